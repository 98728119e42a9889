"""Symmetric device memory across the ranks of one node (CUDA IPC) for kernels that load/store peer memory.

Every rank allocates one block with the same layout, exports it with `cudaIpcGetMemHandle`, and opens the other
ranks' blocks; `SymmetricBlock.peer_ptr(rank, name)` is then a device pointer into rank `rank`'s copy of the named
region that this rank's kernels can dereference over NVLink.  Handles travel through `torch.distributed`
(`all_gather_object`), which is also the bootstrap for the NCCL baseline path.
(Reference: peer publication / attach_peer, rust/crates/cuteafd-daemon/src/shared/peer_split.rs:34-60;
RDMA ring registration plays this role between hosts, cuteafd-transport/src/verbs.rs.)
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from ..ops import native


@dataclass
class Region:
    offset: int
    nbytes: int


class SymmetricBlock:
    """One contiguous allocation per rank with named, 256-byte aligned regions (identical layout on all ranks)."""

    def __init__(self, regions: dict[str, int], device, group=None, rank: int = 0, world: int = 1):
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.regions: dict[str, Region] = {}
        off = 0
        for name, nbytes in regions.items():
            self.regions[name] = Region(off, nbytes)
            off += -(-nbytes // 256) * 256
        self.nbytes = max(off, 256)
        self.buf = torch.zeros(self.nbytes, dtype=torch.uint8, device=self.device)
        from ..utils.memory_ledger import LEDGER
        with LEDGER.scope("peer-split"):
            LEDGER.charge(self.nbytes, "symmetric block")
        self.base = [0] * world
        self.base[rank] = self.buf.data_ptr()
        self._opened: list = []
        if world > 1:
            self._exchange(group)

    def _exchange(self, group):
        import torch.distributed as dist
        handle = (C.c_ubyte * 64)()
        offset = C.c_ulonglong(0)
        native.call("cuteafd_ipc_export", self.buf.data_ptr(), C.addressof(handle), C.addressof(offset))
        mine = (bytes(handle), int(offset.value))
        gathered = [None] * self.world
        dist.all_gather_object(gathered, mine, group=group)
        for r, (h, off) in enumerate(gathered):
            if r == self.rank:
                continue
            hb = (C.c_ubyte * 64).from_buffer_copy(h)
            out = C.c_void_p(0)
            native.call("cuteafd_ipc_open", C.addressof(hb), C.c_ulonglong(off), C.addressof(out))
            self.base[r] = int(out.value)
            self._opened.append((int(out.value), off))
        dist.barrier(group=group)

    def local(self, name: str, dtype=torch.uint8, shape=None) -> torch.Tensor:
        r = self.regions[name]
        t = self.buf[r.offset:r.offset + r.nbytes].view(dtype)
        return t.view(*shape) if shape is not None else t

    def peer_ptr(self, rank: int, name: str, byte_offset: int = 0) -> int:
        return self.base[rank] + self.regions[name].offset + byte_offset

    def ptr_table(self, ranks, name: str, byte_offset: int = 0):
        """ctypes array of void* (host memory) with the region's address on each of `ranks`."""
        arr = (C.c_void_p * len(ranks))()
        for i, r in enumerate(ranks):
            arr[i] = self.peer_ptr(r, name, byte_offset)
        return arr

    def close(self):
        for ptr, off in self._opened:
            try:
                native.call("cuteafd_ipc_close", ptr, C.c_ulonglong(off))
            except Exception:
                pass
        self._opened = []
