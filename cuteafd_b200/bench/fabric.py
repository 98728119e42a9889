"""NVLink / NVSwitch link probes between the GPUs of one node (run under torchrun, one rank per GPU):

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m cuteafd_b200.bench.fabric [--sizes 4096,1048576] [--all-to-all]

Modes, per message size (4 KB ... 256 MB by default), rank 0 <-> rank 1 unless `--all-to-all`:
  copy_engine   cudaMemcpyAsync to the peer's memory (no SM)
  sm_push       SM-issued 16-byte stores into the peer's memory
  sm_pull       SM-issued 16-byte loads from the peer's memory
each one-way (rank 0 only) and both ways at once (every rank pushes / pulls at the same time: full duplex), each launched
eagerly and replayed from a CUDA graph; plus the 8-byte flag round trip (`st.release.sys` / `ld.acquire.sys` ping-pong between
two kernels, one per GPU) whose half is the one-way signalling latency every fused transfer of the split pays per layer.
With `--all-to-all` every rank pushes a slice to every other rank at once (the dispatch / combine pattern).

Times are CUDA events on the launching stream, max over the ranks that took part; bandwidth is payload bytes per direction.
The table this prints is the NVLink denominator of the fused paths' rooflines.
Reference: `cuteafd fabric --p2p` / cuteafd_p2p_probe (native/shared/include/cuteafd_peer_exchange.h:121-138, 353-371: copy
engine vs SM pull vs SM push, one-way vs ping-pong, eager vs graph), commands/bench_rdma*.rs.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from ..ops.native import call, stream
from ..parallel.symm import SymmetricBlock


def _time(fn, iters: int, use_graph: bool) -> float:
    """Milliseconds per call (device time)."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    g = None
    if use_graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        g.replay()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    e0.record()
    for _ in range(iters):
        (g.replay if g is not None else fn)()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="4096,65536,1048576,16777216,268435456")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--all-to-all", action="store_true")
    ap.add_argument("--pingpong-iters", type=int, default=2000)
    a = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    if world < 2:
        print(json.dumps({"error": "the fabric probe needs at least two ranks (torchrun --nproc-per-node 2)"}))
        return 2
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    sizes = [int(s) for s in a.sizes.split(",")]
    big = max(sizes)
    block = SymmetricBlock({"buf": 2 * big, "flags": 256}, dev, None, rank, world)
    src = torch.empty(big, dtype=torch.uint8, device=dev).random_(0, 255)
    local_dst = torch.empty(big, dtype=torch.uint8, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    peer = (rank + 1) % world if not a.all_to_all else None
    rows = []

    def record(mode, size, duplex, graph, ms_local, active):
        t = torch.tensor([ms_local if active else 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            ms = float(t[0])
            rows.append({"mode": mode, "bytes": size, "duplex": duplex, "launch": "graph" if graph else "eager", "us": round(ms * 1e3, 2),
                         "gb_per_s_per_direction": round(size / (ms / 1e3) / 1e9, 1) if ms > 0 else None})

    for size in sizes:
        for graph in (False, True):
            if a.all_to_all:
                part = (size // (world - 1)) // 16 * 16
                if part == 0:
                    continue

                def a2a():
                    for d in range(1, world):
                        p = (rank + d) % world
                        call("cuteafd_peer_copy", block.peer_ptr(p, "buf", rank * part), src.data_ptr(), part, 0, stream())
                ms = _time(a2a, a.iters, graph)
                record("sm_push_all_to_all", part * (world - 1), True, graph, ms, True)
                continue
            modes = {
                "copy_engine": lambda: call("cuteafd_copy_engine", block.peer_ptr(peer, "buf"), src.data_ptr(), size, stream()),
                "sm_push": lambda: call("cuteafd_peer_copy", block.peer_ptr(peer, "buf"), src.data_ptr(), size, 0, stream()),
                "sm_pull": lambda: call("cuteafd_peer_copy", local_dst.data_ptr(), block.peer_ptr(peer, "buf"), size, 0, stream()),
            }
            for mode, fn in modes.items():
                for duplex in (False, True):
                    active = duplex or rank == 0
                    ms = _time(fn if active else (lambda: None), a.iters, graph and active)
                    record(mode, size, duplex, graph, ms, active)
    # 8-byte flag round trip between rank 0 and rank 1 (the other ranks idle)
    out_ns = torch.zeros(1, dtype=torch.int64, device=dev)
    flags = block.local("flags", torch.int32)
    lat = None
    for rep in range(2):                    # first repetition warms both sides up
        dist.barrier()
        torch.cuda.synchronize()
        if rank < 2:
            other = 1 - rank
            call("cuteafd_flag_pingpong", block.peer_ptr(rank, "flags"), block.peer_ptr(other, "flags"), rep * (a.pingpong_iters + 8), a.pingpong_iters,
                 1 if rank == 0 else 0, 2_000_000_000, status.data_ptr(), out_ns.data_ptr(), stream())
        torch.cuda.synchronize()
        lat = float(out_ns[0]) / a.pingpong_iters / 1e3
    t = torch.tensor([lat if rank == 0 else 0.0, float(int(status[0]) != 0)], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"bench": "fabric", "world": world, "gpu": torch.cuda.get_device_name(local),
                          "flag_round_trip_us": round(float(t[0]), 3), "flag_one_way_us": round(float(t[0]) / 2, 3),
                          "status_nonzero": bool(t[1]), "rows": rows}))
    block.close()
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
