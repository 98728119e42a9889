"""Python wrappers of the peer-memory kernels in `csrc/peer.cu` (flags, push, TP2 wait+add, dispatch, combine)."""
from __future__ import annotations

import ctypes as C

import torch

from ..ops.native import call, ptr, stream

WAIT_NS = 2_000_000_000      # two seconds: a flag that has not arrived by then is a failed peer, not a slow one


def step_begin(ctl: torch.Tensor):
    call("cuteafd_step_begin", ptr(ctl), stream())


def wait_flags(flags_ptr: int, n: int, stride: int, ctl, step_offset: int, status, timeout_ns: int = WAIT_NS):
    call("cuteafd_wait_flags", flags_ptr, n, stride, ptr(ctl), step_offset, timeout_ns, ptr(status), stream())


def arm_flag_wait(flags_ptr: int, n: int, stride: int, ctl, status, timeout_ns: int = WAIT_NS):
    """The next route_pack / moe_combine launch waits for these flags inside the kernel (no wait-only launch)."""
    call("cuteafd_arm_flag_wait", flags_ptr, n, stride, ptr(ctl), timeout_ns, ptr(status))


def push_bytes(src: torch.Tensor, peer_dst: int, nbytes: int, peer_flag: int, ctl, step_offset: int, done_counter):
    call("cuteafd_push_bytes", ptr(src), peer_dst, nbytes, peer_flag, ptr(ctl), step_offset, ptr(done_counter), stream())


def wait_add(mine, theirs, residual, out, elems: int, my_rank: int, flag_ptr: int, ctl, step_offset: int, status,
             timeout_ns: int = WAIT_NS):
    call("cuteafd_wait_add", ptr(mine), ptr(theirs), ptr(residual), ptr(out), elems, my_rank, flag_ptr, ptr(ctl), step_offset,
         timeout_ns, ptr(status), stream())


def dispatch_push(x, idx, slot_row, offsets, slab_q_tbl, slab_sf_tbl, idx_tbl, flag_tbl, inv_gs, ctl, done_counter, T0, T1, H, k,
                  E_local, n_ep, kind, sf_ld, rows_cap, step_offset, status):
    call("cuteafd_dispatch_push", ptr(x), ptr(idx), ptr(slot_row), ptr(offsets), C.addressof(slab_q_tbl),
         C.addressof(slab_sf_tbl) if slab_sf_tbl is not None else None, C.addressof(idx_tbl), C.addressof(flag_tbl), ptr(inv_gs), ptr(ctl),
         ptr(done_counter), T0, T1, H, k, E_local, n_ep, kind, sf_ld, rows_cap, step_offset, ptr(status), stream())


def combine_push(y, src_route, n_rows, recv_tbl, flag_tbl, ctl, done_counter, H, n_attn, rows_cap, step_offset):
    call("cuteafd_combine_push", ptr(y), ptr(src_route), ptr(n_rows), C.addressof(recv_tbl), C.addressof(flag_tbl), ptr(ctl),
         ptr(done_counter), H, n_attn, rows_cap, step_offset, stream())
