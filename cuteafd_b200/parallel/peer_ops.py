"""Python wrappers of the peer-memory kernels in `csrc/peer.cu` (flags, push, TP2 wait+add, dispatch, combine)."""
from __future__ import annotations

import ctypes as C

import torch

from ..ops.native import call, ptr, stream

WAIT_NS = 2_000_000_000      # two seconds: a flag that has not arrived by then is a failed peer, not a slow one
WAIT_NS_EAGER = 10_000_000_000   # launches outside graph capture include first-use set-up (module loads, allocations) on the peer


def wait_ns() -> int:
    """Time limit for an in-kernel flag wait: the short limit inside captured graphs (steady state), the long one for eager
    launches, which include each rank's first-use set-up."""
    return WAIT_NS if torch.cuda.is_current_stream_capturing() else WAIT_NS_EAGER

# Flag addresses whose releasing kernel has been launched in the current step, recorded only while a single-GPU scheduler
# (`parallel.local.LocalWorld`) runs several ranks' programs in one stream; None otherwise.
PUBLISHED: set | None = None


def note_published(addrs):
    if PUBLISHED is not None:
        PUBLISHED.update(int(a) for a in addrs)


def step_begin(ctl: torch.Tensor):
    call("cuteafd_step_begin", ptr(ctl), stream())


def wait_flags(flags_ptr: int, n: int, stride: int, ctl, step_offset: int, status, timeout_ns: int | None = None):
    timeout_ns = wait_ns() if timeout_ns is None else timeout_ns
    call("cuteafd_wait_flags", flags_ptr, n, stride, ptr(ctl), step_offset, timeout_ns, ptr(status), stream())


def push_bytes(src: torch.Tensor, peer_dst: int, nbytes: int, peer_flag: int, ctl, step_offset: int, done_counter):
    call("cuteafd_push_bytes", ptr(src), peer_dst, nbytes, peer_flag, ptr(ctl), step_offset, ptr(done_counter), stream())


def wait_add(mine, theirs, residual, out, elems: int, my_rank: int, flag_ptr: int, ctl, step_offset: int, status,
             timeout_ns: int | None = None):
    timeout_ns = wait_ns() if timeout_ns is None else timeout_ns
    call("cuteafd_wait_add", ptr(mine), ptr(theirs), ptr(residual), ptr(out), elems, my_rank, flag_ptr, ptr(ctl), step_offset,
         timeout_ns, ptr(status), stream())


def wait_concat(mine, theirs, out, n_rows: int, w0: int, w1: int, my_rank: int, flag_ptr: int, ctl, step_offset: int, status,
                timeout_ns: int | None = None):
    """out[r] = [share of rank 0 | share of rank 1] (fp32 rows) once the partner's share has landed (vocabulary-parallel head)."""
    timeout_ns = wait_ns() if timeout_ns is None else timeout_ns
    call("cuteafd_wait_concat", ptr(mine), ptr(theirs), ptr(out), n_rows, w0, w1, my_rank, flag_ptr, ptr(ctl), step_offset, timeout_ns,
         ptr(status), stream())


def dispatch_push(x, idx, slot_row, offsets, slab_q_tbl, slab_sf_tbl, idx_tbl, flag_tbl, inv_gs, ctl, done_counter, T0, T1, H, k,
                  E_local, n_ep, kind, sf_ld, rows_cap, step_offset, status):
    call("cuteafd_dispatch_push", ptr(x), ptr(idx), ptr(slot_row), ptr(offsets), C.addressof(slab_q_tbl),
         C.addressof(slab_sf_tbl) if slab_sf_tbl is not None else None, C.addressof(idx_tbl), C.addressof(flag_tbl), ptr(inv_gs), ptr(ctl),
         ptr(done_counter), T0, T1, H, k, E_local, n_ep, kind, sf_ld, rows_cap, step_offset, ptr(status), stream())


def combine_push(y, src_route, n_rows, recv_tbl, flag_tbl, ctl, done_counter, H, n_attn, rows_cap, step_offset):
    call("cuteafd_combine_push", ptr(y), ptr(src_route), ptr(n_rows), C.addressof(recv_tbl), C.addressof(flag_tbl), ptr(ctl),
         ptr(done_counter), H, n_attn, rows_cap, step_offset, stream())


def dispatch_tok_push(x, idx, slab_q_tbl, slab_sf_tbl, idx_tbl, lane_t_tbl, flag_tbl, inv_gs, ctl, done_counter, T0, T1, T, H, k, E, n_ep, kind,
                      sf_ld, step_offset, status, broadcast: bool = False):
    """Token-major dispatch of rows [T0, T1) of a lane that holds T tokens: each row is quantised once and stored into the slab
    of every expert rank owning one of its experts (`broadcast`: of every expert rank - they each hold a slice of every
    expert); the routing rows and T go to every rank; then one flag per rank."""
    call("cuteafd_dispatch_tok_push", ptr(x), ptr(idx), C.addressof(slab_q_tbl), C.addressof(slab_sf_tbl) if slab_sf_tbl is not None else None,
         C.addressof(idx_tbl), C.addressof(lane_t_tbl), C.addressof(flag_tbl), ptr(inv_gs), ptr(ctl), ptr(done_counter), T0, T1, T, H, k, E,
         n_ep, kind, sf_ld, 1 if broadcast else 0, step_offset, ptr(status), stream())


def combine_push_lanes(y, src_route, n_rows, recv_tbl, flag_tbl, ctl, done_counter, H, k, t_cap, tp, n_dst, rows_cap, step_offset, status):
    """Expert outputs back to the attention ranks of every lane that sent rows (route = (lane * t_cap + t) * k + slot)."""
    call("cuteafd_combine_push_lanes", ptr(y), ptr(src_route), ptr(n_rows), C.addressof(recv_tbl), C.addressof(flag_tbl), ptr(ctl),
         ptr(done_counter), H, k, t_cap, tp, n_dst, rows_cap, step_offset, ptr(status), stream())
