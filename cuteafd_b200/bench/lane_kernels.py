"""Per-kernel timing of the lane transfer kernels of the attention/expert layouts on ONE GPU, with "peers" that are local
buffers (`parallel.local.LocalBlocks`): token-major dispatch (quantise once per token + stores into every owning rank's slab),
multi-lane route pack, row gather into expert order, lane combine push, and the ordered combine.  NVLink time is NOT in these
numbers (stores land in local HBM); what they show is the launch + SM cost of each step of a layer's expert round trip, and they
give `ncu` a single-process target:

    python -m cuteafd_b200.bench.lane_kernels --tokens 16 --lanes 8 [--model qwen3-235b|deepseek-v3] [--iters 200]

The run emulates one rank of a colocated layout with `lanes` ranks: it dispatches its `tokens` rows to all ranks' slabs, then
plays expert rank 0, which sees `lanes` lanes of `tokens` rows each (the other lanes' slabs are filled by extra dispatches).
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from .. import ops
from ..config import deepseek_v3_spec, qwen3_235b_spec
from ..ops import ActBuffer, KIND_BY_NAME, native
from ..parallel import peer_ops
from ..parallel.afd import PtrTable, payload_row_bytes, sf_row_bytes
from ..parallel.local import LocalBlocks


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-235b", choices=["qwen3-235b", "deepseek-v3"])
    ap.add_argument("--tokens", type=int, default=16)
    ap.add_argument("--lanes", type=int, default=8)
    ap.add_argument("--iters", type=int, default=200)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    spec = qwen3_235b_spec(1) if a.model == "qwen3-235b" else deepseek_v3_spec(4)
    H, k, E, L, T = spec.hidden, spec.moe.top_k, spec.moe.n_experts, a.lanes, a.tokens
    kind = KIND_BY_NAME[spec.quant.experts]
    rb, sfb = payload_row_bytes(H, kind), sf_row_bytes(H, kind)
    regions = {"slab_q": L * T * rb, "slab_sf": max(256, L * T * sfb), "idx": L * T * k * 4, "lane_T": 256, "y_recv": T * k * H * 2, "flags": 4096}
    blocks = LocalBlocks(regions, dev, L)
    g = torch.Generator(device=dev).manual_seed(0)
    i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
    status, ctl, done = i32(4), i32(4), i32(8)
    inv_gs = torch.tensor([64.0], device=dev)
    xs_in = [torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16) for _ in range(L)]
    logits = torch.randn(L * T, E, generator=g, device=dev)
    idx_all, wts_all = i32(L * T, k), torch.zeros(L * T, k, device=dev)
    ops.router_select(logits, None, idx_all, wts_all, L * T, k, "softmax", True, 1.0)
    ranks = list(range(L))
    views = [blocks.view(r) for r in ranks]

    def tables(lane):
        tb = lambda name, off: PtrTable([views[0].peer_ptr(r, name, off) for r in ranks])
        return (tb("slab_q", lane * T * rb), tb("slab_sf", lane * T * sfb), tb("idx", lane * T * k * 4), tb("lane_T", lane * 4), tb("flags", lane * 4))
    tabs = [tables(l) for l in range(L)]

    def dispatch(lane):
        q, sf, ix, lt, fl = tabs[lane]
        peer_ops.dispatch_tok_push(xs_in[lane], idx_all[lane * T:(lane + 1) * T], q.arr, sf.arr, ix.arr, lt.arr, fl.arr, inv_gs, ctl, done[0:1],
                                   0, T, T, H, k, E, L, kind, sfb, 0, status)
    # expert rank 0
    e_lo, e_hi = 0, E // L
    rows = L * T * k
    tn = ops.pick_tn(min(max(1, -(-rows // E) * 2), 32), swiglu=True)
    max_tiles = (e_hi - e_lo) + rows // tn + 1
    src_token, src_route, slot_row = i32(rows), i32(rows), i32(L * T, k)
    counts, offsets, tiles, n_tiles, n_rows = i32(e_hi), i32(e_hi), i32(max_tiles, 4), i32(1), i32(1)
    v0 = views[0]
    slab_q = v0.local("slab_q", torch.uint8, (L, T, rb))
    slab_sf = v0.local("slab_sf", torch.uint8)[:L * T * sfb].view(L, T, sfb)
    idx_tab, lane_T = v0.local("idx", torch.int32, (L, T, k)), v0.local("lane_T", torch.int32)[:L]
    xs = ActBuffer.alloc(kind, rows, H, tn, dev)
    y2 = torch.randn(rows, H, generator=g, device=dev).to(torch.bfloat16)
    recv = PtrTable([views[0].peer_ptr(r, "y_recv") for r in ranks])
    cflags = PtrTable([views[0].peer_ptr(r, "flags", (64 + 0) * 4) for r in ranks])
    wait_d = native.flag_wait(v0.peer_ptr(0, "flags", 0), L, 1, ctl, status)
    wait_c = native.flag_wait(v0.peer_ptr(0, "flags", 64 * 4), 1, 1, ctl, status)
    y_recv = v0.local("y_recv", torch.bfloat16, (T * k, H))
    ident = torch.arange(T * k, dtype=torch.int32, device=dev).view(T, k).contiguous()
    resid = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    out = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)

    def pack():
        ops.route_pack(idx_tab, src_token, slot_row, counts, offsets, tiles, n_tiles, n_rows, L * T, k, e_lo, e_hi, tn, max_tiles, src_route=src_route,
                       wait=wait_d, lane_T=lane_T, t_cap=T)

    steps = {
        "dispatch_tok_push (my lane -> all ranks)": lambda: dispatch(0),
        "route_pack over all lanes (in-kernel flag wait)": pack,
        "route_gather (slab rows -> expert order)": lambda: ops.route_gather(slab_q, slab_sf, src_token, n_rows, xs, rows, status),
        "combine_push_lanes (expert outputs -> lanes)": lambda: peer_ops.combine_push_lanes(y2, src_route, n_rows, recv.arr, cflags.arr, ctl, done[1:2], H, k, T, 1,
                                                                                           L, rows, 0, status),
        "moe_combine (ordered weighted sum, in-kernel flag wait)": lambda: ops.moe_combine(y_recv, ident, wts_all[:T], None, resid, out, T, k, wait=wait_c),
    }
    peer_ops.step_begin(ctl)
    for lane in range(L):
        dispatch(lane)              # every lane delivered: the waits below are satisfied from the first launch on
    torch.cuda.synchronize()
    res = {}
    for name, fn in steps.items():
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for _ in range(10):
                fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters // 10):
            gr.replay()
        e1.record()
        torch.cuda.synchronize()
        res[name] = round(e0.elapsed_time(e1) * 1e3 / (a.iters // 10 * 10), 2)
    print(json.dumps({"bench": "lane_kernels", "model": spec.name, "tokens_per_lane": T, "lanes": L, "hidden": H, "top_k": k, "experts": E,
                      "expert_format": spec.quant.experts, "rows_on_this_expert_rank": int(n_rows[0]), "status": status.tolist(),
                      "us_per_launch_back_to_back_in_a_graph": res,
                      "note": "peers are local buffers: no NVLink time; kernels replayed back to back from a CUDA graph (launch latency hidden)"}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
