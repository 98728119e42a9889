"""EP dispatch -> grouped GEMM -> combine micro-benchmark (hidden 7168, 256 routed experts, top-8, SwiGLU
intermediate 2048, MXFP4 expert weights, bf16 activations, N(0,1) router logits), swept over tokens per rank.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m cuteafd_b200.bench.ep_microbench \
        --tokens 1,16,128,1024,4096 --comm p2p

All `world` ranks are both senders and expert owners (EP = world).  Per iteration every rank: quantises each of its tokens
once and stores the row into the lane slab of every rank that owns one of its experts (peer stores + flags; routing rows and
token counts travel with them), waits in-kernel for all lanes, packs and gathers the received rows into expert order, runs the
grouped MXFP4 FC1 (SwiGLU, FP4 output) + FC2, pushes the output rows back to the token owners, and forms the ordered weighted
top-k sum (waiting in-kernel for the owners' flags).
`--comm nccl` is the baseline: all_to_all_single of bf16 rows both ways around the same local GEMMs.
Time is CUDA-event device time, max over ranks; the roofline is the slowest of the GEMM flops at the measured bf16
peak (an under-estimate for FP4), the bytes that must cross NVLink at 770 GB/s per direction, and the expert weight bytes that
must stream from HBM at the measured copy bandwidth.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from .. import ops
from ..config import ep_microbench_spec
from ..ops import ActBuffer, KIND_BF16, KIND_MXFP4, TcWeight, native, pick_tn
from ..parallel import peer_ops
from ..parallel.afd import PtrTable
from ..parallel.symm import SymmetricBlock


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="1,16,128,1024,4096")
    ap.add_argument("--comm", default="p2p", choices=["p2p", "nccl"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    spec = ep_microbench_spec()
    H, I, E, k = spec.hidden, spec.moe.intermediate, spec.moe.n_experts, spec.moe.top_k
    e_lo, e_hi = (rank * E) // world, ((rank + 1) * E) // world
    El = e_hi - e_lo
    wg, wu, wd = (TcWeight.random(El, I, H, "mxfp4", dev, seed=10 + rank), TcWeight.random(El, I, H, "mxfp4", dev, seed=20 + rank),
                  TcWeight.random(El, H, I, "mxfp4", dev, seed=30 + rank))
    results = []
    for T in [int(t) for t in a.tokens.split(",")]:
        Tg = T * world                                 # global tokens; every rank knows the full routing table
        rows_cap = Tg * k
        g = torch.Generator(device=dev).manual_seed(1234)            # same stream on every rank -> identical routing tables
        logits = torch.randn(Tg, E, generator=g, device=dev)
        x_all = torch.randn(Tg, H, generator=g, device=dev).to(torch.bfloat16)
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
        idx, wts = i32(Tg, k), torch.zeros(Tg, k, device=dev)
        ops.router_select(logits, None, idx, wts, Tg, k, "softmax", True, 1.0)
        tn = pick_tn(min(max(1, -(-rows_cap // E) * 2), 128), swiglu=True)
        max_tiles = El + rows_cap // tn + 1
        # global packing (dispatch addressing) and local packing (GEMM tile table)
        g_src, g_slot, g_cnt, g_off, g_tiles, g_nt, g_nr = i32(rows_cap), i32(Tg, k), i32(E), i32(E), i32(E + 2, 4), i32(1), i32(1)
        l_src, l_route, l_slot, l_cnt, l_off, l_tiles, l_nt, l_nr = i32(rows_cap), i32(rows_cap), i32(Tg, k), i32(El), i32(El), i32(max_tiles, 4), i32(1), i32(1)
        status, ctl, done = i32(4), i32(4), i32(8)
        inv_gs = torch.ones(1, device=dev)
        sf_ld = H // 32
        block = SymmetricBlock({"slab_q": Tg * H // 2, "slab_sf": Tg * (-(-H // 256) * 8), "idx": Tg * k * 4, "lane_T": 256, "y_recv": T * k * H * 2,
                                "flags": 64 * 4}, dev, None, rank, world) if a.comm == "p2p" else None
        h1 = torch.zeros(rows_cap, I, dtype=torch.bfloat16, device=dev)
        h1q = ActBuffer.alloc(KIND_MXFP4, rows_cap, I, tn, dev)
        y2 = torch.zeros(rows_cap, H, dtype=torch.bfloat16, device=dev)
        out = torch.zeros(Tg, H, dtype=torch.bfloat16, device=dev)
        ident = torch.arange(rows_cap, dtype=torch.int32, device=dev).view(Tg, k).contiguous()
        ranks = list(range(world))
        if a.comm == "p2p":
            # token-major lanes: rank r is lane r on every rank (slab rows [r * T, (r + 1) * T)); each token crosses NVLink once per
            # destination rank, the expert side gathers rows into expert order itself
            sf_pad = -(-H // 256) * 8
            slab_q = block.local("slab_q", torch.uint8, (Tg, H // 2))
            slab_sf = block.local("slab_sf", torch.uint8)[:Tg * sf_pad].view(Tg, sf_pad)
            idx_tab = block.local("idx", torch.int32, (Tg, k))
            lane_T = block.local("lane_T", torch.int32)[:world]
            xs = ActBuffer.alloc(KIND_MXFP4, rows_cap, H, tn, dev)
            mk = lambda name, off: PtrTable([block.peer_ptr(r, name, off) for r in ranks])
            q_tbl, sf_tbl, i_tbl, t_tbl = mk("slab_q", rank * T * (H // 2)), mk("slab_sf", rank * T * sf_pad), mk("idx", rank * T * k * 4), mk("lane_T", rank * 4)
            f_disp = mk("flags", rank * 4)
            recv_tbl = PtrTable([block.peer_ptr(r, "y_recv") for r in ranks])        # lane r's rows return to rank r
            f_comb = PtrTable([block.peer_ptr(r, "flags", (16 + rank) * 4) for r in ranks])
            y_recv = block.local("y_recv", torch.bfloat16, (T * k, H))
            x_mine, idx_mine = x_all[rank * T:(rank + 1) * T].contiguous(), idx[rank * T:(rank + 1) * T].contiguous()
            ident_mine = torch.arange(T * k, dtype=torch.int32, device=dev).view(T, k).contiguous()
            wait_d = native.flag_wait(block.peer_ptr(rank, "flags", 0), world, 1, ctl, status)
            wait_c = native.flag_wait(block.peer_ptr(rank, "flags", 16 * 4), world, 1, ctl, status)
        else:
            xs = ActBuffer.alloc(KIND_MXFP4, rows_cap, H, tn, dev)

        def step_p2p():
            peer_ops.step_begin(ctl)
            peer_ops.dispatch_tok_push(x_mine, idx_mine, q_tbl.arr, sf_tbl.arr, i_tbl.arr, t_tbl.arr, f_disp.arr, inv_gs, ctl, done[0:1], 0, T, T, H, k, E,
                                       world, KIND_MXFP4, sf_pad, 0, status)
            ops.route_pack(idx_tab, l_src, l_slot, l_cnt, l_off, l_tiles, l_nt, l_nr, Tg, k, e_lo, e_hi, tn, max_tiles, src_route=l_route,
                           wait=wait_d, lane_T=lane_T, t_cap=T)
            ops.route_gather(slab_q, slab_sf, l_src, l_nr, xs, rows_cap, status)
            ops.tc_linear(wg, xs, None, rows=rows_cap, w_up=wu, tiles=l_tiles, n_tiles=l_nt, max_tiles=max_tiles, status=status, quant_out=h1q)
            ops.tc_linear(wd, h1q, y2, rows=rows_cap, tiles=l_tiles, n_tiles=l_nt, max_tiles=max_tiles, status=status)
            peer_ops.combine_push_lanes(y2, l_route, l_nr, recv_tbl.arr, f_comb.arr, ctl, done[1:2], H, k, T, 1, world, rows_cap, 0, status)
            ops.moe_combine(y_recv, ident_mine, wts[rank * T:(rank + 1) * T], None, None, out[:T], T, k, wait=wait_c)

        def step_nccl():
            # baseline: every rank already holds the routing table; exchange bf16 rows with all_to_all, GEMMs local
            ops.route_pack(idx, l_src, l_slot, l_cnt, l_off, l_tiles, l_nt, l_nr, Tg, k, e_lo, e_hi, tn, max_tiles, src_route=l_route)
            n_local = int(l_nr[0])
            owner = torch.bucketize(idx[rank * T:(rank + 1) * T].flatten(), torch.tensor([(r * E) // world for r in range(1, world)], device=dev), right=True)
            order = torch.argsort(owner, stable=True)
            send_counts = torch.bincount(owner, minlength=world).tolist()
            send = x_all[rank * T:(rank + 1) * T].repeat_interleave(k, 0)[order].contiguous()
            recv_counts = [int(((idx[r * T:(r + 1) * T] >= e_lo) & (idx[r * T:(r + 1) * T] < e_hi)).sum()) for r in range(world)]
            recv = torch.empty(sum(recv_counts), H, dtype=torch.bfloat16, device=dev)
            dist.all_to_all_single(recv, send, recv_counts, send_counts)
            ops.quant_fp4_rows(x_all, xs, src_rows=l_src, n_rows_dev=l_nr, rows=rows_cap)      # rows gathered from the replicated input
            ops.tc_linear(wg, xs, h1, rows=rows_cap, w_up=wu, tiles=l_tiles, n_tiles=l_nt, max_tiles=max_tiles, status=status)
            ops.quant_fp4_rows(h1, h1q, n_rows_dev=l_nr, rows=rows_cap)
            ops.tc_linear(wd, h1q, y2, rows=rows_cap, tiles=l_tiles, n_tiles=l_nt, max_tiles=max_tiles, status=status)
            back = torch.empty(sum(send_counts), H, dtype=torch.bfloat16, device=dev)
            dist.all_to_all_single(back, y2[:sum(recv_counts)].contiguous(), send_counts, recv_counts)
            inv = torch.empty_like(order); inv[order] = torch.arange(order.numel(), device=dev)
            ops.moe_combine(back[inv].contiguous(), ident[:T], wts[rank * T:(rank + 1) * T], None, None, out[:T], T, k)

        step = step_p2p if a.comm == "p2p" else step_nccl
        if world > 1:
            dist.barrier()
        for _ in range(a.warmup):
            step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        st = int(status[0])
        flops = 2.0 * T * world * k * 3 * H * I / world            # per rank, balanced routing
        nv_bytes = T * k * (H / 2 + H / 32) * (world - 1) / world + T * k * H * 2 * (world - 1) / world
        # weights that must stream from HBM: experts of this rank that receive at least one row (expected value)
        p_hit = 1.0 - (1.0 - 1.0 / E) ** (Tg * k)
        hbm_bytes = El * p_hit * 3 * H * I * (0.5 + 1.0 / 32)
        roof_ms = max(flops / 1.6866e15, nv_bytes / 770e9, hbm_bytes / 6.538e12) * 1e3
        if rank == 0:
            results.append({"tokens_per_rank": T, "ms": round(float(ms[0]), 4), "roofline_ms": round(roof_ms, 4),
                            "fraction_of_roofline": round(roof_ms / float(ms[0]), 4), "status": st})
        if block is not None:
            block.close()
            del block
        if world > 1:
            dist.barrier()
    if rank == 0:
        print(json.dumps({"bench": "ep_dispatch_gemm_combine", "comm": a.comm, "world": world, "hidden": H, "experts": E, "top_k": k,
                          "intermediate": I, "weights": "mxfp4", "results": results,
                          "roofline": "max(GEMM flops / measured bf16 peak 1686.6 TFLOP/s, NVLink bytes / 770 GB/s per direction, touched expert weight bytes / measured HBM copy 6538 GB/s)"}))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
