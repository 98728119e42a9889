"""Micro-benchmarks of the tcgen05 linear kernels (decode-sized token tiles), timed as CUDA-graph replays of several
launches over DISTINCT weights (so nothing is served from L2) with CUDA events.

    python -m cuteafd_b200.bench.gemm --mode stream     # weight streaming: GB/s of large skinny GEMMs per format and K
    python -m cuteafd_b200.bench.gemm --mode small      # decode projections (QKV / O / router shapes) per split-K factor
    python -m cuteafd_b200.bench.gemm --mode trace      # device time stamps of the persistent kernel on small layers
    python -m cuteafd_b200.bench.gemm --mode moe        # grouped FC1 (SwiGLU, FP4 output) and FC2 of a decode step, per kernel
"""
from __future__ import annotations

import argparse

import torch

from .. import ops
from ..ops import ActBuffer, TcWeight


def graph_time_us(fns, reps: int = 5) -> float:
    """Median device time per launch (microseconds) of one graph holding every callable of `fns`."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fns:
            f()
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / len(fns))
    ts.sort()
    return ts[len(ts) // 2]


def stream(dev, T: int = 16):
    st = torch.zeros(4, dtype=torch.int32, device=dev)
    cases = [("bf16 K4096", "bf16", 75776, 4096, False), ("nvfp4 K8192", "nvfp4", 151552, 8192, False),
             ("nvfp4 K4096", "nvfp4", 303104, 4096, False), ("nvfp4 K2048", "nvfp4", 606208, 2048, False),
             ("nvfp4 K1536", "nvfp4", 606208, 1536, False), ("nvfp4 K1024", "nvfp4", 606208, 1024, False),
             ("mxfp4 K4096", "mxfp4", 303104, 4096, False), ("mxfp4 K1536", "mxfp4", 606208, 1536, False),
             ("nvfp4 swiglu K4096", "nvfp4", 151552, 4096, True)]
    for name, kind, N, K, sw in cases:
        copies = 3
        Ws = [TcWeight.random(1, N, K, kind, dev, seed=i) for i in range(copies * (2 if sw else 1))]
        x = ActBuffer.alloc(Ws[0].kind, T, K, ops.pick_tn(T, swiglu=True), dev)
        y = torch.zeros(T, N, dtype=torch.bfloat16, device=dev)
        if sw:
            fns = [(lambda i=i: ops.tc_linear(Ws[2 * i], x, y, w_up=Ws[2 * i + 1], status=st)) for i in range(copies)]
            nbytes = Ws[0].nbytes * 2
        else:
            fns = [(lambda W=W: ops.tc_linear(W, x, y, status=st)) for W in Ws]
            nbytes = Ws[0].nbytes
        us = graph_time_us(fns)
        print(f"{name:20s} N={N} K={K} T={T} {us:8.1f} us  {nbytes / us / 1e3:7.1f} GB/s  ({nbytes / 1e6:.0f} MB)", flush=True)
        del Ws
    print("status", st.tolist())


SMALL = [("wqkv", "nvfp4", 9216, 4096, 12), ("wo", "nvfp4", 4096, 8192, 12), ("router", "bf16", 128, 4096, 64),
         ("shared-ish", "nvfp4", 1536, 4096, 40), ("q_b (mla)", "bf16", 12288, 1536, 8), ("o (mla)", "bf16", 7168, 8192, 4),
         ("q_a fp8", "fp8_block128", 1536, 7168, 12), ("q_b fp8", "fp8_block128", 24576, 1536, 6), ("o fp8", "fp8_block128", 7168, 16384, 4)]


def small(dev, T: int = 16):
    st = torch.zeros(4, dtype=torch.int32, device=dev)
    for name, kind, N, K, copies in SMALL:
        Ws = [TcWeight.random(1, N, K, kind, dev, seed=i) for i in range(copies)]
        x = ActBuffer.alloc(Ws[0].kind, T, K, ops.pick_tn(T, swiglu=True), dev)
        y = torch.zeros(T, N, dtype=torch.bfloat16, device=dev)
        for splits in (1, 2, 3, 4, 8):
            us = graph_time_us([(lambda W=W: ops.tc_linear(W, x, y, splits=splits, status=st)) for W in Ws])
            how = "cluster" if splits in (2, 4, 8) else ("global fix-up" if splits > 1 else "-")
            print(f"{name:10s} T={T} splits={splits} ({how:13s}) {us:8.2f} us/launch  {Ws[0].nbytes / us / 1e3:7.1f} GB/s", flush=True)
    print("status", st.tolist())


def trace(dev, T: int = 16):
    """Period between launches, first load -> end of the last epilogue, and the gap to the next launch's first load
    (tear-down + launch + prologue, and for the global fix-up the fix-up itself), from the kernel's own stamps."""
    import numpy as np
    st = torch.zeros(4, dtype=torch.int32, device=dev)
    for name, kind, N, K, splits in [("wqkv", "nvfp4", 9216, 4096, 1), ("wqkv", "nvfp4", 9216, 4096, 3), ("wo", "nvfp4", 4096, 8192, 1),
                                     ("wo", "nvfp4", 4096, 8192, 3), ("router", "bf16", 128, 4096, 3)]:
        copies = 10
        Ws = [TcWeight.random(1, N, K, kind, dev, seed=i) for i in range(copies)]
        x = ActBuffer.alloc(Ws[0].kind, T, K, 16, dev)
        y = torch.zeros(T, N, dtype=torch.bfloat16, device=dev)
        bufs = [torch.zeros(296, 4, 8, dtype=torch.int64, device=dev) for _ in range(copies)]

        def run():
            for W, b in zip(Ws, bufs):
                ops.tc_trace(b, 4)
                ops.tc_linear(W, x, y, splits=splits, status=st)
            ops.tc_trace(None)
        run()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            run()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        starts, ends = [], []
        for b in bufs:
            t = b.cpu().numpy()
            starts.append(t[:, :, 7][t[:, :, 7] != 0].min())
            ends.append(t[:, :, 3][t[:, :, 3] != 0].max())
        starts, ends = np.array(starts), np.array(ends)
        print(f"{name} splits={splits}: period {np.diff(starts)[2:].mean() / 1e3:.2f} us, first load -> last epilogue "
              f"{(ends - starts)[2:].mean() / 1e3:.2f} us, gap to the next first load {(starts[1:] - ends[:-1])[2:].mean() / 1e3:.2f} us", flush=True)
    print("status", st.tolist())


def moe(dev, T: int = 16, E: int = 128, k: int = 8, H: int = 4096, I: int = 1536, kind: str = "nvfp4"):
    """The two grouped expert GEMMs of one decode step (Qwen3-235B shape by default: 16 tokens x top-8 of 128 experts), each
    timed alone over three distinct weight sets (nothing served from L2); GB/s counts the weights of the ACTIVE experts only."""
    st = torch.zeros(4, dtype=torch.int32, device=dev)
    copies = 3
    g = torch.Generator(device=dev).manual_seed(1)
    logits = torch.randn(T, E, generator=g, device=dev)
    idx, wts = torch.zeros(T, k, dtype=torch.int32, device=dev), torch.zeros(T, k, device=dev)
    ops.router_select(logits, None, idx, wts, T, k, "softmax", True, 1.0)
    rows = T * k
    for tn in (16, 32):
        max_tiles = E + rows // tn + 1
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
        src_token, slot_row, counts, offsets, tiles, n_tiles, n_rows = i32(rows), i32(T, k), i32(E), i32(E), i32(max_tiles, 4), i32(1), i32(1)
        ops.route_pack(idx, src_token, slot_row, counts, offsets, tiles, n_tiles, n_rows, T, k, 0, E, tn, max_tiles)
        torch.cuda.synchronize()
        active = int((counts > 0).sum())
        Wg = [TcWeight.random(E, I, H, kind, dev, seed=10 + i) for i in range(copies)]
        Wu = [TcWeight.random(E, I, H, kind, dev, seed=20 + i) for i in range(copies)]
        Wd = [TcWeight.random(E, H, I, kind, dev, seed=30 + i) for i in range(copies)]
        xs = ActBuffer.alloc(Wg[0].kind, rows, H, tn, dev)
        h1q = ActBuffer.alloc(Wg[0].kind, rows, I, tn, dev)
        y2 = torch.zeros(rows, H, dtype=torch.bfloat16, device=dev)
        per_expert_fc1 = 2 * Wg[0].nbytes / E
        per_expert_fc2 = Wd[0].nbytes / E
        fc1 = [(lambda i=i: ops.tc_linear(Wg[i], xs, None, rows=rows, w_up=Wu[i], tiles=tiles, n_tiles=n_tiles, max_tiles=max_tiles, status=st,
                                          quant_out=h1q, inv_gs_out=Wd[i].inv_act_gs)) for i in range(copies)]
        fc2 = [(lambda i=i: ops.tc_linear(Wd[i], h1q, y2, rows=rows, tiles=tiles, n_tiles=n_tiles, max_tiles=max_tiles, status=st)) for i in range(copies)]
        u1, u2 = graph_time_us(fc1), graph_time_us(fc2)
        both = graph_time_us([f for pair in zip(fc1, fc2) for f in pair]) * 2
        print(f"{kind} tn={tn} T={T} active experts {active}/{E}: FC1 {u1:7.1f} us {active * per_expert_fc1 / u1 / 1e3:7.1f} GB/s | "
              f"FC2 {u2:7.1f} us {active * per_expert_fc2 / u2 / 1e3:7.1f} GB/s | FC1+FC2 back to back {both:7.1f} us", flush=True)
        del Wg, Wu, Wd
    print("status", st.tolist())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="stream", choices=["stream", "small", "trace", "moe"])
    ap.add_argument("--tokens", type=int, default=16)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    {"stream": stream, "small": small, "trace": trace, "moe": moe}[a.mode](dev, a.tokens)


if __name__ == "__main__":
    main()
