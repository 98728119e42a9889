"""Expert-rank lane on ONE GPU with the "peers" mapped to local buffers: route pack -> grouped FC1 (SwiGLU, FP4 output)
-> grouped FC2 whose epilogue stores every output row into [token][slot] of two destination buffers and raises their
flags, against the unfused sequence (FC2 to a local buffer, then the combine_push copy kernel).

The kernels and their arguments are exactly those of the multi-GPU path (`parallel/afd.py`); only the destination
addresses are local, so the kernel can be timed and profiled (ncu) without a second process:

    python -m cuteafd_b200.bench.fused_peer --tokens 64
"""
from __future__ import annotations

import argparse
import ctypes as C

import torch

from .. import ops
from ..ops import ActBuffer, TcWeight
from ..parallel import peer_ops
from .gemm import graph_time_us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--experts", type=int, default=32, help="experts held by this rank")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=1536)
    ap.add_argument("--kind", default="nvfp4")
    ap.add_argument("--layers", type=int, default=6, help="distinct weight sets cycled inside the timed graph (no L2 reuse)")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    T, E, H, I, k = a.tokens, a.experts, a.hidden, a.inter, 8
    rows = T * k
    g = torch.Generator(device=dev).manual_seed(0)
    i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
    idx = torch.stack([torch.randperm(E, device=dev, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    tn = ops.pick_tn(min(max(1, -(-rows // E) * 2), 128), swiglu=True)
    max_tiles = E + rows // tn + 1
    src, route, slot, cnt, off, tiles, nt, nr = i32(rows), i32(rows), i32(T, k), i32(E), i32(E), i32(max_tiles, 4), i32(1), i32(1)
    ops.route_pack(idx, src, slot, cnt, off, tiles, nt, nr, T, k, 0, E, tn, max_tiles, src_route=route)
    kind = ops.KIND_BY_NAME[a.kind]
    xs = ActBuffer.alloc(kind, rows, H, tn, dev)
    xs.data.random_(0, 256, generator=g)
    xs.sf.fill_(0x38 if kind == ops.KIND_NVFP4 else 120)
    h1q = ActBuffer.alloc(kind, rows, I, tn, dev)
    y2 = torch.zeros(rows, H, dtype=torch.bfloat16, device=dev)
    recv = [torch.zeros(rows, H, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    flags = torch.zeros(8, dtype=torch.int32, device=dev)
    ctl, done, st = i32(4), i32(4), i32(4)
    ctl[1] = 1
    W = [(TcWeight.random(E, I, H, kind, dev, seed=3 * l), TcWeight.random(E, I, H, kind, dev, seed=3 * l + 1),
          TcWeight.random(E, H, I, kind, dev, seed=3 * l + 2)) for l in range(a.layers)]
    recv_tbl = (C.c_void_p * 2)(recv[0].data_ptr(), recv[1].data_ptr())
    flag_tbl = (C.c_void_p * 2)(flags.data_ptr(), flags.data_ptr() + 4)

    def fc1(l):
        ops.tc_linear(W[l][0], xs, None, rows=rows, w_up=W[l][1], tiles=tiles, n_tiles=nt, max_tiles=max_tiles, status=st,
                      quant_out=h1q, inv_gs_out=W[l][2].inv_act_gs)

    def fused(l):
        fc1(l)
        ops.tc_linear(W[l][2], h1q, None, rows=rows, tiles=tiles, n_tiles=nt, max_tiles=max_tiles, status=st,
                      peer={"y": [recv[0].data_ptr(), recv[1].data_ptr()], "ld": H, "row_map": route,
                            "flags": [flags.data_ptr(), flags.data_ptr() + 4], "ctl": ctl, "done": done[0:1]})

    def unfused(l):
        fc1(l)
        ops.tc_linear(W[l][2], h1q, y2, rows=rows, tiles=tiles, n_tiles=nt, max_tiles=max_tiles, status=st)
        peer_ops.combine_push(y2, route, nr, recv_tbl, flag_tbl, ctl, done[1:2], H, 2, rows, 0)

    # same result either way
    fused(0)
    torch.cuda.synchronize()
    got = [r.clone() for r in recv]
    for r in recv:
        r.zero_()
    unfused(0)
    torch.cuda.synchronize()
    same = all(torch.equal(x, y) for x, y in zip(got, recv))
    t_f = graph_time_us([(lambda l=l: fused(l)) for l in range(a.layers)])
    t_u = graph_time_us([(lambda l=l: unfused(l)) for l in range(a.layers)])
    t_1 = graph_time_us([(lambda l=l: fc1(l)) for l in range(a.layers)])
    wbytes = W[0][2].nbytes
    print(f"tokens {T} rows {rows} experts {E} kind {a.kind}: FC1 {t_1:.1f} us; FC1 + FC2 with peer-store epilogue {t_f:.1f} us; "
          f"FC1 + FC2 + combine_push {t_u:.1f} us; identical output: {same}; status {st.tolist()} flags {flags[:2].tolist()}")
    print(f"FC2 part: fused {t_f - t_1:.1f} us ({wbytes / (t_f - t_1) / 1e3:.0f} GB/s of expert weights), unfused {t_u - t_1:.1f} us")

    # attention-rank side of the same hand-off: quantise T token rows once and scatter every (token, expert) row, its block
    # scales and the routing table into the owning expert rank's slab (two "ranks" here, both local), then raise their flags
    x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    row_bytes = H * 2 if kind == ops.KIND_BF16 else H // 2
    sf_ld = -(-H // 256) * (256 // (16 if kind == ops.KIND_NVFP4 else 32))
    slab_q = [torch.zeros(rows, row_bytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    slab_sf = [torch.zeros(rows, sf_ld, dtype=torch.uint8, device=dev) for _ in range(2)]
    idx_dst = [i32(T, k) for _ in range(2)]
    tbl = lambda ts: (C.c_void_p * 2)(ts[0].data_ptr(), ts[1].data_ptr())
    q_tbl, sf_tbl, i_tbl = tbl(slab_q), tbl(slab_sf), tbl(idx_dst)
    f_tbl = (C.c_void_p * 2)(flags.data_ptr() + 8, flags.data_ptr() + 12)
    inv_gs = torch.tensor([64.0], device=dev)

    def dispatch():
        peer_ops.dispatch_push(x, idx, slot, off, q_tbl, sf_tbl, i_tbl, f_tbl, inv_gs, ctl, done[2:3], 0, T, H, k, E, 2, kind, sf_ld, rows, 0, st)

    t_d = graph_time_us([dispatch for _ in range(8)])
    moved = rows * (row_bytes + (H // (16 if kind == ops.KIND_NVFP4 else 32) if kind != ops.KIND_BF16 else 0))
    print(f"dispatch_push: {t_d:.1f} us for {rows} rows ({moved / 1e6:.2f} MB stored, {moved / t_d / 1e3:.0f} GB/s); status {st.tolist()}")


if __name__ == "__main__":
    main()
