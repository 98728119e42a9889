"""Attention/FFN disaggregation inside one NVSwitch node.

Ranks split into an attention group (TP over heads; holds embeddings, attention, router, shared expert, LM head and
the KV cache) and an expert group (expert-parallel routed experts).  Per MoE layer:

  attention rank:  ... -> router top-k -> route pack (replicated, deterministic) -> DISPATCH: quantise my half of the
                   tokens and store the rows straight into the owning expert ranks' slabs over NVLink (+ flag)
                   -> shared expert meanwhile -> wait COMBINE flags -> ordered weighted top-k sum + shared + residual
  expert rank:     wait DISPATCH flags -> route pack of its own expert range on the received routing table ->
                   grouped FC1 (SwiGLU) -> quant -> grouped FC2 (tcgen05, TMA from the LOCAL slab) ->
                   COMBINE: store every output row into [token][slot] of both attention ranks (+ flag)
  attention TP2:   wo partial -> push to the peer + flag -> wait -> add in rank order (bit-identical on both ranks)

With several data-parallel attention groups (`Deployment.attn_groups`) every group serves its own sequences and owns a
slab / routing-table / flag lane on each expert rank; an expert rank runs the lanes one after the other per layer, so
it computes group A's experts while group B is in attention (the groups fall out of phase after the first layer).

`comm="p2p"` uses the peer-memory kernels of `csrc/peer.cu`; `comm="nccl"` is the baseline that only calls NCCL
(broadcast activations + routes, all-reduce expert partial sums, all-reduce attention partials).

Reference: the coordinator/Spark split (families/deepseek_v4/engine.rs:1036-1191, 2047-2133), TP2 head split
(engine.rs:1524-1552), ordered combine (native/shared/include/cuteafd_experts.h:136-183).
"""
from __future__ import annotations

import dataclasses
import os
import time

import torch

from .. import ops
from ..config import Deployment, ModelSpec, default_deployment
from ..engine.engine import Engine, Lane, StepShape, PAGE
from ..models.weights import DeviceWeights, LayerWeights
from ..ops import ActBuffer, KIND_BF16, KIND_NVFP4, pick_tn
from . import peer_ops
from .symm import SymmetricBlock

PH_DISPATCH, PH_COMBINE, PH_TP = 0, 1, 2
# GEMM epilogues can store straight into peer memory (output projection -> TP partner, expert FC2 -> attention ranks)
# and publish the flags themselves: CUTEAFD_FUSED_PEER=1; the default keeps the separate push kernels.
FUSED_PEER = os.environ.get("CUTEAFD_FUSED_PEER", "0") == "1"


def local_attention_spec(spec: ModelSpec, tp: int) -> ModelSpec:
    a = spec.attn
    if a.n_heads % tp or a.n_kv_heads % tp:
        raise ValueError(f"heads ({a.n_heads}/{a.n_kv_heads}) do not split over tp={tp}")
    return spec.replace(attn=dataclasses.replace(a, n_heads=a.n_heads // tp, n_kv_heads=a.n_kv_heads // tp))


def make_block(spec: ModelSpec, dep: Deployment, t_max: int, expert_kind: int, rank: int, device, group) -> SymmetricBlock:
    """Symmetric regions (same layout on every rank; each role uses its part)."""
    H, k, G = spec.hidden, spec.moe.top_k, dep.attn_groups
    rows = t_max * k
    row_bytes = H * 2 if expert_kind == KIND_BF16 else H // 2
    vec = 16 if expert_kind == KIND_NVFP4 else 32
    sf_ld = -(-H // 256) * (256 // vec)
    regions = {     # the expert-side regions hold one lane per attention group
        "slab_q": G * rows * row_bytes, "slab_sf": G * rows * sf_ld, "idx": G * rows * 4,
        "y_recv": rows * H * 2, "tp_recv": 2 * t_max * H * 2,
        "flags": 3 * spec.n_layers * 8 * 4,
    }
    return SymmetricBlock(regions, device, group, rank, dep.world)


def flag_offset(spec: ModelSpec, phase: int, layer: int, src: int) -> int:
    return ((phase * spec.n_layers + layer) * 8 + src) * 4


class AttnRankEngine(Engine):
    """Engine of one attention rank: local heads, replicated residual stream, routed experts remote."""

    def __init__(self, spec: ModelSpec, dep: Deployment, rank: int, device, *, t_max: int, n_pages: int, max_seqs: int,
                 max_pages_per_seq: int, comm: str, block: SymmetricBlock | None, expert_kind: int, act_gs: float = 1.0 / 64, seed: int = 1):
        self.full_spec, self.dep, self.rank, self.comm, self.block = spec, dep, rank, comm, block
        self.tp, self.tp_rank = dep.tp, dep.attn_ranks.index(rank) % dep.tp
        self.group = dep.group_of(rank)
        self.group_ranks = dep.group_ranks(self.group)
        self.flag_src = self.group * dep.tp + self.tp_rank       # this rank's slot among the dispatch flags
        lw = self._make_weights(spec, device, seed, act_gs)
        super().__init__(lw, n_pages=n_pages, max_seqs=max_seqs, max_pages_per_seq=max_pages_per_seq, device=device)
        self.remote_kind = expert_kind
        self.t_max = t_max
        m, H = spec.moe, spec.hidden
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=device)
        self.ctl = torch.zeros(4, dtype=torch.int32, device=device)
        self.done = torch.zeros(8, dtype=torch.int32, device=device)
        self.inv_gs = torch.tensor([1.0 / act_gs], dtype=torch.float32, device=device)
        rows = t_max * m.top_k
        self.router_logits = torch.zeros(t_max, m.n_experts, dtype=torch.float32, device=device)
        self.idx, self.wts = i32(t_max, m.top_k), torch.zeros(t_max, m.top_k, dtype=torch.float32, device=device)
        self.src_token, self.slot_row = i32(rows), i32(t_max, m.top_k)
        self.counts, self.offsets = i32(m.n_experts), i32(m.n_experts)
        self.tiles, self.n_tiles, self.n_rows = i32(m.n_experts + rows + 1, 4), i32(1), i32(1)
        self.identity_rows = torch.arange(rows, dtype=torch.int32, device=device).view(t_max, m.top_k).contiguous()
        self.part = torch.zeros(t_max, H, dtype=torch.bfloat16, device=device)
        self.e_local = m.n_experts          # the dispatch kernel derives each rank's expert range from the total
        if block is not None:
            vec = 16 if expert_kind == KIND_NVFP4 else 32
            self.sf_ld = -(-H // 256) * (256 // vec)
            row_bytes = H * 2 if expert_kind == KIND_BF16 else H // 2
            g = self.group                                       # my group's lane on every expert rank
            self.slab_q_tbl = block.ptr_table(dep.expert_ranks, "slab_q", g * rows * row_bytes)
            self.slab_sf_tbl = block.ptr_table(dep.expert_ranks, "slab_sf", g * rows * self.sf_ld)
            self.idx_tbl = block.ptr_table(dep.expert_ranks, "idx", g * rows * 4)
            self.y_recv = block.local("y_recv", torch.bfloat16, (rows, H))
            self.tp_recv = block.local("tp_recv", torch.bfloat16, (2, t_max, H))

    def _make_weights(self, spec, device, seed, act_gs):
        """This rank's share: attention heads split over the TP group, router/shared/dense replicated, no routed experts.
        With bf16 projections the shard is cut out of the full-model weights of the same seed (so the split reproduces
        the single-GPU model exactly); block-scaled projections are generated per shard (synthetic benchmarks)."""
        if self.tp == 1 or spec.quant.dense != "bf16":
            return DeviceWeights.random(local_attention_spec(spec, self.tp), device, seed=seed, experts_range=(0, 0), act_gs=act_gs)
        from ..ops import TcWeight, encode_tmap
        dw = DeviceWeights.random(spec, device, seed=seed, experts_range=(0, 0), act_gs=act_gs)
        a, r, tp = spec.attn, self.tp_rank, self.tp
        hq, hkv, D = a.n_heads // tp, a.n_kv_heads // tp, a.head_dim
        nq, nk = a.n_heads * D, a.n_kv_heads * D
        for lw in dw.layers:
            w = lw.wqkv.data[0]
            rows = torch.cat([w[r * hq * D:(r + 1) * hq * D], w[nq + r * hkv * D:nq + (r + 1) * hkv * D],
                              w[nq + nk + r * hkv * D:nq + nk + (r + 1) * hkv * D]]).unsqueeze(0).contiguous()
            lw.wqkv = TcWeight(KIND_BF16, 1, rows.shape[1], rows.shape[2], rows, encode_tmap(rows, 128))
            cols = lw.wo.data[:, :, r * hq * D:(r + 1) * hq * D].contiguous()
            lw.wo = TcWeight(KIND_BF16, 1, cols.shape[1], cols.shape[2], cols, encode_tmap(cols, 128))
        dw.spec = local_attention_spec(spec, tp)
        return dw

    # -- output projection with the TP all-reduce
    def _attn_out(self, li, lw, oq, L, T):
        if self.tp == 1:
            return super()._attn_out(li, lw, oq, L, T)
        if self.comm == "p2p" and FUSED_PEER and lw.wo.kind != ops.KIND_FP8B:
            # the projection's epilogue writes my partial sum locally AND into the partner's landing buffer, then raises
            # its flag: GEMM -> exchange in one kernel; the wait + ordered add follows
            H, peer, buf = self.full_spec.hidden, self.group_ranks[1 - self.tp_rank], li & 1
            splits = self._splits(lw.wo.N, lw.wo.K, T, oq.tn, lw.wo.kind)
            ops.tc_linear(lw.wo, oq, self.part, rows=T, splits=splits, status=self.status,
                          peer={"y": [self.block.peer_ptr(peer, "tp_recv", buf * self.t_max * H * 2)], "ld": H, "row_map": None,
                                "flags": [self.block.peer_ptr(peer, "flags", flag_offset(self.full_spec, PH_TP, li, self.tp_rank))],
                                "ctl": self.ctl, "done": self.done[2:3]})
            peer_ops.wait_add(self.part, self.tp_recv[buf], L.x, L.x, T * H, self.tp_rank,
                              self.block.peer_ptr(self.rank, "flags", flag_offset(self.full_spec, PH_TP, li, 1 - self.tp_rank)),
                              self.ctl, 0, self.status)
            self.launches_per_step += 2
            return
        self._dense(lw.wo, oq, self.part, T)              # partial sum over my heads, then the TP exchange
        self._tp_allreduce(li, self.part, L.x, T)

    def _tp_allreduce(self, li, part, x, T):
        """x += part(rank 0) + part(rank 1), identical bits on both ranks."""
        H = self.full_spec.hidden
        if self.comm == "nccl":
            import torch.distributed as dist
            dist.all_reduce(part[:T], group=self.tp_group)
            x[:T] += part[:T]
            return
        peer = self.group_ranks[1 - self.tp_rank]
        buf = li & 1
        nbytes = T * H * 2
        peer_ops.push_bytes(part, self.block.peer_ptr(peer, "tp_recv", buf * self.t_max * H * 2), nbytes,
                            self.block.peer_ptr(peer, "flags", flag_offset(self.full_spec, PH_TP, li, self.tp_rank)),
                            self.ctl, 0, self.done[0:1])
        peer_ops.wait_add(part, self.tp_recv[buf], x, x, T * H, self.tp_rank,
                          self.block.peer_ptr(self.rank, "flags", flag_offset(self.full_spec, PH_TP, li, 1 - self.tp_rank)),
                          self.ctl, 0, self.status)
        self.launches_per_step += 2

    # -- FFN: router local, routed experts remote
    def _moe_layer_at(self, li, lw, L, T):
        spec, m, dep = self.full_spec, self.full_spec.moe, self.dep
        ops.add_rmsnorm(L.x, None, lw.ffn_norm, L.xn, spec.rms_eps, rows=T)
        if T <= 64 and lw.router.kind == KIND_BF16 and lw.router.G == 1 and L.xn.stride(0) == lw.router.K \
                and os.environ.get("CUTEAFD_ROUTER_GEMM", "0") != "1":
            ops.router_logits(L.xn, lw.router, self.router_logits, T)      # same kernel as the single-GPU engine (token-exact layouts)
            self.launches_per_step += 1
        else:
            self._dense(lw.router, L.xn_act, self.router_logits, T)
        self.launches_per_step += 2
        shared = None
        if self.comm == "nccl":
            ops.router_select(self.router_logits, lw.router_bias, self.idx, self.wts, T, m.top_k, m.scoring, m.normalize, m.route_scale,
                              m.n_group, m.topk_group)
            return self._moe_nccl(li, lw, L, T)
        if T * m.top_k <= 1024 and m.n_experts <= 512:
            ops.router_select_pack(self.router_logits, lw.router_bias, self.idx, self.wts, T, m.top_k, m.scoring, m.normalize, m.route_scale,
                                   m.n_group, m.topk_group, self.src_token, self.slot_row, self.counts, self.offsets, self.tiles,
                                   self.n_tiles, self.n_rows, 0, m.n_experts, 1 << 20, self.tiles.shape[0])
        else:
            ops.router_select(self.router_logits, lw.router_bias, self.idx, self.wts, T, m.top_k, m.scoring, m.normalize, m.route_scale,
                              m.n_group, m.topk_group)
            ops.route_pack(self.idx, self.src_token, self.slot_row, self.counts, self.offsets, self.tiles, self.n_tiles, self.n_rows,
                           T, m.top_k, 0, m.n_experts, 1 << 20, self.tiles.shape[0])
        # my share of the tokens (the other attention rank sends the rest; both hold identical activations)
        per = -(-T // self.tp)
        t0, t1 = min(T, self.tp_rank * per), min(T, (self.tp_rank + 1) * per)
        flag_tbl = self.block.ptr_table(dep.expert_ranks, "flags", flag_offset(spec, PH_DISPATCH, li, self.flag_src))
        peer_ops.dispatch_push(L.xn, self.idx, self.slot_row, self.offsets, self.slab_q_tbl, self.slab_sf_tbl, self.idx_tbl, flag_tbl,
                               self.inv_gs, self.ctl, self.done[1:2], t0, t1, spec.hidden, m.top_k, self.e_local, dep.ep,
                               self.remote_kind, self.sf_ld, self.t_max * m.top_k, 0, self.status)
        self._keep.append(flag_tbl)
        if lw.ws_gate is not None:
            self._ffn(lw, L, T, L.shared, None)
            shared = L.shared
        peer_ops.arm_flag_wait(self.block.peer_ptr(self.rank, "flags", flag_offset(spec, PH_COMBINE, li, 0)), dep.ep, 1, self.ctl, self.status)
        self._combine(self.y_recv, self.identity_rows, self.wts, shared, L, T, m.top_k)
        self.launches_per_step += 3

    def _moe_nccl(self, li, lw, L, T):
        import torch.distributed as dist
        if self.dep.attn_groups > 1:
            raise NotImplementedError("the NCCL-only baseline runs one attention group")
        m, H = self.full_spec.moe, self.full_spec.hidden
        src = self.dep.attn_ranks[0]
        dist.broadcast(L.xn[:T], src)
        dist.broadcast(self.idx[:T], src)
        dist.broadcast(self.wts[:T], src)
        acc = torch.zeros(T, H, dtype=torch.bfloat16, device=self.device)
        dist.all_reduce(acc)                      # expert ranks contribute their weighted partial sums
        if lw.ws_gate is not None:
            self._ffn(lw, L, T, L.shared, None)
            acc += L.shared[:T]
        L.x[:T] += acc

    def forward(self, sh: StepShape):
        self._keep = []          # ctypes tables referenced by launches of this step
        self._layer_cursor = 0
        if self.block is not None and self.comm == "p2p":
            peer_ops.step_begin(self.ctl)
        return super().forward(sh)

    def _moe_layer(self, lw, L, T):
        li = self._layer_cursor
        self._layer_cursor += 1
        if lw.router is None:
            return super()._moe_layer(lw, L, T)
        return self._moe_layer_at(li, lw, L, T)


class MlaAttnRankEngine(AttnRankEngine):
    """Attention rank of an MLA model (DeepSeek-V3 shape): local heads, replicated latent cache."""

    def _make_weights(self, spec, device, seed, act_gs):
        from ..engine.mla import mla_weights_random
        return mla_weights_random(spec, device, heads_local=spec.attn.n_heads // self.tp, experts_range=(0, 0), act_gs=act_gs, seed=seed)


def _bind_mla(cls):
    """MLA attention methods come from MlaEngine; everything else (TP exchange, remote experts) from AttnRankEngine."""
    from ..engine.mla import MlaEngine
    for name in ("_alloc_attention_state", "_mla_buf", "_head_tiles", "attn_splits_for", "_attention_layer", "_act", "_attn_in_gs"):
        setattr(cls, name, getattr(MlaEngine, name))
    return cls


_bind_mla(MlaAttnRankEngine)


class ExpertRankWorker:
    """One expert-parallel rank: receives dispatched rows, runs its experts, returns rows to the attention ranks."""

    def __init__(self, spec: ModelSpec, dep: Deployment, rank: int, device, *, t_max: int, comm: str, block: SymmetricBlock | None,
                 act_gs: float = 1.0 / 64, seed: int = 1):
        self.spec, self.dep, self.rank, self.comm, self.block, self.device = spec, dep, rank, comm, block, device
        self.ep_rank = dep.expert_ranks.index(rank)
        m = spec.moe
        self.e_lo, self.e_hi = (self.ep_rank * m.n_experts) // dep.ep, ((self.ep_rank + 1) * m.n_experts) // dep.ep
        self.e_local = self.e_hi - self.e_lo
        self.weights = DeviceWeights.random(spec, device, seed=seed, experts_range=(self.e_lo, self.e_hi), with_attention=False, act_gs=act_gs)
        self.kind = next(l.w_gate.kind for l in self.weights.layers if l.w_gate is not None)
        self.t_max, H, k = t_max, spec.hidden, m.top_k
        rows = t_max * k
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=device)
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.ctl, self.done = i32(4), i32(8)
        self.tn = pick_tn(min(max(1, -(-rows // m.n_experts) * 2), 32), swiglu=True)      # <= 32: see Lane.tn_g
        self.max_tiles = self.e_local + rows // self.tn + 1
        self.src_token, self.src_route, self.slot_row = i32(rows), i32(rows), i32(t_max, k)
        self.counts, self.offsets = i32(self.e_local), i32(self.e_local)
        self.tiles, self.n_tiles, self.n_rows = i32(self.max_tiles, 4), i32(1), i32(1)
        self.h1 = torch.zeros(rows, m.intermediate, dtype=torch.bfloat16, device=device)
        self.h1_q = (ActBuffer.alloc(self.kind, rows, m.intermediate, self.tn, device) if self.kind != KIND_BF16
                     else ActBuffer.wrap_bf16(self.h1, self.tn))
        self.y2 = torch.zeros(rows, H, dtype=torch.bfloat16, device=device)
        self.launches_per_step = 0
        G = dep.attn_groups
        if block is not None:
            # one lane (slab, scales, routing table, destination ranks) per attention group
            self.xs_g, self.idx_g, self.recv_tbl_g = [], [], []
            if self.kind == KIND_BF16:
                data_all = block.local("slab_q", torch.bfloat16, (G, rows, H))
                sf_all = None
            else:
                vec = 16 if self.kind == KIND_NVFP4 else 32
                data_all = block.local("slab_q", torch.uint8, (G, rows, H // 2))
                sf_all = block.local("slab_sf", torch.uint8, (G, rows, -(-H // 256) * (256 // vec)))
            idx_all = block.local("idx", torch.int32, (G, t_max, k))
            for g in range(G):
                self.xs_g.append(ActBuffer(self.kind, rows, H, self.tn, data_all[g], ops.encode_tmap(data_all[g], self.tn),
                                           sf_all[g] if sf_all is not None else None))
                self.idx_g.append(idx_all[g])
                self.recv_tbl_g.append(block.ptr_table(dep.group_ranks(g), "y_recv"))
            self.xs, self.idx = self.xs_g[0], self.idx_g[0]
        else:
            self.xs = ActBuffer.alloc(self.kind, rows, H, self.tn, device)
            self.idx = i32(t_max, k)
        self._keep = []

    def layer(self, li: int, T: int):
        spec, m, dep = self.spec, self.spec.moe, self.dep
        lw = self.weights.layer(li)
        if lw.w_gate is None:
            return
        rows = T * m.top_k
        if self.comm == "nccl":
            return self._layer_nccl(li, lw, T)
        for g in range(dep.attn_groups):
            xs, idx = self.xs_g[g], self.idx_g[g]
            peer_ops.arm_flag_wait(self.block.peer_ptr(self.rank, "flags", flag_offset(spec, PH_DISPATCH, li, g * dep.tp)), dep.tp, 1,
                                   self.ctl, self.status)       # the pack kernel waits for this group's dispatch itself
            ops.route_pack(idx, self.src_token, self.slot_row, self.counts, self.offsets, self.tiles, self.n_tiles, self.n_rows,
                           T, m.top_k, self.e_lo, self.e_hi, self.tn, self.max_tiles, src_route=self.src_route)
            if self.kind != KIND_BF16 and m.intermediate % 32 == 0:      # FC1 writes its output quantised for FC2
                ops.tc_linear(lw.w_gate, xs, None, rows=rows, w_up=lw.w_up, tiles=self.tiles, n_tiles=self.n_tiles,
                              max_tiles=self.max_tiles, status=self.status, quant_out=self.h1_q, inv_gs_out=lw.w_down.inv_act_gs)
            else:
                ops.tc_linear(lw.w_gate, xs, self.h1, rows=rows, w_up=lw.w_up, tiles=self.tiles, n_tiles=self.n_tiles,
                              max_tiles=self.max_tiles, status=self.status)
                if self.kind != KIND_BF16:
                    ops.quant_fp4_rows(self.h1, self.h1_q, n_rows_dev=self.n_rows, rows=rows, inv_gs=lw.w_down.inv_act_gs)
            if FUSED_PEER:
                # FC2's epilogue stores every output row straight into [token][slot] of the group's attention ranks and
                # the last CTA raises their flags: grouped GEMM -> combine transfer in one kernel
                ranks = dep.group_ranks(g)
                ops.tc_linear(lw.w_down, self.h1_q, None, rows=rows, tiles=self.tiles, n_tiles=self.n_tiles, max_tiles=self.max_tiles,
                              status=self.status,
                              peer={"y": [self.block.peer_ptr(r, "y_recv") for r in ranks], "ld": spec.hidden, "row_map": self.src_route,
                                    "flags": [self.block.peer_ptr(r, "flags", flag_offset(spec, PH_COMBINE, li, self.ep_rank)) for r in ranks],
                                    "ctl": self.ctl, "done": self.done[0:1]})
                self.launches_per_step += 3
                continue
            ops.tc_linear(lw.w_down, self.h1_q, self.y2, rows=rows, tiles=self.tiles, n_tiles=self.n_tiles, max_tiles=self.max_tiles,
                          status=self.status)
            flag_tbl = self.block.ptr_table(dep.group_ranks(g), "flags", flag_offset(spec, PH_COMBINE, li, self.ep_rank))
            self._keep.append(flag_tbl)
            peer_ops.combine_push(self.y2, self.src_route, self.n_rows, self.recv_tbl_g[g], flag_tbl, self.ctl, self.done[0:1], spec.hidden,
                                  dep.tp, rows, 0)
            self.launches_per_step += 4

    def _layer_nccl(self, li, lw, T):
        import torch.distributed as dist
        m, H = self.spec.moe, self.spec.hidden
        src = self.dep.attn_ranks[0]
        xn = torch.empty(T, H, dtype=torch.bfloat16, device=self.device)
        idx = torch.empty(T, m.top_k, dtype=torch.int32, device=self.device)
        wts = torch.empty(T, m.top_k, dtype=torch.float32, device=self.device)
        dist.broadcast(xn, src); dist.broadcast(idx, src); dist.broadcast(wts, src)
        rows = T * m.top_k
        ops.route_pack(idx, self.src_token, self.slot_row, self.counts, self.offsets, self.tiles, self.n_tiles, self.n_rows,
                       T, m.top_k, self.e_lo, self.e_hi, self.tn, self.max_tiles)
        if self.kind == KIND_BF16:
            ops.gather_rows(xn, self.src_token, self.n_rows, self.xs.data, rows)
        else:
            ops.quant_fp4_rows(xn, self.xs, src_rows=self.src_token, n_rows_dev=self.n_rows, rows=rows, inv_gs=lw.w_gate.inv_act_gs)
        ops.tc_linear(lw.w_gate, self.xs, self.h1, rows=rows, w_up=lw.w_up, tiles=self.tiles, n_tiles=self.n_tiles,
                      max_tiles=self.max_tiles, status=self.status)
        if self.kind != KIND_BF16:
            ops.quant_fp4_rows(self.h1, self.h1_q, n_rows_dev=self.n_rows, rows=rows, inv_gs=lw.w_down.inv_act_gs)
        ops.tc_linear(lw.w_down, self.h1_q, self.y2, rows=rows, tiles=self.tiles, n_tiles=self.n_tiles, max_tiles=self.max_tiles,
                      status=self.status)
        acc = torch.zeros(T, H, dtype=torch.bfloat16, device=self.device)
        ops.moe_combine(self.y2, self.slot_row, wts, None, None, acc, T, m.top_k)
        dist.all_reduce(acc)

    def step(self, T: int):
        self._keep = []
        self.launches_per_step = 0
        if self.comm == "p2p":
            peer_ops.step_begin(self.ctl)
        for li in range(self.spec.n_layers):
            self.layer(li, T)

    def run(self, T: int, graphs: dict, use_graph: bool = True):
        if not use_graph or self.comm != "p2p":
            return self.step(T)
        if T not in graphs:
            raise RuntimeError("expert graph for this step size was not captured")
        graphs[T].replay()


def capture_expert_graph(worker: ExpertRankWorker, T: int) -> torch.cuda.CUDAGraph:
    """Capture one expert-rank step.  Waiting kernels are part of the graph, so the capture itself must not run
    them: capture records launches without executing."""
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        worker.step(T)
    return g
