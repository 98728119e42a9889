"""DeepSeek-V3-shape engine: multi-head latent attention in absorbed form on top of the generic engine.

Per layer: RMSNorm -> q_a (H -> q_lora) -> RMSNorm -> q_b -> split {q_nope head-major, q_rope + RoPE}
           -> grouped GEMM per head  q_lat = q_nope W_UK   (W_UK folded into the query, so keys stay latent)
           kv_a (H -> 512 + 64) -> RMSNorm(c_kv) | RoPE(k_rope) -> paged latent cache row (576 bf16 per token)
           -> `mla_attention` (tcgen05; scores over 576, values = the 512-wide latent, two V halves per tile)
           -> grouped GEMM per head  o = o_lat W_UV^T  -> token-major -> wo (+ residual)
The FFN half (dense first layers, then router + routed + shared experts) is the generic engine's.
The latent cache is replicated on the attention ranks of a TP group (heads are split, the latent is shared), as in
the reference's head-split mode (families/deepseek_v4/engine.rs:97-119).
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from .. import ops
from ..config import ModelSpec
from ..models.weights import DeviceWeights, LayerWeights, _dense_kind, _expert_kind
from ..ops import ActBuffer, KIND_BF16, TcWeight
from ..ops.native import call, ptr, stream
from .engine import Engine, Lane, PAGE, StepShape

DQK, DV = 576, 512


@dataclass
class MlaWeights:
    """Attention weights of one MLA layer (dense kind of the model; the two absorb matrices stay bf16)."""
    wq_a: TcWeight | None
    q_a_norm: torch.Tensor | None
    wq_b: TcWeight              # [Hl * 192, q_lora]  (or [Hl * 192, H] without q compression)
    wkv_a: TcWeight             # [576, H]
    kv_a_norm: torch.Tensor
    w_uk_t: TcWeight            # G = Hl, [512, 128]: q_lat = q_nope @ W_UK
    w_uv: TcWeight              # G = Hl, [128, 512]: o = o_lat @ W_UV^T
    w_kvb: TcWeight | None = None   # [Hl * 256, 512]: per head 128 key rows then 128 value rows (prefill expands the latent cache with it)
    # sparse-attention indexer (AttentionSpec.index_topk > 0): index queries from the compressed query (or the hidden state),
    # index keys and head weights (already scaled by index_heads ** -0.5) from the hidden state
    wq_idx: TcWeight | None = None  # [Hi * Di, q_lora | H]
    wk_idx: TcWeight | None = None  # [Di, H]
    w_idx: TcWeight | None = None   # [Hi, H]

    def ensure_kvb(self) -> TcWeight:
        """The kv_b projection in its checkpoint orientation, rebuilt from the two absorb matrices on first use (prefill only;
        33 MB per layer at 128 heads).  Needs 128-wide key and value heads, the shape the prefill kernel is written for."""
        if self.w_kvb is None:
            uk, uv = self.w_uk_t.data, self.w_uv.data            # [Hl, 512, 128], [Hl, 128, 512]
            if uk.shape[2] != 128 or uv.shape[1] != 128:
                raise ValueError("the MLA prefill path needs qk_nope_head_dim = v_head_dim = 128")
            data = torch.cat([uk.transpose(1, 2), uv], dim=1).reshape(1, uk.shape[0] * 256, uk.shape[1]).contiguous()
            self.w_kvb = TcWeight(KIND_BF16, 1, data.shape[1], data.shape[2], data, ops.encode_tmap(data, 128))
        return self.w_kvb


def _mla_from_masters(spec: ModelSpec, lw: dict, device, dk: str, act_gs: float) -> MlaWeights:
    a = spec.attn
    nope, rope, dv, H = a.qk_nope_head_dim, a.qk_rope_head_dim, a.v_head_dim, a.n_heads
    kvb = lw["wkv_b"].reshape(H, nope + dv, a.kv_lora_rank)
    w_uk_t = kvb[:, :nope].transpose(1, 2).contiguous()          # [H, 512, 128]
    w_uv = kvb[:, nope:].contiguous()                            # [H, 128, 512]
    f32 = lambda t: t.float().to(device).contiguous()
    return MlaWeights(
        wq_a=TcWeight.from_master(lw["wq_a"], dk, device, act_gs) if "wq_a" in lw else None,
        q_a_norm=f32(lw["q_a_norm"]) if "q_a_norm" in lw else None,
        wq_b=TcWeight.from_master(lw["wq_b"] if "wq_b" in lw else lw["wq"], dk, device, act_gs),
        wkv_a=TcWeight.from_master(lw["wkv_a"], dk, device, act_gs), kv_a_norm=f32(lw["kv_a_norm"]),
        w_uk_t=TcWeight.from_master(w_uk_t, "bf16", device), w_uv=TcWeight.from_master(w_uv, "bf16", device),
        wq_idx=TcWeight.from_master(lw["wq_idx"], dk, device, act_gs) if "wq_idx" in lw else None,
        wk_idx=TcWeight.from_master(lw["wk_idx"], dk, device, act_gs) if "wk_idx" in lw else None,
        w_idx=TcWeight.from_master(lw["w_idx"] * (a.index_heads ** -0.5), dk, device, act_gs) if "w_idx" in lw else None)


def mla_weights_from_masters(spec: ModelSpec, masters: dict, device, act_gs: float = 1.0 / 64) -> DeviceWeights:
    """DeviceWeights whose layers carry `.mla` (MlaWeights) instead of a fused QKV projection."""
    dk, ek = _dense_kind(spec), _expert_kind(spec)
    f32 = lambda t: t.float().to(device).contiguous()
    dw = DeviceWeights(spec=spec, embed=masters["embed"].to(torch.bfloat16).to(device).contiguous(), final_norm=f32(masters["final_norm"]),
                       lm_head=TcWeight.from_master(masters["lm_head"], "bf16", device), act_gs=act_gs)
    def layer_from(lw: dict) -> LayerWeights:
        out = LayerWeights(attn_norm=f32(lw["attn_norm"]), ffn_norm=f32(lw["ffn_norm"]), wqkv=None,
                           wo=TcWeight.from_master(lw["wo"], dk, device, act_gs))
        out.mla = _mla_from_masters(spec, lw, device, dk, act_gs)
        if "hc_attn_fn" in lw:         # hyper-connections (the V4 line pairs them with latent attention)
            out.hc_attn = tuple(f32(lw[f"hc_attn_{k}"]) for k in ("fn", "scale", "base"))
            out.hc_ffn = tuple(f32(lw[f"hc_ffn_{k}"]) for k in ("fn", "scale", "base"))
        if "router" in lw:
            out.router = TcWeight.from_master(lw["router"], "bf16", device)
            if "router_bias" in lw:
                out.router_bias = f32(lw["router_bias"])
            if "w_gate" in lw:
                out.w_gate, out.w_up, out.w_down = (TcWeight.from_master(lw[k], ek, device, act_gs) for k in ("w_gate", "w_up", "w_down"))
            if "ws_gate" in lw:
                out.ws_gate, out.ws_up, out.ws_down = (TcWeight.from_master(lw[k], dk, device, act_gs) for k in ("ws_gate", "ws_up", "ws_down"))
        else:
            out.ws_gate, out.ws_up, out.ws_down = (TcWeight.from_master(lw[k], dk, device, act_gs) for k in ("wd_gate", "wd_up", "wd_down"))
        return out

    dw.layers = [layer_from(lw) for lw in masters["layers"]]
    dw.layer_map = list(range(spec.n_layers))
    if "hc_head_fn" in masters:
        dw.hc_head = tuple(f32(masters[f"hc_head_{k}"]) for k in ("fn", "scale", "base"))
    for mw in masters.get("mtp", []):
        dw.mtp.append((f32(mw["enorm"]), f32(mw["hnorm"]), TcWeight.from_master(mw["eh_proj"], "bf16", device), layer_from(mw["layer"]),
                       f32(mw["norm"])))
    return dw


def mla_weights_random(spec: ModelSpec, device, *, heads_local: int | None = None, experts_range: tuple | None = None,
                       distinct_moe_layers: int = 0, act_gs: float = 1.0 / 64, seed: int = 1) -> DeviceWeights:
    """Random weights directly in storage format.  `heads_local` < n_heads builds one TP shard of the attention;
    `distinct_moe_layers` > 0 cycles that many distinct MoE layer sets (every layer still runs at full size)."""
    a, m, h = spec.attn, spec.moe, spec.hidden
    dk, ek = _dense_kind(spec), _expert_kind(spec)
    Hl = heads_local or a.n_heads
    ones = lambda n: torch.ones(n, dtype=torch.float32, device=device)
    e_lo, e_hi = experts_range if experts_range is not None else (0, m.n_experts)
    gen = torch.Generator(device=device).manual_seed(seed)
    dw = DeviceWeights(spec=spec, embed=torch.empty(spec.vocab, h, dtype=torch.bfloat16, device=device).normal_(0, spec.init_std, generator=gen),
                       final_norm=ones(h), lm_head=TcWeight.random(1, spec.vocab, h, "bf16", device, spec.init_std, act_gs, seed + 7), act_gs=act_gs)

    def make(i: int) -> LayerWeights:
        s = seed * 1000 + i * 32
        R = lambda G, N, K, kind, j: TcWeight.random(G, N, K, kind, device, spec.init_std, act_gs, s + j)
        out = LayerWeights(attn_norm=ones(h), ffn_norm=ones(h), wqkv=None, wo=R(1, h, Hl * a.v_head_dim, dk, 1))
        qk = a.qk_nope_head_dim + a.qk_rope_head_dim
        out.mla = MlaWeights(wq_a=R(1, a.q_lora_rank, h, dk, 2) if a.q_lora_rank else None, q_a_norm=ones(a.q_lora_rank) if a.q_lora_rank else None,
                             wq_b=R(1, Hl * qk, a.q_lora_rank or h, dk, 3), wkv_a=R(1, a.kv_lora_rank + a.qk_rope_head_dim, h, dk, 4),
                             kv_a_norm=ones(a.kv_lora_rank), w_uk_t=R(Hl, a.kv_lora_rank, a.qk_nope_head_dim, "bf16", 5),
                             w_uv=R(Hl, a.v_head_dim, a.kv_lora_rank, "bf16", 6))
        if a.index_topk:
            out.mla.wq_idx = R(1, a.index_heads * a.index_dim, a.q_lora_rank or h, dk, 14)
            out.mla.wk_idx, out.mla.w_idx = R(1, a.index_dim, h, dk, 15), R(1, a.index_heads, h, dk, 16)
        if spec.is_moe_layer(i):
            out.router = R(1, m.n_experts, h, "bf16", 7)
            if m.use_bias:
                out.router_bias = torch.zeros(m.n_experts, dtype=torch.float32, device=device)
            if e_hi > e_lo:
                RE = lambda N, K, j: TcWeight.random(m.n_experts, N, K, ek, device, spec.init_std, act_gs, s + j, groups=(e_lo, e_hi))
                out.w_gate, out.w_up, out.w_down = RE(m.intermediate, h, 8), RE(m.intermediate, h, 9), RE(h, m.intermediate, 10)
            if m.shared_inter:
                out.ws_gate, out.ws_up, out.ws_down = R(1, m.shared_inter, h, dk, 11), R(1, m.shared_inter, h, dk, 12), R(1, h, m.shared_inter, dk, 13)
        else:
            inter = m.dense_intermediate or m.intermediate
            out.ws_gate, out.ws_up, out.ws_down = R(1, inter, h, dk, 11), R(1, inter, h, dk, 12), R(1, h, inter, dk, 13)
        return out

    n_dense = min(m.first_dense, spec.n_layers)
    n_moe = spec.n_layers - n_dense
    n_sets = n_moe if distinct_moe_layers <= 0 else min(distinct_moe_layers, n_moe)
    dw.layers = [make(i) for i in range(n_dense)] + [make(n_dense + j) for j in range(n_sets)]
    dw.layer_map = list(range(n_dense)) + [n_dense + (j % n_sets) for j in range(n_moe)]
    for d in range(spec.mtp_layers):        # native next-token draft modules: one full MoE layer each plus the merge projection
        i = spec.n_layers + d
        dw.mtp.append((ones(h), ones(h), TcWeight.random(1, h, 2 * h, "bf16", device, spec.init_std, act_gs, seed * 1000 + i * 32 + 20),
                       make(max(i, n_dense)), ones(h)))
    return dw


class MlaEngine(Engine):
    def _alloc_attention_state(self):
        spec = self.spec
        self.heads_local = self.weights.layers[0].mla.w_uv.G
        # latent cache: one row of 576 bf16 per token and layer (zero-filled: masked slots must hold finite values)
        n_kv = spec.n_layers + len(self.weights.mtp)          # MTP draft layers keep their rows in extra layers
        self.kv = torch.zeros(n_kv, self.n_pages * PAGE, DQK, dtype=torch.bfloat16, device=self.device)
        host = torch.zeros(n_kv, 128, dtype=torch.uint8)
        for l in range(n_kv):
            call("cuteafd_tmap_encode_latent", host[l].data_ptr(), self.kv[l].data_ptr(), self.n_pages * PAGE)
        self.kv_tmaps = host.to(self.device)
        self.mla_bufs: dict = {}
        a = spec.attn
        if a.index_topk:
            if a.index_dim != 128 or a.index_heads % 16 or a.index_heads > 64:
                raise ValueError("the sparse-attention indexer is built for 128-wide index keys and 16..64 index heads (a multiple of 16)")
            # index-key cache: one 128-wide bf16 row per token and layer, same slots as the latent cache
            self.idx_kv = torch.zeros(n_kv, self.n_pages * PAGE, a.index_dim, dtype=torch.bfloat16, device=self.device)
            host = torch.zeros(n_kv, 128, dtype=torch.uint8)
            for l in range(n_kv):
                call("cuteafd_tmap_encode_index_keys", host[l].data_ptr(), self.idx_kv[l].data_ptr(), self.n_pages * PAGE)
            self.idx_tmaps = host.to(self.device)
            self._dsa: dict = {}

    def _mla_buf(self, L: Lane):
        if getattr(L, "mla_buf", None) is None:
            a, dev, Hl, cap = self.spec.attn, self.device, self.heads_local, L.cap
            bf = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)
            i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
            b = {"q_a": bf(cap, max(a.q_lora_rank, 8)), "q_an": bf(cap, max(a.q_lora_rank, 8)), "q": bf(cap, Hl * 192), "kv_a": bf(cap, DQK),
                 "q_nope": bf(Hl * cap, 128), "q_rope": bf(cap, Hl, 64), "q_lat": bf(Hl * cap, DV), "o_lat": bf(Hl * cap, DV),
                 "o_head": bf(Hl * cap, a.v_head_dim), "o_tok": bf(cap, Hl * a.v_head_dim)}
            if a.index_topk:
                b["q_idx"], b["k_idx"] = bf(cap, a.index_heads * a.index_dim), bf(cap, a.index_dim)
                b["w_idx"] = torch.zeros(cap, a.index_heads, dtype=torch.float32, device=dev)
            b["q_an_act"] = (ActBuffer.alloc(self.dense_kind, cap, a.q_lora_rank, L.tn, dev) if self.dense_kind != KIND_BF16 and a.q_lora_rank
                             else ActBuffer.wrap_bf16(b["q_an"], L.tn))
            b["o_tok_act"] = (ActBuffer.alloc(self.dense_kind, cap, Hl * a.v_head_dim, L.tn, dev) if self.dense_kind != KIND_BF16
                              else ActBuffer.wrap_bf16(b["o_tok"], L.tn))
            L.mla_buf = b           # per lane object: micro-batch lanes of the same capacity keep separate buffers
        return L.mla_buf

    def _head_tiles(self, b, T: int, tn: int):
        """Tile table for the per-head grouped GEMMs over head-major buffers laid out [Hl, T, .]."""
        key = ("tiles", T, tn)
        if key not in b:
            rows = []
            for h in range(self.heads_local):
                for r0 in range(0, T, tn):
                    rows.append([h, h * T + r0, min(tn, T - r0), 0])
            b[key] = (torch.tensor(rows, dtype=torch.int32, device=self.device), torch.tensor([len(rows)], dtype=torch.int32, device=self.device), len(rows))
        return b[key]

    def attn_splits_for(self, n_seq: int, max_q_len: int, max_kv: int) -> int:
        tpt = max(1, 128 // self.heads_local)
        ctas = 2 * n_seq * (-(-max_q_len // tpt))
        tiles = max(1, -(-max_kv // 64))         # the kernel walks the cache in 64-key tiles (one page)
        return max(1, min(tiles, 32, self.sm_count // ctas)) if max_q_len <= 16 else 1

    def _attention_layer(self, li: int, lw: LayerWeights, L: Lane, sh: StepShape):
        spec, a, T, md, w = self.spec, self.spec.attn, sh.T, self.md, lw.mla
        Hl = self.heads_local
        b = self._mla_buf(L)
        xq = self._norm_in(lw, L, T)
        qa = None
        if w.wq_a is not None:
            self._dense(w.wq_a, xq, b["q_a"], T)
            if b["q_an_act"].kind in ops.FUSED_QUANT_KINDS and a.q_lora_rank % 256 == 0:      # norm + operand quantisation in one launch
                ops.add_rmsnorm(b["q_a"], None, w.q_a_norm, None, spec.rms_eps, rows=T, quant=b["q_an_act"], inv_gs=w.wq_b.inv_act_gs)
                qa = b["q_an_act"]
            else:
                ops.add_rmsnorm(b["q_a"], None, w.q_a_norm, b["q_an"], spec.rms_eps, rows=T)
                qa = self._quant(b["q_an"], b["q_an_act"], T, w.wq_b.inv_act_gs)
            self._dense(w.wq_b, qa, b["q"], T)
        else:
            self._dense(w.wq_b, xq, b["q"], T)
        if a.index_topk and w.wq_idx is not None:
            # indexer operands of this step's tokens; the index keys join the paged index-key cache at the tokens' slots
            self._dense(w.wq_idx, qa if qa is not None else xq, b["q_idx"], T)
            self._dense(w.wk_idx, xq, b["k_idx"], T)
            self._dense(w.w_idx, xq, b["w_idx"], T)
            call("cuteafd_dsa_scatter_rows", ptr(b["k_idx"]), ptr(md["slot_map"]), ptr(self.idx_kv[li]), T, self.idx_kv.shape[1], a.index_dim * 2,
                 ptr(self.status), stream())
            self.launches_per_step += 1
        self._dense(w.wkv_a, xq, b["kv_a"], T)
        call("cuteafd_mla_kv_prepare", ptr(b["kv_a"]), ptr(w.kv_a_norm), ptr(md["positions"]), ptr(md["slot_map"]), ptr(self.kv[li]), T,
             self.kv.shape[1], a.rope_theta, spec.rms_eps, 1 if a.rope_interleaved else 0, ptr(self.status), stream())
        q_nope, q_lat = b["q_nope"][:Hl * T], b["q_lat"][:Hl * T]
        call("cuteafd_mla_q_split", ptr(b["q"]), ptr(md["positions"]), ptr(q_nope), ptr(b["q_rope"]), T, Hl, a.rope_theta,
             1 if a.rope_interleaved else 0, stream())
        if a.index_topk and w.wq_idx is not None and self._sparse_step(sh):
            tn = ops.pick_tn(T, swiglu=True)
            tiles, n_tiles, max_tiles = self._head_tiles(b, T, tn)
            qn_act = self._act(b, ("qn", T, tn), q_nope, tn)
            ops.tc_linear(w.w_uk_t, qn_act, q_lat, rows=Hl * T, tiles=tiles, n_tiles=n_tiles, max_tiles=max_tiles, status=self.status)
            o_lat = b["o_lat"][:Hl * T]
            self._sparse_attention(li, b, sh, q_lat, o_lat)
            o_head = b["o_head"][:Hl * T]
            ol_act = self._act(b, ("ol", T, tn), o_lat, tn)
            ops.tc_linear(w.w_uv, ol_act, o_head, rows=Hl * T, tiles=tiles, n_tiles=n_tiles, max_tiles=max_tiles, status=self.status)
            oq = self._o_tok(b, o_head, T, lw)
            self._attn_out(li, lw, oq, L, T)
            self.launches_per_step += 10
            return
        if self._use_prefill_path(sh):
            self._prefill_attention(li, w, b, sh, q_nope)
            oq = self._quant(b["o_tok"], b["o_tok_act"], T, lw.wo.inv_act_gs)
            self._attn_out(li, lw, oq, L, T)
            self.launches_per_step += 5
            return
        tn = ops.pick_tn(T, swiglu=True)
        tiles, n_tiles, max_tiles = self._head_tiles(b, T, tn)
        qn_act = self._act(b, ("qn", T, tn), q_nope, tn)
        ops.tc_linear(w.w_uk_t, qn_act, q_lat, rows=Hl * T, tiles=tiles, n_tiles=n_tiles, max_tiles=max_tiles, status=self.status)
        o_lat = b["o_lat"][:Hl * T]
        if sh.attn_splits > 1:
            need = sh.attn_splits * T * Hl
            if getattr(self, "mla_part_o", None) is None or self.mla_part_o.numel() < need * DV:
                self.mla_part_o = torch.empty(need * DV, dtype=torch.float32, device=self.device)
                self.mla_part_ml = torch.empty(need * 2, dtype=torch.float32, device=self.device)
        po, pml = (self.mla_part_o, self.mla_part_ml) if sh.attn_splits > 1 else (None, None)
        scale = (a.qk_nope_head_dim + a.qk_rope_head_dim) ** -0.5
        call("cuteafd_mla_attention", ptr(q_lat), ptr(b["q_rope"]), ptr(self.kv_tmaps[li]), ptr(md["page_table"]), ptr(md["kv_len"]),
             ptr(md["q_start"]), ptr(md["q_len"]), ptr(o_lat), ptr(po), ptr(pml), T, sh.n_seq, sh.max_q_len, Hl, md["page_table"].shape[1],
             sh.attn_splits, scale, ptr(self.status), stream())
        o_head = b["o_head"][:Hl * T]
        ol_act = self._act(b, ("ol", T, tn), o_lat, tn)
        ops.tc_linear(w.w_uv, ol_act, o_head, rows=Hl * T, tiles=tiles, n_tiles=n_tiles, max_tiles=max_tiles, status=self.status)
        oq = self._o_tok(b, o_head, T, lw)
        self._attn_out(li, lw, oq, L, T)
        self.launches_per_step += 7

    def _o_tok(self, b: dict, o_head: torch.Tensor, T: int, lw: LayerWeights) -> ActBuffer:
        """Per-head attention outputs [Hl, T, 128] -> the output projection's operand (token-major; FP8 operands are written by the
        same launch as the transpose)."""
        a, Hl, act = self.spec.attn, self.heads_local, b["o_tok_act"]
        if act.kind == ops.KIND_FP8B and a.v_head_dim == 128:
            call("cuteafd_head_to_token_major_fp8b", ptr(o_head), None, ptr(act.data), ptr(act.sf), T, Hl, 128, stream())
            return act
        call("cuteafd_head_to_token_major", ptr(o_head), ptr(b["o_tok"]), T, Hl, a.v_head_dim, stream())
        return self._quant(b["o_tok"], act, T, lw.wo.inv_act_gs)

    # ------------------------------------------------------------------ sparse attention over the indexer's selection
    SPARSE_MAX_Q = 8          # decode and verify steps (at most this many query rows per sequence) always take the sparse path

    def _sparse_step(self, sh: StepShape) -> bool:
        """Decode / verify steps of a model with an indexer always run score -> top-k -> gather -> attention (a row that sees at
        most k positions selects all of them, which is dense attention), so a captured graph stays valid as contexts grow past
        k.  Longer query runs (prefill chunks) attend densely while every context of the step has at most k tokens; beyond that
        they are refused (per-row selection for prefill chunks is not built)."""
        a = self.spec.attn
        if sh.T == 0:
            return False
        if sh.max_q_len <= self.SPARSE_MAX_Q:
            return True
        if not torch.cuda.is_current_stream_capturing() and max(self.mh["kv_len"][:sh.n_seq].tolist()) > a.index_topk:
            raise NotImplementedError(f"prefill chunks over contexts longer than index_topk = {a.index_topk} need per-row selection, which is not built")
        return False

    def _sparse_attention(self, li: int, b: dict, sh: StepShape, q_lat: torch.Tensor, o_lat: torch.Tensor):
        """index scores of every query row over its sequence's cached index keys -> top-k positions per row -> gather of the
        selected latent rows into per-row pseudo-pages -> the absorbed attention kernel with one "sequence" per query row.
        Reference: v41_index_scores.cu:37, v41_index_topk.cu:25-57, v41_sparse_attention.cu:89."""
        a, Hl, dev, T, md = self.spec.attn, self.heads_local, self.device, sh.T, self.md
        k, kp = a.index_topk, -(-a.index_topk // PAGE) * PAGE
        ld = -(-(self.max_pages * PAGE) // 128) * 128
        key = (T, sh.n_seq, sh.max_q_len, sh.uniform)
        st = self._dsa.get(key)
        if st is None:
            i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
            st = {"seq_of_row": i32([r // sh.max_q_len for r in range(T)]), "q_start": i32(list(range(T))), "q_len": i32([1] * T),
                  "pages": i32([[r * (kp // PAGE) + j for j in range(kp // PAGE)] for r in range(T)]),
                  "sel": torch.zeros(T, k, dtype=torch.int32, device=dev), "count": torch.zeros(T, dtype=torch.int32, device=dev)}
            self._dsa[key] = st
        if not sh.uniform:           # ragged step (eager only): rows -> sequences from the host copy of the step's description
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("a ragged sparse-attention step cannot be captured")
            qs, ql = self.mh["q_start"][:sh.n_seq].tolist(), self.mh["q_len"][:sh.n_seq].tolist()
            rows = [0] * T
            for sq, (q0, n) in enumerate(zip(qs, ql)):
                rows[q0:q0 + n] = [sq] * n
            st["seq_of_row"].copy_(torch.tensor(rows, dtype=torch.int32).pin_memory(), non_blocking=True)
        if self._dsa.get("rows", 0) < T:          # shared scratch, grown to the largest step (zero-filled: unselected rows stay finite)
            self._dsa["scores"] = torch.zeros(T, ld, dtype=torch.float32, device=dev)
            self._dsa["gather"] = torch.zeros(T * kp, DQK, dtype=torch.bfloat16, device=dev)
            host = torch.zeros(128, dtype=torch.uint8)
            call("cuteafd_tmap_encode_latent", host.data_ptr(), self._dsa["gather"].data_ptr(), T * kp)
            self._dsa["gmap"] = host.to(dev)
            self._dsa["rows"] = T
            self.graphs.clear()                    # captured graphs hold the old scratch addresses
        scores, gather = self._dsa["scores"], self._dsa["gather"]
        sp = ptr(self.status)
        call("cuteafd_dsa_index_scores", ptr(b["q_idx"]), ptr(b["w_idx"]), ptr(self.idx_tmaps[li]), ptr(md["page_table"]), ptr(md["kv_len"]),
             ptr(md["q_start"]), ptr(md["q_len"]), ptr(scores), T, sh.n_seq, sh.max_q_len, self.max_pages * PAGE, a.index_heads, ld,
             md["page_table"].shape[1], sp, stream())
        call("cuteafd_dsa_topk", ptr(scores), ld, ptr(md["positions"]), T, k, 1, ptr(st["sel"]), ptr(st["count"]), stream())
        call("cuteafd_dsa_gather_rows", ptr(self.kv[li]), ptr(md["page_table"]), ptr(st["seq_of_row"]), ptr(st["sel"]), ptr(st["count"]), ptr(gather),
             T, k, kp, md["page_table"].shape[1], self.kv.shape[1], DQK * 2, sp, stream())
        splits = self.attn_splits_for(T, 1, k)
        po = pml = None
        if splits > 1:
            need = splits * T * Hl
            if getattr(self, "mla_part_o", None) is None or self.mla_part_o.numel() < need * DV:
                self.mla_part_o = torch.empty(need * DV, dtype=torch.float32, device=dev)
                self.mla_part_ml = torch.empty(need * 2, dtype=torch.float32, device=dev)
            po, pml = self.mla_part_o, self.mla_part_ml
        scale = (a.qk_nope_head_dim + a.qk_rope_head_dim) ** -0.5
        call("cuteafd_mla_attention", ptr(q_lat), ptr(b["q_rope"]), ptr(self._dsa["gmap"]), ptr(st["pages"]), ptr(st["count"]), ptr(st["q_start"]),
             ptr(st["q_len"]), ptr(o_lat), ptr(po), ptr(pml), T, T, 1, Hl, kp // PAGE, splits, scale, sp, stream())

    # ------------------------------------------------------------------ prefill: per-head attention over the expanded context
    PREFILL_MIN_Q = int(os.environ.get("CUTEAFD_MLA_PREFILL_MIN_Q", "128"))          # 0 disables the path
    PREFILL_MAX_BYTES = int(float(os.environ.get("CUTEAFD_MLA_PREFILL_MAX_GIB", "12")) * (1 << 30))

    def _use_prefill_path(self, sh: StepShape) -> bool:
        """Steps whose longest query run is at least one 128-row tile take the non-absorbed path (arithmetic per key 320
        instead of 1088 multiply-adds per head), unless the step is being captured (the context sizes are read on the host),
        was cut into micro-batches, or its expanded context would not fit the scratch budget."""
        a = self.spec.attn
        if not self.PREFILL_MIN_Q or sh.max_q_len < self.PREFILL_MIN_Q or sh.uniform or a.qk_nope_head_dim != 128 or a.v_head_dim != 128:
            return False
        if torch.cuda.is_current_stream_capturing():
            return False
        kv = self.mh["kv_len"][:sh.n_seq].tolist()
        rows = sum(-(-n // 64) * 64 for n in kv) + 64
        return rows * (DQK + self.heads_local * 256) * 2 <= self.PREFILL_MAX_BYTES

    def _prefill_attention(self, li: int, w, b: dict, sh: StepShape, q_nope: torch.Tensor):
        """gather the context's latent rows -> expand them to per-head keys / values (one GEMM with kv_b) -> per-head causal
        attention (`mla_prefill_kernel`), output token-major in b["o_tok"].  Reference: glm_mla_prefill.cu:123-960."""
        a, Hl, dev = self.spec.attn, self.heads_local, self.device
        n_seq, md = sh.n_seq, self.md
        kv = tuple(self.mh["kv_len"][:n_seq].tolist())
        plan = getattr(self, "_pf_plan", None)
        if plan is None or plan[0] != kv:
            starts, tot = [], 0
            for n in kv:
                starts.append(tot)
                tot += -(-n // 64) * 64
            host = torch.tensor(starts, dtype=torch.int32).pin_memory()
            if getattr(self, "_pf_starts", None) is None or self._pf_starts.numel() < n_seq:
                self._pf_starts = torch.zeros(max(n_seq, self.max_seqs), dtype=torch.int32, device=dev)
            self._pf_starts[:n_seq].copy_(host, non_blocking=True)
            self._pf_plan = plan = (kv, tot, host)
        rows = plan[1]
        cap = getattr(self, "_pf_cap", 0)
        if rows + 64 > cap:                       # zero-filled: rows no gather ever wrote are multiplied by zero probabilities
            cap = max(1024, 1 << (rows + 64 - 1).bit_length())
            self._pf_lat = self._pf_kvb = self._pf_act = None
            self._pf_lat = torch.zeros(cap, DQK, dtype=torch.bfloat16, device=dev)
            self._pf_kvb = torch.zeros(cap, Hl * 256, dtype=torch.bfloat16, device=dev)
            view = self._pf_lat[:, :DV]
            self._pf_act = ActBuffer(KIND_BF16, cap, DV, 256, view, ops.encode_tmap(view, 256))
            self._pf_cap = cap
        st = ptr(self.status)
        call("cuteafd_mla_gather_ctx", ptr(self.kv[li]), ptr(md["page_table"]), ptr(self._pf_starts), ptr(md["kv_len"]), ptr(self._pf_lat), n_seq,
             max(kv), md["page_table"].shape[1], self.kv.shape[1], self._pf_cap, st, stream())
        ops.tc_linear(w.ensure_kvb(), self._pf_act, self._pf_kvb, rows=rows, status=self.status)
        scale = (a.qk_nope_head_dim + a.qk_rope_head_dim) ** -0.5
        call("cuteafd_mla_prefill_attention", ptr(q_nope), ptr(b["q_rope"]), ptr(self._pf_kvb), ptr(self._pf_lat), self._pf_cap, ptr(self._pf_starts),
             ptr(md["kv_len"]), ptr(md["q_start"]), ptr(md["q_len"]), ptr(b["o_tok"]), sh.T, n_seq, sh.max_q_len, Hl, scale, st, stream())

    def _attn_in_gs(self, lw):
        return lw.mla.wkv_a.inv_act_gs

    def _act(self, b, key, tensor, tn):
        """bf16 activation operand over a view of a head-major buffer (descriptor cached per shape)."""
        if key not in b:
            b[key] = ActBuffer.wrap_bf16(tensor, tn)
        return b[key]
