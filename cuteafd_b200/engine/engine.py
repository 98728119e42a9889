"""Model engine: runs prefill / decode / speculative-verify steps of a MoE decoder on one GPU (or one rank's
share of it) by launching the native kernels on the current stream, with decode steps replayed from
CUDA graphs keyed by their exact shape.

Shape of one step (reference: Engine::step_inner, families/deepseek_v4/engine.rs:909-1241):
  inputs  -> one packed int32 block copied H2D (tokens, positions, KV slots, per-sequence lengths, page table)
  per layer: RMSNorm -> [act quant] -> QKV GEMM -> head-norm + RoPE + paged KV write -> paged attention ->
             [act quant] -> O GEMM (+residual) -> RMSNorm -> router GEMM + top-k -> route pack ->
             gather + quant into expert order -> grouped FC1 (SwiGLU fused) -> [quant] -> grouped FC2 ->
             shared expert -> ordered weighted combine + shared + residual
  tail    -> gather rows that need logits -> RMSNorm -> LM head GEMM -> token selection on device.
Only token ids / status words return to the host.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass

import torch

from .. import ops
from ..config import ModelSpec
from ..models.weights import DeviceWeights, LayerWeights
from ..ops import ActBuffer, FP4_KINDS, FUSED_QUANT_KINDS, KIND_BF16, KIND_FP8B, native, pick_tn
from ..ops.native import ptr
from ..utils.graph_census import GraphCensus

PAGE = 64
# query rows per sequence from which a step's GQA attention takes the prefill kernel (128-key tiles); 0 = never
PREFILL_ATTN_MIN_Q = int(os.environ.get("CUTEAFD_PREFILL_ATTN_MIN_Q", "64"))


# Decode-sized steps: router logits + selection + packing in one launch.  Opt-in: measured equal to the two-launch form on one GPU
# (265.3 vs 265.4 us per layer) and 0.6 % slower on the multi-GPU layouts (one block selects for every token instead of a block per token).
FP8_FUSE_GATE_UP = os.environ.get("CUTEAFD_FP8_FUSE_GATE_UP", "1") != "0"      # FP8 dense FFNs: gate and up projections as one GEMM
CLUSTER_KINDS = (KIND_BF16,) + tuple(FP4_KINDS)       # operand kinds with a cluster split-K kernel besides FP8
ROUTER_FUSED = os.environ.get("CUTEAFD_ROUTER_FUSED", "0") == "1"


@dataclass
class StepShape:
    """Static shape of a captured step."""
    T: int            # token rows
    n_seq: int
    max_q_len: int
    n_logits: int
    attn_splits: int
    # True when the caller guarantees the regular layout of decode / verify steps: every sequence has max_q_len query rows,
    # sequence s owns rows [s * max_q_len, (s + 1) * max_q_len), and rows that need logits are listed in ascending order.  Such a
    # step can be cut into micro-batches at sequence boundaries.
    uniform: bool = False
    # Speculative verify step of a stack with recurrent (linear-attention) layers: those layers compute their outputs but leave the
    # state and the convolution history as they were; `Engine.commit_state` replays the accepted rows afterwards.
    defer_state: bool = False

    def key(self):
        return (self.T, self.n_seq, self.max_q_len, self.n_logits, self.attn_splits, self.uniform, self.defer_state)


class Lane:
    """Activation buffers for steps of up to `cap` token rows (one lane per row bucket)."""

    def __init__(self, eng: "Engine", cap: int):
        spec, dev, w = eng.spec, eng.device, eng.weights
        a, m, H = spec.attn, spec.moe, spec.hidden
        self.cap = cap
        self.tn = pick_tn(min(cap, int(os.environ.get("CUTEAFD_TN", "128"))), swiglu=True)      # <= 128 so the same descriptors serve the fused SwiGLU GEMMs
        bf = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
        dk, ek = eng.dense_kind, eng.expert_kind
        self.x = bf(cap, H)
        self.xn = bf(cap, H)
        self.xn_act = ActBuffer.wrap_bf16(self.xn, self.tn)
        self.xq = ActBuffer.alloc(dk, cap, H, self.tn, dev) if dk != KIND_BF16 else self.xn_act
        if a.kind == "gqa":
            qkv_n = (a.n_heads + 2 * a.n_kv_heads) * a.head_dim
            self.qkv = bf(cap, qkv_n)
            self.attn = bf(cap, a.n_heads * a.head_dim)
            self.attn_q = (ActBuffer.alloc(dk, cap, a.n_heads * a.head_dim, self.tn, dev) if dk != KIND_BF16
                           else ActBuffer.wrap_bf16(self.attn, self.tn))
        # logits
        self.xl = bf(cap, H)
        self.xln = bf(cap, H)
        self.xln_act = ActBuffer.wrap_bf16(self.xln, self.tn)
        self.logits = torch.zeros(cap, spec.vocab, dtype=torch.float32, device=dev)
        self.next_tok = i32(cap)
        self.tok_status = i32(cap)
        # shared expert / dense FFN intermediates, created on first use per width (always during the
        # un-captured warm-up run of a shape)
        self.ffn_bufs: dict = {}
        self.shared = bf(cap, H)
        # routed experts
        if m.n_experts and eng.n_local_experts:
            rows = cap * m.top_k
            exp_rows = max(1, math.ceil(rows / max(1, m.n_experts)) * 2)
            # token tiles of the grouped expert GEMMs stay <= 32 rows even in prefill: those tiles run two CTAs per SM with
            # double-buffered accumulators, which measured 2x faster end to end than 128-row tiles (one CTA per SM, the
            # SwiGLU epilogue not overlapped); CUTEAFD_TNG overrides for experiments
            self.tn_g = pick_tn(min(exp_rows, int(os.environ.get("CUTEAFD_TNG", "32"))), swiglu=True)
            self.max_tiles = eng.n_local_experts + rows // self.tn_g + 1
            self.router_logits = torch.zeros(cap, m.n_experts, dtype=torch.float32, device=dev)
            self.idx, self.wts = i32(cap, m.top_k), torch.zeros(cap, m.top_k, dtype=torch.float32, device=dev)
            self.src_token, self.slot_row = i32(rows), i32(cap, m.top_k)
            self.counts, self.offsets = i32(eng.n_local_experts), i32(eng.n_local_experts)
            self.tiles, self.n_tiles, self.n_rows = i32(self.max_tiles, 4), i32(1), i32(1)
            self.xs = ActBuffer.alloc(ek, rows, H, self.tn_g, dev)
            self.h1 = bf(rows, m.intermediate)
            self.h1_q = (ActBuffer.alloc(ek, rows, m.intermediate, self.tn_g, dev) if ek != KIND_BF16
                         else ActBuffer.wrap_bf16(self.h1, self.tn_g))
            self.y2 = bf(rows, H)
        if a.linear_every:
            self.lin_buf(eng)
        if spec.hyper_streams:       # hyper-connections: the residual streams, the open sub-layer's output and its spread / mix coefficients
            self.res = bf(cap, spec.hyper_streams, H)
            self.sub = bf(cap, H)
            self.hc_coef = torch.zeros(cap, 20, dtype=torch.float32, device=dev)

    def lin_buf(self, eng) -> dict:
        """Buffers of the linear-attention layers of a hybrid stack."""
        if getattr(self, "_lin", None) is None:
            a, dev, cap = eng.spec.attn, eng.device, self.cap
            Hk, Hv = a.linear_k_heads, a.linear_v_heads
            bf = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)
            f32 = lambda *s: torch.zeros(*s, dtype=torch.float32, device=dev)
            nb = Hv + (Hv * 128 if a.linear_per_channel else Hv)
            on = bf(cap, Hv * 128)
            self._lin = {"qkvz": bf(cap, (2 * Hk + 2 * Hv) * 128), "ba": f32(cap, nb), "conv": bf(cap, (2 * Hk + Hv) * 128), "q": bf(cap, Hv, 128),
                         "k": bf(cap, Hv, 128), "v": bf(cap, Hv, 128), "g": f32(cap, Hv, 128) if a.linear_per_channel else f32(cap, Hv),
                         "beta": f32(cap, Hv), "o": bf(cap, Hv, 128), "on": on, "on_act": ActBuffer.wrap_bf16(on, self.tn)}
        return self._lin

    def lin_save(self, eng) -> list:
        """Per linear-attention layer, what a deferred (speculative verify) step keeps for the replay of its accepted rows."""
        if getattr(self, "_lin_save", None) is None:
            if self.cap > 256:
                raise NotImplementedError("deferred recurrent state is for decode / verify sized steps (<= 256 rows)")
            a, dev, cap = eng.spec.attn, eng.device, self.cap
            Hk, Hv = a.linear_k_heads, a.linear_v_heads
            bf = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)
            f32 = lambda *s: torch.zeros(*s, dtype=torch.float32, device=dev)
            self._lin_save = [{"qkvz": bf(cap, (2 * Hk + 2 * Hv) * 128), "k": bf(cap, Hv, 128), "v": bf(cap, Hv, 128),
                               "g": f32(cap, Hv, 128) if a.linear_per_channel else f32(cap, Hv), "beta": f32(cap, Hv)} for _ in eng.lin_layers]
        return self._lin_save

    def ffn_buf(self, eng, inter: int):
        if inter not in self.ffn_bufs:
            s1 = torch.zeros(self.cap, inter, dtype=torch.bfloat16, device=eng.device)
            act = (ActBuffer.alloc(eng.dense_kind, self.cap, inter, self.tn, eng.device) if eng.dense_kind != KIND_BF16
                   else ActBuffer.wrap_bf16(s1, self.tn))
            self.ffn_bufs[inter] = (s1, act)
        return self.ffn_bufs[inter]


class Engine:
    def __init__(self, weights: DeviceWeights, *, n_pages: int, max_seqs: int = 64, max_pages_per_seq: int = 0,
                 expert_range: tuple | None = None, device=None, sm_count: int = 148):
        self.weights, self.spec = weights, weights.spec
        spec = self.spec
        self.device = device or weights.embed.device
        if spec.attn.kind != "gqa":
            if not hasattr(self, "_alloc_attention_state"):
                raise NotImplementedError("Engine runs GQA models; MLA models use engine.mla.MlaEngine")
            self.dense_kind = weights.layers[0].wo.kind
        else:
            self.dense_kind = weights.layers[0].wo.kind
        self.engram = getattr(weights, "engram", None)          # n-gram memory (specs with engram_layers)
        if self.engram is not None and spec.hyper_streams:
            raise NotImplementedError("the n-gram memory is wired for single-stream stacks (its module gates any number of streams)")
        first_moe = next((l for l in weights.layers if l.w_gate is not None), None)
        self.expert_kind = first_moe.w_gate.kind if first_moe is not None else KIND_BF16
        self.expert_range = expert_range or (0, spec.moe.n_experts)
        self.n_local_experts = first_moe.w_gate.G if first_moe is not None else 0
        self.n_pages, self.max_seqs = n_pages, max_seqs
        self.max_pages = max_pages_per_seq or n_pages
        self.sm_count = sm_count
        a = spec.attn
        # one allocation for every layer's paged KV: [layers, slots, 2, Hkv, D]; zero-filled so masked
        # (never-written) slots hold finite values
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        if spec.attn.kind == "gqa":
            # MTP draft layers keep their KV rows in extra layers of the same store (same pages, same slots)
            self.kv = torch.zeros(spec.n_layers + len(weights.mtp), n_pages * PAGE, 2, a.n_kv_heads, a.head_dim, dtype=torch.bfloat16,
                                  device=self.device)
            # head_dim 128 runs on the tcgen05 attention kernel (one TMA descriptor per layer's K/V store)
            self.kv_tmaps = ops.encode_kv_tmaps(self.kv) if a.head_dim == 128 and 128 % (a.n_heads // a.n_kv_heads) == 0 else None
        else:
            self._alloc_attention_state()
        if spec.hyper_streams:
            if spec.hyper_streams != 4 or weights.hc_head is None or weights.mtp:
                raise NotImplementedError("hyper-connections: four streams, on the single-GPU engines, without an MTP module")
        self._hc_pending = None
        # hybrid stacks: gated delta-rule layers keep a recurrent state and the last three convolution inputs per sequence slot
        self.lin_layers = [i for i in range(spec.n_layers) if spec.layer_is_linear(i)]
        if self.lin_layers:
            if a.kind != "gqa" or a.linear_v_heads % a.linear_k_heads:
                raise ValueError("linear-attention layers: GQA stacks with linear_v_heads a multiple of linear_k_heads")
            self.lin_index = {li: j for j, li in enumerate(self.lin_layers)}
            C = (2 * a.linear_k_heads + a.linear_v_heads) * 128
            self.lin_state = torch.zeros(len(self.lin_layers), max_seqs, a.linear_v_heads, 128, 128, dtype=torch.float32, device=self.device)
            self.lin_carry = torch.zeros(len(self.lin_layers), max_seqs, 3, C, dtype=torch.bfloat16, device=self.device)
        # memory ledger: what this engine holds, by category (reported by `/v1/stats` and `cuteafd doctor`)
        from ..utils.memory_ledger import LEDGER
        with LEDGER.scope("weights"):
            LEDGER.charge_tree(weights, "model weights")
        with LEDGER.scope("kv"):
            LEDGER.charge(self.kv.numel() * self.kv.element_size(), "paged KV store")
        # optional instrumentation of eager steps: per-layer device time (CUDA events, read after the step) and NVTX ranges
        self.layer_clock = None
        if os.environ.get("CUTEAFD_LAYER_CLOCK", "0") == "1":
            from ..utils.trace import DeviceClock
            self.layer_clock = DeviceClock()
        self._nvtx = os.environ.get("CUTEAFD_NVTX", "0") == "1"
        self._l2_prefetch = os.environ.get("CUTEAFD_L2_PREFETCH", "0") == "1"
        self.lanes: dict[int, Lane] = {}
        self.mtp_lanes: dict[int, Lane] = {}
        self.graphs: dict = {}
        self.graph_captures = 0
        self.census = GraphCensus()
        self._meta_cap = 0
        self.launches_per_step = 0

    # ------------------------------------------------------------------ buffers
    def lane(self, T: int) -> Lane:
        cap = next(c for c in (16, 64, 256, 1024, 4096, 16384) if T <= c)
        if cap not in self.lanes:
            self.lanes[cap] = Lane(self, cap)
        return self.lanes[cap]

    def _ensure_meta(self, T: int):
        """Packed int32 step inputs: host (pinned) + device copies and named views."""
        cap = max(T, 16)
        if cap <= self._meta_cap:
            return
        cap = 1 << (cap - 1).bit_length()
        S, MP = self.max_seqs, self.max_pages
        n = 4 * cap + 4 * S + S * MP
        self.meta_host = torch.zeros(n, dtype=torch.int32).pin_memory() if torch.cuda.is_available() else torch.zeros(n, dtype=torch.int32)
        self.meta_dev = torch.zeros(n, dtype=torch.int32, device=self.device)

        def views(buf):
            o = 0
            out = {}
            for name, cnt in (("tokens", cap), ("positions", cap), ("slot_map", cap), ("logit_rows", cap),
                              ("kv_len", S), ("q_start", S), ("q_len", S), ("state_slot", S)):
                out[name] = buf[o:o + cnt]
                o += cnt
            out["page_table"] = buf[o:o + S * MP].view(S, MP)
            return out
        self.mh, self.md = views(self.meta_host), views(self.meta_dev)
        self._meta_cap = cap
        self.graphs.clear()     # views moved: captured graphs are stale
        self.census.invalidate()

    def set_inputs(self, tokens, positions, slot_map, logit_rows, kv_len, q_start, q_len, page_table_rows, state_slots=None, engram_ctx=None):
        """Fill the pinned host block and enqueue ONE host-to-device copy.  `state_slots`: per sequence of the step, the slot of its
        recurrent state (hybrid stacks with linear-attention layers); default: the sequence's index in the step.  `engram_ctx`: per
        sequence, the (up to three) tokens before its first row of this step - models with an n-gram memory address its tables by the
        last four tokens, and the addresses of all rows travel in a second copy."""
        T, S = len(tokens), len(kv_len)
        extra = 0
        if self.engram is not None:
            if engram_ctx is None or len(engram_ctx) != S:
                raise ValueError("this model has an n-gram memory: set_inputs needs engram_ctx (the tokens before each sequence's rows)")
            import numpy as np
            from ..ref.engram import context_hashes
            parts = [context_hashes(self.engram.addr, list(engram_ctx[s]), list(tokens[q_start[s]:q_start[s] + q_len[s]])) for s in range(S)]
            extra = self.engram.set_hashes(np.concatenate(parts, axis=1))
        self._ensure_meta(T)
        mh = self.mh
        mh["tokens"][:T] = torch.as_tensor(tokens, dtype=torch.int32)
        mh["positions"][:T] = torch.as_tensor(positions, dtype=torch.int32)
        mh["slot_map"][:T] = torch.as_tensor(slot_map, dtype=torch.int32)
        nl = len(logit_rows)
        mh["logit_rows"][:nl] = torch.as_tensor(logit_rows, dtype=torch.int32)
        mh["kv_len"][:S] = torch.as_tensor(kv_len, dtype=torch.int32)
        mh["q_start"][:S] = torch.as_tensor(q_start, dtype=torch.int32)
        mh["q_len"][:S] = torch.as_tensor(q_len, dtype=torch.int32)
        mh["state_slot"][:S] = torch.as_tensor(list(state_slots) if state_slots is not None else list(range(S)), dtype=torch.int32)
        for s, row in enumerate(page_table_rows):
            mh["page_table"][s, :len(row)] = torch.as_tensor(row, dtype=torch.int32)
        self.meta_dev.copy_(self.meta_host, non_blocking=True)
        return self.meta_host.numel() * 4 + extra

    def set_input_embeds(self, rows, vals: torch.Tensor | None):
        """Rows of the NEXT eager step whose token embedding is replaced by `vals` (bf16 [n, hidden] on this device): the image rows
        a vision tower produced for the placeholder tokens of a prompt.  One-shot: the step that consumes them clears them.
        Reference: native/families/deepseek_v41/cuda/v41_vision.cu (`image_embed_kernel`: features scattered into the residual)."""
        if vals is None or not len(rows):
            self._embed_over = None
            return
        if vals.dtype != torch.bfloat16 or vals.shape != (len(rows), self.spec.hidden) or vals.device != self.device:
            raise ValueError("set_input_embeds: bf16 [len(rows), hidden] rows on the engine's device")
        self._embed_over = (torch.as_tensor(rows, dtype=torch.int32).to(self.device), vals.contiguous())

    def _apply_input_embeds(self, x: torch.Tensor, T: int):
        over = getattr(self, "_embed_over", None)
        if over is None:
            return
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("input embeddings belong to eager (prefill) steps, not to a captured graph")
        self._embed_over = None
        rows, vals = over
        native.call("cuteafd_dsa_scatter_rows", ptr(vals), ptr(rows), ptr(x), len(rows), T, self.spec.hidden * 2, ptr(self.status), native.stream())
        self.launches_per_step += 1

    # ------------------------------------------------------------------ kernels
    def _splits(self, N: int, K: int, T: int, tn: int, kind: int) -> int:
        """Split-K factor of a dense layer.  Decode-sized token tiles (<= 32 rows) split over a thread-block cluster
        (up to 8 CTAs reduce through distributed shared memory): the largest split that still fits one wave - asked of the
        device, since a cluster must sit inside one GPC - and leaves every CTA at least two pipeline stages of K."""
        tiles = -(-N // 128) * -(-T // tn)
        nkb = K // (64 if kind == KIND_BF16 else (128 if kind == KIND_FP8B else 256))
        if tiles >= self.sm_count or nkb < 4:
            return 1
        if kind == KIND_FP8B and tn <= 32:
            # decode-sized FP8 tiles run two CTAs per SM for splits of up to 4 (the kernel is bound by its per-stage chain of MMA issues):
            # few tiles spread K over the widest cluster, otherwise the largest split that still fits one wave of 2 x SMs CTAs
            # (a cluster needs its CTAs inside one GPC: the device holds e.g. only 15 clusters of 8, so the fit is asked, not computed)
            if tn == 16:
                for s in (8, 7, 6, 5):
                    if nkb // s >= 2 and tiles <= ops.fp8_cluster_capacity(tn, s, K):
                        return s
            for s in (4, 2):      # measured: 224 CTAs of a 4-way split (two rounds of clusters) beat 112 CTAs of a 2-way split on the wo shape
                if tiles * s <= 2 * self.sm_count and nkb // s >= 2:
                    return s
            return 1
        if tn <= 32 or (kind == KIND_FP8B and tn <= 64):      # the FP8 kernel's cluster reduction also takes 64-row tiles
            for s in ((8, 4, 2) if tn == 16 else (4, 2)):
                if tiles * s <= self.sm_count and nkb // s >= 2 and (kind == KIND_FP8B or kind not in CLUSTER_KINDS or tiles <= ops.cluster_capacity(kind, tn, s)):
                    return s
            return 1
        # larger token tiles: global-memory fix-up (measured on B200: its cost grows with the split count, the sweet
        # spot is about one work unit per SM and never more than 8 splits)
        return max(1, min(nkb // 2, 8, self.sm_count // tiles))

    def _dense(self, w, x_act, y, T, residual=None, w_up=None):
        splits = 1 if w_up is not None else self._splits(w.N, w.K, T, x_act.tn, w.kind)
        ops.tc_linear(w, x_act, y, rows=T, w_up=w_up, residual=residual, splits=splits, status=self.status)
        self.launches_per_step += 1

    def _quant(self, x_bf16, act: ActBuffer, T, inv_gs):
        if act.kind == KIND_BF16:
            return act
        ops.quant_fp4_rows(x_bf16, act, rows=T, inv_gs=inv_gs)
        self.launches_per_step += 1
        return act

    def _attn_in_gs(self, lw: LayerWeights):
        """Activation global scale of the first projection of the attention block (NVFP4)."""
        return (lw.wqkv if lw.wqkv is not None else lw.lin_qkvz).inv_act_gs

    def _norm_in(self, lw: LayerWeights, L: Lane, T: int) -> ActBuffer:
        """Input of the attention block: RMSNorm of the residual stream as the GEMM operand (bf16 or FP4, quantised in
        the same launch) - unless the previous layer's combine already produced it."""
        if self.spec.hyper_streams:
            self._hc_boundary(L, T, lw.hc_attn, lw.attn_norm)
            if L.xq.kind != KIND_BF16:
                self._quant(L.xn, L.xq, T, None if L.xq.kind == KIND_FP8B else self._attn_in_gs(lw))
            return L.xq
        if self._pre_normed:
            self._pre_normed = False
            return L.xq
        if L.xq.kind in FUSED_QUANT_KINDS and self.spec.hidden % 256 == 0:
            ops.add_rmsnorm(L.x, None, lw.attn_norm, None, self.spec.rms_eps, rows=T, quant=L.xq, inv_gs=self._attn_in_gs(lw))
        else:
            ops.add_rmsnorm(L.x, None, lw.attn_norm, L.xn, self.spec.rms_eps, rows=T)
            self._quant(L.xn, L.xq, T, None)              # FP8 operands: separate quantiser (no-op for bf16)
        self.launches_per_step += 1
        return L.xq

    def _combine(self, y, rows, wts, shared, L: Lane, T: int, k: int, wait=None):
        """Weighted top-k sum + shared expert + residual; when another layer follows, its input norm (and FP4
        quantisation) rides in the same launch.  `wait`: the kernel first waits for the peers that deliver `y`."""
        nxt = self._next_lw
        if self.spec.hyper_streams:       # the block's output stays apart: the next boundary spreads it over the streams
            ops.moe_combine(y, rows, wts, shared, None, L.sub, T, k, wait=wait)
            return
        if nxt is None or getattr(self, "_next_engram", False):      # an engram layer first adds its memory to the un-normalised rows
            ops.moe_combine(y, rows, wts, shared, L.x, L.x, T, k, wait=wait)
            return
        fp4 = L.xq.kind in FUSED_QUANT_KINDS and self.spec.hidden % 256 == 0      # the quantised operand rides in the same launch
        ops.moe_combine(y, rows, wts, shared, L.x, L.x, T, k, norm_w=nxt.attn_norm, eps=self.spec.rms_eps, xn=None if fp4 else L.xn,
                        quant=L.xq if fp4 else None, inv_gs=self._attn_in_gs(nxt) if fp4 else None, wait=wait)
        if not fp4:
            self._quant(L.xn, L.xq, T, None)              # FP8 operands: separate quantiser (no-op for bf16)
        self._pre_normed = True

    def reset_state_slots(self, slots):
        """A new sequence takes over these recurrent-state slots: zero state, zero convolution history."""
        if getattr(self, "lin_layers", None) and len(slots):
            idx = torch.as_tensor(list(slots), dtype=torch.long, device=self.device)
            self.lin_state.index_fill_(1, idx, 0.0)
            self.lin_carry.index_fill_(1, idx, 0.0)

    def _linear_layer(self, li: int, lw: LayerWeights, L: Lane, sh: StepShape):
        """Gated delta-rule layer: fused projection -> width-4 causal convolution + SiLU -> normalised q / k, gates -> recurrence over
        the sequences' state slots -> gated RMSNorm -> output projection (+ residual).  Oracle: `RefModel.linear_attention`."""
        spec, a, T, md = self.spec, self.spec.attn, sh.T, self.md
        Hk, Hv = a.linear_k_heads, a.linear_v_heads
        C, Nq, j = (2 * Hk + Hv) * 128, (2 * Hk + 2 * Hv) * 128, self.lin_index[li]
        b = L.lin_buf(self)
        pc = 1 if a.linear_per_channel else 0
        # a deferred (speculative verify) step keeps what the replay of the accepted rows needs, per layer: the convolution's input
        # rows and the recurrence's k / v / decay / beta; state and history stay untouched
        sv = L.lin_save(self)[j] if sh.defer_state else None
        qkvz = sv["qkvz"] if sv else b["qkvz"]
        k_, v_, g_, beta_ = (sv["k"], sv["v"], sv["g"], sv["beta"]) if sv else (b["k"], b["v"], b["g"], b["beta"])
        xq = self._norm_in(lw, L, T)
        self._dense(lw.lin_qkvz, xq, qkvz, T)
        if xq.kind != KIND_BF16:           # the gate projection stays bf16: it needs the bf16 normalised rows
            raise NotImplementedError("linear-attention layers run with bf16 dense projections")
        self._dense(lw.lin_ba, L.xn_act, b["ba"], T)
        st, n_seq = ptr(self.status), sh.n_seq
        native.call("cuteafd_short_conv4_peek" if sv else "cuteafd_short_conv4", ptr(qkvz), ptr(lw.lin_conv), ptr(self.lin_carry[j]), ptr(md["state_slot"]),
                    ptr(md["q_start"]), ptr(md["q_len"]), ptr(b["conv"]), n_seq, C, Nq, self.max_seqs, st, native.stream())
        native.call("cuteafd_linear_prepare", ptr(b["conv"]), ptr(b["ba"]), ptr(lw.lin_a_log), ptr(lw.lin_dt_bias), ptr(b["q"]), ptr(k_), ptr(v_),
                    ptr(g_), ptr(beta_), T, Hk, Hv, b["ba"].shape[1], pc, native.stream())
        native.call("cuteafd_gated_delta_step", ptr(b["q"]), ptr(k_), ptr(v_), ptr(g_), ptr(beta_), ptr(self.lin_state[j]),
                    ptr(md["state_slot"]), ptr(md["q_start"]), ptr(md["q_len"]), ptr(b["o"]), None, n_seq, Hv, pc | (2 if sv else 0),
                    self.max_seqs, st, native.stream())
        native.call("cuteafd_gated_rmsnorm", ptr(b["o"]), ptr(qkvz), ptr(lw.lin_norm), ptr(b["on"]), T, Hv, Nq, C, spec.rms_eps, native.stream())
        self._attn_out(li, lw, b["on_act"], L, T)
        self.launches_per_step += 7

    def commit_state(self, sh: StepShape, accepted):
        """After a deferred step (`sh.defer_state`): absorb the first `accepted[s]` rows of every sequence s of that step into the
        recurrent state and the convolution history of every linear-attention layer, by replaying the convolution and the recurrence
        over the rows the step kept.  Must run before the next `set_inputs` (it reads that step's sequence layout)."""
        if not getattr(self, "lin_layers", None):
            return
        if not sh.defer_state or len(accepted) != sh.n_seq:
            raise ValueError("commit_state follows a deferred step and takes one accepted-row count per sequence of it")
        a, md, L = self.spec.attn, self.md, self.lane(sh.T)
        Hk, Hv, pc = a.linear_k_heads, a.linear_v_heads, 1 if a.linear_per_channel else 0
        C, Nq = (2 * Hk + Hv) * 128, (2 * Hk + 2 * Hv) * 128
        if getattr(self, "_acc_host", None) is None:
            self._acc_host = torch.zeros(self.max_seqs, dtype=torch.int32)
            if torch.cuda.is_available():
                self._acc_host = self._acc_host.pin_memory()
            self._acc_dev = torch.zeros(self.max_seqs, dtype=torch.int32, device=self.device)
        self._acc_host[:sh.n_seq] = torch.as_tensor([max(0, min(int(n), sh.max_q_len)) for n in accepted], dtype=torch.int32)
        self._acc_dev.copy_(self._acc_host, non_blocking=True)
        b, save, st = L.lin_buf(self), L.lin_save(self), ptr(self.status)
        for j, li in enumerate(self.lin_layers):
            lw, sv = self.weights.layer(li), save[j]
            native.call("cuteafd_short_conv4", ptr(sv["qkvz"]), ptr(lw.lin_conv), ptr(self.lin_carry[j]), ptr(md["state_slot"]), ptr(md["q_start"]),
                        ptr(self._acc_dev), ptr(b["conv"]), sh.n_seq, C, Nq, self.max_seqs, st, native.stream())
            native.call("cuteafd_gated_delta_step", ptr(sv["k"]), ptr(sv["k"]), ptr(sv["v"]), ptr(sv["g"]), ptr(sv["beta"]), ptr(self.lin_state[j]),
                        ptr(md["state_slot"]), ptr(md["q_start"]), ptr(self._acc_dev), ptr(b["o"]), None, sh.n_seq, Hv, pc, self.max_seqs, st,
                        native.stream())

    def _attention_layer(self, li: int, lw: LayerWeights, L: Lane, sh: StepShape):
        spec, a, T = self.spec, self.spec.attn, sh.T
        md = self.md
        if lw.lin_qkvz is not None:
            return self._linear_layer(li, lw, L, sh)
        xq = self._norm_in(lw, L, T)
        self._dense(lw.wqkv, xq, L.qkv, T)
        window = spec.layer_window(li)                # hybrid stacks: full and sliding-window layers differ in window, sink and theta
        ops.qk_norm_rope_kvwrite(L.qkv, md["positions"], md["slot_map"], lw.q_norm, lw.k_norm, self.kv[li], T,
                                 a.n_heads, a.n_kv_heads, a.head_dim, spec.layer_rope_theta(li), a.rope_interleaved, spec.rms_eps, self.status)
        fused_q = False
        if self.kv_tmaps is not None and sh.attn_splits == 1 and sh.max_q_len >= PREFILL_ATTN_MIN_Q > 0:
            # prefill chunks: 128-key tiles with the query tile in tensor memory (8 + 8 tcgen05.mma per 128 keys instead of
            # 2 x (8 + 4) of the 64-key decode kernel)
            native.call("cuteafd_gqa_prefill_attention", ptr(L.qkv), ptr(self.kv_tmaps[li]), ptr(md["page_table"]), ptr(md["kv_len"]), ptr(md["q_start"]),
                        ptr(md["q_len"]), ptr(lw.sink), ptr(L.attn), T, sh.n_seq, sh.max_q_len, L.qkv.shape[1], a.n_heads, a.n_kv_heads,
                        md["page_table"].shape[1], window, a.head_dim ** -0.5, ptr(self.status), native.stream())
        elif self.kv_tmaps is not None:
            fused_q = ops.paged_attention_tc(L.qkv, self.kv_tmaps[li], md["page_table"], md["kv_len"], md["q_start"], md["q_len"], L.attn,
                                             T=T, n_seq=sh.n_seq, max_q_len=sh.max_q_len, q_stride=L.qkv.shape[1], Hq=a.n_heads,
                                             Hkv=a.n_kv_heads, n_splits=sh.attn_splits, part_o=self.part_o, part_ml=self.part_ml,
                                             window=window, sink=lw.sink, status=self.status, quant=L.attn_q, inv_gs=lw.wo.inv_act_gs)
        else:
            ops.paged_attention(L.qkv, self.kv[li], md["page_table"], md["kv_len"], md["q_start"], md["q_len"], L.attn,
                                T=T, n_seq=sh.n_seq, max_q_len=sh.max_q_len, q_stride=L.qkv.shape[1], Hq=a.n_heads,
                                Hkv=a.n_kv_heads, D=a.head_dim, n_splits=sh.attn_splits, part_o=self.part_o, part_ml=self.part_ml,
                                window=window, sink=lw.sink)
        oq = L.attn_q if fused_q else self._quant(L.attn, L.attn_q, T, lw.wo.inv_act_gs)
        self._attn_out(li, lw, oq, L, T)
        self.launches_per_step += 2 + (1 if sh.attn_splits > 1 else 0)

    _ffn_in_quantised = False

    def _ffn_norm(self, lw: LayerWeights, L: Lane, T: int):
        """RMSNorm in front of the FFN block -> L.xn (router, dispatch and gather read bf16 rows); when a dense or shared expert
        with FP8 operands follows, its quantised input is written by the same launch."""
        if self.spec.hyper_streams:
            self._hc_boundary(L, T, lw.hc_ffn, lw.ffn_norm)
            self._ffn_in_quantised = False
            return
        fuse = L.xq.kind == KIND_FP8B and self.spec.hidden % 256 == 0 and lw.ws_gate is not None and lw.ws_gate.kind == KIND_FP8B
        ops.add_rmsnorm(L.x, None, lw.ffn_norm, L.xn, self.spec.rms_eps, rows=T, quant=L.xq if fuse else None)
        self._ffn_in_quantised = fuse
        self.launches_per_step += 1

    def _attn_out(self, li: int, lw: LayerWeights, oq: ActBuffer, L: Lane, T: int):
        """Output projection + residual (a tensor-parallel rank overrides this with partial sum + exchange)."""
        if self.spec.hyper_streams:
            self._dense(lw.wo, oq, L.sub, T)
            return
        self._dense(lw.wo, oq, L.x, T, residual=L.x)

    def _hc_boundary(self, L: Lane, T: int, hc: tuple, norm_w: torch.Tensor, head: bool = False):
        """Hyper-connections, one launch per sub-layer boundary: close the open sub-layer (spread its output over the four residual
        streams, mix the streams), open the next one (coefficients from 24 projections of the row) and hand its collapsed, normalised
        input to L.xn.  The step's first boundary spreads the embedding; the head's boundary has collapse weights only and also
        leaves the un-normalised hidden rows in L.x."""
        fn, scale, base = hc
        init = self._hc_pending == "init"
        native.call("cuteafd_mhc_boundary", ptr(L.res), ptr(L.x if init else L.sub), None if init else ptr(L.hc_coef), ptr(fn), ptr(scale), ptr(base),
                    ptr(norm_w), ptr(L.x) if head else None, ptr(L.xn), None if head else ptr(L.hc_coef), T, self.spec.hidden, 4 if head else 24,
                    1 if init else 0, self.spec.hyper_sinkhorn_iters, self.spec.rms_eps, native.stream())
        self._hc_pending = "sub"
        self.launches_per_step += 1

    def _ffn(self, lw: LayerWeights, L: Lane, T: int, out, residual):
        """Shared expert / dense FFN: out = residual + down(silu(gate x) * up x)."""
        s1, s_act = L.ffn_buf(self, lw.ws_gate.N)
        if self._ffn_in_quantised:                 # the FFN norm already wrote the FP8 operand (same launch)
            xq, self._ffn_in_quantised = L.xq, False
        else:
            xq = self._quant(L.xn, L.xq, T, lw.ws_gate.inv_act_gs)
        inter = lw.ws_gate.N
        if lw.ws_gate.kind == KIND_FP8B and s_act.kind == KIND_FP8B and inter % 256 == 0 and FP8_FUSE_GATE_UP:
            # no SwiGLU epilogue in the FP8 kernel, but gate and up read the same operand: ONE GEMM over the stacked weight, then
            # silu(g) * u straight into the FP8 operand of the down projection
            gu = getattr(lw, "ws_gate_up", None)
            if gu is None:
                gu = lw.ws_gate_up = ops.TcWeight.fuse_rows_fp8(lw.ws_gate, lw.ws_up)
            key = ("gu", inter)
            if key not in L.ffn_bufs:
                L.ffn_bufs[key] = torch.zeros(L.cap, 2 * inter, dtype=torch.bfloat16, device=self.device)
            s_gu = L.ffn_bufs[key]
            self._dense(gu, xq, s_gu, T)
            native.call("cuteafd_silu_mul_quant_fp8b", ptr(s_gu), ptr(s_gu) + inter * 2, ptr(s_act.data), ptr(s_act.sf), T, inter, 2 * inter, native.stream())
            self.launches_per_step += 1
        elif lw.ws_gate.kind == KIND_FP8B:    # two GEMMs + silu(g) * u
            key = ("up", lw.ws_gate.N)
            if key not in L.ffn_bufs:
                L.ffn_bufs[key] = torch.zeros_like(s1)
            s_up = L.ffn_bufs[key]
            self._dense(lw.ws_gate, xq, s1, T)
            self._dense(lw.ws_up, xq, s_up, T)
            self.launches_per_step += 1
            if s_act.kind == KIND_FP8B and s1.shape[1] % 256 == 0:       # silu(g) * u straight into the FP8 operand of the down projection
                native.call("cuteafd_silu_mul_quant_fp8b", ptr(s1), ptr(s_up), ptr(s_act.data), ptr(s_act.sf), T, s1.shape[1], s1.stride(0), native.stream())
            else:
                ops.silu_mul(s1[:T], s_up[:T], s1[:T])
                self._quant(s1, s_act, T, lw.ws_down.inv_act_gs)
        else:
            self._dense(lw.ws_gate, xq, s1, T, w_up=lw.ws_up)
            self._quant(s1, s_act, T, lw.ws_down.inv_act_gs)
        self._dense(lw.ws_down, s_act, out, T, residual=residual)

    def _moe_layer(self, lw: LayerWeights, L: Lane, T: int):
        spec, m = self.spec, self.spec.moe
        self._ffn_norm(lw, L, T)
        if lw.router is None:
            if self.spec.hyper_streams:
                self._ffn(lw, L, T, L.sub, None)
            else:
                self._ffn(lw, L, T, L.x, L.x)
            return
        e_lo, e_hi = self.expert_range
        fused = False
        simt = T <= 64 and lw.router.kind == KIND_BF16 and lw.router.G == 1 and L.xn.stride(0) == lw.router.K and os.environ.get("CUTEAFD_ROUTER_GEMM", "0") != "1"
        if simt and T * m.top_k <= 1024 and e_hi - e_lo <= 512 and m.n_experts <= 512 and ROUTER_FUSED:
            # decode / verify: logits, selection and packing in ONE launch (the block that finishes its expert's logits last selects and packs)
            ops.router_fused(L.xn, lw.router, L.router_logits, lw.router_bias, L.idx, L.wts, T, m.top_k, m.scoring, m.normalize, m.route_scale,
                             m.n_group, m.topk_group, pack={"src_token": L.src_token, "slot_row": L.slot_row, "counts": L.counts, "offsets": L.offsets,
                                                            "tiles": L.tiles, "n_tiles": L.n_tiles, "n_rows": L.n_rows, "e_lo": e_lo, "e_hi": e_hi,
                                                            "tn": L.tn_g, "max_tiles": L.max_tiles})
            self.launches_per_step -= 1
            fused = True
        elif simt:
            ops.router_logits(L.xn, lw.router, L.router_logits, T)         # SIMT dot products, one block per expert
            self.launches_per_step += 1
        else:
            self._dense(lw.router, L.xn_act, L.router_logits, T)
        if fused:
            pass
        elif T * m.top_k <= 1024 and e_hi - e_lo <= 512:     # decode / verify steps: select and pack in one launch
            ops.router_select_pack(L.router_logits, lw.router_bias, L.idx, L.wts, T, m.top_k, m.scoring, m.normalize, m.route_scale,
                                   m.n_group, m.topk_group, L.src_token, L.slot_row, L.counts, L.offsets, L.tiles, L.n_tiles, L.n_rows,
                                   e_lo, e_hi, L.tn_g, L.max_tiles)
            self.launches_per_step -= 1
        else:
            ops.router_select(L.router_logits, lw.router_bias, L.idx, L.wts, T, m.top_k, m.scoring, m.normalize, m.route_scale,
                              m.n_group, m.topk_group)
            ops.route_pack(L.idx, L.src_token, L.slot_row, L.counts, L.offsets, L.tiles, L.n_tiles, L.n_rows, T, m.top_k,
                           e_lo, e_hi, L.tn_g, L.max_tiles)
        rows = T * m.top_k
        if L.xs.kind == KIND_BF16:
            ops.gather_rows(L.xn, L.src_token, L.n_rows, L.xs.data, rows)
        else:
            ops.quant_fp4_rows(L.xn, L.xs, src_rows=L.src_token, n_rows_dev=L.n_rows, rows=rows, inv_gs=lw.w_gate.inv_act_gs)
        if L.h1_q.kind != KIND_BF16 and m.intermediate % 32 == 0:
            # FC1's epilogue writes silu(g) * u already quantised for FC2 (no bf16 round trip, no quantiser launch)
            ops.tc_linear(lw.w_gate, L.xs, None, rows=rows, w_up=lw.w_up, tiles=L.tiles, n_tiles=L.n_tiles, max_tiles=L.max_tiles,
                          status=self.status, quant_out=L.h1_q, inv_gs_out=lw.w_down.inv_act_gs)
        else:
            ops.tc_linear(lw.w_gate, L.xs, L.h1, rows=rows, w_up=lw.w_up, tiles=L.tiles, n_tiles=L.n_tiles, max_tiles=L.max_tiles,
                          status=self.status)
            if L.h1_q.kind != KIND_BF16:
                ops.quant_fp4_rows(L.h1, L.h1_q, n_rows_dev=L.n_rows, rows=rows, inv_gs=lw.w_down.inv_act_gs)
                self.launches_per_step += 1
        ops.tc_linear(lw.w_down, L.h1_q, L.y2, rows=rows, tiles=L.tiles, n_tiles=L.n_tiles, max_tiles=L.max_tiles, status=self.status)
        shared = None
        if lw.ws_gate is not None:
            self._ffn(lw, L, T, L.shared, None)
            shared = L.shared
        self._combine(L.y2, L.slot_row, L.wts, shared, L, T, m.top_k)
        self.launches_per_step += 6

    def forward(self, sh: StepShape):
        """Launch one step on the current stream.  Inputs come from the device meta block."""
        lane = None
        for item in self.program(sh):
            if isinstance(item, Lane):
                lane = item
        return lane

    def program(self, sh: StepShape):
        """The step as a generator of launches.  A rank of a multi-GPU layout yields the peer flags it is about to wait for
        before it launches the waiting kernel (a scheduler that runs several ranks' programs on one GPU resumes a program
        only when those flags have been published); the last item yielded is the result lane."""
        yield self._forward_single(sh)

    def _forward_single(self, sh: StepShape):
        spec, T = self.spec, sh.T
        L = self.lane(T)
        self._ensure_attn_scratch(sh)
        self.launches_per_step = 0
        self._pre_normed = False
        stage = getattr(self, "stage", None)        # a layer-range split: this engine holds a slice of the stack (parallel/pipeline.py)
        if stage is None or stage.first:
            ops.embed_gather(self.md["tokens"][:T], self.weights.embed, L.x, self.status)
            self.launches_per_step += 1
            self._apply_input_embeds(L.x, T)
        else:
            self.launches_per_step += stage.receive(L.x, T)         # the residual rows arrive from the stage before
        self._hc_pending = "init" if spec.hyper_streams else None
        import contextlib
        from ..utils.trace import nvtx
        timed = self.layer_clock is not None and not torch.cuda.is_current_stream_capturing()
        for li in range(spec.n_layers):
            lw = self.weights.layer(li)
            self._next_lw = self.weights.layer(li + 1) if li + 1 < spec.n_layers else None
            self._next_engram = self.engram is not None and (li + 1) in spec.engram_layers
            if self.engram is not None and li in spec.engram_layers:
                if self._pre_normed:
                    raise RuntimeError("engram layer behind a fused combine + norm: its input rows were normalised before the memory could be added")
                self.launches_per_step += self.engram.apply(spec.engram_layers.index(li), L.x, T)
            with (self.layer_clock.span(f"layer{li}") if timed else contextlib.nullcontext()), (nvtx(f"layer{li}") if self._nvtx else contextlib.nullcontext()):
                self._attention_layer(li, lw, L, sh)
                if self._l2_prefetch and self._next_lw is not None and getattr(self._next_lw, "wqkv", None) is not None:
                    ops.l2_prefetch(self._next_lw.wqkv.data)       # the next layer's first weights ride into L2 under this layer's experts
                self._moe_layer(lw, L, T)
        if stage is not None and not stage.last:
            self.launches_per_step += stage.send(L.x, T)            # hop to the next stage; the head runs on the last one
            return L
        if spec.hyper_streams:      # close the last block, collapse the streams for the head: hidden rows -> L.x, normalised -> L.xn
            self._hc_boundary(L, T, self.weights.hc_head, self.weights.final_norm, head=True)
        if sh.n_logits:
            if spec.hyper_streams:
                ops.gather_rows(L.xn, self.md["logit_rows"], None, L.xln, sh.n_logits)
            else:
                ops.gather_rows(L.x, self.md["logit_rows"], None, L.xl, sh.n_logits)
                ops.add_rmsnorm(L.xl, None, self.weights.final_norm, L.xln, spec.rms_eps, rows=sh.n_logits)
            ops.tc_linear(self.weights.lm_head, L.xln_act, L.logits, rows=sh.n_logits, status=self.status)
            ops.argmax_rows(L.logits, L.next_tok, rows=sh.n_logits, status=L.tok_status)
            self.launches_per_step += 4
        return L

    def _ensure_attn_scratch(self, sh: StepShape):
        a, T = self.spec.attn, sh.T
        if sh.attn_splits > 1:
            need = sh.attn_splits * T * a.n_heads
            if getattr(self, "part_o", None) is None or self.part_o.numel() < need * a.head_dim:
                self.part_o = torch.empty(need * a.head_dim, dtype=torch.float32, device=self.device)
                self.part_ml = torch.empty(need * 2, dtype=torch.float32, device=self.device)
        elif getattr(self, "part_o", None) is None:
            self.part_o = self.part_ml = None

    # ------------------------------------------------------------------ MTP draft module
    def mtp_forward(self, depth: int, sh: StepShape, prev_hidden: torch.Tensor) -> Lane:
        """One step of MTP module `depth` over the rows described by the device meta block (tokens, positions, KV
        slots, lengths - as for `forward`, with the draft layer's own row numbering).  prev_hidden [T, H] bf16 is the
        hidden state paired with each row.  Returns the draft lane: `.x` holds the module's output hidden of every
        row, `.next_tok` the arg-max token of the rows listed in md["logit_rows"].
        (Reference: the MTP head of the DeepSeek families, families/deepseek_v4/engine.rs:2047-2133; oracle
        `RefModel.mtp_forward`.)"""
        spec, T, H = self.spec, sh.T, self.spec.hidden
        enorm, hnorm, eh_proj, lw, norm = self.weights.mtp[depth]
        cap = next(c for c in (16, 64, 256, 1024, 4096, 16384) if T <= c)
        if cap not in self.mtp_lanes:
            L = Lane(self, cap)
            L.cat = torch.zeros(cap, 2 * H, dtype=torch.bfloat16, device=self.device)
            L.cat_act = ActBuffer.wrap_bf16(L.cat, L.tn)
            self.mtp_lanes[cap] = L
        L = self.mtp_lanes[cap]
        self._ensure_attn_scratch(sh)
        ops.embed_gather(self.md["tokens"][:T], self.weights.embed, L.xl, self.status)
        ops.add_rmsnorm(L.xl, None, enorm, L.xln, spec.rms_eps, rows=T)
        L.cat[:T, :H].copy_(L.xln[:T])
        ops.add_rmsnorm(prev_hidden.contiguous(), None, hnorm, L.xln, spec.rms_eps, rows=T)
        L.cat[:T, H:].copy_(L.xln[:T])
        ops.tc_linear(eh_proj, L.cat_act, L.x, rows=T, status=self.status)
        self._pre_normed, self._next_lw = False, None
        self._attention_layer(spec.n_layers + depth, lw, L, sh)
        self._moe_layer(lw, L, T)
        if sh.n_logits:
            ops.gather_rows(L.x, self.md["logit_rows"], None, L.xl, sh.n_logits)
            ops.add_rmsnorm(L.xl, None, norm, L.xln, spec.rms_eps, rows=sh.n_logits)
            ops.tc_linear(self.weights.lm_head, L.xln_act, L.logits, rows=sh.n_logits, status=self.status)
            ops.argmax_rows(L.logits, L.next_tok, rows=sh.n_logits, status=L.tok_status)
        return L

    def mtp_run(self, depth: int, sh: StepShape, prev_hidden: torch.Tensor, use_graph: bool = True) -> Lane:
        """`mtp_forward`, replayed from a CUDA graph per (depth, shape) when `use_graph`: the hidden rows are first copied
        into a buffer of fixed address that the captured step reads."""
        if not use_graph:
            return self.mtp_forward(depth, sh, prev_hidden)
        cap = next(c for c in (16, 64, 256, 1024, 4096, 16384) if sh.T <= c)
        key = ("mtp", depth, cap)
        buf = self.graphs.get(key)
        if buf is None:
            buf = self.graphs[key] = torch.zeros(cap, self.spec.hidden, dtype=torch.bfloat16, device=self.device)
        buf[:sh.T].copy_(prev_hidden[:sh.T])
        gkey = ("mtp", depth) + sh.key()
        g = self.graphs.get(gkey)
        hook = getattr(self, "on_mtp_step", None)
        if g is None:
            lane = self.mtp_forward(depth, sh, buf)          # warm-up outside capture (announces itself on multi-rank runs)
            torch.cuda.synchronize()
            self.on_mtp_step = None                          # the capture launches nothing: nobody must be told
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    lane = self.mtp_forward(depth, sh, buf)
            finally:
                if hook is not None:
                    self.on_mtp_step = hook
                else:
                    del self.on_mtp_step
            self.graphs[gkey] = g = (graph, lane)
            self.graph_captures += 1
        if hook:
            hook(depth, sh)
        g[0].replay()
        return g[1]

    # ------------------------------------------------------------------ CUDA graphs
    def attn_splits_for(self, n_seq: int, max_q_len: int, max_kv: int) -> int:
        a = self.spec.attn
        tpt = max(1, (128 if self.kv_tmaps is not None else 16) // (a.n_heads // a.n_kv_heads))
        ctas = a.n_kv_heads * n_seq * (-(-max_q_len // tpt))
        pages = max(1, -(-max_kv // PAGE))
        if max_q_len > 16:
            return 1
        # fill the machine in ONE wave (two CTAs per SM); a ragged second wave doubles the kernel's time
        return max(1, min(pages, 32, (2 * self.sm_count) // ctas))

    def run(self, sh: StepShape, use_graph: bool = True) -> Lane:
        """Run a step, replaying a captured graph when one exists for this exact shape.  A new shape in graph mode executes
        twice (an eager warm-up, then the first replay of the capture); `on_real_step(sh, replay)` is told of each execution."""
        hook = getattr(self, "on_real_step", None)      # multi-rank runs announce every executed step to their peers
        if not use_graph:
            if hook:
                hook(sh, False)
            self.census.ran_eager(sh.key())
            return self.forward(sh)
        key = sh.key()
        if key not in self.graphs:
            if hook:
                hook(sh, False)
            # the warm-up execution must not advance the recurrent state of linear-attention layers (KV writes repeat harmlessly)
            saved = (self.lin_state.clone(), self.lin_carry.clone()) if getattr(self, "lin_layers", None) else None
            self.forward(sh)                    # warm-up launch outside capture (loads modules, sizes scratch)
            torch.cuda.synchronize()
            if saved is not None:
                self.lin_state.copy_(saved[0])
                self.lin_carry.copy_(saved[1])
            self._capture(sh)
        if hook:
            hook(sh, True)
        g = self.graphs[key]
        g[0].replay()
        self.census.replayed(key)
        self.launches_per_step = g[2]
        return g[1]

    def _capture(self, sh: StepShape):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            lane = self.forward(sh)
        self.graphs[sh.key()] = (graph, lane, self.launches_per_step)
        self.graph_captures += 1
        self.census.captured(sh.key(), self.launches_per_step)

    def execute(self, sh: StepShape, replay: bool) -> Lane:
        """Exactly ONE execution of a step, eager or from its graph (captured first if need be, which executes nothing): what
        a rank does that mirrors another rank's `run` call by call."""
        if not replay:
            return self.forward(sh)
        if sh.key() not in self.graphs:
            torch.cuda.synchronize()
            self._capture(sh)
        g = self.graphs[sh.key()]
        g[0].replay()
        self.launches_per_step = g[2]
        return g[1]

    def layer_times(self) -> dict:
        """Device milliseconds per layer of the eager steps since the last call (needs CUTEAFD_LAYER_CLOCK=1; synchronises)."""
        if self.layer_clock is None:
            return {}
        torch.cuda.synchronize()
        return self.layer_clock.collect()

    def check_status(self):
        word = int(self.status[0])
        if word:
            from ..ops.native import decode_status
            raise RuntimeError(f"device status: {decode_status(word)}")
        if self.engram is not None:
            self.engram.check_status()
