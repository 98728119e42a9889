"""Attention/FFN disaggregation inside one NVSwitch node.

Roles.  An ATTENTION rank holds embeddings, attention (its share of the heads when the group is tensor-parallel), router,
shared expert, LM head and the KV cache; an EXPERT rank holds a contiguous range of routed experts.  In the split layouts
the two sets of ranks are disjoint (the named layout: attention TP2 + experts on the other GPUs); in the colocated layout
every GPU plays both roles for its own sequences (data-parallel attention, expert-parallel FFN).

Lanes.  Every (attention group, micro-batch) pair owns a LANE on every expert rank: a token-major slab for its quantised
rows, its routing table, its token count and its flag words.  Per MoE layer:

  attention rank:  ... router top-k -> DISPATCH: quantise each of my tokens once and store the row into the lane slab of every
                   expert rank that owns one of its experts (+ routing row and token count to all, + flag) -> shared expert
                   meanwhile -> [wait COMBINE flags inside the kernel] ordered weighted top-k sum + shared + residual (+ the
                   next layer's input norm)
  expert rank:     [wait DISPATCH flags inside the kernel] route pack over the lane table(s) -> gather rows into expert
                   order -> grouped FC1 (SwiGLU, FP4 output) -> grouped FC2 (tcgen05, TMA from LOCAL memory) -> COMBINE:
                   store each output row into [token][slot] of the lane's attention ranks (+ flag)
  attention TP2:   wo partial -> push to the partner + flag -> wait -> add in rank order (bit-identical on both ranks)

Overlap.  With `n_micro` = 2 an attention rank cuts a decode / verify step into two micro-batches and interleaves their
layer segments (combine of layer l-1, attention of layer l, dispatch of layer l), so one micro-batch's experts run while
the other micro-batch is in attention (reference: layer-major prefill lanes, families/deepseek_v4/engine.rs:1119-1191).
Expert ranks either run the lanes one after the other as they arrive (`merged=False`, pipelined layouts) or wait for all
lanes and run them as ONE grouped GEMM that streams each expert's weights once (`merged=True`, the colocated layout).

Programs.  A rank's step is a generator of launches (`program`) that yields the peer flag addresses it is about to wait
for.  A real rank simply exhausts it; `LocalWorld` runs several ranks' programs round-robin on ONE GPU, resuming a program
only when the flags it waits for have been published by launches already in the stream - the same kernels and the same
protocol, testable without a second GPU.

`comm="p2p"` uses the peer-memory kernels of `csrc/peer.cu`; `comm="nccl"` is the baseline that only calls NCCL
(broadcast activations + routes, all-reduce expert partial sums, all-reduce attention partials).

Reference: the coordinator/Spark split (families/deepseek_v4/engine.rs:1036-1191, 2047-2133), TP2 head split
(engine.rs:1524-1552), ordered combine (native/shared/include/cuteafd_experts.h:136-183).
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from .. import ops
from ..config import Deployment, ModelSpec
from ..engine.engine import ROUTER_FUSED, Engine, Lane, StepShape
from ..models.weights import DeviceWeights
from ..ops import ActBuffer, KIND_BF16, KIND_BY_NAME, KIND_NVFP4, KIND_W4A8, native, pick_tn
from . import peer_ops
from .shard import attention_masters, expert_masters, local_attention_spec
from .symm import SymmetricBlock

PH_DISPATCH, PH_COMBINE, PH_TP = 0, 1, 2
NFLAG = 32          # flag words per (phase, layer): dispatch lane * tp + tp_rank, combine micro * 8 + expert rank, TP micro * 2 + tp_rank
# A TP pair splits the LM head over the vocabulary: each rank reads half of the head's weights and the halves of the logit rows are
# exchanged over peer memory (reference: families/deepseek_v41/v41_target_head/distributed.rs, the vocab-sharded target head).
VOCAB_PARALLEL = os.environ.get("CUTEAFD_VOCAB_PARALLEL", "1") == "1"
HEAD_ROWS = 512     # logit rows per step the exchange buffers hold
# GEMM epilogues can store straight into peer memory (output projection -> TP partner) and publish the flag themselves
FUSED_PEER = os.environ.get("CUTEAFD_FUSED_PEER", "0") == "1"


@dataclass(frozen=True)
class LanePlan:
    """Static lane geometry shared by all ranks of a run."""
    dep: Deployment
    t_cap: int                  # token rows a lane can carry per step
    n_micro: int = 1            # micro-batches per attention group
    merged: bool = False        # expert ranks run all lanes as one grouped GEMM (needs every lane each layer)
    # Expert TP: every expert rank holds a slice of the intermediate dimension of EVERY expert (instead of whole experts of a
    # range); rows are broadcast to all expert ranks, each returns per-route partial sums, the attention rank adds the ranks in
    # fixed order.  One token's experts then stream from all expert ranks at once - the layout for very small batches.
    expert_tp: bool = False

    @property
    def planes(self) -> int:
        """Receive planes per micro-batch on an attention rank (one per expert rank under expert TP)."""
        return self.dep.ep if self.expert_tp else 1

    @property
    def n_lanes(self) -> int:
        return self.dep.attn_groups * self.n_micro

    def lane(self, group: int, micro: int) -> int:
        return group * self.n_micro + micro

    def check(self):
        if self.n_lanes * self.dep.tp > 8:
            raise ValueError(f"{self.n_lanes} lanes x tp {self.dep.tp} exceed the 8 destinations a combine kernel addresses")
        if self.n_micro > 4 or self.dep.ep > 8:
            raise ValueError("at most 4 micro-batches and 8 expert ranks")


def n_flag_layers(spec: ModelSpec) -> int:
    return spec.n_layers + spec.mtp_layers


def flag_offset(spec: ModelSpec, phase: int, layer: int, slot: int) -> int:
    return ((phase * n_flag_layers(spec) + layer) * NFLAG + slot) * 4


def sf_row_bytes(H: int, kind: int) -> int:
    """Bytes of block scales per dispatched row (padded to whole pipeline stages of the GEMM that reads them)."""
    if kind == KIND_BF16:
        return 0
    if kind == KIND_W4A8:
        return -(-H // 128) * 4
    return -(-H // 256) * (256 // (16 if kind == KIND_NVFP4 else 32))


def payload_row_bytes(H: int, kind: int) -> int:
    return H * 2 if kind == KIND_BF16 else (H if kind == KIND_W4A8 else H // 2)


def block_regions(spec: ModelSpec, plan: LanePlan, expert_kind: int) -> dict:
    """Symmetric regions (same layout on every rank; each role uses its part)."""
    H, k, L, t = spec.hidden, spec.moe.top_k, plan.n_lanes, plan.t_cap
    row_bytes = payload_row_bytes(H, expert_kind)
    return {
        "slab_q": L * t * row_bytes, "slab_sf": max(256, L * t * sf_row_bytes(H, expert_kind)), "idx": L * t * k * 4, "lane_T": 256,
        "y_recv": plan.n_micro * plan.planes * t * k * H * 2, "tp_recv": plan.n_micro * 2 * t * H * 2,
        "flags": 3 * n_flag_layers(spec) * NFLAG * 4,
        "head_recv": min(t, HEAD_ROWS) * max(head_split(spec.vocab)) * 4 if plan.dep.tp == 2 and VOCAB_PARALLEL else 256,
    }


def head_split(vocab: int) -> tuple[int, int]:
    """Vocabulary shares of the two ranks of a TP pair (the cut sits on a 128-row weight tile)."""
    v0 = max(128, (vocab // 2) // 128 * 128)
    return v0, vocab - v0


def make_block(spec: ModelSpec, plan: LanePlan, expert_kind: int, rank: int, device, group=None) -> SymmetricBlock:
    plan.check()
    return SymmetricBlock(block_regions(spec, plan, expert_kind), device, group, rank, plan.dep.world)


class PtrTable:
    """ctypes array of device addresses (what the kernels take) plus the same addresses as Python ints (what the
    single-GPU scheduler tracks)."""

    def __init__(self, addrs):
        import ctypes as C
        self.addrs = [int(a) for a in addrs]
        self.arr = (C.c_void_p * len(self.addrs))(*self.addrs)


class MicroCtx:
    """One micro-batch of a step on an attention rank: its rows, its views of the step inputs, its activation lane."""

    def __init__(self, mb: int, sh: StepShape, md: dict, L: Lane, t0: int, s0: int):
        self.mb, self.sh, self.md, self.L, self.t0, self.s0 = mb, sh, md, L, t0, s0
        self.T = sh.T
        self.pre_normed = False
        self.pending = None         # MoE layer whose combine is outstanding
        self.shared = None


class AttnRankEngine(Engine):
    """Engine of one attention rank: local heads, replicated residual stream, routed experts remote."""

    def __init__(self, spec: ModelSpec, plan: LanePlan, rank: int, device, *, n_pages: int, max_seqs: int, max_pages_per_seq: int, comm: str,
                 block: SymmetricBlock | None, expert_kind: int, act_gs: float = 1.0 / 64, seed: int = 1, masters: dict | None = None):
        dep = plan.dep
        self.full_spec, self.plan, self.dep, self.rank, self.comm, self.block = spec, plan, dep, rank, comm, block
        self.tp, self.tp_rank = dep.tp, dep.attn_ranks.index(rank) % dep.tp
        if spec.hyper_streams:
            raise NotImplementedError("hyper-connections run on the single-GPU engine (the lanes carry one residual stream)")
        if spec.engram_layers:
            raise NotImplementedError("models with an n-gram memory run on the single-GPU engines (the step inputs of the lanes carry no table addresses)")
        if self.tp > 1 and spec.attn.linear_every:
            raise NotImplementedError("hybrid stacks with linear-attention layers run with attention TP 1 (data-parallel attention ranks)")
        self.group = dep.group_of(rank)
        self.group_ranks = dep.group_ranks(self.group)
        lw = self._make_weights(spec, device, seed, act_gs, masters)
        super().__init__(lw, n_pages=n_pages, max_seqs=max_seqs, max_pages_per_seq=max_pages_per_seq, device=device)
        self.remote_kind = expert_kind
        self.t_cap = plan.t_cap
        m, H, k = spec.moe, spec.hidden, spec.moe.top_k
        self.ctl = torch.zeros(4, dtype=torch.int32, device=device)
        self.done = torch.zeros(8, dtype=torch.int32, device=device)
        self.inv_gs = torch.tensor([1.0 / act_gs], dtype=torch.float32, device=device)
        self.expert_inv_gs: dict = {}       # layer -> fp32[1] activation scale of that layer's routed experts (checkpoints)
        self.identity_rows = torch.arange(plan.t_cap * k, dtype=torch.int32, device=device).view(plan.t_cap, k).contiguous()
        self._iota = torch.arange(max(plan.t_cap, 16), dtype=torch.int32, device=device)
        self._qstart: dict = {}
        self._ctx_cache: dict = {}
        self._tp_pending = None
        self.local_worker = None            # colocated layout: the ExpertRankWorker of this same GPU
        self.part = torch.zeros(plan.t_cap, H, dtype=torch.bfloat16, device=device)
        if block is not None:
            self.sf_ld = sf_row_bytes(H, expert_kind)
            row_bytes = payload_row_bytes(H, expert_kind)
            t = plan.t_cap
            self.lane_tbls = []
            for mb in range(plan.n_micro):
                lane = plan.lane(self.group, mb)
                tb = lambda name, off: PtrTable([block.peer_ptr(r, name, off) for r in dep.expert_ranks])
                self.lane_tbls.append({"slab_q": tb("slab_q", lane * t * row_bytes), "slab_sf": tb("slab_sf", lane * t * self.sf_ld) if self.sf_ld else None,
                                       "idx": tb("idx", lane * t * k * 4), "lane_T": tb("lane_T", lane * 4), "lane": lane})
            self.y_recv = block.local("y_recv", torch.bfloat16, (plan.n_micro, plan.planes * t * k, H))
            if plan.expert_tp:
                # pseudo-slots of the rank-ordered sum: slot s of rank e reads row e * (t * k) + token * k + s
                P = plan.planes
                base = self.identity_rows.view(t, k, 1) + (torch.arange(P, dtype=torch.int32, device=device) * (t * k)).view(1, 1, P)
                self.identity_rows_tp = base.reshape(t, k * P).contiguous()
            self.tp_recv = block.local("tp_recv", torch.bfloat16, (plan.n_micro, 2, t, H))
        self.vocab_parallel = False
        head = self.weights.lm_head
        if (VOCAB_PARALLEL and self.tp == 2 and comm == "p2p" and block is not None and head is not None and head.kind == KIND_BF16
                and spec.vocab % 8 == 0 and spec.vocab >= 256):
            from ..ops import TcWeight, encode_tmap
            self.vocab_parallel = True
            self.head_w = head_split(spec.vocab)
            lo = 0 if self.tp_rank == 0 else self.head_w[0]
            rows = head.data[:, lo:lo + self.head_w[self.tp_rank]].contiguous()       # my share of the head; the full matrix is dropped
            self.weights.lm_head = TcWeight(KIND_BF16, 1, rows.shape[1], rows.shape[2], rows, encode_tmap(rows, 128))
            del head
            self.head_rows = min(plan.t_cap, HEAD_ROWS)
            self.head_stage = torch.zeros(self.head_rows, self.head_w[self.tp_rank], dtype=torch.float32, device=device)
            self.head_recv = block.local("head_recv", torch.float32, (self.head_rows, self.head_w[1 - self.tp_rank]))

    def _head(self, L, n: int, mb: int, t0: int, flag_layer: int):
        """Logit rows of `n` gathered, normalised rows in L.xln -> L.logits and L.next_tok.  On a TP pair every rank multiplies by its share
        of the vocabulary only (half the weight bytes per rank) and the two shares are exchanged over peer memory: both ranks end up
        with the same full rows, so selection, sampling and grammar masks are unchanged."""
        if not self.vocab_parallel:
            ops.tc_linear(self.weights.lm_head, L.xln_act, L.logits, rows=n, status=self.status)
            ops.argmax_rows(L.logits, L.next_tok, rows=n, status=L.tok_status)
            self.launches_per_step += 2
            return
        if t0 + n > self.head_rows:
            raise ValueError(f"vocabulary-parallel head: {t0 + n} logit rows in a step (limit {self.head_rows}; CUTEAFD_VOCAB_PARALLEL=0 lifts it)")
        peer, w = self.group_ranks[1 - self.tp_rank], self.head_w
        mine = self.head_stage[t0:t0 + n]
        ops.tc_linear(self.weights.lm_head, L.xln_act, mine, rows=n, status=self.status)
        dst = self.block.peer_ptr(peer, "head_recv", t0 * w[self.tp_rank] * 4)
        flag = self._flag(peer, PH_TP, flag_layer, 16 + mb * 2 + self.tp_rank)
        peer_ops.push_bytes(mine, dst, n * w[self.tp_rank] * 4, flag, self.ctl, 0, self.done[0:1])
        peer_ops.note_published([flag])
        flag = self._flag(self.rank, PH_TP, flag_layer, 16 + mb * 2 + (1 - self.tp_rank))
        yield [flag]
        peer_ops.wait_concat(mine, self.head_recv[t0:t0 + n], L.logits, n, w[0], w[1], self.tp_rank, flag, self.ctl, 0, self.status)
        ops.argmax_rows(L.logits, L.next_tok, rows=n, status=L.tok_status)
        self.launches_per_step += 4

    def _make_weights(self, spec, device, seed, act_gs, masters):
        """This rank's share: attention heads split over the TP group, router / shared expert / dense layers replicated, no
        routed experts.  From masters the shard is cut before quantisation; random bf16 projections are cut out of the
        full-model random weights of the same seed (both reproduce the single-GPU model exactly); random block-scaled
        projections are generated per shard (synthetic benchmarks)."""
        if masters is not None:
            return DeviceWeights.from_masters(local_attention_spec(spec, self.tp), attention_masters(spec, masters, self.tp, self.tp_rank), device, act_gs)
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

    # ------------------------------------------------------------------ flags
    def _flag(self, rank: int, phase: int, layer: int, slot: int) -> int:
        return self.block.peer_ptr(rank, "flags", flag_offset(self.full_spec, phase, layer, slot))

    # ------------------------------------------------------------------ output projection with the TP all-reduce
    def _attn_out(self, li, lw, oq, L, T):
        if self.tp == 1:
            return super()._attn_out(li, lw, oq, L, T)
        c = self._cur
        H, peer, buf = self.full_spec.hidden, self.group_ranks[1 - self.tp_rank], li & 1
        if self.comm == "nccl":
            import torch.distributed as dist
            self._dense(lw.wo, oq, self.part, T)
            dist.all_reduce(self.part[:T], group=self.tp_group)
            L.x[:T] += self.part[:T]
            return
        dst = self.block.peer_ptr(peer, "tp_recv", ((c.mb * 2 + buf) * self.t_cap) * H * 2)
        flag = self._flag(peer, PH_TP, li, c.mb * 2 + self.tp_rank)
        if FUSED_PEER and lw.wo.kind != ops.KIND_FP8B:
            # the projection's epilogue writes my partial sum locally AND into the partner's landing buffer, then raises
            # its flag: GEMM -> exchange in one kernel; the wait + ordered add follows
            splits = self._splits(lw.wo.N, lw.wo.K, T, oq.tn, lw.wo.kind)
            ops.tc_linear(lw.wo, oq, self.part, rows=T, splits=splits, status=self.status,
                          peer={"y": [dst], "ld": H, "row_map": None, "flags": [flag], "ctl": self.ctl, "done": self.done[2:3]})
            self.launches_per_step += 1
        else:
            self._dense(lw.wo, oq, self.part, T)              # partial sum over my heads, then the TP exchange
            peer_ops.push_bytes(self.part, dst, T * H * 2, flag, self.ctl, 0, self.done[0:1])
            self.launches_per_step += 1
        peer_ops.note_published([flag])
        self._tp_pending = (li, T, buf)

    def _tp_finish(self, c: MicroCtx):
        """x += part(rank 0) + part(rank 1), identical bits on both ranks."""
        li, T, buf = self._tp_pending
        self._tp_pending = None
        flag = self._flag(self.rank, PH_TP, li, c.mb * 2 + (1 - self.tp_rank))
        yield [flag]
        peer_ops.wait_add(self.part, self.tp_recv[c.mb, buf], c.L.x, c.L.x, T * self.full_spec.hidden, self.tp_rank, flag, self.ctl, 0, self.status)
        self.launches_per_step += 1

    # ------------------------------------------------------------------ micro-batch contexts
    def _mb_lane(self, cap_rows: int, mb: int, main: Lane, t0: int) -> Lane:
        """Activation lane of a micro-batch; its residual stream, logits and token outputs are views into the step's main lane,
        so the caller reads one contiguous result whatever the cut."""
        cap = next(c for c in (16, 64, 256, 1024, 4096, 16384) if cap_rows <= c)
        key = ("mb", cap, mb, main.cap, t0)
        if key not in self.lanes:
            L = Lane(self, cap)
            n = min(cap, main.cap - t0)
            L.logits, L.next_tok, L.tok_status = main.logits[t0:t0 + n], main.next_tok[t0:t0 + n], main.tok_status[t0:t0 + n]
            L.x = main.x[t0:t0 + n]         # the residual stream too: callers read the step's hidden rows from the main lane
            self.lanes[key] = L
        return self.lanes[key]

    def _routing_bufs(self, L: Lane):
        if getattr(L, "r_idx", None) is None:
            m, dev = self.full_spec.moe, self.device
            L.r_logits = torch.zeros(L.cap, m.n_experts, dtype=torch.float32, device=dev)
            L.r_idx = torch.zeros(L.cap, m.top_k, dtype=torch.int32, device=dev)
            L.r_wts = torch.zeros(L.cap, m.top_k, dtype=torch.float32, device=dev)
        return L

    def _contexts(self, sh: StepShape) -> list:
        """Cuts a step into the plan's micro-batches at a sequence boundary when its layout is regular (`sh.uniform`, logits
        for no row or for every row); any other step runs as one micro-batch and the remaining lanes carry zero tokens (the
        expert ranks still see every lane every layer)."""
        key = sh.key()
        if key in self._ctx_cache:
            ctxs = self._ctx_cache[key]
            for c in ctxs:
                c.pre_normed, c.pending, c.shared = False, None, None
            return ctxs
        if sh.T > self.t_cap * (self.plan.n_micro if sh.uniform else 1):
            raise ValueError(f"step of {sh.T} rows exceeds the lane capacity {self.t_cap}")
        md, nm = self.md, self.plan.n_micro
        main = self.lane(sh.T)
        cut = nm > 1 and self.comm == "p2p" and sh.uniform and sh.n_seq >= nm and sh.n_logits in (0, sh.T) and sh.T == sh.n_seq * sh.max_q_len
        ctxs = []
        if not cut:
            ctxs.append(MicroCtx(0, sh, md, main, 0, 0))
            for mb in range(1, nm if self.comm == "p2p" else 1):
                ctxs.append(MicroCtx(mb, StepShape(0, 0, 1, 0, 1), md, main, 0, 0))
        else:
            q, per = sh.max_q_len, -(-sh.n_seq // nm)
            if q not in self._qstart:
                self._qstart[q] = (torch.arange(self.max_seqs, dtype=torch.int32, device=self.device) * q).contiguous()
            for mb in range(nm):
                s0, s1 = min(sh.n_seq, mb * per), min(sh.n_seq, (mb + 1) * per)
                t0, t1 = s0 * q, s1 * q
                nl = (t1 - t0) if sh.n_logits else 0
                splits = min(32, sh.attn_splits * nm) if sh.attn_splits > 1 else 1
                msh = StepShape(T=t1 - t0, n_seq=s1 - s0, max_q_len=q, n_logits=nl, attn_splits=splits, uniform=True)
                mmd = {"tokens": md["tokens"][t0:t1], "positions": md["positions"][t0:t1], "slot_map": md["slot_map"][t0:t1],
                       "logit_rows": self._iota[:max(nl, 1)], "kv_len": md["kv_len"][s0:s1], "q_start": self._qstart[q][:max(s1 - s0, 1)],
                       "q_len": md["q_len"][s0:s1], "state_slot": md["state_slot"][s0:s1], "page_table": md["page_table"][s0:s1]}
                ctxs.append(MicroCtx(mb, msh, mmd, self._mb_lane(max(t1 - t0, 1), mb, main, t0), t0, s0))
        for c in ctxs:
            c.main = main
        self._ctx_cache[key] = ctxs
        return ctxs

    def set_inputs(self, *args, **kw):
        n = super().set_inputs(*args, **kw)
        hook = getattr(self, "on_inputs", None)     # a leader forwards the packed input block to the ranks that mirror its steps
        if hook:
            hook(self.meta_host)
        return n

    def load_inputs(self, block: torch.Tensor):
        """Mirror side of `set_inputs`: `block` is the leader's packed int32 input block (same engine geometry)."""
        need = (block.numel() - 4 * self.max_seqs - self.max_seqs * self.max_pages) // 4
        self._ensure_meta(need)
        if block.numel() != self.meta_host.numel():
            raise ValueError(f"input block of {block.numel()} words does not fit this engine's layout ({self.meta_host.numel()})")
        self.meta_host.copy_(block)
        self.meta_dev.copy_(self.meta_host, non_blocking=True)

    def _ensure_meta(self, T: int):
        before = self._meta_cap
        super()._ensure_meta(T)
        if self._meta_cap != before:
            self._ctx_cache = {}        # the views of the step inputs moved

    def _bind(self, c: MicroCtx):
        self._cur, self.md, self._pre_normed = c, c.md, c.pre_normed

    def _unbind(self, c: MicroCtx):
        c.pre_normed = self._pre_normed

    # ------------------------------------------------------------------ the step
    def program(self, sh: StepShape):
        spec = self.spec
        if sh.defer_state:
            raise NotImplementedError("speculative steps over linear-attention layers run on the single-GPU engine")
        self._keep = []
        self.launches_per_step = 0
        base_md = self.md
        if self.block is not None and self.comm == "p2p":
            peer_ops.step_begin(self.ctl)
            if self.local_worker is not None:
                self.local_worker.begin()
        ctxs = self._contexts(sh)
        for c in ctxs:
            self._ensure_attn_scratch(c.sh)
        for c in ctxs:
            if c.T:
                ops.embed_gather(c.md["tokens"][:c.T], self.weights.embed, c.L.x, self.status)
                self.launches_per_step += 1
        try:
            for li in range(spec.n_layers):
                lw = self.weights.layer(li)
                for c in ctxs:
                    self._bind(c)
                    yield from self._segment(li, lw, c)
                    self._unbind(c)
                if self.local_worker is not None:       # colocated layout: this GPU's share of the experts, same stream
                    yield from self.local_worker.layer_program(li)
            for c in ctxs:
                self._bind(c)
                if c.pending is not None:
                    yield from self._moe_back(c, None)
                if c.T and c.sh.n_logits:
                    L, n = c.L, c.sh.n_logits
                    ops.gather_rows(L.x, c.md["logit_rows"], None, L.xl, n)
                    ops.add_rmsnorm(L.xl, None, self.weights.final_norm, L.xln, spec.rms_eps, rows=n)
                    self.launches_per_step += 2
                    yield from self._head(L, n, c.mb, c.t0 if c.sh.n_logits == c.sh.T else 0, spec.n_layers - 1)
                self._unbind(c)
        finally:
            self.md = base_md
        yield ctxs[0].main

    def _segment(self, li: int, lw, c: MicroCtx):
        """One layer of one micro-batch: combine of the previous MoE layer, attention, TP exchange, FFN front."""
        if c.pending is not None:
            yield from self._moe_back(c, lw)
        if c.T:
            self._next_lw = None
            self._attention_layer(li, lw, c.L, c.sh)
            if self._tp_pending is not None:
                yield from self._tp_finish(c)
        self._ffn_front(li, lw, c)

    def _ffn_front(self, li: int, lw, c: MicroCtx):
        spec, m, L, T = self.full_spec, self.full_spec.moe, c.L, c.T
        if lw.router is None:
            if T:
                self._next_lw = None
                Engine._moe_layer(self, lw, L, T)          # dense FFN layer: all local
            return
        if T:
            self._routing_bufs(L)
            self._ffn_norm(lw, L, T)
            self.launches_per_step -= 1
            simt = T <= 64 and lw.router.kind == KIND_BF16 and lw.router.G == 1 and L.xn.stride(0) == lw.router.K \
                and os.environ.get("CUTEAFD_ROUTER_GEMM", "0") != "1"
            if simt and ROUTER_FUSED and m.n_experts <= 512:
                # logits + selection in one launch (same arithmetic as the single-GPU engine's fused router: token-exact layouts)
                ops.router_fused(L.xn, lw.router, L.r_logits, lw.router_bias, L.r_idx, L.r_wts, T, m.top_k, m.scoring, m.normalize, m.route_scale,
                                 m.n_group, m.topk_group)
                self.launches_per_step += 2
            else:
                if simt:
                    ops.router_logits(L.xn, lw.router, L.r_logits, T)
                else:
                    self._dense(lw.router, L.xn_act, L.r_logits, T)
                    self.launches_per_step -= 1
                ops.router_select(L.r_logits, lw.router_bias, L.r_idx, L.r_wts, T, m.top_k, m.scoring, m.normalize, m.route_scale, m.n_group, m.topk_group)
                self.launches_per_step += 3
        if self.comm == "nccl":
            if T:
                self._moe_nccl(li, lw, L, T)
            return
        # my share of the tokens (the other attention rank of the group sends the rest; both hold identical activations)
        per = -(-T // self.tp)
        t0, t1 = min(T, self.tp_rank * per), min(T, (self.tp_rank + 1) * per)
        tb = self.lane_tbls[c.mb]
        flags = PtrTable([self._flag(r, PH_DISPATCH, li, tb["lane"] * self.tp + self.tp_rank) for r in self.dep.expert_ranks])
        self._keep.append(flags)
        x = L.xn if T else self.part
        idx = L.r_idx if T else self.identity_rows
        peer_ops.dispatch_tok_push(x, idx, tb["slab_q"].arr, tb["slab_sf"].arr if tb["slab_sf"] else None, tb["idx"].arr, tb["lane_T"].arr,
                                   flags.arr, self.expert_inv_gs.get(li, self.inv_gs), self.ctl, self.done[1:2], t0, t1, T, spec.hidden, m.top_k,
                                   m.n_experts, self.dep.ep, self.remote_kind, self.sf_ld, 0, self.status, broadcast=self.plan.expert_tp)
        peer_ops.note_published(flags.addrs)
        self.launches_per_step += 1
        c.shared = None
        if T and lw.ws_gate is not None:
            self._ffn(lw, L, T, L.shared, None)
            c.shared = L.shared
        c.pending = li

    def _moe_back(self, c: MicroCtx, next_lw):
        """Second half of a MoE layer: wait for the expert ranks' rows, ordered weighted sum + shared + residual."""
        li, L, T = c.pending, c.L, c.T
        c.pending = None
        base = self._flag(self.rank, PH_COMBINE, li, c.mb * 8)
        yield [base + 4 * e for e in range(self.dep.ep)]
        if not T:
            peer_ops.wait_flags(base, self.dep.ep, 1, self.ctl, 0, self.status)
            self.launches_per_step += 1
            return
        self._next_lw = next_lw
        wait = native.flag_wait(base, self.dep.ep, 1, self.ctl, self.status, peer_ops.wait_ns())
        k = self.full_spec.moe.top_k
        if self.plan.expert_tp:
            # every expert rank returned a partial sum per route: fold the ranks into the ordered weighted sum (slot-major,
            # rank-minor, fp32, one rounding) by treating (slot, rank) as k * ranks slots with the slot's weight repeated
            P = self.plan.planes
            if getattr(L, "r_wts_x", None) is None:
                L.r_wts_x = torch.zeros(L.cap, k * P, dtype=torch.float32, device=self.device)
            L.r_wts_x.view(L.cap, k, P)[:T].copy_(L.r_wts[:T].unsqueeze(-1).expand(T, k, P))
            self._combine(self.y_recv[c.mb], self.identity_rows_tp, L.r_wts_x, c.shared, L, T, k * P, wait=wait)
            self.launches_per_step += 2
            return
        self._combine(self.y_recv[c.mb], self.identity_rows, L.r_wts, c.shared, L, T, k, wait=wait)
        self.launches_per_step += 1

    def _moe_nccl(self, li, lw, L, T):
        import torch.distributed as dist
        if self.dep.attn_groups > 1:
            raise NotImplementedError("the NCCL-only baseline runs one attention group")
        H = self.full_spec.hidden
        src = self.dep.attn_ranks[0]
        dist.broadcast(L.xn[:T], src)
        dist.broadcast(L.r_idx[:T], src)
        dist.broadcast(L.r_wts[:T], src)
        acc = torch.zeros(T, H, dtype=torch.bfloat16, device=self.device)
        dist.all_reduce(acc)                      # expert ranks contribute their weighted partial sums
        if lw.ws_gate is not None:
            self._ffn(lw, L, T, L.shared, None)
            acc += L.shared[:T]
        L.x[:T] += acc

    # ------------------------------------------------------------------ MTP draft module on the split
    def mtp_program(self, depth: int, sh: StepShape, prev_hidden: torch.Tensor):
        """One step of draft module `depth` (see `Engine.mtp_forward`): its attention runs here, its routed experts on the
        expert ranks as layer n_layers + depth (they are told to run that single layer)."""
        spec, T, H = self.spec, sh.T, self.spec.hidden
        enorm, hnorm, eh_proj, lw, norm = self.weights.mtp[depth]
        li = spec.n_layers + depth
        cap = next(c for c in (16, 64, 256, 1024, 4096, 16384) if T <= c)
        if cap not in self.mtp_lanes:
            L = Lane(self, cap)
            L.cat = torch.zeros(cap, 2 * H, dtype=torch.bfloat16, device=self.device)
            L.cat_act = ActBuffer.wrap_bf16(L.cat, L.tn)
            self.mtp_lanes[cap] = L
        L = self.mtp_lanes[cap]
        self._keep = []
        self._ensure_attn_scratch(sh)
        if self.block is not None and self.comm == "p2p":
            peer_ops.step_begin(self.ctl)
            if self.local_worker is not None:
                self.local_worker.begin()
        ops.embed_gather(self.md["tokens"][:T], self.weights.embed, L.xl, self.status)
        ops.add_rmsnorm(L.xl, None, enorm, L.xln, spec.rms_eps, rows=T)
        L.cat[:T, :H].copy_(L.xln[:T])
        ops.add_rmsnorm(prev_hidden.contiguous(), None, hnorm, L.xln, spec.rms_eps, rows=T)
        L.cat[:T, H:].copy_(L.xln[:T])
        ops.tc_linear(eh_proj, L.cat_act, L.x, rows=T, status=self.status)
        ctxs = [MicroCtx(0, sh, self.md, L, 0, 0)]
        for mb in range(1, self.plan.n_micro if self.comm == "p2p" else 1):
            ctxs.append(MicroCtx(mb, StepShape(0, 0, 1, 0, 1), self.md, L, 0, 0))
        for c in ctxs:
            self._bind(c)
            yield from self._segment(li, lw, c)
            self._unbind(c)
        if self.local_worker is not None:
            yield from self.local_worker.layer_program(li)
        for c in ctxs:
            self._bind(c)
            if c.pending is not None:
                yield from self._moe_back(c, None)
        if sh.n_logits:
            ops.gather_rows(L.x, self.md["logit_rows"], None, L.xl, sh.n_logits)
            ops.add_rmsnorm(L.xl, None, norm, L.xln, spec.rms_eps, rows=sh.n_logits)
            yield from self._head(L, sh.n_logits, 0, 0, li)
        yield L

    def mtp_forward(self, depth: int, sh: StepShape, prev_hidden: torch.Tensor) -> Lane:
        hook = getattr(self, "on_mtp_step", None)      # multi-rank runs tell the expert ranks to run the draft layer
        if hook:
            hook(depth, sh)
        lane = None
        for item in self.mtp_program(depth, sh, prev_hidden):
            if isinstance(item, Lane):
                lane = item
        return lane


class MlaAttnRankEngine(AttnRankEngine):
    """Attention rank of an MLA model (DeepSeek-V3 shape): local heads, replicated latent cache."""

    def _make_weights(self, spec, device, seed, act_gs, masters):
        from ..engine.mla import mla_weights_from_masters, mla_weights_random
        if masters is not None:
            return mla_weights_from_masters(local_attention_spec(spec, self.tp), attention_masters(spec, masters, self.tp, self.tp_rank), device, act_gs)
        return mla_weights_random(spec, device, heads_local=spec.attn.n_heads // self.tp, experts_range=(0, 0), act_gs=act_gs, seed=seed)


def _bind_mla(cls):
    """MLA attention comes from MlaEngine - every method and class constant it defines (attention layer, its prefill and sparse
    paths, buffers, cache state) - everything else (TP exchange, remote experts) from AttnRankEngine."""
    from ..engine.mla import MlaEngine
    for name, value in vars(MlaEngine).items():
        if not name.startswith("__"):
            setattr(cls, name, value)
    return cls


_bind_mla(MlaAttnRankEngine)


class ExpertRankWorker:
    """One expert-parallel rank: receives dispatched rows, runs its experts, returns rows to the attention ranks."""

    def __init__(self, spec: ModelSpec, plan: LanePlan, rank: int, device, *, comm: str, block: SymmetricBlock | None,
                 act_gs: float = 1.0 / 64, seed: int = 1, masters: dict | None = None):
        dep = plan.dep
        self.spec, self.plan, self.dep, self.rank, self.comm, self.block, self.device = spec, plan, dep, rank, comm, block, device
        self.ep_rank = dep.expert_ranks.index(rank)
        m = spec.moe
        if plan.expert_tp:
            self.e_lo, self.e_hi = 0, m.n_experts           # every expert, a slice of its intermediate dimension
        else:
            self.e_lo, self.e_hi = (self.ep_rank * m.n_experts) // dep.ep, ((self.ep_rank + 1) * m.n_experts) // dep.ep
        self.e_local = self.e_hi - self.e_lo
        self.layers = self._make_weights(spec, device, seed, act_gs, masters)         # per layer (main + MTP): (w_gate, w_up, w_down) or None
        self.kind = next(l[0].kind for l in self.layers if l is not None)
        H, k, t = spec.hidden, m.top_k, plan.t_cap
        n_run = plan.n_lanes if plan.merged else 1          # lanes packed into one grouped GEMM
        rows = n_run * t * k
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=device)
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.ctl, self.done = i32(4), i32(8)
        self.tn = pick_tn(min(max(1, -(-rows // m.n_experts) * 2), 32), swiglu=True)      # <= 32: two CTAs per SM, see Lane.tn_g
        self.max_tiles = self.e_local + rows // self.tn + 1
        self.rows_cap = rows
        self.src_token, self.src_route, self.slot_row = i32(rows), i32(rows), i32(n_run * t, k)
        self.counts, self.offsets = i32(self.e_local), i32(self.e_local)
        self.tiles, self.n_tiles, self.n_rows = i32(self.max_tiles, 4), i32(1), i32(1)
        self.I_local = next(l[0].N for l in self.layers if l is not None)      # intermediate rows this rank computes
        self.xs = ActBuffer.alloc(self.kind, rows, H, self.tn, device)
        self.h1 = torch.zeros(rows, self.I_local, dtype=torch.bfloat16, device=device)
        self.h1_q = (ActBuffer.alloc(self.kind, rows, self.I_local, self.tn, device) if self.kind != KIND_BF16
                     else ActBuffer.wrap_bf16(self.h1, self.tn))
        self.y2 = torch.zeros(rows, H, dtype=torch.bfloat16, device=device)
        self.launches_per_step = 0
        self._keep = []
        if block is not None:
            L = plan.n_lanes
            row_bytes = payload_row_bytes(H, self.kind)
            self.sf_ld = sf_row_bytes(H, self.kind)
            self.slab_q = block.local("slab_q", torch.uint8, (L, t, row_bytes))
            self.slab_sf = block.local("slab_sf", torch.uint8)[:L * t * self.sf_ld].view(L, t, self.sf_ld) if self.sf_ld else None
            self.idx_tab = block.local("idx", torch.int32, (L, t, k))
            self.lane_T = block.local("lane_T", torch.int32)[:L]
            # destinations of each lane: the tp attention ranks of its group, their receive buffer of the lane's micro-batch
            self.recv_addrs, self.lane_ranks = [], []
            for lane in range(L):
                g, mb = lane // plan.n_micro, lane % plan.n_micro
                plane = self.ep_rank if plan.expert_tp else 0
                for r in dep.group_ranks(g):
                    self.recv_addrs.append(block.peer_ptr(r, "y_recv", (mb * plan.planes + plane) * t * k * H * 2))
                    self.lane_ranks.append((r, mb))

    def _make_weights(self, spec, device, seed, act_gs, masters):
        from ..ops import TcWeight
        from ..models.weights import _expert_kind
        tp = self.plan.expert_tp
        granule = 128 if KIND_BY_NAME[_expert_kind(spec)] == KIND_W4A8 else 32
        if masters is not None:
            ek = _expert_kind(spec)
            out = []
            from .shard import expert_tp_masters
            shards = expert_tp_masters(spec, masters, self.ep_rank, self.dep.ep, granule) if tp else expert_masters(spec, masters, self.e_lo, self.e_hi)
            for lw in shards:
                out.append(None if lw is None else tuple(TcWeight.from_master(lw[k], ek, device, act_gs) for k in ("w_gate", "w_up", "w_down")))
            return out
        if tp:      # synthetic benchmarks: random slices of the padded intermediate dimension (no single-GPU twin to match)
            from .shard import expert_tp_slice
            sl = expert_tp_slice(spec.moe.intermediate, self.dep.ep, granule)
            return _random_expert_layers(spec, device, seed + 100 * (self.ep_rank + 1), act_gs, 0, spec.moe.n_experts, intermediate=sl)
        if spec.attn.kind == "mla":
            # expert-only layer sets of an MLA model come from the same generator as the attention ranks' (same seeds per layer)
            return _random_expert_layers(spec, device, seed, act_gs, self.e_lo, self.e_hi)
        dw = DeviceWeights.random(spec, device, seed=seed, experts_range=(self.e_lo, self.e_hi), with_attention=False, act_gs=act_gs)
        return [(l.w_gate, l.w_up, l.w_down) if (l := dw.layer(i)).w_gate is not None else None for i in range(spec.n_layers)]

    # ------------------------------------------------------------------ one layer
    def _flag_local(self, phase: int, layer: int, slot: int) -> int:
        return self.block.peer_ptr(self.rank, "flags", flag_offset(self.spec, phase, layer, slot))

    def layer_program(self, li: int):
        """Runs layer `li` for every lane: all lanes in one grouped GEMM (`merged`) or lane by lane."""
        if self.layers[li] is None:
            return
        L = self.plan.n_lanes
        runs = [(0, L)] if self.plan.merged else [(lane, 1) for lane in range(L)]
        for lane0, n in runs:
            yield from self._run(li, lane0, n)

    def _run(self, li: int, lane0: int, n: int):
        spec, m, dep, plan = self.spec, self.spec.moe, self.dep, self.plan
        w_gate, w_up, w_down = self.layers[li]
        t, k, tp = plan.t_cap, m.top_k, dep.tp
        rows = n * t * k
        base = self._flag_local(PH_DISPATCH, li, lane0 * tp)
        yield [base + 4 * i for i in range(n * tp)]
        wait = native.flag_wait(base, n * tp, 1, self.ctl, self.status, peer_ops.wait_ns())
        ops.route_pack(self.idx_tab[lane0:lane0 + n], self.src_token, self.slot_row, self.counts, self.offsets, self.tiles, self.n_tiles, self.n_rows,
                       n * t, k, self.e_lo, self.e_hi, self.tn, self.max_tiles, src_route=self.src_route, wait=wait,
                       lane_T=self.lane_T[lane0:lane0 + n], t_cap=t)
        ops.route_gather(self.slab_q[lane0:lane0 + n], self.slab_sf[lane0:lane0 + n] if self.slab_sf is not None else None, self.src_token,
                         self.n_rows, self.xs, rows, self.status)
        if self.kind != KIND_BF16 and self.I_local % 32 == 0:      # FC1 writes its output quantised for FC2
            ops.tc_linear(w_gate, self.xs, None, rows=rows, w_up=w_up, tiles=self.tiles, n_tiles=self.n_tiles, max_tiles=self.max_tiles,
                          status=self.status, quant_out=self.h1_q, inv_gs_out=w_down.inv_act_gs)
        else:
            ops.tc_linear(w_gate, self.xs, self.h1, rows=rows, w_up=w_up, tiles=self.tiles, n_tiles=self.n_tiles, max_tiles=self.max_tiles,
                          status=self.status)
            if self.kind != KIND_BF16:
                ops.quant_fp4_rows(self.h1, self.h1_q, n_rows_dev=self.n_rows, rows=rows, inv_gs=w_down.inv_act_gs)
                self.launches_per_step += 1
        ops.tc_linear(w_down, self.h1_q, self.y2, rows=rows, tiles=self.tiles, n_tiles=self.n_tiles, max_tiles=self.max_tiles, status=self.status)
        dst = range(lane0 * tp, (lane0 + n) * tp)
        recv = PtrTable([self.recv_addrs[i] for i in dst])
        flags = PtrTable([self.block.peer_ptr(self.lane_ranks[i][0], "flags", flag_offset(spec, PH_COMBINE, li, self.lane_ranks[i][1] * 8 + self.ep_rank))
                          for i in dst])
        self._keep += [recv, flags]
        peer_ops.combine_push_lanes(self.y2, self.src_route, self.n_rows, recv.arr, flags.arr, self.ctl, self.done[0:1], spec.hidden, k, t, tp,
                                    n * tp, rows, 0, self.status)
        peer_ops.note_published(flags.addrs)
        self.launches_per_step += 5

    def _layer_nccl(self, li: int, T: int):
        import torch.distributed as dist
        if self.layers[li] is None:
            return
        w_gate, w_up, w_down = self.layers[li]
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
            ops.quant_fp4_rows(xn, self.xs, src_rows=self.src_token, n_rows_dev=self.n_rows, rows=rows, inv_gs=w_gate.inv_act_gs)
        ops.tc_linear(w_gate, self.xs, self.h1, rows=rows, w_up=w_up, tiles=self.tiles, n_tiles=self.n_tiles, max_tiles=self.max_tiles, status=self.status)
        if self.kind != KIND_BF16:
            ops.quant_fp4_rows(self.h1, self.h1_q, n_rows_dev=self.n_rows, rows=rows, inv_gs=w_down.inv_act_gs)
        ops.tc_linear(w_down, self.h1_q, self.y2, rows=rows, tiles=self.tiles, n_tiles=self.n_tiles, max_tiles=self.max_tiles, status=self.status)
        acc = torch.zeros(T, H, dtype=torch.bfloat16, device=self.device)
        ops.moe_combine(self.y2, self.slot_row, wts, None, None, acc, T, m.top_k)
        dist.all_reduce(acc)

    # ------------------------------------------------------------------ steps
    def begin(self):
        self._keep = []
        self.launches_per_step = 0
        peer_ops.step_begin(self.ctl)

    def step_program(self, layers=None):
        """All main layers (or the given ones: an MTP draft step runs the single layer n_layers + depth)."""
        self.begin()
        for li in (range(self.spec.n_layers) if layers is None else layers):
            yield from self.layer_program(li)

    def step(self, layers=None):
        for _ in self.step_program(layers):
            pass

    def step_nccl(self, T: int, layers=None):
        for li in (range(self.spec.n_layers) if layers is None else layers):
            self._layer_nccl(li, T)


def _random_expert_layers(spec: ModelSpec, device, seed: int, act_gs: float, e_lo: int, e_hi: int, intermediate: int = 0) -> list:
    """Routed experts [e_lo, e_hi) of every layer of an MLA model (+ its MTP draft layers), generated with the per-layer
    seeds `engine.mla.mla_weights_random` uses, so any expert split holds the experts a single-GPU model would."""
    from ..models.weights import _expert_kind
    from ..ops import TcWeight
    m, h, ek = spec.moe, spec.hidden, _expert_kind(spec)
    inter = intermediate or m.intermediate
    out = []
    for i in range(spec.n_layers + spec.mtp_layers):
        if not spec.is_moe_layer(i):
            out.append(None)
            continue
        s = seed * 1000 + i * 32
        RE = lambda N, K, j: TcWeight.random(m.n_experts, N, K, ek, device, spec.init_std, act_gs, s + j, groups=(e_lo, e_hi))
        out.append((RE(inter, h, 8), RE(inter, h, 9), RE(h, inter, 10)))
    return out


def capture_expert_graph(worker: ExpertRankWorker, layers=None) -> torch.cuda.CUDAGraph:
    """Capture one expert-rank step.  Waiting kernels are part of the graph, so the capture itself must not run
    them: capture records launches without executing."""
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        worker.step(layers)
    return g
