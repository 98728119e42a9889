"""Whole-model fp32 CPU oracle: embedding -> [norm, attention(+RoPE, KV cache), residual, norm,
router + routed experts + shared expert (or dense FFN), residual] x L -> norm -> LM head, plus the
MTP draft module and greedy generation / speculative verification.

This plays the role of the reference's tiny CPU path (python/reference/cuteafd_reference/
layer_ref.py:11-36, prefill_ref.py:42-141, mtp_protocol_ref.py:6-19) extended to a full decoder with
GQA or MLA attention so the same oracle covers the DeepSeek-V3 and Qwen3-MoE shapes at toy sizes.
It is the timed CPU baseline and the comparison target for the GPU engine.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from ..config import ModelSpec
from . import ops


def _randn(gen, *shape, std):
    return torch.randn(*shape, generator=gen, dtype=torch.float32) * std


def init_layer(spec: ModelSpec, gen: torch.Generator, layer: int, force_dense: bool = False) -> dict:
    h, a, m, s = spec.hidden, spec.attn, spec.moe, spec.init_std
    w = {"attn_norm": torch.ones(h), "ffn_norm": torch.ones(h)}
    if a.kind == "mla":
        qk = a.qk_nope_head_dim + a.qk_rope_head_dim
        if a.q_lora_rank:
            w["wq_a"] = _randn(gen, a.q_lora_rank, h, std=s)
            w["q_a_norm"] = torch.ones(a.q_lora_rank)
            w["wq_b"] = _randn(gen, a.n_heads * qk, a.q_lora_rank, std=s)
        else:
            w["wq"] = _randn(gen, a.n_heads * qk, h, std=s)
        w["wkv_a"] = _randn(gen, a.kv_lora_rank + a.qk_rope_head_dim, h, std=s)
        w["kv_a_norm"] = torch.ones(a.kv_lora_rank)
        w["wkv_b"] = _randn(gen, a.n_heads * (a.qk_nope_head_dim + a.v_head_dim), a.kv_lora_rank, std=s)
        w["wo"] = _randn(gen, h, a.n_heads * a.v_head_dim, std=s)
        if a.index_topk:        # indexer: queries from the compressed query (or the hidden state), keys and head weights from the hidden state
            w["wq_idx"] = _randn(gen, a.index_heads * a.index_dim, a.q_lora_rank or h, std=s)
            w["wk_idx"] = _randn(gen, a.index_dim, h, std=s)
            w["w_idx"] = _randn(gen, a.index_heads, h, std=s)
    elif spec.layer_is_linear(layer):
        Hk, Hv = a.linear_k_heads, a.linear_v_heads
        w["w_qkvz"] = _randn(gen, (2 * Hk + 2 * Hv) * 128, h, std=s)          # rows: q [Hk x 128], k [Hk x 128], v [Hv x 128], z [Hv x 128]
        w["w_ba"] = _randn(gen, Hv + (Hv * 128 if a.linear_per_channel else Hv), h, std=s)   # rows: b [Hv], a [Hv] (or a per channel [Hv x 128])
        w["conv_w"] = _randn(gen, (2 * Hk + Hv) * 128, 4, std=0.5)
        w["dt_bias"] = _randn(gen, Hv * 128 if a.linear_per_channel else Hv, std=0.5)
        w["a_log"] = _randn(gen, Hv, std=0.5)
        w["lin_norm"] = torch.ones(128)
        w["wo"] = _randn(gen, h, Hv * 128, std=s)
    else:
        w["wq"] = _randn(gen, a.n_heads * a.head_dim, h, std=s)
        w["wk"] = _randn(gen, a.n_kv_heads * a.head_dim, h, std=s)
        w["wv"] = _randn(gen, a.n_kv_heads * a.head_dim, h, std=s)
        w["wo"] = _randn(gen, h, a.n_heads * a.head_dim, std=s)
        if a.qk_norm:
            w["q_norm"] = torch.ones(a.head_dim)
            w["k_norm"] = torch.ones(a.head_dim)
        if spec.layer_has_sink(layer):
            w["sink"] = _randn(gen, a.n_heads, std=1.0)
    if spec.hyper_streams:
        S = spec.hyper_streams
        for blk in ("attn", "ffn"):        # projections wide enough to move the coefficients off their base values
            w[f"hc_{blk}_fn"] = _randn(gen, S * (S + 2), S * h, std=2.0 / math.sqrt(S * h))
            w[f"hc_{blk}_scale"] = torch.tensor([0.5, 0.5, 0.5])
            w[f"hc_{blk}_base"] = _randn(gen, S * (S + 2), std=0.5)
    if spec.is_moe_layer(layer) and not force_dense:
        w["router"] = _randn(gen, m.n_experts, h, std=s)
        if m.use_bias:
            w["router_bias"] = _randn(gen, m.n_experts, std=0.01)
        w["w_gate"] = _randn(gen, m.n_experts, m.intermediate, h, std=s)
        w["w_up"] = _randn(gen, m.n_experts, m.intermediate, h, std=s)
        w["w_down"] = _randn(gen, m.n_experts, h, m.intermediate, std=s)
        if m.shared_inter:
            w["ws_gate"] = _randn(gen, m.shared_inter, h, std=s)
            w["ws_up"] = _randn(gen, m.shared_inter, h, std=s)
            w["ws_down"] = _randn(gen, h, m.shared_inter, std=s)
    else:
        inter = m.dense_intermediate or m.intermediate
        w["wd_gate"] = _randn(gen, inter, h, std=s)
        w["wd_up"] = _randn(gen, inter, h, std=s)
        w["wd_down"] = _randn(gen, h, inter, std=s)
    return w


def init_weights(spec: ModelSpec, seed: int = 0) -> dict:
    """N(0, init_std) weights from a seed (norm gains = 1).  fp32 masters on CPU."""
    gen = torch.Generator().manual_seed(seed)
    w = {"embed": _randn(gen, spec.vocab, spec.hidden, std=spec.init_std),
         "layers": [init_layer(spec, gen, i) for i in range(spec.n_layers)],
         "final_norm": torch.ones(spec.hidden)}
    w["lm_head"] = w["embed"] if spec.tie_embeddings else _randn(gen, spec.vocab, spec.hidden, std=spec.init_std)
    if spec.hyper_streams:
        S = spec.hyper_streams
        w["hc_head_fn"] = _randn(gen, S, S * spec.hidden, std=2.0 / math.sqrt(S * spec.hidden))
        w["hc_head_scale"] = torch.tensor([0.5, 0.5, 0.5])
        w["hc_head_base"] = _randn(gen, S, std=0.5)
    if spec.engram_layers:
        from .engram import init_engram_weights
        w["engram"] = init_engram_weights(spec.engram_spec(), seed + 17)
    if spec.mtp_layers:
        w["mtp"] = [{"enorm": torch.ones(spec.hidden), "hnorm": torch.ones(spec.hidden),
                     "eh_proj": _randn(gen, spec.hidden, 2 * spec.hidden, std=spec.init_std),
                     "layer": init_layer(spec, gen, spec.n_layers + i),
                     "norm": torch.ones(spec.hidden)} for i in range(spec.mtp_layers)]
    return w


@dataclass
class RefCache:
    """Per-sequence KV history: one (k, v, positions) triple per layer ("mtp{i}" for draft layers)."""
    layers: dict = field(default_factory=dict)
    tokens: list = field(default_factory=list)      # token ids by position (the n-gram memory addresses by the last four)

    def append(self, key, k, v, pos):
        if key in self.layers:
            k0, v0, p0 = self.layers[key]
            k, v, pos = torch.cat([k0, k]), torch.cat([v0, v]), torch.cat([p0, pos])
        self.layers[key] = (k, v, pos)
        return self.layers[key]

    def truncate(self, length: int):
        """Drop cached rows at position >= length (rejected speculative rows)."""
        for key, (k, v, p) in list(self.layers.items()):
            if isinstance(key, tuple) and key[0] == "lin":
                raise NotImplementedError("rows of a linear-attention layer cannot be dropped: the recurrent state has absorbed them")
            keep = p < length
            self.layers[key] = (k[keep], v[keep], p[keep])
        del self.tokens[length:]

    def clone(self) -> "RefCache":
        return RefCache({k: tuple(t.clone() for t in v) for k, v in self.layers.items()}, list(self.tokens))


class RefModel:
    def __init__(self, spec: ModelSpec, weights: dict, act_quant=None):
        """`act_quant`: optional callable(x, kind) -> x emulating activation quantisation ahead of
        quantised linears (kind in {"dense", "expert"})."""
        self.spec, self.w, self.act_quant = spec, weights, act_quant

    # ---- blocks ---------------------------------------------------------
    def _aq(self, x, kind):
        return self.act_quant(x, kind) if self.act_quant else x

    def attention_block(self, lw: dict, x: torch.Tensor, pos: torch.Tensor, cache: RefCache, key, add_residual: bool = True) -> torch.Tensor:
        a, spec = self.spec.attn, self.spec
        T = x.shape[0]
        xn = self._aq(ops.rmsnorm(x, lw["attn_norm"], spec.rms_eps), "dense")
        if a.kind == "mla":
            nope, rope, dv = a.qk_nope_head_dim, a.qk_rope_head_dim, a.v_head_dim
            qa = None
            if "wq_a" in lw:
                qa = ops.rmsnorm(xn @ lw["wq_a"].T, lw["q_a_norm"], spec.rms_eps)
                q = self._aq(qa, "dense") @ lw["wq_b"].T
            else:
                q = xn @ lw["wq"].T
            q = q.reshape(T, a.n_heads, nope + rope)
            q = torch.cat([q[..., :nope], ops.apply_rope(q[..., nope:], pos, a.rope_theta, a.rope_interleaved)], -1)
            kva = xn @ lw["wkv_a"].T
            ckv = ops.rmsnorm(kva[:, :a.kv_lora_rank], lw["kv_a_norm"], spec.rms_eps)
            kr = ops.apply_rope(kva[:, None, a.kv_lora_rank:], pos, a.rope_theta, a.rope_interleaved)[:, 0]
            ckv, kr, kpos = cache.append(key, ckv, kr, pos)
            kvb = (ckv @ lw["wkv_b"].T).reshape(-1, a.n_heads, nope + dv)
            k = torch.cat([kvb[..., :nope], kr[:, None, :].expand(-1, a.n_heads, -1)], -1)
            allowed = None
            if a.index_topk and "wq_idx" in lw:
                # the indexer's operands are bf16 on the device (its score product runs on the tensor cores): round them here too
                b16 = lambda t: t.to(torch.bfloat16).float()
                src = self._aq(qa, "dense") if qa is not None else xn
                q_idx = b16((src @ lw["wq_idx"].T).reshape(T, a.index_heads, a.index_dim))
                k_new = b16(xn @ lw["wk_idx"].T)
                w_idx = (xn @ lw["w_idx"].T) * (a.index_heads ** -0.5)
                k_idx, _, _ = cache.append(("idx", key), k_new, k_new[:, :1], pos)
                if k_idx.shape[0] > a.index_topk:
                    allowed = ops.topk_mask(ops.index_scores(q_idx, w_idx, k_idx, pos, kpos), a.index_topk)
            o = ops.attention(q, k, kvb[..., nope:], pos, kpos, scale=1.0 / math.sqrt(nope + rope), allowed=allowed)
            o = o.reshape(T, a.n_heads * dv)
        elif "w_qkvz" in lw:
            o = self.linear_attention(lw, xn, cache, key)
        else:
            q = (xn @ lw["wq"].T).reshape(T, a.n_heads, a.head_dim)
            k = (xn @ lw["wk"].T).reshape(T, a.n_kv_heads, a.head_dim)
            v = (xn @ lw["wv"].T).reshape(T, a.n_kv_heads, a.head_dim)
            if a.qk_norm:
                q = ops.rmsnorm(q, lw["q_norm"], spec.rms_eps)
                k = ops.rmsnorm(k, lw["k_norm"], spec.rms_eps)
            li = key if isinstance(key, int) else spec.n_layers         # MTP draft layers count as layers past the stack
            theta = spec.layer_rope_theta(li)
            q = ops.apply_rope(q, pos, theta, a.rope_interleaved)
            k = ops.apply_rope(k, pos, theta, a.rope_interleaved)
            k, v, kpos = cache.append(key, k, v, pos)
            o = ops.attention(q, k, v, pos, kpos, window=spec.layer_window(li), sink=lw.get("sink")).reshape(T, -1)
        out = self._aq(o, "dense") @ lw["wo"].T
        return x + out if add_residual else out

    def linear_attention(self, lw: dict, xn: torch.Tensor, cache: RefCache, key) -> torch.Tensor:
        """Gated delta-rule layer (GDN: decay per head; KDA: per key channel): projections -> width-4 causal convolution + SiLU over
        q / k / v -> L2-normalised q (scaled by dk^-1/2) and k -> recurrence over the sequence's carried state -> RMSNorm gated by
        silu(z).  The state and the convolution's last three inputs live in the cache entry ("lin", key).  Intermediate tensors are
        rounded to bf16 where the device path stores them in bf16."""
        a = self.spec.attn
        Hk, Hv, T = a.linear_k_heads, a.linear_v_heads, xn.shape[0]
        b16 = lambda t: t.to(torch.bfloat16).float()
        qkvz = b16(xn @ lw["w_qkvz"].T)
        ba = xn @ lw["w_ba"].T
        C = (2 * Hk + Hv) * 128
        st = cache.layers.get(("lin", key))
        state, carry = (st[0], st[1]) if st is not None else (None, None)
        conv, carry = ops.short_conv4(qkvz[:, :C], lw["conv_w"], carry)
        conv = b16(conv)
        q = conv[:, :Hk * 128].reshape(T, Hk, 128)
        k = conv[:, Hk * 128:2 * Hk * 128].reshape(T, Hk, 128)
        v = conv[:, 2 * Hk * 128:].reshape(T, Hv, 128)
        z = qkvz[:, C:].reshape(T, Hv, 128)
        rep = Hv // Hk
        qn = torch.nn.functional.normalize(q, dim=-1, eps=1e-6) * 128 ** -0.5
        kn = torch.nn.functional.normalize(k, dim=-1, eps=1e-6)
        qe, ke = b16(qn.repeat_interleave(rep, 1)), b16(kn.repeat_interleave(rep, 1))
        beta = torch.sigmoid(ba[:, :Hv])
        if a.linear_per_channel:
            g = torch.exp(-torch.exp(lw["a_log"])[None, :, None] * torch.nn.functional.softplus(ba[:, Hv:].reshape(T, Hv, 128) + lw["dt_bias"].reshape(Hv, 128)))
        else:
            g = torch.exp(-torch.exp(lw["a_log"])[None, :] * torch.nn.functional.softplus(ba[:, Hv:2 * Hv] + lw["dt_bias"]))
        o, state, _ = ops.gated_delta_rule(qe, ke, v, g, beta, state)
        cache.layers[("lin", key)] = (state, b16(carry), torch.zeros(0))
        o = b16(o)
        o = ops.rmsnorm(o, lw["lin_norm"], self.spec.rms_eps) * torch.nn.functional.silu(z)
        return b16(o).reshape(T, Hv * 128)

    def ffn_block(self, lw: dict, x: torch.Tensor, routes_out: list | None = None, add_residual: bool = True) -> torch.Tensor:
        m, spec = self.spec.moe, self.spec
        xn = ops.rmsnorm(x, lw["ffn_norm"], spec.rms_eps)
        if "router" in lw:
            idx, wt = ops.route_topk(xn, lw["router"], m.top_k, m.scoring, m.normalize, m.route_scale,
                                     lw.get("router_bias"), m.n_group, m.topk_group)
            if routes_out is not None:
                routes_out.append((idx, wt))
            y = ops.moe_forward(self._aq(xn, "expert"), lw["w_gate"], lw["w_up"], lw["w_down"], idx, wt, m.swiglu_limit)
            if "ws_gate" in lw:
                y = y + ops.expert_ffn(self._aq(xn, "dense"), lw["ws_gate"], lw["ws_up"], lw["ws_down"])
        else:
            y = ops.expert_ffn(self._aq(xn, "dense"), lw["wd_gate"], lw["wd_up"], lw["wd_down"])
        return x + y if add_residual else y

    # ---- passes ---------------------------------------------------------
    def hidden_states(self, tokens: torch.Tensor, start: int, cache: RefCache, routes_out=None) -> torch.Tensor:
        pos = torch.arange(start, start + tokens.numel())
        x = self.w["embed"][tokens.long()].float()
        if self.spec.hyper_streams:
            return self._hyper_hidden_states(x, pos, cache, routes_out)
        eng_hashes = None
        if self.spec.engram_layers:
            from .engram import EngramAddressing, context_hashes, engram_apply
            espec = self.spec.engram_spec()
            del cache.tokens[start:]
            eng_hashes = context_hashes(EngramAddressing(espec), cache.tokens, tokens.tolist())
            cache.tokens += tokens.tolist()
        for i, lw in enumerate(self.w["layers"]):
            if eng_hashes is not None and i in self.spec.engram_layers:
                e = self.spec.engram_layers.index(i)
                x = engram_apply(espec, self.w["engram"]["layers"][e], x.bfloat16().float()[:, None, :], eng_hashes[e])[:, 0]
            x = self.attention_block(lw, x, pos, cache, i)
            x = self.ffn_block(lw, x, routes_out)
        return x

    def _hyper_hidden_states(self, x: torch.Tensor, pos: torch.Tensor, cache: RefCache, routes_out=None) -> torch.Tensor:
        """The stack with hyper-connections: S residual streams, closed and re-opened around every sub-layer; the streams and the
        sub-layer outputs are rounded to bf16 where the device stores them.  Returns the head's collapse of the streams."""
        spec, S = self.spec, self.spec.hyper_streams
        b16 = lambda t: t.to(torch.bfloat16).float()
        res = b16(x)[:, None, :].expand(-1, S, -1).contiguous()
        sub = post = comb = None
        for i, lw in enumerate(self.w["layers"]):
            for blk in ("attn", "ffn"):
                if sub is not None:
                    res = b16(ops.mhc_close(res, sub, post, comb))
                pre, post, comb = ops.mhc_mixes(res, lw[f"hc_{blk}_fn"], lw[f"hc_{blk}_scale"], lw[f"hc_{blk}_base"], spec.hyper_sinkhorn_iters)
                y = (pre[:, :, None] * res).sum(1)
                if blk == "attn":
                    sub = b16(self.attention_block(lw, y, pos, cache, i, add_residual=False))
                else:
                    sub = b16(self.ffn_block(lw, y, routes_out, add_residual=False))
        res = b16(ops.mhc_close(res, sub, post, comb))
        pre, _, _ = ops.mhc_mixes(res, self.w["hc_head_fn"], self.w["hc_head_scale"], self.w["hc_head_base"])
        return (pre[:, :, None] * res).sum(1)

    def logits_from_hidden(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.w["final_norm"], self.spec.rms_eps).float() @ self.w["lm_head"].float().T

    def forward(self, tokens: torch.Tensor, start: int, cache: RefCache, chunk: int = 0):
        """Returns (logits [T, V], hidden [T, H]).  `chunk` > 0 runs chunked prefill."""
        if chunk and tokens.numel() > chunk:
            hs = [self.hidden_states(tokens[s:s + chunk], start + s, cache) for s in range(0, tokens.numel(), chunk)]
            x = torch.cat(hs)
        else:
            x = self.hidden_states(tokens, start, cache)
        return self.logits_from_hidden(x), x

    def mtp_forward(self, prev_hidden: torch.Tensor, tokens: torch.Tensor, start: int, cache: RefCache, depth: int = 0):
        """MTP draft module: combine the target hidden at position p with the embedding of token p+1,
        run one decoder layer, project with the shared head.  Returns (logits, hidden)."""
        mw = self.w["mtp"][depth]
        e = ops.rmsnorm(self.w["embed"][tokens.long()].float(), mw["enorm"], self.spec.rms_eps)
        hn = ops.rmsnorm(prev_hidden.float(), mw["hnorm"], self.spec.rms_eps)
        x = torch.cat([e, hn], -1) @ mw["eh_proj"].T
        pos = torch.arange(start, start + tokens.numel())
        x = self.attention_block(mw["layer"], x, pos, cache, f"mtp{depth}")
        x = self.ffn_block(mw["layer"], x)
        logits = ops.rmsnorm(x, mw["norm"], self.spec.rms_eps).float() @ self.w["lm_head"].float().T
        return logits, x

    def generate_greedy(self, prompt: torch.Tensor, n_new: int, chunk: int = 0):
        """Prefill + greedy decode.  Returns (tokens list, per-step logits rows)."""
        cache = RefCache()
        logits, _ = self.forward(prompt, 0, cache, chunk)
        out, rows = [], []
        nxt = int(logits[-1].argmax())
        for i in range(n_new):
            out.append(nxt)
            rows.append(logits[-1])
            if i + 1 == n_new:
                break
            logits, _ = self.forward(torch.tensor([nxt]), prompt.numel() + i, cache)
            nxt = int(logits[-1].argmax())
        return out, rows

    def generate_speculative(self, prompt: torch.Tensor, n_new: int, n_draft: int = 3):
        """Greedy generation with MTP drafts + lossless verification; must equal generate_greedy.

        Draft-cache invariant: the MTP row at position q pairs the *target* hidden of position q-1
        with the token at position q.  Rows written from recursive draft hiddens during a round are
        discarded after verification and rebuilt from the verified hiddens.
        Returns (tokens, drafts accepted per round)."""
        cache = RefCache()
        logits, hidden = self.forward(prompt, 0, cache)
        L = prompt.numel()
        if L > 1:
            self.mtp_forward(hidden[:-1], prompt[1:], 1, cache)
        anchor = int(logits[-1].argmax())
        out, acc_hist = [anchor], []
        h_last = hidden[-1:]
        while len(out) < n_new:
            drafts, h, tok = [], h_last, anchor
            for d in range(n_draft):
                dl, h = self.mtp_forward(h, torch.tensor([tok]), L + d, cache)
                tok = int(dl[-1].argmax())
                drafts.append(tok)
            inputs = [anchor] + drafts
            vl, vh = self.forward(torch.tensor(inputs), L, cache)
            accepted, emitted, _, _ = ops.greedy_verify(inputs, vl.argmax(-1).tolist(), None, n_new - len(out))
            acc_hist.append(accepted - 1)
            out.extend(emitted)
            cache.truncate(L + accepted)
            for key in [k for k in cache.layers if isinstance(k, str)]:
                kk, vv, pp = cache.layers[key]
                keep = pp <= L
                cache.layers[key] = (kk[keep], vv[keep], pp[keep])
            if accepted > 1:
                self.mtp_forward(vh[:accepted - 1], torch.tensor(inputs[1:accepted]), L + 1, cache)
            L += accepted
            anchor = emitted[-1]
            h_last = vh[accepted - 1:accepted]
        return out[:n_new], acc_hist
