"""fp32 CPU oracle for every operator the engine runs.

Behaviour follows the reference's tiny CPU path (python/reference/cuteafd_reference/
rmsnorm_ref.py:6-9, rope_ref.py:6-25, attention_ref.py:8-21, router_ref.py:6-23, moe_ref.py:16-36)
and its router kernels (native/shared/cuda/expert_router.cu:73-171): all math in fp32, outputs cast
back to the input dtype.  These functions are the comparison target of each CUDA kernel test.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * weight.float()).to(x.dtype)


def rope_angles(dim: int, positions: torch.Tensor, theta: float = 10000.0) -> torch.Tensor:
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    return torch.outer(positions.float(), inv)          # [T, dim/2]


def apply_rope(x: torch.Tensor, positions: torch.Tensor, theta: float = 10000.0,
               interleaved: bool = True) -> torch.Tensor:
    """x: [T, heads, dim].  interleaved rotates pairs (2i, 2i+1); otherwise (i, i+dim/2)."""
    dim = x.shape[-1]
    ang = rope_angles(dim, positions, theta)
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xf = x.float()
    out = torch.empty_like(xf)
    if interleaved:
        a, b = xf[..., 0::2], xf[..., 1::2]
        out[..., 0::2] = a * cos - b * sin
        out[..., 1::2] = a * sin + b * cos
    else:
        h = dim // 2
        a, b = xf[..., :h], xf[..., h:]
        out[..., :h] = a * cos - b * sin
        out[..., h:] = a * sin + b * cos
    return out.to(x.dtype)


def index_scores(q_idx: torch.Tensor, w: torch.Tensor, k_idx: torch.Tensor, q_pos: torch.Tensor, k_pos: torch.Tensor) -> torch.Tensor:
    """Indexer scores of sparse attention: q_idx [Tq, Hi, Di], w [Tq, Hi], k_idx [Tk, Di] ->
    [Tq, Tk] = sum_h w[t, h] * relu(q_idx[t, h] . k_idx[s]), -inf where the key lies in the query's future."""
    dots = torch.einsum("qhd,kd->qhk", q_idx.float(), k_idx.float())
    s = (torch.relu(dots) * w.float()[:, :, None]).sum(1)
    return s.masked_fill(k_pos[None, :] > q_pos[:, None], float("-inf"))


def topk_mask(scores: torch.Tensor, k: int) -> torch.Tensor:
    """[Tq, Tk] bool: the k best finite entries of every row (all of them when a row has at most k); ties at the threshold
    resolve to the lowest key index (the device kernel's rule)."""
    Tq, Tk = scores.shape
    out = torch.zeros(Tq, Tk, dtype=torch.bool)
    for t in range(Tq):
        row = scores[t]
        vis = torch.isfinite(row)
        n = int(vis.sum())
        if n <= k:
            out[t] = vis
            continue
        order = sorted(range(Tk), key=lambda i: (-float(row[i]), i))        # best first, lowest index among equals
        out[t, torch.tensor(order[:k])] = True
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos: torch.Tensor,
              k_pos: torch.Tensor, scale: float | None = None, window: int = 0,
              sink: torch.Tensor | None = None, allowed: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention by absolute position.  q: [Tq, Hq, D], k: [Tk, Hkv, D], v: [Tk, Hkv, Dv].
    Query at position p sees keys with position <= p (and > p - window when window > 0).
    `sink` ([Hq]) adds one extra softmax logit per head whose value contribution is zero."""
    Tq, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    kf = k.float().repeat_interleave(g, 1)
    vf = v.float().repeat_interleave(g, 1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kf) * scale
    mask = k_pos[None, :] > q_pos[:, None]
    if window > 0:
        mask |= k_pos[None, :] <= (q_pos[:, None] - window)
    if allowed is not None:                 # sparse attention: [Tq, Tk] bool, keys a query may attend to
        mask = mask | ~allowed
    s = s.masked_fill(mask[None], float("-inf"))
    if sink is not None:
        s = torch.cat([s, sink.float()[:, None, None].expand(Hq, Tq, 1)], -1)
    p = torch.softmax(s, -1)
    if sink is not None:
        p = p[..., :-1]
    return torch.einsum("hqk,khd->qhd", p, vf).to(q.dtype)


def router_scores(logits: torch.Tensor, scoring: str) -> torch.Tensor:
    lf = logits.float()
    if scoring == "sigmoid":
        return torch.sigmoid(lf)
    if scoring == "softmax":
        return torch.softmax(lf, -1)
    if scoring == "sqrtsoftplus":
        return torch.sqrt(F.softplus(lf))
    raise ValueError(f"unsupported scoring {scoring!r}")


def route_topk(hidden: torch.Tensor, router_weight: torch.Tensor, top_k: int, scoring: str = "sigmoid",
               normalize: bool = True, route_scale: float = 1.0, bias: torch.Tensor | None = None,
               n_group: int = 1, topk_group: int = 1):
    """Returns (indices [T, k] int64, weights [T, k] fp32).

    `bias` (noaux_tc) only influences the choice; gate weights come from unbiased scores.
    Group-limited routing keeps the `topk_group` groups whose top-2 biased scores sum highest.
    Ties pick the lowest expert id; selected experts are ordered by descending choice score."""
    logits = hidden.float() @ router_weight.float().T
    scores = router_scores(logits, scoring)
    choice = scores + bias.float() if bias is not None else scores
    T, E = scores.shape
    if n_group > 1 and topk_group < n_group:
        grp = choice.reshape(T, n_group, E // n_group)
        gscore = grp.topk(2, -1).values.sum(-1)
        keep = torch.zeros(T, n_group, dtype=torch.bool)
        keep.scatter_(1, _stable_topk(gscore, topk_group), True)
        choice = choice.masked_fill(~keep.repeat_interleave(E // n_group, 1), float("-inf"))
    idx = _stable_topk(choice, top_k)
    w = scores.gather(1, idx)
    if normalize:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-12)
    return idx, w * route_scale


def _stable_topk(x: torch.Tensor, k: int) -> torch.Tensor:
    """top-k indices, descending value, lowest index first among equals."""
    order = torch.sort(x, dim=-1, descending=True, stable=True).indices
    return order[..., :k]


def hash_route(token_ids: torch.Tensor, tid2eid: torch.Tensor):
    """Hash routing: a per-token-id table names the experts (reference select_hash_kernel)."""
    return tid2eid[token_ids.long()]


def swiglu(gate: torch.Tensor, up: torch.Tensor, limit: float = 0.0) -> torch.Tensor:
    g, u = gate.float(), up.float()
    if limit > 0:
        g = g.clamp(max=limit)
        u = u.clamp(-limit, limit)
    return F.silu(g) * u


def expert_ffn(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
               limit: float = 0.0) -> torch.Tensor:
    xf = x.float()
    return swiglu(xf @ w_gate.float().T, xf @ w_up.float().T, limit) @ w_down.float().T


def moe_forward(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
                idx: torch.Tensor, weights: torch.Tensor, limit: float = 0.0) -> torch.Tensor:
    """Routed experts.  w_*: [E, ...].  Accumulates routes in slot order in fp32 (the combine
    contract: fixed order fp32 sum, one final rounding)."""
    out = torch.zeros(x.shape, dtype=torch.float32)
    for e in idx.unique().tolist():
        rows, slots = (idx == e).nonzero(as_tuple=True)
        y = expert_ffn(x[rows], w_gate[e], w_up[e], w_down[e], limit)
        out.index_put_((rows,), y * weights[rows, slots].float()[:, None], accumulate=True)
    return out


def greedy_verify(inputs: list[int], target_next: list[int], eos: int | None, remaining: int):
    """Lossless greedy verification (reference: cuteafd-core/src/dspark_verify.rs:21-69).
    inputs = anchor followed by drafts; target_next[i] = target argmax after input row i.
    Returns (accepted_inputs, emitted, hit_eos, hit_length)."""
    assert inputs and len(inputs) == len(target_next) and remaining > 0
    accepted, emitted, hit_eos, hit_len = 1, [], False, False
    for i, tok in enumerate(target_next):
        matched = i + 1 < len(inputs) and inputs[i + 1] == tok
        emitted.append(tok)
        if matched:
            accepted += 1
        hit_eos = eos is not None and tok == eos
        hit_len = len(emitted) == remaining
        if not matched or hit_eos or hit_len:
            break
    return accepted, emitted, hit_eos, hit_len


def gated_delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                     state: torch.Tensor | None = None):
    """Recurrent gated delta rule of the GDN / KDA linear-attention layers, one sequence: q, k [T, H, dk], v [T, H, dv],
    g [T, H] (one decay per head) or [T, H, dk] (per key channel), beta [T, H]; state [H, dk, dv] or None (zeros).
    Returns (o [T, H, dv] fp32, final state, list of the states after every token)."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv) if state is None else state.float().clone()
    out, snaps = [], []
    for t in range(T):
        gt = g[t].float()
        S = S * (gt[:, :, None] if gt.dim() == 2 else gt[:, None, None])
        u = torch.einsum("hkv,hk->hv", S, k[t].float())
        d = beta[t].float()[:, None] * (v[t].float() - u)
        S = S + k[t].float()[:, :, None] * d[:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S, q[t].float()))
        snaps.append(S.clone())
    return torch.stack(out), S, snaps


def short_conv4(x: torch.Tensor, w: torch.Tensor, carry: torch.Tensor | None = None):
    """Causal depthwise convolution of width 4 + SiLU over one sequence: x [T, C], w [C, 4], carry [3, C] (the three inputs before
    x, zeros when None).  Returns (y [T, C] fp32, new carry [3, C])."""
    T, C = x.shape
    hist = torch.cat([torch.zeros(3, C) if carry is None else carry.float(), x.float()])
    y = sum(hist[i:i + T] * w[:, i].float()[None, :] for i in range(4))
    return F.silu(y), hist[-3:]


def mhc_mixes(res: torch.Tensor, fn: torch.Tensor, scale: torch.Tensor, base: torch.Tensor, iters: int = 20):
    """Hyper-connection coefficients of one boundary.  res [T, S, H] (the residual streams), fn [P, S*H] with P = S*(S+2)
    (collapse, spread and stream-mix projections) or P = S (collapse only), scale [3], base [P].
    Returns (pre [T, S], post [T, S] | None, comb [T, S, S] | None); comb[t, s, d] is the weight of source stream s in
    destination stream d, made doubly stochastic by `iters` Sinkhorn sweeps.
    Reference: native/families/deepseek_v41/cuda/v41_hc.cu (mixes_kernel)."""
    T, S, H = res.shape
    flat = res.reshape(T, S * H).float()
    proj = (flat @ fn.float().T) * torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + 1e-20)
    pre = torch.sigmoid(proj[:, :S] * scale[0] + base[:S]) + 1e-6
    if fn.shape[0] == S:
        return pre, None, None
    post = 2 * torch.sigmoid(proj[:, S:2 * S] * scale[1] + base[S:2 * S])
    c = torch.softmax((proj[:, 2 * S:] * scale[2] + base[2 * S:]).reshape(T, S, S), -1) + 1e-6
    c = c / (c.sum(1, keepdim=True) + 1e-6)
    for _ in range(iters - 1):
        c = c / (c.sum(2, keepdim=True) + 1e-6)
        c = c / (c.sum(1, keepdim=True) + 1e-6)
    return pre, post, c


def mhc_close(res: torch.Tensor, sub: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    """res'[t, d] = post[t, d] * sub[t] + sum_s comb[t, s, d] * res[t, s]."""
    return post[:, :, None] * sub[:, None, :].float() + torch.einsum("tsd,tsh->tdh", comb, res.float())


def compress_pool(kv: torch.Tensor, scores: torch.Tensor, ratio: int, norm_w: torch.Tensor, eps: float, pos0: int = 0, state=None):
    """Learned KV compressor (CSA / HCA / CED caches): blocks of `ratio` consecutive positions pooled per channel with a softmax over
    their scores, rounded to bf16, RMS-normalised and scaled.  kv, scores: fp32 [T, D] rows of positions pos0 .. pos0 + T - 1;
    `state` = (max, sum, weighted sum) [3, D] of a block an earlier call left open.  Returns (rows of the blocks completed here [n, D],
    state of the block left open or None).  Reference: native/families/deepseek_v41/cuda/v41_compressor.cu (`pool_kernel`)."""
    T, D = kv.shape
    mx, l, acc = (state[0].clone(), state[1].clone(), state[2].clone()) if state is not None else (
        torch.full((D,), float("-inf")), torch.zeros(D), torch.zeros(D))
    if state is None and pos0 % ratio:
        raise ValueError("a step that starts inside a block needs the block's state")
    out = []
    for t in range(T):
        nm = torch.maximum(mx, scores[t])
        r = torch.where(torch.isinf(mx), torch.zeros_like(mx), torch.exp(mx - nm))
        e = torch.exp(scores[t] - nm)
        l, acc, mx = l * r + e, acc * r + e * kv[t], nm
        if (pos0 + t + 1) % ratio == 0:
            pooled = (acc / l).to(torch.bfloat16).float()
            out.append(pooled * torch.rsqrt(pooled.pow(2).mean() + eps) * norm_w)
            mx, l, acc = torch.full((D,), float("-inf")), torch.zeros(D), torch.zeros(D)
    open_block = (pos0 + T) % ratio != 0
    return (torch.stack(out) if out else torch.zeros(0, D)), (torch.stack([mx, l, acc]) if open_block else None)
