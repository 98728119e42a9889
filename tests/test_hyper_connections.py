"""Hyper-connections (four residual streams mixed at every sub-layer boundary): the oracle's coefficients and stack."""
import torch

from cuteafd_b200.config import tiny_spec
from cuteafd_b200.ref import ops
from cuteafd_b200.ref.model import RefCache, RefModel, init_weights


def test_mixes_are_bounded_and_the_stream_mix_is_doubly_stochastic():
    g = torch.Generator().manual_seed(0)
    T, S, H = 6, 4, 64
    res = torch.randn(T, S, H, generator=g)
    fn = torch.randn(S * (S + 2), S * H, generator=g) * 0.2
    pre, post, comb = ops.mhc_mixes(res, fn, torch.tensor([1.0, 1.0, 1.0]), torch.randn(S * (S + 2), generator=g))
    assert pre.shape == (T, S) and post.shape == (T, S) and comb.shape == (T, S, S)
    assert float(pre.min()) > 0 and float(pre.max()) < 1.0001 and float(post.min()) > 0 and float(post.max()) < 2
    assert torch.allclose(comb.sum(1), torch.ones(T, S), atol=1e-3) and torch.allclose(comb.sum(2), torch.ones(T, S), atol=0.05)    # the last sweep normalises the columns
    only_pre, none_a, none_b = ops.mhc_mixes(res, fn[:S], torch.tensor([1.0, 1.0, 1.0]), torch.zeros(S))
    assert only_pre.shape == (T, S) and none_a is None and none_b is None
    # scaling every stream by a constant leaves the coefficients unchanged (the projections see the RMS-normalised row)
    pre2, post2, comb2 = ops.mhc_mixes(res * 7.0, fn, torch.tensor([1.0, 1.0, 1.0]), torch.zeros(S * (S + 2)))
    pre1, post1, comb1 = ops.mhc_mixes(res, fn, torch.tensor([1.0, 1.0, 1.0]), torch.zeros(S * (S + 2)))
    assert torch.allclose(pre1, pre2, atol=1e-5) and torch.allclose(comb1, comb2, atol=1e-5)


def test_close_spreads_the_output_and_mixes_the_streams():
    T, S, H = 2, 4, 8
    res = torch.arange(T * S * H, dtype=torch.float32).reshape(T, S, H)
    sub = torch.ones(T, H)
    eye = torch.eye(S).expand(T, S, S)
    out = ops.mhc_close(res, sub, torch.tensor([[1.0, 0.0, 2.0, 0.5]] * T), eye)
    assert torch.equal(out[:, 1], res[:, 1]) and torch.equal(out[:, 0], res[:, 0] + 1) and torch.equal(out[:, 2], res[:, 2] + 2)
    swap = torch.zeros(T, S, S)
    swap[:, 0, 1] = swap[:, 1, 0] = swap[:, 2, 2] = swap[:, 3, 3] = 1.0          # source 0 -> destination 1, source 1 -> destination 0
    out = ops.mhc_close(res, sub, torch.zeros(T, S), swap)
    assert torch.equal(out[:, 1], res[:, 0]) and torch.equal(out[:, 0], res[:, 1])


def test_hyper_stack_chunked_prefill_equals_whole_prompt_and_differs_from_plain_stack():
    spec = tiny_spec().replace(n_layers=2, hyper_streams=4)
    masters = init_weights(spec, 1)
    assert masters["layers"][0]["hc_attn_fn"].shape == (24, 4 * spec.hidden) and masters["hc_head_fn"].shape == (4, 4 * spec.hidden)
    ref = RefModel(spec, masters)
    p = torch.randint(0, spec.vocab, (14,), generator=torch.Generator().manual_seed(2))
    whole, _ = ref.forward(p, 0, RefCache())
    c = RefCache()
    ref.forward(p[:6], 0, c)
    tail, _ = ref.forward(p[6:], 6, c)
    assert float((tail[-1] - whole[-1]).abs().max()) < 5e-3        # the streams are rounded to bf16 at every boundary
    plain = RefModel(tiny_spec().replace(n_layers=2), masters)
    other, _ = plain.forward(p, 0, RefCache())
    assert float((other[-1] - whole[-1]).abs().max()) > 5e-2
