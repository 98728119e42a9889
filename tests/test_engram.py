"""N-gram memory: addressing, request-owned history (prepare / commit / fork / resume), row format and the gate (CPU oracle)."""
import numpy as np
import pytest
import torch

from cuteafd_b200.ref.engram import (COLUMNS, EngramAddressing, EngramHistory, EngramSpec, context_hashes, dequantize_rows, engram_apply,
                                     engram_gate, init_engram_weights, quantize_rows)


def test_addressing_is_a_pure_function_of_the_last_four_ids_and_stays_inside_each_heads_table():
    spec = EngramSpec(layers=(1, 3), vocab=1000, prime_floor=300)
    addr = EngramAddressing(spec)
    assert addr.primes.shape == (2, COLUMNS) and len(set(addr.primes.reshape(-1).tolist())) == 2 * COLUMNS
    assert all(int(m) % 2 == 1 for m in addr.mult.reshape(-1))
    ids = np.array([0, 0, 0, 5, 9, 2, 7, 5, 9, 2, 7], dtype=np.int64)
    h = addr.hashes(ids)
    assert h.shape == (2, 8, COLUMNS)
    for l in range(2):
        lo, hi = addr.offsets[l], addr.offsets[l] + addr.primes[l]
        assert (h[l] >= lo[None, :]).all() and (h[l] < hi[None, :]).all() and int(hi[-1]) == addr.rows[l]
    # positions 3 and 7 end the same 4-gram (5 9 2 7): every order agrees; positions 2 and 6 (.. 5 9 2) agree in orders 2 and 3 only
    assert (h[:, 3] == h[:, 7]).all()
    assert (h[:, 2, :16] == h[:, 6, :16]).all() and (h[:, 2, 16:] != h[:, 6, 16:]).any()
    # wrap-around arithmetic against Python integers
    m, p = [int(x) for x in addr.mult[0]], [int(x) for x in addr.primes[0]]
    r = (7 * m[0]) % 2 ** 64
    r ^= (2 * m[1]) % 2 ** 64
    assert int(h[0, 3, 0]) == r % p[0] and int(h[0, 3, 1]) == r % p[1] + p[0]


def test_history_prepares_without_side_effects_and_commits_only_what_was_accepted():
    spec = EngramSpec(layers=(0,), vocab=500)
    addr = EngramAddressing(spec)
    seq = [11, 12, 13, 14, 15, 16, 17]
    want = context_hashes(addr, [], seq)
    h = EngramHistory(spec.pad_id)
    b1 = h.prepare(addr, seq[:4])
    assert (b1.hashes == want[:, :4]).all() and h.position == 0
    h.commit(b1, 4)
    drafts = h.prepare(addr, [15, 99, 98])                # a speculative batch: only the first token is accepted
    h.commit(drafts, 1)
    with pytest.raises(ValueError):
        h.commit(drafts, 1)                               # prepared against the state before that commit
    b3 = h.prepare(addr, seq[5:])
    assert (b3.hashes == want[:, 5:]).all()
    fork = h.fork()
    with pytest.raises(ValueError):
        fork.commit(b3, 2)                                # another request identity
    h.commit(b3, 2)
    assert h.position == 7 and h.recent == (17, 16, 15)
    again = EngramHistory.from_recent(spec.pad_id, 7, [15, 16, 17])
    assert (again.prepare(addr, [3]).hashes == h.prepare(addr, [3]).hashes).all()
    with pytest.raises(ValueError):
        EngramHistory.from_recent(spec.pad_id, 7, [16, 17])


def test_an_image_position_is_a_barrier():
    spec = EngramSpec(layers=(0,), vocab=500, pad_id=1)
    addr = EngramAddressing(spec)
    h = EngramHistory(spec.pad_id)
    b = h.prepare(addr, [21, 22, None, 23, 24])
    assert b.is_image(2) and not b.is_image(3)
    fresh = context_hashes(addr, [], [23, 24])            # behind the image the lookback starts over
    assert (b.hashes[:, 3:] == fresh).all()


def test_row_format_round_trip_and_gate_limits():
    g = torch.Generator().manual_seed(0)
    rows = torch.randn(50, 256, generator=g) * torch.logspace(-3, 2, 50)[:, None]
    q, e = quantize_rows(rows)
    back = dequantize_rows(q, e)
    assert q.shape == (50, 256) and e.shape == (50, 8)
    assert float(((back - rows).abs() / rows.abs().clamp(min=1e-6)).median()) < 0.04
    x = torch.randn(6, 4, 64, generator=g)
    kv = torch.randn(6, 5, 64, generator=g)
    ones = torch.ones(4, 64)
    out = engram_gate(x, kv, ones, ones)
    gate = ((out - x) / kv[:, 4][:, None, :]).mean(-1)
    assert ((gate > 0) & (gate < 1)).all()
    aligned = engram_gate(x, torch.cat([x * 3, kv[:, 4:]], dim=1), ones, ones)          # key parallel to the stream: the gate opens
    assert (((aligned - x) / kv[:, 4][:, None, :]).mean(-1) > 0.9).all()
    mask = torch.tensor([True, False, True, True, False, True])
    masked = engram_gate(x, kv, ones, ones, mask)
    assert torch.equal(masked[1], x[1]) and torch.equal(masked[0], out[0])


def test_apply_reads_the_addressed_rows():
    spec = EngramSpec(layers=(0,), vocab=200, row_dim=64, prime_floor=100, streams=2, hidden=32)
    w = init_engram_weights(spec, 1)
    addr = EngramAddressing(spec)
    hs = context_hashes(addr, [5, 6, 7], [8, 9])
    x = torch.randn(2, 2, 32, generator=torch.Generator().manual_seed(2))
    out = engram_apply(spec, w["layers"][0], x, hs[0])
    assert out.shape == x.shape and (out != x).any()
    lw = dict(w["layers"][0])
    lw["table_q"] = lw["table_q"].clone()
    lw["table_q"][int(hs[0, 1, 5])] ^= 0x40              # one addressed row of the second token changes: only that token moves
    out2 = engram_apply(spec, lw, x, hs[0])
    assert torch.equal(out2[0], out[0]) and not torch.equal(out2[1], out[1])


def test_oracle_model_with_an_ngram_memory_is_causal_and_chunk_invariant():
    """The stack with engram layers: chunked prefill equals one-shot prefill (the lookback crosses chunk borders through the cache's
    token list), later tokens do not change earlier rows, and the memory does change the output."""
    from cuteafd_b200.config import tiny_spec
    from cuteafd_b200.ref.model import RefCache, RefModel, init_weights
    spec = tiny_spec().replace(engram_layers=(0, 1), engram_row_dim=64, engram_prime_floor=200)
    w = init_weights(spec, 3)
    assert len(w["engram"]["layers"]) == 2
    m = RefModel(spec, w)
    toks = torch.randint(0, spec.vocab, (21,), generator=torch.Generator().manual_seed(4))
    full, _ = m.forward(toks, 0, RefCache())
    chunked, _ = m.forward(toks, 0, RefCache(), chunk=8)
    assert torch.allclose(full, chunked, atol=2e-4)
    c = RefCache()
    part, _ = m.forward(toks[:13], 0, c)
    assert torch.allclose(part, full[:13], atol=2e-4)
    step, _ = m.forward(toks[13:14], 13, c)                      # a decode step continues the same addressing
    assert torch.allclose(step[0], full[13], atol=2e-4)
    plain = RefModel(spec.replace(engram_layers=()), w)
    off, _ = plain.forward(toks, 0, RefCache())
    assert float((off - full).abs().max()) > 1e-3
    from cuteafd_b200.config import spec_from_json, spec_to_json
    import json
    assert spec_from_json(json.loads(json.dumps(spec_to_json(spec)))) == spec
