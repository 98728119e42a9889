"""Sparse attention with a learned indexer (DSA): index-score kernel, top-k selection and row gather against plain PyTorch
references, and the MLA engine's sparse path against the fp32 oracle."""
import pytest
import torch

from cuteafd_b200.config import AttentionSpec, ModelSpec, MoESpec, QuantSpec
from cuteafd_b200.engine.generate import BatchGenerator
from cuteafd_b200.engine.mla import MlaEngine, mla_weights_from_masters
from cuteafd_b200.ops.native import call, ptr, stream
from cuteafd_b200.ref import ops as rops
from cuteafd_b200.ref.model import RefModel, init_weights

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _paged(n_seq, lens, max_pages, n_pages, gen):
    """Random page tables: sequence s owns ceil(len / 64) distinct pages."""
    perm = (torch.randperm(n_pages - 1, generator=gen) + 1).tolist()
    table = torch.zeros(n_seq, max_pages, dtype=torch.int32)
    for s, n in enumerate(lens):
        for j in range(-(-n // 64)):
            table[s, j] = perm.pop()
    return table


def test_index_scores_topk_and_gather():
    g = torch.Generator().manual_seed(4)
    Hi, Di, n_pages, max_pages = 32, 128, 24, 8
    kv_len, q_len = [300, 70, 129], [1, 3, 2]
    n_seq, T = len(kv_len), sum(q_len)
    q_start = [0, 1, 4]
    table = _paged(n_seq, kv_len, max_pages, n_pages, g)
    cache = torch.randn(n_pages * 64, Di, generator=g).to(torch.bfloat16)
    q_idx = torch.randn(T, Hi, Di, generator=g).to(torch.bfloat16)
    w = torch.randn(T, Hi, generator=g)
    ld = max_pages * 64
    d = lambda t: t.to(DEV)
    cache_d, q_d, w_d, table_d = d(cache), d(q_idx), d(w), d(table)
    kv_d, qs_d, ql_d = d(torch.tensor(kv_len, dtype=torch.int32)), d(torch.tensor(q_start, dtype=torch.int32)), d(torch.tensor(q_len, dtype=torch.int32))
    tmap = torch.zeros(128, dtype=torch.uint8)
    call("cuteafd_tmap_encode_index_keys", tmap.data_ptr(), cache_d.data_ptr(), n_pages * 64)
    tmap_d = d(tmap)
    scores = torch.full((T, ld), 7.0, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    call("cuteafd_dsa_index_scores", ptr(q_d), ptr(w_d), ptr(tmap_d), ptr(table_d), ptr(kv_d), ptr(qs_d), ptr(ql_d), ptr(scores), T, n_seq, max(q_len),
         ld, Hi, ld, max_pages, ptr(status), stream())
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    got = scores.cpu()
    positions, seq_of_row = [], []
    for s in range(n_seq):
        keys = torch.stack([cache[int(table[s, p // 64]) * 64 + p % 64] for p in range(kv_len[s])])
        qpos = torch.arange(kv_len[s] - q_len[s], kv_len[s])
        rows = slice(q_start[s], q_start[s] + q_len[s])
        want = rops.index_scores(q_idx[rows], w[rows], keys, qpos, torch.arange(kv_len[s]))
        g_rows = got[rows, :kv_len[s]]
        fin = torch.isfinite(want)
        assert torch.equal(torch.isfinite(g_rows), fin)
        err = float((g_rows[fin] - want[fin]).abs().max() / want[fin].abs().max())
        assert err < 2e-3, f"sequence {s}: relative error {err}"
        positions += qpos.tolist()
        seq_of_row += [s] * q_len[s]
    # top-k over the device's own scores: the set must be the k best of each row, ties to the lowest position
    k = 64
    pos_d = d(torch.tensor(positions, dtype=torch.int32))
    sel, cnt = torch.zeros(T, k, dtype=torch.int32, device=DEV), torch.zeros(T, dtype=torch.int32, device=DEV)
    call("cuteafd_dsa_topk", ptr(scores), ld, ptr(pos_d), T, k, 1, ptr(sel), ptr(cnt), stream())
    torch.cuda.synchronize()
    for r in range(T):
        n = positions[r] + 1
        want = rops.topk_mask(got[r:r + 1, :n], k)[0].nonzero().flatten().tolist()
        c = int(cnt[r])
        assert c == min(n, k) and sorted(sel[r, :c].tolist()) == want and (sel[r, c:] == -1).all()
    # gather of the selected rows of a 576-wide paged cache into per-row pseudo-pages
    lat = torch.randn(n_pages * 64, 576, generator=g).to(torch.bfloat16)
    lat_d = d(lat)
    kp = 64
    dst = torch.zeros(T * kp, 576, dtype=torch.bfloat16, device=DEV)
    sor_d = d(torch.tensor(seq_of_row, dtype=torch.int32))
    call("cuteafd_dsa_gather_rows", ptr(lat_d), ptr(table_d), ptr(sor_d), ptr(sel), ptr(cnt), ptr(dst), T, k, kp,
         max_pages, n_pages * 64, 1152, ptr(status), stream())
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    out = dst.cpu().view(T, kp, 576)
    for r in range(T):
        s = seq_of_row[r]
        for j in range(int(cnt[r])):
            p = int(sel[r, j])
            assert torch.equal(out[r, j], lat[int(table[s, p // 64]) * 64 + p % 64])


def dsa_spec(topk):
    return ModelSpec(name="mla-dsa", family="deepseek_v3", vocab=512, hidden=256, n_layers=2, rms_eps=1e-6,
                     attn=AttentionSpec(kind="mla", n_heads=4, n_kv_heads=4, head_dim=192, q_lora_rank=64, kv_lora_rank=512, qk_nope_head_dim=128,
                                        qk_rope_head_dim=64, v_head_dim=128, index_topk=topk, index_heads=32, index_dim=128),
                     moe=MoESpec(n_experts=8, top_k=2, intermediate=128, n_shared=1, scoring="sigmoid", use_bias=True, n_group=4, topk_group=2,
                                 route_scale=2.5, first_dense=1, dense_intermediate=256),
                     quant=QuantSpec(experts="bf16", dense="bf16"))


def _bf16(tree):
    if isinstance(tree, torch.Tensor):
        return tree.to(torch.bfloat16).float() if tree.dim() >= 2 else tree
    if isinstance(tree, dict):
        return {k: _bf16(v) for k, v in tree.items()}
    if isinstance(tree, list):
        return [_bf16(v) for v in tree]
    return tree


@pytest.mark.parametrize("topk,prompt_lens,chunk", [(256, (70, 33), 4096), (64, (150, 90), 8)])
def test_engine_sparse_path_tracks_the_oracle(topk, prompt_lens, chunk):
    """topk 256 covers every context: the sparse path (score, select, gather, attend) must reproduce dense attention.  topk 64 with
    150-token prompts fed eight rows at a time: every row beyond position 63 attends to its 64 selected positions only, in the
    engine and in the oracle; a token may differ only where the oracle's own top-2 margin is small (a selection or rounding flip)."""
    spec = dsa_spec(topk)
    masters = _bf16(init_weights(spec, 2))
    eng = MlaEngine(mla_weights_from_masters(spec, masters, DEV), n_pages=32, max_seqs=4, max_pages_per_seq=6)
    ref = RefModel(spec, masters)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, spec.vocab, (n,), generator=g).tolist() for n in prompt_lens]
    used = []
    orig = MlaEngine._sparse_attention

    def spy(self, *a, **k):
        used.append(1)
        return orig(self, *a, **k)
    MlaEngine._sparse_attention = spy
    try:
        gen = BatchGenerator(eng, prefill_chunk=chunk)
        out = [[t] for t in gen.prefill(prompts)]
        for _ in range(5):
            for o, t in zip(out, gen.decode_step(use_graph=True)):
                o.append(t)
    finally:
        MlaEngine._sparse_attention = orig
    torch.cuda.synchronize()
    eng.check_status()
    gen.release()
    assert used, "the sparse path did not run"
    for i, p in enumerate(prompts):
        want, rows = ref.generate_greedy(torch.tensor(p), 6, chunk=chunk if chunk < 4096 else 0)
        for j, (a_, b_) in enumerate(zip(out[i], want)):
            if a_ != b_:
                top2 = rows[j].topk(2).values
                assert float(top2[0] - top2[1]) < 0.05, f"prompt {i} step {j}: {a_} != {b_}"
                break
