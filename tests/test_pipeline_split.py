"""Layer-range split: stage planning on the CPU; on the GPU the stages of a split run one after the other on one device (the real
hop kernels: push + release flag, bounded wait + copy) and must generate the single-GPU engine's tokens."""
import dataclasses

import pytest
import torch

from cuteafd_b200.config import AttentionSpec, tiny_spec
from cuteafd_b200.parallel.pipeline import stage_masters, stage_ranges, stage_spec


def test_stage_ranges_are_consecutive_even_and_respect_the_layer_period():
    assert stage_ranges(8, 2) == [(0, 4), (4, 8)]
    assert stage_ranges(7, 3) == [(0, 2), (2, 5), (5, 7)]
    assert stage_ranges(12, 2, period=4) == [(0, 8), (8, 12)] or stage_ranges(12, 2, period=4) == [(0, 4), (4, 12)]
    for lo, hi in stage_ranges(12, 3, period=4):
        assert lo % 4 == 0 and hi > lo
    with pytest.raises(ValueError):
        stage_ranges(4, 5)


def test_stage_spec_keeps_the_meaning_of_layer_indices():
    base = tiny_spec()
    spec = base.replace(n_layers=6, moe=dataclasses.replace(base.moe, first_dense=2, dense_intermediate=128))
    a, b, c = stage_spec(spec, 0, 1), stage_spec(spec, 1, 4), stage_spec(spec, 4, 6)
    assert (a.n_layers, a.moe.first_dense) == (1, 1) and (b.n_layers, b.moe.first_dense) == (3, 1) and (c.n_layers, c.moe.first_dense) == (2, 0)
    hybrid = base.replace(n_layers=8, attn=dataclasses.replace(base.attn, window=16, full_every=4))
    assert stage_spec(hybrid, 4, 8).layer_is_full(0) == hybrid.layer_is_full(4)
    with pytest.raises(ValueError):
        stage_spec(hybrid, 2, 8)
    with pytest.raises(NotImplementedError):
        stage_spec(spec.replace(mtp_layers=1), 0, 3)
    m = {"embed": 1, "lm_head": 2, "final_norm": 3, "layers": list(range(6)), "mtp": []}
    assert stage_masters(m, 1, 4) == {"embed": 1, "lm_head": 2, "final_norm": 3, "layers": [1, 2, 3]}


@pytest.mark.gpu
@pytest.mark.parametrize("n_stages,first_dense", [(2, 0), (4, 1)])
def test_stages_on_one_gpu_generate_the_single_gpu_tokens(n_stages, first_dense):
    from cuteafd_b200.parallel.local import LocalBlocks
    from cuteafd_b200.parallel.pipeline import PipelineRank, generate_pipeline, hop_regions
    from cuteafd_b200.parallel.selftest import reference_tokens, tokens_agree
    from cuteafd_b200.ref.model import init_weights
    dev = "cuda:0"
    base = tiny_spec()
    spec = base.replace(n_layers=4, moe=dataclasses.replace(base.moe, first_dense=first_dense, dense_intermediate=128))
    masters = init_weights(spec, 7)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, spec.vocab, (n,), generator=g).tolist() for n in (19, 33, 7)]
    want, top2 = reference_tokens(spec, masters, prompts, 8, torch.device(dev))
    blocks = LocalBlocks(hop_regions(spec, 256), dev, n_stages)
    ranks = [PipelineRank(spec, r, n_stages, dev, n_pages=32, max_seqs=8, max_pages_per_seq=4, t_cap=256, masters=masters, block=blocks.view(r))
             for r in range(n_stages)]
    assert [(r.engine.lo, r.engine.hi) for r in ranks] == [(i * 4 // n_stages, (i + 1) * 4 // n_stages) for i in range(n_stages)]
    assert sum(r.engine.kv.shape[0] for r in ranks) == 4                 # every stage caches its own layers only
    got = generate_pipeline(ranks, prompts, 8)
    # the last layer of a stage cannot fuse the next layer's norm into its combine: a near tie may round the other way
    assert tokens_agree(got, want, top2, exact=False), (got, want)
    assert ranks[0].link.hop_bytes > 0 and ranks[-1].link.hop_bytes == 0
