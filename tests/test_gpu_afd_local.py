"""Multi-rank layouts of the attention/expert split run as one process on one GPU (`parallel.local.LocalWorld`): the real
peer kernels and flag protocol, scheduled so that every wait is already satisfied.  Every layout must generate exactly the
single-GPU engine's tokens."""
import dataclasses

import pytest
import torch

from cuteafd_b200.config import AttentionSpec, MoESpec, QuantSpec, colocated_deployment, default_deployment, tiny_spec
from cuteafd_b200.ref.model import init_weights

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _prompts(spec, seed, n=2, length=24):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, spec.vocab, (length + 3 * i,), generator=g).tolist() for i in range(n)]


def _single_gpu_tokens(spec, masters, prompts, n_new):
    from cuteafd_b200.engine.engine import Engine
    from cuteafd_b200.engine.generate import generate
    from cuteafd_b200.models.weights import DeviceWeights
    eng = Engine(DeviceWeights.from_masters(spec, masters, DEV), n_pages=32, max_seqs=8, max_pages_per_seq=4)
    return generate(eng, prompts, n_new, use_graph=False)


def _world(spec, masters, dep, n_micro, merged, t_cap=128):
    from cuteafd_b200.parallel.afd import LanePlan
    from cuteafd_b200.parallel.local import LocalWorld
    return LocalWorld(spec, LanePlan(dep, t_cap=t_cap, n_micro=n_micro, merged=merged), DEV, n_pages=32, max_seqs=8, max_pages_per_seq=4,
                      masters=masters)


LAYOUTS = [
    ("1 attention + 1 expert rank", lambda: default_deployment(2), 1, False),
    ("TP2 + EP2, two micro-batches in flight", lambda: default_deployment(4), 2, False),
    ("two attention groups + EP2, lane by lane", lambda: default_deployment(4, 2), 1, False),
    ("two attention groups + EP2, lanes merged into one grouped GEMM", lambda: default_deployment(4, 2), 1, True),
    ("colocated x4", lambda: colocated_deployment(4), 1, True),
    ("colocated x2, two micro-batches", lambda: colocated_deployment(2), 2, True),
]


@pytest.mark.parametrize("experts", ["nvfp4", "bf16"])
@pytest.mark.parametrize("name,dep_fn,n_micro,merged", LAYOUTS, ids=[l[0] for l in LAYOUTS])
def test_layout_generates_the_single_gpu_tokens(name, dep_fn, n_micro, merged, experts):
    from cuteafd_b200.parallel.local import generate_local
    spec = tiny_spec().replace(quant=QuantSpec(experts=experts, dense="bf16"))
    masters = init_weights(spec, 5)
    dep = dep_fn()
    world = _world(spec, masters, dep, n_micro, merged)
    prompts = [_prompts(spec, 3 + g, n=3) for g in range(dep.attn_groups)]
    got = generate_local(world, prompts, 6)
    for g in range(dep.attn_groups):
        assert got[g] == _single_gpu_tokens(spec, masters, prompts[g], 6), (name, g)


def test_idle_group_still_takes_part():
    """A data-parallel group with no sequences dispatches an empty lane every layer; the busy groups are unaffected."""
    from cuteafd_b200.parallel.local import generate_local
    spec = tiny_spec().replace(quant=QuantSpec(experts="mxfp4", dense="bf16"))
    masters = init_weights(spec, 6)
    world = _world(spec, masters, colocated_deployment(4), 1, True)
    prompts = [_prompts(spec, 11), [], _prompts(spec, 12, n=1), []]
    got = generate_local(world, prompts, 5)
    assert got[0] == _single_gpu_tokens(spec, masters, prompts[0], 5)
    assert got[2] == _single_gpu_tokens(spec, masters, prompts[2], 5)


def test_mla_split_generates_the_single_gpu_tokens():
    """DeepSeek-V3-style attention (MLA) on the split: TP2 over heads + EP2, two micro-batches."""
    from cuteafd_b200.parallel.local import generate_local
    base = tiny_spec()
    spec = base.replace(attn=AttentionSpec(kind="mla", n_heads=8, n_kv_heads=8, head_dim=192, q_lora_rank=64, kv_lora_rank=512,
                                           qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128),
                        moe=dataclasses.replace(base.moe, first_dense=1, dense_intermediate=256),
                        quant=QuantSpec(experts="mxfp4", dense="bf16"))
    masters = init_weights(spec, 7)
    prompts = _prompts(spec, 21, n=4)
    from cuteafd_b200.parallel.selftest import reference_tokens, tokens_agree
    want, top2 = reference_tokens(spec, masters, prompts, 5, DEV)
    for dep, n_micro, merged in ((default_deployment(2), 2, False), (default_deployment(4), 2, False), (colocated_deployment(2), 1, True)):
        world = _world(spec, masters, dep, n_micro, merged)
        groups = [prompts] if dep.attn_groups == 1 else [prompts[:2], prompts[2:]]
        got = generate_local(world, groups, 5)
        flat = [o for g in got for o in g]
        # heads split over two ranks sum two bf16-rounded partial projections: a near tie of the reference may flip there;
        # every other layout computes exactly what the single-GPU engine computes
        assert tokens_agree(flat, want, top2, exact=dep.tp == 1), (dep.describe(), flat, want)


@pytest.mark.parametrize("experts", ["nvfp4", "bf16"])
def test_expert_tp_layouts(experts):
    """Expert TP: every expert rank holds an intermediate-dimension slice of every expert; rows are broadcast, the attention
    rank adds the ranks' partial sums in fixed order.  Three expert ranks make the slices uneven (zero-padded)."""
    from cuteafd_b200.config import Deployment
    from cuteafd_b200.parallel.afd import LanePlan
    from cuteafd_b200.parallel.local import LocalWorld, generate_local
    from cuteafd_b200.parallel.selftest import reference_tokens, tokens_agree
    spec = tiny_spec().replace(quant=QuantSpec(experts=experts, dense="bf16"))
    masters = init_weights(spec, 5)
    prompts = _prompts(spec, 31, n=3)
    want, top2 = reference_tokens(spec, masters, prompts, 6, DEV)
    deps = [(default_deployment(2), 1), (Deployment(world=4, attn_ranks=(0,), expert_ranks=(1, 2, 3), colocated=False), 2), (colocated_deployment(2), 1)]
    for dep, n_micro in deps:
        plan = LanePlan(dep, t_cap=128, n_micro=n_micro, merged=dep.colocated, expert_tp=True)
        world = LocalWorld(spec, plan, DEV, n_pages=32, max_seqs=8, max_pages_per_seq=4, masters=masters)
        groups = [prompts] if dep.attn_groups == 1 else [prompts[:2], prompts[2:]]
        got = generate_local(world, groups, 6)
        flat = [o for g in got for o in g]
        # each rank rounds its partial FC2 sum to bf16 before the ranks are added: a near tie of the reference may flip
        assert tokens_agree(flat, want, top2, exact=False), (dep.describe(), flat, want)


def test_scheduler_refuses_a_wait_without_a_push():
    """The single-GPU scheduler never launches a kernel whose flags nobody publishes: it raises instead."""
    from cuteafd_b200.parallel.local import Deadlock, run_programs

    def lonely():
        yield [0xdead0]
        raise AssertionError("resumed although the flag was never published")

    with pytest.raises(Deadlock):
        run_programs({"a": lonely()})


def test_tp_pair_splits_the_head_over_the_vocabulary():
    """On a TP pair each rank keeps and multiplies by its share of the LM head only; the shares of the logit rows are exchanged over
    peer memory, so both ranks select from the same complete rows (tokens equal the single-GPU engine's: the layout test above).
    Here: the split is engaged, the weights are halved, and both ranks hold bit-identical full logits after a step."""
    from cuteafd_b200.parallel.afd import head_split
    from cuteafd_b200.parallel.local import generate_local
    spec = tiny_spec().replace(quant=QuantSpec(experts="bf16", dense="bf16"))
    masters = init_weights(spec, 5)
    dep = default_deployment(4)
    world = _world(spec, masters, dep, 1, False)
    a, b = (world.engines[r] for r in dep.attn_ranks[:2])
    assert a.vocab_parallel and b.vocab_parallel
    w = head_split(spec.vocab)
    assert (a.weights.lm_head.N, b.weights.lm_head.N) == w and sum(w) == spec.vocab
    prompts = [_prompts(spec, 3, n=3)]
    got = generate_local(world, prompts, 4)
    assert got[0] == _single_gpu_tokens(spec, masters, prompts[0], 4)
    la, lb = a.lane(3).logits[:3], b.lane(3).logits[:3]
    assert torch.equal(la, lb) and float(la.abs().max()) > 0
