"""Rank layouts of the attention/expert split (CPU)."""
import pytest

from cuteafd_b200.config import default_deployment


def test_named_layouts():
    d = default_deployment(8)
    assert (d.attn_ranks, d.expert_ranks, d.tp, d.ep, d.attn_groups) == ((0, 1), (2, 3, 4, 5, 6, 7), 2, 6, 1)
    assert d.describe() == "attn-tp2+ep6"
    assert default_deployment(1).describe() == "single"
    d2 = default_deployment(2)
    assert (d2.attn_ranks, d2.expert_ranks, d2.tp) == ((0,), (1,), 1)


@pytest.mark.parametrize("world,groups,attn,experts,tp", [(4, 2, (0, 1), (2, 3), 1), (8, 2, (0, 1, 2, 3), (4, 5, 6, 7), 2),
                                                          (8, 4, (0, 1, 2, 3), (4, 5, 6, 7), 1)])
def test_data_parallel_attention_groups(world, groups, attn, experts, tp):
    d = default_deployment(world, groups)
    assert (d.attn_ranks, d.expert_ranks, d.tp, d.attn_groups) == (attn, experts, tp, groups)
    seen = []
    for g in range(groups):
        ranks = d.group_ranks(g)
        assert len(ranks) == tp and all(d.group_of(r) == g for r in ranks)
        seen += list(ranks)
    assert tuple(seen) == attn
    assert f"dp{groups}x" in d.describe()


def test_groups_need_an_expert_rank():
    with pytest.raises(ValueError):
        default_deployment(4, 4)


def test_dispatch_flag_slots_are_distinct_per_group_and_tp_rank():
    from cuteafd_b200.config import tiny_spec
    from cuteafd_b200.parallel.afd import PH_COMBINE, PH_DISPATCH, PH_TP, flag_offset
    spec = tiny_spec()
    d = default_deployment(8, 2)
    offs = set()
    for ph in (PH_DISPATCH, PH_COMBINE, PH_TP):
        for layer in range(spec.n_layers):
            for src in range(8):
                offs.add(flag_offset(spec, ph, layer, src))
    assert len(offs) == 3 * spec.n_layers * 8 and max(offs) < 3 * spec.n_layers * 8 * 4
    assert {g * d.tp + t for g in range(d.attn_groups) for t in range(d.tp)} == {0, 1, 2, 3}


def test_plan_deployment_decisions_for_two_attention_groups():
    from cuteafd_b200.loader.plan import deployment_decisions, plan
    rep = plan("qwen3-235b", world=8, layout=True, attn_groups=2)
    d = deployment_decisions(rep.layout, "qwen3-235b")
    assert d["parallelism"] == "attn-dp2xtp2+ep4" and d["expert_ranks"] == [4, 5, 6, 7]
    assert [g["ranks"] for g in d["attention_groups"]] == [[0, 1], [2, 3]]
    r3, r6 = d["ranks"][3], d["ranks"][6]
    assert r3["attention_group"] == 1 and r3["tp_rank"] == 1 and r6["ep_rank"] == 2 and "attention_group" not in r6
    assert "--attn-groups 2" in d["launch"]["decode_bench"] and d["env"] == {"NCCL_NVLS_ENABLE": "0"}
    one = deployment_decisions(plan("qwen3-235b", world=1, layout=True).layout, "qwen3-235b")
    assert one["parallelism"] == "single" and one["launch"]["serve"].endswith("--model qwen3-235b")


def test_flag_words_of_every_layout_are_disjoint_and_pair_up():
    """Host-side fixture of the peer-flag protocol: for every layout the benchmark uses, each (phase, layer, publisher)
    has its own flag word inside the flags region, and every waiter's range covers exactly its publishers."""
    from cuteafd_b200.config import default_deployment, tiny_spec
    from cuteafd_b200.parallel.afd import PH_COMBINE, PH_DISPATCH, PH_TP, flag_offset
    spec = tiny_spec().replace(n_layers=5)
    region = 3 * spec.n_layers * 8 * 4
    for world, groups in ((2, 1), (4, 1), (4, 2), (8, 1), (8, 2), (8, 4)):
        dep = default_deployment(world, groups)
        for li in range(spec.n_layers):
            seen = {}
            # dispatch: every attention rank raises its own word on the expert ranks; an expert rank waits, per group, on
            # `tp` consecutive words starting at the group's first slot
            pub = {}
            for r in dep.attn_ranks:
                g = dep.group_of(r)
                src = g * dep.tp + list(dep.group_ranks(g)).index(r)
                off = flag_offset(spec, PH_DISPATCH, li, src)
                assert off not in seen and 0 <= off < region and off % 4 == 0
                seen[off] = ("dispatch", r)
                pub.setdefault(g, set()).add(off)
            for g in range(dep.attn_groups):
                first = flag_offset(spec, PH_DISPATCH, li, g * dep.tp)
                assert {first + 4 * i for i in range(dep.tp)} == pub[g]
            # combine: every expert rank raises word `ep_rank` on the attention ranks, which wait on `ep` consecutive words
            for i, r in enumerate(dep.expert_ranks):
                off = flag_offset(spec, PH_COMBINE, li, i)
                assert off not in seen and off < region
                seen[off] = ("combine", r)
            first = flag_offset(spec, PH_COMBINE, li, 0)
            assert {first + 4 * i for i in range(dep.ep)} == {o for o, (k, _) in seen.items() if k == "combine"}
            # tensor-parallel pair: rank t raises word t on its partner and waits on word 1 - t of its own block
            for t in range(min(2, dep.tp)):
                off = flag_offset(spec, PH_TP, li, t)
                assert off not in seen and off < region
                seen[off] = ("tp", t)
        assert dep.attn_groups * dep.tp <= 8 and dep.ep <= 8            # the region has eight words per (phase, layer)
