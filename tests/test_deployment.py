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
    from cuteafd_b200.parallel.afd import NFLAG, PH_COMBINE, PH_DISPATCH, PH_TP, flag_offset, n_flag_layers
    spec = tiny_spec().replace(mtp_layers=1)
    d = default_deployment(8, 2)
    offs = set()
    for ph in (PH_DISPATCH, PH_COMBINE, PH_TP):
        for layer in range(n_flag_layers(spec)):            # the MTP draft layer has its own words
            for src in range(NFLAG):
                offs.add(flag_offset(spec, ph, layer, src))
    assert len(offs) == 3 * n_flag_layers(spec) * NFLAG and max(offs) < 3 * n_flag_layers(spec) * NFLAG * 4
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
    """Host-side fixture of the peer-flag protocol: for every layout and micro-batch count, each (phase, layer, publisher)
    has its own flag word inside the flags region, and every waiter's range covers exactly its publishers."""
    from cuteafd_b200.config import colocated_deployment, default_deployment, tiny_spec
    from cuteafd_b200.parallel.afd import NFLAG, PH_COMBINE, PH_DISPATCH, PH_TP, LanePlan, block_regions, flag_offset
    spec = tiny_spec().replace(n_layers=5)
    cases = [(default_deployment(w, g), m, mg) for w, g in ((2, 1), (4, 1), (4, 2), (8, 1), (8, 2)) for m in (1, 2) for mg in (False, True)]
    cases += [(colocated_deployment(w), m, True) for w in (2, 4, 8) for m in (1, 2) if w * m <= 8]
    for dep, n_micro, merged in cases:
        plan = LanePlan(dep, t_cap=16, n_micro=n_micro, merged=merged)
        plan.check()
        region = block_regions(spec, plan, 1)["flags"]
        for li in range(spec.n_layers):
            seen = {}
            # dispatch: attention rank (group g, tp rank t) raises word lane * tp + t on every expert rank for each of its
            # micro-batch lanes; an expert rank waits on the tp words of one lane, or on all lanes * tp words when merged
            pub = {}
            for r in dep.attn_ranks:
                g = dep.group_of(r)
                t = list(dep.group_ranks(g)).index(r)
                for mb in range(n_micro):
                    lane = plan.lane(g, mb)
                    off = flag_offset(spec, PH_DISPATCH, li, lane * dep.tp + t)
                    assert off not in seen and 0 <= off < region and off % 4 == 0
                    seen[off] = ("dispatch", r, mb)
                    pub.setdefault(lane, set()).add(off)
            runs = [(0, plan.n_lanes)] if merged else [(lane, 1) for lane in range(plan.n_lanes)]
            covered = set()
            for lane0, n in runs:
                first = flag_offset(spec, PH_DISPATCH, li, lane0 * dep.tp)
                waits = {first + 4 * i for i in range(n * dep.tp)}
                assert waits == set().union(*(pub[l] for l in range(lane0, lane0 + n)))
                covered |= waits
            assert covered == {o for o, v in seen.items() if v[0] == "dispatch"}
            # combine: expert rank e raises word mb * 8 + e on the attention ranks of a lane; micro-batch mb of an attention
            # rank waits on `ep` consecutive words starting at mb * 8
            for mb in range(n_micro):
                words = set()
                for e in range(dep.ep):
                    off = flag_offset(spec, PH_COMBINE, li, mb * 8 + e)
                    assert off not in seen and off < region
                    seen[off] = ("combine", e, mb)
                    words.add(off)
                first = flag_offset(spec, PH_COMBINE, li, mb * 8)
                assert {first + 4 * i for i in range(dep.ep)} == words
            # tensor-parallel pair: rank t raises word mb * 2 + t on its partner and waits on word mb * 2 + (1 - t) of its own block
            for mb in range(n_micro):
                for t in range(min(2, dep.tp)):
                    off = flag_offset(spec, PH_TP, li, mb * 2 + t)
                    assert off not in seen and off < region
                    seen[off] = ("tp", t, mb)
        assert plan.n_lanes * dep.tp <= 8 and dep.ep <= 8 and n_micro * 8 <= NFLAG
