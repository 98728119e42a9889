"""Checkpoint reader: HF-layout snapshots (bf16, FP8 128x128, NVFP4, MXFP4; sharded) decode to the oracle's masters."""
import dataclasses

import pytest
import torch

from cuteafd_b200.config import tiny_spec
from cuteafd_b200.loader import checkpoint as ck
from cuteafd_b200.loader.formats import detect_all
from cuteafd_b200.loader.safetensors_io import catalog
from cuteafd_b200.ref import quant
from cuteafd_b200.ref.model import RefModel, init_weights


def bf16r(t):
    return t.to(torch.bfloat16).float()


def test_bf16_snapshot_round_trip_and_same_tokens(tmp_path):
    spec = tiny_spec().replace(mtp_layers=1)
    masters = init_weights(spec, 3)
    snap = ck.export_snapshot(spec, masters, tmp_path / "snap", shard_layers=1)
    assert len(list(snap.glob("*.safetensors"))) == spec.n_layers
    got = ck.read_masters(snap, spec)
    assert torch.equal(got["embed"], bf16r(masters["embed"])) and torch.equal(got["lm_head"], bf16r(masters["lm_head"]))
    for a, b in zip(got["layers"] + [got["mtp"][0]["layer"]], masters["layers"] + [masters["mtp"][0]["layer"]]):
        assert set(a) == set(b)
        for k in b:
            want = b[k].float() if k in ("router_bias", "sink") else bf16r(b[k])
            assert torch.equal(a[k], want), k
    assert torch.equal(got["mtp"][0]["eh_proj"], bf16r(masters["mtp"][0]["eh_proj"]))
    prompt = torch.randint(0, spec.vocab, (9,), generator=torch.Generator().manual_seed(0))
    rounded = RefModel(spec, got).generate_greedy(prompt, 5)[0]
    spec_toks, _ = RefModel(spec, got).generate_speculative(prompt, 5, 2)
    assert rounded == spec_toks


@pytest.mark.parametrize("experts", ["nvfp4", "mxfp4"])
def test_fp4_expert_snapshot_decodes_to_the_oracle_quantisation(tmp_path, experts):
    spec = tiny_spec()
    masters = init_weights(spec, 4)
    snap = ck.export_snapshot(spec, masters, tmp_path / "snap", experts=experts)
    ops, bad = detect_all(catalog(snap))
    assert not bad
    assert ops["model.layers.0.mlp.experts.3.up_proj"].format == experts
    got = ck.read_masters(snap, spec)
    for li, lw in enumerate(masters["layers"]):
        if "w_up" not in lw:
            continue
        for e in (0, spec.moe.n_experts - 1):
            w = lw["w_down"][e]
            if experts == "nvfp4":
                p, s, g = quant.nvfp4_quantize(w)
                want = quant.nvfp4_dequantize(p, s, g)
            else:
                p, s = quant.mxfp4_quantize(w)
                want = quant.mxfp4_dequantize(p, s)
            assert torch.equal(got["layers"][li]["w_down"][e], want)
    assert torch.equal(got["layers"][0]["wq"], bf16r(masters["layers"][0]["wq"]))      # dense stays bf16


def test_fp8_block_dense_snapshot(tmp_path):
    base = tiny_spec()
    spec = base.replace(attn=dataclasses.replace(base.attn, n_kv_heads=4))           # k/v projections of 128 rows: whole scale blocks
    masters = init_weights(spec, 5)
    snap = ck.export_snapshot(spec, masters, tmp_path / "snap", dense="fp8_block128")
    ops, bad = detect_all(catalog(snap))
    assert not bad and ops["model.layers.1.self_attn.o_proj"].format == "fp8_block128"
    got = ck.read_masters(snap, spec)
    q, s = quant.fp8_block_quantize(masters["layers"][1]["wo"])
    assert torch.equal(got["layers"][1]["wo"], quant.fp8_block_dequantize(q, s))
    assert torch.equal(got["layers"][0]["router"], bf16r(masters["layers"][0]["router"]))


def test_plan_lists_the_files_each_rank_reads(tmp_path, capsys):
    """Role-sliced view of a snapshot: attention ranks read everything but routed experts, expert ranks their expert range."""
    from cuteafd_b200 import cli
    from cuteafd_b200.config import default_deployment, tiny_spec
    from cuteafd_b200.loader.checkpoint import export_snapshot
    from cuteafd_b200.loader.plan import files_for_rank
    from cuteafd_b200.ref.model import init_weights
    spec = tiny_spec()
    export_snapshot(spec, init_weights(spec, 0), tmp_path, shard_layers=1)
    dep = default_deployment(4)
    per_rank = [files_for_rank(tmp_path, dep, r, spec.moe.n_experts) for r in range(4)]
    attn = [p for p in per_rank if p["role"] == "attention"]
    exp = [p for p in per_rank if p["role"] == "experts"]
    assert attn and exp and all(p["experts"] is None for p in attn)
    ranges = sorted(tuple(p["experts"]) for p in exp)
    assert ranges[0][0] == 0 and ranges[-1][1] == spec.moe.n_experts and all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    total = sum(t.nbytes for t in __import__("cuteafd_b200.loader.safetensors_io", fromlist=["catalog"]).catalog(tmp_path).values())
    assert attn[0]["bytes"] + sum(p["bytes"] for p in exp) == total            # every tensor has exactly one kind of reader
    assert cli.main(["plan", str(tmp_path), "--gpus", "4", "--rank", "3"]) == 0
    assert '"role": "experts"' in capsys.readouterr().out


def test_hybrid_linear_and_hyper_connection_snapshots_round_trip(tmp_path):
    """Snapshots of stacks with gated delta-rule layers (per-head and per-channel decay) and hyper-connections: every weight comes back
    (bf16-rounded projections, fp32 taps / decay parameters / mixing coefficients exactly) and the oracle gives the same logits."""
    import dataclasses
    from cuteafd_b200.ref.model import RefCache, RefModel
    base = tiny_spec()
    lin = dataclasses.replace(base.attn, n_heads=4, n_kv_heads=2, head_dim=128, linear_every=2, linear_k_heads=1, linear_v_heads=2)
    for name, spec in (("gdn", base.replace(n_layers=4, attn=lin)),
                       ("kda_hyper", base.replace(n_layers=2, hyper_streams=4, attn=dataclasses.replace(lin, linear_per_channel=True)))):
        masters = init_weights(spec, 3)
        from cuteafd_b200.config import spec_from_snapshot
        ck.export_snapshot(spec, masters, tmp_path / name)
        back = ck.read_masters(tmp_path / name, spec_from_snapshot(tmp_path / name))
        assert set(back["layers"][0]) == set(masters["layers"][0])
        b16 = lambda t: t.to(torch.bfloat16).float()
        for key in ("conv_w", "dt_bias", "a_log"):
            assert torch.equal(back["layers"][0][key], masters["layers"][0][key])
        assert torch.equal(back["layers"][0]["w_qkvz"], b16(masters["layers"][0]["w_qkvz"]))
        if spec.hyper_streams:
            assert torch.equal(back["hc_head_fn"], masters["hc_head_fn"]) and torch.equal(back["layers"][1]["hc_ffn_base"], masters["layers"][1]["hc_ffn_base"])
        p = torch.randint(0, spec.vocab, (9,), generator=torch.Generator().manual_seed(0))
        a, _ = RefModel(spec, masters).forward(p, 0, RefCache())
        c, _ = RefModel(spec_from_snapshot(tmp_path / name), back).forward(p, 0, RefCache())
        assert float((a[-1] - c[-1]).abs().max()) < 0.2          # the snapshot holds bf16-rounded projections
