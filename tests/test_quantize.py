"""Resumable re-quantisation pipeline: run store, recovery identity, continuation after a crash, publication (CPU only)."""
import json

import pytest
import torch

from cuteafd_b200.config import tiny_spec
from cuteafd_b200.loader.checkpoint import export_snapshot, read_masters
from cuteafd_b200.loader.quantize import RUN_FILE, Interrupted, quantize_snapshot
from cuteafd_b200.ref.model import init_weights


def _digest(d):
    return {f.name: f.read_bytes() for f in sorted(d.glob("unit-*.safetensors"))}


def test_interrupted_run_continues_and_matches_a_one_shot_run(tmp_path):
    spec = tiny_spec()
    masters = init_weights(spec, 0)
    export_snapshot(spec, masters, tmp_path / "src")
    with pytest.raises(Interrupted):
        quantize_snapshot(tmp_path / "src", tmp_path / "a", spec, dense="nvfp4", experts="mxfp4", stop_after=2)
    run = json.loads((tmp_path / "a" / RUN_FILE).read_text())
    assert run["state"] == "running" and len(run["done"]) == 2 and not (tmp_path / "a" / "model.safetensors.index.json").exists()
    (tmp_path / "a" / ".unit-layer-0001.partial").write_bytes(b"torn write")              # what a crash mid-write leaves behind
    r = quantize_snapshot(tmp_path / "src", tmp_path / "a", spec, dense="nvfp4", experts="mxfp4")
    assert r["skipped"] == ["head", "layer-0000"] and r["written"] == ["layer-0001"] and r["published"]
    assert not list((tmp_path / "a").glob(".unit-*.partial"))
    quantize_snapshot(tmp_path / "src", tmp_path / "b", spec, dense="nvfp4", experts="mxfp4")
    assert _digest(tmp_path / "a") == _digest(tmp_path / "b")                             # continuation == one shot, byte for byte
    index = json.loads((tmp_path / "a" / "model.safetensors.index.json").read_text())
    assert index["weight_map"]["model.embed_tokens.weight"] == "unit-head.safetensors"
    # the result decodes back close to the source (FP4 error) and a third run has nothing left to do
    w = read_masters(tmp_path / "a", spec)
    a, b = masters["layers"][1]["wo"], w["layers"][1]["wo"]
    assert float((a - b).norm() / a.norm()) < 0.15
    again = quantize_snapshot(tmp_path / "src", tmp_path / "a", spec, dense="nvfp4", experts="mxfp4")
    assert again["written"] == [] and len(again["skipped"]) == 3


def test_run_store_of_another_run_is_refused_and_a_lost_shard_is_redone(tmp_path):
    spec = tiny_spec()
    export_snapshot(spec, init_weights(spec, 1), tmp_path / "src")
    quantize_snapshot(tmp_path / "src", tmp_path / "q", spec, dense="bf16", experts="mxfp4")
    with pytest.raises(ValueError, match="another run"):
        quantize_snapshot(tmp_path / "src", tmp_path / "q", spec, dense="nvfp4", experts="mxfp4")
    (tmp_path / "q" / "unit-layer-0000.safetensors").unlink()
    r = quantize_snapshot(tmp_path / "src", tmp_path / "q", spec, dense="bf16", experts="mxfp4")
    assert r["written"] == ["layer-0000"]
    r = quantize_snapshot(tmp_path / "src", tmp_path / "q", spec, dense="nvfp4", experts="nvfp4", restart=True)
    assert len(r["written"]) == 3 and json.loads((tmp_path / "q" / RUN_FILE).read_text())["dense"] == "nvfp4"


def test_quantize_and_plan_commands_work_on_a_synthetic_snapshot(tmp_path, capsys):
    """Synthetic snapshots carry their spec, so the commands that take a snapshot directory work on them."""
    from cuteafd_b200 import cli
    from cuteafd_b200.config import spec_from_snapshot
    spec = tiny_spec()
    export_snapshot(spec, init_weights(spec, 2), tmp_path / "src")
    assert spec_from_snapshot(tmp_path / "src") == spec
    assert cli.main(["quantize", str(tmp_path / "src"), str(tmp_path / "q"), "--dense", "bf16", "--experts", "mxfp4"]) == 0
    assert '"published": true' in capsys.readouterr().out
    q = spec_from_snapshot(tmp_path / "q")
    assert q.quant.experts == "mxfp4" and q.quant.dense == "bf16" and q.replace(quant=spec.quant) == spec
    assert cli.main(["plan", str(tmp_path / "q"), "--gpus", "1", "--layout"]) == 0
    out = capsys.readouterr().out
    assert "mxfp4" in out and "supported: True" in out
