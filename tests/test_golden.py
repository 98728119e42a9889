"""Golden windows: sealing from the fp32 oracle, the file format, and the fidelity check's verdicts (CPU: the 'engine' is the
oracle itself, exact or perturbed).  The GPU engine against golden windows is covered in tests/test_gpu_model.py."""
import json

import pytest
import torch

from cuteafd_b200.bench.golden import check_logits, make_windows, read_golden, spec_digest, write_golden
from cuteafd_b200.config import tiny_spec
from cuteafd_b200.ref.model import RefCache, RefModel, init_weights
from cuteafd_b200.serving.chat_templates import template_round_trip


def test_golden_windows_seal_and_check(tmp_path):
    spec = tiny_spec()
    masters = init_weights(spec, 0)
    path = str(tmp_path / "tiny.golden.json")
    gold = write_golden(path, spec, masters, n=3, length=24, tail=8, topk=4)
    assert read_golden(path) == json.loads(json.dumps(gold)) and gold["digest"] == spec_digest(spec) and len(gold["windows"]) == 3
    assert make_windows(spec.vocab, 3, 24) == [w["tokens"] for w in gold["windows"]]            # windows are reproducible from the seed
    ref = RefModel(spec, masters)
    exact = lambda toks: ref.forward(torch.tensor(toks), 0, RefCache())[0]
    rep = check_logits(exact, gold, spec=spec)
    assert rep["pass"] and all(r["top1_agreement"] == 1.0 and r["rel_l2_topk"] < 1e-5 for r in rep["windows"])
    # a different model (another seed) must fail the gate
    other = RefModel(spec, init_weights(spec, 1))
    rep2 = check_logits(lambda toks: other.forward(torch.tensor(toks), 0, RefCache())[0], gold, spec=spec)
    assert not rep2["pass"]
    # small noise passes (a quantised engine), the digest guards against checking the wrong model
    g = torch.Generator().manual_seed(0)
    noisy = lambda toks: exact(toks) + 1e-3 * torch.randn(len(toks), spec.vocab, generator=g)
    assert check_logits(noisy, gold, spec=spec)["pass"]
    with pytest.raises(ValueError):
        check_logits(exact, gold, spec=spec.replace(n_layers=spec.n_layers + 1))
    with pytest.raises(ValueError):
        (tmp_path / "bad.json").write_text("{}")
        read_golden(str(tmp_path / "bad.json"))


def test_template_round_trip_gate():
    for model in ("qwen3-235b", "qwen3-coder", "deepseek-v3", "glm-5", "tiny", None):
        assert template_round_trip(model), model
