"""Checkpoint -> GPU engine: weights loaded from an HF-layout snapshot in their stored formats generate the oracle's tokens."""
import dataclasses

import pytest
import torch

from cuteafd_b200.config import QuantSpec, tiny_spec
from cuteafd_b200.loader import checkpoint as ck
from cuteafd_b200.ref.model import RefModel, init_weights

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("dense,experts", [("bf16", "bf16"), ("bf16", "nvfp4"), ("bf16", "mxfp4"), ("fp8_block128", "mxfp4")])
def test_snapshot_loads_into_the_engine(tmp_path, dense, experts):
    from cuteafd_b200.engine.engine import Engine
    from cuteafd_b200.engine.generate import generate
    base = tiny_spec()
    spec = base.replace(attn=dataclasses.replace(base.attn, n_kv_heads=4), quant=QuantSpec(experts=experts, dense=dense))
    masters = init_weights(spec, 6)
    snap = ck.export_snapshot(spec, masters, tmp_path / "snap", dense=dense, experts=experts, shard_layers=1)
    dw = ck.load_device_weights(snap, spec, DEV)
    # the payloads are the stored ones: dequantising the device weights gives what the host reader decodes
    host = ck.read_masters(snap, spec)
    back = dw.dequantized_masters()
    for li in range(spec.n_layers):
        for k in ("wq", "wo", "w_down", "router"):
            if k in host["layers"][li]:
                assert torch.allclose(back["layers"][li][k], host["layers"][li][k], rtol=0, atol=1e-6), (li, k)
    eng = Engine(dw, n_pages=16, max_seqs=4, max_pages_per_seq=4)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, spec.vocab, (n,), generator=g).tolist() for n in (6, 15)]
    out = generate(eng, prompts, 6, use_graph=False)
    if dense == "bf16" and experts == "bf16":
        ref = RefModel(spec, host)
        for p, o in zip(prompts, out):
            assert o == ref.generate_greedy(torch.tensor(p), 6)[0]
    else:
        assert all(len(o) == 6 for o in out)      # quantised activations: run to completion (numerics are covered per kernel)
    eng.check_status()
