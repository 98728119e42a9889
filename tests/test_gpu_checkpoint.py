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


def test_nvfp4_activation_scale_comes_from_the_checkpoint(tmp_path):
    """ModelOpt NVFP4 snapshots carry a calibrated `input_scale` per linear.  With it, activations far above the range a
    fixed 1/64 scale can express (6 * 448 / 64 = 42) survive quantisation; the expert gate/up pair shares one scale."""
    from cuteafd_b200 import ops
    from cuteafd_b200.ops import ActBuffer
    from cuteafd_b200.ref import quant
    spec = tiny_spec().replace(quant=QuantSpec(experts="nvfp4", dense="nvfp4"))
    masters = init_weights(spec, 9)
    amax = 300.0
    snap = ck.export_snapshot(spec, masters, tmp_path / "snap", dense="nvfp4", experts="nvfp4", input_amax=amax)
    catalog_ops = ck._ops_of(snap)
    stems = ck.layer_stems(spec, 0)
    wo = ck._tc_from_operands([catalog_ops[stems["wo"]]], DEV, 1.0 / 64)
    want_gs = amax / (448.0 * 6.0)
    assert abs(1.0 / float(wo.inv_act_gs[0]) - want_gs) < 1e-6
    gs_w = float(ck.read_tensor(catalog_ops[stems["wo"]].members["weight_scale_2"]))
    assert abs(float(wo.alpha[0]) - gs_w * want_gs) < 1e-9
    # activations with outliers up to ~amax
    K, T = wo.K, 8
    g = torch.Generator().manual_seed(4)
    x = torch.randn(T, K, generator=g) * 20.0
    x[:, ::17] *= 10.0
    x = x.clamp(-amax, amax)
    xb = x.to(torch.bfloat16).to(DEV).contiguous()
    xq = ActBuffer.alloc(wo.kind, T, K, 16, DEV)
    ops.quant_fp4_rows(xb, xq, inv_gs=wo.inv_act_gs)
    y = torch.zeros(T, wo.N, dtype=torch.float32, device=DEV)
    ops.tc_linear(wo, xq, y)
    torch.cuda.synchronize()
    xd = quant.nvfp4_dequantize(xq.data.cpu(), xq.sf.cpu()[:, :K // 16], want_gs)
    wd = wo.dequantize()[0]
    ref_q = xd @ wd.T
    assert (y.cpu() - ref_q).norm() / ref_q.norm() < 2e-3
    ref_full = xb.float().cpu() @ wd.T                                   # unquantised activations: FP4 noise only, no clipping
    assert (y.cpu() - ref_full).norm() / ref_full.norm() < 0.15
    # the same input through a fixed 1/64 scale saturates its blocks and is far off
    fixed = torch.tensor([64.0], device=DEV)
    ops.quant_fp4_rows(xb, xq, inv_gs=fixed)
    xc = quant.nvfp4_dequantize(xq.data.cpu(), xq.sf.cpu()[:, :K // 16], 1.0 / 64)
    assert (xc - xb.float().cpu()).norm() / xb.float().cpu().norm() > 0.3
    # expert gate and up multiply the same quantised rows: one shared scale
    spec2 = spec.replace(quant=QuantSpec(experts="nvfp4", dense="bf16"))
    snap2 = ck.export_snapshot(spec2, masters, tmp_path / "snap2", dense="bf16", experts="nvfp4", input_amax=amax)
    lw = ck.load_device_weights(snap2, spec2, DEV).layers[0]
    assert float(lw.w_gate.inv_act_gs[0]) == float(lw.w_up.inv_act_gs[0]) == pytest.approx(1.0 / want_gs)
