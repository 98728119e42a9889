"""Loader / planner on CPU: safetensors round trip, sliced reads, format detection of every shipped layout, plan."""
import json

import numpy as np
import torch

from cuteafd_b200.config import deepseek_v3_spec, qwen3_235b_spec, from_hf_config
from cuteafd_b200.loader import formats, placement
from cuteafd_b200.loader.plan import plan
from cuteafd_b200.loader.safetensors_io import catalog, read_rows, read_tensor, write_file
from cuteafd_b200.loader.tokenizer import ByteTokenizer, StreamDecoder
from cuteafd_b200.ref import quant, exl3


def _snapshot(tmp_path):
    w = torch.randn(256, 512) * 0.02
    fp8, s128 = quant.fp8_block_quantize(w)
    mx_p, mx_s = quant.mxfp4_quantize(w)
    nv_p, nv_s, nv_g = quant.nvfp4_quantize(w)
    tr = torch.from_numpy(exl3.encode_tiles_greedy(np.random.default_rng(0).standard_normal((128, 128)).astype(np.float32), 3).view(np.int16))
    tensors = {
        "model.norm.weight": torch.ones(512, dtype=torch.bfloat16),
        "l0.q_proj.weight": w.to(torch.bfloat16),
        "l0.kv.weight": fp8, "l0.kv.weight_scale_inv": s128,
        "l0.e0.down.weight": mx_p, "l0.e0.down.weight_scale": mx_s,
        "l0.e1.up.weight": nv_p, "l0.e1.up.weight_scale": nv_s, "l0.e1.up.weight_scale_2": nv_g.reshape(1), "l0.e1.up.input_scale": torch.ones(1),
        "l0.e2.gate.trellis": tr, "l0.e2.gate.suh": torch.ones(128, dtype=torch.float16), "l0.e2.gate.svh": torch.ones(128, dtype=torch.float16),
        "l0.bad.weight": mx_p,                                   # packed 4-bit without scales
    }
    write_file(tmp_path / "model-00001.safetensors", tensors,
               dtypes={"l0.kv.weight": "F8_E4M3", "l0.e1.up.weight_scale": "F8_E4M3", "l0.e0.down.weight_scale": "F8_E8M0"})
    cfg = {"architectures": ["Qwen3MoeForCausalLM"], "hidden_size": 512, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128,
           "num_hidden_layers": 2, "vocab_size": 1000, "num_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 256,
           "quantization_config": {"quant_method": "modelopt", "quant_algo": "NVFP4"}}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    return tensors, w


def test_safetensors_roundtrip_and_row_windows(tmp_path):
    tensors, w = _snapshot(tmp_path)
    cat = catalog(tmp_path)
    assert set(cat) == set(tensors)
    got = read_tensor(cat["l0.q_proj.weight"])
    assert torch.equal(got, tensors["l0.q_proj.weight"])
    rows = read_rows(cat["l0.q_proj.weight"], 100, 164)           # a TP shard / one expert's window
    assert torch.equal(rows, tensors["l0.q_proj.weight"][100:164])
    assert cat["l0.kv.weight"].dtype == "F8_E4M3"


def test_format_detection_covers_every_shipped_layout(tmp_path):
    _snapshot(tmp_path)
    ops, bad = formats.detect_all(catalog(tmp_path))
    assert ops["l0.q_proj"].format == "bf16"
    assert ops["l0.kv"].format == "fp8_block128" and ops["l0.kv"].scale_encoding == "f32"
    assert ops["l0.e0.down"].format == "mxfp4" and ops["l0.e0.down"].logical == (256, 512)
    nv = ops["l0.e1.up"]
    assert nv.format == "nvfp4" and nv.global_scale and nv.input_scale and nv.block == (1, 16)
    ex = ops["l0.e2.gate"]
    assert ex.format == "exl3_k3" and ex.logical == (128, 128)
    assert [b.stem for b in bad] == ["l0.bad"] and "scales" in bad[0].reason


def test_plan_reports_results_not_exceptions(tmp_path):
    _snapshot(tmp_path)
    rep = plan(str(tmp_path), layout=True, files=True, world=8)
    assert rep.family == "qwen3_moe" and rep.format_counts["nvfp4"] == 1
    assert not rep.supported and any("l0.bad" in p for p in rep.problems)
    assert any("EXL3" in h for h in rep.hints) and rep.files == ["model-00001.safetensors"]
    assert rep.layout is not None and "pool tokens" in rep.text()
    assert not plan("no-such-model").supported
    ok = plan("qwen3-235b", layout=True)
    assert ok.supported and ok.layout.fits


def test_placement_of_the_benchmark_shapes():
    lay = placement.solve(deepseek_v3_spec(), world=8)
    assert lay.fits and [r.role for r in lay.ranks] == ["attention"] * 2 + ["experts"] * 6
    assert 50 < lay.ranks[2].weight_bytes / placement.GIB < 62          # 256 MXFP4 experts x 58 layers over EP6
    assert lay.pool_tokens > 1_000_000                                  # MLA latent cache is tiny
    one = placement.solve(deepseek_v3_spec(), world=1)
    assert not one.fits and one.ranks[0].shortfall > 0
    q = placement.solve(qwen3_235b_spec(), world=1)
    assert q.fits and q.pool_tokens > 100_000
    assert not placement.solve(qwen3_235b_spec(), world=8, pool_tokens=10**9).fits


def test_hf_config_reader_and_stream_decoder():
    spec = from_hf_config({"architectures": ["DeepseekV3ForCausalLM"], "hidden_size": 7168, "num_attention_heads": 128, "kv_lora_rank": 512,
                           "q_lora_rank": 1536, "qk_nope_head_dim": 128, "qk_rope_head_dim": 64, "v_head_dim": 128, "num_hidden_layers": 61,
                           "vocab_size": 129280, "n_routed_experts": 256, "num_experts_per_tok": 8, "moe_intermediate_size": 2048,
                           "n_shared_experts": 1, "scoring_func": "sigmoid", "topk_method": "noaux_tc", "n_group": 8, "topk_group": 4,
                           "first_k_dense_replace": 3, "intermediate_size": 18432, "routed_scaling_factor": 2.5, "num_nextn_predict_layers": 1,
                           "quantization_config": {"quant_method": "fp8", "weight_block_size": [128, 128]}})
    assert spec.attn.kind == "mla" and spec.moe.use_bias and spec.quant.dense == "fp8_block128" and spec.mtp_layers == 1
    tok = ByteTokenizer()
    dec = StreamDecoder(tok)
    ids = tok.encode("héllo")
    pieces = [dec.push([i]) for i in ids]
    assert "".join(pieces) == "héllo" and "�" not in "".join(pieces)
