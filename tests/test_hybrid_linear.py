"""Hybrid stacks with gated delta-rule layers: layer pattern, oracle consistency, recurrent-state slots of the serving runner."""
import dataclasses
from types import SimpleNamespace

import pytest
import torch

from cuteafd_b200.config import spec_by_name, tiny_spec
from cuteafd_b200.ref.model import RefCache, RefModel, init_weights
from cuteafd_b200.serving.runner import EngineRunner


def _spec(per_channel=False):
    base = tiny_spec()
    return base.replace(n_layers=4, attn=dataclasses.replace(base.attn, n_heads=4, n_kv_heads=2, head_dim=128, linear_every=2, linear_k_heads=1,
                                                             linear_v_heads=2, linear_per_channel=per_channel))


def test_layer_pattern_and_presets():
    spec = _spec()
    assert [spec.layer_is_linear(i) for i in range(4)] == [True, False, True, False]
    assert not any(tiny_spec().layer_is_linear(i) for i in range(2))
    g = spec_by_name("hybrid-gdn", n_layers=8)
    assert [g.layer_is_linear(i) for i in range(8)] == [True, True, True, False] * 2 and not g.attn.linear_per_channel
    assert spec_by_name("hybrid-kda").attn.linear_per_channel


@pytest.mark.parametrize("per_channel", [False, True])
def test_oracle_chunked_prefill_equals_whole_prompt(per_channel):
    spec = _spec(per_channel)
    masters = init_weights(spec, 5)
    lw = masters["layers"][0]
    assert "w_qkvz" in lw and "wq" not in lw and "wq" in masters["layers"][1]
    assert lw["w_ba"].shape[0] == (2 + 256 if per_channel else 4)
    ref = RefModel(spec, masters)
    p = torch.randint(0, spec.vocab, (24,), generator=torch.Generator().manual_seed(1))
    whole, _ = ref.forward(p, 0, RefCache())
    c = RefCache()
    ref.forward(p[:7], 0, c)
    ref.forward(p[7:15], 7, c)
    tail, _ = ref.forward(p[15:], 15, c)
    assert float((tail[-1] - whole[-1]).abs().max()) < 1e-3
    with pytest.raises(Exception):
        c.truncate(10)           # a recurrent state cannot step back


def test_runner_assigns_and_recycles_state_slots():
    resets = []
    eng = SimpleNamespace(lin_layers=[0], max_seqs=2, reset_state_slots=lambda s: resets.append(list(s)))
    r = EngineRunner(eng, max_rows=64)
    a, b, c = object(), object(), object()
    row = lambda st, pos, n: SimpleNamespace(state=st, start_pos=pos, tokens=[1] * n)
    s = r._slots_of([row(a, 0, 5), row(b, 0, 3)])
    assert sorted(s) == [0, 1] and sorted(resets[-1]) == [0, 1]
    assert r._slots_of([row(a, 5, 1), row(b, 3, 1)]) == s and resets[-1] == []
    with pytest.raises(RuntimeError, match="step back"):
        r._slots_of([row(a, 4, 1)])
    with pytest.raises(RuntimeError, match="slots"):
        r._slots_of([row(c, 0, 2)])
    with pytest.raises(RuntimeError, match="cached pages"):
        r._slots_of([row(object(), 8, 2)])
    r.forget(a)
    assert r._slots_of([row(c, 0, 2)]) == [s[0]] and resets[-1] == [s[0]]
    # a preempted sequence restarts from position 0 in its own slot
    assert r._slots_of([row(b, 0, 4)]) == [s[1]] and resets[-1] == [s[1]]


def test_hf_configs_of_hybrid_and_sparse_families_map_to_specs():
    from cuteafd_b200.config import from_hf_config
    s = from_hf_config({"architectures": ["Qwen3NextForCausalLM"], "hidden_size": 2048, "num_attention_heads": 16, "num_key_value_heads": 2, "head_dim": 128,
                        "num_hidden_layers": 48, "vocab_size": 151936, "full_attention_interval": 4, "linear_num_key_heads": 16,
                        "linear_num_value_heads": 32, "linear_key_head_dim": 128, "linear_value_head_dim": 128, "linear_conv_kernel_dim": 4,
                        "num_experts": 512, "num_experts_per_tok": 10, "moe_intermediate_size": 512,
                        "layer_types": ["linear_attention"] * 3 + ["full_attention"]})
    assert s.family == "hybrid_linear" and (s.attn.linear_every, s.attn.linear_k_heads, s.attn.linear_v_heads) == (4, 16, 32)
    assert [s.layer_is_linear(i) for i in range(8)] == [True, True, True, False] * 2 and s.attn.full_every == 0
    with pytest.raises(ValueError):
        from_hf_config({"architectures": ["Qwen3NextForCausalLM"], "hidden_size": 2048, "num_attention_heads": 16, "num_hidden_layers": 4, "vocab_size": 1000,
                        "full_attention_interval": 4, "linear_num_key_heads": 16, "linear_num_value_heads": 32, "linear_key_head_dim": 256})
    d = from_hf_config({"architectures": ["DeepseekV32ForCausalLM"], "hidden_size": 7168, "num_attention_heads": 128, "kv_lora_rank": 512, "q_lora_rank": 1536,
                        "qk_nope_head_dim": 128, "qk_rope_head_dim": 64, "v_head_dim": 128, "num_hidden_layers": 61, "vocab_size": 129280,
                        "index_topk": 2048, "index_n_heads": 64, "index_head_dim": 128, "n_routed_experts": 256, "num_experts_per_tok": 8,
                        "moe_intermediate_size": 2048})
    assert (d.attn.index_topk, d.attn.index_heads, d.attn.index_dim) == (2048, 64, 128)
    assert spec_by_name("deepseek-v32", n_layers=4).attn.index_topk == 2048
