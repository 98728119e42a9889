"""Model geometry and deployment descriptions.

A `ModelSpec` is the single description every layer of the framework consumes: the
CPU oracle, the weight initialiser, the planner/placement solver, the engine and the
benchmarks.  The reference derives the same facts from a snapshot's `config.json`
(reference: rust/crates/cuteafd-loader/src/plan/family.rs, cuteafd-core/src/constants.rs);
here they are plain dataclasses plus a `from_hf_config` reader.
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional


@dataclass(frozen=True)
class AttentionSpec:
    kind: str = "gqa"              # "gqa" | "mla"
    n_heads: int = 8
    n_kv_heads: int = 2
    head_dim: int = 32
    rope_theta: float = 10000.0
    rope_interleaved: bool = True   # pair (2i, 2i+1) rotation; False = half-split (HF llama style)
    qk_norm: bool = False           # per-head RMSNorm on q and k (Qwen3)
    # MLA (DeepSeek-V3 style); ignored for gqa
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    window: int = 0                 # sliding window (0 = full)
    sink: bool = False              # learned attention sink logit per head
    # Hybrid stacks (MiMo-V2 style: full causal layers interleaved with sliding-window layers that carry the sinks): with
    # full_every = n > 0, layers i with i % n == 0 are full attention (no window, no sink, `rope_theta`), the others use `window`,
    # the sink and `swa_rope_theta` (0 = the same theta).  0 = every layer as configured above.
    full_every: int = 0
    swa_rope_theta: float = 0.0
    # Sparse attention with a learned indexer (DSA of the DeepSeek-V3.2 / GLM-5 lines; MLA only): with index_topk = k > 0 every
    # query token scores the visible cached positions with `index_heads` small heads of `index_dim` dimensions
    # (score = sum_h w_h * relu(q_h . k)), and attends only to its k best positions once it can see more than k.
    index_topk: int = 0
    index_heads: int = 32
    index_dim: int = 128
    # Hybrid stacks with linear-attention layers (the Qwen 3.8 / GLM 5.3 Flash lines; GQA models only): with linear_every = n > 0,
    # layer i is a full-attention layer when (i + 1) % n == 0 and a gated delta-rule layer otherwise (n = 4: three linear layers,
    # then one full).  Linear layers have `linear_k_heads` query / key heads and `linear_v_heads` value heads of 128 dimensions,
    # a width-4 causal convolution in front of q / k / v, and a per-sequence recurrent state instead of KV pages.
    # `linear_per_channel`: one decay per key channel (KDA) instead of one per head (GDN).
    linear_every: int = 0
    linear_k_heads: int = 2
    linear_v_heads: int = 4
    linear_per_channel: bool = False

    @property
    def q_dim(self) -> int:
        if self.kind == "mla":
            return self.n_heads * (self.qk_nope_head_dim + self.qk_rope_head_dim)
        return self.n_heads * self.head_dim

    @property
    def kv_token_elems(self) -> int:
        """Cached elements per token per layer."""
        if self.kind == "mla":
            return self.kv_lora_rank + self.qk_rope_head_dim
        return 2 * self.n_kv_heads * self.head_dim


@dataclass(frozen=True)
class MoESpec:
    n_experts: int = 16
    top_k: int = 4
    intermediate: int = 128
    n_shared: int = 1
    shared_intermediate: int = 0    # 0 -> n_shared * intermediate
    scoring: str = "sigmoid"        # sigmoid | softmax | sqrtsoftplus | hash
    normalize: bool = True
    route_scale: float = 1.0
    use_bias: bool = False          # noaux_tc selection bias (affects choice only)
    n_group: int = 1
    topk_group: int = 1
    first_dense: int = 0            # leading dense layers
    dense_intermediate: int = 0
    swiglu_limit: float = 0.0       # clamp on gate/up (0 = off)

    @property
    def shared_inter(self) -> int:
        return self.shared_intermediate or self.n_shared * self.intermediate


@dataclass(frozen=True)
class QuantSpec:
    """Weight formats as shipped in the checkpoint (no repacking on disk)."""
    experts: str = "bf16"           # bf16 | fp8_block128 | mxfp4 | nvfp4 | exl3
    dense: str = "bf16"             # bf16 | fp8_block128 | fp8_block32 | nvfp4
    kv: str = "bf16"                # bf16 | fp8
    exl3_bits: int = 4


@dataclass(frozen=True)
class ModelSpec:
    name: str = "tiny"
    family: str = "tiny"
    vocab: int = 1024
    hidden: int = 256
    n_layers: int = 2
    rms_eps: float = 1e-5
    attn: AttentionSpec = field(default_factory=AttentionSpec)
    moe: MoESpec = field(default_factory=MoESpec)
    quant: QuantSpec = field(default_factory=QuantSpec)
    mtp_layers: int = 0             # native next-n (MTP) draft layers
    # Hyper-connections (the V4 line): 0 = one residual stream; 4 = four streams mixed at every sub-layer boundary by per-token
    # coefficients (collapse weights, spread weights and a Sinkhorn-normalised 4 x 4 stream mix from 24 projections of the row)
    hyper_streams: int = 0
    hyper_sinkhorn_iters: int = 20
    # N-gram memory (the V4.1 line's "engram"): decoder layers whose input takes a gated projection of hashed table rows addressed by the
    # 2- to 4-grams ending at the token; the tables have engram_prime_floor-sized heads (24 consecutive primes above it per layer)
    engram_layers: tuple = ()
    engram_row_dim: int = 256
    engram_prime_floor: int = 500
    engram_vocab: int = 0           # compressed vocabulary of the addressing (0: the model's vocabulary, identity map)
    init_std: float = 0.02
    tie_embeddings: bool = False
    max_context: int = 1 << 20

    def replace(self, **kw) -> "ModelSpec":
        return dataclasses.replace(self, **kw)

    def engram_spec(self):
        """Addressing / shape of the n-gram memory, or None for models without one."""
        if not self.engram_layers:
            return None
        from .ref.engram import EngramSpec
        return EngramSpec(layers=tuple(self.engram_layers), vocab=self.engram_vocab or self.vocab, pad_id=0, row_dim=self.engram_row_dim,
                          prime_floor=self.engram_prime_floor, streams=1, hidden=self.hidden)

    # ---- per-layer attention program ---------------------------------------
    def layer_is_full(self, layer: int) -> bool:
        """Full causal attention (True) or the sliding-window variant (False); MTP draft layers (>= n_layers) are full."""
        a = self.attn
        if a.full_every <= 0:
            return a.window == 0
        return layer >= self.n_layers or layer % a.full_every == 0

    def layer_is_linear(self, layer: int) -> bool:
        """A gated delta-rule (linear attention) layer; MTP draft layers (>= n_layers) are full-attention layers."""
        n = self.attn.linear_every
        return n > 0 and layer < self.n_layers and (layer + 1) % n != 0

    def layer_window(self, layer: int) -> int:
        a = self.attn
        return a.window if (a.full_every <= 0 or not self.layer_is_full(layer)) else 0

    def layer_has_sink(self, layer: int) -> bool:
        a = self.attn
        return a.sink and (a.full_every <= 0 or not self.layer_is_full(layer))

    def layer_rope_theta(self, layer: int) -> float:
        a = self.attn
        if a.full_every > 0 and a.swa_rope_theta and not self.layer_is_full(layer):
            return a.swa_rope_theta
        return a.rope_theta

    # ---- derived sizes -------------------------------------------------
    def is_moe_layer(self, layer: int) -> bool:
        return layer >= self.moe.first_dense

    def expert_params(self) -> int:
        return 3 * self.hidden * self.moe.intermediate

    def attn_params(self) -> int:
        a, h = self.attn, self.hidden
        if a.kind == "mla":
            qk = a.qk_nope_head_dim + a.qk_rope_head_dim
            q = h * a.q_lora_rank + a.q_lora_rank * a.n_heads * qk if a.q_lora_rank else h * a.n_heads * qk
            kv = h * (a.kv_lora_rank + a.qk_rope_head_dim) + a.kv_lora_rank * a.n_heads * (a.qk_nope_head_dim + a.v_head_dim)
            return q + kv + a.n_heads * a.v_head_dim * h
        return h * (a.n_heads + 2 * a.n_kv_heads) * a.head_dim + a.n_heads * a.head_dim * h

    def bits(self, fmt: str) -> float:
        return {"bf16": 16.0, "fp8_block128": 8.0 + 32.0 / (128 * 128), "fp8_block32": 8.0 + 8.0 / (32 * 32),
                "mxfp4": 4.25, "nvfp4": 4.5, "exl3": float(self.quant.exl3_bits)}[fmt]

    def weight_bytes(self) -> dict:
        """Bytes per category for the whole model (planner input)."""
        moe_layers = self.n_layers - self.moe.first_dense
        eb = self.bits(self.quant.experts) / 8
        db = self.bits(self.quant.dense) / 8
        routed = moe_layers * self.moe.n_experts * self.expert_params() * eb
        shared = moe_layers * 3 * self.hidden * self.moe.shared_inter * db
        dense_ffn = self.moe.first_dense * 3 * self.hidden * self.moe.dense_intermediate * db
        attn = self.n_layers * self.attn_params() * db
        router = moe_layers * self.moe.n_experts * self.hidden * 2
        embed = self.vocab * self.hidden * 2 * (1 if self.tie_embeddings else 2)
        return {"routed_experts": routed, "shared_experts": shared, "dense_ffn": dense_ffn,
                "attention": attn, "router": router, "embed_head": embed}

    def kv_bytes_per_token(self) -> float:
        per = 1.0 if self.quant.kv == "fp8" else 2.0
        return self.n_layers * self.attn.kv_token_elems * per


# ---------------------------------------------------------------------------
# Named configurations
# ---------------------------------------------------------------------------

def tiny_spec() -> ModelSpec:
    """Tiny synthetic MoE decoder (CPU oracle config): vocab 1024, hidden 256, 2 layers,
    GQA 8q/2kv/32, 16 experts sigmoid-normalised top-4 + 1 shared, SwiGLU I=128."""
    return ModelSpec()


def deepseek_v3_spec(n_layers: int = 61) -> ModelSpec:
    """DeepSeek-V3-shape: 61 layers, hidden 7168, MLA 128 heads (q_lora 1536, kv_lora 512,
    rope 64), 256 experts top-8 + 1 shared, I=2048, vocab 129280; FP8 128x128 dense, MXFP4 experts."""
    return ModelSpec(
        name="deepseek-v3-shape", family="deepseek_v3", vocab=129280, hidden=7168, n_layers=n_layers,
        rms_eps=1e-6,
        attn=AttentionSpec(kind="mla", n_heads=128, n_kv_heads=128, head_dim=192, rope_theta=10000.0,
                           q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128,
                           qk_rope_head_dim=64, v_head_dim=128),
        moe=MoESpec(n_experts=256, top_k=8, intermediate=2048, n_shared=1, scoring="sigmoid",
                    normalize=True, route_scale=2.5, use_bias=True, n_group=8, topk_group=4,
                    first_dense=min(3, n_layers), dense_intermediate=18432),
        quant=QuantSpec(experts="mxfp4", dense="fp8_block128", kv="bf16"),
        mtp_layers=1)


def qwen3_235b_spec(n_layers: int = 94) -> ModelSpec:
    """Qwen3-235B-A22B-shape with NVFP4 weights: 94 layers, hidden 4096, GQA 64q/4kv/128,
    128 experts top-8, I=1536, vocab 151936."""
    return ModelSpec(
        name="qwen3-235b-a22b-shape", family="qwen3_moe", vocab=151936, hidden=4096, n_layers=n_layers,
        rms_eps=1e-6,
        attn=AttentionSpec(kind="gqa", n_heads=64, n_kv_heads=4, head_dim=128, rope_theta=1e6,
                           rope_interleaved=False, qk_norm=True),
        moe=MoESpec(n_experts=128, top_k=8, intermediate=1536, n_shared=0, scoring="softmax",
                    normalize=True),
        quant=QuantSpec(experts="nvfp4", dense="nvfp4", kv="bf16"))


def ep_microbench_spec() -> ModelSpec:
    """EP dispatch -> grouped GEMM -> combine microbench layer: hidden 7168, 256 experts, top-8,
    I=2048, MXFP4 weights."""
    return ModelSpec(name="ep-microbench", family="microbench", hidden=7168, n_layers=1, vocab=1024,
                     moe=MoESpec(n_experts=256, top_k=8, intermediate=2048, n_shared=0,
                                 scoring="softmax", normalize=True),
                     quant=QuantSpec(experts="mxfp4"))


def deepseek_v32_spec(n_layers: int = 61) -> ModelSpec:
    """DeepSeek-V3.2-shape: the V3 shape with the sparse-attention indexer (64 index heads of 128, 2048 positions kept per query)."""
    base = deepseek_v3_spec(n_layers)
    return base.replace(name="deepseek-v32-shape", attn=dataclasses.replace(base.attn, index_topk=2048, index_heads=64, index_dim=128))


def hybrid_gdn_spec(n_layers: int = 48, per_channel: bool = False) -> ModelSpec:
    """Hybrid linear-attention MoE shape (the Qwen-Next line): three gated delta-rule layers (16 q/k heads, 32 value heads of 128)
    then one full GQA layer (16q/2kv/128), hidden 2048, 128 experts top-8 I=768 + 1 shared, vocab 151936, bf16 dense projections and
    NVFP4 experts.  `per_channel`: one decay per key channel (the KDA variant of the GLM Flash line) instead of one per head."""
    return ModelSpec(
        name="hybrid-kda-shape" if per_channel else "hybrid-gdn-shape", family="hybrid_linear", vocab=151936, hidden=2048, n_layers=n_layers, rms_eps=1e-6,
        attn=AttentionSpec(kind="gqa", n_heads=16, n_kv_heads=2, head_dim=128, rope_theta=1e6, rope_interleaved=False, qk_norm=True,
                           linear_every=4, linear_k_heads=16, linear_v_heads=32, linear_per_channel=per_channel),
        moe=MoESpec(n_experts=128, top_k=8, intermediate=768, n_shared=1, scoring="softmax", normalize=True),
        quant=QuantSpec(experts="nvfp4", dense="bf16", kv="bf16"))


NAMED_SPECS = {
    "tiny": tiny_spec,
    "hybrid-gdn": hybrid_gdn_spec,
    "hybrid-kda": lambda **kw: hybrid_gdn_spec(per_channel=True, **kw),
    "deepseek-v3": deepseek_v3_spec,
    "deepseek-v32": deepseek_v32_spec,
    "qwen3-235b": qwen3_235b_spec,
    "ep-microbench": ep_microbench_spec,
}


def spec_by_name(name: str, **kw) -> ModelSpec:
    if name not in NAMED_SPECS:
        raise KeyError(f"unknown model spec {name!r}; known: {sorted(NAMED_SPECS)}")
    return NAMED_SPECS[name](**kw)


# ---------------------------------------------------------------------------
# HF config.json -> ModelSpec (family detection, reference: commands/family.rs)
# ---------------------------------------------------------------------------

FAMILY_BY_ARCH = {
    "DeepseekV3ForCausalLM": "deepseek_v3",
    "DeepseekV32ForCausalLM": "deepseek_v3",
    "DeepseekV4ForCausalLM": "deepseek_v4",
    "Qwen3MoeForCausalLM": "qwen3_moe",
    "Qwen3ForCausalLM": "qwen3_dense",
    "Glm4MoeForCausalLM": "glm_moe",
    "GlmMoeDsaForCausalLM": "glm_moe",
    "MiMoV2FlashForCausalLM": "mimo_v2",
    "MixtralForCausalLM": "mixtral",
    "Qwen3NextForCausalLM": "hybrid_linear",
}


def detect_quant(cfg: dict) -> QuantSpec:
    q = cfg.get("quantization_config") or {}
    method = (q.get("quant_method") or q.get("quant_algo") or "").lower()
    fmt = (q.get("fmt") or q.get("format") or "").lower()
    if method == "fp8":
        blk = q.get("weight_block_size") or [128, 128]
        dense = "fp8_block32" if list(blk) == [32, 32] else "fp8_block128"
        experts = "mxfp4" if "mxfp4" in json.dumps(q).lower() else dense
        return QuantSpec(experts=experts, dense=dense)
    if method in ("mxfp4",):
        return QuantSpec(experts="mxfp4", dense="bf16")
    if method in ("modelopt", "nvfp4") or "nvfp4" in fmt or q.get("quant_algo", "").upper() == "NVFP4":
        return QuantSpec(experts="nvfp4", dense="nvfp4")
    if method in ("exl3",) or "exl3" in fmt:
        return QuantSpec(experts="exl3", dense="bf16", exl3_bits=int(round(float(q.get("bits", 4)))))
    return QuantSpec()


def from_hf_config(cfg: dict | str | Path) -> ModelSpec:
    """Build a ModelSpec from a Hugging Face `config.json` (dict or path)."""
    if not isinstance(cfg, dict):
        p = Path(cfg)
        p = p / "config.json" if p.is_dir() else p
        cfg = json.loads(p.read_text())
    archs = cfg.get("architectures") or ["?"]
    family = FAMILY_BY_ARCH.get(archs[0])
    if family is None:
        raise ValueError(f"unsupported architecture {archs[0]!r} (supported: {sorted(FAMILY_BY_ARCH)})")
    hidden = cfg["hidden_size"]
    heads = cfg["num_attention_heads"]
    if "kv_lora_rank" in cfg:
        attn = AttentionSpec(kind="mla", n_heads=heads, n_kv_heads=heads,
                             head_dim=cfg["qk_nope_head_dim"] + cfg["qk_rope_head_dim"],
                             rope_theta=cfg.get("rope_theta", 1e4),
                             q_lora_rank=cfg.get("q_lora_rank") or 0, kv_lora_rank=cfg["kv_lora_rank"],
                             qk_nope_head_dim=cfg["qk_nope_head_dim"], qk_rope_head_dim=cfg["qk_rope_head_dim"],
                             v_head_dim=cfg["v_head_dim"],
                             # sparse attention with a learned indexer (the V3.2 / GLM-5 line)
                             index_topk=cfg.get("index_topk") or 0, index_heads=cfg.get("index_n_heads") or 0,
                             index_dim=cfg.get("index_head_dim") or 0)
    else:
        attn = AttentionSpec(kind="gqa", n_heads=heads, n_kv_heads=cfg.get("num_key_value_heads", heads),
                             head_dim=cfg.get("head_dim") or hidden // heads,
                             rope_theta=cfg.get("rope_theta", 1e4), rope_interleaved=False,
                             qk_norm=family in ("qwen3_moe", "qwen3_dense"),
                             window=cfg.get("sliding_window_size") or cfg.get("sliding_window") or 0)
        if cfg.get("full_attention_interval") and cfg.get("linear_num_value_heads"):
            # hybrid linear-attention stack (the Qwen-Next line): gated delta-rule layers, every n-th layer full attention
            if cfg.get("linear_key_head_dim", 128) != 128 or cfg.get("linear_value_head_dim", 128) != 128 or cfg.get("linear_conv_kernel_dim", 4) != 4:
                raise ValueError("linear-attention layers: 128-wide key / value heads and a width-4 convolution are supported")
            attn = dataclasses.replace(attn, linear_every=int(cfg["full_attention_interval"]), linear_k_heads=int(cfg["linear_num_key_heads"]),
                                       linear_v_heads=int(cfg["linear_num_value_heads"]), qk_norm=True)
        pattern = cfg.get("hybrid_layer_pattern")            # MiMo-V2: 0 = full attention, 1 = sliding window (+ sinks)
        if attn.linear_every:
            pattern = None                                    # `layer_types` then names the linear layers, not sliding windows
        if pattern is None and cfg.get("layer_types") and not attn.linear_every:
            pattern = [0 if t == "full_attention" else 1 for t in cfg["layer_types"]]
        if pattern and any(pattern):
            full = [i for i, p in enumerate(pattern) if not p]
            period = (full[1] - full[0]) if len(full) > 1 else len(pattern)
            if not full or full[0] != 0 or any(bool(p) == (i % period == 0) for i, p in enumerate(pattern)):
                raise ValueError("unsupported layer pattern: full-attention layers must sit at layer 0 and every n-th layer after it")
            attn = dataclasses.replace(attn, full_every=period, swa_rope_theta=float(cfg.get("swa_rope_theta") or 0.0),
                                       sink=bool(cfg.get("add_swa_attention_sink_bias", True)))
    n_exp = cfg.get("n_routed_experts") or cfg.get("num_experts") or cfg.get("num_local_experts") or 0
    moe = MoESpec(
        n_experts=n_exp, top_k=cfg.get("num_experts_per_tok", 1),
        intermediate=cfg.get("moe_intermediate_size") or cfg.get("intermediate_size", 0),
        n_shared=cfg.get("n_shared_experts") or 0,
        scoring=cfg.get("scoring_func", "softmax"), normalize=cfg.get("norm_topk_prob", True),
        route_scale=cfg.get("routed_scaling_factor", 1.0),
        use_bias=cfg.get("topk_method") == "noaux_tc", n_group=cfg.get("n_group") or 1,
        topk_group=cfg.get("topk_group") or 1, first_dense=cfg.get("first_k_dense_replace", 0),
        dense_intermediate=cfg.get("intermediate_size", 0))
    return ModelSpec(name=cfg.get("_name_or_path") or family, family=family, vocab=cfg["vocab_size"],
                     hidden=hidden, n_layers=cfg["num_hidden_layers"], rms_eps=cfg.get("rms_norm_eps", 1e-6),
                     attn=attn, moe=moe, quant=detect_quant(cfg),
                     mtp_layers=cfg.get("num_nextn_predict_layers", 0),
                     tie_embeddings=cfg.get("tie_word_embeddings", False),
                     max_context=cfg.get("max_position_embeddings", 1 << 20))


SPEC_FILE = "cuteafd_spec.json"


def spec_to_json(spec: ModelSpec) -> dict:
    """Lossless dump of a model spec (written next to synthetic snapshots, whose shapes have no Hugging Face architecture)."""
    return dataclasses.asdict(spec)


def spec_from_json(d: dict) -> ModelSpec:
    d = dict(d)
    if "engram_layers" in d:
        d["engram_layers"] = tuple(d["engram_layers"])
    return ModelSpec(attn=AttentionSpec(**d.pop("attn")), moe=MoESpec(**d.pop("moe")), quant=QuantSpec(**d.pop("quant")), **d)


def spec_from_snapshot(path: str | Path) -> ModelSpec:
    """Model spec of a snapshot directory: the native spec file when the snapshot has one, else its `config.json`."""
    p = Path(path)
    if (p / SPEC_FILE).exists():
        return spec_from_json(json.loads((p / SPEC_FILE).read_text()))
    return from_hf_config(p)


@dataclass(frozen=True)
class Deployment:
    """How ranks of one node are used (reference: SparkWorld / placement decisions).

    attention ranks run attention + dense backbone + router + shared expert (+ head);
    expert ranks hold routed experts, expert-parallel.  With `colocated=True` every rank does both."""
    world: int = 1
    attn_ranks: tuple = (0,)
    expert_ranks: tuple = (0,)
    colocated: bool = True
    attn_groups: int = 1        # data-parallel attention groups; each group is `tp` consecutive entries of attn_ranks

    @property
    def tp(self) -> int:
        return len(self.attn_ranks) // max(1, self.attn_groups)

    @property
    def ep(self) -> int:
        return len(self.expert_ranks)

    def group_of(self, rank: int) -> int:
        return self.attn_ranks.index(rank) // self.tp

    def group_ranks(self, g: int) -> tuple:
        return tuple(self.attn_ranks[g * self.tp:(g + 1) * self.tp])

    def describe(self) -> str:
        if self.world == 1:
            return "single"
        dp = f"dp{self.attn_groups}x" if self.attn_groups > 1 else ""
        return f"attn-{dp}tp{self.tp}+ep{self.ep}" if not self.colocated else f"colocated attn-{dp}tp{self.tp} + ep{self.ep} on the same GPUs"


def default_deployment(world: int, attn_groups: int = 1) -> Deployment:
    """North-star split: attention TP2 on ranks 0-1, experts EP on the rest (8 GPUs -> TP2 + EP6).  With
    `attn_groups` > 1 the attention side is that many data-parallel groups (each serving its own sequences, all
    sending to the same expert ranks, which work on one group's tokens while the other groups run attention):
    4 GPUs -> 2 x TP1 + EP2, 8 GPUs -> 2 x TP2 + EP4."""
    if world == 1:
        return Deployment()
    if world == 2:
        return Deployment(world=2, attn_ranks=(0,), expert_ranks=(1,), colocated=False)
    if attn_groups <= 1:
        return Deployment(world=world, attn_ranks=(0, 1), expert_ranks=tuple(range(2, world)), colocated=False)
    n_attn = max(attn_groups, (world // 2 // attn_groups) * attn_groups)
    if n_attn >= world:
        raise ValueError(f"{attn_groups} attention groups leave no expert rank in a world of {world}")
    return Deployment(world=world, attn_ranks=tuple(range(n_attn)), expert_ranks=tuple(range(n_attn, world)), colocated=False,
                      attn_groups=attn_groups)


def colocated_deployment(world: int) -> Deployment:
    """Every GPU is an attention rank for its own sequences (data-parallel attention, TP1) AND an expert rank for its share
    of the routed experts (reference counterpart: routed layers resident on the coordinator GPUs, `--rtx-expert-layers`,
    shared/experts/local.rs; on NVSwitch every GPU can afford both roles)."""
    if world == 1:
        return Deployment()
    ranks = tuple(range(world))
    return Deployment(world=world, attn_ranks=ranks, expert_ranks=ranks, colocated=True, attn_groups=world)


def deployment_by_name(layout: str, world: int, attn_groups: int = 1) -> Deployment:
    """`split` = disjoint attention / expert ranks (`default_deployment`), `colocated` = both roles on every GPU."""
    if layout == "colocated":
        return colocated_deployment(world)
    if layout == "split":
        return default_deployment(world, attn_groups)
    raise ValueError(f"unknown layout {layout!r} (split | colocated)")
