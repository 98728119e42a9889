"""Device-resident model weights in the formats the kernels consume.

Two constructors:
  * `DeviceWeights.from_masters(spec, masters, device)` - quantise fp32 masters (the oracle's `init_weights`)
    with the CPU format oracles; used by tests and small models so GPU results can be compared with the
    oracle evaluated on the *dequantised* weights.
  * `DeviceWeights.random(spec, device, ...)` - random-init weights generated directly in storage format on
    the GPU (synthetic benchmarks of the 235B / 671B shapes; there are no checkpoints to read here).
    `distinct_layers` bounds how many distinct layer weight sets are materialised (layer i uses set
    i % distinct_layers) for shapes that exceed one GPU's memory; every layer still runs at full size.

Layout mirrors what the loader produces from an HF snapshot: projections stay [out, in] (K-major), experts
stay separate per-expert matrices addressed through per-expert TMA descriptors, block scales are re-tiled
once on the device into the tensor-core scale-factor atom layout (reference: expert_pack.cu:9,
nvfp4_scale.cu:22 do the equivalent one-time device-side preparation).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import os

import torch

from ..config import ModelSpec
from ..ops import TcWeight, KIND_BF16, KIND_BY_NAME


def _dense_kind(spec: ModelSpec) -> str:
    return {"bf16": "bf16", "nvfp4": "nvfp4", "mxfp4": "mxfp4", "fp8_block128": "fp8_block128"}.get(spec.quant.dense, "bf16")


def _expert_kind(spec: ModelSpec) -> str:
    return {"bf16": "bf16", "nvfp4": "nvfp4", "mxfp4": "mxfp4"}.get(spec.quant.experts, "bf16")


# n-gram memory: rows of a step the module's buffers hold, and where the tables live ("device", or "host": pinned host memory read in place)
ENGRAM_ROWS = int(os.environ.get("CUTEAFD_ENGRAM_ROWS", "4096"))
ENGRAM_TABLES = os.environ.get("CUTEAFD_ENGRAM_TABLES", "device")

@dataclass
class LayerWeights:
    attn_norm: torch.Tensor
    ffn_norm: torch.Tensor
    wqkv: TcWeight
    wo: TcWeight
    q_norm: torch.Tensor | None = None
    k_norm: torch.Tensor | None = None
    sink: torch.Tensor | None = None
    router: TcWeight | None = None
    router_bias: torch.Tensor | None = None
    w_gate: TcWeight | None = None
    w_up: TcWeight | None = None
    w_down: TcWeight | None = None
    ws_gate: TcWeight | None = None     # shared expert, or the dense FFN of a non-MoE layer
    ws_up: TcWeight | None = None
    ws_down: TcWeight | None = None
    # gated delta-rule (linear attention) layers: fused q / k / v / z projection, gate projection (fp32 output), convolution taps,
    # decay parameters, output norm; `wo` is then [hidden, Hv * 128] and `wqkv` is None
    lin_qkvz: TcWeight | None = None
    lin_ba: TcWeight | None = None
    lin_conv: torch.Tensor | None = None
    lin_dt_bias: torch.Tensor | None = None
    lin_a_log: torch.Tensor | None = None
    lin_norm: torch.Tensor | None = None
    # hyper-connections: (fn [24, 4H] fp32, scale [3], base [24]) of the boundary in front of the attention and of the FFN block
    hc_attn: tuple | None = None
    hc_ffn: tuple | None = None

    def nbytes(self) -> int:
        n = 0
        for name, v in vars(self).items():
            if name == "ws_gate_up":         # the fused gate + up weight: ws_gate and ws_up are views into it
                continue
            if isinstance(v, TcWeight):
                n += v.nbytes
            elif isinstance(v, torch.Tensor):
                n += v.numel() * v.element_size()
            elif isinstance(v, tuple):
                n += sum(t.numel() * t.element_size() for t in v)
        return n


@dataclass
class DeviceWeights:
    spec: ModelSpec
    embed: torch.Tensor
    final_norm: torch.Tensor
    lm_head: TcWeight
    layers: list = field(default_factory=list)     # distinct layer sets
    layer_map: list = field(default_factory=list)  # layer index -> index into `layers`
    mtp: list = field(default_factory=list)        # [(enorm, hnorm, eh_proj TcWeight, LayerWeights, norm)]
    act_gs: float = 1.0 / 64
    engram: object | None = None                   # n-gram memory (`models/engram.py::EngramModule`) of specs with engram_layers
    hc_head: tuple | None = None                   # hyper-connections: (fn [4, 4H], scale [3], base [4]) of the head's collapse

    def layer(self, i: int) -> LayerWeights:
        return self.layers[self.layer_map[i]]

    def nbytes(self) -> int:
        return sum(l.nbytes() for l in self.layers) + self.embed.numel() * 2 + (self.lm_head.nbytes if self.lm_head else 0)

    # ------------------------------------------------------------------ from fp32 masters
    @staticmethod
    def from_masters(spec: ModelSpec, masters: dict, device, act_gs: float = 1.0 / 64) -> "DeviceWeights":
        dk, ek = _dense_kind(spec), _expert_kind(spec)
        f32 = lambda t: t.float().to(device).contiguous()

        def layer_from(lw: dict) -> LayerWeights:
            if spec.attn.kind != "gqa":
                raise NotImplementedError("from_masters: MLA layers are built by models.mla")
            if "w_qkvz" in lw:       # linear-attention layer
                out = LayerWeights(attn_norm=f32(lw["attn_norm"]), ffn_norm=f32(lw["ffn_norm"]), wqkv=None,
                                   wo=TcWeight.from_master(lw["wo"], dk, device, act_gs),
                                   lin_qkvz=TcWeight.from_master(lw["w_qkvz"], dk, device, act_gs), lin_ba=TcWeight.from_master(lw["w_ba"], "bf16", device),
                                   lin_conv=f32(lw["conv_w"]), lin_dt_bias=f32(lw["dt_bias"]), lin_a_log=f32(lw["a_log"]), lin_norm=f32(lw["lin_norm"]))
            else:
                wqkv = torch.cat([lw["wq"], lw["wk"], lw["wv"]], 0)
                out = LayerWeights(attn_norm=f32(lw["attn_norm"]), ffn_norm=f32(lw["ffn_norm"]),
                                   wqkv=TcWeight.from_master(wqkv, dk, device, act_gs),
                                   wo=TcWeight.from_master(lw["wo"], dk, device, act_gs))
            if "hc_attn_fn" in lw:
                out.hc_attn = tuple(f32(lw[f"hc_attn_{k}"]) for k in ("fn", "scale", "base"))
                out.hc_ffn = tuple(f32(lw[f"hc_ffn_{k}"]) for k in ("fn", "scale", "base"))
            if "q_norm" in lw:
                out.q_norm, out.k_norm = f32(lw["q_norm"]), f32(lw["k_norm"])
            if "sink" in lw:
                out.sink = f32(lw["sink"])
            if "router" in lw:
                out.router = TcWeight.from_master(lw["router"], "bf16", device)
                if "router_bias" in lw:
                    out.router_bias = f32(lw["router_bias"])
                if "w_gate" in lw:      # an attention rank of a split layout holds no routed experts
                    out.w_gate = TcWeight.from_master(lw["w_gate"], ek, device, act_gs)
                    out.w_up = TcWeight.from_master(lw["w_up"], ek, device, act_gs)
                    out.w_down = TcWeight.from_master(lw["w_down"], ek, device, act_gs)
                if "ws_gate" in lw:
                    out.ws_gate = TcWeight.from_master(lw["ws_gate"], dk, device, act_gs)
                    out.ws_up = TcWeight.from_master(lw["ws_up"], dk, device, act_gs)
                    out.ws_down = TcWeight.from_master(lw["ws_down"], dk, device, act_gs)
            else:
                out.ws_gate = TcWeight.from_master(lw["wd_gate"], dk, device, act_gs)
                out.ws_up = TcWeight.from_master(lw["wd_up"], dk, device, act_gs)
                out.ws_down = TcWeight.from_master(lw["wd_down"], dk, device, act_gs)
            return out

        dw = DeviceWeights(spec=spec, embed=masters["embed"].to(torch.bfloat16).to(device).contiguous(),
                           final_norm=f32(masters["final_norm"]),
                           lm_head=TcWeight.from_master(masters["lm_head"], "bf16", device), act_gs=act_gs)
        dw.layers = [layer_from(lw) for lw in masters["layers"]]
        dw.layer_map = list(range(spec.n_layers))
        if "hc_head_fn" in masters:
            dw.hc_head = tuple(f32(masters[f"hc_head_{k}"]) for k in ("fn", "scale", "base"))
        if "engram" in masters and spec.engram_layers:
            from .engram import EngramModule
            dw.engram = EngramModule(spec.engram_spec(), masters["engram"], device, cap=ENGRAM_ROWS, tables=ENGRAM_TABLES)
        for mw in masters.get("mtp", []):
            dw.mtp.append((f32(mw["enorm"]), f32(mw["hnorm"]), TcWeight.from_master(mw["eh_proj"], "bf16", device),
                           layer_from(mw["layer"]), f32(mw["norm"])))
        return dw

    def dequantized_masters(self) -> dict:
        """fp32 masters equivalent to what the kernels compute with (oracle input for quantised models)."""
        a, spec = self.spec.attn, self.spec
        nq, nk = a.n_heads * a.head_dim, a.n_kv_heads * a.head_dim

        def layer_to(l: LayerWeights) -> dict:
            if l.lin_qkvz is not None:
                d = {"attn_norm": l.attn_norm.cpu(), "ffn_norm": l.ffn_norm.cpu(), "w_qkvz": l.lin_qkvz.dequantize()[0], "w_ba": l.lin_ba.dequantize()[0],
                     "conv_w": l.lin_conv.cpu(), "dt_bias": l.lin_dt_bias.cpu(), "a_log": l.lin_a_log.cpu(), "lin_norm": l.lin_norm.cpu(),
                     "wo": l.wo.dequantize()[0]}
            else:
                qkv = l.wqkv.dequantize()[0]
                d = {"attn_norm": l.attn_norm.cpu(), "ffn_norm": l.ffn_norm.cpu(), "wq": qkv[:nq], "wk": qkv[nq:nq + nk],
                     "wv": qkv[nq + nk:], "wo": l.wo.dequantize()[0]}
            if l.hc_attn is not None:
                for blk, t in (("attn", l.hc_attn), ("ffn", l.hc_ffn)):
                    d[f"hc_{blk}_fn"], d[f"hc_{blk}_scale"], d[f"hc_{blk}_base"] = (x.cpu() for x in t)
            if l.q_norm is not None:
                d["q_norm"], d["k_norm"] = l.q_norm.cpu(), l.k_norm.cpu()
            if l.sink is not None:
                d["sink"] = l.sink.cpu()
            if l.router is not None:
                d["router"] = l.router.dequantize()[0]
                if l.router_bias is not None:
                    d["router_bias"] = l.router_bias.cpu()
                d["w_gate"], d["w_up"], d["w_down"] = l.w_gate.dequantize(), l.w_up.dequantize(), l.w_down.dequantize()
                if l.ws_gate is not None:
                    d["ws_gate"], d["ws_up"], d["ws_down"] = (l.ws_gate.dequantize()[0], l.ws_up.dequantize()[0], l.ws_down.dequantize()[0])
            else:
                d["wd_gate"], d["wd_up"], d["wd_down"] = (l.ws_gate.dequantize()[0], l.ws_up.dequantize()[0], l.ws_down.dequantize()[0])
            return d

        m = {"embed": self.embed.float().cpu(), "final_norm": self.final_norm.cpu(), "lm_head": self.lm_head.dequantize()[0],
             "layers": [layer_to(self.layer(i)) for i in range(spec.n_layers)]}
        if self.hc_head is not None:
            m["hc_head_fn"], m["hc_head_scale"], m["hc_head_base"] = (x.cpu() for x in self.hc_head)
        if self.engram is not None:
            m["engram"] = {"layers": [{"table_q": l["tq"].cpu(), "table_e": l["te"].cpu(), "proj": l["proj"].dequantize()[0], "wq": l["wq"].cpu(),
                                       "wk": l["wk"].cpu()} for l in self.engram.layers]}
        if self.mtp:
            m["mtp"] = [{"enorm": e.cpu(), "hnorm": h.cpu(), "eh_proj": p.dequantize()[0], "layer": layer_to(l), "norm": n.cpu()}
                        for e, h, p, l, n in self.mtp]
        return m

    # ------------------------------------------------------------------ random, directly in storage format
    @staticmethod
    def random(spec: ModelSpec, device, distinct_layers: int = 0, act_gs: float = 1.0 / 64, seed: int = 0,
               experts_range: tuple | None = None, with_attention: bool = True) -> "DeviceWeights":
        if spec.attn.kind != "gqa" and with_attention:
            raise NotImplementedError("random: MLA attention layers are built by engine.mla.mla_weights_random")
        a, m, h = spec.attn, spec.moe, spec.hidden
        dk, ek = _dense_kind(spec), _expert_kind(spec)
        n_sets = spec.n_layers if distinct_layers <= 0 else min(distinct_layers, spec.n_layers)
        if a.linear_every and n_sets < spec.n_layers and n_sets % a.linear_every:
            raise ValueError("random: with linear-attention layers, distinct_layers must be a multiple of linear_every (the weight sets repeat)")
        ones = lambda n: torch.ones(n, dtype=torch.float32, device=device)
        e_lo, e_hi = experts_range if experts_range else (0, m.n_experts)

        def make_layer(i: int) -> LayerWeights:
            s = seed * 1000 + i * 16
            R = lambda G, N, K, kind, j: TcWeight.random(G, N, K, kind, device, spec.init_std, act_gs, s + j)
            RE = lambda N, K, j: TcWeight.random(m.n_experts, N, K, ek, device, spec.init_std, act_gs, s + j, groups=(e_lo, e_hi))
            if with_attention and spec.layer_is_linear(i):
                Hk, Hv = a.linear_k_heads, a.linear_v_heads
                C = (2 * Hk + Hv) * 128
                gl = torch.Generator(device=device).manual_seed(s + 9)
                nb = Hv + (Hv * 128 if a.linear_per_channel else Hv)
                out = LayerWeights(attn_norm=ones(h), ffn_norm=ones(h), wqkv=None, wo=R(1, h, Hv * 128, dk, 1),
                                   lin_qkvz=R(1, (2 * Hk + 2 * Hv) * 128, h, dk, 0), lin_ba=R(1, nb, h, "bf16", 10),
                                   lin_conv=torch.empty(C, 4, device=device).normal_(0, 0.5, generator=gl),
                                   lin_dt_bias=torch.empty(Hv * 128 if a.linear_per_channel else Hv, device=device).normal_(0, 0.5, generator=gl),
                                   lin_a_log=torch.empty(Hv, device=device).normal_(0, 0.5, generator=gl), lin_norm=ones(128))
            else:
                out = LayerWeights(attn_norm=ones(h), ffn_norm=ones(h),
                                   wqkv=R(1, (a.n_heads + 2 * a.n_kv_heads) * a.head_dim, h, dk, 0) if with_attention else None,
                                   wo=R(1, h, a.n_heads * a.head_dim, dk, 1) if with_attention else None)
            if spec.hyper_streams and with_attention:
                S = spec.hyper_streams
                gh = torch.Generator(device=device).manual_seed(s + 11)
                mk = lambda: (torch.empty(S * (S + 2), S * h, device=device).normal_(0, 2.0 / (S * h) ** 0.5, generator=gh),
                              torch.full((3,), 0.5, device=device), torch.empty(S * (S + 2), device=device).normal_(0, 0.5, generator=gh))
                out.hc_attn, out.hc_ffn = mk(), mk()
            if not with_attention:      # expert rank: routed experts only
                if spec.is_moe_layer(i) and e_hi > e_lo:
                    out.w_gate, out.w_up, out.w_down = RE(m.intermediate, h, 3), RE(m.intermediate, h, 4), RE(h, m.intermediate, 5)
                return out
            if a.qk_norm:
                out.q_norm, out.k_norm = ones(a.head_dim), ones(a.head_dim)
            if spec.is_moe_layer(i):
                out.router = R(1, m.n_experts, h, "bf16", 2)
                if m.use_bias:
                    out.router_bias = torch.zeros(m.n_experts, dtype=torch.float32, device=device)
                if e_hi > e_lo:
                    out.w_gate, out.w_up, out.w_down = RE(m.intermediate, h, 3), RE(m.intermediate, h, 4), RE(h, m.intermediate, 5)
                if m.shared_inter:
                    out.ws_gate, out.ws_up = R(1, m.shared_inter, h, dk, 6), R(1, m.shared_inter, h, dk, 7)
                    out.ws_down = R(1, h, m.shared_inter, dk, 8)
            else:
                inter = m.dense_intermediate or m.intermediate
                out.ws_gate, out.ws_up, out.ws_down = R(1, inter, h, dk, 6), R(1, inter, h, dk, 7), R(1, h, inter, dk, 8)
            return out

        gen = torch.Generator(device=device).manual_seed(seed)
        if with_attention:
            embed = torch.empty(spec.vocab, h, dtype=torch.bfloat16, device=device).normal_(0, spec.init_std, generator=gen)
            head = TcWeight.random(1, spec.vocab, h, "bf16", device, spec.init_std, act_gs, seed + 7)
        else:
            embed, head = torch.zeros(8, h, dtype=torch.bfloat16, device=device), None
        dw = DeviceWeights(spec=spec, embed=embed, final_norm=ones(h), lm_head=head, act_gs=act_gs)
        dw.layers = [make_layer(i) for i in range(n_sets)]
        dw.layer_map = [i % n_sets for i in range(spec.n_layers)]
        if spec.hyper_streams and with_attention:
            S = spec.hyper_streams
            dw.hc_head = (torch.empty(S, S * h, device=device).normal_(0, 2.0 / (S * h) ** 0.5, generator=gen), torch.full((3,), 0.5, device=device),
                          torch.empty(S, device=device).normal_(0, 0.5, generator=gen))
        if spec.engram_layers and with_attention:
            from ..ref.engram import init_engram_weights
            from .engram import EngramModule
            dw.engram = EngramModule(spec.engram_spec(), init_engram_weights(spec.engram_spec(), seed + 17), device, cap=ENGRAM_ROWS, tables=ENGRAM_TABLES)
        return dw
