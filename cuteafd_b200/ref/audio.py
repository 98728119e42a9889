"""fp32 oracle of the audio tower: waveform -> log-mel frames -> two width-3 convolutions (the second with stride 2) -> sinusoidal
positions -> bidirectional pre-norm transformer blocks -> final LayerNorm -> pairs of frames averaged -> projection to the decoder's
hidden size (the Whisper-encoder shape that Qwen-Audio / Omni style models put in front of the decoder).

Reference: native/shared/cuda/audio_runtime.cu (audio tower driver: FFT, mel filter bank, convolution front end, encoder blocks),
rust/crates/cuteafd-daemon/src/shared/vision.rs (the encoder owner also serves audio).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace

import torch
import torch.nn.functional as F

from .vision import _norm, encoder_blocks


@dataclass(frozen=True)
class AudioSpec:
    hidden: int = 128
    depth: int = 2
    n_heads: int = 2
    head_dim: int = 64
    intermediate: int = 256
    out_hidden: int = 256
    n_mels: int = 128
    sample_rate: int = 16000
    n_fft: int = 400
    hop: int = 160
    max_seconds: float = 30.0
    norm: str = "layernorm"
    mlp: str = "gelu"
    qkv_bias: bool = True
    qk_norm: bool = False
    eps: float = 1e-5

    def replace(self, **kw) -> "AudioSpec":
        return replace(self, **kw)


def mel_filters(spec: AudioSpec) -> torch.Tensor:
    """Triangular filters on the mel scale (Slaney: linear below 1 kHz, logarithmic above; area-normalised): fp32 [n_mels, n_fft / 2 + 1]."""
    def hz_to_mel(f):
        f = torch.as_tensor(f, dtype=torch.float64)
        return torch.where(f < 1000.0, f / (200.0 / 3), 15.0 + torch.log(f.clamp(min=1e-9) / 1000.0) / (math.log(6.4) / 27.0))

    def mel_to_hz(m):
        return torch.where(m < 15.0, m * (200.0 / 3), 1000.0 * torch.exp((m - 15.0) * (math.log(6.4) / 27.0)))

    n_freq = spec.n_fft // 2 + 1
    freqs = torch.linspace(0, spec.sample_rate / 2, n_freq, dtype=torch.float64)
    pts = mel_to_hz(torch.linspace(float(hz_to_mel(0.0)), float(hz_to_mel(spec.sample_rate / 2)), spec.n_mels + 2, dtype=torch.float64))
    lower = (freqs[None, :] - pts[:-2, None]) / (pts[1:-1] - pts[:-2])[:, None]
    upper = (pts[2:, None] - freqs[None, :]) / (pts[2:] - pts[1:-1])[:, None]
    fb = torch.clamp(torch.minimum(lower, upper), min=0.0)
    return (fb * (2.0 / (pts[2:] - pts[:-2]))[:, None]).float()


def log_mel(wave: torch.Tensor, spec: AudioSpec) -> torch.Tensor:
    """Mono fp32 waveform at `sample_rate` -> log-mel frames fp32 [frames, n_mels] (an even number of frames: the tower halves them twice)."""
    wave = wave.float().flatten()[: int(spec.max_seconds * spec.sample_rate)]
    st = torch.stft(wave, spec.n_fft, spec.hop, window=torch.hann_window(spec.n_fft), return_complex=True)
    power = st[:, :-1].abs() ** 2
    mel = torch.log10((mel_filters(spec) @ power).clamp(min=1e-10))
    mel = (torch.maximum(mel, mel.max() - 8.0) + 4.0) / 4.0
    frames = mel.T.contiguous()
    n = frames.shape[0] // 4 * 4
    if n == 0:
        raise ValueError("audio clip shorter than four frames")
    return frames[:n]


def sinusoid_positions(n: int, dim: int) -> torch.Tensor:
    inc = math.log(10000.0) / (dim // 2 - 1)
    t = torch.arange(n, dtype=torch.float32)[:, None] * torch.exp(-inc * torch.arange(dim // 2, dtype=torch.float32))[None, :]
    return torch.cat([t.sin(), t.cos()], dim=1)


def init_audio_weights(spec: AudioSpec, seed: int = 0) -> dict:
    from .vision import VisionSpec, init_vision_weights
    v = VisionSpec(hidden=spec.hidden, depth=spec.depth, n_heads=spec.n_heads, head_dim=spec.head_dim, intermediate=spec.intermediate,
                   out_hidden=spec.out_hidden, norm=spec.norm, mlp=spec.mlp, qkv_bias=spec.qkv_bias, qk_norm=spec.qk_norm, patch=2)
    base = init_vision_weights(v, seed)
    g = torch.Generator().manual_seed(seed + 101)
    H = spec.hidden
    w = {"blocks": base["blocks"], "merger_norm_w": base["merger_norm_w"]}
    if "merger_norm_b" in base:
        w["merger_norm_b"] = base["merger_norm_b"]
    w["conv1_w"] = torch.randn(H, spec.n_mels, 3, generator=g) * (3 * spec.n_mels) ** -0.5
    w["conv1_b"] = torch.randn(H, generator=g) * 0.1
    w["conv2_w"] = torch.randn(H, H, 3, generator=g) * (3 * H) ** -0.5
    w["conv2_b"] = torch.randn(H, generator=g) * 0.1
    w["proj_w"] = torch.randn(spec.out_hidden, H, generator=g) * H ** -0.5
    w["proj_b"] = torch.randn(spec.out_hidden, generator=g) * 0.1
    return w


def audio_bf16_round(w):
    if isinstance(w, dict):
        return {k: audio_bf16_round(v) if isinstance(v, (dict, list)) else (v.bfloat16().float() if v.dim() >= 2 else v) for k, v in w.items()}
    return [audio_bf16_round(v) for v in w]


def audio_forward(spec: AudioSpec, w: dict, frames: torch.Tensor) -> torch.Tensor:
    """Log-mel frames [n, n_mels] (n a multiple of 4) -> [n / 4, out_hidden]."""
    x = F.gelu(F.conv1d(frames.T[None], w["conv1_w"], w["conv1_b"], padding=1))
    x = F.gelu(F.conv1d(x, w["conv2_w"], w["conv2_b"], stride=2, padding=1))[0].T          # [n / 2, H]
    x = x + sinusoid_positions(x.shape[0], spec.hidden)
    x = encoder_blocks(spec, w["blocks"], x, None)
    h = _norm(x, w["merger_norm_w"], w.get("merger_norm_b"), spec.eps)
    h = h.reshape(h.shape[0] // 2, 2, -1).mean(dim=1)
    return h @ w["proj_w"].T + w["proj_b"]
