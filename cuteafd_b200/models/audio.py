"""Audio tower on the GPU: log-mel frames -> rows of the decoder's hidden size that replace the audio placeholder tokens of a prompt.

The front end is two width-3 convolutions over the frame axis run as GEMMs (`audio_im2col3` builds the operand rows, `tc_linear`
multiplies, `vision_bias_act` adds the bias and the GELU); blocks and merger are the encoder tower shared with the vision model
(`models/vision.py::EncoderTower`: bf16 tcgen05 GEMMs, bidirectional tcgen05 attention over heads padded to 128, fused glue) with the
rotary table set to the identity (positions are sinusoids added to the residual) and the merger reduced to the average of two frames
followed by one projection - folded into ONE GEMM over the concatenated pair with the projection's weight halved and duplicated.
The mel spectrogram (FFT + filter bank, `ref/audio.py::log_mel`) is computed once per clip on the host with torch's FFT.

Reference: native/shared/cuda/audio_runtime.cu (audio tower driver), rust/crates/cuteafd-daemon/src/shared/vision.rs (encoder owners).
"""
from __future__ import annotations

import torch

from ..ops import native
from ..ops.native import ptr
from ..ref.audio import AudioSpec, log_mel, sinusoid_positions
from .vision import EncoderTower


def load_audio(data, spec: AudioSpec) -> torch.Tensor:
    """WAV bytes / base64 string / fp32 waveform tensor (mono, at the tower's sample rate) -> log-mel frames fp32 [n, n_mels]."""
    if isinstance(data, torch.Tensor):
        return log_mel(data, spec)
    import base64
    import io
    import wave

    import numpy as np
    if isinstance(data, str):
        data = base64.b64decode(data.split(",", 1)[1] if data.startswith("data:") else data)
    with wave.open(io.BytesIO(data)) as wf:
        if wf.getsampwidth() != 2:
            raise ValueError("audio input: 16-bit PCM WAV")
        pcm = np.frombuffer(wf.readframes(wf.getnframes()), dtype="<i2").astype(np.float32) / 32768.0
        if wf.getnchannels() > 1:
            pcm = pcm.reshape(-1, wf.getnchannels()).mean(axis=1)
        rate = wf.getframerate()
    x = torch.from_numpy(pcm.copy())
    if rate != spec.sample_rate:            # linear resampling: enough for speech front ends, no extra dependency
        n = int(round(x.numel() * spec.sample_rate / rate))
        x = torch.nn.functional.interpolate(x[None, None], size=n, mode="linear", align_corners=False)[0, 0]
    return log_mel(x, spec)


def audio_tokens(frames: torch.Tensor) -> int:
    return frames.shape[0] // 4


class AudioTower(EncoderTower):
    def __init__(self, spec: AudioSpec, masters: dict, device, max_frames: int = 12000, max_clips: int = 8):
        H = spec.hidden
        if spec.n_mels % 8:
            raise ValueError("audio tower: n_mels must be a multiple of 8")
        base = dict(masters)
        half = masters["proj_w"].float() / 2
        base["merger_fc2_w"], base["merger_fc2_b"] = torch.cat([half, half], dim=1), masters["proj_b"]        # mean of two frames, then proj
        super().__init__(spec, base, device, max_frames // 2, max_clips, 2)
        dev, N = self.device, self.max_patches
        # conv weight [out, in, 3] -> GEMM weight [out, 3 * in] with columns (tap, channel), the order audio_im2col3 writes
        self.conv1_w = self._mat(masters["conv1_w"].float().permute(0, 2, 1).reshape(H, -1))
        self.conv2_w = self._mat(masters["conv2_w"].float().permute(0, 2, 1).reshape(H, -1))
        self.conv1_b, self.conv2_b = self._vec(masters["conv1_b"]), self._vec(masters["conv2_b"])
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.mel = torch.zeros(2 * N, spec.n_mels, **bf)
        self.rows1 = torch.zeros(2 * N, 3 * spec.n_mels, **bf)
        self.f1 = torch.zeros(2 * N, H, **bf)
        self.h1 = torch.zeros(2 * N, H, **bf)
        self.rows2 = torch.zeros(N, 3 * H, **bf)
        self.g2 = torch.zeros(N, H, **bf)
        self.cs[:, : spec.head_dim // 2] = 1.0            # identity rotation: cos 1, sin 0
        self._pos: dict = {}

    def nbytes(self) -> int:
        return super().nbytes() + self.conv1_w.nbytes + self.conv2_w.nbytes + sum(t.numel() * 2 for t in (self.mel, self.rows1, self.f1, self.h1, self.rows2, self.g2))

    @torch.no_grad()
    def encode(self, clips: list[torch.Tensor]) -> list[torch.Tensor]:
        """`clips`: log-mel frames fp32 [n, n_mels], n a multiple of 4 (`load_audio`).  Returns one bf16 [n / 4, out_hidden] tensor per clip."""
        spec, H = self.spec, self.spec.hidden
        if not clips:
            return []
        if len(clips) > self.max_images:
            raise ValueError(f"audio tower: {len(clips)} clips in one call (limit {self.max_images})")
        n_in = [c.shape[0] for c in clips]
        if any(n % 4 or n == 0 for n in n_in) or any(c.shape[1] != spec.n_mels for c in clips):
            raise ValueError("audio tower: clips are [frames, n_mels] with a multiple of 4 frames")
        Nin, counts = sum(n_in), [n // 2 for n in n_in]
        N = Nin // 2
        if N > self.max_patches:
            raise ValueError(f"audio tower: {Nin} frames in one call (limit {2 * self.max_patches})")
        self.mel[:Nin].copy_(torch.cat(clips).to(torch.bfloat16))
        st = native.stream()
        off = 0
        for n in n_in:
            native.call("cuteafd_audio_im2col3", ptr(self.mel[off:]), ptr(self.rows1[off:]), n, spec.n_mels, 1, st)
            off += n
        self._linear(self.conv1_w, "rows1", self.rows1, self.f1, Nin)
        self._bias_act(self.f1, self.conv1_b, self.h1, Nin, H, "gelu")
        off = 0
        for n in n_in:
            native.call("cuteafd_audio_im2col3", ptr(self.h1[off:]), ptr(self.rows2[off // 2:]), n, H, 2, st)
            off += n
        self._linear(self.conv2_w, "rows2", self.rows2, self.y, N)
        self._bias_act(self.y, self.conv2_b, self.g2, N, H, "gelu")
        pos = []
        for c in counts:
            if c not in self._pos:
                if len(self._pos) >= 64:
                    self._pos.clear()
                self._pos[c] = sinusoid_positions(c, H).to(self.device)
            pos.append(self._pos[c])
        self.x[:N].copy_(torch.cat(pos))
        self._add_norm(self.g2, None, self._first_norm(), self.h, N)
        return self._finish(counts)
