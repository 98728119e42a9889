"""Vision tower throughput on one GPU: images per second and the share of the measured bf16 GEMM peak, random weights of the
Qwen3-VL tower shape (27 blocks, hidden 1152, 16 heads of 72, MLP 4304, patch 16, 2 x 2 merger).

    python -m cuteafd_b200.bench.vision --side 1024 --images 4          # four 1024 x 1024 images per call (4096 patches each)

Timed with CUDA events over `--iters` encode calls after warm-up; the inputs (RGB bytes) are re-uploaded by every call, so the
figure includes the host-to-device copy of the pixels.  FLOPs counted are the model's (head_dim 72), not the padded ones the
attention kernel executes (128 per head).
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from ..models.vision import VisionTower
from ..ref.vision import VisionSpec, init_vision_weights


def tower_flops(spec: VisionSpec, counts: list[int]) -> float:
    H, HD, I, M = spec.hidden, spec.n_heads * spec.head_dim, spec.intermediate, spec.merge ** 2 * spec.hidden
    n = sum(counts)
    per_tok = 2 * H * 3 * HD + 2 * HD * H + 2 * H * I * (3 if spec.mlp == "swiglu" else 2)
    attn = sum(4.0 * c * c * HD for c in counts)
    merger = (n / spec.merge ** 2) * (2 * M * M + 2 * M * spec.out_hidden)
    return spec.depth * (n * per_tok + attn) + n * 2 * spec.patch_dim * H + merger


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--side", type=int, default=1024, help="image side in pixels (a multiple of 32)")
    ap.add_argument("--images", type=int, default=4)
    ap.add_argument("--depth", type=int, default=27)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out-hidden", type=int, default=4096)
    a = ap.parse_args()
    spec = VisionSpec(hidden=1152, depth=a.depth, n_heads=16, head_dim=72, intermediate=4304, patch=16, out_hidden=a.out_hidden, pos_grid=48,
                      mlp="gelu_tanh")
    dev = torch.device("cuda", 0)
    g = a.side // spec.patch
    tower = VisionTower(spec, init_vision_weights(spec, 0), dev, max_patches=a.images * g * g, max_images=a.images)
    gen = torch.Generator().manual_seed(0)
    images = [torch.randint(0, 256, (a.side, a.side, 3), generator=gen, dtype=torch.uint8).pin_memory() for _ in range(a.images)]
    for _ in range(a.warmup):
        tower.encode(images)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        tower.encode(images)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.iters
    counts = [g * g] * a.images
    fl = tower_flops(spec, counts)
    peaks = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    peak = json.loads(peaks.read_text()).get("bf16_tflops") if peaks.exists() else None
    out = {"bench": "vision_tower", "images": a.images, "side": a.side, "patches": sum(counts), "tokens_out": sum(counts) // spec.merge ** 2,
           "depth": a.depth, "ms_per_call": round(ms, 3), "images_per_s": round(a.images / ms * 1e3, 1), "tflops": round(fl / ms / 1e9, 1),
           "weights_mib": round(tower.nbytes() / 2 ** 20)}
    if peak:
        out["of_measured_bf16_peak"] = round(fl / ms / 1e9 / peak, 3)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
