#!/usr/bin/env python
"""Headline benchmark: decode throughput (tokens/s, whole job) of the Qwen3-235B-A22B-shape MoE with NVFP4
weights, 16 sequences per GPU at 4k context (weak scaling: 1 GPU = batch 16 ... 8 GPUs = batch 128 with
attention TP2 + experts EP6), random-init weights, synthetic token ids, bf16 activations / NVFP4 GEMMs.

    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Prints ONE JSON line on rank 0.  `value` is timed on the device with CUDA events around K graph-replayed
decode steps (max over ranks); `e2e` times the same K steps through the public generation API including the
per-step host-to-device input copy (pinned) and the device-to-host token read.  Other workloads of the
benchmark plan are reachable with --config (see `cuteafd_b200/bench/`).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

BASELINE_TOKS = 657.0   # reference's closest published number: Qwen3.8-Flash-Next NVFP4, C16 aggregate tok/s
BASELINE_SRC = "benchmarks/qwen4/2026-10-18-smoke-qwen3-8-flash-next-nvfp4-1rtx-2spark-qwen38-nvfp4-min/report.json:563 (C16 aggregate)"


class ClockSampler:
    """nvidia-smi sampling during the timed region (read-only queries)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.path = gpu_index, None, f"/tmp/cuteafd_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1])); mx.append(float(p[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def reference_arm(args):
    out = {"impl": "reference", "unavailable": "reference cannot be built offline: its GEMM/attention/expert kernels are AOT exports "
           "of the empty third_party/sparkinfer submodule and target sm_120/sm_121 only (the reference tree holds no pip-installable package)"}
    print(json.dumps(out))
    return 0


def deepseek_headline(args, rank: int, world: int, local: int) -> dict | None:
    """DeepSeek-V3-shape decode with the one-layer MTP drafter, batch 64 and batch 1 at 8k context: batch 64 on the default
    layout (colocated: every GPU attention + experts; `--layout split` selects the named attention TP2 + expert ranks), batch 1 on
    the split (one sequence has one attention group).  Rank 0 gets the record."""
    import torch
    from cuteafd_b200.bench.mtp_decode import run_mtp_decode_bench
    from cuteafd_b200.config import deepseek_v3_spec
    from cuteafd_b200.parallel.selftest import run_selftest
    if world < 4:
        raise SystemExit("the DeepSeek-V3 shape needs the attention/expert split on at least 4 GPUs")
    spec = deepseek_v3_spec(args.layers or 61)
    context = 8192 if args.context == 4096 else args.context
    ok = None
    if not args.no_selftest and args.comm == "p2p":
        from cuteafd_b200.parallel.runner import default_layout
        lay = args.layout or default_layout(spec, world, args.comm)["layout"]
        ok = run_selftest(rank, world, local, layout=lay, groups=(world if lay == "colocated" else (args.attn_groups or 1)),
                          n_micro=(1 if lay == "colocated" else (args.n_micro or 2)), comm="p2p", experts="mxfp4", model="mla", verbose=False)
    out = {}
    clocks = ClockSampler(local)
    for name, batch in (("bs64", args.batch_total or 64), ("bs1", 1)):
        out[name] = run_mtp_decode_bench(args, spec, rank, world, local, clocks, batch=batch, context=context, n_draft=args.mtp,
                                         rounds=max(3, min(args.steps, 10)), warmup=3)
        import gc
        gc.collect(); torch.cuda.empty_cache()
        if args.batch_total:
            break
    if rank != 0:
        return None
    main = out.get("bs64") or next(iter(out.values()))
    return {"metric": "decode_tokens_per_s", "value": main["tokens_per_s_measured"], "unit": "tokens/s", "n_gpus": world,
            "steps": main["rounds"], "warmup": main["warmup"], "ms_per_step": main["round_ms"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": f"bf16 activations, {spec.quant.experts} experts / {spec.quant.dense} dense",
            "data": "synthetic token ids, random-init weights (so the drafter's proposals are almost never accepted), context KV random-filled",
            "config": {"model": spec.name + (f" (DEBUG {args.layers} layers: INVALID)" if args.layers else ""), "global_batch": main["batch"],
                       "seq_len": context, "parallelism": main["parallelism"], "mtp_draft_tokens": args.mtp, "layers": spec.n_layers,
                       "l2": "inputs (weights + KV) far larger than L2; no flush needed"},
            "timing": "end to end: host clock around K draft/verify rounds through MtpSpeculator, each step copying its inputs H2D and reading tokens back",
            "selftest": None if ok is None else ("ok" if ok else "FAILED"), "results": out, "clocks": main.get("clocks")}


def deepseek_ttft(args, rank: int, world: int, local: int) -> dict | None:
    """Long-prefill + exact prefix-cache workload on the DeepSeek-V3 shape through the serving stack on the split (scheduler,
    chunked prefill, prefix cache on the attention leader; its TP partner mirrors it; expert ranks serve): sessions share a
    28k-token prefix and append 4k unique tokens; cold TTFT, prefix-restore TTFT (p50), then decode tokens per session."""
    import argparse as ap
    import torch
    import torch.distributed as dist
    from cuteafd_b200.bench.ttft import measure_sessions
    from cuteafd_b200.serving.split import build_split_serving
    prompt, shared, decode = args.ttft_prompt, args.ttft_shared, args.ttft_decode
    a = ap.Namespace(model="deepseek-v3", device=local, layers=args.layers, pool_tokens=(prompt + decode + 512) * 3 // 64 * 64, max_sequences=2,
                     max_context=prompt + decode + 256, prefill_batch_tokens=4096, host_cache_gib=0.0, host_cache_headroom_gib=0.0,
                     host_cache_min_tokens=512, prefix_cache_entries=16, prefix_cache_min_tokens=64, draft="off", decode_share=0.2, draft_limit=3,
                     http_queue=16, queue_wait_s=0, n_micro=args.n_micro or 1)
    built = build_split_serving(a, world)
    res = None
    if built is not None:
        spec, sched = built
        res = measure_sessions(sched, spec.vocab, prompt=prompt, shared=shared, sessions=args.ttft_sessions, decode=decode)
        sched.runner.eng.check_status()
        res.update(model=spec.name + (f" (DEBUG {args.layers} layers: INVALID)" if args.layers else ""), layers=spec.n_layers,
                   parallelism=sched.afd_runner.dep.describe(), prefix_cache=sched.prefix.snapshot(),
                   timing="host clock from submit to first token (device synchronised), through Scheduler + EngineRunner on the split",
                   data="synthetic token ids, random-init weights")
        sched.afd_runner.shutdown()
    dist.barrier()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="qwen3-235b-decode", choices=["qwen3-235b-decode", "deepseek-v3-decode", "deepseek-v3-plain", "deepseek-v3-ttft", "hybrid-gdn-decode", "hybrid-kda-decode"],
                    help="deepseek-v3-plain: one-token-per-step decode of the DeepSeek-V3 shape through the generic path (any --layout; no drafter)")
    ap.add_argument("--ttft-prompt", type=int, default=32768); ap.add_argument("--ttft-shared", type=int, default=28672)
    ap.add_argument("--ttft-sessions", type=int, default=8); ap.add_argument("--ttft-decode", type=int, default=256)
    ap.add_argument("--hyper-streams", type=int, default=0, help="1 GPU: run the shape with this many residual streams (hyper-connections; 4)")
    ap.add_argument("--batch-per-gpu", type=int, default=16)
    ap.add_argument("--batch-total", type=int, default=0, help="fixed global batch instead of a per-GPU batch (DeepSeek-V3 decode: 1 or 64)")
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (the result is then marked invalid)")
    ap.add_argument("--comm", default="p2p", choices=["p2p", "nccl"], help="multi-GPU transport: fused peer-memory kernels, or the NCCL-only baseline")
    ap.add_argument("--attn-groups", type=int, default=0, help="data-parallel attention groups in the split layout (0 = the config's default)")
    ap.add_argument("--layout", default=None, choices=["split", "colocated"],
                    help="multi-GPU layout: disjoint attention / expert ranks, or both roles on every GPU (default: per model, see parallel.runner.default_layout)")
    ap.add_argument("--n-micro", type=int, default=0, help="micro-batches an attention rank keeps in flight (0 = the layout's default)")
    ap.add_argument("--expert-tp", action="store_true",
                    help="expert ranks hold a slice of every expert's intermediate dimension (rows broadcast, rank-ordered partial sums) instead of whole experts")
    ap.add_argument("--no-selftest", action="store_true", help="skip the token-exactness check of the layout on the tiny model (N > 1)")
    ap.add_argument("--no-nccl-baseline", action="store_true", help="skip the NCCL-only arm that N > 1 runs report beside the main number")
    ap.add_argument("--real-prefill", action="store_true", help="build the context by running prefill instead of filling KV")
    ap.add_argument("--mtp", type=int, default=3, help="deepseek-v3-decode: draft tokens the MTP module proposes per round")
    ap.add_argument("--no-ttft", action="store_true", help="8 GPUs, default config: skip the 32k-prefill / prefix-restore sub-result")
    ap.add_argument("--no-headline", action="store_true",
                    help="8 GPUs, default config: skip the DeepSeek-V3-shape sub-results (batch 1 and 64 at 8k with the MTP drafter)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")

    if args.config == "deepseek-v3-ttft":
        res = deepseek_ttft(args, rank, world, local)
        if rank == 0:
            print(json.dumps({"metric": "ttft_s", "value": res["cold_ttft_s"], "unit": "s", "n_gpus": world, "steps": res["sessions"], "warmup": 0,
                              "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 activations, mxfp4 experts / fp8_block128 dense",
                              "data": res["data"], "config": {"model": res["model"], "global_batch": 1, "seq_len": res["prompt_tokens"],
                                                               "parallelism": res["parallelism"]}, "results": res}))
        import torch.distributed as dist
        dist.destroy_process_group()
        return 0
    if args.config == "deepseek-v3-decode":
        res = deepseek_headline(args, rank, world, local)
        if rank == 0:
            print(json.dumps(res))
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()
        return 0
    from cuteafd_b200.bench.decode import run_decode_bench
    selftest = None
    if world > 1 and not args.no_selftest and args.comm == "p2p":
        # the layout about to be timed must first generate the single-GPU engine's tokens on the tiny model
        from cuteafd_b200.config import deepseek_v3_spec, qwen3_235b_spec
        from cuteafd_b200.parallel.runner import default_layout
        from cuteafd_b200.parallel.selftest import run_selftest
        big = deepseek_v3_spec(2) if args.config.startswith("deepseek-v3") else qwen3_235b_spec(2)
        lay = default_layout(big, world, args.comm)
        layout = args.layout or lay["layout"]
        ok = run_selftest(rank, world, local, layout=layout, groups=(args.attn_groups or (1 if layout == "split" else world)),
                          n_micro=args.n_micro or lay["n_micro"], comm="p2p", experts="nvfp4" if big.quant.experts == "nvfp4" else "mxfp4",
                          model=big.attn.kind, verbose=False)
        selftest = "ok" if ok else "FAILED"
    res = run_decode_bench(args, rank, world, local, ClockSampler(local))
    nccl = None
    if world > 1 and args.comm == "p2p" and not args.no_nccl_baseline:
        # like-for-like baseline row: the same model, batch and context over the NCCL-only path (split layout, eager)
        import copy
        import gc
        import torch
        gc.collect(); torch.cuda.empty_cache()
        a2 = copy.copy(args)
        a2.comm, a2.layout, a2.n_micro, a2.attn_groups = "nccl", "split", 1, 1
        a2.steps, a2.warmup = max(3, min(args.steps, 5)), 3
        a2.batch_total = args.batch_total or args.batch_per_gpu * world
        r2 = run_decode_bench(a2, rank, world, local, ClockSampler(local))
        if rank == 0:
            nccl = {"value": r2["value"], "unit": r2["unit"], "ms_per_step": r2["ms_per_step"], "steps": r2["steps"],
                    "parallelism": r2["config"]["parallelism"], "e2e_value": r2["e2e"]["value"]}
    headline = None
    if world == 8 and args.comm == "p2p" and not args.no_headline and not args.layers and args.config == "qwen3-235b-decode":
        # the DeepSeek-V3-shape configuration (attention TP2 + experts on six GPUs, one-layer MTP drafter) rides along as sub-results
        import gc
        import torch
        gc.collect(); torch.cuda.empty_cache()
        try:
            headline = deepseek_headline(args, rank, world, local)
        except Exception as e:           # the main record must survive a failure of the sub-results
            headline = {"error": f"{type(e).__name__}: {e}"}
        if not args.no_ttft:
            gc.collect(); torch.cuda.empty_cache()
            try:
                import copy
                a3 = copy.copy(args)
                a3.ttft_sessions, a3.ttft_decode = min(args.ttft_sessions, 3), min(args.ttft_decode, 32)    # bounded: 1 cold + 2 restores
                ttft = deepseek_ttft(a3, rank, world, local)
            except Exception as e:
                ttft = {"error": f"{type(e).__name__}: {e}"}
            if rank == 0 and headline is not None:
                headline["ttft_32k"] = ttft
    if rank == 0:
        if headline is not None:
            res["deepseek_v3_headline"] = headline
        res["vs_baseline"] = round(res["value"] / BASELINE_TOKS, 3)
        res["baseline_ref"] = BASELINE_SRC
        res["vs_baseline_comparable"] = False     # a different, smaller model on other hardware: context only, see nccl_baseline
        if selftest is not None:
            res["selftest"] = selftest
        if nccl is not None:
            res["nccl_baseline"] = nccl
            res["vs_nccl_baseline"] = round(res["value"] / nccl["value"], 3) if nccl["value"] else None
        print(json.dumps(res))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
