"""Serving self-test on a multi-GPU layout (run under torchrun with 2+ ranks): the scheduler, prefix cache and n-gram drafter
run on the attention leader over the attention/expert split, and must produce byte-identical tokens

  * for a prefix-restored request and a cold one (exact prefix cache on the split),
  * for drafted and undrafted decoding (lossless speculation on the split),
  * and the tokens of plain single-GPU generation of the same model.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m cuteafd_b200.serving.split_selftest
"""
from __future__ import annotations

import argparse
import os
import sys

import torch


def main() -> int:
    import torch.distributed as dist
    from ..cli import build_serving
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    a = argparse.Namespace(model="tiny", device=local, layers=0, pool_tokens=64 * 64, max_sequences=4, max_context=1024, prefill_batch_tokens=64,
                           host_cache_gib=0.0, host_cache_headroom_gib=0.0, host_cache_min_tokens=512, prefix_cache_entries=8,
                           prefix_cache_min_tokens=64, draft=os.environ.get("CUTEAFD_SERVE_DRAFT", "ngram"), decode_share=0.2, draft_limit=3,
                           http_queue=16, queue_wait_s=0, n_micro=int(os.environ.get("CUTEAFD_SERVE_MICRO", "0")))
    built = build_serving(a)
    if built is None:
        dist.destroy_process_group()
        return 0
    spec, sched = built
    from ..serving.scheduler import Request
    g = torch.Generator().manual_seed(9)
    shared = torch.randint(0, spec.vocab, (150,), generator=g).tolist()
    # a repetitive tail makes the n-gram drafter propose (and sometimes be right)
    tail = [5, 6, 7, 8] * 6
    prompts = [shared + tail + [11], shared + tail + [11], shared + [3, 4, 5]]
    outs = []

    def ask(tag, prompt, n_new, cache=True):
        toks = []
        sched.submit(Request(tag, list(prompt), max_tokens=n_new, on_token=lambda new, done, reason: toks.extend(new), use_cache=cache))
        sched.run_until_idle()
        return toks
    cold = ask("cold", prompts[0], 12)
    hits0 = sched.prefix.stats["hit_tokens"]
    warm = ask("warm", prompts[1], 12)              # same prompt: the shared pages come back from the prefix cache
    hit = sched.prefix.stats["hit_tokens"] - hits0
    other = ask("other", prompts[2], 8)
    drafted = sched.stats["drafted"]
    sched.drafter = None
    plain = ask("plain", prompts[0], 12, cache=False)   # no cache, no drafts
    other_plain = ask("other-plain", prompts[2], 8, cache=False)
    # single-GPU reference on this rank's GPU
    from ..engine.engine import Engine
    from ..engine.generate import generate
    from ..models.weights import DeviceWeights
    from ..ref.model import init_weights
    ref = Engine(DeviceWeights.from_masters(spec, init_weights(spec, 0), torch.device("cuda", local)), n_pages=64, max_seqs=4, max_pages_per_seq=16)
    want = generate(ref, [prompts[0], prompts[2]], 12, use_graph=False)
    ok = cold == warm == plain == want[0] and other == other_plain == want[1][:8] and hit >= 128 and len(cold) == 12
    print(f"[serve-selftest] world={world} layout={sched.afd_runner.dep.describe()} prefix_hit_tokens={hit} drafted={drafted} "
          f"{'OK' if ok else 'MISMATCH'} cold={cold} warm={warm} plain={plain} want={want[0]} other={other} other_plain={other_plain} want1={want[1][:8]}",
          flush=True)
    sched.afd_runner.shutdown()                      # OP_STOP: followers and expert ranks leave their loops
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
