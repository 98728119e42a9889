"""Multi-GPU self-test (run under torchrun with 2+ ranks): the attention/expert split must generate exactly the
tokens of the single-GPU engine, over the peer-memory kernels and over the NCCL baseline.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m cuteafd_b200.parallel.selftest
"""
from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist

from ..config import QuantSpec, tiny_spec
from ..engine.engine import Engine
from ..engine.generate import BatchGenerator, generate
from ..engine.kv import PagePool
from ..models.weights import DeviceWeights
from .runner import AfdRunner, OP_STOP


def main() -> int:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    experts = os.environ.get("CUTEAFD_SELFTEST_EXPERTS", "nvfp4")
    spec = tiny_spec().replace(quant=QuantSpec(experts=experts, dense="bf16"))
    groups = int(os.environ.get("CUTEAFD_SELFTEST_GROUPS", "1"))
    n_new = 6
    ok = True
    from ..config import default_deployment
    dep = default_deployment(world, groups)
    leaders = [dep.group_ranks(g)[0] for g in range(dep.attn_groups)]
    want = prompts = None
    if rank in leaders:
        # every attention group serves its own prompts; its leader checks them against the single-GPU engine
        g = torch.Generator().manual_seed(3 + dep.group_of(rank))
        prompts = [torch.randint(0, spec.vocab, (24,), generator=g).tolist() for _ in range(2)]
        ref_eng = Engine(DeviceWeights.random(spec, "cuda", seed=1), n_pages=16, max_seqs=4, max_pages_per_seq=4)
        want = generate(ref_eng, prompts, n_new, use_graph=False)
        del ref_eng
    elif rank in dep.attn_ranks:
        g = torch.Generator().manual_seed(3 + dep.group_of(rank))
        prompts = [torch.randint(0, spec.vocab, (24,), generator=g).tolist() for _ in range(2)]
    for comm in (("p2p", "nccl") if groups == 1 else ("p2p",)):
        run = AfdRunner(spec, rank, world, local, t_max=64, n_pages=16, max_seqs=4, max_pages_per_seq=4, comm=comm, seed=1, attn_groups=groups)
        if run.is_attn:
            gen = BatchGenerator(run.engine, PagePool(16))
            out = [[t] for t in gen.prefill(prompts)]
            for _ in range(n_new - 1):
                for o, t in zip(out, gen.decode_step(use_graph=(comm == "p2p" and not os.environ.get("CUTEAFD_SELFTEST_EAGER")))):
                    o.append(t)
            run.control(OP_STOP)
            run.check()
            if rank in leaders:
                same = out == want
                print(f"[selftest] comm={comm} experts={experts} world={world} layout={dep.describe()} rank={rank}: "
                      f"{'OK' if same else 'MISMATCH'} {out} vs {want}", flush=True)
                ok = ok and same
        else:
            run.serve_loop()
            run.check()
        run.close()
        dist.barrier()
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    return 0 if int(flag[0]) else 1


if __name__ == "__main__":
    sys.exit(main())
