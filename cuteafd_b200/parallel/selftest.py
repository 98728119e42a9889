"""Multi-GPU self-test (run under torchrun with 2+ ranks): every layout of the attention/expert split must generate exactly
the tokens of the single-GPU engine, over the peer-memory kernels and over the NCCL baseline.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m cuteafd_b200.parallel.selftest
    CUTEAFD_SELFTEST_LAYOUT=colocated|split  CUTEAFD_SELFTEST_GROUPS=n  CUTEAFD_SELFTEST_MICRO=n  CUTEAFD_SELFTEST_MODEL=gqa|mla

`run_selftest` is also what `bench.py` runs on the tiny model before its timed region at N > 1, so every multi-GPU record
carries a token-exactness check of the layout it timed.
"""
from __future__ import annotations

import dataclasses
import os
import sys

import torch
import torch.distributed as dist

from ..config import AttentionSpec, QuantSpec, deployment_by_name, tiny_spec
from ..engine.generate import BatchGenerator, generate
from ..engine.kv import PagePool
from .runner import AfdRunner, OP_STOP


def selftest_spec(model: str, experts: str):
    base = tiny_spec()
    if model == "mla":
        return base.replace(attn=AttentionSpec(kind="mla", n_heads=8, n_kv_heads=8, head_dim=192, q_lora_rank=64, kv_lora_rank=512,
                                               qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128),
                            moe=dataclasses.replace(base.moe, first_dense=1, dense_intermediate=256),
                            quant=QuantSpec(experts=experts, dense="bf16"))
    return base.replace(quant=QuantSpec(experts=experts, dense="bf16"))


def reference_tokens(spec, masters, prompts, n_new, device):
    """Greedy tokens of the single-GPU engine plus, per prompt and step, its two best tokens and the logit margin between them
    (a layout that sums tensor-parallel partials rounds differently and may legitimately flip a near tie)."""
    from ..models.weights import DeviceWeights
    if spec.attn.kind == "mla":
        from ..engine.mla import MlaEngine, mla_weights_from_masters
        eng = MlaEngine(mla_weights_from_masters(spec, masters, device), n_pages=32, max_seqs=8, max_pages_per_seq=4)
    else:
        from ..engine.engine import Engine
        eng = Engine(DeviceWeights.from_masters(spec, masters, device), n_pages=32, max_seqs=8, max_pages_per_seq=4)
    gen = BatchGenerator(eng)
    n = len(prompts)
    out, top2 = [[] for _ in prompts], [[] for _ in prompts]

    def record(toks):
        lane = eng.lane(sum(len(p) for p in prompts)) if not out[0] else eng.lane(n)
        best = lane.logits[:n].float().topk(2, dim=-1)
        for i, t in enumerate(toks):
            out[i].append(t)
            top2[i].append((best.indices[i].tolist(), float(best.values[i, 0] - best.values[i, 1])))
    record(gen.prefill(prompts))
    for _ in range(n_new - 1):
        record(gen.decode_step(use_graph=False))
    eng.check_status()
    gen.release()
    return out, top2


def tokens_agree(got, want, top2, exact: bool, margin: float = 0.05) -> bool:
    """Every prompt's tokens equal the reference's; unless `exact`, the first difference of a prompt may be a flipped near tie
    (the reference's second choice, less than `margin` behind its first), after which that prompt is no longer compared."""
    for g, w, t2 in zip(got, want, top2):
        if len(g) != len(w):
            return False
        for j, (a, b) in enumerate(zip(g, w)):
            if a != b:
                if exact or a != t2[j][0][1] or t2[j][1] > margin:
                    return False
                break
    return True


def run_selftest(rank: int, world: int, local: int, *, layout: str = "split", groups: int = 1, n_micro: int = 1, comm: str = "p2p",
                 experts: str = "nvfp4", model: str = "gqa", n_new: int = 6, use_graph: bool = True, verbose: bool = True) -> bool:
    """One layout, one transport: True when every attention group generated the single-GPU engine's tokens (agreed over all
    ranks).  Needs an initialised NCCL process group."""
    from ..ref.model import init_weights
    spec = selftest_spec(model, experts)
    masters = init_weights(spec, 5)
    dep = deployment_by_name(layout, world, groups)
    dev = torch.device("cuda", local)
    ok = True
    want = prompts = top2 = None
    if rank in dep.attn_ranks:
        grp = dep.group_of(rank)
        g = torch.Generator().manual_seed(3 + grp)
        prompts = [torch.randint(0, spec.vocab, (24,), generator=g).tolist() for _ in range(4)]
        if rank == dep.group_ranks(grp)[0]:
            want, top2 = reference_tokens(spec, masters, prompts, n_new, dev)
    run = AfdRunner(spec, rank, world, local, t_cap=128, n_pages=32, max_seqs=8, max_pages_per_seq=4, comm=comm, layout=layout,
                    attn_groups=dep.attn_groups, n_micro=n_micro, masters=masters)
    if run.is_attn:
        gen = BatchGenerator(run.engine, PagePool(32))
        out = [[t] for t in gen.prefill(prompts)]
        for _ in range(n_new - 1):
            for o, t in zip(out, gen.decode_step(use_graph=use_graph and comm == "p2p")):
                o.append(t)
        run.control(OP_STOP)
        run.check()
        if want is not None:
            # heads split over two ranks sum two bf16-rounded partial projections: a near tie of the reference may flip there;
            # every other layout computes exactly what the single-GPU engine computes
            ok = tokens_agree(out, want, top2, exact=dep.tp == 1)
            if verbose:
                print(f"[selftest] model={model} comm={comm} experts={experts} world={world} layout={dep.describe()} micro={n_micro} "
                      f"rank={rank}: {'OK' if ok else 'MISMATCH'} {out if not ok else ''} {want if not ok else ''}", flush=True)
    else:
        run.serve_loop()
        run.check()
    run.close()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(int(flag[0]))


def main() -> int:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    experts = os.environ.get("CUTEAFD_SELFTEST_EXPERTS", "nvfp4")
    layout = os.environ.get("CUTEAFD_SELFTEST_LAYOUT", "split")
    groups = int(os.environ.get("CUTEAFD_SELFTEST_GROUPS", "1"))
    n_micro = int(os.environ.get("CUTEAFD_SELFTEST_MICRO", "1"))
    model = os.environ.get("CUTEAFD_SELFTEST_MODEL", "gqa")
    eager = bool(os.environ.get("CUTEAFD_SELFTEST_EAGER"))
    ok = True
    comms = ("p2p", "nccl") if (layout == "split" and groups == 1 and n_micro == 1) else ("p2p",)
    for comm in comms:
        ok = run_selftest(rank, world, local, layout=layout, groups=groups, n_micro=n_micro, comm=comm, experts=experts, model=model,
                          use_graph=not eager) and ok
        dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
