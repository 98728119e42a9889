"""Layer-range split over real GPUs: one process per stage, hops over CUDA-IPC peer memory, token broadcast through NCCL."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

WORKER = r'''
import dataclasses, os, sys, torch, torch.distributed as dist
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
from cuteafd_b200.config import tiny_spec
from cuteafd_b200.parallel.pipeline import PipelineRank, generate_pipeline
from cuteafd_b200.parallel.selftest import reference_tokens, tokens_agree
from cuteafd_b200.ref.model import init_weights
base = tiny_spec()
spec = base.replace(n_layers=4)
masters = init_weights(spec, 7)
g = torch.Generator().manual_seed(2)
prompts = [torch.randint(0, spec.vocab, (n,), generator=g).tolist() for n in (19, 33, 7)]
dev = torch.device("cuda", rank)
want, top2 = reference_tokens(spec, masters, prompts, 8, dev)
pr = PipelineRank(spec, rank, world, dev, n_pages=32, max_seqs=8, max_pages_per_seq=4, t_cap=256, masters=masters)
got = generate_pipeline([pr], prompts, 8)
ok = tokens_agree(got, want, top2, exact=False)
flag = torch.tensor([1 if ok else 0], device=dev)
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
if rank == 0:
    print("PIPELINE_OK" if int(flag) else f"PIPELINE_MISMATCH {got} {want}", flush=True)
dist.barrier()
pr.block.close()
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_stage_split_over_two_gpus(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29631",
           str(script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "PIPELINE_OK" in r.stdout, r.stdout[-3000:]
