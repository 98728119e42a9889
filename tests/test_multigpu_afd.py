"""2-GPU run of the attention/expert split (child processes under torchrun): tokens must equal the single-GPU engine."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("experts", ["nvfp4", "bf16"])
def test_afd_two_ranks_match_single_gpu(experts):
    env = dict(os.environ, CUTEAFD_SELFTEST_EXPERTS=experts, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29541", "-m", "cuteafd_b200.parallel.selftest"]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "MISMATCH" not in r.stdout


def test_afd_two_attention_groups_match_single_gpu():
    """4 ranks: two data-parallel attention groups (TP1 each) share two expert ranks; every group's tokens must equal
    the single-GPU engine's for its own prompts."""
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 CUDA devices")
    env = dict(os.environ, CUTEAFD_SELFTEST_EXPERTS="nvfp4", CUTEAFD_SELFTEST_GROUPS="2", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1",
           "--master-port", "29543", "-m", "cuteafd_b200.parallel.selftest"]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "MISMATCH" not in r.stdout and r.stdout.count("OK") >= 2
