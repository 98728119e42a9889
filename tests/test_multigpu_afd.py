"""Multi-GPU runs of the attention/expert layouts (child processes under torchrun): tokens must equal the single-GPU
engine's.  The same layouts also run on one GPU in `test_gpu_afd_local.py`; these cases add real NVLink peers."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _selftest(nproc, port, **env):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} CUDA devices")
    e = dict(os.environ, NCCL_NVLS_ENABLE="0", **{f"CUTEAFD_SELFTEST_{k.upper()}": str(v) for k, v in env.items()})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), "-m", "cuteafd_b200.parallel.selftest"]
    r = subprocess.run(cmd, cwd=ROOT, env=e, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "MISMATCH" not in r.stdout
    return r.stdout


@pytest.mark.parametrize("experts", ["nvfp4", "bf16"])
def test_afd_two_ranks_match_single_gpu(experts):
    """1 attention + 1 expert rank, over the peer-memory kernels and over the NCCL-only baseline."""
    out = _selftest(2, 29541, experts=experts)
    assert out.count("OK") >= 2


def test_colocated_two_ranks_match_single_gpu():
    assert _selftest(2, 29542, layout="colocated").count("OK") >= 2


def test_mla_two_ranks_match_single_gpu():
    _selftest(2, 29546, model="mla", experts="mxfp4")


def test_afd_two_attention_groups_match_single_gpu():
    """4 ranks: two data-parallel attention groups (TP1 each) share two expert ranks."""
    assert _selftest(4, 29543, groups=2).count("OK") >= 2


def test_tp2_with_two_micro_batches_matches_single_gpu():
    """4 ranks: attention TP2 + EP2, two micro-batches in flight per step (GQA and MLA attention)."""
    _selftest(4, 29544, micro=2)
    _selftest(4, 29547, micro=2, model="mla", experts="mxfp4")


def test_colocated_four_ranks_match_single_gpu():
    assert _selftest(4, 29545, layout="colocated").count("OK") >= 4


def _serve_selftest(nproc, port, **env):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} CUDA devices")
    e = dict(os.environ, NCCL_NVLS_ENABLE="0", **{f"CUTEAFD_SERVE_{k.upper()}": str(v) for k, v in env.items()})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), "-m", "cuteafd_b200.serving.split_selftest"]
    r = subprocess.run(cmd, cwd=ROOT, env=e, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "[serve-selftest]" in r.stdout and "MISMATCH" not in r.stdout
    return r.stdout


def test_serving_on_the_split_two_ranks():
    """Scheduler + prefix cache + n-gram drafter over 1 attention + 1 expert rank: a prefix-restored request, a cold one, drafted
    and undrafted decoding all give the single-GPU tokens."""
    _serve_selftest(2, 29551)


def test_serving_on_the_split_tp2_mirrors_the_leader():
    """4 ranks: attention TP2 (the partner mirrors the leader's inputs and steps through the mailbox) + EP2, two micro-batches."""
    _serve_selftest(4, 29552, micro=2)
