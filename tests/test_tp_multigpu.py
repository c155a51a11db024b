"""Tensor-parallel engine on 2+ GPUs (child processes under torch.distributed.run): NCCL baseline and the fused
NVLink kernels against the single-GPU engine."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = Path(__file__).resolve().parent.parent


def _run(kind, world, batch, port, moe=False):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TP_TEST_BATCH=str(batch), TP_TEST_MOE="1" if moe else "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(ROOT / "tests" / "tp_worker.py"), kind]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("TPRESULT") == world, r.stdout[-2000:]   # ranks may interleave their lines


@pytest.mark.parametrize("kind", ["nccl", "fused", "fused_rsag"])
@pytest.mark.parametrize("batch", [1, 5, 16])
def test_tp2_matches_single_gpu(kind, batch):
    _run(kind, 2, batch, 29541)


@pytest.mark.parametrize("kind", ["nccl", "fused", "fused_rsag"])
def test_tp_all_gpus_matches_single_gpu(kind):
    n = torch.cuda.device_count()
    world = 8 if n >= 8 else (4 if n >= 4 else 2)
    if world == 2:
        pytest.skip("covered by the 2-GPU test")
    _run(kind, world, 7, 29543)


@pytest.mark.parametrize("kind", ["nccl", "fused"])
def test_expert_parallel_matches_single_gpu(kind):
    """One expert per rank, attention tensor-parallel; the fused form pushes the gate-scaled expert output into every
    rank's inbox from the GEMM epilogue."""
    n = torch.cuda.device_count()
    world = 8 if n >= 8 else (4 if n >= 4 else 2)
    _run(kind, world, 6, 29545, moe=True)


@pytest.mark.xfail(strict=False, reason="pipeline stages over NCCL point-to-point: not yet run on devices")
def test_pipeline_two_stages_match_single_gpu():
    """Layer pipeline over two GPUs: stage hand-off by NCCL send / recv, rank 0 drives, rank 1 follows."""
    import json
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", POOT_PP_CUDA="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29547", str(ROOT / "tests" / "pp_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    out = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert out["ok"], out


@pytest.mark.xfail(strict=False, reason="tensor-parallel shares of the families beyond the plain layer: not yet run on devices")
def test_tensor_parallel_families_match_single_gpu():
    """Two GPUs over NCCL (library collectives) with the real kernels: the gathered logits of every family equal one
    GPU's within bf16 noise."""
    import json
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    families = ["gemma2", "gemma3", "olmo2", "olmoe", "smollm3-nope-layer", "granite", "mpt", "bloom", "gpt_oss", "minimax_m2"]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", POOT_TP_CUDA="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29549", str(ROOT / "tests" / "tp_family_worker.py"), *families]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=str(ROOT / "tests"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    out = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    for rank_flags in out["ranks"]:
        assert all(ok for ok, _ in rank_flags.values()), out
