"""Layer-pipeline placement as separate processes (gloo, CPU): each rank loads only its stage's layers, rank 0 drives,
the other ranks follow its step announcements; generation equals the single-process model."""
import json
import os
import subprocess
import sys

import pytest


@pytest.mark.parametrize("world", [2, 3])
def test_pipeline_ranks_generate_what_one_process_generates(world):
    worker = os.path.join(os.path.dirname(__file__), "pp_worker.py")
    port = 29600 + world + (os.getpid() % 200)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), worker]
    env = dict(os.environ, OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    assert out["ok"], out
    assert out["sent_bytes"] > 0


def test_tensor_parallel_ranks_over_the_library_collectives_match_one_process():
    """Two ranks over gloo with emulated kernels: Megatron shares, all-reduce after the row-parallel projections,
    expert-parallel MoE, vocabulary-parallel head with the greedy pick merged from per-shard partial tables."""
    worker = os.path.join(os.path.dirname(__file__), "tp_cpu_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29700 + os.getpid() % 200), worker]
    r = subprocess.run(cmd, env=dict(os.environ, OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES=""), capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    out = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert out["ok"], out
