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
