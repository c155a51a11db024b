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


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_ranks_over_the_library_collectives_match_one_process(world):
    """Ranks over gloo with emulated kernels: Megatron shares, all-reduce after the row-parallel projections,
    expert-parallel MoE with two experts per rank (each rank groups only its own experts' rows), vocabulary-parallel
    head with the greedy pick merged from per-shard partial tables."""
    worker = os.path.join(os.path.dirname(__file__), "tp_cpu_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29700 + world + os.getpid() % 200), worker]
    r = subprocess.run(cmd, env=dict(os.environ, OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES=""), capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    out = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert out["ok"], out


def test_tensor_parallel_shares_of_the_model_families_match_one_process():
    """Families beyond the plain layer under two ranks (gloo, emulated kernels, library collectives): biases joining a
    reduced sum once, norms behind a row-parallel projection, a norm spanning every rank's heads, ALiBi slopes and sink
    logits per rank's heads, LayerNorm stacks, routed experts replicated beside sharded attention."""
    worker = os.path.join(os.path.dirname(__file__), "tp_family_worker.py")
    families = ["gemma2", "gemma3", "olmo2", "olmoe", "smollm3-nope-layer", "granite", "mpt", "bloom", "gpt_oss", "minimax_m2"]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29900 + os.getpid() % 90), worker, *families]
    r = subprocess.run(cmd, env=dict(os.environ, OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES=""), capture_output=True,
                       text=True, timeout=900, cwd=os.path.dirname(__file__))
    assert r.returncode == 0, r.stderr[-3000:]
    out = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    for rank_flags in out["ranks"]:
        assert all(ok for ok, _ in rank_flags.values()), out
    assert sorted(k for k in out if k != "ranks") == sorted(families)


def test_families_without_a_sharding_rule_refuse_tensor_parallelism():
    import torch
    from poot_b200.models.registry import Registry
    from poot_b200.oracle.runner import random_weights_f32
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.weights import UnsupportedOnDevice, from_named_tensors
    from poot_b200.utils.kernel_emulation import emulated_kernels
    from test_engine_emulated import HF_BASE, HF_FAMILIES

    class Comm:                      # stands for a process group: the refusal comes before any collective
        fused = False
    model = Registry.builtin().resolve_hf({**HF_BASE, **HF_FAMILIES["deepseek2"]})
    named = {k: torch.from_numpy(v) for k, v in random_weights_f32(model, seed=0).items()}
    cfg = model.cfg
    for l in [l for l in range(cfg.n_layers) if cfg.moe_layer(l)]:
        for e in range(cfg.n_experts):
            named[f"layers.{l}.experts.{e}.gate"] = named[f"layers.{l}.experts_in"][e, :cfg.moe_ffn]
            named[f"layers.{l}.experts.{e}.up"] = named[f"layers.{l}.experts_in"][e, cfg.moe_ffn:]
            named[f"layers.{l}.experts.{e}.down"] = named[f"layers.{l}.experts_out"][e]
    with emulated_kernels():
        w = from_named_tensors(cfg, named, "cpu")
        with pytest.raises(UnsupportedOnDevice, match="no sharding rule"):
            DecoderEngine(w, num_blocks=4, max_seqs=1, max_tokens=32, max_blocks_per_seq=2, comm=Comm(), device="cpu", use_graphs=False)
        Comm.fused = True
        with pytest.raises(UnsupportedOnDevice, match="fused tensor-parallel programs"):
            DecoderEngine(w, num_blocks=4, max_seqs=1, max_tokens=32, max_blocks_per_seq=2, comm=Comm(), device="cpu", use_graphs=False)
