"""Every typed error of the package is reached by a test that names it (the guard in ``test_repo_guards.py`` checks the
naming); this file holds the ones no other test touches."""
import socket
import threading

import numpy as np
import pytest
import torch


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_control_plane_reports_a_failed_rank_and_a_lost_leader():
    from poot_b200.serve.control import ControlPlane, LeaderLost, RankFailed
    port = _free_port()
    leader = ControlPlane(0, 2, port=port, ready_deadline=5, step_deadline=5, heartbeat=0.05, heartbeat_timeout=0.4)
    follower = ControlPlane(1, 2, port=port, heartbeat=0.05, heartbeat_timeout=0.4)
    leader.start_heartbeat()
    follower.start_heartbeat()
    n = leader.announce({"tokens": [1, 2, 3]})
    kind, payload = follower.next_step()
    assert kind == "step" and payload == {"tokens": [1, 2, 3]}
    follower.ready(n)
    leader.wait_ready(n)
    follower.ack(n, "DeviceWaitTimeout: peer flag of rank 0 never arrived")
    with pytest.raises(RankFailed) as e:
        leader.wait_acks(n)
    assert e.value.rank == 1 and e.value.step == n and "peer flag" in e.value.report
    leader._hb_paused = True                       # rank 0 stops answering without saying so
    with pytest.raises(LeaderLost):
        follower.next_step()
    follower.close()
    leader.close()


def test_sampler_fault_fails_one_sequence():
    from poot_b200.driver.driver import Driver, SamplerFault
    from poot_b200.driver.engines import FakeStepEngine
    from poot_b200.driver.sampler import SamplingParams

    class NonFinite(FakeStepEngine):
        def run_step(self, inp):
            picked, lp = super().run_step(inp)
            picked[0, 1] = 17                       # index of a non-finite logit in the first sampling row
            return picked, lp

    d = Driver(NonFinite(100, 40), 32, 2, 64, 100, prefill_chunk=16)
    sid = d.open([1, 2, 3], SamplingParams(max_tokens=4))
    with pytest.raises(SamplerFault) as e:
        d.step([sid])
    assert e.value.seq_id == sid and e.value.index == 17


def test_native_library_errors():
    from poot_b200.ops import _lib
    with pytest.raises(_lib.KernelError) as e:
        _lib.check(700, "gemm")                     # a launcher's non-zero return code
    assert "gemm" in str(e.value) and "700" in str(e.value)
    _lib.check(0, "gemm")
    with pytest.raises(_lib.NativeLibraryMissing):
        _lib._load("libpoot_nothing.so", "no_such_builder")


def test_graph_and_trace_errors():
    from poot_b200.ir.builder import Builder, TraceBudgetExceeded, TraceLimits
    from poot_b200.ir.graph import GraphError
    from poot_b200.tensor import DType
    b = Builder()
    x = b.slot("x", (2, 3), DType.F32, "activation")
    with pytest.raises(GraphError):
        b.reshape(x, (4, 2))                        # element count changes
    with pytest.raises(GraphError):
        b.slot("x", (2, 3), DType.F32, "activation")          # duplicate input
    small = Builder(limits=TraceLimits(max_equations=3))
    y = small.slot("y", (2,), DType.F32, "activation")
    with pytest.raises(TraceBudgetExceeded):
        for _ in range(8):
            y = y + y


def test_eval_errors_name_the_input():
    from poot_b200.ir.builder import Builder
    from poot_b200.oracle.eval import EvalError, eval_graph
    from poot_b200.tensor import DType
    b = Builder()
    t = b.slot("tokens", (4,), DType.I32, "token", range=(0, 9))
    b.output(t + t, "twice", "result")
    g = b.finish()
    with pytest.raises(EvalError, match="missing input"):
        eval_graph(g, {})
    with pytest.raises(EvalError, match="shape"):
        eval_graph(g, {"tokens": np.zeros(5, np.int32)})
    with pytest.raises(EvalError, match="declared range"):
        eval_graph(g, {"tokens": np.array([0, 1, 2, 10], np.int32)})


def test_checkpoint_layout_and_lowering_refusals():
    from poot_b200.load.hf_map import CheckpointLayout, first_axis
    from poot_b200.plan.lower import LoweringRefused, lower
    from poot_b200.quant.weights import PackedWeight
    planar = PackedWeight("experts", "E4M3_CHANNEL", (4, 8, 16), np.zeros(0, np.uint8),
                          planar={"weight": np.zeros((4, 8, 16), np.uint8), "weight_scale": np.ones(32, np.float32)})
    with pytest.raises(CheckpointLayout):
        first_axis(planar, 1)
    from poot_b200.models.config import DecoderConfig
    from poot_b200.models.model import Model, StepSpec
    from poot_b200.plan.compile import compile_graph
    cfg = DecoderConfig(n_layers=2, hidden=128, n_heads=4, n_kv_heads=2, head_dim=32, ffn=256, vocab=320, max_position=128,
                        layer_kinds=["gdn", "attention"], gdn_k_heads=2, gdn_v_heads=4, gdn_head_dim=64, gdn_conv=4)
    prog = compile_graph(Model(cfg).trace(StepSpec(rows=1, tokens=1, capacity=32, paged=True, pool_slots=64)))
    with pytest.raises(LoweringRefused):             # a recurrent layer's equations have no launcher in the plan walker
        lower(prog)


def test_lora_bank_and_embedder_errors(tmp_path):
    from poot_b200.embed import EmbedError, Embedder
    from poot_b200.runtime.lora_bank import LoraBankError
    from poot_b200.models.config import DecoderConfig
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.weights import random_weights
    from poot_b200.utils.kernel_emulation import emulated_kernels
    cfg = DecoderConfig(n_layers=1, hidden=128, n_heads=4, n_kv_heads=2, head_dim=32, ffn=256, vocab=320, max_position=128)
    with emulated_kernels():
        eng = DecoderEngine(random_weights(cfg, "cpu"), num_blocks=4, max_seqs=2, max_tokens=16, max_blocks_per_seq=2,
                            device="cpu", use_graphs=False)
        eng.enable_adapters(2, 8)
        with pytest.raises(LoraBankError):
            eng.lora.slot_of("no-such-adapter")
    with pytest.raises(EmbedError):
        Embedder.load(str(tmp_path), backend="tpu")


def test_base_classes_catch_their_families():
    from poot_b200.driver.expert_residency import ExpertIdOutOfRange, PoolTooSmall, ResidencyError
    from poot_b200.runtime.lifecycle import ExecError, Fault, NeedsReset, Poisoned, Validation
    from poot_b200.parallel.symm import PeerLinkError
    assert issubclass(PoolTooSmall, ResidencyError) and issubclass(ExpertIdOutOfRange, ResidencyError)
    assert all(issubclass(c, ExecError) for c in (Fault, NeedsReset, Poisoned, Validation))
    assert issubclass(PeerLinkError, RuntimeError) and "did not arrive" in str(PeerLinkError("rank 1: 3 words did not arrive"))
