"""Stand-ins for a sanitizer: guard words around peer-written communication regions, the checked kernel build that
records out-of-range indices instead of trapping, and the run-twice determinism check."""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from poot_b200.parallel.guarded_layout import ALIGN, GUARD_BYTES, CommBufferOverrun, GuardedLayout


def test_guarded_layout_places_a_guard_right_behind_every_region():
    lay = GuardedLayout([("flags", 128), ("inbox", 2 * 4 * 128 * 4096 * 2), ("xs", 1000), ("ax", 4 * 777)])
    regs = list(lay.regions.values())
    for a, b in zip(regs, regs[1:]):
        assert a.offset % ALIGN == 0 and b.offset % ALIGN == 0
        assert a.offset + a.nbytes <= a.guard_offset < a.guard_offset + GUARD_BYTES <= b.offset
        assert a.guard_offset - (a.offset + a.nbytes) < 4            # no gap an overrun could hide in
    assert lay.total % ALIGN == 0 and lay.total >= regs[-1].guard_offset + GUARD_BYTES
    with pytest.raises(ValueError):
        GuardedLayout([("a", 16), ("a", 16)])
    with pytest.raises(ValueError):
        GuardedLayout([("a", 0)])


def test_guard_check_names_the_overrun_region():
    lay = GuardedLayout([("flags", 128), ("inbox", 4096), ("xs", 1000)])
    mem = np.zeros(lay.total // 4, dtype=np.int32)
    store = lambda off, words: mem.__setitem__(slice(off // 4, off // 4 + len(words)), words)
    load = lambda off, n: mem[off // 4: off // 4 + n].tolist()
    lay.write(3, store)
    lay.check(3, load)                                              # intact
    inbox = lay.regions["inbox"]
    mem[inbox.offset // 4: (inbox.offset + inbox.nbytes) // 4] = -1  # the whole region may be written
    lay.check(3, load)
    mem[(inbox.offset + inbox.nbytes) // 4] = 0x1234                 # one element past its end
    with pytest.raises(CommBufferOverrun) as e:
        lay.check(3, load)
    assert e.value.region == "inbox" and e.value.rank == 3 and e.value.word == 0
    lay.write(3, store)
    lay.check(3, load)
    with pytest.raises(CommBufferOverrun):                           # guards are per rank: another rank's pattern fails
        lay.check(2, load)


def test_checked_library_registers_every_translation_unit():
    from poot_b200 import build
    lib_dir = build.LIB_DIR
    dbg = lib_dir / "libpoot_kernels_dbg.so"
    build.build_kernels_checked()            # rebuilds only what is older than its sources
    checked, release = ctypes.CDLL(str(dbg)), ctypes.CDLL(str(lib_dir / "libpoot_kernels.so"))
    assert checked.poot_debug_bounds_enabled() == 1 and release.poot_debug_bounds_enabled() == 0
    n_units = len(list((build.CSRC / "kernels").glob("*.cu")))
    assert checked.poot_debug_bounds_units() == n_units and release.poot_debug_bounds_units() == 0
    out = (ctypes.c_int * 4)(7, 7, 7, 7)
    assert release.poot_debug_bounds_read(out) == 0 and list(out) == [0, 0, 0, 0]
    assert release.poot_debug_bounds_limit(9, ctypes.c_longlong(1)) != 0        # unknown limit id


def test_loader_picks_the_checked_library_from_the_environment():
    code = ("from poot_b200.ops import cuda_ops as K; print(int(K.bounds_checking()))")
    for flag, want in (("1", "1"), ("0", "0")):
        env = dict(os.environ, POOT_DEBUG_BOUNDS=flag)
        r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=300)
        assert r.returncode == 0 and r.stdout.strip().endswith(want), r.stderr


def test_index_fault_is_a_typed_error():
    from poot_b200.ops import cuda_ops as K
    e = K.DeviceIndexOutOfRange(3, 95, 70000, 4096)
    assert "K/V block id 70000 outside [0, 4096)" in str(e) and e.line == 95


def test_run_twice_accepts_a_deterministic_step_and_names_a_racy_tensor():
    from poot_b200.models.config import DecoderConfig
    from poot_b200.runtime.engine import DecoderEngine, StepShape
    from poot_b200.runtime.session import FixedBatchSession
    from poot_b200.runtime.weights import random_weights
    from poot_b200.utils.determinism import NotDeterministic, diff_report, run_twice
    from poot_b200.utils.kernel_emulation import emulated_kernels
    cfg = DecoderConfig(n_layers=2, hidden=128, n_heads=4, n_kv_heads=2, head_dim=64, ffn=256, vocab=512, max_position=256)
    with emulated_kernels():
        w = random_weights(cfg, "cpu", seed=0, std=0.05)
        eng = DecoderEngine(w, num_blocks=9, max_seqs=2, max_tokens=32, max_blocks_per_seq=4, device="cpu", use_graphs=False)
        sess = FixedBatchSession(eng, 2, 64)
        g = torch.Generator().manual_seed(0)
        sess.prefill_fast(torch.randint(0, cfg.vocab, (2, 9), generator=g, dtype=torch.int32))
        sess._bind_decode_inputs([5, 6])
        shape = StepShape(2, 2, 0)
        eng.bind(sess.h_tokens[:2], sess.h_pos[:2], sess.h_slots[:2], sess.h_seq[:2], sess.h_ctx[:2], sess.h_lidx[:2])
        run_twice(eng, shape, step=lambda: eng.run(shape))
        calls = [0]

        def racy():
            eng.run(shape)
            calls[0] += 1
            eng.logits[0, 17] += 1e-3 * calls[0]         # what a second writer would do

        with pytest.raises(NotDeterministic) as e:
            run_twice(eng, shape, step=racy)
        assert e.value.name == "logits" and e.value.differing == 1 and e.value.first == 17
    a = torch.tensor([1.0, float("nan")])
    assert diff_report("x", a, a.clone()) is None                  # bits, not values: NaN equals itself


@pytest.mark.gpu
def test_checked_build_records_an_out_of_range_token_and_the_context_survives():
    """A child process loads the checked library, feeds one token id beyond the vocabulary to the embedding gather and
    reads the record: site, index and bound; the release behaviour (row 0 substituted) is kept and later work runs."""
    code = r'''
import torch
from poot_b200.ops import cuda_ops as K
assert K.bounds_checking()
table = torch.randn(64, 128, device="cuda").to(torch.bfloat16)
ids = torch.tensor([3, 99, 5], dtype=torch.int32, device="cuda")
out = K.embed_gather(ids, table)
try:
    K.check_bounds()
    raise SystemExit("no fault recorded")
except K.DeviceIndexOutOfRange as e:
    assert (e.site, e.index, e.bound) == (1, 99, 64), (e.site, e.index, e.bound)
assert torch.equal(out[1], table[0]) and torch.equal(out[2], table[5])
K.check_bounds()                                   # the record was cleared
assert torch.equal(K.embed_gather(ids[:1], table)[0], table[3])
K.check_bounds()
print("ok")
'''
    env = dict(os.environ, POOT_DEBUG_BOUNDS="1")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr


@pytest.mark.gpu
def test_decode_step_is_bit_identical_when_run_twice():
    from poot_b200.models.config import DecoderConfig
    from poot_b200.runtime.engine import DecoderEngine, StepShape
    from poot_b200.runtime.session import FixedBatchSession
    from poot_b200.runtime.weights import random_weights
    from poot_b200.utils.determinism import run_twice
    cfg = DecoderConfig(n_layers=2, hidden=1024, n_heads=8, n_kv_heads=2, head_dim=128, ffn=2048, vocab=4096, max_position=512)
    w = random_weights(cfg, "cuda", seed=0, std=0.05)
    eng = DecoderEngine(w, num_blocks=64, max_seqs=4, max_tokens=128, max_blocks_per_seq=8, device="cuda", use_graphs=False)
    sess = FixedBatchSession(eng, 4, 128)
    g = torch.Generator().manual_seed(0)
    sess.prefill_fast(torch.randint(0, cfg.vocab, (4, 40), generator=g, dtype=torch.int32))
    sess._bind_decode_inputs([5, 6, 7, 8])
    shape = StepShape(4, 4, 0)
    eng.bind(sess.h_tokens[:4], sess.h_pos[:4], sess.h_slots[:4], sess.h_seq[:4], sess.h_ctx[:4], sess.h_lidx[:4])
    run_twice(eng, shape, step=lambda: eng.run(shape))
