"""Shared runtime pieces: the upload ring's policy and the memory counters by buffer role."""
import numpy as np
import pytest
import torch


def test_upload_ring_policy():
    from poot_b200.ops._lib import kernels
    from poot_b200.runtime.upload import CHUNK_BYTES, slot_bytes, upload
    from ctypes import c_ulonglong
    assert slot_bytes(1) == 64 << 10 and slot_bytes((64 << 10) + 1) == 128 << 10 and slot_bytes(1 << 40) == CHUNK_BYTES
    lib = kernels()
    lib.poot_ring_chunk_count.argtypes, lib.poot_ring_chunk_count.restype = [c_ulonglong, c_ulonglong], c_ulonglong
    assert lib.poot_ring_chunk_count(0, CHUNK_BYTES) == 0 and lib.poot_ring_chunk_count(CHUNK_BYTES, CHUNK_BYTES) == 1
    assert lib.poot_ring_chunk_count(CHUNK_BYTES + 1, CHUNK_BYTES) == 2
    a = np.arange(12, dtype=np.uint16).reshape(3, 4)
    t = upload(a, "cpu", torch.bfloat16)                       # no device: a plain copy with the same view rule
    assert t.dtype == torch.bfloat16 and tuple(t.shape) == (3, 4) and t.view(torch.int16)[2, 3].item() == 11


def test_memory_counters_by_role_on_the_emulated_engine():
    from poot_b200.models.config import DecoderConfig
    from poot_b200.profile.memory import MemoryCounters, account
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.weights import random_weights
    from poot_b200.utils.kernel_emulation import emulated_kernels
    cfg = DecoderConfig(n_layers=2, hidden=128, n_heads=4, n_kv_heads=2, head_dim=32, ffn=256, vocab=512, max_position=128)
    with emulated_kernels():
        w = random_weights(cfg, "cpu", seed=0)
        eng = DecoderEngine(w, num_blocks=8, max_seqs=2, max_tokens=32, max_blocks_per_seq=4, device="cpu", use_graphs=False)
        m = account(eng)
    b = m.bytes_by_role
    assert b["weight"] == w.nbytes()
    assert b["state"] == eng.kv.buf.numel() * eng.kv.buf.element_size()
    assert b["activation"] > 0 and b["input"] > 0 and b["output"] >= eng.logits.numel() * 4 and b["staging"] == 0
    c = m.classes()
    assert c["weights_bytes"] == b["weight"] and c["kv_bytes"] == b["state"] and sum(c.values()) == m.total
    again = MemoryCounters()
    again.add("weight", [w.embed, w.embed, w.lm_head])           # shared storage is counted once
    tied = w.lm_head is w.embed
    assert again.bytes_by_role["weight"] == (1 if tied else 2) * w.embed.numel() * 2
    with pytest.raises(ValueError):
        again.add("cache", [w.embed])


@pytest.mark.gpu
def test_upload_ring_moves_bytes_in_chunks():
    from poot_b200.runtime.upload import UploadRing
    ring = UploadRing(slot_hint=1 << 20)
    src = np.random.default_rng(0).integers(0, 255, (5 << 20) + 123, dtype=np.uint8)
    dst = torch.zeros(src.size, dtype=torch.uint8, device="cuda")
    ring.upload(src, dst)
    ring.drain()
    assert torch.equal(dst.cpu(), torch.from_numpy(src))
    st = ring.stats()
    assert st["bytes"] == src.size and st["chunks"] == 6 and st["slot_bytes"] == 1 << 20
    ring.close()
