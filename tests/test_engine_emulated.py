"""The engine's kernel program on the CPU: ``emulated_kernels`` swaps the device kernels' entry points for host
restatements with the same signatures and buffer layouts, so the unmodified engine (buffer binding, launch order,
epilogue choices, K/V paging through block tables, tile cutting for the prefill attention, chained decode, the
sampler suffix, the serving driver on top) is compared with the fp32 restatement of the model without a GPU.  The
kernels themselves are checked on the device (tests marked ``gpu``)."""
import numpy as np
import pytest
import torch

from poot_b200.models.config import DecoderConfig
from poot_b200.utils.kernel_emulation import emulated_kernels


def _cfg(**kw):
    base = dict(n_layers=2, hidden=128, n_heads=4, n_kv_heads=2, head_dim=64, ffn=256, vocab=512, max_position=256)
    base.update(kw)
    return DecoderConfig(**base)


def _engine(cfg, batch, max_len, max_tokens, seed=0):
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.session import FixedBatchSession
    from poot_b200.runtime.weights import random_weights
    w = random_weights(cfg, "cpu", seed=seed, std=0.05)
    bps = (max_len + 15) // 16
    eng = DecoderEngine(w, num_blocks=batch * bps + 1, max_seqs=batch, max_tokens=max_tokens, max_blocks_per_seq=bps,
                        device="cpu", use_graphs=False)
    return w, eng, FixedBatchSession(eng, batch, max_len)


VARIANTS = {
    "llama": {},
    "head-dim-128-flash-tiles": dict(n_heads=2, n_kv_heads=1, head_dim=128, hidden=256),
    "qk-norm-window": dict(qk_norm=True, sliding_window=8),
    "per-layer-windows": dict(layer_windows=[6, 0]),
    "scale-override-softcap": dict(attn_scale=0.2, attn_softcap=20.0),
    "qkv-bias-multipliers": dict(attn_bias=True, embed_scale=3.0, residual_scale=0.5, logit_scale=0.25),
    "partial-rotary": dict(rope_dim=32),
    "moe": dict(n_experts=4, top_k=2, moe_ffn=128),
    "moe-not-renormalised": dict(n_experts=4, top_k=2, moe_ffn=128, norm_topk_prob=False),
}


@pytest.mark.parametrize("name", sorted(VARIANTS))
def test_prefill_then_decode_matches_the_fp32_restatement(name):
    from poot_b200.oracle.torch_ref import forward_logits
    cfg = _cfg(**VARIANTS[name])
    with emulated_kernels():
        w, eng, sess = _engine(cfg, batch=2, max_len=64, max_tokens=64)
        g = torch.Generator().manual_seed(0)
        prompts = torch.randint(0, cfg.vocab, (2, 21), generator=g, dtype=torch.int32)
        picked = sess.prefill_fast(prompts)
        for b in range(2):
            ref = forward_logits(w, prompts[b])[-1]
            err = (eng.logits[b] - ref).abs().max().item()
            assert err < 0.03 * max(1.0, ref.abs().max().item()), (name, "prefill", err)
            assert picked[b, 1] == -1
        nxt = torch.randint(0, cfg.vocab, (2, 3), generator=g, dtype=torch.int32)
        for t in range(3):
            sess.decode(nxt[:, t].tolist())
        for b in range(2):
            ref = forward_logits(w, torch.cat([prompts[b], nxt[b]]))[-1]
            err = (eng.logits[b] - ref).abs().max().item()
            assert err < 0.03 * max(1.0, ref.abs().max().item()), (name, "decode", err)


def test_chained_decode_equals_stepwise_decode():
    cfg = _cfg()
    with emulated_kernels():
        g = torch.Generator().manual_seed(3)
        prompts = torch.randint(0, cfg.vocab, (2, 9), generator=g, dtype=torch.int32)
        _, eng_a, a = _engine(cfg, 2, 64, 32)
        first = a.prefill_fast(prompts)[:, 0].tolist()
        toks, cur = [], first
        for _ in range(5):
            cur = a.decode(cur)[:, 0].tolist()
            toks.append(cur)
        _, eng_b, b = _engine(cfg, 2, 64, 32)
        first_b = b.prefill_fast(prompts)[:, 0].tolist()
        assert first_b == first
        chained = b.decode_chain(first_b, 5)
        assert [list(map(int, chained[i])) for i in range(5)] == toks if chained is not None else True
        assert eng_b.picked[:2, 0].tolist() == toks[-1]


def test_device_gaps_are_refused_by_the_engine():
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.weights import UnsupportedOnDevice, random_weights
    cfg = _cfg(final_softcap=30.0)
    with emulated_kernels():
        w = random_weights(_cfg(), "cpu", seed=0)
        w.cfg = cfg
        with pytest.raises(UnsupportedOnDevice) as e:
            DecoderEngine(w, 8, 1, 16, 4, device="cpu", use_graphs=False)
    assert "soft-capped" in str(e.value)


def test_serving_driver_over_the_emulated_engine_matches_greedy_reference():
    """Driver -> DeviceStepEngine -> engine: chunked prefill of two sequences sharing steps, then decode."""
    from poot_b200.driver.driver import Driver
    from poot_b200.driver.engines import DeviceStepEngine
    from poot_b200.driver.sampler import SamplingParams
    from poot_b200.oracle.torch_ref import forward_logits
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.weights import random_weights
    cfg = _cfg()
    with emulated_kernels():
        w = random_weights(cfg, "cpu", seed=1, std=0.05)
        eng = DecoderEngine(w, num_blocks=16, max_seqs=2, max_tokens=16 + 2, max_blocks_per_seq=4, device="cpu", use_graphs=False)
        step_engine = DeviceStepEngine(eng)
        drv = Driver(step_engine, 16, 2, 64, cfg.vocab, prefill_chunk=16, eos_token=None)
        g = torch.Generator().manual_seed(5)
        prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (37, 6)]
        sp = SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True)
        ids = [drv.open(p, sp) for p in prompts]
        got = {i: [] for i in ids}
        live = set(ids)
        while live:
            for r in drv.step(sorted(live)):
                if r.token is None:
                    continue
                drv.commit(r.seq_id, [r.token])
                got[r.seq_id].append(r.token)
                if drv.finished(r.seq_id, r.token):
                    drv.release(r.seq_id)
                    live.discard(r.seq_id)
    for i, p in zip(ids, prompts):
        seq = list(p)
        for t in got[i]:
            ref = forward_logits(w, torch.tensor(seq, dtype=torch.int32))[-1]
            top2 = torch.topk(ref, 2).values
            if float(top2[0] - top2[1]) > 0.05:        # bf16 storage can flip a near-tie
                assert t == int(ref.argmax())
            seq.append(t)


@pytest.mark.parametrize("kw", [{}, dict(n_experts=4, top_k=2, moe_ffn=128)], ids=["dense", "moe"])
def test_long_prefill_takes_the_tiled_split_k_route(kw):
    """More than 128 tokens in a step: the tiled GEMM, split-K partial slices folded into the next norm, expert
    chunks of 128 rows."""
    from poot_b200.oracle.torch_ref import forward_logits
    cfg = _cfg(hidden=1024, ffn=512, n_heads=4, n_kv_heads=2, head_dim=64, **kw)
    with emulated_kernels():
        w, eng, sess = _engine(cfg, batch=2, max_len=96, max_tokens=192)
        g = torch.Generator().manual_seed(4)
        prompts = torch.randint(0, cfg.vocab, (2, 80), generator=g, dtype=torch.int32)
        sess.prefill_fast(prompts)
        for b in range(2):
            ref = forward_logits(w, prompts[b])[-1]
            err = (eng.logits[b] - ref).abs().max().item()
            assert err < 0.03 * max(1.0, ref.abs().max().item()), err
