"""Mixture-of-experts path on one GPU: router, grouped expert GEMM (both regimes), whole model vs the torch reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_moe_route_matches_topk_softmax():
    from poot_b200.ops import moe_ops as M
    T, E, k = 37, 8, 2
    logits = torch.randn(T, E, device="cuda")
    logits[3, 1] = logits[3, 5] = 4.0          # tie: lower index first
    logits[4, 2] = float("nan")
    ids = torch.zeros(T * k, dtype=torch.int32, device="cuda")
    gates = torch.zeros(T * k, device="cuda")
    dense = torch.zeros(E, T, device="cuda")
    M.moe_route(logits, k, True, ids, gates, dense)
    ids, gates = ids.view(T, k), gates.view(T, k)
    clean = torch.nan_to_num(logits, nan=-3.4e38)
    tv, ti = torch.topk(clean, k, dim=-1)
    for t in range(T):
        if t == 3:
            assert ids[t].tolist() == [1, 5]
            continue
        assert ids[t].tolist() == ti[t].tolist(), t
        assert torch.allclose(gates[t], torch.softmax(tv[t], -1), atol=1e-5)
        assert abs(float(dense[:, t].sum()) - 1.0) < 1e-5
    assert 2 not in ids[4].tolist()


@pytest.mark.first_device_run          # steps with more rows than experts ride the row-grouped kernels
@pytest.mark.parametrize("batch,prompt", [(1, 9), (12, 6), (2, 100)])
def test_mixtral_like_model_matches_reference(batch, prompt):
    from poot_b200.models.config import DecoderConfig
    from poot_b200.ops import cuda_ops as K
    from poot_b200.oracle.torch_ref import forward_logits
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.session import FixedBatchSession
    from poot_b200.runtime.weights import random_weights
    cfg = DecoderConfig(family="mixtral", n_layers=2, hidden=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn=1024,
                        vocab=2048, max_position=256, n_experts=8, top_k=2, moe_ffn=768)
    w = random_weights(cfg, "cuda", seed=5, std=0.05)
    bps = 8
    eng = DecoderEngine(w, num_blocks=batch * bps, max_seqs=batch, max_tokens=max(batch * prompt, batch),
                        max_blocks_per_seq=bps)
    sess = FixedBatchSession(eng, batch, 128)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, cfg.vocab, (batch, prompt), generator=g, dtype=torch.int32)
    sess.prefill_fast(toks)
    K.check_status()
    for b in range(min(batch, 3)):
        ref = forward_logits(w, toks[b].cuda())[-1]
        err = (eng.logits[b] - ref).abs().max().item() / max(1.0, ref.abs().max().item())
        assert err < 0.06, (b, err)
    nxt = torch.randint(0, cfg.vocab, (batch,), generator=g, dtype=torch.int32)
    sess.decode(nxt.tolist())                 # decode step: slot regime at batch 1, dense regime above
    K.check_status()
    ref = forward_logits(w, torch.cat([toks[0], nxt[:1]]).cuda())[-1]
    err = (eng.logits[0] - ref).abs().max().item() / max(1.0, ref.abs().max().item())
    assert err < 0.06, err


@pytest.mark.xfail(strict=False, reason="router variant: not yet run on a device")
def test_sigmoid_router_with_selection_bias_matches_the_host_restatement():
    from poot_b200.ops import moe_ops as M
    from poot_b200.utils import kernel_emulation as emu
    g = torch.Generator().manual_seed(0)
    T, E, k = 37, 64, 6
    logits = torch.randn(T, E, generator=g) * 2
    bias = torch.randn(E, generator=g) * 0.3
    for renorm in (True, False):
        want = [torch.zeros(T * k, dtype=torch.int32), torch.zeros(T * k), torch.zeros(E * T)]
        emu.moe_route(logits, k, renorm, *want, mode="sigmoid", select_bias=bias, scale=2.5)
        got = [torch.zeros(T * k, dtype=torch.int32, device="cuda"), torch.zeros(T * k, device="cuda"), torch.zeros(E * T, device="cuda")]
        M.moe_route(logits.cuda(), k, renorm, *got, mode="sigmoid", select_bias=bias.cuda(), scale=2.5)
        assert torch.equal(got[0].cpu(), want[0])
        assert torch.allclose(got[1].cpu(), want[1], rtol=1e-5, atol=1e-6) and torch.allclose(got[2].cpu(), want[2], rtol=1e-5, atol=1e-6)
