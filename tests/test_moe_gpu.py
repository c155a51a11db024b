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


@pytest.mark.xfail(strict=False, reason="new kernels: not yet run on a device")
@pytest.mark.parametrize("world,S,k,E", [(2, 8, 2, 8), (4, 16, 4, 16)])
def test_expert_exchange_kernels_with_every_rank_on_one_device(world, S, k, E):
    """Dispatch -> mask -> gather -> (identity experts) -> combine -> finish with all ranks' areas on one device and the
    phases launched rank after rank in one stream, so a kernel never waits for a flag that is not set yet.  With the
    experts replaced by "multiply the row by its gate", every token must come back as its row times the sum of its gates."""
    import ctypes
    from ctypes import c_int, c_void_p
    import torch
    from poot_b200.ops import cuda_ops as K, moe_ops as M
    H, e_local, cap = 256, E // world, S * k
    dev = "cuda"
    i32 = dict(dtype=torch.int32, device=dev)
    flags = [torch.zeros(6 * 8, **i32) for _ in range(world)]
    recv = [torch.zeros(2, world, cap, H, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    meta = [torch.zeros(2, world, cap, 4, **i32) for _ in range(world)]
    count = [torch.zeros(2, world, **i32) for _ in range(world)]
    back = [torch.zeros(2, cap, H, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    arr = lambda ts: (c_void_p * world)(*[t.data_ptr() for t in ts])
    epoch = [torch.ones(1, **i32) for _ in range(world)]
    ticket = [torch.zeros(1, **i32) for _ in range(world)]
    st = K.status_word(torch.device(dev))
    P, ep_common = c_void_p, [c_int] * 9 + [c_void_p] * 9
    K.register_signature("poot_ep_plan", [P, c_int, c_int, c_int, P, P, P, P])
    K.register_signature("poot_ep_dispatch", [P, c_int, P, P, P, P, P] + ep_common)
    K.register_signature("poot_ep_mask", [P, P, P, P] + ep_common)
    K.register_signature("poot_ep_gather", [P, P, P, P, c_int, c_int, P, P] + ep_common)
    K.register_signature("poot_ep_combine", [P, P, P] + ep_common)
    K.register_signature("poot_ep_finish", [P, P] + ep_common)
    common = lambda r: (world, r, S, k, cap, H, e_local, 0, 1, epoch[r].data_ptr(), flags[r].data_ptr(), arr(flags), arr(recv),
                        arr(meta), arr(count), arr(back), ticket[r].data_ptr(), st.data_ptr(), K._stream())
    g = torch.Generator().manual_seed(0)
    x = [(torch.randn(S, H, generator=g) * 0.5).to(torch.bfloat16).to(dev) for _ in range(world)]
    ids = [torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(S)]).reshape(-1).to(torch.int32).to(dev) for _ in range(world)]
    gates = [torch.rand(S * k, generator=g).to(dev) for _ in range(world)]
    h = [torch.zeros(S, H, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    ck = lambda rc, what: (_ for _ in ()).throw(RuntimeError(f"{what}: {rc}")) if rc else None
    for r in range(world):
        dest, dpos, cnt = torch.zeros(cap, **i32), torch.zeros(cap, **i32), torch.zeros(8, **i32)
        ck(K.fn("poot_ep_plan")(ids[r].data_ptr(), S * k, e_local, world, dest.data_ptr(), dpos.data_ptr(), cnt.data_ptr(), K._stream()), "plan")
        ck(K.fn("poot_ep_dispatch")(x[r].data_ptr(), H, ids[r].data_ptr(), gates[r].data_ptr(), dest.data_ptr(), dpos.data_ptr(),
                                    cnt.data_ptr(), *common(r)), "dispatch")
        assert int(cnt[:world].sum()) == S * k
    n = world * cap
    pos_all = []
    for r in range(world):
        rids, rg = torch.zeros(n, **i32), torch.zeros(n, dtype=torch.float32, device=dev)
        ck(K.fn("poot_ep_mask")(meta[r].data_ptr(), count[r].data_ptr(), rids.data_ptr(), rg.data_ptr(), *common(r)), "mask")
        live = rids >= 0
        assert int(live.sum()) == int(count[r][1].sum()) and bool(((rids[live] // e_local) == r).all())
        block = 16
        max_tiles = M.group_capacity(n, e_local, block)
        pos, srt = torch.zeros(n, **i32), torch.zeros(max_tiles * block, **i32)
        te, nt = torch.zeros(max_tiles, **i32), torch.zeros(1, **i32)
        M.moe_align(rids, r * e_local, e_local, block, max_tiles, pos, srt, te, nt)
        xs = torch.zeros(max_tiles * block, H, dtype=torch.bfloat16, device=dev)
        gs = torch.zeros(max_tiles * block, dtype=torch.float32, device=dev)
        ck(K.fn("poot_ep_gather")(recv[r].data_ptr(), srt.data_ptr(), rg.data_ptr(), nt.data_ptr(), block, max_tiles, xs.data_ptr(),
                                  gs.data_ptr(), *common(r)), "gather")
        y = (xs.float() * gs[:, None]).to(torch.bfloat16)             # the "expert": scale the row by its gate
        ck(K.fn("poot_ep_combine")(y.data_ptr(), pos.data_ptr(), meta[r].data_ptr(), *common(r)), "combine")
        pos_all.append(pos)
    for r in range(world):
        ck(K.fn("poot_ep_finish")(h[r].data_ptr(), back[r].data_ptr(), *common(r)), "finish")
    K.check_status()
    for r in range(world):
        want = torch.zeros(S, H)
        for t in range(S):
            for j in range(k):
                want[t] += (x[r][t].float().cpu() * gates[r][t * k + j].item()).to(torch.bfloat16).float()
        err = (h[r].float().cpu() - want).abs().max().item()
        assert err <= 0.02 * max(1.0, want.abs().max().item()), (r, err)
