"""Numerics of every CUDA kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from poot_b200.ops import cuda_ops
    return cuda_ops


def bf(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def close(a, b, rtol=2e-2, atol=2e-2):
    a, b = a.float(), b.float()
    assert torch.isfinite(a).all()
    err = (a - b).abs().max().item()
    ref = b.abs().max().item()
    assert err <= atol + rtol * ref, f"max err {err} vs ref max {ref}"


def test_embed_gather(K):
    table = bf(1000, 256)
    ids = torch.randint(0, 1000, (37,), device="cuda", dtype=torch.int32)
    out = K.embed_gather(ids, table)
    assert torch.equal(out, table[ids.long()])


@pytest.mark.parametrize("D", [256, 2048, 4096, 8192])
def test_rmsnorm(K, D):
    x, w = bf(5, D, seed=1), bf(D, seed=2)
    y = K.rmsnorm(x, w, 1e-5)
    xf = x.float()
    ref = xf / torch.sqrt((xf * xf).mean(-1, keepdim=True) + 1e-5) * w.float()
    close(y, ref, 1e-2, 1e-2)


def test_rmsnorm_partials(K):
    T, D, P = 7, 4096, 3
    h, w = bf(T, D, seed=1), bf(D, seed=2)
    parts = torch.randn(P, T, D, device="cuda")
    h2 = h.clone()
    y = K.rmsnorm(h2, w, 1e-5, partials=parts, h_out=h2)
    hn = (h.float() + parts.sum(0)).to(torch.bfloat16)
    close(h2, hn, 1e-2, 1e-2)
    xf = hn.float()
    ref = xf / torch.sqrt((xf * xf).mean(-1, keepdim=True) + 1e-5) * w.float()
    close(y, ref, 1e-2, 2e-2)


@pytest.mark.parametrize("inter", [True, False])
def test_swiglu(K, inter):
    T, F = 9, 688
    gu = bf(T, 2 * F)
    out = K.swiglu(gu, inter)
    g, u = (gu[:, 0::2], gu[:, 1::2]) if inter else (gu[:, :F], gu[:, F:])
    close(out, torch.nn.functional.silu(g.float()) * u.float(), 1e-2, 1e-2)


@pytest.mark.parametrize("M", [1, 2, 4])
@pytest.mark.parametrize("N,Kd", [(512, 256), (6144, 4096), (4096, 14336), (1026, 520)])
def test_gemv(K, M, N, Kd):
    x, W = bf(M, Kd, seed=1), bf(N, Kd, scale=0.05, seed=2)
    ref = x.float() @ W.float().T
    close(K.gemv(x, W, K.EPI_STORE), ref)
    close(K.gemv(x, W, K.EPI_F32), ref, 1e-3, 1e-3)
    res = bf(M, N, seed=3)
    close(K.gemv(x, W, K.EPI_RESID, resid=res), ref + res.float())
    sw = K.gemv(x, W, K.EPI_SWIGLU)
    close(sw, torch.nn.functional.silu(ref[:, 0::2]) * ref[:, 1::2])


@pytest.mark.parametrize("bn", [64, 128, 256])
@pytest.mark.parametrize("M,N,Kd", [(128, 256, 64), (64, 512, 4096), (512, 1024, 1024), (300, 776, 520), (5, 64, 128)])
def test_gemm_tcgen05(K, bn, M, N, Kd):
    x, W = bf(M, Kd, seed=1), bf(N, Kd, scale=0.05, seed=2)
    ref = x.float() @ W.float().T
    out = K.gemm(x, W, K.EPI_STORE, bn=bn)
    K.check_status()
    close(out, ref)
    close(K.gemm(x, W, K.EPI_F32, bn=bn), ref, 1e-3, 1e-3)
    res = bf(M, N, seed=3)
    close(K.gemm(x, W, K.EPI_RESID, resid=res, bn=bn), ref + res.float())
    if N % 16 == 0:
        close(K.gemm(x, W, K.EPI_SWIGLU, bn=bn), torch.nn.functional.silu(ref[:, 0::2]) * ref[:, 1::2])
    K.check_status()


@pytest.mark.parametrize("M", [1, 3, 16, 17, 64, 100, 128])
@pytest.mark.parametrize("N,Kd,ck", [(4096, 4096, 8), (6144, 4096, 4), (1024, 14336, 8), (28672, 1024, 1), (776, 520, 2),
                                     (256, 192, 4)])
def test_gemm_skinny(K, M, N, Kd, ck):
    x, W = bf(M, Kd, seed=1), bf(N, Kd, scale=0.05, seed=2)
    ref = x.float() @ W.float().T
    close(K.gemm_skinny(x, W, K.EPI_F32, ck=ck), ref, 1e-3, 1e-3)
    res = bf(M, N, seed=3)
    close(K.gemm_skinny(x, W, K.EPI_RESID, resid=res, ck=ck), ref + res.float())
    close(K.gemm_skinny(x, W, K.EPI_SWIGLU, ck=ck), torch.nn.functional.silu(ref[:, 0::2]) * ref[:, 1::2])
    h = res.clone()
    K.gemm_skinny(x, W, K.EPI_RESID, out=h, resid=h)
    close(h, ref + res.float())
    K.check_status()


def test_pdl_chain_matches_plain(K):
    """A chain of dependent kernels gives the same result with programmatic dependent launch on and off."""
    x, W1, W2 = bf(8, 1024, seed=1), bf(2048, 1024, scale=0.05, seed=2), bf(1024, 1024, scale=0.05, seed=3)
    w = bf(1024, seed=4)

    def chain():
        a = K.gemm_skinny(x, W1, K.EPI_SWIGLU)
        b = K.gemm_skinny(a, W2, K.EPI_RESID, resid=x)
        return K.rmsnorm(b, w, 1e-5)

    plain = chain().clone()
    K.set_pdl(True)
    try:
        for _ in range(5):
            got = chain()
        torch.cuda.synchronize()
    finally:
        K.set_pdl(False)
    assert torch.equal(plain, got)


@pytest.mark.parametrize("splits", [2, 4, 7])
def test_gemm_tcgen05_splitk(K, splits):
    M, N, Kd = 64, 4096, 14336
    x, W = bf(M, Kd, seed=1), bf(N, Kd, scale=0.02, seed=2)
    parts = K.gemm(x, W, K.EPI_PARTIAL, bn=64, splits=splits)
    K.check_status()
    close(parts.sum(0), x.float() @ W.float().T, 2e-3, 2e-3)


def test_gemm_inplace_residual(K):
    M, N, Kd = 64, 4096, 1024
    x, W, h = bf(M, Kd, seed=1), bf(N, Kd, scale=0.05, seed=2), bf(M, N, seed=3)
    ref = h.float() + x.float() @ W.float().T
    K.gemm(x, W, K.EPI_RESID, out=h, resid=h)
    close(h, ref)


def _paged_setup(nseq, ctx_lens, Hkv, D, seed=0):
    blocks_per = (max(ctx_lens) + 15) // 16 + 1
    nb = nseq * blocks_per
    perm = torch.randperm(nb, generator=torch.Generator().manual_seed(seed)).to(torch.int32)
    bt = perm.view(nseq, blocks_per).cuda()
    kpool, vpool = bf(nb, Hkv, 16, D, seed=seed + 1), bf(nb, Hkv, 16, D, seed=seed + 2)
    return bt, kpool, vpool


def _gather_kv(pool, bt_row, n):
    blocks = pool[bt_row.long()]            # [nblk, Hkv, 16, D]
    x = blocks.permute(1, 0, 2, 3).reshape(pool.shape[1], -1, pool.shape[3])  # [Hkv, pos, D]
    return x[:, :n]


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (4, 2, 64), (64, 8, 128), (8, 8, 128), (4, 4, 64)])
@pytest.mark.parametrize("splits", [1, 4])
def test_attn_paged(K, Hq, Hkv, D, splits):
    ctx = [1, 17, 100, 333]
    bt, kpool, vpool = _paged_setup(len(ctx), ctx, Hkv, D)
    R = len(ctx)
    q = bf(R, Hq * D, seed=5)
    row_seq = torch.arange(R, device="cuda", dtype=torch.int32)
    row_ctx = torch.tensor(ctx, device="cuda", dtype=torch.int32)
    scale = 1 / math.sqrt(D)
    out = K.attn_paged(q, kpool, vpool, bt, row_seq, row_ctx, Hq, Hkv, D, scale, splits=splits)
    n_rep = Hq // Hkv
    for r in range(R):
        k = _gather_kv(kpool, bt[r], ctx[r]).float().repeat_interleave(n_rep, 0)
        v = _gather_kv(vpool, bt[r], ctx[r]).float().repeat_interleave(n_rep, 0)
        qq = q[r].float().view(Hq, D)
        p = torch.softmax(torch.einsum("hd,hsd->hs", qq, k) * scale, -1)
        ref = torch.einsum("hs,hsd->hd", p, v).reshape(-1)
        close(out[r], ref, 2e-2, 1e-2)


def test_attn_paged_window_softcap(K):
    Hq, Hkv, D = 8, 2, 128
    ctx = [50, 200]
    bt, kpool, vpool = _paged_setup(2, ctx, Hkv, D)
    q = bf(2, Hq * D, seed=5)
    row_ctx = torch.tensor(ctx, device="cuda", dtype=torch.int32)
    scale, cap, win = 1 / math.sqrt(D), 30.0, 64
    out = K.attn_paged(q, kpool, vpool, bt, None, row_ctx, Hq, Hkv, D, scale, softcap=cap, window=win)
    for r in range(2):
        k = _gather_kv(kpool, bt[r], ctx[r]).float().repeat_interleave(4, 0)
        v = _gather_kv(vpool, bt[r], ctx[r]).float().repeat_interleave(4, 0)
        s = torch.einsum("hd,hsd->hs", q[r].float().view(Hq, D), k) * scale
        s = cap * torch.tanh(s / cap)
        first = max(0, ctx[r] - win)
        s[:, :first] = float("-inf")
        ref = torch.einsum("hs,hsd->hd", torch.softmax(s, -1), v).reshape(-1)
        close(out[r], ref, 2e-2, 1e-2)


def test_rope_kv_write(K):
    from poot_b200.models.config import DecoderConfig
    from poot_b200.runtime.rope import rope_tables
    Hq, Hkv, D, T = 8, 2, 128, 19
    cfg = DecoderConfig(head_dim=D, rope_theta=500000.0)
    cos, sin = rope_tables(cfg, 512)
    cos, sin = cos.cuda(), sin.cuda()
    qkv = bf(T, (Hq + 2 * Hkv) * D, seed=3)
    pos = torch.randint(0, 512, (T,), device="cuda", dtype=torch.int32)
    nb = 8
    slots = torch.randperm(nb * 16)[:T].to(torch.int32).cuda()
    slots[3] = -1
    kpool = torch.zeros(nb, Hkv, 16, D, dtype=torch.bfloat16, device="cuda")
    vpool = torch.zeros_like(kpool)
    q_out = torch.empty(T, Hq * D, dtype=torch.bfloat16, device="cuda")
    K.rope_kv_write(qkv, q_out, kpool, vpool, pos, slots, cos, sin, Hq, Hkv, D)

    def rope(x):  # [T,H,D]
        c, s = cos[pos.long()][:, None, :], sin[pos.long()][:, None, :]
        x1, x2 = x[..., :D // 2].float(), x[..., D // 2:].float()
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)

    qr = rope(qkv[:, :Hq * D].view(T, Hq, D))
    close(q_out.view(T, Hq, D), qr, 1e-2, 1e-2)
    kr = rope(qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)).to(torch.bfloat16)
    vr = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        close(kpool[s // 16, :, s % 16], kr[t], 1e-2, 1e-2)
        assert torch.equal(vpool[s // 16, :, s % 16], vr[t])
    assert kpool.float().abs().sum() > 0


def test_argmax(K):
    logits = torch.randn(5, 128256, device="cuda")
    logits[1, 777] = 100.0
    logits[2, 5] = float("nan")
    logits[3, 10] = logits[3, 20] = 50.0
    out = K.argmax(logits).cpu()
    assert out[0, 0] == logits[0].argmax().item() and out[0, 1] == -1
    assert out[1, 0] == 777
    assert out[2, 0] == 0 and out[2, 1] == 5
    assert out[3, 0] == 10


def test_random_uniform_matches_hash(K):
    seeds = torch.tensor([1, 12345], dtype=torch.int32, device="cuda")
    u = K.random_uniform(seeds, 1000).cpu()
    from poot_b200.oracle.sampling import random_uniform_at
    for r, s in enumerate([1, 12345]):
        for c in (0, 1, 999):
            assert u[r, c].item() == random_uniform_at(s, c)


@pytest.mark.parametrize("rule", [1, 2, 3])
def test_sample_gumbel_matches_oracle(K, rule):
    from poot_b200.oracle.sampling import sample_rows
    rows, vocab = 4, 5000
    logits = torch.randn(rows, vocab, device="cuda") * 3
    params = torch.tensor([[1.0, -3.0, 1.0, 0.9], [0.5, -1e30, 1.0, 0.5], [2.0, -2.0, 1.0, 1.0], [1.0, -5.0, 1.0, 0.0]],
                          device="cuda")
    top_k = torch.tensor([40, 0, 5, 10], dtype=torch.int32, device="cuda")
    seeds = torch.tensor([1, 2, 3, 4], dtype=torch.int32, device="cuda")
    out = K.sample_gumbel(logits, params, top_k, seeds, rule).cpu()
    ref = sample_rows(logits.cpu().numpy(), params.cpu().numpy(), top_k.cpu().numpy(), seeds.cpu().numpy(), rule)
    # device exp/log differ from the host's by ulps, so allow a different pick only on a near tie of scores
    agree = (out[:, 0].numpy() == ref[:, 0]).mean()
    assert agree >= 0.75, (out, ref)
    assert (out[:, 1] == -1).all()


@pytest.mark.parametrize("window", [0, 48])
@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (4, 4)])
def test_flash_prefill_matches_reference_over_paged_kv(window, Hq, Hkv):
    """Tensor-core prefill attention: several sequences, pieces that start mid-sequence, ragged tiles, shuffled pages."""
    from poot_b200.ops import cuda_ops as K
    torch.manual_seed(0)
    D, nblocks, max_blocks = 128, 96, 32
    # (block-table row, first position, tokens): a fresh 200-token prompt, a 70-token chunk continuing at 300, a short piece
    segs = [(0, 0, 200), (1, 300, 70), (2, 5, 16), (3, 0, 129)]
    kpool = (torch.randn(nblocks, Hkv, 16, D, device="cuda") * 0.5).to(torch.bfloat16)
    vpool = (torch.randn(nblocks, Hkv, 16, D, device="cuda") * 0.5).to(torch.bfloat16)
    perm = torch.randperm(nblocks)
    bt = torch.zeros(4, max_blocks, dtype=torch.int32)
    nxt = 0
    for r, p0, n in segs:
        need = (p0 + n + 15) // 16
        bt[r, :need] = perm[nxt:nxt + need].to(torch.int32)
        nxt += need
    row_seq = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, _, n in segs])
    positions = torch.cat([torch.arange(p0, p0 + n, dtype=torch.int32) for _, p0, n in segs])
    T = row_seq.numel()
    q = (torch.randn(T, Hq * D, device="cuda") * 0.5).to(torch.bfloat16)
    tiles, covered = K.flash_tiles(row_seq.numpy(), positions.numpy())
    assert covered.all() and tiles.shape[0] == 2 + 1 + 1 + 2
    tiles_dev = torch.zeros(tiles.shape[0] + 3, 4, dtype=torch.int32, device="cuda")     # trailing empty slots are skipped
    tiles_dev[:tiles.shape[0]] = torch.from_numpy(tiles).cuda()
    out = torch.zeros(T, Hq * D, dtype=torch.bfloat16, device="cuda")
    scale = D ** -0.5
    K.attn_flash_prefill(q, kpool, vpool, bt.cuda(), tiles_dev, Hq, Hkv, scale, out, window=window)
    torch.cuda.synchronize()
    K.check_status()
    n_rep = Hq // Hkv
    worst = 0.0
    for i in range(0, T, 7):           # a spread of rows, every segment and tile boundary included
        r, p = int(row_seq[i]), int(positions[i])
        ctx = p + 1
        blocks = bt[r, :(ctx + 15) // 16].long().cuda()
        k = kpool[blocks].permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, :ctx].float()
        v = vpool[blocks].permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, :ctx].float()
        lo = max(0, ctx - window) if window else 0
        qi = q[i].float().view(Hq, D)
        for h in range(Hq):
            s = (k[h // n_rep, lo:] @ qi[h]) * scale
            ref = torch.softmax(s, 0) @ v[h // n_rep, lo:]
            worst = max(worst, (out[i].float().view(Hq, D)[h] - ref).abs().max().item())
    assert worst < 2e-2, worst
    assert torch.isfinite(out.float()).all()


@pytest.mark.xfail(strict=False, reason="new kernels: not yet run on a device")
@pytest.mark.parametrize("act", ["silu", "gelu_tanh", "gelu_erf"])
def test_gated_activation_and_logit_softcap(act):
    from poot_b200.ops import cuda_ops as K
    g = torch.Generator(device="cuda").manual_seed(0)
    gu = (torch.randn(37, 2 * 264, device="cuda", generator=g) * 2).to(torch.bfloat16)
    fn = {"silu": torch.nn.functional.silu, "gelu_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh"),
          "gelu_erf": torch.nn.functional.gelu}[act]
    for interleaved in (True, False):
        x = gu.float()
        gate, up = (x[:, 0::2], x[:, 1::2]) if interleaved else (x[:, :264], x[:, 264:])
        ref = fn(gate) * up
        got = K.gated_act(gu, interleaved, act).float()
        assert (got - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 1e-3
    logits = torch.randn(5, 1000, device="cuda", generator=g) * 40
    ref = 30.0 * torch.tanh(logits / 30.0)
    K.softcap_(logits, 30.0)
    assert (logits - ref).abs().max().item() < 1e-3


@pytest.mark.xfail(strict=False, reason="gated delta net kernels: not yet run on a device")
@pytest.mark.parametrize("D", [64, 128])
def test_gdn_kernels_match_their_host_restatements(D):
    """Causal conv + SiLU, the gated delta rule scan, the gated RMSNorm and the sigmoid gate against the host
    restatements the emulated-engine tests use (which are in turn checked against the graph oracle)."""
    from poot_b200.ops import cuda_ops as K
    from poot_b200.utils import kernel_emulation as emu
    g = torch.Generator().manual_seed(0)
    nk, nv, Kc, rows = 2, 4, 4, 3
    C = (2 * nk + nv) * D
    N = C + nv * D + 2 * nv
    T = 23
    x = (torch.randn(T, N, generator=g) * 0.5).to(torch.bfloat16)
    w = torch.randn(C, Kc, generator=g) * 0.3
    segs = torch.tensor([[0, 9, 2, 0], [9, 1, 0, 5], [10, 13, 1, 16], [0, 0, 0, 0]], dtype=torch.int32)
    cstate = torch.randn(rows, Kc - 1, C, generator=g) * 0.2
    sstate = torch.randn(rows, nv, D, D, generator=g) * 0.05
    dt_bias, a_log = torch.randn(nv, generator=g) * 0.3, torch.log(torch.rand(nv, generator=g) * 3 + 0.5)
    # host
    c_ref, s_ref = cstate.clone(), sstate.clone()
    conv_ref = torch.zeros(T, C, dtype=torch.bfloat16)
    emu.causal_conv_silu(x, 0, C, w, c_ref, segs, conv_ref)
    y_ref = torch.zeros(T, nv * D, dtype=torch.bfloat16)
    emu.gdn_scan(conv_ref, x, C + nv * D, C + nv * D + nv, dt_bias, a_log, s_ref, segs, y_ref, nk, nv, D)
    gn_w = (1 + 0.1 * torch.randn(D, generator=g)).to(torch.bfloat16)
    n_ref = torch.zeros_like(y_ref)
    emu.gated_rmsnorm(y_ref, x, C, gn_w, 1e-6, n_ref, nv, D)
    # device
    xd, segd = x.cuda(), segs.cuda()
    c_dev, s_dev = cstate.cuda(), sstate.cuda()
    conv = torch.zeros(T, C, dtype=torch.bfloat16, device="cuda")
    K.causal_conv_silu(xd, 0, C, w.cuda(), c_dev, segd, conv)
    y = torch.zeros(T, nv * D, dtype=torch.bfloat16, device="cuda")
    K.gdn_scan(conv, xd, C + nv * D, C + nv * D + nv, dt_bias.cuda(), a_log.cuda(), s_dev, segd, y, nk, nv, D)
    n = torch.zeros_like(y)
    K.gated_rmsnorm(y, xd, C, gn_w.cuda(), 1e-6, n, nv, D)
    K.check_status()
    tol = lambda a, b: (a.float().cpu() - b.float()).abs().max().item() <= 0.02 * b.float().abs().max().item() + 2e-3
    assert tol(conv, conv_ref) and tol(c_dev, c_ref)
    assert tol(y, y_ref) and tol(s_dev, s_ref)
    assert tol(n, n_ref)
    a = torch.randn(7, 96, generator=g).to(torch.bfloat16)
    gt = torch.randn(7, 96, generator=g).to(torch.bfloat16)
    want = (a.float() * torch.sigmoid(gt.float()))
    got = K.sigmoid_mul(a.cuda(), gt.cuda())
    assert tol(got, want)


@pytest.mark.xfail(strict=False, reason="new kernel: not yet run on a device")
def test_ngram_hash_matches_its_host_restatement():
    """Ids and carried histories of pieces that start a sequence, continue one (one token: a decode step) and contain
    an end-of-sequence id and an out-of-vocabulary token, against the host restatement in Python integers."""
    from poot_b200.models.ngram import ngram_tables
    from poot_b200.ops import cuda_ops as K
    from poot_b200.utils import kernel_emulation as emu
    g = torch.Generator().manual_seed(2)
    vocab, eos, rows, T = 1000, 7, 3, 24
    for order, per in ((3, 2), (2, 3)):
        tb = ngram_tables(1, order, per, 5000, 64, 99, vocab)
        ctx, heads = order - 1, len(tb.primes)
        tokens = torch.randint(0, vocab, (T,), generator=g, dtype=torch.int32)
        tokens[4], tokens[15] = eos, vocab + 5
        segs = torch.tensor([[0, 9, 2, 0], [9, 1, 0, 5], [10, 14, 1, 16], [0, 0, 0, 0]], dtype=torch.int32)
        hist = torch.randint(0, vocab, (rows, ctx), generator=g, dtype=torch.int32)
        mult = torch.tensor([m - (1 << 64) if m >= 1 << 63 else m for m in tb.multipliers], dtype=torch.int64)
        primes, offsets = torch.tensor(tb.primes, dtype=torch.int32), torch.tensor(tb.offsets, dtype=torch.int32)
        h_ref, i_ref = hist.clone(), torch.zeros(T, heads, dtype=torch.int32)
        emu.ngram_hash(tokens, h_ref, segs, mult, primes, offsets, per, eos, vocab, i_ref)
        h_dev, ids = hist.cuda(), torch.zeros(T, heads, dtype=torch.int32, device="cuda")
        K.ngram_hash(tokens.cuda(), h_dev, segs.cuda(), mult.cuda(), primes.cuda(), offsets.cuda(), per, eos, vocab, ids)
        K.check_status()
        assert torch.equal(ids.cpu(), i_ref) and torch.equal(h_dev.cpu(), h_ref)


@pytest.mark.xfail(strict=False, reason="new kernel: not yet run on a device")
@pytest.mark.parametrize("D", [64, 128])
def test_kda_scan_matches_its_host_restatement(D):
    """The delta rule with a decay per key channel against the host restatement (itself checked against the graph
    oracle's scan equation): outputs and carried states of pieces that start at zero and that continue."""
    from poot_b200.ops import cuda_ops as K
    from poot_b200.utils import kernel_emulation as emu
    g = torch.Generator().manual_seed(1)
    heads, rows, T = 3, 3, 21
    C = heads * D
    qkv = (torch.randn(T, 3 * C, generator=g) * 0.5).to(torch.bfloat16)
    f = (torch.randn(T, C, generator=g)).to(torch.bfloat16)
    bm = (torch.randn(T, heads + 5, generator=g)).to(torch.bfloat16)
    segs = torch.tensor([[0, 8, 2, 0], [8, 1, 0, 5], [9, 12, 1, 16], [0, 0, 0, 0]], dtype=torch.int32)
    state = torch.randn(rows, heads, D, D, generator=g) * 0.05
    dt_bias, a_log = torch.randn(C, generator=g) * 0.3, torch.log(torch.rand(heads, generator=g) * 2 + 0.5)
    s_ref, y_ref = state.clone(), torch.zeros(T, C, dtype=torch.bfloat16)
    emu.kda_scan(qkv, f, bm, 2, dt_bias, a_log, -5.0, s_ref, segs, y_ref, heads, D)
    s_dev, y = state.cuda(), torch.zeros(T, C, dtype=torch.bfloat16, device="cuda")
    K.kda_scan(qkv.cuda(), f.cuda(), bm.cuda(), 2, dt_bias.cuda(), a_log.cuda(), -5.0, s_dev, segs.cuda(), y, heads, D)
    K.check_status()
    tol = lambda a, b: (a.float().cpu() - b.float()).abs().max().item() <= 0.02 * b.float().abs().max().item() + 2e-3
    assert tol(y, y_ref) and tol(s_dev, s_ref)


@pytest.mark.xfail(strict=False, reason="general attention kernel: not yet run on a device")
@pytest.mark.parametrize("Dk,Dv,extras", [(256, 256, False), (192, 128, False), (64, 64, True)])
def test_general_attention_matches_its_host_restatement(Dk, Dv, extras):
    from poot_b200.ops import cuda_ops as K
    from poot_b200.utils import kernel_emulation as emu
    g = torch.Generator().manual_seed(0)
    Hq, Hkv, blocks, R = 4, 2, 12, 5
    pd = max(Dk, Dv)
    kpool = (torch.randn(blocks, Hkv, 16, pd, generator=g) * 0.5).to(torch.bfloat16)
    vpool = (torch.randn(blocks, Hkv, 16, pd, generator=g) * 0.5).to(torch.bfloat16)
    bt = torch.tensor([[3, 1, 7, 0], [5, 2, 9, 11]], dtype=torch.int32)
    row_seq = torch.tensor([0, 0, 1, 1, 0], dtype=torch.int32)
    row_ctx = torch.tensor([1, 37, 64, 20, 0], dtype=torch.int32)
    q = (torch.randn(R, Hq * Dk, generator=g) * 0.5).to(torch.bfloat16)
    alibi = torch.tensor([0.5, 0.25, 0.125, 0.0625]) if extras else None
    sinks = torch.randn(Hq, generator=g) if extras else None
    for window, cap in ((0, 0.0), (9, 5.0)):
        want = torch.zeros(R, Hq * Dv, dtype=torch.bfloat16)
        emu.attn_general(q, kpool, vpool, bt, row_seq, row_ctx, Hq, Hkv, Dk, Dv, 0.11, want, cap, window, alibi, sinks)
        got = torch.zeros(R, Hq * Dv, dtype=torch.bfloat16, device="cuda")
        K.attn_general(q.cuda(), kpool.cuda(), vpool.cuda(), bt.cuda(), row_seq.cuda(), row_ctx.cuda(), Hq, Hkv, Dk, Dv, 0.11, got,
                       cap, window, None if alibi is None else alibi.cuda(), None if sinks is None else sinks.cuda())
        assert (got.float().cpu() - want.float()).abs().max().item() < 0.02


@pytest.mark.xfail(strict=False, reason="latent attention assembly and group-limited routing: not yet run on a device")
def test_mla_assembly_and_group_limited_router_match_their_host_restatements():
    from poot_b200.ops import cuda_ops as K
    from poot_b200.ops import moe_ops as M
    from poot_b200.utils import kernel_emulation as emu
    g = torch.Generator().manual_seed(0)
    T, nh, dn, dr, dv, rk, blocks = 9, 4, 64, 32, 64, 48, 6
    q = torch.randn(T, nh * (dn + dr), generator=g).to(torch.bfloat16)
    kvb = torch.randn(T, nh * (dn + dv), generator=g).to(torch.bfloat16)
    kva = torch.randn(T, rk + dr, generator=g).to(torch.bfloat16)
    pos = torch.arange(3, 3 + T, dtype=torch.int32)
    slots = torch.tensor([5, 6, 7, -1, 40, 41, 42, 43, 90], dtype=torch.int32)
    ang = torch.arange(64)[:, None] * (1.0 / 10000 ** (torch.arange(dr // 2) / (dr // 2)))[None]
    cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    ref = [torch.zeros(T, nh * (dn + dr), dtype=torch.bfloat16), torch.zeros(blocks, nh, 16, dn + dr, dtype=torch.bfloat16),
           torch.zeros(blocks, nh, 16, dn + dr, dtype=torch.bfloat16)]
    emu.mla_qkv_write(q, kvb, kva, rk, ref[0], ref[1], ref[2], pos, slots, cos, sin, nh, dn, dr, dv)
    dev = [torch.zeros_like(t).cuda() for t in ref]
    K.mla_qkv_write(q.cuda(), kvb.cuda(), kva.cuda(), rk, dev[0], dev[1], dev[2], pos.cuda(), slots.cuda(), cos.cuda(), sin.cuda(),
                    nh, dn, dr, dv)
    for a, b in zip(dev, ref):
        assert (a.float().cpu() - b.float()).abs().max().item() < 0.02
    E, k = 32, 6
    logits = torch.randn(21, E, generator=g) * 2
    bias = torch.randn(E, generator=g) * 0.2
    want = [torch.zeros(21 * k, dtype=torch.int32), torch.zeros(21 * k), torch.zeros(E * 21)]
    emu.moe_route(logits, k, True, *want, mode="sigmoid", select_bias=bias, scale=2.5, n_group=8, topk_group=3)
    got = [torch.zeros(21 * k, dtype=torch.int32, device="cuda"), torch.zeros(21 * k, device="cuda"), torch.zeros(E * 21, device="cuda")]
    M.moe_route(logits.cuda(), k, True, *got, mode="sigmoid", select_bias=bias.cuda(), scale=2.5, n_group=8, topk_group=3)
    assert torch.equal(got[0].cpu(), want[0]) and torch.allclose(got[1].cpu(), want[1], rtol=1e-5, atol=1e-6)


@pytest.mark.xfail(strict=False, reason="row replacement (image rows in place of embeddings): not yet run on a device")
def test_replace_rows_takes_the_flagged_rows_only():
    from poot_b200.ops import cuda_ops as K
    g = torch.Generator().manual_seed(0)
    for T, D in ((37, 576), (1, 8), (300, 2048)):
        h = torch.randn(T, D, generator=g).to(torch.bfloat16)
        rows = torch.randn(T, D, generator=g).to(torch.bfloat16)
        flags = (torch.rand(T, generator=g) < 0.4).to(torch.int32)
        want = torch.where(flags.bool()[:, None], rows, h)
        got = K.replace_rows_(h.clone().cuda(), rows.cuda(), flags.cuda())
        assert torch.equal(got.cpu(), want)


@pytest.mark.xfail(strict=False, reason="LayerNorm, plain activations and the clamped SwiGLU: not yet run on a device")
def test_layernorm_plain_activations_and_clamped_swiglu():
    from poot_b200.ops import cuda_ops as K
    from poot_b200.utils import kernel_emulation as emu
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(19, 384, generator=g) * 2 + 0.5).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(384, generator=g)).to(torch.bfloat16)
    b = (0.1 * torch.randn(384, generator=g)).to(torch.bfloat16)
    close = lambda a, r: (a.float().cpu() - r.float()).abs().max().item() <= 0.02 * r.float().abs().max().item() + 2e-3
    for bias in (b, None):
        assert close(K.layernorm(x.cuda(), w.cuda(), None if bias is None else bias.cuda(), 1e-5), emu.layernorm(x, w, bias, 1e-5))
    for act in ("silu", "gelu_tanh", "gelu_erf", "relu2"):
        assert close(K.act_(x.clone().cuda(), act), emu.act_(x.clone(), act))
    gu = (torch.randn(11, 2 * 96, generator=g) * 6).to(torch.bfloat16)
    assert close(K.gated_act(gu.cuda(), True, "swiglu_clamped", limit=7.0, alpha=1.702),
                 emu.gated_act(gu, True, "swiglu_clamped", limit=7.0, alpha=1.702))


@pytest.mark.xfail(strict=False, reason="Mamba2 kernels: not yet run on a device")
@pytest.mark.parametrize("P,N", [(64, 128), (32, 16)])
def test_mamba2_kernels_match_their_host_restatements(P, N):
    from poot_b200.ops import cuda_ops as K
    from poot_b200.utils import kernel_emulation as emu
    g = torch.Generator().manual_seed(0)
    nh, G, Kc, rows, T = 4, 2, 4, 3, 21
    I = nh * P
    C = I + 2 * G * N
    width = -(-(I + C + nh) // 8) * 8
    x = (torch.randn(T, width, generator=g) * 0.5).to(torch.bfloat16)
    w, cb = torch.randn(C, Kc, generator=g) * 0.3, torch.randn(C, generator=g) * 0.1
    segs = torch.tensor([[0, 8, 2, 0], [8, 1, 0, 5], [9, 12, 1, 16], [0, 0, 0, 0]], dtype=torch.int32)
    cstate = torch.randn(rows, Kc - 1, C, generator=g) * 0.2
    hstate = torch.randn(rows, nh, N, P, generator=g) * 0.05
    dt_bias, a_log, dskip = torch.randn(nh, generator=g) * 0.3, torch.log(torch.rand(nh, generator=g) * 3 + 0.5), torch.randn(nh, generator=g)
    gn = (1 + 0.1 * torch.randn(I, generator=g)).to(torch.bfloat16)
    c_ref, h_ref = cstate.clone(), hstate.clone()
    conv_ref = torch.zeros(T, C, dtype=torch.bfloat16)
    emu.causal_conv_silu(x, I, C, w, c_ref, segs, conv_ref, bias=cb)
    y_ref = torch.zeros(T, I, dtype=torch.bfloat16)
    emu.ssd_scan(conv_ref, x, I + C, dt_bias, a_log, dskip, h_ref, segs, y_ref, nh, G, N, P)
    n_ref = torch.zeros_like(y_ref)
    emu.gated_rmsnorm(y_ref, x, 0, gn, 1e-5, n_ref, G, I // G, gate_first=True)
    xd, segd, c_dev, h_dev = x.cuda(), segs.cuda(), cstate.cuda(), hstate.cuda()
    conv = torch.zeros(T, C, dtype=torch.bfloat16, device="cuda")
    K.causal_conv_silu(xd, I, C, w.cuda(), c_dev, segd, conv, bias=cb.cuda())
    y = torch.zeros(T, I, dtype=torch.bfloat16, device="cuda")
    K.ssd_scan(conv, xd, I + C, dt_bias.cuda(), a_log.cuda(), dskip.cuda(), h_dev, segd, y, nh, G, N, P)
    n = torch.zeros_like(y)
    K.gated_rmsnorm(y, xd, 0, gn.cuda(), 1e-5, n, G, I // G, gate_first=True)
    K.check_status()
    tol = lambda a, b: (a.float().cpu() - b.float()).abs().max().item() <= 0.02 * b.float().abs().max().item() + 2e-3
    assert tol(conv, conv_ref) and tol(c_dev, c_ref) and tol(y, y_ref) and tol(h_dev, h_ref) and tol(n, n_ref)


@pytest.mark.xfail(strict=False, reason="new kernels: not yet run on a device")
def test_small_pointwise_and_row_movement_kernels():
    """bias add (plain, strided, f32, per-expert), scale, row gather at three alignments, per-row sigmoid gate: each
    against the fp32 statement of the op."""
    from poot_b200.ops import cuda_ops as K
    g = torch.Generator().manual_seed(3)
    bf = lambda *s: (torch.randn(*s, generator=g)).to(torch.bfloat16).cuda()
    x, b = bf(37, 520), bf(520)
    ref = (x.float() + b.float()).to(torch.bfloat16)
    assert torch.equal(K.bias_add_(x.clone(), b), ref)
    assert torch.equal(K.bias_add_(x.clone(), b.float()), ref)
    wide = bf(37, 1040)
    want = wide.clone()
    want[:, 520:] = (wide[:, 520:].float() + b.float()).to(torch.bfloat16)
    K.bias_add_(wide[:, 520:], b)
    assert torch.equal(wide, want)
    lf, bfl = torch.randn(9, 130, generator=g).cuda(), torch.randn(130, generator=g).cuda()
    assert torch.equal(K.bias_add_(lf.clone(), bfl), lf + bfl)
    assert torch.equal(K.scale_(x.clone(), 0.37), (x.float() * 0.37).to(torch.bfloat16))
    table, idx = bf(6, 520), torch.tensor([2, -1, 5, 0], dtype=torch.int32).cuda()
    rows, gate = bf(32, 520), torch.rand(32, generator=g).cuda()
    e = idx.long().repeat_interleave(8)
    want = torch.where((e >= 0)[:, None],
                       (rows.float() + table[e.clamp(min=0)].float() * gate[:, None]).to(torch.bfloat16), rows)
    assert torch.equal(K.bias_add_indexed_(rows.clone(), table, idx, 8, 0, gate=gate), want)
    for dtype, width in ((torch.bfloat16, 520), (torch.float32, 131), (torch.bfloat16, 129)):
        src = torch.randn(50, width, generator=g).to(dtype).cuda()
        pick = torch.tensor([49, 0, 7, 7, 13], dtype=torch.int64).cuda()
        out = torch.zeros(5, width, dtype=dtype, device="cuda")
        assert torch.equal(K.gather_rows(src, pick, out), src[pick])
    gg = torch.randn(37, 8, generator=g).cuda()
    want = (x.float() * torch.sigmoid(gg[:, :1])).to(torch.bfloat16)
    got = K.sigmoid_gate_rows_(x.clone(), gg)
    assert (got.float() - want.float()).abs().max().item() <= 1e-2 * want.float().abs().max().item()


@pytest.mark.xfail(strict=False, reason="new kernels: not yet run on a device")
@pytest.mark.parametrize("ni,Di,dr,topk", [(6, 32, 32, 5), (64, 128, 64, 48), (32, 128, 64, 2048)])
def test_sparse_indexer_kernels_and_selected_attention(ni, Di, dr, topk):
    """Index-key write (LayerNorm + rotary + paged write), query rotary, scores over the visible keys, exact top-k
    selection and attention over the kept positions, each against the host restatement of the same entry point."""
    from poot_b200.ops import cuda_ops as K
    from poot_b200.utils import kernel_emulation as emu
    g = torch.Generator().manual_seed(7)
    T, blocks, max_pos = 40, 8, 128
    bf = lambda *s: (torch.randn(*s, generator=g) * 0.5).to(torch.bfloat16)
    kraw, nw, nb = bf(T, Di), (1 + 0.1 * torch.randn(Di, generator=g)).to(torch.bfloat16), bf(Di)
    pos = torch.arange(T, dtype=torch.int32)
    slots = (16 + pos).to(torch.int32)                      # blocks 1, 2, 3 of the pool
    ang = torch.rand(max_pos, max(dr // 2, 1), generator=g) * 6.28
    cos, sin = torch.cos(ang), torch.sin(ang)
    pool_ref = torch.zeros(blocks, 16, Di, dtype=torch.bfloat16)
    emu.index_k_write(kraw, nw, nb, 1e-6, pos, slots, cos, sin, pool_ref, dr)
    pool = torch.zeros(blocks, 16, Di, dtype=torch.bfloat16, device="cuda")
    K.index_k_write(kraw.cuda(), nw.cuda(), nb.cuda(), 1e-6, pos.cuda(), slots.cuda(), cos.cuda(), sin.cuda(), pool, dr)
    assert (pool.cpu().float() - pool_ref.float()).abs().max().item() <= 0.02 * pool_ref.float().abs().max().item()
    q = bf(T, ni * Di)
    q_ref = emu.index_q_rope(q.clone(), pos, cos, sin, ni, Di, dr)
    q_dev = K.index_q_rope(q.cuda(), pos.cuda(), cos.cuda(), sin.cuda(), ni, Di, dr)
    assert (q_dev.cpu().float() - q_ref.float()).abs().max().item() <= 0.02 * q_ref.float().abs().max().item()
    bt = torch.zeros(2, 4, dtype=torch.int32)
    bt[0, :3] = torch.tensor([1, 2, 3])
    ctx = (pos + 1).to(torch.int32)
    w = torch.rand(T, (ni + 7) // 8 * 8, generator=g)
    sc_ref = torch.full((T, 64), -7.0)
    emu.index_scores(q_ref, w, pool_ref, bt, None if False else torch.zeros(T, dtype=torch.int32), ctx, sc_ref, ni, Di, 64, Di ** -0.5)
    sc = torch.full((T, 64), -7.0, device="cuda")
    K.index_scores(q_ref.cuda(), w.cuda(), pool_ref.cuda(), bt.cuda(), torch.zeros(T, dtype=torch.int32, device="cuda"), ctx.cuda(),
                   sc, ni, Di, 64, Di ** -0.5)
    assert (sc.cpu() - sc_ref).abs().max().item() <= 2e-3 * max(1.0, sc_ref.abs().max().item())
    k_sel = min(topk, 24)
    sel_ref = torch.zeros(T, k_sel, dtype=torch.int32)
    emu.index_select(sc_ref, ctx, sel_ref)
    sel = torch.zeros(T, k_sel, dtype=torch.int32, device="cuda")
    K.index_select(sc_ref.cuda(), ctx.cuda(), sel)
    assert torch.equal(sel.cpu(), sel_ref)
    ties = torch.zeros(3, 64)
    ties[1, 5], ties[1, 9] = 1.0, float("nan")
    n = torch.tensor([64, 64, 3], dtype=torch.int32)
    want = torch.zeros(3, 4, dtype=torch.int32)
    emu.index_select(ties, n, want)
    got = torch.zeros(3, 4, dtype=torch.int32, device="cuda")
    K.index_select(ties.cuda(), n.cuda(), got)
    assert torch.equal(got.cpu(), want) and want[0].tolist() == [0, 1, 2, 3] and want[1].tolist() == [0, 1, 2, 5]
    Hq, Dk, Dv = 4, 64, 32
    aq, kp, vp = bf(T, Hq * Dk), bf(blocks, 1, 16, Dk), bf(blocks, 1, 16, Dk)
    out_ref = torch.zeros(T, Hq * Dv, dtype=torch.bfloat16)
    rs = torch.zeros(T, dtype=torch.int32)
    emu.attn_general(aq, kp, vp, bt, rs, ctx, Hq, 1, Dk, Dv, 0.125, out_ref, sel=sel_ref)
    out = torch.zeros(T, Hq * Dv, dtype=torch.bfloat16, device="cuda")
    K.attn_general(aq.cuda(), kp.cuda(), vp.cuda(), bt.cuda(), rs.cuda(), ctx.cuda(), Hq, 1, Dk, Dv, 0.125, out, sel=sel_ref.cuda())
    assert (out.cpu().float() - out_ref.float()).abs().max().item() <= 0.03 * out_ref.float().abs().max().item() + 2e-3


@pytest.mark.xfail(strict=False, reason="new kernels: not yet run on a device")
@pytest.mark.parametrize("world", [2, 4])
def test_tiled_gemm_tensor_parallel_form_with_every_rank_on_one_device(world):
    """The sharded program's prefill-sized pieces with all ranks' areas on one device and the phases launched rank after
    rank in one stream (a kernel never waits for a flag that is not set yet): norm + push (all-gather), tiled GEMM over
    the gathered rows, tiled GEMM scattering its rows to the owners' inboxes, reduce + norm."""
    from ctypes import c_float, c_int, c_void_p
    from poot_b200.ops import cuda_ops as K
    P = c_void_p
    K.register_signature("poot_tp_norm", [P, P, P, P, P, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                          P, P, P, P, P, P])
    K.register_signature("poot_gemm_tiled_tp", [c_int, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                c_int, c_int, P, P, P, P, c_int, P, P, P])
    H, N, R = 256, 384, 256
    S = R // world
    dev = "cuda"
    i32 = dict(dtype=torch.int32, device=dev)
    g = torch.Generator().manual_seed(5)
    bf = lambda *s: (torch.randn(*s, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    flags = [torch.zeros(6 * 8, **i32) for _ in range(world)]
    xs = [torch.zeros(2, R, H, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    inbox = [torch.zeros(2, world, S, H, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    arr = lambda ts: (c_void_p * world)(*[t.data_ptr() for t in ts])
    epoch = [torch.ones(1, **i32) for _ in range(world)]
    ticket = [torch.zeros(1, **i32) for _ in range(world)]
    st = K.status_word(torch.device(dev))
    h = [bf(S, H) for _ in range(world)]
    h0 = [t.clone() for t in h]
    wn = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).to(dev)
    Wcol = [bf(N, H) for _ in range(world)]            # column-parallel weight shares (qkv / gate_up kind)
    Wrow = [bf(H, N) for _ in range(world)]            # row-parallel weight shares (o / down kind)
    ck = lambda rc, what: (_ for _ in ()).throw(RuntimeError(f"{what}: CUDA error {rc}")) if rc else None
    ag_sites, rs_sites = 3, 2
    for r in range(world):                             # site 0: every rank normalises its rows and pushes them everywhere
        ck(K.fn("poot_tp_norm")(h[r].data_ptr(), inbox[r].data_ptr(), wn.data_ptr(), arr(xs), None, S, H, 1e-5, world, r, S, 0,
                                ag_sites, -1, rs_sites, epoch[r].data_ptr(), flags[r].data_ptr(), arr(flags), ticket[r].data_ptr(),
                                st.data_ptr(), K._stream()), "tp_norm")
    full = torch.cat(h0, 0).float()
    normed = (full * torch.rsqrt(full.pow(2).mean(-1, keepdim=True) + 1e-5) * wn.float()).to(torch.bfloat16)
    outs = []
    for r in range(world):                             # all-gather + GEMM
        out = torch.zeros(R, N, dtype=torch.bfloat16, device=dev)
        ck(K.fn("poot_gemm_tiled_tp")(0, xs[r].data_ptr(), Wcol[r].data_ptr(), out.data_ptr(), N, H, H, N, world, r, S, 0,
                                      ag_sites, -1, rs_sites, epoch[r].data_ptr(), flags[r].data_ptr(), arr(flags), None, H,
                                      ticket[r].data_ptr(), st.data_ptr(), K._stream()), "gemm ag")
        want = normed.float() @ Wcol[r].float().T
        assert (out.float() - want).abs().max().item() <= 0.02 * want.abs().max().item()
        outs.append(out)
    for r in range(world):                             # GEMM + reduce-scatter: rank r's partial of every row goes to its owner
        ck(K.fn("poot_gemm_tiled_tp")(0, outs[r].data_ptr(), Wrow[r].data_ptr(), None, H, N, N, H, world, r, S, -1, ag_sites, 0,
                                      rs_sites, epoch[r].data_ptr(), flags[r].data_ptr(), arr(flags), arr(inbox), H,
                                      ticket[r].data_ptr(), st.data_ptr(), K._stream()), "gemm rs")
    xl = [torch.zeros(S, H, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    for r in range(world):                             # the owner adds the ranks' partials in rank order and normalises
        ck(K.fn("poot_tp_norm")(h[r].data_ptr(), inbox[r].data_ptr(), wn.data_ptr(), None, xl[r].data_ptr(), S, H, 1e-5, world, r,
                                S, 0, ag_sites, 0, rs_sites, epoch[r].data_ptr(), flags[r].data_ptr(), arr(flags),
                                ticket[r].data_ptr(), st.data_ptr(), K._stream()), "tp_norm reduce")
    K.check_status()
    total = sum(outs[r].float() @ Wrow[r].float().T for r in range(world))
    for r in range(world):
        want = h0[r].float() + total[r * S:(r + 1) * S]
        assert (h[r].float() - want).abs().max().item() <= 0.03 * want.abs().max().item()
