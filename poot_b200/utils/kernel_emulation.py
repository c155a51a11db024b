"""Host restatements of the device kernels' entry points, for checking the engine's program on a machine
without a GPU.

``with emulated_kernels():`` replaces the functions of ``ops.cuda_ops`` / ``ops.moe_ops`` / ``ops.suffix_ops`` by
PyTorch code over CPU tensors with the same signatures, buffer layouts and rounding points (fp32 accumulation, bf16
stores where the kernels store bf16).  A ``DecoderEngine(device="cpu", use_graphs=False)`` built inside the block
then runs its unmodified kernel program - buffer binding, the order of launches, epilogue choices, K/V paging,
chained decode, the sampler suffix - and can be compared with the fp32 restatement of the model.  This is a test
harness only: nothing selects it automatically, the engine never falls back to it, and on a GPU box the ops keep
failing loudly when the CUDA library is missing.  What it cannot check is the kernels themselves; those are
compared with PyTorch references on the device.
"""
from __future__ import annotations

import math
from contextlib import contextmanager
from typing import Optional

import numpy as np
import torch

from ..ops import cuda_ops as K

BF = torch.bfloat16


def _bf(x: torch.Tensor) -> torch.Tensor:
    return x.to(BF)


def embed_gather(ids, table, out=None):
    r = table[ids.long()]
    if out is None:
        return r.clone()
    out.copy_(r)
    return out


def rmsnorm(x, w, eps, out=None, partials=None, h_out=None):
    h = x.float()
    if partials is not None:
        p = partials if partials.dim() == 3 else partials.unsqueeze(0)
        h = _bf(h + p.float().sum(0)).float()
        if h_out is not None:
            h_out.copy_(_bf(h))
    y = h / torch.sqrt((h * h).mean(-1, keepdim=True) + eps) * w.float()
    if out is None:
        return _bf(y)
    out.copy_(_bf(y))
    return out


def reduce_partials(h, partials, out):
    s = partials.float().sum(0)
    if h is not None:
        s = s + h.float()
    out.copy_(_bf(s))
    return out


def swiglu(gu, interleaved, out=None):
    g = gu.float()
    F = g.shape[1] // 2
    a = torch.nn.functional.silu(g[:, 0::2]) * g[:, 1::2] if interleaved else torch.nn.functional.silu(g[:, :F]) * g[:, F:]
    if out is None:
        return _bf(a)
    out.copy_(_bf(a))
    return out


def gated_act(gu, interleaved, act, out=None, limit=0.0, alpha=1.702):
    g = gu.float()
    F = g.shape[1] // 2
    gate, up = (g[:, 0::2], g[:, 1::2]) if interleaved else (g[:, :F], g[:, F:])
    if act == "swiglu_clamped":
        gate = gate.clamp(max=limit)
        r = _bf((up.clamp(-limit, limit) + 1.0) * gate * torch.sigmoid(alpha * gate))
    else:
        fn = {"silu": torch.nn.functional.silu, "gelu_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh"),
              "gelu_erf": torch.nn.functional.gelu}[act]
        r = _bf(fn(gate) * up)
    if out is None:
        return r
    out.copy_(r)
    return out


def layernorm(x, w, b, eps, out=None):
    h = x.float()
    mean = h.mean(-1, keepdim=True)
    var = ((h - mean) ** 2).mean(-1, keepdim=True)
    y = (h - mean) / torch.sqrt(var + eps) * w.float()
    if b is not None:
        y = y + b.float()
    if out is None:
        return _bf(y)
    out.copy_(_bf(y))
    return out


def act_(x, act):
    fn = {"silu": torch.nn.functional.silu, "gelu_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh"),
          "gelu_erf": torch.nn.functional.gelu, "relu2": lambda t: torch.relu(t) ** 2}[act]
    x.copy_(_bf(fn(x.float())))
    return x


def replace_rows_(h, rows, flags):
    sel = flags.bool()
    h[sel] = rows[sel]
    return h


def softcap_(x, cap):
    x.copy_(cap * torch.tanh(x / cap))
    return x


def causal_conv_silu(x, col0, C, w, state, segs, out, bias=None):
    Kc = w.shape[1]
    for first, n, seq, pos0 in segs.tolist():
        if n == 0:
            continue
        prev = torch.zeros(Kc - 1, C) if pos0 == 0 else state[seq].clone()
        xp = torch.cat([prev, x[first:first + n, col0:col0 + C].float()], 0)
        acc = sum(xp[k:k + n] * w[:, k] for k in range(Kc))
        if bias is not None:
            acc = acc + bias.float()
        out[first:first + n] = _bf(torch.nn.functional.silu(acc))
        state[seq] = xp[n:]
    return out


def gdn_scan(qkv, ba, b_col, a_col, dt_bias, a_log, state, segs, out, nk, nv, D):
    rep = nv // nk
    for first, n, seq, pos0 in segs.tolist():
        if n == 0:
            continue
        S = torch.zeros(nv, D, D) if pos0 == 0 else state[seq].clone()
        x = qkv[first:first + n].float()
        q = x[:, :nk * D].reshape(n, nk, D)
        k = x[:, nk * D:2 * nk * D].reshape(n, nk, D)
        v = x[:, 2 * nk * D:].reshape(n, nv, D)
        unit = lambda t: t / torch.sqrt((t * t).sum(-1, keepdim=True) + 1e-6)
        q = unit(q).repeat_interleave(rep, 1) * (D ** -0.5)
        k = unit(k).repeat_interleave(rep, 1)
        b = ba[first:first + n, b_col:b_col + nv].float()
        a = ba[first:first + n, a_col:a_col + nv].float()
        beta = torch.sigmoid(b)
        g = -torch.exp(a_log.float()) * torch.nn.functional.softplus(a + dt_bias.float())
        for t in range(n):
            S = S * torch.exp(g[t])[:, None, None]
            kv = torch.einsum("hk,hkv->hv", k[t], S)
            d = (v[t] - kv) * beta[t][:, None]
            S = S + k[t][:, :, None] * d[:, None, :]
            out[first + t] = _bf(torch.einsum("hk,hkv->hv", q[t], S).reshape(-1))
        state[seq] = S
    return out


def ngram_hash(tokens, history, segs, mult, primes, offsets, per_order, eos, vocab, ids):
    M = (1 << 64) - 1
    ctx, heads = history.shape[1], ids.shape[1]
    m = [int(v) & M for v in mult.tolist()]
    pr = [int(v) & 0xFFFFFFFF for v in primes.tolist()]
    off = offsets.tolist()
    for first, n, seq, pos0 in segs.tolist():
        if n == 0:
            continue
        before = [eos] * ctx if pos0 == 0 else [int(v) ^ eos for v in history[seq].tolist()]
        toks = [t if 0 <= t < vocab else 0 for t in tokens[first:first + n].tolist()]
        run = before + toks
        for i in range(n):
            s0, s1 = run[ctx + i], run[ctx + i - 1]
            mix2 = ((s0 * m[0]) & M) ^ ((s1 * m[1]) & M)
            for h in range(heads):
                mix = mix2
                if h >= per_order:
                    s2 = eos if s1 == eos else run[ctx + i - 2]
                    mix ^= (s2 * m[2]) & M
                ids[first + i, h] = mix % pr[h] + off[h]
        history[seq] = torch.tensor([v ^ eos for v in run[-ctx:]], dtype=history.dtype)
    return ids


def kda_scan(qkv, f, bm, b_col, dt_bias, a_log, lower_bound, state, segs, out, heads, D):
    C = heads * D
    for first, n, seq, pos0 in segs.tolist():
        if n == 0:
            continue
        S = torch.zeros(heads, D, D) if pos0 == 0 else state[seq].clone()
        x = qkv[first:first + n].float()
        unit = lambda t: t / torch.sqrt((t * t).sum(-1, keepdim=True) + 1e-6)
        q = unit(x[:, :C].reshape(n, heads, D)) * (D ** -0.5)
        k = unit(x[:, C:2 * C].reshape(n, heads, D))
        v = x[:, 2 * C:].reshape(n, heads, D)
        gate = torch.sigmoid(torch.exp(a_log.float())[None, :, None] * (f[first:first + n].float() + dt_bias.float()).reshape(n, heads, D))
        decay = torch.exp(lower_bound * gate)
        beta = torch.sigmoid(bm[first:first + n, b_col:b_col + heads].float())
        for t in range(n):
            S = S * decay[t][:, :, None]
            kv = torch.einsum("hk,hkv->hv", k[t], S)
            d = (v[t] - kv) * beta[t][:, None]
            S = S + k[t][:, :, None] * d[:, None, :]
            out[first + t] = _bf(torch.einsum("hk,hkv->hv", q[t], S).reshape(-1))
        state[seq] = S
    return out


def gated_rmsnorm(y, z, z_col, w, eps, out, heads, D, gate_first=False):
    T = y.shape[0]
    yy = y.float().reshape(T, heads, D)
    zz = torch.nn.functional.silu(z[:, z_col:z_col + heads * D].float().reshape(T, heads, D))
    ww = w.float().reshape(heads, D) if w.numel() == heads * D else w.float()
    if gate_first:
        v = yy * zz
        r = v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * ww
    else:
        r = yy / torch.sqrt((yy * yy).mean(-1, keepdim=True) + eps) * ww * zz
    out.copy_(_bf(r.reshape(T, heads * D)))
    return out


def ssd_scan(xbc, dtm, dt_col, dt_bias, a_log, dskip, state, segs, out, nh, groups, N, P):
    I, rep = nh * P, nh // groups
    for first, n, seq, pos0 in segs.tolist():
        if n == 0:
            continue
        H = torch.zeros(nh, N, P) if pos0 == 0 else state[seq].clone()
        r = xbc[first:first + n].float()
        x = r[:, :I].reshape(n, nh, P)
        B = r[:, I:I + groups * N].reshape(n, groups, N).repeat_interleave(rep, 1)
        C = r[:, I + groups * N:].reshape(n, groups, N).repeat_interleave(rep, 1)
        dt = torch.nn.functional.softplus(dtm[first:first + n, dt_col:dt_col + nh].float() + dt_bias.float())
        A = -torch.exp(a_log.float())
        for t in range(n):
            H = torch.exp(dt[t] * A)[:, None, None] * H + (dt[t][:, None] * B[t])[:, :, None] * x[t][:, None, :]
            y = torch.einsum("hn,hnp->hp", C[t], H) + dskip.float()[:, None] * x[t]
            out[first + t] = _bf(y.reshape(-1))
        state[seq] = H
    return out


def sigmoid_mul(a, g):
    a.copy_(_bf(a.float() * torch.sigmoid(g.float())))
    return a


def add(a, b, out=None):
    r = _bf(a.float() + b.float())
    if out is None:
        return r
    out.copy_(r)
    return out


def bias_add_(x, bias):
    x.copy_((x.float() + bias.float()).to(x.dtype))
    return x


def bias_add_indexed_(x, table, idx, div=1, e0=0, gate=None):
    R = x.shape[0]
    e = idx.long().repeat_interleave(div)[:R]
    live = (e >= 0) & (e + e0 < table.shape[0])
    b = table[(e + e0).clamp(0, table.shape[0] - 1)].float()
    if gate is not None:
        b = b * gate[:R, None]
    x.copy_(torch.where(live[:, None], _bf(x.float() + b), x))
    return x


def scale_(x, s):
    x.copy_(_bf(x.float() * s))
    return x


def gather_rows(src, idx, out):
    out.copy_(src[idx[:out.shape[0]].clamp(0, src.shape[0] - 1)])
    return out


def sigmoid_gate_rows_(x, g):
    x.copy_(_bf(x.float() * torch.sigmoid(g[:, :1])))
    return x


def _epilogue(y: torch.Tensor, epi: int, out, resid):
    """``y`` fp32 ``[M, N]`` -> the epilogue's stored form."""
    if epi == K.EPI_F32:
        r = y
    elif epi == K.EPI_SWIGLU:
        r = _bf(torch.nn.functional.silu(y[:, 0::2]) * y[:, 1::2])
    elif epi == K.EPI_RESID:
        r = _bf(y + resid.float())
    else:
        r = _bf(y)
    if out is None:
        return r.clone()
    out.copy_(r)
    return out


def _planar_f32(W) -> torch.Tensor:
    """The decoded weight of a ``PlanarWeight`` through the host codec (cached on the object)."""
    w = getattr(W, "_emulated_f32", None)
    if w is None:
        from ..quant import codec
        np_ = lambda t: None if t is None else t.cpu().numpy()
        if W.fmt in ("GPTQ", "AWQ"):
            ops = {"qweight": np_(W.w), "qzeros": np_(W.zeros), "scales": np_(W.scale)}
            if W.g_idx is not None:
                ops["g_idx"] = np_(W.g_idx)
        else:
            key = "weight_scale_inv" if W.fmt == "E4M3_BLOCK128" else "weight_scale"
            ops = {"weight": np_(W.w), key: np_(W.scale)}
        w = torch.from_numpy(codec.dequantize_planar(W.fmt, ops, W.group).astype("float32"))
        W._emulated_f32 = w
    return w


def _packed_expert_f32(P, which: str, e: int) -> torch.Tensor:
    cache = P.__dict__.setdefault("_emulated", {})
    if (which, e) not in cache:
        from ..quant import codec
        w, sc = getattr(P, which)
        key = "weight_scale_inv" if P.fmt == "E4M3_BLOCK128" else "weight_scale"
        cache[(which, e)] = torch.from_numpy(codec.dequantize_planar(P.fmt, {"weight": w[e].cpu().numpy(), key: sc[e].cpu().numpy()}).astype("float32"))
    return cache[(which, e)]


def planar_gemv_grouped(x, P, which, ids, out, groups, x_row_div=0, row_scale=None, act="silu", alpha=1.702, limit=0.0):
    for g in range(groups):
        e = int(ids[g]) if ids is not None else g
        if e < 0 or e >= P.E:
            out[g, :(P.F if which == "in" else P.H)] = 0
            continue
        xr = x[g // x_row_div if x_row_div > 0 else g].float()
        if which == "in":
            gt, up = _packed_expert_f32(P, "gate", e) @ xr, _packed_expert_f32(P, "up", e) @ xr
            if P.bias_gate is not None:
                gt, up = gt + P.bias_gate[e].float(), up + P.bias_up[e].float()
            if limit > 0:
                gt, up = gt.clamp(max=limit), up.clamp(-limit, limit)
                v = (up + 1.0) * gt * torch.sigmoid(alpha * gt)
            else:
                v = torch.nn.functional.silu(gt) * up
            out[g, :P.F] = _bf(v)
        else:
            v = _packed_expert_f32(P, "down", e) @ xr
            if P.bias_down is not None:
                v = v + P.bias_down[e].float()
            if row_scale is not None:
                v = v * row_scale[g]
            out[g, :P.H] = _bf(v)
    return out


def linear(x, W, epi=K.EPI_STORE, out=None, resid=None):
    if isinstance(W, K.QuantWeight):
        raise NotImplementedError("packed weights are not emulated")
    if isinstance(W, K.PlanarWeight):
        w = _planar_f32(W)
        if x.shape[0] > 4:              # larger steps decode the weight to bf16 first and multiply with the dense GEMM
            w = _bf(w).float()
        return _epilogue(x.float() @ w.T, epi, out, resid)
    return _epilogue(x.float() @ W.float().T, epi, out, resid)


def gemm(x, W, epi=K.EPI_STORE, out=None, resid=None, bn=None, splits=1):
    if epi == K.EPI_PARTIAL:        # split-K partial slices: the sum over slices is the product
        y = x.float() @ W.float().T
        if out is None:
            out = torch.zeros(splits, *y.shape, dtype=torch.float32)
        out.zero_()
        Kd = x.shape[1]
        step = -(-Kd // splits)
        for s in range(splits):
            out[s].copy_(x[:, s * step:(s + 1) * step].float() @ W[:, s * step:(s + 1) * step].float().T)
        return out
    return linear(x, W, epi, out, resid)


def gemm_skinny(x, W, epi=K.EPI_STORE, out=None, resid=None, ck=None, wm=1):
    assert x.shape[0] <= 128
    return linear(x, W, epi, out, resid)


def gemv(x, W, epi=K.EPI_STORE, out=None, resid=None):
    return linear(x, W, epi, out, resid)


def rope_kv_write(qkv, q_out, kpool, vpool, positions, slots, cos, sin, Hq, Hkv, D, rot=None, q_norm_w=None,
                  k_norm_w=None, norm_eps=1e-6):
    T = qkv.shape[0]
    rot = D if rot is None else rot
    half = rot // 2
    x = qkv.float()
    q = x[:, :Hq * D].reshape(T, Hq, D)
    k = x[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D)
    v = x[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)

    def norm(t, w):
        return t if w is None else t / torch.sqrt((t * t).mean(-1, keepdim=True) + norm_eps) * w.float()

    def rope(t):
        c = cos[positions.long()].unsqueeze(1)      # [T, 1, half]
        s = sin[positions.long()].unsqueeze(1)
        a, b = t[..., :half], t[..., half:rot]
        return torch.cat([a * c - b * s, b * c + a * s, t[..., rot:]], -1)

    q, k = rope(norm(q, q_norm_w)), rope(norm(k, k_norm_w))
    q_out.copy_(_bf(q.reshape(T, Hq * D)))
    live = slots >= 0
    if live.any():
        sl = slots[live].long()
        kpool[sl // K.KV_BLOCK, :, sl % K.KV_BLOCK] = _bf(k[live])
        vpool[sl // K.KV_BLOCK, :, sl % K.KV_BLOCK] = _bf(v[live])


def _attend(qrow: torch.Tensor, kpool, vpool, blocks: torch.Tensor, first_key: int, n_keys: int, Hq: int, Hkv: int,
            D: int, scale: float, softcap: float) -> torch.Tensor:
    """One query row ``[Hq, D]`` over keys ``first_key .. n_keys-1`` of the sequence whose block list is ``blocks``."""
    pos = torch.arange(first_key, n_keys)
    blk = blocks[(pos // K.KV_BLOCK).long()].long()
    kk = kpool[blk, :, (pos % K.KV_BLOCK).long()].float()      # [S, Hkv, D]
    vv = vpool[blk, :, (pos % K.KV_BLOCK).long()].float()
    rep = Hq // Hkv
    kk, vv = kk.repeat_interleave(rep, 1), vv.repeat_interleave(rep, 1)
    s = torch.einsum("hd,shd->hs", qrow.float(), kk) * scale
    if softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    return torch.einsum("hs,shd->hd", torch.softmax(s, -1), vv)


def attn_paged(q, kpool, vpool, block_tables, row_seq, row_ctx, Hq, Hkv, D, scale, out=None, splits=1, scratch=None,
               softcap=0.0, window=0):
    R = q.shape[0]
    if out is None:
        out = torch.zeros(R, Hq * D, dtype=BF)
    for r in range(R):
        ctx = int(row_ctx[r])
        if ctx <= 0:
            continue
        seq = int(row_seq[r]) if row_seq is not None else r
        first = ctx - window if (window > 0 and ctx > window) else 0
        o = _attend(q[r].reshape(Hq, D), kpool, vpool, block_tables[seq], first, ctx, Hq, Hkv, D, scale, softcap)
        out[r].copy_(_bf(o.reshape(-1)))
    return out


def mla_qkv_write(q, kvb, kva, rope_col, q_out, kpool, vpool, positions, slots, cos, sin, nh, dn, dr, dv):
    T, half = q.shape[0], dr // 2
    c = cos[positions.long()].unsqueeze(1)
    s = sin[positions.long()].unsqueeze(1)

    def rot(t):
        a, b = t[..., :half], t[..., half:]
        return torch.cat([a * c - b * s, b * c + a * s], -1)

    qq = q.float().reshape(T, nh, dn + dr)
    q_out.copy_(_bf(torch.cat([qq[..., :dn], rot(qq[..., dn:])], -1).reshape(T, -1)))
    kb = kvb.float().reshape(T, nh, dn + dv)
    kr = rot(kva[:, rope_col:rope_col + dr].float().reshape(T, 1, dr)).expand(T, nh, dr)
    kfull = torch.cat([kb[..., :dn], kr], -1)
    live = slots >= 0
    if live.any():
        sl = slots[live].long()
        kpool[sl // K.KV_BLOCK, :, sl % K.KV_BLOCK] = _bf(kfull[live])
        vpool[sl // K.KV_BLOCK, :, sl % K.KV_BLOCK, :dv] = _bf(kb[live][..., dn:])


def attn_general(q, kpool, vpool, block_tables, row_seq, row_ctx, Hq, Hkv, Dk, Dv, scale, out, softcap=0.0, window=0,
                 alibi=None, sinks=None, sel=None):
    rep = Hq // Hkv
    for r in range(q.shape[0]):
        ctx = int(row_ctx[r])
        if ctx <= 0:
            continue
        seq = int(row_seq[r]) if row_seq is not None else r
        first = ctx - window if (window > 0 and ctx > window) else 0
        pos = torch.arange(first, ctx)
        if sel is not None:
            pos = sel[r].long()
            pos = pos[(pos >= 0) & (pos < ctx)]
        blk = block_tables[seq][(pos // K.KV_BLOCK).long()].long()
        kk = kpool[blk, :, (pos % K.KV_BLOCK).long()][..., :Dk].float().repeat_interleave(rep, 1)     # [S, Hq, Dk]
        vv = vpool[blk, :, (pos % K.KV_BLOCK).long()][..., :Dv].float().repeat_interleave(rep, 1)
        s = torch.einsum("hd,shd->hs", q[r, :Hq * Dk].reshape(Hq, Dk).float(), kk) * scale
        if softcap > 0:
            s = softcap * torch.tanh(s / softcap)
        if alibi is not None:
            s = s + alibi.float()[:, None] * (pos - (ctx - 1)).float()[None, :]
        if sinks is not None:
            full = torch.cat([s, sinks.float()[:, None]], 1)
            p = torch.softmax(full, -1)[:, :-1]
        else:
            p = torch.softmax(s, -1)
        out[r, :Hq * Dv] = _bf(torch.einsum("hs,shd->hd", p, vv).reshape(-1))
    return out


def _half_rope(x, cos_row, sin_row, dr):
    """Half-split rotary on the leading ``dr`` channels of the last axis."""
    half = dr // 2
    x1, x2 = x[..., :half], x[..., half:dr]
    return torch.cat([x1 * cos_row - x2 * sin_row, x2 * cos_row + x1 * sin_row, x[..., dr:]], -1)


def index_k_write(kraw, norm_w, norm_b, eps, positions, slots, cos, sin, pool, dr):
    T, Di = kraw.shape
    x = kraw.float()
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    y = (x - mean) * torch.rsqrt(var + eps) * norm_w.float() + (norm_b.float() if norm_b is not None else 0.0)
    y = _bf(y).float()                                      # the kernel rounds the normalised row before rotating it
    flat = pool.view(-1, Di)
    for t in range(T):
        slot = int(slots[t])
        if slot < 0:
            continue
        p = min(max(int(positions[t]), 0), cos.shape[0] - 1)
        flat[slot] = _bf(_half_rope(y[t], cos[p], sin[p], dr)) if dr else _bf(y[t])


def index_q_rope(q, positions, cos, sin, ni, Di, dr):
    if dr == 0:
        return q
    T = q.shape[0]
    p = positions[:T].long().clamp(0, cos.shape[0] - 1)
    x = q.view(T, ni, Di).float()
    q.copy_(_bf(_half_rope(x, cos[p][:, None, :], sin[p][:, None, :], dr)).view(T, ni * Di))
    return q


def index_scores(q, w, pool, block_tables, row_seq, row_ctx, scores, ni, Di, max_ctx, scale):
    flat = pool.view(-1, Di)
    for r in range(q.shape[0]):
        ctx = int(row_ctx[r])
        if ctx <= 0:
            continue
        seq = int(row_seq[r]) if row_seq is not None else r
        pos = torch.arange(ctx)
        keys = flat[block_tables[seq][(pos // K.KV_BLOCK).long()].long() * K.KV_BLOCK + pos % K.KV_BLOCK].float()   # [ctx, Di]
        dots = torch.relu(q[r].view(ni, Di).float() @ keys.T * scale)                                                # [ni, ctx]
        scores[r, :ctx] = (w[r, :ni].float()[:, None] * dots).sum(0)
    return scores


def index_select(scores, row_ctx, sel):
    k = sel.shape[1]
    sel.fill_(-1)
    for r in range(sel.shape[0]):
        n = max(int(row_ctx[r]), 0)
        if n <= k:
            sel[r, :n] = torch.arange(n, dtype=sel.dtype)
            continue
        s = scores[r, :n].float().clone()
        s[torch.isnan(s) | (s == float("-inf"))] = torch.finfo(torch.float32).min
        order = torch.sort(s, descending=True, stable=True).indices[:k]        # ties: lowest position first
        sel[r] = torch.sort(order).values.to(sel.dtype)
    return sel


def attn_flash_prefill(q, kpool, vpool, block_tables, tiles, Hq, Hkv, scale, out, window=0):
    D = kpool.shape[-1]
    for first_row, rows, seq, first_pos in tiles.tolist():
        for i in range(rows):
            ctx = first_pos + i + 1
            first = ctx - window if (window > 0 and ctx > window) else 0
            o = _attend(q[first_row + i].reshape(Hq, D), kpool, vpool, block_tables[seq], first, ctx, Hq, Hkv, D, scale, 0.0)
            out[first_row + i].copy_(_bf(o.reshape(-1)))


def argmax_scratch(rows, vocab, device):
    return torch.zeros(rows, K.argmax_groups(vocab), 3, dtype=torch.int32)


def argmax(logits, out=None, scratch=None):
    from ..oracle.sampling import GREEDY, sample_rows
    r = torch.from_numpy(sample_rows(logits.float().numpy(), None, None, None, GREEDY))
    if out is None:
        return r
    out.copy_(r)
    return out


def argmax_partials(logits, idx_offset, vocab_total, part):
    """Stage 1 over one vocabulary shard: per (row, chunk) the best finite value (as its bit pattern), its global index
    and the first non-finite global index (``vocab_total`` when there is none)."""
    rows, vocab = logits.shape
    chunk = K.ARGMAX_CHUNK
    x = logits.float()
    for g in range(part.shape[1]):
        seg = x[:, g * chunk:(g + 1) * chunk]
        fin = torch.isfinite(seg)
        masked = torch.where(fin, seg, torch.full_like(seg, -float("inf")))
        best = masked.argmax(-1)                                        # first maximum
        val = masked.gather(-1, best[:, None])[:, 0]
        any_fin = fin.any(-1)
        part[:, g, 0] = torch.where(any_fin, val, torch.zeros_like(val)).view(torch.int32)
        part[:, g, 1] = torch.where(any_fin, best + idx_offset + g * chunk, torch.full_like(best, -1)).to(torch.int32)
        bad = torch.where(fin, torch.full_like(seg, float(vocab_total)),
                          (torch.arange(seg.shape[1]) + idx_offset + g * chunk).float().expand_as(seg)).min(-1).values
        part[:, g, 2] = bad.to(torch.int32)
    return part


def argmax_combine(parts, rows, groups, vocab_total, out):
    p = parts.reshape(-1, rows, groups, 3).permute(1, 0, 2, 3).reshape(rows, -1, 3)
    for r in range(rows):
        vals = p[r, :, 0].contiguous().view(torch.float32)
        idx = p[r, :, 1]
        live = idx >= 0
        bad = int(p[r, :, 2].min())
        tok = 0
        if live.any():
            v = torch.where(live, vals, torch.full_like(vals, -float("inf")))
            m = v.max()
            tok = int(idx[(v == m) & live].min())
        out[r, 0] = 0 if bad < vocab_total else tok
        out[r, 1] = bad if bad < vocab_total else -1
    return out


def sample_gumbel(logits, params, top_k, seeds, rule, out=None):
    from ..oracle.sampling import sample_rows
    r = torch.from_numpy(sample_rows(logits.float().numpy(), params.numpy(), top_k.numpy(), seeds.numpy(), rule))
    if out is None:
        return r
    out.copy_(r)
    return out


def decode_advance(picked, tokens, positions, slots, ctx, block_tables, row_seq, B):
    maxb = block_tables.shape[1]
    for i in range(B):
        if int(slots[i]) < 0:
            continue
        tokens[i] = picked[i, 0]
        pos = int(positions[i]) + 1
        positions[i] = pos
        ctx[i] = pos + 1
        seq = int(row_seq[i]) if row_seq is not None else i
        b = pos // K.KV_BLOCK
        slots[i] = int(block_tables[seq, b]) * K.KV_BLOCK + pos % K.KV_BLOCK if b < maxb else -1


def adjust_logits(logits, idx, val, guided=None):
    fmin = torch.finfo(torch.float32).min
    for r in range(logits.shape[0]):
        for t, v in zip(idx[r].tolist(), val[r].tolist()):
            if 0 <= t < logits.shape[1]:
                l = float(logits[r, t]) + v[0]
                logits[r, t] = (l * v[1] if l > 0 else l * v[2]) + v[3]
        if guided is not None:
            m = guided[r]
            logits[r] = torch.where(m <= fmin, torch.full_like(m, fmin), torch.where(m != 0, logits[r] + m, logits[r]))


def token_logprob(logits, picked, out=None):
    lp = torch.log_softmax(logits.float(), -1)[torch.arange(logits.shape[0]), picked[:, 0].long()]
    if out is None:
        return lp
    out.copy_(lp)
    return out


def moe_route(logits, k, renorm, ids, gates, dense, mode="softmax", select_bias=None, scale=1.0, n_group=1, topk_group=1):
    T, E = logits.shape
    s = torch.nan_to_num(logits.float(), nan=torch.finfo(torch.float32).min, posinf=torch.finfo(torch.float32).max,
                         neginf=torch.finfo(torch.float32).min)
    if mode == "sigmoid":
        score = torch.sigmoid(s)
        rankv = score + (select_bias.float() if select_bias is not None else 0.0)
        if n_group > 1:
            gs = rankv.reshape(T, n_group, E // n_group).topk(2, dim=-1).values.sum(-1)
            gorder = torch.sort(gs, dim=-1, descending=True, stable=True).indices[:, :topk_group]
            keep = torch.zeros(T, n_group, dtype=torch.bool).scatter_(1, gorder, True)
            rankv = torch.where(keep.repeat_interleave(E // n_group, 1), rankv, torch.zeros_like(rankv))
        order = torch.sort(rankv, dim=-1, descending=True, stable=True).indices[:, :k]
        g = score.gather(-1, order)
        if renorm:
            g = g / (g.sum(-1, keepdim=True) + 1e-20)
    else:
        order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :k]       # ties: lower index first
        top = s.gather(-1, order)
        g = torch.softmax(top, -1) if renorm else torch.softmax(s, -1).gather(-1, order)
    g = g * scale
    ids.view(T, k).copy_(order.to(torch.int32))
    gates.view(T, k).copy_(g)
    d = dense.view(E, T)
    d.zero_()
    d.T.scatter_(1, order, g)


def moe_combine(h, parts, out, T, H, groups, gstride, per_token=0):
    p = parts.reshape(-1).float()
    acc = torch.zeros(T, H) if h is None else h.float().clone()
    if per_token:      # group g belongs to token g / per_token
        for g in range(groups):
            acc[g // per_token] += p[g * gstride:g * gstride + H]
    else:
        for g in range(groups):
            acc += p[g * gstride:g * gstride + T * H].view(T, H)
    out.copy_(_bf(acc))


def gemm_grouped(epi, x, W, out, M, groups, group_expert=None, x_row_div=0, x_row_mul=0, x_col_per_expert=0,
                 out_group_stride=0, row_scale=None, ldo=None, K_dim=None, tp=None):
    if tp is not None:
        # one group whose result goes to every rank's inbox: compute it into a scratch, then push through the comm
        comm, rs_site = tp
        if not hasattr(comm, "push_rows"):
            raise NotImplementedError("peer pushes are emulated over utils.tp_emulation only")
        scratch = torch.zeros(M, W.shape[1], dtype=torch.bfloat16)
        gemm_grouped(epi, x, W, scratch, M, groups, group_expert, x_row_div, x_row_mul, x_col_per_expert, 0, row_scale,
                     W.shape[1], K_dim)
        comm.push_rows(scratch, M, rs_site)
        return
    E, N, Kw = W.shape
    Kd = K_dim or Kw
    n_out = N // 2 if epi == K.EPI_SWIGLU else N
    flat = out.reshape(-1)
    for g in range(groups):
        e = int(group_expert[g]) if group_expert is not None else g
        row0 = (g // x_row_div if x_row_div > 0 else 0) + g * x_row_mul
        col0 = e * x_col_per_expert
        if e < 0:
            y = torch.zeros(M, N)
        else:
            y = x[row0:row0 + M, col0:col0 + Kd].float() @ W[e].float().T
        if row_scale is not None:
            y = y * row_scale.reshape(-1)[g * M:(g + 1) * M].float().unsqueeze(1)
        r = _bf(torch.nn.functional.silu(y[:, 0::2]) * y[:, 1::2]) if epi == K.EPI_SWIGLU else _bf(y)
        for m in range(M):
            o = g * out_group_stride + m * ldo
            flat[o:o + n_out] = r[m]


def moe_align(ids, e0, e_local, block, max_tiles, pos, sorted_rows, tile_expert, n_tiles):
    from ..plan.moe_align import group_expert_rows
    flat = ids.reshape(-1).long()
    local = (flat >= e0) & (flat < e0 + e_local)
    idx = torch.nonzero(local).reshape(-1)
    rows, tiles, padded = group_expert_rows((flat[idx] - e0).numpy(), e_local, block)
    sorted_rows.fill_(-1)
    pos.fill_(-1)
    tile_expert.fill_(-1)
    n_tiles[0] = padded // block
    if padded:
        sr = torch.from_numpy(rows)
        live = sr >= 0
        mapped = torch.where(live, idx[sr.clamp(min=0)], torch.full_like(sr, -1))
        sorted_rows[:padded] = mapped.to(sorted_rows.dtype)
        pos[mapped[live]] = torch.nonzero(live).reshape(-1).to(pos.dtype)
        tile_expert[:padded // block] = torch.from_numpy(tiles)


def moe_gather_rows(x, sorted_rows, gates, n_tiles, block, max_tiles, k, xs, gate_sorted):
    n = int(n_tiles[0]) * block
    sr = sorted_rows[:n].long()
    live = sr >= 0
    xs[:n] = torch.where(live[:, None], x[(sr.clamp(min=0) // k)], torch.zeros_like(xs[:n]))
    gate_sorted[:n] = torch.where(live, gates.reshape(-1)[sr.clamp(min=0)], torch.zeros_like(gate_sorted[:n]))


def moe_scatter_combine(h, y, pos, out, T, H, k):
    acc = h[:T].float().clone() if h is not None else torch.zeros(T, H)
    p = pos[:T * k].view(T, k).long()
    for j in range(k):                                      # slot order, as the kernel adds
        live = p[:, j] >= 0
        acc = acc + torch.where(live[:, None], y[p[:, j].clamp(min=0)].float(), torch.zeros(T, H))
    out[:T].copy_(_bf(acc))


def moe_scatter_combine_push(y, pos, T, H, k, tp):
    comm, rs_site = tp
    part = torch.zeros(T, H, dtype=torch.bfloat16)
    moe_scatter_combine(None, y, pos, part, T, H, k)
    comm.push_rows(part, T, rs_site)


def gemm_grouped_tiled(epi, x, W, out, tile_expert, row_scale=None):
    for t, ex in enumerate(tile_expert.tolist()):
        if ex < 0:
            continue
        rows = slice(t * 128, (t + 1) * 128)
        y = x[rows].float() @ W[ex].float().T
        if row_scale is not None:
            y = y * row_scale[rows].reshape(-1, 1)
        _epilogue(y, epi, out[rows], None)


_status = torch.zeros(16, dtype=torch.int32)


@contextmanager
def emulated_kernels():
    """Run the engine's kernel program against the host restatements above (tests only)."""
    from ..ops import moe_ops, suffix_ops
    table = {
        K: dict(embed_gather=embed_gather, rmsnorm=rmsnorm, reduce_partials=reduce_partials, swiglu=swiglu, add=add,
                gated_act=gated_act, softcap_=softcap_, layernorm=layernorm, act_=act_, replace_rows_=replace_rows_, causal_conv_silu=causal_conv_silu, gdn_scan=gdn_scan, kda_scan=kda_scan, ngram_hash=ngram_hash, planar_gemv_grouped=planar_gemv_grouped, ssd_scan=ssd_scan,
                gated_rmsnorm=gated_rmsnorm, sigmoid_mul=sigmoid_mul,
                bias_add_=bias_add_, bias_add_indexed_=bias_add_indexed_, scale_=scale_, gather_rows=gather_rows,
                sigmoid_gate_rows_=sigmoid_gate_rows_,
                linear=linear, gemm=gemm, gemm_skinny=gemm_skinny, gemv=gemv, rope_kv_write=rope_kv_write,
                index_k_write=index_k_write, index_q_rope=index_q_rope, index_scores=index_scores,
                index_select=index_select,
                attn_paged=attn_paged, attn_general=attn_general, mla_qkv_write=mla_qkv_write, attn_flash_prefill=attn_flash_prefill, argmax_scratch=argmax_scratch,
                argmax=argmax, argmax_partials=argmax_partials, argmax_combine=argmax_combine,
                sample_gumbel=sample_gumbel, decode_advance=decode_advance,
                status_word=lambda device=None: _status, check_status=lambda device=None: None),
        moe_ops: dict(moe_route=moe_route, moe_combine=moe_combine, gemm_grouped=gemm_grouped, moe_align=moe_align,
                      moe_gather_rows=moe_gather_rows, moe_scatter_combine=moe_scatter_combine,
                      moe_scatter_combine_push=moe_scatter_combine_push,
                      gemm_grouped_tiled=gemm_grouped_tiled),
        suffix_ops: dict(adjust_logits=adjust_logits, token_logprob=token_logprob),
    }
    saved = {(mod, name): getattr(mod, name) for mod, fns in table.items() for name in fns}
    try:
        for mod, fns in table.items():
            for name, fn in fns.items():
                setattr(mod, name, fn)
        yield
    finally:
        for (mod, name), fn in saved.items():
            setattr(mod, name, fn)
