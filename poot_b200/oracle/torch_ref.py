"""Plain PyTorch fp32 restatement of the decoder stack, used as the numerics reference of the device engine.

It consumes the same fused weight layouts as the engine (``DecoderWeights`` at world size 1), runs a whole
sequence with a dense causal mask, and follows the op definitions of the reference's op library: RMSNorm
``x / sqrt(mean(x^2)+eps) * w`` (crates/poot-graph-ir/src/ops/norm.rs:18-29), half-split RoPE (ops/rope.rs:30-58),
``silu(g)*u`` (ops/activation.rs:94-143), blocked GQA ``repeat_kv`` and masked softmax attention
(ops/attention.rs:260-337), Mixtral routing (softmax over the selected top-k, ops/moe.rs).  Constant multipliers of a
family (residual and logit scales) are already folded into the weights it is given; the embedding scale and the q/k/v
bias are applied here as the engine applies them.
"""
from __future__ import annotations

import math

import torch

from ..models.config import DecoderConfig
from ..runtime.rope import rope_tables
from ..runtime.weights import DecoderWeights


def rmsnorm(x, w, eps):
    x = x.float()
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.float()


def rope(x, cos, sin, rot):
    # x [T, H, D]; cos/sin [T, rot/2]
    half = rot // 2
    x1, x2, rest = x[..., :half], x[..., half:rot], x[..., rot:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)


def moe_ffn(cfg: DecoderConfig, L, x):
    logits = x @ L.router.float().T
    top_v, top_i = torch.topk(logits, cfg.top_k, dim=-1)  # ties: lower index first for equal values
    if cfg.norm_topk_prob:
        gates = torch.softmax(top_v, dim=-1)
    else:       # softmax over all experts, read at the selected ones, not renormalised
        gates = torch.softmax(logits, dim=-1).gather(-1, top_i)
    out = torch.zeros_like(x)
    for e in range(cfg.n_experts):
        sel = (top_i == e)
        if not sel.any():
            continue
        rows = sel.any(-1)
        g = (gates * sel).sum(-1)[rows]
        xe = x[rows]
        gu = xe @ L.ex_wgu[e].float().T
        a = torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]
        out[rows] += (a @ L.ex_wdown[e].float().T) * g[:, None]
    return out


@torch.no_grad()
def forward_logits(w: DecoderWeights, tokens: torch.Tensor, round_bf16: bool = True) -> torch.Tensor:
    """Logits ``[T, vocab]`` (fp32) for one sequence of token ids with positions ``0..T-1``.

    ``round_bf16`` rounds activations to bf16 where the device engine stores them in bf16, so the comparison
    measures kernel error and not the storage format.
    """
    cfg = w.cfg
    dev = w.embed.device
    T = tokens.numel()
    D, Hq, Hkv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads

    def r(t):
        return t.to(torch.bfloat16).float() if round_bf16 else t

    cos, sin = rope_tables(cfg, T)
    cos, sin = cos.to(dev), sin.to(dev)
    h = w.embed[tokens.long()].float()
    if cfg.embed_scale != 1.0:
        h = r(h * cfg.embed_scale)
    pos = torch.arange(T, device=dev)
    causal = pos[None, :] <= pos[:, None]
    scale = float(cfg.attn_scale) if cfg.attn_scale is not None else 1.0 / math.sqrt(D)
    for li, L in enumerate(w.layers):
        mask = causal
        if cfg.window_of(li) > 0:
            mask = causal & (pos[None, :] > (pos[:, None] - cfg.window_of(li)))
        x = r(rmsnorm(h, L.ln1, cfg.norm_eps))
        qkv = x @ L.wqkv.float().T
        if L.bqkv is not None:
            qkv = r(qkv) + L.bqkv.float()
        qkv = r(qkv)
        q = qkv[:, :Hq * D].view(T, Hq, D)
        k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
        v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        if L.q_norm is not None:
            q = r(rmsnorm(q, L.q_norm, cfg.norm_eps))
            k = r(rmsnorm(k, L.k_norm, cfg.norm_eps))
        q = r(rope(q, cos, sin, cfg.rot))
        k = r(rope(k, cos, sin, cfg.rot))
        kk = k.repeat_interleave(cfg.n_rep, dim=1)
        vv = v.repeat_interleave(cfg.n_rep, dim=1)
        s = torch.einsum("thd,shd->hts", q, kk) * scale
        if cfg.attn_softcap > 0:
            s = cfg.attn_softcap * torch.tanh(s / cfg.attn_softcap)
        s = s.masked_fill(~mask[None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        a = r(torch.einsum("hts,shd->thd", p, vv).reshape(T, Hq * D))
        h = r(h + a @ L.wo.float().T)
        x = r(rmsnorm(h, L.ln2, cfg.norm_eps))
        if cfg.is_moe:
            h = r(h + moe_ffn(cfg, L, x))
        else:
            gu = x @ L.wgu.float().T
            act = r(torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2])
            h = r(h + act @ L.wdown.float().T)
    x = r(rmsnorm(h, w.final_norm, cfg.norm_eps))
    return x @ w.lm_head.float().T
