"""BERT-style encoders on the device: the program of ``models/encoder.py`` over the decoder engine's kernels
(crates/poot-models/src/architectures/bert.rs: embedders and cross-encoder rerankers run on the device executor).

A batch is ragged: only the real tokens of every sequence are laid out, one after another.  Per layer the fused q | k | v
projection (tcgen05 GEMM) feeds the rotary / K-V write kernel with an identity table, which lands the keys and values of
sequence ``r`` in its own blocks of a paged pool; the general attention kernel then runs every token with the whole
sequence visible (``row_ctx`` = the sequence's length, so attention is bidirectional and padding never exists); output
and FFN projections add their residual in the GEMM epilogue and LayerNorm follows each.  Biases are added by the
elementwise kernel; GELU by the activation kernel.  Pooling (``[CLS]``, mean) and the classifier head of a reranker
are a few rows and stay in tensor arithmetic on the device.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..models.encoder import EncoderConfig
from ..ops import cuda_ops as K

KV_BLOCK = K.KV_BLOCK


class EncoderEngine:
    def __init__(self, cfg: EncoderConfig, tensors: Dict[str, torch.Tensor], device, max_tokens: int = 4096, max_rows: int = 64):
        if cfg.head_dim % 32 or cfg.head_dim > 512:
            raise ValueError(f"encoder head width {cfg.head_dim}: the attention kernel takes multiples of 32 up to 512")
        self.cfg, self.device = cfg, torch.device(device)
        dev, bf = self.device, torch.bfloat16
        self.max_tokens, self.max_rows = max_tokens, max_rows
        get = lambda n: tensors[n].to(device=dev, dtype=bf).contiguous()
        self.embed, self.embed_pos, self.embed_type = get("embed"), get("embed_pos"), get("embed_type")
        self.embed_norm, self.embed_norm_b = get("embed_norm"), get("embed_norm_bias")
        self.layers = []
        for l in range(cfg.n_layers):
            p = f"layers.{l}."
            self.layers.append({
                "wqkv": torch.cat([get(p + "attn_q"), get(p + "attn_k"), get(p + "attn_v")], 0).contiguous(),
                "bqkv": torch.cat([get(p + "attn_q_bias"), get(p + "attn_k_bias"), get(p + "attn_v_bias")], 0).contiguous(),
                "wo": get(p + "attn_o"), "bo": get(p + "attn_o_bias"), "ln1": get(p + "attn_post_norm"),
                "ln1_b": get(p + "attn_post_norm_bias"), "wup": get(p + "ffn_up"), "bup": get(p + "ffn_up_bias"),
                "wdown": get(p + "ffn_down"), "bdown": get(p + "ffn_down_bias"), "ln2": get(p + "ffn_post_norm"),
                "ln2_b": get(p + "ffn_post_norm_bias")})
        self.head = None
        if cfg.labels:
            self.head = {k: tensors[k].to(device=dev, dtype=torch.float32) for k in ("pooler", "pooler_bias", "classifier", "classifier_bias")}
        H, nh, D = cfg.hidden, cfg.n_heads, cfg.head_dim
        T = max_tokens
        z = lambda *s, dt=bf: torch.zeros(*s, dtype=dt, device=dev)
        self.h, self.x, self.qkv, self.q, self.attn, self.act = z(T, H), z(T, H), z(T, 3 * H), z(T, H), z(T, H), z(T, cfg.ffn)
        self.blocks_per_seq = -(-cfg.max_position // KV_BLOCK)
        self.pool_blocks = -(-T // KV_BLOCK) + max_rows
        self.kpool, self.vpool = z(self.pool_blocks, nh, KV_BLOCK, D), z(self.pool_blocks, nh, KV_BLOCK, D)
        i32 = torch.int32
        self.tokens, self.pos, self.types, self.slots, self.row_seq, self.row_ctx = (z(T, dt=i32) for _ in range(6))
        self.block_tables = z(max_rows, self.blocks_per_seq, dt=i32)
        # identity rotation: the K/V write kernel is the rotary kernel reading a one-row table of cos = 1, sin = 0
        self.cos = torch.ones(1, D // 2, dtype=torch.float32, device=dev)
        self.sin = torch.zeros(1, D // 2, dtype=torch.float32, device=dev)
        self.zero_pos = z(T, dt=i32)
        self.launches = 0

    # ---- host-side layout --------------------------------------------------------------------------------------
    def _bind(self, seqs: Sequence[Sequence[int]], types: Optional[Sequence[Sequence[int]]]):
        lens = [len(s) for s in seqs]
        N = sum(lens)
        if len(seqs) > self.max_rows or N > self.max_tokens:
            raise ValueError(f"{len(seqs)} sequences / {N} tokens exceed the engine's {self.max_rows} / {self.max_tokens}")
        if max(lens) > self.cfg.max_position:
            raise ValueError(f"a sequence of {max(lens)} tokens exceeds the position table of {self.cfg.max_position}")
        tok, pos, typ = np.zeros(N, np.int32), np.zeros(N, np.int32), np.zeros(N, np.int32)
        slots, row_seq, row_ctx = np.zeros(N, np.int32), np.zeros(N, np.int32), np.zeros(N, np.int32)
        bt = np.zeros((len(seqs), self.blocks_per_seq), np.int32)
        off = blk = 0
        for r, s in enumerate(seqs):
            n = lens[r]
            nb = -(-n // KV_BLOCK)
            bt[r, :nb] = np.arange(blk, blk + nb)
            p = np.arange(n)
            sl = slice(off, off + n)
            tok[sl], pos[sl] = np.asarray(s, np.int32), p
            typ[sl] = 0 if types is None else np.asarray(types[r], np.int32)
            slots[sl] = (blk + p // KV_BLOCK) * KV_BLOCK + p % KV_BLOCK
            row_seq[sl], row_ctx[sl] = r, n                  # every token sees its whole sequence
            off += n
            blk += nb
        for dst, src in ((self.tokens, tok), (self.pos, pos), (self.types, typ), (self.slots, slots), (self.row_seq, row_seq),
                         (self.row_ctx, row_ctx)):
            dst[:N].copy_(torch.from_numpy(src))
        self.block_tables[:len(seqs)].copy_(torch.from_numpy(bt))
        return N, lens

    def _count(self, n: int = 1):
        self.launches += n

    # ---- the program -------------------------------------------------------------------------------------------
    def forward(self, seqs: Sequence[Sequence[int]], types: Optional[Sequence[Sequence[int]]] = None) -> List[torch.Tensor]:
        """Final hidden states of every sequence: a list of ``[len, hidden]`` fp32 tensors (on the device)."""
        cfg = self.cfg
        N, lens = self._bind(seqs, types)
        H, nh, D = cfg.hidden, cfg.n_heads, cfg.head_dim
        h, x, qkv, q, attn = self.h[:N], self.x[:N], self.qkv[:N], self.q[:N], self.attn[:N]
        self.launches = 0
        K.embed_gather(self.tokens[:N], self.embed, out=h)
        K.embed_gather(self.pos[:N], self.embed_pos, out=x)
        K.add(h, x, out=h)
        K.embed_gather(self.types[:N], self.embed_type, out=x)
        K.add(h, x, out=h)
        K.layernorm(h, self.embed_norm, self.embed_norm_b, cfg.norm_eps, out=h)
        self._count(6)
        scale = 1.0 / math.sqrt(D)
        for L in self.layers:
            K.linear(h, L["wqkv"], K.EPI_STORE, qkv)
            qkv.add_(L["bqkv"])
            K.rope_kv_write(qkv, q, self.kpool, self.vpool, self.zero_pos[:N], self.slots[:N], self.cos, self.sin, nh, nh, D, D)
            K.attn_general(q, self.kpool, self.vpool, self.block_tables, self.row_seq[:N], self.row_ctx[:N], nh, nh, D, D,
                           scale, attn)
            K.linear(attn, L["wo"], K.EPI_RESID, h, h)
            h.add_(L["bo"])
            K.layernorm(h, L["ln1"], L["ln1_b"], cfg.norm_eps, out=h)
            up = self.act[:N]
            K.linear(h, L["wup"], K.EPI_STORE, up)
            up.add_(L["bup"])
            K.act_(up, cfg.act)
            K.linear(up, L["wdown"], K.EPI_RESID, h, h)
            h.add_(L["bdown"])
            K.layernorm(h, L["ln2"], L["ln2_b"], cfg.norm_eps, out=h)
            self._count(13)
        out, off = [], 0
        hf = h.float()
        for n in lens:
            out.append(hf[off:off + n])
            off += n
        return out

    def scores(self, seqs, types=None) -> torch.Tensor:
        """Classifier logits ``[rows, labels]`` over the pooled ``[CLS]`` state (cross-encoder rerankers)."""
        if self.head is None:
            raise ValueError("the checkpoint has no classifier head")
        cls = torch.stack([s[0] for s in self.forward(seqs, types)])
        pooled = torch.tanh(cls @ self.head["pooler"].T + self.head["pooler_bias"])
        return pooled @ self.head["classifier"].T + self.head["classifier_bias"]
