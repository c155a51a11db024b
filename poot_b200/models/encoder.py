"""BERT-style bidirectional encoder behind the same graph IR: sentence embedders (MiniLM, BGE, E5) and, with the
classifier head, cross-encoder rerankers (crates/poot-models/src/architectures/bert.rs:1-11, 210-215, 588-593).

A step is ``rows`` right-padded sequences of ``tokens`` positions.  Four inputs bind per step: token ids, absolute
positions, the segment id of every token and which tokens are real; a padded token is never attended to, so a
row's output does not depend on how far its batch pads it.  The step returns every position's final hidden state
(pooled on the host) or, with the classifier, the ``[CLS]`` position's logits.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict

from ..ir import oplib as O
from ..ir.builder import Builder
from ..ir.graph import Graph
from ..tensor import DType

F32, I32 = DType.F32, DType.I32


@dataclass
class EncoderConfig:
    name: str = "bert"
    family: str = "bert"
    n_layers: int = 2
    hidden: int = 64
    n_heads: int = 4
    ffn: int = 256
    vocab: int = 30522
    max_position: int = 512
    type_vocab: int = 2
    norm_eps: float = 1e-12
    act: str = "gelu_erf"
    labels: int = 0                # > 0: BertForSequenceClassification (pooler + classifier over [CLS])
    pad_token: int = 0

    @property
    def head_dim(self) -> int:
        return self.hidden // self.n_heads


class EncoderModel:
    kind = "encoder"

    def __init__(self, cfg: EncoderConfig):
        self.cfg = cfg

    def weight_shapes(self) -> Dict[str, tuple]:
        c = self.cfg
        H = c.hidden
        s = {"embed": (c.vocab, H), "embed_pos": (c.max_position, H), "embed_type": (c.type_vocab, H),
             "embed_norm": (H,), "embed_norm_bias": (H,)}
        for l in range(c.n_layers):
            p = f"layers.{l}."
            for r in ("attn_q", "attn_k", "attn_v", "attn_o"):
                s[p + r], s[p + r + "_bias"] = (H, H), (H,)
            s.update({p + "attn_post_norm": (H,), p + "attn_post_norm_bias": (H,), p + "ffn_up": (c.ffn, H),
                      p + "ffn_up_bias": (c.ffn,), p + "ffn_down": (H, c.ffn), p + "ffn_down_bias": (H,),
                      p + "ffn_post_norm": (H,), p + "ffn_post_norm_bias": (H,)})
        if c.labels:
            s.update({"pooler": (H, H), "pooler_bias": (H,), "classifier": (c.labels, H), "classifier_bias": (c.labels,)})
        return s

    def trace(self, rows: int, tokens: int, weight_dtype: DType = DType.F32) -> Graph:
        c = self.cfg
        b = Builder()
        R, T, H, nh, D = rows, tokens, c.hidden, c.n_heads, c.head_dim
        shapes = self.weight_shapes()
        consts = {}

        def W(name):
            if name not in consts:
                consts[name] = b.const(name, shapes[name], weight_dtype).cast(F32)
            return consts[name]

        def ln(x, name):
            return O.layernorm(b, x, W(name), W(name + "_bias"), c.norm_eps)

        ids = b.slot("tokens", (R, T), I32, "token", range=(0, c.vocab - 1))
        pos = b.slot("positions", (R, T), I32, "pos", range=(0, c.max_position - 1))
        typ = b.slot("token_type", (R, T), I32, "activation", range=(0, c.type_vocab - 1))
        real = b.slot("real_tokens", (R, T), I32, "activation", range=(0, 1))
        flat = lambda x: b.reshape(x, (R * T,))
        h = b.gather(W("embed"), flat(ids), 0) + b.gather(W("embed_pos"), flat(pos), 0) + b.gather(W("embed_type"), flat(typ), 0)
        h = ln(h, "embed_norm")
        # key s is visible to every query of its row iff it is a real token
        vis = b.broadcast(b.reshape(real, (R, 1, T)), (R, T, T))
        mask = b.select(vis, b.broadcast(b.scalar(0.0, F32), (R, T, T)), b.broadcast(b.scalar(O.MASK_HIDDEN, F32), (R, T, T)))
        scale = 1.0 / math.sqrt(D)
        for l in range(c.n_layers):
            p = f"layers.{l}."
            heads = lambda x: b.transpose(b.reshape(x, (R, T, nh, D)), (0, 2, 1, 3))
            q = heads(O.linear(b, h, W(p + "attn_q"), W(p + "attn_q_bias")))
            k = heads(O.linear(b, h, W(p + "attn_k"), W(p + "attn_k_bias")))
            v = heads(O.linear(b, h, W(p + "attn_v"), W(p + "attn_v_bias")))
            a = O.attention_masked(b, q, k, v, mask, scale)
            a = b.reshape(b.transpose(a, (0, 2, 1, 3)), (R * T, H))
            h = ln(h + O.linear(b, a, W(p + "attn_o"), W(p + "attn_o_bias")), p + "attn_post_norm")
            u = O.ffn_activation(b, O.linear(b, h, W(p + "ffn_up"), W(p + "ffn_up_bias")), None, c.act)
            h = ln(h + O.linear(b, u, W(p + "ffn_down"), W(p + "ffn_down_bias")), p + "ffn_post_norm")
        hid = b.reshape(h, (R, T, H))
        if c.labels:
            cls = b.reshape(b.slice(hid, 1, 0, 1), (R, H))
            pooled = b.unary("tanh", O.linear(b, cls, W("pooler"), W("pooler_bias")))
            b.output(O.linear(b, pooled, W("classifier"), W("classifier_bias")), "scores", "result")
        else:
            b.output(hid, "hidden", "result")
        return b.finish()
