"""Vision front end of the vision-language families: a SigLIP-style patch encoder and the connector that turns its
patch states into rows of the text model's embedding space (crates/poot-models: the Idefics3 / SmolVLM front end).

An image is cut on the host into non-overlapping ``patch x patch`` squares (``patchify``: the strided convolution of
the checkpoint written as a matrix product over flattened patches); the graph embeds them, adds the learned position
rows, runs pre-norm bidirectional transformer blocks (LayerNorm, biased attention, GELU MLP), the final LayerNorm,
then the connector: a pixel shuffle that folds ``scale x scale`` neighbouring patches into one row, and a linear
projection into the text width.  The text stack receives those rows in place of the embeddings of its image tokens
(``StepSpec.embeds``)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict

import numpy as np

from ..ir import oplib as O
from ..ir.builder import Builder
from ..ir.graph import Graph
from ..tensor import DType

F32, I32 = DType.F32, DType.I32


@dataclass
class VisionConfig:
    hidden: int = 64
    ffn: int = 128
    n_layers: int = 2
    n_heads: int = 4
    channels: int = 3
    image_size: int = 32
    patch: int = 8
    norm_eps: float = 1e-6
    act: str = "gelu_tanh"
    scale: int = 2                  # pixel-shuffle factor of the connector
    text_hidden: int = 64

    @property
    def per_side(self) -> int:
        return self.image_size // self.patch

    @property
    def n_patches(self) -> int:
        return self.per_side ** 2

    @property
    def patch_dim(self) -> int:
        return self.channels * self.patch * self.patch

    @property
    def rows_per_image(self) -> int:
        return self.n_patches // (self.scale ** 2)


def patchify(pixels: np.ndarray, patch: int) -> np.ndarray:
    """``[B, C, H, W]`` -> ``[B, (H/p)(W/p), C p p]`` in the element order of a convolution weight ``[out, C, p, p]``.
    Pixels past the last whole patch are dropped, as an unpadded strided convolution drops them (384 / 14)."""
    B, C, H, W = pixels.shape
    H, W = H // patch * patch, W // patch * patch
    pixels = pixels[:, :, :H, :W]
    x = pixels.reshape(B, C, H // patch, patch, W // patch, patch)
    return np.ascontiguousarray(x.transpose(0, 2, 4, 1, 3, 5)).reshape(B, (H // patch) * (W // patch), C * patch * patch)


def position_ids(cfg: VisionConfig, rows: int, cols: int) -> np.ndarray:
    """Position row of every patch of a ``rows x cols`` patch grid: fractional coordinates bucketed onto the
    ``per_side x per_side`` table the checkpoint learned (identity for a full square image)."""
    n = cfg.per_side
    bounds = np.arange(1.0 / n, 1.0, 1.0 / n, dtype=np.float32)
    fh = np.minimum(np.arange(rows, dtype=np.float32) * np.float32(1.0 / rows), np.float32(1.0 - 1e-6))
    fw = np.minimum(np.arange(cols, dtype=np.float32) * np.float32(1.0 / cols), np.float32(1.0 - 1e-6))
    bh = np.searchsorted(bounds, fh, side="right")
    bw = np.searchsorted(bounds, fw, side="right")
    return (bh[:, None] * n + bw[None, :]).reshape(-1).astype(np.int32)


class VisionTower:
    def __init__(self, cfg: VisionConfig):
        self.cfg = cfg

    def weight_shapes(self) -> Dict[str, tuple]:
        c = self.cfg
        H = c.hidden
        s = {"vision.patch_embed": (H, c.patch_dim), "vision.patch_embed_bias": (H,), "vision.pos_embed": (c.n_patches, H),
             "vision.post_norm": (H,), "vision.post_norm_bias": (H,),
             "vision.projector": (c.text_hidden, H * c.scale * c.scale)}
        for l in range(c.n_layers):
            p = f"vision.layers.{l}."
            for r in ("attn_q", "attn_k", "attn_v", "attn_o"):
                s[p + r], s[p + r + "_bias"] = (H, H), (H,)
            s.update({p + "attn_norm": (H,), p + "attn_norm_bias": (H,), p + "ffn_norm": (H,), p + "ffn_norm_bias": (H,),
                      p + "ffn_up": (c.ffn, H), p + "ffn_up_bias": (c.ffn,), p + "ffn_down": (H, c.ffn), p + "ffn_down_bias": (H,)})
        return s

    def trace(self, images: int, weight_dtype: DType = DType.F32) -> Graph:
        """``patches[images, n_patches, patch_dim]``, ``pos_ids[images, n_patches]`` -> ``rows[images * rows_per_image, text_hidden]``."""
        c = self.cfg
        b = Builder()
        B, N, H, nh = images, c.n_patches, c.hidden, c.n_heads
        D = H // nh
        shapes = self.weight_shapes()
        consts = {}

        def W(name):
            if name not in consts:
                consts[name] = b.const(name, shapes[name], weight_dtype).cast(F32)
            return consts[name]

        def ln(x, name):
            return O.layernorm(b, x, W(name), W(name + "_bias"), c.norm_eps)

        patches = b.slot("patches", (B, N, c.patch_dim), F32, "activation")
        pos = b.slot("pos_ids", (B, N), I32, "pos", range=(0, c.n_patches - 1))
        x = b.reshape(patches, (B * N, c.patch_dim))
        h = O.linear(b, x, W("vision.patch_embed"), W("vision.patch_embed_bias"), precision="exact")
        h = h + b.gather(W("vision.pos_embed"), b.reshape(pos, (B * N,)), 0)
        mask = b.broadcast(b.scalar(0.0, F32), (B, N, N))               # every patch sees every patch of its image
        scale = 1.0 / math.sqrt(D)
        for l in range(c.n_layers):
            p = f"vision.layers.{l}."
            y = ln(h, p + "attn_norm")
            heads = lambda t: b.transpose(b.reshape(t, (B, N, nh, D)), (0, 2, 1, 3))
            q = heads(O.linear(b, y, W(p + "attn_q"), W(p + "attn_q_bias")))
            k = heads(O.linear(b, y, W(p + "attn_k"), W(p + "attn_k_bias")))
            v = heads(O.linear(b, y, W(p + "attn_v"), W(p + "attn_v_bias")))
            a = O.attention_masked(b, q, k, v, mask, scale)
            a = b.reshape(b.transpose(a, (0, 2, 1, 3)), (B * N, H))
            h = h + O.linear(b, a, W(p + "attn_o"), W(p + "attn_o_bias"))
            y = ln(h, p + "ffn_norm")
            u = O.ffn_activation(b, O.linear(b, y, W(p + "ffn_up"), W(p + "ffn_up_bias")), None, c.act)
            h = h + O.linear(b, u, W(p + "ffn_down"), W(p + "ffn_down_bias"))
        h = ln(h, "vision.post_norm")
        # connector: fold scale x scale neighbouring patches into one row (pixel shuffle), then project into the text width
        s, side = c.scale, c.per_side
        x = b.reshape(h, (B, side, side // s, H * s))
        x = b.transpose(x, (0, 2, 1, 3))
        x = b.reshape(x, (B, side // s, side // s, H * s * s))
        x = b.transpose(x, (0, 2, 1, 3))
        x = b.reshape(x, (B * (N // (s * s)), H * s * s))
        b.output(O.linear(b, x, W("vision.projector")), "image_rows", "result")
        return b.finish()


class VisionLanguageModel:
    """A text decoder with a vision front end: ``text`` is the standard stack (its tracer takes the image rows through
    ``StepSpec.embeds``), ``vision`` the patch encoder + connector, ``image_token`` the id whose embeddings they replace."""
    kind = "vlm"

    def __init__(self, text, vision: VisionTower, image_token: int):
        self.text, self.vision, self.image_token = text, vision, image_token
        self.cfg = text.cfg

    def weight_shapes(self) -> Dict[str, tuple]:
        return {**self.text.weight_shapes(), **self.vision.weight_shapes()}

    def trace(self, spec):
        return self.text.trace(spec)
