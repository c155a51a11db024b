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
from typing import Dict, Optional

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


# ---- Qwen2.5-VL ----------------------------------------------------------------------------------------------------
@dataclass
class QwenVisionConfig:
    """Vision tower of Qwen2.5-VL (crates/poot-models/src/multimodal/qwen_vl/tower.rs): patches of
    ``temporal x patch x patch`` pixels, 2-D rotary positions, attention inside windows of merged patches except on the
    ``full_layers``, RMSNorm, biased SwiGLU, and a merger that folds ``merge x merge`` patches into one text row."""
    hidden: int = 64
    ffn: int = 128
    n_layers: int = 2
    n_heads: int = 4
    channels: int = 3
    patch: int = 14
    temporal: int = 2
    merge: int = 2
    window: int = 112                      # pixels
    full_layers: tuple = (1,)
    out_hidden: int = 64
    act: str = "silu"
    norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    video_token: int = -1                  # id of the video placeholder (-1: the checkpoint names none)
    tokens_per_second: float = 2.0         # time positions per second of video

    @property
    def patch_dim(self) -> int:
        return self.channels * self.temporal * self.patch * self.patch

    @property
    def head_dim(self) -> int:
        return self.hidden // self.n_heads

    @property
    def unit(self) -> int:
        return self.merge * self.merge


def qwen_vision_inputs(cfg: QwenVisionConfig, grids) -> Dict[str, np.ndarray]:
    """Host-side inputs of the tower for images of ``grids = [(t, h, w), ...]`` patches, in the processor's patch order
    (frame, merged row, merged column, row in the merge cell, column in the merge cell): rotary tables from each patch's
    (row, column), and the two additive masks - patches of one frame see each other on the full layers, patches of one
    window of ``window / merge / patch`` merged cells on the others."""
    rows, cols, frame_id, window_id = [], [], [], []
    m, vws = cfg.merge, max(cfg.window // cfg.merge // cfg.patch, 1)
    frames = windows = 0
    for t, h, w in grids:
        lh, lw = h // m, w // m
        r = np.arange(h)[:, None].repeat(w, 1).reshape(lh, m, lw, m).transpose(0, 2, 1, 3).reshape(-1)
        c = np.arange(w)[None, :].repeat(h, 0).reshape(lh, m, lw, m).transpose(0, 2, 1, 3).reshape(-1)
        wh = -(-lh // vws)
        win = ((r // m) // vws) * (-(-lw // vws)) + (c // m) // vws
        for f in range(t):
            rows.append(r); cols.append(c)
            frame_id.append(np.full(h * w, frames + f))
            window_id.append(windows + f * wh * (-(-lw // vws)) + win)
        frames += t
        windows += t * wh * (-(-lw // vws))
    rows, cols = np.concatenate(rows), np.concatenate(cols)
    frame_id, window_id = np.concatenate(frame_id), np.concatenate(window_id)
    quarter = cfg.head_dim // 4
    inv = 1.0 / (cfg.rope_theta ** (np.arange(0, cfg.head_dim // 2, 2, dtype=np.float32) / np.float32(cfg.head_dim // 2)))
    ang = np.concatenate([rows[:, None].astype(np.float32) * inv[None, :quarter], cols[:, None].astype(np.float32) * inv[None, :quarter]], 1)
    ang = np.concatenate([ang, ang], 1)
    hidden = np.float32(O.MASK_HIDDEN)
    return {"rope_cos": np.cos(ang).astype(np.float32), "rope_sin": np.sin(ang).astype(np.float32),
            "mask_full": np.where(frame_id[:, None] == frame_id[None, :], np.float32(0), hidden)[None].astype(np.float32),
            "mask_window": np.where(window_id[:, None] == window_id[None, :], np.float32(0), hidden)[None].astype(np.float32)}


class QwenVisionTower:
    def __init__(self, cfg: QwenVisionConfig):
        self.cfg = cfg

    def weight_shapes(self) -> Dict[str, tuple]:
        c = self.cfg
        H, U = c.hidden, c.hidden * c.unit
        s = {"vision.patch_embed": (H, c.patch_dim), "vision.merger_norm": (H,), "vision.merger_fc1": (U, U),
             "vision.merger_fc1_bias": (U,), "vision.merger_fc2": (c.out_hidden, U), "vision.merger_fc2_bias": (c.out_hidden,)}
        for l in range(c.n_layers):
            p = f"vision.layers.{l}."
            for r, shape in (("attn_q", (H, H)), ("attn_k", (H, H)), ("attn_v", (H, H)), ("attn_o", (H, H)),
                             ("ffn_gate", (c.ffn, H)), ("ffn_up", (c.ffn, H)), ("ffn_down", (H, c.ffn))):
                s[p + r], s[p + r + "_bias"] = shape, (shape[0],)
            s[p + "attn_norm"], s[p + "ffn_norm"] = (H,), (H,)
        return s

    def trace(self, patches: int, weight_dtype: DType = DType.F32) -> Graph:
        """``patches[N, patch_dim]`` + the inputs of ``qwen_vision_inputs`` -> ``image_rows[N / merge^2, out_hidden]``."""
        c = self.cfg
        b = Builder()
        N, H, nh, D = patches, c.hidden, c.n_heads, c.head_dim
        shapes = self.weight_shapes()
        consts = {}

        def W(name):
            if name not in consts:
                consts[name] = b.const(name, shapes[name], weight_dtype).cast(F32)
            return consts[name]

        x = b.slot("patches", (N, c.patch_dim), F32, "activation")
        cos = b.slot("rope_cos", (N, D), F32, "activation")
        sin = b.slot("rope_sin", (N, D), F32, "activation")
        masks = {True: b.slot("mask_full", (1, N, N), F32, "activation"), False: b.slot("mask_window", (1, N, N), F32, "activation")}
        h = O.linear(b, x, W("vision.patch_embed"), precision="exact")
        scale = 1.0 / math.sqrt(D)
        for l in range(c.n_layers):
            p = f"vision.layers.{l}."
            y = O.rmsnorm(b, h, W(p + "attn_norm"), c.norm_eps)
            q = O.rope(b, b.reshape(O.linear(b, y, W(p + "attn_q"), W(p + "attn_q_bias")), (N, nh, D)), cos, sin, D)
            k = O.rope(b, b.reshape(O.linear(b, y, W(p + "attn_k"), W(p + "attn_k_bias")), (N, nh, D)), cos, sin, D)
            v = b.reshape(O.linear(b, y, W(p + "attn_v"), W(p + "attn_v_bias")), (N, nh, D))
            heads = lambda t: b.transpose(b.reshape(t, (1, N, nh, D)), (0, 2, 1, 3))
            a = O.attention_masked(b, heads(q), heads(k), heads(v), masks[l in c.full_layers], scale)
            a = b.reshape(b.transpose(a, (0, 2, 1, 3)), (N, H))
            h = h + O.linear(b, a, W(p + "attn_o"), W(p + "attn_o_bias"))
            y = O.rmsnorm(b, h, W(p + "ffn_norm"), c.norm_eps)
            g = O.ffn_activation(b, O.linear(b, y, W(p + "ffn_gate"), W(p + "ffn_gate_bias")),
                                 O.linear(b, y, W(p + "ffn_up"), W(p + "ffn_up_bias")), c.act)
            h = h + O.linear(b, g, W(p + "ffn_down"), W(p + "ffn_down_bias"))
        m = b.reshape(O.rmsnorm(b, h, W("vision.merger_norm"), c.norm_eps), (N // c.unit, H * c.unit))
        m = O.gelu_erf(b, O.linear(b, m, W("vision.merger_fc1"), W("vision.merger_fc1_bias")))
        b.output(O.linear(b, m, W("vision.merger_fc2"), W("vision.merger_fc2_bias")), "image_rows", "result")
        return b.finish()


def mrope_positions(tokens, image_token: int, grids, merge: int, video_token: Optional[int] = None, seconds_per_step=None,
                    tokens_per_second: float = 2.0) -> np.ndarray:
    """Rotary position streams ``[3, len(tokens)]`` (time, row, column) of a prompt whose runs of ``image_token`` (or
    ``video_token``) stand for the media of ``grids = [(t, h, w), ...]`` patches, in prompt order (multimodal/mrope.rs;
    ``get_rope_index``): text tokens count up with three equal values; an image starting at ``s`` gives ``(s, s + row,
    s + column)`` per merged cell and the text after it continues at ``s + max(rows, columns)`` of merged cells.  A video
    (``seconds_per_step[i]`` is the time one temporal step of grid ``i`` covers, ``None`` for an image) advances its time
    stream by ``floor(step * seconds * tokens_per_second)`` per temporal step, and the text continues after the largest
    position of any stream."""
    toks = np.asarray(tokens).reshape(-1)
    out = np.zeros((3, len(toks)), dtype=np.int32)
    i, nxt, image = 0, 0, 0
    secs = list(seconds_per_step) if seconds_per_step is not None else [None] * len(grids)
    while i < len(toks):
        if video_token is not None and toks[i] == video_token:
            if image >= len(grids) or secs[image] is None:
                raise ValueError("a video run in the prompt without a video at that place")
            t, h, w = grids[image]
            lh, lw = h // merge, w // merge
            n = t * lh * lw
            if len(toks[i:i + n]) != n or not np.all(toks[i:i + n] == video_token):
                raise ValueError(f"video {image}: the prompt holds fewer than {n} video tokens in a run")
            step = np.floor(np.arange(t) * float(secs[image]) * float(tokens_per_second)).astype(np.int64)
            out[0, i:i + n] = nxt + np.repeat(step, lh * lw)
            out[1, i:i + n] = nxt + np.tile(np.repeat(np.arange(lh), lw), t)
            out[2, i:i + n] = nxt + np.tile(np.tile(np.arange(lw), lh), t)
            nxt = int(out[:, i:i + n].max()) + 1
            i += n
            image += 1
            continue
        if toks[i] != image_token:
            out[:, i] = nxt
            nxt += 1
            i += 1
            continue
        if image < len(grids) and secs[image] is not None:
            raise ValueError(f"medium {image} is a video but the prompt holds an image run there")
        if image >= len(grids):
            raise ValueError("more image runs in the prompt than images")
        t, h, w = grids[image]
        lh, lw = h // merge, w // merge
        n = t * lh * lw
        if not np.all(toks[i:i + n] == image_token) or len(toks[i:i + n]) != n:
            raise ValueError(f"image {image}: the prompt holds fewer than {n} image tokens in a run")
        out[0, i:i + n] = nxt                   # frames of one image share the start (no time interval between them)
        out[1, i:i + n] = nxt + np.tile(np.repeat(np.arange(lh), lw), t)
        out[2, i:i + n] = nxt + np.tile(np.tile(np.arange(lw), lh), t)
        nxt += max(lh, lw)
        i += n
        image += 1
    if image != len(grids):
        raise ValueError(f"{len(grids)} images for {image} image runs in the prompt")
    return out
