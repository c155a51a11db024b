"""The Idefics3 / SmolVLM vision tower and connector on the device: the program of ``models/vision.py::VisionTower`` over
the decoder engine's kernels (crates/poot-models/src/multimodal/idefics3/tower.rs runs the tower on a driver of its own).

Every frame is one sequence of ``n_patches`` rows.  The patch embedding is a GEMM over flattened patches (the strided
convolution written as a matrix product) plus the learned position rows; each pre-norm block is LayerNorm, the fused
q | k | v GEMM, the K/V write kernel with an identity rotary table, the general attention kernel with every patch of the
frame visible, the output GEMM with the residual in its epilogue, LayerNorm, and the GELU FFN the same way; the final
LayerNorm, the pixel shuffle (a reshape / permute of the rows) and the projection GEMM give the rows the text stack
takes in place of its image tokens.  Head widths must be multiples of 32 (the attention kernel's constraint: the
SigLIP-base towers of the small SmolVLM checkpoints qualify, the 72-wide heads of the so400m tower do not).
"""
from __future__ import annotations

import math
from typing import Dict

import numpy as np
import torch

from ..models.vision import VisionConfig, patchify, position_ids
from ..ops import cuda_ops as K

KV_BLOCK = K.KV_BLOCK


class VisionEngine:
    def __init__(self, cfg: VisionConfig, tensors: Dict[str, torch.Tensor], device, max_frames: int = 17):
        D = cfg.hidden // cfg.n_heads
        if D % 32 or D > 512:
            raise ValueError(f"vision head width {D}: the attention kernel takes multiples of 32 up to 512")
        if cfg.act != "gelu_tanh":
            raise ValueError(f"vision activation {cfg.act!r}: the device program has the tanh GELU")
        self.cfg, self.device, self.max_frames, self.D = cfg, torch.device(device), max_frames, D
        dev, bf = self.device, torch.bfloat16
        get = lambda n: tensors[n].to(device=dev, dtype=bf).contiguous()
        pd = cfg.patch_dim
        self.pd_pad = -(-pd // 8) * 8                          # GEMM rows of 16-byte multiples
        w = torch.zeros(cfg.hidden, self.pd_pad, dtype=bf, device=dev)
        w[:, :pd] = get("vision.patch_embed")
        self.patch_embed, self.patch_bias, self.pos_embed = w, get("vision.patch_embed_bias"), get("vision.pos_embed")
        self.post_norm, self.post_norm_b, self.projector = get("vision.post_norm"), get("vision.post_norm_bias"), get("vision.projector")
        self.layers = []
        for l in range(cfg.n_layers):
            p = f"vision.layers.{l}."
            self.layers.append({
                "ln1": get(p + "attn_norm"), "ln1_b": get(p + "attn_norm_bias"), "ln2": get(p + "ffn_norm"), "ln2_b": get(p + "ffn_norm_bias"),
                "wqkv": torch.cat([get(p + "attn_q"), get(p + "attn_k"), get(p + "attn_v")], 0).contiguous(),
                "bqkv": torch.cat([get(p + "attn_q_bias"), get(p + "attn_k_bias"), get(p + "attn_v_bias")], 0).contiguous(),
                "wo": get(p + "attn_o"), "bo": get(p + "attn_o_bias"), "wup": get(p + "ffn_up"), "bup": get(p + "ffn_up_bias"),
                "wdown": get(p + "ffn_down"), "bdown": get(p + "ffn_down_bias")})
        N, H, nh = cfg.n_patches, cfg.hidden, cfg.n_heads
        T = max_frames * N
        z = lambda *s, dt=bf: torch.zeros(*s, dtype=dt, device=dev)
        self.patches = z(T, self.pd_pad)
        self.h, self.x, self.qkv, self.q, self.attn, self.act = z(T, H), z(T, H), z(T, 3 * H), z(T, H), z(T, H), z(T, cfg.ffn)
        self.rows = z(max_frames * cfg.rows_per_image, cfg.text_hidden)
        bpf = -(-N // KV_BLOCK)                                # K/V blocks of one frame
        self.kpool, self.vpool = z(max_frames * bpf, nh, KV_BLOCK, D), z(max_frames * bpf, nh, KV_BLOCK, D)
        i32 = torch.int32
        frame = np.repeat(np.arange(max_frames), N)
        inside = np.tile(np.arange(N), max_frames)
        to = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
        self.slots = to((frame * bpf + inside // KV_BLOCK) * KV_BLOCK + inside % KV_BLOCK)
        self.row_seq, self.row_ctx = to(frame), to(np.full(T, N))            # every patch sees its whole frame
        self.block_tables = to(np.arange(max_frames * bpf).reshape(max_frames, bpf))
        self.pos_ids = to(np.tile(position_ids(cfg, cfg.per_side, cfg.per_side), max_frames))
        self.zero_pos = z(T, dt=i32)
        self.cos = torch.ones(1, D // 2, dtype=torch.float32, device=dev)     # identity rotation for the K/V write kernel
        self.sin = torch.zeros(1, D // 2, dtype=torch.float32, device=dev)
        self.launches = 0

    def forward(self, pixels: np.ndarray) -> torch.Tensor:
        """``pixels[frames, C, S, S]`` (normalised, host) -> ``[frames * rows_per_image, text_hidden]`` bf16 on the device."""
        cfg = self.cfg
        F_ = pixels.shape[0]
        if F_ > self.max_frames:
            raise ValueError(f"{F_} frames exceed the engine's {self.max_frames}")
        N, H, nh, D = cfg.n_patches, cfg.hidden, cfg.n_heads, self.D
        T = F_ * N
        flat = torch.from_numpy(patchify(np.asarray(pixels, np.float32), cfg.patch).reshape(T, cfg.patch_dim))
        self.patches[:T, :cfg.patch_dim].copy_(flat.to(torch.bfloat16))
        h, x, qkv, q, attn, up = self.h[:T], self.x[:T], self.qkv[:T], self.q[:T], self.attn[:T], self.act[:T]
        K.linear(self.patches[:T], self.patch_embed, K.EPI_STORE, h)
        h.add_(self.patch_bias)
        K.embed_gather(self.pos_ids[:T], self.pos_embed, out=x)
        K.add(h, x, out=h)
        self.launches = 4
        scale = 1.0 / math.sqrt(D)
        for L in self.layers:
            K.layernorm(h, L["ln1"], L["ln1_b"], cfg.norm_eps, out=x)
            K.linear(x, L["wqkv"], K.EPI_STORE, qkv)
            qkv.add_(L["bqkv"])
            K.rope_kv_write(qkv, q, self.kpool, self.vpool, self.zero_pos[:T], self.slots[:T], self.cos, self.sin, nh, nh, D, D)
            K.attn_general(q, self.kpool, self.vpool, self.block_tables, self.row_seq[:T], self.row_ctx[:T], nh, nh, D, D,
                           scale, attn)
            K.linear(attn, L["wo"], K.EPI_RESID, h, h)
            h.add_(L["bo"])
            K.layernorm(h, L["ln2"], L["ln2_b"], cfg.norm_eps, out=x)
            K.linear(x, L["wup"], K.EPI_STORE, up)
            up.add_(L["bup"])
            K.act_(up, cfg.act)
            K.linear(up, L["wdown"], K.EPI_RESID, h, h)
            h.add_(L["bdown"])
            self.launches += 13
        K.layernorm(h, self.post_norm, self.post_norm_b, cfg.norm_eps, out=x)
        s, side = cfg.scale, cfg.per_side
        # pixel shuffle: scale x scale neighbouring patches fold into one row (the permutes of the graph's connector)
        y = x.view(F_, side, side // s, H * s).permute(0, 2, 1, 3).reshape(F_, side // s, side // s, H * s * s)
        y = y.permute(0, 2, 1, 3).reshape(F_ * cfg.rows_per_image, H * s * s).contiguous()
        out = self.rows[:F_ * cfg.rows_per_image]
        K.linear(y, self.projector, K.EPI_STORE, out)
        self.launches += 3
        return out
