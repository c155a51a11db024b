"""Host codecs: dequantise / quantise any supported format.

Block (GGUF) formats run in the C++ host library (csrc/host/quant_codec.cpp); planar (safetensors) formats -
E4M3 per-channel and 128x128 block scales, E2M1 rows of 32, GPTQ and AWQ int4 - are a few numpy lines each.
``check_scales`` is the content check of the reference (crates/poot-quant/src/content.rs:1-7): a block whose
scale is NaN/Inf is rejected before the store is published.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_void_p
from typing import Dict, Optional, Tuple

import numpy as np

from ..ops._lib import host
from ..tensor import e4m3_bits_to_f32, e8m0_bits_to_f32, f32_to_e4m3_bits
from .formats import FORMATS, UnsupportedFormat, descriptor, packed_nbytes

_E2M1 = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)
_AWQ_ORDER = np.array([0, 4, 1, 5, 2, 6, 3, 7])


def _lib():
    lib = host()
    if not getattr(lib, "_quant_bound", False):
        lib.poot_dequantize.argtypes = [c_int, c_void_p, c_void_p, c_longlong]
        lib.poot_quantize.argtypes = [c_int, c_void_p, c_void_p, c_longlong]
        lib.poot_quant_check_scales.argtypes = [c_int, c_void_p, c_longlong]
        lib.poot_quant_check_scales.restype = c_longlong
        lib._quant_bound = True
    return lib


def dequantize(fmt: str, packed: np.ndarray, shape) -> np.ndarray:
    """Packed bytes of a block format -> f32 array of ``shape``."""
    d = descriptor(fmt)
    if not d.decode:
        raise UnsupportedFormat(f"{fmt}: {d.note}")
    if d.storage == "planar":
        raise UnsupportedFormat(f"{fmt} is planar: use dequantize_planar")
    n = int(np.prod(shape))
    raw = np.ascontiguousarray(packed).view(np.uint8).reshape(-1)
    if raw.size != packed_nbytes(fmt, n):
        raise ValueError(f"{fmt}: {raw.size} bytes for {n} values, expected {packed_nbytes(fmt, n)}")
    out = np.empty(n, dtype=np.float32)
    rc = _lib().poot_dequantize(d.ggml_type, raw.ctypes.data, out.ctypes.data, n)
    if rc != 0:
        raise UnsupportedFormat(f"{fmt}: host decoder refused ({rc})")
    return out.reshape(shape)


def quantize(fmt: str, x: np.ndarray) -> np.ndarray:
    """f32 array (last axis a multiple of the block size) -> packed bytes (uint8, rows concatenated)."""
    d = descriptor(fmt)
    if not d.encode or d.storage == "planar":
        raise UnsupportedFormat(f"{fmt}: no block encoder")
    x = np.ascontiguousarray(x, dtype=np.float32)
    if x.shape[-1] % d.block_elems:
        raise UnsupportedFormat(f"{fmt}: row length {x.shape[-1]} is not a multiple of {d.block_elems}")
    out = np.empty(packed_nbytes(fmt, x.size), dtype=np.uint8)
    rc = _lib().poot_quantize(d.ggml_type, x.ctypes.data, out.ctypes.data, x.size)
    if rc != 0:
        raise UnsupportedFormat(f"{fmt}: host encoder refused ({rc})")
    return out


def check_scales(fmt: str, packed: np.ndarray, n_elems: int) -> None:
    d = descriptor(fmt)
    if d.storage != "blocks":
        return
    raw = np.ascontiguousarray(packed).view(np.uint8).reshape(-1)
    bad = _lib().poot_quant_check_scales(d.ggml_type, raw.ctypes.data, n_elems)
    if bad >= 0:
        raise ValueError(f"{fmt}: block {bad} has a non-finite scale")


# ---- planar formats ------------------------------------------------------------------------------------------------
def quantize_planar(fmt: str, w: np.ndarray, group: int = 128) -> Dict[str, np.ndarray]:
    w = np.asarray(w, dtype=np.float32)
    N, K = w.shape
    if fmt == "E4M3_CHANNEL":
        scale = np.maximum(np.abs(w).max(axis=1), 1e-12) / 448.0
        return {"weight": f32_to_e4m3_bits(w / scale[:, None]), "weight_scale": scale.astype(np.float32)}
    if fmt == "E4M3_BLOCK128":
        nb, kb = (N + 127) // 128, (K + 127) // 128
        scale = np.zeros((nb, kb), dtype=np.float32)
        q = np.zeros((N, K), dtype=np.uint8)
        for i in range(nb):
            for j in range(kb):
                blk = w[i * 128:(i + 1) * 128, j * 128:(j + 1) * 128]
                s = max(float(np.abs(blk).max()), 1e-12) / 448.0
                scale[i, j] = s
                q[i * 128:(i + 1) * 128, j * 128:(j + 1) * 128] = f32_to_e4m3_bits(blk / s)
        return {"weight": q, "weight_scale_inv": scale}
    if fmt == "E2M1_ROW32":
        assert K % 32 == 0
        blocks = w.reshape(N, K // 32, 32)
        amax = np.maximum(np.abs(blocks).max(axis=2), 1e-30)
        e = np.clip(np.ceil(np.log2(amax / 6.0)) + 127, 0, 254).astype(np.uint8)
        s = e8m0_bits_to_f32(e)[..., None]
        codes = np.abs((blocks / s)[..., None] - _E2M1[None, None, None, :]).argmin(-1).astype(np.uint8)
        packed = (codes[..., 0::2] | (codes[..., 1::2] << 4)).reshape(N, K // 2)
        return {"weight": packed, "weight_scale": e}
    if fmt in ("GPTQ", "AWQ"):
        assert K % group == 0 and N % 8 == 0 and K % 8 == 0
        wt = w.T.reshape(K // group, group, N)                      # [groups, group, N]
        mn, mx = wt.min(axis=1), wt.max(axis=1)
        scale = np.maximum((mx - mn) / 15.0, 1e-8).astype(np.float32)        # [groups, N]
        zero = np.clip(np.rint(-mn / scale), 0, 15).astype(np.uint32)
        q = np.clip(np.rint(wt / scale[:, None, :]) + zero[:, None, :], 0, 15).astype(np.uint32).reshape(K, N)
        if fmt == "GPTQ":
            qweight = np.zeros((K // 8, N), dtype=np.uint32)
            for i in range(8):
                qweight |= q[i::8] << (4 * i)
            zz = zero - 1                                            # GPTQ v1 stores zero - 1
            qzeros = np.zeros((K // group, N // 8), dtype=np.uint32)
            for i in range(8):
                qzeros |= (zz[:, i::8] & 0xF) << (4 * i)
            return {"qweight": qweight.view(np.int32), "qzeros": qzeros.view(np.int32), "scales": scale,
                    "g_idx": (np.arange(K) // group).astype(np.int32)}
        qweight = np.zeros((K, N // 8), dtype=np.uint32)
        qzeros = np.zeros((K // group, N // 8), dtype=np.uint32)
        for i in range(8):
            qweight |= q[:, _AWQ_ORDER[i]::8] << (4 * i)
            qzeros |= zero[:, _AWQ_ORDER[i]::8] << (4 * i)
        return {"qweight": qweight.view(np.int32), "qzeros": qzeros.view(np.int32), "scales": scale}
    raise UnsupportedFormat(f"{fmt}: no planar encoder")


def dequantize_planar(fmt: str, t: Dict[str, np.ndarray], group: int = 128) -> np.ndarray:
    """Planar operands -> f32 ``[out, in]`` weight."""
    if fmt == "E4M3_CHANNEL":
        return e4m3_bits_to_f32(t["weight"]) * np.asarray(t["weight_scale"], dtype=np.float32).reshape(-1, 1)
    if fmt == "E4M3_BLOCK128":
        w = e4m3_bits_to_f32(t["weight"])
        s = np.asarray(t["weight_scale_inv"], dtype=np.float32)
        return w * np.repeat(np.repeat(s, 128, axis=0), 128, axis=1)[:w.shape[0], :w.shape[1]]
    if fmt == "E2M1_ROW32":
        p = t["weight"]
        N, K2 = p.shape
        codes = np.empty((N, K2 * 2), dtype=np.uint8)
        codes[:, 0::2], codes[:, 1::2] = p & 0xF, p >> 4
        s = e8m0_bits_to_f32(t["weight_scale"]).reshape(N, -1)
        return _E2M1[codes] * np.repeat(s, 32, axis=1)
    if fmt in ("GPTQ", "AWQ"):
        qw, qz = t["qweight"].view(np.uint32), t["qzeros"].view(np.uint32)
        scale = np.asarray(t["scales"], dtype=np.float32)
        if fmt == "GPTQ":
            K, N = qw.shape[0] * 8, qw.shape[1]
            q = np.zeros((K, N), dtype=np.float32)
            for i in range(8):
                q[i::8] = (qw >> (4 * i)) & 0xF
            zero = np.zeros((qz.shape[0], N), dtype=np.float32)
            for i in range(8):
                zero[:, i::8] = ((qz >> (4 * i)) & 0xF) + 1
            g_idx = t.get("g_idx")
            gi = np.asarray(g_idx) if g_idx is not None else np.arange(K) // group
        else:
            K, N = qw.shape[0], qw.shape[1] * 8
            q = np.zeros((K, N), dtype=np.float32)
            zero = np.zeros((qz.shape[0], N), dtype=np.float32)
            for i in range(8):
                q[:, _AWQ_ORDER[i]::8] = (qw >> (4 * i)) & 0xF
                zero[:, _AWQ_ORDER[i]::8] = (qz >> (4 * i)) & 0xF
            gi = np.arange(K) // group
        return ((q - zero[gi]) * scale[gi]).T.copy()
    raise UnsupportedFormat(f"{fmt}: no planar decoder")
