"""Quantised safetensors checkpoints: the tensors a quantisation method stores for one linear layer become ONE stored
weight in a planar format.

``config.json``'s ``quantization_config`` names the method; the checkpoint then holds, per linear ``X``:

* fp8 (``quant_method: fp8``): ``X.weight`` as e4m3 codes with ``X.weight_scale_inv`` ``[N/128, K/128]`` when
  ``weight_block_size`` is ``[128, 128]`` (DeepSeek-V3 layout) -> ``E4M3_BLOCK128``; otherwise ``X.weight_scale`` as a
  scalar, ``[N]`` or ``[N, 1]`` -> ``E4M3_CHANNEL`` (a scalar is broadcast over the rows);
* GPTQ (``quant_method: gptq``, 4 bits): ``X.qweight [K/8, N]``, ``X.qzeros [K/g, N/8]``, ``X.scales [K/g, N]``,
  ``X.g_idx [K]`` -> ``GPTQ``;
* AWQ (``quant_method: awq``, 4 bits, GEMM layout): ``X.qweight [K, N/8]``, ``X.qzeros``, ``X.scales`` -> ``AWQ``.

``planar_view`` wraps a weight store so that the name tables see ``X.weight`` as one ``PackedWeight`` whose ``planar``
operands are the stored arrays (zero-copy views of the mapped files); the operand names disappear.  Anything the
method leaves unquantised (embeddings, norms, the head, routers) passes through.  Formats and layouts follow the
reference's planar descriptors (crates/poot-quant/src/format.rs:141-207); other methods are typed refusals.
"""
from __future__ import annotations

from typing import Dict, Iterable, Optional

import numpy as np

from ..quant.formats import UnsupportedFormat
from ..quant.weights import PackedWeight

_OPERANDS = ("weight_scale_inv", "weight_scale", "qweight", "qzeros", "scales", "g_idx", "input_scale")


def _raw(w: PackedWeight) -> np.ndarray:
    if w.planar is not None and "__raw__" in w.planar:
        return w.planar["__raw__"]
    return w.to_f32()


class PlanarView:
    """Store-like: ``names()`` / ``__getitem__`` / ``__contains__`` over the assembled weights."""

    def __init__(self, store, qcfg: dict):
        self.store, self.metadata, self.source = store, getattr(store, "metadata", {}), getattr(store, "source", None)
        method = str(qcfg.get("quant_method", "")).lower()
        self.method = method
        bits = int(qcfg.get("bits", qcfg.get("w_bit", 4)) or 4)
        self.group = int(qcfg.get("group_size", qcfg.get("q_group_size", 128)) or 128)
        if method in ("gptq", "awq"):
            if bits != 4:
                raise UnsupportedFormat(f"{method} with {bits}-bit weights (4-bit layouts only)")
            if self.group <= 0:
                raise UnsupportedFormat(f"{method} with one group per column (group_size -1)")
            if method == "awq" and str(qcfg.get("version", "gemm")).lower() != "gemm":
                raise UnsupportedFormat(f"awq version {qcfg.get('version')!r} (the GEMM layout only)")
        elif method == "fp8":
            blk = qcfg.get("weight_block_size")
            if blk not in (None, [128, 128], (128, 128)):
                raise UnsupportedFormat(f"fp8 with weight blocks {blk} (128 x 128 only)")
            if str(qcfg.get("fmt", "e4m3")).lower() not in ("e4m3", "float8_e4m3fn"):
                raise UnsupportedFormat(f"fp8 format {qcfg.get('fmt')!r}")
        else:
            raise UnsupportedFormat(f"quantisation method {method!r} (fp8, gptq and awq checkpoints load)")
        self._made: Dict[str, PackedWeight] = {}
        self._hidden = set()
        names = set(store.names())
        for n in names:
            stem, _, leaf = n.rpartition(".")
            if leaf in _OPERANDS and (stem + ".weight" in names or stem + ".qweight" in names):
                self._hidden.add(n)
        self._quantised = set()
        for n in names:
            stem, _, leaf = n.rpartition(".")
            if leaf == "qweight" and method in ("gptq", "awq"):
                self._quantised.add(stem + ".weight")
            elif leaf == "weight" and method == "fp8" and (stem + ".weight_scale_inv" in names or stem + ".weight_scale" in names):
                self._quantised.add(n)

    def names(self) -> Iterable[str]:
        plain = [n for n in self.store.names() if n not in self._hidden and n not in self._quantised]
        return plain + sorted(self._quantised)

    def __contains__(self, name: str) -> bool:
        return name in self._quantised or (name in self.store and name not in self._hidden)

    def nbytes(self) -> int:
        return self.store.nbytes()

    def __getitem__(self, name: str) -> PackedWeight:
        if name not in self._quantised:
            if name in self._hidden:
                raise KeyError(name)
            return self.store[name]
        w = self._made.get(name)
        if w is None:
            w = self._made[name] = self._assemble(name)
        return w

    def _assemble(self, name: str) -> PackedWeight:
        stem = name[:-len(".weight")]
        get = lambda leaf: _raw(self.store[stem + "." + leaf])
        has = lambda leaf: stem + "." + leaf in self.store
        empty = np.zeros(0, np.uint8)
        if self.method == "fp8":
            codes = get("weight")
            if codes.dtype != np.uint8:
                codes = codes.view(np.uint8)
            N, K = codes.shape
            if has("weight_scale_inv"):
                s = np.asarray(get("weight_scale_inv"), np.float32)
                if s.shape != ((N + 127) // 128, (K + 127) // 128):
                    raise UnsupportedFormat(f"{name}: block scales {s.shape} do not cover {(N, K)} in 128 x 128 blocks")
                return PackedWeight(name, "E4M3_BLOCK128", (N, K), empty, planar={"weight": codes, "weight_scale_inv": s})
            s = np.asarray(get("weight_scale"), np.float32).reshape(-1)
            if s.size == 1:
                s = np.full(N, s[0], np.float32)
            if s.size != N:
                raise UnsupportedFormat(f"{name}: {s.size} scales for {N} output channels")
            return PackedWeight(name, "E4M3_CHANNEL", (N, K), empty, planar={"weight": codes, "weight_scale": s})
        qw, qz = get("qweight").view(np.int32), get("qzeros").view(np.int32)
        sc = np.asarray(get("scales"), np.float32)
        if self.method == "gptq":
            K, N = qw.shape[0] * 8, qw.shape[1]
            ops = {"qweight": qw, "qzeros": qz, "scales": sc}
            if has("g_idx"):
                g = np.asarray(get("g_idx")).astype(np.int32)
                if not np.array_equal(g, np.arange(K, dtype=np.int32) // self.group):
                    ops["g_idx"] = g                   # act-order: groups are not contiguous along K
            fmt = "GPTQ"
        else:
            K, N = qw.shape[0], qw.shape[1] * 8
            ops, fmt = {"qweight": qw, "qzeros": qz, "scales": sc}, "AWQ"
        if sc.shape != (K // self.group, N) or qz.shape != (K // self.group, N // 8):
            raise UnsupportedFormat(f"{name}: scales {sc.shape} / zeros {qz.shape} do not match {(N, K)} in groups of {self.group}")
        return PackedWeight(name, fmt, (N, K), empty, planar=ops, group=self.group)


def planar_view(store, hf_config: dict):
    """``store`` itself when the checkpoint is not quantised, else the assembled view."""
    qcfg: Optional[dict] = hf_config.get("quantization_config")
    if not qcfg:
        return store
    return PlanarView(store, qcfg)


# ---- row surgery on planar weights (fused projections keep their packed form) -----------------------------------------
_AWQ_ORDER = np.array([0, 4, 1, 5, 2, 6, 3, 7])


def _unpack_cols(words: np.ndarray, awq: bool) -> np.ndarray:
    """int32 words holding eight 4-bit values along the LAST axis -> uint8 ``[..., 8 * words]``."""
    u = words.view(np.uint32)
    out = np.empty(u.shape[:-1] + (u.shape[-1] * 8,), np.uint8)
    for i in range(8):
        out[..., (_AWQ_ORDER[i] if awq else i)::8] = (u >> (4 * i)) & 0xF
    return out


def _pack_cols(vals: np.ndarray, awq: bool) -> np.ndarray:
    u = np.zeros(vals.shape[:-1] + (vals.shape[-1] // 8,), np.uint32)
    for i in range(8):
        u |= vals[..., (_AWQ_ORDER[i] if awq else i)::8].astype(np.uint32) << (4 * i)
    return u.view(np.int32)


def planar_take_rows(w: PackedWeight, order: np.ndarray) -> PackedWeight:
    """Output rows ``order`` of a planar weight, still packed (exact: codes, scales and zero points move with their rows).
    128 x 128 block scales survive only when ``order`` moves whole aligned row blocks; otherwise ``ValueError``."""
    order = np.asarray(order, np.int64)
    p, fmt, (N, K) = w.planar, w.format, w.shape
    n = len(order)
    if fmt == "E4M3_CHANNEL":
        ops = {"weight": p["weight"][order], "weight_scale": np.asarray(p["weight_scale"], np.float32).reshape(-1)[order]}
    elif fmt == "E2M1_ROW32":
        ops = {"weight": p["weight"][order], "weight_scale": p["weight_scale"].reshape(N, -1)[order]}
    elif fmt == "E4M3_BLOCK128":
        if n % 128 or np.any(order.reshape(-1, 128)[:, 0] % 128) or np.any(np.diff(order.reshape(-1, 128), axis=1) != 1):
            raise ValueError("128 x 128 block scales: rows move in whole aligned blocks only")
        ops = {"weight": p["weight"][order], "weight_scale_inv": p["weight_scale_inv"][order.reshape(-1, 128)[:, 0] // 128]}
    elif fmt in ("GPTQ", "AWQ"):
        if n % 8:
            raise ValueError("int4 planar formats: a multiple of eight output columns")
        awq = fmt == "AWQ"
        zeros = _unpack_cols(p["qzeros"], awq)[:, order]
        ops = {"qzeros": _pack_cols(zeros, awq), "scales": np.asarray(p["scales"], np.float32)[:, order]}
        if awq:
            ops["qweight"] = _pack_cols(_unpack_cols(p["qweight"], True)[:, order], True)
        else:
            ops["qweight"] = np.ascontiguousarray(p["qweight"][:, order])
            if "g_idx" in p:
                ops["g_idx"] = p["g_idx"]
    else:
        raise ValueError(f"{fmt} is not a planar format")
    return PackedWeight(w.name, fmt, (n, K), np.zeros(0, np.uint8), planar=ops, group=w.group)


def planar_cat_rows(parts) -> PackedWeight:
    """Row concatenation of planar weights of one format, group size and K (a fused q|k|v or gate|up projection)."""
    parts = list(parts)
    fmt, K, group = parts[0].format, parts[0].shape[1], parts[0].group
    if any(x.format != fmt or x.shape[1] != K or x.group != group for x in parts):
        raise ValueError("fused projection mixes planar formats, widths or group sizes")
    if any(("g_idx" in x.planar) != ("g_idx" in parts[0].planar) for x in parts) or \
            ("g_idx" in parts[0].planar and any(not np.array_equal(x.planar["g_idx"], parts[0].planar["g_idx"]) for x in parts)):
        raise ValueError("fused projection mixes act-order group maps")
    if fmt == "E4M3_BLOCK128" and any(x.shape[0] % 128 for x in parts[:-1]):
        raise ValueError("128 x 128 block scales: every part but the last must be a multiple of 128 rows")
    if fmt in ("GPTQ", "AWQ") and any(x.shape[0] % 8 for x in parts):
        raise ValueError("int4 planar formats: parts of a multiple of eight output columns")
    N = sum(x.shape[0] for x in parts)
    axis = {"weight": 0, "weight_scale": 0, "weight_scale_inv": 0, "qweight": 1, "qzeros": 1, "scales": 1}
    ops = {}
    for k in parts[0].planar:
        if k == "g_idx":
            ops[k] = parts[0].planar[k]
            continue
        arrs = [np.asarray(x.planar[k]).reshape(x.shape[0], -1) if (k == "weight_scale" and fmt != "E4M3_CHANNEL") else
                (np.asarray(x.planar[k]).reshape(-1) if k == "weight_scale" else x.planar[k]) for x in parts]
        ops[k] = np.ascontiguousarray(np.concatenate(arrs, axis=axis[k]))
    return PackedWeight("+".join(x.name for x in parts), fmt, (N, K), np.zeros(0, np.uint8), planar=ops, group=group)
