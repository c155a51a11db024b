"""The one dtype vocabulary and the typed host tensor carrier.

Counterpart of the reference's foundation crate (crates/poot-tensor/src/lib.rs:22-58, src/host.rs): fifteen
dtypes that a checkpoint header or a graph value can name, and ``HostTensor`` / ``HostView`` as the typed host
carrier the loaders, the oracle and the executors exchange.  Storage dtypes without arithmetic of their own
(bf16, f16, E4M3FN, E8M0) are carried as raw integer words with exact conversion helpers.
"""
from __future__ import annotations

import math

import enum
from dataclasses import dataclass
from typing import Sequence, Tuple

import numpy as np


class DType(enum.Enum):
    BOOL = "bool"
    I8 = "i8"
    U8 = "u8"
    I16 = "i16"
    U16 = "u16"
    I32 = "i32"
    U32 = "u32"
    I64 = "i64"
    U64 = "u64"
    F16 = "f16"
    BF16 = "bf16"
    F32 = "f32"
    F64 = "f64"
    E4M3FN = "e4m3fn"
    E8M0 = "e8m0"

    @property
    def size(self) -> int:
        return _SIZES[self]

    @property
    def is_float(self) -> bool:
        return self in (DType.F16, DType.BF16, DType.F32, DType.F64, DType.E4M3FN)

    @property
    def is_int(self) -> bool:
        return self in (DType.I8, DType.U8, DType.I16, DType.U16, DType.I32, DType.U32, DType.I64, DType.U64)

    @property
    def storage_numpy(self):
        """numpy dtype of the raw storage words."""
        return _NP[self]

    def __str__(self) -> str:
        return self.value


_SIZES = {DType.BOOL: 1, DType.I8: 1, DType.U8: 1, DType.I16: 2, DType.U16: 2, DType.I32: 4, DType.U32: 4,
          DType.I64: 8, DType.U64: 8, DType.F16: 2, DType.BF16: 2, DType.F32: 4, DType.F64: 8, DType.E4M3FN: 1,
          DType.E8M0: 1}
_NP = {DType.BOOL: np.bool_, DType.I8: np.int8, DType.U8: np.uint8, DType.I16: np.int16, DType.U16: np.uint16,
       DType.I32: np.int32, DType.U32: np.uint32, DType.I64: np.int64, DType.U64: np.uint64, DType.F16: np.float16,
       DType.BF16: np.uint16, DType.F32: np.float32, DType.F64: np.float64, DType.E4M3FN: np.uint8, DType.E8M0: np.uint8}

SAFETENSORS_NAMES = {"BOOL": DType.BOOL, "I8": DType.I8, "U8": DType.U8, "I16": DType.I16, "U16": DType.U16,
                     "I32": DType.I32, "U32": DType.U32, "I64": DType.I64, "U64": DType.U64, "F16": DType.F16,
                     "BF16": DType.BF16, "F32": DType.F32, "F64": DType.F64, "F8_E4M3": DType.E4M3FN,
                     "F8_E8M0": DType.E8M0}


# ---- exact narrow-float conversions ---------------------------------------------------------------------------
def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round to nearest even; NaN stays NaN."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    nan = np.isnan(x)
    return np.where(nan, (u >> 16) | 0x40, rounded).astype(np.uint16)


def round_bf16(x: np.ndarray) -> np.ndarray:
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def round_f16(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


_E4M3_TABLE = None


def e4m3_table() -> np.ndarray:
    """All 256 E4M3FN values as f32 (S.EEEE.MMM, bias 7, no infinities, 0x7F / 0xFF are NaN)."""
    global _E4M3_TABLE
    if _E4M3_TABLE is None:
        t = np.zeros(256, dtype=np.float32)
        for b in range(256):
            s = -1.0 if b & 0x80 else 1.0
            e, m = (b >> 3) & 0xF, b & 7
            if e == 0xF and m == 7:
                v = np.nan
            elif e == 0:
                v = s * (m / 8.0) * 2.0 ** -6
            else:
                v = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
            t[b] = v
        _E4M3_TABLE = t
    return _E4M3_TABLE


def e4m3_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return e4m3_table()[bits.astype(np.uint8)]


def f32_to_e4m3_bits(x: np.ndarray) -> np.ndarray:
    """Round to nearest even, saturating to +-448 (the FN format has no infinity)."""
    x = np.asarray(x, dtype=np.float32)
    t = e4m3_table()
    pos = t[:0x7F].astype(np.float64)               # codes 0x00..0x7E ascending
    a = np.minimum(np.abs(x.astype(np.float64)), 448.0)
    idx = np.clip(np.searchsorted(pos, a), 1, len(pos) - 1)
    lo, hi = pos[idx - 1], pos[idx]
    pick_hi = (a - lo > hi - a) | ((a - lo == hi - a) & (idx % 2 == 0))
    code = np.where(pick_hi, idx, idx - 1).astype(np.uint8)
    code = np.where(a == 0, 0, code).astype(np.uint8)
    out = code | np.where(np.signbit(x), 0x80, 0).astype(np.uint8)
    return np.where(np.isnan(x), np.uint8(0x7F), out).astype(np.uint8)


def e8m0_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    b = bits.astype(np.int32)
    return np.where(b == 255, np.nan, np.ldexp(np.float32(1.0), b - 127)).astype(np.float32)


@dataclass
class HostTensor:
    """A typed host array: ``data`` holds the raw storage words of ``dtype`` in row-major order."""
    shape: Tuple[int, ...]
    dtype: DType
    data: np.ndarray

    @staticmethod
    def f32(shape: Sequence[int], data) -> "HostTensor":
        return HostTensor(tuple(shape), DType.F32, np.asarray(data, dtype=np.float32).reshape(shape))

    @staticmethod
    def i32(shape: Sequence[int], data) -> "HostTensor":
        return HostTensor(tuple(shape), DType.I32, np.asarray(data, dtype=np.int32).reshape(shape))

    @staticmethod
    def from_numpy(a: np.ndarray, dtype: DType = None) -> "HostTensor":
        if dtype is None:
            dtype = {np.dtype(v): k for k, v in _NP.items() if k not in (DType.BF16, DType.E4M3FN, DType.E8M0)}[a.dtype]
        return HostTensor(tuple(a.shape), dtype, np.ascontiguousarray(a))

    def to_f32(self) -> np.ndarray:
        d = self.dtype
        if d == DType.BF16:
            return bf16_bits_to_f32(self.data)
        if d == DType.E4M3FN:
            return e4m3_bits_to_f32(self.data)
        if d == DType.E8M0:
            return e8m0_bits_to_f32(self.data)
        return self.data.astype(np.float32)

    @property
    def nbytes(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n * self.dtype.size

    def view(self, start_row: int, rows: int) -> "HostTensor":
        """A zero-copy view of a run of leading-axis rows (``HostView`` of the reference)."""
        return HostTensor((rows,) + tuple(self.shape[1:]), self.dtype, self.data[start_row:start_row + rows])


# ---- position helpers shared by the tracer and the device engine ------------------------------------------------
def alibi_slopes(n_heads: int, kind: str = "bloom", bias_max: float = 8.0) -> list:
    """Per-head ALiBi slopes.  ``bloom``: geometric series of the closest power of two, the remaining heads take the
    odd powers of the next series (Press et al.); ``mpt``: ``2^-(i * bias_max / n2)`` over the next power of two
    ``n2``, odd entries first when ``n_heads`` is not a power of two."""
    if kind == "mpt":
        n2 = 2 ** math.ceil(math.log2(n_heads))
        sl = [1.0 / 2.0 ** (i * bias_max / n2) for i in range(1, n2 + 1)]
        if n2 != n_heads:
            sl = (sl[1::2] + sl[::2])[:n_heads]
        return sl
    cp2 = 2 ** math.floor(math.log2(n_heads))
    base = 2.0 ** (-(2.0 ** -(math.log2(cp2) - 3)))
    sl = [base ** i for i in range(1, cp2 + 1)]
    if cp2 != n_heads:
        extra = 2.0 ** (-(2.0 ** -(math.log2(2 * cp2) - 3)))
        sl += [extra ** i for i in range(1, 1 + 2 * min(cp2, n_heads - cp2), 2)]
    return sl
