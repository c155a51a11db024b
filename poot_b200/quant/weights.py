"""Packed weights and the weight store.

``PackedWeight`` = a stored tensor in its checkpoint format (payload bytes kept as a zero-copy view of the
memory-mapped file, crates/poot-quant/src/stored.rs:1-7); ``WeightStore`` = name -> stored tensor for one
checkpoint, published only after every tensor passed its content check (crates/poot-quant/src/weights.rs:1-6).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, Optional, Tuple

import numpy as np

from . import codec
from .formats import descriptor


@dataclass
class PackedWeight:
    name: str
    format: str                  # key of formats.FORMATS
    shape: Tuple[int, ...]       # logical shape (rows = out features, last axis = K)
    payload: np.ndarray          # raw bytes (uint8 view) for dense / block formats
    planar: Optional[Dict[str, np.ndarray]] = None
    group: int = 128             # int4 planar formats: values per (scale, zero point) along K

    @property
    def nbytes(self) -> int:
        if self.planar is not None:
            return sum(int(v.nbytes) for v in self.planar.values())
        return int(self.payload.nbytes)

    def to_f32(self) -> np.ndarray:
        d = descriptor(self.format)
        if d.storage == "planar":
            return codec.dequantize_planar(self.format, self.planar, self.group)
        return codec.dequantize(self.format, self.payload, self.shape)

    def rows(self, start: int, count: int) -> "PackedWeight":
        """Row range of a block-format matrix without decoding (tensor-parallel output split)."""
        d = descriptor(self.format)
        if d.storage == "planar":
            raise ValueError("row views of planar formats go through their operands")
        row_bytes = self.shape[-1] // d.block_elems * d.block_bytes
        raw = self.payload.reshape(-1)
        return PackedWeight(self.name, self.format, (count,) + tuple(self.shape[1:]),
                            raw[start * row_bytes:(start + count) * row_bytes])

    def cols(self, start: int, count: int) -> "PackedWeight":
        """Column (K) range; legal only on encoding-block boundaries (the reference's IllegalEncodingSplit)."""
        d = descriptor(self.format)
        if start % d.block_elems or count % d.block_elems:
            raise ValueError(f"{self.format}: a K split at {start}+{count} cuts an encoding block of {d.block_elems}")
        N, K = self.shape
        bpr = K // d.block_elems
        raw = self.payload.reshape(N, bpr, d.block_bytes)
        part = np.ascontiguousarray(raw[:, start // d.block_elems:(start + count) // d.block_elems])
        return PackedWeight(self.name, self.format, (N, count), part.reshape(-1))


class WeightStore:
    def __init__(self):
        self._entries: Dict[str, PackedWeight] = {}
        self.metadata: Dict[str, object] = {}
        self.source: Optional[str] = None
        self._published = False

    def add(self, w: PackedWeight) -> None:
        if self._published:
            raise RuntimeError("store is already published")
        if w.name in self._entries:
            raise ValueError(f"duplicate tensor {w.name!r}")
        self._entries[w.name] = w

    def publish(self, check: bool = True) -> "WeightStore":
        if check:
            for w in self._entries.values():
                if w.planar is None:
                    codec.check_scales(w.format, w.payload, int(np.prod(w.shape)))
        self._published = True
        return self

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def __getitem__(self, name: str) -> PackedWeight:
        return self._entries[name]

    def names(self) -> Iterable[str]:
        return self._entries.keys()

    def nbytes(self) -> int:
        return sum(w.nbytes for w in self._entries.values())
