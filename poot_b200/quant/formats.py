"""Every weight storage format as data.

Counterpart of the reference's ``WeightFormat`` + ``FormatDescriptor`` (crates/poot-quant/src/format.rs:141-207):
one descriptor per format - storage shape (self-contained ``blocks`` along K as in GGUF, or ``planar`` with one
tensor per operand role as in safetensors), block geometry, the ggml type id and which code paths exist for it
(host decoder, host encoder, fused device GEMV).  ``IQ2_XS`` / ``IQ3_XXS`` / ``IQ3_S`` are listed but not decodable
in this build: their codebook grids are ggml data tables that are not reproduced here, so loading them is a
typed refusal.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional


@dataclass(frozen=True)
class FormatDescriptor:
    name: str
    storage: str                 # dense | blocks | planar
    block_elems: int = 1
    block_bytes: int = 0
    ggml_type: Optional[int] = None
    decode: bool = True          # host decoder present
    encode: bool = False         # host encoder present
    device_gemv: bool = False    # dequant-fused device GEMV present (others are expanded to bf16 at load)
    note: str = ""

    @property
    def bits_per_weight(self) -> float:
        return 8.0 * self.block_bytes / self.block_elems if self.block_bytes else 0.0


_F = FormatDescriptor
FORMATS: Dict[str, FormatDescriptor] = {f.name: f for f in [
    _F("F32", "dense", 1, 4, 0), _F("F16", "dense", 1, 2, 1, encode=True), _F("BF16", "dense", 1, 2, 30),
    _F("Q4_0", "blocks", 32, 18, 2, encode=True, device_gemv=True), _F("Q4_1", "blocks", 32, 20, 3, encode=True, device_gemv=True),
    _F("Q5_0", "blocks", 32, 22, 6, encode=True, device_gemv=True), _F("Q5_1", "blocks", 32, 24, 7, encode=True, device_gemv=True),
    _F("Q8_0", "blocks", 32, 34, 8, encode=True, device_gemv=True),
    _F("Q2_K", "blocks", 256, 84, 10, encode=True, device_gemv=True), _F("Q3_K", "blocks", 256, 110, 11, encode=True, device_gemv=True),
    _F("Q4_K", "blocks", 256, 144, 12, encode=True, device_gemv=True),
    _F("Q5_K", "blocks", 256, 176, 13, encode=True, device_gemv=True),
    _F("Q6_K", "blocks", 256, 210, 14, encode=True, device_gemv=True),
    _F("IQ4_NL", "blocks", 32, 18, 20, device_gemv=True), _F("IQ4_XS", "blocks", 256, 136, 23, device_gemv=True),
    _F("IQ2_XS", "blocks", 256, 74, 17, decode=False, note="codebook grid not reproduced"),
    _F("IQ3_XXS", "blocks", 256, 98, 18, decode=False, note="codebook grid not reproduced"),
    _F("IQ3_S", "blocks", 256, 110, 21, decode=False, note="codebook grid not reproduced"),
    _F("MXFP4", "blocks", 32, 17, 39, encode=True, device_gemv=True),
    _F("E4M3_CHANNEL", "planar", device_gemv=True, note="fp8 weight + per-output-channel f32 scale", encode=True),
    _F("E4M3_BLOCK128", "planar", device_gemv=True, note="fp8 weight + 128x128 block scales", encode=True),
    _F("E2M1_ROW32", "planar", device_gemv=True, note="fp4 codes + e8m0 scale per 32 values of a row", encode=True),
    _F("GPTQ", "planar", device_gemv=True, note="int4 qweight/qzeros/scales (+g_idx for act-order)", encode=True),
    _F("AWQ", "planar", device_gemv=True, note="int4 qweight/qzeros/scales in AWQ nibble order", encode=True),
]}
GGML_TYPE_TO_FORMAT = {f.ggml_type: f.name for f in FORMATS.values() if f.ggml_type is not None}
# ggml types that exist but are refused by name (as the reference's type table does, crates/poot-load/src/gguf/format.rs:476-520)
GGML_REFUSED = {9: "Q8_1", 15: "Q8_K", 16: "IQ2_XXS", 19: "IQ1_S", 22: "IQ2_S", 29: "IQ1_M", 34: "TQ1_0", 35: "TQ2_0"}


class UnsupportedFormat(ValueError):
    """A stored format this build cannot decode (typed refusal naming the format)."""


def descriptor(name: str) -> FormatDescriptor:
    try:
        return FORMATS[name]
    except KeyError:
        raise UnsupportedFormat(f"unknown weight format {name!r}") from None


def packed_nbytes(name: str, n_elems: int) -> int:
    d = descriptor(name)
    if n_elems % d.block_elems:
        raise UnsupportedFormat(f"{name}: {n_elems} values do not fill whole blocks of {d.block_elems}")
    return n_elems // d.block_elems * d.block_bytes
