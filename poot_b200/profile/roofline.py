"""Rooflines: decode (bytes the plan reads per token against the measured copy bandwidth) and fused
compute+collective kernels (the slower of FLOPs at the measured GEMM peak and bytes over NVLink)
(crates/poot-profile/src/roofline.rs:1-120; the reference pins one ceiling row per device in data/ceilings.tsv)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..target import DeviceCaps, b200


@dataclass
class Roofline:
    achieved: float          # GB/s or TFLOP/s
    ceiling: float
    unit: str
    bound: str               # "hbm" | "tensor" | "nvlink"
    basis: str               # "of measured" | "of fallback"

    @property
    def fraction(self) -> float:
        return self.achieved / self.ceiling if self.ceiling else 0.0

    def __str__(self) -> str:
        return f"{self.achieved:.0f} {self.unit} = {self.fraction:.2f} {self.basis} {self.bound} ceiling ({self.ceiling:.0f} {self.unit})"


def decode_roofline(bytes_per_token: int, ms_per_token: float, caps: Optional[DeviceCaps] = None, ranks: int = 1) -> Roofline:
    """``bytes_per_token`` = whole-model read traffic of one decode step; each of ``ranks`` GPUs streams its share."""
    caps = caps or b200()
    gbs = bytes_per_token / ranks / (ms_per_token * 1e-3) / 1e9
    return Roofline(gbs, caps.hbm_gbs, "GB/s", "hbm", f"of {caps.measured}")


def gemm_roofline(flops: float, ms: float, caps: Optional[DeviceCaps] = None, sustained: bool = False) -> Roofline:
    caps = caps or b200()
    peak = caps.bf16_tflops_sustained if sustained else caps.bf16_tflops
    return Roofline(flops / (ms * 1e-3) / 1e12, peak, "TFLOP/s", "tensor", f"of {caps.measured}")


def fused_collective_roofline(flops: float, nvlink_bytes_per_gpu: float, ms: float, caps: Optional[DeviceCaps] = None,
                              hbm_bytes: float = 0.0) -> Roofline:
    """Target time = the slowest of compute at the measured GEMM peak, bytes that must cross NVLink at the measured
    per-direction link bandwidth, and (for skinny decode shapes) weight bytes at the measured copy bandwidth."""
    caps = caps or b200()
    t_c = flops / (caps.bf16_tflops * 1e12)
    t_l = nvlink_bytes_per_gpu / (caps.nvlink_gbs_measured * 1e9)
    t_m = hbm_bytes / (caps.hbm_gbs * 1e9)
    target = max(t_c, t_l, t_m)
    bound = "tensor" if target == t_c else ("nvlink" if target == t_l else "hbm")
    return Roofline(target / (ms * 1e-3), 1.0, "x target time", bound, f"of {caps.measured}")
