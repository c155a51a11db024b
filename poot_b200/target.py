"""Device description the planner and the capacity fit read (crates/poot-target/src/lib.rs:474-545).

One target: NVIDIA B200 (sm_100a).  Nominal figures come from the public datasheet; the roofline denominators are
the figures MEASURED on the deployment's own GPUs (a STREAM-style copy and a library bf16 GEMM, burst and sustained)
when a ``MEASURED_PEAKS.json`` is present next to the package root, else the recorded fallback of an earlier
measurement on the same kind of machine.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, Optional


@dataclass(frozen=True)
class MatrixUnits:
    """5th-generation tensor cores: one elected thread issues ``tcgen05.mma``; accumulators live in tensor memory."""
    m: int = 128
    n_max: int = 256
    k_bf16: int = 16
    tmem_columns: int = 512          # 256 KB per SM
    cta_pair: bool = True            # cta_group::2
    dense_tflops: Dict[str, float] = field(default_factory=lambda: {"bf16": 2250.0, "f16": 2250.0, "fp8": 4500.0,
                                                                    "fp4": 9000.0, "tf32": 1100.0})


@dataclass(frozen=True)
class DeviceCaps:
    name: str = "NVIDIA B200"
    arch: str = "sm_100a"
    sms: int = 148
    dies: int = 2
    warp: int = 32
    smem_per_cta: int = 227 * 1024
    l2_bytes: int = 126 << 20
    hbm_bytes: int = 180 * 10**9
    hbm_gbs_nominal: float = 7700.0
    sm_max_mhz: float = 1965.0
    max_cluster: int = 8
    nvlink_gbs_per_dir: float = 900.0
    nvlink_gbs_measured: float = 770.0       # peer copy, per direction
    allreduce_busbw_gbs_measured: float = 725.0
    peer_transport: str = "nvlink5-nvswitch"
    matrix: MatrixUnits = field(default_factory=MatrixUnits)
    # measured roofline denominators
    hbm_gbs: float = 6650.0
    bf16_tflops: float = 1590.0
    bf16_tflops_sustained: float = 1400.0
    measured: str = "fallback"               # "measured" when read from MEASURED_PEAKS.json

    def tma_x_multiple(self, itemsize: int) -> int:
        """Innermost TMA coordinate granularity: the copy must start on a 16-byte boundary."""
        return max(1, 16 // itemsize)

    def grid_for(self, ctas_per_sm: int = 1) -> int:
        return self.sms * ctas_per_sm


def _peaks_path() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")


def b200(peaks_file: Optional[str] = None) -> DeviceCaps:
    path = peaks_file or _peaks_path()
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return DeviceCaps(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]),
                          bf16_tflops_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                          sm_max_mhz=float(p.get("sm_max_mhz", 1965.0)), measured="measured")
    return DeviceCaps()


def from_device(index: int = 0) -> DeviceCaps:
    """Caps with the live device's SM count and memory (requires a GPU)."""
    import dataclasses
    import torch
    props = torch.cuda.get_device_properties(index)
    if props.major != 10:
        raise RuntimeError(f"{props.name} is compute capability {props.major}.{props.minor}; this build targets sm_100a only")
    return dataclasses.replace(b200(), name=props.name, sms=props.multi_processor_count, hbm_bytes=props.total_memory)
