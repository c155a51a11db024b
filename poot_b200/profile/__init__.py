"""Timing snapshots and rooflines (crates/poot-profile/src/timing.rs:30-506, src/roofline.rs:1-120)."""
from .roofline import Roofline, decode_roofline, fused_collective_roofline
from .timing import ExecutionCounters, Report, TimingOptions, TimingSnapshot
