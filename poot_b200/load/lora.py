"""LoRA (PEFT) adapters: ``adapter_config.json`` + ``adapter_model.safetensors``
(crates/poot-load/src/lora.rs:42-119).

An adapter adds ``scale * B @ A`` to each targeted projection (``scale = lora_alpha / r``, or ``/ sqrt(r)`` with
rsLoRA).  The reference selects an adapter per request with an indexed contraction
(crates/poot-graph-plan/src/passes/lora.rs:1-7); here adapters are MERGED into the bf16 projection weights when the
model is loaded (one resident adapter per served model: at decode the projections are bandwidth-bound, so a merged
weight costs nothing per token, and switching adapters is a reload).  Refused, typed: adapters over packed
(block-quantised) projections, unknown target modules, rank / shape mismatches, DoRA and bias training.
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass
from typing import Dict, Tuple

import numpy as np

from . import safetensors as st
from .names import HF_LAYER


class LoraError(ValueError):
    pass


@dataclass
class LoraAdapter:
    name: str
    rank: int
    scale: float
    deltas: Dict[str, Tuple[np.ndarray, np.ndarray]]       # canonical weight name -> (A [r, in], B [out, r]) as f32

    def delta(self, canonical: str) -> np.ndarray:
        a, b = self.deltas[canonical]
        return self.scale * (b @ a)


_KEY = re.compile(r"(?:base_model\.model\.)?model\.layers\.(\d+)\.(.+?)\.lora_([AB])\.weight$")


def load_adapter(path: str, name: str = "") -> LoraAdapter:
    cfg_path = os.path.join(path, "adapter_config.json")
    if not os.path.exists(cfg_path):
        raise LoraError(f"{path}: no adapter_config.json")
    with open(cfg_path) as f:
        cfg = json.load(f)
    if cfg.get("peft_type", "LORA") != "LORA":
        raise LoraError(f"adapter type {cfg.get('peft_type')!r} is not LoRA")
    if cfg.get("use_dora"):
        raise LoraError("DoRA adapters are not supported")
    if cfg.get("bias", "none") != "none":
        raise LoraError("adapters that train biases are not supported")
    r = int(cfg.get("r", 0))
    if r < 1:
        raise LoraError("adapter rank must be positive")
    alpha = float(cfg.get("lora_alpha", r))
    scale = alpha / (r ** 0.5) if cfg.get("use_rslora") else alpha / r
    tensors = st.read_tensors(os.path.join(path, "adapter_model.safetensors"))
    halves: Dict[str, Dict[str, np.ndarray]] = {}
    for key, val in tensors.items():
        if key == "__mmap__":
            continue
        m = _KEY.match(key)
        if not m:
            raise LoraError(f"adapter tensor {key!r} does not target a decoder projection")
        layer, module, which = m.group(1), m.group(2) + ".weight", m.group(3)
        if module not in HF_LAYER:
            raise LoraError(f"adapter targets unknown module {m.group(2)!r}")
        dt, shape, raw = val
        arr = st.as_numpy(dt, shape, raw)
        if dt.value == "bf16":
            arr = (arr.astype(np.uint32) << 16).view(np.float32)
        halves.setdefault(f"layers.{layer}.{HF_LAYER[module]}", {})[which] = np.asarray(arr, dtype=np.float32)
    deltas = {}
    for canon, ab in halves.items():
        if set(ab) != {"A", "B"}:
            raise LoraError(f"{canon}: adapter has only lora_{next(iter(ab))}")
        a, b = ab["A"], ab["B"]
        if a.shape[0] != r or b.shape[1] != r:
            raise LoraError(f"{canon}: factors {a.shape} / {b.shape} do not have rank {r}")
        deltas[canon] = (a, b)
    if not deltas:
        raise LoraError("adapter has no tensors")
    return LoraAdapter(name or os.path.basename(os.path.normpath(path)), r, scale, deltas)


def merge_into(named: Dict[str, np.ndarray], adapter: LoraAdapter) -> Dict[str, np.ndarray]:
    """``named``: canonical name -> f32 ``[out, in]`` weights; returns a copy with the adapter's deltas added."""
    out = dict(named)
    for canon in adapter.deltas:
        if canon not in named:
            raise LoraError(f"adapter targets {canon}, which the model does not have")
        w = named[canon]
        d = adapter.delta(canon)
        if d.shape != w.shape:
            raise LoraError(f"{canon}: adapter delta {d.shape} does not match the weight {w.shape}")
        out[canon] = (w.astype(np.float32) + d).astype(w.dtype)
    return out
