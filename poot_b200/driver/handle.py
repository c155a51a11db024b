"""Model handle: checkpoint -> family, configuration, weight store -> device weights.

``ModelHandle.load`` resolves the family from ``config.json`` (HF directory) or the GGUF header before any weight
is read, maps the checkpoint tensor names to canonical roles, and keeps the stored tensors as zero-copy views of
the mapped files (crates/poot-llm/src/driver/handle.rs:233; crates/poot-load/src/plan.rs:51-115).
``device_weights`` uploads a rank's share in the layouts the kernels read: packed GGUF formats with a fused device
GEMV stay packed (``QuantWeight``), every other stored format is expanded to bf16 once at load.
"""
from __future__ import annotations

import json
import re
import os
from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np

from ..load import gguf, names, safetensors as st
from ..models.config import DecoderConfig
from ..models.model import Model
from ..models.registry import Registry
from ..quant import codec
from ..quant.formats import FORMATS
from ..quant.weights import PackedWeight, WeightStore


@dataclass
class ModelHandle:
    model: Model
    store: WeightStore
    canonical: Dict[str, PackedWeight]     # canonical role name -> stored tensor
    source: str
    kind: str                              # "hf" | "gguf"
    tokenizer_dir: Optional[str] = None
    adapter: Optional[str] = None          # name of the merged LoRA adapter, if any

    @property
    def cfg(self) -> DecoderConfig:
        return self.model.cfg

    @staticmethod
    def load(path: str, registry: Optional[Registry] = None) -> "ModelHandle":
        registry = registry or Registry.builtin()
        if os.path.isdir(path):
            with open(os.path.join(path, "config.json")) as f:
                hf_config = json.load(f)
            model = registry.resolve_hf(hf_config)
            from ..load.planar import planar_view
            store = planar_view(st.load_weight_store(path), hf_config)    # fp8 / GPTQ / AWQ linears become planar weights
            from ..load.hf_map import map_checkpoint
            canon = map_checkpoint(model.cfg, store)
            return ModelHandle(model, store, canon, path, "hf", path)
        store = gguf.read_gguf(path)
        arch = store.metadata.get("general.architecture")
        meta = store.metadata
        if arch == "gemma4":
            # what this family's header leaves to the tensor list: the global layers' rotary tail is NoPE where
            # ``rope_freqs.weight`` divides a frequency away, a global layer without ``attn_v`` reads its value from the
            # key projection, and ``output.weight`` is there only when the head is not the embedding
            meta = dict(meta)
            have = set(store.names())
            if "rope_freqs.weight" in have:
                f = store["rope_freqs.weight"].to_f32()
                meta["tensors.rope_proportion"] = float((f == 1.0).sum()) / max(1, f.size)
            local = [bool(x) for x in meta.get("gemma4.attention.sliding_window_pattern", [])]
            meta["tensors.value_is_key"] = any(not loc and f"blk.{l}.attn_v.weight" not in have for l, loc in enumerate(local))
            meta["tensors.has_output"] = "output.weight" in have
        model = registry.resolve_gguf(arch, meta)
        canon = {}
        stacked = {}
        fam = model.cfg.family
        paired = fam in names.GGUF_PAIRED_QK
        bias_parts = {}
        latent_parts = {}
        cfg = model.cfg
        for n in store.names():
            m = re.match(r"blk\.(\d+)\.(.+)$", n)
            if m and int(m.group(1)) >= cfg.n_layers:
                continue                                       # blocks a converter appends after the stack (multi-token prediction)
            x = re.match(r"blk\.(\d+)\.ffn_(gate_up|down)_exps\.weight#(\d+)$", n)
            if x and fam == "gemma4":                          # this tracer reads the experts as the stacks the file holds
                stacked.setdefault((int(x.group(1)), "experts_in" if x.group(2) == "gate_up" else "experts_out"), {})[int(x.group(3))] = store[n].to_f32()
                continue
            if n == "rope_freqs.weight":
                continue
            if m and fam == "qwen38_27b":
                from ..load.hf_map import qwen35_gguf_tensor
                if qwen35_gguf_tensor(cfg, f"layers.{m.group(1)}.", m.group(2), store[n], canon):
                    continue
            c = names.canonical_from_gguf(n, fam)
            if c is None:
                m = re.match(r"blk\.(\d+)\.ffn_(gate|up|down)_exps\.bias$", n)          # gpt-oss: one bias row per expert
                if m:
                    bias_parts.setdefault(int(m.group(1)), {})[m.group(2)] = store[n].to_f32()
                m = re.match(r"blk\.(\d+)\.(attn_qkv)\.(weight|bias)$", n)
                if m and m.group(2) + "." + m.group(3) in names.GGUF_FUSED_QKV:          # q rows | k rows | v rows
                    from ..load.hf_map import f32_weight
                    p, w = f"layers.{m.group(1)}.", store[n]
                    nq, nk = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
                    if w.shape[0] != nq + 2 * nk:
                        raise KeyError(f"{n}: {w.shape[0]} rows, expected {nq} + 2 x {nk}")
                    suffix = "" if m.group(3) == "weight" else "_bias"
                    for role, lo, cnt in (("attn_q", 0, nq), ("attn_k", nq, nk), ("attn_v", nq + nk, nk)):
                        canon[p + role + suffix] = w.rows(lo, cnt) if suffix == "" else f32_weight(p + role + suffix, w.to_f32()[lo:lo + cnt])
                m = re.match(r"blk\.(\d+)\.attn_(k|v)_b\.weight$", n)                    # the latent up-projection stored per head
                if m and fam == "deepseek2":
                    latent_parts.setdefault(int(m.group(1)), {})[m.group(2)] = store[n].to_f32()
                continue
            w = store[n]
            if paired and c.endswith(("attn_q", "attn_k")) and len(w.shape) == 2:
                heads = model.cfg.n_heads if c.endswith("attn_q") else model.cfg.n_kv_heads
                w = _permute_rows(w, names.gguf_qk_row_order(w.shape[0], heads))
            canon[c] = w
        for l, parts in bias_parts.items():
            from ..load.hf_map import f32_weight
            if {"gate", "up", "down"} - set(parts):
                raise KeyError(f"blk.{l}: expert biases without {sorted({'gate', 'up', 'down'} - set(parts))}")
            canon[f"layers.{l}.experts_in_bias"] = f32_weight(f"layers.{l}.experts_in_bias", np.concatenate([parts["gate"], parts["up"]], 1))
            canon[f"layers.{l}.experts_out_bias"] = f32_weight(f"layers.{l}.experts_out_bias", parts["down"])
        for (l, role), parts in stacked.items():
            from ..load.hf_map import f32_weight
            canon[f"layers.{l}.{role}"] = f32_weight(f"layers.{l}.{role}", np.stack([parts[e] for e in sorted(parts)]))
        if fam == "gemma4":
            for l in range(cfg.n_layers):                      # K/V of a layer that reads another layer's cache are stored and unused
                for role in ("attn_k", "attn_v", "attn_k_norm"):
                    if cfg.kv_source(l) is not None or (role == "attn_v" and cfg.value_is_key(l)):
                        canon.pop(f"layers.{l}.{role}", None)
        for l, parts in latent_parts.items():
            # ``attn_k_b`` [heads, latent, nope] and ``attn_v_b`` [heads, value, latent] are the two halves of each head's
            # rows of the up-projection the tracer reads as one matrix: nope rows (the key half transposed back), then value rows
            from ..load.hf_map import f32_weight
            if set(parts) != {"k", "v"}:
                raise KeyError(f"blk.{l}: attn_k_b and attn_v_b come as a pair")
            k_b = parts["k"].reshape(cfg.n_heads, cfg.kv_lora_rank, cfg.qk_nope_dim).transpose(0, 2, 1)
            v_b = parts["v"].reshape(cfg.n_heads, cfg.v_head_dim, cfg.kv_lora_rank)
            canon[f"layers.{l}.attn_kv_b"] = f32_weight(f"layers.{l}.attn_kv_b", np.concatenate([k_b, v_b], 1).reshape(-1, cfg.kv_lora_rank))
        if fam == "deepseek2" and cfg.rope_interleaved:
            from ..load.hf_map import _mla_halfsplit
            _mla_halfsplit(cfg, canon)                         # the converter keeps the rotary pairs interleaved, like the source checkpoint
        if "lm_head" not in canon and "embed" in canon:
            model.cfg.tie_embeddings = True
        return ModelHandle(model, store, canon, path, "gguf", None)

    def f32(self, name: str) -> np.ndarray:
        return self.canonical[name].to_f32()

    def apply_adapter(self, adapter) -> None:
        """Merge a LoRA adapter into the targeted projections (``W + scale * B @ A``), replacing their stored tensors
        by f32 ones; refused over block-quantised projections."""
        from ..load.lora import LoraError
        from .features import Feature, Incompatible
        for canon in adapter.deltas:
            if canon not in self.canonical:
                raise LoraError(f"adapter targets {canon}, which the model does not have")
            w = self.canonical[canon]
            if w.format not in ("F32", "F16", "BF16"):
                raise Incompatible(Feature.ADAPTERS, Feature.PACKED_WEIGHTS, f"{canon} is stored as {w.format}")
            d = adapter.delta(canon)
            if tuple(d.shape) != tuple(w.shape):
                raise LoraError(f"{canon}: adapter delta {d.shape} does not match the weight {tuple(w.shape)}")
            merged = (w.to_f32() + d).astype(np.float32)
            self.canonical[canon] = PackedWeight(w.name, "F32", tuple(w.shape), merged.view(np.uint8).reshape(-1))
        self.adapter = adapter.name

    def _stack_experts(self, out: Dict[str, np.ndarray], p: str) -> None:
        c = self.cfg
        if p + "experts_in" in out:          # the family's checkpoint stores the experts stacked in this layout
            return
        if c.gated_ffn:
            gi = np.stack([np.concatenate([self.f32(p + f"experts.{e}.gate"), self.f32(p + f"experts.{e}.up")], 0)
                           for e in range(c.n_experts)])
        else:
            gi = np.stack([self.f32(p + f"experts.{e}.up") for e in range(c.n_experts)])
        out[p + "experts_in"] = gi
        out[p + "experts_out"] = np.stack([self.f32(p + f"experts.{e}.down") for e in range(c.n_experts)])

    def packed_oracle_weights(self):
        """``(weights, formats)`` for the oracle over packed weights: the 2-D weights the checkpoint stores in a GGUF
        block format stay as their bytes (``formats[name]`` names the format), everything else is decoded to f32.
        Families whose tracer declares every weight dense (their own tracers, routed experts) decode as usual."""
        from ..quant.formats import FORMATS
        out = self.oracle_weights(skip_packed=True)
        formats = {}
        if type(self.model).__name__ == "Model":
            for n, w in self.canonical.items():
                d = FORMATS[w.format]
                if n not in out and d.storage == "blocks" and len(w.shape) == 2:
                    out[n] = np.ascontiguousarray(w.payload).view(np.uint8).reshape(-1)
                    formats[n] = w.format
        for n, w in self.canonical.items():          # what the packed declaration does not cover is decoded after all
            if n not in out and ".experts." not in n and not n.startswith("mtp.") and not n.startswith(f"layers.{self.cfg.n_layers}."):
                out[n] = w.to_f32()
        return out, formats

    def oracle_weights(self, skip_packed: bool = False) -> Dict[str, np.ndarray]:
        """Every canonical weight decoded to f32 in the tracer's layout (experts stacked gate-then-up).  ``skip_packed``
        leaves out the 2-D weights stored in a quantised block format (``packed_oracle_weights`` keeps those as stored)."""
        from ..quant.formats import FORMATS
        c = self.cfg
        out = {}
        if skip_packed:
            keep = lambda w: not (FORMATS[w.format].storage == "blocks" and w.format not in ("F32", "F16", "BF16") and len(w.shape) == 2)
            tail = f"layers.{c.n_layers}."
            for n, w in self.canonical.items():
                if ".experts." not in n and not n.startswith(tail) and not n.startswith("mtp.") and keep(w):
                    out[n] = w.to_f32()
            for l in range(c.n_layers):
                if c.has_ffn(l) and c.moe_layer(l):
                    self._stack_experts(out, f"layers.{l}.")
            if c.tie_embeddings:
                out.pop("lm_head", None)
            return out
        tail = f"layers.{c.n_layers}."          # a multi-token-prediction layer's block: ``mtp_oracle_weights``
        for n, w in self.canonical.items():
            if ".experts." not in n and not n.startswith(tail) and not n.startswith("mtp."):
                out[n] = w.to_f32()
        if getattr(self.model, "kind", "decoder") == "encoder":
            return out
        for l in range(c.n_layers):
            if c.has_ffn(l) and c.moe_layer(l):
                self._stack_experts(out, f"layers.{l}.")
        if c.tie_embeddings:
            out.pop("lm_head", None)
        return out

    @property
    def has_mtp(self) -> bool:
        """The configuration names a multi-token-prediction layer AND the checkpoint stores it (conversions often
        drop it)."""
        return self.cfg.mtp_layers > 0 and "mtp.eh_proj" in self.canonical

    def mtp_named(self) -> Dict[str, PackedWeight]:
        """Canonical names of the multi-token-prediction layer as a one-layer model (block renamed to layer 0, its
        closing norm as ``final_norm``, the target's embedding and head)."""
        c = self.cfg
        if not self.has_mtp:
            raise KeyError(f"{self.source} stores no multi-token-prediction layer")
        tail = f"layers.{c.n_layers}."
        out = {"layers.0." + n[len(tail):]: w for n, w in self.canonical.items() if n.startswith(tail)}
        for n in ("mtp.enorm", "mtp.hnorm", "mtp.eh_proj"):
            out[n] = self.canonical[n]
        out["final_norm"], out["embed"] = self.canonical["mtp.head_norm"], self.canonical["embed"]
        if not c.tie_embeddings and "lm_head" in self.canonical:
            out["lm_head"] = self.canonical["lm_head"]
        return out

    def mtp_oracle_weights(self) -> Dict[str, np.ndarray]:
        """The multi-token-prediction layer as the one-layer model ``models.config.mtp_config`` describes: its block
        renamed to layer 0, its closing norm as ``final_norm``, the target's embedding and head."""
        c = self.cfg
        if not self.has_mtp:
            raise KeyError(f"{self.source} stores no multi-token-prediction layer")
        tail = f"layers.{c.n_layers}."
        out = {"layers.0." + n[len(tail):]: w.to_f32() for n, w in self.canonical.items()
               if n.startswith(tail) and ".experts." not in n}
        if self.model.mtp_model().cfg.moe_layer(0):
            src = {}
            self._stack_experts(src, tail)
            out.update({"layers.0." + k[len(tail):]: v for k, v in src.items()})
        for n in ("mtp.enorm", "mtp.hnorm", "mtp.eh_proj"):
            out[n] = self.f32(n)
        out["final_norm"] = self.f32("mtp.head_norm")
        out["embed"] = self.f32("embed")
        if not c.tie_embeddings:
            out["lm_head"] = self.f32("lm_head")
        return out


def _permute_rows(w: PackedWeight, order: np.ndarray) -> PackedWeight:
    d = FORMATS[w.format]
    row_bytes = w.shape[-1] // d.block_elems * d.block_bytes
    raw = np.ascontiguousarray(w.payload).view(np.uint8).reshape(w.shape[0], row_bytes)
    return PackedWeight(w.name, w.format, w.shape, np.ascontiguousarray(raw[order]).reshape(-1))


# ---- device upload ---------------------------------------------------------------------------------------------
def _rows(w: PackedWeight, start: int, count: int) -> PackedWeight:
    if FORMATS[w.format].storage == "planar":
        if start == 0 and count == w.shape[0]:
            return w
        from ..load.planar import planar_take_rows
        return planar_take_rows(w, np.arange(start, start + count))
    return w.rows(start, count)


def _planar(w: PackedWeight) -> bool:
    return FORMATS[w.format].storage == "planar"


def _dense_f32(w: PackedWeight) -> PackedWeight:
    a = np.ascontiguousarray(w.to_f32(), dtype=np.float32)
    return PackedWeight(w.name, "F32", tuple(a.shape), a.view(np.uint8).reshape(-1))


def _cat_rows(parts) -> PackedWeight:
    fmt = parts[0].format
    if any(p.format != fmt for p in parts):
        raise ValueError("fused projection mixes storage formats")
    n = sum(p.shape[0] for p in parts)
    return PackedWeight("+".join(p.name for p in parts), fmt, (n, parts[0].shape[1]),
                        np.concatenate([np.ascontiguousarray(p.payload).view(np.uint8).reshape(-1) for p in parts]))


def _interleave_rows(a: PackedWeight, b: PackedWeight) -> PackedWeight:
    d = FORMATS[a.format]
    rb = a.shape[1] // d.block_elems * d.block_bytes
    ra = np.ascontiguousarray(a.payload).view(np.uint8).reshape(a.shape[0], rb)
    rbb = np.ascontiguousarray(b.payload).view(np.uint8).reshape(b.shape[0], rb)
    return PackedWeight(a.name + "|" + b.name, a.format, (2 * a.shape[0], a.shape[1]),
                        np.stack([ra, rbb], 1).reshape(-1))


def to_device(w: PackedWeight, device, keep_packed: bool = True):
    """bf16 tensor, or a ``QuantWeight`` when the format has fused device kernels."""
    import torch
    from ..ops import cuda_ops as K
    d = FORMATS[w.format]
    if d.storage == "planar":
        if keep_packed and w.format in K.PLANAR_DEVICE_FORMATS and len(w.shape) == 2:
            ops = {k: torch.from_numpy(np.array(v)).to(device) for k, v in w.planar.items()}     # a copy: the mapped file is read-only
            return K.PlanarWeight(w.format, ops, w.shape[0], w.shape[1], w.group)
        return torch.from_numpy(w.to_f32()).to(device=device, dtype=torch.bfloat16)
    from ..runtime.upload import upload       # stored bytes go to the device through the pinned ring, as stored
    if keep_packed and d.device_gemv and len(w.shape) == 2 and w.shape[1] % 256 == 0:
        raw = upload(np.ascontiguousarray(w.payload).view(np.uint8).reshape(-1), device, torch.uint8)
        return K.QuantWeight(w.format, raw, w.shape[0], w.shape[1])
    if w.format == "BF16":
        return upload(np.ascontiguousarray(w.payload).view(np.uint16).reshape(w.shape), device, torch.bfloat16)
    return torch.from_numpy(w.to_f32()).to(device=device, dtype=torch.bfloat16)


def mtp_device_weights(handle: ModelHandle, device, target=None):
    """Device weights of the checkpoint's multi-token-prediction layer (dense bf16, canonical-name builder); with
    ``target`` given the layer uses the target's embedding and head tensors instead of copies."""
    import torch
    from ..models.config import mtp_config
    from ..runtime.weights import from_named_tensors, share_tables
    named = {n: torch.from_numpy(np.ascontiguousarray(w.to_f32())) for n, w in handle.mtp_named().items()}
    w = from_named_tensors(mtp_config(handle.cfg), named, device)
    return share_tables(w, target) if target is not None else w


def packed_experts(handle: ModelHandle, device, layers) -> dict:
    """Layer -> ``PackedExperts`` for the layers of ``layers`` whose routed experts are all stored in one row-major
    planar format (fp8 per channel or per 128 x 128 block, fp4 rows of 32): the stored operands go to the device as
    they are, stacked per projection.  Layers stored otherwise are left out (their experts are decoded to bf16)."""
    import torch
    from ..ops import cuda_ops as K
    c, canon = handle.cfg, handle.canonical
    out = {}
    if not (c.is_moe and c.gated_ffn and c.act == "silu"):
        return out
    for l in layers:
        p = f"layers.{l}."
        if not (c.has_ffn(l) and c.moe_layer(l)) or p + "experts.0.gate" not in canon:
            continue
        ws = [canon[p + f"experts.{e}.{r}"] for e in range(c.n_experts) for r in ("gate", "up", "down")]
        fmt = ws[0].format
        if fmt not in K.PACKED_EXPERT_FORMATS or any(w.format != fmt for w in ws):
            continue
        key = "weight_scale_inv" if fmt == "E4M3_BLOCK128" else "weight_scale"

        def stack(role):
            parts = [canon[p + f"experts.{e}.{role}"].planar for e in range(c.n_experts)]
            codes = np.stack([np.ascontiguousarray(q["weight"]).view(np.uint8) for q in parts])
            sc = np.stack([np.asarray(q[key]) for q in parts])
            sc = sc if fmt == "E2M1_ROW32" else sc.astype(np.float32).reshape(c.n_experts, -1) if fmt == "E4M3_CHANNEL" else sc.astype(np.float32)
            return torch.from_numpy(codes).to(device), torch.from_numpy(np.ascontiguousarray(sc)).to(device)
        bias = {}
        if c.expert_bias:
            b, F = handle.f32(p + "experts_in_bias"), c.moe_ffn
            f32dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device)
            bias = {"bias_gate": f32dev(b[:, :F]), "bias_up": f32dev(b[:, F:]), "bias_down": f32dev(handle.f32(p + "experts_out_bias"))}
        out[l] = K.PackedExperts(fmt, stack("gate"), stack("up"), stack("down"), c.n_experts, c.moe_ffn, c.hidden, **bias)
    return out


def device_weights(handle: ModelHandle, device, tp_rank: int = 0, tp_world: int = 1, keep_packed: bool = True, stage=None):
    """Rank-local ``DecoderWeights``: fused QKV, interleaved gate/up, Megatron shares."""
    import torch
    from ..runtime.weights import DecoderWeights, LayerWeights
    c, canon = handle.cfg, handle.canonical
    gaps = c.device_gaps()
    if gaps:                 # refused before any tensor is read: the loader below knows the device program's layouts only
        from ..runtime.weights import UnsupportedOnDevice
        raise UnsupportedOnDevice(f"{c.family}: the device program lacks " + "; ".join(gaps) +
                                  " (the CPU oracle evaluates this checkpoint: --backend oracle)")
    if not c.plain_block or c.router_select_bias or c.shared_width or c.first_dense_layers or c.dense_layers or c.n_group > 1 \
            or c.router != "softmax":
        # hybrid stacks and the less common layer variants go through the canonical-name builder (dense bf16)
        from ..runtime.weights import StageSpec, from_named_tensors
        st_ = stage or StageSpec.whole(c)
        packed = packed_experts(handle, device, range(st_.l0, st_.l1)) if (keep_packed and tp_world == 1) else {}
        skip = tuple(f"layers.{l}.experts." for l in packed)
        named = {n: torch.from_numpy(np.ascontiguousarray(w.to_f32())) for n, w in canon.items() if not n.startswith(skip or ("\0",))}
        return from_named_tensors(c, named, device, tp_rank, tp_world, stage=stage, packed_experts=packed)
    D = c.head_dim
    hq, hkv = c.n_heads // tp_world, max(c.n_kv_heads // tp_world, 1)
    k0 = tp_rank * hkv if c.n_kv_heads >= tp_world else tp_rank * c.n_kv_heads // tp_world
    if tp_world > 1 and any(_planar(w) for w in canon.values()):
        # planar quantised linears are cut along K for the row-parallel projections, which their group layouts do not
        # allow in general: a device group runs them decoded
        canon = {n: (_dense_f32(w) if _planar(w) else w) for n, w in canon.items()}

    def dense(name):
        return torch.from_numpy(canon[name].to_f32()).to(device=device, dtype=torch.bfloat16)

    layers = []
    from ..runtime.weights import StageSpec
    st = stage or StageSpec.whole(c)
    packed = packed_experts(handle, device, range(st.l0, st.l1)) if (keep_packed and tp_world == 1) else {}
    for l in range(st.l0, st.l1):
        p = f"layers.{l}."
        q, k, v = canon[p + "attn_q"], canon[p + "attn_k"], canon[p + "attn_v"]
        wqkv = None
        if len({q.format, k.format, v.format}) == 1 and _planar(q) and keep_packed:
            try:                # one planar weight over q | k | v rows, still packed
                from ..load.planar import planar_cat_rows
                wqkv = to_device(planar_cat_rows([q, k, v]), device, keep_packed)
            except ValueError:
                wqkv = None     # parts that do not line up with the format's groups: decoded below
        if wqkv is not None:
            pass
        elif len({q.format, k.format, v.format}) == 1 and not _planar(q):
            wqkv = to_device(_cat_rows([_rows(q, tp_rank * hq * D, hq * D), _rows(k, k0 * D, hkv * D),
                                        _rows(v, k0 * D, hkv * D)]), device, keep_packed)
        else:   # mixed formats (e.g. Q4_K_M keeps V in Q6_K): expand to bf16
            wqkv = torch.cat([torch.from_numpy(_rows(x, s, n).to_f32()) for x, s, n in
                              ((q, tp_rank * hq * D, hq * D), (k, k0 * D, hkv * D), (v, k0 * D, hkv * D))]
                             ).to(device=device, dtype=torch.bfloat16)
        o = canon[p + "attn_o"]
        n_in = o.shape[1] // tp_world
        wo = to_device(o.cols(tp_rank * n_in, n_in) if tp_world > 1 else o, device, keep_packed)
        pre = c.block in ("pre", "sandwich")
        L = LayerWeights(ln1=dense(p + "attn_norm") if pre else None, ln2=dense(p + "ffn_norm") if pre else None, wqkv=wqkv, wo=wo)
        if c.block in ("post", "sandwich"):
            L.post1, L.post2 = dense(p + "attn_post_norm"), dense(p + "ffn_post_norm")
        if c.attn_bias:
            from ..runtime.weights import fuse_qkv_bias
            L.bqkv = fuse_qkv_bias(dense(p + "attn_q_bias"), dense(p + "attn_k_bias"), dense(p + "attn_v_bias"), c,
                                   tp_rank, tp_world)
        if c.qk_norm:
            L.q_norm, L.k_norm = dense(p + "attn_q_norm"), dense(p + "attn_k_norm")
        if c.is_moe:
            L.router = dense(p + "ffn_router")
            if c.router_select_bias:
                L.select_bias = torch.from_numpy(handle.f32(p + "ffn_router_select_bias")).to(device=device, dtype=torch.float32)
            if l in packed:
                L.ex_packed = packed[l]
            else:
                gus, downs = [], []
                for e in range(c.n_experts):
                    g, u = handle.f32(p + f"experts.{e}.gate"), handle.f32(p + f"experts.{e}.up")
                    gus.append(torch.from_numpy(np.stack([g, u], 1).reshape(2 * g.shape[0], -1)))
                    downs.append(torch.from_numpy(handle.f32(p + f"experts.{e}.down")))
                L.ex_wgu = torch.stack(gus).to(device=device, dtype=torch.bfloat16)
                L.ex_wdown = torch.stack(downs).to(device=device, dtype=torch.bfloat16)
        else:
            g, u, dn = canon[p + "ffn_gate"], canon[p + "ffn_up"], canon[p + "ffn_down"]
            F = g.shape[0] // tp_world
            wgu = None
            if g.format == u.format and _planar(g) and keep_packed:
                try:            # gate and up rows interleaved inside the packed form (codes, scales, zero points move together)
                    from ..load.planar import planar_cat_rows, planar_take_rows
                    order = np.stack([np.arange(F), F + np.arange(F)], 1).reshape(-1)
                    wgu = to_device(planar_take_rows(planar_cat_rows([g, u]), order), device, keep_packed)
                except ValueError:
                    wgu = None
            if wgu is not None:
                L.wgu = wgu
            elif g.format == u.format and not _planar(g):
                L.wgu = to_device(_interleave_rows(_rows(g, tp_rank * F, F), _rows(u, tp_rank * F, F)), device, keep_packed)
            else:
                gf, uf = _rows(g, tp_rank * F, F).to_f32(), _rows(u, tp_rank * F, F).to_f32()
                L.wgu = torch.from_numpy(np.stack([gf, uf], 1).reshape(2 * F, -1)).to(device=device, dtype=torch.bfloat16)
            L.wdown = to_device(dn.cols(tp_rank * F, F) if tp_world > 1 else dn, device, keep_packed)
        layers.append(L)
    head = canon.get("lm_head")
    tied = c.tie_embeddings or head is None
    embed = to_device(canon["embed"], device, keep_packed) if (st.first or (st.last and tied)) else None
    lm_head = None
    if st.last and tied:
        lm_head = embed
    elif st.last:
        vl = head.shape[0] // tp_world
        lm_head = to_device(_rows(head, tp_rank * vl, vl) if tp_world > 1 else head, device, keep_packed)
    if not st.first:
        embed = None
    from ..runtime.weights import fold_scales
    return fold_scales(DecoderWeights(cfg=c, embed=embed, final_norm=dense("final_norm") if st.last else None,
                                      lm_head=lm_head, layers=layers, tp_rank=tp_rank, tp_world=tp_world, stage=stage))


def write_random_gguf(path: str, cfg: DecoderConfig, proj_format: str = "Q4_K", embed_format: str = "Q8_0",
                      seed: int = 0, std: float = 0.02) -> None:
    """A synthetic GGUF checkpoint of ``cfg`` quantised from random N(0, std) weights (projections in
    ``proj_format``, token embeddings in ``embed_format``, norms in F32) - the benchmark's stand-in for a download."""
    rng = np.random.default_rng(seed)
    arch = "llama"
    meta = {"general.architecture": arch, "general.name": cfg.name, f"{arch}.block_count": cfg.n_layers,
            f"{arch}.embedding_length": cfg.hidden, f"{arch}.attention.head_count": cfg.n_heads,
            f"{arch}.attention.head_count_kv": cfg.n_kv_heads, f"{arch}.feed_forward_length": cfg.ffn,
            f"{arch}.rope.freq_base": float(cfg.rope_theta), f"{arch}.attention.layer_norm_rms_epsilon": float(cfg.norm_eps),
            f"{arch}.context_length": cfg.max_position, f"{arch}.vocab_size": cfg.vocab,
            f"{arch}.attention.key_length": cfg.head_dim, "tokenizer.ggml.bos_token_id": cfg.bos_token,
            "tokenizer.ggml.eos_token_id": cfg.eos_token}
    tensors = []

    def add(name, shape, fmt, permute_heads=0):
        w = (rng.standard_normal(shape) * std).astype(np.float32)
        if permute_heads:
            w = w[names.hf_to_gguf_qk_row_order(shape[0], permute_heads)]
        if fmt == "F32":
            tensors.append(PackedWeight(name, "F32", shape, w.view(np.uint8).reshape(-1)))
        else:
            tensors.append(PackedWeight(name, fmt, shape, codec.quantize(fmt, w)))

    H = cfg.hidden
    add("token_embd.weight", (cfg.vocab, H), embed_format)
    for l in range(cfg.n_layers):
        b = f"blk.{l}."
        tensors.append(PackedWeight(b + "attn_norm.weight", "F32", (H,), np.ones(H, np.float32).view(np.uint8)))
        tensors.append(PackedWeight(b + "ffn_norm.weight", "F32", (H,), np.ones(H, np.float32).view(np.uint8)))
        add(b + "attn_q.weight", (cfg.q_size, H), proj_format, cfg.n_heads)
        add(b + "attn_k.weight", (cfg.kv_size, H), proj_format, cfg.n_kv_heads)
        add(b + "attn_v.weight", (cfg.kv_size, H), proj_format)
        add(b + "attn_output.weight", (H, cfg.q_size), proj_format)
        add(b + "ffn_gate.weight", (cfg.ffn, H), proj_format)
        add(b + "ffn_up.weight", (cfg.ffn, H), proj_format)
        add(b + "ffn_down.weight", (H, cfg.ffn), proj_format)
    tensors.append(PackedWeight("output_norm.weight", "F32", (H,), np.ones(H, np.float32).view(np.uint8)))
    add("output.weight", (cfg.vocab, H), proj_format)
    gguf.write_gguf(path, meta, tensors)


def prove_step_ranges(cfg: DecoderConfig, prefill_chunk: int = 64) -> None:
    """Trace the decode and prefill step graphs and prove every index (token ids, positions, slot maps, expert ids)
    inside its extent; raises ``ValueError`` naming the first unproven use."""
    from ..ir.analysis import index_guards
    from ..models.model import Model, StepSpec
    for tokens in (1, min(prefill_chunk, 64)):
        g = Model(cfg).trace(StepSpec(rows=1, tokens=tokens, capacity=64))
        bad = [x for x in index_guards(g) if not x.proven]
        if bad:
            raise ValueError(f"{len(bad)} index uses are not proven in range, first: {bad[0]}")
