"""GGUF reader and writer.

Layout (crates/poot-load/src/gguf.rs:1-9): magic ``GGUF``, version, tensor count, KV count, the KV metadata, the
tensor directory (name, dims in ggml order = innermost first, ggml type, offset), padding to
``general.alignment`` (32), then the tensor data.  Payloads are returned as zero-copy views of a memory map; split
shards (``-00001-of-0000N``) are merged; ggml types that exist but cannot be decoded are refused by name
(crates/poot-load/src/gguf/format.rs:476-560).  A quantised rank-3 expert tensor becomes one packed owner per
expert (gguf.rs:79-88).
"""
from __future__ import annotations

import mmap
import os
import re
import struct
from dataclasses import dataclass
from typing import Any, BinaryIO, Dict, List, Optional, Tuple

import numpy as np

from ..models.config import DecoderConfig, RopeScaling
from ..quant.formats import FORMATS, GGML_REFUSED, GGML_TYPE_TO_FORMAT, UnsupportedFormat, packed_nbytes
from ..quant.weights import PackedWeight, WeightStore

MAGIC = 0x46554747
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
MAX_STRING = 1 << 28
MAX_ARRAY = 1 << 28


class GgufError(ValueError):
    pass


@dataclass
class GgufTensorInfo:
    name: str
    shape: Tuple[int, ...]      # logical (outermost first)
    ggml_type: int
    offset: int


class _Reader:
    def __init__(self, buf, size):
        self.b, self.p, self.n = buf, 0, size

    def take(self, fmt: str):
        sz = struct.calcsize(fmt)
        if self.p + sz > self.n:
            raise GgufError("truncated GGUF header")
        v = struct.unpack_from(fmt, self.b, self.p)[0]
        self.p += sz
        return v

    def string(self) -> str:
        n = self.take("<Q")
        if n > MAX_STRING or self.p + n > self.n:
            raise GgufError(f"string of {n} bytes overruns the file")
        s = bytes(self.b[self.p:self.p + n]).decode("utf-8", errors="replace")
        self.p += n
        return s

    def value(self, t: int, depth: int = 0):
        if t in _SCALAR:
            return self.take(_SCALAR[t])
        if t == 8:
            return self.string()
        if t == 9:
            if depth > 2:
                raise GgufError("array nesting too deep")
            et, cnt = self.take("<I"), self.take("<Q")
            if cnt > MAX_ARRAY:
                raise GgufError(f"array of {cnt} elements")
            if et in _SCALAR:
                fmt = _SCALAR[et]
                sz = struct.calcsize(fmt)
                if self.p + sz * cnt > self.n:
                    raise GgufError("array overruns the file")
                arr = np.frombuffer(self.b, dtype=np.dtype(fmt[1:]).newbyteorder("<"), count=cnt, offset=self.p)
                self.p += sz * cnt
                return arr.tolist() if cnt <= 4096 else arr
            return [self.value(et, depth + 1) for _ in range(cnt)]
        raise GgufError(f"unknown metadata value type {t}")


@dataclass
class GgufIndex:
    path: str
    version: int
    metadata: Dict[str, Any]
    tensors: List[GgufTensorInfo]
    data_start: int
    alignment: int


def read_index(path: str) -> Tuple[GgufIndex, mmap.mmap]:
    f = open(path, "rb")
    size = os.fstat(f.fileno()).st_size
    if size < 24:
        raise GgufError("file too small for a GGUF header")
    mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    r = _Reader(mm, size)
    if r.take("<I") != MAGIC:
        raise GgufError("not a GGUF file (bad magic)")
    version = r.take("<I")
    if version not in (2, 3):
        raise GgufError(f"unsupported GGUF version {version}")
    n_tensors, n_kv = r.take("<Q"), r.take("<Q")
    if n_tensors > 1 << 20 or n_kv > 1 << 20:
        raise GgufError("implausible tensor / metadata count")
    meta: Dict[str, Any] = {}
    for _ in range(n_kv):
        key = r.string()
        if key in meta:
            raise GgufError(f"duplicate metadata key {key!r}")
        meta[key] = r.value(r.take("<I"))
    infos = []
    seen = set()
    for _ in range(n_tensors):
        name = r.string()
        if name in seen:
            raise GgufError(f"duplicate tensor {name!r}")
        seen.add(name)
        nd = r.take("<I")
        if nd > 4:
            raise GgufError(f"tensor {name!r} has {nd} dimensions")
        dims = [r.take("<Q") for _ in range(nd)]
        infos.append(GgufTensorInfo(name, tuple(reversed(dims)), r.take("<I"), r.take("<Q")))
    align = int(meta.get("general.alignment", 32))
    if align <= 0 or align & (align - 1):
        raise GgufError(f"alignment {align} is not a power of two")
    data_start = (r.p + align - 1) // align * align
    return GgufIndex(path, version, meta, infos, data_start, align), mm


def _format_of(info: GgufTensorInfo) -> str:
    if info.ggml_type in GGML_REFUSED:
        raise UnsupportedFormat(f"tensor {info.name!r}: ggml type {GGML_REFUSED[info.ggml_type]} is not supported")
    try:
        return GGML_TYPE_TO_FORMAT[info.ggml_type]
    except KeyError:
        raise UnsupportedFormat(f"tensor {info.name!r}: unknown ggml type {info.ggml_type}") from None


def shard_paths(path: str) -> List[str]:
    m = re.search(r"-(\d{5})-of-(\d{5})\.gguf$", path)
    if not m:
        return [path]
    total = int(m.group(2))
    return [path[:m.start()] + f"-{i:05d}-of-{total:05d}.gguf" for i in range(1, total + 1)]


def read_gguf(path: str, check: bool = True) -> WeightStore:
    store = WeightStore()
    store.source = path
    store._maps = []
    for k, sp in enumerate(shard_paths(path)):
        idx, mm = read_index(sp)
        store._maps.append(mm)
        if k == 0:
            store.metadata = idx.metadata
        raw = np.frombuffer(mm, dtype=np.uint8)
        for t in idx.tensors:
            fmt = _format_of(t)
            n = int(np.prod(t.shape)) if t.shape else 1
            nbytes = packed_nbytes(fmt, n)
            lo = idx.data_start + t.offset
            if t.offset % idx.alignment or lo + nbytes > raw.size:
                raise GgufError(f"tensor {t.name!r} overruns the file or is misaligned")
            payload = raw[lo:lo + nbytes]
            if len(t.shape) == 3 and (FORMATS[fmt].storage == "blocks" or t.name.endswith("_exps.weight")):
                # a stacked expert tensor becomes one owner per expert, in any storage format
                per = nbytes // t.shape[0]
                for e in range(t.shape[0]):
                    store.add(PackedWeight(f"{t.name}#{e}", fmt, tuple(t.shape[1:]), payload[e * per:(e + 1) * per]))
            else:
                store.add(PackedWeight(t.name, fmt, tuple(t.shape), payload))
    return store.publish(check)


# ---- writer -----------------------------------------------------------------------------------------------------
def _put_string(out: bytearray, s: str) -> None:
    b = s.encode("utf-8")
    out += struct.pack("<Q", len(b)) + b


def _put_value(out: bytearray, v) -> None:
    if isinstance(v, bool):
        out += struct.pack("<I?", 7, v)
    elif isinstance(v, int):
        out += struct.pack("<Iq", 11, v) if v < 0 or v > 0xFFFFFFFF else struct.pack("<II", 4, v)
    elif isinstance(v, float):
        out += struct.pack("<If", 6, v)
    elif isinstance(v, str):
        out += struct.pack("<I", 8)
        _put_string(out, v)
    elif isinstance(v, (list, tuple, np.ndarray)):
        v = list(v)
        out += struct.pack("<I", 9)
        if v and isinstance(v[0], str):
            out += struct.pack("<IQ", 8, len(v))
            for s in v:
                _put_string(out, s)
        elif v and isinstance(v[0], (bool, np.bool_)):
            out += struct.pack("<IQ", 7, len(v)) + struct.pack(f"<{len(v)}?", *[bool(x) for x in v])
        elif v and isinstance(v[0], float):
            out += struct.pack("<IQ", 6, len(v)) + struct.pack(f"<{len(v)}f", *v)
        else:
            out += struct.pack("<IQ", 5, len(v)) + struct.pack(f"<{len(v)}i", *[int(x) for x in v])
    else:
        raise GgufError(f"cannot encode metadata value of type {type(v)}")


def write_gguf(path: str, metadata: Dict[str, Any], tensors: List[PackedWeight], alignment: int = 32) -> None:
    head = bytearray(struct.pack("<IIQQ", MAGIC, 3, len(tensors), len(metadata)))
    for k, v in metadata.items():
        _put_string(head, k)
        _put_value(head, v)
    offsets, off = [], 0
    for t in tensors:
        offsets.append(off)
        off = (off + t.payload.nbytes + alignment - 1) // alignment * alignment
    for t, o in zip(tensors, offsets):
        _put_string(head, t.name)
        dims = list(reversed(t.shape))
        head += struct.pack("<I", len(dims)) + struct.pack(f"<{len(dims)}Q", *dims)
        head += struct.pack("<IQ", FORMATS[t.format].ggml_type, o)
    pad = (-len(head)) % alignment
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        for t in tensors:
            raw = np.ascontiguousarray(t.payload).view(np.uint8).reshape(-1)
            f.write(raw.tobytes())
            f.write(b"\0" * ((-raw.nbytes) % alignment))


# ---- metadata -> configuration ---------------------------------------------------------------------------------
def hf_header_from_gguf(arch: str, meta: Dict[str, Any], family: str) -> Dict[str, Any]:
    """The Hugging Face style header a family's table reads, rebuilt from a GGUF's metadata keys (``<arch>.block_count``,
    ``.embedding_length``, ... as llama.cpp's converter writes them), so one header table per family serves both
    containers.  What a GGUF does not state takes the value llama.cpp's graph uses: Gemma's query scale is the head
    width, gpt-oss slides on every even layer, SmolLM3 leaves every fourth layer without rotary positions."""
    def g(key, default=None):
        return meta.get(f"{arch}.{key}", default)

    def one(v):
        return v[0] if isinstance(v, (list, np.ndarray)) else v

    H, nh = int(g("embedding_length")), int(g("attention.head_count"))
    L = int(g("block_count"))
    tokens = meta.get("tokenizer.ggml.tokens")
    vocab = int(g("vocab_size", len(tokens) if tokens is not None else 0))
    ids = {"bos_token_id": meta.get("tokenizer.ggml.bos_token_id"), "eos_token_id": meta.get("tokenizer.ggml.eos_token_id")}
    if family == "mpt":                                  # the LayerNorm families keep their own header spelling
        return {"d_model": H, "n_heads": nh, "n_layers": L, "vocab_size": vocab, "max_seq_len": int(g("context_length", 2048)),
                "layer_norm_epsilon": float(g("attention.layer_norm_epsilon", 1e-5)), "expansion_ratio": int(one(g("feed_forward_length", 4 * H))) / H,
                "no_bias": True, "attn_config": {"alibi": float(g("attention.max_alibi_bias", 8.0)) > 0.0, "alibi_bias_max": float(g("attention.max_alibi_bias", 8.0)),
                                                 "clip_qkv": g("attention.clamp_kqv")}, **ids}
    if family == "gemma4":
        # per-layer facts come as arrays: which layers slide, and the K/V head count of each (local and global layers differ);
        # ``tensors.*`` are facts read off the tensor list by the loader (a GGUF header does not state them)
        local = [bool(x) for x in g("attention.sliding_window_pattern")]
        kv = [int(x) for x in np.atleast_1d(g("attention.head_count_kv"))]
        kv = kv * L if len(kv) == 1 else kv
        kv_local = [n for n, loc in zip(kv, local) if loc] or kv
        kv_global = [n for n, loc in zip(kv, local) if not loc]
        experts = int(g("expert_count", 0) or 0)
        return {"hidden_size": H, "num_hidden_layers": L, "num_attention_heads": nh, "num_key_value_heads": kv_local[0],
                "num_global_key_value_heads": kv_global[0] if kv_global else 0, "head_dim": int(g("attention.key_length_swa", g("attention.key_length"))),
                "global_head_dim": int(g("attention.key_length")), "intermediate_size": int(one(g("feed_forward_length"))), "vocab_size": vocab,
                "rms_norm_eps": float(g("attention.layer_norm_rms_epsilon", 1e-6)), "max_position_embeddings": int(g("context_length", 131072)),
                "layer_types": ["sliding_attention" if loc else "full_attention" for loc in local], "sliding_window": int(g("attention.sliding_window", 0) or 0),
                "rope_parameters": {"full_attention": {"rope_type": "proportional", "rope_theta": float(g("rope.freq_base", 1e6)),
                                                       "partial_rotary_factor": float(meta.get("tensors.rope_proportion", 1.0))},
                                    "sliding_attention": {"rope_type": "default", "rope_theta": float(g("rope.freq_base_swa", 10000.0))}},
                "final_logit_softcapping": g("final_logit_softcapping"), "attention_k_eq_v": bool(meta.get("tensors.value_is_key", False)),
                "tie_word_embeddings": not meta.get("tensors.has_output", False), "enable_moe_block": experts > 0, "num_experts": experts,
                "top_k_experts": int(g("expert_used_count", 0) or 0), "moe_intermediate_size": int(g("expert_feed_forward_length", 0) or 0), **ids}
    if family == "bloom":
        return {"hidden_size": H, "n_head": nh, "n_layer": L, "vocab_size": vocab, "seq_length": int(g("context_length", 2048)),
                "layer_norm_epsilon": float(g("attention.layer_norm_epsilon", 1e-5)), **ids}
    h: Dict[str, Any] = {
        "hidden_size": H, "num_hidden_layers": L, "num_attention_heads": nh,
        "num_key_value_heads": int(one(g("attention.head_count_kv", nh))), "head_dim": int(g("attention.key_length", H // nh)),
        "intermediate_size": int(one(g("feed_forward_length", 4 * H))),
        "vocab_size": int(g("vocab_size", len(tokens) if tokens is not None else 0)),
        "rms_norm_eps": float(g("attention.layer_norm_rms_epsilon", 1e-6)), "rope_theta": float(g("rope.freq_base", 10000.0)),
        "max_position_embeddings": int(g("context_length", 8192)), "tie_word_embeddings": False,
        "bos_token_id": int(meta.get("tokenizer.ggml.bos_token_id", 1)), "eos_token_id": int(meta.get("tokenizer.ggml.eos_token_id", 2))}
    if g("rope.scaling.type") in ("linear", "yarn"):
        h["rope_scaling"] = {"rope_type": g("rope.scaling.type"), "factor": float(g("rope.scaling.factor", 1.0)),
                             "original_max_position_embeddings": int(g("rope.scaling.original_context_length", 8192))}
    if g("expert_count"):
        h["num_local_experts"], h["num_experts_per_tok"] = int(g("expert_count")), int(g("expert_used_count", 0))
        if g("expert_feed_forward_length"):
            h["intermediate_size"] = int(g("expert_feed_forward_length"))
    win = g("attention.sliding_window")
    if family in ("gemma2", "gemma3"):
        h.update({"sliding_window": int(win) if win else h["max_position_embeddings"], "query_pre_attn_scalar": h["head_dim"],
                  "attn_logit_softcapping": g("attn_logit_softcapping"), "final_logit_softcapping": g("final_logit_softcapping"),
                  "rope_local_base_freq": float(g("rope.freq_base_swa", 10000.0))})
    elif family == "gpt_oss":
        h.update({"sliding_window": int(win or 128), "attention_bias": True,
                  "layer_types": ["sliding_attention" if l % 2 == 0 else "full_attention" for l in range(L)]})
    elif family == "granite":
        h.update({"embedding_multiplier": float(g("embedding_scale", 1.0)), "residual_multiplier": float(g("residual_scale", 1.0)),
                  "logits_scaling": float(g("logit_scale", 1.0)), "attention_multiplier": g("attention.scale")})
    elif family == "smollm3":
        h["no_rope_layers"] = [int((l + 1) % 4 != 0) for l in range(L)]
    elif family == "qwen38_27b":
        # the multi-token-prediction blocks a converter appends count in ``block_count`` and are not part of the stack
        nextn = int(g("nextn_predict_layers", 0) or 0)
        if nextn >= L:
            raise ValueError(f"{arch}.nextn_predict_layers {nextn} leaves no block of {L} for the stack")
        rot = int(g("rope.dimension_count", h["head_dim"]))
        h.update({"num_hidden_layers": L - nextn, "linear_num_key_heads": int(g("ssm.group_count")), "linear_num_value_heads": int(g("ssm.time_step_rank")),
                  "linear_key_head_dim": int(g("ssm.state_size")), "linear_value_head_dim": int(g("ssm.state_size")),
                  "linear_conv_kernel_dim": int(g("ssm.conv_kernel", 4)), "full_attention_interval": int(g("full_attention_interval", 4)),
                  "partial_rotary_factor": rot / h["head_dim"]})
        if int(g("ssm.inner_size", h["linear_num_value_heads"] * h["linear_key_head_dim"])) != h["linear_num_value_heads"] * h["linear_key_head_dim"]:
            raise ValueError(f"{arch}.ssm.inner_size is not value heads x head width")
    elif family == "minimax_m2":
        rot = int(g("rope.dimension_count", h["head_dim"]))
        if rot != h["head_dim"]:
            h["partial_rotary_factor"] = rot / h["head_dim"]
        if int(g("expert_gating_func", 2)) != 2:
            raise ValueError(f"{arch}.expert_gating_func {g('expert_gating_func')}: this family's router is the sigmoid one (2)")
    elif family == "deepseek2":
        # converters that store the absorbed form describe the one shared latent head in ``key_length`` / ``value_length``
        # and the per-head widths in the ``_mla`` keys; older files have the per-head widths in the plain keys
        rope = int(g("rope.dimension_count"))
        key = int(g("attention.key_length_mla", g("attention.key_length")))
        if int(g("expert_gating_func", 1)) != 1:
            raise ValueError(f"{arch}.expert_gating_func {g('expert_gating_func')}: DeepSeek-V2 routes by softmax (1)")
        h.update({"q_lora_rank": int(g("attention.q_lora_rank", 0) or 0) or None, "kv_lora_rank": int(g("attention.kv_lora_rank")),
                  "qk_rope_head_dim": rope, "qk_nope_head_dim": key - rope, "head_dim": key,
                  "v_head_dim": int(g("attention.value_length_mla", g("attention.value_length"))), "num_key_value_heads": nh,
                  "n_routed_experts": int(g("expert_count", 0) or 0), "num_experts_per_tok": int(g("expert_used_count", 0) or 0),
                  "moe_intermediate_size": int(g("expert_feed_forward_length", 0) or 0), "n_shared_experts": int(g("expert_shared_count", 0) or 0),
                  "first_k_dense_replace": int(g("leading_dense_block_count", 0) or 0), "routed_scaling_factor": float(g("expert_weights_scale", 1.0)),
                  "norm_topk_prob": bool(g("expert_weights_norm", False)), "topk_method": "greedy"})
        h.pop("num_local_experts", None)
        h["intermediate_size"] = int(one(g("feed_forward_length", 4 * H)))
    return h


def config_from_gguf_metadata(arch: str, meta: Dict[str, Any], family: str) -> DecoderConfig:
    def g(key, default=None):
        return meta.get(f"{arch}.{key}", default)

    H, nh = int(g("embedding_length")), int(g("attention.head_count"))
    nkv = g("attention.head_count_kv", nh)
    nkv = int(nkv[0] if isinstance(nkv, (list, np.ndarray)) else nkv)
    head_dim = int(g("attention.key_length", H // nh))
    tokens = meta.get("tokenizer.ggml.tokens")
    vocab = int(g("vocab_size", len(tokens) if tokens is not None else 0))
    n_exp = int(g("expert_count", 0) or 0)
    ffn = g("feed_forward_length", 4 * H)
    ffn = int(ffn[0] if isinstance(ffn, (list, np.ndarray)) else ffn)
    scaling = RopeScaling()
    if g("rope.scaling.type") in ("linear", "yarn"):
        scaling = RopeScaling(kind=g("rope.scaling.type"), factor=float(g("rope.scaling.factor", 1.0)),
                              original_max_position=int(g("rope.scaling.original_context_length", 8192)))
    return DecoderConfig(
        name=str(meta.get("general.name", family)), family="mixtral" if (family == "llama" and n_exp) else family,
        n_layers=int(g("block_count")), hidden=H, n_heads=nh, n_kv_heads=nkv, head_dim=head_dim, ffn=ffn, vocab=vocab,
        norm_eps=float(g("attention.layer_norm_rms_epsilon", 1e-6)), rope_theta=float(g("rope.freq_base", 10000.0)),
        rope_dim=int(g("rope.dimension_count", head_dim)) if int(g("rope.dimension_count", head_dim)) != head_dim else None,
        rope_scaling=scaling, max_position=int(g("context_length", 8192)),
        tie_embeddings=False, qk_norm=family in ("qwen3", "qwen3moe", "olmo2", "olmoe"), attn_bias=family == "qwen2",
        n_experts=n_exp, top_k=int(g("expert_used_count", 0) or 0), moe_ffn=int(g("expert_feed_forward_length", ffn)) if n_exp else 0,
        bos_token=int(meta.get("tokenizer.ggml.bos_token_id", 1)), eos_token=int(meta.get("tokenizer.ggml.eos_token_id", 2)))
