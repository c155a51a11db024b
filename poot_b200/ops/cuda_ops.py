"""PyTorch-facing wrappers over the hand-written sm_100a kernels.

Every wrapper validates shapes and dtypes, allocates its output with torch when the caller passes none,
and launches on the current CUDA stream, so all of them can be captured into a CUDA graph.  There is no
PyTorch fallback: a tensor that is not on a CUDA device is an error.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from ._lib import check, kernels

EPI_STORE, EPI_F32, EPI_RESID, EPI_SWIGLU, EPI_PARTIAL = 0, 1, 2, 3, 4
KV_BLOCK = 16

_P = c_void_p
_SIGS = {
    "poot_embed_gather": [_P, _P, _P, c_int, c_int, c_int, _P],
    "poot_rmsnorm": [_P, _P, _P, c_int, c_longlong, _P, _P, c_int, c_int, c_float, _P],
    "poot_swiglu": [_P, _P, c_int, c_int, c_int, _P],
    "poot_gated_act": [_P, _P, c_int, c_int, c_int, c_int, c_float, c_float, _P],
    "poot_softcap_f32": [_P, c_longlong, c_float, _P],
    "poot_layernorm": [_P, _P, _P, c_float, _P, c_int, c_int, _P],
    "poot_act_bf16": [_P, c_longlong, c_int, _P],
    "poot_replace_rows": [_P, _P, _P, c_int, c_int, _P],
    "poot_causal_conv_silu": [_P, c_int, c_int, c_int, c_int, _P, _P, _P, c_int, _P, c_int, _P, _P],
    "poot_ssd_scan": [_P, _P, c_int, c_int, _P, _P, _P, _P, c_int, _P, c_int, _P, c_int, c_int, c_int, c_int, _P],
    "poot_gdn_scan": [_P, _P, c_int, c_int, c_int, _P, _P, _P, c_int, _P, c_int, _P, c_int, c_int, c_int, _P],
    "poot_ngram_hash": [_P, _P, c_int, _P, c_int, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P, _P],
    "poot_kda_scan": [_P, _P, _P, c_int, c_int, _P, _P, c_float, _P, c_int, _P, c_int, _P, c_int, c_int, _P],
    "poot_gated_rmsnorm": [_P, _P, c_int, c_int, _P, c_int, c_float, c_int, _P, c_int, c_int, c_int, _P],
    "poot_sigmoid_mul": [_P, _P, c_longlong, _P],
    "poot_add_bf16": [_P, _P, _P, c_longlong, _P],
    "poot_bias_add": [_P, _P, c_int, c_int, c_int, c_int, c_int, _P],
    "poot_bias_add_indexed": [_P, _P, _P, c_int, c_int, c_int, _P, c_int, c_int, _P],
    "poot_scale_bf16": [_P, c_longlong, c_float, _P],
    "poot_gather_rows": [_P, c_longlong, c_int, _P, _P, c_longlong, c_int, c_int, _P],
    "poot_sigmoid_gate_rows": [_P, _P, c_int, c_int, c_int, _P],
    "poot_reduce_partials": [_P, _P, c_int, c_longlong, _P, c_longlong, _P],
    "poot_cast_f32_bf16": [_P, _P, c_longlong, _P],
    "poot_cast_bf16_f32": [_P, _P, c_longlong, _P],
    "poot_gemv_bf16": [c_int, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P],
    "poot_gemm_bf16_tcgen05": [c_int, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_longlong,
                               _P, _P],
    "poot_gemm_skinny": [c_int, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P],
    "poot_rope_kv_write": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_float, c_int, c_int, c_int, c_int, c_int, c_int,
                           c_int, _P],
    "poot_attn_paged": [_P, c_int, _P, _P, _P, c_int, _P, _P, _P, c_int, _P, _P, c_int, c_int, c_int, c_int, c_float,
                        c_float, c_int, c_int, _P],
    "poot_mla_qkv_write": [_P, _P, _P, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P],
    "poot_attn_general": [_P, c_int, _P, _P, c_int, _P, c_int, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                          c_float, c_int, _P, _P, _P, c_int, _P],
    "poot_index_k_write": [_P, _P, _P, c_float, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P],
    "poot_index_q_rope": [_P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P],
    "poot_index_scores": [_P, _P, c_int, _P, _P, c_int, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_float, _P],
    "poot_index_select": [_P, c_int, _P, _P, c_int, c_int, _P],
    "poot_attn_flash_prefill": [_P, c_int, c_int, _P, _P, c_longlong, _P, c_int, _P, c_int, _P, c_int, c_int, c_int,
                                c_float, c_int, _P, _P],
    "poot_decode_advance": [_P, _P, _P, _P, _P, _P, c_int, _P, c_int, _P],
    "poot_argmax": [_P, c_int, c_int, c_int, _P, _P, _P],
    "poot_argmax_partials": [_P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P],
    "poot_argmax_combine": [_P, c_int, c_longlong, c_int, c_int, c_int, _P, _P],
    "poot_sample_gumbel": [_P, c_int, c_int, _P, _P, _P, c_int, _P, _P],
    "poot_random_uniform": [_P, c_int, c_int, _P, _P],
}
_bound = {}


_timing_sink = None   # when a list: every launch is bracketed by CUDA events and appended as (name, e0, e1)
launch_total = 0      # launchers called since import (cheap always-on counter)


def _fn(name: str):
    f = _bound.get(name)
    if f is None:
        raw = getattr(kernels(), name)
        raw.argtypes = _SIGS[name]
        raw.restype = c_int

        def f(*args, _raw=raw, _name=name):
            global launch_total
            launch_total += 1
            if _timing_sink is None:
                return _raw(*args)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = _raw(*args)
            e1.record()
            _timing_sink.append((_name, e0, e1))
            return r

        _bound[name] = f
    return f


def start_device_timing() -> None:
    """Opt-in detailed device timing: bracket every launch with CUDA events (eager launches only)."""
    global _timing_sink
    _timing_sink = []


def timed_region(name: str):
    """Context manager that times a non-library region (e.g. an NCCL collective) into the same sink."""
    class _R:
        def __enter__(self_inner):
            if _timing_sink is not None:
                self_inner.e0 = torch.cuda.Event(enable_timing=True)
                self_inner.e0.record()
            return self_inner

        def __exit__(self_inner, *exc):
            if _timing_sink is not None:
                e1 = torch.cuda.Event(enable_timing=True)
                e1.record()
                _timing_sink.append((name, self_inner.e0, e1))
            return False
    return _R()


def stop_device_timing():
    """Stop timing; returns ``{launcher name: (count, total microseconds)}`` (synchronises the device)."""
    global _timing_sink
    sink, _timing_sink = _timing_sink, None
    torch.cuda.synchronize()
    out = {}
    for name, e0, e1 in sink or []:
        c, t = out.get(name, (0, 0.0))
        out[name] = (c + 1, t + e0.elapsed_time(e1) * 1e3)
    return out


def register_signature(name: str, argtypes) -> None:
    """Let other op modules of the package declare launchers that live in the same library."""
    _SIGS[name] = argtypes


def fn(name: str):
    return _fn(name)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("poot_b200.ops: tensor must live on a CUDA device (no CPU fallback)")


_status = {}
_abort = {}            # device -> (host pointer of the mapped abort word, device-visible address)
CTL_WORDS = 16         # control block: [0] first failure, [1] detail, [2:4] deadline ns, [4:6] abort-word address,
                       # [6:8] step budget ns, [8] waits given up (csrc/kernels/common.cuh)
DEFAULT_STEP_BUDGET_S = 5.0

STATUS_NAMES = {1: "TMA producer", 2: "MMA issuer", 3: "epilogue", 4: "peer flag", 5: "bad argument",
                6: "host abort", 7: "step deadline", 8: "peer failed"}


def _canon(device=None) -> torch.device:
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.index is None:       # "cuda" and "cuda:N" must name the same block
        dev = torch.device("cuda", torch.cuda.current_device())
    return dev


def status_word(device=None) -> torch.Tensor:
    """Per-device control block (``CTL_WORDS`` int32 words) that every launcher receives as its ``status`` pointer.

    Word 0 is the first failure of a bounded wait since the block was last cleared; the block also carries the
    step deadline, the step budget and the address of a host-mapped abort word (see ``request_abort``)."""
    dev = _canon(device)
    s = _status.get(dev)
    if s is None:
        s = torch.zeros(CTL_WORDS, dtype=torch.int32, device=dev)
        _status[dev] = s
        lib = kernels()
        lib.poot_abort_word_alloc.argtypes = [ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p)]
        lib.poot_abort_word_set.argtypes = [c_void_p, c_int]
        lib.poot_abort_word_set.restype = None
        hp, dp = c_void_p(), c_void_p()
        with torch.cuda.device(dev):
            check(lib.poot_abort_word_alloc(ctypes.byref(hp), ctypes.byref(dp)), "abort_word_alloc")
        _abort[dev] = (hp.value, dp.value)
        s[4:6].copy_(torch.tensor([dp.value], dtype=torch.int64).view(torch.int32))
        set_step_budget(DEFAULT_STEP_BUDGET_S, dev)
    return s


def set_step_budget(seconds: float, device=None) -> None:
    """Budget shared by all cross-rank waits of one tensor-parallel step (0 = no deadline: each wait has its own
    limit of about a second)."""
    s = _status.get(_canon(device))
    if s is None:
        s = status_word(device)
    ns = int(max(0.0, seconds) * 1e9)
    s[6:8].copy_(torch.tensor([ns], dtype=torch.int64).view(torch.int32))
    s[2:4].zero_()      # a deadline left by an earlier step must not end the waits of a program that sets none


def request_abort(device=None) -> None:
    """Host side of the abort word: every pending and future cross-rank wait on the device gives up at once, so
    queued kernels run to their end and ``torch.cuda.synchronize`` returns.  Plain host store (async-signal-safe
    once the block exists); it works while kernels are running.  Call ``clear_abort`` before using the device again."""
    devs = [_canon(device)] if device is not None else list(_abort)
    for d in devs:
        if d in _abort:
            kernels().poot_abort_word_set(_abort[d][0], 1)


def clear_abort(device=None) -> None:
    devs = [_canon(device)] if device is not None else list(_abort)
    for d in devs:
        if d in _abort:
            kernels().poot_abort_word_set(_abort[d][0], 0)


class DeviceWaitTimeout(RuntimeError):
    """A bounded device-side wait ran out; the kernel returned early and its output is invalid."""

    def __init__(self, message: str, code: int = 0, detail: int = -1):
        super().__init__(message)
        self.code, self.detail = code, detail


def read_status(device=None):
    """``(code, detail, waits_given_up)`` of the control block (synchronises the device)."""
    words = status_word(device)[:9].tolist()
    return words[0], words[1], words[8]


def describe_status(code: int, detail: int) -> str:
    what = STATUS_NAMES.get(code, str(code))
    if code in (4, 7, 8) and detail >= 0:
        if detail >= (1 << 20):
            return f"{what} (greedy-pick exchange, waiting for rank {detail - (1 << 20)})"
        return f"{what} (site {detail // 16}, waiting for rank {detail % 16})"
    return what


def check_status(device=None) -> None:
    """Raise ``DeviceWaitTimeout`` if a wait gave up since the last check; the failure words are cleared."""
    code, detail, gave_up = read_status(device)
    if code != 0:
        s = status_word(device)
        s[0:2].zero_()
        s[8:9].zero_()
        raise DeviceWaitTimeout(f"device wait timed out in {describe_status(code, detail)}"
                                f" ({gave_up} wait(s) gave up)", code, detail)


# ---- checked build ------------------------------------------------------------------------------------------------
BOUNDS_SITES = {1: "token id", 2: "K/V slot", 3: "K/V block id", 4: "position", 5: "expert id", 6: "row map",
                7: "logit index", 8: "sequence row", 9: "recurrent-state row", 10: "gathered row"}
BOUNDS_LIMITS = {"pool_slots": 0, "pool_blocks": 1, "state_rows": 2}


class DeviceIndexOutOfRange(RuntimeError):
    """The checked kernel library saw a data-dependent index outside its bound (the kernel substituted a safe index
    and carried on; the step's results are not to be used)."""

    def __init__(self, site: int, line: int, index: int, bound: int):
        super().__init__(f"device index out of range: {BOUNDS_SITES.get(site, f'site {site}')} {index} outside "
                         f"[0, {bound}) (kernel source line {line})")
        self.site, self.line, self.index, self.bound = site, line, index, bound


def _dbg(name: str, argtypes):
    f = getattr(kernels(), name)            # host-only entry points: not launches, so not counted as such
    f.argtypes, f.restype = argtypes, c_int
    return f


def bounds_checking() -> bool:
    """True when the loaded kernel library is the checked flavour (``POOT_DEBUG_BOUNDS=1`` at import)."""
    return bool(_dbg("poot_debug_bounds_enabled", [])())


def set_bounds_limits(**limits: int) -> None:
    """Bounds the kernels are not given as arguments: ``pool_slots``, ``pool_blocks``, ``state_rows``."""
    for name, v in limits.items():
        check(_dbg("poot_debug_bounds_limit", [c_int, c_longlong])(BOUNDS_LIMITS[name], int(v)), "debug_bounds_limit")


def check_bounds() -> None:
    """Raise ``DeviceIndexOutOfRange`` for the first recorded fault (and clear the record).  Synchronises the device;
    a no-op on the release library."""
    if not bounds_checking():
        return
    out = (c_int * 4)()
    check(_dbg("poot_debug_bounds_read", [_P])(out), "debug_bounds_read")
    if out[0] != 0:
        check(_dbg("poot_debug_bounds_clear", [])(), "debug_bounds_clear")
        raise DeviceIndexOutOfRange(out[0], out[1], out[2], out[3])


# ----------------------------------------------------------------------------------------------------------------
def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need_cuda(ids, table)
    assert ids.dtype == torch.int32 and table.dtype == torch.bfloat16 and table.is_contiguous()
    T, (V, D) = ids.numel(), table.shape
    if out is None:
        out = torch.empty(T, D, dtype=torch.bfloat16, device=table.device)
    check(_fn("poot_embed_gather")(_ptr(ids), _ptr(table), _ptr(out), T, D, V, _stream()), "embed_gather")
    return out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None,
            partials: Optional[torch.Tensor] = None, h_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y = rmsnorm(x + sum(partials)) * w``; the updated residual stream goes to ``h_out`` (may be ``x``)."""
    _need_cuda(x, w)
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and w.dtype == torch.bfloat16
    T, D = x.shape
    if out is None:
        out = torch.empty_like(x)
    P, stride = 0, 0
    if partials is not None:
        if partials.dim() == 2:
            partials = partials.unsqueeze(0)
        assert partials.dtype == torch.float32 and partials.shape[-2:] == (T, D)
        assert partials.stride(2) == 1 and partials.stride(1) == D
        P, stride = partials.shape[0], partials.stride(0)
    check(_fn("poot_rmsnorm")(_ptr(x), _ptr(h_out), _ptr(partials), P, stride, _ptr(w), _ptr(out), T, D, float(eps),
                              _stream()), "rmsnorm")
    return out


def reduce_partials(h: Optional[torch.Tensor], partials: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    P = partials.shape[0]
    n = out.numel()
    assert partials.stride(2) == 1 and partials.stride(1) == out.shape[1] and out.is_contiguous()
    check(_fn("poot_reduce_partials")(_ptr(h), _ptr(partials), P, partials.stride(0), _ptr(out), n, _stream()),
          "reduce_partials")
    return out


def swiglu(gu: torch.Tensor, interleaved: bool, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need_cuda(gu)
    assert gu.dtype == torch.bfloat16 and gu.is_contiguous()
    T, F2 = gu.shape
    if out is None:
        out = torch.empty(T, F2 // 2, dtype=torch.bfloat16, device=gu.device)
    check(_fn("poot_swiglu")(_ptr(gu), _ptr(out), T, F2 // 2, int(interleaved), _stream()), "swiglu")
    return out


GATED_ACTS = {"silu": 0, "gelu_tanh": 1, "gelu_erf": 2, "swiglu_clamped": 3}


def gated_act(gu: torch.Tensor, interleaved: bool, act: str, out: Optional[torch.Tensor] = None, limit: float = 0.0,
              alpha: float = 1.702) -> torch.Tensor:
    """``act(gate) * up`` over a ``[T, 2F]`` projection output (GeGLU and the other gated FFNs that are not SwiGLU);
    ``swiglu_clamped``: ``(clamp(up, +-limit) + 1) * g * sigmoid(alpha * g)`` with ``g = min(gate, limit)``."""
    _need_cuda(gu)
    assert gu.dtype == torch.bfloat16 and gu.is_contiguous()
    T, F2 = gu.shape
    if out is None:
        out = torch.empty(T, F2 // 2, dtype=torch.bfloat16, device=gu.device)
    check(_fn("poot_gated_act")(_ptr(gu), _ptr(out), T, F2 // 2, int(interleaved), GATED_ACTS[act], float(limit), float(alpha),
                                _stream()), "gated_act")
    return out


def layernorm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``(x - mean) / sqrt(var + eps) * w (+ b)`` over the last axis (bf16)."""
    _need_cuda(x, w)
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and w.dtype == torch.bfloat16
    if out is None:
        out = torch.empty_like(x)
    check(_fn("poot_layernorm")(_ptr(x), _ptr(w), _ptr(b), float(eps), _ptr(out), x.shape[0], x.shape[1], _stream()), "layernorm")
    return out


PLAIN_ACTS = {"silu": 0, "gelu_tanh": 1, "gelu_erf": 2, "relu2": 4}


def act_(x: torch.Tensor, act: str) -> torch.Tensor:
    """``x = act(x)`` in place (bf16): the activation of FFNs without a gate."""
    _need_cuda(x)
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    check(_fn("poot_act_bf16")(_ptr(x), x.numel(), PLAIN_ACTS[act], _stream()), "act")
    return x


def replace_rows_(h: torch.Tensor, rows: torch.Tensor, flags: torch.Tensor) -> torch.Tensor:
    """``h[t] = rows[t]`` where ``flags[t] != 0`` (bf16 ``[T, D]``, int32 ``[T]``): rows of another modality (a vision
    connector's output) in place of the token embeddings."""
    _need_cuda(h, rows, flags)
    assert h.dtype == rows.dtype == torch.bfloat16 and flags.dtype == torch.int32
    assert h.is_contiguous() and rows.is_contiguous() and h.shape == rows.shape and flags.numel() == h.shape[0]
    check(_fn("poot_replace_rows")(_ptr(h), _ptr(rows), _ptr(flags), h.shape[0], h.shape[1], _stream()), "replace_rows")
    return h


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """``x = cap * tanh(x / cap)`` in place (fp32 logits)."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    check(_fn("poot_softcap_f32")(_ptr(x), x.numel(), float(cap), _stream()), "softcap")
    return x


def add(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need_cuda(a, b)
    if out is None:
        out = torch.empty_like(a)
    check(_fn("poot_add_bf16")(_ptr(a), _ptr(b), _ptr(out), a.numel(), _stream()), "add")
    return out


def bias_add_(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``x[t, :] += bias`` in place.  ``x`` is a bf16 or f32 matrix whose rows may be a column slice of a wider
    buffer (unit inner stride); ``bias`` is bf16 or f32 (an f32 ``x`` takes an f32 bias)."""
    _need_cuda(x, bias)
    assert x.dim() == 2 and x.stride(1) == 1 and bias.is_contiguous() and bias.numel() == x.shape[1]
    assert x.dtype in (torch.bfloat16, torch.float32) and bias.dtype in (torch.bfloat16, torch.float32)
    T, N = x.shape
    check(_fn("poot_bias_add")(_ptr(x), _ptr(bias), T, N, x.stride(0) if T > 1 else N,
                               int(x.dtype == torch.float32), int(bias.dtype == torch.float32), _stream()), "bias_add")
    return x


def bias_add_indexed_(x: torch.Tensor, table: torch.Tensor, idx: torch.Tensor, div: int = 1, e0: int = 0,
                      gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x[r] += table[idx[r // div] + e0] * (gate[r] if gate is given else 1)`` in place; rows whose index is negative
    are left alone.  ``x`` and ``table`` are contiguous bf16, ``idx`` int32, ``gate`` f32."""
    _need_cuda(x, table, idx)
    assert x.dtype == table.dtype == torch.bfloat16 and x.is_contiguous() and table.is_contiguous()
    assert idx.dtype == torch.int32 and idx.is_contiguous() and table.shape[1] == x.shape[1]
    R, N = x.shape
    assert idx.numel() * div >= R
    if gate is not None:
        assert gate.dtype == torch.float32 and gate.is_contiguous() and gate.numel() >= R
    check(_fn("poot_bias_add_indexed")(_ptr(x), _ptr(table), _ptr(idx), int(div), int(e0), table.shape[0],
                                       _ptr(gate) if gate is not None else None, R, N, _stream()), "bias_add_indexed")
    return x


def scale_(x: torch.Tensor, s: float) -> torch.Tensor:
    """``x *= s`` in place (bf16, contiguous)."""
    _need_cuda(x)
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    check(_fn("poot_scale_bf16")(_ptr(x), x.numel(), float(s), _stream()), "scale")
    return x


def gather_rows(src: torch.Tensor, idx: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[b] = src[idx[b]]`` for 2-D tensors of one dtype (16-byte chunks when rows and pitches allow, narrower otherwise); ``idx`` is int64
    with ``out.shape[0]`` entries read."""
    _need_cuda(src, idx, out)
    assert src.dim() == 2 and out.dim() == 2 and src.dtype == out.dtype and src.shape[1] == out.shape[1]
    assert src.stride(1) == 1 and out.stride(1) == 1 and idx.dtype == torch.int64 and idx.is_contiguous()
    assert idx.numel() >= out.shape[0]
    es = src.element_size()
    B = out.shape[0]
    check(_fn("poot_gather_rows")(_ptr(src), src.stride(0) * es, src.shape[0], _ptr(idx), _ptr(out),
                                  (out.stride(0) if B > 1 else out.shape[1]) * es, B, src.shape[1] * es, _stream()),
          "gather_rows")
    return out


def sigmoid_gate_rows_(x: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """``x[t, :] *= sigmoid(g[t, 0])`` in place: ``x`` bf16 contiguous ``[T, N]``, ``g`` f32 ``[T, >=1]``."""
    _need_cuda(x, g)
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and g.dtype == torch.float32 and g.dim() == 2
    assert g.shape[0] == x.shape[0] and g.stride(1) == 1
    check(_fn("poot_sigmoid_gate_rows")(_ptr(x), _ptr(g), g.stride(0), x.shape[0], x.shape[1], _stream()),
          "sigmoid_gate_rows")
    return x


def _out_for(epi: int, M: int, N: int, device, out):
    if out is not None:
        return out
    if epi == EPI_F32:
        return torch.empty(M, N, dtype=torch.float32, device=device)
    if epi == EPI_SWIGLU:
        return torch.empty(M, N // 2, dtype=torch.bfloat16, device=device)
    return torch.empty(M, N, dtype=torch.bfloat16, device=device)


def gemv(x: torch.Tensor, W: torch.Tensor, epi: int = EPI_STORE, out: Optional[torch.Tensor] = None,
         resid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Skinny GEMM ``x[M,K] @ W[N,K]^T`` for ``M <= 4`` (decode)."""
    _need_cuda(x, W)
    assert x.dtype == torch.bfloat16 and W.dtype == torch.bfloat16 and W.is_contiguous()
    M, K = x.shape
    N = W.shape[0]
    assert W.shape[1] == K and x.stride(1) == 1
    out = _out_for(epi, M, N, x.device, out)
    check(_fn("poot_gemv_bf16")(epi, _ptr(x), _ptr(W), _ptr(out), _ptr(resid), M, N, K, x.stride(0), out.stride(0),
                                _stream()), "gemv_bf16")
    return out


def _pick_bn(M: int, N: int) -> int:
    m_tiles = (M + 127) // 128
    if m_tiles * ((N + 255) // 256) >= 148:
        return 256
    if m_tiles * ((N + 127) // 128) >= 120:
        return 128
    return 64


def gemm(x: torch.Tensor, W: torch.Tensor, epi: int = EPI_STORE, out: Optional[torch.Tensor] = None,
         resid: Optional[torch.Tensor] = None, bn: Optional[int] = None, splits: int = 1) -> torch.Tensor:
    """tcgen05 GEMM ``x[M,K] @ W[N,K]^T``.  With ``epi == EPI_PARTIAL`` the result is fp32 ``[splits, M, N]``."""
    _need_cuda(x, W)
    assert x.dtype == torch.bfloat16 and W.dtype == torch.bfloat16 and W.is_contiguous()
    M, K = x.shape
    N = W.shape[0]
    assert W.shape[1] == K and x.stride(1) == 1
    if bn is None:
        bn = _pick_bn(M, N)
    pstride = 0
    if epi == EPI_PARTIAL:
        if out is None:
            out = torch.empty(splits, M, N, dtype=torch.float32, device=x.device)
        pstride = out.stride(0)
        ldo = out.stride(1)
    else:
        out = _out_for(epi, M, N, x.device, out)
        ldo = out.stride(0)
    st = status_word(x.device)
    check(_fn("poot_gemm_bf16_tcgen05")(epi, _ptr(x), _ptr(W), _ptr(out), _ptr(resid), M, N, K, x.stride(0), ldo, bn,
                                        splits, pstride, _ptr(st), _stream()), "gemm_bf16_tcgen05")
    return out


def skinny_cluster(N: int, Kd: int) -> int:
    """Cluster size (K split) that fills the 148 SMs for a weight of N rows."""
    row_tiles = (N + 127) // 128
    ck = 1
    while ck < 8 and row_tiles * ck < 148 and (Kd // 64) // (ck * 2) >= 4:
        ck *= 2
    return ck


def gemm_skinny(x: torch.Tensor, W: torch.Tensor, epi: int = EPI_STORE, out: Optional[torch.Tensor] = None,
                resid: Optional[torch.Tensor] = None, ck: Optional[int] = None, wm: int = 1) -> torch.Tensor:
    """Swap-AB tcgen05 GEMM for ``M <= 128`` tokens with cluster split-K reduced through DSMEM."""
    _need_cuda(x, W)
    assert x.dtype == torch.bfloat16 and W.dtype == torch.bfloat16 and W.is_contiguous()
    M, Kd = x.shape
    N = W.shape[0]
    assert W.shape[1] == Kd and x.stride(1) == 1 and M <= 128 and epi != EPI_PARTIAL
    if ck is None:
        ck = skinny_cluster(N, Kd)
    out = _out_for(epi, M, N, x.device, out)
    st = status_word(x.device)
    check(_fn("poot_gemm_skinny")(epi, _ptr(x), _ptr(W), _ptr(out), _ptr(resid), M, N, Kd, x.stride(0), out.stride(0),
                                  ck, wm, 0, _ptr(st), _stream()), "gemm_skinny")
    return out


GEMV_MAX_M = 0          # rows served by the SIMT GEMV; 0 routes every decode GEMM to the tensor-core kernel


def set_pdl(on: bool) -> None:
    """Library-wide switch: launch kernels with programmatic stream serialization."""
    lib = kernels()
    lib.poot_set_pdl.argtypes = [c_int]
    lib.poot_set_pdl.restype = None
    lib.poot_set_pdl(int(on))


def linear(x: torch.Tensor, W: torch.Tensor, epi: int = EPI_STORE, out: Optional[torch.Tensor] = None,
           resid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Pick the decode GEMV (``M <= 4``), the skinny swap-AB GEMM (``M <= 128``) or the tiled GEMM."""
    M = x.shape[0]
    if M <= GEMV_MAX_M:
        return gemv(x, W, epi, out, resid)
    if M <= 128:
        return gemm_skinny(x, W, epi, out, resid)
    return gemm(x, W, epi, out, resid)


def rope_kv_write(qkv: torch.Tensor, q_out: torch.Tensor, kpool: torch.Tensor, vpool: torch.Tensor,
                  positions: torch.Tensor, slots: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, Hq: int,
                  Hkv: int, D: int, rot: Optional[int] = None, q_norm_w: Optional[torch.Tensor] = None,
                  k_norm_w: Optional[torch.Tensor] = None, norm_eps: float = 1e-6) -> None:
    _need_cuda(qkv, kpool)
    T = qkv.shape[0]
    assert qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and qkv.shape[1] == (Hq + 2 * Hkv) * D
    assert positions.dtype == torch.int32 and slots.dtype == torch.int32
    assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous()
    rot = D if rot is None else rot
    assert cos.shape[1] == rot // 2
    check(_fn("poot_rope_kv_write")(_ptr(qkv), _ptr(q_out), _ptr(kpool), _ptr(vpool), _ptr(positions), _ptr(slots),
                                    _ptr(cos), _ptr(sin), _ptr(q_norm_w), _ptr(k_norm_w), float(norm_eps), T, Hq, Hkv,
                                    D, rot, cos.shape[0], 0, _stream()), "rope_kv_write")


def attn_paged(q: torch.Tensor, kpool: torch.Tensor, vpool: torch.Tensor, block_tables: torch.Tensor,
               row_seq: Optional[torch.Tensor], row_ctx: torch.Tensor, Hq: int, Hkv: int, D: int, scale: float,
               out: Optional[torch.Tensor] = None, splits: int = 1, scratch=None, softcap: float = 0.0,
               window: int = 0) -> torch.Tensor:
    """Paged attention for R query rows; ``q`` is ``[R, Hq*D]``; pools are ``[blocks, Hkv, 16, D]``."""
    _need_cuda(q, kpool, vpool)
    R = q.shape[0]
    assert q.dtype == torch.bfloat16 and q.stride(1) == 1
    assert block_tables.dtype == torch.int32 and row_ctx.dtype == torch.int32
    if out is None:
        out = torch.empty(R, Hq * D, dtype=torch.bfloat16, device=q.device)
    po = pml = None
    if splits > 1:
        if scratch is None:
            po = torch.empty(R * Hq * splits * D, dtype=torch.float32, device=q.device)
            pml = torch.empty(R * Hq * splits * 2, dtype=torch.float32, device=q.device)
        else:
            po, pml = scratch
            assert po.numel() >= R * Hq * splits * D and pml.numel() >= R * Hq * splits * 2
    check(_fn("poot_attn_paged")(_ptr(q), q.stride(0), _ptr(kpool), _ptr(vpool), _ptr(block_tables),
                                 block_tables.shape[1], _ptr(row_seq), _ptr(row_ctx), _ptr(out), out.stride(0),
                                 _ptr(po), _ptr(pml), R, Hq, Hkv, D, float(scale), float(softcap), int(window),
                                 int(splits), _stream()), "attn_paged")
    return out


def mla_qkv_write(q: torch.Tensor, kvb: torch.Tensor, kva: torch.Tensor, rope_col: int, q_out: torch.Tensor, kpool: torch.Tensor,
                  vpool: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, nh: int,
                  dn: int, dr: int, dv: int) -> None:
    """Latent attention, expanded form: rotate the rotary parts, write the query rows ``[T, nh * (dn + dr)]`` and the key
    ``[no-position | shared rotary]`` and value rows into the pools (rows ``dn + dr`` wide; a value uses the first ``dv``)."""
    _need_cuda(q, kpool)
    T = q.shape[0]
    assert q.is_contiguous() and kvb.is_contiguous() and kva.stride(1) == 1 and q_out.is_contiguous()
    assert kpool.shape[-1] == dn + dr and cos.shape[1] == dr // 2 and cos.dtype == torch.float32
    check(_fn("poot_mla_qkv_write")(_ptr(q), _ptr(kvb), _ptr(kva), kva.stride(0), rope_col, _ptr(q_out), _ptr(kpool), _ptr(vpool),
                                    _ptr(positions), _ptr(slots), _ptr(cos), _ptr(sin), T, nh, dn, dr, dv, cos.shape[0], _stream()),
          "mla_qkv_write")


def attn_general(q: torch.Tensor, kpool: torch.Tensor, vpool: torch.Tensor, block_tables: torch.Tensor,
                 row_seq: Optional[torch.Tensor], row_ctx: torch.Tensor, Hq: int, Hkv: int, Dk: int, Dv: int, scale: float,
                 out: torch.Tensor, softcap: float = 0.0, window: int = 0, alibi: Optional[torch.Tensor] = None,
                 sinks: Optional[torch.Tensor] = None, sel: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Paged attention for the shapes the tuned kernels do not serve: key width ``Dk`` and value width ``Dv`` (multiples of
    32 up to 512), optional per-head ALiBi slopes and sink logits (fp32 ``[Hq]``).  Pools are ``[blocks, Hkv, 16, pool_d]``.
    ``sel[rows, k]`` int32 (ascending key positions, -1 after the last) restricts each row to the listed keys."""
    _need_cuda(q, kpool, vpool)
    if sel is not None:
        assert sel.dtype == torch.int32 and sel.is_contiguous() and sel.shape[0] >= q.shape[0]
    assert q.dtype == torch.bfloat16 and q.stride(1) == 1 and kpool.is_contiguous() and vpool.is_contiguous()
    assert kpool.shape == vpool.shape and block_tables.dtype == torch.int32 and row_ctx.dtype == torch.int32
    check(_fn("poot_attn_general")(_ptr(q), q.stride(0), _ptr(kpool), _ptr(vpool), kpool.shape[-1], _ptr(block_tables),
                                   block_tables.shape[1], _ptr(row_seq), _ptr(row_ctx), _ptr(out), out.stride(0), q.shape[0], Hq,
                                   Hkv, Dk, Dv, float(scale), float(softcap), int(window), _ptr(alibi), _ptr(sinks), _ptr(sel),
                                   sel.shape[1] if sel is not None else 0, _stream()),
          "attn_general")
    return out


# ---- sparse attention indexer ---------------------------------------------------------------------------------------
def index_k_write(kraw: torch.Tensor, norm_w: torch.Tensor, norm_b: Optional[torch.Tensor], eps: float,
                  positions: torch.Tensor, slots: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pool: torch.Tensor,
                  dr: int) -> None:
    """Indexer keys of a step: ``LayerNorm(kraw)`` with the rotary on the leading ``dr`` channels (half-split), written
    to ``pool[blocks, 16, Di]`` at the tokens' slots."""
    _need_cuda(kraw, pool)
    T, Di = kraw.shape
    assert kraw.dtype == torch.bfloat16 and kraw.is_contiguous() and pool.is_contiguous() and pool.shape[-1] == Di
    assert cos.dtype == torch.float32 and (dr == 0 or cos.shape[1] == dr // 2)
    check(_fn("poot_index_k_write")(_ptr(kraw), _ptr(norm_w), _ptr(norm_b), float(eps), _ptr(positions), _ptr(slots), _ptr(cos),
                                    _ptr(sin), _ptr(pool), T, Di, dr, cos.shape[0], _stream()), "index_k_write")


def index_q_rope(q: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, ni: int, Di: int,
                 dr: int) -> torch.Tensor:
    """The rotary on the leading ``dr`` channels of each indexer query head, in place: ``q[T, ni * Di]``."""
    _need_cuda(q)
    assert q.dtype == torch.bfloat16 and q.is_contiguous() and q.shape[1] == ni * Di
    check(_fn("poot_index_q_rope")(_ptr(q), _ptr(positions), _ptr(cos), _ptr(sin), q.shape[0], ni, Di, dr, cos.shape[0],
                                   _stream()), "index_q_rope")
    return q


def index_scores(q: torch.Tensor, w: torch.Tensor, pool: torch.Tensor, block_tables: torch.Tensor,
                 row_seq: Optional[torch.Tensor], row_ctx: torch.Tensor, scores: torch.Tensor, ni: int, Di: int,
                 max_ctx: int, scale: float) -> torch.Tensor:
    """``scores[r, j] = sum_h w[r, h] * relu(q[r, h] . key[j] * scale)`` for every visible key ``j < row_ctx[r]``;
    entries at and beyond a row's context are left as they were.  ``w`` is f32 ``[rows, >= ni]``."""
    _need_cuda(q, w, pool, scores)
    assert q.dtype == torch.bfloat16 and q.is_contiguous() and w.dtype == torch.float32 and w.stride(1) == 1
    assert scores.dtype == torch.float32 and scores.stride(1) == 1 and scores.shape[1] >= max_ctx
    check(_fn("poot_index_scores")(_ptr(q), _ptr(w), w.stride(0), _ptr(pool), _ptr(block_tables), block_tables.shape[1],
                                   _ptr(row_seq), _ptr(row_ctx), _ptr(scores), scores.stride(0), q.shape[0], ni, Di,
                                   int(max_ctx), float(scale), _stream()), "index_scores")
    return scores


def index_select(scores: torch.Tensor, row_ctx: torch.Tensor, sel: torch.Tensor) -> torch.Tensor:
    """Per row the ``sel.shape[1]`` best of its ``row_ctx[r]`` scores (ties at the cut: lowest position first), as
    ascending positions with -1 after the last kept; a row with no more scores than that keeps them all."""
    _need_cuda(scores, sel)
    assert scores.dtype == torch.float32 and sel.dtype == torch.int32 and sel.is_contiguous()
    check(_fn("poot_index_select")(_ptr(scores), scores.stride(0), _ptr(row_ctx), _ptr(sel), sel.shape[0], sel.shape[1],
                                   _stream()), "index_select")
    return sel


FLASH_MIN_TOKENS = 16      # prefill pieces at least this long go to the tensor-core kernel


def flash_tiles(row_seq, positions, min_tokens: int = FLASH_MIN_TOKENS):
    """Split a step's rows into tensor-core tiles and rows left to the per-row kernel.

    ``row_seq`` / ``positions``: host int arrays of the step's T rows.  A *segment* is a maximal run of rows of one
    sequence at consecutive positions; segments of at least ``min_tokens`` rows are cut into tiles of up to 128 rows
    ``(first row, rows, block-table row, first position)``.  Returns ``(tiles [n, 4] int32, covered [T] bool)``."""
    import numpy as np
    seq = np.asarray(row_seq, dtype=np.int64)
    pos = np.asarray(positions, dtype=np.int64)
    T = seq.shape[0]
    covered = np.zeros(T, dtype=bool)
    if T == 0:
        return np.zeros((0, 4), np.int32), covered
    brk = np.flatnonzero((seq[1:] != seq[:-1]) | (pos[1:] != pos[:-1] + 1)) + 1
    starts = np.concatenate([[0], brk])
    ends = np.concatenate([brk, [T]])
    tiles = []
    for a, b in zip(starts.tolist(), ends.tolist()):
        if b - a < min_tokens:
            continue
        covered[a:b] = True
        for t0 in range(a, b, 128):
            tiles.append((t0, min(128, b - t0), int(seq[a]), int(pos[a]) + (t0 - a)))
    return np.asarray(tiles, dtype=np.int32).reshape(-1, 4), covered


def step_segments(row_seq, positions, row_ctx):
    """The sequence pieces of a step: maximal runs of live rows (context > 0) of one sequence at consecutive positions,
    as ``[n, 4]`` int32 ``(first row, rows, block-table row, first position)``."""
    import numpy as np
    seq = np.asarray(row_seq, dtype=np.int64)
    pos = np.asarray(positions, dtype=np.int64)
    live = np.asarray(row_ctx) > 0
    out, t, T = [], 0, seq.shape[0]
    while t < T:
        if not live[t]:
            t += 1
            continue
        e = t + 1
        while e < T and live[e] and seq[e] == seq[t] and pos[e] == pos[e - 1] + 1:
            e += 1
        out.append((t, e - t, int(seq[t]), int(pos[t])))
        t = e
    return np.asarray(out, dtype=np.int32).reshape(-1, 4)


def causal_conv_silu(x: torch.Tensor, col0: int, C: int, w: torch.Tensor, state: torch.Tensor, segs: torch.Tensor,
                     out: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Depthwise causal convolution + SiLU over columns ``[col0, col0 + C)`` of ``x[T, ld]`` (bf16), per sequence piece
    of ``segs``, continuing from and updating ``state[rows, K-1, C]`` (fp32; a piece at position 0 starts from zeros)."""
    _need_cuda(x, state)
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and w.dtype == torch.float32 and w.is_contiguous()
    assert state.dtype == torch.float32 and state.is_contiguous() and segs.dtype == torch.int32 and out.is_contiguous()
    Kc = w.shape[1]
    check(_fn("poot_causal_conv_silu")(_ptr(x), x.stride(0), col0, C, Kc, _ptr(w), _ptr(bias), _ptr(state), state.shape[0],
                                       _ptr(segs), segs.shape[0], _ptr(out), _stream()), "causal_conv_silu")
    return out


def gdn_scan(qkv: torch.Tensor, ba: torch.Tensor, b_col: int, a_col: int, dt_bias: torch.Tensor, a_log: torch.Tensor,
             state: torch.Tensor, segs: torch.Tensor, out: torch.Tensor, nk: int, nv: int, D: int) -> torch.Tensor:
    """Gated delta rule over each sequence piece (crates/poot-graph-ir/src/ops/ssm.rs).  ``qkv[T, (2 nk + nv) D]`` holds
    q | k | v after the convolution; ``ba[T, ld]`` holds the raw b and a projections at columns ``b_col`` / ``a_col``;
    q and k are normalised to unit length, q scaled by ``D^-1/2``, ``g = -exp(a_log) softplus(a + dt_bias)``,
    ``beta = sigmoid(b)``; ``state[rows, nv, D, D]`` fp32 is read (unless the piece starts at position 0) and updated."""
    _need_cuda(qkv, state)
    assert qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and ba.dtype == torch.bfloat16 and ba.stride(1) == 1
    assert state.dtype == torch.float32 and state.is_contiguous() and out.is_contiguous() and D in (64, 128)
    check(_fn("poot_gdn_scan")(_ptr(qkv), _ptr(ba), ba.stride(0), b_col, a_col, _ptr(dt_bias), _ptr(a_log), _ptr(state),
                               state.shape[0], _ptr(segs), segs.shape[0], _ptr(out), nk, nv, D, _stream()), "gdn_scan")
    return out


def ngram_hash(tokens: torch.Tensor, history: torch.Tensor, segs: torch.Tensor, mult: torch.Tensor, primes: torch.Tensor,
               offsets: torch.Tensor, per_order: int, eos: int, vocab: int, ids: torch.Tensor) -> torch.Tensor:
    """Hashed n-gram ids ``ids[T, heads]`` (int32) of the step's tokens, piece by piece (crates/poot-models/src/components/
    ple.rs ``row_ids``): head ``h`` is ``((m0 * s0) ^ (m1 * s1) [^ (m2 * s2)]) % primes[h] + offsets[h]`` over wrapping
    64-bit words.  ``history[rows, ctx]`` int32 holds each sequence's last ``ctx`` tokens xor-ed with ``eos`` (a piece at
    position 0 ignores it) and is updated; ``mult`` is int64 holding the unsigned multipliers' bits, ``primes`` int32
    holding unsigned moduli."""
    _need_cuda(tokens, history)
    ctx, heads = history.shape[1], ids.shape[1]
    assert tokens.dtype == torch.int32 and history.dtype == torch.int32 and ids.dtype == torch.int32 and segs.dtype == torch.int32
    assert mult.dtype == torch.int64 and mult.numel() == ctx + 1 and primes.dtype == torch.int32 and offsets.dtype == torch.int32
    assert primes.numel() == heads == offsets.numel() and heads == ctx * per_order and ids.is_contiguous() and history.is_contiguous()
    check(_fn("poot_ngram_hash")(_ptr(tokens), _ptr(history), history.shape[0], _ptr(segs), segs.shape[0], _ptr(mult), _ptr(primes),
                                 _ptr(offsets), ctx, heads, per_order, eos, vocab, _ptr(ids), _stream()), "ngram_hash")
    return ids


def kda_scan(qkv: torch.Tensor, f: torch.Tensor, bm: torch.Tensor, b_col: int, dt_bias: torch.Tensor, a_log: torch.Tensor,
             lower_bound: float, state: torch.Tensor, segs: torch.Tensor, out: torch.Tensor, heads: int, D: int) -> torch.Tensor:
    """Kimi delta attention's recurrence over each sequence piece (crates/poot-models/src/components/kda.rs): the delta
    rule of :func:`gdn_scan` with a decay per key channel.  ``qkv[T, 3 * heads * D]`` holds q | k | v after the
    convolution, ``f[T, heads * D]`` the raw low-rank gate projection, ``bm[T, ld]`` the raw beta projection at column
    ``b_col``; row ``i`` of a head's state decays by ``exp(lower_bound * sigmoid(exp(a_log[h]) * (f[h, i] + dt_bias[h, i])))``."""
    _need_cuda(qkv, state)
    assert qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and f.dtype == torch.bfloat16 and f.is_contiguous()
    assert bm.dtype == torch.bfloat16 and bm.stride(1) == 1 and qkv.shape[1] == 3 * heads * D and f.shape[1] == heads * D
    assert state.dtype == torch.float32 and state.is_contiguous() and out.is_contiguous() and D in (64, 128) and lower_bound < 0
    check(_fn("poot_kda_scan")(_ptr(qkv), _ptr(f), _ptr(bm), bm.stride(0), b_col, _ptr(dt_bias), _ptr(a_log), float(lower_bound),
                               _ptr(state), state.shape[0], _ptr(segs), segs.shape[0], _ptr(out), heads, D, _stream()), "kda_scan")
    return out


def gated_rmsnorm(y: torch.Tensor, z: torch.Tensor, z_col: int, w: torch.Tensor, eps: float, out: torch.Tensor,
                  heads: int, D: int, gate_first: bool = False) -> torch.Tensor:
    """``out = rmsnorm_D(y) * w * silu(z)`` per head (``w[D]`` shared by the heads), or with ``gate_first``
    ``rmsnorm_D(y * silu(z)) * w`` per channel group (``w[heads * D]``); ``z`` is read at columns
    ``[z_col, z_col + heads * D)`` of its rows."""
    _need_cuda(y, z)
    assert y.dtype == torch.bfloat16 and y.is_contiguous() and z.stride(1) == 1 and w.dtype == torch.bfloat16
    per_head = int(w.numel() == heads * D and heads > 1)
    assert w.numel() in (D, heads * D)
    check(_fn("poot_gated_rmsnorm")(_ptr(y), _ptr(z), z.stride(0), z_col, _ptr(w), per_head, float(eps), int(gate_first), _ptr(out),
                                    y.shape[0], heads, D, _stream()), "gated_rmsnorm")
    return out


def ssd_scan(xbc: torch.Tensor, dtm: torch.Tensor, dt_col: int, dt_bias: torch.Tensor, a_log: torch.Tensor, dskip: torch.Tensor,
             state: torch.Tensor, segs: torch.Tensor, out: torch.Tensor, nh: int, groups: int, N: int, P: int) -> torch.Tensor:
    """Mamba2 selective state-space recurrence over each sequence piece (crates/poot-graph-ir/src/ops/ssm.rs):
    ``xbc[T, nh P + 2 groups N]`` holds x | B | C after the convolution, the raw time steps are columns
    ``[dt_col, dt_col + nh)`` of ``dtm``; ``state[rows, nh, N, P]`` fp32 is read (unless the piece starts at position 0)
    and updated; ``out[T, nh P]``."""
    _need_cuda(xbc, state)
    assert xbc.dtype == torch.bfloat16 and xbc.is_contiguous() and dtm.stride(1) == 1 and state.dtype == torch.float32
    assert state.is_contiguous() and out.is_contiguous() and P in (32, 64, 128)
    check(_fn("poot_ssd_scan")(_ptr(xbc), _ptr(dtm), dtm.stride(0), dt_col, _ptr(dt_bias), _ptr(a_log), _ptr(dskip), _ptr(state),
                               state.shape[0], _ptr(segs), segs.shape[0], _ptr(out), nh, groups, N, P, _stream()), "ssd_scan")
    return out


def sigmoid_mul(a: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """``a *= sigmoid(g)`` elementwise (bf16, same shape)."""
    _need_cuda(a, g)
    assert a.dtype == torch.bfloat16 and a.is_contiguous() and g.is_contiguous() and a.shape == g.shape
    check(_fn("poot_sigmoid_mul")(_ptr(a), _ptr(g), a.numel(), _stream()), "sigmoid_mul")
    return a


def attn_flash_prefill(q: torch.Tensor, kpool: torch.Tensor, vpool: torch.Tensor, block_tables: torch.Tensor,
                       tiles: torch.Tensor, Hq: int, Hkv: int, scale: float, out: torch.Tensor, window: int = 0) -> None:
    """Tensor-core causal attention over paged K/V for the rows named by ``tiles`` (``[n, 4]`` int32 on the device;
    entries with zero rows are skipped).  head_dim 128 only; pools are ``[blocks, Hkv, 16, 128]`` bf16."""
    _need_cuda(q, kpool, vpool)
    assert q.dtype == torch.bfloat16 and q.stride(1) == 1 and kpool.shape[-1] == 128 and kpool.is_contiguous()
    assert tiles.dtype == torch.int32 and tiles.shape[1] == 4 and tiles.is_contiguous()
    st = status_word(q.device)
    check(_fn("poot_attn_flash_prefill")(_ptr(q), q.stride(0), q.shape[0], _ptr(kpool), _ptr(vpool), kpool.shape[0],
                                         _ptr(block_tables), block_tables.shape[1], _ptr(tiles), tiles.shape[0],
                                         _ptr(out), out.stride(0), Hq, Hkv, float(scale), int(window), _ptr(st),
                                         _stream()), "attn_flash_prefill")


ARGMAX_CHUNK = 2048


def argmax_groups(vocab: int) -> int:
    return max(1, (vocab + ARGMAX_CHUNK - 1) // ARGMAX_CHUNK)


def argmax_scratch(rows: int, vocab: int, device) -> torch.Tensor:
    """int32 ``[rows, groups, 3]`` partial table ``(bits of best value, best index, first non-finite index)``."""
    return torch.empty(rows, argmax_groups(vocab), 3, dtype=torch.int32, device=device)


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None, scratch=None) -> torch.Tensor:
    """Greedy pick per row: ``out[r] = (token, non_finite_index)``."""
    _need_cuda(logits)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty(rows, 2, dtype=torch.int32, device=logits.device)
    part = scratch if scratch is not None else argmax_scratch(rows, vocab, logits.device)
    check(_fn("poot_argmax")(_ptr(logits), rows, vocab, ARGMAX_CHUNK, _ptr(part), _ptr(out), _stream()), "argmax")
    return out


def argmax_partials(logits: torch.Tensor, idx_offset: int, vocab_total: int, part: torch.Tensor) -> torch.Tensor:
    """Stage 1 of the greedy pick over one vocabulary shard (indices are global)."""
    rows, vocab = logits.shape
    check(_fn("poot_argmax_partials")(_ptr(logits), rows, vocab, logits.stride(0), idx_offset, vocab_total,
                                      ARGMAX_CHUNK, _ptr(part), _stream()), "argmax_partials")
    return part


def argmax_combine(parts: torch.Tensor, rows: int, groups: int, vocab_total: int, out: torch.Tensor) -> torch.Tensor:
    """Stage 2 over ``parts[nparts, rows, groups, 3]`` (one table per vocabulary shard)."""
    nparts = parts.shape[0]
    check(_fn("poot_argmax_combine")(_ptr(parts), nparts, parts.stride(0), rows, groups, vocab_total, _ptr(out),
                                     _stream()), "argmax_combine")
    return out


def sample_gumbel(logits: torch.Tensor, params: torch.Tensor, top_k: torch.Tensor, seeds: torch.Tensor, rule: int,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gumbel-max sampling; ``params[r] = (inv_temp, floor_offset, noise_scale, top_p)``; rule 1..3."""
    _need_cuda(logits)
    rows, vocab = logits.shape
    assert params.shape == (rows, 4) and params.dtype == torch.float32
    assert top_k.dtype == torch.int32 and seeds.dtype == torch.int32
    if out is None:
        out = torch.empty(rows, 2, dtype=torch.int32, device=logits.device)
    check(_fn("poot_sample_gumbel")(_ptr(logits), rows, vocab, _ptr(params), _ptr(top_k), _ptr(seeds), rule, _ptr(out),
                                    _stream()), "sample_gumbel")
    return out


def random_uniform(seeds: torch.Tensor, cols: int) -> torch.Tensor:
    rows = seeds.numel()
    out = torch.empty(rows, cols, dtype=torch.float32, device=seeds.device)
    check(_fn("poot_random_uniform")(_ptr(seeds), rows, cols, _ptr(out), _stream()), "random_uniform")
    return out


def decode_advance(picked: torch.Tensor, tokens: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                   ctx: torch.Tensor, block_tables: torch.Tensor, row_seq: Optional[torch.Tensor], B: int) -> None:
    """Feed sampled tokens back and advance positions / write slots on the device (chained decode)."""
    check(_fn("poot_decode_advance")(_ptr(picked), _ptr(tokens), _ptr(positions), _ptr(slots), _ptr(ctx),
                                     _ptr(block_tables), block_tables.shape[1], _ptr(row_seq), B, _stream()),
          "decode_advance")


# ---- GGUF block-quantised weights ---------------------------------------------------------------------------------
register_signature("poot_quant_gemv", [c_int, c_int, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P])
register_signature("poot_quant_row_gather", [c_int, _P, _P, _P, c_int, c_int, c_int, _P])
register_signature("poot_quant_dequant_bf16", [c_int, _P, _P, c_int, c_int, _P])
# block formats with dequant-fused device kernels (name -> ggml type id, the id the launchers take)
QUANT_DEVICE_FORMATS = {"Q4_0": 2, "Q4_1": 3, "Q5_0": 6, "Q5_1": 7, "Q8_0": 8, "Q2_K": 10, "Q3_K": 11, "Q4_K": 12,
                        "Q5_K": 13, "Q6_K": 14, "IQ4_NL": 20, "IQ4_XS": 23, "MXFP4": 39}


class QuantWeight:
    """A packed ``[N, K]`` weight resident on the device in its checkpoint block layout."""

    def __init__(self, fmt: str, packed: torch.Tensor, N: int, K: int):
        if fmt not in QUANT_DEVICE_FORMATS:
            raise ValueError(f"{fmt} has no fused device kernels (expand it to bf16 at load time)")
        assert packed.dtype == torch.uint8 and packed.is_cuda and packed.is_contiguous()
        self.fmt, self.packed, self.N, self.K = fmt, packed, N, K
        self.type_id = QUANT_DEVICE_FORMATS[fmt]
        self.shape = (N, K)
        self._scratch = None

    @property
    def device(self):
        return self.packed.device

    def nbytes(self) -> int:
        return self.packed.numel()


_dequant_scratch = {}
# Decode batches of 5 to 128 rows over packed weights: the dequant-fused tensor-core kernel (the packed weight is read
# once and never written back as bf16) instead of "decode the whole matrix to bf16, then the dense GEMM".  Opt-in
# (POOT_QUANT_FUSED_GEMM=1) until the kernel has been checked on a device.
QUANT_FUSED_GEMM = os.environ.get("POOT_QUANT_FUSED_GEMM", "0") not in ("", "0")
_SIGS["poot_quant_gemm_skinny"] = [c_int, c_int, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P, _P]


def quant_gemm_skinny(x: torch.Tensor, W: "QuantWeight", epi: int = EPI_STORE, out: Optional[torch.Tensor] = None,
                      resid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x[M <= 128, K] @ dequant(W)^T`` with the block decode fused into the tcgen05 GEMM's weight stage."""
    _need_cuda(x, W.packed)
    M, Kd = x.shape
    assert Kd == W.K and x.dtype == torch.bfloat16 and x.stride(1) == 1 and M <= 128
    out = _out_for(epi, M, W.N, x.device, out)
    check(_fn("poot_quant_gemm_skinny")(W.type_id, epi, _ptr(x), _ptr(W.packed), _ptr(out), _ptr(resid), M, W.N, Kd,
                                        x.stride(0), out.stride(0), status_word(x.device).data_ptr(), _stream()),
          "quant_gemm_skinny")
    return out



def quant_gemv(x: torch.Tensor, W: QuantWeight, epi: int = EPI_STORE, out: Optional[torch.Tensor] = None,
               resid: Optional[torch.Tensor] = None) -> torch.Tensor:
    M, Kd = x.shape
    assert Kd == W.K and x.dtype == torch.bfloat16 and x.stride(1) == 1
    out = _out_for(epi, M, W.N, x.device, out)
    check(_fn("poot_quant_gemv")(W.type_id, epi, _ptr(x), _ptr(W.packed), _ptr(out), _ptr(resid), M, W.N, Kd,
                                 x.stride(0), out.stride(0), _stream()), "quant_gemv")
    return out


def quant_row_gather(ids: torch.Tensor, W: QuantWeight, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    T = ids.numel()
    if out is None:
        out = torch.empty(T, W.K, dtype=torch.bfloat16, device=W.device)
    check(_fn("poot_quant_row_gather")(W.type_id, _ptr(ids), _ptr(W.packed), _ptr(out), T, W.K, W.N, _stream()),
          "quant_row_gather")
    return out


def quant_dequant(W: QuantWeight, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if out is None:
        out = torch.empty(W.N, W.K, dtype=torch.bfloat16, device=W.device)
    check(_fn("poot_quant_dequant_bf16")(W.type_id, _ptr(W.packed), _ptr(out), W.N, W.K, _stream()), "quant_dequant")
    return out


_plain_linear = linear


PLANAR_DEVICE_FORMATS = {"E4M3_CHANNEL": 0, "E4M3_BLOCK128": 1, "E2M1_ROW32": 2, "GPTQ": 3, "AWQ": 4}
_SIGS["poot_planar_gemv"] = [c_int, c_int, _P, c_int, _P, _P, _P, _P, c_int, _P, _P, c_int, c_int, c_int, c_int, _P]
_SIGS["poot_planar_dequant"] = [c_int, _P, _P, _P, _P, c_int, _P, c_int, c_int, _P]


class PlanarWeight:
    """A ``[N, K]`` weight resident on the device as the tensors its safetensors checkpoint stores (codes, scales,
    zero points): fp8 with per-channel or 128 x 128 block scales, fp4 rows of 32, GPTQ and AWQ int4."""

    def __init__(self, fmt: str, ops: dict, N: int, K: int, group: int = 128):
        if fmt not in PLANAR_DEVICE_FORMATS:
            raise ValueError(f"{fmt} is not a planar format with device kernels")
        self.fmt, self.type_id, self.N, self.K, self.group = fmt, PLANAR_DEVICE_FORMATS[fmt], N, K, group
        self.shape = (N, K)
        if fmt in ("GPTQ", "AWQ"):
            self.w, self.zeros = ops["qweight"].contiguous(), ops["qzeros"].contiguous()
            self.scale = ops["scales"].to(torch.float32).contiguous()
            g = ops.get("g_idx")
            self.g_idx = None if g is None or fmt == "AWQ" else g.to(torch.int32).contiguous()
        else:
            self.w, self.zeros, self.g_idx = ops["weight"].contiguous(), None, None
            sc = ops["weight_scale_inv"] if fmt == "E4M3_BLOCK128" else ops["weight_scale"]
            self.scale = (sc if fmt == "E2M1_ROW32" else sc.to(torch.float32).reshape(-1) if fmt == "E4M3_CHANNEL"
                          else sc.to(torch.float32)).contiguous()

    @property
    def device(self):
        return self.w.device

    def tensors(self):
        return [t for t in (self.w, self.scale, self.zeros, self.g_idx) if t is not None]

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors())


def planar_gemv(x: torch.Tensor, W: PlanarWeight, epi: int = EPI_STORE, out: Optional[torch.Tensor] = None,
                resid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x[M <= 4, K] @ W^T`` decoded from the checkpoint's own tensors inside the product."""
    _need_cuda(x, W.w)
    M, Kd = x.shape
    assert Kd == W.K and x.dtype == torch.bfloat16 and x.stride(1) == 1 and epi in (EPI_STORE, EPI_F32, EPI_RESID)
    out = _out_for(epi, M, W.N, x.device, out)
    check(_fn("poot_planar_gemv")(W.type_id, {EPI_STORE: 0, EPI_F32: 1, EPI_RESID: 2}[epi], _ptr(x), x.stride(0), _ptr(W.w),
                                  _ptr(W.scale), _ptr(W.zeros), _ptr(W.g_idx), W.group, _ptr(out), _ptr(resid), out.stride(0),
                                  M, W.N, Kd, _stream()), "planar_gemv")
    return out


_SIGS["poot_planar_gemv_grouped"] = [c_int, _P, c_int, c_int, _P, _P, _P, _P, _P, _P, c_int, c_float, c_float, _P, _P, _P, c_int,
                                     c_int, c_int, c_int, c_int, _P]
PACKED_EXPERT_FORMATS = ("E4M3_CHANNEL", "E4M3_BLOCK128", "E2M1_ROW32")


class PackedExperts:
    """A layer's routed experts resident as their checkpoint stores them: per projection (``gate``, ``up``, ``down``) one
    stack of code tensors ``[E, N, K or K / 2]`` and one of scales (``[E, N]`` f32 per channel, ``[E, N / 128, K / 128]``
    f32 per block, ``[E, N, K / 32]`` e8m0 bytes for fp4 rows of 32).  Optional f32 biases ``[E, N]`` per projection."""

    def __init__(self, fmt: str, gate, up, down, E: int, F: int, H: int, bias_gate=None, bias_up=None, bias_down=None):
        if fmt not in PACKED_EXPERT_FORMATS:
            raise ValueError(f"{fmt}: experts stay packed in the row-major planar formats only")
        self.fmt, self.type_id, self.E, self.F, self.H = fmt, PLANAR_DEVICE_FORMATS[fmt], E, F, H
        self.gate, self.up, self.down = gate, up, down                   # (codes, scales) each
        self.bias_gate, self.bias_up, self.bias_down = bias_gate, bias_up, bias_down
        for (w, sc), (n, k) in ((gate, (F, H)), (up, (F, H)), (down, (H, F))):
            assert w.dtype == torch.uint8 and w.is_contiguous() and sc.is_contiguous() and w.shape[0] == E and w.shape[1] == n
            assert w.shape[2] == (k // 2 if fmt == "E2M1_ROW32" else k)

    @property
    def device(self):
        return self.gate[0].device

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for pair in (self.gate, self.up, self.down) for t in pair)


def planar_gemv_grouped(x: torch.Tensor, P: PackedExperts, which: str, ids: Optional[torch.Tensor], out: torch.Tensor, groups: int,
                        x_row_div: int = 0, row_scale: Optional[torch.Tensor] = None, act: str = "silu", alpha: float = 1.702,
                        limit: float = 0.0) -> torch.Tensor:
    """One activation row per group against the group's expert, decoded inside the product.  ``which="in"``:
    ``out[g] = act(gate_e(x) + b, up_e(x) + b)`` (SwiGLU, or the clamped form when ``limit > 0``) with ``x`` row
    ``g // x_row_div``; ``which="out"``: ``out[g] = (down_e(x[g]) + b) * row_scale[g]``.  ``ids[g]`` names the expert
    (negative: the row is zero)."""
    _need_cuda(x, P.gate[0])
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and out.dtype == torch.bfloat16 and out.stride(1) == 1
    assert ids is None or (ids.dtype == torch.int32 and ids.numel() >= groups)
    if which == "in":
        assert act == "silu" and x.shape[1] == P.H and out.shape[1] >= P.F
        check(_fn("poot_planar_gemv_grouped")(P.type_id, _ptr(x), x.stride(0), x_row_div, _ptr(P.gate[0]), _ptr(P.gate[1]), _ptr(P.up[0]),
                                              _ptr(P.up[1]), _ptr(P.bias_gate), _ptr(P.bias_up), 2 if limit > 0 else 1, float(alpha),
                                              float(limit), _ptr(ids), None, _ptr(out), out.stride(0), groups, P.E, P.F, P.H, _stream()),
              "planar_gemv_grouped")
    else:
        assert x.shape[1] == P.F and out.shape[1] >= P.H and (row_scale is None or row_scale.dtype == torch.float32)
        check(_fn("poot_planar_gemv_grouped")(P.type_id, _ptr(x), x.stride(0), x_row_div, _ptr(P.down[0]), _ptr(P.down[1]), None, None,
                                              _ptr(P.bias_down), None, 0, 0.0, 0.0, _ptr(ids), _ptr(row_scale), _ptr(out),
                                              out.stride(0), groups, P.E, P.H, P.F, _stream()), "planar_gemv_grouped")
    return out


def planar_dequant(W: PlanarWeight, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The whole weight as bf16 ``[N, K]``."""
    _need_cuda(W.w)
    if out is None:
        out = torch.empty(W.N, W.K, dtype=torch.bfloat16, device=W.device)
    check(_fn("poot_planar_dequant")(W.type_id, _ptr(W.w), _ptr(W.scale), _ptr(W.zeros), _ptr(W.g_idx), W.group, _ptr(out),
                                     W.N, W.K, _stream()), "planar_dequant")
    return out


def linear(x, W, epi: int = EPI_STORE, out: Optional[torch.Tensor] = None, resid: Optional[torch.Tensor] = None):
    """``x @ W^T`` for a bf16 weight, a packed ``QuantWeight`` or a ``PlanarWeight`` (fused GEMV at decode, expand + GEMM
    for larger M)."""
    if isinstance(W, PlanarWeight):
        if x.shape[0] <= 4 and epi in (EPI_STORE, EPI_F32, EPI_RESID):
            return planar_gemv(x, W, epi, out, resid)
        if x.shape[0] <= 4 and epi == EPI_SWIGLU:           # interleaved (gate, up) rows: product, then the gated activation
            key = (W.device, "gu", W.N)
            gu = _dequant_scratch.get(key)
            if gu is None:
                gu = _dequant_scratch[key] = torch.empty(4, W.N, dtype=torch.bfloat16, device=W.device)
            return swiglu(planar_gemv(x, W, EPI_STORE, gu[:x.shape[0]]), True, out)
        key = (W.device, W.N * W.K)
        buf = _dequant_scratch.get(key)
        if buf is None:
            buf = torch.empty(W.N * W.K, dtype=torch.bfloat16, device=W.device)
            _dequant_scratch[key] = buf
        return _plain_linear(x, planar_dequant(W, buf.view(W.N, W.K)), epi, out, resid)
    if isinstance(W, QuantWeight):
        if x.shape[0] <= 4:
            return quant_gemv(x, W, epi, out, resid)
        if x.shape[0] <= 128 and QUANT_FUSED_GEMM and epi in (EPI_STORE, EPI_F32, EPI_RESID, EPI_SWIGLU):
            return quant_gemm_skinny(x, W, epi, out, resid)
        key = (W.device, W.N * W.K)
        buf = _dequant_scratch.get(key)
        if buf is None:
            buf = torch.empty(W.N * W.K, dtype=torch.bfloat16, device=W.device)
            _dequant_scratch[key] = buf
        return _plain_linear(x, quant_dequant(W, buf.view(W.N, W.K)), epi, out, resid)
    return _plain_linear(x, W, epi, out, resid)
