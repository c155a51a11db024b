"""Native inner loops of the host evaluator (``csrc/host/oracle_ops.cpp``): contractions over block-quantised weights
decoded inside the product, the two scan recurrences and the rank-to-ids step.  ``EvalOptions(native=True)`` routes the
evaluator through them; the NumPy paths stay the definition they are checked against (``tests/test_oracle_native.py``)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import numpy as np

from ..ops._lib import host
from ..quant.formats import descriptor


def _lib():
    lib = host()
    if not getattr(lib, "_oracle_bound", False):
        lib.poot_host_packed_matmul.argtypes = [c_int, c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_int]
        lib.poot_host_delta_rule.argtypes = [c_void_p] * 4 + [c_int] + [c_void_p] * 3 + [c_int] * 4
        lib.poot_host_ssd.argtypes = [c_void_p] * 8 + [c_int] * 5
        lib.poot_host_arg_top_k.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p]
        lib._oracle_bound = True
    return lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def packed_matmul(x: np.ndarray, packed: np.ndarray, fmt: str, shape, narrow: bool, threads: int = 0) -> np.ndarray:
    """``x[..., K] @ W^T`` for ``W[N, K]`` stored in the block format ``fmt``, decoded row by row inside the product."""
    N, K = shape
    d = descriptor(fmt)
    lead = x.shape[:-1]
    x2 = _f32(x).reshape(-1, K)
    raw = np.ascontiguousarray(packed).view(np.uint8).reshape(-1)
    out = np.empty((x2.shape[0], N), np.float32)
    rc = _lib().poot_host_packed_matmul(d.ggml_type, raw.ctypes.data, N, K, x2.ctypes.data, x2.shape[0], out.ctypes.data, int(narrow), threads)
    if rc != 0:
        raise ValueError(f"{fmt}: the native contraction refused the weight ({rc})")
    return out.reshape(lead + (N,))


def scan(family: str, ins, threads: int = 0) -> np.ndarray:
    """The scan equation's packed result ``[1, H, L + S, W]`` (sequence rows, then the carried state)."""
    if family == "delta_rule":
        q, k, v, g, beta, s = (_f32(a[0]) for a in ins)
        H, L, D = q.shape
        state, y = s.copy(), np.empty((H, L, D), np.float32)
        _lib().poot_host_delta_rule(q.ctypes.data, k.ctypes.data, v.ctypes.data, g.ctypes.data, g.shape[-1], beta.ctypes.data,
                                    state.ctypes.data, y.ctypes.data, H, L, D, threads)
        return np.concatenate([y, state], 1)[None]
    x, b, c, delta, a, d, h = (_f32(z[0]) for z in ins)
    H, L, P = x.shape
    N = b.shape[-1]
    state, y = h.copy(), np.empty((H, L, P), np.float32)
    _lib().poot_host_ssd(x.ctypes.data, b.ctypes.data, c.ctypes.data, delta.ctypes.data, a.ctypes.data, d.ctypes.data,
                         state.ctypes.data, y.ctypes.data, H, L, P, N, threads)
    return np.concatenate([y, state], 1)[None]


def arg_top_k(rank: np.ndarray, k: int) -> np.ndarray:
    r = np.ascontiguousarray(rank, dtype=np.int32)
    ids = np.empty((r.shape[0], k), np.int32)
    _lib().poot_host_arg_top_k(r.ctypes.data, r.shape[0], r.shape[1], k, ids.ctypes.data)
    return ids
