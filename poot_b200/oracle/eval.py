"""CPU eager oracle: one walk over a graph, the correctness reference of every kernel and every pass.

Counterpart of the reference's ``poot-eval`` (crates/poot-eval/src/walk.rs:89-140,432-566): float values are held
in f32 (f64 for F64), narrow storage dtypes (bf16, f16, e4m3) are exact round trips through their bit patterns,
integers keep their own lanes; composites are evaluated through their decomposition; ``all_reduce`` is the
identity at world 1 (ops/collective.rs:12-34) and, on a rank walk, the left fold of the ranks' partials in rank
order.  Heavy inner loops (contractions, packed dequantisation) call the C++ host library when it is present.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence

import numpy as np

from ..ir.graph import Eqn, Graph, GraphError
from ..tensor import DType, round_bf16, round_f16, e4m3_bits_to_f32, f32_to_e4m3_bits
from . import sampling as S


class EvalError(RuntimeError):
    pass


@dataclass
class EvalOptions:
    matmul_precision: Optional[str] = None     # override every matmul's precision attr: exact | narrow | split
    narrow_dtype: DType = DType.BF16
    collectives: Optional[Callable[[str, Eqn, List[np.ndarray]], np.ndarray]] = None   # rank-walk hook
    keep_intermediates: bool = False
    native: bool = False          # contractions over packed weights, scans and rank-to-ids through the C++ loops (oracle/native.py)


@dataclass
class Evaluation:
    outputs: Dict[str, np.ndarray]
    values: Dict[int, np.ndarray] = field(default_factory=dict)
    equations: int = 0


def _np_dtype(dt: DType):
    if dt in (DType.F32, DType.BF16, DType.F16, DType.E4M3FN, DType.E8M0):
        return np.float32
    if dt == DType.F64:
        return np.float64
    if dt == DType.BOOL:
        return np.int32
    return dt.storage_numpy


def round_to(x: np.ndarray, dt: DType) -> np.ndarray:
    if dt == DType.BF16:
        return round_bf16(x)
    if dt == DType.F16:
        return round_f16(x)
    if dt == DType.E4M3FN:
        return e4m3_bits_to_f32(f32_to_e4m3_bits(x))
    return x


def _erf(x: np.ndarray) -> np.ndarray:
    return np.vectorize(math.erf, otypes=[np.float32])(x).astype(np.float32)


def _narrow(x: np.ndarray, precision: str, dt: DType) -> np.ndarray:
    if precision == "exact" or x.dtype != np.float32:
        return x
    return round_to(x, dt)


def _matmul(a: np.ndarray, b: np.ndarray, precision: str, dt: DType) -> np.ndarray:
    """Exact: f32 operands; narrow: operands rounded to bf16/f16; split: hi + lo halves of each operand (three
    products), all accumulated in f32 (semantics of website/docs/architecture/graph-ir.mdx:128-147)."""
    if precision == "split":
        ah, bh = round_to(a, dt), round_to(b, dt)
        al, bl = round_to(a - ah, dt), round_to(b - bh, dt)
        return (np.matmul(ah, bh) + np.matmul(ah, bl) + np.matmul(al, bh)).astype(np.float32)
    return np.matmul(_narrow(a, precision, dt), _narrow(b, precision, dt)).astype(np.float32)


def computed_constant(kind: str, params: tuple, shape, dtype: DType) -> np.ndarray:
    if kind == "literal":
        return np.array(params[0], dtype=_np_dtype(dtype)).reshape(shape)
    if kind in ("rope_cos", "rope_sin"):
        from ..runtime.rope import inv_frequencies
        dim, theta, positions = params[0], params[1], params[2]
        scaling = params[3] if len(params) > 3 else None
        inv, att = inv_frequencies(dim, theta, scaling, positions)
        ang = np.arange(positions, dtype=np.float64)[:, None] * inv[None, :]
        t = (np.cos(ang) if kind == "rope_cos" else np.sin(ang)) * att
        return np.concatenate([t, t], axis=1).astype(np.float32).reshape(shape)   # duplicated halves
    if kind == "iota":                                     # a folded ``iota`` equation: counts along one axis
        ax = params[0]
        view = [1] * len(shape)
        view[ax] = shape[ax]
        return np.broadcast_to(np.arange(shape[ax], dtype=_np_dtype(dtype)).reshape(view), shape).copy()
    raise EvalError(f"unknown computed constant {kind!r}")


def _scan(family: str, ins) -> np.ndarray:
    """The two recurrences, one token at a time, vectorised over heads; f32 throughout
    (crates/poot-graph-ir/src/ops/ssm.rs: gated delta rule and the Mamba2 SSD)."""
    if family == "delta_rule":
        q, k, v, g, beta, s = (x[0] for x in ins)          # [H,L,D] ... s [H,D,D]
        H, L, D = q.shape
        s = s.copy()
        y = np.zeros((H, L, D), np.float32)
        for t in range(L):
            s = s * np.exp(g[:, t])[:, :, None]                 # g [H,1]: the whole state; [H,D]: row i by exp(g[i])
            kv = np.einsum("hk,hkv->hv", k[:, t], s)
            d = (v[:, t] - kv) * beta[:, t]
            s = (s + k[:, t][:, :, None] * d[:, None, :]).astype(np.float32)
            y[:, t] = np.einsum("hk,hkv->hv", q[:, t], s)
        return np.concatenate([y, s], 1)[None].astype(np.float32)
    x, b, c, delta, a, d, h = (z[0] for z in ins)            # x [H,L,P], b/c [H,L,N], delta [H,L,1], a/d [H,1,1], h [H,N,P]
    H, L, P = x.shape
    h = h.copy()
    y = np.zeros((H, L, P), np.float32)
    for t in range(L):
        dt = delta[:, t]                                      # [H,1]
        h = (np.exp(dt * a[:, 0])[:, :, None] * h + (dt * b[:, t])[:, :, None] * x[:, t][:, None, :]).astype(np.float32)
        y[:, t] = np.einsum("hn,hnp->hp", c[:, t], h) + d[:, 0] * x[:, t]
    return np.concatenate([y, h], 1)[None].astype(np.float32)


def eval_graph(g: Graph, inputs: Dict[str, np.ndarray], options: Optional[EvalOptions] = None) -> Evaluation:
    opt = options or EvalOptions()
    env: Dict[int, np.ndarray] = {}
    for i in g.inputs:
        ty = g.types[i.value]
        if i.storage == "computed" and i.name not in inputs:
            env[i.value] = computed_constant(i.computed[0], i.computed[1], ty.shape, ty.dtype)
            continue
        if i.name not in inputs:
            raise EvalError(f"missing input {i.name!r}")
        a = np.asarray(inputs[i.name])
        if tuple(a.shape) != tuple(ty.shape):
            raise EvalError(f"input {i.name!r}: shape {a.shape}, graph expects {ty.shape}")
        a = a.astype(_np_dtype(ty.dtype), copy=False)
        if i.range is not None and a.size and (a.min() < i.range[0] or a.max() > i.range[1]):
            raise EvalError(f"input {i.name!r} outside its declared range {i.range}")
        env[i.value] = round_to(a, ty.dtype) if ty.dtype.is_float else a
    n = 0
    for e in g.eqns:
        ins = [env[v] for v in e.inputs]
        outs = _eval_eqn(g, e, ins, opt)
        for o, val in zip(e.outputs, outs):
            ty = g.types[o]
            if tuple(val.shape) != tuple(ty.shape):
                raise EvalError(f"{e.op}: produced {val.shape}, inferred {ty.shape}")
            env[o] = val
        n += 1
    outs = {o.name: env[o.value] for o in g.outputs}
    return Evaluation(outs, env if opt.keep_intermediates else {}, n)


def _eval_eqn(g: Graph, e: Eqn, ins: List[np.ndarray], opt: EvalOptions) -> List[np.ndarray]:
    op, at = e.op, e.attrs
    out_ty = g.types[e.outputs[0]]
    with np.errstate(all="ignore"):
        if op == "neg": return [-ins[0]]
        if op == "exp": return [np.exp(ins[0]).astype(ins[0].dtype)]
        if op == "log": return [np.log(ins[0]).astype(ins[0].dtype)]
        if op == "sqrt": return [np.sqrt(ins[0]).astype(ins[0].dtype)]
        if op == "recip": return [(1.0 / ins[0]).astype(ins[0].dtype)]
        if op == "tanh": return [np.tanh(ins[0]).astype(ins[0].dtype)]
        if op == "erf": return [_erf(ins[0])]
        if op == "not": return [np.bitwise_not(ins[0])]
        if op == "clz":
            x = ins[0].astype(np.uint32)
            return [np.where(x == 0, 32, 31 - np.floor(np.log2(np.maximum(x, 1))).astype(np.int32)).astype(ins[0].dtype)]
        if op in ("add", "sub", "mul", "div"):
            a, b = ins
            r = {"add": np.add, "sub": np.subtract, "mul": np.multiply, "div": np.divide}[op](a, b)
            if a.dtype.kind in "iu" and op == "div":
                r = np.floor_divide(a, np.where(b == 0, 1, b))
            return [r.astype(a.dtype)]
        if op == "max":                       # max-number: NaN operands are ignored
            return [np.fmax(ins[0], ins[1])]
        if op == "ge": return [(ins[0] >= ins[1]).astype(np.int32)]
        if op == "geu": return [(ins[0].astype(np.uint32) >= ins[1].astype(np.uint32)).astype(np.int32)]
        if op == "remu":
            b = ins[1].astype(np.uint32)
            return [(ins[0].astype(np.uint32) % np.where(b == 0, 1, b)).astype(ins[0].dtype)]
        if op == "and": return [ins[0] & ins[1]]
        if op == "or": return [ins[0] | ins[1]]
        if op == "xor": return [ins[0] ^ ins[1]]
        if op == "shl": return [(ins[0].astype(np.uint32) << (ins[1].astype(np.uint32) & 31)).astype(ins[0].dtype)]
        if op == "shr": return [(ins[0].astype(np.uint32) >> (ins[1].astype(np.uint32) & 31)).astype(ins[0].dtype)]
        if op == "select":
            c, t, f = ins
            return [np.where(c != 0, t, f)]
        if op == "reduce":
            fn = np.sum if at.get("kind", "sum") == "sum" else np.max
            x = ins[0]
            if at.get("kind") == "max" and x.dtype.kind == "f":
                r = np.fmax.reduce(x, axis=at["axis"], keepdims=at.get("keepdim", False), initial=-np.inf)
            else:
                r = fn(x, axis=at["axis"], keepdims=at.get("keepdim", False))
            return [np.asarray(r).astype(x.dtype)]
        if op == "broadcast": return [np.broadcast_to(ins[0], at["shape"])]
        if op == "cast":
            dt = at["dtype"]
            x = ins[0]
            if dt.is_float:
                return [round_to(x.astype(_np_dtype(dt)), dt)]
            if x.dtype.kind == "f":
                x = np.trunc(np.nan_to_num(x, nan=0.0, posinf=2147483647.0, neginf=-2147483648.0))
            return [x.astype(_np_dtype(dt))]
        if op == "reshape": return [np.reshape(ins[0], at["shape"])]
        if op == "transpose": return [np.transpose(ins[0], at["perm"])]
        if op == "slice":
            sl = tuple(slice(s, s + n) for s, n in zip(at["starts"], at["sizes"]))
            return [ins[0][sl]]
        if op == "concat": return [np.concatenate(ins, axis=at["axis"])]
        if op == "iota":
            shape, ax = at["shape"], at["axis"]
            v = np.arange(shape[ax], dtype=_np_dtype(at.get("dtype", DType.I32)))
            view = [1] * len(shape)
            view[ax] = shape[ax]
            return [np.broadcast_to(v.reshape(view), shape).copy()]
        if op == "gather":
            x, idx = ins
            ax = at.get("axis", 0)
            if idx.size and (idx.min() < 0 or idx.max() >= x.shape[ax]):
                raise EvalError(f"gather index out of range [0, {x.shape[ax]})")
            return [np.take(x, idx, axis=ax)]
        if op == "scatter_update":
            x, idx, upd = ins
            live = idx[idx >= 0]
            if len(set(live.tolist())) != live.size:
                raise EvalError("scatter_update: duplicate write slots")
            if live.size and live.max() >= x.shape[0]:
                raise EvalError("scatter_update: slot out of range")
            out = x.copy()
            out[live] = round_to(upd[idx >= 0], out_ty.dtype)
            return [out]
        if op == "dynamic_update_slice":
            x, upd, start = ins
            ax = at["axis"]
            s = int(np.asarray(start).reshape(-1)[0])
            s = max(0, min(s, x.shape[ax] - upd.shape[ax]))
            out = x.copy()
            sl = [slice(None)] * x.ndim
            sl[ax] = slice(s, s + upd.shape[ax])
            out[tuple(sl)] = round_to(upd, out_ty.dtype)
            return [out]
        if op == "matmul":
            prec = opt.matmul_precision or at.get("precision", "narrow")
            return [_matmul(ins[0], ins[1], prec, opt.narrow_dtype)]
        if op == "indexed_matmul":
            x, w, idx = ins
            prec = opt.matmul_precision or at.get("precision", "narrow")
            if idx.size and (idx.min() < 0 or idx.max() >= w.shape[0]):
                raise EvalError("indexed_matmul: expert id out of range")
            out = np.zeros((x.shape[0], w.shape[2]), dtype=np.float32)
            for ex in np.unique(idx):
                rows = idx == ex
                out[rows] = _matmul(x[rows], w[ex], prec, opt.narrow_dtype)
            return [out]
        if op == "packed_dequant":
            from ..quant import codec
            return [codec.dequantize(at["format"], ins[0], at["shape"])]
        if op == "ngram_hash":
            ctx, per, eos = at["context"], at["heads_per_order"], at["eos"]
            win = ins[0].astype(np.int64).astype(np.uint64)
            t = win.shape[0] - ctx
            m = [np.uint64(v & 0xFFFFFFFFFFFFFFFF) for v in at["multipliers"]]
            s0, s1 = win[ctx:ctx + t], win[ctx - 1:ctx - 1 + t]
            with np.errstate(over="ignore"):
                mix = [(s0 * m[0]) ^ (s1 * m[1])]
                if ctx == 2:
                    s2 = np.where(s1 == np.uint64(eos), np.uint64(eos), win[0:t])
                    mix.append(mix[0] ^ (s2 * m[2]))
            cols = [(mix[h // per] % np.uint64(at["primes"][h])).astype(np.int64) + at["offsets"][h] for h in range(ctx * per)]
            return [np.stack(cols, 1).astype(np.int32)]
        if op == "arg_top_k" and opt.native:
            from . import native
            return [native.arg_top_k(ins[0], at["k"])]
        if op == "arg_top_k":
            rank = ins[0]
            k = at["k"]
            ids = np.zeros((rank.shape[0], k), dtype=np.int32)
            for r in range(rank.shape[0]):
                for ex, rk in enumerate(rank[r]):
                    if 0 <= rk < k:
                        ids[r, rk] = ex
            return [ids]
        if op == "random_uniform":
            seed = ins[0].reshape(-1)
            out = np.stack([S.random_uniform_row(int(s) & 0xFFFFFFFF, at["cols"]) for s in seed])
            return [out.reshape(tuple(ins[0].shape) + (at["cols"],))]
        if op == "sample_token":
            return [_sample_token(at, ins)]
        if op == "all_reduce":
            if opt.collectives is not None:
                return [opt.collectives("all_reduce", e, ins)]
            return [ins[0]]
        if op in ("all_gather", "all_to_all"):
            if opt.collectives is None:
                if op == "all_gather" and at.get("world", 1) == 1:
                    return [ins[0]]
                raise EvalError(f"{op} needs a rank walk (world > 1)")
            return [opt.collectives(op, e, ins)]
        if op == "scan" and opt.native:
            from . import native
            return [native.scan(at["family"], ins)]
        if op == "scan":
            return [_scan(at["family"], [np.asarray(x, np.float32) for x in ins])]
        if opt.native and op == "packed_contraction" and len(ins) == 2:
            # the composite's body is ``matmul(x, transpose(packed_dequant(p)))``: decode inside the product instead
            from . import native
            deq = next(b_ for b_ in e.body.eqns if b_.op == "packed_dequant")
            prec = opt.matmul_precision or at.get("precision", "narrow")
            packed_first = e.body.inputs[0].value == deq.inputs[0]
            x, pk = (ins[1], ins[0]) if packed_first else (ins[0], ins[1])
            if prec in ("exact", "narrow") and opt.narrow_dtype == DType.BF16:
                return [native.packed_matmul(x, pk, at["format"], deq.attrs["shape"], prec == "narrow")]
        if opt.native and op == "packed_row_gather" and len(ins) == 2:
            # only the gathered rows are decoded (the body would expand the whole table first)
            from ..quant import codec
            from ..quant.formats import packed_nbytes
            deq = next(b_ for b_ in e.body.eqns if b_.op == "packed_dequant")
            gat = next(b_ for b_ in e.body.eqns if b_.op == "gather")
            packed_first = e.body.inputs[0].value == deq.inputs[0]
            pk, ids = (ins[0], ins[1]) if packed_first else (ins[1], ins[0])
            N, K = deq.attrs["shape"]
            if gat.attrs.get("axis", 0) == 0 and (ids.size == 0 or (ids.min() >= 0 and ids.max() < N)):
                rows = np.ascontiguousarray(pk).view(np.uint8).reshape(N, packed_nbytes(at["format"], K))[ids.reshape(-1)]
                return [codec.dequantize(at["format"], rows.reshape(-1), (ids.size, K)).reshape(tuple(ids.shape) + (K,))]
        if e.body is not None:
            sub_inputs = {bi.name: v for bi, v in zip(e.body.inputs, ins)}
            ev = eval_graph(e.body, sub_inputs, opt)
            return [ev.outputs[o.name] for o in e.body.outputs]
    raise EvalError(f"no evaluation rule for {op!r}")


def _sample_token(at, ins) -> np.ndarray:
    rule = {"greedy": S.GREEDY, "gumbel": S.GUMBEL, "gumbel_top_k": S.GUMBEL_TOPK,
            "gumbel_top_k_top_p": S.GUMBEL_TOPK_TOPP}[at["rule"]]
    logits = ins[0]
    lead = logits.shape[:-1]
    rows = int(np.prod(lead)) if lead else 1
    L = logits.reshape(rows, logits.shape[-1])
    k = 1
    noise = params = top_k = None
    if at.get("has_noise"):
        noise = ins[k].reshape(rows, -1); k += 1
    if at.get("has_params"):
        params = ins[k].reshape(rows, -1); k += 1
    if at.get("has_top_k"):
        top_k = ins[k].reshape(rows); k += 1
    out = np.zeros((rows, 2), dtype=np.int32)
    for r in range(rows):
        if rule == S.GREEDY:
            out[r] = S.sample_one_row(L[r], None, None, None, None)
        else:
            kk = int(top_k[r]) if (top_k is not None and rule >= S.GUMBEL_TOPK) else None
            tp = float(params[r][3]) if rule >= S.GUMBEL_TOPK_TOPP else None
            out[r] = S.sample_one_row(L[r], noise[r], params[r][:3], kk, tp)
    return out.reshape(tuple(lead) + (2,))
