"""Shape and dtype inference of every op (the reference's ``OpKind::infer``, crates/poot-graph-ir/src/op.rs:1633-2520)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

from ..tensor import DType
from .graph import BINARY, COMPOSITES, UNARY, GraphError, TensorType

I32 = DType.I32
F32 = DType.F32


def broadcast_shapes(a: Sequence[int], b: Sequence[int]) -> tuple:
    out = []
    ra, rb = list(reversed(a)), list(reversed(b))
    for i in range(max(len(ra), len(rb))):
        x = ra[i] if i < len(ra) else 1
        y = rb[i] if i < len(rb) else 1
        if x != y and x != 1 and y != 1:
            raise GraphError(f"shapes {tuple(a)} and {tuple(b)} do not broadcast")
        out.append(max(x, y))
    return tuple(reversed(out))


def _axis(ax: int, rank: int) -> int:
    if ax < 0:
        ax += rank
    if not 0 <= ax < rank:
        raise GraphError(f"axis {ax} out of range for rank {rank}")
    return ax


def infer(op: str, attrs: Dict[str, Any], ins: List[TensorType], body=None) -> List[TensorType]:
    if op in UNARY:
        (x,) = ins
        if op in ("not", "clz") and not (x.dtype.is_int or x.dtype == DType.BOOL):
            raise GraphError(f"{op} needs an integer operand, got {x.dtype}")
        return [x]
    if op in BINARY:
        a, b = ins
        if a.dtype != b.dtype:
            raise GraphError(f"{op}: operand dtypes differ ({a.dtype} vs {b.dtype})")
        if op in ("geu", "remu", "and", "or", "xor", "shl", "shr") and not a.dtype.is_int:
            raise GraphError(f"{op} needs integer operands")
        out_dtype = I32 if op in ("ge", "geu") else a.dtype   # comparisons yield a 0/1 I32 predicate
        return [TensorType(broadcast_shapes(a.shape, b.shape), out_dtype)]
    if op == "select":
        c, t, f = ins
        if t.dtype != f.dtype:
            raise GraphError("select: branch dtypes differ")
        return [TensorType(broadcast_shapes(c.shape, broadcast_shapes(t.shape, f.shape)), t.dtype)]
    if op == "reduce":
        (x,) = ins
        ax = _axis(attrs["axis"], x.rank)
        if attrs.get("kind", "sum") not in ("sum", "max"):
            raise GraphError("reduce kind must be sum or max")
        shape = list(x.shape)
        if attrs.get("keepdim", False):
            shape[ax] = 1
        else:
            del shape[ax]
        return [TensorType(tuple(shape), x.dtype)]
    if op == "broadcast":
        (x,) = ins
        shape = tuple(attrs["shape"])
        if broadcast_shapes(x.shape, shape) != shape:
            raise GraphError(f"cannot broadcast {x.shape} to {shape}")
        return [TensorType(shape, x.dtype)]
    if op == "cast":
        (x,) = ins
        return [TensorType(x.shape, attrs["dtype"])]
    if op == "reshape":
        (x,) = ins
        shape = tuple(attrs["shape"])
        n = 1
        for s in shape:
            n *= s
        if n != x.numel:
            raise GraphError(f"reshape {x.shape} -> {shape} changes the element count")
        return [TensorType(shape, x.dtype)]
    if op == "transpose":
        (x,) = ins
        perm = tuple(attrs["perm"])
        if sorted(perm) != list(range(x.rank)):
            raise GraphError(f"bad permutation {perm}")
        return [TensorType(tuple(x.shape[p] for p in perm), x.dtype)]
    if op == "slice":
        (x,) = ins
        starts, sizes = attrs["starts"], attrs["sizes"]
        if len(starts) != x.rank or len(sizes) != x.rank:
            raise GraphError("slice: starts/sizes must cover every axis")
        for s, n, d in zip(starts, sizes, x.shape):
            if s < 0 or n < 0 or s + n > d:
                raise GraphError(f"slice [{s}:{s + n}] out of bounds for extent {d}")
        return [TensorType(tuple(sizes), x.dtype)]
    if op == "concat":
        ax = _axis(attrs["axis"], ins[0].rank)
        shape = list(ins[0].shape)
        for t in ins[1:]:
            if t.dtype != ins[0].dtype or t.rank != ins[0].rank:
                raise GraphError("concat: operands differ in dtype or rank")
            for i, (p, q) in enumerate(zip(shape, t.shape)):
                if i != ax and p != q:
                    raise GraphError("concat: off-axis extents differ")
            shape[ax] += t.shape[ax]
        return [TensorType(tuple(shape), ins[0].dtype)]
    if op == "iota":
        shape = tuple(attrs["shape"])
        _axis(attrs["axis"], len(shape))
        return [TensorType(shape, attrs.get("dtype", I32))]
    if op == "gather":
        x, idx = ins
        if idx.dtype != I32:
            raise GraphError("gather indices must be I32")
        ax = _axis(attrs.get("axis", 0), x.rank)
        return [TensorType(tuple(x.shape[:ax]) + tuple(idx.shape) + tuple(x.shape[ax + 1:]), x.dtype)]
    if op == "scatter_update":
        x, idx, upd = ins
        if idx.dtype != I32 or idx.rank != 1:
            raise GraphError("scatter_update: indices must be rank-1 I32")
        if upd.shape != (idx.shape[0],) + tuple(x.shape[1:]):
            raise GraphError(f"scatter_update: update shape {upd.shape} does not match rows of {x.shape}")
        return [TensorType(x.shape, x.dtype)]
    if op == "dynamic_update_slice":
        x, upd, start = ins
        ax = _axis(attrs["axis"], x.rank)
        if upd.rank != x.rank or upd.shape[ax] > x.shape[ax]:
            raise GraphError("dynamic_update_slice: update does not fit")
        return [x]
    if op == "matmul":
        a, b = ins[0], ins[1]
        if a.rank < 2 or b.rank < 2 or a.shape[-1] != b.shape[-2]:
            raise GraphError(f"matmul: {a.shape} x {b.shape}")
        batch = broadcast_shapes(a.shape[:-2], b.shape[:-2])
        return [TensorType(batch + (a.shape[-2], b.shape[-1]), attrs.get("out_dtype", F32))]
    if op == "indexed_matmul":
        x, w, idx = ins   # x [M,K], w [E,K,N], idx [M]
        if w.rank != 3 or x.shape[-1] != w.shape[1] or idx.shape != (x.shape[0],):
            raise GraphError(f"indexed_matmul: {x.shape} {w.shape} {idx.shape}")
        return [TensorType((x.shape[0], w.shape[2]), attrs.get("out_dtype", F32))]
    if op == "packed_dequant":
        (x,) = ins
        return [TensorType(tuple(attrs["shape"]), F32)]
    if op == "arg_top_k":
        (rank,) = ins     # stable descending rank [rows, E] -> ids [rows, k]
        return [TensorType((rank.shape[0], attrs["k"]), I32)]
    if op == "scan":
        fam = attrs.get("family")
        first = ins[0]
        if fam not in ("delta_rule", "ssd") or first.rank != 4 or first.shape[0] != 1 or any(t.dtype != F32 for t in ins):
            raise GraphError(f"scan: family {fam!r}, lead operand {first.shape}")
        _, h, l, w = first.shape
        if fam == "delta_rule":
            # the log decay is one value per head and token, or one per key channel (a row of the state each)
            decay = (1, h, l, w) if len(ins) > 3 and tuple(ins[3].shape) == (1, h, l, w) else (1, h, l, 1)
            want = [(1, h, l, w), (1, h, l, w), (1, h, l, w), decay, (1, h, l, 1), (1, h, w, w)]
            rows = w
        else:
            n = ins[1].shape[3] if ins[1].rank == 4 else 0
            want = [(1, h, l, w), (1, h, l, n), (1, h, l, n), (1, h, l, 1), (1, h, 1, 1), (1, h, 1, 1), (1, h, n, w)]
            rows = n
        if len(ins) != len(want) or any(tuple(t.shape) != s_ for t, s_ in zip(ins, want)) or rows == 0:
            raise GraphError(f"scan {fam}: operands {[tuple(t.shape) for t in ins]}, expected {want}")
        if tuple(attrs["shape"]) != (1, h, l + rows, w):
            raise GraphError("scan: packed shape does not match the operands")
        return [TensorType((1, h, l + rows, w), F32)]
    if op == "ngram_hash":
        (win,) = ins
        ctx, per = attrs["context"], attrs["heads_per_order"]
        heads = ctx * per
        if win.dtype != I32 or win.rank != 1 or win.shape[0] <= ctx or ctx not in (1, 2) or per < 1:
            raise GraphError(f"ngram_hash: window {win.shape} {win.dtype}, context {ctx}, {per} heads per order")
        if len(attrs["multipliers"]) != ctx + 1 or len(attrs["primes"]) != heads or len(attrs["offsets"]) != heads:
            raise GraphError("ngram_hash: one multiplier per n-gram position and one prime / offset per head")
        if any(not 1 < p_ < 2 ** 32 for p_ in attrs["primes"]):
            raise GraphError("ngram_hash: every head's modulus fits an unsigned 32-bit word")
        return [TensorType((win.shape[0] - ctx, heads), I32)]
    if op == "random_uniform":
        (seed,) = ins
        return [TensorType(tuple(seed.shape) + (attrs["cols"],), F32)]
    if op == "sample_token":
        logits = ins[0]
        return [TensorType(tuple(logits.shape[:-1]) + (2,), I32)]
    if op == "all_reduce":
        return [ins[0]]
    if op == "all_gather":
        (x,) = ins
        ax = _axis(attrs["axis"], x.rank)
        shape = list(x.shape)
        shape[ax] *= attrs["world"]
        return [TensorType(tuple(shape), x.dtype)]
    if op == "all_to_all":
        return [TensorType(tuple(attrs.get("shape", ins[0].shape)), ins[0].dtype)]
    if op in COMPOSITES:
        if body is None:
            raise GraphError(f"composite {op} carries no decomposition")
        if len(body.inputs) != len(ins):
            raise GraphError(f"composite {op}: {len(ins)} operands for a body of {len(body.inputs)} inputs")
        for k, (bi, t) in enumerate(zip(body.inputs, ins)):
            if body.types[bi.value] != t:
                raise GraphError(f"composite {op}: operand {k} is {t}, body expects {body.types[bi.value]}")
        return [body.types[o.value] for o in body.outputs]
    raise GraphError(f"no inference rule for {op!r}")
