"""The graph IR evaluated with tensors on a device: the general executor behind ``--backend graph``.

Every family's tracer emits the same primitive equations, so one evaluator runs every family wherever tensors live.
The hand-written engine (``runtime/engine.py``) is the fast path for the families it has programs for; this executor is
the general path for the rest (Gemma 4, GLM-5.3-Flash, DeepSeek-V4, Qwen3.8-Flash-Next) and the device-side twin of the
CPU oracle (``eval.py`` beside this file): same equations, same semantics, f32 arithmetic, one library or extension launch per
equation.  It is launch-bound by construction - the point is that the family RUNS on the device with its weights and
its paged pools resident there, not that it is fast (crates/poot-executor walks a planned program the same way, with a
generated kernel where this file has a tensor op).

Differences from the oracle that follow from staying on the device:

* ``scatter_update`` into a paged pool writes in place when the pool is one of the step's state tensors (the tracer never
  reads the old pool after the write); the skipped slots (``-1``) go to a spare row the state tensors carry at their end,
  so no host decision is taken per step;
* index and range checks of the oracle (duplicate slots, ids out of range) are the driver's validation gate's business and
  are not repeated here;
* ``ngram_hash`` runs the extension kernel on a CUDA device and 64-bit host arithmetic elsewhere.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

from ..ir.graph import Eqn, Graph
from ..tensor import DType

_T = {DType.F32: torch.float32, DType.BF16: torch.bfloat16, DType.F16: torch.float16, DType.I32: torch.int32, DType.U8: torch.uint8}


def torch_dtype(dt: DType):
    try:
        return _T[dt]
    except KeyError:
        raise ValueError(f"the device evaluator has no tensor type for {dt}")


class StateTensor:
    """A step's state on the device with one spare row at its end (where skipped writes land)."""

    def __init__(self, shape, dtype, device):
        self.storage = torch.zeros((shape[0] + 1,) + tuple(shape[1:]), dtype=dtype, device=device)
        self.view = self.storage[:shape[0]]


def _erf(x):
    return torch.erf(x)


def eval_graph_torch(g: Graph, inputs: Dict[str, torch.Tensor], device, in_place: Optional[Dict[int, StateTensor]] = None,
                     donated=None) -> Dict[str, torch.Tensor]:
    """Evaluate ``g`` over ``inputs`` (tensors on ``device``, computed constants are materialised here); returns the
    outputs by name.  ``in_place``: graph value -> state tensor behind it; ``donated``: indices of the equations the state
    commit plan lets overwrite their state in place (``plan/state_commit.py``; ``None``: every update of a state tensor)."""
    from .eval import computed_constant
    env: Dict[int, torch.Tensor] = {}
    for i in g.inputs:
        ty = g.types[i.value]
        if i.storage == "computed" and i.name not in inputs:
            key = (i.computed[0], tuple(map(str, i.computed[1])), tuple(ty.shape), str(device))
            t = _CONST_CACHE.get(key)
            if t is None:
                t = torch.from_numpy(np.ascontiguousarray(computed_constant(i.computed[0], i.computed[1], ty.shape, ty.dtype))).to(device)
                _CONST_CACHE[key] = t
            env[i.value] = t
            continue
        a = inputs[i.name]
        if tuple(a.shape) != tuple(ty.shape):
            raise ValueError(f"input {i.name!r}: shape {tuple(a.shape)}, graph expects {ty.shape}")
        env[i.value] = a
    owner = dict(in_place or {})
    for k, e in enumerate(g.eqns):
        ins = [env[v] for v in e.inputs]
        if e.op == "cast" and e.inputs[0] in owner and ins[0].dtype == torch_dtype(e.attrs["dtype"]):
            owner[e.outputs[0]] = owner[e.inputs[0]]          # a cast to the pool's own type is the pool
        outs = _eval(g, e, ins, device, owner if (donated is None or k in donated) else {})
        for o, val in zip(e.outputs, outs):
            env[o] = val
    return {o.name: env[o.value] for o in g.outputs}


_CONST_CACHE: Dict[tuple, torch.Tensor] = {}


def _eval(g: Graph, e: Eqn, ins: List[torch.Tensor], device, owner) -> List[torch.Tensor]:
    op, at = e.op, e.attrs
    if op == "neg": return [-ins[0]]
    if op == "exp": return [torch.exp(ins[0])]
    if op == "log": return [torch.log(ins[0])]
    if op == "sqrt": return [torch.sqrt(ins[0])]
    if op == "recip": return [1.0 / ins[0]]
    if op == "tanh": return [torch.tanh(ins[0])]
    if op == "erf": return [_erf(ins[0])]
    if op == "not": return [torch.bitwise_not(ins[0])]
    if op in ("add", "sub", "mul"):
        return [{"add": torch.add, "sub": torch.sub, "mul": torch.mul}[op](ins[0], ins[1])]
    if op == "div":
        a, b = ins
        if not a.dtype.is_floating_point:
            return [torch.div(a, torch.where(b == 0, torch.ones_like(b), b), rounding_mode="floor")]
        return [a / b]
    if op == "max":                                   # max-number: a NaN operand is ignored
        return [torch.fmax(ins[0], ins[1])]
    if op == "ge": return [(ins[0] >= ins[1]).to(torch.int32)]
    if op in ("and", "or", "xor"):
        return [{"and": torch.bitwise_and, "or": torch.bitwise_or, "xor": torch.bitwise_xor}[op](ins[0], ins[1])]
    if op in ("geu", "remu", "shl", "shr", "clz"):
        a = ins[0].to(torch.int64) & 0xFFFFFFFF
        if op == "clz":
            r = torch.where(a == 0, torch.full_like(a, 32), 31 - torch.floor(torch.log2(a.clamp(min=1).to(torch.float64))).to(torch.int64))
            return [r.to(ins[0].dtype)]
        b = ins[1].to(torch.int64) & 0xFFFFFFFF
        if op == "geu": return [(a >= b).to(torch.int32)]
        if op == "remu": r = a % torch.where(b == 0, torch.ones_like(b), b)
        elif op == "shl": r = (a << (b & 31)) & 0xFFFFFFFF
        else: r = a >> (b & 31)
        r = torch.where(r >= 2 ** 31, r - 2 ** 32, r)
        return [r.to(ins[0].dtype)]
    if op == "select":
        return [torch.where(ins[0] != 0, ins[1], ins[2])]
    if op == "reduce":
        x, ax, keep = ins[0], at["axis"], at.get("keepdim", False)
        if at.get("kind", "sum") == "sum":
            return [x.sum(dim=ax, keepdim=keep, dtype=x.dtype)]
        if x.dtype.is_floating_point:                 # max-number reduce
            return [torch.nan_to_num(x, nan=float("-inf")).amax(dim=ax, keepdim=keep)]
        return [x.amax(dim=ax, keepdim=keep)]
    if op == "broadcast": return [ins[0].expand(tuple(at["shape"]))]
    if op == "cast":
        dt, x = at["dtype"], ins[0]
        if dt.is_float:
            return [x.to(torch_dtype(dt))]
        if x.dtype.is_floating_point:
            x = torch.trunc(torch.nan_to_num(x, nan=0.0, posinf=2147483647.0, neginf=-2147483648.0))
        return [x.to(torch_dtype(dt))]
    if op == "reshape": return [ins[0].reshape(tuple(at["shape"]))]
    if op == "transpose": return [ins[0].permute(tuple(at["perm"]))]
    if op == "slice":
        x = ins[0]
        for ax, (s, n) in enumerate(zip(at["starts"], at["sizes"])):
            if s != 0 or n != x.shape[ax]:
                x = x.narrow(ax, s, n)
        return [x]
    if op == "concat": return [torch.cat(ins, dim=at["axis"])]
    if op == "iota":
        shape, ax = tuple(at["shape"]), at["axis"]
        v = torch.arange(shape[ax], dtype=torch_dtype(at.get("dtype", DType.I32)), device=device)
        view = [1] * len(shape)
        view[ax] = shape[ax]
        return [v.reshape(view).expand(shape)]
    if op == "gather":
        x, idx = ins
        ax = at.get("axis", 0)
        return [torch.index_select(x, ax, idx.reshape(-1).to(torch.int64)).reshape(tuple(x.shape[:ax]) + tuple(idx.shape) + tuple(x.shape[ax + 1:]))]
    if op == "scatter_update":
        x, idx, upd = ins
        st = owner.get(e.inputs[0])
        rows = x.shape[0]
        slot = torch.where(idx >= 0, idx, torch.full_like(idx, rows)).to(torch.int64)
        if st is not None and st.view.data_ptr() == x.data_ptr():
            st.storage.index_copy_(0, slot, upd.to(st.storage.dtype))
            owner[e.outputs[0]] = st
            return [st.view]
        out = torch.cat([x, x.new_zeros((1,) + tuple(x.shape[1:]))], 0)
        out.index_copy_(0, slot, upd.to(x.dtype))
        return [out[:rows]]
    if op == "dynamic_update_slice":
        x, upd, start = ins
        ax = at["axis"]
        s = start.reshape(-1)[0].to(torch.int64).clamp(0, x.shape[ax] - upd.shape[ax])
        index = (s + torch.arange(upd.shape[ax], device=device)).to(torch.int64)
        return [x.index_copy(ax, index, upd.to(x.dtype))]
    if op == "matmul":
        a, b = ins
        return [torch.matmul(a.to(torch.float32), b.to(torch.float32))]
    if op == "indexed_matmul":
        x, w, idx = ins
        return [torch.bmm(x.unsqueeze(1), w.index_select(0, idx.to(torch.int64))).squeeze(1)]
    if op == "packed_dequant":
        from ..quant import codec
        return [torch.from_numpy(codec.dequantize(at["format"], ins[0].cpu().numpy(), at["shape"])).to(device)]
    if op == "arg_top_k":
        rank, k = ins[0], at["k"]
        ids = torch.zeros((rank.shape[0], k + 1), dtype=torch.int32, device=device)
        place = torch.where((rank >= 0) & (rank < k), rank, torch.full_like(rank, k)).to(torch.int64)
        src = torch.arange(rank.shape[1], dtype=torch.int32, device=device).expand(rank.shape[0], -1)
        ids.scatter_(1, place, src)
        return [ids[:, :k].contiguous()]
    if op == "scan":
        return [_scan(at["family"], ins)]
    if op == "ngram_hash":
        return [_ngram_hash(at, ins[0], device)]
    if op in ("all_reduce", "all_gather") and at.get("world", 1) == 1:
        return [ins[0]]
    if e.body is not None:
        sub = {bi.name: v for bi, v in zip(e.body.inputs, ins)}
        out = eval_graph_torch(e.body, sub, device)
        return [out[o.name] for o in e.body.outputs]
    raise NotImplementedError(f"the device evaluator has no rule for {op!r}")


def _scan(family: str, ins) -> torch.Tensor:
    """Both recurrences token by token over tensors (heads vectorised)."""
    if family == "delta_rule":
        q, k, v, g, beta, s = (x[0].to(torch.float32) for x in ins)          # [H, L, D] ...; s [H, D, D]
        H, L, D = q.shape
        s = s.clone()
        ys = []
        for t in range(L):
            s = s * torch.exp(g[:, t]).unsqueeze(-1)
            kv = torch.einsum("hk,hkv->hv", k[:, t], s)
            d = (v[:, t] - kv) * beta[:, t]
            s = s + k[:, t].unsqueeze(-1) * d.unsqueeze(1)
            ys.append(torch.einsum("hk,hkv->hv", q[:, t], s))
        return torch.cat([torch.stack(ys, 1), s], 1).unsqueeze(0)
    x, b, c, delta, a, d, h = (z[0].to(torch.float32) for z in ins)
    H, L, P = x.shape
    h = h.clone()
    ys = []
    for t in range(L):
        dt = delta[:, t]
        h = torch.exp(dt * a[:, 0]).unsqueeze(-1) * h + (dt * b[:, t]).unsqueeze(-1) * x[:, t].unsqueeze(1)
        ys.append(torch.einsum("hn,hnp->hp", c[:, t], h) + d[:, 0] * x[:, t])
    return torch.cat([torch.stack(ys, 1), h], 1).unsqueeze(0)


def _ngram_hash(at, win: torch.Tensor, device) -> torch.Tensor:
    ctx, per, eos = at["context"], at["heads_per_order"], at["eos"]
    heads = ctx * per
    t = win.shape[0] - ctx
    if win.is_cuda:
        from ..ops import cuda_ops as K
        mult = torch.tensor([m - (1 << 64) if m >= 1 << 63 else m for m in at["multipliers"]], dtype=torch.int64, device=device)
        primes = torch.tensor([p - (1 << 32) if p >= 1 << 31 else p for p in at["primes"]], dtype=torch.int32, device=device)
        offsets = torch.tensor(at["offsets"], dtype=torch.int32, device=device)
        # the kernel reads the context from a carried history (xor-ed with eos) and the tokens from the step
        hist = (win[:ctx] ^ eos).reshape(1, ctx).contiguous()
        ids = torch.zeros(t, heads, dtype=torch.int32, device=device)
        segs = torch.tensor([[0, t, 0, 1]], dtype=torch.int32, device=device)            # position 1: the history is read
        K.ngram_hash(win[ctx:].contiguous(), hist, segs, mult, primes, offsets, per, eos, 1 << 30, ids)
        return ids
    w = win.cpu().numpy().astype(np.int64).astype(np.uint64)
    m = [np.uint64(v & 0xFFFFFFFFFFFFFFFF) for v in at["multipliers"]]
    s0, s1 = w[ctx:ctx + t], w[ctx - 1:ctx - 1 + t]
    with np.errstate(over="ignore"):
        mix = [(s0 * m[0]) ^ (s1 * m[1])]
        if ctx == 2:
            s2 = np.where(s1 == np.uint64(eos), np.uint64(eos), w[0:t])
            mix.append(mix[0] ^ (s2 * m[2]))
    cols = [(mix[h // per] % np.uint64(at["primes"][h])).astype(np.int64) + at["offsets"][h] for h in range(heads)]
    return torch.from_numpy(np.stack(cols, 1).astype(np.int32)).to(device)
