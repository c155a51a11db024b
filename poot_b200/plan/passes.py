"""The pass pipeline, in the reference's order (crates/poot-graph-plan/src/compile.rs:923-1210):
canonicalize -> cse -> rope_fusion -> flash_attention -> dce -> recognize packed contractions / row gathers ->
fold dense contractions -> fuse contraction epilogues -> fuse (row regions, pointwise regions).

Every rewrite keeps the primitives it folds as the composite's body, so each pass is checked by evaluating the graph
before and after on the CPU oracle: the results must be bit-identical.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Set, Tuple

from ..ir.graph import BINARY, UNARY, Eqn, Graph
from .edit import Decline, fold_region, literal_value

POINTWISE = set(UNARY) | set(BINARY) | {"select", "cast"}
NO_CSE = {"random_uniform", "sample_token", "all_reduce", "all_gather", "all_to_all", "scatter_update",
          "dynamic_update_slice"}


def _replace_uses(g: Graph, rep: Dict[int, int]) -> None:
    if not rep:
        return

    def r(v):
        while v in rep:
            v = rep[v]
        return v
    for e in g.eqns:
        e.inputs = [r(v) for v in e.inputs]
    for o in g.outputs:
        o.value = r(o.value)


def canonicalize(g: Graph) -> int:
    """reshape∘reshape and transpose∘transpose collapse; identity movement disappears.  Returns rewrites made."""
    n = 0
    changed = True
    while changed:
        changed = False
        prod = g.producers()
        rep: Dict[int, int] = {}
        for e in g.eqns:
            if e.op == "reshape":
                src = e.inputs[0]
                if src in prod and g.eqns[prod[src]].op == "reshape":
                    e.inputs = [g.eqns[prod[src]].inputs[0]]
                    changed = True
                    n += 1
                if g.types[e.inputs[0]].shape == tuple(e.attrs["shape"]):
                    rep[e.outputs[0]] = e.inputs[0]
            elif e.op == "transpose":
                src = e.inputs[0]
                if src in prod and g.eqns[prod[src]].op == "transpose":
                    inner = g.eqns[prod[src]]
                    e.attrs = {"perm": tuple(inner.attrs["perm"][p] for p in e.attrs["perm"])}
                    e.inputs = [inner.inputs[0]]
                    changed = True
                    n += 1
                if tuple(e.attrs["perm"]) == tuple(range(len(e.attrs["perm"]))):
                    rep[e.outputs[0]] = e.inputs[0]
            elif e.op == "broadcast" and g.types[e.inputs[0]].shape == tuple(e.attrs["shape"]):
                rep[e.outputs[0]] = e.inputs[0]
        if rep:
            g.eqns = [e for e in g.eqns if e.outputs[0] not in rep]
            _replace_uses(g, rep)
            changed = True
            n += len(rep)
    if n:
        dce(g)          # the inner equations of collapsed chains are dead now
    return n


def cse(g: Graph) -> int:
    seen: Dict[tuple, List[int]] = {}
    rep: Dict[int, int] = {}
    keep: List[Eqn] = []
    for e in g.eqns:
        e.inputs = [rep.get(v, v) for v in e.inputs]
        if e.op in NO_CSE:
            keep.append(e)
            continue
        key = (e.op, tuple(e.inputs), tuple(sorted((k, repr(v)) for k, v in e.attrs.items())),
               e.body.digest() if e.body else "")
        if key in seen:
            for a, b in zip(e.outputs, seen[key]):
                rep[a] = b
        else:
            seen[key] = e.outputs
            keep.append(e)
    removed = len(g.eqns) - len(keep)
    g.eqns = keep
    for o in g.outputs:
        o.value = rep.get(o.value, o.value)
    return removed


def dce(g: Graph) -> int:
    live: Set[int] = {o.value for o in g.outputs}
    keep: List[Eqn] = []
    for e in reversed(g.eqns):
        if any(o in live for o in e.outputs):
            keep.append(e)
            live.update(e.inputs)
    removed = len(g.eqns) - len(keep)
    g.eqns = keep[::-1]
    used = live
    g.inputs = [i for i in g.inputs if i.value in used or i.storage in ("state", "slot")]
    return removed


# ---- rotate-half chain -> rope ---------------------------------------------------------------------------------
def rope_fusion(g: Graph, declines: Optional[list] = None) -> int:
    n = 0
    while True:
        prod, users = g.producers(), g.users()
        hit = None
        for ci, c in enumerate(g.eqns):
            if c.op != "concat" or len(c.inputs) != 2:
                continue
            a, b = c.inputs
            if a not in prod or b not in prod:
                continue
            ne, s1 = g.eqns[prod[a]], g.eqns[prod[b]]
            if ne.op != "neg" or s1.op != "slice" or ne.inputs[0] not in prod:
                continue
            s2 = g.eqns[prod[ne.inputs[0]]]
            if s2.op != "slice" or s2.inputs[0] != s1.inputs[0]:
                continue
            x = s1.inputs[0]
            rot = g.types[x].shape[-1]
            if tuple(s1.attrs["starts"])[-1] != 0 or tuple(s2.attrs["starts"])[-1] != rot // 2:
                continue
            region = {ci, prod[a], prod[b], prod[ne.inputs[0]]}
            muls = [u for u in users.get(c.outputs[0], []) if g.eqns[u].op == "mul"]
            xmuls = [u for u in users.get(x, []) if g.eqns[u].op == "mul" and u not in region]
            adds = [k for k, e in enumerate(g.eqns) if e.op == "add" and muls and xmuls and
                    set(e.inputs) == {g.eqns[xmuls[0]].outputs[0], g.eqns[muls[0]].outputs[0]}]
            if len(muls) != 1 or len(xmuls) != 1 or len(adds) != 1:
                (declines if declines is not None else []).append(("rope", ci, "rotate-half found without x*cos + rot*sin"))
                continue
            region |= {muls[0], xmuls[0], adds[0]}
            tables = []
            for mi in (xmuls[0], muls[0]):       # fold the reshape/broadcast that shape cos and sin
                for v in g.eqns[mi].inputs:
                    if v in (x, c.outputs[0]):
                        continue
                    chain = []
                    while v in prod and g.eqns[prod[v]].op in ("broadcast", "reshape") and len(users.get(v, [])) == 1:
                        chain.append(prod[v])
                        v = g.eqns[prod[v]].inputs[0]
                    region |= set(chain)
                    tables.append(v)
            hit = (region, rot, [x] + tables)
            break
        if hit is None:
            return n
        try:
            fold_region(g, hit[0], "rope", {"rot": hit[1]}, input_order=hit[2] if len(set(hit[2])) == 3 else None)
            n += 1
        except Decline as d:
            (declines if declines is not None else []).append(("rope", min(hit[0]), str(d)))
            return n


# ---- primitive attention chain -> attention --------------------------------------------------------------------
def flash_attention(g: Graph, declines: Optional[list] = None) -> int:
    n = 0
    skip: Set[int] = set()
    while True:
        prod, users = g.producers(), g.users()
        found = None
        for ei, ex in enumerate(g.eqns):
            if ex.op != "exp" or ex.outputs[0] in skip:
                continue
            try:
                found = _match_attention(g, ei, prod, users)
            except Decline as d:
                skip.add(ex.outputs[0])
                if ex.inputs[0] in prod and g.eqns[prod[ex.inputs[0]]].op == "sub":     # looked like a softmax
                    (declines if declines is not None else []).append(("attention", ei, str(d)))
                continue
            break
        if found is None:
            return n
        region, attrs = found
        try:
            fold_region(g, region, "attention", attrs)
            n += 1
        except Decline as d:
            (declines if declines is not None else []).append(("attention", min(region), str(d)))
            skip.add(g.eqns[max(region)].outputs[0])
            return n


def _match_attention(g: Graph, ei: int, prod, users) -> Tuple[Set[int], dict]:
    E = g.eqns
    ex = E[ei]

    def P(v, op=None):
        if v not in prod:
            raise Decline("operand is a graph input")
        e = E[prod[v]]
        if op is not None and e.op != op:
            raise Decline(f"expected {op}, found {e.op}")
        return prod[v], e

    region = {ei}
    si, sub = P(ex.inputs[0], "sub")
    scores = sub.inputs[0]
    bi, bm = P(sub.inputs[1], "broadcast")
    ri, rmax = P(bm.inputs[0], "reduce")
    if rmax.attrs["kind"] != "max" or rmax.inputs[0] != scores:
        raise Decline("not a max-shifted softmax")
    region |= {si, bi, ri}
    divs = [u for u in users.get(ex.outputs[0], []) if E[u].op == "div"]
    sums = [u for u in users.get(ex.outputs[0], []) if E[u].op == "reduce" and E[u].attrs["kind"] == "sum"]
    if len(divs) != 1 or len(sums) != 1:
        raise Decline("softmax normaliser not found")
    bs = [u for u in users.get(E[sums[0]].outputs[0], []) if E[u].op == "broadcast"]
    if len(bs) != 1 or E[divs[0]].inputs != [ex.outputs[0], E[bs[0]].outputs[0]]:
        raise Decline("softmax normaliser not found")
    region |= {divs[0], sums[0], bs[0]}
    pv = [u for u in users.get(E[divs[0]].outputs[0], []) if E[u].op == "matmul"]
    if len(pv) != 1 or E[pv[0]].inputs[0] != E[divs[0]].outputs[0]:
        raise Decline("probabilities do not feed a P·V matmul")
    region.add(pv[0])
    attrs = {"softcap": 0.0, "mask": "additive", "key": "single", "bound": "capacity", "sink": "absent"}
    # scores = [softcap](q k^T * scale) + mask
    ai, add = P(scores, "add")
    region.add(ai)
    qk = None
    mask = None
    for side in add.inputs:
        v, chain = side, []
        while v in prod and E[prod[v]].op in ("broadcast", "reshape"):
            chain.append(prod[v])
            v = E[prod[v]].inputs[0]
        if v in prod and E[prod[v]].op in ("mul", "matmul", "tanh"):
            qk = side
        else:
            mask, mchain = v, chain
    if qk is None or mask is None:
        raise Decline("score / mask operands not told apart")
    region |= set(mchain)
    v = qk
    while True:
        k_, e = P(v)
        region.add(k_)
        if e.op == "matmul":
            mm = e
            break
        if e.op == "mul":
            lit = [literal_value(g, o) for o in e.inputs]
            other = [o for o, l in zip(e.inputs, lit) if l is None]
            val = [l for l in lit if l is not None]
            if len(other) != 1 or len(val) != 1:
                raise Decline("score scaling is not by a literal")
            for o in e.inputs:           # literal broadcast
                if o != other[0] and o in prod:
                    region.add(prod[o])
            if "scale" not in attrs and E[prod[other[0]]].op == "matmul":
                attrs["scale"] = val[0]
            elif E[prod[other[0]]].op == "tanh":
                attrs["softcap"] = val[0]
            elif "scale" in attrs:
                attrs["scale"] *= val[0]          # the 1/cap inside the soft cap
            v = other[0]
        elif e.op == "tanh":
            v = e.inputs[0]
        else:
            raise Decline(f"unexpected {e.op} between q·kᵀ and the mask")
    if attrs["softcap"]:
        attrs["scale"] = attrs["scale"] * attrs["softcap"]      # scores*scale/cap was folded into scale above
    q = mm.inputs[0]
    ti, tr = P(mm.inputs[1], "transpose")
    region.add(ti)

    def kv_chain(v):
        """repeat_kv (reshape, broadcast, reshape) and paged_view (gather, transpose) in front of K / V."""
        rep = 1
        if v in prod and E[prod[v]].op == "reshape":
            a = E[prod[v]]
            if a.inputs[0] in prod and E[prod[a.inputs[0]]].op == "broadcast":
                b_ = E[prod[a.inputs[0]]]
                if b_.inputs[0] in prod and E[prod[b_.inputs[0]]].op == "reshape":
                    c = E[prod[b_.inputs[0]]]
                    region.update({prod[v], prod[a.inputs[0]], prod[b_.inputs[0]]})
                    rep = tuple(b_.attrs["shape"])[2]
                    v = c.inputs[0]
        paged = False
        if v in prod and E[prod[v]].op == "transpose" and E[prod[v]].inputs[0] in prod and \
                E[prod[E[prod[v]].inputs[0]]].op == "gather" and len(users.get(E[prod[v]].inputs[0], [])) == 1 and \
                len(users.get(v, [])) == 1:
            region.update({prod[v], prod[E[prod[v]].inputs[0]]})
            paged = True
        elif v in prod and E[prod[v]].op == "gather" and len(users.get(v, [])) == 1:
            region.add(prod[v])          # the paged view's transpose was merged into the q·kᵀ transpose
            paged = True
        return rep, paged

    rep_k, paged_k = kv_chain(tr.inputs[0])
    rep_v, paged_v = kv_chain(E[pv[0]].inputs[1])
    if rep_k != rep_v or paged_k != paged_v:
        raise Decline("K and V are prepared differently")
    attrs["n_rep"] = rep_k
    attrs["key"] = "paged" if paged_k else "single"
    attrs.setdefault("scale", 1.0)
    _ = q
    return region, attrs


# ---- contractions ----------------------------------------------------------------------------------------------
def recognize_packed(g: Graph) -> int:
    """``matmul(x, transpose(packed_dequant(p)))`` -> packed_contraction; ``gather(packed_dequant(p), ids)`` -> packed_row_gather."""
    n = 0
    while True:
        prod, users = g.producers(), g.users()
        hit = None
        for k, e in enumerate(g.eqns):
            if e.op == "matmul" and e.inputs[1] in prod and g.eqns[prod[e.inputs[1]]].op == "transpose":
                t = g.eqns[prod[e.inputs[1]]]
                if t.inputs[0] in prod and g.eqns[prod[t.inputs[0]]].op == "packed_dequant" and \
                        len(users.get(e.inputs[1], [])) == 1 and len(users.get(t.inputs[0], [])) == 1:
                    d = g.eqns[prod[t.inputs[0]]]
                    hit = ({k, prod[e.inputs[1]], prod[t.inputs[0]]}, "packed_contraction",
                           {"format": d.attrs["format"], "precision": e.attrs.get("precision", "narrow")})
                    break
            if e.op == "gather" and e.inputs[0] in prod and g.eqns[prod[e.inputs[0]]].op == "packed_dequant" and \
                    len(users.get(e.inputs[0], [])) == 1:
                d = g.eqns[prod[e.inputs[0]]]
                hit = ({k, prod[e.inputs[0]]}, "packed_row_gather", {"format": d.attrs["format"]})
                break
        if hit is None:
            return n
        fold_region(g, hit[0], hit[1], hit[2])
        n += 1


def _is_weight(g: Graph, v: int) -> bool:
    prod = g.producers()
    while v in prod and g.eqns[prod[v]].op == "cast":
        v = g.eqns[prod[v]].inputs[0]
    return any(i.value == v and i.storage == "const" for i in g.inputs)


def fold_dense_contractions(g: Graph) -> int:
    """``matmul(x, transpose(W))`` with a checkpoint-order ``W[N, K]`` constant -> dense_contraction (no transpose runs)."""
    n = 0
    while True:
        prod, users = g.producers(), g.users()
        hit = None
        for k, e in enumerate(g.eqns):
            if e.op != "matmul" or e.inputs[1] not in prod:
                continue
            t = g.eqns[prod[e.inputs[1]]]
            if t.op == "transpose" and tuple(t.attrs["perm"]) == (1, 0) and _is_weight(g, t.inputs[0]) and \
                    len(users.get(e.inputs[1], [])) == 1:
                hit = {k, prod[e.inputs[1]]}
                attrs = {"precision": e.attrs.get("precision", "narrow")}
                break
        if hit is None:
            return n
        fold_region(g, hit, "dense_contraction", attrs)
        n += 1


def fuse_contraction_epilogues(g: Graph) -> int:
    """A contraction whose only user is a residual add keeps the add in its epilogue (``contraction_epilogue``)."""
    n = 0
    heads = ("dense_contraction", "packed_contraction")
    while True:
        users = g.users()
        outs = {o.value for o in g.outputs}
        hit = None
        for k, e in enumerate(g.eqns):
            if e.op not in heads or e.outputs[0] in outs:
                continue
            u = users.get(e.outputs[0], [])
            if len(u) == 1 and g.eqns[u[0]].op == "add" and g.types[g.eqns[u[0]].outputs[0]] == g.types[e.outputs[0]]:
                hit = ({k, u[0]}, {"head": e.op, "region": "residual_add"})
                break
        if hit is None:
            return n
        try:
            fold_region(g, hit[0], "contraction_epilogue", hit[1])
            n += 1
        except Decline:
            return n


# ---- row and pointwise fusion ----------------------------------------------------------------------------------
def fuse(g: Graph, declines: Optional[list] = None) -> Dict[str, int]:
    out = {"rmsnorm": 0, "swiglu": 0, "pointwise": 0}
    out["rmsnorm"] = _fuse_rmsnorm(g, declines)
    out["swiglu"] = _fuse_swiglu(g)
    out["pointwise"] = _fuse_pointwise(g)
    return out


def _lits(g, e, prod, region):
    """Pull literal broadcasts feeding ``e`` into the region."""
    for v in e.inputs:
        if literal_value(g, v) is not None and v in prod:
            region.add(prod[v])


def _fuse_rmsnorm(g: Graph, declines) -> int:
    n = 0
    done: Set[int] = set()
    while True:
        prod, users = g.producers(), g.users()
        hit = None
        for k, s in enumerate(g.eqns):
            if s.op != "sqrt" or s.outputs[0] in done:
                continue
            done.add(s.outputs[0])
            try:
                region = {k}
                ai = prod[s.inputs[0]]; add = g.eqns[ai]
                assert add.op == "add"
                _lits(g, add, prod, region)
                eps = [literal_value(g, v) for v in add.inputs if literal_value(g, v) is not None][0]
                ms = [v for v in add.inputs if literal_value(g, v) is None][0]
                mi = prod[ms]; mul = g.eqns[mi]
                assert mul.op == "mul"
                _lits(g, mul, prod, region)
                ss = [v for v in mul.inputs if literal_value(g, v) is None][0]
                ri = prod[ss]; red = g.eqns[ri]
                assert red.op == "reduce" and red.attrs["kind"] == "sum"
                qi = prod[red.inputs[0]]; sq = g.eqns[qi]
                assert sq.op == "mul" and sq.inputs[0] == sq.inputs[1]
                x = sq.inputs[0]
                region |= {ai, mi, ri, qi}
                bd = [u for u in users[s.outputs[0]] if g.eqns[u].op == "broadcast"]
                dv = [u for u in users[g.eqns[bd[0]].outputs[0]] if g.eqns[u].op == "div" and g.eqns[u].inputs[0] == x]
                wm = [u for u in users[g.eqns[dv[0]].outputs[0]] if g.eqns[u].op == "mul"]
                assert len(bd) == 1 and len(dv) == 1 and len(wm) == 1
                region |= {bd[0], dv[0], wm[0]}
                for v in g.eqns[wm[0]].inputs:           # the weight's broadcast
                    if v in prod and g.eqns[prod[v]].op == "broadcast" and len(users.get(v, [])) == 1:
                        region.add(prod[v])
                hit = (region, float(eps))
                break
            except (AssertionError, KeyError, IndexError):
                continue
        if hit is None:
            return n
        try:
            fold_region(g, hit[0], "fused_row", {"kind": "rmsnorm", "eps": hit[1]})
            n += 1
        except Decline as d:
            (declines if declines is not None else []).append(("rmsnorm", min(hit[0]), str(d)))


def _fuse_swiglu(g: Graph) -> int:
    """``gate / (1 + exp(-gate)) * up`` -> fused{swiglu}."""
    n = 0
    done: Set[int] = set()
    while True:
        prod, users = g.producers(), g.users()
        hit = None
        for k, ex in enumerate(g.eqns):
            if ex.op != "exp" or ex.outputs[0] in done:
                continue
            done.add(ex.outputs[0])
            try:
                region = {k}
                ni = prod[ex.inputs[0]]; neg = g.eqns[ni]
                assert neg.op == "neg"
                gate = neg.inputs[0]
                a = [u for u in users[ex.outputs[0]] if g.eqns[u].op == "add"]
                assert len(a) == 1 and len(users[ex.outputs[0]]) == 1
                _lits(g, g.eqns[a[0]], prod, region)
                d = [u for u in users[g.eqns[a[0]].outputs[0]] if g.eqns[u].op == "div" and g.eqns[u].inputs[0] == gate]
                assert len(d) == 1
                m = [u for u in users[g.eqns[d[0]].outputs[0]] if g.eqns[u].op == "mul"]
                assert len(m) == 1 and len(users[g.eqns[d[0]].outputs[0]]) == 1
                region |= {ni, a[0], d[0], m[0]}
                hit = region
                break
            except (AssertionError, KeyError, IndexError):
                continue
        if hit is None:
            return n
        try:
            fold_region(g, hit, "fused", {"kind": "swiglu"})
            n += 1
        except Decline:
            pass


def _fuse_pointwise(g: Graph) -> int:
    """Greedy chains of single-use pointwise equations (with their literal broadcasts) -> fused{pointwise}."""
    n = 0
    while True:
        prod, users = g.producers(), g.users()
        outs = {o.value for o in g.outputs}
        hit = None
        for k, e in enumerate(g.eqns):
            if e.op not in POINTWISE:
                continue
            region = {k}
            cur = e
            while True:
                u = users.get(cur.outputs[0], [])
                if len(u) != 1 or cur.outputs[0] in outs or g.eqns[u[0]].op not in POINTWISE:
                    break
                if g.types[g.eqns[u[0]].outputs[0]].shape != g.types[cur.outputs[0]].shape:
                    break
                region.add(u[0])
                cur = g.eqns[u[0]]
            if len(region) < 2:
                continue
            for r in list(region):
                _lits(g, g.eqns[r], prod, region)
            hit = region
            break
        if hit is None:
            return n
        try:
            fold_region(g, hit, "fused", {"kind": "pointwise", "ops": len(hit)})
            n += 1
        except Decline:
            return n
