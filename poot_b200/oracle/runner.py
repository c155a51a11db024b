"""Step-by-step generation on the CPU oracle (the tiny end-to-end reference of the whole stack).

Runs prefill and decode steps of a traced model with the carried state (paged or contiguous KV) fed back
from ``state_next`` outputs, a block table of 16-position blocks and greedy or seeded sampling - the same
open / step / commit loop as the device driver, on the oracle.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np

from ..models.model import Model, StepSpec
from ..tensor import DType
from .eval import EvalOptions, eval_graph

BLOCK = 16


def random_weights_f32(model: Model, seed: int = 0, std: float = 0.02) -> Dict[str, np.ndarray]:
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in model.weight_shapes().items():
        if name.endswith("norm"):
            out[name] = np.ones(shape, dtype=np.float32)
        else:
            out[name] = (rng.standard_normal(shape) * std).astype(np.float32)
    return out


class OracleSession:
    """One sequence per row; every row advances in lockstep (enough for the oracle's purposes)."""

    def __init__(self, model: Model, weights: Dict[str, np.ndarray], rows: int = 1, capacity: int = 64,
                 paged: bool = True, options: Optional[EvalOptions] = None, block_order: Optional[Sequence[int]] = None,
                 world: int = 1, rank: int = 0, graph_transform=None, logit_rows: str = "last"):
        self.logit_rows = logit_rows               # "all": ``step`` returns the logits of every token of the step
        self.model, self.weights, self.rows, self.capacity, self.paged = model, weights, rows, capacity, paged
        self.options = options or EvalOptions(matmul_precision="exact")
        self.graphs: Dict[int, object] = {}
        self.state: Dict[str, np.ndarray] = {}
        self.length = 0
        self.world, self.rank = world, rank
        self.graph_transform = graph_transform     # e.g. the planner's pass pipeline (pass-soundness checks)
        nblocks = rows * capacity // BLOCK
        order = list(block_order) if block_order is not None else list(range(nblocks))
        self.block_table = np.asarray(order, dtype=np.int32).reshape(rows, capacity // BLOCK)
        self.last_logits: Optional[np.ndarray] = None

    def _graph(self, tokens: int, embeds: bool = False, mrope: bool = False):
        key = (tokens, embeds, mrope) if mrope else (tokens, embeds)
        if key not in self.graphs:
            spec = StepSpec(rows=self.rows, tokens=tokens, capacity=self.capacity, paged=self.paged, world=self.world,
                            embeds=embeds, mrope=mrope, logit_rows=self.logit_rows)
            g = self.model.trace(spec)
            self.graphs[key] = self.graph_transform(g) if self.graph_transform is not None else g
        return self.graphs[key]

    def slot(self, row: int, pos: int) -> int:
        return int(self.block_table[row, pos // BLOCK]) * BLOCK + pos % BLOCK

    def step(self, tokens: np.ndarray, embed_rows: Optional[np.ndarray] = None,
             embed_flags: Optional[np.ndarray] = None, rope_positions: Optional[np.ndarray] = None) -> np.ndarray:
        """Feed ``tokens[rows, T]`` at the current position; returns logits ``[rows, vocab]`` of the last token.
        ``embed_rows[rows * T, hidden]`` replace the embeddings of the tokens whose ``embed_flags`` entry is 1;
        ``rope_positions[3, rows * T]`` are the rotary position streams of a sectioned-rope model (the K/V index of a
        token stays its place in the sequence)."""
        tokens = np.asarray(tokens, dtype=np.int32).reshape(self.rows, -1)
        T = tokens.shape[1]
        g = self._graph(T, embed_rows is not None, True) if rope_positions is not None else self._graph(T, embed_rows is not None)
        pos = np.arange(self.length, self.length + T, dtype=np.int32)[None, :].repeat(self.rows, 0)
        inputs: Dict[str, np.ndarray] = {"tokens": tokens, "positions": pos}
        if rope_positions is not None:
            inputs["rope_positions"] = np.asarray(rope_positions, dtype=np.int32).reshape(3, self.rows * T)
        if embed_rows is not None:
            inputs["embed_rows"] = np.asarray(embed_rows, dtype=np.float32).reshape(self.rows * T, -1)
            inputs["embed_flags"] = np.asarray(embed_flags, dtype=np.int32).reshape(self.rows * T)
        if self.paged:
            read = np.zeros((self.rows, self.capacity), dtype=np.int32)
            for r in range(self.rows):
                for p in range(self.capacity):
                    read[r, p] = self.slot(r, p)
            write = np.array([self.slot(r, self.length + t) for r in range(self.rows) for t in range(T)], dtype=np.int32)
            inputs["read_map"], inputs["write_map"] = read, write
        for i in g.inputs:
            if i.storage == "const":
                inputs[i.name] = self._weight(i.name, g.types[i.value].shape)
            elif i.storage == "state":
                if i.name not in self.state:
                    self.state[i.name] = np.zeros(g.types[i.value].shape, dtype=np.float32)
                inputs[i.name] = self.state[i.name]
        ev = eval_graph(g, inputs, self.options)
        for o in g.outputs:
            if o.role == "state_next":
                self.state[o.state_of] = ev.outputs[o.name]
        self.length += T
        self.last_logits = ev.outputs["logits"]
        return self.last_logits

    def _weight(self, name: str, shape) -> np.ndarray:
        w = self.weights[name]
        if tuple(w.shape) == tuple(shape):
            return w
        # tensor-parallel share: split on the axis whose extent shrank (Megatron layouts)
        for ax in range(w.ndim):
            if w.shape[ax] != shape[ax]:
                n = shape[ax]
                sl = [slice(None)] * w.ndim
                sl[ax] = slice(self.rank * n, (self.rank + 1) * n)
                return np.ascontiguousarray(w[tuple(sl)])
        return w

    def generate(self, prompt: Sequence[int], n: int) -> List[int]:
        logits = self.step(np.asarray(prompt, dtype=np.int32).reshape(1, -1))
        out = []
        for _ in range(n):
            tok = int(np.argmax(logits[0]))
            out.append(tok)
            logits = self.step(np.array([[tok]], dtype=np.int32))
        return out


class RankWalk:
    """Evaluate the ``world`` rank-local graphs of a tensor-parallel model in lockstep on the CPU.

    Each rank runs its own :class:`OracleSession` on a thread; at an ``all_reduce`` every rank deposits its partial
    and all of them continue with the left fold of the partials in rank order, which is the sum the device's
    rank-ordered reduction produces (crates/poot-eval/src/ops/collective.rs:12-34; the reference's
    ``expand_ranks`` walk, crates/poot-graph-plan/src/passes/sharding.rs:1165-1357).
    """

    def __init__(self, model: Model, weights: Dict[str, np.ndarray], world: int, rows: int = 1, capacity: int = 64,
                 paged: bool = True, graph_transform=None):
        import threading
        self.world = world
        self._barrier = threading.Barrier(world)
        self._box: List[Optional[np.ndarray]] = [None] * world
        self.sessions = []
        for r in range(world):
            opt = EvalOptions(matmul_precision="exact", collectives=self._hook(r))
            self.sessions.append(OracleSession(model, weights, rows, capacity, paged, opt, world=world, rank=r,
                                               graph_transform=graph_transform))

    def _hook(self, rank: int):
        def collective(op, eqn, ins):
            self._box[rank] = ins[0]
            self._barrier.wait()
            if op == "all_reduce":
                acc = self._box[0].copy()
                for r in range(1, self.world):
                    acc = acc + self._box[r]
            elif op == "all_gather":
                acc = np.concatenate(self._box, axis=eqn.attrs["axis"])
            else:
                raise NotImplementedError(op)
            self._barrier.wait()         # nobody overwrites the box before every rank has read it
            return acc
        return collective

    def step(self, tokens: np.ndarray) -> List[np.ndarray]:
        import threading
        out: List[Optional[np.ndarray]] = [None] * self.world
        errs: List[BaseException] = []

        def run(r):
            try:
                out[r] = self.sessions[r].step(tokens)
            except BaseException as e:      # a failed rank must not leave the others waiting at the barrier
                errs.append(e)
                self._barrier.abort()

        ts = [threading.Thread(target=run, args=(r,)) for r in range(self.world)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        if errs:
            raise errs[0]
        return out
