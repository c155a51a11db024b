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
                 world: int = 1, rank: int = 0):
        self.model, self.weights, self.rows, self.capacity, self.paged = model, weights, rows, capacity, paged
        self.options = options or EvalOptions(matmul_precision="exact")
        self.graphs: Dict[int, object] = {}
        self.state: Dict[str, np.ndarray] = {}
        self.length = 0
        self.world, self.rank = world, rank
        nblocks = rows * capacity // BLOCK
        order = list(block_order) if block_order is not None else list(range(nblocks))
        self.block_table = np.asarray(order, dtype=np.int32).reshape(rows, capacity // BLOCK)
        self.last_logits: Optional[np.ndarray] = None

    def _graph(self, tokens: int):
        if tokens not in self.graphs:
            spec = StepSpec(rows=self.rows, tokens=tokens, capacity=self.capacity, paged=self.paged, world=self.world)
            self.graphs[tokens] = self.model.trace(spec)
        return self.graphs[tokens]

    def slot(self, row: int, pos: int) -> int:
        return int(self.block_table[row, pos // BLOCK]) * BLOCK + pos % BLOCK

    def step(self, tokens: np.ndarray) -> np.ndarray:
        """Feed ``tokens[rows, T]`` at the current position; returns logits ``[rows, vocab]`` of the last token."""
        tokens = np.asarray(tokens, dtype=np.int32).reshape(self.rows, -1)
        T = tokens.shape[1]
        g = self._graph(T)
        pos = np.arange(self.length, self.length + T, dtype=np.int32)[None, :].repeat(self.rows, 0)
        inputs: Dict[str, np.ndarray] = {"tokens": tokens, "positions": pos}
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
