"""Run-twice determinism check: the stand-in for a race detector.

Every kernel of the engine is written to be order-independent (fixed-order reductions, no float atomics on results),
so a step run twice from the same state must give the same bits.  A difference means two writers raced for a buffer,
a kernel read something before its producer finished, or scratch memory leaked from one step into the next.
``run_twice`` snapshots the engine's mutable state (K/V pool, recurrent state, step inputs), runs the step, restores
the state, runs it again and compares logits, picked tokens and the K/V pool bit for bit; ``diff_report`` names the
first tensor that differs and how many elements do.  It works on the device engine and, on a machine without a GPU,
on the same engine under ``emulated_kernels()``.  (The reference relies on structural rules instead of a race
detector - one writer per slot, declared slot ranges checked at bind; website/docs/architecture/graph-ir.mdx.)
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch

STATE_NAMES = ("gdn_state", "gdn_conv_state", "ssm_state", "ssm_conv_state")


class NotDeterministic(AssertionError):
    def __init__(self, name: str, differing: int, total: int, first: int):
        super().__init__(f"'{name}' differs between two runs of the same step: {differing} of {total} elements, "
                         f"first at flat index {first}")
        self.name, self.differing, self.total, self.first = name, differing, total, first


def _bits(t: torch.Tensor) -> torch.Tensor:
    t = t.detach().contiguous()
    view = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[t.element_size()]
    return t.view(view).reshape(-1)


def diff_report(name: str, a: torch.Tensor, b: torch.Tensor) -> Optional[NotDeterministic]:
    ne = _bits(a) != _bits(b)
    n = int(ne.sum())
    if n == 0:
        return None
    return NotDeterministic(name, n, ne.numel(), int(torch.nonzero(ne)[0]))


def engine_state(engine) -> Dict[str, torch.Tensor]:
    """The tensors a step mutates besides its outputs."""
    st = {"kv": engine.kv.buf}
    for n in STATE_NAMES:
        t = getattr(engine, n, None)
        if t is not None:
            st[n] = t
    return st


def engine_outputs(engine, shape) -> Dict[str, torch.Tensor]:
    B = shape.logit_rows
    out = {"picked": engine.picked[:B]}
    logits = getattr(engine, "logits", None)
    if logits is not None:
        out["logits"] = logits[:B]
    return out


def run_twice(engine, shape, step: Optional[Callable[[], None]] = None, sync: Optional[Callable[[], None]] = None,
              extra: Optional[Callable[[], Dict[str, torch.Tensor]]] = None) -> None:
    """Run ``step`` (default: ``engine.forward(shape)``) twice from the same state and raise ``NotDeterministic`` for
    the first tensor whose bits differ.  The engine's state after the call is the state after one run."""
    step = step or (lambda: engine.forward(shape))
    if sync is None:
        sync = (lambda: torch.cuda.synchronize(engine.device)) if engine.device.type == "cuda" else (lambda: None)
    state = engine_state(engine)
    saved = {k: v.clone() for k, v in state.items()}
    sync()
    step()
    sync()
    outs = lambda: {**engine_outputs(engine, shape), **(extra() if extra else {})}
    first = {k: v.clone() for k, v in {**outs(), **state}.items()}
    for k, v in state.items():
        v.copy_(saved[k])
    sync()
    step()
    sync()
    second = {**outs(), **state}
    problems: List[NotDeterministic] = [p for k in first if (p := diff_report(k, first[k], second[k])) is not None]
    if problems:
        raise problems[0]
