"""Failure lifecycle of a step engine: typed errors, the validation gate, ``NeedsReset`` and ``Poisoned``.

The contract is the reference executor's (crates/poot-executor/src/error.rs:12-57, src/engine.rs:9-14):

* every step runs as one transaction; a failure anywhere in it calls the engine's ``abort`` exactly once;
* a failure that may have left state dirty (K/V written for half a step, a recurrent state advanced, cross-rank
  counters out of step) marks the engine ``needs_reset``: ``run_step`` refuses with ``NeedsReset`` until a *complete*
  ``reset()`` has restored it;
* an ``abort`` or ``reset`` that itself fails poisons the engine for good: ``Poisoned`` on every later call, and a
  reset cannot clear it;
* a step whose inputs fail validation is refused *before* anything is launched (``Validation``): nothing was touched,
  the engine stays usable.  The reference computes a validation packet on the device and checks it before any output
  is read back (crates/poot-graph-plan/src/device_validation.rs:1-8); here the packet is the step's index arrays,
  checked on the host against the engine's static limits, because every index a kernel of this engine dereferences
  comes from those arrays;
* a kernel-reported failure (a bounded wait that gave up: ``DeviceWaitTimeout``) is a ``Fault`` and dirties state.

``GuardedStepEngine`` wraps any step engine of the driver (device, oracle, fake) and is what the coordinator tests
drive with injected failures (crates/poot-executor/tests/coordinator.rs:55-80).
"""
from __future__ import annotations

from typing import Callable, Optional

import numpy as np


class ExecError(RuntimeError):
    """Base of the step-engine failures."""


class Fault(ExecError):
    """A kernel reported a failure through the control block, or the engine raised in the middle of a step."""

    def __init__(self, message: str, code: int = 0, detail: int = -1):
        super().__init__(message)
        self.code, self.detail = code, detail


class Validation(ExecError):
    """A step input is outside what the engine's buffers and tables can hold; nothing was launched."""


class NeedsReset(ExecError):
    """State may be dirty after an earlier failure: a complete ``reset()`` has to come first."""


class Poisoned(ExecError):
    """Cleaning up after a failure failed as well; the engine accepts no further work and cannot be reset."""


class StepLimits:
    """Static limits a step's index arrays are checked against."""

    def __init__(self, vocab: int, max_tokens: int, max_rows: int, pool_slots: int, max_position: int):
        self.vocab, self.max_tokens, self.max_rows = vocab, max_tokens, max_rows
        self.pool_slots, self.max_position = pool_slots, max_position

    @staticmethod
    def of(engine, vocab: Optional[int] = None) -> Optional["StepLimits"]:
        e = getattr(engine, "e", None)          # DeviceStepEngine holds the DecoderEngine as .e
        if e is not None and hasattr(e, "kv"):
            return StepLimits(e.cfg.vocab, e.max_tokens, e.max_seqs, e.kv.num_blocks * 16, e.cfg.max_position)
        if vocab is not None and hasattr(engine, "max_tokens"):
            big = 1 << 30
            return StepLimits(vocab, engine.max_tokens, big, big, big)
        return None


def validate_step(inp, lim: StepLimits) -> None:
    """The validation packet of one step.  Raises ``Validation`` naming the first field that is out of range."""
    T, B = len(inp.tokens), len(inp.logit_idx)

    def bad(what):
        raise Validation(f"step refused before launch: {what}")
    if T > lim.max_tokens:
        bad(f"{T} token rows exceed the engine's {lim.max_tokens}")
    if B > lim.max_rows:
        bad(f"{B} sampling rows exceed the engine's {lim.max_rows}")
    live = inp.live_tokens if inp.live_tokens else T
    tok = np.asarray(inp.tokens[:live])
    if tok.size and (tok.min() < 0 or tok.max() >= lim.vocab):
        bad(f"token id {int(tok.max() if tok.max() >= lim.vocab else tok.min())} outside [0, {lim.vocab})")
    slots = np.asarray(inp.slots[:live])
    if slots.size and (slots.max() >= lim.pool_slots or slots.min() < -1):
        bad(f"K/V slot {int(slots.max())} outside the pool of {lim.pool_slots} slots")
    pos = np.asarray(inp.positions[:live])
    if pos.size and (pos.min() < 0 or pos.max() >= lim.max_position):
        bad(f"position {int(pos.max())} outside [0, {lim.max_position})")
    li = np.asarray(inp.logit_idx[:inp.live_rows if inp.live_rows else B])
    if li.size and (li.min() < 0 or li.max() >= T):
        bad(f"logit row index {int(li.max())} outside the step's {T} rows")
    ctx = np.asarray(inp.row_ctx[:live])
    if ctx.size and ctx.min() < 0:
        bad("negative context length")


class GuardedStepEngine:
    """Transaction wrapper: ``ready`` -> (failure) -> ``needs_reset`` -> ``reset()`` -> ``ready``; a failing clean-up
    leads to ``poisoned``.  Everything else is passed through to the wrapped engine."""

    def __init__(self, inner, limits: Optional[StepLimits] = None, on_reset: Optional[Callable[[], None]] = None):
        self.inner = inner
        self.limits = limits
        self.on_reset = on_reset            # the owner's part of a complete reset (the driver drops its sequences)
        self.state = "ready"                # ready | needs_reset | poisoned
        self.cause: Optional[str] = None
        self.aborts = 0

    def __getattr__(self, name):
        return getattr(self.inner, name)

    def _refuse_unless_ready(self) -> None:
        if self.state == "poisoned":
            raise Poisoned(f"the engine is poisoned and cannot accept further work ({self.cause})")
        if self.state == "needs_reset":
            raise NeedsReset(f"the engine needs a complete reset before its next step ({self.cause})")

    def write_block_table(self, row: int, blocks) -> None:
        self._refuse_unless_ready()
        self.inner.write_block_table(row, blocks)

    def run_step(self, inp):
        self._refuse_unless_ready()
        if self.limits is not None:
            validate_step(inp, self.limits)     # raises before anything is launched: the engine stays ready
        try:
            return self.inner.run_step(inp)
        except Exception as e:
            self.state, self.cause = "needs_reset", f"{type(e).__name__}: {e}"
            self._abort_once()
            if isinstance(e, ExecError):
                raise
            code, detail = getattr(e, "code", 0), getattr(e, "detail", -1)
            raise Fault(f"step failed: {e}", code, detail) from e

    def _abort_once(self) -> None:
        """The engine's own clean-up after a failed transaction (drain the device, clear the control block)."""
        self.aborts += 1
        cleanup = getattr(self.inner, "abort_cleanup", None)
        if cleanup is None:
            return
        try:
            cleanup()
        except Exception as e:
            self.state, self.cause = "poisoned", f"clean-up after a failed step failed: {type(e).__name__}: {e}"

    def reset(self) -> None:
        """Complete reset: the wrapped engine restores its state (K/V contents are dropped, recurrent state and
        cross-rank counters start over), then the owner drops what it built on that state."""
        if self.state == "poisoned":
            raise Poisoned(f"the engine is poisoned; a reset cannot clear it ({self.cause})")
        try:
            r = getattr(self.inner, "reset_state", None)
            if r is not None:
                r()
            if self.on_reset is not None:
                self.on_reset()
        except Exception as e:
            self.state, self.cause = "poisoned", f"reset failed: {type(e).__name__}: {e}"
            raise Poisoned(self.cause) from e
        self.state, self.cause = "ready", None
