"""Host-side control plane of a multi-rank server: step announcements, readiness, acknowledgements, heartbeats.

Every exchange goes through a ``torch.distributed.TCPStore`` that rank 0 hosts, never through a collective, so every
wait has its own short limit and a rank that has left, or that stalls, is noticed on the host *before* the others
launch a step whose kernels or collectives would wait for it:

* rank 0 announces step ``n`` (``step/n``), every follower answers ``ready/n/rank`` when it holds the step and is about
  to launch it, and rank 0 launches only after all of them answered within ``ready_deadline``;
* after the step every follower writes ``ack/n/rank`` with its own result (``ok`` or the failure it saw); rank 0 reads
  them within ``step_deadline``;
* every rank refreshes ``hb/rank`` from a thread with a connection of its own; a follower that waits for the next
  announcement gives up when rank 0's heartbeat is stale, and rank 0 names the rank whose heartbeat stopped;
* ``stop`` carries the cause when rank 0 ends the group, so the followers leave their loops between two steps.

The reference keeps one engine thread per model and one process for all devices
(crates/poot-serve/src/batch/engine.rs:520-560); its coordinator contract on failing devices is tested on fakes
(crates/poot-executor/tests/coordinator.rs:55-80).  With one process per GPU the same contract needs this plane.
"""
from __future__ import annotations

import pickle
import threading
import time
from datetime import timedelta
from typing import Any, Optional, Tuple


class RankLost(RuntimeError):
    """A rank did not answer within its limit (it left, died or stalled)."""

    def __init__(self, rank: int, step: int, why: str):
        super().__init__(f"rank {rank} lost at step {step}: {why}")
        self.rank, self.step, self.why = rank, step, why


class RankFailed(RuntimeError):
    """A rank finished the step and reported a failure of its own."""

    def __init__(self, rank: int, step: int, report: str):
        super().__init__(f"rank {rank} failed step {step}: {report}")
        self.rank, self.step, self.report = rank, step, report


class LeaderLost(RuntimeError):
    """Rank 0 stopped refreshing its heartbeat while a follower was waiting for the next step."""


class ControlPlane:
    def __init__(self, rank: int, world: int, host: str = "127.0.0.1", port: int = 29600,
                 ready_deadline: float = 5.0, step_deadline: float = 30.0, heartbeat: float = 0.25,
                 heartbeat_timeout: float = 3.0, connect_timeout: float = 60.0, ready_check: bool = True):
        from torch.distributed import TCPStore
        self.rank, self.world = rank, world
        self.ready_deadline, self.step_deadline = ready_deadline, step_deadline
        self.heartbeat, self.heartbeat_timeout = heartbeat, heartbeat_timeout
        self.ready_check = ready_check
        mk = lambda master: TCPStore(host, port, world_size=None, is_master=master,
                                     timeout=timedelta(seconds=connect_timeout), wait_for_workers=False)
        self.store = mk(rank == 0)
        self._hb_store = mk(False)          # the heartbeat thread's own connection: a long wait must not block it
        self._hb_stop = threading.Event()
        self._hb_thread: Optional[threading.Thread] = None
        self._hb_paused = False             # tests: a rank that stops answering without exiting
        self.n = 0                          # next step number

    # ---- heartbeat -----------------------------------------------------------------------------------------------
    def start_heartbeat(self) -> None:
        def beat():
            while not self._hb_stop.is_set():
                if not self._hb_paused:
                    try:
                        self._hb_store.set(f"hb/{self.rank}", repr(time.time()))
                    except Exception:
                        return
                self._hb_stop.wait(self.heartbeat)
        self._hb_store.set(f"hb/{self.rank}", repr(time.time()))
        self._hb_thread = threading.Thread(target=beat, name=f"poot-heartbeat-{self.rank}", daemon=True)
        self._hb_thread.start()

    def stale(self, rank: int) -> Optional[float]:
        """Seconds since ``rank``'s last heartbeat when that is beyond the limit, else ``None``."""
        if not self.store.check([f"hb/{rank}"]):
            return None                 # not started yet: readiness and acknowledgements cover it
        age = time.time() - float(self.store.get(f"hb/{rank}").decode())
        return age if age > self.heartbeat_timeout else None

    # ---- waits -----------------------------------------------------------------------------------------------------
    def _wait(self, key: str, limit: float) -> bool:
        try:
            self.store.wait([key], timedelta(seconds=max(limit, 1e-3)))
            return True
        except Exception:               # the store's timeout error type differs between torch versions
            return self.store.check([key])

    def _gather(self, prefix: str, n: int, limit: float, what: str):
        """Values of ``prefix/n/rank`` for every follower; ``RankLost`` names the first one missing."""
        end = time.monotonic() + limit
        out = {}
        for r in range(1, self.world):
            key = f"{prefix}/{n}/{r}"
            while True:
                left = end - time.monotonic()
                if self._wait(key, min(max(left, 0.0), 0.25)):
                    out[r] = self.store.get(key).decode()
                    break
                if self.store.check([f"left/{r}"]):
                    raise RankLost(r, n, "the rank left the group: " + self.store.get(f"left/{r}").decode())
                age = self.stale(r)
                if age is not None:
                    raise RankLost(r, n, f"no heartbeat for {age:.1f} s")
                if left <= 0:
                    raise RankLost(r, n, f"no {what} within {limit:.1f} s")
        return out

    # ---- rank 0 ----------------------------------------------------------------------------------------------------
    def announce(self, payload: Any) -> int:
        n = self.n
        self.n += 1
        self.store.set(f"step/{n}", pickle.dumps(payload))
        if n >= 2:                      # keys of finished steps
            for key in [f"step/{n - 2}"] + [f"{p}/{n - 2}/{r}" for p in ("ready", "ack") for r in range(1, self.world)]:
                try:
                    self.store.delete_key(key)
                except Exception:
                    pass
        return n

    def wait_ready(self, n: int) -> None:
        """Every follower holds step ``n`` and is about to launch it.  Raises ``RankLost`` before anything was
        launched here, so no kernel or collective of this rank ever waits for a rank that is gone."""
        if self.ready_check:
            self._gather("ready", n, self.ready_deadline, "readiness")

    def wait_acks(self, n: int) -> None:
        for r, report in self._gather("ack", n, self.step_deadline, "acknowledgement").items():
            if report != "ok":
                raise RankFailed(r, n, report)

    def stop(self, cause: str = "", linger: float = 0.0) -> None:
        """Publish the end of the group.  With ``linger`` rank 0 then waits (bounded) until every follower that still
        answers has said that it left: the store lives in rank 0's process, so leaving at once would take the message
        away from a follower that has not read it yet."""
        try:
            if not self.store.check(["stop"]):
                self.store.set("stop", cause or "stopped")
        except Exception:
            return
        end = time.monotonic() + linger
        for r in range(1, self.world):
            while time.monotonic() < end:
                try:
                    if self.store.check([f"left/{r}"]) or self.stale(r) is not None:
                        break
                except Exception:
                    return
                time.sleep(0.02)

    def stopped(self) -> Optional[str]:
        """The cause if rank 0 ended the group, else ``None``."""
        try:
            return self.store.get("stop").decode() if self.store.check(["stop"]) else None
        except Exception:
            return "rank 0 is gone (the control store does not answer)"

    # ---- followers -------------------------------------------------------------------------------------------------
    def next_step(self) -> Tuple[str, Any]:
        """``("step", payload)`` of the next announcement, or ``("stop", cause)``."""
        key = f"step/{self.n}"
        while True:
            if self._wait(key, 0.25):
                self.n += 1
                return "step", pickle.loads(self.store.get(key))
            if self.store.check(["stop"]):
                return "stop", self.store.get("stop").decode()
            age = self.stale(0)
            if age is not None:
                raise LeaderLost(f"rank 0 sent no heartbeat for {age:.1f} s")

    def ready(self, n: int) -> None:
        self.store.set(f"ready/{n}/{self.rank}", "1")

    def ack(self, n: int, report: str = "ok") -> None:
        self.store.set(f"ack/{n}/{self.rank}", report)

    def leave(self, why: str) -> None:
        """Say that this rank leaves the group (between two steps, nothing of it in flight)."""
        try:
            self.store.set(f"left/{self.rank}", why)
        except Exception:
            pass

    def close(self) -> None:
        self._hb_stop.set()
        if self._hb_thread is not None:
            self._hb_thread.join(timeout=2)
