"""Leaving a multi-rank process without a resident waiting kernel.

A process that exits (or is killed) while one of its kernels is still spinning on a flag that a peer writes, or while a
library collective is still waiting for a peer, has its context torn down under a running kernel; kernels that hold
tensor memory and a cluster cannot be switched out for that, and the GPU can be left unusable.  So every exit path of
a multi-rank program - normal end, exception, watchdog, SIGTERM / SIGINT - goes through ``drain_and_exit``:

1. set the host-mapped abort word: every pending and future device-side wait of this rank returns at once
   (``csrc/kernels/common.cuh`` control block, ``cuda_ops.request_abort``);
2. abort the NCCL communicators, so that a library collective that waits for a rank that is gone ends as well;
3. wait for the device to go idle (bounded: a helper thread reports when the wait outlives its limit);
4. unmap the peers' symmetric memory, flush the streams' output, and only then leave with ``os._exit``.

The reference's equivalent is ``Device::abort`` of a scoped transaction followed by teardown in one process
(crates/poot-executor/src/engine.rs:9-14); with one process per GPU the abort has to reach kernels that wait on
another process, hence the abort word.
"""
from __future__ import annotations

import os
import signal
import sys
import threading
from typing import Callable, Optional

_state = {"comm": None, "on_exit": None, "draining": False}


def _abort_library_collectives() -> None:
    try:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_backend() == "nccl":
            from torch.distributed import distributed_c10d as c10d
            c10d._abort_process_group()
    except Exception:
        pass


def drain(sync_limit: float = 20.0) -> bool:
    """Steps 1-3.  Returns whether the device went idle within ``sync_limit`` seconds."""
    import torch
    from ..ops import cuda_ops as K
    if not torch.cuda.is_available():
        return True
    K.request_abort()
    _abort_library_collectives()
    done = threading.Event()

    def sync():
        try:
            torch.cuda.synchronize()
        except Exception:
            pass
        done.set()
    t = threading.Thread(target=sync, name="poot-drain", daemon=True)
    t.start()
    return done.wait(sync_limit)


def drain_and_exit(code: int, message: Optional[str] = None) -> None:
    """Drain this rank's device, release peer mappings and leave the process with ``code``."""
    if _state["draining"]:
        return
    _state["draining"] = True
    if message:
        print(message, file=sys.stderr, flush=True)
    idle = drain()
    comm = _state["comm"]
    if idle and comm is not None and getattr(comm, "block", None) is not None:
        try:
            comm.block.close()
        except Exception:
            pass
    cb = _state["on_exit"]
    if cb is not None:
        try:
            cb(code)
        except Exception:
            pass
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(code if idle else max(code, 4))


def install(comm=None, watchdog_seconds: Optional[float] = None, on_exit: Optional[Callable[[int], None]] = None,
            signals=(signal.SIGTERM, signal.SIGINT)) -> Optional[threading.Timer]:
    """Route SIGTERM / SIGINT and an optional watchdog through ``drain_and_exit``.  ``on_exit(code)`` runs after the
    drain (print a result line, say).  Returns the watchdog timer (cancel it when the run finished in time)."""
    _state["comm"], _state["on_exit"] = comm, on_exit

    # The Python-level handler of a signal only runs when the main thread is between two bytecodes; a main thread that
    # sits in a device synchronise or in a collective would never get there.  The C-level handler, however, writes the
    # signal number to the wake-up descriptor at once, and a helper thread reads it and runs the drain.
    if threading.current_thread() is threading.main_thread():
        r, w = os.pipe()
        os.set_blocking(w, False)
        try:
            signal.set_wakeup_fd(w, warn_on_full_buffer=False)
            for sig in signals:
                signal.signal(sig, lambda *_: None)
        except (ValueError, OSError):
            pass
        else:
            def waiter():
                while True:
                    try:
                        data = os.read(r, 1)
                    except OSError:
                        return
                    if data and data[0] in [int(s) for s in signals]:
                        drain_and_exit(128 + data[0], f"signal {data[0]}: draining the device before exit")
                        return
            threading.Thread(target=waiter, name="poot-signal-drain", daemon=True).start()
    dog = None
    if watchdog_seconds:
        dog = threading.Timer(watchdog_seconds, drain_and_exit,
                              args=(3, f"watchdog: the run did not finish within {watchdog_seconds:.0f} s; draining"))
        dog.daemon = True
        dog.start()
    return dog


def set_comm(comm) -> None:
    _state["comm"] = comm
