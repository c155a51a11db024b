"""Layer-pipeline placement: the hand-off of the residual stream between stages, one process per GPU.

A step runs its stages in order (no micro-batching: crates/poot-executor/src/coordinator/mod.rs:19-22): stage ``i``
receives ``h[T, hidden]`` from stage ``i - 1``, runs its layers and sends ``h`` on; the last stage samples and
returns the picked tokens to the first stage, whose host driver owns the sequences.  The transfers are
point-to-point ``torch.distributed`` operations on the step's stream (NCCL over NVLink between GPUs; gloo in the
host tests), so they are ordered with the kernels on both sides and need no host synchronisation in between.
"""
from __future__ import annotations

from typing import Optional

import torch


class PipelineLink:
    """Point-to-point plumbing of one stage (``rank`` of ``world`` in ``group``)."""

    def __init__(self, rank: int, world: int, group=None):
        self.rank, self.world, self.group = rank, world, group
        self.sent_bytes = 0

    def recv_hidden(self, h: torch.Tensor) -> None:
        import torch.distributed as dist
        dist.recv(h, src=self.rank - 1, group=self.group)

    def send_hidden(self, h: torch.Tensor) -> None:
        import torch.distributed as dist
        dist.send(h, dst=self.rank + 1, group=self.group)
        self.sent_bytes += h.numel() * h.element_size()

    def return_picked(self, picked: torch.Tensor, extra: Optional[torch.Tensor] = None) -> None:
        """Last stage -> first stage: the sampled tokens (and the log-probabilities when asked for)."""
        import torch.distributed as dist
        if self.world == 1:
            return
        if self.rank == self.world - 1:
            dist.send(picked, dst=0, group=self.group)
            if extra is not None:
                dist.send(extra, dst=0, group=self.group)
        elif self.rank == 0:
            dist.recv(picked, src=self.world - 1, group=self.group)
            if extra is not None:
                dist.recv(extra, src=self.world - 1, group=self.group)


class LocalLink:
    """All stages in one process, one thread per stage (tests): blocking queues stand in for the transfers."""

    def __init__(self, queues: dict, index: int, count: int):
        import queue
        self.q, self.rank, self.world = queues, index, count
        for key in [("h", i) for i in range(1, count)] + ["picked"]:
            queues.setdefault(key, queue.Queue())
        self.sent_bytes = 0

    def recv_hidden(self, h: torch.Tensor) -> None:
        h.copy_(self.q[("h", self.rank)].get(timeout=60))

    def send_hidden(self, h: torch.Tensor) -> None:
        self.q[("h", self.rank + 1)].put(h.clone())
        self.sent_bytes += h.numel() * h.element_size()

    def return_picked(self, picked: torch.Tensor, extra: Optional[torch.Tensor] = None) -> None:
        if self.world == 1:
            return
        if self.rank == self.world - 1:
            self.q["picked"].put((picked.clone(), None if extra is None else extra.clone()))
        elif self.rank == 0:
            p, e = self.q["picked"].get(timeout=60)
            picked.copy_(p)
            if extra is not None and e is not None:
                extra.copy_(e)
