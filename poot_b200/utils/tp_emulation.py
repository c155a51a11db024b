"""Host restatement of the fused tensor-parallel kernels, with the ranks as threads of one process (tests only).

``EmulatedFusedComm`` offers what ``parallel.tp.FusedComm`` offers the engine, but its "symmetric memory" is a set of
host tensors that all rank threads share, and each launch is a Python function that does what the kernel does, in the
kernel's order: write the partial rows into the peers' inboxes, publish the site's flag (and the poison word when this
rank has recorded a failure), wait for the peers' flags under the rules of ``csrc/kernels/tp_common.cuh`` - a recorded
failure, the host's abort word, the step deadline and a peer's poison word each end a wait - then reduce in rank order.

So the engine's unmodified fused programs (site numbering, flag targets across steps, buffer parity, the greedy-pick
exchange) run at any world size without a GPU, and the failure rules can be driven from the host: a rank thread that
never starts, a stall longer than the step budget, an abort while a wait is pending.  With fewer GPUs than ranks this
is also the only form in which kernels that wait on one another may be run at all.  Nothing in the product selects it.
"""
from __future__ import annotations

import threading
import time
from typing import List, Optional

import torch

from ..ops import cuda_ops as K
from . import kernel_emulation as E

CH_RS, CH_AG, CH_POISON, CH_AX, CH_EPD, CH_EPC = 0, 1, 2, 3, 4, 5
MAX_ROWS = 128
OK, TIMEOUT_PEER_FLAG, ABORTED, STEP_DEADLINE, PEER_FAILED = 0, 4, 6, 7, 8
NO_DEADLINE_BUDGET_S = 1.0


class EmulatedGroup:
    """What the ranks of one node share: every rank's flag block, inbox, gather buffer, exchange area, control block."""

    def __init__(self, world: int, hidden: int, ax_cap: int = 4096, max_rows: int = MAX_ROWS):
        self.world, self.H, self.ax_cap = world, hidden, ax_cap
        self.max_rows = max(MAX_ROWS, max_rows // 128 * 128)       # largest padded step of the sharded program
        self.flags = torch.zeros(world, 6, 8, dtype=torch.int64)
        self.inbox = [torch.zeros(2, world, self.max_rows, hidden, dtype=torch.bfloat16) for _ in range(world)]
        self.xs = [torch.zeros(2, self.max_rows, hidden, dtype=torch.bfloat16) for _ in range(world)]
        self.ax = [torch.zeros(2, world, ax_cap, dtype=torch.int32) for _ in range(world)]
        # control blocks: first failure, detail, deadline (monotonic seconds; 0 = none), abort word, step budget
        self.ctl = [dict(code=0, detail=-1, deadline=0.0, abort=0, budget=5.0, gave_up=0) for _ in range(world)]
        self.barrier = threading.Barrier(world)
        self.lock = threading.Lock()
        self.ep_recv = self.ep_meta = self.ep_gatev = self.ep_count = self.ep_back = None

    def ensure_ep(self, cap: int) -> None:
        """Receive and combine areas of the expert-parallel exchange (first rank to attach a routed model makes them)."""
        with self.lock:
            if self.ep_recv is None:
                w, H = self.world, self.H
                self.ep_recv = [torch.zeros(2, w, cap, H, dtype=torch.bfloat16) for _ in range(w)]
                self.ep_meta = [torch.zeros(2, w, cap, 4, dtype=torch.int32) for _ in range(w)]
                self.ep_gatev = [torch.zeros(2, w, cap, dtype=torch.float32) for _ in range(w)]
                self.ep_count = [torch.zeros(2, w, dtype=torch.int32) for _ in range(w)]
                self.ep_back = [torch.zeros(2, cap, H, dtype=torch.bfloat16) for _ in range(w)]

    # ---- control block rules (csrc/kernels/common.cuh) ---------------------------------------------------------
    def fail(self, rank: int, code: int, detail: int = -1) -> None:
        with self.lock:
            c = self.ctl[rank]
            if c["code"] == 0:                  # first cause only
                c["code"], c["detail"] = code, detail
            c["gave_up"] += 1

    def stop_reason(self, rank: int) -> int:
        c = self.ctl[rank]
        if c["code"] != 0:
            return c["code"]
        if c["abort"]:
            return ABORTED
        if c["deadline"] and time.monotonic() > c["deadline"]:
            return STEP_DEADLINE
        return 0

    def request_abort(self, rank: Optional[int] = None) -> None:
        for r in (range(self.world) if rank is None else [rank]):
            self.ctl[r]["abort"] = 1

    def status(self, rank: int):
        c = self.ctl[rank]
        return c["code"], c["detail"]

    def clear(self, rank: int) -> None:
        self.ctl[rank].update(code=0, detail=-1, gave_up=0)

    # ---- flags (csrc/kernels/tp_common.cuh) ----------------------------------------------------------------------
    def wait_flag(self, rank: int, ch: int, src: int, target: int) -> int:
        f = self.flags[rank, ch]
        if int(f[src]) >= target:
            return 0
        why = self.stop_reason(rank)
        if why:
            return why
        has_deadline = bool(self.ctl[rank]["deadline"])
        t0 = time.monotonic()
        while int(f[src]) < target:
            if bool((self.flags[rank, CH_POISON, :self.world] != 0).any()):
                return PEER_FAILED
            why = self.stop_reason(rank)
            if why:
                return why
            if not has_deadline and time.monotonic() - t0 > NO_DEADLINE_BUDGET_S:
                return TIMEOUT_PEER_FLAG
            time.sleep(0.0002)
        return 0

    def wait_all(self, rank: int, ch: int, target: int, site: int, skip_self: bool = False) -> bool:
        for r in range(self.world):             # a peer that gave up ran ahead and published every flag: its poison word tells
            if int(self.flags[rank, CH_POISON, r]) != 0:
                self.fail(rank, PEER_FAILED, site * 16 + r)
                return False
        for r in range(self.world):
            if skip_self and r == rank:
                continue
            why = self.wait_flag(rank, ch, r, target)
            if why:
                self.fail(rank, why, site * 16 + r)
                return False
        return True

    def signal_all(self, rank: int, ch: int, target: int) -> None:
        code = self.ctl[rank]["code"]
        for d in range(self.world):
            if code and d != rank:
                self.flags[d, CH_POISON, rank] = code
            self.flags[d, ch, rank] = target


class EmulatedFusedComm:
    fused = True
    MAX_ROWS = MAX_ROWS

    def __init__(self, rank: int, group: EmulatedGroup):
        self.rank, self.world, self.g = rank, group.world, group
        self.device = torch.device("cpu")
        self.epoch = 0
        self.ax_count = 0
        self.library_collectives = 0
        self.block = None
        self.log: List[tuple] = []          # (kind, site, target) of every cross-rank launch, for the tests

    def attach(self, engine) -> None:
        H = engine.cfg.hidden
        assert H == self.g.H
        self.H = H
        self.max_rows = max(MAX_ROWS, min(self.g.max_rows, engine.max_tokens // 128 * 128))
        self.s_max = self.max_rows // self.world
        self.h_shard = torch.zeros(self.s_max, H, dtype=torch.bfloat16)
        L = engine.cfg.n_layers
        self.rs_sites, self.ag_sites = 2 * L, 2 * L + 1
        self.partial = torch.zeros(engine.max_tokens, H, dtype=torch.bfloat16)
        self.ep_cap, self.ep_sites = 0, L
        if engine.cfg.is_moe and getattr(engine.w, "ep_world", 1) == self.world:
            self.ep_cap = self.s_max * engine.cfg.top_k
            self.g.ensure_ep(self.ep_cap)

    # ---- geometry (same rules as FusedComm) ----------------------------------------------------------------------
    def rows_for(self, T: int) -> int:
        need = max(T, 8 * self.world)
        for r in (16, 32, 64, 128):
            if r >= need and r % (8 * self.world) == 0:
                return r
        r = (need + 127) // 128 * 128
        return r if r <= self.max_rows else 0

    def oneshot_ok(self, T: int) -> bool:
        return T <= 128 and T * (self.world - 1) <= 512

    def _target(self, site: int, sites: int) -> int:
        return (self.epoch - 1) * sites + site + 1

    # ---- launches --------------------------------------------------------------------------------------------------
    def rendezvous(self) -> None:
        self.g.barrier.wait(timeout=60)

    def begin_step(self) -> None:
        self.epoch += 1
        c = self.g.ctl[self.rank]
        c["deadline"] = time.monotonic() + c["budget"] if c["budget"] else 0.0

    def end_step(self) -> None:
        self.g.ctl[self.rank]["deadline"] = 0.0

    def gather_rows(self, idx, out, rows: int, S: int, ag_site: int) -> None:
        target = self._target(ag_site, self.ag_sites)
        ok = self.g.wait_all(self.rank, CH_AG, target, ag_site)
        X = self.g.xs[self.rank][target & 1, :self.world * S]
        out[:rows] = X[idx[:rows].long().clamp(0, self.world * S - 1)] if ok else 0

    def gemm_allreduce(self, x, W, rows: int, rs_site: int) -> None:
        y = E._bf(x[:rows].float() @ W.float().T)
        target = self._target(rs_site, self.rs_sites)
        for d in range(self.world):
            self.g.inbox[d][target & 1, self.rank, :rows] = y
        self.log.append(("rs", rs_site, target))
        self.g.signal_all(self.rank, CH_RS, target)

    def push_rows(self, y, rows: int, rs_site: int) -> None:
        """A producer that is not the row-parallel GEMM (the expert-parallel combine) sends its partial rows the same way."""
        target = self._target(rs_site, self.rs_sites)
        for d in range(self.world):
            self.g.inbox[d][target & 1, self.rank, :rows] = y[:rows]
        self.log.append(("rs", rs_site, target))
        self.g.signal_all(self.rank, CH_RS, target)

    # ---- expert-parallel exchange over the token-sharded stream ------------------------------------------------------
    def norm_local(self, w, x_out, S: int, eps: float, rs_site: int) -> None:
        if rs_site >= 0:
            self._reduce(self.h_shard, S, rs_site)
        E.rmsnorm(self.h_shard[:S], w, eps, out=x_out[:S])

    def _ep_target(self, site: int) -> int:
        return (self.epoch - 1) * self.ep_sites + site + 1

    def ep_dispatch(self, x, ids, gates, S: int, k: int, e_local: int, site: int) -> None:
        target = self._ep_target(site)
        par, g = target & 1, self.g
        counts = [0] * self.world
        for i in range(S * k):
            d = int(ids[i]) // e_local
            p = counts[d]
            counts[d] += 1
            g.ep_recv[d][par, self.rank, p] = x[i // k]
            g.ep_meta[d][par, self.rank, p] = torch.tensor([int(ids[i]), i, 0, 0], dtype=torch.int32)
            g.ep_gatev[d][par, self.rank, p] = gates[i]
        for d in range(self.world):
            g.ep_count[d][par, self.rank] = counts[d]
        self.log.append(("epd", site, target))
        g.signal_all(self.rank, CH_EPD, target)

    def ep_mask(self, S: int, k: int, e_local: int, site: int):
        target = self._ep_target(site)
        par, g = target & 1, self.g
        ok = g.wait_all(self.rank, CH_EPD, target, site)
        cap = self.ep_cap
        ids = torch.full((self.world * cap,), -1, dtype=torch.int32)
        gate = torch.zeros(self.world * cap, dtype=torch.float32)
        if ok:
            for src in range(self.world):
                n = int(g.ep_count[self.rank][par, src])
                ids[src * cap:src * cap + n] = g.ep_meta[self.rank][par, src, :n, 0]
                gate[src * cap:src * cap + n] = g.ep_gatev[self.rank][par, src, :n]
        self.ep_ids, self.ep_gate = ids, gate
        return ids, gate

    def ep_gather(self, sorted_rows, n_tiles, block: int, max_tiles: int, xs, gate_sorted, S: int, k: int, e_local: int,
                  site: int) -> None:
        par = self._ep_target(site) & 1
        flat = self.g.ep_recv[self.rank][par].reshape(self.world * self.ep_cap, -1)
        for p in range(int(n_tiles[0]) * block):
            i = int(sorted_rows[p])
            if i < 0:
                xs[p].zero_()
                gate_sorted[p] = 0.0
            else:
                xs[p] = flat[i]
                gate_sorted[p] = self.ep_gate[i]

    def ep_combine(self, y, pos, S: int, k: int, e_local: int, site: int) -> None:
        target = self._ep_target(site)
        par, g, cap = target & 1, self.g, self.ep_cap
        for idx in range(self.world * cap):
            p = int(pos[idx])
            if p < 0:
                continue
            src = idx // cap
            row = int(g.ep_meta[self.rank][par, src, idx - src * cap, 1])
            g.ep_back[src][par, row] = y[p]
        self.log.append(("epc", site, target))
        g.signal_all(self.rank, CH_EPC, target)

    def ep_finish(self, S: int, k: int, e_local: int, site: int) -> None:
        target = self._ep_target(site)
        par = target & 1
        if not self.g.wait_all(self.rank, CH_EPC, target, site):
            return
        back = self.g.ep_back[self.rank][par]
        for t in range(S):
            v = self.h_shard[t].float()
            for j in range(k):
                v = v + back[t * k + j].float()
            self.h_shard[t] = E._bf(v)

    def _reduce(self, h, rows: int, rs_site: int, slot_rows_from=None):
        target = self._target(rs_site, self.rs_sites)
        self.g.wait_all(self.rank, CH_RS, target, rs_site)
        v = h[:rows].float()
        for r in range(self.world):             # rank order: every rank computes the same sums
            v = v + self.g.inbox[self.rank][target & 1, r, :rows].float()
        h[:rows] = E._bf(v)

    def norm_oneshot(self, h, w, x_out, rows: int, eps: float, rs_site: int) -> None:
        if rs_site >= 0:
            self._reduce(h, rows, rs_site)
        E.rmsnorm(h[:rows], w, eps, out=x_out[:rows])

    def norm(self, w, S: int, eps: float, ag_site: int, rs_site: int) -> None:
        if rs_site >= 0:
            self._reduce(self.h_shard, S, rs_site)
        y = E.rmsnorm(self.h_shard[:S], w, eps)
        target = self._target(ag_site, self.ag_sites)
        for d in range(self.world):
            self.g.xs[d][target & 1, self.rank * S:(self.rank + 1) * S] = y
        self.log.append(("ag", ag_site, target))
        self.g.signal_all(self.rank, CH_AG, target)

    def gemm(self, epi, x, W, out, S: int, ag_site: int = -1, rs_site: int = -1) -> None:
        R = self.world * S
        if ag_site >= 0:
            target = self._target(ag_site, self.ag_sites)
            self.g.wait_all(self.rank, CH_AG, target, ag_site)
            X = self.g.xs[self.rank][target & 1, :R]
        else:
            X = x[:R]
        y = X.float() @ W.float().T
        if rs_site >= 0:
            target = self._target(rs_site, self.rs_sites)
            yb = E._bf(y)
            for d in range(self.world):         # token row t belongs to rank t // S
                self.g.inbox[d][target & 1, self.rank, :S] = yb[d * S:(d + 1) * S]
            self.log.append(("rs", rs_site, target))
            self.g.signal_all(self.rank, CH_RS, target)
        else:
            E._epilogue(y, epi, out[:R], None)

    def argmax_exchange(self, part, rows: int, groups: int, vocab_total: int, out) -> None:
        target = self.ax_count + 1
        n = rows * groups * 3
        flat = part.reshape(-1)[:n]
        for d in range(self.world):
            if d != self.rank:
                self.g.ax[d][target & 1, self.rank, :n] = flat
        self.g.signal_all(self.rank, CH_AX, target)
        self.ax_count = target
        ok = True
        for r in range(self.world):
            if r == self.rank:
                continue
            why = self.g.wait_flag(self.rank, CH_AX, r, target)
            if not why and int(self.g.flags[self.rank, CH_POISON, r]) != 0:
                why = PEER_FAILED
            if why:
                self.g.fail(self.rank, why, (1 << 20) + r)
                ok = False
                break
        if not ok:
            out[:rows, 0], out[:rows, 1] = 0, -1
            return
        tables = [flat if r == self.rank else self.g.ax[self.rank][target & 1, r, :n] for r in range(self.world)]
        E.argmax_combine(torch.stack(tables).view(self.world, rows, groups, 3), rows, groups, vocab_total, out)

    # ---- the library-collective interface, for steps that are not fused (prefill chunks, sampling rules) ----------
    def _exchange_host(self, t: torch.Tensor) -> List[torch.Tensor]:
        box = self.g.__dict__.setdefault("_box", [None] * self.world)
        box[self.rank] = t.clone()
        self.g.barrier.wait(timeout=60)
        got = [b.clone() for b in box]
        self.g.barrier.wait(timeout=60)
        return got

    def row_parallel(self, engine, x, W, T: int):
        p = self.partial[:T]
        engine._linear(x, W, K.EPI_STORE, p)
        self.all_reduce(p)
        engine._count()
        K.add(engine.h[:T], p, out=engine.h[:T])
        return None

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        self.library_collectives += 1           # what a step on the library path would hand to NCCL
        parts = self._exchange_host(t)
        acc = parts[0].float()
        for p in parts[1:]:
            acc = acc + p.float()
        t.copy_(acc.to(t.dtype))
        return t

    def all_gather(self, out: torch.Tensor, inp: torch.Tensor) -> None:
        self.library_collectives += 1
        parts = self._exchange_host(inp)
        out.view(self.world, -1).copy_(torch.stack([p.reshape(-1) for p in parts]))

    def drain(self) -> None:
        self.g.request_abort(self.rank)

    def close(self) -> None:
        pass
