"""Tensor-parallel communication back ends of the device engine.

``NcclComm`` is the baseline: a row-parallel projection writes its partial result, NCCL all-reduces it and a
kernel adds it to the residual stream - one library collective per projection, captured in the step graph.

``FusedComm`` is the product path for steps of up to 128 padded token rows (decode batches): the o_proj /
down_proj GEMMs scatter their output tiles straight into the owner ranks' inboxes over NVLink
(GEMM + reduce-scatter in one kernel), the consumer kernel reduces the inboxes into the token-sharded
residual stream and normalises it (reduce + RMSNorm), pushes the rows into every rank's gather buffer, and the following qkv / gate_up GEMM's producer
warp waits for the ranks' flags before its first activation load (all-gather + GEMM without a separate collective;
a remote row crosses NVLink once and is then read from local memory by every CTA).
Larger steps (prefill chunks) fall back to the NCCL form.

Sharding follows the reference's Megatron layouts (crates/poot-graph-plan/src/passes/sharding.rs:219-251);
its collective lowering - every rank reads every peer's partial once, summed in rank order so all ranks get
bit-identical results (sharding.rs:1219-1250) - is kept, but runs inside kernels instead of as
world*(world-1) host-issued copies per collective.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import cuda_ops as K
from ..ops._lib import check, kernels
from .guarded_layout import CommBufferOverrun, GuardedLayout
from .symm import SymmetricBlock

FLAG_BYTES = 6 * 8 * 4             # six channels of eight int32 flag words (tp_common.cuh: TP_FLAG_WORDS)

_P = c_void_p


class NcclComm:
    """All-reduce through NCCL after a local GEMM (the baseline, not the product)."""

    fused = False

    def __init__(self, rank: int, world: int, device: torch.device, group=None):
        self.rank, self.world, self.device, self.group = rank, world, device, group

    def attach(self, engine) -> None:
        T, H = engine.max_tokens, engine.cfg.hidden
        self.partial = torch.zeros(T, H, dtype=torch.bfloat16, device=self.device)

    def row_parallel(self, engine, x: torch.Tensor, W: torch.Tensor, T: int):
        """``h += allreduce(x @ W^T)``."""
        p = self.partial[:T]
        engine._linear(x, W, K.EPI_STORE, p)
        with K.timed_region("nccl_all_reduce"):
            dist.all_reduce(p, group=self.group)
        engine._count()
        K.add(engine.h[:T], p, out=engine.h[:T])
        return None

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        """Sum ``t`` over the ranks in place (a projection's partial that a norm consumes before the residual add)."""
        with K.timed_region("nccl_all_reduce"):
            dist.all_reduce(t, group=self.group)
        return t

    def all_gather(self, out: torch.Tensor, inp: torch.Tensor) -> None:
        with K.timed_region("nccl_all_gather"):
            # flat views: the same bytes, and the form every backend of the process group accepts
            dist.all_gather_into_tensor(out.view(-1), inp.reshape(-1), group=self.group)

    def rendezvous(self) -> None:
        """Host rendezvous of all ranks with the device idle on both sides: everything queued so far has finished
        on every rank when this returns.  Called before the first launch of any program whose kernels wait on other
        ranks, so no rank can start such a program seconds ahead of its peers."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)


class FusedComm(NcclComm):
    """In-kernel NVLink reduce-scatter / all-gather fused with the projections' GEMMs."""

    fused = True
    MAX_ROWS = 128                 # rows of a one-shot slot, and the largest step the skinny (swap-AB) kernels serve
    MAX_SHARD_ROWS = 4096          # largest padded step of the token-sharded program (tiled GEMMs above 128 rows)

    def __init__(self, rank: int, world: int, device: torch.device, group=None, probe: bool = True):
        super().__init__(rank, world, device, group)
        self.probe_links = probe
        self.block: Optional[SymmetricBlock] = None

    def attach(self, engine) -> None:
        super().attach(engine)
        H, w = engine.cfg.hidden, self.world
        self.H = H
        # the sharded program serves steps up to max_rows padded rows: what the engine's buffers hold, in whole 128-row tiles
        self.max_rows = max(self.MAX_ROWS, min(self.MAX_SHARD_ROWS, engine.max_tokens // 128 * 128))
        self.s_max = self.max_rows // w
        # layout of the symmetric block: 1 KiB aligned regions, each followed by guard words that check_guards() reads
        # inbox: one-shot form [2][world][MAX_ROWS][H] or sharded form [2][world][S][H] with world * S <= max_rows
        inbox_bytes = 2 * max(w * self.MAX_ROWS, self.max_rows) * H * 2
        xs_bytes = 2 * self.max_rows * H * 2
        # greedy-pick exchange: [2][world][ax_cap] int32, one stage-1 table [rows, groups, 3] per rank and parity
        self.ax_cap = engine.max_seqs * K.argmax_groups(max(1, engine.cfg.vocab // w)) * 3
        ax_bytes = 2 * w * self.ax_cap * 4
        regions = [("flags", FLAG_BYTES), ("inbox", inbox_bytes), ("xs", xs_bytes), ("ax", ax_bytes)]
        self.ep_cap = 0
        cfg = engine.cfg
        if cfg.is_moe and getattr(engine.w, "ep_world", 1) == w:
            # expert-parallel exchange over a token-sharded stream: receive area [2][world][cap][H] with its metadata
            # and counts, combine area [2][cap][H]; cap = a rank's (token, slot) rows of the largest sharded step
            self.ep_cap = self.s_max * cfg.top_k
            regions += [("ep_recv", 2 * w * self.ep_cap * H * 2), ("ep_meta", 2 * w * self.ep_cap * 16),
                        ("ep_count", 2 * w * 4), ("ep_back", 2 * self.ep_cap * H * 2)]
        self.layout = GuardedLayout(regions)
        self.off_flags, self.off_inbox = self.layout.offset("flags"), self.layout.offset("inbox")
        self.off_xs, self.off_ax = self.layout.offset("xs"), self.layout.offset("ax")
        self.block = SymmetricBlock(self.layout.total, self.rank, w, self.device, self.group)
        if self.probe_links:
            self.block.probe(self.group)                  # leaves the block zeroed
        self._write_guards()
        self.last_overrun: Optional[CommBufferOverrun] = None
        self.flags_peer = self.block.ptr_array(self.off_flags)
        self.inbox_peer = self.block.ptr_array(self.off_inbox)
        self.xs_peer = self.block.ptr_array(self.off_xs)
        self.ax_peer = self.block.ptr_array(self.off_ax)
        if self.ep_cap:
            i32 = dict(dtype=torch.int32, device=self.device)
            self.ep_peers = [self.block.ptr_array(self.layout.offset(n)) for n in ("ep_recv", "ep_meta", "ep_count", "ep_back")]
            self.ep_sites = engine.cfg.n_layers
            self.ep_dest, self.ep_dpos = torch.zeros(self.ep_cap, **i32), torch.zeros(self.ep_cap, **i32)
            self.ep_counts = torch.zeros(8, **i32)
            self.ep_ids = torch.zeros(w * self.ep_cap, **i32)
            self.ep_gate = torch.zeros(w * self.ep_cap, dtype=torch.float32, device=self.device)
            ep_common = [c_int] * 9 + [_P] * 9
            K.register_signature("poot_ep_plan", [_P, c_int, c_int, c_int, _P, _P, _P, _P])
            K.register_signature("poot_ep_dispatch", [_P, c_int, _P, _P, _P, _P, _P] + ep_common)
            K.register_signature("poot_ep_mask", [_P, _P, _P, _P] + ep_common)
            K.register_signature("poot_ep_gather", [_P, _P, _P, _P, c_int, c_int, _P, _P] + ep_common)
            K.register_signature("poot_ep_combine", [_P, _P, _P] + ep_common)
            K.register_signature("poot_ep_finish", [_P, _P] + ep_common)
        self.ax_count = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.ticket = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.h_shard = torch.zeros(self.s_max, H, dtype=torch.bfloat16, device=self.device)
        L = engine.cfg.n_layers
        self.rs_sites = 2 * L
        self.ag_sites = 2 * L + 1
        K.register_signature("poot_tp_begin_step", [_P, _P, _P])
        K.register_signature("poot_tp_argmax_exchange", [_P, c_int, c_int, c_int, c_int, _P, _P, c_int, c_int, _P, _P, _P,
                                                         _P, _P, _P])
        self._exchange = K.fn("poot_tp_argmax_exchange")
        K.register_signature("poot_tp_norm", [_P, _P, _P, _P, _P, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_int,
                                              c_int, c_int, _P, _P, _P, _P, _P, _P])
        K.register_signature("poot_gemm_skinny_tp", [c_int, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                     c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P, c_int, c_int, _P,
                                                     _P, _P])
        K.register_signature("poot_tp_end_step", [_P, _P])
        K.register_signature("poot_gemm_tiled_tp", [c_int, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                    c_int, c_int, c_int, _P, _P, _P, _P, c_int, _P, _P, _P])
        self._gemm_tiled = K.fn("poot_gemm_tiled_tp")
        self._begin = K.fn("poot_tp_begin_step")
        self._end = K.fn("poot_tp_end_step")
        self._norm = K.fn("poot_tp_norm")
        self._gemm = K.fn("poot_gemm_skinny_tp")

    # ---- geometry -------------------------------------------------------------------------------------------
    def rows_for(self, T: int) -> int:
        """Padded step rows (world * S): one of 16/32/64/128 for the skinny kernels, whole 128-row tiles above that for
        the tiled ones; 0 when the step is too large for the sharded program."""
        need = max(T, 8 * self.world)
        for r in (16, 32, 64, 128):
            if r >= need and r % (8 * self.world) == 0:
                return r
        r = (need + 127) // 128 * 128
        return r if r <= self.max_rows else 0

    # ---- launches -------------------------------------------------------------------------------------------
    def begin_step(self) -> None:
        """First launch of a fused step: advances the epoch and starts the step's wait budget."""
        check(self._begin(self.epoch.data_ptr(), K.status_word(self.device).data_ptr(), K._stream()), "tp_begin_step")

    def gather_rows(self, idx: torch.Tensor, out: torch.Tensor, rows: int, S: int, ag_site: int) -> None:
        """``out[b] = gathered rows[idx[b]]`` of ``ag_site`` once every rank's rows have landed (int64 ``idx``)."""
        K.register_signature("poot_tp_gather_rows", [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P])
        b = self.block
        check(K.fn("poot_tp_gather_rows")(b.ptr(self.rank, self.off_xs), idx.data_ptr(), out.data_ptr(), rows, self.H,
                                          self.world, self.rank, S, ag_site, self.ag_sites, self.epoch.data_ptr(),
                                          b.ptr(self.rank, self.off_flags), K.status_word(self.device).data_ptr(),
                                          K._stream()), "tp_gather_rows")

    def end_step(self) -> None:
        """Last launch of a fused step: clears the step deadline, so a later step that does not begin with
        ``begin_step`` (one on the library collectives) is not judged against a deadline that has passed."""
        check(self._end(K.status_word(self.device).data_ptr(), K._stream()), "tp_end_step")

    def argmax_exchange(self, part: torch.Tensor, rows: int, groups: int, vocab_total: int, out: torch.Tensor) -> None:
        """Greedy pick over the ranks' vocabulary shards: push this rank's stage-1 table ``part`` [rows, groups, 3]
        into every peer's exchange area and combine the tables received, in one kernel and without a library
        collective (a fused step's graph holds no library collective at all)."""
        b = self.block
        check(self._exchange(part.data_ptr(), rows, groups, self.ax_cap, vocab_total, out.data_ptr(),
                             self.ax_count.data_ptr(), self.world, self.rank, b.ptr(self.rank, self.off_flags),
                             self.flags_peer, self.ax_peer, self.ticket.data_ptr(),
                             K.status_word(self.device).data_ptr(), K._stream()), "tp_argmax_exchange")

    def norm_oneshot(self, h: torch.Tensor, w: torch.Tensor, x_out: torch.Tensor, rows: int, eps: float,
                     rs_site: int) -> None:
        """One-shot all-reduce consumer: ``h += sum_r inbox[r]`` (rank order), ``x_out = rmsnorm(h) * w``; all local."""
        b = self.block
        check(self._norm(h.data_ptr(), b.ptr(self.rank, self.off_inbox), w.data_ptr(), None, x_out.data_ptr(), rows,
                         self.H, float(eps), self.world, self.rank, self.MAX_ROWS, 0, self.ag_sites, rs_site,
                         self.rs_sites, self.epoch.data_ptr(), b.ptr(self.rank, self.off_flags), self.flags_peer,
                         self.ticket.data_ptr(), K.status_word(self.device).data_ptr(), K._stream()), "tp_norm")

    def gemm_allreduce(self, x: torch.Tensor, W: torch.Tensor, rows: int, rs_site: int) -> None:
        """Row-parallel projection whose epilogue writes the partial into every rank's inbox (one-shot all-reduce)."""
        N, Kd = W.shape
        b = self.block
        check(self._gemm(K.EPI_STORE, x.data_ptr(), W.data_ptr(), None, N, Kd, x.stride(0), self.H,
                         K.skinny_cluster(N, Kd), self.world, self.rank, self.MAX_ROWS, -1, self.ag_sites, rs_site,
                         self.rs_sites, self.epoch.data_ptr(), b.ptr(self.rank, self.off_flags), self.flags_peer,
                         self.inbox_peer, self.H, rows, self.ticket.data_ptr(),
                         K.status_word(self.device).data_ptr(), K._stream()), "gemm_skinny_tp")

    def oneshot_ok(self, T: int) -> bool:
        """One-shot all-reduce pays while the partial (T x hidden, sent to world-1 peers) stays small."""
        return T <= 128 and T * (self.world - 1) <= 512

    def norm(self, w: torch.Tensor, S: int, eps: float, ag_site: int, rs_site: int) -> None:
        """Reduce the inboxes of ``rs_site`` (if >= 0) into the residual shard, normalise, publish for ``ag_site``."""
        b = self.block
        check(self._norm(self.h_shard.data_ptr(), b.ptr(self.rank, self.off_inbox), w.data_ptr(),
                         self.xs_peer, None, S, self.H, float(eps), self.world, self.rank, S, ag_site,
                         self.ag_sites, rs_site, self.rs_sites, self.epoch.data_ptr(), b.ptr(self.rank, self.off_flags),
                         self.flags_peer, self.ticket.data_ptr(), K.status_word(self.device).data_ptr(), K._stream()),
              "tp_norm")

    def gemm(self, epi: int, x: Optional[torch.Tensor], W: torch.Tensor, out: Optional[torch.Tensor], S: int,
             ag_site: int = -1, rs_site: int = -1) -> None:
        """Skinny GEMM with a gathered X operand (``ag_site``) and / or a scattered output (``rs_site``)."""
        N, Kd = W.shape
        ck = K.skinny_cluster(N, Kd)
        ldx = x.stride(0) if x is not None else Kd
        ldo = out.stride(0) if out is not None else self.H
        b = self.block
        xptr = b.ptr(self.rank, self.off_xs) if ag_site >= 0 else x.data_ptr()
        if self.world * S > self.MAX_ROWS:
            # prefill-sized step: the tiled tcgen05 GEMM with the gathered operand and / or the scattered result
            check(self._gemm_tiled(epi, xptr, W.data_ptr(), None if out is None else out.data_ptr(), N, Kd, ldx, ldo,
                                   self.world, self.rank, S, ag_site, self.ag_sites, rs_site, self.rs_sites,
                                   self.epoch.data_ptr(), b.ptr(self.rank, self.off_flags), self.flags_peer, self.inbox_peer,
                                   self.H, self.ticket.data_ptr(), K.status_word(self.device).data_ptr(), K._stream()),
                  "gemm_tiled_tp")
            return
        check(self._gemm(epi, xptr, W.data_ptr(), None if out is None else out.data_ptr(),
                         N, Kd, ldx, ldo, ck, self.world, self.rank, S, ag_site, self.ag_sites, rs_site, self.rs_sites,
                         self.epoch.data_ptr(), b.ptr(self.rank, self.off_flags), self.flags_peer, self.inbox_peer,
                         self.H, 0, self.ticket.data_ptr(), K.status_word(self.device).data_ptr(), K._stream()),
              "gemm_skinny_tp")

    # ---- expert-parallel exchange over the token-sharded stream (csrc/kernels/ep_exchange.cu) ---------------------------
    def norm_local(self, w: torch.Tensor, x_out: torch.Tensor, S: int, eps: float, rs_site: int) -> None:
        """Reduce the inboxes of ``rs_site`` (if >= 0) into the residual shard and normalise this rank's own rows into
        ``x_out``; nothing is published (the expert exchange sends each row only where its experts are)."""
        b = self.block
        check(self._norm(self.h_shard.data_ptr(), b.ptr(self.rank, self.off_inbox), w.data_ptr(), None, x_out.data_ptr(), S,
                         self.H, float(eps), self.world, self.rank, S, 0, self.ag_sites, rs_site, self.rs_sites,
                         self.epoch.data_ptr(), b.ptr(self.rank, self.off_flags), self.flags_peer,
                         self.ticket.data_ptr(), K.status_word(self.device).data_ptr(), K._stream()), "tp_norm")

    def _ep_common(self, S: int, k: int, e_local: int, site: int):
        b = self.block
        return (self.world, self.rank, S, k, self.ep_cap, self.H, e_local, site, self.ep_sites, self.epoch.data_ptr(),
                b.ptr(self.rank, self.off_flags), self.flags_peer, *self.ep_peers, self.ticket.data_ptr(),
                K.status_word(self.device).data_ptr(), K._stream())

    def _ep_local(self, name: str) -> int:
        return self.block.ptr(self.rank, self.layout.offset(name))

    def ep_dispatch(self, x: torch.Tensor, ids: torch.Tensor, gates: torch.Tensor, S: int, k: int, e_local: int,
                    site: int) -> None:
        """Send every (token, slot) row of this rank's ``S`` tokens to the rank that holds its expert."""
        n = S * k
        check(K.fn("poot_ep_plan")(ids.data_ptr(), n, e_local, self.world, self.ep_dest.data_ptr(), self.ep_dpos.data_ptr(),
                                   self.ep_counts.data_ptr(), K._stream()), "ep_plan")
        check(K.fn("poot_ep_dispatch")(x.data_ptr(), x.stride(0), ids.data_ptr(), gates.data_ptr(), self.ep_dest.data_ptr(),
                                       self.ep_dpos.data_ptr(), self.ep_counts.data_ptr(), *self._ep_common(S, k, e_local, site)),
              "ep_dispatch")

    def ep_mask(self, S: int, k: int, e_local: int, site: int):
        """Wait for every rank's rows; returns ``(expert ids or -1, gates)`` over the ``world * cap`` receive slots."""
        check(K.fn("poot_ep_mask")(self._ep_local("ep_meta"), self._ep_local("ep_count"), self.ep_ids.data_ptr(),
                                   self.ep_gate.data_ptr(), *self._ep_common(S, k, e_local, site)), "ep_mask")
        return self.ep_ids, self.ep_gate

    def ep_gather(self, sorted_rows, n_tiles, block: int, max_tiles: int, xs, gate_sorted, S: int, k: int, e_local: int,
                  site: int) -> None:
        check(K.fn("poot_ep_gather")(self._ep_local("ep_recv"), sorted_rows.data_ptr(), self.ep_gate.data_ptr(),
                                     n_tiles.data_ptr(), block, max_tiles, xs.data_ptr(), gate_sorted.data_ptr(),
                                     *self._ep_common(S, k, e_local, site)), "ep_gather")

    def ep_combine(self, y: torch.Tensor, pos: torch.Tensor, S: int, k: int, e_local: int, site: int) -> None:
        """Send every result row back to the rank that owns its token."""
        check(K.fn("poot_ep_combine")(y.data_ptr(), pos.data_ptr(), self._ep_local("ep_meta"),
                                      *self._ep_common(S, k, e_local, site)), "ep_combine")

    def ep_finish(self, S: int, k: int, e_local: int, site: int) -> None:
        """Wait for every rank's results and add each token's ``k`` rows to the residual shard, in slot order."""
        check(K.fn("poot_ep_finish")(self.h_shard.data_ptr(), self._ep_local("ep_back"),
                                     *self._ep_common(S, k, e_local, site)), "ep_finish")

    def _write_guards(self) -> None:
        def store(off, words):
            self.block.local_tensor(off, (len(words),), torch.int32).copy_(torch.tensor(words, dtype=torch.int32))
        self.layout.write(self.rank, store)
        torch.cuda.synchronize(self.device)

    def check_guards(self) -> None:
        """Read the guard words behind every region of this rank's block (host read after a device sync); raises
        ``CommBufferOverrun`` naming the region a store ran past.  Called at close, before a reset clears the block,
        and by debug runs after a step."""
        torch.cuda.synchronize(self.device)
        self.layout.check(self.rank, lambda off, n: self.block.local_tensor(off, (n,), torch.int32).cpu().tolist())

    def reset(self) -> None:
        """Collective restart of the cross-rank protocol after a failed step: every rank drains, all meet, each zeroes
        its own block (flags, poison words, inboxes) and its counters, all meet again.  Between the two meetings no rank
        launches anything, so no rank can see a half-cleared peer."""
        self.drain()
        K.clear_abort(self.device)
        self.rendezvous()
        try:                            # what the failed step left behind is evidence: look before clearing it
            self.check_guards()
        except CommBufferOverrun as e:
            self.last_overrun = e
        self.block.local_tensor(0, (self.block.nbytes,), torch.uint8).zero_()
        self._write_guards()
        self.epoch.zero_()
        self.ticket.zero_()
        self.ax_count.zero_()
        self.rendezvous()

    def drain(self) -> None:
        """Make every kernel of this rank that is waiting on a peer give up (host abort word), then wait for the
        device to go idle.  After this no kernel of this rank is resident, so the process can unmap peers' memory and
        exit without tearing a context down under a waiting kernel."""
        K.request_abort(self.device)
        torch.cuda.synchronize(self.device)

    def close(self) -> None:
        if self.block is not None:
            self.drain()
            overrun = self.last_overrun
            try:
                self.check_guards()
            except CommBufferOverrun as e:
                overrun = e
            self.block.close()
            self.block = None
            K.clear_abort(self.device)
            if overrun is not None:
                raise overrun


# What "auto" means wherever a tensor-parallel group is built without an explicit choice.  The fused programs are the
# product path; they are selected explicitly (``--comm fused``) until they have been re-validated on more than two
# GPUs with the step deadline, abort word and rendezvous rules in place.
DEFAULT_COMM = "nccl"


def make_comm(kind: str, rank: int, world: int, device: torch.device, group=None):
    if kind == "auto":
        kind = DEFAULT_COMM
    if kind == "nccl":
        return NcclComm(rank, world, device, group)
    if kind == "fused":
        return FusedComm(rank, world, device, group)
    raise ValueError(f"unknown comm kind {kind!r}")
