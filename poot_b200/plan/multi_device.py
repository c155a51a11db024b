"""Multi-device plan: topology, placement, communication rows and per-device accounting, admitted before any device
work.

The four parts of the reference's multi-device planner (crates/poot-graph-plan/src/multi_device/{topology,placement,
communication,accounting}.rs):

* ``Topology`` - every device and every directed link is supplied explicitly: identity, usable bytes, and what each link
  can do (peer loads / stores, in-switch reductions) at what measured rate.  Nothing is inferred from a shape; the
  order of the devices is meaningful (the same set in another order is another plan).
* ``Placement`` - each host-owned weight is resident either replicated on named devices or as exact disjoint byte
  ranges, never both and never overlapping; ranges respect the owner's encoding granule (a packed block is not cut).
* ``Communication`` - the ordered transfer / reduction / exchange rows of one step with their participants, bytes and
  explicit producer -> consumer edges, each admitted against the capabilities of the links it crosses.
* ``Accounting`` - per-device byte categories with checked totals; every device passes on its own (aggregate capacity
  across the group is never consulted: one deficient device rejects the plan).

``plan_tensor_parallel`` builds all four for the engine's tensor- / expert-parallel program of a decoder configuration,
which is what ``poot-serve`` admits a ``tensor:`` or ``expert:`` placement against before any rank loads a byte, and what
the roofline of a fused compute + collective launch is computed from (bytes that must cross a link over the link's
measured rate against the launch's FLOPs over the measured GEMM rate).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from ..models.config import DecoderConfig


class MultiDeviceError(ValueError):
    """A plan that cannot be admitted; the message names the device, link or row."""


# ---- topology ----------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Device:
    id: int
    usable_bytes: int
    backend: str = "sm_100a"


@dataclass(frozen=True)
class Link:
    src: int
    dst: int
    gbs: float                       # measured rate of this direction
    peer_access: bool = True         # loads and stores from a kernel on ``src`` into ``dst``'s memory
    in_switch_reduce: bool = False   # multimem reductions through the switch


@dataclass
class Topology:
    devices: List[Device]
    links: List[Link]

    def __post_init__(self):
        ids = [d.id for d in self.devices]
        if len(set(ids)) != len(ids):
            raise MultiDeviceError("device identities repeat")
        known = set(ids)
        for l in self.links:
            if l.src not in known or l.dst not in known or l.src == l.dst:
                raise MultiDeviceError(f"link {l.src}->{l.dst} names a device outside the topology")
        self._link = {(l.src, l.dst): l for l in self.links}

    def link(self, src: int, dst: int) -> Link:
        l = self._link.get((src, dst))
        if l is None:
            raise MultiDeviceError(f"no link from device {src} to device {dst}")
        return l

    @staticmethod
    def nvswitch(ordinals: Sequence[int], usable_bytes: int, gbs: float = 770.0, in_switch_reduce: bool = True) -> "Topology":
        """Every listed GPU reaches every other at full rate through the switch (one B200 node)."""
        devs = [Device(o, usable_bytes) for o in ordinals]
        links = [Link(a, b, gbs, True, in_switch_reduce) for a in ordinals for b in ordinals if a != b]
        return Topology(devs, links)


# ---- placement -----------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class HostOwner:
    name: str
    nbytes: int
    granule: int = 1                 # bytes of one encoding unit: a resident range starts and ends on a multiple


@dataclass(frozen=True)
class Resident:
    owner: str
    device: int
    lo: int
    hi: int                          # byte range [lo, hi) of the owner; the whole extent for a replica


@dataclass
class Placement:
    owners: Dict[str, HostOwner] = field(default_factory=dict)
    residents: List[Resident] = field(default_factory=list)

    def replicate(self, owner: HostOwner, devices: Sequence[int]) -> None:
        self.owners[owner.name] = owner
        self.residents += [Resident(owner.name, d, 0, owner.nbytes) for d in devices]

    def shard(self, owner: HostOwner, devices: Sequence[int]) -> None:
        """Equal disjoint ranges in device order, cut on granule boundaries."""
        self.owners[owner.name] = owner
        n = len(devices)
        units = owner.nbytes // owner.granule
        if owner.nbytes % owner.granule or units % n:
            raise MultiDeviceError(f"{owner.name}: {owner.nbytes} bytes do not split into {n} ranges of whole {owner.granule}-byte units")
        per = units // n * owner.granule
        self.residents += [Resident(owner.name, d, i * per, (i + 1) * per) for i, d in enumerate(devices)]

    def validate(self, topo: Topology) -> None:
        known = {d.id for d in topo.devices}
        by_owner: Dict[str, List[Resident]] = {}
        for r in self.residents:
            if r.device not in known:
                raise MultiDeviceError(f"{r.owner}: resident on device {r.device}, which the topology does not have")
            o = self.owners[r.owner]
            if not (0 <= r.lo < r.hi <= o.nbytes) or r.lo % o.granule or r.hi % o.granule:
                raise MultiDeviceError(f"{r.owner}: range [{r.lo}, {r.hi}) is outside the owner or cuts a {o.granule}-byte unit")
            by_owner.setdefault(r.owner, []).append(r)
        for name, rs in by_owner.items():
            o = self.owners[name]
            whole = [r for r in rs if (r.lo, r.hi) == (0, o.nbytes)]
            if whole and len(whole) != len(rs):
                raise MultiDeviceError(f"{name}: replicated and sharded at the same time")
            if whole:
                if len({r.device for r in whole}) != len(whole):
                    raise MultiDeviceError(f"{name}: replicated twice on one device")
                continue
            spans = sorted((r.lo, r.hi) for r in rs)
            pos = 0
            for lo, hi in spans:
                if lo != pos:
                    raise MultiDeviceError(f"{name}: byte ranges {'overlap' if lo < pos else 'leave a gap'} at {min(lo, pos)}")
                pos = hi
            if pos != o.nbytes:
                raise MultiDeviceError(f"{name}: ranges cover {pos} of {o.nbytes} bytes")

    def bytes_on(self, device: int) -> int:
        return sum(r.hi - r.lo for r in self.residents if r.device == device)


# ---- communication ---------------------------------------------------------------------------------------------------
KINDS = ("all_reduce", "reduce_scatter", "all_gather", "all_to_all", "send")


@dataclass
class CommRow:
    id: int
    kind: str
    participants: Tuple[int, ...]
    bytes_per_rank: int                  # bytes each participant contributes
    after: Tuple[int, ...] = ()          # rows that must have completed (producer -> consumer edges)
    fused_into: Optional[str] = None     # the launch that performs it in-kernel (None: a library collective)
    needs: str = "peer_access"           # capability every crossed link must have: peer_access | in_switch_reduce

    def link_bytes(self) -> int:
        """Bytes that leave one participant over its links (what the link-time side of the roofline divides)."""
        w = len(self.participants)
        if w < 2:
            return 0
        if self.kind == "all_reduce":
            # one-shot form: every rank sends its whole partial to every peer; ring / in-switch forms send 2 (w-1)/w
            return self.bytes_per_rank * (w - 1) if self.fused_into else 2 * self.bytes_per_rank * (w - 1) // w
        if self.kind in ("reduce_scatter", "all_gather", "all_to_all"):
            return self.bytes_per_rank * (w - 1) // w
        return self.bytes_per_rank


@dataclass
class Communication:
    rows: List[CommRow] = field(default_factory=list)

    def add(self, kind: str, participants: Sequence[int], bytes_per_rank: int, after: Sequence[int] = (),
            fused_into: Optional[str] = None, needs: str = "peer_access") -> int:
        if kind not in KINDS:
            raise MultiDeviceError(f"unknown collective {kind!r}")
        rid = len(self.rows)
        if any(a >= rid or a < 0 for a in after):
            raise MultiDeviceError(f"row {rid} depends on a row that does not precede it")
        self.rows.append(CommRow(rid, kind, tuple(participants), int(bytes_per_rank), tuple(after), fused_into, needs))
        return rid

    def validate(self, topo: Topology) -> None:
        for r in self.rows:
            if len(set(r.participants)) != len(r.participants) or len(r.participants) < 2:
                raise MultiDeviceError(f"row {r.id} ({r.kind}): participants must be two or more distinct devices")
            for a in r.participants:
                for b in r.participants:
                    if a == b:
                        continue
                    l = topo.link(a, b)
                    if not getattr(l, r.needs):
                        raise MultiDeviceError(f"row {r.id} ({r.kind}): link {a}->{b} lacks {r.needs}")

    def seconds(self, topo: Topology) -> float:
        """Lower bound on the link time of the rows as ordered (rows are serial along their dependency chain)."""
        t = 0.0
        for r in self.rows:
            gbs = min(topo.link(a, b).gbs for a in r.participants for b in r.participants if a != b)
            t += r.link_bytes() / (gbs * 1e9)
        return t


# ---- accounting ------------------------------------------------------------------------------------------------------
CATEGORIES = ("weights", "kv", "activations", "exchange", "workspace")


@dataclass
class Accounting:
    per_device: Dict[int, Dict[str, int]] = field(default_factory=dict)

    def charge(self, device: int, category: str, nbytes: int) -> None:
        if category not in CATEGORIES:
            raise MultiDeviceError(f"unknown byte category {category!r}")
        if nbytes < 0:
            raise MultiDeviceError(f"device {device}: negative {category} bytes")
        d = self.per_device.setdefault(device, {c: 0 for c in CATEGORIES})
        d[category] += int(nbytes)

    def total(self, device: int) -> int:
        return sum(self.per_device.get(device, {}).values())

    def admit(self, topo: Topology, reserve: int = 256 << 20) -> None:
        """Every device passes its own total; a deficient device in any position rejects the plan."""
        for d in topo.devices:
            need = self.total(d.id) + reserve
            if need > d.usable_bytes:
                cats = ", ".join(f"{c} {v / 2**30:.2f}" for c, v in self.per_device.get(d.id, {}).items() if v)
                raise MultiDeviceError(f"device {d.id}: {need / 2**30:.2f} GiB planned ({cats}; reserve "
                                       f"{reserve / 2**30:.2f}) exceeds its {d.usable_bytes / 2**30:.2f} GiB")


# ---- the engine's tensor- / expert-parallel program ----------------------------------------------------------------------
@dataclass
class MultiDevicePlan:
    topology: Topology
    placement: Placement
    communication: Communication
    accounting: Accounting
    flops_per_rank: float = 0.0

    def validate(self, reserve: int = 256 << 20) -> "MultiDevicePlan":
        self.placement.validate(self.topology)
        self.communication.validate(self.topology)
        self.accounting.admit(self.topology, reserve)
        return self

    def roofline_seconds(self, tflops: float, hbm_gbs: float) -> Dict[str, float]:
        """The three floors of one step per rank: math at the measured GEMM rate, resident weight bytes at the measured
        copy rate, and link bytes at the links' measured rate.  The target time is the largest."""
        topo = self.topology
        d0 = topo.devices[0].id
        w = self.accounting.per_device.get(d0, {}).get("weights", 0)
        out = {"compute": self.flops_per_rank / (tflops * 1e12), "hbm": w / (hbm_gbs * 1e9),
               "links": self.communication.seconds(topo)}
        out["target"] = max(out.values())
        return out


def plan_tensor_parallel(cfg: DecoderConfig, topo: Topology, rows: int, num_blocks: int, step_tokens: int,
                         comm: str = "fused", itemsize: int = 2, program: str = "one_shot") -> MultiDevicePlan:
    """Placement, communication rows, accounting and FLOPs of one step of ``step_tokens`` tokens on the engine's
    tensor-parallel (dense) or expert-parallel (routed) program over the devices of ``topo``.

    ``program="one_shot"``: every rank holds every token; each projection that ends a block is an all-reduce.
    ``program="rs_ag"``: the token-sharded program - a block's result is reduce-scattered into the rank's share of the
    rows and all-gathered in front of the next block's first projection; a routed block exchanges rows instead: an
    all-to-all that sends every (token, slot) row to the rank owning its expert and one that brings the results back
    (``runtime/moe.py::moe_forward_sharded``, ``csrc/kernels/ep_exchange.cu``)."""
    if program not in ("one_shot", "rs_ag"):
        raise MultiDeviceError(f"unknown tensor-parallel program {program!r}")
    devs = [d.id for d in topo.devices]
    w = len(devs)
    H, D, L, V = cfg.hidden, cfg.head_dim, cfg.n_layers, cfg.vocab
    if cfg.n_heads % w or (cfg.n_kv_heads % w and w % cfg.n_kv_heads):
        raise MultiDeviceError(f"{cfg.n_heads} query / {cfg.n_kv_heads} K/V heads do not divide over {w} devices")
    place = Placement()
    q, kv = cfg.n_heads * D, cfg.n_kv_heads * D
    for l in range(L):
        p = f"layers.{l}."
        for name, rows_, cols in ((p + "attn_q", q, H), (p + "attn_k", kv, H), (p + "attn_v", kv, H)):
            own = HostOwner(name, rows_ * cols * itemsize, cols * itemsize)                 # cut by output rows
            (place.shard if rows_ // D >= w else place.replicate)(own, devs)
        place.shard(HostOwner(p + "attn_o", H * q * itemsize, itemsize * (q // w)), devs)     # cut along the input dim
        for n in ("attn_norm", "ffn_norm"):
            place.replicate(HostOwner(p + n, H * itemsize), devs)
        if cfg.moe_layer(l):
            E, F = cfg.n_experts, cfg.moe_ffn
            if E % w:
                raise MultiDeviceError(f"{E} experts do not divide over {w} devices")
            place.replicate(HostOwner(p + "ffn_router", E * H * itemsize), devs)
            place.shard(HostOwner(p + "experts_in", E * 2 * F * H * itemsize, 2 * F * H * itemsize), devs)   # whole experts
            place.shard(HostOwner(p + "experts_out", E * H * F * itemsize, H * F * itemsize), devs)
        else:
            F = cfg.ffn
            place.shard(HostOwner(p + "ffn_gate_up", 2 * F * H * itemsize, 2 * H * itemsize), devs)
            place.shard(HostOwner(p + "ffn_down", H * F * itemsize, itemsize * (F // w)), devs)
    place.replicate(HostOwner("embed", V * H * itemsize), devs)
    place.replicate(HostOwner("final_norm", H * itemsize), devs)
    place.shard(HostOwner("lm_head", V * H * itemsize, H * itemsize), devs)

    T = step_tokens
    fused = comm == "fused" and T <= 128
    cm = Communication()
    prev: Tuple[int, ...] = ()
    S = -(-T // w)                                  # a rank's share of the step's rows under the sharded program
    for l in range(L):
        for site in ("o_proj", "down_proj"):
            if program == "rs_ag":
                if site == "down_proj" and cfg.moe_layer(l):
                    # every (token, slot) row of the rank's share travels to its expert's rank and back
                    out_rows = S * cfg.top_k * H * itemsize
                    rid = cm.add("all_to_all", devs, out_rows, prev, fused_into=f"ep_dispatch[{l}]" if comm == "fused" else None)
                    rid = cm.add("all_to_all", devs, out_rows, (rid,), fused_into=f"ep_combine[{l}]" if comm == "fused" else None)
                    prev = (rid,)
                    continue
                gemm = "gemm_tiled_tp" if w * S > 128 else "gemm_skinny_tp"
                rid = cm.add("reduce_scatter", devs, w * S * H * itemsize, prev, fused_into=f"{gemm}[{l}.{site}]" if comm == "fused" else None)
                rid = cm.add("all_gather", devs, w * S * H * itemsize, (rid,), fused_into=f"{gemm}[{l}.{site}.next]" if comm == "fused" else None)
            elif fused:
                rid = cm.add("all_reduce", devs, T * H * itemsize, prev, fused_into=f"gemm_skinny_tp[{l}.{site}]")
            else:
                rid = cm.add("all_reduce", devs, T * H * itemsize, prev, needs="peer_access")
            prev = (rid,)
    cm.add("all_gather", devs, rows * 3 * 4 * max(1, (V // w + 2047) // 2048), prev,
           fused_into="tp_argmax_exchange" if fused else None)

    acct = Accounting()
    for d in devs:
        acct.charge(d, "weights", place.bytes_on(d))
        hkv = max(cfg.n_kv_heads // w, 1)
        acct.charge(d, "kv", num_blocks * L * 2 * hkv * 16 * D * itemsize)            # blocks of 16 positions, K and V
        tok = max(T, 128 if w > 1 else T)
        ffn_local = cfg.moe_ffn if cfg.is_moe else cfg.ffn // w
        acct.charge(d, "activations", itemsize * tok * (2 * H + (cfg.n_heads // w + 2 * hkv) * D + 2 * (cfg.n_heads // w) * D + ffn_local)
                    + rows * (V // w) * 4 * 3)
        if comm == "fused":
            acct.charge(d, "exchange", 1024 + 2 * w * 128 * H * itemsize + 2 * 128 * H * itemsize)
    ffn_flops = (cfg.top_k * 3 * cfg.moe_ffn if cfg.is_moe else 3 * cfg.ffn) * H
    flops = 2.0 * T * L * ((q + 2 * kv) * H + q * H + ffn_flops) / w + 2.0 * rows * V * H / w
    return MultiDevicePlan(topo, place, cm, acct, flops)
