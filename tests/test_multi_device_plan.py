"""The multi-device planner: explicit topology, placement without duplication, communication rows admitted against
link capabilities, independent per-device accounting (crates/poot-graph-plan/src/multi_device/)."""
import pytest

from poot_b200.models.config import PRESETS
from poot_b200.plan.multi_device import (Accounting, Communication, Device, HostOwner, Link, MultiDeviceError, Placement,
                                         Topology, plan_tensor_parallel)

GIB = 1 << 30


def test_topology_is_explicit_and_ordered():
    t = Topology.nvswitch([0, 1, 2, 3], 170 * GIB)
    assert len(t.links) == 12 and t.link(2, 1).gbs == 770.0
    with pytest.raises(MultiDeviceError, match="no link"):
        Topology([Device(0, GIB), Device(1, GIB)], [Link(0, 1, 100.0)]).link(1, 0)     # links are directed
    with pytest.raises(MultiDeviceError, match="repeat"):
        Topology([Device(0, GIB), Device(0, GIB)], [])
    with pytest.raises(MultiDeviceError, match="outside"):
        Topology([Device(0, GIB)], [Link(0, 5, 1.0)])


def test_placement_never_duplicates_or_cuts_an_encoding_unit():
    t = Topology.nvswitch([0, 1], GIB)
    p = Placement()
    p.shard(HostOwner("w", 144 * 8, granule=144), [0, 1])          # eight Q4_K blocks: four per device
    p.replicate(HostOwner("norm", 64), [0, 1])
    p.validate(t)
    assert p.bytes_on(0) == 144 * 4 + 64
    with pytest.raises(MultiDeviceError, match="whole 144-byte units"):
        Placement().shard(HostOwner("w", 144 * 7, granule=144), [0, 1])
    bad = Placement()
    bad.shard(HostOwner("w", 100), [0, 1])
    bad.residents.append(bad.residents[0])                          # the same range twice
    with pytest.raises(MultiDeviceError, match="overlap"):
        bad.validate(t)
    mixed = Placement()
    mixed.replicate(HostOwner("w", 100), [0])
    mixed.residents.append(type(mixed.residents[0])("w", 1, 0, 50))
    with pytest.raises(MultiDeviceError, match="replicated and sharded"):
        mixed.validate(t)
    gap = Placement()
    gap.owners["w"] = HostOwner("w", 100)
    gap.residents.append(type(mixed.residents[0])("w", 0, 0, 40))
    with pytest.raises(MultiDeviceError, match="cover 40 of 100"):
        gap.validate(t)


def test_communication_rows_are_admitted_against_link_capabilities():
    slow = Topology([Device(0, GIB), Device(1, GIB)], [Link(0, 1, 50.0, peer_access=True), Link(1, 0, 50.0, peer_access=False)])
    c = Communication()
    a = c.add("all_reduce", [0, 1], 1 << 20)
    c.add("all_gather", [0, 1], 1 << 10, after=[a])
    with pytest.raises(MultiDeviceError, match="lacks peer_access"):
        c.validate(slow)
    with pytest.raises(MultiDeviceError, match="does not precede"):
        c.add("send", [0, 1], 8, after=[7])
    ok = Topology.nvswitch([0, 1], GIB, in_switch_reduce=False)
    c.validate(ok)
    nvls = Communication()
    nvls.add("all_reduce", [0, 1], 1 << 20, needs="in_switch_reduce")
    with pytest.raises(MultiDeviceError, match="in_switch_reduce"):
        nvls.validate(ok)
    assert c.seconds(ok) == pytest.approx(((1 << 20) + (1 << 9)) / 770e9)


def test_every_device_is_admitted_on_its_own_total():
    t = Topology([Device(0, 10 * GIB), Device(1, 10 * GIB), Device(2, 4 * GIB)], [])
    a = Accounting()
    for d in (0, 1, 2):
        a.charge(d, "weights", 3 * GIB)
        a.charge(d, "kv", 2 * GIB)
    with pytest.raises(MultiDeviceError, match="device 2"):      # the aggregate has room; device 2 alone does not
        a.admit(t)
    a2 = Accounting()
    a2.charge(0, "weights", GIB)
    a2.admit(t)
    with pytest.raises(MultiDeviceError):
        a2.charge(0, "mystery", 1)


def test_llama_70b_over_eight_devices_and_what_does_not_fit():
    cfg = PRESETS["llama-3-70b"]()
    topo = Topology.nvswitch(list(range(8)), 178 * GIB)
    plan = plan_tensor_parallel(cfg, topo, rows=64, num_blocks=64 * 80, step_tokens=64).validate()
    per = plan.accounting.per_device[0]
    assert 16 * GIB < per["weights"] < 20 * GIB                 # 141 GB of bf16 weights over eight ranks + a replicated embedding
    rows = plan.communication.rows
    assert len(rows) == 2 * cfg.n_layers + 1 and all(r.fused_into for r in rows)
    assert rows[5].after == (4,)
    roof = plan.roofline_seconds(tflops=1658.0, hbm_gbs=6549.0)
    assert roof["target"] == roof["hbm"] and 2e-3 < roof["hbm"] < 4e-3     # decode is bound by the weights a rank reads
    assert roof["links"] < roof["hbm"]
    # the same model on two devices of 64 GiB does not fit: device 0 says so by itself
    with pytest.raises(MultiDeviceError, match="device 0"):
        plan_tensor_parallel(cfg, Topology.nvswitch([0, 1], 64 * GIB), 64, 64 * 80, 64).validate()
    # a library-collective plan has no fused rows
    lib = plan_tensor_parallel(cfg, topo, 64, 64 * 80, 64, comm="nccl")
    assert not any(r.fused_into for r in lib.communication.rows)
    with pytest.raises(MultiDeviceError, match="do not divide"):
        plan_tensor_parallel(PRESETS["mixtral-8x7b"](), Topology.nvswitch(list(range(3)), 178 * GIB), 8, 64, 8)


def test_sharded_program_plans_scatter_gather_pairs_and_expert_exchanges():
    """The token-sharded program: a dense block ends in a reduce-scatter whose rows the next block's first projection
    gathers; a routed block sends every (token, slot) row of the rank's share to its expert's rank and back as two
    all-to-alls.  Their link bytes follow the rows that cross, and an unknown program is refused."""
    from poot_b200.models.config import PRESETS
    cfg = PRESETS["mixtral-8x7b"]()
    topo = Topology.nvswitch(list(range(8)), 178 * GIB)
    plan = plan_tensor_parallel(cfg, topo, rows=64, num_blocks=64 * 16, step_tokens=1024, program="rs_ag").validate()
    kinds = [r.kind for r in plan.communication.rows]
    L = cfg.n_layers
    assert kinds.count("all_to_all") == 2 * L and kinds.count("reduce_scatter") == L and kinds.count("all_gather") == L + 1
    S = 1024 // 8
    a2a = next(r for r in plan.communication.rows if r.kind == "all_to_all")
    assert a2a.bytes_per_rank == S * cfg.top_k * cfg.hidden * 2 and a2a.fused_into.startswith("ep_dispatch")
    assert a2a.link_bytes() == a2a.bytes_per_rank * 7 // 8
    rs = next(r for r in plan.communication.rows if r.kind == "reduce_scatter")
    assert rs.fused_into.startswith("gemm_tiled_tp") and rs.bytes_per_rank == 1024 * cfg.hidden * 2
    lib = plan_tensor_parallel(cfg, topo, 64, 64 * 16, 1024, comm="nccl", program="rs_ag")
    assert all(r.fused_into is None for r in lib.communication.rows)
    dense = plan_tensor_parallel(PRESETS["llama-3-8b"](), Topology.nvswitch([0, 1], 178 * GIB), 64, 64 * 16, 64, program="rs_ag")
    assert [r.kind for r in dense.communication.rows].count("all_to_all") == 0
    assert next(r for r in dense.communication.rows if r.kind == "reduce_scatter").fused_into.startswith("gemm_skinny_tp")
    with pytest.raises(MultiDeviceError):
        plan_tensor_parallel(cfg, topo, 64, 64 * 16, 64, program="ring")
