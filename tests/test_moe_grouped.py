"""Row-grouped mixture of experts: block-aligned grouping, gather, grouped GEMMs over the tiles, scatter-combine.
The host restatements are checked against an fp32 dense statement of the routed FFN on the CPU; the device kernels are
checked against the same statement on a GPU (`-m gpu`)."""
import numpy as np
import pytest
import torch

from poot_b200.plan.moe_align import group_expert_rows


def _routed_reference(x, wgu, wdown, ids, gates):
    """fp32: out[t] = sum_j gate[t, j] * down_e(silu(gate_e(x_t)) * up_e(x_t)), e = ids[t, j]; wgu rows interleave
    (gate, up)."""
    T, k = ids.shape
    out = torch.zeros(T, wdown.shape[1])
    for t in range(T):
        for j in range(k):
            e = int(ids[t, j])
            gu = wgu[e].float() @ x[t].float()
            a = torch.nn.functional.silu(gu[0::2]) * gu[1::2]
            a = a.to(torch.bfloat16).float()
            out[t] += float(gates[t, j]) * (wdown[e].float() @ a).to(torch.bfloat16).float()
    return out


def _case(T, E, k, H=128, F=64, seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(T, H, generator=g) * 0.5).to(torch.bfloat16)
    wgu = (torch.randn(E, 2 * F, H, generator=g) * 0.1).to(torch.bfloat16)
    wdown = (torch.randn(E, H, F, generator=g) * 0.1).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    gates = torch.softmax(torch.randn(T, k, generator=g), -1)
    return [t.to(device) for t in (x, wgu, wdown, ids, gates)]


def _grouped_forward(M, K, x, wgu, wdown, ids, gates, e0=0, e_local=None, force_block=None):
    """The launch sequence of runtime/moe.py's row-grouped regime on stand-alone buffers; returns (out, pos, n_tiles)."""
    T, k = ids.shape
    E, W2, H = wgu.shape
    e_local = E if e_local is None else e_local
    F = W2 // 2
    dev = x.device
    n = T * k
    block = force_block or M.group_block(n, E)
    max_tiles = M.group_capacity(n, e_local, block)
    cap = max_tiles * block
    i32 = dict(dtype=torch.int32, device=dev)
    pos, sorted_rows = torch.zeros(n, **i32), torch.zeros(cap, **i32)
    tile_expert, n_tiles = torch.zeros(max_tiles, **i32), torch.zeros(1, **i32)
    xs = torch.zeros(cap, H, dtype=torch.bfloat16, device=dev)
    gate_s = torch.zeros(cap, dtype=torch.float32, device=dev)
    act = torch.zeros(cap, F, dtype=torch.bfloat16, device=dev)
    y = torch.zeros(cap, H, dtype=torch.bfloat16, device=dev)
    M.moe_align(ids.reshape(-1).contiguous(), e0, e_local, block, max_tiles, pos, sorted_rows, tile_expert, n_tiles)
    M.moe_gather_rows(x, sorted_rows, gates.reshape(-1).contiguous().float(), n_tiles, block, max_tiles, k, xs, gate_s)
    wl, dl = wgu[e0:e0 + e_local].contiguous(), wdown[e0:e0 + e_local].contiguous()
    if block == 128 and W2 % 128 == 0 and H % 128 == 0:
        M.gemm_grouped_tiled(K.EPI_SWIGLU, xs, wl, act, tile_expert)
        M.gemm_grouped_tiled(K.EPI_STORE, act, dl, y, tile_expert, row_scale=gate_s)
    else:
        M.gemm_grouped(K.EPI_SWIGLU, xs, wl, act, block, max_tiles, group_expert=tile_expert, x_row_mul=block,
                       out_group_stride=block * F, ldo=F)
        M.gemm_grouped(K.EPI_STORE, act, dl, y, block, max_tiles, group_expert=tile_expert, x_row_mul=block,
                       out_group_stride=block * H, row_scale=gate_s, ldo=H)
    out = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
    M.moe_scatter_combine(None, y, pos, out, T, H, k)
    return out, pos, sorted_rows, tile_expert, int(n_tiles[0]), block


def _check_grouping(ids, pos, sorted_rows, tile_expert, n_tiles, block, e0, e_local):
    flat = ids.reshape(-1).cpu().numpy()
    pos, sorted_rows, tile_expert = pos.cpu().numpy(), sorted_rows.cpu().numpy(), tile_expert.cpu().numpy()
    local = (flat >= e0) & (flat < e0 + e_local)
    want_rows, want_tiles, padded = group_expert_rows(flat[local] - e0, e_local, block)
    assert n_tiles == padded // block
    assert list(tile_expert[:n_tiles]) == list(want_tiles) and (tile_expert[n_tiles:] == -1).all()
    assert (pos[~local] == -1).all() and (pos[local] >= 0).all()
    assert len(set(pos[local])) == local.sum()                            # a permutation: no two rows share a position
    for i in np.nonzero(local)[0]:
        p = pos[i]
        assert sorted_rows[p] == i and tile_expert[p // block] == flat[i] - e0      # the row sits in a tile of its expert
    live = sorted_rows[:n_tiles * block] >= 0
    assert live.sum() == local.sum()


@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (64, 8, 2), (300, 8, 2), (64, 128, 8), (1024, 128, 8)])
def test_row_grouped_experts_equal_the_routed_reference_on_the_host(T, E, k):
    from poot_b200.ops import cuda_ops as K, moe_ops as M
    from poot_b200.utils.kernel_emulation import emulated_kernels
    x, wgu, wdown, ids, gates = _case(T, E, k, H=64 if T > 500 else 128, F=32 if T > 500 else 64)
    with emulated_kernels():
        out, pos, sr, te, nt, block = _grouped_forward(M, K, x, wgu, wdown, ids, gates)
    _check_grouping(ids, pos, sr, te, nt, block, 0, E)
    rows = list(range(T)) if T <= 64 else list(range(0, T, max(1, T // 24)))
    ref = _routed_reference(x[rows], wgu, wdown, ids[rows], gates[rows])
    err = (out[rows].float() - ref).abs().max().item() / max(1.0, ref.abs().max().item())
    assert err < 0.03, err
    # the work is the routed work: T * k rows plus less than one tile of padding per expert
    assert nt * block < T * k + E * block


def test_expert_parallel_shards_group_only_their_own_rows_and_sum_to_the_whole():
    from poot_b200.ops import cuda_ops as K, moe_ops as M
    from poot_b200.utils.kernel_emulation import emulated_kernels
    T, E, k, world = 40, 8, 2, 4
    x, wgu, wdown, ids, gates = _case(T, E, k)
    with emulated_kernels():
        whole, *_ = _grouped_forward(M, K, x, wgu, wdown, ids, gates)
        total = torch.zeros(T, x.shape[1])
        for r in range(world):                         # two experts per rank
            part, pos, sr, te, nt, block = _grouped_forward(M, K, x, wgu, wdown, ids, gates, e0=2 * r, e_local=2)
            _check_grouping(ids, pos, sr, te, nt, block, 2 * r, 2)
            total += part.float()
    err = (total - whole.float()).abs().max().item() / max(1.0, whole.float().abs().max().item())
    assert err < 0.02, err


@pytest.mark.gpu
@pytest.mark.first_device_run
@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (64, 8, 2), (1024, 8, 2), (64, 128, 8), (1024, 128, 8)])
def test_row_grouped_experts_on_the_device(T, E, k):
    """The device kernels (align, gather, grouped swap-AB and tiled tcgen05 GEMMs, scatter-combine) against the fp32
    statement; T = 1024 with 8 experts runs tiles of 128 rows through the tiled kernel."""
    from poot_b200.ops import cuda_ops as K, moe_ops as M
    x, wgu, wdown, ids, gates = _case(T, E, k, H=256, F=128, device="cuda")
    out, pos, sr, te, nt, block = _grouped_forward(M, K, x, wgu, wdown, ids, gates)
    K.check_status()
    _check_grouping(ids, pos, sr, te, nt, block, 0, E)
    rows = list(range(T)) if T <= 64 else list(range(0, T, T // 16))
    ref = _routed_reference(x[rows].cpu(), wgu.cpu(), wdown.cpu(), ids[rows].cpu(), gates[rows].cpu())
    err = (out[rows].float().cpu() - ref).abs().max().item() / max(1.0, ref.abs().max().item())
    assert err < 0.03, err


@pytest.mark.gpu
@pytest.mark.first_device_run
def test_expert_shard_on_the_device_leaves_other_ranks_rows_out():
    from poot_b200.ops import cuda_ops as K, moe_ops as M
    T, E, k = 96, 8, 2
    x, wgu, wdown, ids, gates = _case(T, E, k, H=256, F=128, device="cuda")
    whole, *_ = _grouped_forward(M, K, x, wgu, wdown, ids, gates)
    total = torch.zeros(T, 256, device="cuda")
    for r in range(4):
        part, pos, sr, te, nt, block = _grouped_forward(M, K, x, wgu, wdown, ids, gates, e0=2 * r, e_local=2)
        _check_grouping(ids, pos, sr, te, nt, block, 2 * r, 2)
        total += part.float()
    K.check_status()
    assert (total - whole.float()).abs().max().item() / max(1.0, whole.float().abs().max().item()) < 0.02
