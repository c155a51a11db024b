"""The fused row-parallel GEMM + one-shot all-reduce + RMSNorm pair of a tensor-parallel decode step, with every
rank of the group emulated on ONE GPU (for profiling: the profiler captures single-GPU programs only).

    python benchmarks/tp_oneshot_emulated.py [world] [rows] [hidden] [k_local] [rounds]

Each emulated rank owns its flag block, inbox, step counter and weight shard, all in this GPU's memory, so the
"peer" stores of the GEMM epilogue land locally.  Launch order per round: every rank's GEMM, then every rank's
reduce+norm; a kernel that waits on flags is only launched after the kernels that set them have been enqueued on
the same stream, so nothing waits on a later launch.  The result is checked against fp32 PyTorch.
"""
import ctypes
import sys
from ctypes import c_float, c_int, c_void_p

import torch

sys.path.insert(0, ".")
from poot_b200.ops import cuda_ops as K  # noqa: E402
from poot_b200.ops._lib import check  # noqa: E402

_P = c_void_p
world = int(sys.argv[1]) if len(sys.argv) > 1 else 2
T = int(sys.argv[2]) if len(sys.argv) > 2 else 64
H = int(sys.argv[3]) if len(sys.argv) > 3 else 4096
Kl = int(sys.argv[4]) if len(sys.argv) > 4 else 7168
rounds = int(sys.argv[5]) if len(sys.argv) > 5 else 6
MAX_ROWS, RS_SITES, AG_SITES = 128, 2, 3
dev = torch.device("cuda")
K.register_signature("poot_tp_begin_step", [_P, _P])
K.register_signature("poot_tp_norm", [_P, _P, _P, _P, _P, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_int,
                                      c_int, c_int, _P, _P, _P, _P, _P, _P])
K.register_signature("poot_gemm_skinny_tp", [c_int, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                             c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P, c_int, c_int, _P, _P, _P])
begin, norm, gemm = K.fn("poot_tp_begin_step"), K.fn("poot_tp_norm"), K.fn("poot_gemm_skinny_tp")

torch.manual_seed(0)
flags = [torch.zeros(256, dtype=torch.int32, device=dev) for _ in range(world)]
inbox = [torch.zeros(2 * world * MAX_ROWS * H, dtype=torch.bfloat16, device=dev) for _ in range(world)]
epoch = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(world)]
ticket = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(world)]
copies = 3          # rotate weight copies so that every launch streams cold weights (inputs larger than L2)
W = [[(torch.randn(H, Kl, device=dev) * 0.02).to(torch.bfloat16) for _ in range(copies)] for _ in range(world)]
for r in range(world):
    for c in range(1, copies):
        W[r][c].copy_(W[r][0])
x = [(torch.randn(T, Kl, device=dev) * 0.5).to(torch.bfloat16) for _ in range(world)]
h = [(torch.randn(T, H, device=dev) * 0.5).to(torch.bfloat16) for _ in range(world)]
for r in range(1, world):
    h[r].copy_(h[0])
h0 = h[0].clone()
wn = torch.ones(H, dtype=torch.bfloat16, device=dev)
xo = [torch.zeros(T, H, dtype=torch.bfloat16, device=dev) for _ in range(world)]
flags_peer = (c_void_p * world)(*[f.data_ptr() for f in flags])
inbox_peer = (c_void_p * world)(*[b.data_ptr() for b in inbox])
st = K.status_word(dev)
stream = K._stream()
ck = K.skinny_cluster(H, Kl)

e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
times = []
for it in range(rounds):
    for r in range(world):
        check(begin(epoch[r].data_ptr(), stream), "begin")
    e0.record()
    for r in range(world):
        check(gemm(K.EPI_STORE, x[r].data_ptr(), W[r][it % copies].data_ptr(), None, H, Kl, Kl, H, ck, world, r, MAX_ROWS,
                   -1, AG_SITES, 0, RS_SITES, epoch[r].data_ptr(), flags[r].data_ptr(), flags_peer, inbox_peer, H, T,
                   ticket[r].data_ptr(), st.data_ptr(), stream), "gemm_skinny_tp")
    e1.record()
    for r in range(world):
        check(norm(h[r].data_ptr(), inbox[r].data_ptr(), wn.data_ptr(), None, xo[r].data_ptr(), T, H, 1e-5, world, r,
                   MAX_ROWS, 0, AG_SITES, 0, RS_SITES, epoch[r].data_ptr(), flags[r].data_ptr(), flags_peer,
                   ticket[r].data_ptr(), st.data_ptr(), stream), "tp_norm")
    if "--plain" in sys.argv:       # the same contraction without the collective epilogue, for comparison in a launch list
        K.gemm_skinny(x[0], W[0][it % copies], K.EPI_STORE, out=xo[0])
    torch.cuda.synchronize()
    times.append(e0.elapsed_time(e1) * 1e3 / world)
K.check_status()

# the same rounds inside one CUDA graph (programmatic dependent launch on): per-rank time of GEMM + reduce/norm as it
# runs inside a decode step, without host launch gaps
if "--graph" in sys.argv:
    K.set_pdl(True)
    n_graph = 8
    s2 = torch.cuda.Stream()
    s2.wait_stream(torch.cuda.current_stream())

    def rounds_on(stream_ptr, n):
        for it in range(n):
            for r in range(world):
                check(begin(epoch[r].data_ptr(), stream_ptr), "begin")
            for r in range(world):
                check(gemm(K.EPI_STORE, x[r].data_ptr(), W[r][it % copies].data_ptr(), None, H, Kl, Kl, H, ck, world, r,
                           MAX_ROWS, -1, AG_SITES, 0, RS_SITES, epoch[r].data_ptr(), flags[r].data_ptr(), flags_peer,
                           inbox_peer, H, T, ticket[r].data_ptr(), st.data_ptr(), stream_ptr), "gemm_skinny_tp")
            for r in range(world):
                check(norm(h[r].data_ptr(), inbox[r].data_ptr(), wn.data_ptr(), None, xo[r].data_ptr(), T, H, 1e-5, world,
                           r, MAX_ROWS, 0, AG_SITES, 0, RS_SITES, epoch[r].data_ptr(), flags[r].data_ptr(), flags_peer,
                           ticket[r].data_ptr(), st.data_ptr(), stream_ptr), "tp_norm")

    with torch.cuda.stream(s2):
        rounds_on(K._stream(), 1)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s2):
        rounds_on(K._stream(), n_graph)
    reps = []
    for _ in range(6):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        reps.append(a.elapsed_time(b) * 1e3 / (n_graph * world))
    K.check_status()
    rounds += 1 + 6 * n_graph          # the residual stream kept accumulating
    print(f"in-graph: {sorted(reps[1:])[len(reps[1:]) // 2]:.2f} us per rank for GEMM + reduce/norm "
          f"(HBM floor {H * Kl * 2 / 6549e3:.2f} us for the weights)")
delta = sum(x[r].float() @ W[r][0].float().T for r in range(world))
ref_h = h0.float() + rounds * delta
err = (h[0].float() - ref_h).abs().max().item() / max(1.0, ref_h.abs().max().item())
same = all(torch.equal(h[0], h[r]) for r in range(1, world))
print(f"world={world} rows={T} N={H} K_local={Kl} cluster={ck}: gemm {sorted(times)[len(times) // 2]:.1f} us per rank "
      f"(weights {H * Kl * 2 / 1e6:.1f} MB), residual rel err {err:.4f}, ranks identical {same}")
assert err < 0.05 and same
