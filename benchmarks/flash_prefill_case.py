"""One tensor-core prefill attention launch over a paged cache, timed with CUDA events.

    python benchmarks/flash_prefill_case.py [tokens] [sequences] [q_heads] [kv_heads]
"""
import sys

import torch

sys.path.insert(0, ".")
from poot_b200.ops import cuda_ops as K  # noqa: E402

L = int(sys.argv[1]) if len(sys.argv) > 1 else 2048
B = int(sys.argv[2]) if len(sys.argv) > 2 else 1
Hq = int(sys.argv[3]) if len(sys.argv) > 3 else 32
Hkv = int(sys.argv[4]) if len(sys.argv) > 4 else 8
D = 128
torch.manual_seed(0)
bps = (L + 15) // 16
nblocks = B * bps
kpool = (torch.randn(nblocks, Hkv, 16, D, device="cuda") * 0.5).to(torch.bfloat16)
vpool = (torch.randn(nblocks, Hkv, 16, D, device="cuda") * 0.5).to(torch.bfloat16)
bt = torch.randperm(nblocks).to(torch.int32).view(B, bps).cuda()
row_seq = torch.arange(B, dtype=torch.int32).repeat_interleave(L)
positions = torch.arange(L, dtype=torch.int32).repeat(B)
tiles, covered = K.flash_tiles(row_seq.numpy(), positions.numpy())
tiles = torch.from_numpy(tiles).cuda()
q = (torch.randn(B * L, Hq * D, device="cuda") * 0.5).to(torch.bfloat16)
out = torch.empty_like(q)
times = []
for _ in range(6):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    K.attn_flash_prefill(q, kpool, vpool, bt, tiles, Hq, Hkv, D ** -0.5, out)
    e1.record()
    torch.cuda.synchronize()
    times.append(e0.elapsed_time(e1))
K.check_status()
ms = sorted(times[1:])[len(times[1:]) // 2]
flops = 4.0 * B * Hq * D * (L * (L + 1) / 2)            # causal: q·kᵀ and p·v over the visible keys only
tile_flops = 4.0 * Hq * D * 128 * 128 * sum((int(t[3]) + int(t[1]) + 127) // 128 for t in tiles.cpu())
print(f"tokens={L} x {B} seqs, heads {Hq}/{Hkv}: {ms * 1e3:.1f} us, {flops / ms / 1e9:.0f} TFLOP/s causal-useful, "
      f"{tile_flops / ms / 1e9:.0f} TFLOP/s issued (whole 128x128 tiles)")
