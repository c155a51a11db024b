"""The allocation-free attention entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory when they call into it (they are inside a stream
capture, or their host runtime forbids cudaMalloc after start-up, or the device is full).  For them
``poot_attn_paged_noalloc`` keeps the split-KV scratch in an array that lives inside the library.  This test
calls it twice in a row with different inputs and checks each result against the ordinary entry point, which
takes caller-allocated scratch.  It is collected last so that a failure here cannot hide another test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, R, Hq, Hkv, D, ctx_max):
    g = torch.Generator(device="cuda").manual_seed(seed)
    blocks_per = (ctx_max + 15) // 16
    nb = R * blocks_per
    perm = torch.randperm(nb, generator=torch.Generator().manual_seed(seed)).to(torch.int32)
    bt = perm.view(R, blocks_per).cuda()
    kpool = torch.randn(nb, Hkv, 16, D, generator=g, device="cuda").to(torch.bfloat16)
    vpool = torch.randn(nb, Hkv, 16, D, generator=g, device="cuda").to(torch.bfloat16)
    q = torch.randn(R, Hq * D, generator=g, device="cuda").to(torch.bfloat16)
    ctx = torch.randint(1, ctx_max + 1, (R,), generator=torch.Generator().manual_seed(seed + 1)).to(torch.int32).cuda()
    return q, kpool, vpool, bt, ctx


def test_noalloc_attention_matches_regular_entry_point_twice():
    from poot_b200.ops import cuda_ops as K
    from poot_b200.ops._lib import kernels
    lib = kernels()
    f = lib.poot_attn_paged_noalloc
    P = c_void_p
    f.argtypes = [P, c_int, P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int,
                  P]
    f.restype = c_int
    Hq, Hkv, D, splits = 32, 8, 128, 4
    for call, (seed, R, ctx_max) in enumerate([(11, 6, 300), (23, 3, 97)]):
        q, kpool, vpool, bt, ctx = _case(seed, R, Hq, Hkv, D, ctx_max)
        scale = 1.0 / math.sqrt(D)
        ref = K.attn_paged(q, kpool, vpool, bt, None, ctx, Hq, Hkv, D, scale, splits=splits)
        out = torch.empty_like(ref)
        stream = torch.cuda.current_stream().cuda_stream
        code = f(q.data_ptr(), q.stride(0), kpool.data_ptr(), vpool.data_ptr(), bt.data_ptr(), bt.shape[1], None,
                 ctx.data_ptr(), out.data_ptr(), out.stride(0), R, Hq, Hkv, D, scale, 0.0, 0, splits, stream)
        assert code == 0, f"call {call}: CUDA error {code}"
        torch.cuda.synchronize()
        a, b = out.float(), ref.float()
        assert torch.isfinite(a).all()
        err = (a - b).abs().max().item()
        assert err <= 2e-2 + 2e-2 * b.abs().max().item(), f"call {call}: max err {err}"


def test_noalloc_rejects_requests_beyond_the_built_in_scratch():
    from poot_b200.ops._lib import kernels
    lib = kernels()
    f = lib.poot_attn_paged_noalloc
    P = c_void_p
    f.argtypes = [P, c_int, P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int,
                  P]
    f.restype = c_int
    # 4096 rows x 32 heads x 16 splits x 130 floats is far beyond 2 Mi floats: refused before any launch
    code = f(None, 0, None, None, None, 0, None, None, None, 0, 4096, 32, 8, 128, 1.0, 0.0, 0, 16, None)
    assert code == 1
    # head counts that cannot be divided are refused the same way, not by a trap on the host
    for hq, hkv in ((32, 0), (32, -8), (32, 5), (0, 8)):
        assert f(None, 0, None, None, None, 0, None, None, None, 0, 4, hq, hkv, 128, 1.0, 0.0, 0, 2, None) == 1
