"""Device kernels over GGUF block formats against the host codec (which is checked against hand-built blocks)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
FMTS = ["Q4_K", "Q5_K", "Q6_K", "Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q2_K", "Q3_K", "IQ4_NL", "IQ4_XS", "MXFP4"]


def _packed(fmt, N, Kd, seed=0):
    from poot_b200.ops import cuda_ops as K
    from poot_b200.quant import codec
    from poot_b200.quant.formats import FORMATS
    rng = np.random.default_rng(seed)
    d = FORMATS[fmt]
    if d.encode:
        p = codec.quantize(fmt, (rng.standard_normal((N, Kd)) * 0.05).astype(np.float32))
    else:           # decoder-only formats (IQ4_NL, IQ4_XS): random code bytes under finite f16 block scales
        raw = rng.integers(0, 256, size=(N, Kd // d.block_elems, d.block_bytes), dtype=np.uint8)
        raw[:, :, 0:2] = (rng.standard_normal((N, Kd // d.block_elems)) * 0.01).astype(np.float16).view(np.uint8).reshape(N, -1, 2)
        p = raw.reshape(-1)
    deq = codec.dequantize(fmt, p, (N, Kd))
    return K.QuantWeight(fmt, torch.from_numpy(p).cuda(), N, Kd), torch.from_numpy(deq).cuda()


@pytest.mark.first_device_run          # eight of the formats' decoders have not run on a device
@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("M", [1, 3])
@pytest.mark.parametrize("N,Kd", [(1026, 1024), (258, 5376), (36, 14336)])     # 14336 = the down projection's K of Llama-3-8B
def test_quant_gemv_matches_dequantised_reference(fmt, M, N, Kd):
    from poot_b200.ops import cuda_ops as K
    W, deq = _packed(fmt, N, Kd)
    x = (torch.randn(M, Kd, device="cuda")).to(torch.bfloat16)
    ref = x.float() @ deq.T
    out = K.quant_gemv(x, W, K.EPI_F32)
    assert (out - ref).abs().max() <= 2e-3 * ref.abs().max() + 1e-3
    res = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    o2 = K.quant_gemv(x, W, K.EPI_RESID, resid=res)
    assert (o2.float() - (ref + res.float())).abs().max() <= 2e-2 * (ref.abs().max() + 3)
    sw = K.quant_gemv(x, W, K.EPI_SWIGLU)
    r2 = torch.nn.functional.silu(ref[:, 0::2]) * ref[:, 1::2]
    assert (sw.float() - r2).abs().max() <= 2e-2 * r2.abs().max() + 1e-2


@pytest.mark.first_device_run
@pytest.mark.parametrize("fmt", FMTS)
def test_quant_dequant_and_row_gather_are_exact(fmt):
    from poot_b200.ops import cuda_ops as K
    W, deq = _packed(fmt, 300, 512, seed=3)
    full = K.quant_dequant(W)
    assert torch.equal(full, deq.to(torch.bfloat16))
    ids = torch.tensor([0, 7, 299, 7], dtype=torch.int32, device="cuda")
    rows = K.quant_row_gather(ids, W)
    assert torch.equal(rows, deq[ids.long()].to(torch.bfloat16))


def test_linear_dispatches_packed_weights_for_prefill_shapes():
    from poot_b200.ops import cuda_ops as K
    W, deq = _packed("Q4_K", 512, 1024, seed=5)
    x = torch.randn(200, 1024, device="cuda").to(torch.bfloat16)
    out = K.linear(x, W)
    ref = x.float() @ deq.to(torch.bfloat16).float().T
    assert (out.float() - ref).abs().max() <= 2e-2 * ref.abs().max() + 2e-2
    K.check_status()


@pytest.mark.xfail(strict=False, reason="new kernel: not yet run on a device")
@pytest.mark.parametrize("fmt", ["Q4_K", "Q8_0", "Q6_K", "Q4_0", "MXFP4", "Q3_K"])
@pytest.mark.parametrize("M", [5, 17, 64, 128])
def test_dequant_fused_skinny_gemm_matches_dequantised_reference(fmt, M):
    """Decode batches over packed weights on the tensor cores: the decoders write the weight tile straight into the
    swizzled stage.  Every epilogue against ``x @ dequant(W)^T`` in fp32 (N = 264: two full row tiles and a ragged one)."""
    from poot_b200.ops import cuda_ops as K
    N, Kd = 264, 1024
    W, deq = _packed(fmt, N, Kd, seed=3)
    g = torch.Generator().manual_seed(M)
    x = (torch.randn(M, Kd, generator=g) * 0.5).to(torch.bfloat16).cuda()
    ref = x.float() @ deq.to(torch.bfloat16).float().T
    tol = 2e-2 * ref.abs().max().item() + 2e-2
    out = K.quant_gemm_skinny(x, W, K.EPI_STORE)
    assert (out.float() - ref).abs().max().item() <= tol
    f32 = K.quant_gemm_skinny(x, W, K.EPI_F32)
    assert (f32 - ref).abs().max().item() <= tol
    res = (torch.randn(M, N, generator=g)).to(torch.bfloat16).cuda()
    rs = K.quant_gemm_skinny(x, W, K.EPI_RESID, resid=res)
    assert (rs.float() - (ref + res.float())).abs().max().item() <= tol + 1e-2
    sw = K.quant_gemm_skinny(x, W, K.EPI_SWIGLU)
    want = torch.nn.functional.silu(ref[:, 0::2]) * ref[:, 1::2]
    assert (sw.float() - want).abs().max().item() <= 3e-2 * want.abs().max().item() + 2e-2
    K.check_status()
