"""Quant codecs: block geometry, encode/decode round trips within the format's step, hand-built reference blocks."""
import struct

import numpy as np
import pytest

from poot_b200.quant import codec
from poot_b200.quant.formats import FORMATS, UnsupportedFormat, packed_nbytes

BLOCK_ENC = [n for n, f in FORMATS.items() if f.storage == "blocks" and f.encode]


def test_descriptor_table_is_complete():
    assert len(FORMATS) == 24
    assert FORMATS["Q4_K"].block_bytes == 144 and FORMATS["Q8_0"].block_bytes == 34
    assert abs(FORMATS["Q4_K"].bits_per_weight - 4.5) < 1e-9


@pytest.mark.parametrize("fmt", BLOCK_ENC)
def test_round_trip_error_is_bounded_by_the_quant_step(fmt):
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((8, 1024)) * 0.02).astype(np.float32)
    packed = codec.quantize(fmt, w)
    assert packed.nbytes == packed_nbytes(fmt, w.size)
    back = codec.dequantize(fmt, packed, w.shape)
    bits = FORMATS[fmt].bits_per_weight
    levels = {"Q8_0": 127, "Q4_0": 8, "Q4_1": 15, "Q5_0": 16, "Q5_1": 31, "MXFP4": 4, "Q2_K": 3, "Q3_K": 4, "Q4_K": 15,
              "Q5_K": 31, "Q6_K": 32}[fmt]
    tol = 1.3 * np.abs(w).max() / levels
    assert np.abs(back - w).max() <= tol, (fmt, np.abs(back - w).max(), tol, bits)
    codec.check_scales(fmt, packed, w.size)


def test_q8_0_reference_block():
    d = np.float16(0.5)
    qs = np.arange(-16, 16, dtype=np.int8)
    blk = np.frombuffer(d.tobytes() + qs.tobytes(), dtype=np.uint8)
    out = codec.dequantize("Q8_0", blk, (32,))
    assert np.array_equal(out, qs.astype(np.float32) * 0.5)


def test_q4_k_reference_block_follows_the_ggml_layout():
    # d = 1, dmin = 0.5, sub-block j: scale j+1, min j (6-bit fields, j >= 4 use the split encoding)
    ls, lm = list(range(1, 9)), list(range(8))
    sc = bytearray(12)
    for j in range(8):
        if j < 4:
            sc[j], sc[j + 4] = ls[j], lm[j]
        else:
            sc[j + 4] = (ls[j] & 0xF) | ((lm[j] & 0xF) << 4)
            sc[j - 4] |= (ls[j] >> 4) << 6
            sc[j] |= (lm[j] >> 4) << 6
    qs = bytes(((l % 16) | (((l + 3) % 16) << 4)) for l in range(128))
    blk = np.frombuffer(np.float16(1.0).tobytes() + np.float16(0.5).tobytes() + bytes(sc) + qs, dtype=np.uint8)
    out = codec.dequantize("Q4_K", blk, (256,))
    for i in (0, 31, 32, 63, 64, 200, 255):
        j, h, l = i // 64, (i % 64) // 32, i % 32      # element i = j*64 + h*32 + l is nibble h of qs[j*32 + l]
        byte = qs[j * 32 + l]
        q = (byte >> 4) if h else (byte & 0xF)
        sub = 2 * j + h
        assert out[i] == np.float32(1.0 * ls[sub] * q - 0.5 * lm[sub]), i


def test_non_finite_scale_is_rejected():
    blk = np.frombuffer(np.float16(np.inf).tobytes() + bytes(32), dtype=np.uint8)
    with pytest.raises(ValueError):
        codec.check_scales("Q8_0", blk, 32)


def test_unsupported_grid_formats_are_typed_refusals():
    with pytest.raises(UnsupportedFormat):
        codec.dequantize("IQ3_S", np.zeros(110, dtype=np.uint8), (256,))


@pytest.mark.parametrize("fmt,tol", [("E4M3_CHANNEL", 0.07), ("E4M3_BLOCK128", 0.07), ("E2M1_ROW32", 0.3), ("GPTQ", 0.08),
                                      ("AWQ", 0.08)])
def test_planar_round_trip(fmt, tol):
    rng = np.random.default_rng(2)
    w = (rng.standard_normal((256, 256)) * 0.05).astype(np.float32)
    back = codec.dequantize_planar(fmt, codec.quantize_planar(fmt, w))
    assert back.shape == w.shape
    assert np.abs(back - w).max() <= tol * np.abs(w).max() + 1e-6


def test_packed_row_and_column_views():
    from poot_b200.quant.weights import PackedWeight
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((8, 512)) * 0.02).astype(np.float32)
    pw = PackedWeight("w", "Q4_K", w.shape, codec.quantize("Q4_K", w))
    full = pw.to_f32()
    assert np.array_equal(pw.rows(2, 4).to_f32(), full[2:6])
    assert np.array_equal(pw.cols(256, 256).to_f32(), full[:, 256:])
    with pytest.raises(ValueError):
        pw.cols(100, 256)


def _random_blocks(fmt, rows, K, seed=3):
    """Packed rows of ``fmt``: encoded from random weights where an encoder exists, otherwise random bytes with
    finite f16 scale fields (IQ4_NL / IQ4_XS have a decoder only)."""
    rng = np.random.default_rng(seed)
    d = FORMATS[fmt]
    if d.encode:
        return codec.quantize(fmt, (rng.standard_normal((rows, K)) * 0.05).astype(np.float32)).reshape(rows, -1)
    raw = rng.integers(0, 256, size=(rows, K // d.block_elems, d.block_bytes), dtype=np.uint8)
    scale = (rng.standard_normal((rows, K // d.block_elems)) * 0.01).astype(np.float16).view(np.uint8).reshape(rows, -1, 2)
    raw[:, :, 0:2] = scale
    return raw.reshape(rows, -1)


DEVICE_BLOCK_FORMATS = [n for n, f in FORMATS.items() if f.storage == "blocks" and f.device_gemv]


@pytest.mark.parametrize("fmt", DEVICE_BLOCK_FORMATS)
def test_device_block_decoders_equal_the_host_codec(fmt):
    """The block decoders that the device kernels run are also built for the host (the same source): every value of
    every format equals the host codec's, so a wrong nibble order, bit plane or scale index cannot hide until a GPU run."""
    import ctypes
    from poot_b200.ops._lib import kernels
    from poot_b200.ops.cuda_ops import QUANT_DEVICE_FORMATS
    lib = kernels()
    f = lib.poot_quant_decode8_host
    f.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    f.restype = ctypes.c_int
    assert len(DEVICE_BLOCK_FORMATS) == 13 and set(DEVICE_BLOCK_FORMATS) == set(QUANT_DEVICE_FORMATS)
    rows, K = 3, 1024
    packed = np.ascontiguousarray(_random_blocks(fmt, rows, K))
    want = codec.dequantize(fmt, packed, (rows, K))
    got = np.zeros((rows, K), np.float32)
    out8 = np.zeros(8, np.float32)
    for r in range(rows):
        row = np.ascontiguousarray(packed[r])
        for k in range(0, K, 8):
            assert f(QUANT_DEVICE_FORMATS[fmt], row.ctypes.data, k, out8.ctypes.data) == 0
            got[r, k:k + 8] = out8
    # the kernels factor a block as scale * q - offset in f32; the host codec multiplies in a slightly different order
    assert np.allclose(got, want, rtol=2e-6, atol=1e-7), (fmt, np.abs(got - want).max())
    assert f(QUANT_DEVICE_FORMATS[fmt], packed.ctypes.data, 4, out8.ctypes.data) == 1      # k must be a multiple of 8
    assert f(99, packed.ctypes.data, 0, out8.ctypes.data) == 1
