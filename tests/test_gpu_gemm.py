"""Prefill GEMM on the tcgen05 tensor cores against the CPU dequant + matmul (Q4_0 / Q8_0 weights
times 16-bit activations, f32 accumulation).

Operands are 16-bit, accumulation f32.  Mode 0 (bf16): activations rounded to bf16, weights
bf16(bf16(d) * (n - 8)) for Q4_0 and bf16(d * q) for Q8_0.  Mode 1 (f16): activations rounded to IEEE
half, weights f16(d * q).  Mode 2 (compensated f16, the session's): hi + lo planes of both operands.
Tolerance: rounding both operands costs 2^-8 (bf16) or 2^-11 (f16) relative per product and
averages out over K; the bound used is norm-relative (|x|.|w| per output), and 1e-5 of that norm
against a reference that applies the same operand rounding.  The compensated mode must be within
2e-6 of that norm of the exact product (f32 accumulation is all that is left)."""
import numpy as np
import pytest

from oracle import oracle as O
from rustgrad_b200 import quant, session, synth

pytestmark = pytest.mark.gpu


def to_bf16(a):
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((b >> 16) & 1) + 0x7FFF
    return (((b + r) >> 16) << 16).astype(np.uint32).view(np.float32)


def to_f16(a):
    return np.asarray(a, dtype=np.float32).astype(np.float16).astype(np.float32)


def operand_weight(kind, data, n, k, f16):
    """The operand the kernel builds from the blocks."""
    dense = O.dequantize(kind, data, n * k).reshape(n, k // 32, 32)
    if f16:
        return to_f16(dense).reshape(n, k)
    if kind == quant.Q8_0:
        return to_bf16(dense).reshape(n, k)
    bb = quant.BLOCK_BYTES[kind]
    d = data.reshape(n, k // 32, bb)[:, :, :2].copy().view(np.float16).astype(np.float32)  # [n, blocks, 1]
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(d != 0, np.rint(dense / d), 0.0).astype(np.float32)
    return to_bf16(to_bf16(d) * q).reshape(n, k)


@pytest.mark.parametrize("mode", [0, 1, 2], ids=["bf16", "f16", "f16x3"])
@pytest.mark.parametrize("kind", [quant.Q4_0, quant.Q8_0])
@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (16, 128, 512), (200, 300, 1024), (33, 4096, 4096), (512, 1024, 4096)])
def test_qgemm_matches_cpu_dequant_matmul(kind, m, n, k, mode):
    rng = np.random.default_rng(m + n + k)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    data = quant.encode(kind, w)
    got, _ = session.qgemm(kind, data, n, k, x, operand_mode=mode)
    dense = O.dequantize(kind, data, n * k).reshape(n, k)
    scale = np.sqrt((x.astype(np.float64) ** 2).sum(1))[:, None] * np.sqrt((dense.astype(np.float64) ** 2).sum(1))[None, :]
    want = x.astype(np.float64) @ dense.astype(np.float64).T
    if mode == 2:
        assert (np.abs(got - want) / scale).max() < 2e-6
        return
    f16 = mode == 1
    assert (np.abs(got - want) / scale).max() < (2e-2 if not f16 else 2.5e-3) / np.sqrt(k) * 8
    rx = to_f16(x) if f16 else to_bf16(x)
    same_rounding = rx.astype(np.float64) @ operand_weight(kind, data, n, k, f16).astype(np.float64).T
    assert (np.abs(got - same_rounding) / scale).max() < 1e-5


def test_f16_operands_saturate_large_finite_activations():
    n, k = 128, 256
    rng = np.random.default_rng(5)
    data = quant.encode(quant.Q8_0, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    x = np.zeros((16, k), dtype=np.float32)
    x[0, 0] = 1.0e6  # beyond the f16 range: enters as 65504
    x[1, 3] = -3.0
    got, _ = session.qgemm(quant.Q8_0, data, n, k, x, operand_mode=1)
    w = to_f16(O.dequantize(quant.Q8_0, data, n * k).reshape(n, k))
    assert np.isfinite(got).all()
    np.testing.assert_allclose(got[0], 65504.0 * w[:, 0], rtol=1e-6)
    np.testing.assert_allclose(got[1], -3.0 * w[:, 3], rtol=1e-6)


def test_compensated_mode_keeps_small_and_large_magnitudes():
    """Weights and activations far from 1 (lo planes in the f16 subnormal range, hi near its top)."""
    n, k, m = 256, 512, 40
    rng = np.random.default_rng(11)
    for wstd, xstd in ((1e-3, 1e-2), (0.5, 300.0), (0.02, 1.0)):
        data = quant.encode(quant.Q4_0, (rng.standard_normal((n, k)) * wstd).astype(np.float32))
        x = (rng.standard_normal((m, k)) * xstd).astype(np.float32)
        got, _ = session.qgemm(quant.Q4_0, data, n, k, x, operand_mode=2)
        dense = O.dequantize(quant.Q4_0, data, n * k).reshape(n, k).astype(np.float64)
        want = x.astype(np.float64) @ dense.T
        scale = np.sqrt((x.astype(np.float64) ** 2).sum(1))[:, None] * np.sqrt((dense ** 2).sum(1))[None, :]
        assert (np.abs(got - want) / scale).max() < 1e-5, (wstd, xstd)


def _check_qgemm(kind, m, n, k, mode, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k), dtype=np.float32)
    data = synth.device_weight(kind, n, k, seed=4)  # N(0, 0.02) quantized on the device, read back
    got, _ = session.qgemm(kind, data, n, k, x, operand_mode=mode)
    dense = O.dequantize(kind, data, n * k).reshape(n, k)
    # f32 matmul on the host BLAS is the CPU dequant + matmul at these sizes; its own error
    # (2^-24 sqrt(k) relative to the norm) is far below the bounds used here
    scale = np.sqrt((x.astype(np.float64) ** 2).sum(1))[:, None].astype(np.float32) * \
        np.sqrt((dense.astype(np.float64) ** 2).sum(1))[None, :].astype(np.float32)
    want = x @ dense.T
    f16 = mode == 1
    assert (np.abs(got - want) / scale).max() < (2e-2 if not f16 else 2.5e-3) / np.sqrt(k) * 8
    rx = to_f16(x) if f16 else to_bf16(x)
    same_rounding = rx @ operand_weight(kind, data, n, k, f16).T
    assert (np.abs(got - same_rounding) / scale).max() < 1e-5


@pytest.mark.parametrize("mode", [0, 1], ids=["bf16", "f16"])
@pytest.mark.parametrize("m,n,k", [(512, 12288, 512), (700, 12416, 256), (2048, 4096, 4096), (512, 14336, 4096),
                                   (2048, 14336, 4096)])
def test_wide_tile_kernel_matches_cpu_dequant_matmul(m, n, k, mode):
    """More than 256 tokens with one operand plane on a grid of at least 96 CTAs select the
    128 x 512-tile kernel (two tensor-memory accumulators per dequantised weight tile); the
    prefill shapes [14336, 4096] and [4096, 4096] at 512 and 2048 tokens are among the cases, and a
    ragged one (700 tokens, 12416 rows).  The launch counter proves which kernel ran."""
    before_wide, before_tc = session.launch_count("qgemm_tc_wide"), session.launch_count("qgemm_tc")
    _check_qgemm(quant.Q4_0, m, n, k, mode, seed=m + n + k + mode)
    assert session.launch_count("qgemm_tc_wide") == before_wide + 1
    assert session.launch_count("qgemm_tc") == before_tc


@pytest.mark.parametrize("m,n,k", [(128, 14336, 4096), (128, 4096, 4096), (512, 4096, 4096)])
def test_prefill_shapes_below_the_wide_tile_threshold(m, n, k):
    """The remaining prefill GEMM shapes (128 tokens; 512 tokens on [4096, 4096]: 32 CTAs) stay on the
    256-token-tile kernel; checked at their full size in bf16 and in the session's compensated mode."""
    before = session.launch_count("qgemm_tc_wide")
    _check_qgemm(quant.Q4_0, m, n, k, 0, seed=m + n + k)
    assert session.launch_count("qgemm_tc_wide") == before
    rng = np.random.default_rng(m * 7 + n)
    data = synth.device_weight(quant.Q4_0, n, k, seed=4)
    x = rng.standard_normal((m, k), dtype=np.float32)
    got, _ = session.qgemm(quant.Q4_0, data, n, k, x, operand_mode=2)
    dense = O.dequantize(quant.Q4_0, data, n * k).reshape(n, k).astype(np.float64)
    want = x.astype(np.float64) @ dense.T
    scale = np.sqrt((x.astype(np.float64) ** 2).sum(1))[:, None] * np.sqrt((dense ** 2).sum(1))[None, :]
    assert (np.abs(got - want) / scale).max() < 2e-6
