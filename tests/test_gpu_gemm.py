"""Prefill GEMM on the tcgen05 tensor cores against the CPU dequant + matmul (BASELINE config 3).

Operands are bf16 (activations rounded to bf16, weights bf16(bf16(d) * (n - 8))), accumulation f32.
Tolerance: the error of rounding both operands to bf16 is 2^-8 relative per product and averages
out over K; the bound used is 2e-2 of |x|.|w| per output (norm-relative), and 1e-3 of it against a
reference that applies the same operand rounding."""
import numpy as np
import pytest

from oracle import oracle as O
from rustgrad_b200 import quant, session

pytestmark = pytest.mark.gpu


def to_bf16(a):
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((b >> 16) & 1) + 0x7FFF
    return (((b + r) >> 16) << 16).astype(np.uint32).view(np.float32)


def bf16_weight(kind, data, n, k):
    """The operand the kernel builds: bf16(bf16(d) * q) for Q4_0, bf16(d * q) for Q8_0."""
    dense = O.dequantize(kind, data, n * k).reshape(n, k // 32, 32)
    bb = quant.BLOCK_BYTES[kind]
    d = data.reshape(n, k // 32, bb)[:, :, :2].copy().view(np.float16).astype(np.float32)  # [n, blocks, 1]
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(d != 0, np.rint(dense / d), 0.0).astype(np.float32)
    if kind == quant.Q8_0:
        return to_bf16(dense).reshape(n, k)
    return to_bf16(to_bf16(d) * q).reshape(n, k)


@pytest.mark.parametrize("kind", [quant.Q4_0, quant.Q8_0])
@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (16, 128, 512), (200, 300, 1024), (33, 4096, 4096), (512, 1024, 4096)])
def test_qgemm_matches_cpu_dequant_matmul(kind, m, n, k):
    rng = np.random.default_rng(m + n + k)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    data = quant.encode(kind, w)
    got, _ = session.qgemm(kind, data, n, k, x)
    dense = O.dequantize(kind, data, n * k).reshape(n, k)
    scale = np.sqrt((x.astype(np.float64) ** 2).sum(1))[:, None] * np.sqrt((dense.astype(np.float64) ** 2).sum(1))[None, :]
    want = x.astype(np.float64) @ dense.astype(np.float64).T
    assert (np.abs(got - want) / scale).max() < 2e-2 / np.sqrt(k) * 8
    same_rounding = to_bf16(x).astype(np.float64) @ bf16_weight(kind, data, n, k).astype(np.float64).T
    assert (np.abs(got - same_rounding) / scale).max() < 1e-5
