"""GPU parity of the operator-level entry points against the CPU checker, through the C ABI.

Bar: block decode and row gather bit-exact; quantized matmul within 1e-3 relative of the f64
blockwise plan (src/matmul/quantized.rs:126-182), measured against the row's magnitude scale."""
import numpy as np
import pytest

from oracle import oracle as O
from rustgrad_b200 import quant, session, synth

pytestmark = pytest.mark.gpu


def q4_0_block(scale_bits, low, high):
    return bytes([scale_bits & 0xFF, scale_bits >> 8] + [(low & 15) | ((high & 15) << 4)] * 16)


def q8_0_block(scale_bits):
    return bytes([scale_bits & 0xFF, scale_bits >> 8] + [v & 0xFF for v in range(-16, 16)])


def test_known_answer_blocks_on_device():
    # src/gguf/tests.rs:109-119,179-187 and src/matmul/quantized.rs:356-369
    blk = np.frombuffer(bytes([0x00, 0x3C] + [((15 - i) << 4) | i for i in range(16)]), np.uint8)
    got = session.dequantize(quant.Q4_0, blk, 32)
    assert got.tolist() == [float(v) for v in range(-8, 8)] + [float(v) for v in range(7, -9, -1)]
    blk = np.frombuffer(bytes([0x00, 0x38, 0x80, 0xFF, 0x00, 0x01, 0x7F] + [0] * 27), np.uint8)
    assert session.dequantize(quant.Q8_0, blk, 32)[:5].tolist() == [-64.0, -0.5, 0.0, 0.5, 63.5]
    got = session.dequantize(quant.Q4_0, np.frombuffer(q4_0_block(0x3C00, 3, 14), np.uint8), 32)
    assert got[:16].tolist() == [-5.0] * 16 and got[16:].tolist() == [6.0] * 16
    got = session.dequantize(quant.Q8_0, np.frombuffer(q8_0_block(0x3800), np.uint8), 32)
    assert got[0] == -8.0 and got[31] == 7.5


@pytest.mark.parametrize("kind", [quant.Q4_0, quant.Q8_0, quant.F16])
def test_dequantize_is_bit_exact_including_subnormal_scales(kind):
    rng = np.random.default_rng(7)
    n = 32 * 4096
    if kind == quant.F16:
        data = rng.integers(0, 65536, n, dtype=np.uint16)
        data = data[np.isfinite(data.view(np.float16))]
        n = data.size
        data = data.view(np.uint8)
    else:
        bb = quant.BLOCK_BYTES[kind]
        data = rng.integers(0, 256, (n // 32, bb), dtype=np.uint8)
        scales = rng.integers(0, 0x7C00, n // 32, dtype=np.uint16)      # every finite magnitude, subnormals included
        scales |= rng.integers(0, 2, n // 32, dtype=np.uint16) << 15
        scales[:4] = [0x0001, 0x8001, 0x03FF, 0x0000]
        data[:, :2] = scales.view(np.uint8).reshape(-1, 2)
        data = data.reshape(-1)
    want = O.dequantize(kind, data, n)
    got = session.dequantize(kind, data, n)
    assert got.view(np.uint32).tolist() == want.view(np.uint32).tolist()


def test_non_finite_scale_is_a_typed_error():
    for kind, n in ((quant.Q4_0, 18), (quant.Q8_0, 34)):
        blk = np.frombuffer(bytes([0x00, 0x7C] + [1] * (n - 2)), np.uint8)
        with pytest.raises(session.RgError) as e:
            session.dequantize(kind, blk, 32)
        assert e.value.status == 4
        w = np.tile(blk, 8 * 4)
        with pytest.raises(session.RgError) as e:
            session.qmatmul(kind, w, 4, 256, np.ones((1, 256), np.float32))
        assert e.value.status == 4


def rel_err(got, want, x, wdense):
    scale = np.sqrt((x.astype(np.float64) ** 2).sum(axis=1))[:, None] * np.sqrt((wdense.astype(np.float64) ** 2).sum(axis=1))[None, :]
    return np.abs(got.astype(np.float64) - want.astype(np.float64)) / (scale + 1e-30)


@pytest.mark.parametrize("kind", [quant.Q4_0, quant.Q8_0])
@pytest.mark.parametrize("n,k", [(64, 256), (45, 512), (688, 256), (300, 1024), (1000, 4096), (37, 14336)])
def test_qmatmul_matches_f64_blockwise_plan(kind, n, k):
    rng = np.random.default_rng(n * 31 + k)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    data = quant.encode(kind, w)
    dense = O.dequantize(kind, data, n * k).reshape(n, k)
    for m in (1, 2, 3, 4, 5, 8, 9, 13, 16):  # 9..16: four column tiles
        x = rng.standard_normal((m, k)).astype(np.float32)
        want = O.quantized_matmul(kind, data, n, k, x)
        got = session.qmatmul(kind, data, n, k, x)
        assert got.shape == (m, n)
        err = rel_err(got, want, x, dense)
        assert err.max() < 2e-6, (m, err.max())
        assert np.abs(got - want).max() <= 1e-3 * np.abs(want).max()


@pytest.mark.parametrize("kind", [quant.Q4_0, quant.Q8_0], ids=["q4_0", "q8_0"])
@pytest.mark.parametrize("n,k", [(4096, 4096), (14336, 4096), (4096, 14336), (128256, 4096)])
def test_qmatmul_at_the_decode_sweep_shapes(kind, n, k):
    """The isolated GEMV sweep at its own sizes: weights N(0, 0.02) quantized to Q4_0 / Q8_0,
    activations N(0, 1), 1, 2, 4 and 8 rows (1-2: integer tensor-core kernel, 4-8: f16-MMA kernel),
    against the f64 blockwise plan.  Same bars as the small shapes above."""
    rng = np.random.default_rng(3)
    data = synth.device_weight(kind, n, k, seed=2)
    x8 = rng.standard_normal((8, k), dtype=np.float32)
    want8 = O.quantized_matmul(kind, data, n, k, x8)
    bb = quant.BLOCK_BYTES[kind]
    rows = data.reshape(n, k // 32 * bb)
    wnorm = np.empty(n)
    for r0 in range(0, n, 8192):  # row norms of the decoded weight, a slab at a time
        slab = O.dequantize(kind, rows[r0:r0 + 8192].reshape(-1), rows[r0:r0 + 8192].shape[0] * k)
        wnorm[r0:r0 + 8192] = np.sqrt((slab.reshape(-1, k).astype(np.float64) ** 2).sum(axis=1))
    i8, f16 = session.launch_count("qgemv_i8"), session.launch_count("qgemv")
    for m in (1, 2, 4, 8):
        got = session.qmatmul(kind, data, n, k, x8[:m])
        want = want8[:m]
        scale = np.sqrt((x8[:m].astype(np.float64) ** 2).sum(axis=1))[:, None] * wnorm[None, :]
        err = np.abs(got.astype(np.float64) - want.astype(np.float64)) / scale
        assert err.max() < 2e-6, (m, err.max())
        assert np.abs(got - want).max() <= 1e-3 * np.abs(want).max()
    assert session.launch_count("qgemv_i8") == i8 + 2 and session.launch_count("qgemv") == f16 + 2


def test_qmatmul_more_than_eight_rows_and_dense_weights():
    rng = np.random.default_rng(5)
    n, k = 96, 512
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    x = rng.standard_normal((19, k)).astype(np.float32)
    data = quant.encode(quant.Q8_0, w)
    got = session.qmatmul(quant.Q8_0, data, n, k, x)
    want = O.quantized_matmul(quant.Q8_0, data, n, k, x)
    assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
    for kind in (quant.F32, quant.F16):
        k2 = 688  # not a multiple of 32: only dense storage can hold it
        w2 = (rng.standard_normal((n, k2)) * 0.05).astype(np.float32)
        x2 = rng.standard_normal((3, k2)).astype(np.float32)
        d2 = quant.encode(kind, w2)
        dense = O.dequantize(kind, d2, n * k2).reshape(n, k2)
        got = session.qmatmul(kind, d2, n, k2, x2)
        want = (x2.astype(np.float64) @ dense.astype(np.float64).T)
        assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())


def test_qmatmul_extreme_activations_keep_f32_precision():
    # the hi/lo f16 split must not lose small or large activation magnitudes
    rng = np.random.default_rng(9)
    n, k = 64, 1024
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    data = quant.encode(quant.Q4_0, w)
    dense = O.dequantize(quant.Q4_0, data, n * k).reshape(n, k)
    for scale in (1e-4, 1.0, 3e3):
        for m in (2, 4, 12):  # integer kernel; f16-MMA kernel with one and with four column tiles
            x = (rng.standard_normal((m, k)) * scale).astype(np.float32)
            got = session.qmatmul(quant.Q4_0, data, n, k, x)
            want = O.quantized_matmul(quant.Q4_0, data, n, k, x)
            assert rel_err(got, want, x, dense).max() < 4e-6, (scale, m)


def test_qmatmul_rejects_unsupported_geometry_and_types():
    w = np.zeros(18 * 3, np.uint8)
    with pytest.raises(session.RgError) as e:
        session.qmatmul(quant.Q4_0, w, 1, 96, np.ones((1, 96), np.float32))
    assert e.value.status == 20
    with pytest.raises(session.RgError) as e:
        session.qmatmul(13, w, 1, 256, np.ones((1, 256), np.float32))  # Q5_K is outside this path
    assert e.value.status == 2
    with pytest.raises(session.RgError) as e:
        session.qmatmul(quant.Q4_0, w, 1, 40, np.ones((1, 40), np.float32))
    assert e.value.status == 3


def test_row_gather_is_bit_exact_and_preflights_indices():
    rng = np.random.default_rng(3)
    rows, cols = 50, 256
    for kind in (quant.Q8_0, quant.Q4_0, quant.F32):
        data = quant.encode(kind, (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32))
        idx = [49, 0, 7, 7, 13]
        got = session.row_gather(kind, data, rows, cols, idx)
        want = O.row_gather(kind, data, rows, cols, idx)
        assert got.tobytes() == want.tobytes()
        for bad in ([0, 50], [-1]):
            with pytest.raises(session.RgError) as e:
                session.row_gather(kind, data, rows, cols, bad)
            assert e.value.status == 5
        assert session.row_gather(kind, data, rows, cols, []).shape == (0, cols)


@pytest.mark.parametrize("heads,kv_heads,hd", [(4, 4, 64), (8, 2, 128), (32, 8, 128), (16, 2, 128)])
@pytest.mark.parametrize("n_pos", [1, 31, 128, 129, 700])
def test_decode_attention_matches_reference_softmax_composition(heads, kv_heads, hd, n_pos):
    # tolerance: 1e-5 absolute on outputs that are convex combinations of N(0,1) values
    rng = np.random.default_rng(heads * 1000 + n_pos)
    q = rng.standard_normal((heads, hd)).astype(np.float32)
    k = rng.standard_normal((kv_heads, n_pos, hd)).astype(np.float32)
    v = rng.standard_normal((kv_heads, n_pos, hd)).astype(np.float32)
    want = O.attention_decode(q, k, v)
    got = session.attention_decode(q, k, v)
    assert np.abs(got - want).max() <= 1e-5
    k16, v16 = k.astype(np.float16), v.astype(np.float16)
    want16 = O.attention_decode(q, k16.astype(np.float32), v16.astype(np.float32))
    got16 = session.attention_decode(q, k16, v16)
    assert np.abs(got16 - want16).max() <= 1e-5


def test_decode_attention_rejects_unsupported_head_geometry():
    q = np.zeros((6, 96), np.float32)
    kv = np.zeros((2, 4, 96), np.float32)
    with pytest.raises(session.RgError) as e:
        session.attention_decode(q, kv, kv)
    assert e.value.status == 20


def test_opt_in_row_gemv_matches_f64_blockwise_plan():
    """The second 3..16-row GEMV (qgemv_rows.cu, switched on by RG_B200_ROWS_GEMV=1 when the library
    loads, hence the child process): tall row tiles, K split over CTAs for matrices with few rows and
    the in-order merge by the last CTA to arrive; 3..16 rows against the f64 blockwise plan."""
    import os
    import subprocess
    import sys
    code = r'''
import numpy as np
from oracle import oracle as O
from rustgrad_b200 import quant, session
rng = np.random.default_rng(7)
before = session.launch_count("qgemv_rows")
for n, k in ((64, 256), (45, 512), (300, 1024), (1000, 4096), (4096, 4096), (37, 14336), (6144, 1024)):
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    data = quant.encode(quant.Q4_0, w)
    dense = O.dequantize(quant.Q4_0, data, n * k).reshape(n, k)
    wn = np.sqrt((dense.astype(np.float64) ** 2).sum(axis=1))
    for m in (3, 4, 8, 11, 16):
        x = rng.standard_normal((m, k)).astype(np.float32)
        want = O.quantized_matmul(quant.Q4_0, data, n, k, x)
        got = session.qmatmul(quant.Q4_0, data, n, k, x)
        scale = np.sqrt((x.astype(np.float64) ** 2).sum(axis=1))[:, None] * wn[None, :]
        err = np.abs(got.astype(np.float64) - want.astype(np.float64)) / (scale + 1e-30)
        assert err.max() < 2e-6, (n, k, m, err.max())
assert session.launch_count("qgemv_rows") == before + 7 * 5
print("ok")
'''
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, RG_B200_ROWS_GEMV="1", PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr
