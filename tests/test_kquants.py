"""Q4_K / Q6_K super-blocks (src/gguf/quantization/blocks.rs:1164-1187,1219-1240,1511-1522): decode pinned
on the reference's formula-defined fixtures (src/matmul/quantized.rs:266-301), GPU decode bit-exact, and a
small model with K-quant projections against the CPU checker."""
import numpy as np
import pytest

from oracle import oracle as O
from rustgrad_b200 import quant, synth


def f16_bytes(bits):
    return [bits & 0xFF, bits >> 8]


def reference_q4_k_block():
    """q4_k_block() of matmul/quantized.rs:266-286, rebuilt from its formula."""
    scales = [1, 2, 3, 4, 17, 33, 49, 63]
    mins = [0, 1, 2, 3, 16, 32, 48, 62]
    packed = [0] * 12
    for lane in range(4):
        packed[lane] = scales[lane] | ((scales[4 + lane] >> 4) << 6)
        packed[4 + lane] = mins[lane] | ((mins[4 + lane] >> 4) << 6)
        packed[8 + lane] = (scales[4 + lane] & 15) | ((mins[4 + lane] & 15) << 4)
    out = f16_bytes(0x3800) + f16_bytes(0x3400) + packed  # d = 0.5, dmin = 0.25
    for pair in range(4):
        out += [(pair * 2 + 1) | ((pair * 2 + 2) << 4)] * 32
    return np.array(out, dtype=np.uint8), scales, mins


def reference_q6_k_block():
    """q6_k_block() of matmul/quantized.rs:288-301."""
    out = np.zeros(210, dtype=np.uint8)
    for index in range(256):
        raw = (index * 29 + 7) & 63
        half_index, within = index // 128, index % 128
        out[half_index * 64 + within % 64] |= (raw & 15) << ((within // 64) * 4)
        out[128 + half_index * 32 + within % 32] |= ((raw >> 4) & 3) << ((within // 32) * 2)
    for index, scale in enumerate(range(-8, 8)):
        out[192 + index] = scale & 0xFF
    out[208:210] = f16_bytes(0x0001)  # smallest half subnormal
    return out


def test_geometry_table():
    # src/gguf/tests.rs:872-879
    assert (quant.BLOCK_ELEMS[quant.Q4_K], quant.BLOCK_BYTES[quant.Q4_K]) == (256, 144)
    assert (quant.BLOCK_ELEMS[quant.Q6_K], quant.BLOCK_BYTES[quant.Q6_K]) == (256, 210)
    assert quant.Q4_K == 12 and quant.Q6_K == 14


def test_checker_decodes_the_reference_fixture_blocks():
    block, scales, mins = reference_q4_k_block()
    got = O.dequantize(quant.Q4_K, block, 256)
    # group g holds the constant quant g + 1: value = 0.5 * scale * (g + 1) - 0.25 * min
    want = np.repeat([np.float32(0.5) * s * (g + 1) - np.float32(0.25) * m for g, (s, m) in enumerate(zip(scales, mins))], 32)
    assert np.array_equal(got, want.astype(np.float32))
    assert got[0] == 0.5 and got[32] == 1.75 and got[255] == 236.5
    block6 = reference_q6_k_block()
    got6 = O.dequantize(quant.Q6_K, block6, 256)
    d = np.float32(2.0 ** -24)
    want6 = np.array([d * np.float32((((i * 29 + 7) & 63) - 32) * (-8 + i // 16)) for i in range(256)], dtype=np.float32)
    assert np.array_equal(got6, want6)
    # a non-finite super-block scale is a decode error
    bad = block.copy()
    bad[2:4] = f16_bytes(0x7C00)
    with pytest.raises(O.OracleError):
        O.dequantize(quant.Q4_K, bad, 256)


@pytest.mark.gpu
@pytest.mark.parametrize("kind", [quant.Q4_K, quant.Q6_K], ids=["q4_k", "q6_k"])
def test_gpu_block_decode_row_gather_and_matmul(kind):
    from rustgrad_b200 import session
    rng = np.random.default_rng(3)
    rows, cols = 24, 768
    data = quant.random_k_blocks(kind, rows * cols // 256, rng)
    want = O.dequantize(kind, data, rows * cols)
    got = session.dequantize(kind, data, rows * cols)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))  # bit-exact
    fixture = reference_q4_k_block()[0] if kind == quant.Q4_K else reference_q6_k_block()
    assert np.array_equal(session.dequantize(kind, fixture, 256), O.dequantize(kind, fixture, 256))
    idx = np.array([5, 0, 23, 5], dtype=np.int64)
    assert np.array_equal(session.row_gather(kind, data, rows, cols, idx), want.reshape(rows, cols)[idx])
    x = rng.standard_normal((3, cols)).astype(np.float32)
    y = session.qmatmul(kind, data, rows, cols, x)
    ref = x.astype(np.float64) @ want.reshape(rows, cols).astype(np.float64).T
    assert np.abs(y - ref).max() <= 2e-6 * np.abs(ref).max() + 1e-7
    bad = data.copy()
    bad[(1 if kind == quant.Q4_K else 209)] = 0x7C  # infinite d
    with pytest.raises(session.RgError) as err:
        session.dequantize(kind, bad, rows * cols)
    assert err.value.status == 4  # NON_FINITE_SCALE


@pytest.mark.gpu
def test_model_with_k_quant_projections_matches_cpu_path():
    from rustgrad_b200 import session
    cfg = synth.scaled(synth.TINY, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn_dim=512, vocab=384, n_layers=2)
    rng = np.random.default_rng(7)
    tensors = {}
    for name, rows, cols, is_norm in synth.tensor_inventory(cfg, tied_head=False):
        if is_norm:
            tensors[name] = (quant.F32, 1, cols, np.ones(cols, dtype=np.float32).view(np.uint8))
        else:
            kind = quant.Q6_K if name in ("token_embd.weight", "output.weight", "blk.0.ffn_down.weight") else quant.Q4_K
            tensors[name] = (kind, rows, cols, quant.random_k_blocks(kind, rows * cols // 256, rng, scale=0.05))
    prompt = synth.prompt_ids(cfg, 11, seed=3)
    oracle = O.OracleModel(cfg, tensors, threads=4)
    s = session.LlamaCudaPlan.from_tensors(cfg, tensors, session.CudaSessionTarget(kv_f32=True)).prepare()
    want = oracle.forward(prompt)
    got = s.prefill_ids(prompt)
    diff = np.abs(got - want).max()
    assert diff <= 1e-2 and diff <= 1e-3 * np.abs(want).max() + 1e-6, (diff, np.abs(want).max())
    tok = O.select_greedy(want)
    for _ in range(5):
        w = oracle.forward([tok])
        logits, greedy = s.decode([tok], want_logits=True)
        d = np.abs(logits[0] - w).max()
        assert d <= 1e-2 and d <= 1e-3 * np.abs(w).max() + 1e-6
        assert int(greedy[0]) == O.select_greedy(w)
        tok = int(greedy[0])
