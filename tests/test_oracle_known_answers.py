"""Pins the CPU checker against the known-answer vectors of rustgrad's own tests.

Sources: src/gguf/tests.rs:105-187,413-441,872-876 (block order, packed retention, geometry
table) and src/matmul/quantized.rs:254-264,356-416 (fixture blocks, blockwise plan == dense f64
oracle), src/gguf/quantization/row_gather.rs (index preflight).
"""
import numpy as np
import pytest

from oracle import oracle as O


def q4_0_block(scale_bits, low, high):
    return bytes([scale_bits & 0xFF, scale_bits >> 8] + [(low & 15) | ((high & 15) << 4)] * 16)


def q8_0_block(scale_bits):
    return bytes([scale_bits & 0xFF, scale_bits >> 8] + [v & 0xFF for v in range(-16, 16)])


def test_q4_0_block_order_known_answer():
    # src/gguf/tests.rs:109-110,179-185: d = 1.0, byte i = ((15 - i) << 4) | i
    blk = bytes([0x00, 0x3C] + [((15 - i) << 4) | i for i in range(16)])
    got = O.dequantize(O.Q4_0, np.frombuffer(blk, np.uint8), 32)
    want = [float(v) for v in range(-8, 8)] + [float(v) for v in range(7, -9, -1)]
    assert got.tolist() == want
    two = O.dequantize(O.Q4_0, np.frombuffer(blk + blk, np.uint8), 64)
    assert two[:32].tolist() == want and two[32:].tolist() == want


def test_q8_0_block_known_answer():
    # src/gguf/tests.rs:117-119,186-187: d = 0.5, bytes 80 ff 00 01 7f
    blk = bytes([0x00, 0x38, 0x80, 0xFF, 0x00, 0x01, 0x7F] + [0] * 27)
    got = O.dequantize(O.Q8_0, np.frombuffer(blk, np.uint8), 32)
    assert got[:5].tolist() == [-64.0, -0.5, 0.0, 0.5, 63.5]
    assert not got[5:].any()


def test_matmul_fixture_blocks_known_answer():
    # src/matmul/quantized.rs:254-264,356-369
    q4 = O.dequantize(O.Q4_0, np.frombuffer(q4_0_block(0x3C00, 3, 14), np.uint8), 32)
    assert q4[:16].tolist() == [-5.0] * 16 and q4[16:].tolist() == [6.0] * 16
    q8 = O.dequantize(O.Q8_0, np.frombuffer(q8_0_block(0x3800), np.uint8), 32)
    assert q8[0] == -8.0 and q8[31] == 7.5


def test_rank_two_packed_weight_decodes_rowwise():
    # src/gguf/tests.rs:413-441: [2,32] Q4_0, d = 1, every byte 0xe3 -> low 3, high 14
    blk = bytes([0x00, 0x3C] + [0xE3] * 16)
    got = O.dequantize(O.Q4_0, np.frombuffer(blk + blk, np.uint8), 64).reshape(2, 32)
    assert (got[:, :16] == -5.0).all() and (got[:, 16:] == 6.0).all()


def test_geometry_table():
    # src/gguf/tests.rs:872-879: (raw id, block elements, block bytes)
    L = O.lib()
    assert (L.rgo_block_elements(2), L.rgo_block_bytes(2)) == (32, 18)
    assert (L.rgo_block_elements(8), L.rgo_block_bytes(8)) == (32, 34)
    assert (L.rgo_block_elements(0), L.rgo_block_bytes(0)) == (1, 4)
    assert (L.rgo_block_elements(1), L.rgo_block_bytes(1)) == (1, 2)
    assert (L.rgo_block_elements(12), L.rgo_block_bytes(12)) == (256, 144)
    assert (L.rgo_block_elements(14), L.rgo_block_bytes(14)) == (256, 210)
    assert L.rgo_block_elements(13) == 0  # Q5_K is outside this path


@pytest.mark.parametrize("kind,block", [(O.Q4_0, q4_0_block(0x3C00, 3, 14)), (O.Q8_0, q8_0_block(0x3800))])
def test_blockwise_plan_equals_dense_f64_oracle(kind, block):
    # src/matmul/quantized.rs:389-416: fixture(kind, rows=3, blocks_per_row=2); activation
    # ((index % 13) - 6) / 7 for shapes [k] and [2,2,k]; results must be bit-equal.
    rows, bpr = 3, 2
    k = 32 * bpr
    w = np.frombuffer(block * (rows * bpr), np.uint8)
    dense = O.dequantize(kind, w, rows * k).reshape(rows, k).astype(np.float64)
    for m in (1, 4):
        a = (((np.arange(m * k) % 13).astype(np.float32) - np.float32(6.0)) / np.float32(7.0)).astype(np.float32)
        got = O.quantized_matmul(kind, w, rows, k, a)
        want = np.empty((m, rows), np.float32)
        for r in range(m):
            for c in range(rows):
                acc = 0.0
                for i in range(k):  # k ascending, f64 accumulate, one cast
                    acc += float(a[r * k + i]) * float(dense[c, i])
                want[r, c] = np.float32(acc)
        assert got.tobytes() == want.tobytes()


def test_f16_conversion_exhaustive_against_numpy():
    # src/tensor/scalar.rs:110-135: exact for every half bit pattern, subnormals included
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([O.f16_to_f32(int(b)) for b in bits], dtype=np.float32)
    finite = np.isfinite(want)
    assert (got[finite].view(np.uint32) == want[finite].view(np.uint32)).all()
    assert (np.isnan(got) == np.isnan(want)).all() and (np.isinf(got) == np.isinf(want)).all()
    assert O.f16_to_f32(0x0001) == 2.0 ** -24  # smallest subnormal (quantized.rs:299)


def test_f32_to_f16_round_to_nearest_even():
    rng = np.random.default_rng(11)
    xs = np.concatenate([rng.standard_normal(4000).astype(np.float32) * np.float32(s) for s in (1e-7, 1e-3, 1, 300, 7e4)])
    xs = np.concatenate([xs, np.array([0.0, -0.0, 65504.0, 65520.0, 1e-8, 6.1e-5, np.inf, -np.inf], np.float32)])
    want = xs.astype(np.float16).view(np.uint16)
    got = np.array([O.f32_to_f16(float(x)) for x in xs], dtype=np.uint16)
    assert (got == want).all()


def test_non_finite_scale_is_rejected():
    # src/gguf/quantization/blocks.rs:1246-1249,1496-1498
    for kind, n in ((O.Q4_0, 18), (O.Q8_0, 34)):
        for scale in (0x7C00, 0xFC00, 0x7E00):
            blk = bytes([scale & 0xFF, scale >> 8] + [1] * (n - 2))
            with pytest.raises(O.OracleError) as e:
                O.dequantize(kind, np.frombuffer(blk, np.uint8), 32)
            assert e.value.code == O.ERR_NON_FINITE


def test_row_gather_preflights_every_index():
    # src/gguf/quantization/row_gather.rs:187-226: a bad index fails before any decode; repeats allowed
    rows = [q8_0_block(0x3800), q8_0_block(0x3C00), q8_0_block(0x4000)]
    w = np.frombuffer(b"".join(rows), np.uint8)
    got = O.row_gather(O.Q8_0, w, 3, 32, [2, 0, 2])
    assert got[0, 0] == -32.0 and got[1, 0] == -8.0 and (got[0] == got[2]).all()
    for bad in ([0, 3], [-1], [1, 2, 99]):
        with pytest.raises(O.OracleError) as e:
            O.row_gather(O.Q8_0, w, 3, 32, bad)
        assert e.value.code == O.ERR_INDEX
    assert O.row_gather(O.Q8_0, w, 3, 32, []).shape == (0, 32)


def test_greedy_lowest_id_wins_ties_and_rejects_non_finite():
    # src/models/transformer/generation.rs:268-287
    assert O.select_greedy(np.array([0.5, 2.0, 2.0, -1.0], np.float32)) == 1
    assert O.select_greedy(np.array([-3.0], np.float32)) == 0
    for bad in (np.nan, np.inf, -np.inf):
        with pytest.raises(O.OracleError) as e:
            O.select_greedy(np.array([0.0, bad, 5.0], np.float32))
        assert e.value.code == O.ERR_NON_FINITE_LOGITS
