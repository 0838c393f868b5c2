"""Pins the strict CPU forward on rustgrad's formula-defined model fixtures.

The reference has no golden logits; its model tests compare against an independent f64 forward on
deterministic weights (src/models/transformer/model_tests.rs:16-87,343-377: 3e-5 abs) and compare
a packed model against its dequantized control (packed_tests.rs:339-351,620-679: 1e-3 abs, equal
greedy ids).  The fixture weights are regenerated here from their formula.
"""
import numpy as np

from oracle import oracle as O
from rustgrad_b200 import quant, synth

DENSE_CFG = dict(n_layers=2, d_model=8, n_heads=2, n_kv_heads=1, head_dim=4, ffn_dim=10, vocab=12, max_context=8,
                 norm_eps=1e-5, rope_theta=10.0, eos_id=1, eot_id=2)


def values(n, salt, scale):
    i = np.arange(n, dtype=np.int64)
    return (((i * 17 + salt * 11) % 29).astype(np.float32) - np.float32(14.0)) * np.float32(scale)


def dense_fixture():
    c = DENSE_CFG
    d, hid, qw, kw = c["d_model"], c["ffn_dim"], c["n_heads"] * c["head_dim"], c["n_kv_heads"] * c["head_dim"]

    def t(rows, cols, salt, scale):
        return (O.F32, rows, cols, values(rows * cols, salt, scale).view(np.uint8))

    def vec(fn):
        return (O.F32, 1, d, np.array([fn(i) for i in range(d)], dtype=np.float32).view(np.uint8))

    f32 = np.float32
    tensors = {"token_embd.weight": t(c["vocab"], d, 1, 0.018),
               "output_norm.weight": vec(lambda i: f32(0.92) + f32(i) * f32(0.015))}
    for layer in range(2):
        p, salt = f"blk.{layer}.", layer * 9
        tensors[p + "attn_norm.weight"] = vec(lambda i: f32(1.03) - f32(i) * f32(0.01) + f32(layer) * f32(0.005))
        tensors[p + "attn_q.weight"] = t(qw, d, salt + 2, 0.012)
        tensors[p + "attn_k.weight"] = t(kw, d, salt + 3, 0.014)
        tensors[p + "attn_v.weight"] = t(kw, d, salt + 4, 0.013)
        tensors[p + "attn_output.weight"] = t(d, qw, salt + 5, 0.011)
        tensors[p + "ffn_norm.weight"] = vec(lambda i: f32(0.97) + f32(i) * f32(0.008) + f32(layer) * f32(0.004))
        tensors[p + "ffn_gate.weight"] = t(hid, d, salt + 6, 0.010)
        tensors[p + "ffn_up.weight"] = t(hid, d, salt + 7, 0.009)
        tensors[p + "ffn_down.weight"] = t(d, hid, salt + 8, 0.010)
    return tensors


def test_strict_forward_matches_independent_f64_forward_on_dense_fixture():
    m = O.OracleModel(DENSE_CFG, dense_fixture(), threads=1)
    tokens = [3, 4, 5]
    got = m.forward(tokens, O.MODE_STRICT, all_logits=True)
    want = m.forward_f64(tokens)
    assert got.shape == (3, 12)
    assert np.abs(got - want).max() <= 3e-5
    assert np.abs(want).max() > 1e-3  # the fixture is not degenerate


def variant_fixture(qk_norm, rope_dim=2):
    """The dense fixture with partial rotary lanes, q / k RMS norms and q / k / v biases, weights by the
    formulas of src/models/transformer/model_tests.rs:258-297."""
    c = dict(DENSE_CFG, rope_dim=rope_dim, qk_norm=qk_norm, qkv_bias=1)
    if qk_norm == 2:  # per projection: equal query and key widths only (model.rs:262-268)
        c["n_kv_heads"] = c["n_heads"]
    hd, qw, kw = c["head_dim"], c["n_heads"] * c["head_dim"], c["n_kv_heads"] * c["head_dim"]
    tensors = dense_fixture()
    if qk_norm == 2:
        for layer in range(2):
            p, salt = f"blk.{layer}.", layer * 9
            for name, s_, sc in (("attn_k.weight", 3, 0.014), ("attn_v.weight", 4, 0.013)):
                tensors[p + name] = (O.F32, kw, c["d_model"], values(kw * c["d_model"], salt + s_, sc).view(np.uint8))
    f32 = np.float32
    for layer in range(2):
        p = f"blk.{layer}."
        nq, nk = (hd, hd) if qk_norm == 1 else (qw, kw)
        tensors[p + "attn_q_norm.weight"] = (O.F32, 1, nq, np.array(
            [f32(0.91) + f32(layer) * f32(0.02) + f32(i % hd) * f32(0.03) for i in range(nq)], dtype=np.float32).view(np.uint8))
        tensors[p + "attn_k_norm.weight"] = (O.F32, 1, nk, np.array(
            [f32(1.07) - f32(layer) * f32(0.01) - f32(i % hd) * f32(0.02) for i in range(nk)], dtype=np.float32).view(np.uint8))
        for name, width, salt in (("attn_q.bias", qw, 3), ("attn_k.bias", kw, 5), ("attn_v.bias", kw, 7)):
            tensors[p + name] = (O.F32, 1, width, np.array(
                [(f32(i + layer * 3 + salt) - f32(8.0)) * f32(0.004) for i in range(width)], dtype=np.float32).view(np.uint8))
    return c, tensors


def test_partial_rotary_qk_norms_and_biases_match_independent_f64_forward():
    # src/models/transformer/model_tests.rs:380-411 (per head, rope_dim 2: 5e-5) and :457 (per projection)
    for qk_norm, rope_dim in ((1, 2), (2, 2), (0, 2), (1, 4)):
        cfg, tensors = variant_fixture(qk_norm, rope_dim)
        if qk_norm == 0:
            cfg["qk_norm"] = 0
            tensors = {k: v for k, v in tensors.items() if "_norm.weight" not in k or "attn_q_norm" not in k and "attn_k_norm" not in k}
        m = O.OracleModel(cfg, tensors, threads=1)
        tokens = [3, 4, 5]
        full = m.forward(tokens, O.MODE_STRICT, all_logits=True)
        assert np.abs(full - m.forward_f64(tokens)).max() <= 5e-5, (qk_norm, rope_dim)
        m.reset()
        step = np.stack([m.forward([t]) for t in tokens])
        m.reset()
        chunk = np.concatenate([m.forward(tokens[:2], all_logits=True), m.forward(tokens[2:], all_logits=True)])
        assert np.abs(full - step).max() <= 5e-5 and np.abs(full - chunk).max() <= 5e-5
    # the variants change the result: the same weights without them give other logits
    plain = O.OracleModel(DENSE_CFG, dense_fixture(), threads=1).forward([3, 4, 5])
    cfg, tensors = variant_fixture(1, 2)
    assert np.abs(O.OracleModel(cfg, tensors, threads=1).forward([3, 4, 5]) - plain).max() > 1e-4
    # a variant tensor the configuration does not name is refused, a missing one too
    try:
        O.OracleModel(DENSE_CFG, tensors, threads=1)
        raise AssertionError("expected a refusal")
    except O.OracleError:
        pass
    missing = {k: v for k, v in tensors.items() if k != "blk.1.attn_v.bias"}
    try:
        O.OracleModel(cfg, missing, threads=1)
        raise AssertionError("expected a refusal")
    except O.OracleError:
        pass


def test_full_equals_tokenwise_equals_chunked_cache():
    # src/models/transformer/model_tests.rs:643-669
    m = O.OracleModel(DENSE_CFG, dense_fixture(), threads=1)
    tokens = [3, 4, 5, 6, 3]
    full = m.forward(tokens, all_logits=True)
    m.reset()
    step = np.stack([m.forward([t]) for t in tokens])
    m.reset()
    chunk = np.concatenate([m.forward(tokens[:2], all_logits=True), m.forward(tokens[2:], all_logits=True)])
    assert np.abs(full - step).max() <= 1e-6 and np.abs(full - chunk).max() <= 1e-6
    assert m.position == 5


def test_cache_commits_only_on_success():
    # src/models/transformer/model.rs:917-920; generation.rs:115-124
    m = O.OracleModel(DENSE_CFG, dense_fixture(), threads=1)
    m.forward([3, 4])
    for bad, code in (([12], O.ERR_TOKEN_RANGE), ([-1], O.ERR_TOKEN_RANGE), ([3] * 7, O.ERR_CONTEXT)):
        try:
            m.forward(bad)
            raise AssertionError("expected a typed failure")
        except O.OracleError as e:
            assert e.code == code
        assert m.position == 2


def packed_model(body, seed=5):
    cfg = dict(n_layers=2, d_model=256, n_heads=2, n_kv_heads=1, head_dim=128, ffn_dim=512, vocab=96, max_context=48,
               norm_eps=1e-5, rope_theta=10000.0)
    return cfg, synth.build_tensors(cfg, seed, body_type=body, std=0.05)


def test_packed_model_strict_fast_and_f64_agree_and_pick_equal_greedy_ids():
    for body in (quant.Q4_0, quant.Q8_0):
        cfg, tensors = packed_model(body)
        m = O.OracleModel(cfg, tensors, threads=4)
        prompt = synth.prompt_ids(cfg, 9, seed=3)
        strict = m.forward(prompt, O.MODE_STRICT, all_logits=True)
        m.reset()
        fast = m.forward(prompt, O.MODE_FAST, all_logits=True)
        f64 = m.forward_f64(prompt)
        assert np.abs(strict - f64).max() <= 1e-3
        assert np.abs(fast - strict).max() <= 1e-4
        ids_strict, _ = m.generate_greedy(prompt, 12, O.MODE_STRICT)
        ids_fast, _ = m.generate_greedy(prompt, 12, O.MODE_FAST)
        assert ids_strict == ids_fast and len(ids_strict) == 12


def test_packed_head_uses_f64_blockwise_plan():
    # src/models/transformer/model.rs:1036-1064: a packed (here tied) head runs the f64-accumulating plan
    cfg, tensors = packed_model(quant.Q8_0)
    m = O.OracleModel(cfg, tensors, threads=1)
    logits = m.forward([7])
    t, rows, cols, data = tensors["token_embd.weight"]
    # recompute the final normalized state through an F32 copy of the head and compare the two rules
    dense = O.dequantize(t, data, rows * cols).reshape(rows, cols)
    tensors_dense = dict(tensors)
    tensors_dense["output.weight"] = (O.F32, rows, cols, dense.view(np.uint8).reshape(-1))
    m2 = O.OracleModel(cfg, tensors_dense, threads=1)
    logits_dense_rule = m2.forward([7])
    assert np.abs(logits - logits_dense_rule).max() <= 1e-5
    assert (logits != logits_dense_rule).any()  # f64 vs sequential f32 accumulation differ in the last bits


def test_generate_stops_on_eos_and_does_not_feed_last_token():
    # src/models/transformer/generation.rs:141-151
    cfg, tensors = packed_model(quant.Q8_0)
    m = O.OracleModel(cfg, tensors, threads=2)
    prompt = synth.prompt_ids(cfg, 5, seed=1)
    ids, stopped = m.generate_greedy(prompt, 6)
    assert not stopped and m.position == 5 + 6 - 1
    cfg2 = dict(cfg, eos_id=ids[2])
    m2 = O.OracleModel(cfg2, tensors, threads=2)
    ids2, stopped2 = m2.generate_greedy(prompt, 6)
    first = ids.index(ids[2])
    assert stopped2 and ids2 == ids[: first + 1]
