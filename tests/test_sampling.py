"""Gumbel-max sampling with an explicit uniform tape (src/models/transformer/generation.rs:10-19,227-287)."""
import numpy as np
import pytest

from oracle import oracle as O
from rustgrad_b200 import quant, synth


def reference_formula(row, temperature, u):
    """The reference's expression in float32, token by token, strict '>' (lowest id wins ties)."""
    best, best_score = -1, None
    t = max(np.float32(temperature), np.float32(1e-12))
    for i, logit in enumerate(row):
        uu = max(np.float32(u[i]), np.float32(1e-12))
        with np.errstate(divide="ignore"):
            score = np.float32(np.float32(logit) / t) - np.log(-np.log(uu, dtype=np.float32), dtype=np.float32)
        if best < 0 or score > best_score:
            best, best_score = i, score
    return best


def test_checker_gumbel_selection_follows_the_reference_expression():
    rng = np.random.default_rng(0)
    for trial in range(20):
        row = rng.standard_normal(97).astype(np.float32) * 3
        u = rng.random(97, dtype=np.float32)
        if trial == 3:
            u[5] = 0.0       # clamped to 1e-12
        if trial == 4:
            u[7] = 1.0       # ln(1) = 0 -> -ln(-0) = +inf score: allowed, only logits are checked
        for temp in (1.0, 0.7, 0.0):
            assert O.select_gumbel(row, temp, u) == reference_formula(row, temp, u)
    # greedy limit: a vanishing temperature makes the largest logit win whatever the noise
    row = np.array([0.0, 2.0, 1.0], dtype=np.float32)
    assert O.select_gumbel(row, 0.0, np.array([0.3, 0.01, 0.9], dtype=np.float32)) == 1
    with pytest.raises(O.OracleError):
        O.select_gumbel(np.array([0.0, np.inf], dtype=np.float32), 1.0, np.array([0.5, 0.5], dtype=np.float32))


@pytest.mark.gpu
def test_sampled_generation_and_batched_sampled_decode_match_the_checker():
    from rustgrad_b200 import session
    cfg = dict(synth.TINY)
    tensors = synth.build_tensors(cfg, seed=0, body_type=quant.Q8_0)
    prompt = synth.prompt_ids(cfg, 9, seed=5)
    rng = np.random.default_rng(1)
    steps, temp = 12, 0.8
    tape = rng.random((steps, cfg["vocab"]), dtype=np.float32)
    oracle = O.OracleModel(cfg, tensors, threads=1)
    want = []
    logits = oracle.forward(prompt)
    for step in range(steps):
        tok = O.select_gumbel(logits, temp, tape[step])
        want.append(tok)
        if step + 1 < steps:
            logits = oracle.forward([tok])
    s = session.LlamaCudaPlan.from_tensors(cfg, tensors, session.CudaSessionTarget(kv_f32=True)).prepare()
    gen = s.generate_ids(prompt, steps, temperature=temp, uniforms=tape)
    assert gen.generated_ids == want
    # the greedy path is untouched by an earlier sampled call
    s.reset_sequence()
    greedy = s.generate_ids(prompt, 6).generated_ids
    oracle.reset()
    assert greedy == oracle.generate_greedy(prompt, 6)[0]
    # two rows sampled in one step, each with its own row of uniforms
    b = session.LlamaCudaPlan.from_tensors(cfg, tensors, session.CudaSessionTarget(kv_f32=True, max_batch=2)).prepare()
    oracles = [O.OracleModel(cfg, tensors, threads=1) for _ in range(2)]
    toks = []
    for r in range(2):
        p = synth.prompt_ids(cfg, 5 + r, seed=20 + r)
        b.prefill_ids(p, row=r)
        toks.append(O.select_greedy(oracles[r].forward(p)))
    u = rng.random((2, cfg["vocab"]), dtype=np.float32)
    lg, ids = b.decode(toks, want_logits=True, temperature=1.3, uniforms=u)
    for r in range(2):
        assert int(ids[r]) == O.select_gumbel(oracles[r].forward([toks[r]]), 1.3, u[r])
    with pytest.raises(ValueError):
        b.decode(toks, temperature=1.0, uniforms=np.zeros((1, 3), dtype=np.float32))  # wrong tape shape
