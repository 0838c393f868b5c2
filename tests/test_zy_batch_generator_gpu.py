"""The fixed-size batch generator (LlamaBatchGenerator, src/models/transformer/batch_generation.rs:58-189)
over a GPU session: every row must produce exactly the tokens it produces alone, greedy and with the
[step, batch, vocabulary] Gumbel-max tape, with a row that stops early, and the committed lengths."""
import numpy as np
import pytest

from rustgrad_b200 import quant, serving, session, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model():
    cfg = dict(synth.TINY)
    tensors = synth.build_tensors(cfg, seed=0, body_type=quant.Q8_0)
    return cfg, synth.gguf_bytes(cfg, tensors)


def make_session(data, **kw):
    target = session.CudaSessionTarget(**kw)
    return target.prepare(session.LlamaCudaPlan.from_gguf_bytes(data, target))


def alone(data, prompt, max_new, temperature=None, uniforms=None):
    s = make_session(data, max_batch=1, kv_f32=True)
    return s.generate_ids(prompt, max_new, temperature=temperature, uniforms=uniforms).generated_ids


def test_batch_rows_match_isolated_generation(model):
    cfg, data = model
    batch, steps = 3, 6
    prompts = [synth.prompt_ids(cfg, 5 + 2 * r, seed=30 + r) for r in range(batch)]
    want = [alone(data, p, steps) for p in prompts]
    s = make_session(data, max_batch=batch, kv_f32=True)
    gen = serving.LlamaBatchGenerator(s, batch_size=batch)
    seqs = gen.generate_ids(prompts, steps)
    assert [q.generated_ids for q in seqs] == want and not any(q.stopped for q in seqs)
    assert gen.cache_lengths() == [len(p) + steps - 1 for p in prompts]  # the last token is not fed back
    # a stop id that row 1 emits as its third token: that row ends there, the others run on
    stop = want[1][2]
    stopping = serving.LlamaBatchGenerator(s, batch_size=batch, stop_ids=[stop])
    seqs = stopping.generate_ids(prompts, steps)
    for q, w in zip(seqs, want):
        cut = w[:w.index(stop) + 1] if stop in w else w
        assert q.generated_ids == cut and q.stopped == (stop in w)
    # Gumbel-max: row r reads tape row step * batch + r
    rng = np.random.default_rng(5)
    tape = rng.random((steps * batch, cfg["vocab"]), dtype=np.float32)
    seqs = gen.generate_ids(prompts, steps, serving.Sampling(0.8, tape))
    for r, p in enumerate(prompts):
        assert seqs[r].generated_ids == alone(data, p, steps, temperature=0.8, uniforms=tape[r::batch])
    with pytest.raises(serving.BatchGenerationError) as e:
        gen.generate_ids(prompts[:2], steps)
    assert (e.value.kind, e.value.value, e.value.value2) == ("BatchSize", batch, 2)
