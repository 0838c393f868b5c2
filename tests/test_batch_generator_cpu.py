"""The fixed-size batch generator of include/rg_b200_serving.h (LlamaBatchGenerator,
src/models/transformer/batch_generation.rs:58-247) driven through a table of Python callables: the
compiled host logic -- checks in the reference's order, per-row stop state, the [step, batch,
vocabulary] tape, lengths committed only on success -- without a device."""
import numpy as np
import pytest

from rustgrad_b200 import serving
from test_serving_cpu import VOCAB, BatchingSession, FakeSession, alone, fake_logits, next_token, pick


def sampled_alone(prompt, n, temperature, tape, row, batch, stop=()):
    """One row on its own with the tape rows (step * batch + row) the batch run gives it."""
    history, out = list(prompt), []
    for step in range(n):
        out.append(pick(fake_logits(history), temperature, tape[step * batch + row]))
        history.append(out[-1])
        if out[-1] in stop:
            break
    return out


def test_rows_are_independent_and_lengths_commit_on_success():
    fake = BatchingSession()
    prompts = [[1, 2, 3], [4, 5], [6, 7, 8, 9]]
    stop = next_token([4, 5])  # row 1 stops at its first token
    gen = serving.LlamaBatchGenerator(fake, batch_size=3, stop_ids=[stop])
    assert gen.cache_lengths() == [0, 0, 0]
    seqs = gen.generate_ids(prompts, 4)
    for r, (q, p) in enumerate(zip(seqs, prompts)):
        want = alone(p, 4, stop=(stop,))
        assert (q.prompt_ids, q.generated_ids, q.stopped, q.decoded, q.request_id) == (p, want, want[-1] == stop, "", r)
    assert seqs[1].stopped and len(seqs[1].generated_ids) == 1
    # one pass over all prompts, then one launch sequence per step over the rows still running;
    # the last token is not fed back: three decode steps for four tokens
    assert ("prefill_rows", (0, 1, 2), (3, 2, 4)) in fake.calls
    decodes = [c for c in fake.calls if c[0] == "decode"]
    assert len(decodes) == 3 and all(c[1] == (0, 2) for c in decodes)
    assert gen.cache_lengths() == [3 + 3, 2, 4 + 3]
    # every generate starts from empty rows
    again = gen.generate_ids(prompts, 2)
    assert [q.generated_ids for q in again] == [alone(p, 2, stop=(stop,)) for p in prompts]
    assert sum(1 for c in fake.calls if c[0] == "reset") == 6
    gen.clear()
    assert gen.cache_lengths() == [0, 0, 0]


def test_gumbel_tape_is_indexed_by_step_batch_and_row():
    fake = FakeSession()
    rng = np.random.default_rng(4)
    batch, steps, t = 2, 3, 0.7
    tape = rng.random((steps * batch, VOCAB), dtype=np.float32)
    prompts = [[3, 1], [2, 2, 2]]
    gen = serving.LlamaBatchGenerator(fake, batch_size=batch)
    seqs = gen.generate_ids(prompts, steps, serving.Sampling(t, tape))
    for r, p in enumerate(prompts):
        assert seqs[r].generated_ids == sampled_alone(p, steps, t, tape, r, batch)
    assert not any(c[0] == "prefill_rows" for c in fake.calls)  # sampled prompts are prefilled row by row


def test_checks_come_in_the_reference_order_before_any_work():
    fake = FakeSession()
    gen = serving.LlamaBatchGenerator(fake, batch_size=2)
    tape = np.full((2 * 2, VOCAB), 0.5, np.float32)

    def kind(*a, **k):
        with pytest.raises(serving.BatchGenerationError) as e:
            gen.generate_ids(*a, **k)
        return e.value

    e = kind([[1]], 2)
    assert (e.kind, e.value, e.value2) == ("BatchSize", 2, 1)
    e = kind([[1], []], 2)
    assert (e.kind, e.row) == ("EmptyPrompt", 1)
    e = kind([[1] * 60, [1]], 5)  # the row check wins over the bad token behind it
    assert (e.kind, e.row, e.value, e.value2) == ("ContextLength", 0, 65, 64)
    e = kind([[1], [2, VOCAB]], 2)
    assert (e.kind, e.row, e.value, e.value2) == ("TokenOutOfRange", 1, VOCAB, VOCAB)
    e = kind([[1], [2, VOCAB]], 2, serving.Sampling(0.0, tape))  # tokens are checked before the sampling
    assert e.kind == "TokenOutOfRange"
    assert kind([[1], [2]], 2, serving.Sampling(float("nan"), tape)).kind == "InvalidTemperature"
    e = kind([[1], [2]], 3, serving.Sampling(0.5, tape))
    assert (e.kind, e.value, e.value2) == ("UniformTapeLength", 3 * 2 * VOCAB, 2 * 2 * VOCAB)
    bad = tape.copy()
    bad[1, 7] = 1.0
    e = kind([[1], [2]], 2, serving.Sampling(0.5, bad))
    assert (e.kind, e.value) == ("InvalidUniform", VOCAB + 7)
    assert fake.calls == [] and gen.cache_lengths() == [0, 0]
    # no new tokens: empty rows without touching the cache
    seqs = gen.generate_ids([[1], [2]], 0)
    assert [q.generated_ids for q in seqs] == [[], []] and fake.calls == []


def test_a_failed_generation_keeps_the_committed_lengths():
    fake = FakeSession()
    gen = serving.LlamaBatchGenerator(fake, batch_size=2)
    gen.generate_ids([[1, 2], [3]], 3)
    assert gen.cache_lengths() == [4, 3]
    fake.fail["decode"] = 7
    with pytest.raises(serving.BatchGenerationError) as e:
        gen.generate_ids([[5], [6, 7, 8]], 4)
    assert (e.value.kind, e.value.value) == ("Session", 7)
    assert gen.cache_lengths() == [4, 3]
    seqs = gen.generate_ids([[5], [6, 7, 8]], 4)  # and the generator works on
    assert [q.generated_ids for q in seqs] == [alone([5], 4), alone([6, 7, 8], 4)]
    assert gen.cache_lengths() == [1 + 3, 3 + 3]
