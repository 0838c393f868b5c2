"""The compiled serving scheduler (include/rg_b200_serving.h) driven without a device, through a
table of Python callables in place of the session verbs: admission, arrival order, cache rows,
stop ids, sampling tapes, the prefix cache (PrefixCache of
src/models/transformer/serving/mod.rs:192-352) and what a failed step leaves behind."""
import numpy as np
import pytest

from rustgrad_b200 import serving

VOCAB = 50


def next_token(history):
    """The fake model: a pure function of everything its row holds."""
    return (sum(history) * 7 + len(history) * 3 + 1) % VOCAB


def fake_logits(history):
    out = np.zeros(VOCAB, dtype=np.float32)
    out[next_token(history)] = 1.0
    return out


def pick(logits, temperature, uniforms):
    """Greedy, or Gumbel-max over the tape (serving/mod.rs:649-665)."""
    if uniforms is None or temperature <= 0:
        return int(np.argmax(logits))
    u = np.maximum(uniforms.astype(np.float64), 1e-30)
    return int(np.argmax(logits.astype(np.float64) / temperature - np.log(-np.log(u))))


class FakeSession(serving.ServingBackend):
    vocab, max_context = VOCAB, 64

    def __init__(self, snapshot_bytes=1000):
        self.rows, self.snapshots, self.next_handle = {}, {}, 1
        self.snapshot_bytes = snapshot_bytes
        self.calls = []
        self.fail = {}            # verb -> status to return once

    def _failing(self, verb):
        return self.fail.pop(verb, 0)

    def reset_row(self, row):
        self.calls.append(("reset", row))
        self.rows[row] = []
        return 0

    def prefill_select(self, row, ids, temperature, uniforms, last_logits):
        self.calls.append(("prefill", row, len(ids)))
        rc = self._failing("prefill")
        if rc:
            return rc, -1
        self.rows.setdefault(row, []).extend(ids)
        last_logits[:] = fake_logits(self.rows[row])
        return 0, pick(last_logits, temperature, uniforms)

    def decode_rows(self, rows, tokens, temperatures, uniforms):
        self.calls.append(("decode", tuple(rows)))
        rc = self._failing("decode")
        if rc:
            return rc, []
        out = []
        for i, (row, tok) in enumerate(zip(rows, tokens)):
            self.rows[row].append(tok)
            out.append(pick(fake_logits(self.rows[row]), temperatures[i], None if uniforms is None else uniforms[i]))
        return 0, out

    def select(self, logits, temperature, uniforms):
        self.calls.append(("select",))
        return 0, pick(logits, temperature, uniforms)

    def snapshot_create(self, row, length):
        h = self.next_handle
        self.next_handle += 1
        self.snapshots[h] = list(self.rows[row][:length])
        return 0, h, self.snapshot_bytes

    def snapshot_restore(self, handle, row):
        self.calls.append(("restore", row, len(self.snapshots[handle])))
        self.rows[row] = list(self.snapshots[handle])
        return 0

    def snapshot_free(self, handle):
        del self.snapshots[handle]


def alone(prompt, n, stop=()):
    history, out = list(prompt), []
    for _ in range(n):
        out.append(next_token(history))
        history.append(out[-1])
        if out[-1] in stop:
            break
    return out


def run_all(sched, limit=200):
    steps = []
    while sched.pending() and len(steps) < limit:
        steps.append(sched.step())
    assert sched.pending() == 0
    return steps


def entry_bytes(tokens, nbytes=1000):
    return nbytes + VOCAB * 4 + len(tokens) * 4


def test_arrival_order_batch_size_and_row_reuse():
    fake = FakeSession()
    sched = serving.LlamaServingScheduler(fake, batch_size=2, max_rows=3)
    prompts = [[1, 2, 3], [4, 5], [6], [7, 8, 9, 10]]
    lengths = [3, 5, 2, 4]
    ids = [sched.submit_ids(p, serving.GenerationConfig(n)) for p, n in zip(prompts, lengths)]
    assert [sched.status(i) for i in ids] == ["queued"] * 4
    first = sched.step()
    assert [(e.request_id, e.arrival_order, e.generation_step) for e in first] == [(ids[0], 0, 0), (ids[1], 1, 0)]
    assert [sched.status(i) for i in ids] == ["running", "running", "queued", "queued"]
    assert [c for c in fake.calls if c[0] == "prefill"] == [("prefill", 0, 3), ("prefill", 1, 2)]
    second = sched.step()
    assert ("decode", (0, 1)) in fake.calls and [e.generation_step for e in second] == [1, 1]
    run_all(sched)
    for i, p, n in zip(ids, prompts, lengths):
        r = sched.result(i)
        assert (r.generated_ids, r.prompt_ids, r.stopped, r.decoded) == (alone(p, n), p, False, "")
    assert [r.request_id for r in sched.completed_results()] == ids
    # the third request got the row the first one handed back; no request ever saw row 2
    assert {c[1] for c in fake.calls if c[0] == "prefill"} == {0, 1}
    assert sched.step() == []


def test_one_decode_launch_sequence_per_step_and_late_arrivals_wait():
    fake = FakeSession()
    sched = serving.LlamaServingScheduler(fake, batch_size=3)
    a = sched.submit_ids([1], serving.GenerationConfig(4))
    sched.step()
    b = sched.submit_ids([2], serving.GenerationConfig(4))
    fake.calls.clear()
    events = sched.step()      # one running row decodes, one new prompt is prefilled
    assert [e.request_id for e in events] == [a, b]
    assert [c[0] for c in fake.calls] == ["prefill", "decode"] and fake.calls[1] == ("decode", (0,))
    fake.calls.clear()
    sched.step()
    assert fake.calls == [("decode", (0, 1))]


def test_stop_ids_end_a_request_and_the_stop_token_is_reported():
    p = [3, 1, 4]
    want = alone(p, 8)
    stop = want[3]
    fake = FakeSession()
    sched = serving.LlamaServingScheduler(fake, batch_size=1, stop_ids=[stop, 49])
    rid = sched.submit_ids(p, serving.GenerationConfig(8))
    events = [e for step in run_all(sched) for e in step]
    r = sched.result(rid)
    assert r.generated_ids == want[: want.index(stop) + 1] and r.stopped
    assert (events[-1].stopped, events[-1].complete, events[-1].token_id) == (True, True, stop)
    assert not any(e.complete for e in events[:-1])


def test_admission_checks_come_before_an_id_is_given():
    fake = FakeSession()
    sched = serving.LlamaServingScheduler(fake, batch_size=1)
    cases = [([], 1, None, "EmptyPrompt", None), ([VOCAB], 1, None, "TokenOutOfRange", (VOCAB, VOCAB)),
             ([-1], 1, None, "TokenOutOfRange", (-1, VOCAB)), ([1] * 60, 5, None, "ContextLength", (65, 64)),
             ([1], 2, serving.Sampling(0.0, np.zeros((2, VOCAB), np.float32)), "InvalidTemperature", None),
             ([1], 2, serving.Sampling(float("nan"), np.zeros((2, VOCAB), np.float32)), "InvalidTemperature", None),
             ([1], 2, serving.Sampling(1.0, np.zeros(3, np.float32)), "UniformTapeLength", (2 * VOCAB, 3)),
             ([1], 2, serving.Sampling(1.0, None), "UniformTapeLength", (2 * VOCAB, 0)),
             ([1], 1, serving.Sampling(1.0, np.ones(VOCAB, np.float32)), "InvalidUniform", (0, 0))]
    for prompt, n, sampling, kind, numbers in cases:
        with pytest.raises(serving.ServingError) as e:
            sched.submit_ids(prompt, serving.GenerationConfig(n, sampling or serving.Sampling()))
        assert e.value.kind == kind
        if numbers:
            assert (e.value.value, e.value.value2) == numbers
    bad = np.zeros((1, VOCAB), np.float32)
    bad[0, 17] = -0.5
    with pytest.raises(serving.ServingError) as e:
        sched.submit_ids([1], serving.GenerationConfig(1, serving.Sampling(1.0, bad)))
    assert (e.value.kind, e.value.value) == ("InvalidUniform", 17)
    assert sched.submit_ids([1], serving.GenerationConfig(1)) == 0      # no id was spent on the rejected ones
    z = sched.submit_ids([1], serving.GenerationConfig(0))
    assert sched.status(z) == "complete" and sched.result(z).generated_ids == []
    for kw in (dict(batch_size=0), dict(batch_size=3, max_rows=2)):
        with pytest.raises(serving.ServingError) as e:
            serving.LlamaServingScheduler(fake, **kw)
        assert e.value.kind == "EmptyBatch"
    with pytest.raises(serving.ServingError):       # text needs a tokenizer
        sched.submit_text("hello", serving.GenerationConfig(1))


def test_gumbel_tape_rows_follow_the_generation_step():
    rng = np.random.default_rng(3)
    tape = rng.random((4, VOCAB), dtype=np.float32)
    history, want = [5, 6], []
    for step in range(4):
        want.append(pick(fake_logits(history), 0.8, tape[step]))
        history.append(want[-1])
    assert want != alone([5, 6], 4)
    fake = FakeSession()
    sched = serving.LlamaServingScheduler(fake, batch_size=2)
    g = sched.submit_ids([9], serving.GenerationConfig(4))
    s = sched.submit_ids([5, 6], serving.GenerationConfig(4, serving.Sampling(0.8, tape)))
    run_all(sched)
    assert sched.result(s).generated_ids == want and sched.result(g).generated_ids == alone([9], 4)


def test_remove_frees_the_row_and_unknown_ids_are_reported():
    fake = FakeSession()
    sched = serving.LlamaServingScheduler(fake, batch_size=1)
    a = sched.submit_ids([1, 2], serving.GenerationConfig(5))
    b = sched.submit_ids([3], serving.GenerationConfig(2))
    sched.step()
    assert sched.result(a) is None                  # not complete yet
    assert sched.remove(a) and not sched.remove(a) and sched.status(a) is None
    assert ("reset", 0) in fake.calls
    run_all(sched)
    assert sched.result(b).generated_ids == alone([3], 2) and sched.pending() == 0


def test_prefix_cache_longest_match_extension_and_full_hit():
    fake = FakeSession()
    sched = serving.LlamaServingScheduler(fake, batch_size=1, prefix_max_entries=8, prefix_max_bytes=1 << 20)
    base, longer = [1, 2, 3, 4], [1, 2, 3, 4, 5, 6]
    a = sched.submit_ids(base, serving.GenerationConfig(3))
    run_all(sched)
    st = sched.prefix_stats()
    assert (st["entries"], st["hits"], st["misses"], st["bytes"]) == (1, 0, 1, entry_bytes(base))
    fake.calls.clear()
    b = sched.submit_ids(base, serving.GenerationConfig(1))      # the whole prompt is cached: selection only
    run_all(sched)
    assert [c[0] for c in fake.calls if c[0] != "reset"] == ["restore", "select"]
    fake.calls.clear()
    c = sched.submit_ids(longer, serving.GenerationConfig(3))    # four cached positions, two prefilled
    run_all(sched)
    assert ("restore", 0, 4) in fake.calls and ("prefill", 0, 2) in fake.calls
    d = sched.submit_ids([1, 2, 9], serving.GenerationConfig(2))  # shares two tokens with an entry but no whole entry
    run_all(sched)
    assert sched.result(a).generated_ids == alone(base, 3) and sched.result(b).generated_ids == alone(base, 1)
    assert sched.result(c).generated_ids == alone(longer, 3) and sched.result(d).generated_ids == alone([1, 2, 9], 2)
    st = sched.prefix_stats()
    assert (st["entries"], st["hits"], st["misses"]) == (3, 2, 2)
    assert st["bytes"] == entry_bytes(base) + entry_bytes(longer) + entry_bytes([1, 2, 9])


def test_prefix_cache_evicts_least_recently_used_under_both_budgets():
    fake = FakeSession()
    sched = serving.LlamaServingScheduler(fake, batch_size=1, prefix_max_entries=2, prefix_max_bytes=1 << 20)
    for p in ([1], [2]):
        sched.submit_ids(p, serving.GenerationConfig(1))
    run_all(sched)
    sched.submit_ids([1, 5], serving.GenerationConfig(1))        # touches [1]; its own entry evicts [2], the oldest
    run_all(sched)
    st = sched.prefix_stats()
    assert (st["entries"], st["evictions"]) == (2, 1)
    assert sorted(len(v) for v in fake.snapshots.values()) == [1, 2] and [1] in fake.snapshots.values()
    sched.submit_ids([2], serving.GenerationConfig(1))           # [2] is gone: a miss
    run_all(sched)
    assert sched.prefix_stats()["misses"] == 3
    # re-inserting a key replaces it without an eviction
    before = sched.prefix_stats()
    sched.invalidate_prefix_cache()
    assert fake.snapshots == {}                                   # device copies are released with their entries
    st = sched.prefix_stats()
    assert (st["entries"], st["bytes"], st["generation"]) == (0, 0, before["generation"] + 1)
    # byte budget: room for one entry only, and an entry larger than the whole budget is not kept
    small = serving.LlamaServingScheduler(FakeSession(), batch_size=1, prefix_max_entries=8, prefix_max_bytes=1500)
    for p in ([1], [2]):
        small.submit_ids(p, serving.GenerationConfig(1))
    run_all(small)
    st = small.prefix_stats()
    assert (st["entries"], st["evictions"], st["bytes"]) == (1, 1, entry_bytes([2]))
    none = serving.LlamaServingScheduler(FakeSession(snapshot_bytes=4000), batch_size=1, prefix_max_entries=8, prefix_max_bytes=1500)
    none.submit_ids([1], serving.GenerationConfig(1))
    run_all(none)
    assert none.prefix_stats()["entries"] == 0
    off = serving.LlamaServingScheduler(FakeSession(), batch_size=1, prefix_max_entries=0, prefix_max_bytes=1 << 20)
    off.submit_ids([1], serving.GenerationConfig(1))
    run_all(off)
    assert off.prefix_stats()["entries"] == 0 and off.session.snapshots == {}


def test_a_failed_step_can_be_run_again_as_a_whole():
    fake = FakeSession()
    sched = serving.LlamaServingScheduler(fake, batch_size=2)
    a = sched.submit_ids([1, 2], serving.GenerationConfig(4))
    sched.step()
    b = sched.submit_ids([3, 4, 5], serving.GenerationConfig(3))
    fake.fail["decode"] = 9                                       # the decode launch of this step fails
    with pytest.raises(serving.ServingError) as e:
        sched.step()
    assert (e.value.kind, e.value.value) == ("Session", 9)
    assert sched.status(a) == "running" and sched.status(b) == "queued"   # b was un-admitted, its row reset
    assert fake.rows[1] == []
    fake.fail["prefill"] = 12
    with pytest.raises(serving.ServingError) as e:
        sched.step()
    assert e.value.value == 12 and sched.status(b) == "queued"
    run_all(sched)
    assert sched.result(a).generated_ids == alone([1, 2], 4) and sched.result(b).generated_ids == alone([3, 4, 5], 3)


class BatchingSession(FakeSession):
    """A back end that also offers the several-prompts-in-one-pass verb."""

    def prefill_rows(self, rows, prompts, last_logits):
        self.calls.append(("prefill_rows", tuple(rows), tuple(len(p) for p in prompts)))
        rc = self._failing("prefill_rows")
        if rc:
            return rc, []
        out = []
        for i, (row, ids) in enumerate(zip(rows, prompts)):
            self.rows.setdefault(row, []).extend(ids)
            last_logits[i, :] = fake_logits(self.rows[row])
            out.append(int(np.argmax(last_logits[i])))
        return 0, out


def test_greedy_prompts_admitted_together_are_prefilled_in_one_pass():
    fake = BatchingSession()
    sched = serving.LlamaServingScheduler(fake, batch_size=4, prefix_max_entries=8, prefix_max_bytes=1 << 20)
    rng = np.random.default_rng(1)
    tape = rng.random((3, VOCAB), dtype=np.float32)
    prompts = [[1, 2, 3], [4, 5], [6, 7, 8, 9]]
    ids = [sched.submit_ids(p, serving.GenerationConfig(3)) for p in prompts]
    sampled = sched.submit_ids([9, 9], serving.GenerationConfig(3, serving.Sampling(0.9, tape)))
    sched.step()
    assert ("prefill_rows", (0, 1, 2), (3, 2, 4)) in fake.calls          # the three greedy prompts in one call
    assert [c for c in fake.calls if c[0] == "prefill"] == [("prefill", 3, 2)]   # the sampled one alone
    run_all(sched)
    for rid, p in zip(ids, prompts):
        assert sched.result(rid).generated_ids == alone(p, 3)
    assert sched.prefix_stats()["entries"] == 4
    # a prompt that extends one waiting in the same step still finds it in the prefix cache
    fake.calls.clear()
    a = sched.submit_ids([20, 21], serving.GenerationConfig(2))
    b = sched.submit_ids([20, 21, 22], serving.GenerationConfig(2))
    c = sched.submit_ids([30], serving.GenerationConfig(2))
    sched.step()
    assert ("restore", 1, 2) in fake.calls and sched.prefix_stats()["hits"] == 1
    run_all(sched)
    assert [sched.result(r).generated_ids for r in (a, b, c)] == [alone([20, 21], 2), alone([20, 21, 22], 2), alone([30], 2)]
    # a failing pass un-admits all of its prompts
    d = sched.submit_ids([40, 41], serving.GenerationConfig(1))
    e = sched.submit_ids([42], serving.GenerationConfig(1))
    fake.fail["prefill_rows"] = 9
    with pytest.raises(serving.ServingError):
        sched.step()
    assert [sched.status(r) for r in (d, e)] == ["queued", "queued"]
    run_all(sched)
    assert sched.result(d).generated_ids == alone([40, 41], 1) and sched.result(e).generated_ids == alone([42], 1)


def test_rebind_needs_an_idle_scheduler_and_drops_prefixes_only_for_another_session():
    """LlamaServingScheduler::rebind (serving/mod.rs:528-547): refused while a request is unfinished; the same
    session keeps the cached prefixes; another session drops them (freed through the session that made them)
    and serves the next requests; finished results stay readable; new stop ids apply from then on."""
    a, b = FakeSession(), FakeSession()
    sched = serving.LlamaServingScheduler(a, batch_size=2, prefix_max_entries=8, prefix_max_bytes=1 << 20)
    first = sched.submit_ids([1, 2, 3, 4], serving.GenerationConfig(3))
    sched.step()
    with pytest.raises(serving.ServingError) as e:
        sched.rebind(b)
    assert e.value.kind == "ActiveRequests" and e.value.value == 1
    run_all(sched)
    assert sched.prefix_stats()["entries"] == 1 and len(a.snapshots) == 1
    # the same session: nothing is dropped, and the cached prefix still serves a hit
    assert sched.rebind(a) is False
    assert sched.prefix_stats()["entries"] == 1 and len(a.snapshots) == 1
    again = sched.submit_ids([1, 2, 3, 4, 5], serving.GenerationConfig(2))
    run_all(sched)
    assert sched.prefix_stats()["hits"] == 1
    assert sched.result(again).generated_ids == alone([1, 2, 3, 4, 5], 2)
    # another session: every prefix goes, its snapshots are freed by the session that made them
    held = len(a.snapshots)
    assert held >= 1
    assert sched.rebind(b, stop_ids=[next_token([9, 8, 7])]) is True
    assert sched.prefix_stats()["entries"] == 0 and len(a.snapshots) == 0
    assert sched.result(first).generated_ids == alone([1, 2, 3, 4], 3)  # finished results are kept
    before = len(a.calls)
    late = sched.submit_ids([9, 8, 7], serving.GenerationConfig(4))
    run_all(sched)
    assert len(a.calls) == before and any(c[0] == "prefill" for c in b.calls)  # only the new session works
    r = sched.result(late)
    assert r.generated_ids == alone([9, 8, 7], 4, stop=(next_token([9, 8, 7]),)) and r.stopped
    assert sched.prefix_stats()["misses"] >= 1
