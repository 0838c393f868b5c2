"""Continuous batching over one GPU session (the scheduler of include/rg_b200_serving.h, after
src/models/transformer/serving/mod.rs): every request must produce exactly the tokens it produces
alone, whatever it shares a step with and whether or not its prompt came from the prefix cache."""
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


def run_all(sched):
    events = []
    for _ in range(200):
        if sched.pending() == 0:
            break
        events.append(sched.step())
    assert sched.pending() == 0
    return events


def test_staggered_requests_match_isolated_generation(model):
    cfg, data = model
    prompts = [synth.prompt_ids(cfg, 5 + 2 * r, seed=30 + r) for r in range(5)]
    want = [alone(data, p, 6) for p in prompts]
    s = make_session(data, max_batch=4, kv_f32=True)
    sched = serving.LlamaServingScheduler(s, batch_size=3, max_rows=4)
    ids = [sched.submit_ids(p, serving.GenerationConfig(6)) for p in prompts[:3]]
    assert [sched.status(i) for i in ids] == ["queued"] * 3
    first = sched.step()
    assert [e.request_id for e in first] == ids and [e.generation_step for e in first] == [0, 0, 0]
    assert [e.arrival_order for e in first] == [0, 1, 2]
    assert [sched.status(i) for i in ids] == ["running"] * 3
    second = sched.step()
    assert [e.generation_step for e in second] == [1, 1, 1]
    ids += [sched.submit_ids(p, serving.GenerationConfig(6)) for p in prompts[3:]]
    third = sched.step()  # the batch is full: the two late arrivals wait
    assert [e.request_id for e in third] == ids[:3]
    assert [sched.status(i) for i in ids[3:]] == ["queued"] * 2
    run_all(sched)
    for i, w, p in zip(ids, want, prompts):
        r = sched.result(i)
        assert r.generated_ids == w and r.prompt_ids == list(p) and not r.stopped
        assert sched.status(i) == "complete"
    assert [r.request_id for r in sched.completed_results()] == ids
    assert all(s.position(row) == 0 for row in range(4))  # every slot was handed back


def test_mixed_greedy_and_gumbel_rows_in_one_step(model):
    cfg, data = model
    vocab = cfg["vocab"]
    rng = np.random.default_rng(5)
    prompts = [synth.prompt_ids(cfg, 7, seed=50 + r) for r in range(3)]
    tapes = [None, rng.random((5, vocab), dtype=np.float32), rng.random((5, vocab), dtype=np.float32)]
    temps = [None, 0.7, 1.3]
    want = [alone(data, p, 5, temperature=t, uniforms=u) for p, t, u in zip(prompts, temps, tapes)]
    assert want[1] != alone(data, prompts[1], 5)  # the tape really changes the choice
    s = make_session(data, max_batch=3, kv_f32=True)
    sched = serving.LlamaServingScheduler(s, batch_size=3)
    ids = [sched.submit_ids(p, serving.GenerationConfig(5, serving.Sampling(t, u))) for p, t, u in zip(prompts, temps, tapes)]
    run_all(sched)
    assert [sched.result(i).generated_ids for i in ids] == want


def test_prefix_cache_hits_extend_and_evict(model):
    cfg, data = model
    base = synth.prompt_ids(cfg, 12, seed=70)
    longer = list(base) + list(synth.prompt_ids(cfg, 5, seed=71))
    other = synth.prompt_ids(cfg, 9, seed=72)
    want_base, want_longer, want_other = alone(data, base, 4), alone(data, longer, 4), alone(data, other, 4)
    s = make_session(data, max_batch=2, kv_f32=True)
    sched = serving.LlamaServingScheduler(s, batch_size=2, prefix_max_entries=2, prefix_max_bytes=1 << 24)
    a = sched.submit_ids(base, serving.GenerationConfig(4))
    run_all(sched)
    st = sched.prefix_stats()
    assert (st["entries"], st["hits"], st["misses"]) == (1, 0, 1) and st["bytes"] > 0
    launches = s.report()["kernel_launches"]
    b = sched.submit_ids(base, serving.GenerationConfig(1))  # the whole prompt is cached: selection only
    run_all(sched)
    assert s.report()["kernel_launches"] - launches <= 2
    assert sched.result(b).generated_ids == want_base[:1]
    c = sched.submit_ids(longer, serving.GenerationConfig(4))  # 12 cached positions + 5 new
    d = sched.submit_ids(base, serving.GenerationConfig(4))
    run_all(sched)
    assert sched.result(a).generated_ids == want_base and sched.result(d).generated_ids == want_base
    assert sched.result(c).generated_ids == want_longer
    st = sched.prefix_stats()
    assert st["hits"] == 3 and st["entries"] == 2 and st["evictions"] == 0
    e = sched.submit_ids(other, serving.GenerationConfig(4))  # a third entry evicts the least recently used
    run_all(sched)
    assert sched.result(e).generated_ids == want_other
    st = sched.prefix_stats()
    assert st["entries"] == 2 and st["evictions"] == 1
    sched.invalidate_prefix_cache()
    st = sched.prefix_stats()
    assert st["entries"] == 0 and st["bytes"] == 0 and st["generation"] == 1
    f = sched.submit_ids(base, serving.GenerationConfig(4))
    run_all(sched)
    assert sched.result(f).generated_ids == want_base and sched.prefix_stats()["misses"] == st["misses"] + 1


def test_stop_tokens_removal_and_admission_errors(model):
    cfg, data = model
    p = synth.prompt_ids(cfg, 6, seed=90)
    want = alone(data, p, 6)
    s = make_session(data, max_batch=2, kv_f32=True)
    sched = serving.LlamaServingScheduler(s, batch_size=2, stop_ids=[want[2]])
    a = sched.submit_ids(p, serving.GenerationConfig(6))
    b = sched.submit_ids(p, serving.GenerationConfig(6))
    events = sched.step()
    assert sched.remove(b) and not sched.remove(b) and sched.status(b) is None
    events = [e for e in events if e.request_id == a] + [e for step in run_all(sched) for e in step]
    r = sched.result(a)
    assert r.generated_ids == want[: want.index(want[2]) + 1] and r.stopped
    assert events[-1].stopped and events[-1].complete
    z = sched.submit_ids(p, serving.GenerationConfig(0))
    assert sched.status(z) == "complete" and sched.result(z).generated_ids == []
    for bad, kind in [([], "EmptyPrompt"), ([cfg["vocab"]], "TokenOutOfRange"), ([1] * cfg["max_context"], "ContextLength")]:
        with pytest.raises(serving.ServingError) as e:
            sched.submit_ids(bad, serving.GenerationConfig(1))
        assert e.value.kind == kind
    with pytest.raises(serving.ServingError) as e:
        sched.submit_ids(p, serving.GenerationConfig(2, serving.Sampling(0.0, np.zeros((2, cfg["vocab"]), np.float32))))
    assert e.value.kind == "InvalidTemperature"
    with pytest.raises(serving.ServingError) as e:
        sched.submit_ids(p, serving.GenerationConfig(2, serving.Sampling(1.0, np.zeros(3, np.float32))))
    assert e.value.kind == "UniformTapeLength" and (e.value.value, e.value.value2) == (2 * cfg["vocab"], 3)
    with pytest.raises(serving.ServingError) as e:
        sched.submit_ids(p, serving.GenerationConfig(1, serving.Sampling(1.0, np.ones(cfg["vocab"], np.float32))))
    assert e.value.kind == "InvalidUniform" and e.value.value == 0
    with pytest.raises(serving.ServingError):
        serving.LlamaServingScheduler(s, batch_size=0)


def test_snapshot_restore_round_trip_and_shape_checks(model):
    cfg, data = model
    p = synth.prompt_ids(cfg, 10, seed=95)
    s = make_session(data, max_batch=2, kv_f32=False)
    logits = s.prefill_ids(p, row=0)
    snap = session.KvSnapshot(s, 0, 10)
    assert snap.bytes == 2 * cfg["n_layers"] * cfg["n_kv_heads"] * 10 * cfg["head_dim"] * 2
    snap.restore(s, 1)
    assert s.position(1) == 10
    tok = int(np.argmax(logits))
    out, _ = s.decode([tok, tok], want_logits=True)  # both rows now continue the same sequence
    np.testing.assert_array_equal(out[0], out[1])
    other = make_session(data, max_batch=1, kv_f32=True)
    with pytest.raises(session.RgError):
        snap.restore(other, 0)
    with pytest.raises(session.RgError):
        session.KvSnapshot(s, 0, 50)


def test_decode_rows_rejections_leave_positions_unchanged(model):
    import ctypes as C
    from rustgrad_b200 import _lib
    cfg, data = model
    s = make_session(data, max_batch=3, kv_f32=True)
    L = _lib.load()
    for r in range(3):
        s.prefill_ids(synth.prompt_ids(cfg, 4 + r, seed=r), row=r, want_logits=False)
    before = [s.position(r) for r in range(3)]

    def call(rows, toks):
        rows, toks = np.array(rows, np.int32), np.array(toks, np.int32)
        ids = np.empty(len(rows), np.int32)
        i32 = C.POINTER(C.c_int32)
        return L.rg_b200_decode_rows(s._h, rows.ctypes.data_as(i32), toks.ctypes.data_as(i32), len(rows), None, None, None,
                                     ids.ctypes.data_as(i32)), ids

    assert call([0, 0], [1, 1])[0] == 1          # the same row twice: RG_INVALID_ARGUMENT
    assert call([0, 3], [1, 1])[0] == 1          # row out of range
    assert call([0, 1], [1, cfg["vocab"]])[0] == 5  # RG_TOKEN_OUT_OF_RANGE
    assert [s.position(r) for r in range(3)] == before
    rc, ids = call([2, 0], [1, 2])               # any order, any subset
    assert rc == 0 and [s.position(r) for r in range(3)] == [before[0] + 1, before[1], before[2] + 1]
    solo = make_session(data, max_batch=1, kv_f32=True)
    solo.prefill_ids(synth.prompt_ids(cfg, 6, seed=2), want_logits=False)
    _, want = solo.decode([1])
    assert int(ids[0]) == int(want[0])           # column 0 fed row 2, whose prompt had seed 2


def test_text_and_chat_requests_share_steps_and_decode_their_results():
    """submit_text / submit_chat (serving/mod.rs:408-477): the scheduler encodes with the model's own
    tokenizer (BOS in front of plain text, the checked template for chat) and decodes each result."""
    from oracle import tokenizer_oracle as T
    from rustgrad_b200 import gguf_writer, tokenizer
    cfg = dict(synth.TINY)
    tensors = synth.build_tensors(cfg, seed=0, body_type=quant.Q8_0)
    data = synth.gguf_bytes(cfg, tensors, chat_tokens=True)
    tokens, types, ids = gguf_writer.chat_token_table(cfg["vocab"])
    normal = [(t, i) for i, (t, ty) in enumerate(zip(tokens, types)) if ty == 1]
    special = [(t, i) for i, (t, ty) in enumerate(zip(tokens, types)) if ty != 1]
    check_tok = T.SimpleTokenizer(normal, special, eos_id=ids["eos"], eot_id=ids["eot"], bos_id=ids["bos"])
    g = session.GgufFile(data)
    tok = tokenizer.SimpleTokenizer.from_gguf(g)
    g.close()
    s = make_session(data, max_batch=2, kv_f32=True)
    stops = [ids["eos"], ids["eot"]]
    sched = serving.LlamaServingScheduler(s, tokenizer=tok, batch_size=2, stop_ids=stops, bos_id=ids["bos"])
    a = sched.submit_text("hello world", serving.GenerationConfig(6))
    messages = [("system", "be brief"), ("user", "hello")]
    b = sched.submit_chat(messages, serving.GenerationConfig(6))
    run_all(sched)
    want_a = [ids["bos"]] + check_tok.encode("hello world")
    want_b = check_tok.encode(tokenizer.LlamaChatTemplate().render(tok, messages, True))
    for rid, prompt in ((a, want_a), (b, want_b)):
        r = sched.result(rid)
        assert r.prompt_ids == prompt
        gen = alone(data, prompt, 6)
        cut = next((i + 1 for i, t in enumerate(gen) if t in stops), len(gen))
        assert r.generated_ids == gen[:cut] and r.decoded == check_tok.decode(gen[:cut])


def test_rebind_moves_an_idle_scheduler_to_another_session(model):
    """rebind (serving/mod.rs:528-547) over device sessions: the prefixes cached from the first session are
    dropped (their device copies freed), and requests after the rebind run on the second session's weights."""
    cfg, data = model
    other = synth.gguf_bytes(cfg, synth.build_tensors(cfg, seed=3, body_type=quant.Q8_0))
    a, b = make_session(data, max_batch=2, kv_f32=True), make_session(other, max_batch=2, kv_f32=True)
    prompt = synth.prompt_ids(cfg, 9, seed=61)
    sched = serving.LlamaServingScheduler(a, batch_size=2, prefix_max_entries=4, prefix_max_bytes=1 << 28)
    first = sched.submit_ids(prompt, serving.GenerationConfig(5))
    sched.step()
    with pytest.raises(serving.ServingError) as e:
        sched.rebind(b)
    assert e.value.kind == "ActiveRequests"
    run_all(sched)
    assert sched.result(first).generated_ids == alone(data, prompt, 5)
    assert sched.prefix_stats()["entries"] == 1
    assert sched.rebind(a) is False and sched.prefix_stats()["entries"] == 1
    assert sched.rebind(b) is True and sched.prefix_stats()["entries"] == 0
    second = sched.submit_ids(prompt, serving.GenerationConfig(5))
    run_all(sched)
    assert sched.result(second).generated_ids == alone(other, prompt, 5)
    assert sched.result(first).generated_ids == alone(data, prompt, 5)  # finished results are kept
