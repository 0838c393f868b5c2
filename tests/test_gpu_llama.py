"""GPU parity of the Llama session against the CPU checker on seeded synthetic models.

Bar (floating point): every logit within 1e-2 absolute and 1e-3 relative of the reference CPU
path (|a-b| <= 1e-2 and |a-b| <= 1e-3 * max|logit|), identical greedy token sequences."""
import numpy as np
import pytest

from oracle import oracle as O
from rustgrad_b200 import quant, session, synth

pytestmark = pytest.mark.gpu

ATOL, RTOL = 1e-2, 1e-3


def assert_logits_close(got, want):
    diff = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert diff.max() <= ATOL, diff.max()
    assert diff.max() <= RTOL * np.abs(want).max() + 1e-6, (diff.max(), np.abs(want).max())


@pytest.fixture(scope="module")
def tiny():
    """The tiny end-to-end model: 2 layers, d 256, 4 heads, ffn 688, vocab 512, Q8_0, tied head, as a GGUF file."""
    cfg = dict(synth.TINY)
    tensors = synth.build_tensors(cfg, seed=0, body_type=quant.Q8_0)
    data = synth.gguf_bytes(cfg, tensors)
    prompt = synth.prompt_ids(cfg, 16, seed=1)
    return cfg, tensors, data, prompt


def make_session(data, **kw):
    target = session.CudaSessionTarget(**kw)
    plan = session.LlamaCudaPlan.from_gguf_bytes(data, target)
    return target.prepare(plan)


def test_config1_logits_and_greedy_tokens_match_reference_cpu_path(tiny):
    cfg, tensors, data, prompt = tiny
    oracle = O.OracleModel(cfg, tensors, threads=1)
    want_ids, _ = oracle.generate_greedy(prompt, 32, O.MODE_STRICT)
    s = make_session(data, kv_f32=True)
    gen = s.generate_ids(prompt, 32)
    assert gen.generated_ids == want_ids
    assert not gen.stopped and s.position() == 16 + 31
    # logits of the prefill and of every decode step
    oracle.reset()
    s.reset_sequence()
    assert_logits_close(s.prefill_ids(prompt), oracle.forward(prompt))
    for tok in want_ids[:8]:
        assert_logits_close(s.run_token(tok), oracle.forward([tok]))
    assert s.report()["fallback_count"] == 0 and s.report()["kernel_launches"] > 0


def test_f16_kv_cache_matches_checker_with_f16_cache(tiny):
    cfg, tensors, data, prompt = tiny
    oracle = O.OracleModel(cfg, tensors, kv_f16=True, threads=1)
    s = make_session(data)  # f16 cache is the default
    assert_logits_close(s.prefill_ids(prompt), oracle.forward(prompt))
    for tok in (5, 77, 300):
        assert_logits_close(s.run_token(tok), oracle.forward([tok]))


def test_prefill_equals_token_steps_and_graph_equals_direct_launch(tiny):
    cfg, tensors, data, prompt = tiny
    a = make_session(data, kv_f32=True)
    full = a.prefill_ids(prompt)
    b = make_session(data, kv_f32=True, disable_graph=True, disable_pdl=True)
    for tok in prompt[:-1]:
        b.run_token(int(tok))
    step = b.run_token(int(prompt[-1]))
    assert np.abs(full - step).max() <= 1e-4
    c = make_session(data, kv_f32=True)
    for tok in prompt[:-1]:
        c.run_token(int(tok))
    assert np.array_equal(c.run_token(int(prompt[-1])), step)  # graph + PDL replay is bit-identical


def test_batched_rows_decode_independently(tiny):
    cfg, tensors, data, _ = tiny
    rows = [synth.prompt_ids(cfg, 6, seed=10 + r) for r in range(3)]
    s = make_session(data, max_batch=3, kv_f32=True)
    oracles = [O.OracleModel(cfg, tensors, threads=1) for _ in rows]
    firsts = []
    for r, p in enumerate(rows):
        lg = s.prefill_ids(p, row=r)
        want = oracles[r].forward(p)
        assert_logits_close(lg, want)
        firsts.append(O.select_greedy(want))
    toks = firsts
    for _ in range(5):
        logits, greedy = s.decode(toks, want_logits=True)
        nxt = []
        for r in range(3):
            want = oracles[r].forward([toks[r]])
            assert_logits_close(logits[r], want)
            nxt.append(O.select_greedy(want))
        assert greedy.tolist() == nxt
        toks = nxt
    assert [s.position(r) for r in range(3)] == [11, 11, 11]


def test_device_resident_loop_equals_host_driven_generation(tiny):
    cfg, tensors, data, prompt = tiny
    s = make_session(data, kv_f32=True)
    gen = s.generate_ids(prompt, 20)
    t = make_session(data, kv_f32=True)
    logits = t.prefill_ids(prompt)
    first = int(np.argmax(logits))
    assert first == gen.generated_ids[0]
    ids, ms = t.decode_loop([first], 19)
    assert ids[:, 0].tolist() == gen.generated_ids[1:]
    assert ms > 0 and t.position() == 16 + 19


def test_q4_0_body_with_explicit_q8_0_head():
    cfg = synth.scaled(synth.TINY, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn_dim=1024, vocab=640, n_layers=3,
                       rope_theta=500000.0)
    tensors = synth.build_tensors(cfg, seed=6, body_type=quant.Q4_0, embed_type=quant.Q8_0, head_type=quant.Q8_0,
                                  tied_head=False)
    prompt = synth.prompt_ids(cfg, 13, seed=2)
    oracle = O.OracleModel(cfg, tensors, threads=4)
    want_ids, _ = oracle.generate_greedy(prompt, 16, O.MODE_STRICT)
    s = session.LlamaCudaPlan.from_tensors(cfg, tensors, session.CudaSessionTarget(kv_f32=True)).prepare()
    assert s.generate_ids(prompt, 16).generated_ids == want_ids
    oracle.reset()
    s.reset_sequence()
    assert_logits_close(s.prefill_ids(prompt), oracle.forward(prompt))
    # the fused small-batch decode path (integer GEMV) and the general path agree step by step
    g = session.LlamaCudaPlan.from_tensors(cfg, tensors, session.CudaSessionTarget(kv_f32=True, general_path_only=True)).prepare()
    g.prefill_ids(prompt)
    for tok in want_ids[:6]:
        a, b, w = s.run_token(tok), g.run_token(tok), oracle.forward([tok])
        assert_logits_close(a, w)
        assert_logits_close(b, w)
        assert np.abs(a - b).max() <= 1e-4


def test_tensor_core_path_for_long_prompts_and_wide_decode_batches():
    """Prompts of more than 8 tokens and decode batches of 9..32 rows run the projections on the
    tcgen05 GEMM (f16 operands); both must stay inside the logit bar and agree with the GEMV paths."""
    cfg = synth.scaled(synth.TINY, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn_dim=1024, vocab=640, n_layers=3,
                       rope_theta=500000.0, max_context=512)
    tensors = synth.build_tensors(cfg, seed=9, body_type=quant.Q4_0, embed_type=quant.Q8_0, head_type=quant.Q8_0,
                                  tied_head=False)
    prompt = synth.prompt_ids(cfg, 300, seed=3)  # two chunks: 256 + 44
    oracle = O.OracleModel(cfg, tensors, threads=8)
    want = oracle.forward(prompt, O.MODE_FAST)
    wide = session.LlamaCudaPlan.from_tensors(cfg, tensors, session.CudaSessionTarget(kv_f32=True, max_context=512)).prepare()
    narrow = session.LlamaCudaPlan.from_tensors(
        cfg, tensors, session.CudaSessionTarget(kv_f32=True, max_context=512, general_path_only=True)).prepare()
    a, b = wide.prefill_ids(prompt), narrow.prefill_ids(prompt)
    assert_logits_close(a, want)
    assert_logits_close(b, want)
    assert wide.report()["kernel_launches"] < narrow.report()["kernel_launches"] / 4  # 2 chunks instead of 38
    # both caches now continue identically under the small-batch decode path
    tok = O.select_greedy(want)
    for _ in range(3):
        w = oracle.forward([tok], O.MODE_FAST)
        assert_logits_close(wide.run_token(tok), w)
        tok = O.select_greedy(w)
    # 16 rows decoding together: the f16-MMA GEMV with four column tiles streams the weights once
    rows = 16
    before = session.launch_count("qgemv")
    s = session.LlamaCudaPlan.from_tensors(cfg, tensors, session.CudaSessionTarget(kv_f32=True, max_batch=rows,
                                                                                  max_context=64)).prepare()
    oracles = [O.OracleModel(cfg, tensors, threads=2) for _ in range(rows)]
    toks = []
    for r in range(rows):
        p = synth.prompt_ids(cfg, 3 + r % 5, seed=40 + r)
        s.prefill_ids(p, row=r)
        toks.append(O.select_greedy(oracles[r].forward(p, O.MODE_FAST)))
    near_ties = []
    for _ in range(3):
        logits, greedy = s.decode(toks, want_logits=True)
        nxt = []
        for r in range(rows):
            w = oracles[r].forward([toks[r]], O.MODE_FAST)
            assert_logits_close(logits[r], w)
            nxt.append(O.select_greedy(w))
            if int(greedy[r]) != nxt[r]:
                top2 = np.sort(w)[-2:]
                near_ties.append((r, float(top2[1] - top2[0])))
        toks = nxt
    # a differing greedy id is a finding, never silently accepted: none is expected on this model
    print(f"greedy ids differing from the checker on the 16-row decode path: {len(near_ties)} {near_ties}")
    assert not near_ties
    assert session.launch_count("qgemv") > before


def test_twenty_rows_decode_on_the_tensor_core_path(monkeypatch):
    """Decode batches of 17..32 rows: by default cut into equal chunks of at most 16 rows that run the GEMV path
    (20 rows = two steps of 10); with RG_B200_WIDE_DECODE_ONE_STEP=1 (and, with the GEMV route switched off,
    for 9..16 rows) the projections run on the tcgen05 GEMM with compensated f16 operands.  Logit bar and
    greedy ids against the checker for all three."""
    cfg = synth.scaled(synth.TINY, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn_dim=1024, vocab=640, n_layers=3,
                       rope_theta=500000.0, max_context=64)
    tensors = synth.build_tensors(cfg, seed=9, body_type=quant.Q4_0, embed_type=quant.Q8_0, head_type=quant.Q8_0,
                                  tied_head=False)
    for rows, env, kernel in ((20, None, "qgemv"), (20, "RG_B200_WIDE_DECODE_ONE_STEP", "qgemm_tc"), (12, "RG_B200_NO_GEMV16", "qgemm_tc")):
        if env:
            monkeypatch.setenv(env, "1")
        s = session.LlamaCudaPlan.from_tensors(cfg, tensors, session.CudaSessionTarget(kv_f32=True, max_batch=rows,
                                                                                      max_context=64)).prepare()
        oracles = [O.OracleModel(cfg, tensors, threads=2) for _ in range(rows)]
        toks = []
        for r in range(rows):
            p = synth.prompt_ids(cfg, 3 + r % 5, seed=70 + r)
            s.prefill_ids(p, row=r)
            toks.append(O.select_greedy(oracles[r].forward(p, O.MODE_FAST)))
        before = {k: session.launch_count(k) for k in ("qgemv", "qgemm_tc")}
        differing = 0
        for _ in range(2):
            logits, greedy = s.decode(toks, want_logits=True)
            nxt = []
            for r in range(rows):
                w = oracles[r].forward([toks[r]], O.MODE_FAST)
                assert_logits_close(logits[r], w)
                nxt.append(O.select_greedy(w))
                differing += int(greedy[r]) != nxt[r]
            toks = nxt
        print(f"{rows} rows ({env or 'chunked'}): greedy ids differing from the checker: {differing}")
        assert differing == 0
        assert session.launch_count(kernel) > before[kernel]
        if kernel == "qgemv":
            assert session.launch_count("qgemm_tc") == before["qgemm_tc"]
        if env:
            monkeypatch.delenv(env)


def test_stop_on_eos_and_last_token_not_fed_back(tiny):
    cfg, tensors, data, prompt = tiny
    s = make_session(data, kv_f32=True)
    ids = s.generate_ids(prompt, 10).generated_ids
    cfg2 = dict(cfg, eos_id=ids[3])
    plan = session.LlamaCudaPlan.from_tensors(cfg2, tensors, session.CudaSessionTarget(kv_f32=True))
    s2 = plan.prepare()
    gen = s2.generate_ids(prompt, 10)
    first = ids.index(ids[3])
    assert gen.stopped and gen.generated_ids == ids[: first + 1]
    assert s2.position() == 16 + first  # the stop token is never fed back


def test_typed_failures_leave_the_session_unchanged(tiny):
    cfg, tensors, data, prompt = tiny
    s = make_session(data, kv_f32=True)
    E = session
    with pytest.raises(E.EmptyPrompt):
        s.generate_ids([], 4)
    with pytest.raises(E.TokenOutOfRange):
        s.generate_ids([1, 512], 4)
    with pytest.raises(E.TokenOutOfRange):
        s.prefill_ids([-1])
    with pytest.raises(E.ContextExhausted):
        s.generate_ids(prompt, cfg["max_context"])
    assert s.position() == 0
    assert s.generate_ids(prompt, 0).generated_ids == []
    s.prefill_ids(prompt)
    with pytest.raises(E.FreshSessionRequired):
        s.generate_ids(prompt, 2)
    with pytest.raises(E.ContextExhausted):
        s.prefill_ids([1] * (cfg["max_context"] - 15))
    with pytest.raises(E.InvalidArgument):
        s.decode([1, 2])  # batch above max_batch
    assert s.position() == 16 and not s.is_full()
    s.reset_sequence()
    assert s.position() == 0
    assert s.generate_ids(prompt, 3).generated_ids == make_session(data, kv_f32=True).generate_ids(prompt, 3).generated_ids


def test_binding_rejections_precede_device_work(tiny):
    cfg, tensors, _, _ = tiny
    E = session
    target = E.CudaSessionTarget()

    def plan_with(change):
        t = dict(tensors)
        change(t)
        return E.LlamaCudaPlan.from_tensors(cfg, t, target)

    with pytest.raises(E.UnexpectedTensor):
        plan_with(lambda t: t.update({"blk.0.attn_q.extra": t["blk.0.attn_q.weight"]}))
    with pytest.raises(E.ShapeMismatch):
        plan_with(lambda t: t.update({"blk.0.attn_k.weight": (quant.Q8_0, 128, 256, t["blk.0.attn_k.weight"][3][: 128 * 272])}))
    with pytest.raises(E.UnsupportedType):
        plan_with(lambda t: t.update({"output_norm.weight": (quant.Q8_0, 1, 256, np.zeros(272, np.uint8))}))
    with pytest.raises(E.UnsupportedType):
        plan_with(lambda t: t.update({"blk.1.ffn_up.weight": (13, 688, 256, np.zeros(688 * 176, np.uint8))}))  # Q5_K

    def poison(t):
        kind, rows, cols, data = t["blk.1.ffn_gate.weight"]
        data = data.copy()
        data[34 * 5 + 1] = 0x7C
        t["blk.1.ffn_gate.weight"] = (kind, rows, cols, data)

    with pytest.raises(E.NonFiniteScale):
        plan_with(poison)
    missing = dict(tensors)
    del missing["blk.1.ffn_norm.weight"]
    with pytest.raises(E.MissingTensor):
        E.LlamaCudaPlan.from_tensors(cfg, missing, target).prepare()


def test_host_injected_failures_are_typed_and_recoverable(tiny):
    """Fault injection on the host side of the runtime (no GPU fault is ever provoked)."""
    from rustgrad_b200 import _lib
    cfg, tensors, data, prompt = tiny
    L = _lib.load()
    s = make_session(data, kv_f32=True, disable_graph=True)
    s.prefill_ids(prompt[:4])
    L.rg_b200_test_fail_after(b"launch", 5)
    with pytest.raises(session.CudaError):
        s.run_token(3)
    assert s.position() == 4                      # position unchanged
    logits = s.run_token(3)                       # retry succeeds
    ref = make_session(data, kv_f32=True, disable_graph=True)
    ref.prefill_ids(prompt[:4])
    assert np.array_equal(logits, ref.run_token(3))
    L.rg_b200_test_fail_after(b"sync", 0)
    with pytest.raises(session.Poisoned):         # completion unprovable -> poisoned
        s.run_token(4)
    L.rg_b200_test_fail_after(b"sync", -1)
    with pytest.raises(session.Poisoned):
        s.run_token(4)
    L.rg_b200_test_fail_after(b"malloc", 3)
    with pytest.raises(session.OutOfMemory):
        make_session(data)
    L.rg_b200_test_fail_after(b"malloc", -1)
    make_session(data).prefill_ids(prompt)


def test_device_synthesized_weights_match_host_recipe():
    """The device generator + GGML quantizer are reproducible on the host, bit for bit."""
    cfg = synth.scaled(synth.TINY, n_layers=1, vocab=64)
    plan = session.LlamaCudaPlan.empty(cfg, session.CudaSessionTarget())
    for name, kind, rows, cols in (("blk.0.attn_q.weight", quant.Q4_0, 256, 256), ("blk.0.ffn_gate.weight", quant.Q8_0, 688, 256),
                                   ("blk.0.ffn_down.weight", quant.F32, 256, 688), ("token_embd.weight", quant.F16, 64, 256)):
        plan.synth_tensor(name, kind, rows, cols, seed=42, std=0.02)
        got = plan.read_tensor(name)
        e = np.arange(rows * cols, dtype=np.uint64)
        total = np.zeros(rows * cols, dtype=np.uint64)
        with np.errstate(over="ignore"):
            for i in range(4):
                z = np.uint64(42) * np.uint64(0xD1342543DE82EF95) + e * np.uint64(4) + np.uint64(i)
                z = z + np.uint64(0x9E3779B97F4A7C15)
                z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
                z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
                z = z ^ (z >> np.uint64(31))
                for sh in (0, 16, 32, 48):
                    total += (z >> np.uint64(sh)) & np.uint64(0xFFFF)
        normal = (total.astype(np.int64) - 524280).astype(np.float32) * np.float32(1.0 / 75674.5234375)
        w = (normal * np.float32(0.02)).astype(np.float32)
        assert abs(float(normal.std()) - 1.0) < 0.02 and abs(float(normal.mean())) < 0.02
        want = quant.encode(kind, w.reshape(rows, cols))
        assert np.array_equal(got, want.reshape(-1)), name


def test_llama3_8b_width_model_matches_cpu_path_on_device_synthesized_weights():
    """The Llama-3-8B shape at full width (d 4096, 32/8 heads of 128, ffn 14336, vocab 128256, Q4_0 body,
    Q8_0 embedding + head, f16 KV) with 3 of the 32 layers, so the CPU checker finishes in seconds.
    The weights are generated on the device and read back, so both sides see the same bytes."""
    cfg = synth.scaled(synth.LLAMA_8B, n_layers=3, max_context=256)
    target = session.CudaSessionTarget(max_context=256)
    plan = session.LlamaCudaPlan.synthetic(cfg, target, seed=6)
    tensors = {}
    for name, rows, cols, is_norm in synth.tensor_inventory(cfg, tied_head=False):
        kind = quant.F32 if is_norm else quant.Q8_0 if name in ("token_embd.weight", "output.weight") else quant.Q4_0
        tensors[name] = (kind, rows, cols, plan.read_tensor(name))
    s = plan.prepare()
    oracle = O.OracleModel(cfg, tensors, kv_f16=True)
    prompt = synth.prompt_ids(cfg, 24, seed=1)
    want = oracle.forward(prompt, O.MODE_FAST)
    got = s.prefill_ids(prompt)
    assert_logits_close(got, want)
    tok = O.select_greedy(want)
    assert int(np.argmax(got)) == tok
    for _ in range(4):
        want = oracle.forward([tok], O.MODE_FAST)
        logits, greedy = s.decode([tok], want_logits=True)
        assert_logits_close(logits[0], want)
        nxt = O.select_greedy(want)
        assert int(greedy[0]) == nxt, ("greedy id differs from the checker", np.sort(want)[-2:])
        tok = nxt


def test_full_size_8b_shape_properties():
    """The Llama-3-8B shape at its full size (32 layers, 4.5 GB of Q4_0 / Q8_0 weights synthesised on the
    device): size-independent properties of the path, the same sequence through different kernels
    and call patterns (the comparison with the CPU checker at this size is the test below)."""
    cfg = synth.scaled(synth.LLAMA_8B, max_context=1024)
    prompt = synth.prompt_ids(cfg, 300, seed=1)

    def make(**kw):
        target = session.CudaSessionTarget(max_context=1024, **kw)
        return session.LlamaCudaPlan.synthetic(cfg, target, seed=6).prepare()

    a = make(max_batch=2)
    full = a.prefill_ids(prompt)                       # one tensor-core chunk
    assert np.isfinite(full).all() and full.shape == (cfg["vocab"],)
    first = int(np.argmax(full))
    # the same prompt in two calls (chunk boundary inside the cache) and on the second row
    part = a.prefill_ids(prompt[:173], row=1, want_logits=False)
    assert part is None
    again = a.prefill_ids(prompt[173:], row=1)
    assert np.abs(again - full).max() <= 2e-3 * max(1.0, np.abs(full).max())
    # two identical rows decode identically through the batch-2 kernels, and like a batch-1 session
    ids2, _ = a.decode_loop([first, first], 12)
    assert ids2[:, 0].tolist() == ids2[:, 1].tolist()
    b = make()
    assert np.abs(b.prefill_ids(prompt) - full).max() <= 1e-4
    ids1, _ = b.decode_loop([first], 12)
    assert ids1[:, 0].tolist() == ids2[:, 0].tolist()
    # host-driven steps (graph replay per call, logits read back) follow the device-resident loop
    c = make()
    c.prefill_ids(prompt)
    tok, host_ids = first, []
    for _ in range(12):
        logits, greedy = c.decode([tok], want_logits=True)
        assert int(np.argmax(logits[0])) == int(greedy[0])
        tok = int(greedy[0])
        host_ids.append(tok)
    assert host_ids == ids1[:, 0].tolist()


def test_thirty_two_rows_at_full_width_match_one_row():
    """A decode batch of 32 at the 8B width (2 layers): the K-split tensor-core path has its
    largest partial-sum footprint here (every projection, 32 tokens); all rows carry the same
    sequence, so every row must reproduce the one-row session."""
    cfg = synth.scaled(synth.LLAMA_8B, n_layers=2, max_context=64)
    prompt = synth.prompt_ids(cfg, 5, seed=3)

    def make(batch):
        target = session.CudaSessionTarget(max_context=64, max_batch=batch)
        return session.LlamaCudaPlan.synthetic(cfg, target, seed=6).prepare()

    one = make(1)
    tok = int(np.argmax(one.prefill_ids(prompt)))
    want, _ = one.decode([tok], want_logits=True)
    many = make(32)
    for r in range(32):
        many.prefill_ids(prompt, row=r, want_logits=False)
    got, greedy = many.decode([tok] * 32, want_logits=True)
    for r in range(32):
        assert_logits_close(got[r], want[0])
    assert len(set(greedy.tolist())) == 1
    # a 32-token prompt remainder after a restored prefix takes the same path (prefill, m = 32)
    again = make(1)
    long_prompt = synth.prompt_ids(cfg, 40, seed=4)
    full = again.prefill_ids(long_prompt)
    split = make(1)
    split.prefill_ids(long_prompt[:8], want_logits=False)
    assert_logits_close(split.prefill_ids(long_prompt[8:]), full)


def device_model(cfg, seed, embed=quant.Q8_0, head=quant.Q8_0, **target_kw):
    """A model synthesised on the device and read back, so the session and the checker hold the same bytes."""
    target = session.CudaSessionTarget(**target_kw)
    plan = session.LlamaCudaPlan.synthetic(cfg, target, seed=seed, embed_type=embed, head_type=head)
    tensors = {}
    for name, rows, cols, is_norm in synth.tensor_inventory(cfg, tied_head=False):
        kind = quant.F32 if is_norm else embed if name == "token_embd.weight" else head if name == "output.weight" else quant.Q4_0
        tensors[name] = (kind, rows, cols, plan.read_tensor(name))
    return plan.prepare(), tensors


def check_prefill_and_decode(s, oracle, prompt, steps):
    """Prefill logits, then `steps` decode steps: every logit inside the bar, every greedy id equal."""
    want = oracle.forward(prompt, O.MODE_FAST)
    got = s.prefill_ids(prompt)
    assert_logits_close(got, want)
    tok = O.select_greedy(want)
    assert int(np.argmax(got)) == tok
    worst = float(np.abs(got - want).max())
    for _ in range(steps):
        want = oracle.forward([tok], O.MODE_FAST)
        logits, greedy = s.decode([tok], want_logits=True)
        assert_logits_close(logits[0], want)
        worst = max(worst, float(np.abs(logits[0] - want).max()))
        tok = O.select_greedy(want)
        assert int(greedy[0]) == tok, ("greedy id differs from the checker", np.sort(want)[-2:])
    return worst


def test_llama3_8b_shape_at_full_depth_matches_cpu_path():
    """All 32 layers of the Llama-3-8B shape (Q4_0 body, Q8_0 embedding + head, f16 KV cache): a
    16-token prompt (tensor-core path, compensated operands) and 4 decode steps (integer GEMV, fused
    attention) against the CPU checker on the same bytes: logit bar, identical greedy ids."""
    cfg = synth.scaled(synth.LLAMA_8B, max_context=64)
    s, tensors = device_model(cfg, seed=6, max_context=64)
    oracle = O.OracleModel(cfg, tensors, kv_f16=True)
    worst = check_prefill_and_decode(s, oracle, synth.prompt_ids(cfg, 16, seed=1), 4)
    print(f"32 layers: max |logit - checker| = {worst:.3e}")
    assert session.launch_count("qgemv_i8") > 0 and session.launch_count("attn_fused") > 0


def test_long_prompt_at_depth_on_the_tensor_core_path():
    """A 300-token prompt through 8 full-width layers: two tensor-core chunks with the tiled causal
    attention, then decode steps over a cache of 300 positions."""
    cfg = synth.scaled(synth.LLAMA_8B, n_layers=8, max_context=320)
    s, tensors = device_model(cfg, seed=6, max_context=320)
    oracle = O.OracleModel(cfg, tensors, kv_f16=True)
    before = session.launch_count("attn_prefill"), session.launch_count("qgemm_tc")
    worst = check_prefill_and_decode(s, oracle, synth.prompt_ids(cfg, 300, seed=2), 2)
    print(f"8 layers, 300-token prompt: max |logit - checker| = {worst:.3e}")
    assert session.launch_count("attn_prefill") > before[0] and session.launch_count("qgemm_tc") > before[1]


def test_llama3_70b_width_on_one_gpu_matches_cpu_path():
    """The Llama-3-70B width (d 8192, 64 / 8 heads of 128, ffn 28672, full vocabulary, everything
    Q4_0) with 2 of the 80 layers on one GPU against the CPU checker."""
    cfg = synth.scaled(synth.LLAMA_70B, n_layers=2, max_context=64)
    s, tensors = device_model(cfg, seed=7, embed=quant.Q4_0, head=quant.Q4_0, max_context=64)
    oracle = O.OracleModel(cfg, tensors, kv_f16=True)
    worst = check_prefill_and_decode(s, oracle, synth.prompt_ids(cfg, 16, seed=1), 4)
    print(f"70B width, 2 layers: max |logit - checker| = {worst:.3e}")


@pytest.fixture(scope="module")
def small_hd128():
    """A model every projection of which qualifies for the integer GEMV and the one-launch attention."""
    cfg = synth.scaled(synth.TINY, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn_dim=1024, vocab=640, n_layers=3,
                       rope_theta=500000.0, max_context=1100)
    tensors = synth.build_tensors(cfg, seed=21, body_type=quant.Q4_0, embed_type=quant.Q8_0, head_type=quant.Q8_0,
                                  tied_head=False)
    return cfg, tensors


def test_two_token_prompt_chunks_see_their_own_first_token(small_hd128):
    """A chunk of exactly two prompt tokens runs the two-column GEMV path; its second column reads the
    K / V row its first column appends, so the two must not share the one-launch attention kernel.
    Cases: a 2-token prompt, a prompt of 1024 + 2 tokens, and 2 tokens after a cached prefix."""
    cfg, tensors = small_hd128
    mk = lambda: session.LlamaCudaPlan.from_tensors(  # noqa: E731
        cfg, tensors, session.CudaSessionTarget(kv_f32=True, max_context=1100)).prepare()
    oracle = O.OracleModel(cfg, tensors, threads=4)
    pair = [17, 301]
    s = mk()
    got = s.prefill_ids(pair)
    assert_logits_close(got, oracle.forward(pair, O.MODE_FAST))
    steps = mk()
    steps.run_token(pair[0])
    assert np.abs(steps.run_token(pair[1]) - got).max() <= 1e-4
    # 1026 tokens: a 1024-token tensor-core chunk, then a 2-token chunk
    long_prompt = synth.prompt_ids(cfg, 1026, seed=5)
    oracle.reset()
    want = oracle.forward(long_prompt, O.MODE_FAST)
    s = mk()
    assert_logits_close(s.prefill_ids(long_prompt), want)
    # 2 tokens after 5 cached ones (what a prefix-cache hit leaves to prefill)
    oracle.reset()
    want = oracle.forward(long_prompt[:7], O.MODE_FAST)
    s = mk()
    s.prefill_ids(long_prompt[:5], want_logits=False)
    assert_logits_close(s.prefill_ids(long_prompt[5:7]), want)


def test_gguf_without_stop_keys_stops_on_token_zero():
    """rustgrad takes the stop ids from the tokenizer: without `tokenizer.ggml.eos_token_id` the eos
    id is 0 (src/tokenizer/mod.rs:284-296, model.rs:288-292).  The embedding rows of token 0 and of
    the token this model emits first are swapped (the head is tied; the prompt is renamed alike), so the
    greedy run emits 0."""
    cfg = dict(synth.TINY)
    tensors = synth.build_tensors(cfg, seed=0, body_type=quant.Q8_0)
    prompt = synth.prompt_ids(cfg, 16, seed=1)
    base = O.OracleModel(cfg, tensors, threads=1)
    first = base.generate_greedy(prompt, 1, O.MODE_STRICT)[0][0]
    assert first != 0
    kind, rows, cols, data = tensors["token_embd.weight"]
    emb = data.reshape(rows, -1).copy()
    emb[[0, first]] = emb[[first, 0]]
    swapped = dict(tensors)
    swapped["token_embd.weight"] = (kind, rows, cols, emb.reshape(-1))
    # the same renaming in the prompt: the model now behaves as before with ids 0 and `first` exchanged
    prompt = np.where(prompt == first, 0, np.where(prompt == 0, first, prompt)).astype(np.int32)
    data = synth.gguf_bytes(cfg, swapped)  # the writer emits no eos / eot key
    g = session.GgufFile(data)
    got_cfg = g.llama_config()
    g.close()
    assert got_cfg["eos_id"] == 0 and got_cfg["eot_id"] == -1
    s = make_session(data, kv_f32=True)
    gen = s.generate_ids(prompt, 8)
    assert gen.generated_ids == [0] and gen.stopped and s.position() == 16
    # the checker with the reference's default agrees; with no stop id the run goes on
    oracle = O.OracleModel(dict(cfg, eos_id=0), swapped, threads=1)
    assert oracle.generate_greedy(prompt, 8, O.MODE_STRICT) == ([0], True)


def test_bounded_device_wait_that_runs_out_is_a_timeout_then_poisoned(tiny):
    """A device-side wait never spins for ever: it gives up, records a status and the kernel
    returns.  The hook launches the exchange kernel against a flag nobody writes with a short poll
    limit; the step that follows reports the time-out and the session refuses further work."""
    cfg, tensors, data, prompt = tiny
    s = make_session(data, kv_f32=True)
    s.prefill_ids(prompt[:4])
    before = session.launch_count("tp_exchange")
    s.expire_device_wait()
    assert session.launch_count("tp_exchange") == before + 1
    with pytest.raises(session.Timeout):
        s.run_token(3)
    assert s.position() == 4
    with pytest.raises(session.Poisoned):
        s.run_token(3)
    with pytest.raises(session.Poisoned):
        s.reset_sequence()
    # other sessions of the process are untouched
    assert np.isfinite(make_session(data, kv_f32=True).prefill_ids(prompt)).all()


def test_packed_rows_of_any_whole_number_of_blocks():
    """rustgrad accepts packed tensors whose K is a multiple of 32 (src/gguf/quantization/data.rs:268-270).
    Rows that are not whole groups of 256 elements take the generic decode-and-multiply GEMV."""
    # q width 256 and k width 128 over K = 160, ffn_down over K = 224: neither a multiple of 256
    cfg = synth.scaled(synth.TINY, d_model=160, n_heads=4, n_kv_heads=2, head_dim=64, ffn_dim=224, vocab=96, n_layers=2)
    tensors = synth.build_tensors(cfg, seed=3, body_type=quant.Q4_0, embed_type=quant.Q8_0, head_type=quant.Q8_0, tied_head=False)
    oracle = O.OracleModel(cfg, tensors, threads=2)
    s = session.LlamaCudaPlan.from_tensors(cfg, tensors, session.CudaSessionTarget(kv_f32=True)).prepare()
    prompt = synth.prompt_ids(cfg, 11, seed=4)
    want_ids, _ = oracle.generate_greedy(prompt, 10, O.MODE_STRICT)
    assert s.generate_ids(prompt, 10).generated_ids == want_ids
    oracle.reset()
    s.reset_sequence()
    assert_logits_close(s.prefill_ids(prompt), oracle.forward(prompt))


VARIANTS = [dict(rope_dim=32, qk_norm=1, qkv_bias=1), dict(rope_dim=16), dict(qk_norm=2, n_kv_heads=4), dict(qkv_bias=1),
            dict(rope_dim=2, qk_norm=1, qkv_bias=1, body=quant.Q4_0, head_dim=128, n_heads=2, n_kv_heads=1)]


@pytest.mark.parametrize("variant", VARIANTS, ids=lambda v: "-".join(f"{k}{v[k]}" for k in sorted(v)))
def test_model_variants_match_cpu_path(variant):
    """Partial rotary lanes (the query permuted over its last rope_dim lanes, the key over the head),
    RMS norms of q and k per head or per projection, and q / k / v biases
    (src/models/transformer/layer.rs:274-346,481-571; model.rs:253-282): prefill in chunks, token
    steps and batched decode against the CPU checker, through a GGUF file."""
    variant = dict(variant)
    body = variant.pop("body", quant.Q8_0)
    base = dict(d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn_dim=512, vocab=320, n_layers=2, max_context=96)
    base.update(variant)
    cfg = synth.scaled(synth.TINY, **base)
    tensors = synth.build_tensors(cfg, seed=8, body_type=body)
    data = synth.gguf_bytes(cfg, tensors)
    g = session.GgufFile(data)
    got_cfg = g.llama_config()
    g.close()
    for key in ("rope_dim", "qk_norm", "qkv_bias"):
        want = cfg.get(key, 0)
        assert got_cfg[key] == (0 if key == "rope_dim" and want == cfg["head_dim"] else want), key
    s = make_session(data, kv_f32=True, max_batch=3)
    oracle = O.OracleModel(cfg, tensors, threads=2)
    prompt = synth.prompt_ids(cfg, 21, seed=9)       # one tensor-core chunk when the model qualifies, else chunks of 8
    assert_logits_close(s.prefill_ids(prompt), oracle.forward(prompt))
    tok = 5
    for _ in range(4):                                # token steps
        want = oracle.forward([tok])
        got = s.run_token(tok)
        assert_logits_close(got, want)
        tok = O.select_greedy(want)
        assert int(np.argmax(got)) == tok
    # three rows decoding together at different positions
    oracles = [oracle] + [O.OracleModel(cfg, tensors, threads=2) for _ in range(2)]
    toks = [tok]
    for r in (1, 2):
        p = synth.prompt_ids(cfg, 3 + 4 * r, seed=20 + r)
        s.prefill_ids(p, row=r, want_logits=False)
        toks.append(O.select_greedy(oracles[r].forward(p)))
    logits, greedy = s.decode(toks, want_logits=True)
    for r in range(3):
        want = oracles[r].forward([toks[r]])
        assert_logits_close(logits[r], want)
        assert int(greedy[r]) == O.select_greedy(want)


def test_incomplete_variant_families_are_refused():
    cfg = synth.scaled(synth.TINY, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn_dim=512, vocab=320, n_layers=2,
                       qk_norm=1, qkv_bias=1)
    tensors = synth.build_tensors(cfg, seed=8)
    target = session.CudaSessionTarget()
    missing = {k: v for k, v in tensors.items() if k != "blk.1.attn_k.bias"}
    with pytest.raises(session.MissingTensor):
        session.LlamaCudaPlan.from_tensors(cfg, missing, target).prepare()
    plain = synth.scaled(cfg, qk_norm=0, qkv_bias=0)
    with pytest.raises(session.UnexpectedTensor):   # variant tensors a plain configuration does not name
        session.LlamaCudaPlan.from_tensors(plain, tensors, target)
    # a file with only the query norm, or only two of the three biases, has no configuration
    for drop in ("blk.0.attn_k_norm.weight", "blk.0.attn_v.bias"):
        partial = {k: v for k, v in tensors.items() if k != drop}
        g = session.GgufFile(synth.gguf_bytes(cfg, partial))
        with pytest.raises(session.UnsupportedVariant):
            g.llama_config()
        g.close()


def test_batched_prompt_prefill_matches_per_prompt_prefill(small_hd128, tiny):
    """Several prompts in one pass (rg_b200_prefill_rows; src/models/transformer/batch.rs:177-325):
    one chunk holding five prompts of very different lengths (logits of five arbitrary columns),
    prompts cut across two chunks, a row that continues from cached positions, and a model that is
    not on the tensor-core path; every prompt must see exactly what it sees alone, and the decode
    step that follows must find every cache row in place."""
    cfg, tensors = small_hd128
    mk = lambda **kw: session.LlamaCudaPlan.from_tensors(  # noqa: E731
        cfg, tensors, session.CudaSessionTarget(kv_f32=True, max_context=1100, **kw)).prepare()

    def check(s, prompts, model_cfg, model_tensors, mode=O.MODE_FAST, kv_f16=False):
        before = {r: s.position(r) for r in prompts}
        logits, greedy = s.prefill_rows(prompts)
        oracles = {}
        for i, (row, p) in enumerate(prompts.items()):
            o = oracles[row] = O.OracleModel(model_cfg, model_tensors, kv_f16=kv_f16, threads=4)
            want = o.forward(p, mode)
            assert_logits_close(logits[i], want)
            assert int(greedy[i]) == O.select_greedy(want)
            assert s.position(row) == before[row] + len(p)
        return oracles, [int(g) for g in greedy]

    s = mk(max_batch=5)
    prompts = {2: synth.prompt_ids(cfg, 40, seed=1), 0: synth.prompt_ids(cfg, 7, seed=2), 4: synth.prompt_ids(cfg, 300, seed=3),
               1: synth.prompt_ids(cfg, 1, seed=4), 3: synth.prompt_ids(cfg, 2, seed=5)}
    before = session.launch_count("attn_prefill")
    oracles, toks = check(s, prompts, cfg, tensors)
    assert session.launch_count("attn_prefill") == before + 5 * cfg["n_layers"]   # one chunk, one attention launch per prompt
    order = list(prompts)                                     # decode all five rows together: row r feeds its own token
    by_row = {row: toks[i] for i, row in enumerate(order)}
    logits, _ = s.decode([by_row[r] for r in range(5)], want_logits=True)
    for r in range(5):
        assert_logits_close(logits[r], oracles[r].forward([by_row[r]], O.MODE_FAST))
    # 700 + 500 + 30 tokens: the second prompt is cut by the 1024-column chunk boundary
    s = mk(max_batch=3)
    check(s, {0: synth.prompt_ids(cfg, 700, seed=6), 1: synth.prompt_ids(cfg, 500, seed=7), 2: synth.prompt_ids(cfg, 30, seed=8)},
          cfg, tensors)
    # the same with the f16 cache: every run of the chunk goes through the tensor-core attention kernel
    s = session.LlamaCudaPlan.from_tensors(cfg, tensors, session.CudaSessionTarget(max_context=1100, max_batch=3)).prepare()
    before = session.launch_count("attn_prefill_tc")
    check(s, {2: synth.prompt_ids(cfg, 90, seed=14), 0: synth.prompt_ids(cfg, 33, seed=15), 1: synth.prompt_ids(cfg, 200, seed=16)},
          cfg, tensors, kv_f16=True)
    assert session.launch_count("attn_prefill_tc") == before + 3 * cfg["n_layers"]
    # a row that already holds positions continues from them
    s = mk(max_batch=2)
    head, tail = synth.prompt_ids(cfg, 9, seed=9), synth.prompt_ids(cfg, 20, seed=10)
    s.prefill_ids(head, row=1, want_logits=False)
    logits, _ = s.prefill_rows({1: tail, 0: head})
    o = O.OracleModel(cfg, tensors, threads=4)
    assert_logits_close(logits[0], o.forward(np.concatenate([head, tail]), O.MODE_FAST))
    # typed refusals leave every position as it was
    for bad, err in (({0: head, 1: [cfg["vocab"]]}, session.TokenOutOfRange), ({0: head, 1: []}, session.EmptyPrompt),
                     ({0: head, 1: synth.prompt_ids(cfg, 1100, seed=1)}, session.ContextExhausted)):
        with pytest.raises(err):
            s.prefill_rows(bad)
        assert (s.position(0), s.position(1)) == (9, 29)
    import ctypes as C
    from rustgrad_b200 import _lib
    rows = (C.c_int32 * 2)(0, 0)
    lens = (C.c_size_t * 2)(1, 1)
    ids = (C.c_int32 * 2)(1, 2)
    assert _lib.load().rg_b200_prefill_rows(s._h, rows, ids, lens, 2, None, None) == 1   # a row listed twice
    # a model with a dense projection (K = 688): the prompts run one after the other
    tcfg, ttensors, tdata, _ = tiny
    s = make_session(tdata, kv_f32=True, max_batch=3)
    check(s, {1: synth.prompt_ids(tcfg, 12, seed=11), 0: synth.prompt_ids(tcfg, 5, seed=12), 2: synth.prompt_ids(tcfg, 20, seed=13)},
          tcfg, ttensors, O.MODE_STRICT)


@pytest.mark.parametrize("heads,kv_heads", [(4, 1), (4, 2), (2, 2), (8, 1)])
def test_prompt_attention_on_tensor_cores_with_f16_cache(heads, kv_heads):
    """Prompt chunks of a session with the f16 cache run the tensor-core attention kernel
    (attn_prefill_tc.cu): 1, 2, 4 and 8 query heads per kv head, a chunk whose last tile is ragged
    (700 tokens), a second chunk that sees 1024 cached positions (1030 tokens), and the same prompt
    through the f32 kernel; against the checker with an f16 cache."""
    cfg = synth.scaled(synth.TINY, d_model=heads * 128, n_heads=heads, n_kv_heads=kv_heads, head_dim=128, ffn_dim=512, vocab=320,
                       n_layers=2, rope_theta=500000.0, max_context=1100)
    tensors = synth.build_tensors(cfg, seed=31, body_type=quant.Q8_0)
    oracle = O.OracleModel(cfg, tensors, kv_f16=True, threads=4)
    for n in (700, 1030):
        prompt = synth.prompt_ids(cfg, n, seed=n)
        s = session.LlamaCudaPlan.from_tensors(cfg, tensors, session.CudaSessionTarget(max_context=1100)).prepare()
        before = session.launch_count("attn_prefill_tc")
        got = s.prefill_ids(prompt)
        assert session.launch_count("attn_prefill_tc") >= before + cfg["n_layers"]
        oracle.reset()
        want = oracle.forward(prompt, O.MODE_FAST)
        assert_logits_close(got, want)
        tok = O.select_greedy(want)
        assert_logits_close(s.run_token(tok), oracle.forward([tok], O.MODE_FAST))   # the cache rows it left are the checker's


@pytest.mark.parametrize("heads,kv_heads", [(4, 1), (4, 2), (2, 2), (8, 1)])
def test_batched_decode_attention_on_tensor_cores_with_f16_cache(heads, kv_heads):
    """Eight or more rows decoding together on f16 caches run the tensor-core decode attention
    (attn_decode_tc.cu): 1, 2, 4 and 8 query heads per kv head; rows at different positions, so spans end in
    ragged 16-key tiles, some warps of a CTA get no tile, and long rows are cut into several spans; every
    row against its own checker with an f16 cache, three steps."""
    cfg = synth.scaled(synth.TINY, d_model=heads * 128, n_heads=heads, n_kv_heads=kv_heads, head_dim=128, ffn_dim=512, vocab=320,
                       n_layers=2, rope_theta=500000.0, max_context=700)
    tensors = synth.build_tensors(cfg, seed=33, body_type=quant.Q4_0)
    # 9 and 16 rows: one step; 20 rows: two steps of 10 rows
    for rows, lengths in ((9, (1, 15, 16, 17, 63, 64, 65, 130, 600)), (16, tuple(5 + 41 * r for r in range(16))),
                          (20, tuple(3 + 29 * r for r in range(20)))):
        s = session.LlamaCudaPlan.from_tensors(cfg, tensors, session.CudaSessionTarget(max_context=700, max_batch=rows)).prepare()
        oracles = [O.OracleModel(cfg, tensors, kv_f16=True, threads=2) for _ in range(rows)]
        toks = []
        for r in range(rows):
            p = synth.prompt_ids(cfg, lengths[r], seed=200 + r)
            s.prefill_ids(p, row=r)
            toks.append(O.select_greedy(oracles[r].forward(p, O.MODE_FAST)))
        before = session.launch_count("attn_decode_tc")
        for _ in range(3):
            logits, greedy = s.decode(toks, want_logits=True)
            nxt = []
            for r in range(rows):
                w = oracles[r].forward([toks[r]], O.MODE_FAST)
                assert_logits_close(logits[r], w)
                nxt.append(O.select_greedy(w))
            toks = nxt
        assert session.launch_count("attn_decode_tc") >= before + cfg["n_layers"]  # later steps may replay a captured graph
