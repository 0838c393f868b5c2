"""The prompt-to-tokens facade (include/rg_b200_workflow.h, rustgrad_b200/workflow.py): text in,
token ids and text out, against the checker's tokenizer restatement and CPU model
(src/models/transformer/workflow.rs:66-124, generation.rs:92-160, examples/llama_prompt.rs)."""
import numpy as np
import pytest

from oracle import oracle as O
from oracle import tokenizer_oracle as T
from rustgrad_b200 import gguf_writer, llama_prompt, quant, session, synth, workflow


def test_command_line_arguments_follow_the_reference_parser():
    assert llama_prompt.parse_args(["fixture.gguf", "hello", "4"]) == ("fixture.gguf", "hello", 4)
    assert llama_prompt.parse_args(["fixture.gguf", "hello"]) == ("fixture.gguf", "hello", 16)
    for bad in ([], ["only.gguf"], ["a.gguf", "hi", "x"], ["a.gguf", "hi", "3", "extra"], ["a.gguf", "hi", "-1"]):
        with pytest.raises(ValueError):
            llama_prompt.parse_args(bad)
    assert llama_prompt.main(["missing-prompt.gguf"]) == 2


def test_chat_token_table_encodes_text_like_the_checker():
    tokens, types, ids = gguf_writer.chat_token_table(512)
    assert len(tokens) == 512 == len(types) and len(set(tokens)) == 512
    normal = [(t, i) for i, (t, ty) in enumerate(zip(tokens, types)) if ty == 1]
    special = [(t, i) for i, (t, ty) in enumerate(zip(tokens, types)) if ty != 1]
    tok = T.SimpleTokenizer(normal, special, eos_id=ids["eos"], eot_id=ids["eot"], bos_id=ids["bos"])
    got = tok.encode("hello world")
    assert tok.decode(got) == "hello world" and len(got) == 2   # "hello" and " world" are merged tokens
    assert tok.encode("<|eot_id|>") == [ids["eot"]]


@pytest.fixture(scope="module")
def chat_model():
    cfg = dict(synth.TINY)
    tensors = synth.build_tensors(cfg, seed=0, body_type=quant.Q8_0)
    data = synth.gguf_bytes(cfg, tensors, chat_tokens=True)
    tokens, types, ids = gguf_writer.chat_token_table(cfg["vocab"])
    normal = [(t, i) for i, (t, ty) in enumerate(zip(tokens, types)) if ty == 1]
    special = [(t, i) for i, (t, ty) in enumerate(zip(tokens, types)) if ty != 1]
    tok = T.SimpleTokenizer(normal, special, eos_id=ids["eos"], eot_id=ids["eot"], bos_id=ids["bos"])
    oracle = O.OracleModel(dict(cfg, eos_id=ids["eos"], eot_id=ids["eot"]), tensors, threads=1)
    return cfg, data, tok, oracle, ids


@pytest.mark.gpu
def test_generate_text_matches_checker_and_streams(chat_model):
    cfg, data, tok, oracle, ids = chat_model
    wf = workflow.LlamaPromptWorkflow.from_gguf_bytes(data, session.CudaSessionTarget(kv_f32=True))
    pieces = []
    out = wf.generate("hello world, the tiny model", 12, on_text=lambda t, s: pieces.append((t, s)))
    want_prompt = [ids["bos"]] + tok.encode("hello world, the tiny model")
    assert out.rendered_prompt == "hello world, the tiny model"
    assert out.generation.prompt_ids == want_prompt
    want_ids, stopped = oracle.generate_greedy(want_prompt, 12, O.MODE_STRICT)
    assert out.generation.generated_ids == want_ids and out.generation.stopped == stopped
    assert out.generation.decoded == tok.decode(want_ids)
    assert [t for t, _ in pieces if t >= 0] == want_ids
    # the streamed text is the decoded text whenever every byte sequence completes (replacement
    # characters of sequences cut by a token boundary may be placed differently)
    streamed = "".join(s for _, s in pieces)
    assert streamed.replace("�", "") == out.generation.decoded.replace("�", "")
    # every request starts from a fresh sequence: the same call twice gives the same result
    again = wf.generate("hello world, the tiny model", 12)
    assert again.generation.generated_ids == want_ids
    assert wf.generate("hello", 0).generation.generated_ids == []


@pytest.mark.gpu
def test_generate_chat_renders_the_checked_template(chat_model):
    cfg, data, tok, oracle, ids = chat_model
    wf = workflow.LlamaPromptWorkflow.from_gguf_bytes(data, session.CudaSessionTarget(kv_f32=True))
    messages = [("system", "be brief"), ("user", "hello")]
    out = wf.generate_chat(messages, 6)
    rendered = ("<|begin_of_text|>" + "".join(f"<|start_header_id|>{r}<|end_header_id|>\n\n{c}<|end_of_text|>" for r, c in messages)
                + "<|start_header_id|>assistant<|end_header_id|>\n\n")
    assert out.rendered_prompt == rendered
    want_prompt = [ids["bos"]] + tok.encode(rendered)
    assert out.generation.prompt_ids == want_prompt
    want_ids, stopped = oracle.generate_greedy(want_prompt, 6, O.MODE_STRICT)
    assert out.generation.generated_ids == want_ids and out.generation.stopped == stopped


@pytest.mark.gpu
def test_request_failures_are_typed_and_precede_device_work(chat_model):
    cfg, data, tok, oracle, ids = chat_model
    wf = workflow.LlamaPromptWorkflow.from_gguf_bytes(data, session.CudaSessionTarget(kv_f32=True))
    with pytest.raises(session.ContextExhausted):
        wf.generate("hello", cfg["max_context"])
    long_message = "x" * (1024 * 1024 + 1)
    with pytest.raises(workflow.TokenizerFailure) as e:
        wf.generate_chat([("user", long_message)], 2)
    assert e.value.tokenizer_status == 16          # message above the 1 MiB bound
    # a file whose chat template is not the supported one is refused at open
    bad = synth.gguf_bytes(cfg, synth.build_tensors(cfg, seed=0, body_type=quant.Q8_0), chat_tokens=True)
    import io
    md = gguf_writer.llama_metadata(cfg, chat_tokens=True) + [gguf_writer.kv_str("tokenizer.chat_template", "{{ messages }}")]
    buf = io.BytesIO()
    gguf_writer.write_gguf(buf, md, synth.build_tensors(cfg, seed=0, body_type=quant.Q8_0))
    with pytest.raises(session.InvalidArgument):
        workflow.LlamaPromptWorkflow.from_gguf_bytes(buf.getvalue())
    assert wf.generate("hello", 3).generation.generated_ids  # the handle is still usable
