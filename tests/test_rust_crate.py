"""The Rust binding crate is source only (no Rust toolchain in this image): check that its extern
block declares exactly the functions the headers declare, with the same number of parameters, and
that its #[repr(C)] structs have the fields of the C structs in the same order."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CRATE = ROOT / "rust" / "rustgrad-b200-sys"


def c_declarations():
    out = {}
    for h in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        for m in re.finditer(r"\n[a-zA-Z_][^;{}()]*?\b(rg_b200_\w+)\s*\(([^;]*?)\);", text):
            args = " ".join(m.group(2).split())
            out[m.group(1)] = 0 if args in ("", "void") else len(args.split(","))
    return out


def rust_declarations():
    text = (CRATE / "src" / "lib.rs").read_text()
    block = text[text.index('unsafe extern "C" {'):]
    out = {}
    for m in re.finditer(r"pub fn (rg_b200_\w+)\((.*?)\)(?: -> [^;]+)?;", block):
        args = m.group(2).strip()
        out[m.group(1)] = 0 if not args else len(args.split(", "))
    return out


def test_bindings_cover_every_export_with_matching_arity():
    c, r = c_declarations(), rust_declarations()
    assert set(c) == set(r), (sorted(set(c) - set(r)), sorted(set(r) - set(c)))
    assert c == r, {k: (c[k], r[k]) for k in c if c[k] != r[k]}
    from rustgrad_b200 import _lib
    assert set(c) == set(_lib.EXPORTS)


def c_struct_fields(header, name):
    text = re.sub(r"/\*.*?\*/", "", (ROOT / "include" / header).read_text(), flags=re.S)
    m = re.search(r"typedef struct(?: \w+)? \{([^}]*)\} " + name + ";", text)
    fields = []
    for line in m.group(1).split(";"):
        line = line.strip()
        if line:
            first, *more = line.split(",")          # `uint64_t a, b;` declares two fields
            for part in [first.split()[-1]] + [m.strip() for m in more]:
                fields.append(re.sub(r"\[.*\]", "", part).lstrip("*"))
    return fields


def rust_struct_fields(name):
    text = (CRATE / "src" / "lib.rs").read_text()
    m = re.search(r"pub struct " + name + r" \{(.*?)\n\}", text, flags=re.S)
    return re.findall(r"pub (\w+):", m.group(1))


def test_repr_c_structs_list_the_c_fields_in_order():
    for header, name in (("rg_b200.h", "rg_llama_config"), ("rg_b200.h", "rg_options"), ("rg_b200.h", "rg_report"),
                         ("rg_b200.h", "rg_device_info"),
                         ("rg_b200_tokenizer.h", "rg_tok_config"), ("rg_b200_tokenizer.h", "rg_tok_error"),
                         ("rg_b200_workflow.h", "rg_prompt_output"), ("rg_b200_serving.h", "rg_serving_error"),
                         ("rg_b200_serving.h", "rg_serving_options"), ("rg_b200_serving.h", "rg_serving_sampling"),
                         ("rg_b200_serving.h", "rg_token_event"), ("rg_b200_serving.h", "rg_serving_result"),
                         ("rg_b200_serving.h", "rg_prefix_stats"), ("rg_b200_serving.h", "rg_batch_error")):
        assert c_struct_fields(header, name) == rust_struct_fields(name), name


def test_facade_files_exist_and_name_the_reference_trait():
    safe = (CRATE / "src" / "safe.rs").read_text()
    for item in ("CudaSessionTarget", "LlamaCudaPlan", "LlamaCudaSession", "LlamaCudaGenerationError", "LlamaCudaProgress"):
        assert f"pub struct {item}" in safe or f"pub enum {item}" in safe, item
    integration = (CRATE / "integration" / "cuda_generation.rs").read_text()
    assert "impl SessionTarget<LlamaCudaModelPlan> for CudaSessionTarget" in integration
    assert "[dependencies]\n\n" in (CRATE / "Cargo.toml").read_text()  # none
