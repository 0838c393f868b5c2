"""Run one bounded chat request from a supported local GGUF on the GPU.

    python -m rustgrad_b200.llama_prompt path/to/model.gguf "hello" 16

The command-line counterpart of rustgrad's ``examples/llama_prompt.rs``: one user message through
the checked chat template, greedy, the decoded text on stdout (streamed as it is generated).
"""
from __future__ import annotations

import sys

USAGE = "usage: llama_prompt <model.gguf> <prompt> [max_tokens]"


def parse_args(args):
    """(path, prompt, max_new_tokens); raises ValueError(USAGE) like the reference's parser."""
    args = list(args)
    if len(args) < 2 or len(args) > 3:
        raise ValueError(USAGE)
    max_new = 16
    if len(args) == 3:
        if not args[2].isdigit():
            raise ValueError(USAGE)
        max_new = int(args[2])
    return args[0], args[1], max_new


def main(argv=None) -> int:
    try:
        path, prompt, max_new = parse_args(sys.argv[1:] if argv is None else argv)
    except ValueError as e:
        print(e, file=sys.stderr)
        return 2
    from .workflow import LlamaPromptWorkflow
    workflow = LlamaPromptWorkflow.from_path(path)
    workflow.generate_chat([("user", prompt)], max_new, on_text=lambda _tok, text: (sys.stdout.write(text), sys.stdout.flush()))
    sys.stdout.write("\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
