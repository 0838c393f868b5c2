"""Host-side statement of the tensor-parallel split used by the CUDA runtime.

Megatron-style: Q/K/V, gate/up and the vocabulary head are split by output rows (a contiguous
byte range of the GGML tensor), attention-output and down projections are split along K at
32-element block boundaries (a per-row range of whole blocks), so no block is ever re-encoded.
A contracting-axis split needs a sum all-reduce (src/sharding.rs:642-667); partial sums are
combined in rank order (src/sharded_graph.rs:715-724).  The C++ runtime applies the same rule
with one strided device copy per tensor; this module exists for tests and tools.
"""
from __future__ import annotations

import numpy as np

from .quant import BLOCK_BYTES, BLOCK_ELEMS

ROW_SPLIT = ("attn_q.weight", "attn_k.weight", "attn_v.weight", "ffn_gate.weight", "ffn_up.weight")
COL_SPLIT = ("attn_output.weight", "ffn_down.weight")


def split_kind(name: str) -> str:
    if name == "output.weight" or name.endswith(ROW_SPLIT):
        return "rows"
    if name.endswith(COL_SPLIT):
        return "cols"
    return "none"


def shard(name: str, ggml_type: int, rows: int, cols: int, data: np.ndarray, rank: int, world: int):
    """Returns (local_rows, local_cols, bytes) of `rank`'s shard of one tensor."""
    data = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
    kind = split_kind(name)
    if world == 1 or kind == "none":
        return rows, cols, data
    be, bb = BLOCK_ELEMS[ggml_type], BLOCK_BYTES[ggml_type]
    row_bytes = cols // be * bb
    table = data.reshape(rows, row_bytes)
    if kind == "rows":
        if rows % world:
            raise ValueError(f"{name}: rows do not divide by the world size")
        lr = rows // world
        return lr, cols, np.ascontiguousarray(table[rank * lr:(rank + 1) * lr]).reshape(-1)
    if cols % (world * 32):
        raise ValueError(f"{name}: columns do not split at block boundaries")
    lc = cols // world
    lo = rank * lc // be * bb
    return rows, lc, np.ascontiguousarray(table[:, lo:lo + lc // be * bb]).reshape(-1)
