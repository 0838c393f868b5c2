"""The tensor-parallel split of the CUDA runtime, for tests and tools: ``rg_b200_tp_shard`` gives the
rank's row and column range (the rule the library applies when a tensor is added to a plan of a
tensor-parallel rank), and the shard is cut out of the unmodified GGML bytes here.

Megatron-style: Q/K/V, gate/up and the vocabulary head are split by output rows (a contiguous
byte range of the GGML tensor), attention-output and down projections along K at block boundaries
(a per-row range of whole blocks), so no block is ever re-encoded.  A contracting-axis split needs
a sum all-reduce (src/sharding.rs:642-667); partial sums are combined in rank order
(src/sharded_graph.rs:715-724).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .quant import BLOCK_BYTES, BLOCK_ELEMS
from .session import check


def shard_range(name: str, ggml_type: int, rows: int, cols: int, rank: int, world: int):
    """(row0, n_rows, col0, n_cols) of `rank`'s share, from the library."""
    out = [C.c_uint64() for _ in range(4)]
    check(_lib.load().rg_b200_tp_shard(name.encode(), ggml_type, rows, cols, rank, world, *[C.byref(o) for o in out]))
    return tuple(o.value for o in out)


def shard(name: str, ggml_type: int, rows: int, cols: int, data: np.ndarray, rank: int, world: int):
    """Returns (local_rows, local_cols, bytes) of `rank`'s shard of one tensor."""
    data = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
    r0, lr, c0, lc = shard_range(name, ggml_type, rows, cols, rank, world)
    be, bb = BLOCK_ELEMS[ggml_type], BLOCK_BYTES[ggml_type]
    table = data.reshape(rows, cols // be * bb)
    return lr, lc, np.ascontiguousarray(table[r0:r0 + lr, c0 // be * bb:(c0 + lc) // be * bb]).reshape(-1)
