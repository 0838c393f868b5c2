"""World-size-2 check of the tensor-parallel split on CPU ranks (gloo): row-split projections
concatenate, K-split projections sum under an all-reduce, and a rank's shard is a byte range of
the unmodified GGML tensor (no block is re-encoded)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O
from rustgrad_b200 import quant, tp


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(0)  # same data on every rank
    n, k = 96, 512
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    x = rng.standard_normal((3, k)).astype(np.float32)
    ok = True
    for kind in (quant.Q4_0, quant.Q8_0):
        data = quant.encode(kind, w)
        full = O.quantized_matmul(kind, data, n, k, x)
        # column-parallel (rows of W): every rank owns a slice of the outputs
        lr, lc, part = tp.shard("blk.0.ffn_up.weight", kind, n, k, data, rank, world)
        mine = torch.from_numpy(O.quantized_matmul(kind, part, lr, lc, x))
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        ok &= bool(np.array_equal(torch.cat(gathered, dim=1).numpy(), full))
        # row-parallel (K of W): partial sums all-reduced in rank order
        lr, lc, part = tp.shard("blk.0.ffn_down.weight", kind, n, k, data, rank, world)
        partial = torch.from_numpy(O.quantized_matmul(kind, part, lr, lc, x[:, rank * lc:(rank + 1) * lc]))
        dist.all_reduce(partial)
        ok &= bool(np.abs(partial.numpy() - full).max() <= 1e-5 * max(1.0, float(np.abs(full).max())))
        # the shard is a byte range of the original rows
        bb = quant.BLOCK_BYTES[kind]
        table = data.reshape(n, k // 32 * bb)
        ok &= bool(np.array_equal(part.reshape(n, -1), table[:, rank * (lc // 32) * bb:(rank + 1) * (lc // 32) * bb]))
    # replicated tensors are untouched
    lr, lc, part = tp.shard("blk.0.attn_norm.weight", quant.F32, 1, 8, np.arange(32, dtype=np.uint8), rank, world)
    ok &= (lr, lc, part.size) == (1, 8, 32)
    flag = torch.tensor([int(ok)])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        open(os.path.join(out_dir, "ok"), "w").write(str(int(flag.item())))
    dist.destroy_process_group()


def test_two_rank_split_reproduces_the_unsharded_projection(tmp_path):
    mp.spawn(worker, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok").read_text() == "1"


def test_split_rejects_shapes_that_would_cut_a_block():
    from rustgrad_b200 import session
    data = np.zeros(18 * 3 * 4, np.uint8)
    with pytest.raises(session.UnsupportedGeometry):
        tp.shard("blk.0.ffn_down.weight", quant.Q4_0, 4, 96, data, 0, 2)   # 96 / 2 = 48: not whole blocks
    with pytest.raises(session.UnsupportedGeometry):
        tp.shard("blk.0.attn_q.weight", quant.Q4_0, 3, 128, np.zeros(18 * 4 * 3, np.uint8), 0, 2)
    with pytest.raises(session.UnsupportedGeometry):  # a K-quant super-block holds 256 elements: 512 / 4 cuts one
        tp.shard_range("blk.0.attn_output.weight", quant.Q4_K, 8, 512, 0, 4)


def test_split_ranges_by_name_and_type():
    # rows for the projections that produce heads / hidden units and the head, the contracting axis for
    # the two that consume them, everything else whole
    assert tp.shard_range("blk.3.attn_k.weight", quant.Q8_0, 1024, 4096, 3, 8) == (384, 128, 0, 4096)
    assert tp.shard_range("output.weight", quant.Q8_0, 128256, 4096, 1, 2) == (64128, 64128, 0, 4096)
    assert tp.shard_range("blk.0.ffn_down.weight", quant.Q4_0, 8192, 28672, 5, 8) == (0, 8192, 17920, 3584)
    assert tp.shard_range("blk.0.attn_output.weight", quant.Q4_K, 8, 1024, 1, 4) == (0, 8, 256, 256)
    assert tp.shard_range("token_embd.weight", quant.Q8_0, 100, 64, 1, 2) == (0, 100, 0, 64)
    assert tp.shard_range("blk.0.attn_norm.weight", quant.F32, 1, 64, 1, 2) == (0, 1, 0, 64)
    assert tp.shard_range("blk.0.ffn_up.weight", quant.Q4_0, 96, 512, 0, 1) == (0, 96, 0, 512)
