"""Tensor-parallel session on 2, 4 and 8 GPUs (one process per GPU, NCCL) against the CPU checker and
the single-GPU session.  A case is skipped when fewer devices are visible than it needs.  The
model has 16 query heads over 8 kv heads, so a rank owns 4, 2 or 1 kv heads as the 70B shape does
at the same world sizes."""
import os
import socket

import numpy as np
import pytest

from rustgrad_b200 import quant, synth

pytestmark = pytest.mark.gpu

CFG = synth.scaled(synth.TINY, d_model=1024, n_heads=16, n_kv_heads=8, head_dim=128, ffn_dim=2048, vocab=640, n_layers=2,
                   rope_theta=500000.0, max_context=128)


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, out_dir, fused=True):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    from rustgrad_b200 import session
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    box = [session.nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    tensors = synth.build_tensors(CFG, seed=6, body_type=quant.Q4_0, embed_type=quant.Q8_0, head_type=quant.Q8_0, tied_head=False)
    target = session.CudaSessionTarget(device=rank, kv_f32=True, tp_rank=rank, tp_world=world, nccl_id=box[0],
                                       disable_fused_allreduce=not fused)
    s = session.LlamaCudaPlan.from_tensors(CFG, tensors, target).prepare()
    prompt = synth.prompt_ids(CFG, 11, seed=2)
    logits = [s.prefill_ids(prompt)]
    tok = int(np.argmax(logits[0]))
    ids = [tok]
    for _ in range(6):
        lg, greedy = s.decode([tok], want_logits=True)
        logits.append(lg[0])
        tok = int(greedy[0])
        ids.append(tok)
    np.save(os.path.join(out_dir, f"logits{rank}.npy"), np.stack(logits))
    np.save(os.path.join(out_dir, f"ids{rank}.npy"), np.array(ids))
    ids_loop, _ = s.decode_loop([tok], 5)  # graph replays with the exchange kernel inside
    np.save(os.path.join(out_dir, f"loop{rank}.npy"), ids_loop[:, 0])
    np.save(os.path.join(out_dir, f"peer{rank}.npy"), np.array([s.report()["peer_reduce_launches"]]))
    # a 40-token prompt: exchanges of more than 32 columns go through ncclAllReduce even with the peer kernel on
    s.reset_sequence()
    np.save(os.path.join(out_dir, f"long{rank}.npy"), s.prefill_ids(synth.prompt_ids(CFG, 40, seed=3)))
    dist.barrier()
    s.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_matches_single_gpu_and_cpu_path(tmp_path, world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    from oracle import oracle as O
    from rustgrad_b200 import session
    mp.spawn(worker, args=(world, free_port(), str(tmp_path)), nprocs=world, join=True)
    l0, i0 = np.load(tmp_path / "logits0.npy"), np.load(tmp_path / "ids0.npy")
    for r in range(1, world):  # every rank holds identical logits
        assert np.array_equal(l0, np.load(tmp_path / f"logits{r}.npy")) and np.array_equal(i0, np.load(tmp_path / f"ids{r}.npy"))
    tensors = synth.build_tensors(CFG, seed=6, body_type=quant.Q4_0, embed_type=quant.Q8_0, head_type=quant.Q8_0, tied_head=False)
    oracle = O.OracleModel(CFG, tensors, threads=4)
    prompt = synth.prompt_ids(CFG, 11, seed=2)
    want = [oracle.forward(prompt)]
    ids = [O.select_greedy(want[0])]
    for _ in range(6):
        want.append(oracle.forward([ids[-1]]))
        ids.append(O.select_greedy(want[-1]))
    assert i0.tolist() == ids
    diff = np.abs(l0 - np.stack(want)).max()
    assert diff <= 1e-2 and diff <= 1e-3 * np.abs(np.stack(want)).max() + 1e-6
    single = session.LlamaCudaPlan.from_tensors(CFG, tensors, session.CudaSessionTarget(kv_f32=True)).prepare()
    assert np.abs(single.prefill_ids(prompt) - l0[0]).max() <= 1e-4
    # the partial sums went through the peer-memory kernel, and the graph-replayed loop agrees with the checker
    assert all(np.load(tmp_path / f"peer{r}.npy")[0] > 0 for r in range(world))
    loop_want = []
    t = ids[-1]
    for _ in range(5):
        t = O.select_greedy(oracle.forward([t]))
        loop_want.append(t)
    assert all(np.load(tmp_path / f"loop{r}.npy").tolist() == loop_want for r in range(world))
    oracle.reset()
    long_want = oracle.forward(synth.prompt_ids(CFG, 40, seed=3))
    for r in range(world):
        diff = np.abs(np.load(tmp_path / f"long{r}.npy") - long_want).max()
        assert diff <= 1e-2 and diff <= 1e-3 * np.abs(long_want).max() + 1e-6
    # the same run through NCCL all-reduce + add gives the same logits up to summation order
    nccl_dir = tmp_path / "nccl"
    nccl_dir.mkdir()
    mp.spawn(worker, args=(world, free_port(), str(nccl_dir), False), nprocs=world, join=True)
    assert np.load(nccl_dir / "peer0.npy")[0] == 0
    assert np.abs(np.load(nccl_dir / "logits0.npy") - l0).max() <= 1e-4


def kquant_tensors():
    """Q4_K projections, Q6_K embedding / head / one down projection: random valid super-blocks."""
    rng = np.random.default_rng(7)
    tensors = {}
    for name, rows, cols, is_norm in synth.tensor_inventory(CFG, tied_head=False):
        if is_norm:
            tensors[name] = (quant.F32, 1, cols, np.ones(cols, dtype=np.float32).view(np.uint8))
        else:
            kind = quant.Q6_K if name in ("token_embd.weight", "output.weight", "blk.0.ffn_down.weight") else quant.Q4_K
            tensors[name] = (kind, rows, cols, quant.random_k_blocks(kind, rows * cols // 256, rng, scale=0.05))
    return tensors


def kquant_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    from rustgrad_b200 import session
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    box = [session.nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    target = session.CudaSessionTarget(device=rank, kv_f32=True, tp_rank=rank, tp_world=world, nccl_id=box[0])
    s = session.LlamaCudaPlan.from_tensors(CFG, kquant_tensors(), target).prepare()
    logits = [s.prefill_ids(synth.prompt_ids(CFG, 11, seed=2))]
    tok = int(np.argmax(logits[0]))
    for _ in range(4):
        lg, greedy = s.decode([tok], want_logits=True)
        logits.append(lg[0])
        tok = int(greedy[0])
    np.save(os.path.join(out_dir, f"logits{rank}.npy"), np.stack(logits))
    dist.barrier()
    s.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_k_quant_tensors_shard_at_super_block_boundaries(tmp_path, world):
    """Q4_K / Q6_K projections under tensor parallelism: rows split as for any type, the contracting
    axis of attn_output / ffn_down at 256-element super-blocks (src/sharding.rs:642-667 on the block
    geometry of src/gguf/tensor.rs:88-155)."""
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    from oracle import oracle as O
    mp.spawn(kquant_worker, args=(world, free_port(), str(tmp_path)), nprocs=world, join=True)
    l0 = np.load(tmp_path / "logits0.npy")
    for r in range(1, world):
        assert np.array_equal(l0, np.load(tmp_path / f"logits{r}.npy"))
    oracle = O.OracleModel(CFG, kquant_tensors(), threads=4)
    want = [oracle.forward(synth.prompt_ids(CFG, 11, seed=2))]
    for _ in range(4):
        want.append(oracle.forward([O.select_greedy(want[-1])]))
    want = np.stack(want)
    assert [int(np.argmax(r)) for r in l0] == [O.select_greedy(w) for w in want]
    diff = np.abs(l0 - want).max()
    assert diff <= 1e-2 and diff <= 1e-3 * np.abs(want).max() + 1e-6, (diff, np.abs(want).max())
