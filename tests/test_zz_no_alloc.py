"""The allocation-free decode attention against the ordinary entry point, through the C ABI.

Some users of this library cannot allocate device memory while they run: a host runtime that took
all of its HBM into its own arena when it started, a serving loop where the device-wide stall of a
cudaMalloc is not acceptable, code between the begin and end of a stream capture.  For them the
library keeps the attention's split-context partials in a fixed 4 MiB array of its own.  This test
hands the entry point device buffers it did not allocate (torch tensors) and checks two calls in a
row, with different inputs and sizes, against `rg_b200_attention_decode`, which allocates its
scratch with cudaMalloc.  Tolerance: 1e-6 absolute, the same kernels run in both, so in practice
the results are identical.  The file name sorts last so a run that stops at the first failure has
already been through every other test.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O
from rustgrad_b200 import _lib, session

pytestmark = pytest.mark.gpu


def run_noalloc(q, k, v, ctx):
    import torch
    heads, hd = q.shape
    kv_heads, n_pos, _ = k.shape
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    # caches with `ctx` rows per kv head of which the first n_pos are filled
    kd = torch.zeros((kv_heads, ctx, hd), dtype=torch.from_numpy(k[:0]).dtype, device=dev)
    vd = torch.zeros_like(kd)
    kd[:, :n_pos] = torch.from_numpy(k).to(dev)
    vd[:, :n_pos] = torch.from_numpy(v).to(dev)
    qd = torch.from_numpy(q).to(dev)
    out = torch.full((heads, hd), float("nan"), dtype=torch.float32, device=dev)
    torch.cuda.synchronize()
    rc = _lib.load().rg_b200_attention_decode_noalloc(
        C.c_void_p(qd.data_ptr()), C.c_void_p(kd.data_ptr()), C.c_void_p(vd.data_ptr()), heads, kv_heads, hd, ctx, n_pos,
        int(k.dtype == np.float32), C.c_void_p(out.data_ptr()), None, 1)
    session.check(rc)
    return out.cpu().numpy()


def case(seed, heads, kv_heads, hd, n_pos, dtype):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((heads, hd)).astype(np.float32)
    k = rng.standard_normal((kv_heads, n_pos, hd)).astype(dtype)
    v = rng.standard_normal((kv_heads, n_pos, hd)).astype(dtype)
    return q, k, v


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    # second call is smaller than the first: stale partials of the first call stay in the shared
    # array and must not leak into the result
    for seed, (heads, kv_heads, hd, n_pos, ctx, dtype) in enumerate([(32, 8, 128, 1500, 2048, np.float16),
                                                                      (8, 2, 128, 77, 256, np.float32),
                                                                      (4, 4, 64, 1, 128, np.float16)]):
        q, k, v = case(seed, heads, kv_heads, hd, n_pos, dtype)
        want = session.attention_decode(q, k, v)
        got = run_noalloc(q, k, v, ctx)
        assert np.isfinite(got).all()
        assert np.abs(got - want).max() <= 1e-6, (heads, n_pos)
        # and against the CPU checker's softmax composition (summation order differs: 2e-5)
        ref = O.attention_decode(q, k.astype(np.float32), v.astype(np.float32))
        assert np.abs(got - ref).max() <= 2e-5, (heads, n_pos)


def test_sizes_beyond_the_fixed_array_are_refused():
    import torch
    torch.cuda.set_device(0)
    buf = torch.zeros(16, device="cuda")
    p = C.c_void_p(buf.data_ptr())
    L = _lib.load()
    # 64 heads, 128 dims, ctx 16384: 64 * 128 * 130 = 1 064 960 floats > 1 048 576
    rc = L.rg_b200_attention_decode_noalloc(p, p, p, 64, 8, 128, 16384, 1, 0, p, None, 1)
    assert rc == 20 and b"1048576" in L.rg_b200_last_error()
    assert L.rg_b200_attention_decode_noalloc(p, p, p, 64, 8, 128, 64, 65, 0, p, None, 1) == 1   # n_pos > ctx
    assert L.rg_b200_attention_decode_noalloc(p, p, p, 6, 2, 96, 64, 1, 0, p, None, 1) == 20     # head geometry
    assert L.rg_b200_attention_decode_noalloc(None, p, p, 8, 2, 128, 64, 1, 0, p, None, 1) == 1  # null pointer
    # a cache pointer cut from the middle of an arena at an odd offset would fault the bulk copies
    odd = C.c_void_p(buf.data_ptr() + 4)
    assert L.rg_b200_attention_decode_noalloc(p, odd, p, 8, 2, 128, 64, 1, 0, p, None, 1) == 1
    assert L.rg_b200_attention_decode_noalloc(p, p, odd, 8, 2, 128, 64, 1, 0, p, None, 1) == 1
    assert b"16-byte" in L.rg_b200_last_error()
    assert L.rg_b200_attention_decode_noalloc(C.c_void_p(buf.data_ptr() + 2), p, p, 8, 2, 128, 64, 1, 0, p, None, 1) == 1
