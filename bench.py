"""Decode-throughput benchmark of the GGUF-quantized Llama session (one JSON line on stdout).

    python bench.py --gpus 1 --steps 256 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...        # the CPU restatement of the reference path
    python bench.py --workload gemv [--shapes 14336x4096 --types q4_0 --batches 1]   # isolated GEMV sweep
    python bench.py --workload gemm [--shapes 14336x4096 --tokens 2048 --modes 0,2]  # prefill GEMM sweep
    python bench.py --workload serving [--requests 16 --batch 8 --prompt-tokens 128 --new-tokens 64]  # continuous batching

A step is one greedy decode step (one new token per row) of a seeded synthetic model:
  * N = 1: Llama-3-8B shape, Q4_0 projections, Q8_0 embedding and head, f16 KV cache, batch 1,
    decoded after a 2048-token prefill;
  * N > 1: Llama-3-70B shape, all Q4_0, tensor-parallel over N GPUs (strong scaling).
`value` times K replays of the decode graph with the selected token fed back on the device
(inputs resident in HBM); `e2e` times K calls of the session's decode verb with host tokens in
and host ids out.  The weights (4.5 GB / 39 GB) are far larger than L2, so every step reads HBM.
At N > 1 a two-layer model of the 70B width first runs through the tensor-parallel session and is
compared with the CPU checker and the single-GPU session (`tp_parity`; a mismatch exits non-zero).
At N = 1 the line also carries the 70B shape on one GPU (`scale_anchor`), the point the N > 1
lines scale from.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402

from rustgrad_b200 import quant, synth  # noqa: E402

PREFILL = 2048
# (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes of one integer-GEMV launch, from
# the ncu captures summarised in profiles/: 33.112 MB / 33.104 MB on Q4_0 [14336, 4096] and
# 580.1 MB / 558.7 MB on Q8_0 [128256, 4096].  DRAM traffic grows in proportion to the bytes a launch
# streams, so the traffic of the average launch of a step is its algorithmic bytes times this ratio.
NCU_TRAFFIC_OVER_ALGORITHMIC = {"q4_0": 1.000, "q8_0": 1.038}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        peaks = json.loads(path.read_text())
        return float(peaks["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def workload(n_gpus: int):
    if n_gpus == 1:
        return dict(name="llama3_8b_shape_q4_0_decode_b1", cfg=dict(synth.LLAMA_8B), seed=6, body=quant.Q4_0, embed=quant.Q8_0,
                    head=quant.Q8_0)
    return dict(name=f"llama3_70b_shape_q4_0_decode_b1_tp{n_gpus}", cfg=dict(synth.LLAMA_70B), seed=7, body=quant.Q4_0,
                embed=quant.Q4_0, head=quant.Q4_0)


def gemv_bytes_per_step(cfg: dict, wl: dict, tp: int, batch: int):
    """Algorithmic bytes of the quantized GEMV launches of one decode step on one rank:
    packed weight bytes + f32 activations in + f32 results out (N*K*18/32 + 4*B*K + 4*B*N)."""
    d, f, hd = cfg["d_model"], cfg["ffn_dim"], cfg["head_dim"]
    qw, kw = cfg["n_heads"] * hd // tp, cfg["n_kv_heads"] * hd // tp
    fl = f // tp

    def one(n, k, t):
        return n * k * quant.BLOCK_BYTES[t] // 32 + 4 * batch * k + 4 * batch * n

    body = wl["body"]
    layer = one(qw + 2 * kw, d, body) + one(d, qw, body) + one(2 * fl, d, body) + one(d, fl, body)
    head = one(cfg["vocab"] // tp, d, wl["head"])
    launches = 4 * cfg["n_layers"] + 1
    return cfg["n_layers"] * layer + head, launches


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.proc = device, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.device)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.summary = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.proc:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            self.summary = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                            "samples": len(sm)}


def random_blocks(rng, kind, n, k):
    """Random block bytes with a sane f16 scale: as good as encoded weights for timing."""
    w = rng.integers(0, 256, (n * k // 32, quant.BLOCK_BYTES[kind]), dtype=np.uint8)
    w[:, 1] = 0x20
    return w.reshape(-1)


def cpu_reference_arm(args, wl, threads, context):
    """Times the CPU restatement of the reference path on a bounded sample of the workload.

    One decode token costs t_head + L * t_layer.  The sample runs the full-width model with 1 and
    with 3 layers and an eighth of the vocabulary rows in embedding and head, takes
    t_layer = (T3 - T1) / 2 and t_head = 8 * (T1 - t_layer), and scales to the model's layer count.
    The decode steps run at the GPU arm's context: the checker's KV cache is filled to `context`
    positions with seeded values first, so attention reads as many rows as on the GPU.  Weights are
    random block bytes with a sane scale (the time of the CPU path does not depend on the values).
    """
    from oracle import oracle as O
    cfg = wl["cfg"]
    steps = max(1, min(args.steps, 3))
    vocab_div = 8
    rng = np.random.default_rng(wl["seed"])
    sub3 = synth.scaled(cfg, n_layers=3, max_context=context + steps + 8, vocab=cfg["vocab"] // vocab_div)
    tensors3 = {}
    for name, rows, cols, is_norm in synth.tensor_inventory(sub3, tied_head=False):
        if is_norm:
            tensors3[name] = (quant.F32, 1, cols, np.ones(cols, dtype=np.float32).view(np.uint8))
        else:
            kind = wl["embed"] if name == "token_embd.weight" else wl["head"] if name == "output.weight" else wl["body"]
            tensors3[name] = (kind, rows, cols, random_blocks(rng, kind, rows, cols))
    times = {}
    for layers in (1, 3):
        sub = synth.scaled(sub3, n_layers=layers)
        keep = {k: v for k, v in tensors3.items() if not k.startswith("blk.") or int(k.split(".")[1]) < layers}
        m = O.OracleModel(sub, keep, kv_f16=True, threads=threads)
        m.fill_cache_seeded(context, seed=1)
        m.forward([1], O.MODE_FAST)  # warm-up step
        t0 = time.perf_counter()
        for i in range(steps):
            m.forward([2 + i], O.MODE_FAST)
        times[layers] = (time.perf_counter() - t0) / steps
        m.close()
    t_layer = max((times[3] - times[1]) / 2.0, 1e-9)
    t_head = max(times[1] - t_layer, 0.0) * vocab_div
    t_token = t_head + cfg["n_layers"] * t_layer
    sample = (f"{steps} decode steps at context {context} each of a 1-layer and a 3-layer full-width model with "
              f"vocab/{vocab_div} rows, scaled to {cfg['n_layers']} layers and the full vocabulary")
    return 1.0 / t_token, t_token, sample


GGML = {"q4_0": quant.Q4_0, "q8_0": quant.Q8_0}


def op_sweep(args):
    """Isolated kernels on one GPU, one JSON line per case (the second and third benchmark
    configurations: quantized GEMV at B in {1,2,4,8}, prefill GEMM at M in {128,512,2048})."""
    from rustgrad_b200 import session
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    tflops = float(peaks.get("bf16_tflops", 1590.0))
    rng = np.random.default_rng(2)
    shapes = [tuple(int(v) for v in sh.split("x")) for sh in args.shapes.split(",")]
    for name in args.types.split(","):
        kind = GGML[name]
        for n, k in shapes:
            w = random_blocks(rng, kind, n, k)
            if args.workload == "gemv":
                rotate = max(2, int(600e6 // w.size) + 1)  # distinct weight copies in turn: every launch reads HBM
                for b in (int(v) for v in args.batches.split(",")):
                    x = rng.standard_normal((b, k)).astype(np.float32)
                    _, ms = session.qmatmul_bench(kind, w, n, k, x, rotate=rotate, iters=args.iters, warmup=args.op_warmup)
                    nbytes = w.size + 4 * b * k + 4 * b * n
                    print(json.dumps({"op": "qgemv", "type": name, "n": n, "k": k, "batch": b, "us": ms * 1e3,
                                      "algorithmic_bytes": nbytes, "gbs": nbytes / ms / 1e6,
                                      "frac_of_measured_hbm": nbytes / ms / 1e6 / hbm}), flush=True)
            else:
                for m in (int(v) for v in args.tokens.split(",")):
                    x = rng.standard_normal((m, k)).astype(np.float32)
                    for mode in (int(v) for v in args.modes.split(",")):
                        _, ms = session.qgemm(kind, w, n, k, x, iters=args.iters, operand_mode=mode)
                        fl = 2.0 * m * n * k
                        print(json.dumps({"op": "qgemm", "type": name, "n": n, "k": k, "tokens": m,
                                          "operands": ["bf16", "f16", "f16 hi+lo (3 products)"][mode], "us": ms * 1e3,
                                          "tflops": fl / ms / 1e9, "frac_of_measured_bf16_burst": fl / ms / 1e9 / tflops,
                                          "tensor_work_frac": fl * (3 if mode == 2 else 1) / ms / 1e9 / tflops}), flush=True)


def serving_run(args):
    """Continuous batching on the 8B shape, one GPU: `requests` prompts that share a prefix arrive
    at once, `batch` of them run per step; wall-clock tokens/s of the whole job through the
    scheduler (host tokens in, host tokens out), with and without the prefix cache."""
    from rustgrad_b200 import serving, session
    cfg = dict(synth.LLAMA_8B)
    B = max(1, min(args.batch if args.batch > 1 else 8, 32))
    target = session.CudaSessionTarget(max_batch=B, max_context=args.prompt_tokens + args.new_tokens + 8)
    s = session.LlamaCudaPlan.synthetic(cfg, target, seed=6).prepare()
    shared = synth.prompt_ids(cfg, args.shared_prefix, seed=11).tolist()
    prompts = [shared + synth.prompt_ids(cfg, args.prompt_tokens - args.shared_prefix, seed=100 + r).tolist()
               for r in range(args.requests)]
    for label, entries in (("no prefix cache", 0), ("prefix cache", 64)):
        sched = serving.LlamaServingScheduler(s, batch_size=B, prefix_max_entries=entries, prefix_max_bytes=8 << 30)
        if entries:  # the shared prefix is resident before the requests arrive
            warm = sched.submit_ids(shared, serving.GenerationConfig(1))
            while sched.pending():
                sched.step()
            sched.remove(warm)
        t0 = time.perf_counter()
        ids = [sched.submit_ids(p, serving.GenerationConfig(args.new_tokens)) for p in prompts]
        steps = 0
        while sched.pending():
            sched.step()
            steps += 1
        dt = time.perf_counter() - t0
        generated = sum(len(sched.result(i).generated_ids) for i in ids)
        print(json.dumps({"op": "serving", "config": label, "requests": args.requests, "batch": B,
                          "prompt_tokens": args.prompt_tokens, "shared_prefix": args.shared_prefix,
                          "new_tokens": args.new_tokens, "steps": steps, "seconds": dt,
                          "generated_tokens_per_s": generated / dt,
                          "prompt_and_generated_tokens_per_s": (generated + args.requests * args.prompt_tokens) / dt,
                          "prefix": sched.prefix_stats()}), flush=True)


def tp_parity_check(n, rank, local_rank, dist, threads):
    """Two layers of the 70B width (d 8192, 64 / 8 heads, ffn 28672, Q4_0, a quarter of the
    vocabulary) through the tensor-parallel session: a 16-token prompt and 4 decode steps.  Rank 0
    compares its logits with the CPU checker and with the single-GPU session on the same bytes;
    every rank's greedy ids must equal rank 0's.  Returns the `tp_parity` object (on every rank)."""
    import torch
    from rustgrad_b200 import session
    cfg = synth.scaled(synth.LLAMA_70B, n_layers=2, max_context=64, vocab=32064)
    box = [session.nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    target = session.CudaSessionTarget(device=local_rank, tp_rank=rank, tp_world=n, nccl_id=box[0], max_context=64)
    sess = session.LlamaCudaPlan.synthetic(cfg, target, seed=7, body_type=quant.Q4_0, embed_type=quant.Q4_0,
                                           head_type=quant.Q4_0).prepare()
    prompt = synth.prompt_ids(cfg, 16, seed=1)
    logits = [sess.prefill_ids(prompt)]
    ids = [int(np.argmax(logits[0]))]
    for _ in range(4):
        lg, greedy = sess.decode([ids[-1]], want_logits=True)
        logits.append(lg[0])
        ids.append(int(greedy[0]))
    fused = sess.report().get("peer_reduce_launches", 0) > 0
    sess.close()
    mine = torch.tensor(ids, dtype=torch.int64, device="cuda")
    everyone = [torch.empty_like(mine) for _ in range(n)]
    dist.all_gather(everyone, mine)
    ids_equal = all(bool((t == everyone[0]).all()) for t in everyone)
    out = {"world": n, "layers": 2, "width": "llama3_70b", "prompt_tokens": 16, "decode_steps": 4, "ids_equal": ids_equal,
           "exchange": "peer-memory kernel" if fused else "nccl all-reduce + add"}
    verdict = torch.zeros(3, dtype=torch.float64, device="cuda")
    if rank == 0:
        from oracle import oracle as O
        single_target = session.CudaSessionTarget(device=local_rank, max_context=64)
        plan = session.LlamaCudaPlan.synthetic(cfg, single_target, seed=7, body_type=quant.Q4_0, embed_type=quant.Q4_0,
                                               head_type=quant.Q4_0)
        tensors = {}
        for name, rows, cols, is_norm in synth.tensor_inventory(cfg, tied_head=False):
            tensors[name] = (quant.F32 if is_norm else quant.Q4_0, rows, cols, plan.read_tensor(name))
        single = plan.prepare()
        oracle = O.OracleModel(cfg, tensors, kv_f16=True, threads=threads)
        want = [oracle.forward(prompt, O.MODE_FAST)]
        one = [single.prefill_ids(prompt)]
        want_ids = [O.select_greedy(want[0])]
        for _ in range(4):
            want.append(oracle.forward([want_ids[-1]], O.MODE_FAST))
            one.append(single.decode([want_ids[-1]], want_logits=True)[0][0])
            want_ids.append(O.select_greedy(want[-1]))
        oracle.close()
        single.close()
        got, want, one = np.stack(logits), np.stack(want), np.stack(one)
        max_abs = float(np.abs(got - want).max())
        ok = ids == want_ids and max_abs <= 1e-2 and max_abs <= 1e-3 * float(np.abs(want).max()) + 1e-6
        verdict = torch.tensor([max_abs, float(np.abs(got - one).max()), float(ok)], dtype=torch.float64, device="cuda")
    dist.broadcast(verdict, src=0)
    out.update({"max_abs": float(verdict[0]), "max_abs_vs_single_gpu": float(verdict[1]), "bar": "1e-2 abs, 1e-3 of max |logit|",
                "ids_equal_checker": bool(verdict[2] > 0.5) and ids_equal, "ok": bool(verdict[2] > 0.5) and ids_equal})
    return out


def scale_anchor(args, local_rank):
    """The 70B shape (all Q4_0, 39 GB) on ONE GPU: decode tokens/s after a 2048-token prefill, the
    point the tensor-parallel lines at N = 2, 4, 8 scale from."""
    from rustgrad_b200 import session
    wl = workload(2)
    cfg = wl["cfg"]
    steps = max(8, min(args.steps, 32))
    target = session.CudaSessionTarget(device=local_rank, max_batch=1)
    sess = session.LlamaCudaPlan.synthetic(cfg, target, seed=wl["seed"], body_type=wl["body"], embed_type=wl["embed"],
                                           head_type=wl["head"]).prepare()
    logits = sess.prefill_ids(synth.prompt_ids(cfg, min(args.prefill, 2048), seed=1))
    prefill_ms = sess.report()["last_prefill_ms"]
    ids, _ = sess.decode_loop([int(np.argmax(logits))], 3)
    ids, gpu_ms = sess.decode_loop([int(ids[-1][0])], steps)
    sess.close()
    gemv_bytes, _ = gemv_bytes_per_step(cfg, wl, 1, 1)
    ms = gpu_ms / steps
    return {"workload": "llama3_70b_shape_q4_0_decode_b1_tp1", "value": steps / (gpu_ms * 1e-3), "unit": "tokens/s",
            "ms_per_step": ms, "steps": steps, "prefill_ms": prefill_ms,
            "step_bytes_over_step_time_gbs": gemv_bytes / (ms * 1e-3) / 1e9}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="decode", choices=["decode", "gemv", "gemm", "serving"])
    ap.add_argument("--requests", type=int, default=16)
    ap.add_argument("--prompt-tokens", type=int, default=128)
    ap.add_argument("--new-tokens", type=int, default=64)
    ap.add_argument("--shared-prefix", type=int, default=96, help="leading prompt tokens every request shares")
    ap.add_argument("--shapes", default="4096x4096,14336x4096,4096x14336,128256x4096")
    ap.add_argument("--types", default="q4_0,q8_0")
    ap.add_argument("--batches", default="1,2,4,8")
    ap.add_argument("--tokens", default="128,512,2048")
    ap.add_argument("--modes", default="0,1,2")
    ap.add_argument("--iters", type=int, default=40)
    ap.add_argument("--op-warmup", type=int, default=5)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--prefill", type=int, default=PREFILL)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-tp-parity", action="store_true", help="skip the tensor-parallel parity check at N > 1")
    ap.add_argument("--no-scale-anchor", action="store_true", help="skip the 70B single-GPU figure at N = 1")
    ap.add_argument("--batch", type=int, default=1, help="rows decoded together (the headline workload is 1)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.workload == "serving":
        return serving_run(args)
    if args.workload != "decode":
        return op_sweep(args)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    n = args.gpus
    wl = workload(n)
    cfg = wl["cfg"]
    threads = os.cpu_count() or 1

    prefill = min(args.prefill, cfg["max_context"] - 2 * (args.steps + args.warmup) - 80)

    if args.impl == "reference":
        if rank != 0:
            return
        tok_s, t_token, sample = cpu_reference_arm(args, wl, threads, prefill + args.warmup)
        line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": n,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_token * 1e3, "higher_is_better": True,
                "scaling": "weak" if n == 1 else "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": wl["name"], "batch": 1, "prefill_tokens": prefill, "context": prefill + args.warmup,
                           "kv_cache": "f16", "weights": "Q4_0 body, Q8_0 embedding+head" if n == 1 else "Q4_0",
                           "parallelism": "host cores"},
                "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
                "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    import torch
    from rustgrad_b200 import session
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: rustgrad_b200 has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dist = None
    nccl_id = b""
    if n > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # keep stdout to the one JSON line
        if world != n:
            raise SystemExit(f"--gpus {n} needs torchrun with {n} ranks (WORLD_SIZE={world})")
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        box = [session.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        nccl_id = box[0]

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    B = args.batch
    parity = None
    if n > 1 and not args.no_tp_parity:
        parity = tp_parity_check(n, rank, local_rank, dist, threads)
        if not parity["ok"]:
            if rank == 0:
                print(json.dumps({"tp_parity": parity}))
            dist.destroy_process_group()
            raise SystemExit("tensor-parallel parity check failed")
    target = session.CudaSessionTarget(device=local_rank, max_batch=B, tp_rank=rank if n > 1 else 0, tp_world=n, nccl_id=nccl_id)
    plan = session.LlamaCudaPlan.synthetic(cfg, target, seed=wl["seed"], body_type=wl["body"], embed_type=wl["embed"],
                                           head_type=wl["head"])
    sess = target.prepare(plan)
    first = []
    for r in range(B):  # every row gets its own prompt of the same length
        logits = sess.prefill_ids(synth.prompt_ids(cfg, prefill, seed=1 + r), row=r)
        first.append(int(np.argmax(logits)))
    prefill_ms = sess.report()["last_prefill_ms"]

    # ---- device-resident loop: W warm-up steps, then exactly K timed steps
    ids, _ = sess.decode_loop(first, args.warmup)
    tok = [int(v) for v in ids[-1]]
    r0 = sess.report()
    barrier()
    with ClockSampler(local_rank) as clocks:
        ids, gpu_ms = sess.decode_loop(tok, args.steps)
        torch.cuda.synchronize()
    barrier()
    r1 = sess.report()
    tok = [int(v) for v in ids[-1]]
    launches = r1["kernel_launches"] - r0["kernel_launches"]

    # ---- end to end through the decode verb: host token in, host id out, every step
    for _ in range(3):
        _, g = sess.decode(tok)
        tok = [int(v) for v in g]
    r2 = sess.report()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        _, g = sess.decode(tok)
        tok = [int(v) for v in g]
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()
    r3 = sess.report()

    # ---- profiling pass: CUDA events between kernel families (serialized, no overlap)
    prof = sess.decode_profile(tok, 16, in_step=True)   # launch attributes as in the timed step
    prof_serial = sess.decode_profile(tok, 16)          # every kernel alone, no overlap
    prof_sites = sess.decode_profile_projections(tok, 16) if B <= 2 else None
    position = sess.position()

    t = torch.tensor([gpu_ms, e2e_s * 1e3], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    gpu_ms, e2e_ms = float(t[0]), float(t[1])
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peaks()
    gemv_bytes, gemv_launches = gemv_bytes_per_step(cfg, wl, n, B)
    proj_kernel = ("qgemv_i8_kernel" if B <= 2 else "qgemv_kernel" if B <= 16 else "qgemm_tc_kernel") + " (all projection launches of a step)"
    gemv_ms = prof["gemv"]["ms_per_step"]
    achieved = gemv_bytes / (gemv_ms * 1e-3) / 1e9 if gemv_ms > 0 else None
    ms_per_step = gpu_ms / args.steps
    line = {
        "metric": "decode_tokens_per_s", "value": B * args.steps / (gpu_ms * 1e-3), "unit": "tokens/s", "n_gpus": n,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak" if n == 1 else "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl["name"].replace("_b1", f"_b{B}"), "batch": B, "prefill_tokens": prefill, "context_at_end": position,
                   "kv_cache": "f16", "weights": "Q4_0 body, Q8_0 embedding+head" if n == 1 else "Q4_0",
                   "parallelism": "single GPU" if n == 1 else f"tp{n}", "l2": "inputs larger than L2 (weights >> 126 MB)",
                   "prefill_ms": prefill_ms},
        "e2e": {"value": B * args.steps / (e2e_ms * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": (r3["h2d_bytes"] - r2["h2d_bytes"]) / args.steps,
                "d2h_bytes_per_step": (r3["d2h_bytes"] - r2["d2h_bytes"]) / args.steps},
        "gpu_launches": launches,
        "clocks": clocks.summary,
        "roofline": {"bound": "hbm", "kernel": proj_kernel, "achieved": achieved,
                     "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak if achieved else None,
                     "traffic": gemv_bytes / gemv_launches * NCU_TRAFFIC_OVER_ALGORITHMIC["q4_0"],
                     "traffic_note": ("not measured in this run: algorithmic bytes of the average GEMV launch x the "
                                      "dram/algorithmic ratio (1.000) of the ncu capture summarised under profiles/"),
                     "launches_per_step": gemv_launches,
                     "algorithmic_bytes_per_step": gemv_bytes, "kernel_ms_per_step": gemv_ms,
                     "kernel_ms_per_step_serialized": prof_serial["gemv"]["ms_per_step"],
                     "timing": ("CUDA events around 16 replays of the step's GEMV launches alone, with the dependent-launch "
                                "edges they have inside the step; `..._serialized` is the same without any overlap"),
                     "step_bytes_over_step_time_gbs": (gemv_bytes / (ms_per_step * 1e-3) / 1e9)},
        "profile_ms_per_step": {k: v["ms_per_step"] for k, v in prof.items()},
        "profile_ms_per_step_serialized": {k: v["ms_per_step"] for k, v in prof_serial.items()},
        "gemv_ms_per_step_by_projection": prof_sites,
    }
    if n > 1:
        # tensor parallel: what the exchange of partial sums costs (the "other" family is the 160 exchanges plus
        # embedding, selection and the logits all-gather) and what each GPU streams
        line["tensor_parallel"] = {
            "exchange": "peer-memory kernel" if r1.get("peer_reduce_launches", 0) > 0 else "nccl all-reduce + add",
            "exchange_and_other_ms_per_step": prof["other"]["ms_per_step"],
            "exchange_and_other_share": prof["other"]["ms_per_step"] / prof["total"]["ms_per_step"],
            "per_gpu_projection_gbs": achieved,
        }
    if parity is not None:
        line["tp_parity"] = parity
    if B > 16 and n == 1:
        line["profile_note"] = ("the timed steps run as equal chunks of at most 16 rows; `roofline` and `profile_ms_per_step` "
                                "describe ONE step over all rows on the 17..32-row path (RG_B200_WIDE_DECODE_ONE_STEP=1 times that)")
    if not args.no_cpu_baseline:
        tok_s, t_token, sample = cpu_reference_arm(args, wl, threads, prefill + args.warmup)
        line["cpu_baseline"] = {"value": tok_s, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample}
    if n == 1 and B == 1 and not args.no_scale_anchor:
        sess.close()
        line["scale_anchor"] = scale_anchor(args, local_rank)
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
