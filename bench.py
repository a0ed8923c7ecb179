#!/usr/bin/env python
"""Headline benchmark: greedy decode tokens/s of the full random-init 4-bit decoder.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...   (N > 1)

A step is one decoded token of BASELINE config 4 (36 layers, hidden 4096, intermediate 12288,
32 x 8 x 128 heads, vocab 151936, all linear layers affine u4 group 64, fp16 embedding and LM
head) after a 512-token seeded prompt; weights are random-init synthetic, drawn per tensor
from seeded streams.  The timed region replays a captured CUDA graph per token on the
library's stream, timed with CUDA events on that stream; every step streams ~5.2 GB of
weights, far more than L2.  N > 1 runs the model tensor-parallel (column-parallel Q/K/V/gate/up,
row-parallel O/down, all-reduce after O and down), so per-GPU work shrinks: strong scaling.

Rank 0 prints ONE JSON line.  --impl reference times the CPU oracle (the port of the
reference's scalar path; the reference itself is Swift + Metal and cannot run here) on the
host's cores for the same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PROMPT_LEN = 512
SEED = 0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.rows, self.proc, self.device_index, self.marks = [], None, device_index, []

    def mark(self):
        """Brackets the timed region: called when it starts and when it ends."""
        self.marks.append(time.time())

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([time.time()] + [c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        # Samples inside the timed region when it is long enough to hold some, else every sample
        # since the warm-up began (the GPU is under the same load there).
        lo, hi = (self.marks[0], self.marks[-1]) if len(self.marks) >= 2 else (0.0, float("inf"))
        inside = [r for r in self.rows if lo <= r[0] <= hi + 0.1]
        rows, window = (inside, "timed region") if len(inside) >= 2 else (self.rows, "warm-up + timed region")
        sm, mx, reasons = [], [], set()
        for r in rows:
            try:
                sm.append(float(r[2])); mx.append(float(r[3]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], r[6:10]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": window}


def token_bytes(cfg, ctx_len: int, batch: int, world: int, vocab_parallel: bool) -> dict:
    """Algorithmic bytes one decoded token moves per GPU: packed weights + scales + biases of every
    linear layer (0.5625 B/weight at group 64), the fp16 LM head (this rank's vocab rows when the
    head is vocab-parallel), and the live KV prefix."""
    per_layer = (cfg.n_q * cfg.head_dim * cfg.hidden * 2 + 2 * cfg.n_kv * cfg.head_dim * cfg.hidden + 3 * cfg.inter * cfg.hidden)
    linear = cfg.layers * per_layer * 0.5625 / world
    head = cfg.vocab * cfg.hidden * 2 / (world if vocab_parallel else 1)
    kv = cfg.layers * 2 * cfg.n_kv * cfg.head_dim * 2 * ctx_len * batch / world
    return {"linear": linear, "lm_head": head, "kv": kv, "total": linear + head + kv}


def setup_dist(n_gpus: int):
    if n_gpus <= 1:
        return 0, 1, None
    import torch
    import torch.distributed as dist

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    return rank, world, dist


GOLDEN = os.path.join(ROOT, "tests", "golden", "full_model_tokens.json")


def parity_check(dec, prompts, args, capacity) -> dict:
    """Teacher-forced replay of the committed known-good tokens (sequence 0; same model, seed and
    prompt) right after the prompt: the fixture's token goes in at every step, the argmax of every
    step is compared.  Runs on every rank, so at N > 1 each GPU's tokens are checked."""
    from smelt_b200 import package

    if not os.path.exists(GOLDEN):
        return {"checked": 0, "note": "fixture missing"}
    with open(GOLDEN) as f:
        gold = json.load(f)
    if gold["seed"] != SEED or gold["prompt_len"] != args.prompt_len or gold["config"] != package.FULL_MODEL.as_dict():
        return {"checked": 0, "note": "no fixture for this prompt length"}
    n = min(gold["n_decode"], capacity - args.prompt_len - 1)
    tokens = np.array(gold["tokens"][:n], np.int32)
    got = np.zeros(n, np.int32)
    cur = dec.graph_decode(1, read=True)[0]  # the prompt's last token was seeded by the caller
    for i in range(n):
        got[i] = cur[0]
        if i + 1 < n:
            feed = np.array(cur, np.int32)
            feed[0] = tokens[i]
            dec.graph_seed(feed, args.prompt_len + i)
            cur = dec.graph_decode(1, read=True)[0]
    v = package.compare_greedy(got, tokens, np.array(gold["runner_up"][:n]), np.array(gold["top2_margin"][:n]))
    v["fixture"] = "tests/golden/full_model_tokens.json"
    return v


def qmv_block(args) -> list:
    """The metric's second half: achieved HBM GB/s of the quantised matvec kernels alone, one
    line per shape: config 0 with its weights resident in L2 and rotating through more copies than
    L2 holds, and the four matvec launches of a config-4 layer (rotating)."""
    from smelt_b200 import kernel_bench

    b = kernel_bench.Bench(reps=10, quiet=True)
    try:
        b.affine("config0 (L2-resident: one weight copy)", 4096, 1024, 1, copies=1)
        b.affine("config0 (HBM: rotating copies > L2)", 4096, 1024, 1)
        b.affine("config4 Q|K|V", 6144, 4096, 1, "matvec")
        b.affine("config4 O + residual", 4096, 4096, 1, "add")
        b.affine("config4 gate/up + SwiGLU", 12288, 4096, 1, "gate_up")
        b.affine("config4 down + residual", 4096, 12288, 1, "add")
    finally:
        b.ctx.close()
    keep = ("config", "kernel", "shape", "batch", "bytes_per_launch", "us_per_launch", "achieved_gbs", "frac_of_peak", "frac_of_8tbs", "distinct_operand_sets")
    return [{k: r[k] for k in keep} for r in b.rows]


def prefill_block(ctx, dec, prompt, args):
    """tok/s of the prompt through ``smelt_cuda_prefill`` (host token ids in, argmax out; wall
    clock around the synchronous call, best of three) in chunks of 512 and 128 positions, and
    whether the token after the prompt is the fixture's."""
    out = {"prompt_len": int(len(prompt)), "unit": "tok/s", "timing": "wall clock around the synchronous call, best of 3"}
    first = None
    for chunk in (512, 128):
        best = None
        for _ in range(3):
            ctx.synchronize()
            t0 = time.perf_counter()
            first = dec.prefill(prompt, 0, chunk)
            dt = time.perf_counter() - t0
            best = dt if best is None or dt < best else best
        out["chunk_%d" % chunk] = {"ms": round(best * 1e3, 3), "tok_s": round(len(prompt) / best, 1),
                                   "launches": int(ctx.lib.smelt_cuda_last_launch_count(ctx.h))}
    gold_path = os.path.join(ROOT, "tests", "golden", "full_model_tokens.json")
    if os.path.exists(gold_path) and args.prompt_len == 512:
        with open(gold_path) as f:
            gold = json.load(f)
        if gold["seed"] == SEED and gold["prompt_len"] == len(prompt):
            ok = first == gold["tokens"][0] or (gold["top2_margin"][0] < 0.02 and first == gold["runner_up"][0])
            out["first_token_matches_fixture"] = bool(ok)
    dec.reset_cache()
    return out


def run_ours(args):
    from smelt_b200 import capi, package

    rank, world, dist = setup_dist(args.gpus)
    local = int(os.environ.get("LOCAL_RANK", 0)) if world > 1 else 0
    cfg = package.FULL_MODEL
    B = args.batch
    capacity = args.prompt_len + max(args.warmup + 2 * args.steps, 64) + 16  # room for the 64-step parity replay
    ctx = capi.Context(local)

    if world > 1:
        import torch

        ident = np.zeros(capi.TP_ID_BYTES, np.uint8)
        if rank == 0:
            st = ctx.lib.smelt_cuda_tp_unique_id(ident.ctypes.data_as(C.c_void_p))
            assert st == 0, "ncclGetUniqueId failed"
        t = torch.from_numpy(ident).cuda()
        dist.broadcast(t, 0)
        ident = t.cpu().numpy()
        ctx._check(ctx.lib.smelt_cuda_tp_init(ctx.h, rank, world, ident.ctypes.data_as(C.c_void_p)))
        if args.collective == "peer":
            package.open_tp_exchange(ctx, dist, world)

    t0 = time.time()
    pkg = package.SyntheticPackage(cfg, SEED)
    keep = rank == 0 and world == 1 and not args.no_cpu_baseline
    peer = world > 1 and args.collective == "peer"
    image, desc, layers = package.build_image(pkg, rank, world, keep_for_oracle=keep, vocab_parallel=peer)
    fuse = (3 if args.table == "fused" else 0) | (12 if peer else 0)  # 4: fused all-reduce + add, 8: vocab-parallel LM head
    dec = package.Decoder(ctx, image, desc, layers, capacity, B, fuse_residual=fuse)
    del image
    dec.build_graph()
    gen_s = time.time() - t0

    prompts = np.stack([np.random.Generator(np.random.Philox(key=[SEED, 1000 + b])).integers(0, cfg.vocab, size=args.prompt_len) for b in range(B)]).astype(np.int32)
    if dist is not None:
        # Ranks finish building their weight shards seconds apart; the exchange's bounded wait is
        # about a second, so every rank waits here until all are ready to decode.
        ctx.synchronize()
        dist.barrier()
    # ── prefill (one GPU, batch 1): the same prompt through smelt_cuda_prefill, timed for the
    # `prefill` block; the token-by-token pass below then overwrites the caches with what the
    # headline measures ──
    prefill = None
    if world == 1 and B == 1 and not args.no_prefill:
        prefill = prefill_block(ctx, dec, prompts[0], args)
    for i in range(args.prompt_len):  # the reference's no-prefill path: one decode step per prompt token
        dec.graph_seed(prompts[:, i], i)
        if i + 1 < args.prompt_len:
            dec.graph_decode(1, read=False)

    def barrier():
        ctx.synchronize()
        if dist is not None:
            dist.barrier()
            ctx.synchronize()

    # ── parity, before anything is timed: the known-good greedy tokens of this model, seed and
    # prompt (a committed fixture written by the CPU restatement of the reference's scalar path)
    # are replayed teacher-forced on every rank and the argmax of every step is compared ──
    parity = parity_check(dec, prompts, args, capacity)
    dec.graph_seed(prompts[:, args.prompt_len - 1], args.prompt_len - 1)  # back to the end of the prompt
    device_error = ctx.device_error_flags()

    ms = C.c_float(0)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # before the warm-up, so that short timed regions still hold samples
    dec.graph_decode(args.warmup, read=False)
    barrier()
    sampler.mark()
    # ── value: K graph replays, inputs resident, CUDA events on the launching stream ──
    ctx.call("timer_start")
    dec.graph_decode(args.steps, read=False)
    ctx._check(ctx.lib.smelt_cuda_timer_stop(ctx.h, C.byref(ms)))
    barrier()
    sampler.mark()
    dev_ms = float(ms.value)
    launches = ctx.lib.smelt_cuda_last_launch_count(ctx.h) * args.steps
    # the ids the timed steps generated (device ring): every rank must hold the same ones
    timed_tokens = np.zeros((min(args.steps, 1024), B), np.int32)
    ctx._check(ctx.lib.smelt_cuda_graph_generated(ctx.h, timed_tokens.shape[0], timed_tokens.ctypes.data_as(C.c_void_p)))
    device_error |= ctx.device_error_flags()

    # ── e2e: K steps through the public graph_step call with host token buffers ──
    pos = args.prompt_len - 1 + args.warmup + args.steps
    cur = np.zeros(B, np.int32)
    out = np.zeros(B, np.int32)
    ctx._check(ctx.lib.smelt_cuda_read_slot(ctx.h, package.ARGMAX_SLOT, 0, cur.ctypes.data_as(C.c_void_p), B * 4))
    barrier()
    t1 = time.perf_counter()
    for i in range(args.steps):
        ctx._check(ctx.lib.smelt_cuda_graph_step(ctx.h, cur.ctypes.data_as(C.c_void_p), pos + i, out.ctypes.data_as(C.c_void_p)))
        cur[:] = out
    barrier()
    e2e_s = time.perf_counter() - t1
    clocks = sampler.stop() if rank == 0 else None
    device_error |= ctx.device_error_flags()

    tokens_match = True
    if dist is not None:
        import torch

        tt = torch.tensor([dev_ms, e2e_s, float(device_error), float(bool(parity.get("wrong")))], device="cuda", dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dev_ms, e2e_s = float(tt[0]), float(tt[1])
        device_error = device_error or int(tt[2])
        parity["all_ranks_ok"] = bool(tt[3] == 0)
        tk = torch.from_numpy(timed_tokens.astype(np.int64)).cuda()
        lo, hi = tk.clone(), tk.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        tokens_match = bool(torch.equal(lo, hi))

    result = None
    if rank == 0:
        peak, peak_kind = measured_peaks()
        tok_s = args.steps * B / (dev_ms / 1e3)
        ctx_len = args.prompt_len + args.warmup + args.steps // 2
        tb = token_bytes(cfg, ctx_len, B, world, peer)
        wptr = C.c_void_p()
        ctx._check(ctx.lib.smelt_cuda_slot_ptr(ctx.h, package.WEIGHTS_SLOT, C.byref(wptr), None))
        base = wptr.value
        tensors = [(base + L.gate.packed, base + L.gate.scales, base + L.gate.biases, base + L.up.packed, base + L.up.scales, base + L.up.biases)
                   for L in (dec.layers[l] for l in range(cfg.layers))]
        roof = kernel_roofline(ctx, tensors, desc.inter, desc.hidden, desc.group, peak, peak_kind)
        result = {
            "metric": "decode tok/s at batch 1 (1/2/4/8 B200); qmv achieved HBM GB/s vs 8 TB/s",
            "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "u4 weights x fp16 activations, fp32 accumulate", "data": "synthetic",
            "config": {"workload": "config4: full 36-layer 4096/12288 decoder, affine u4 g64, greedy decode after a %d-token prompt" % args.prompt_len,
                       "batch": B, "prompt_len": args.prompt_len, "parallelism": f"tp{world}" + (f" ({args.collective} all-reduce)" if world > 1 else ""),
                       "table": args.table + (" (norm+QKV, RoPE+append, O+add, norm+gate/up+SwiGLU, down+add per layer)" if args.table == "fused" else " (the reference emitter's record sequence)"),
                       "l2_policy": "inputs larger than L2: each step streams %.2f GB of weights per GPU" % (tb["total"] / 1e9)},
            "e2e": {"value": args.steps * B / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 4 * B + 4, "d2h_bytes_per_step": 4 * B},
            "gpu_launches": launches,
            "clocks": clocks,
            "parity": parity, "tokens_match_across_ranks": tokens_match, "device_error": device_error,
            "roofline": roof,
            "token_roofline": {"bytes_per_token_per_gpu": tb["total"], "achieved_gbs": tb["total"] / (dev_ms / args.steps / 1e3) / 1e9,
                               "peak_gbs": peak, "frac": tb["total"] / (dev_ms / args.steps / 1e3) / 1e9 / peak, "peak_kind": peak_kind,
                               "frac_of_8tbs": tb["total"] / (dev_ms / args.steps / 1e3) / 1e9 / 8000.0},
            "setup_s": gen_s,
        }
        if prefill is not None:
            result["prefill"] = prefill
        if world == 1 and not args.no_qmv:
            result["qmv"] = qmv_block(args)
        if keep:
            result["cpu_baseline"] = cpu_baseline(pkg, cfg, budget_s=25.0, prompt_len=args.prompt_len)
    if device_error or not tokens_match or parity.get("wrong"):
        # a run whose exchanges timed out, whose ranks disagree or whose tokens are wrong is not a measurement
        if result is not None:
            result["invalid"] = "device_error=%s tokens_match=%s parity_wrong=%s" % (device_error, tokens_match, parity.get("wrong"))
    if result is not None:
        print(json.dumps(result), flush=True)  # before any teardown, so that the line survives whatever follows
    ctx.synchronize()
    if dist is not None:
        dist.barrier()
    dec.ctx = None
    ctx.close()  # graphs, then the communicator
    if dist is not None:
        dist.destroy_process_group()
    return None


# dram__bytes_read.sum + dram__bytes_write.sum of one gate/up launch at the full shape
# (12288 x 4096 x 2), from the ncu capture summarised in profiles/; scaled by the weight bytes
# for other shapes (the traffic is the weight stream).
GATE_UP_TRAFFIC_FULL = 56.77e6


def kernel_roofline(ctx, tensors, I, H, G, peak, peak_kind, reps=6):
    """The dominant kernel alone: the fused gate/up SwiGLU matvec (two [inter, hidden] u4 matrices
    per launch), launched over every layer's weights in turn so that consecutive launches never
    share cached weights (the set is larger than L2), timed with CUDA events on the library's
    stream.  tensors: per layer the six device addresses gate (w, s, b), up (w, s, b)."""
    x = ctx.to_device(np.random.default_rng(1).standard_normal(H).astype(np.float16))
    y = ctx.alloc(I * 2)
    def launch_all():
        for t in tensors:
            ctx.call("affine_gate_up_swiglu", *t, x, y, I, H, G, 1)
    launch_all()  # eager once: sets the kernel attributes
    ctx.synchronize()
    # one pass over every weight set recorded, then replayed between two CUDA events on the
    # library's stream: no host launch overhead inside the timed region
    ctx.call("capture_begin")
    launch_all()
    ctx.call("capture_end")
    ms = C.c_float(0)
    ctx._check(ctx.lib.smelt_cuda_capture_replay(ctx.h, 3, reps, C.byref(ms)))
    ms = C.c_float(ms.value * reps)
    n = reps * len(tensors)
    per_launch_s = ms.value / 1e3 / n
    alg_bytes = 2 * I * H * 0.5625 + H * 2 + I * 2
    achieved = alg_bytes / per_launch_s / 1e9
    traffic = GATE_UP_TRAFFIC_FULL * (I * H) / (12288 * 4096) if GATE_UP_TRAFFIC_FULL else None
    return {"bound": "hbm", "kernel": "affine_imma_kernel<gate_up> (fused_affine_gate_up_swiglu %dx%d x2, u4 g64, batch 1)" % (I, H),
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
            "frac_of_8tbs": achieved / 8000.0, "bytes_per_launch": alg_bytes, "us_per_launch": per_launch_s * 1e6,
            "launches_timed": n, "traffic": traffic,
            "note": "timed alone: a recorded pass over %d distinct weight sets (%.0f MB, larger than L2) replayed back to back" % (len(tensors), len(tensors) * alg_bytes / 1e6)}


def run_kernel_only(args):
    """Only the dominant kernel, on a few layers' worth of synthetic gate/up weights: the small
    case for profiler captures (a few hundred MB on the device)."""
    from smelt_b200 import capi, package, synth

    cfg = package.FULL_MODEL
    I, H, G = cfg.inter, cfg.hidden, 64
    ctx = capi.Context(0)
    tensors = []
    for l in range(args.kernel_layers):
        gate = synth.affine_u4_model(SEED, f"k{l}.gate", I, H, G)
        up = synth.affine_u4_model(SEED, f"k{l}.up", I, H, G)
        tensors.append(tuple(ctx.to_device(a) for a in (*gate, *up)))
    peak, peak_kind = measured_peaks()
    roof = kernel_roofline(ctx, tensors, I, H, G, peak, peak_kind, reps=args.steps)
    ctx.synchronize()
    return {"metric": "qmv achieved HBM GB/s (gate/up kernel alone)", "value": roof["achieved"], "unit": "GB/s", "n_gpus": 1,
            "steps": args.steps, "warmup": 3, "ms_per_step": roof["us_per_launch"] / 1e3, "higher_is_better": True,
            "config": {"workload": "kernel-only: fused gate/up SwiGLU matvec over %d weight sets" % args.kernel_layers},
            "gpu_launches": (args.steps + 3) * args.kernel_layers, "roofline": roof}


def cpu_baseline(pkg, cfg, budget_s: float, prompt_len: int, threads: int | None = None):
    """The oracle (a port of the reference's scalar CPU path) timed on the host's cores on a bounded
    sample of the same workload: greedy decode steps at the GPU arm's context.  The prompt is not
    decoded on the CPU (512 steps would take a quarter of an hour); its KV cache is filled with
    seeded K and V rows of the benchmark's distribution (N(0,1)/sqrt(head_dim)) instead, so every
    timed step streams the same weights and walks the same number of keys as the GPU arm's."""
    import oracle
    from smelt_b200 import synth

    # all the host threads this process may use; a launcher's OMP_NUM_THREADS=1 does not apply
    oracle.set_num_threads(threads or len(os.sched_getaffinity(0)))
    cores = oracle.num_threads()
    max_steps = 24
    m = oracle.model_from_package(pkg, prompt_len + max_steps + 8)
    for l in range(cfg.layers):
        k = synth.kv_cache(SEED, f"cpu_baseline.k{l}", 1, cfg.n_kv, prompt_len, cfg.head_dim)[0]
        v = synth.kv_cache(SEED, f"cpu_baseline.v{l}", 1, cfg.n_kv, prompt_len, cfg.head_dim)[0]
        m.fill_kv(l, k, v)
    rng = np.random.Generator(np.random.Philox(key=[SEED, 1000]))
    tok = int(rng.integers(0, cfg.vocab))
    t0 = time.perf_counter()
    tok = m.decode_step(tok, prompt_len)  # untimed in the result: pages the weights in, sizes the sample
    per = time.perf_counter() - t0
    n = max(1, min(max_steps - 1, int(budget_s / max(per, 1e-3)) - 1))
    t0 = time.perf_counter()
    for i in range(n):
        tok = m.decode_step(int(tok), prompt_len + 1 + i)
    dt = time.perf_counter() - t0
    m.close()
    return {"value": n / dt, "unit": "tok/s", "cores": cores, "kind": "port", "same_config": True,
            "sample": f"{n} greedy decode steps of the full config-4 model at context {prompt_len + 2}..{prompt_len + 1 + n} "
                      f"(KV cache of the {prompt_len}-token prompt filled with seeded N(0,1)/sqrt(d) rows, not decoded), OpenMP over output rows on {cores} threads"}


def run_reference(args):
    """The reference's own CPU path for this workload.  The reference is Swift + Metal and cannot be
    built on Linux, so this arm runs the C port of its scalar oracles on all host threads."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return None
    from smelt_b200 import package

    cfg = package.FULL_MODEL
    pkg = package.SyntheticPackage(cfg, SEED)
    package.build_image(pkg, keep_for_oracle=True)
    base = cpu_baseline(pkg, cfg, budget_s=min(150.0, 6.0 * max(args.steps, 1)), prompt_len=args.prompt_len)
    tok_s = base["value"]
    return {"impl": "reference", "metric": "decode tok/s at batch 1 (1/2/4/8 B200); qmv achieved HBM GB/s vs 8 TB/s",
            "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 / tok_s, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "u4 weights x fp16 activations, fp32 accumulate", "data": "synthetic",
            "config": {"workload": "config4: full 36-layer 4096/12288 decoder, affine u4 g64, greedy decode after a %d-token prompt" % args.prompt_len,
                       "batch": 1, "prompt_len": args.prompt_len, "parallelism": "cpu"},
            "cpu_baseline": base, "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-qmv", action="store_true", help="skip the per-shape matvec bandwidth block (N = 1)")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill timing block (N = 1, batch 1)")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="prompt tokens decoded before the timed region (512 = the headline configuration; smaller for profiler captures)")
    ap.add_argument("--table", default="fused", choices=["fused", "reference"],
                    help="fused: the builder's fused record table; reference: the reference emitter's record sequence")
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="N > 1: all-reduce + residual add as one peer-memory launch, or ncclAllReduce + elementwise_add")
    ap.add_argument("--kernel-only", action="store_true", help="time only the dominant kernel on a few synthetic weight sets (profiler captures)")
    ap.add_argument("--kernel-layers", type=int, default=6)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.kernel_only:
        result = run_kernel_only(args)
    else:
        result = run_reference(args) if args.impl == "reference" else run_ours(args)
    if result is not None:
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
