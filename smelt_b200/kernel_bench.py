"""Per-kernel bandwidth of the decode kernels at the benchmark configurations.

    python -m smelt_b200.kernel_bench [--configs 0,1,2,3,4] [--reps 20] [--markdown] [--only CASE]

Every case launches its kernel over enough distinct copies of its weights (or KV caches) to
exceed the 126 MB L2, records one pass over all copies with smelt_cuda_capture_begin / _end
and replays it between CUDA events, so a launch never finds its operands cached and no host
launch overhead is inside the timed region.  One JSON line per case: algorithmic bytes per
launch (packed weights + scales + biases + activations in and out), microseconds per launch,
achieved GB/s and its fraction of the measured copy bandwidth (MEASURED_PEAKS.json).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os

import numpy as np

from . import capi, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
L2_BYTES = 126e6
TARGET_BYTES = 320e6  # per case: copies * bytes >= this (2.5 x L2)


def measured_peak() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def copies_for(nbytes: float, cap: int = 128) -> int:
    return int(max(1, min(cap, np.ceil(TARGET_BYTES / nbytes))))


class Bench:
    def __init__(self, reps: int, only: str = "", quiet: bool = False):
        self.ctx = capi.Context(0)
        self.reps = reps
        self.quiet = quiet  # collect rows without printing them
        self.only = only  # substring of a case label: run only the affine / attention cases it matches
        self.peak, self.peak_kind = measured_peak()
        self.rows: list[dict] = []

    def dev_copies(self, arrays, n):
        """n device copies of each host array (same content, distinct addresses)."""
        return [[self.ctx.to_device(a) for a in arrays] for _ in range(n)]

    def run(self, config: str, kernel: str, shape: str, batch: int, alg_bytes: float, launches: int, enqueue, flops: float = 0.0):
        ctx = self.ctx
        enqueue()  # eager once: validates arguments, sets kernel attributes
        ctx.synchronize()
        ctx.call("capture_begin")
        enqueue()
        ctx.call("capture_end")
        ms = C.c_float(0)
        ctx._check(ctx.lib.smelt_cuda_capture_replay(ctx.h, 3, self.reps, C.byref(ms)))
        us = ms.value * 1e3 / launches
        gbs = alg_bytes / (us * 1e-6) / 1e9
        row = {"config": config, "kernel": kernel, "shape": shape, "batch": batch, "bytes_per_launch": alg_bytes,
               "us_per_launch": round(us, 3), "achieved_gbs": round(gbs, 1), "frac_of_peak": round(gbs / self.peak, 4),
               "peak_gbs": self.peak, "peak_kind": self.peak_kind, "frac_of_8tbs": round(gbs / 8000.0, 4),
               "launches_timed": launches * self.reps, "distinct_operand_sets": launches}
        if flops:  # multiply-adds x 2 of the contraction: what the tensor pipe is asked for at large batch
            row["tflops"] = round(flops / (us * 1e-6) / 1e12, 2)
        self.rows.append(row)
        if not self.quiet:
            print(json.dumps(row), flush=True)

    # ── affine u4 family ──
    def affine(self, config, rows, cols, batch, mode="matvec", copies=None):
        ctx, G = self.ctx, 64
        if self.only and self.only not in f"{mode} {rows}x{cols} b{batch}":
            return
        nmat = 2 if mode in ("gate_up", "dual") else 1
        alg = nmat * rows * cols * 0.5625 + batch * cols * 2 + batch * rows * 2 * (2 if mode == "dual" else 1) + (batch * rows * 2 if mode == "add" else 0)
        n = copies or copies_for(alg)
        host = synth.affine_u4(0, f"kb{rows}x{cols}", rows, cols, G)
        sets = self.dev_copies(host * nmat, n)
        x = ctx.to_device(synth.activations(0, "kbx", batch, cols))
        y, y2 = ctx.alloc(batch * rows * 2), ctx.alloc(batch * rows * 2)
        def enqueue():
            for s in sets:
                if mode == "matvec":
                    ctx.call("affine_matvec", *s, x, y, rows, cols, G, batch)
                elif mode == "add":
                    ctx.call("affine_matvec_add", *s, x, y2, y, rows, cols, G, batch)
                elif mode == "gate_up":
                    ctx.call("affine_gate_up_swiglu", *s, x, y, rows, cols, G, batch)
                else:
                    ctx.call("affine_dual_matvec", *s, x, y, y2, rows, cols, G, batch)
        name = {"matvec": "affine_matvec", "add": "fused_affine_matvec_add", "gate_up": "fused_affine_gate_up_swiglu", "dual": "fused_dual_affine_matvec"}[mode]
        self.run(config, name, f"{rows}x{cols}" + (" x2" if nmat == 2 else ""), batch, alg, n, enqueue, flops=2.0 * nmat * rows * cols * batch)
        for s in sets:
            for b in s:
                b.free()
        for b in (x, y, y2):
            b.free()

    def layer_set(self, config, hidden, inter, n_q, n_kv, d, batch, layers=8):
        """Q, K|V, O(+residual), gate/up+SwiGLU, down(+residual) of one decoder layer, back to back."""
        ctx, G = self.ctx, 64
        qd, kvd = n_q * d, n_kv * d
        shapes = {"q": (qd, hidden), "k": (kvd, hidden), "v": (kvd, hidden), "o": (hidden, qd), "gate": (inter, hidden), "up": (inter, hidden), "down": (hidden, inter)}
        host = {k: synth.affine_u4(1, f"ls{k}", r, c, G) for k, (r, c) in shapes.items()}
        wbytes = sum(r * c for r, c in shapes.values()) * 0.5625
        act = batch * 2 * (3 * hidden + 2 * qd + 2 * kvd + 2 * inter + 4 * hidden)
        sets = [{k: [ctx.to_device(a) for a in v] for k, v in host.items()} for _ in range(layers)]
        xh, xq, xi = (ctx.to_device(synth.activations(1, n, batch, c)) for n, c in (("xh", hidden), ("xq", qd), ("xi", inter)))
        yq, yk, yv, yh, yi = (ctx.alloc(batch * c * 2) for c in (qd, kvd, kvd, hidden, inter))
        res = ctx.to_device(synth.activations(1, "res", batch, hidden))
        def enqueue():
            for s in sets:
                ctx.call("affine_matvec", *s["q"], xh, yq, qd, hidden, G, batch)
                ctx.call("affine_dual_matvec", *s["k"], *s["v"], xh, yk, yv, kvd, hidden, G, batch)
                ctx.call("affine_matvec_add", *s["o"], xq, res, yh, hidden, qd, G, batch)
                ctx.call("affine_gate_up_swiglu", *s["gate"], *s["up"], xh, yi, inter, hidden, G, batch)
                ctx.call("affine_matvec_add", *s["down"], xi, res, yh, hidden, inter, G, batch)
        self.run(config, "decoder-layer qmm set (Q, K|V, O+add, gate/up+SwiGLU, down+add: 5 launches)", f"hidden {hidden} inter {inter} {n_q}x{n_kv}x{d}", batch, wbytes + act, layers, enqueue)
        for s in sets:
            for v in s.values():
                for b in v:
                    b.free()
        for b in (xh, xq, xi, yq, yk, yv, yh, yi, res):
            b.free()

    # ── binary / ternary ──
    def signed(self, config, fmt, rows, cols, batch=1):
        ctx = self.ctx
        if self.only and self.only not in f"signed fmt{fmt} {rows}x{cols} b{batch}":
            return
        maker, bpw, name = (synth.binary1, 1 / 8, "signed_binary_matvec_g128") if fmt == 1 else (synth.ternary2, 2 / 8, "signed_ternary_matvec_g128")
        alg = rows * cols * (bpw + 2 / 128) + batch * cols * 2 + batch * rows * 2
        n = copies_for(alg)
        sets = self.dev_copies(maker(2, f"sg{fmt}{rows}", rows, cols), n)
        x = ctx.to_device(synth.activations(2, "sx", batch, cols))
        y = ctx.alloc(batch * rows * 2)
        def enqueue():
            for s in sets:
                ctx.call("signed_matvec", fmt, *s, x, y, rows, cols, batch)
        self.run(config, name, f"{rows}x{cols}", batch, alg, n, enqueue)
        for s in sets:
            for b in s:
                b.free()
        x.free(); y.free()

    def bitplane(self, config, fmt, planes, rows, cols, batch=1):
        """The low-bit activation path: bit-plane view of x (producer) + popcount matvec (consumer), two launches;
        batch > 1: prompt rows through the batched view and the weight-sharing tile."""
        ctx = self.ctx
        if self.only and self.only not in f"bitplane fmt{fmt} i{planes} {rows}x{cols} b{batch}":
            return
        maker, bpw = (synth.binary1, 1 / 8) if fmt == 1 else (synth.ternary2, 2 / 8)
        groups = cols // 128
        alg = rows * cols * (bpw + 2 / 128) + batch * (cols * 2 + rows * 2 + 2 * (groups * planes * 16 + groups * 2))  # planes written once, read once
        n = copies_for(alg)
        sets = self.dev_copies(maker(2, f"bp{fmt}{rows}", rows, cols), n)
        x = ctx.to_device(synth.activations(2, "bpx", batch, cols))
        pl, sc, y = ctx.alloc(batch * groups * planes * 16), ctx.alloc(batch * groups * 2), ctx.alloc(batch * rows * 2)
        def enqueue():
            for s in sets:
                ctx.call("signed_activation_bitplanes", x, None, pl, sc, cols, planes, batch)
                ctx.call("signed_bitplane_matvec", fmt, 0, *s, None, None, pl, sc, None, y, rows, cols, planes, batch)
        name = ("signed_binary" if fmt == 1 else "signed_ternary") + f"_bitplane_i{planes}_matvec_g128 (+ view producer)"
        self.run(config, name, f"{rows}x{cols}", batch, alg, n, enqueue)
        for s in sets:
            for b in s:
                b.free()
        for b in (x, pl, sc, y):
            b.free()

    # ── attention ──
    def attention(self, config, n_q, n_kv, d, ctx_len, batch):
        ctx = self.ctx
        if self.only and self.only not in f"attention {n_q}x{n_kv}x{d} ctx{ctx_len} b{batch}":
            return
        cap = ctx_len
        kv_bytes = 2 * n_kv * d * 2 * ctx_len * batch
        alg = kv_bytes + 2 * n_q * d * 2 * batch
        n = copies_for(alg, cap=48)
        k = synth.kv_cache(3, "k", 1, n_kv, min(cap, 4096), d)[0]
        # one seeded block of keys repeated along the context: the values do not change the timing
        reps = int(np.ceil(cap / k.shape[1]))
        kfull = np.ascontiguousarray(np.tile(k, (batch, 1, reps, 1))[:, :, :cap, :])
        caches = [(ctx.to_device(kfull), ctx.to_device(kfull)) for _ in range(n)]
        q = ctx.to_device(synth.activations(3, "q", batch, n_q, d))
        out = ctx.alloc(batch * n_q * d * 2)
        scale = C.c_float(1 / np.sqrt(d))
        def enqueue():
            for kc, vc in caches:
                ctx.call("attention_decode", q, kc, vc, out, n_q, n_kv, d, cap, ctx_len, scale, 0, batch, C.c_size_t(n_kv * cap * d))
        self.run(config, "attention_decode (split-K flash decode)", f"{n_q}q x {n_kv}kv x d{d}, ctx {ctx_len}", batch, alg, n, enqueue)
        for kc, vc in caches:
            kc.free(); vc.free()
        q.free(); out.free()

    def attention_prefill(self, config, n_q, n_kv, d, n_pos, start):
        """Chunked causal attention of a prompt chunk: n_pos query positions from `start`."""
        ctx = self.ctx
        if self.only and self.only not in f"prefill attention {n_q}x{n_kv}x{d} n{n_pos} s{start}":
            return
        cap = start + n_pos
        # K and V of the keys any position of the chunk sees cross HBM once per group of eight positions at worst;
        # the algorithmic figure is one pass over them plus q and out
        alg = 2 * n_kv * d * 2 * cap + 2 * n_pos * n_q * d * 2
        k = synth.kv_cache(5, "pk", 1, n_kv, cap, d)[0]
        n = copies_for(alg, cap=32)
        caches = [(ctx.to_device(k), ctx.to_device(k)) for _ in range(n)]
        q = ctx.to_device(synth.activations(5, "pq", n_pos, n_q, d))
        out = ctx.alloc(n_pos * n_q * d * 2)
        scale = C.c_float(1 / np.sqrt(d))
        def enqueue():
            for kc, vc in caches:
                ctx.call("attention_prefill", q, kc, vc, out, n_q, n_kv, d, n_pos, start, cap, scale, 0)
        # multiply-adds x 2 of QK^T and PV over the causal triangle
        keys = sum(start + t + 1 for t in range(n_pos))
        self.run(config, "attention_prefill (chunked causal)", f"{n_q}q x {n_kv}kv x d{d}, {n_pos} positions from {start}", 1, alg, n, enqueue,
                 flops=4.0 * n_q * d * keys)
        for kc, vc in caches:
            kc.free(); vc.free()
        q.free(); out.free()

    def deltanet(self, config, d, hv, hqk, seq_len):
        """The recurrence of a DeltaNet layer: one decode step (seq_len 1) or a prompt chunk."""
        ctx = self.ctx
        if self.only and self.only not in f"deltanet d{d} h{hv} qk{hqk} t{seq_len}":
            return
        rng = np.random.default_rng(seq_len)
        width = (2 * hqk + hv) * d
        alg = 2 * hv * d * d * 2 + seq_len * (width + hv * d + 2 * hv) * 2
        n = copies_for(alg, cap=32)
        states = [ctx.to_device((rng.standard_normal((hv, d, d)) * 0.05).astype(np.float16)) for _ in range(n)]
        qkv = rng.standard_normal((seq_len, 2 * hqk + hv, d)).astype(np.float32)
        qkv[:, :2 * hqk] /= np.linalg.norm(qkv[:, :2 * hqk], axis=2, keepdims=True)
        dq = ctx.to_device(qkv.astype(np.float16))
        b, a = (ctx.to_device(rng.standard_normal(seq_len * hv).astype(np.float16)) for _ in range(2))
        a_log, dt = ctx.to_device(rng.uniform(-2, 0.5, hv).astype(np.float16)), ctx.to_device(rng.uniform(-0.5, 0.5, hv).astype(np.float16))
        out = ctx.alloc(seq_len * hv * d * 2)
        def enqueue():
            for st in states:
                if seq_len == 1:
                    ctx.call("deltanet_recurrence_decode", st, dq, b, a, a_log, dt, out, d, hv, hqk)
                else:
                    ctx.call("deltanet_recurrence_prefill", st, dq, b, a, a_log, dt, out, d, hv, hqk, seq_len, None)
        name = "deltanet_recurrence_mlx_decode" if seq_len == 1 else "deltanet_recurrence_mlx_prefill"
        self.run(config, name, f"d{d} h{hv} qk{hqk}, {seq_len} positions", 1, alg, n, enqueue)
        for t in states + [dq, b, a, a_log, dt, out]:
            t.free()

    def lm_head(self, config, vocab, hidden):
        ctx = self.ctx
        w = ctx.to_device(synth.normal_f16(4, "head", (vocab, hidden), 0.02))
        x = ctx.to_device(synth.activations(4, "x", 1, hidden))
        y = ctx.alloc(vocab * 2)
        alg = vocab * hidden * 2 + hidden * 2 + vocab * 2
        self.run(config, "fp16_matvec (LM head)", f"{vocab}x{hidden}", 1, alg, 1, lambda: ctx.call("fp16_matvec", w, x, y, vocab, hidden, 1))
        for b in (w, x, y):
            b.free()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="0,1,2,3,4")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--markdown", action="store_true", help="print a markdown table after the JSON lines")
    ap.add_argument("--quick", action="store_true", help="fewer attention cases")
    ap.add_argument("--only", default="", help='only the affine cases whose "<mode> <rows>x<cols> b<batch>" the attention cases whose "attention <n_q>x<n_kv>x<d> ctx<len> b<batch>" and the low-bit cases whose "signed fmt<1|2> <rows>x<cols> b<batch>" contain this (small runs for profiler captures)')
    args = ap.parse_args()
    want = {c.strip() for c in args.configs.split(",")}
    b = Bench(args.reps, args.only)
    if "0" in want:
        b.affine("config0", 4096, 1024, 1)
    if "1" in want:
        for batch in (1, 4, 8, 16, 32, 64):  # 17 rows and more run on the tcgen05 QMM
            b.layer_set("config1", 2048, 6144, 16, 4, 128, batch)
    if "2" in want:
        for fmt in (1, 2):
            b.signed("config2", fmt, 17408, 5120)
            b.signed("config2", fmt, 5120, 17408)
        b.bitplane("config2", 1, 4, 17408, 5120)
        b.bitplane("config2", 1, 4, 5120, 17408)
        b.bitplane("config2", 2, 5, 17408, 5120)
        b.bitplane("config2", 2, 5, 5120, 17408)
        b.bitplane("config2", 1, 4, 17408, 5120, batch=8)   # prompt rows: the weight-sharing tile
        b.bitplane("config2", 1, 4, 5120, 17408, batch=8)
    if "3" in want:
        for (nq, nkv, d) in ((16, 4, 128), (8, 2, 256)):
            for ctx_len in ((1024, 32768) if args.quick else (1024, 4096, 16384, 32768)):
                for batch in (1, 8):
                    b.attention("config3", nq, nkv, d, ctx_len, batch)
    if "4" in want:
        b.affine("config4", 12288, 4096, 1, "gate_up")
        b.affine("config4", 4096, 12288, 1, "add")
        b.affine("config4", 4096, 4096, 1, "add")
        b.affine("config4", 4096, 4096, 1, "matvec")
        b.affine("config4", 1024, 4096, 1, "dual")
        b.affine("config4", 12288, 4096, 8, "gate_up")
        b.affine("config4", 4096, 12288, 8, "add")
        for batch in (64, 512):  # tcgen05 QMM (prompt chunks, large decode batches)
            b.affine("config4", 12288, 4096, batch, "gate_up")
            b.affine("config4", 4096, 12288, batch, "add")
            b.affine("config4", 4096, 4096, batch, "matvec")
        b.attention_prefill("config4", 32, 8, 128, 512, 0)
        b.attention_prefill("config4", 32, 8, 128, 128, 384)
        if not args.only:
            b.lm_head("config4", 151936, 4096)
    if "deltanet" in want:  # not one of the headline configurations: the recurrence of a hybrid model's linear-attention layers
        for t in (1, 64, 512):
            b.deltanet("deltanet", 128, 32, 16, t)
    if args.markdown:
        print("\n| config | kernel | shape | batch | MB / launch | us / launch | GB/s | of %s peak %.0f GB/s |" % (b.peak_kind, b.peak))
        print("|---|---|---|---|---|---|---|---|")
        for r in b.rows:
            print("| %s | %s | %s | %d | %.2f | %.2f | %.0f | %.3f |" % (r["config"], r["kernel"], r["shape"], r["batch"], r["bytes_per_launch"] / 1e6,
                                                                      r["us_per_launch"], r["achieved_gbs"], r["frac_of_peak"]))


if __name__ == "__main__":
    main()
