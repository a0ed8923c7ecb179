"""Time of one tensor-parallel exchange (``smelt_tp_reduce_add``: all-reduce of the ranks'
partials over peer memory + residual add) at N ranks, one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P -m smelt_b200.tp_bench [--hidden 4096] [--launches 72] [--reps 20] [--collective peer|nccl]

Every rank records ``launches`` exchanges of ``hidden`` fp16 values (the decode table issues two
per layer: 72 per token of the 36-layer model) with ``smelt_cuda_capture_begin / _end`` and replays
the recording between CUDA events; rank 0 prints one JSON line with the slowest rank's time per
exchange.  ``--collective nccl`` times ncclAllReduce + ``elementwise_add`` instead."""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os

import numpy as np


def main():
    import torch
    import torch.distributed as dist

    from smelt_b200 import capi, package, synth

    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--launches", type=int, default=72)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--collective", choices=("peer", "nccl"), default="peer")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl")
    ctx = capi.Context(local)
    ident = np.zeros(capi.TP_ID_BYTES, np.uint8)
    if rank == 0:
        assert ctx.lib.smelt_cuda_tp_unique_id(ident.ctypes.data_as(C.c_void_p)) == 0
    t = torch.from_numpy(ident).cuda()
    dist.broadcast(t, 0)
    ctx._check(ctx.lib.smelt_cuda_tp_init(ctx.h, rank, world, t.cpu().numpy().ctypes.data_as(C.c_void_p)))
    if args.collective == "peer":
        package.open_tp_exchange(ctx, dist, world)
    n = args.hidden
    partial = ctx.to_device(synth.activations(50 + rank, "partial", 1, n))
    residual = ctx.to_device(synth.activations(50, "residual", 1, n))
    out = ctx.alloc(n * 2)
    work = ctx.alloc(n * 2).fill(0)

    def enqueue():
        for _ in range(args.launches):
            if args.collective == "peer":
                ctx.call("tp_reduce_add", partial, residual, out, C.c_size_t(n))
            else:  # the baseline: all-reduce in place (a zero buffer, so repeated sums stay finite), then the residual add
                ctx.call("tp_all_reduce_f16", work, C.c_size_t(n))
                ctx.call("elementwise_add", work, residual, out, C.c_size_t(n))

    ctx.synchronize()
    dist.barrier()  # every rank is set up: the exchange's bounded wait is about a second
    enqueue()
    ctx.synchronize()
    dist.barrier()
    ctx.call("capture_begin")
    enqueue()
    ctx.call("capture_end")
    ms = C.c_float(0)
    dist.barrier()
    ctx._check(ctx.lib.smelt_cuda_capture_replay(ctx.h, 3, args.reps, C.byref(ms)))
    err = ctx.device_error_flags()
    worst = torch.tensor([ms.value, float(err)], device="cuda")
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"metric": "us per tensor-parallel exchange (max over ranks)", "n_gpus": world, "collective": args.collective,
                          "hidden": n, "launches_per_replay": args.launches, "replays": args.reps,
                          "us_per_exchange": round(float(worst[0]) * 1e3 / args.launches, 3), "device_error": int(worst[1])}), flush=True)
    ctx.synchronize()
    dist.barrier()
    ctx.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
