"""One tensor-parallel rank of the multi-GPU parity test (launched by test_gpu_tp.py through
torch.distributed.run): a small synthetic decoder sharded over the ranks, replayed
teacher-forced on the CPU oracle's greedy tokens, must give the oracle's id at every step (a
differing id only as the oracle's runner-up at a top-2 margin under 0.02), eagerly and from the
captured graph, for the NCCL table, the peer-memory table and the vocab-parallel table."""
import ctypes as C
import faulthandler
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
faulthandler.dump_traceback_later(150, exit=True)  # a stuck rank ends itself with a traceback

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from smelt_b200 import capi, package  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl")
    ctx = capi.Context(local)
    ident = np.zeros(capi.TP_ID_BYTES, np.uint8)
    if rank == 0:
        assert ctx.lib.smelt_cuda_tp_unique_id(ident.ctypes.data_as(C.c_void_p)) == 0
    t = torch.from_numpy(ident).cuda()
    dist.broadcast(t, 0)
    ident = t.cpu().numpy()
    ctx._check(ctx.lib.smelt_cuda_tp_init(ctx.h, rank, world, ident.ctypes.data_as(C.c_void_p)))

    buf = ctx.to_device(np.full(4096, rank + 1, np.float16))
    ctx._check(ctx.lib.smelt_cuda_tp_all_reduce_f16(ctx.h, C.c_void_p(buf.ptr), C.c_size_t(4096)))
    ctx.synchronize()
    assert np.all(buf.download(np.float16, (4096,)) == world * (world + 1) / 2)

    cfg = package.DecoderConfig(layers=2, hidden=2048, inter=6144, n_q=16, n_kv=4, head_dim=128, vocab=8192)
    pkg = package.SyntheticPackage(cfg, 7)
    prompt, n_dec = np.array([5, 17, 99, 4000], np.int32), 24
    gold = torch.zeros(3, n_dec, dtype=torch.float64, device="cuda")
    if rank == 0:
        import oracle

        ref = oracle.model_from_package(pkg, 64)
        gold.copy_(torch.tensor(ref.greedy_top2(prompt, n_dec), dtype=torch.float64))
        ref.close()
    dist.broadcast(gold, 0)
    want, runner, margins = (gold[i].cpu().numpy() for i in range(3))
    want, runner = want.astype(np.int32), runner.astype(np.int32)
    results = {}
    for fuse in (0, 2, 6, 14):
        if fuse == 6:  # all-reduce + residual add over peer memory
            package.open_tp_exchange(ctx, dist, world)
        image, desc, layers = package.build_image(pkg, rank, world, vocab_parallel=bool(fuse & 8))  # 14: + vocab-parallel LM head
        dec = package.Decoder(ctx, image, desc, layers, 64, 1, fuse_residual=fuse)
        ctx.synchronize()
        dist.barrier()  # ranks start decoding together: the exchange's bounded wait is about a second
        eager = dec.teacher_forced(prompt, want, use_graph=False)[:, 0]
        dec.reset_cache()
        graph = dec.teacher_forced(prompt, want, use_graph=True)[:, 0]
        assert np.array_equal(eager, graph), (fuse, eager, graph)
        v = package.compare_greedy(graph, want, runner, margins)
        assert not v["wrong"], (fuse, v, graph.tolist(), want.tolist())
        results[fuse] = graph
        if rank == 0:
            print("TP_PARITY fuse=%d world=%d: %d of %d steps identical to the oracle, %d tie breaks" % (fuse, world, v["identical"], v["checked"], v["tie_breaks"]), flush=True)
    assert np.array_equal(results[0], results[2])
    # two ranks: the sum of two fp16 partials rounded once is what the fp16 all-reduce returns too
    assert world != 2 or np.array_equal(results[6], results[2])
    assert np.array_equal(results[14], results[6]), "the vocab-parallel argmax must pick the same ids"
    flags = C.c_uint32(0)
    ctx._check(ctx.lib.smelt_cuda_device_error(ctx.h, C.byref(flags)))
    assert flags.value == 0, "a bounded device wait gave up"
    # every rank holds the same tokens
    tt = torch.from_numpy(np.concatenate([results[f] for f in (0, 2, 6, 14)]).astype(np.int64)).cuda()
    lo, hi = tt.clone(), tt.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    assert torch.equal(lo, hi)
    dist.barrier()
    ctx.close()
    dist.destroy_process_group()
    if rank == 0:
        print("TP_WORKER_OK", flush=True)


if __name__ == "__main__":
    main()
