"""Tensor-parallel sharding on CPU: two gloo ranks each hold their shard of a small synthetic
decoder (the arrays package.build_image lays out for that rank), run the oracle's kernels on it
and all-reduce the row-parallel partial outputs where the record table places
smelt_tp_all_reduce.  The result must match the unsharded oracle model."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from smelt_b200 import package, synth

CFG = package.DecoderConfig(layers=2, hidden=256, inter=512, n_q=4, n_kv=2, head_dim=64, vocab=512)
CFG4 = package.DecoderConfig(layers=2, hidden=256, inter=1024, n_q=8, n_kv=4, head_dim=64, vocab=512)  # one KV head per rank at 4 ranks
SEED, CAP, STEPS = 21, 16, 5


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _all_reduce_f16(partial: np.ndarray) -> np.ndarray:
    """Sum of fp16 partials over the ranks, rounded once to fp16 (what an fp16 all-reduce with
    fp32 accumulation returns)."""
    t = torch.from_numpy(partial.astype(np.float32))
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t.numpy().astype(np.float16)


def _sharded_decode(oracle, c, rank: int, world: int):
    pkg = package.SyntheticPackage(c, SEED)
    nq, nkv, D, H, I, G = c.n_q // world, c.n_kv // world, c.head_dim, c.hidden, c.inter // world, c.group
    shard = {}
    for l in range(c.layers):
        for name in ("q", "k", "v", "o", "gate", "up", "down"):
            t = pkg.layer_tensor(l, name)
            shard[(l, name)] = package.shard_cols(t, rank, world, G) if name in ("o", "down") else package.shard_rows(t, rank, world)
    emb, head, fin = pkg.embedding(), pkg.lm_head(), pkg.norm_delta("final_norm")
    kc = [np.zeros((nkv, CAP, D), np.float16) for _ in range(c.layers)]
    vc = [np.zeros((nkv, CAP, D), np.float16) for _ in range(c.layers)]
    base_log2 = float(np.log2(np.float32(c.rope_theta)))
    tokens = synth.rng_for(SEED, "prompt").integers(0, c.vocab, size=STEPS)
    out = []
    for pos, tok in enumerate(tokens):
        h = emb[int(tok)].copy()
        for l in range(c.layers):
            n_in, n_post = pkg.norm_delta(f"layer{l}.input_norm"), pkg.norm_delta(f"layer{l}.post_norm")
            x = oracle.rms_norm_1pw(h, n_in, c.eps)
            q = oracle.affine_matvec(*shard[(l, "q")], x, nq * D, H, G)[0]
            k = oracle.affine_matvec(*shard[(l, "k")], x, nkv * D, H, G)[0]
            v = oracle.affine_matvec(*shard[(l, "v")], x, nkv * D, H, G)[0]
            q = oracle.apply_rope(q, D, D, nq, 1, pos, base_log2, 1)
            kc[l] = oracle.rope_kv_cache_update(kc[l], k, CAP, D, pos, nkv, D, 1, base_log2, 1).reshape(nkv, CAP, D)
            vc[l] = oracle.kv_cache_update(vc[l], v, CAP, D, pos, nkv).reshape(nkv, CAP, D)
            a = oracle.attention_decode(q, kc[l], vc[l], nq, nkv, D, CAP, pos + 1)
            o = _all_reduce_f16(oracle.affine_matvec(*shard[(l, "o")], a.reshape(-1), H, nq * D, G)[0])
            h = oracle.elementwise_add(h, o)
            x = oracle.rms_norm_1pw(h, n_post, c.eps)
            act = oracle.affine_gate_up_swiglu(*shard[(l, "gate")], *shard[(l, "up")], x, I, H, G)[0]
            d = _all_reduce_f16(oracle.affine_matvec(*shard[(l, "down")], act, H, I, G)[0])
            h = oracle.elementwise_add(h, d)
        logits = oracle.fp16_matvec(head, oracle.rms_norm_1pw(h, fin, c.eps), c.vocab, H)[0]
        out.append(logits)
    return tokens, np.stack(out)


def _worker(rank: int, world: int, port: int, ret, cfg):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle

        tokens, logits = _sharded_decode(oracle, cfg, rank, world)
        # every rank ends with the same (replicated) hidden state, hence the same logits
        t = torch.from_numpy(logits.astype(np.float32))
        lo, hi = t.clone(), t.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        assert torch.equal(lo, hi), "ranks disagree on the replicated logits"
        if rank == 0:
            pkg = package.SyntheticPackage(cfg, SEED)
            ref = oracle.model_from_package(pkg, CAP)
            for pos, tok in enumerate(tokens):
                ref_tok, ref_logits = ref.decode_step(int(tok), pos, want_logits=True)
                r32 = ref_logits.astype(np.float32)
                err = float(np.max(np.abs(logits[pos].astype(np.float32) - r32)) / np.sqrt(np.mean(r32 * r32)))
                assert err < 1e-2, f"sharded decode diverged at position {pos}: {err}"
            ret["ok"] = True
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,cfg", [(2, CFG), (4, CFG4)])
def test_sharded_decode_matches_the_full_model(world, cfg):
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), ret, cfg), nprocs=world, join=True)
        assert ret.get("ok")


def test_shards_of_the_benchmark_model_at_4_and_8_ranks():
    """Per-rank geometry of the 36-layer benchmark decoder: head counts, column shards on group
    boundaries, LM-head row shards."""
    cfg = package.DecoderConfig(layers=1, hidden=4096, inter=12288, n_q=32, n_kv=8, head_dim=128, vocab=1024)
    pkg = package.SyntheticPackage(cfg, SEED)
    for world in (4, 8):
        for rank in (world - 1,):
            _, desc, _ = package.build_image(pkg, rank, world)
            assert (desc.n_q, desc.n_kv, desc.inter) == (32 // world, 8 // world, 12288 // world)
            assert (desc.tp_world, desc.tp_rank) == (world, rank)
            assert desc.inter % 128 == 0 and (desc.n_q * cfg.head_dim) % 128 == 0  # integer-MMA kernel eligibility


def test_shards_tile_the_full_tensors():
    pkg = package.SyntheticPackage(CFG, SEED)
    full = pkg.layer_tensor(0, "down")
    parts = [package.shard_cols(full, r, 2, CFG.group) for r in range(2)]
    assert np.array_equal(np.concatenate([p[0] for p in parts], axis=1), full[0])
    assert np.array_equal(np.concatenate([p[1] for p in parts], axis=1), full[1])
    full = pkg.layer_tensor(0, "gate")
    parts = [package.shard_rows(full, r, 2) for r in range(2)]
    assert all(np.array_equal(np.concatenate([p[i] for p in parts], axis=0), full[i]) for i in range(3))
    _, desc, _ = package.build_image(pkg, 1, 2)
    assert (desc.n_q, desc.n_kv, desc.inter, desc.tp_world, desc.tp_rank) == (2, 1, 256, 2, 1)
