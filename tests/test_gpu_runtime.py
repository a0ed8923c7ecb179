"""The dispatch-record runtime on a B200: a small synthetic decoder replayed through
SmeltDispatchRecord tables must reproduce the CPU oracle's greedy tokens and logits."""
import ctypes as C

import numpy as np
import pytest

from smelt_b200 import capi, package, synth
from helpers import rel_err

pytestmark = pytest.mark.gpu

SMALL = package.DecoderConfig(layers=3, hidden=512, inter=1536, n_q=8, n_kv=2, head_dim=64, vocab=4096)
MID = package.DecoderConfig(layers=2, hidden=2048, inter=6144, n_q=16, n_kv=4, head_dim=128, vocab=8192)


@pytest.fixture(scope="module")
def ctx():
    c = capi.Context(0)
    yield c
    c.close()


def make(ctx, cfg, seed, capacity, batch=1, fuse=0):
    pkg = package.SyntheticPackage(cfg, seed)
    image, desc, layers = package.build_image(pkg, keep_for_oracle=True)
    return pkg, package.Decoder(ctx, image, desc, layers, capacity, batch, fuse_residual=fuse)


@pytest.mark.parametrize("cfg", [SMALL, MID])
def test_decode_step_matches_oracle(ctx, oracle, cfg):
    pkg, dec = make(ctx, cfg, 11, 64)
    ref = oracle.model_from_package(pkg, 64)
    prompt = synth.rng_for(11, "prompt").integers(0, cfg.vocab, size=6)
    for pos, tok in enumerate(prompt):
        got_tok = dec.decode_step([tok], pos)[0]
        ref_tok, ref_logits = ref.decode_step(int(tok), pos, want_logits=True)
        got_logits = dec.logits()[0]
        # Every kernel output may differ from the oracle's by an fp16 ulp (other fp32 summation
        # order), and the differences travel through the layers: bound the worst logit error by
        # one percent of the logits' RMS.
        ref32 = ref_logits.astype(np.float32)
        err = float(np.max(np.abs(got_logits.astype(np.float32) - ref32)) / np.sqrt(np.mean(ref32 * ref32)))
        assert err < 1e-2, f"logits diverged at position {pos}: {err}"
        top2 = np.sort(ref_logits.astype(np.float32))[-2:]
        if top2[1] - top2[0] > 4 * np.spacing(np.float16(top2[1])):
            assert got_tok == ref_tok


def test_greedy_tokens_match_oracle_eager_graph_and_fused(ctx, oracle):
    """Teacher-forced: the oracle's token is fed at every step and every step's argmax is
    compared; a differing id passes only as the oracle's runner-up at a margin under 0.02."""
    cfg, cap, n_dec = SMALL, 96, 48
    pkg, dec = make(ctx, cfg, 5, cap)
    ref = oracle.model_from_package(pkg, cap)
    prompt = synth.rng_for(5, "prompt").integers(0, cfg.vocab, size=12).astype(np.int32)
    want, runner, margins = ref.greedy_top2(prompt, n_dec)
    eager = dec.teacher_forced(prompt, want, use_graph=False)[:, 0]
    dec.reset_cache()
    graph = dec.teacher_forced(prompt, want, use_graph=True)[:, 0]
    assert np.array_equal(eager, graph), "graph replay must equal eager interpretation"
    v = package.compare_greedy(eager, want, runner, margins)
    print("small model: %d of %d steps identical, %d tie breaks" % (v["identical"], v["checked"], v["tie_breaks"]))
    assert not v["wrong"], v
    _, fused = make(ctx, cfg, 5, cap, fuse=True)
    assert np.array_equal(fused.teacher_forced(prompt, want, use_graph=True)[:, 0], graph), "fused residual add must not change tokens"
    # free-running greedy decode equals the teacher-forced ids up to the first step the two differ at
    free = dec.generate(prompt, n_dec, use_graph=True)[:, 0]
    split = next((i for i in range(n_dec) if free[i] != want[i]), n_dec)
    assert np.array_equal(free[:split + 1], graph[:split + 1])


def test_fused_table_keeps_tokens_and_logits(ctx, oracle):
    """Norm folded into the projections, one Q/K/V launch, one RoPE + append + attention launch:
    the same rounding points and the same summation order per output row, so the same logits bit
    for bit as the reference-shaped table, and the oracle's tokens."""
    cfg, cap, n_dec = MID, 64, 24
    prompt = synth.rng_for(6, "prompt").integers(0, cfg.vocab, size=9).astype(np.int32)
    pkg, plain = make(ctx, cfg, 6, cap)
    want, runner, margins = oracle.model_from_package(pkg, cap).greedy_top2(prompt, n_dec)
    got_plain = plain.teacher_forced(prompt, want, use_graph=True)[:, 0]
    logits_plain = plain.logits()[0].copy()
    _, fused = make(ctx, cfg, 6, cap, fuse=3)
    assert len(fused.table) < len(plain.table) - 6 * cfg.layers
    eager = fused.teacher_forced(prompt, want, use_graph=False)[:, 0]
    assert np.array_equal(fused.logits()[0].view(np.uint16), logits_plain.view(np.uint16)), "same rounding points, same bits"
    fused.reset_cache()
    graph = fused.teacher_forced(prompt, want, use_graph=True)[:, 0]
    assert np.array_equal(eager, graph) and np.array_equal(graph, got_plain)
    assert not package.compare_greedy(graph, want, runner, margins)["wrong"]


def test_batch_of_independent_sequences(ctx, oracle):
    cfg, cap, B, n_dec = SMALL, 48, 4, 8
    pkg, dec = make(ctx, cfg, 7, cap, batch=B)
    prompts = synth.rng_for(7, "prompts").integers(0, cfg.vocab, size=(B, 5)).astype(np.int32)
    ref = oracle.model_from_package(pkg, cap)
    gold = [ref.greedy_top2(prompts[b], n_dec) for b in range(B)]
    got = dec.teacher_forced(prompts, np.array([g[0] for g in gold]).T, use_graph=True)
    for b in range(B):
        v = package.compare_greedy(got[:, b], *gold[b])
        assert not v["wrong"], (b, v)


def test_runtime_errors(ctx):
    pkg, dec = make(ctx, SMALL, 3, 16)
    st = ctx.lib.smelt_cuda_decode_step(ctx.h, dec.table, dec.n_records, np.array([0], np.int32).ctypes.data_as(C.c_void_p), 16, None)
    assert st == capi.OUT_OF_RANGE and "position" in ctx.last_error()
    st = ctx.lib.smelt_cuda_decode_step(ctx.h, dec.table, dec.n_records, np.array([SMALL.vocab], np.int32).ctypes.data_as(C.c_void_p), 0, None)
    assert st == capi.OUT_OF_RANGE and "tokenId" in ctx.last_error()
    assert ctx.call_status("register_pipeline", 200, "fused_lut_matvec") == capi.UNKNOWN_PIPELINE
    assert ctx.call_status("register_pipeline", 200, "attention_decode_softcap") == capi.UNKNOWN_PIPELINE
    rec = (capi.DispatchRecord * 1)()
    rec[0].pipeline = 999
    st = ctx.lib.smelt_cuda_decode_step(ctx.h, rec, 1, np.array([0], np.int32).ctypes.data_as(C.c_void_p), 0, None)
    assert st == capi.UNKNOWN_PIPELINE
    rec[0].pipeline = dec.table[0].pipeline  # embedding_gather, but bound to a slot that was never allocated
    rec[0].buffer_count = 1
    rec[0].buf[0].slot = 250
    st = ctx.lib.smelt_cuda_decode_step(ctx.h, rec, 1, np.array([0], np.int32).ctypes.data_as(C.c_void_p), 0, None)
    assert st == capi.OUT_OF_RANGE
    assert ctx.device_error() == 0


def test_kv_slot_growth_preserves_contents(ctx):
    heads, d, old, new, live = 2, 64, 16, 40, 11
    ctx.call("alloc_slot", 200, C.c_size_t(heads * old * d * 2))
    data = synth.activations(1, "kv", heads, old, d)
    ctx.call("write_slot", 200, C.c_size_t(0), data, C.c_size_t(data.nbytes))
    ctx.call("resize_kv_slot", 200, heads, d, old, new, live)
    out = np.empty((heads, new, d), np.float16)
    ctx.call("read_slot", 200, C.c_size_t(0), out, C.c_size_t(out.nbytes))
    assert np.array_equal(out[:, :live].view(np.uint16), data[:, :live].view(np.uint16))
    assert not out[:, live:].any()
    assert ctx.call_status("resize_kv_slot", 200, heads, d, new, new + 8, new + 1) == capi.BAD_ARGUMENT


def test_skip_guards_follow_position(ctx):
    """Constant kinds 10 / 11 (skip unless pos+1 < / >= literal, SmeltDispatchTable.swift:80-83)."""
    ctx.call("alloc_slot", 201, C.c_size_t(64))
    ctx.call("alloc_slot", 202, C.c_size_t(64))
    ctx.call("alloc_slot", 203, C.c_size_t(64))
    ctx.call("alloc_slot", 204, C.c_size_t(64))
    ctx.call("alloc_slot", 205, C.c_size_t(64))
    cfg = capi.RuntimeConfig(token_id_slot=204, position_slot=205, weights_slot=30, argmax_slot=204, cur_slot=201, alt_slot=202,
                             cache_seq_capacity=64, context_limit=64, vocab_size=10, batch=1)
    ctx._check(ctx.lib.smelt_cuda_configure(ctx.h, C.byref(cfg)))
    ctx.call("register_pipeline", 0, "elementwise_add")
    one = np.ones(32, np.float16)
    for slot in (201, 202):
        ctx.call("write_slot", slot, C.c_size_t(0), one, C.c_size_t(64))
    rec = (capi.DispatchRecord * 2)()
    for i, (kind, lit) in enumerate([(capi.CONST_SKIP_UNLESS_POS1_LT, 4), (capi.CONST_SKIP_UNLESS_POS1_GE, 4)]):
        r = rec[i]
        r.pipeline, r.buffer_count, r.constant_count = 0, 3, 2
        r.grid[0] = r.grid[1] = r.grid[2] = 1
        for j, (slot, binding) in enumerate([(capi.SLOT_CUR, 0), (202, 1), (203, 2)]):
            r.buf[j].slot, r.buf[j].binding_index = slot, binding
        r.con[0].kind, r.con[0].binding_index, r.con[0].value = 0, 3, 32
        r.con[1].kind, r.con[1].binding_index, r.con[1].value = kind, 255, lit
    tok = np.array([0], np.int32).ctypes.data_as(C.c_void_p)
    for pos, ran in [(2, [True, False]), (3, [False, True]), (10, [False, True])]:
        for i in range(2):
            ctx.call("zero_slot", 203)
            ctx._check(ctx.lib.smelt_cuda_decode_step(ctx.h, C.byref(rec[i]), 1, tok, pos, None))
            out = np.empty(32, np.float16)
            ctx.call("read_slot", 203, C.c_size_t(0), out, C.c_size_t(64))
            assert bool(out.any()) == ran[i], (pos, i)


def test_capture_replay_runs_the_recorded_launches(ctx, oracle):
    rows, cols = 512, 2048
    w, s, b = synth.affine_u4(9, "cap", rows, cols, 64)
    x = synth.activations(9, "x", 1, cols)
    dw, ds, db, dx = (ctx.to_device(a) for a in (w, s, b, x))
    y = ctx.alloc(rows * 2).fill(0)
    ctx.call("capture_begin")
    ctx.call("affine_matvec", dw, ds, db, dx, y, rows, cols, 64, 1)
    assert ctx.call_status("capture_begin") == capi.BAD_ARGUMENT  # already open
    ctx.call("capture_end")
    assert not np.any(y.download(np.uint16, (rows,)))  # recorded, not run
    ms = C.c_float(-1)
    ctx._check(ctx.lib.smelt_cuda_capture_replay(ctx.h, 1, 3, C.byref(ms)))
    assert 0 < ms.value < 50
    assert rel_err(y.download(np.float16, (1, rows)), oracle.affine_matvec(w, s, b, x, rows, cols, 64)) < 2e-3
    assert ctx.call_status("capture_end") == capi.BAD_ARGUMENT  # nothing open


def test_exchange_wait_gives_up_and_reports():
    """A reduction whose peer never arrives runs into its bounded wait, raises bit 8 of the device
    error word and returns; the context keeps working.  (The peer is a local buffer nobody writes.)"""
    c = capi.Context(0)
    try:
        c.call("tp_exchange_open_loopback", 2)
        n = 4096
        part = c.to_device(synth.activations(12, "p", 1, n))
        res = c.to_device(synth.activations(12, "r", 1, n))
        out = c.alloc(n * 2)
        c.call("tp_reduce_add", part, res, out, C.c_size_t(n))
        c.synchronize()
        with pytest.raises(capi.SmeltError) as caught:  # reading a non-zero error word reports DEVICE_TIMEOUT and clears it
            c.device_error()
        assert caught.value.status == capi.DEVICE_TIMEOUT and "256" in str(caught.value)
        assert c.device_error() == 0
        c.call("clear_device_error")
        y = c.alloc(n * 2)
        c.call("elementwise_add", part, res, y, n)  # the context is still usable
        want = (synth.activations(12, "p", 1, n).astype(np.float16) + synth.activations(12, "r", 1, n).astype(np.float16))
        assert np.array_equal(y.download(np.float16, (1, n)), want)
    finally:
        c.close()
