"""Prefill on a B200: the batched RoPE + KV write and the chunked causal attention against the
oracle's per-position kernels, and the prefill driver against token-by-token decoding
(prefill_rope_kv.metal:64-187, prefill_attention.metal:14-413; SmeltModel.swift:619-631 decodes
the prompt token by token when a package has no prefill table)."""
import ctypes as C

import numpy as np
import pytest

from smelt_b200 import capi, package, synth
from helpers import INF_TOL, REL_TOL, inf_err, rel_err

pytestmark = pytest.mark.gpu

SMALL = package.DecoderConfig(layers=3, hidden=512, inter=1536, n_q=8, n_kv=2, head_dim=64, vocab=4096)
MID = package.DecoderConfig(layers=2, hidden=2048, inter=6144, n_q=16, n_kv=4, head_dim=128, vocab=8192)


@pytest.fixture(scope="module")
def ctx():
    c = capi.Context(0)
    yield c
    c.close()


@pytest.mark.parametrize("layout,rope_dim,math_mode", [(1, 64, 1), (0, 64, 1), (1, 32, 0), (0, 32, 0), (2, 32, 0), (1, 64, 0)])
def test_rope_kv_prefill_is_the_per_position_kernels(ctx, oracle, layout, rope_dim, math_mode):
    """Bit-exact against apply_rope + rope_kv_cache_update + kv_cache_update applied position by
    position (attention.metal:48-209), analytic and table mode, every pair layout."""
    d, n_q, n_kv, n_pos, start, cap = 64, 6, 2, 13, 9, 40
    q = synth.activations(31, "pq", n_pos, n_q, d)
    k = synth.activations(31, "pk", n_pos, n_kv, d)
    v = synth.activations(31, "pv", n_pos, n_kv, d)
    kc0 = synth.kv_cache(31, "kc", 1, n_kv, cap, d)[0]
    vc0 = synth.kv_cache(31, "vc", 1, n_kv, cap, d)[0]
    base_log2 = float(np.log2(10000.0))
    cos = sin = None
    if math_mode == 0:
        ang = synth.rng_for(31, "ang").uniform(-3.0, 3.0, size=(cap, rope_dim)).astype(np.float32)
        cos, sin = np.cos(ang).astype(np.float16), np.sin(ang).astype(np.float16)
    dq, dk, dv, dkc, dvc = (ctx.to_device(a) for a in (q, k, v, kc0, vc0))
    dcos = ctx.to_device(cos) if cos is not None else None
    dsin = ctx.to_device(sin) if sin is not None else None
    ctx.call("rope_kv_prefill", dq, dk, dv, dcos, dsin, dkc, dvc, d, rope_dim, n_q, n_kv, n_pos, start, cap, layout, C.c_float(base_log2), math_mode)
    got_q = dq.download(np.float16, (n_pos, n_q, d))
    got_kc = dkc.download(np.float16, (n_kv, cap, d))
    got_vc = dvc.download(np.float16, (n_kv, cap, d))
    want_kc, want_vc = kc0.copy(), vc0.copy()
    for t in range(n_pos):
        pos = start + t
        row = None if cos is None else (cos[pos], sin[pos])
        want_q = oracle.apply_rope(q[t], d, rope_dim, n_q, layout, pos, base_log2, math_mode, *(row or (None, None)))
        assert np.array_equal(got_q[t].view(np.uint16), want_q.reshape(n_q, d).view(np.uint16)), f"q at position {pos}"
        want_kc = oracle.rope_kv_cache_update(want_kc, k[t], cap, d, pos, n_kv, rope_dim, layout, base_log2, math_mode, *(row or (None, None))).reshape(n_kv, cap, d)
        want_vc = oracle.kv_cache_update(want_vc, v[t], cap, d, pos, n_kv).reshape(n_kv, cap, d)
    assert np.array_equal(got_kc.view(np.uint16), want_kc.view(np.uint16))
    assert np.array_equal(got_vc.view(np.uint16), want_vc.view(np.uint16))
    # beyond the capacity: refused, nothing written
    st = ctx.call_status("rope_kv_prefill", dq, dk, dv, dcos, dsin, dkc, dvc, d, rope_dim, n_q, n_kv, n_pos, cap - 3, cap, layout, C.c_float(base_log2), math_mode)
    assert st == capi.OUT_OF_RANGE


@pytest.mark.parametrize("n_q,n_kv,d", [(16, 4, 128), (8, 2, 256), (8, 8, 64), (16, 1, 64), (32, 8, 128)])
@pytest.mark.parametrize("n_pos,start,window", [(37, 0, 0), (64, 200, 0), (5, 1000, 0), (40, 90, 48)])
def test_attention_prefill_matches_the_oracle_per_position(ctx, oracle, n_q, n_kv, d, n_pos, start, window):
    cap = start + n_pos + 5
    k = synth.kv_cache(32, "k", 1, n_kv, cap, d)[0]
    v = synth.kv_cache(32, "v", 1, n_kv, cap, d)[0]
    q = synth.activations(32, "q", n_pos, n_q, d)
    dq, dk, dv = (ctx.to_device(a) for a in (q, k, v))
    out = ctx.alloc(n_pos * n_q * d * 2).fill(0)
    ctx.call("attention_prefill", dq, dk, dv, out, n_q, n_kv, d, n_pos, start, cap, C.c_float(1 / np.sqrt(d)), window)
    got = out.download(np.float16, (n_pos, n_q, d))
    for t in range(n_pos):
        ref = oracle.attention_decode(q[t], k, v, n_q, n_kv, d, cap, start + t + 1, sliding_window=window)
        assert rel_err(got[t], ref) < REL_TOL, f"position {start + t}"
        assert inf_err(got[t], ref) < INF_TOL
    for b in (dq, dk, dv, out):
        b.free()


def rms_err(got, ref) -> float:
    g, r = got.astype(np.float32), ref.astype(np.float32)
    return float(np.max(np.abs(g - r)) / np.sqrt(np.mean(r * r)))


def make(ctx, cfg, seed, capacity):
    pkg = package.SyntheticPackage(cfg, seed)
    image, desc, layers = package.build_image(pkg, keep_for_oracle=True)
    return pkg, package.Decoder(ctx, image, desc, layers, capacity, 1, fuse_residual=3)


def kv_of(dec, cfg, cap):
    rows = []
    for l in range(2 * cfg.layers):
        raw = np.zeros(cfg.n_kv * cap * cfg.head_dim, np.float16)
        dec.ctx._check(dec.ctx.lib.smelt_cuda_read_slot(dec.ctx.h, package.KV_BASE_SLOT + l, 0, raw.ctypes.data_as(C.c_void_p), raw.nbytes))
        rows.append(raw.reshape(cfg.n_kv, cap, cfg.head_dim))
    return rows


@pytest.mark.parametrize("cfg,n_prompt,chunk", [(SMALL, 45, 0), (SMALL, 45, 7), (MID, 70, 32), (MID, 20, 0)])
def test_prefill_equals_token_by_token_decoding(ctx, oracle, cfg, n_prompt, chunk):
    """Same caches (within kernel tolerance), same next token and logits as feeding the prompt
    through decode steps; then the teacher-forced continuation matches the oracle's tokens."""
    cap, n_dec = n_prompt + 40, 24
    pkg, dec = make(ctx, cfg, 17, cap)
    prompt = synth.rng_for(17, "prefill prompt").integers(0, cfg.vocab, size=n_prompt).astype(np.int32)
    ref = oracle.model_from_package(pkg, cap)
    want, runner, margins = ref.greedy_top2(prompt, n_dec)
    tok_seq = None
    for i, t in enumerate(prompt):
        tok_seq = int(dec.decode_step([t], i)[0])
    logits_seq = dec.logits()[0].astype(np.float32)
    kv_seq = kv_of(dec, cfg, cap)
    dec.reset_cache()
    tok_pre = dec.prefill(prompt, 0, chunk)
    logits_pre = dec.logits()[0].astype(np.float32)
    kv_pre = kv_of(dec, cfg, cap)
    for l, (a, b) in enumerate(zip(kv_pre, kv_seq)):
        assert not a[:, n_prompt:].any(), "nothing is written beyond the prompt"
        # an fp16 ulp of difference per kernel (other fp32 summation order) travels up through the
        # layers: bound the worst element error by one percent of the cache's RMS, as for the logits
        assert rms_err(a[:, :n_prompt], b[:, :n_prompt]) < 1e-2, f"cache slot {l}"
    err = float(np.max(np.abs(logits_pre - logits_seq)) / np.sqrt(np.mean(logits_seq * logits_seq)))
    assert err < 1e-2, err
    v0 = package.compare_greedy(np.array([tok_pre]), want[:1], runner[:1], margins[:1])
    assert not v0["wrong"], (tok_pre, tok_seq, v0)
    # continue decoding from the prompt's end, teacher-forced on the oracle's tokens
    got = [tok_pre]
    for i in range(n_dec - 1):
        got.append(int(dec.decode_step([want[i]], n_prompt + i)[0]))
    v = package.compare_greedy(np.array(got), want, runner, margins)
    print("prefill + decode: %d of %d identical, %d tie breaks" % (v["identical"], v["checked"], v["tie_breaks"]))
    assert v["checked"] == n_dec and not v["wrong"], v


def test_prefill_in_two_calls_continues_the_cache(ctx, oracle):
    cfg, cap = SMALL, 64
    pkg, dec = make(ctx, cfg, 19, cap)
    prompt = synth.rng_for(19, "prefill prompt").integers(0, cfg.vocab, size=33).astype(np.int32)
    whole = dec.prefill(prompt)
    kv_whole = kv_of(dec, cfg, cap)
    dec.reset_cache()
    dec.prefill(prompt[:20])
    split = dec.prefill(prompt[20:], start_pos=20)
    assert split == whole
    for a, b in zip(kv_of(dec, cfg, cap), kv_whole):
        assert rms_err(a[:, :33], b[:, :33]) < 1e-2
    # past the capacity: refused before anything runs
    st = ctx.lib.smelt_cuda_prefill(ctx.h, C.byref(dec.desc), dec.layers, prompt.ctypes.data_as(C.c_void_p), 33, 40, 0, None)
    assert st == capi.OUT_OF_RANGE and "pass the limit" in ctx.last_error()


@pytest.mark.parametrize("cfg,n_prompt,chunk", [(SMALL, 45, 16), (MID, 70, 64), (MID, 20, 512)])
def test_prefill_table_equals_the_typed_driver(ctx, oracle, cfg, n_prompt, chunk):
    """The prompt through the prefill dispatch table in the reference's record shapes (seqLen / startPos constants,
    grid kinds, last-row offset) against the typed driver: same caches and logits within kernel tolerance, same next
    token; then the oracle's continuation from the table-filled cache."""
    cap, n_dec = n_prompt + 40, 16
    pkg, dec = make(ctx, cfg, 23, cap)
    prompt = synth.rng_for(23, "prefill prompt").integers(0, cfg.vocab, size=n_prompt).astype(np.int32)
    ref = oracle.model_from_package(pkg, cap)
    want, runner, margins = ref.greedy_top2(prompt, n_dec)
    tok_typed = dec.prefill(prompt, 0, chunk)
    logits_typed = dec.logits()[0].astype(np.float32)
    kv_typed = kv_of(dec, cfg, cap)
    dec.reset_cache()
    dec.build_prefill_table(chunk)
    tok_table = dec.prefill_by_table(prompt)
    logits_table = dec.logits()[0].astype(np.float32)
    kv_table = kv_of(dec, cfg, cap)
    for l, (a, b) in enumerate(zip(kv_table, kv_typed)):
        assert not a[:, n_prompt:].any(), "nothing is written beyond the prompt"
        assert rms_err(a[:, :n_prompt], b[:, :n_prompt]) < 1e-2, f"cache slot {l}"
    err = float(np.max(np.abs(logits_table - logits_typed)) / np.sqrt(np.mean(logits_typed * logits_typed)))
    assert err < 1e-2, err
    v0 = package.compare_greedy(np.array([tok_table]), want[:1], runner[:1], margins[:1])
    assert not v0["wrong"], (tok_table, tok_typed, v0)
    got = [tok_table]
    for i in range(n_dec - 1):
        got.append(int(dec.decode_step([want[i]], n_prompt + i)[0]))
    v = package.compare_greedy(np.array(got), want, runner, margins)
    assert v["checked"] == n_dec and not v["wrong"], v


def test_prefill_table_refuses_what_it_cannot_run(ctx):
    pkg, dec = make(ctx, SMALL, 29, 64)
    dec.build_prefill_table(16)
    toks = np.arange(20, dtype=np.int32)
    lib, h = ctx.lib, ctx.h
    n = len(dec.prefill_records)
    assert lib.smelt_cuda_enqueue_prefill(h, dec.prefill_records, n, toks.ctypes.data_as(C.c_void_p), 10, 60) == capi.OUT_OF_RANGE  # past the cache
    assert lib.smelt_cuda_enqueue_prefill(h, dec.prefill_records, n, toks.ctypes.data_as(C.c_void_p), 20, 0) == capi.OUT_OF_RANGE  # token slot holds 16 ids
    bad = toks.copy(); bad[3] = SMALL.vocab
    assert lib.smelt_cuda_enqueue_prefill(h, dec.prefill_records, n, bad.ctypes.data_as(C.c_void_p), 8, 0) == capi.OUT_OF_RANGE
    # a decode step refuses the prompt-chunk record kinds
    tok = np.zeros(1, np.int32)
    assert lib.smelt_cuda_enqueue_decode(h, dec.prefill_records, n, tok.ctypes.data_as(C.c_void_p), 0) == capi.UNSUPPORTED
