"""Prompt-state snapshots on a B200: the live prefix of the KV cache captured into private
device memory, restored (whole, partially, into a cache of another capacity, through host
bytes), must let decoding continue with exactly the tokens of the uninterrupted run
(SmeltRuntime.capturePromptSnapshot / restorePromptSnapshot, SmeltRuntime.swift:1254-1553)."""
import ctypes as C

import numpy as np
import pytest

from smelt_b200 import capi, package, synth

pytestmark = pytest.mark.gpu

CFG = package.DecoderConfig(layers=3, hidden=512, inter=1536, n_q=8, n_kv=2, head_dim=64, vocab=4096)


@pytest.fixture(scope="module")
def ctx():
    c = capi.Context(0)
    yield c
    c.close()


def make(ctx, capacity, batch=1, seed=21):
    pkg = package.SyntheticPackage(CFG, seed)
    image, desc, layers = package.build_image(pkg)
    return package.Decoder(ctx, image, desc, layers, capacity, batch, fuse_residual=3)


def feed(dec, tokens, start):
    """Decode `tokens` ([n, batch]) at positions start, start + 1, ...; returns the argmax after each."""
    out = []
    for i, t in enumerate(tokens):
        out.append(dec.decode_step(t, start + i).copy())
    return np.array(out)


def cache_rows(dec, layer, cap):
    raw = np.zeros(CFG.n_kv * dec.batch * cap * CFG.head_dim, np.uint16)
    dec.ctx._check(dec.ctx.lib.smelt_cuda_read_slot(dec.ctx.h, package.KV_BASE_SLOT + layer, 0, raw.ctypes.data_as(C.c_void_p), raw.nbytes))
    return raw.reshape(CFG.n_kv * dec.batch, cap, CFG.head_dim)


@pytest.mark.parametrize("batch", [1, 3])
def test_restore_continues_with_the_same_tokens(ctx, batch):
    cap, n_prompt, n_more = 64, 20, 12
    dec = make(ctx, cap, batch)
    prompt = synth.rng_for(3, "snap prompt").integers(0, CFG.vocab, size=(n_prompt, batch)).astype(np.int32)
    more = synth.rng_for(3, "snap more").integers(0, CFG.vocab, size=(n_more, batch)).astype(np.int32)
    feed(dec, prompt, 0)
    snap = dec.capture_snapshot(n_prompt, prompt_length=n_prompt, next_token=7)
    info = snap.info()
    assert (info.captured_length, info.prompt_length, info.next_token, info.n_slots) == (n_prompt, n_prompt, 7, 2 * CFG.layers)
    assert info.byte_count == 2 * CFG.layers * CFG.n_kv * batch * n_prompt * CFG.head_dim * 2
    want = feed(dec, more, n_prompt)
    k_before = cache_rows(dec, 1, cap)[:, :n_prompt].copy()
    dec.reset_cache()
    dec.restore_snapshot(snap)
    assert np.array_equal(cache_rows(dec, 1, cap)[:, :n_prompt], k_before), "the restored prefix is the captured one"
    assert not cache_rows(dec, 1, cap)[:, n_prompt:].any(), "nothing beyond the prefix is written"
    got = feed(dec, more, n_prompt)
    assert np.array_equal(got, want)
    snap.close()


def test_partial_restore_equals_the_shorter_prompt(ctx):
    """restorePromptSnapshot(_:length:) with length < captured: the cache holds the first
    `length` positions only, so decoding from there equals a run that never saw the rest."""
    cap, n_prompt, keep, n_more = 64, 24, 15, 8
    dec = make(ctx, cap)
    prompt = synth.rng_for(4, "snap prompt").integers(0, CFG.vocab, size=(n_prompt, 1)).astype(np.int32)
    more = synth.rng_for(4, "snap more").integers(0, CFG.vocab, size=(n_more, 1)).astype(np.int32)
    feed(dec, prompt[:keep], 0)
    want = feed(dec, more, keep)
    dec.reset_cache()
    feed(dec, prompt, 0)
    snap = dec.capture_snapshot(n_prompt)
    dec.reset_cache()
    dec.restore_snapshot(snap, keep)
    assert not cache_rows(dec, 0, cap)[:, keep:].any()
    assert np.array_equal(feed(dec, more, keep), want)
    # beyond the captured length: the reference throws (SmeltRuntime.swift:1333-1337)
    st = ctx.lib.smelt_cuda_snapshot_restore(ctx.h, snap.h, n_prompt + 1)
    assert st == capi.OUT_OF_RANGE and "outside [0, 24]" in ctx.last_error()
    snap.close()


def test_snapshot_survives_a_capacity_change_and_host_bytes(ctx):
    """A snapshot taken at capacity 32 is restored into a context whose caches hold 80
    positions (other row stride), directly and through the exported host blob."""
    n_prompt, n_more = 18, 10
    prompt = synth.rng_for(5, "snap prompt").integers(0, CFG.vocab, size=(n_prompt, 1)).astype(np.int32)
    more = synth.rng_for(5, "snap more").integers(0, CFG.vocab, size=(n_more, 1)).astype(np.int32)
    small = make(ctx, 32)
    feed(small, prompt, 0)
    snap = small.capture_snapshot(n_prompt)
    want = feed(small, more, n_prompt)
    blob = snap.export()
    assert blob.nbytes == snap.info().blob_bytes
    big = make(ctx, 80)  # same slots of the same context, reallocated at the larger capacity
    big.restore_snapshot(snap)
    assert np.array_equal(feed(big, more, n_prompt), want)
    big.reset_cache()
    again = package.Snapshot.from_blob(ctx, blob)
    assert again.info().byte_count == snap.info().byte_count
    big.restore_snapshot(again)
    assert np.array_equal(feed(big, more, n_prompt), want)
    # a damaged blob is refused, not trusted
    bad = blob.copy(); bad[0] ^= 0xFF
    h = C.c_void_p()
    assert ctx.lib.smelt_cuda_snapshot_import(ctx.h, bad.ctypes.data_as(C.c_void_p), C.c_size_t(bad.nbytes), C.byref(h)) == capi.BAD_ARGUMENT
    assert ctx.lib.smelt_cuda_snapshot_import(ctx.h, blob.ctypes.data_as(C.c_void_p), C.c_size_t(blob.nbytes - 64), C.byref(h)) == capi.BAD_ARGUMENT
    snap.close(); again.close()


def test_state_slots_are_copied_whole_and_cannot_be_rewound(ctx):
    """Position-less state (the recurrent / convolutional slots of hybrid packages): captured and
    restored whole; a restore shorter than the capture is refused (SmeltRuntime.swift:1338-1345)."""
    slot, nbytes = 30, 4096
    ctx.call("alloc_slot", slot, C.c_size_t(nbytes))
    state = synth.rng_for(6, "state").integers(0, 65536, size=nbytes // 2).astype(np.uint16)
    ctx._check(ctx.lib.smelt_cuda_write_slot(ctx.h, slot, C.c_size_t(0), state.ctypes.data_as(C.c_void_p), C.c_size_t(nbytes)))
    slots = (C.c_int32 * 2)(slot, 31)  # slot 31 does not exist: skipped, as the reference skips it
    h = C.c_void_p()
    ctx._check(ctx.lib.smelt_cuda_snapshot_capture(ctx.h, None, 0, slots, 2, 10, 10, 0, C.byref(h)))
    snap = package.Snapshot(ctx, h)
    assert snap.info().n_slots == 1 and snap.info().byte_count == nbytes
    ctx.call("zero_slot", slot)
    assert ctx.lib.smelt_cuda_snapshot_restore(ctx.h, snap.h, 5) == capi.UNSUPPORTED
    ctx._check(ctx.lib.smelt_cuda_snapshot_restore(ctx.h, snap.h, 10))
    back = np.zeros_like(state)
    ctx._check(ctx.lib.smelt_cuda_read_slot(ctx.h, slot, C.c_size_t(0), back.ctypes.data_as(C.c_void_p), C.c_size_t(nbytes)))
    assert np.array_equal(back, state)
    snap.close()
