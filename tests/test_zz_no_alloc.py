"""smelt_cuda_attention_decode_static: the attention entry point whose split partials live in a
fixed device array.  It must give the bits of smelt_cuda_attention_decode, call after call, and
refuse shapes its array cannot hold.  The file name sorts last so that it also runs after every
other GPU test has used the device; it depends on none of them."""
import ctypes as C

import numpy as np
import pytest

from smelt_b200 import capi, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = capi.Context(0)
    yield c
    c.close()


def _case(ctx, seed, n_q, n_kv, d, seq_len, batch):
    cap = seq_len + 8
    k = synth.kv_cache(seed, "k", batch, n_kv, cap, d)
    v = synth.kv_cache(seed, "v", batch, n_kv, cap, d)
    q = synth.activations(seed, "q", batch, n_q, d)
    dq, dk, dv = (ctx.to_device(a) for a in (q, k, v))
    args = (n_q, n_kv, d, cap, seq_len, C.c_float(1 / np.sqrt(d)), 0, batch, C.c_size_t(n_kv * cap * d))
    return dq, dk, dv, args


def test_static_scratch_matches_the_allocating_entry_point_twice_in_a_row(ctx):
    # Calls in a row on different shapes: each reuses the array the one before wrote.  Up to 4096
    # keys the splits of a KV head merge inside a thread-block cluster and the array is not
    # touched; the cases above 4096 keys are the ones whose partials really live in it (and
    # are merged by the separate merge kernel, since this entry point owns no counters).
    for seed, (n_q, n_kv, d, seq_len, batch) in enumerate([(16, 4, 128, 8192, 1), (16, 4, 128, 6000, 4), (8, 2, 256, 20000, 1),
                                                            (32, 8, 128, 4096, 1), (16, 4, 128, 1000, 4)]):
        dq, dk, dv, args = _case(ctx, 40 + seed, n_q, n_kv, d, seq_len, batch)
        want = ctx.alloc(batch * n_q * d * 2).fill(0)
        got = ctx.alloc(batch * n_q * d * 2).fill(0xFF)
        ctx.call("attention_decode", dq, dk, dv, want, *args)
        ctx.call("attention_decode_static", dq, dk, dv, got, *args)
        w = want.download(np.uint16, (batch, n_q, d))
        g = got.download(np.uint16, (batch, n_q, d))
        assert np.array_equal(g, w)
        assert np.abs(w.view(np.float16).astype(np.float32)).max() > 1e-3
        # once more with the same inputs: no state carried from call to call
        ctx.call("attention_decode_static", dq, dk, dv, got.fill(0xFF), *args)
        assert np.array_equal(got.download(np.uint16, (batch, n_q, d)), w)
        for b in (dq, dk, dv, want, got):
            b.free()


def test_static_scratch_refuses_what_it_cannot_hold(ctx):
    d = ctx.alloc(4096)
    # batch * n_q * (head_dim + 2) = 8 * 32 * 130 = 33280 > 32768: refused before anything is read
    st = ctx.call_status("attention_decode_static", d, d, d, d, 32, 8, 128, 64, 64, C.c_float(0.088), 0, 8, 0)
    assert st == capi.OUT_OF_RANGE
    assert "32768" in ctx.last_error() and "smelt_cuda_attention_decode" in ctx.last_error()
    assert ctx.call_status("attention_decode_static", d, d, d, None, 32, 8, 128, 64, 64, C.c_float(0.088), 0, 1, 0) == capi.BAD_ARGUMENT
    assert ctx.call_status("attention_decode_static", d, d, d, d, 32, 8, 96, 64, 64, C.c_float(0.1), 0, 1, 0) == capi.UNSUPPORTED
    d.free()
