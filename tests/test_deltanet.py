"""DeltaNet decode step: the oracle's restatement of the Metal kernels pinned on the closed-form
fixtures and float references the reference's own tests use (PrefillKernelTests.swift:583-609,
:1493-1577, :4352-4552), then the CUDA kernels against the oracle, typed and as records."""
import ctypes as C

import numpy as np
import pytest

from smelt_b200 import capi
from helpers import ulp_diff_f16

F = np.float32


def recurrence_fixture(head_dim=128, heads=16):
    """The inputs of testDeltaNetRecurrenceMlxDecode_GenericAndSpecializedMatchReference
    (PrefillKernelTests.swift:4400-4421): closed-form sin / cos ramps, Q and K L2-normalised
    (Q also times 1/sqrt(D)) in fp32 and rounded to fp16."""
    hidden = head_dim * heads
    i = np.arange(heads * head_dim * head_dim, dtype=F)
    state = (np.sin(i * F(0.0007)) * F(0.03)).astype(np.float16)
    c = np.arange(3 * hidden, dtype=F)
    qkv = (np.sin(c * F(0.0019)) * F(0.4)).astype(np.float16)
    h = np.arange(heads, dtype=F)
    b = (np.cos(h * F(0.017)) * F(0.9)).astype(np.float16)
    a = (np.sin(h * F(0.013)) * F(0.7)).astype(np.float16)
    a_log = (F(-1.2) + h * F(0.03)).astype(np.float16)
    dt_bias = (F(-0.2) + h * F(0.02)).astype(np.float16)
    q = qkv[:hidden].astype(F).reshape(heads, head_dim)
    k = qkv[hidden:2 * hidden].astype(F).reshape(heads, head_dim)
    q = q * (F(1 / np.sqrt(F(head_dim))) / np.maximum(np.sqrt((q * q).sum(1, keepdims=True)), F(1e-6)))
    k = k * (F(1) / np.maximum(np.sqrt((k * k).sum(1, keepdims=True)), F(1e-6)))
    qkv = np.concatenate([q.astype(np.float16).reshape(-1), k.astype(np.float16).reshape(-1), qkv[2 * hidden:]])
    return state, qkv, b, a, a_log, dt_bias


def recurrence_float_reference(state, qkv, b, a, a_log, dt_bias, head_dim, heads):
    """The test's own float reference (PrefillKernelTests.swift:4423-4441): no fp16 staging."""
    hidden = head_dim * heads
    st = state.astype(np.float64).reshape(heads, head_dim, head_dim).copy()
    x = qkv.astype(np.float64)
    out = np.zeros((heads, head_dim))
    for h in range(heads):
        q, k, v = x[h * head_dim:(h + 1) * head_dim], x[hidden + h * head_dim:hidden + (h + 1) * head_dim], x[2 * hidden + h * head_dim:2 * hidden + (h + 1) * head_dim]
        beta = 1 / (1 + np.exp(-float(b[h])))
        sp_in = float(a[h]) + float(dt_bias[h])
        sp = sp_in if sp_in > 20 else np.log1p(np.exp(sp_in))
        decay = np.exp(-np.exp(float(a_log[h])) * sp)
        st[h] *= decay
        delta = (v - st[h] @ k) * beta
        st[h] += np.outer(delta, k)
        out[h] = st[h] @ q
    return st, out


def test_oracle_recurrence_is_within_the_references_own_bound(oracle):
    """The reference asserts max |kernel - float reference| < 0.06 over output and state
    (PrefillKernelTests.swift:4551); the oracle's staged-fp16 restatement must sit well inside."""
    fx = recurrence_fixture()
    st, out = oracle.deltanet_recurrence_decode(*fx, 128, 16, 16)
    ref_st, ref_out = recurrence_float_reference(*fx, 128, 16)
    assert np.max(np.abs(out.astype(np.float64) - ref_out)) < 2e-3
    assert np.max(np.abs(st.astype(np.float64).reshape(ref_st.shape) - ref_st)) < 2e-3


def test_oracle_gated_norm_matches_the_references_cpu_reference(oracle):
    """testRmsNormGatedBatched_Qwen0808Shape_MatchesCPUReference: bound 1e-3 (PrefillKernelTests.swift:1577)."""
    d, heads = 128, 16 * 18
    i = np.arange(heads * d, dtype=F)
    x = (np.sin(i * F(0.0131)) * F(0.2)).astype(np.float16)
    g = (np.cos(i * F(0.0097)) * F(2.0)).astype(np.float16)
    w = (F(0.9) + F(0.2) * np.sin(np.arange(d, dtype=F) * F(0.021))).astype(np.float16)
    got = oracle.rms_norm_gated(x, g, w, d, 1e-6, heads).astype(F)
    xf, gf = x.astype(F).reshape(heads, d), g.astype(F).reshape(heads, d)
    rs = F(1) / np.sqrt((xf * xf).sum(1, keepdims=True) / F(d) + F(1e-6))
    ref = (w.astype(F) * (xf * rs) * (gf / (F(1) + np.exp(-gf)))).astype(np.float16).astype(F)
    assert np.max(np.abs(got - ref)) < 1e-3


def test_oracle_precise_gated_norm_matches_the_references_cpu_reference(oracle):
    """testRmsNormGatedD128Batched_Qwen0808Shape_MatchesCPUReference: 65 rows of 16 heads, bound 0.0021
    (PrefillKernelTests.swift:1585-1668); and the threadgroup-width form against the plain one."""
    d, heads = 128, 16 * 65
    i = np.arange(heads * d, dtype=F)
    x = (np.sin(i * F(0.0131)) * F(0.2)).astype(np.float16)
    g = (np.cos(i * F(0.0097)) * F(2.0)).astype(np.float16)
    w = (F(0.9) + F(0.2) * np.sin(np.arange(d, dtype=F) * F(0.021))).astype(np.float16)
    xf, gf = x.astype(F).reshape(heads, d), g.astype(F).reshape(heads, d)
    rs = F(1) / np.sqrt((xf * xf).sum(1, keepdims=True) / F(d) + F(1e-6))
    ref = (w.astype(F) * (xf * rs) * (gf / (F(1) + np.exp(-gf)))).astype(np.float16).astype(F)  # the test's reference rounds to fp16
    got = oracle.rms_norm_gated_d128(x, g, w, heads).astype(F)
    assert np.max(np.abs(got - ref)) < 0.0021
    for tgs in (32, 128):
        tg = oracle.rms_norm_gated_tg(x, g, w, d, 1e-6, heads, tgs)
        assert np.max(ulp_diff_f16(tg, oracle.rms_norm_gated(x, g, w, d, 1e-6, heads))) <= 1


def test_oracle_conv1d_shifts_and_activates(oracle):
    c, k = 96, 4
    rng = np.random.default_rng(3)
    state = rng.standard_normal((c, k)).astype(np.float16)
    new = rng.standard_normal(c).astype(np.float16)
    w = (rng.standard_normal((c, k)) * 0.5).astype(np.float16)
    st, out = oracle.conv1d_update_silu(state, new, w, c, k)
    st = st.reshape(c, k)
    assert np.array_equal(st[:, :3], state[:, 1:]) and np.array_equal(st[:, 3], new)
    acc = (st.astype(F) * w.astype(F)).sum(1).astype(np.float16).astype(F)
    ref = (acc / (1 + np.exp(-acc))).astype(np.float16)
    assert np.max(ulp_diff_f16(out, ref)) <= 2  # the staged fp16 sigmoid against the float one
    # an underflowed product is +0, never -0 (conv1d.metal:9-14)
    zs, zo = oracle.conv1d_update_silu(np.zeros((1, 4), np.float16), np.array([0x8001], np.uint16).view(np.float16), np.ones((1, 4), np.float16), 1, 4)
    assert zo.view(np.uint16)[0] == 0


# ── CUDA against the oracle ──
@pytest.fixture(scope="module")
def ctx():
    c = capi.Context(0)
    yield c
    c.close()


@pytest.mark.gpu
@pytest.mark.parametrize("channels,ksize", [(6144, 4), (1000, 4), (512, 3), (64, 8)])
def test_conv1d_update_silu(ctx, oracle, channels, ksize):
    rng = np.random.default_rng(channels + ksize)
    state = rng.standard_normal((channels, ksize)).astype(np.float16)
    new = rng.standard_normal(channels).astype(np.float16)
    w = (rng.standard_normal((channels, ksize)) * 0.5).astype(np.float16)
    ds, dn, dw = (ctx.to_device(a) for a in (state, new, w))
    out = ctx.alloc(channels * 2)
    ctx.call("conv1d_update_silu", ds, dn, dw, out, channels, ksize)
    want_state, want = oracle.conv1d_update_silu(state, new, w, channels, ksize)
    assert np.array_equal(ds.download(np.uint16, (channels * ksize,)), want_state.view(np.uint16).reshape(-1)), "the shifted state is exact"
    assert np.max(ulp_diff_f16(out.download(np.float16, (channels,)), want)) <= 1  # expf of the two libraries


@pytest.mark.gpu
@pytest.mark.parametrize("head_dim,qk_heads,v_heads,batch", [(128, 16, 16, 1), (128, 16, 32, 3), (64, 4, 4, 2), (256, 2, 2, 1)])
def test_rms_scale_qk(ctx, oracle, head_dim, qk_heads, v_heads, batch):
    qkv_dim = (2 * qk_heads + v_heads) * head_dim
    x = np.random.default_rng(head_dim).standard_normal((batch, qkv_dim)).astype(np.float16)
    dx = ctx.to_device(x)
    ctx.call("rms_scale_qk", dx, head_dim, C.c_float(1e-6), qkv_dim, qk_heads, batch)
    got = dx.download(np.float16, (batch, qkv_dim))
    want = oracle.rms_scale_qk(x, head_dim, 1e-6, qkv_dim, qk_heads, batch).reshape(batch, qkv_dim)
    assert np.array_equal(got[:, 2 * qk_heads * head_dim:], x[:, 2 * qk_heads * head_dim:]), "V is not touched"
    # another fp32 order of the sum of squares can flip the first fp16 rounding by an ulp, and the
    # second rounding (times the edge scale) can carry that to two
    assert np.max(ulp_diff_f16(got, want)) <= 2


@pytest.mark.gpu
@pytest.mark.parametrize("head_dim,v_heads,qk_heads", [(128, 16, 16), (128, 32, 16), (128, 48, 16), (64, 8, 4), (256, 4, 2)])
def test_deltanet_recurrence_decode(ctx, oracle, head_dim, v_heads, qk_heads):
    rng = np.random.default_rng(head_dim + v_heads)
    state = (rng.standard_normal((v_heads, head_dim, head_dim)) * 0.05).astype(np.float16)
    qkv = rng.standard_normal((2 * qk_heads + v_heads) * head_dim).astype(F)
    for g in range(2 * qk_heads):  # unit-norm q and k, as rms_scale_qk leaves them up to the edge scales
        seg = qkv[g * head_dim:(g + 1) * head_dim]
        seg /= np.linalg.norm(seg)
    qkv = qkv.astype(np.float16)
    b, a = rng.standard_normal(v_heads).astype(np.float16), rng.standard_normal(v_heads).astype(np.float16)
    a_log = rng.uniform(-2, 0.5, v_heads).astype(np.float16)
    dt = rng.uniform(-0.5, 0.5, v_heads).astype(np.float16)
    dev = [ctx.to_device(t) for t in (state, qkv, b, a, a_log, dt)]
    out = ctx.alloc(v_heads * head_dim * 2)
    want_state, want = oracle.deltanet_recurrence_decode(state, qkv, b, a, a_log, dt, head_dim, v_heads, qk_heads)
    for step in range(2):  # two steps: the second reads the state the first wrote
        ctx.call("deltanet_recurrence_decode", *dev, out, head_dim, v_heads, qk_heads)
        got = out.download(np.float16, (v_heads, head_dim))
        got_state = dev[0].download(np.float16, (v_heads, head_dim, head_dim))
        assert np.max(np.abs(got.astype(F) - want.astype(F))) <= 2e-3 * max(1.0, float(np.max(np.abs(want.astype(F))))), f"step {step}"
        assert np.max(ulp_diff_f16(got_state, want_state.reshape(got_state.shape))) <= 1 + step, f"state, step {step}"
        want_state, want = oracle.deltanet_recurrence_decode(want_state, qkv, b, a, a_log, dt, head_dim, v_heads, qk_heads)


@pytest.mark.gpu
def test_deltanet_reference_fixture(ctx):
    """The reference test's fixture through the CUDA kernel, against the reference test's float
    reference and bound (0.06, PrefillKernelTests.swift:4551)."""
    fx = recurrence_fixture()
    dev = [ctx.to_device(t) for t in fx]
    out = ctx.alloc(16 * 128 * 2)
    ctx.call("deltanet_recurrence_decode", *dev, out, 128, 16, 16)
    ref_st, ref_out = recurrence_float_reference(*fx, 128, 16)
    assert np.max(np.abs(out.download(np.float16, (16, 128)).astype(np.float64) - ref_out)) < 0.06
    assert np.max(np.abs(dev[0].download(np.float16, (16, 128, 128)).astype(np.float64) - ref_st)) < 0.06


@pytest.mark.gpu
@pytest.mark.parametrize("head_dim,heads", [(128, 16), (128, 288), (64, 5), (256, 3)])
def test_rms_norm_gated(ctx, oracle, head_dim, heads):
    rng = np.random.default_rng(heads)
    x = (rng.standard_normal((heads, head_dim)) * 0.3).astype(np.float16)
    g = (rng.standard_normal((heads, head_dim)) * 2).astype(np.float16)
    w = (0.9 + 0.2 * rng.standard_normal(head_dim)).astype(np.float16)
    dx, dg, dw = (ctx.to_device(t) for t in (x, g, w))
    ctx.call("rms_norm_gated", dx, dg, dw, dx, head_dim, C.c_float(1e-6), heads)  # in place, as the emitter binds it
    got = dx.download(np.float16, (heads, head_dim))
    want = oracle.rms_norm_gated(x, g, w, head_dim, 1e-6, heads)
    assert np.max(ulp_diff_f16(got, want)) <= 1


@pytest.mark.gpu
@pytest.mark.parametrize("tgs,precise", [(32, 1), (32, 0), (128, 0), (64, 0)])
def test_rms_norm_gated_threadgroup_forms(ctx, oracle, tgs, precise):
    heads, d = 97, 128
    rng = np.random.default_rng(tgs + precise)
    x = (rng.standard_normal((heads, d)) * 0.3).astype(np.float16)
    g = (rng.standard_normal((heads, d)) * 2).astype(np.float16)
    w = (0.9 + 0.2 * rng.standard_normal(d)).astype(np.float16)
    dx, dg, dw = (ctx.to_device(t) for t in (x, g, w))
    out = ctx.alloc(heads * d * 2)
    ctx.call("rms_norm_gated_ex", dx, dg, dw, out, d, C.c_float(1e-6), heads, tgs, precise)
    want = oracle.rms_norm_gated_d128(x, g, w, heads) if precise else oracle.rms_norm_gated_tg(x, g, w, d, 1e-6, heads, tgs)
    ulp = ulp_diff_f16(out.download(np.float16, (heads, d)), want)
    assert np.max(ulp) <= 1 and np.mean(ulp == 0) > 0.99  # expf of the two libraries


@pytest.mark.gpu
def test_deltanet_records_run_the_layer_core(ctx, oracle):
    """The four records the reference's emitter writes for a DeltaNet layer's core
    (DeltaNetPlugin.swift:196-318), with its pipeline names and bindings, eagerly."""
    d, hqk, hv, k = 128, 16, 32, 4
    qkv_dim = (2 * hqk + hv) * d
    rng = np.random.default_rng(9)
    conv_state = rng.standard_normal((qkv_dim, k)).astype(np.float16)
    qkv_in = rng.standard_normal(qkv_dim).astype(np.float16)
    conv_w = (rng.standard_normal((qkv_dim, k)) * 0.5).astype(np.float16)
    rec_state = (rng.standard_normal((hv, d, d)) * 0.05).astype(np.float16)
    b, a = rng.standard_normal(hv).astype(np.float16), rng.standard_normal(hv).astype(np.float16)
    a_log, dt = rng.uniform(-2, 0.5, hv).astype(np.float16), rng.uniform(-0.5, 0.5, hv).astype(np.float16)
    z = (rng.standard_normal(hv * d) * 2).astype(np.float16)
    norm_w = (0.9 + 0.2 * rng.standard_normal(d)).astype(np.float16)
    tensors = {2: conv_state, 3: qkv_in, 4: conv_w, 5: rec_state, 6: b, 7: a, 9: a_log, 10: dt, 11: np.zeros(hv * d, np.float16), 12: z, 13: norm_w}
    for slot, t in tensors.items():
        ctx.call("alloc_slot", slot, C.c_size_t(t.nbytes))
        ctx._check(ctx.lib.smelt_cuda_write_slot(ctx.h, slot, C.c_size_t(0), t.ctypes.data_as(C.c_void_p), C.c_size_t(t.nbytes)))
    cfg = capi.RuntimeConfig(0, 1, 2, 2, 0, 1, 64, 64, 16, 1)
    for slot in (0, 1):
        ctx.call("alloc_slot", slot, C.c_size_t(64))
    ctx._check(ctx.lib.smelt_cuda_configure(ctx.h, C.byref(cfg)))
    names = ["conv1d_update_silu", "rms_scale_qk", "deltanet_recurrence_mlx_decode_d128_h32_qk16", "rms_norm_gated_d128"]
    for i, n in enumerate(names):
        ctx._check(ctx.lib.smelt_cuda_register_pipeline(ctx.h, i, n.encode()))
    f32 = lambda v: int(np.array([v], F).view(np.uint32)[0])

    def rec(pipe, grid, bufs, cons):
        r = capi.DispatchRecord()
        r.op_kind, r.pipeline, r.buffer_count, r.constant_count = 0, pipe, len(bufs), len(cons)
        r.grid[0], r.grid[1], r.grid[2] = grid[0], grid[1], 1
        for j, (binding, slot) in enumerate(bufs):
            r.buf[j].slot, r.buf[j].binding_index, r.buf[j].offset_kind, r.buf[j].offset = slot, binding, 0, 0
        for j, (binding, kind, value) in enumerate(cons):
            r.con[j].kind, r.con[j].binding_index, r.con[j].value = kind, binding, value
        return r

    table = (capi.DispatchRecord * 4)(
        rec(0, (qkv_dim, 1), [(0, 2), (1, 3), (2, 4), (3, 3)], [(4, 0, qkv_dim), (5, 0, k)]),
        rec(1, (2 * hqk, 1), [(0, 3)], [(1, 0, d), (2, 1, f32(1e-6)), (3, 0, qkv_dim), (4, 0, hqk)]),
        rec(2, (32, d), [(0, 5), (1, 3), (2, 6), (3, 7), (4, 9), (5, 10), (6, 11)], []),
        rec(3, (hv, 1), [(0, 11), (1, 12), (2, 13), (3, 11)], []))
    tok = np.zeros(1, np.int32)
    ctx._check(ctx.lib.smelt_cuda_enqueue_decode(ctx.h, table, 4, tok.ctypes.data_as(C.c_void_p), 0))
    ctx.synchronize()
    got = np.zeros(hv * d, np.float16)
    ctx._check(ctx.lib.smelt_cuda_read_slot(ctx.h, 11, C.c_size_t(0), got.ctypes.data_as(C.c_void_p), C.c_size_t(got.nbytes)))
    st, act = oracle.conv1d_update_silu(conv_state, qkv_in, conv_w, qkv_dim, k)
    scaled = oracle.rms_scale_qk(act, d, 1e-6, qkv_dim, hqk)
    rst, core = oracle.deltanet_recurrence_decode(rec_state, scaled, b, a, a_log, dt, d, hv, hqk)
    want = oracle.rms_norm_gated_d128(core, z, norm_w, hv).reshape(-1)  # the record names the precise d128 form
    err = float(np.max(np.abs(got.astype(F) - want.astype(F))) / np.sqrt(np.mean(want.astype(F) ** 2)))
    assert err < 5e-3, err


# ── prompt-chunk forms (conv1d.metal:129-268, prefill_recurrence.metal:290-775) ──
def prefill_fixture(seq_len, head_dim=128, heads=16):
    """The inputs of testDeltaNetRecurrenceMlxPrefill_LargeBatchBoundaries
    (PrefillKernelTests.swift:4253-4264): the decode fixture's ramps over seq_len rows."""
    hidden = head_dim * heads
    i = np.arange(heads * head_dim * head_dim, dtype=F)
    state = (np.sin(i * F(0.0007)) * F(0.03)).astype(np.float16)
    c = np.arange(seq_len * 3 * hidden, dtype=F)
    qkv = (np.sin(c * F(0.0019)) * F(0.4)).astype(np.float16).reshape(seq_len, 3 * hidden)
    j = np.arange(seq_len * heads, dtype=F)
    b = (np.cos(j * F(0.017)) * F(0.9)).astype(np.float16)
    a = (np.sin(j * F(0.013)) * F(0.7)).astype(np.float16)
    h = np.arange(heads, dtype=F)
    a_log = (F(-1.2) + h * F(0.03)).astype(np.float16)
    dt_bias = (F(-0.2) + h * F(0.02)).astype(np.float16)
    q = qkv[:, :hidden].astype(F).reshape(seq_len, heads, head_dim)
    k = qkv[:, hidden:2 * hidden].astype(F).reshape(seq_len, heads, head_dim)
    q = q * (F(1 / np.sqrt(F(head_dim))) / np.maximum(np.sqrt((q * q).sum(2, keepdims=True)), F(1e-6)))
    k = k * (F(1) / np.maximum(np.sqrt((k * k).sum(2, keepdims=True)), F(1e-6)))
    qkv = np.concatenate([q.astype(np.float16).reshape(seq_len, hidden), k.astype(np.float16).reshape(seq_len, hidden), qkv[:, 2 * hidden:]], axis=1)
    return state, np.ascontiguousarray(qkv), b, a, a_log, dt_bias


def prefill_float_reference(state, qkv, b, a, a_log, dt_bias, head_dim, heads, seq_len):
    """The test's own float reference (PrefillKernelTests.swift:4275-4304)."""
    st = state.reshape(heads, head_dim, head_dim)
    out = np.zeros((seq_len, heads, head_dim))
    bb, aa = b.reshape(seq_len, heads), a.reshape(seq_len, heads)
    for pos in range(seq_len):
        row = (qkv[pos], bb[pos], aa[pos], a_log, dt_bias)
        st, out[pos] = recurrence_float_reference(st, *row, head_dim, heads)
    return st, out


def random_chunk(rng, seq_len, head_dim, v_heads, qk_heads):
    state = (rng.standard_normal((v_heads, head_dim, head_dim)) * 0.05).astype(np.float16)
    qkv = rng.standard_normal((seq_len, 2 * qk_heads + v_heads, head_dim)).astype(F)
    qkv[:, :2 * qk_heads] /= np.linalg.norm(qkv[:, :2 * qk_heads], axis=2, keepdims=True)
    qkv = qkv.astype(np.float16).reshape(seq_len, -1)
    b, a = rng.standard_normal(seq_len * v_heads).astype(np.float16), rng.standard_normal(seq_len * v_heads).astype(np.float16)
    a_log = rng.uniform(-2, 0.5, v_heads).astype(np.float16)
    dt = rng.uniform(-0.5, 0.5, v_heads).astype(np.float16)
    return state, qkv, b, a, a_log, dt


@pytest.mark.parametrize("seq_len", [64, 65])
def test_oracle_prefill_recurrence_is_within_the_references_own_bound(oracle, seq_len):
    """The reference asserts max |kernel - float reference| < 0.03 over outputs and final state
    at 64 and 65 positions (PrefillKernelTests.swift:4349)."""
    fx = prefill_fixture(seq_len)
    st, out, _ = oracle.deltanet_recurrence_prefill(*fx, 128, 16, 16, seq_len)
    ref_st, ref_out = prefill_float_reference(*fx, 128, 16, seq_len)
    assert np.max(np.abs(out.astype(np.float64) - ref_out)) < 3e-3
    assert np.max(np.abs(st.astype(np.float64).reshape(ref_st.shape) - ref_st)) < 3e-3


def test_oracle_prefill_of_one_position_is_the_decode_step(oracle):
    """testDeltaNetGenericRecurrenceSingleTokenPrefillIsBitExactWithDecode (PrefillKernelTests.swift:4977):
    same bits; and the checkpoint form over T positions is T decode steps, history included."""
    rng = np.random.default_rng(5)
    d, hv, hqk, t = 64, 8, 4, 5
    fx = random_chunk(rng, t, d, hv, hqk)
    state, qkv, b, a, a_log, dt = fx
    st1, out1, _ = oracle.deltanet_recurrence_prefill(state, qkv[:1], b[:hv], a[:hv], a_log, dt, d, hv, hqk, 1)
    st_d, out_d = oracle.deltanet_recurrence_decode(state, qkv[0], b[:hv], a[:hv], a_log, dt, d, hv, hqk)
    assert np.array_equal(st1.view(np.uint16), st_d.view(np.uint16)) and np.array_equal(out1.reshape(-1).view(np.uint16), out_d.reshape(-1).view(np.uint16))
    st_c, out_c, hist = oracle.deltanet_recurrence_prefill(*fx, d, hv, hqk, t, history=True)
    st_i = state
    assert np.array_equal(hist[0].view(np.uint16), state.view(np.uint16))
    for pos in range(t):
        st_i, o = oracle.deltanet_recurrence_decode(st_i, qkv[pos], b[pos * hv:(pos + 1) * hv], a[pos * hv:(pos + 1) * hv], a_log, dt, d, hv, hqk)
        assert np.array_equal(o.view(np.uint16), out_c[pos].view(np.uint16)), pos
        assert np.array_equal(st_i.reshape(hv, d, d).view(np.uint16), hist[pos + 1].view(np.uint16)), pos
    assert np.array_equal(st_c.view(np.uint16), st_i.view(np.uint16))
    # the fp32-resident form is a different trajectory: close, not equal
    st_f, out_f, _ = oracle.deltanet_recurrence_prefill(*fx, d, hv, hqk, t)
    assert np.max(np.abs(out_f.astype(F) - out_c.astype(F))) < 2e-2


def test_oracle_conv1d_prefill_is_the_iterated_update(oracle):
    rng = np.random.default_rng(6)
    c, k, t = 96, 4, 7
    state = rng.standard_normal((c, k)).astype(np.float16)
    x = rng.standard_normal((t, c)).astype(np.float16)
    w = (rng.standard_normal((c, k)) * 0.5).astype(np.float16)
    st, y, hist = oracle.conv1d_update_silu_prefill(state, x, w, t, c, k, history=True)
    cur = state
    assert np.array_equal(hist[0].view(np.uint16), state.view(np.uint16))
    for pos in range(t):
        cur, o = oracle.conv1d_update_silu(cur, x[pos], w, c, k)
        assert np.array_equal(o.view(np.uint16), y[pos].view(np.uint16))
        assert np.array_equal(cur.reshape(c, k).view(np.uint16), hist[pos + 1].view(np.uint16))
    assert np.array_equal(st.view(np.uint16), cur.view(np.uint16))


@pytest.mark.gpu
@pytest.mark.parametrize("channels,ksize,seq_len,history", [(6144, 4, 65, False), (6144, 4, 3, True), (1000, 4, 64, False), (512, 3, 17, True), (64, 8, 1, False), (64, 8, 0, False)])
def test_conv1d_update_silu_prefill(ctx, oracle, channels, ksize, seq_len, history):
    rng = np.random.default_rng(channels + ksize + seq_len)
    state = rng.standard_normal((channels, ksize)).astype(np.float16)
    x = rng.standard_normal((max(seq_len, 1), channels)).astype(np.float16)
    w = (rng.standard_normal((channels, ksize)) * 0.5).astype(np.float16)
    ds, dx, dw = (ctx.to_device(t) for t in (state, x, w))
    hist = ctx.alloc((seq_len + 1) * channels * ksize * 2).fill(0) if history else None
    ctx.call("conv1d_update_silu_prefill", ds, dx, dw, seq_len, channels, ksize, hist)
    want_state, want, want_hist = oracle.conv1d_update_silu_prefill(state, x[:seq_len], w, seq_len, channels, ksize, history=history)
    assert np.array_equal(ds.download(np.uint16, (channels * ksize,)), want_state.view(np.uint16).reshape(-1)), "the taps are exact"
    got = dx.download(np.float16, x.shape)
    if seq_len:
        assert np.max(ulp_diff_f16(got[:seq_len], want)) <= 1  # expf of the two libraries
    else:
        assert np.array_equal(got.view(np.uint16), x.view(np.uint16))
    if history:
        assert np.array_equal(hist.download(np.uint16, want_hist.shape), want_hist.view(np.uint16))


@pytest.mark.gpu
@pytest.mark.parametrize("head_dim,v_heads,qk_heads,seq_len,history",
                         [(128, 16, 16, 65, False), (128, 32, 16, 64, False), (128, 48, 16, 130, False), (64, 8, 4, 255, False), (256, 4, 2, 33, False),
                          (128, 16, 16, 1, False), (128, 16, 16, 9, True), (64, 8, 4, 130, True)])
def test_deltanet_recurrence_prefill(ctx, oracle, head_dim, v_heads, qk_heads, seq_len, history):
    rng = np.random.default_rng(head_dim + v_heads + seq_len)
    fx = random_chunk(rng, seq_len, head_dim, v_heads, qk_heads)
    dev = [ctx.to_device(t) for t in fx]
    out = ctx.alloc(seq_len * v_heads * head_dim * 2)
    hist = ctx.alloc((seq_len + 1) * v_heads * head_dim * head_dim * 2).fill(0) if history else None
    ctx.call("deltanet_recurrence_prefill", *dev, out, head_dim, v_heads, qk_heads, seq_len, hist)
    want_state, want, want_hist = oracle.deltanet_recurrence_prefill(*fx, head_dim, v_heads, qk_heads, seq_len, history=history)
    got = out.download(np.float16, want.shape).astype(F)
    got_state = dev[0].download(np.float16, (v_heads, head_dim, head_dim))
    # the same fp32 operations in the same order; a gate whose expf differs by an ulp between the two
    # libraries can move one fp16 rounding, which the following positions carry along
    scale = max(1.0, float(np.max(np.abs(want.astype(F)))))
    assert np.max(np.abs(got - want.astype(F))) <= 2e-3 * scale
    assert np.max(np.abs(got_state.astype(F) - want_state.reshape(got_state.shape).astype(F))) <= 2e-3
    assert np.mean(got.view(np.uint32) == want.astype(F).view(np.uint32)) > 0.98, "all but a few values carry the same bits"
    if history:
        gh = hist.download(np.float16, want_hist.shape).astype(F)
        assert np.array_equal(gh[0], fx[0].astype(F))
        assert np.max(np.abs(gh - want_hist.astype(F))) <= 2e-3


@pytest.mark.gpu
def test_deltanet_prefill_reference_fixture(ctx):
    """The reference test's fixture at 65 positions through the CUDA kernel, against the test's
    float reference and bound (0.03, PrefillKernelTests.swift:4349)."""
    fx = prefill_fixture(65)
    dev = [ctx.to_device(t) for t in fx]
    out = ctx.alloc(65 * 16 * 128 * 2)
    ctx.call("deltanet_recurrence_prefill", *dev, out, 128, 16, 16, 65, None)
    ref_st, ref_out = prefill_float_reference(*fx, 128, 16, 65)
    assert np.max(np.abs(out.download(np.float16, (65, 16, 128)).astype(np.float64) - ref_out)) < 0.03
    assert np.max(np.abs(dev[0].download(np.float16, (16, 128, 128)).astype(np.float64) - ref_st)) < 0.03


@pytest.mark.gpu
def test_deltanet_prefill_records(ctx, oracle):
    """The prompt-chunk records with the reference's pipeline names and bindings, eagerly:
    conv1d_update_silu_c6144_k4_prefill -> rms_scale_qk (grid.y = positions) ->
    deltanet_recurrence_mlx_prefill_d128_h16."""
    d, h, k, t = 128, 16, 4, 12
    qkv_dim = 3 * h * d
    rng = np.random.default_rng(11)
    conv_state = rng.standard_normal((qkv_dim, k)).astype(np.float16)
    x = rng.standard_normal((t, qkv_dim)).astype(np.float16)
    conv_w = (rng.standard_normal((qkv_dim, k)) * 0.5).astype(np.float16)
    rec_state = (rng.standard_normal((h, d, d)) * 0.05).astype(np.float16)
    b, a = rng.standard_normal(t * h).astype(np.float16), rng.standard_normal(t * h).astype(np.float16)
    a_log, dt = rng.uniform(-2, 0.5, h).astype(np.float16), rng.uniform(-0.5, 0.5, h).astype(np.float16)
    tensors = {2: conv_state, 3: x, 4: conv_w, 5: rec_state, 6: b, 7: a, 9: a_log, 10: dt, 11: np.zeros(t * h * d, np.float16)}
    for slot, tens in tensors.items():
        ctx.call("alloc_slot", slot, C.c_size_t(tens.nbytes))
        ctx._check(ctx.lib.smelt_cuda_write_slot(ctx.h, slot, C.c_size_t(0), tens.ctypes.data_as(C.c_void_p), C.c_size_t(tens.nbytes)))
    cfg = capi.RuntimeConfig(0, 1, 2, 2, 0, 1, 64, 64, 16, 1)
    for slot in (0, 1):
        ctx.call("alloc_slot", slot, C.c_size_t(64))
    ctx._check(ctx.lib.smelt_cuda_configure(ctx.h, C.byref(cfg)))
    names = ["conv1d_update_silu_c6144_k4_prefill", "rms_scale_qk", "deltanet_recurrence_mlx_prefill_d128_h16"]
    for i, n in enumerate(names):
        ctx._check(ctx.lib.smelt_cuda_register_pipeline(ctx.h, 8 + i, n.encode()))
    f32 = lambda v: int(np.array([v], F).view(np.uint32)[0])

    def rec(pipe, grid, bufs, cons):
        r = capi.DispatchRecord()
        r.op_kind, r.pipeline, r.buffer_count, r.constant_count = 0, pipe, len(bufs), len(cons)
        r.grid[0], r.grid[1], r.grid[2] = grid[0], grid[1], 1
        for j, (binding, slot) in enumerate(bufs):
            r.buf[j].slot, r.buf[j].binding_index, r.buf[j].offset_kind, r.buf[j].offset = slot, binding, 0, 0
        for j, (binding, kind, value) in enumerate(cons):
            r.con[j].kind, r.con[j].binding_index, r.con[j].value = kind, binding, value
        return r

    table = (capi.DispatchRecord * 3)(
        rec(8, (qkv_dim, 1), [(0, 2), (1, 3), (2, 4)], [(3, 0, t)]),
        rec(9, (2 * h, t), [(0, 3)], [(1, 0, d), (2, 1, f32(1e-6)), (3, 0, qkv_dim), (4, 0, h)]),
        rec(10, (32, d), [(0, 5), (1, 3), (2, 6), (3, 7), (4, 9), (5, 10), (6, 11)], [(7, 0, t)]))
    tok = np.zeros(1, np.int32)
    ctx._check(ctx.lib.smelt_cuda_enqueue_decode(ctx.h, table, 3, tok.ctypes.data_as(C.c_void_p), 0))
    ctx.synchronize()
    got = np.zeros(t * h * d, np.float16)
    ctx._check(ctx.lib.smelt_cuda_read_slot(ctx.h, 11, C.c_size_t(0), got.ctypes.data_as(C.c_void_p), C.c_size_t(got.nbytes)))
    st, act, _ = oracle.conv1d_update_silu_prefill(conv_state, x, conv_w, t, qkv_dim, k)
    scaled = oracle.rms_scale_qk(act, d, 1e-6, qkv_dim, h, t).reshape(t, qkv_dim)
    rst, core, _ = oracle.deltanet_recurrence_prefill(rec_state, scaled, b, a, a_log, dt, d, h, h, t)
    want = core.reshape(-1).astype(F)
    err = float(np.max(np.abs(got.astype(F) - want)) / np.sqrt(np.mean(want ** 2)))
    assert err < 5e-3, err


@pytest.mark.gpu
def test_fused_conv_l2_record_equals_the_staged_pair(ctx, oracle):
    """conv1d_update_silu_l2_qk_c6144_k4_d128_h16 against conv1d_update_silu_c6144_k4 then l2_normalize_d128 on the 32
    Q / K heads (the reference's own assertion, PrefillKernelTests.swift:5294-5364), in place as the emitter binds it."""
    rng = np.random.default_rng(21)
    c, k = 6144, 4
    state = rng.standard_normal((c, k)).astype(np.float16)
    new = rng.standard_normal(c).astype(np.float16)
    w = (rng.standard_normal((c, k)) * 0.5).astype(np.float16)
    for slot, t in {2: state, 3: new, 4: w}.items():
        ctx.call("alloc_slot", slot, C.c_size_t(t.nbytes))
        ctx._check(ctx.lib.smelt_cuda_write_slot(ctx.h, slot, C.c_size_t(0), t.ctypes.data_as(C.c_void_p), C.c_size_t(t.nbytes)))
    cfg = capi.RuntimeConfig(0, 1, 2, 2, 0, 1, 64, 64, 16, 1)
    for slot in (0, 1):
        ctx.call("alloc_slot", slot, C.c_size_t(64))
    ctx._check(ctx.lib.smelt_cuda_configure(ctx.h, C.byref(cfg)))
    ctx._check(ctx.lib.smelt_cuda_register_pipeline(ctx.h, 80, b"conv1d_update_silu_l2_qk_c6144_k4_d128_h16"))
    r = capi.DispatchRecord()
    r.op_kind, r.pipeline, r.buffer_count, r.constant_count = 0, 80, 4, 0
    r.grid[0], r.grid[1], r.grid[2] = 48, 1, 1
    r.threadgroup[0] = 128
    for j, (binding, slot) in enumerate([(0, 2), (1, 3), (2, 4), (3, 3)]):
        r.buf[j].slot, r.buf[j].binding_index = slot, binding
    tok = np.zeros(1, np.int32)
    ctx._check(ctx.lib.smelt_cuda_enqueue_decode(ctx.h, (capi.DispatchRecord * 1)(r), 1, tok.ctypes.data_as(C.c_void_p), 0))
    ctx.synchronize()
    got = np.zeros(c, np.float16)
    ctx._check(ctx.lib.smelt_cuda_read_slot(ctx.h, 3, C.c_size_t(0), got.ctypes.data_as(C.c_void_p), C.c_size_t(got.nbytes)))
    got_state = np.zeros((c, k), np.float16)
    ctx._check(ctx.lib.smelt_cuda_read_slot(ctx.h, 2, C.c_size_t(0), got_state.ctypes.data_as(C.c_void_p), C.c_size_t(got_state.nbytes)))
    want_state, act = oracle.conv1d_update_silu(state, new, w, c, k)
    want = act.copy()
    want[:32 * 128] = oracle.row_norm(act[:32 * 128].reshape(32, 128), None, topology=2, value=4, tgs=128, scale=1)[0].reshape(-1)
    assert np.array_equal(got_state.view(np.uint16), want_state.reshape(c, k).view(np.uint16))
    assert np.max(ulp_diff_f16(got, want)) <= 2  # expf of the two libraries inside the staged SiLU, carried through the norm
    assert np.array_equal(got[32 * 128:].view(np.uint16) == act[32 * 128:].view(np.uint16), np.ones(c - 32 * 128, bool)) or np.max(ulp_diff_f16(got[32 * 128:], act[32 * 128:])) <= 1


def test_hybrid_table_follows_the_plugins_record_order():
    """smelt_cuda_build_hybrid_decoder without a context: a DeltaNet layer is norm, four projections, conv, Q / K
    scaling, recurrence, gated norm, output projection + residual (DeltaNetPlugin.swift:60-420), then the feed-forward half."""
    from smelt_b200 import package
    cfg = package.DecoderConfig(layers=2, hidden=512, inter=1024, n_q=4, n_kv=2, head_dim=64, vocab=512, delta_layers=(0,),
                                delta_value_heads=8, delta_qk_heads=4, delta_head_dim=64)
    image, desc, layers, hy = package.build_hybrid_image(package.SyntheticPackage(cfg, 1))
    lib = capi.load()
    n = C.c_size_t(0)
    assert lib.smelt_cuda_build_hybrid_decoder(None, C.byref(desc), layers, C.byref(hy.desc), hy.refs, hy.kinds, 32, None, C.byref(n)) == 0
    table = (capi.DispatchRecord * n.value)()
    assert lib.smelt_cuda_build_hybrid_decoder(None, C.byref(desc), layers, C.byref(hy.desc), hy.refs, hy.kinds, 32, table, C.byref(n)) == 0
    dispatches = [r for r in table if r.op_kind == 0]
    # embedding + delta layer (11 mixer records incl. the residual add, 4 feed-forward) + attention layer (9 + 4) + 4 final
    assert len(dispatches) == 1 + (11 + 4) + (9 + 4) + 4
    bad = capi.DeltaDesc(8, 3, 64, 4)  # value heads not a multiple of the q / k heads
    assert lib.smelt_cuda_build_hybrid_decoder(None, C.byref(desc), layers, C.byref(bad), hy.refs, hy.kinds, 32, None, C.byref(n)) == capi.BAD_ARGUMENT


def test_oracle_chunked_prefill_against_token_by_token_decoding(oracle):
    """so_model_prefill: an attention-only model gives the decode steps' logits bit for bit at any chunking; a hybrid
    model does so at chunks of one position (the prompt-chunk recurrence of one position is the decode step) and
    stays close at longer chunks, where its rows are kept in fp32 across the chunk."""
    from smelt_b200 import package
    prompt = np.array([5, 9, 100, 7, 3, 200, 11, 64, 300], np.int32)
    plain = package.DecoderConfig(layers=2, hidden=512, inter=1024, n_q=4, n_kv=2, head_dim=64, vocab=512)
    m = oracle.model_from_package(package.SyntheticPackage(plain, 4), 32)
    m.reset()
    seq = [m.decode_step(int(t), i, True) for i, t in enumerate(prompt)][-1]
    for chunk in (1, 4, 16):
        m.reset()
        tok, logits = m.prefill(prompt, 0, chunk, want_logits=True)
        assert tok == seq[0] and np.array_equal(logits.view(np.uint16), seq[1].view(np.uint16)), chunk
    hybrid = package.DecoderConfig(layers=3, hidden=512, inter=1024, n_q=4, n_kv=2, head_dim=64, vocab=512, delta_layers=(0, 1),
                                   delta_value_heads=8, delta_qk_heads=4, delta_head_dim=64)
    h = oracle.model_from_package(package.SyntheticPackage(hybrid, 5), 32)
    h.reset()
    seq = [h.decode_step(int(t), i, True) for i, t in enumerate(prompt)][-1]
    h.reset()
    tok, logits = h.prefill(prompt, 0, 1, want_logits=True)
    assert tok == seq[0] and np.array_equal(logits.view(np.uint16), seq[1].view(np.uint16))
    h.reset()
    tok, logits = h.prefill(prompt, 0, 4, want_logits=True)
    ref = seq[1].astype(F)
    assert float(np.max(np.abs(logits.astype(F) - ref)) / np.sqrt(np.mean(ref * ref))) < 2e-2
