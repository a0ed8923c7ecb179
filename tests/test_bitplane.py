"""Signed activation bit-planes (the Bonsai low-bit path): the oracle's restatement pinned on the
fixture and expectation the reference's own test uses (SignedQuantKernelTests.swift:664-677,
:1630-1648), then the CUDA producers and popcount consumers against the oracle.  The view and the
integer dots are exact, so planes and scales must be bit-identical; the fp32 accumulation follows
the same lane partition, so the outputs are compared bit for bit too."""
import ctypes as C

import numpy as np
import pytest

from smelt_b200 import capi, synth

F = np.float32


def reference_fixture(rows=9, cols=256):
    """packedCodes / weightScales / input of testBatchedBinaryBitplaneGEMMIsBitExactWithIndependentRows."""
    groups = cols // 128
    bits = np.array([[(r * 13 + c * 7) & 1 for c in range(cols)] for r in range(rows)], np.uint8)
    codes = np.packbits(bits, axis=1, bitorder="little")
    ws = np.array([0.001953125 * ((i % 7) + 1) for i in range(rows * groups)], np.float16)
    x = np.array([np.sin(F(i * 17 + 3)) * F(0.75) for i in range(cols)], F).astype(np.float16)
    return bits, codes, ws, x


@pytest.mark.parametrize("planes", [2, 3, 4, 5, 6])
def test_oracle_matches_the_reference_tests_expectation(oracle, planes):
    """expected = sum_c q_c * activation_scale * sign * weight_scale, bound max(0.02, 1 %)
    (SignedQuantKernelTests.swift:1630-1648)."""
    rows, cols = 9, 256
    bits, codes, ws, x = reference_fixture(rows, cols)
    pl, sc = oracle.signed_activation_bitplanes(x, cols, planes)
    y = oracle.signed_bitplane_matvec(1, codes, ws, pl, sc, rows, cols, planes).astype(F)
    max_q = (1 << (planes - 1)) - 1
    a = sc.astype(F)[np.arange(cols) // 128]
    q = np.sign(x.astype(F) / a) * np.floor(np.abs(np.clip(x.astype(F) / a, -max_q, max_q)) + F(0.5))  # round half away from zero
    sign = np.where(bits == 0, F(-1), F(1))
    w = ws.astype(F).reshape(rows, cols // 128)[:, np.arange(cols) // 128]
    expected = (q[None, :] * a[None, :] * sign * w).astype(np.float64).sum(1)
    assert np.all(np.abs(y - expected) <= np.maximum(0.02, np.abs(expected) * 0.01))
    # the planes reconstruct q: sign plane + magnitude planes, word w bit l = column 32 w + l
    mag = np.zeros(cols, np.int64)
    for p in range(planes - 1):
        for g in range(cols // 128):
            for wd in range(4):
                mag[g * 128 + wd * 32:g * 128 + wd * 32 + 32] += ((int(pl[g, p, wd]) >> np.arange(32)) & 1) << p
    neg = np.concatenate([[(int(pl[g, planes - 1, wd]) >> l) & 1 for wd in range(4) for l in range(32)] for g in range(cols // 128)])
    assert np.array_equal(np.where(neg == 1, -mag, mag), q.astype(np.int64))


def test_oracle_ternary_consumer_equals_the_dequantised_dot(oracle):
    rows, cols, planes = 7, 384, 5
    rng = np.random.default_rng(5)
    sem = rng.integers(-1, 2, size=(rows, cols))
    code = (sem + 1).astype(np.uint8)  # 0 / 1 / 2 = -1 / 0 / +1
    packed = np.zeros((rows, cols // 4), np.uint8)
    for i in range(4):
        packed |= code[:, i::4] << (2 * i)
    ws = (rng.uniform(0.001, 0.02, size=(rows, cols // 128))).astype(np.float16)
    x = rng.standard_normal(cols).astype(np.float16)
    pl, sc = oracle.signed_activation_bitplanes(x, cols, planes)
    y = oracle.signed_bitplane_matvec(2, packed, ws, pl, sc, rows, cols, planes).astype(np.float64)
    a = sc.astype(np.float64)[np.arange(cols) // 128]
    q = np.sign(x.astype(F) / a.astype(F)) * np.floor(np.abs(np.clip(x.astype(F) / a.astype(F), -15, 15)) + F(0.5))
    w = ws.astype(np.float64)[:, np.arange(cols) // 128]
    expected = (q[None, :] * a[None, :] * sem * w).sum(1)
    assert np.max(np.abs(y - expected)) < 2e-3 * max(1.0, float(np.max(np.abs(expected))))


# ── CUDA against the oracle ──
@pytest.fixture(scope="module")
def ctx():
    c = capi.Context(0)
    yield c
    c.close()


def weights(fmt, rows, cols, seed):
    if fmt == 1:
        codes, scales = synth.binary1(seed, "bp", rows, cols)
    else:
        codes, scales = synth.ternary2(seed, "bp", rows, cols)
    return np.ascontiguousarray(codes), np.ascontiguousarray(scales)


@pytest.mark.gpu
@pytest.mark.parametrize("planes", [2, 3, 4, 5, 6])
@pytest.mark.parametrize("cols,batch", [(5120, 1), (256, 5), (17408, 2)])
def test_producer_is_bit_exact(ctx, oracle, planes, cols, batch):
    x = synth.activations(40 + planes, "bpx", batch, cols)
    x[0, :128] = 0  # an all-zero group: scale 1, every plane empty
    dx = ctx.to_device(x)
    groups = cols // 128
    dpl, dsc = ctx.alloc(batch * groups * planes * 16), ctx.alloc(batch * groups * 2)
    ctx.call("signed_activation_bitplanes", dx, None, dpl, dsc, cols, planes, batch)
    got_pl = dpl.download(np.uint32, (batch, groups, planes, 4))
    got_sc = dsc.download(np.uint16, (batch, groups))
    for b in range(batch):
        pl, sc = oracle.signed_activation_bitplanes(x[b], cols, planes)
        assert np.array_equal(got_sc[b], sc.view(np.uint16)), "scales"
        assert np.array_equal(got_pl[b], pl), "planes"


@pytest.mark.gpu
def test_swiglu_producer_is_bit_exact(ctx, oracle):
    cols = 17408
    gate, up = synth.activations(46, "bpg", cols), synth.activations(46, "bpu", cols)
    dg, du = ctx.to_device(gate), ctx.to_device(up)
    dpl, dsc = ctx.alloc(cols // 128 * 5 * 16), ctx.alloc(cols // 128 * 2)
    ctx.call("signed_activation_bitplanes", dg, du, dpl, dsc, cols, 5, 1)
    pl, sc = oracle.swiglu_signed_activation_bitplanes_i5(gate, up, cols)
    got_sc = dsc.download(np.uint16, (cols // 128,))
    # expf of the two libraries can differ by an ulp inside the staged sigmoid: where the scale agrees the planes must
    same = got_sc == sc.view(np.uint16)
    assert same.mean() > 0.95
    got_pl = dpl.download(np.uint32, (cols // 128, 5, 4))
    flips = sum(bin(int(a) ^ int(b)).count("1") for a, b in zip(got_pl[same].reshape(-1), pl[same].reshape(-1)))
    assert flips <= cols // 1000, flips


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,planes", [(1, 2), (1, 3), (1, 4), (1, 5), (1, 6), (2, 4), (2, 5), (2, 6)])
@pytest.mark.parametrize("rows,cols,batch", [(17408, 5120, 1), (5120, 17408, 1), (9, 256, 3), (130, 384, 1)])
def test_consumer_matvec_is_bit_exact(ctx, oracle, fmt, planes, rows, cols, batch):
    codes, scales = weights(fmt, rows, cols, 50 + planes)
    x = synth.activations(51, "bpx", batch, cols)
    groups = cols // 128
    pls = np.zeros((batch, groups, planes, 4), np.uint32)
    scs = np.zeros((batch, groups), np.float16)
    for b in range(batch):
        pls[b], scs[b] = oracle.signed_activation_bitplanes(x[b], cols, planes)
    dc, ds, dp, da = (ctx.to_device(a) for a in (codes, scales, pls, scs))
    out = ctx.alloc(batch * rows * 2)
    ctx.call("signed_bitplane_matvec", fmt, 0, dc, ds, None, None, dp, da, None, out, rows, cols, planes, batch)
    got = out.download(np.uint16, (batch, rows))
    for b in range(batch):
        want = oracle.signed_bitplane_matvec(fmt, codes, scales, pls[b], scs[b], rows, cols, planes)
        assert np.array_equal(got[b], want.view(np.uint16)), f"batch row {b}"
    for d in (dc, ds, dp, da, out):
        d.free()


@pytest.mark.gpu
@pytest.mark.parametrize("planes", [3, 5])
def test_consumer_add_and_gate_up_are_bit_exact(ctx, oracle, planes):
    rows, cols = 5120, 17408
    gc, gs = weights(1, rows, cols, 60)
    uc, us = weights(1, rows, cols, 61)
    x = synth.activations(62, "bpx", cols)
    res = synth.activations(62, "bpr", rows)
    pl, sc = oracle.signed_activation_bitplanes(x, cols, planes)
    dgc, dgs, duc, dus, dp, da, dr = (ctx.to_device(a) for a in (gc, gs, uc, us, pl, sc, res))
    out = ctx.alloc(rows * 2)
    ctx.call("signed_bitplane_matvec", 1, 1, dgc, dgs, None, None, dp, da, dr, out, rows, cols, planes, 1)
    want = oracle.signed_bitplane_matvec(1, gc, gs, pl, sc, rows, cols, planes, residual=res)
    assert np.array_equal(out.download(np.uint16, (rows,)), want.view(np.uint16))
    ctx.call("signed_bitplane_matvec", 1, 2, dgc, dgs, duc, dus, dp, da, None, out, rows, cols, planes, 1)
    want = oracle.signed_bitplane_gate_up_swiglu(1, gc, gs, uc, us, pl, sc, rows, cols, planes)
    got = out.download(np.float16, (rows,))
    from helpers import ulp_diff_f16
    assert np.max(ulp_diff_f16(got, want)) <= 2  # the staged sigmoid's expf; gate and up themselves are exact
    assert np.mean(got.view(np.uint16) == want.view(np.uint16)) > 0.98


@pytest.mark.gpu
def test_bitplane_records_producer_then_consumer(ctx, oracle):
    """signed_activation_bitplanes_i4_g128 then signed_binary_bitplane_i4_matvec_g128_rows8 as records, with
    the reference's bindings (signed_quant.metal:757-762, :1564-1572)."""
    rows, cols, planes = 1024, 2048, 4
    codes, scales = weights(1, rows, cols, 70)
    x = synth.activations(71, "bpx", cols)
    groups = cols // 128
    tensors = {2: codes, 3: scales, 4: x, 5: np.zeros(groups * planes * 4, np.uint32), 6: np.zeros(groups, np.float16), 7: np.zeros(rows, np.float16)}
    for slot, t in tensors.items():
        ctx.call("alloc_slot", slot, C.c_size_t(t.nbytes))
        ctx._check(ctx.lib.smelt_cuda_write_slot(ctx.h, slot, C.c_size_t(0), t.ctypes.data_as(C.c_void_p), C.c_size_t(t.nbytes)))
    for slot in (0, 1):
        ctx.call("alloc_slot", slot, C.c_size_t(64))
    cfg = capi.RuntimeConfig(0, 1, 2, 2, 0, 1, 64, 64, 16, 1)
    ctx._check(ctx.lib.smelt_cuda_configure(ctx.h, C.byref(cfg)))
    ctx._check(ctx.lib.smelt_cuda_register_pipeline(ctx.h, 0, b"signed_activation_bitplanes_i4_g128"))
    ctx._check(ctx.lib.smelt_cuda_register_pipeline(ctx.h, 1, b"signed_binary_bitplane_i4_matvec_g128_rows8"))

    def rec(pipe, grid, bufs, cons):
        r = capi.DispatchRecord()
        r.op_kind, r.pipeline, r.buffer_count, r.constant_count = 0, pipe, len(bufs), len(cons)
        r.grid[0], r.grid[1], r.grid[2] = grid, 1, 1
        for j, (binding, slot) in enumerate(bufs):
            r.buf[j].slot, r.buf[j].binding_index, r.buf[j].offset_kind, r.buf[j].offset = slot, binding, 0, 0
        for j, (binding, value) in enumerate(cons):
            r.con[j].kind, r.con[j].binding_index, r.con[j].value = 0, binding, value
        return r

    table = (capi.DispatchRecord * 2)(rec(0, groups, [(0, 4), (1, 5), (2, 6)], [(3, cols)]),
                                      rec(1, (rows + 7) // 8, [(0, 2), (1, 3), (2, 5), (3, 6), (4, 7)], [(5, rows), (6, cols)]))
    tok = np.zeros(1, np.int32)
    ctx._check(ctx.lib.smelt_cuda_enqueue_decode(ctx.h, table, 2, tok.ctypes.data_as(C.c_void_p), 0))
    ctx.synchronize()
    got = np.zeros(rows, np.uint16)
    ctx._check(ctx.lib.smelt_cuda_read_slot(ctx.h, 7, C.c_size_t(0), got.ctypes.data_as(C.c_void_p), C.c_size_t(got.nbytes)))
    pl, sc = oracle.signed_activation_bitplanes(x, cols, planes)
    want = oracle.signed_bitplane_matvec(1, codes, scales, pl, sc, rows, cols, planes)
    assert np.array_equal(got, want.view(np.uint16))


# ── producers with another kernel's arithmetic in front; signed embedding gathers ──
def fused_fixture(cols=5120):
    """input / weight of testRMSNormActivationViewsAreBitExactWithStagedGraph (SignedQuantKernelTests.swift:2080-2087)."""
    i = np.arange(cols)
    x = (np.sin((i * 17 + 3).astype(F)) * (F(0.125) + ((i // 128) % 13).astype(F) * F(0.375))).astype(np.float16)
    w = (np.cos((i * 7 + 5).astype(F)) * F(0.25)).astype(np.float16)
    return x, w


@pytest.mark.parametrize("planes", [2, 3, 4, 5, 6])
def test_oracle_norm_scale_view_equals_the_staged_graph(oracle, planes):
    """The reference asserts fused == rms_norm_1pw then the plain builder, bit for bit
    (SignedQuantKernelTests.swift:2077-2200): here with the norm's value written in numpy halves."""
    cols = 5120
    x, w = fused_fixture(cols)
    rs = F(1) / np.sqrt(np.mean(x.astype(F) ** 2, dtype=F) + F(1e-6))
    staged = (x.astype(F) * rs).astype(np.float16) * (F(1) + w.astype(F)).astype(np.float16)  # half * half, rounded once
    assert staged.dtype == np.float16
    want_pl, want_sc = oracle.signed_activation_bitplanes(staged, cols, planes)
    pl, sc = oracle.norm_scale_signed_activation_bitplanes(float(rs), x, w, cols, planes)
    assert np.array_equal(pl, want_pl) and np.array_equal(sc.view(np.uint16), want_sc.view(np.uint16))


def gated_fixture(heads=48):
    """input / gate / weight of the fused gated-norm test (SignedQuantKernelTests.swift:2302-2313)."""
    d = 128
    i = np.arange(heads * d)
    x = (np.sin((i * 17 + 3).astype(F)) * (F(0.125) + ((i // d) % 12).astype(F) * F(0.625))).astype(np.float16)
    g = (np.cos((i * 11 + 5).astype(F)) * (F(0.25) + ((i // d) % 9).astype(F) * F(0.5))).astype(np.float16)
    w = (F(0.5) + ((np.arange(d) * 7) % 31).astype(F) / F(32)).astype(np.float16)
    return x, g, w


@pytest.mark.parametrize("tgs", [32, 128])
def test_oracle_gated_norm_view_equals_the_staged_graph(oracle, tgs):
    heads = 48
    x, g, w = gated_fixture(heads)
    staged = oracle.rms_norm_gated_d128(x, g, w, heads) if tgs == 32 else oracle.rms_norm_gated_tg(x, g, w, 128, 1e-6, heads, 128)
    want_pl, want_sc = oracle.signed_activation_bitplanes(staged.reshape(-1), heads * 128, 6)
    pl, sc = oracle.rms_norm_gated_d128_signed_activation_bitplanes_i6(x, g, w, heads, 1e-6, tgs)
    assert np.array_equal(pl, want_pl) and np.array_equal(sc.view(np.uint16), want_sc.view(np.uint16))
    # the precise form is the gated norm up to its extra fp16 boundary
    plain = oracle.rms_norm_gated(x, g, w, 128, 1e-6, heads)
    assert np.max(np.abs(staged.astype(F) - plain.astype(F))) <= 2e-3 * max(1.0, float(np.max(np.abs(plain.astype(F)))))


def test_oracle_sigmoid_mul_view_equals_the_staged_graph(oracle):
    cols = 2048
    rng = np.random.default_rng(8)
    a, b = rng.standard_normal(cols).astype(np.float16), (rng.standard_normal(cols) * 3).astype(np.float16)
    one = np.float16(1)
    tail = one / (one + np.exp(np.abs(b)).astype(np.float16))
    staged = a * np.where(b < 0, tail, one - tail).astype(np.float16)
    want_pl, want_sc = oracle.signed_activation_bitplanes(staged, cols, 6)
    pl, sc = oracle.sigmoid_mul_signed_activation_bitplanes_i6(a, b, cols)
    agree = sc.view(np.uint16) == want_sc.view(np.uint16)
    assert agree.mean() > 0.9  # numpy's half exp may round another way than expf + one rounding
    assert np.array_equal(pl[agree], want_pl[agree]) or np.mean(pl[agree] == want_pl[agree]) > 0.99


@pytest.mark.parametrize("fmt", [1, 2])
def test_oracle_signed_embedding_gather(oracle, fmt):
    rows, hidden = 40, 384
    codes, scales = weights(fmt, rows, hidden, 3)
    ids = np.array([7, 0, 39, 7], np.int32)
    got = oracle.signed_embedding_gather(fmt, codes, scales, ids, hidden).astype(F)
    if fmt == 1:
        sem = np.unpackbits(codes.reshape(rows, -1), axis=1, bitorder="little")[:, :hidden].astype(F) * 2 - 1
    else:
        b = codes.reshape(rows, -1)
        sem = np.stack([(b >> (2 * i)) & 3 for i in range(4)], axis=2).reshape(rows, -1)[:, :hidden].astype(F) - 1
    want = (sem * scales.reshape(rows, hidden // 128).astype(F)[:, np.arange(hidden) // 128]).astype(np.float16).astype(F)
    assert np.array_equal(got, want[ids])


@pytest.mark.gpu
@pytest.mark.parametrize("planes", [2, 3, 4, 5, 6])
def test_norm_scale_producer_is_bit_exact(ctx, oracle, planes):
    cols = 5120
    x, w = fused_fixture(cols)
    rs = np.array([1 / np.sqrt(np.mean(x.astype(F) ** 2, dtype=F) + F(1e-6))], F)
    dx, dw, drs = ctx.to_device(x), ctx.to_device(w), ctx.to_device(rs)
    dpl, dsc = ctx.alloc(cols // 128 * planes * 16), ctx.alloc(cols // 128 * 2)
    ctx.call("fused_activation_bitplanes", 3, dx, None, dw, drs, dpl, dsc, cols, planes, C.c_float(0), 32)
    pl, sc = oracle.norm_scale_signed_activation_bitplanes(float(rs[0]), x, w, cols, planes)
    assert np.array_equal(dsc.download(np.uint16, (cols // 128,)), sc.view(np.uint16))
    assert np.array_equal(dpl.download(np.uint32, pl.shape), pl)


@pytest.mark.gpu
@pytest.mark.parametrize("tgs", [32, 128])
def test_gated_norm_producer_equals_the_staged_kernels(ctx, oracle, tgs):
    """Fused == gated norm kernel then the plain builder, bit for bit, on the device (the reference's own
    assertion, SignedQuantKernelTests.swift:2296-2400), and within the expf difference of the oracle."""
    heads = 48
    x, g, w = gated_fixture(heads)
    dx, dg, dw = ctx.to_device(x), ctx.to_device(g), ctx.to_device(w)
    staged = ctx.alloc(heads * 256)
    ctx.call("rms_norm_gated_ex", dx, dg, dw, staged, 128, C.c_float(1e-6), heads, tgs, 1 if tgs == 32 else 0)
    spl, ssc = ctx.alloc(heads * 6 * 16), ctx.alloc(heads * 2)
    ctx.call("signed_activation_bitplanes", staged, None, spl, ssc, heads * 128, 6, 1)
    fpl, fsc = ctx.alloc(heads * 6 * 16), ctx.alloc(heads * 2)
    ctx.call("fused_activation_bitplanes", 4, dx, dg, dw, None, fpl, fsc, heads * 128, 6, C.c_float(1e-6), tgs)
    assert np.array_equal(fsc.download(np.uint16, (heads,)), ssc.download(np.uint16, (heads,)))
    assert np.array_equal(fpl.download(np.uint32, (heads, 6, 4)), spl.download(np.uint32, (heads, 6, 4)))
    want = oracle.rms_norm_gated_d128(x, g, w, heads) if tgs == 32 else oracle.rms_norm_gated_tg(x, g, w, 128, 1e-6, heads, 128)
    got = staged.download(np.float16, (heads, 128))
    ulp = np.abs(got.view(np.int16).astype(np.int32) - want.view(np.int16).astype(np.int32))
    assert ulp.max() <= 1 and (ulp == 0).mean() > 0.99


@pytest.mark.gpu
def test_sigmoid_mul_producer(ctx, oracle):
    cols = 17408
    a, b = synth.activations(47, "sma", cols), synth.activations(47, "smb", cols)
    da, db = ctx.to_device(a), ctx.to_device(b)
    dpl, dsc = ctx.alloc(cols // 128 * 6 * 16), ctx.alloc(cols // 128 * 2)
    ctx.call("fused_activation_bitplanes", 2, da, db, None, None, dpl, dsc, cols, 6, C.c_float(0), 32)
    pl, sc = oracle.sigmoid_mul_signed_activation_bitplanes_i6(a, b, cols)
    got_sc = dsc.download(np.uint16, (cols // 128,))
    same = got_sc == sc.view(np.uint16)  # expf of the two libraries inside the staged sigmoid
    assert same.mean() > 0.95
    got_pl = dpl.download(np.uint32, (cols // 128, 6, 4))
    flips = sum(bin(int(p) ^ int(q)).count("1") for p, q in zip(got_pl[same].reshape(-1), pl[same].reshape(-1)))
    assert flips <= cols // 1000, flips


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", [1, 2])
def test_signed_embedding_gather(ctx, oracle, fmt):
    rows, hidden = 300, 5120
    codes, scales = weights(fmt, rows, hidden, 4)
    ids = np.array([7, 0, 299, 7, 150], np.int32)
    dc, ds, di = ctx.to_device(codes), ctx.to_device(scales), ctx.to_device(ids)
    out = ctx.alloc(len(ids) * hidden * 2)
    ctx.call("signed_embedding_gather", fmt, dc, ds, di, out, hidden, len(ids))
    want = oracle.signed_embedding_gather(fmt, codes, scales, ids, hidden)
    assert np.array_equal(out.download(np.uint16, want.shape), want.view(np.uint16))


@pytest.mark.gpu
def test_fused_producer_and_gather_records(ctx, oracle):
    """The fused producers and the signed gather as records with the reference's names and bindings."""
    heads, hidden, rows = 16, 2048, 64
    x, g, w = gated_fixture(heads)
    codes, scales = weights(2, rows, hidden, 5)
    ids = np.array([5], np.int32)
    nx, nw = fused_fixture(hidden)
    rs = np.array([0.75], F)
    tensors = {2: x, 3: g, 4: w, 5: np.zeros(heads * 24, np.uint32), 6: np.zeros(heads, np.float16), 7: codes, 8: scales, 9: ids,
               10: np.zeros(hidden, np.float16), 11: nx, 12: nw, 13: rs, 14: np.zeros(hidden // 128 * 16, np.uint32), 15: np.zeros(hidden // 128, np.float16)}
    for slot, t in tensors.items():
        t = np.ascontiguousarray(t)
        ctx.call("alloc_slot", slot, C.c_size_t(t.nbytes))
        ctx._check(ctx.lib.smelt_cuda_write_slot(ctx.h, slot, C.c_size_t(0), t.ctypes.data_as(C.c_void_p), C.c_size_t(t.nbytes)))
    cfg = capi.RuntimeConfig(0, 1, 2, 2, 0, 1, 64, 64, 16, 1)
    for slot in (0, 1):
        ctx.call("alloc_slot", slot, C.c_size_t(64))
    ctx._check(ctx.lib.smelt_cuda_configure(ctx.h, C.byref(cfg)))
    names = ["rms_norm_gated_d128_signed_activation_bitplanes_i6_g128", "signed_ternary_embedding_gather_g128", "norm_scale_signed_activation_bitplanes_i4_g128"]
    for i, n in enumerate(names):
        ctx._check(ctx.lib.smelt_cuda_register_pipeline(ctx.h, 20 + i, n.encode()))
    f32 = lambda v: int(np.array([v], F).view(np.uint32)[0])

    def rec(pipe, grid, tg, bufs, cons):
        r = capi.DispatchRecord()
        r.op_kind, r.pipeline, r.buffer_count, r.constant_count = 0, pipe, len(bufs), len(cons)
        r.grid[0], r.grid[1], r.grid[2] = grid[0], grid[1], 1
        r.threadgroup[0], r.threadgroup[1], r.threadgroup[2] = tg, 1, 1
        for j, (binding, slot) in enumerate(bufs):
            r.buf[j].slot, r.buf[j].binding_index, r.buf[j].offset_kind, r.buf[j].offset = slot, binding, 0, 0
        for j, (binding, kind, value) in enumerate(cons):
            r.con[j].kind, r.con[j].binding_index, r.con[j].value = kind, binding, value
        return r

    table = (capi.DispatchRecord * 3)(
        rec(20, (heads, 1), 128, [(0, 2), (1, 3), (2, 4), (3, 5), (4, 6)], [(5, 0, 128), (6, 1, f32(1e-6))]),
        rec(21, (hidden, 1), 32, [(0, 7), (1, 8), (2, 9), (3, 10)], [(4, 0, hidden)]),
        rec(22, (hidden // 128, 1), 32, [(0, 13), (1, 11), (2, 12), (3, 14), (4, 15)], [(5, 0, hidden)]))
    tok = np.zeros(1, np.int32)
    ctx._check(ctx.lib.smelt_cuda_enqueue_decode(ctx.h, table, 3, tok.ctypes.data_as(C.c_void_p), 0))
    ctx.synchronize()

    def read(slot, dtype, n):
        out = np.zeros(n, dtype)
        ctx._check(ctx.lib.smelt_cuda_read_slot(ctx.h, slot, C.c_size_t(0), out.ctypes.data_as(C.c_void_p), C.c_size_t(out.nbytes)))
        return out

    pl, sc = oracle.rms_norm_gated_d128_signed_activation_bitplanes_i6(x, g, w, heads, 1e-6, 128)
    got_sc = read(6, np.uint16, heads)
    same = got_sc == sc.view(np.uint16)
    assert same.mean() >= 0.9
    assert np.mean(read(5, np.uint32, heads * 24).reshape(heads, 6, 4)[same] == pl[same]) > 0.99
    assert np.array_equal(read(10, np.uint16, hidden), oracle.signed_embedding_gather(2, codes, scales, ids, hidden).view(np.uint16).reshape(-1))
    npl, nsc = oracle.norm_scale_signed_activation_bitplanes(0.75, nx, nw, hidden, 4)
    assert np.array_equal(read(15, np.uint16, hidden // 128), nsc.view(np.uint16))
    assert np.array_equal(read(14, np.uint32, hidden // 128 * 16).reshape(npl.shape), npl)


@pytest.mark.gpu
def test_bank_and_prompt_row_records(ctx, oracle):
    """Projection banks and the prompt-row tiles as records with the reference's names and bindings
    (signed_quant.metal:2475-2497 bank of four over one view, :1438-1452 batched tiles, :2867-2882 packed
    bank of four over the fp16 input): every member row must be the standalone kernel's value."""
    cols, planes, members = 384, 3, (40, 24, 0, 16)
    total = sum(members)
    codes, scales = weights(1, total, cols, 80)
    groups = cols // 128
    xs = synth.activations(81, "bank", 5, cols)
    pls, scs = zip(*(oracle.signed_activation_bitplanes(xs[b], cols, planes) for b in range(5)))
    pl5, sc5 = np.stack(pls), np.stack(scs)
    pl4 = np.stack([oracle.signed_activation_bitplanes(xs[b], cols, 4)[0] for b in range(5)])
    sc4 = np.stack([oracle.signed_activation_bitplanes(xs[b], cols, 4)[1] for b in range(5)])
    tensors = {2: codes, 3: scales, 4: pl5[0], 5: sc5[0], 6: np.zeros(40, np.float16), 7: np.zeros(24, np.float16), 8: np.zeros(8, np.float16),
               9: np.zeros(16, np.float16), 10: pl4, 11: sc4, 12: np.zeros((5, total), np.float16), 13: xs[0],
               14: np.zeros(40, np.float16), 15: np.zeros(24, np.float16), 16: np.zeros(16, np.float16)}
    for slot, t in tensors.items():
        t = np.ascontiguousarray(t)
        ctx.call("alloc_slot", slot, C.c_size_t(t.nbytes))
        ctx._check(ctx.lib.smelt_cuda_write_slot(ctx.h, slot, C.c_size_t(0), t.ctypes.data_as(C.c_void_p), C.c_size_t(t.nbytes)))
    for slot in (0, 1):
        ctx.call("alloc_slot", slot, C.c_size_t(64))
    cfg = capi.RuntimeConfig(0, 1, 2, 2, 0, 1, 64, 64, 16, 1)
    ctx._check(ctx.lib.smelt_cuda_configure(ctx.h, C.byref(cfg)))
    names = ["signed_binary_bitplane_i3_bank4_matvec_g128_rows8", "signed_binary_bitplane_i4_matvec_g128_rows8_batched_b8", "signed_binary_packed_bank4_matvec_g128_rows8"]
    for i, n in enumerate(names):
        ctx._check(ctx.lib.smelt_cuda_register_pipeline(ctx.h, 40 + i, n.encode()))

    def rec(pipe, grid, bufs, cons):
        r = capi.DispatchRecord()
        r.op_kind, r.pipeline, r.buffer_count, r.constant_count = 0, pipe, len(bufs), len(cons)
        r.grid[0], r.grid[1], r.grid[2] = grid[0], grid[1], 1
        for j, (binding, slot) in enumerate(bufs):
            r.buf[j].slot, r.buf[j].binding_index, r.buf[j].offset_kind, r.buf[j].offset = slot, binding, 0, 0
        for j, (binding, value) in enumerate(cons):
            r.con[j].kind, r.con[j].binding_index, r.con[j].value = 0, binding, value
        return r

    table = (capi.DispatchRecord * 3)(
        rec(40, ((total + 7) // 8, 1), [(0, 2), (1, 3), (2, 4), (3, 5), (4, 6), (5, 7), (6, 8), (7, 9)], [(8, 40), (9, 24), (10, 0), (11, 16), (12, cols)]),
        rec(41, ((total + 3) // 4, 1), [(0, 2), (1, 3), (2, 10), (3, 11), (4, 12)], [(5, total), (6, cols), (7, 5)]),
        rec(42, ((total + 7) // 8, 1), [(0, 2), (1, 3), (2, 13), (3, 14), (4, 15), (5, 8), (6, 16)], [(7, 40), (8, 24), (9, 0), (10, 16), (11, cols)]))
    tok = np.zeros(1, np.int32)
    ctx._check(ctx.lib.smelt_cuda_enqueue_decode(ctx.h, table, 3, tok.ctypes.data_as(C.c_void_p), 0))
    ctx.synchronize()

    def read(slot, shape):
        out = np.zeros(shape, np.float16)
        ctx._check(ctx.lib.smelt_cuda_read_slot(ctx.h, slot, C.c_size_t(0), out.ctypes.data_as(C.c_void_p), C.c_size_t(out.nbytes)))
        return out

    whole = oracle.signed_bitplane_matvec(1, codes, scales, pl5[0], sc5[0], total, cols, planes)
    assert np.array_equal(read(6, 40), whole[:40]) and np.array_equal(read(7, 24), whole[40:64]) and np.array_equal(read(9, 16), whole[64:])
    got = read(12, (5, total))
    for b in range(5):
        assert np.array_equal(got[b], oracle.signed_bitplane_matvec(1, codes, scales, pl4[b], sc4[b], total, cols, 4)), b
    direct = oracle.signed_matvec(1, codes, scales, xs[0], total, cols).astype(F)
    packed = np.concatenate([read(14, 40), read(15, 24), read(16, 16)]).astype(F)
    assert np.max(np.abs(packed - direct)) <= 2e-3 * max(1.0, float(np.max(np.abs(direct))))


@pytest.mark.gpu
def test_ternary_affine_records(ctx, oracle):
    """The MLX-affine ternary forms as records (signed_quant_precise.metal:41-420: matvec, + residual, gate / up +
    SwiGLU, bank of four, prompt-row QMM), whose bias scales repeat the scales: the ternary kernels' values."""
    rows, cols, batch = 96, 512, 3
    members = (40, 0, 24, 32)
    codes, scales = weights(2, rows, cols, 90)
    codes2, scales2 = weights(2, rows, cols, 91)
    xs = synth.activations(92, "ta", batch, cols)
    res = synth.activations(93, "tr", rows)
    tensors = {2: codes, 3: scales, 4: codes2, 5: scales2, 6: xs, 7: res, 8: np.zeros(rows, np.float16), 9: np.zeros(rows, np.float16), 10: np.zeros(40, np.float16),
               11: np.zeros(8, np.float16), 12: np.zeros(24, np.float16), 13: np.zeros(32, np.float16), 14: np.zeros((batch, rows), np.float16)}
    for slot, t in tensors.items():
        t = np.ascontiguousarray(t)
        ctx.call("alloc_slot", slot, C.c_size_t(t.nbytes))
        ctx._check(ctx.lib.smelt_cuda_write_slot(ctx.h, slot, C.c_size_t(0), t.ctypes.data_as(C.c_void_p), C.c_size_t(t.nbytes)))
    for slot in (0, 1):
        ctx.call("alloc_slot", slot, C.c_size_t(64))
    cfg = capi.RuntimeConfig(0, 1, 2, 2, 0, 1, 64, 64, 16, 1)
    ctx._check(ctx.lib.smelt_cuda_configure(ctx.h, C.byref(cfg)))
    names = ["signed_ternary_affine_matvec_add_g128_rows8", "signed_ternary_affine_gate_up_swiglu_g128_rows8", "signed_ternary_affine_bank4_matvec_g128_rows8",
             "signed_ternary_affine_qmm_g128_bm32_bn32_bk32"]
    for i, n in enumerate(names):
        ctx._check(ctx.lib.smelt_cuda_register_pipeline(ctx.h, 60 + i, n.encode()))

    def rec(pipe, bufs, cons):
        r = capi.DispatchRecord()
        r.op_kind, r.pipeline, r.buffer_count, r.constant_count = 0, pipe, len(bufs), len(cons)
        r.grid[0], r.grid[1], r.grid[2] = 1, 1, 1
        for j, (binding, slot) in enumerate(bufs):
            r.buf[j].slot, r.buf[j].binding_index, r.buf[j].offset_kind, r.buf[j].offset = slot, binding, 0, 0
        for j, (binding, value) in enumerate(cons):
            r.con[j].kind, r.con[j].binding_index, r.con[j].value = 0, binding, value
        return r

    table = (capi.DispatchRecord * 4)(
        rec(60, [(0, 2), (1, 3), (2, 3), (3, 6), (4, 8), (5, 7)], [(6, rows), (7, cols)]),
        rec(61, [(0, 2), (1, 3), (2, 3), (3, 4), (4, 5), (5, 5), (6, 6), (7, 9)], [(8, rows), (9, cols)]),
        rec(62, [(0, 2), (1, 3), (2, 3), (3, 6), (4, 10), (5, 11), (6, 12), (7, 13)], [(8, 40), (9, 0), (10, 24), (11, 32), (12, cols)]),
        rec(63, [(0, 2), (1, 3), (2, 3), (3, 6), (4, 14)], [(5, rows), (6, cols), (7, batch)]))
    tok = np.zeros(1, np.int32)
    ctx._check(ctx.lib.smelt_cuda_enqueue_decode(ctx.h, table, 4, tok.ctypes.data_as(C.c_void_p), 0))
    ctx.synchronize()

    def read(slot, shape):
        out = np.zeros(shape, np.float16)
        ctx._check(ctx.lib.smelt_cuda_read_slot(ctx.h, slot, C.c_size_t(0), out.ctypes.data_as(C.c_void_p), C.c_size_t(out.nbytes)))
        return out.astype(F)

    def close(got, want):
        want = want.astype(F)
        return np.max(np.abs(got - want)) <= 2e-3 * max(1.0, float(np.max(np.abs(want))))

    assert close(read(8, rows), oracle.signed_matvec_add(2, codes, scales, xs[0], res, rows, cols))
    assert close(read(9, rows), oracle.signed_gate_up_swiglu(2, codes, scales, codes2, scales2, xs[0], rows, cols))
    whole = oracle.signed_matvec(2, codes, scales, xs[0], rows, cols)
    assert close(np.concatenate([read(10, 40), read(12, 24), read(13, 32)]), whole)
    got = read(14, (batch, rows))
    for b in range(batch):
        assert close(got[b], oracle.signed_matvec(2, codes, scales, xs[b], rows, cols)), b
