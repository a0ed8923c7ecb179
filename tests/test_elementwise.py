"""The small kernels between a layer's projections: element-wise activations and products
(Resources/Shaders/activations.metal:4-210, activations_precise.metal:22-35), the per-head RMS
norms with their reduction topologies and the gate split (attention_fused.metal:11-330), the
batched embedding gathers (lut_matvec.metal:1081-1134).  The oracle against plain float formulas,
then the CUDA kernels against the oracle, typed and as records under the reference's names."""
import ctypes as C

import numpy as np
import pytest

from smelt_b200 import capi
from helpers import ulp_diff_f16

F = np.float32


def halves(rng, *shape, scale=1.0):
    return (rng.standard_normal(shape) * scale).astype(np.float16)


def test_oracle_elementwise_against_float_formulas(oracle):
    rng = np.random.default_rng(1)
    x, b = halves(rng, 3, 500, scale=3), halves(rng, 3, 500)
    xf, bf = x.astype(F), b.astype(F)
    cases = [
        (oracle.EW_SILU, None, 0.0, xf / (1 + np.exp(-xf))),
        (oracle.EW_SIGMOID, None, 0.0, 1 / (1 + np.exp(-xf))),
        (oracle.EW_SOFTPLUS, None, 0.0, np.where(xf > 20, xf, np.log1p(np.exp(xf)))),
        (oracle.EW_SCALAR_MUL, None, 0.37, xf * F(0.37)),
        (oracle.EW_LOGIT_CAP, None, 30.0, F(30) * np.tanh(xf / F(30))),
        (oracle.EW_MUL, b, 0.0, xf * bf),
        (oracle.EW_SIGMOID_MUL, b, 0.0, xf / (1 + np.exp(-bf))),
        (oracle.EW_GEGLU, b, 0.0, 0.5 * xf * (1 + np.tanh(np.clip(F(0.7978845608) * (xf + F(0.044715) * xf ** 3), -20, 20))) * bf),
    ]
    for op, second, scalar, ref in cases:
        got = oracle.elementwise(op, x, second, scalar)
        close = (ulp_diff_f16(got, ref.astype(np.float16)) <= 2) | (np.abs(got.astype(F) - ref) < 1e-6)  # 1 + tanh cancels near -1: tiny values
        assert np.all(close), op  # staged fp16 roundings against the float formula
    assert np.array_equal(oracle.elementwise(oracle.EW_COPY, x).view(np.uint16), x.view(np.uint16))
    bias = halves(rng, 500)
    assert np.array_equal(oracle.elementwise(oracle.EW_BIAS_ADD, x, bias), x + bias[None, :])
    # the strided form reads row r of `up` at r * stride
    up = halves(rng, 3, 700)
    got = oracle.elementwise(oracle.EW_GEGLU, x, up, b_stride=700)
    assert np.array_equal(got, oracle.elementwise(oracle.EW_GEGLU, x, np.ascontiguousarray(up[:, :500])))


@pytest.mark.parametrize("head_dim,tgs", [(128, 32), (256, 64), (256, 256), (512, 128), (96, 32)])
def test_oracle_head_norms_against_float_formulas(oracle, head_dim, tgs):
    rng = np.random.default_rng(head_dim)
    heads = 11
    x, w = halves(rng, heads, head_dim), halves(rng, head_dim, scale=0.2)
    xf = x.astype(F)
    rs = 1 / np.sqrt((xf * xf).mean(1, keepdims=True) + F(1e-6))
    direct = oracle.head_norm(oracle.HEAD_NORM_DIRECT, x, w, heads, head_dim, 1e-6, tgs)
    one_pw = oracle.head_norm(oracle.HEAD_NORM_1PW, x, w, heads, head_dim, 1e-6, tgs)
    plain = oracle.head_norm(oracle.HEAD_NORM_NOSCALE, x, None, heads, head_dim, 1e-6, tgs)
    assert np.max(ulp_diff_f16(direct, (w.astype(F) * (xf * rs).astype(np.float16).astype(F)).astype(np.float16))) <= 1
    assert np.max(ulp_diff_f16(one_pw, (xf * rs * (1 + w.astype(F))).astype(np.float16))) <= 1
    assert np.max(ulp_diff_f16(plain, (xf * rs).astype(np.float16))) <= 1
    # the sequential restatement the earlier tests use agrees to an ulp
    assert np.max(ulp_diff_f16(direct, oracle.per_head_rms_norm(x.reshape(-1), w, heads, head_dim, 1e-6).reshape(heads, head_dim))) <= 1


@pytest.fixture(scope="module")
def ctx():
    c = capi.Context(0)
    yield c
    c.close()


@pytest.mark.gpu
@pytest.mark.parametrize("op,exact", [(0, False), (1, False), (2, False), (3, True), (4, True), (5, False), (6, True), (7, False), (8, False), (9, True)])
def test_elementwise_kernels(ctx, oracle, op, exact):
    rng = np.random.default_rng(op)
    batch, count = (3, 5000) if op in (8, 9) else (1, 12288)
    x, b = halves(rng, batch, count, scale=3), halves(rng, batch, count)
    stride = count
    if op == 8:
        b, stride = halves(rng, batch, count + 300), count + 300
    if op == 9:
        b = halves(rng, count)
    scalar = {4: 0.37, 5: 30.0}.get(op, 0.0)
    dx, db, dy = ctx.to_device(x), ctx.to_device(b), ctx.alloc(x.nbytes)
    ctx.call("elementwise", op, dx, db if op >= 6 else None, dy, count, batch, stride, C.c_float(scalar))
    got = dy.download(np.float16, x.shape)
    want = oracle.elementwise(op, x, b if op >= 6 else None, scalar, stride)
    if exact:
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    else:
        ulp = ulp_diff_f16(got, want)  # expf / tanhf / logf of the two libraries
        tiny = np.abs(got.astype(F) - want.astype(F)) < 1e-6  # 1 + tanh cancels near -1
        assert np.all((ulp <= 1) | tiny) and np.mean(ulp == 0) > 0.98
    if op == 4:  # scalar_mul_weight: the factor comes from the device
        dw = ctx.to_device(np.array([0.37], np.float16))
        ctx.call("elementwise", 10, dx, dw, dy, count, batch, count, C.c_float(0))
        assert np.array_equal(dy.download(np.float16, x.shape), oracle.elementwise(4, x, None, float(np.float16(0.37))))


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("head_dim,tgs", [(128, 32), (256, 64), (256, 256), (512, 128), (96, 32)])
def test_head_norm_kernels_are_bit_exact(ctx, oracle, mode, head_dim, tgs):
    rng = np.random.default_rng(head_dim + mode)
    heads = 37
    x, w = halves(rng, heads, head_dim), halves(rng, head_dim, scale=0.2)
    dx, dw = ctx.to_device(x), ctx.to_device(w)
    ctx.call("head_norm", mode, dx, None if mode == 2 else dw, dx, heads, head_dim, C.c_float(1e-6), tgs)  # in place
    want = oracle.head_norm(mode, x, None if mode == 2 else w, heads, head_dim, 1e-6, tgs)
    assert np.array_equal(dx.download(np.uint16, (heads, head_dim)), want.view(np.uint16))  # IEEE operations only: same bits


@pytest.mark.gpu
def test_gate_split_and_batched_gathers(ctx, oracle):
    rng = np.random.default_rng(3)
    heads, d = 12, 256
    x = halves(rng, heads, 2 * d)
    dq, dg = ctx.alloc(heads * d * 2), ctx.alloc(heads * d * 2)
    ctx.call("gate_split", ctx.to_device(x), dq, dg, heads, d)
    q, g = oracle.gate_split(x, heads, d)
    assert np.array_equal(dq.download(np.float16, (heads, d)), q) and np.array_equal(dg.download(np.float16, (heads, d)), g)


@pytest.mark.gpu
def test_glue_records(ctx, oracle):
    """gate_split -> per_head_rms_norm_1pw (threadgroup of 64) -> sigmoid_mul -> geglu_fused_strided_batched,
    embedding_gather_batched, with the reference's names and bindings."""
    rng = np.random.default_rng(4)
    heads, d, vocab, hidden, batch = 8, 256, 50, 512, 3
    x = halves(rng, heads, 2 * d)
    w = halves(rng, d, scale=0.2)
    att = halves(rng, heads * d)
    gate_rows, up_rows = halves(rng, batch, 400, scale=2), halves(rng, batch, 640)
    table = halves(rng, vocab, hidden)
    ids = np.array([7, 0, 49], np.int32)
    tensors = {2: x, 3: np.zeros(heads * d, np.float16), 4: np.zeros(heads * d, np.float16), 5: w, 6: att, 7: np.zeros(heads * d, np.float16),
               8: gate_rows, 9: up_rows, 10: np.zeros((batch, 400), np.float16), 11: table, 12: ids, 13: np.zeros((batch, hidden), np.float16)}
    for slot, t in tensors.items():
        t = np.ascontiguousarray(t)
        ctx.call("alloc_slot", slot, C.c_size_t(t.nbytes))
        ctx._check(ctx.lib.smelt_cuda_write_slot(ctx.h, slot, C.c_size_t(0), t.ctypes.data_as(C.c_void_p), C.c_size_t(t.nbytes)))
    cfg = capi.RuntimeConfig(0, 1, 2, 2, 0, 1, 64, 64, 16, 1)
    for slot in (0, 1):
        ctx.call("alloc_slot", slot, C.c_size_t(64))
    ctx._check(ctx.lib.smelt_cuda_configure(ctx.h, C.byref(cfg)))
    names = ["gate_split", "per_head_rms_norm_1pw", "sigmoid_mul", "geglu_fused_strided_batched", "embedding_gather_batched"]
    for i, n in enumerate(names):
        ctx._check(ctx.lib.smelt_cuda_register_pipeline(ctx.h, 30 + i, n.encode()))
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

    tbl = (capi.DispatchRecord * 5)(
        rec(30, (d, heads), 32, [(0, 2), (1, 3), (2, 4)], [(3, 0, heads), (4, 0, d)]),
        rec(31, (heads, 1), 64, [(0, 3), (1, 5), (2, 3)], [(3, 0, d), (4, 1, f32(1e-6))]),
        rec(32, (heads * d, 1), 32, [(0, 6), (1, 4), (2, 7)], [(3, 0, heads * d)]),
        rec(33, (400, batch), 32, [(0, 8), (1, 9), (2, 10)], [(3, 0, 400), (4, 0, 640)]),
        rec(34, (hidden, batch), 32, [(0, 11), (1, 12), (2, 13)], [(3, 0, hidden), (4, 0, batch)]))
    tok = np.zeros(1, np.int32)
    ctx._check(ctx.lib.smelt_cuda_enqueue_decode(ctx.h, tbl, 5, tok.ctypes.data_as(C.c_void_p), 0))
    ctx.synchronize()

    def read(slot, shape):
        out = np.zeros(shape, np.float16)
        ctx._check(ctx.lib.smelt_cuda_read_slot(ctx.h, slot, C.c_size_t(0), out.ctypes.data_as(C.c_void_p), C.c_size_t(out.nbytes)))
        return out

    q, g = oracle.gate_split(x, heads, d)
    assert np.array_equal(read(3, (heads, d)), oracle.head_norm(oracle.HEAD_NORM_1PW, q, w, heads, d, 1e-6, 64))
    assert np.max(ulp_diff_f16(read(7, (heads * d,)), oracle.elementwise(oracle.EW_SIGMOID_MUL, att, g.reshape(-1)))) <= 1
    gg, gw = read(10, (batch, 400)), oracle.elementwise(oracle.EW_GEGLU, gate_rows, up_rows, b_stride=640)
    assert np.all((ulp_diff_f16(gg, gw) <= 1) | (np.abs(gg.astype(F) - gw.astype(F)) < 1e-6))
    assert np.array_equal(read(13, (batch, hidden)), table[ids])


# ── the row norms of norms.metal beyond rms_norm_1pw ──
ROW_NORM_CASES = [  # (dim, topology, value, scale, tgs, residual, scalar, pre)
    (2048, 1, 2, 0, 0, False, False, False),    # rms_norm_1pw_d2048
    (1536, 1, 2, 0, 0, True, False, False),     # rms_norm_1pw_d1536_add(_batched)
    (2560, 1, 2, 0, 0, False, False, False),    # rms_norm_1pw_d2560
    (256, 2, 3, 0, 256, True, True, False),     # rms_norm_1pw_d256_add_scalar_weight
    (4096, 0, 1, 0, 256, False, False, False),  # rms_norm_1pw_batched
    (1000, 0, 1, 0, 128, False, False, False),  # ... with a ragged last tile
    (5120, 2, 0, 0, 512, False, False, True),   # residual_add_rms_norm_scale_only_precise
    (128, 2, 4, 1, 128, False, False, False),   # l2_normalize_d128
]


@pytest.mark.parametrize("dim,topology,value,scale,tgs,residual,scalar,pre", ROW_NORM_CASES)
def test_oracle_row_norms_against_float_formulas(oracle, dim, topology, value, scale, tgs, residual, scalar, pre):
    rng = np.random.default_rng(dim)
    rows = 3
    x, w = halves(rng, rows, dim), halves(rng, dim, scale=0.2)
    res = halves(rng, rows, dim) if residual else None
    pr = halves(rng, rows, dim) if pre else None
    sc = np.array([0.75], np.float16) if scalar else None
    y, scales = oracle.row_norm(x, w, topology=topology, value=value, tgs=tgs or 256, scale=scale, pre=pr, residual=res, scalar=sc)
    v = (x + pr).astype(F) if pre else x.astype(F)
    total = (v.astype(np.float64) ** 2).sum(1)
    ref_scale = 1 / np.sqrt(total / dim + 1e-6) if scale == 0 else 1 / np.maximum(np.sqrt(total), 1e-6)
    assert np.allclose(scales, ref_scale, rtol=2e-6)
    if value == 0:
        assert np.array_equal(y, x + pr)
        return
    rs = scales[:, None]
    ref = {1: (1 + w.astype(F)).astype(np.float16).astype(F) * (v * rs).astype(np.float16).astype(F), 2: v * (rs * (1 + w.astype(F))),
           3: v * rs * (1 + w.astype(F)), 4: v * rs}[value].astype(np.float16)
    if residual:
        ref = ref + res
    if scalar:
        ref = (ref.astype(F) * F(np.float16(0.75))).astype(np.float16)
    assert np.max(ulp_diff_f16(y, ref)) <= 1


@pytest.mark.gpu
@pytest.mark.parametrize("dim,topology,value,scale,tgs,residual,scalar,pre", ROW_NORM_CASES)
def test_row_norm_kernels_are_bit_exact(ctx, oracle, dim, topology, value, scale, tgs, residual, scalar, pre):
    rng = np.random.default_rng(dim + 1)
    rows = 5
    x, w = halves(rng, rows, dim), halves(rng, dim, scale=0.2)
    res = halves(rng, rows, dim) if residual else None
    pr = halves(rng, rows, dim) if pre else None
    sc = np.array([0.75], np.float16) if scalar else None
    dev = lambda a: ctx.to_device(a) if a is not None else None
    dx, dy, dscale = ctx.to_device(x), ctx.alloc(x.nbytes), ctx.alloc(rows * 4)
    ctx.call("row_norm", dx, dev(pr), ctx.to_device(w), dev(res), dev(sc), dy, dscale, rows, dim, C.c_float(1e-6), topology, tgs or 256, value, scale)
    want_y, want_scale = oracle.row_norm(x, w, topology=topology, value=value, tgs=tgs or 256, scale=scale, pre=pr, residual=res, scalar=sc)
    assert np.array_equal(dscale.download(np.uint32, (rows,)), want_scale.view(np.uint32))  # IEEE operations only: same bits
    assert np.array_equal(dy.download(np.uint16, x.shape), want_y.view(np.uint16))


@pytest.mark.gpu
def test_row_norm_records_feed_the_norm_scale_view(ctx, oracle):
    """residual_add_rms_norm_scale_only_precise -> norm_scale_signed_activation_bitplanes_i4_g128 (the Bonsai
    layer entry), rms_norm_1pw_d2048, rms_norm_1pw_d1536_add_batched and l2_normalize_d128 as records."""
    rng = np.random.default_rng(9)
    hidden = 5120
    a, b, nw = halves(rng, hidden), halves(rng, hidden), halves(rng, hidden, scale=0.2)
    x2048, w2048 = halves(rng, 2048), halves(rng, 2048, scale=0.2)
    x1536, w1536, r1536 = halves(rng, 3, 1536), halves(rng, 1536, scale=0.2), halves(rng, 3, 1536)
    qk = halves(rng, 6, 128)
    groups = hidden // 128
    tensors = {2: a, 3: b, 4: np.zeros(hidden, np.float16), 5: np.zeros(1, F), 6: nw, 7: np.zeros(groups * 16, np.uint32), 8: np.zeros(groups, np.float16),
               9: x2048, 10: w2048, 11: np.zeros(2048, np.float16), 12: x1536, 13: w1536, 14: r1536, 15: np.zeros((3, 1536), np.float16), 16: qk}
    for slot, t in tensors.items():
        t = np.ascontiguousarray(t)
        ctx.call("alloc_slot", slot, C.c_size_t(t.nbytes))
        ctx._check(ctx.lib.smelt_cuda_write_slot(ctx.h, slot, C.c_size_t(0), t.ctypes.data_as(C.c_void_p), C.c_size_t(t.nbytes)))
    cfg = capi.RuntimeConfig(0, 1, 2, 2, 0, 1, 64, 64, 16, 1)
    for slot in (0, 1):
        ctx.call("alloc_slot", slot, C.c_size_t(64))
    ctx._check(ctx.lib.smelt_cuda_configure(ctx.h, C.byref(cfg)))
    names = ["residual_add_rms_norm_scale_only_precise", "norm_scale_signed_activation_bitplanes_i4_g128", "rms_norm_1pw_d2048", "rms_norm_1pw_d1536_add_batched", "l2_normalize_d128"]
    for i, n in enumerate(names):
        ctx._check(ctx.lib.smelt_cuda_register_pipeline(ctx.h, 50 + i, n.encode()))
    f32 = lambda v: int(np.array([v], F).view(np.uint32)[0])

    def rec(pipe, grid, tg, bufs, cons):
        r = capi.DispatchRecord()
        r.op_kind, r.pipeline, r.buffer_count, r.constant_count = 0, pipe, len(bufs), len(cons)
        r.grid[0], r.grid[1], r.grid[2] = grid, 1, 1
        r.threadgroup[0], r.threadgroup[1], r.threadgroup[2] = tg, 1, 1
        for j, (binding, slot) in enumerate(bufs):
            r.buf[j].slot, r.buf[j].binding_index, r.buf[j].offset_kind, r.buf[j].offset = slot, binding, 0, 0
        for j, (binding, kind, value) in enumerate(cons):
            r.con[j].kind, r.con[j].binding_index, r.con[j].value = kind, binding, value
        return r

    tbl = (capi.DispatchRecord * 5)(
        rec(50, 1, 512, [(0, 2), (1, 3), (2, 4), (3, 5)], [(4, 0, hidden), (5, 1, f32(1e-6))]),
        rec(51, groups, 32, [(0, 5), (1, 4), (2, 6), (3, 7), (4, 8)], [(5, 0, hidden)]),
        rec(52, 1, 256, [(0, 9), (1, 10), (2, 11)], []),
        rec(53, 3, 192, [(0, 12), (1, 13), (2, 14), (3, 15)], []),
        rec(54, 6, 128, [(0, 16)], []))
    tok = np.zeros(1, np.int32)
    ctx._check(ctx.lib.smelt_cuda_enqueue_decode(ctx.h, tbl, 5, tok.ctypes.data_as(C.c_void_p), 0))
    ctx.synchronize()

    def read(slot, shape, dtype=np.float16):
        out = np.zeros(shape, dtype)
        ctx._check(ctx.lib.smelt_cuda_read_slot(ctx.h, slot, C.c_size_t(0), out.ctypes.data_as(C.c_void_p), C.c_size_t(out.nbytes)))
        return out

    summed, scale = oracle.row_norm(a, None, topology=2, value=0, tgs=512, pre=b)
    assert np.array_equal(read(4, hidden), summed) and np.array_equal(read(5, 1, F).view(np.uint32), scale.view(np.uint32))
    pl, sc = oracle.norm_scale_signed_activation_bitplanes(float(scale[0]), summed, nw, hidden, 4)
    assert np.array_equal(read(8, groups).view(np.uint16), sc.view(np.uint16)) and np.array_equal(read(7, groups * 16, np.uint32).reshape(pl.shape), pl)
    assert np.array_equal(read(11, 2048), oracle.row_norm(x2048, w2048, topology=1, value=2)[0])
    assert np.array_equal(read(15, (3, 1536)), oracle.row_norm(x1536, w1536, topology=1, value=2, residual=r1536)[0])
    assert np.array_equal(read(16, (6, 128)), oracle.row_norm(qk, None, topology=2, value=4, tgs=128, scale=1)[0])


@pytest.mark.gpu
def test_l2_normalize_prefill_records(ctx, oracle):
    """The Q and K heads of a prompt chunk's qkv rows normalised in place (norms.metal:1192-1378): the generic
    forms with their constants and the d128 / c6144 / h16 specialisations."""
    rng = np.random.default_rng(12)
    cases = [("l2_normalize_q_prefill", 64, 4, 6, 64 * 14, False), ("l2_normalize_k_prefill", 64, 4, 6, 64 * 14, True),
             ("l2_normalize_q_d128_c6144_h16_prefill", 128, 16, 3, 6144, False), ("l2_normalize_k_d128_c6144_h16_prefill", 128, 16, 3, 6144, True)]
    cfg = capi.RuntimeConfig(0, 1, 2, 2, 0, 1, 64, 64, 16, 1)
    for slot in (0, 1):
        ctx.call("alloc_slot", slot, C.c_size_t(64))
    ctx._check(ctx.lib.smelt_cuda_configure(ctx.h, C.byref(cfg)))
    f32 = lambda v: int(np.array([v], F).view(np.uint32)[0])
    for i, (name, d, heads, positions, qkv_dim, k_heads) in enumerate(cases):
        x = halves(rng, positions, qkv_dim)
        ctx.call("alloc_slot", 2, C.c_size_t(x.nbytes))
        ctx._check(ctx.lib.smelt_cuda_write_slot(ctx.h, 2, C.c_size_t(0), x.ctypes.data_as(C.c_void_p), C.c_size_t(x.nbytes)))
        ctx._check(ctx.lib.smelt_cuda_register_pipeline(ctx.h, 70 + i, name.encode()))
        r = capi.DispatchRecord()
        generic = "d128" not in name
        r.op_kind, r.pipeline, r.buffer_count, r.constant_count = 0, 70 + i, 1, 4 if generic else 0
        r.grid[0], r.grid[1], r.grid[2] = heads, positions, 1
        r.threadgroup[0], r.threadgroup[1], r.threadgroup[2] = 64 if generic else 128, 1, 1
        r.buf[0].slot, r.buf[0].binding_index = 2, 0
        if generic:
            for j, (binding, kind, value) in enumerate([(1, 0, d), (2, 1, f32(1e-6)), (3, 0, qkv_dim), (4, 0, heads)]):
                r.con[j].kind, r.con[j].binding_index, r.con[j].value = kind, binding, value
        tok = np.zeros(1, np.int32)
        ctx._check(ctx.lib.smelt_cuda_enqueue_decode(ctx.h, (capi.DispatchRecord * 1)(r), 1, tok.ctypes.data_as(C.c_void_p), 0))
        ctx.synchronize()
        got = np.zeros_like(x)
        ctx._check(ctx.lib.smelt_cuda_read_slot(ctx.h, 2, C.c_size_t(0), got.ctypes.data_as(C.c_void_p), C.c_size_t(got.nbytes)))
        want = x.copy()
        first = heads * d if k_heads else 0
        region = np.ascontiguousarray(x[:, first:first + heads * d]).reshape(positions * heads, d)
        want[:, first:first + heads * d] = oracle.row_norm(region, None, topology=2, value=4, tgs=64 if generic else 128, scale=1)[0].reshape(positions, heads * d)
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), name
