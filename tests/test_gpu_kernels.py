"""Parity of every CUDA kernel against the CPU oracle, called through the C ABI on a B200."""
import ctypes as C

import numpy as np
import pytest

from smelt_b200 import capi, synth
from helpers import INF_TOL, REL_TOL, add_rel_err, inf_err, rel_err, ulp_diff_f16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = capi.Context(0)
    yield c
    assert c.device_error() == 0
    c.close()


def dev(ctx, *arrs):
    return [ctx.to_device(a) for a in arrs]


# ── bit-exact unpack / dequant ──────────────────────────────────────────────
@pytest.mark.parametrize("rows,cols,group", [(4096, 1024, 64), (257, 512, 64), (64, 256, 32), (16, 1536, 128)])
def test_affine_dequant_bit_exact(ctx, oracle, rows, cols, group):
    w, s, b = synth.affine_u4(0, "deq", rows, cols, group)
    dw, ds, db = dev(ctx, w, s, b)
    o32, o16 = ctx.alloc(rows * cols * 4), ctx.alloc(rows * cols * 2)
    ctx.call("affine_dequantize", dw, ds, db, o32, o16, rows, cols, group)
    got32 = o32.download(np.float32, (rows, cols))
    got16 = o16.download(np.float16, (rows, cols))
    assert np.array_equal(got32.view(np.uint32), oracle.affine_dequantize(w, s, b, cols, group).view(np.uint32))
    assert np.array_equal(got16.view(np.uint16), oracle.affine_dequantize_f16(w, s, b, rows, cols, group).view(np.uint16))


@pytest.mark.parametrize("fmt,maker", [(1, synth.binary1), (2, synth.ternary2)])
def test_signed_dequant_bit_exact(ctx, oracle, fmt, maker):
    rows, cols = 64, 5120
    codes, scales = maker(1, "sdeq", rows, cols)
    dc, ds = dev(ctx, codes, scales)
    out = ctx.alloc(rows * cols * 4)
    bad = C.c_int(-1)
    ctx.call("signed_dequantize", fmt, dc, ds, out, rows, cols, C.byref(bad))
    got = out.download(np.float32, (rows, cols))
    ref = np.stack([oracle.signed_dequantize_row(fmt, codes[r], scales[r], cols, cols, 128) for r in range(rows)])
    assert bad.value == 0
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


def test_signed_dequant_flags_ternary_code_three(ctx):
    codes = np.full((1, 32), 0b11100100, np.uint8)  # every fourth code is the reserved value 3
    scales = np.ones((1, 1), np.float16)
    dc, ds = dev(ctx, codes, scales)
    out = ctx.alloc(128 * 4)
    bad = C.c_int(0)
    ctx.call("signed_dequantize", 2, dc, ds, out, 1, 128, C.byref(bad))
    assert bad.value == 1


# ── affine matvec family ────────────────────────────────────────────────────
AFFINE_SHAPES = [
    (4096, 1024, 64, 1),    # BASELINE config 0
    (257, 512, 64, 1),      # row tail (RegionExactnessTests)
    (5, 256, 64, 5),        # tiny, batch tail
    (2048, 2048, 64, 4), (512, 2048, 64, 8), (2048, 6144, 64, 16),  # config 1
    (1024, 4096, 64, 1), (512, 12288, 64, 1), (256, 12288, 64, 8),  # config 4 (K split over a cluster)
    (128, 1536, 128, 3), (96, 512, 32, 2), (64, 1024, 64, 20),
    (4096, 512, 64, 1), (4096, 1536, 64, 1), (4096, 3072, 64, 2), (512, 4096, 64, 1),  # per-rank shards, 4 / 8 ranks
]


@pytest.mark.parametrize("rows,cols,group,batch", AFFINE_SHAPES)
def test_affine_matvec(ctx, oracle, rows, cols, group, batch):
    w, s, b = synth.affine_u4(0, "mv", rows, cols, group)
    x = synth.activations(0, "x", batch, cols)
    dw, ds, db, dx = dev(ctx, w, s, b, x)
    y = ctx.alloc(batch * rows * 2 + 64).fill(0xFF)
    ctx.call("affine_matvec", dw, ds, db, dx, y, rows, cols, group, batch)
    got = y.download(np.float16, (batch, rows))
    ref = oracle.affine_matvec(w, s, b, x, rows, cols, group)
    assert rel_err(got, ref) < REL_TOL
    assert inf_err(got, ref) < INF_TOL
    canary = y.download(np.uint8, (64,), offset=batch * rows * 2)
    assert np.all(canary == 0xFF)  # nothing written past the output


def test_affine_matvec_reference_fixture(ctx, oracle):
    """The reference's own production-shape check (PrefillKernelTests.swift:11982-12061): 4096x1024, abs tol 0.02."""
    rows, cols, g = 4096, 1024, 64
    w, s, b = synth.ref_affine_fixture(rows, cols, g, 1)
    x = synth.ref_float16_vector(cols, float(synth.REGION_SEED_PRIMARY), 0.5)
    dw, ds, db, dx = dev(ctx, w, s, b, x)
    y = ctx.alloc(rows * 2)
    ctx.call("affine_matvec", dw, ds, db, dx, y, rows, cols, g, 1)
    got = y.download(np.float16, (rows,)).astype(np.float32)
    ref = oracle.affine_matvec(w, s, b, x, rows, cols, g)[0].astype(np.float32)
    assert np.max(np.abs(got - ref)) < 0.02
    assert np.max(np.abs(got)) > 1e-2


@pytest.mark.parametrize("batch", [1, 4, 8, 16])
def test_config1_layer_set(ctx, oracle, batch):
    """BASELINE config 1: the seven matrices of a 2048 / 6144 decoder layer (Q, K, V, O, gate, up,
    down; 16 x 4 x 128 heads), each at every batch of the config, through the records' kernels:
    Q as affine_matvec, K | V as fused_dual_affine_matvec, O and down as fused_affine_matvec_add,
    gate / up as fused_affine_gate_up_swiglu (fp32 gate and up, one rounding)."""
    H, I, KV, G = 2048, 6144, 512, 64
    t = {name: synth.affine_u4(21, name, r, c, G) for name, (r, c) in
         {"q": (H, H), "k": (KV, H), "v": (KV, H), "o": (H, H), "gate": (I, H), "up": (I, H), "down": (H, I)}.items()}
    x = synth.activations(21, "x", batch, H)
    xi = synth.activations(21, "xi", batch, I)
    res = synth.activations(21, "res", batch, H)
    d = {name: dev(ctx, *t[name]) for name in t}
    dx, dxi, dres = dev(ctx, x, xi, res)
    y, y2 = ctx.alloc(batch * I * 2), ctx.alloc(batch * I * 2)

    def check(got_buf, rows, ref):
        got = got_buf.download(np.float16, (batch, rows))
        assert rel_err(got, ref) < REL_TOL
        assert inf_err(got, ref) < INF_TOL

    ctx.call("affine_matvec", *d["q"], dx, y, H, H, G, batch)
    check(y, H, oracle.affine_matvec(*t["q"], x, H, H, G))
    ctx.call("affine_dual_matvec", *d["k"], *d["v"], dx, y, y2, KV, H, G, batch)
    check(y, KV, oracle.affine_matvec(*t["k"], x, KV, H, G))
    check(y2, KV, oracle.affine_matvec(*t["v"], x, KV, H, G))
    ctx.call("affine_matvec_add", *d["o"], dx, dres, y, H, H, G, batch)
    got = y.download(np.float16, (batch, H))
    assert add_rel_err(got, oracle.affine_matvec_add(*t["o"], x, res, H, H, G), oracle.affine_matvec(*t["o"], x, H, H, G)) < REL_TOL
    ctx.call("affine_gate_up_swiglu", *d["gate"], *d["up"], dx, y, I, H, G, batch)
    check(y, I, oracle.affine_gate_up_swiglu(*t["gate"], *t["up"], x, I, H, G, round_gate_up=False))
    ctx.call("affine_matvec_add", *d["down"], dxi, dres, y, H, I, G, batch)
    got = y.download(np.float16, (batch, H))
    assert add_rel_err(got, oracle.affine_matvec_add(*t["down"], xi, res, H, I, G), oracle.affine_matvec(*t["down"], xi, H, I, G)) < REL_TOL
    for bufs in list(d.values()) + [[dx, dxi, dres, y, y2]]:
        for b in bufs:
            b.free()


# batches of seventeen rows and more run on the tcgen05 QMMs (weights on the MMA's M, batch on its N): up to 64 rows
# with one accumulator slot per group drained in fp32, beyond that with every K step accumulated in tensor memory
@pytest.mark.parametrize("batch", [17, 32, 33, 64, 65, 100, 128, 200, 300, 512, 600])
@pytest.mark.parametrize("rows,cols", [(2048, 2048), (200, 512), (192, 512), (2048, 6144)])
def test_affine_qmm_modes(ctx, oracle, rows, cols, batch):
    """agent_affine_qmm_fixed_batched_full and the fused gate/up QMM (agent_affine_qmm.h:107-316, :360-742)
    at M = 17 ... 600: every epilogue, row tails (200 and 192 rows: the paired wide form needs a multiple of 64),
    a long K, two chunks of 256 batch rows, a second pass beyond 512."""
    if batch > 128 and cols == 6144:
        pytest.skip("the long-K case is covered up to 128 rows")
    a = synth.affine_u4(33, "qa", rows, cols, 64)
    b = synth.affine_u4(33, "qb", rows, cols, 64)
    x = synth.activations(33, "qx", batch, cols)
    res = synth.activations(33, "qres", batch, rows)
    d = dev(ctx, *a, *b, x, res)
    y0, y1 = ctx.alloc(batch * rows * 2 + 64).fill(0xFF), ctx.alloc(batch * rows * 2)
    ctx.call("affine_matvec", *d[:3], d[6], y0, rows, cols, 64, batch)
    ref_a = oracle.affine_matvec(*a, x, rows, cols, 64)
    got = y0.download(np.float16, (batch, rows))
    assert rel_err(got, ref_a) < REL_TOL and inf_err(got, ref_a) < INF_TOL
    assert np.all(y0.download(np.uint8, (64,), offset=batch * rows * 2) == 0xFF)
    ctx.call("affine_matvec_add", *d[:3], d[6], d[7], y1, rows, cols, 64, batch)
    assert add_rel_err(y1.download(np.float16, (batch, rows)), oracle.affine_matvec_add(*a, x, res, rows, cols, 64), ref_a) < REL_TOL
    ctx.call("affine_dual_matvec", *d[:7], y0, y1, rows, cols, 64, batch)
    assert rel_err(y0.download(np.float16, (batch, rows)), ref_a) < REL_TOL
    assert rel_err(y1.download(np.float16, (batch, rows)), oracle.affine_matvec(*b, x, rows, cols, 64)) < REL_TOL
    ctx.call("affine_gate_up_swiglu", *d[:7], y0, rows, cols, 64, batch)
    ref = oracle.affine_gate_up_swiglu(*a, *b, x, rows, cols, 64, round_gate_up=False)
    assert rel_err(y0.download(np.float16, (batch, rows)), ref) < REL_TOL
    assert ctx.device_error() == 0
    for buf in d + [y0, y1]:
        buf.free()


# batch 1 and 2 run on the integer-MMA kernel: every mode, row / K tails, long K, few chunks per warp
IMMA_SHAPES = [(4096, 4096, 1), (4096, 12288, 1), (100, 128, 2), (48, 256, 1), (1000, 2048, 2), (6144, 4096, 2), (16, 8192, 1)]


@pytest.mark.parametrize("rows,cols,batch", IMMA_SHAPES)
def test_affine_integer_mma_modes(ctx, oracle, rows, cols, batch):
    a = synth.affine_u4(30, "a", rows, cols, 64)
    b = synth.affine_u4(30, "b", rows, cols, 64)
    x = synth.activations(30, "x", batch, cols)
    res = synth.activations(30, "res", batch, rows)
    d = dev(ctx, *a, *b, x, res)
    y0, y1 = ctx.alloc(batch * rows * 2 + 64).fill(0xFF), ctx.alloc(batch * rows * 2)
    ctx.call("affine_matvec", *d[:3], d[6], y0, rows, cols, 64, batch)
    ref_a = oracle.affine_matvec(*a, x, rows, cols, 64)
    assert rel_err(y0.download(np.float16, (batch, rows)), ref_a) < REL_TOL
    assert np.all(y0.download(np.uint8, (64,), offset=batch * rows * 2) == 0xFF)
    # against the fp32 oracle the fixed-point activations cost less than fp16 output rounding
    ref32 = oracle.affine_matvec(*a, x, rows, cols, 64, f32=True)
    assert rel_err(y0.download(np.float16, (batch, rows)), ref32) < 6e-4
    ctx.call("affine_matvec_add", *d[:3], d[6], d[7], y1, rows, cols, 64, batch)
    assert rel_err(y1.download(np.float16, (batch, rows)), oracle.affine_matvec_add(*a, x, res, rows, cols, 64)) < REL_TOL
    ctx.call("affine_dual_matvec", *d[:7], y0, y1, rows, cols, 64, batch)
    assert rel_err(y0.download(np.float16, (batch, rows)), ref_a) < REL_TOL
    assert rel_err(y1.download(np.float16, (batch, rows)), oracle.affine_matvec(*b, x, rows, cols, 64)) < REL_TOL
    ctx.call("affine_gate_up_swiglu", *d[:7], y0, rows, cols, 64, batch)
    ref = oracle.affine_gate_up_swiglu(*a, *b, x, rows, cols, 64, round_gate_up=False)
    assert rel_err(y0.download(np.float16, (batch, rows)), ref) < REL_TOL


def test_affine_integer_mma_extreme_activations(ctx, oracle):
    """One huge activation sets the fixed-point scale of the row; the small ones must still count."""
    rows, cols = 256, 4096
    w, s, b = synth.affine_u4(31, "w", rows, cols, 64)
    x = (synth.activations(31, "x", 2, cols).astype(np.float32) * 1e-3).astype(np.float16)
    x[0, 77] = np.float16(900.0)
    x[1, :] = 0
    x[1, 5] = np.float16(6e-5)
    dw, ds, db, dx = dev(ctx, w, s, b, x)
    y = ctx.alloc(2 * rows * 2)
    ctx.call("affine_matvec", dw, ds, db, dx, y, rows, cols, 64, 2)
    assert rel_err(y.download(np.float16, (2, rows)), oracle.affine_matvec(w, s, b, x, rows, cols, 64)) < REL_TOL
    x[:] = 0
    ctx.call("affine_matvec", dw, ds, db, ctx.to_device(x), y, rows, cols, 64, 2)
    assert not np.any(y.download(np.uint16, (2, rows)) & 0x7FFF)  # all-zero activations give (signed) zeros


def test_affine_batched_equals_iterated_bitwise(ctx):
    """Batched == iterated, bit for bit (the reference pins this GPU-vs-GPU, PrefillKernelTests.swift:9101-9993)."""
    rows, cols, g, batch = 512, 2048, 64, 2
    w, s, b = synth.affine_u4(3, "bi", rows, cols, g)
    x = synth.activations(3, "x", batch, cols)
    dw, ds, db, dx = dev(ctx, w, s, b, x)
    y = ctx.alloc(batch * rows * 2)
    ctx.call("affine_matvec", dw, ds, db, dx, y, rows, cols, g, batch)
    batched = y.download(np.uint16, (batch, rows))
    y1 = ctx.alloc(rows * 2)
    for i in range(batch):
        ctx.call("affine_matvec", dw, ds, db, dx.at(i * cols * 2), y1, rows, cols, g, 1)
        assert np.array_equal(y1.download(np.uint16, (rows,)), batched[i])
    ctx.call("affine_matvec", dw, ds, db, dx, y, rows, cols, g, batch)
    assert np.array_equal(y.download(np.uint16, (batch, rows)), batched)  # run-to-run determinism


@pytest.mark.parametrize("rows,cols,batch", [(2048, 6144, 1), (257, 512, 3), (512, 12288, 8), (330, 12288, 13), (2048, 6144, 16),
                                             (4096, 1536, 1), (4096, 512, 1), (4096, 1536, 8)])
def test_affine_matvec_add(ctx, oracle, rows, cols, batch):
    w, s, b = synth.affine_u4(1, "add", rows, cols, 64)
    x = synth.activations(1, "x", batch, cols)
    res = synth.activations(1, "res", batch, rows)
    dw, ds, db, dx, dr = dev(ctx, w, s, b, x, res)
    ctx.call("affine_matvec_add", dw, ds, db, dx, dr, dr, rows, cols, 64, batch)  # in place on the residual
    got = dr.download(np.float16, (batch, rows))
    ref = oracle.affine_matvec_add(w, s, b, x, res, rows, cols, 64)
    assert rel_err(got, ref) < REL_TOL


@pytest.mark.parametrize("rows,cols,batch", [(6144, 2048, 1), (261, 512, 4), (1024, 4096, 16)])
def test_affine_gate_up_swiglu(ctx, oracle, rows, cols, batch):
    gw, gs, gb = synth.affine_u4(2, "gate", rows, cols, 64)
    uw, us, ub = synth.affine_u4(2, "up", rows, cols, 64)
    x = synth.activations(2, "x", batch, cols)
    d = dev(ctx, gw, gs, gb, uw, us, ub, x)
    y = ctx.alloc(batch * rows * 2)
    ctx.call("affine_gate_up_swiglu", *d, y, rows, cols, 64, batch)
    got = y.download(np.float16, (batch, rows))
    ref = oracle.affine_gate_up_swiglu(gw, gs, gb, uw, us, ub, x, rows, cols, 64, round_gate_up=False)
    assert rel_err(got, ref) < REL_TOL


def test_affine_dual_matvec(ctx, oracle):
    rows, cols, batch = 512, 2048, 2
    a = synth.affine_u4(4, "k", rows, cols, 64)
    b = synth.affine_u4(4, "v", rows, cols, 64)
    x = synth.activations(4, "x", batch, cols)
    d = dev(ctx, *a, *b, x)
    y0, y1 = ctx.alloc(batch * rows * 2), ctx.alloc(batch * rows * 2)
    ctx.call("affine_dual_matvec", *d, y0, y1, rows, cols, 64, batch)
    assert rel_err(y0.download(np.float16, (batch, rows)), oracle.affine_matvec(*a, x, rows, cols, 64)) < REL_TOL
    assert rel_err(y1.download(np.float16, (batch, rows)), oracle.affine_matvec(*b, x, rows, cols, 64)) < REL_TOL


# ── fused extension kernels: same rounding points as the kernels they replace ──
def _device_norm(ctx, x, nw, eps):
    """rms_norm_1pw on the device (itself checked against the oracle below): a folded norm uses the
    same reduction order, so the kernels that fold it are compared on these exact activations."""
    batch, cols = x.shape
    dx, dn = dev(ctx, x, nw)
    dy = ctx.alloc(batch * cols * 2)
    ctx.call("rms_norm_1pw", dx, dn, dy, cols, C.c_float(eps), batch)
    return dy.download(np.float16, (batch, cols)), dy


def _multi(ctx, tensors, x, norm_w, eps, cols, batch):
    arr = (capi.AffineTensor * len(tensors))()
    outs = []
    for i, (w, s, b, rows) in enumerate(tensors):
        dw, ds, db = dev(ctx, w, s, b)
        y = ctx.alloc(batch * rows * 2).fill(0xFF)
        arr[i] = capi.AffineTensor(dw.ptr, ds.ptr, db.ptr, y.ptr, rows)
        outs.append((y, rows, (dw, ds, db)))
    dx = ctx.to_device(x)
    dn = ctx.to_device(norm_w) if norm_w is not None else None
    st = ctx.call_status("affine_multi_matvec", C.cast(arr, C.c_void_p), len(tensors), dx, dn, C.c_float(eps), cols, 64, batch)
    return st, [y.download(np.float16, (batch, rows)) for y, rows, _ in outs]


@pytest.mark.parametrize("rows,cols,batch,norm", [((4096, 1024, 1024), 4096, 1, True), ((256, 64, 72), 1024, 3, True),
                                                  ((512, 128, 128), 2048, 8, False), ((48, 16, 5), 1024, 1, True),
                                                  ((256, 64, 40), 4096, 11, True), ((512, 128, 128), 4096, 1, True)])
def test_affine_multi_matvec(ctx, oracle, rows, cols, batch, norm):
    eps = 1e-6
    tensors = [(*synth.affine_u4(21, f"t{i}", r, cols, 64), r) for i, r in enumerate(rows)]
    x = synth.activations(21, "x", batch, cols)
    nw = synth.normal_f16(21, "norm", (cols,), 0.1) if norm else None
    st, got = _multi(ctx, tensors, x, nw, eps, cols, batch)
    assert st == 0, ctx.last_error()
    xn, dxn = _device_norm(ctx, x, nw, eps) if norm else (x, ctx.to_device(x))
    for (w, s, b, r), g in zip(tensors, got):
        assert rel_err(g, oracle.affine_matvec(w, s, b, xn, r, cols, 64)) < REL_TOL
        y = ctx.alloc(batch * r * 2)
        ctx.call("affine_matvec", *dev(ctx, w, s, b), dxn, y, r, cols, 64, batch)
        sep = y.download(np.float16, (batch, r))
        assert np.array_equal(g.view(np.uint16), sep.view(np.uint16)), "one launch per tensor must give the same bits"


def test_affine_multi_matvec_rejects_ineligible_shapes(ctx):
    t = [(*synth.affine_u4(22, "a", 24, 1024, 64), 24), (*synth.affine_u4(22, "b", 16, 1024, 64), 16)]
    x = synth.activations(22, "x", 1, 1024)
    st, _ = _multi(ctx, t, x, None, 1e-6, 1024, 1)  # first tensor's rows are not a multiple of 16
    assert st in (capi.BAD_ARGUMENT, capi.UNSUPPORTED)
    t = [(*synth.affine_u4(22, "c", 16, 192, 64), 16)]
    nw = synth.normal_f16(22, "norm", (192,), 0.1)
    st, _ = _multi(ctx, t, synth.activations(22, "x2", 1, 192), nw, 1e-6, 192, 1)  # a folded norm needs cols % 128 == 0
    assert st in (capi.BAD_ARGUMENT, capi.UNSUPPORTED)


@pytest.mark.parametrize("rows,cols,batch", [(12288, 4096, 1), (200, 1024, 4), (1024, 2048, 8), (520, 4096, 16), (1536, 4096, 1)])
def test_rmsnorm_affine_gate_up_swiglu(ctx, oracle, rows, cols, batch):
    eps = 1e-6
    gw, gs, gb = synth.affine_u4(23, "gate", rows, cols, 64)
    uw, us, ub = synth.affine_u4(23, "up", rows, cols, 64)
    x = synth.activations(23, "x", batch, cols)
    nw = synth.normal_f16(23, "norm", (cols,), 0.1)
    d = dev(ctx, gw, gs, gb, uw, us, ub, x, nw)
    y = ctx.alloc(batch * rows * 2)
    ctx.call("rmsnorm_affine_gate_up_swiglu", *d, C.c_float(eps), y, rows, cols, 64, batch)
    xn, dxn = _device_norm(ctx, x, nw, eps)
    ref = oracle.affine_gate_up_swiglu(gw, gs, gb, uw, us, ub, xn, rows, cols, 64, round_gate_up=False)
    assert rel_err(y.download(np.float16, (batch, rows)), ref) < REL_TOL
    y2 = ctx.alloc(batch * rows * 2)
    ctx.call("affine_gate_up_swiglu", *d[:6], dxn, y2, rows, cols, 64, batch)
    assert np.array_equal(y.download(np.uint16, (batch, rows)), y2.download(np.uint16, (batch, rows)))


@pytest.mark.parametrize("position,layout", [(0, 1), (77, 1), (4095, 0), (32767, 1)])
def test_rope_qkv_append_is_the_three_kernels(ctx, oracle, position, layout):
    nq, nkv, d, cap = 8, 2, 128, 32768
    base_log2 = float(np.log2(np.float32(1e6)))
    q = synth.activations(24, "q", nq, d)
    k = synth.activations(24, "k", nkv, d)
    v = synth.activations(24, "v", nkv, d)
    dq, dk, dv = dev(ctx, q, k, v)
    kc = ctx.alloc(nkv * cap * d * 2).fill(0)
    vc = ctx.alloc(nkv * cap * d * 2).fill(0)
    ctx.call("rope_qkv_append", dq, dk, dv, kc, vc, cap, d, nq, nkv, layout, position, C.c_float(base_log2), 1, 0)
    # the separate kernels on the same inputs: bit-identical results
    dq2, dk2, dv2 = dev(ctx, q, k, v)
    kc2 = ctx.alloc(nkv * cap * d * 2).fill(0)
    vc2 = ctx.alloc(nkv * cap * d * 2).fill(0)
    ctx.call("apply_rope", dq2, None, None, d, d, nq, layout, position, C.c_float(base_log2), 1, 1)
    ctx.call("rope_kv_cache_update", kc2, dk2, None, None, cap, d, position, nkv, d, layout, C.c_float(base_log2), 1, 1, 0)
    ctx.call("kv_cache_update", vc2, dv2, cap, d, position, nkv, 1, 0)
    assert np.array_equal(dq.download(np.uint16, (nq, d)), dq2.download(np.uint16, (nq, d)))
    assert np.array_equal(kc.download(np.uint16, (nkv, cap, d)), kc2.download(np.uint16, (nkv, cap, d)))
    assert np.array_equal(vc.download(np.uint16, (nkv, cap, d)), vc2.download(np.uint16, (nkv, cap, d)))
    # and the oracle
    assert np.array_equal(dq.download(np.uint16, (nq * d,)), oracle.apply_rope(q, d, d, nq, layout, position, base_log2, 1).view(np.uint16).ravel())
    refk = oracle.rope_kv_cache_update(np.zeros((nkv, cap, d), np.float16), k, cap, d, position, nkv, d, layout, base_log2, 1)
    assert np.array_equal(kc.download(np.uint16, (nkv, cap, d)), refk.view(np.uint16).reshape(nkv, cap, d))
    assert ctx.call_status("rope_qkv_append", dq, dk, dv, kc, vc, cap, d, nq, nkv, layout, cap, C.c_float(base_log2), 1, 0) == capi.OUT_OF_RANGE


def test_affine_rejects_bad_arguments(ctx):
    d = ctx.alloc(4096)
    assert ctx.call_status("affine_matvec", d, d, d, d, d, 16, 100, 64, 1) == capi.BAD_ARGUMENT  # cols % group
    assert ctx.call_status("affine_matvec", d, d, d, d, d, 16, 128, 48, 1) == capi.BAD_ARGUMENT  # group
    assert ctx.call_status("affine_matvec", d, d, d, None, d, 16, 128, 64, 1) == capi.BAD_ARGUMENT
    assert ctx.call_status("affine_matvec", d.at(8), d, d, d, d, 16, 128, 64, 1) == capi.BAD_ARGUMENT  # alignment
    assert "16-byte" in ctx.last_error()


# ── dense fp16 matvec (LM head) ─────────────────────────────────────────────
@pytest.mark.parametrize("rows,cols,batch", [(4099, 4096, 1), (1000, 2048, 8), (333, 1024, 11), (18992, 4096, 1)])
def test_fp16_matvec(ctx, oracle, rows, cols, batch):
    w = synth.normal_f16(5, "head", (rows, cols), 0.02)
    x = synth.activations(5, "x", batch, cols)
    dw, dx = dev(ctx, w, x)
    y = ctx.alloc(batch * rows * 2)
    ctx.call("fp16_matvec", dw, dx, y, rows, cols, batch)
    got = y.download(np.float16, (batch, rows))
    assert rel_err(got, oracle.fp16_matvec(w, x, rows, cols)) < REL_TOL


def test_fp16_matvec_clamps(ctx):
    w = np.full((8, 64), 60000.0, np.float16)
    x = np.ones(64, np.float16)
    dw, dx = dev(ctx, w, x)
    y = ctx.alloc(16)
    ctx.call("fp16_matvec", dw, dx, y, 8, 64, 1)
    assert np.all(y.download(np.float16, (8,)) == np.float16(65504))


# ── binary / ternary ────────────────────────────────────────────────────────
def _ref_signed_case(fmt):
    """SignedQuantKernelTests.swift:989-1047: rows 5, cols 256, batch 5."""
    rows, cols, batches = 5, 256, 5
    r = np.arange(rows)[:, None]
    c = np.arange(cols)[None, :]
    code = ((r * 13 + c * 7) & 1 if fmt == 1 else (r * 13 + c * 7) % 3).astype(np.uint8)
    codes = synth.pack_codes(code, fmt)
    scales = (np.float32(0.03125) * ((np.arange(rows * 2) % 5) + 1)).astype(np.float16).reshape(rows, 2)
    x = (np.sin((np.arange(batches * cols) * 17 + 3).astype(np.float32)) * np.float32(0.75)).astype(np.float16).reshape(batches, cols)
    return rows, cols, batches, codes, scales, x


@pytest.mark.parametrize("fmt", [1, 2])
def test_signed_matvec_reference_fixture(ctx, oracle, fmt):
    rows, cols, batches, codes, scales, x = _ref_signed_case(fmt)
    dc, ds, dx = dev(ctx, codes, scales, x)
    y = ctx.alloc(batches * rows * 2)
    ctx.call("signed_matvec", fmt, dc, ds, dx, y, rows, cols, batches)
    got = y.download(np.float16, (batches, rows)).astype(np.float32)
    ref = oracle.signed_matvec(fmt, codes, scales, x, rows, cols, f32=True)
    assert np.all(np.abs(got - ref) <= np.maximum(0.02, np.abs(ref) * 0.01))  # the reference's tolerance
    assert rel_err(got, ref) < REL_TOL


def test_ternary_matches_mlx_golden_bits(ctx):
    """SignedQuantKernelTests.swift:87-106, :143-164: operands are dyadic, so any fp32 order gives these bits."""
    for rows, cols, batches, unit, expected in [
        (9, 512, 1, 0.03125, [0xb190, 0x3468, 0xb0b0, 0x2e20, 0xa580, 0x3370, 0xb518, 0x3498, 0xb170]),
        (9, 5120, 3, 0.00390625, [0xa160, 0x9dc0, 0x2420, 0xa160, 0x9dc0, 0x2420, 0xa160, 0x9dc0, 0x2420,
                                  0x2520, 0xa650, 0x1cc0, 0x2520, 0xa650, 0x1cc0, 0x2520, 0xa650, 0x1cc0,
                                  0x2280, 0x1700, 0xa360, 0x2280, 0x1700, 0xa360, 0x2280, 0x1700, 0xa360]),
    ]:
        r = np.arange(rows)[:, None]
        c = np.arange(cols)[None, :]
        codes = synth.pack_codes(((r * 13 + c * 7) % 3).astype(np.uint8), 2)
        groups = cols // 128
        scales = (np.float32(unit) * ((np.arange(rows * groups) % 5) + 1)).astype(np.float16).reshape(rows, groups)
        i = np.arange(batches * cols)
        x = (((i * 17 + 3) % 31 - 15).astype(np.float32) / 16).astype(np.float16).reshape(batches, cols)
        dc, ds, dx = dev(ctx, codes, scales, x)
        y = ctx.alloc(batches * rows * 2)
        ctx.call("signed_matvec", 2, dc, ds, dx, y, rows, cols, batches)
        assert y.download(np.uint16, (batches * rows,)).tolist() == expected


@pytest.mark.parametrize("fmt,maker", [(1, synth.binary1), (2, synth.ternary2)])
@pytest.mark.parametrize("rows,cols", [(1024, 5120), (512, 17408)])
def test_signed_matvec_27b_shapes(ctx, oracle, fmt, maker, rows, cols):
    codes, scales = maker(6, "sm", rows, cols)
    x = synth.activations(6, "x", 1, cols)
    dc, ds, dx = dev(ctx, codes, scales, x)
    y = ctx.alloc(rows * 2)
    ctx.call("signed_matvec", fmt, dc, ds, dx, y, rows, cols, 1)
    assert rel_err(y.download(np.float16, (1, rows)), oracle.signed_matvec(fmt, codes, scales, x, rows, cols)) < REL_TOL


@pytest.mark.parametrize("fmt,maker", [(1, synth.binary1), (2, synth.ternary2)])
def test_signed_matvec_add_and_gate_up(ctx, oracle, fmt, maker):
    rows, cols, batch = 261, 1024, 3
    gc, gs = maker(7, "g", rows, cols)
    uc, us = maker(7, "u", rows, cols)
    x = synth.activations(7, "x", batch, cols)
    res = synth.activations(7, "r", batch, rows)
    dgc, dgs, duc, dus, dx, dr = dev(ctx, gc, gs, uc, us, x, res)
    y = ctx.alloc(batch * rows * 2)
    ctx.call("signed_matvec_add", fmt, dgc, dgs, dx, dr, y, rows, cols, batch)
    assert rel_err(y.download(np.float16, (batch, rows)), oracle.signed_matvec_add(fmt, gc, gs, x, res, rows, cols)) < REL_TOL
    ctx.call("signed_gate_up_swiglu", fmt, dgc, dgs, duc, dus, dx, y, rows, cols, batch)
    got = y.download(np.float16, (batch, rows))
    staged = oracle.signed_gate_up_swiglu(fmt, gc, gs, uc, us, x, rows, cols, staged=True)
    plain = oracle.signed_gate_up_swiglu(fmt, gc, gs, uc, us, x, rows, cols, staged=False).astype(np.float32)
    assert rel_err(got, staged) < 4e-3  # a one-ulp flip of gate or up moves the staged fp16 chain by a few ulp
    g32 = got.astype(np.float32)
    assert np.all(np.abs(g32 - plain) <= np.maximum(0.03, np.abs(plain) * 0.015))  # the reference's tolerance (:1227-1232)


@pytest.mark.parametrize("fmt,maker", [(1, synth.binary1), (2, synth.ternary2)])
@pytest.mark.parametrize("rows,cols,batch", [(1024, 5120, 2), (100, 512, 1), (48, 1536, 2), (17408, 5120, 1)])
def test_signed_integer_mma_modes(ctx, oracle, fmt, maker, rows, cols, batch):
    """Batch 1 and 2 with cols % 512 == 0 run on the integer-MMA kernel: every mode, row tails, uneven K split."""
    gc, gs = maker(32, "g", rows, cols)
    uc, us = maker(32, "u", rows, cols)
    x = synth.activations(32, "x", batch, cols)
    res = synth.activations(32, "r", batch, rows)
    dgc, dgs, duc, dus, dx, dr = dev(ctx, gc, gs, uc, us, x, res)
    y = ctx.alloc(batch * rows * 2 + 64).fill(0xFF)
    ctx.call("signed_matvec", fmt, dgc, dgs, dx, y, rows, cols, batch)
    got = y.download(np.float16, (batch, rows))
    assert rel_err(got, oracle.signed_matvec(fmt, gc, gs, x, rows, cols)) < REL_TOL
    assert rel_err(got, oracle.signed_matvec(fmt, gc, gs, x, rows, cols, f32=True)) < 6e-4  # fp16 output rounding only
    assert np.all(y.download(np.uint8, (64,), offset=batch * rows * 2) == 0xFF)
    ctx.call("signed_matvec_add", fmt, dgc, dgs, dx, dr, y, rows, cols, batch)
    assert add_rel_err(y.download(np.float16, (batch, rows)), oracle.signed_matvec_add(fmt, gc, gs, x, res, rows, cols),
                       oracle.signed_matvec(fmt, gc, gs, x, rows, cols)) < REL_TOL
    ctx.call("signed_gate_up_swiglu", fmt, dgc, dgs, duc, dus, dx, y, rows, cols, batch)
    staged = oracle.signed_gate_up_swiglu(fmt, gc, gs, uc, us, x, rows, cols, staged=True)
    assert rel_err(y.download(np.float16, (batch, rows)), staged) < 4e-3


# ── attention ───────────────────────────────────────────────────────────────
@pytest.mark.parametrize("seq_len,window", [(32, 0), (32, 8), (192, 0), (1, 0), (17, 0)])
def test_attention_reference_fixture(ctx, oracle, seq_len, window):
    """RegionExactnessTests.swift:1271-1357: 4 q heads, 2 kv heads, head_dim 128."""
    n_q, n_kv, d = 4, 2, 128
    cap = max(seq_len, 64)
    q, k, v = synth.ref_attention_inputs(n_q, n_kv, d, cap, 1)
    dq, dk, dv = dev(ctx, q, k, v)
    out = ctx.alloc(n_q * d * 2)
    ctx.call("attention_decode", dq, dk, dv, out, n_q, n_kv, d, cap, seq_len, C.c_float(1 / np.sqrt(d)), window, 1, 0)
    got = out.download(np.float16, (n_q, d))
    ref = oracle.attention_decode(q, k, v, n_q, n_kv, d, cap, seq_len, sliding_window=window)
    assert rel_err(got, ref) < REL_TOL
    assert np.max(np.abs(got.astype(np.float32))) > 1e-3


def _attention_case(ctx, oracle, n_q, n_kv, d, ctx_len, batch):
    cap = ctx_len + 8
    k = synth.kv_cache(8, "k", batch, n_kv, cap, d)
    v = synth.kv_cache(8, "v", batch, n_kv, cap, d)
    q = synth.activations(8, "q", batch, n_q, d)
    dq, dk, dv = dev(ctx, q, k, v)
    out = ctx.alloc(batch * n_q * d * 2)
    ctx.call("attention_decode", dq, dk, dv, out, n_q, n_kv, d, cap, ctx_len, C.c_float(1 / np.sqrt(d)), 0, batch, C.c_size_t(n_kv * cap * d))
    got = out.download(np.float16, (batch, n_q, d))
    for b in range(batch):
        ref = oracle.attention_decode(q[b], k[b], v[b], n_q, n_kv, d, cap, ctx_len)
        assert rel_err(got[b], ref) < REL_TOL
        assert inf_err(got[b], ref) < INF_TOL
    for buf in (dq, dk, dv, out):
        buf.free()


@pytest.mark.parametrize("n_q,n_kv,d", [(16, 4, 128), (8, 2, 256)])
@pytest.mark.parametrize("ctx_len", [1024, 4096, 16384, 32768])
@pytest.mark.parametrize("batch", [1, 8])
def test_attention_config3(ctx, oracle, n_q, n_kv, d, ctx_len, batch):
    """BASELINE config 3, every cell: both head shapes x contexts 1k / 4k / 16k / 32k x batch 1 / 8."""
    _attention_case(ctx, oracle, n_q, n_kv, d, ctx_len, batch)


@pytest.mark.parametrize("n_q,n_kv,d", [(32, 8, 128), (16, 1, 64), (4, 1, 128), (8, 2, 128)])
@pytest.mark.parametrize("ctx_len,batch", [(1024, 1), (4096, 1), (1000, 8), (5000, 2)])
def test_attention_other_head_shapes(ctx, oracle, n_q, n_kv, d, ctx_len, batch):
    _attention_case(ctx, oracle, n_q, n_kv, d, ctx_len, batch)


@pytest.mark.parametrize("n_q,n_kv,d,position,batch,layout", [(32, 8, 128, 0, 1, 1), (32, 8, 128, 530, 1, 1), (16, 4, 128, 4095, 2, 1),
                                                              (8, 2, 256, 777, 1, 0), (16, 1, 64, 129, 3, 1), (4, 1, 128, 600, 1, 1), (8, 2, 128, 5000, 1, 1)])
def test_rope_attention_decode_is_the_four_kernels(ctx, oracle, n_q, n_kv, d, position, batch, layout):
    """RoPE on q, RoPE + append of K, append of V and attention in one launch: the bits of the
    four separate launches, with the new token as the last key."""
    cap = position + 9
    base_log2 = float(np.log2(np.float32(1e6)))
    k = synth.kv_cache(33, "k", batch, n_kv, cap, d)
    v = synth.kv_cache(33, "v", batch, n_kv, cap, d)
    q = synth.activations(33, "q", batch, n_q, d)
    kn = (synth.activations(33, "kn", batch, n_kv, d).astype(np.float32) / np.sqrt(d)).astype(np.float16)
    vn = (synth.activations(33, "vn", batch, n_kv, d).astype(np.float32) / np.sqrt(d)).astype(np.float16)
    stride = C.c_size_t(n_kv * cap * d)
    scale = C.c_float(1 / np.sqrt(d))
    # separate launches
    dq, dk, dv, dkn, dvn = dev(ctx, q, k, v, kn, vn)
    want = ctx.alloc(batch * n_q * d * 2)
    ctx.call("rope_qkv_append", dq, dkn, dvn, dk, dv, cap, d, n_q, n_kv, layout, position, C.c_float(base_log2), batch, stride)
    ctx.call("attention_decode", dq, dk, dv, want, n_q, n_kv, d, cap, position + 1, scale, 0, batch, stride)
    # one launch
    dq2, dk2, dv2 = dev(ctx, q, k, v)
    got = ctx.alloc(batch * n_q * d * 2).fill(0xFF)
    ctx.call("rope_attention_decode", dq2, dkn, dvn, dk2, dv2, got, n_q, n_kv, d, cap, position, scale, 0, layout, C.c_float(base_log2), batch, stride)
    assert np.array_equal(got.download(np.uint16, (batch, n_q, d)), want.download(np.uint16, (batch, n_q, d)))
    assert np.array_equal(dk2.download(np.uint16, (batch, n_kv, cap, d)), dk.download(np.uint16, (batch, n_kv, cap, d)))
    assert np.array_equal(dv2.download(np.uint16, (batch, n_kv, cap, d)), dv.download(np.uint16, (batch, n_kv, cap, d)))
    assert np.array_equal(dq2.download(np.uint16, (batch, n_q, d)), q.view(np.uint16))  # q itself is left alone
    # twice in a row: the split counters are back at zero
    ctx.call("rope_attention_decode", dq2, dkn, dvn, dk2, dv2, got.fill(0), n_q, n_kv, d, cap, position, scale, 0, layout, C.c_float(base_log2), batch, stride)
    assert np.array_equal(got.download(np.uint16, (batch, n_q, d)), want.download(np.uint16, (batch, n_q, d)))
    # and in place
    ctx.call("rope_attention_decode", dq2, dkn, dvn, dk2, dv2, dq2, n_q, n_kv, d, cap, position, scale, 0, layout, C.c_float(base_log2), batch, stride)
    assert np.array_equal(dq2.download(np.uint16, (batch, n_q, d)), want.download(np.uint16, (batch, n_q, d)))
    assert ctx.call_status("rope_attention_decode", dq2, dkn, dvn, dk2, dv2, got, n_q, n_kv, d, cap, cap, scale, 0, layout, C.c_float(base_log2), batch, stride) == capi.OUT_OF_RANGE


def test_attention_in_place(ctx, oracle):
    n_q, n_kv, d, cap, seq = 16, 4, 128, 600, 555
    k = synth.kv_cache(9, "k", 1, n_kv, cap, d)[0]
    v = synth.kv_cache(9, "v", 1, n_kv, cap, d)[0]
    q = synth.activations(9, "q", n_q, d)
    dq, dk, dv = dev(ctx, q, k, v)
    ctx.call("attention_decode", dq, dk, dv, dq, n_q, n_kv, d, cap, seq, C.c_float(1 / np.sqrt(d)), 0, 1, 0)
    assert rel_err(dq.download(np.float16, (n_q, d)), oracle.attention_decode(q, k, v, n_q, n_kv, d, cap, seq)) < REL_TOL


# ── glue ────────────────────────────────────────────────────────────────────
@pytest.mark.parametrize("dim,batch", [(2048, 1), (4096, 3), (5120, 1), (100, 2)])
def test_rms_norm_1pw(ctx, oracle, dim, batch):
    x = synth.activations(10, "x", batch, dim)
    w = (synth.activations(10, "w", dim).astype(np.float32) * 0.1).astype(np.float16)
    dx, dw = dev(ctx, x, w)
    y = ctx.alloc(batch * dim * 2)
    ctx.call("rms_norm_1pw", dx, dw, y, dim, C.c_float(1e-6), batch)
    got = y.download(np.float16, (batch, dim))
    for b in range(batch):
        ref = oracle.rms_norm_1pw(x[b], w, 1e-6, two_stage=True)
        d = ulp_diff_f16(got[b], ref)
        assert d.max() <= 2 and np.mean(d > 0) < 0.01  # summation order may move rsqrt by an fp32 ulp
        assert rel_err(got[b], oracle.rms_norm_1pw(x[b], w, 1e-6, two_stage=False)) < REL_TOL


def test_per_head_rms_norm(ctx, oracle):
    heads, d = 16, 128
    x = synth.activations(11, "x", heads, d)
    w = (1 + synth.activations(11, "w", d).astype(np.float32) * 0.1).astype(np.float16)
    dx, dw = dev(ctx, x, w)
    ctx.call("per_head_rms_norm", dx, dw, dx, heads, d, C.c_float(1e-6))
    d_ulp = ulp_diff_f16(dx.download(np.float16, (heads, d)), oracle.per_head_rms_norm(x, w, heads, d, 1e-6))
    assert d_ulp.max() <= 1 and np.mean(d_ulp > 0) < 0.01


def test_elementwise_add_and_swiglu(ctx, oracle):
    n = 6144 * 3 + 5
    a, b = synth.activations(12, "a", n), synth.activations(12, "b", n)
    da, db = dev(ctx, a, b)
    y = ctx.alloc(n * 2)
    ctx.call("elementwise_add", da, db, y, C.c_size_t(n))
    assert np.array_equal(y.download(np.uint16, (n,)), oracle.elementwise_add(a, b).view(np.uint16))
    a4 = (a.astype(np.float32) * 4).astype(np.float16)
    da4 = ctx.to_device(a4)
    ctx.call("swiglu_fused", da4, db, y, C.c_size_t(n))
    d = ulp_diff_f16(y.download(np.float16, (n,)), oracle.swiglu_staged(a4, b))
    assert d.max() <= 2 and np.mean(d > 0) < 0.02  # expf differs from the host's by an ulp at most


def test_embedding_gathers(ctx, oracle):
    vocab, hidden = 1000, 2048
    table = synth.normal_f16(13, "emb", (vocab, hidden), 0.02)
    tok = np.array([7, 999, 0], np.int32)
    dt, dtok = dev(ctx, table, tok)
    y = ctx.alloc(3 * hidden * 2)
    ctx.call("embedding_gather", dt, dtok, y, hidden, 3)
    assert np.array_equal(y.download(np.uint16, (3, hidden)), table[tok].view(np.uint16))
    w, s, b = synth.affine_u4(13, "aemb", vocab, hidden, 64)
    dw, ds, db = dev(ctx, w, s, b)
    ctx.call("affine_embedding_gather", dw, ds, db, dtok.at(4), y, hidden, 64)
    ref = oracle.affine_dequantize_f16(w[999:1000], s[999:1000], b[999:1000], 1, hidden, 64)
    assert np.array_equal(y.download(np.uint16, (1, hidden)), ref.view(np.uint16))


@pytest.mark.parametrize("layout", [0, 1, 2])
def test_rope_table_mode_bit_exact(ctx, oracle, layout):
    heads, d, rope = 4, 128, 64
    qk = synth.ref_float16_vector(heads * d, float(synth.REGION_SEED_PRIMARY), 0.5, 0.1)
    cos = synth.ref_float16_vector(rope, float(synth.REGION_SEED_SECONDARY), 0.9, phase=0.0237)
    sin = synth.ref_float16_vector(rope, float(synth.REGION_SEED_TERTIARY), 0.9, phase=0.0193)
    dq, dc, dsn = dev(ctx, qk, cos, sin)
    ctx.call("apply_rope", dq, dc, dsn, d, rope, heads, layout, 0, C.c_float(0), 0, 1)
    ref = oracle.apply_rope(qk, d, rope, heads, layout, 0, math_mode=0, cos=cos, sin=sin)
    assert np.array_equal(dq.download(np.uint16, (heads * d,)), ref.view(np.uint16))


@pytest.mark.parametrize("position", [0, 1, 77, 4095, 32767])
def test_rope_analytic_and_kv_append(ctx, oracle, position):
    heads, d, cap = 8, 128, 32768
    base_log2 = float(np.log2(np.float32(1e6)))
    qk = synth.activations(14, "qk", heads, d)
    dq = ctx.to_device(qk)
    ctx.call("apply_rope", dq, None, None, d, d, heads, 1, position, C.c_float(base_log2), 1, 1)
    ref = oracle.apply_rope(qk, d, d, heads, 1, position, base_log2, 1)
    du = ulp_diff_f16(dq.download(np.float16, (heads, d)), ref.reshape(heads, d))
    assert du.max() <= 1 and np.mean(du > 0) < 0.02  # device sincosf / exp2f vs the host's
    cache = ctx.alloc(heads * cap * d * 2).fill(0)
    new = ctx.to_device(qk)
    ctx.call("kv_cache_update", cache, new, cap, d, position, heads, 1, 0)
    row = cache.download(np.uint16, (heads, cap, d))
    assert np.array_equal(row[:, position, :], qk.view(np.uint16))
    assert row.sum(dtype=np.uint64) == qk.view(np.uint16).sum(dtype=np.uint64)  # nothing else touched
    ctx.call("rope_kv_cache_update", cache, new, None, None, cap, d, position, heads, d, 1, C.c_float(base_log2), 1, 1, 0)
    got = cache.download(np.float16, (heads, cap, d))[:, position, :]
    assert ulp_diff_f16(got, ref.reshape(heads, d)).max() <= 1
    assert ctx.call_status("kv_cache_update", cache, new, cap, d, cap, heads, 1, 0) == capi.OUT_OF_RANGE


def test_argmax_ties_and_full_vocab(ctx, oracle):
    out = ctx.alloc(8 * 4)
    for arr in [np.array([1, 3, 3, 2], np.float16), np.array([0x8000, 0x0000, 0x8000], np.uint16).view(np.float16),
                np.array([-5, -2, -2], np.float16), np.full(5000, -65504, np.float16)]:
        d = ctx.to_device(arr)
        ctx.call("argmax_f16", d, out, arr.size, 1)
        assert int(out.download(np.int32, (1,))[0]) == oracle.argmax_f16(arr)
    logits = synth.activations(15, "logits", 3, 151936)
    logits[1, 150000] = logits[1, 17] = np.float16(9.0)
    d = ctx.to_device(logits)
    ctx.call("argmax_f16", d, out, 151936, 3)
    got = out.download(np.int32, (3,))
    assert got.tolist() == [oracle.argmax_f16(logits[b]) for b in range(3)]
    assert got[1] == 17
