"""The DeltaNet step as the reference's older pipelines cut it (Resources/Shaders/recurrence.metal:44-503,
:836-862; prefill_recurrence.metal:42-285): compute_gates, state_decay, kv_mem_readout, compute_delta,
outer_product_update, query_readout, their fused pairs, and the two one-threadgroup-per-head fused kernels.
The reference has no test or scalar oracle for them (its emitters dispatch the tiled forms), so the oracle's
restatement is checked for consistency (fused pairs against the separate steps, fused kernels against the tiled
forms that are pinned on the reference's fixtures), then the CUDA kernels against the oracle as records under
the reference's names and bindings."""
import ctypes as C

import numpy as np
import pytest

from smelt_b200 import capi
from helpers import ulp_diff_f16

F = np.float32


def halves(rng, *shape, scale=1.0):
    return (rng.standard_normal(shape) * scale).astype(np.float16)


def step_inputs(seed, heads, d):
    rng = np.random.default_rng(seed)
    return dict(state=halves(rng, heads, d, d, scale=0.1), key=halves(rng, heads, d, scale=0.1), query=halves(rng, heads, d, scale=0.1),
                value=halves(rng, heads, d), b=halves(rng, heads), a=halves(rng, heads), a_log=halves(rng, heads, scale=0.3),
                dt_bias=halves(rng, heads, scale=0.3))


def test_oracle_gates_are_the_float_formulas(oracle):
    t = step_inputs(1, 24, 64)
    beta, g = oracle.dn_compute_gates(t["b"], t["a"], t["a_log"], t["dt_bias"], 24)
    x = t["a"].astype(np.float64) + t["dt_bias"].astype(np.float64)
    want_g = -np.exp(t["a_log"].astype(np.float64)) * np.log1p(np.exp(x))
    assert np.max(ulp_diff_f16(beta, (1 / (1 + np.exp(-t["b"].astype(np.float64)))).astype(np.float16))) <= 1
    assert np.max(ulp_diff_f16(g, want_g.astype(np.float16))) <= 1


def test_oracle_fused_pairs_equal_the_separate_steps(oracle):
    """kv_readout_delta applies exp(g) to the readout instead of rounding the decayed state to fp16, state_decay_update
    decays and updates in one rounding: both stay within fp16 rounding of the separate launches."""
    heads, d = 3, 64
    t = step_inputs(2, heads, d)
    beta, g = oracle.dn_compute_gates(t["b"], t["a"], t["a_log"], t["dt_bias"], heads)
    decayed = oracle.dn_state_decay(t["state"], g, d, heads)
    want_decay = np.exp(g.astype(F))[:, None, None] * t["state"].astype(F)
    assert np.max(ulp_diff_f16(decayed, want_decay.astype(np.float16))) <= 1
    kv = oracle.dn_kv_mem_readout(decayed, t["key"], d, heads)
    assert np.allclose(kv, np.einsum("hkv,hk->hv", decayed.astype(np.float64), t["key"].astype(np.float64)), atol=1e-5)
    delta = oracle.dn_compute_delta(t["value"], kv, beta, d, heads)
    fused = oracle.dn_kv_readout_delta(t["state"], t["key"], t["value"], g, beta, d, heads)
    assert np.max(np.abs(fused - delta)) < 1e-3
    fused_gates, g2 = oracle.dn_gates_kv_readout_delta(t["state"], t["key"], t["value"], t["b"], t["a"], t["a_log"], t["dt_bias"], d, heads)
    assert np.array_equal(g2.view(np.uint16), g.view(np.uint16))
    assert np.max(np.abs(fused_gates - fused)) < 2e-3  # beta and g in fp32 here, fp16 there
    two = oracle.dn_outer_product_update(decayed, t["key"], delta, d, heads)
    one = oracle.dn_outer_product_update(t["state"], t["key"], delta, d, heads, g_val=g)
    assert np.max(np.abs(one.astype(F) - two.astype(F))) < 5e-4  # one fp16 rounding against two, values up to 0.5
    out = oracle.dn_query_readout(two, t["query"], d, 0.125, heads)
    want = np.einsum("hkv,hk->hv", two.astype(np.float64), t["query"].astype(np.float64) * 0.125)
    assert np.max(np.abs(out.astype(np.float64) - want)) < 2e-4


def fused_inputs(seed, heads, d, k, t=0):
    rng = np.random.default_rng(seed)
    c = 3 * heads * d
    lead = (t,) if t else ()
    return dict(state=halves(rng, heads, d, d, scale=0.05), qkv=halves(rng, *lead, c), conv_state=halves(rng, c, k), conv_weight=halves(rng, c, k, scale=0.5),
                b=halves(rng, *lead, heads), a=halves(rng, *lead, heads), a_log=halves(rng, heads, scale=0.3), dt_bias=halves(rng, heads, scale=0.3),
                z=halves(rng, heads, d), norm_w=(1 + 0.1 * rng.standard_normal(d)).astype(np.float16))


def l2_rows(x, scale):
    return x / np.maximum(np.linalg.norm(x, axis=-1, keepdims=True), 1e-6) * scale


def test_oracle_fused_decode_follows_the_tiled_step(oracle):
    """deltanet_recurrence_fused against conv1d_update_silu -> L2 norms -> deltanet_recurrence_mlx_decode -> rms_norm_gated:
    the same step with other staging (plain fp32 SiLU and gates, no fp16 between the stages)."""
    heads, d, k = 3, 128, 4
    t = fused_inputs(3, heads, d, k)
    c, scale = 3 * heads * d, 1 / np.sqrt(d)
    st, cs, out = oracle.deltanet_recurrence_fused(t["state"], t["qkv"], t["b"], t["a"], t["a_log"], t["dt_bias"], t["conv_state"], t["conv_weight"],
                                                   t["z"], t["norm_w"], d, scale, c, k, heads, 1e-6, 256)
    cs2, act = oracle.conv1d_update_silu(t["conv_state"], t["qkv"], t["conv_weight"], c, k)
    assert np.array_equal(cs.view(np.uint16), cs2.reshape(c, k).view(np.uint16))
    x = act.astype(F).reshape(3, heads, d)
    qkv2 = np.concatenate([l2_rows(x[0], scale).reshape(-1), l2_rows(x[1], 1.0).reshape(-1), x[2].reshape(-1)]).astype(np.float16)
    st2, core = oracle.deltanet_recurrence_decode(t["state"], qkv2, t["b"], t["a"], t["a_log"], t["dt_bias"], d, heads, heads)
    want = oracle.rms_norm_gated(core, t["z"], t["norm_w"], d, 1e-6, heads)
    assert np.max(np.abs(st.astype(F) - st2.astype(F))) < 2e-3
    assert np.max(np.abs(out.astype(F) - want.astype(F))) < 1e-2 * np.max(np.abs(want.astype(F)))


def test_oracle_fused_prefill_follows_the_tiled_chunk(oracle):
    heads, d, k, n = 2, 128, 4, 7
    t = fused_inputs(4, heads, d, k, n)
    c, scale = 3 * heads * d, 1 / np.sqrt(d)
    st, cs, x, out = oracle.deltanet_recurrence_prefill_fused(t["state"], t["conv_state"], t["qkv"], t["conv_weight"], t["a_log"], t["dt_bias"], t["b"], t["a"],
                                                              d, heads, n, c, k, scale, 1e-6)
    cs2, act, _ = oracle.conv1d_update_silu_prefill(t["conv_state"], t["qkv"], t["conv_weight"], n, c, k)
    assert np.array_equal(cs.view(np.uint16), cs2.reshape(c, k).view(np.uint16))
    xm = act.astype(F).reshape(n, 3, heads, d)
    x2 = np.concatenate([l2_rows(xm[:, 0], scale).reshape(n, -1), l2_rows(xm[:, 1], 1.0).reshape(n, -1), xm[:, 2].reshape(n, -1)], axis=1).astype(np.float16)
    # the kernel leaves the conv output and the normalised Q (unscaled) and K in qkv
    assert np.max(ulp_diff_f16(x[:, 2 * heads * d:], act[:, 2 * heads * d:])) <= 2
    assert np.max(np.abs(x[:, heads * d:2 * heads * d].astype(F) - x2[:, heads * d:2 * heads * d].astype(F))) < 2e-3
    st2, out2, _ = oracle.deltanet_recurrence_prefill(t["state"], x2, t["b"], t["a"], t["a_log"], t["dt_bias"], d, heads, heads, n)
    assert np.max(np.abs(st.astype(F) - st2.astype(F))) < 4e-3
    assert np.max(np.abs(out.astype(F) - out2.astype(F))) < 2e-2 * np.max(np.abs(out2.astype(F)))


@pytest.fixture()
def ctx():
    c = capi.Context(0)
    yield c
    c.close()


def f32bits(v):
    return int(np.array([v], F).view(np.uint32)[0])


def rec(pipe, grid, tg, bufs, cons, style=0):
    r = capi.DispatchRecord()
    r.op_kind, r.pipeline, r.style, r.buffer_count, r.constant_count = 0, pipe, style, len(bufs), len(cons)
    r.grid[0], r.grid[1], r.grid[2] = grid, 1, 1
    r.threadgroup[0], r.threadgroup[1], r.threadgroup[2] = tg, 1, 1
    for j, (binding, slot) in enumerate(bufs):
        r.buf[j].slot, r.buf[j].binding_index, r.buf[j].offset_kind, r.buf[j].offset = slot, binding, 0, 0
    for j, (binding, kind, value) in enumerate(cons):
        r.con[j].kind, r.con[j].binding_index, r.con[j].value = kind, binding, value
    return r


def load_slots(ctx, tensors):
    for slot, t in tensors.items():
        t = np.ascontiguousarray(t)
        ctx.call("alloc_slot", slot, C.c_size_t(t.nbytes))
        ctx._check(ctx.lib.smelt_cuda_write_slot(ctx.h, slot, C.c_size_t(0), t.ctypes.data_as(C.c_void_p), C.c_size_t(t.nbytes)))
    cfg = capi.RuntimeConfig(0, 1, 2, 2, 0, 1, 64, 64, 16, 1)
    for slot in (0, 1):
        ctx.call("alloc_slot", slot, C.c_size_t(64))
    ctx._check(ctx.lib.smelt_cuda_configure(ctx.h, C.byref(cfg)))


def read_slot(ctx, slot, shape, dtype=np.float16):
    out = np.zeros(shape, dtype)
    ctx._check(ctx.lib.smelt_cuda_read_slot(ctx.h, slot, C.c_size_t(0), out.ctypes.data_as(C.c_void_p), C.c_size_t(out.nbytes)))
    return out


def run_table(ctx, records):
    tok = np.zeros(1, np.int32)
    ctx._check(ctx.lib.smelt_cuda_enqueue_decode(ctx.h, (capi.DispatchRecord * len(records))(*records), len(records), tok.ctypes.data_as(C.c_void_p), 0))
    ctx.synchronize()


@pytest.mark.gpu
@pytest.mark.parametrize("heads,d", [(16, 128), (5, 64), (2, 256)])
def test_step_records_separate_launches(ctx, oracle, heads, d):
    """compute_gates -> state_decay -> kv_mem_readout -> compute_delta -> outer_product_update -> query_readout on one
    copy of the state, kv_readout_delta / gates_kv_readout_delta -> state_decay_update on two others."""
    t = step_inputs(10 + heads, heads, d)
    z2, z4 = np.zeros(heads, np.float16), np.zeros((heads, d), F)
    tensors = {2: t["state"], 3: t["state"], 4: t["state"], 5: t["key"], 6: t["query"], 7: t["value"], 8: t["b"], 9: t["a"], 10: t["a_log"], 11: t["dt_bias"],
               12: z2, 13: z2, 14: z4, 15: z4, 16: np.zeros((heads, d), np.float16), 17: z4, 18: z4, 19: z2}
    load_slots(ctx, tensors)
    names = ["compute_gates", "state_decay", "kv_mem_readout", "compute_delta", "outer_product_update", "query_readout", "kv_readout_delta",
             "gates_kv_readout_delta", "state_decay_update"]
    for i, n in enumerate(names):
        ctx._check(ctx.lib.smelt_cuda_register_pipeline(ctx.h, 40 + i, n.encode()))
    scale = 1 / np.sqrt(d)
    run_table(ctx, [
        rec(40, heads, 1, [(0, 8), (1, 9), (2, 10), (3, 11), (4, 12), (5, 13)], [(6, 0, heads)], style=1),
        rec(41, heads, 256, [(0, 2), (1, 13)], [(2, 0, d)]),
        rec(42, heads, d, [(0, 2), (1, 5), (2, 14)], [(3, 0, d)]),
        rec(43, heads * d, 1, [(0, 7), (1, 14), (2, 12), (3, 15)], [(4, 0, d)], style=1),
        rec(44, heads, 256, [(0, 2), (1, 5), (2, 15)], [(3, 0, d)]),
        rec(45, heads, d, [(0, 2), (1, 6), (2, 16)], [(3, 0, d), (4, 1, f32bits(scale))]),
        rec(46, heads, d, [(0, 3), (1, 5), (2, 7), (3, 13), (4, 12), (5, 17)], [(6, 0, d)]),
        rec(47, heads, d, [(0, 4), (1, 5), (2, 7), (3, 8), (4, 9), (5, 10), (6, 11), (7, 18), (8, 19)], [(9, 0, d)]),
        rec(48, heads, 256, [(0, 3), (1, 13), (2, 5), (3, 17)], [(4, 0, d)]),
    ])
    beta, g = oracle.dn_compute_gates(t["b"], t["a"], t["a_log"], t["dt_bias"], heads)
    got_beta, got_g = read_slot(ctx, 12, heads), read_slot(ctx, 13, heads)
    assert np.max(ulp_diff_f16(got_beta, beta)) <= 1 and np.max(ulp_diff_f16(got_g, g)) <= 1
    # everything downstream from the GPU's own gates: a one-ulp difference in a gate is not the later kernels' error
    decayed = oracle.dn_state_decay(t["state"], got_g, d, heads)
    kv = oracle.dn_kv_mem_readout(decayed, t["key"], d, heads)
    delta = oracle.dn_compute_delta(t["value"], kv, got_beta, d, heads)
    updated = oracle.dn_outer_product_update(decayed, t["key"], delta, d, heads)
    out = oracle.dn_query_readout(updated, t["query"], d, scale, heads)
    got_kv, got_delta = read_slot(ctx, 14, (heads, d), F), read_slot(ctx, 15, (heads, d), F)
    # exp(g) comes from two maths libraries: one fp32 ulp of the decay can move a state element by one fp16 ulp (2.4e-4 at 0.25 .. 0.5)
    assert np.max(np.abs(got_kv - kv)) < 1e-4 and np.max(np.abs(got_delta - delta)) < 1e-4
    assert np.max(np.abs(read_slot(ctx, 2, (heads, d, d)).astype(F) - updated.astype(F))) < 5e-4
    assert np.max(np.abs(read_slot(ctx, 16, (heads, d)).astype(F) - out.astype(F))) < 1e-4
    fused = oracle.dn_kv_readout_delta(t["state"], t["key"], t["value"], got_g, got_beta, d, heads)
    got_fused = read_slot(ctx, 17, (heads, d), F)
    assert np.max(np.abs(got_fused - fused)) < 1e-5
    fused_gates, g2 = oracle.dn_gates_kv_readout_delta(t["state"], t["key"], t["value"], t["b"], t["a"], t["a_log"], t["dt_bias"], d, heads)
    assert np.max(np.abs(read_slot(ctx, 18, (heads, d), F) - fused_gates)) < 1e-4  # exp of an fp32 gate from two maths libraries
    assert np.max(ulp_diff_f16(read_slot(ctx, 19, heads), g2)) <= 1
    want3 = oracle.dn_outer_product_update(t["state"], t["key"], got_fused, d, heads, g_val=got_g)
    assert np.max(np.abs(read_slot(ctx, 3, (heads, d, d)).astype(F) - want3.astype(F))) < 5e-4
    assert np.array_equal(read_slot(ctx, 4, (heads, d, d)).view(np.uint16), t["state"].view(np.uint16))  # the readouts leave the state alone


@pytest.mark.gpu
@pytest.mark.parametrize("heads,d,k,tgs", [(16, 128, 4, 256), (3, 64, 3, 128), (2, 256, 4, 512)])
def test_fused_decode_record(ctx, oracle, heads, d, k, tgs):
    t = fused_inputs(20 + d, heads, d, k)
    c, scale = 3 * heads * d, 1 / np.sqrt(d)
    load_slots(ctx, {2: t["state"], 3: t["qkv"], 4: t["b"], 5: t["a"], 6: t["a_log"], 7: t["dt_bias"], 8: np.zeros((heads, d), np.float16), 9: t["conv_state"],
                     10: t["conv_weight"], 11: t["z"], 12: t["norm_w"]})
    ctx._check(ctx.lib.smelt_cuda_register_pipeline(ctx.h, 50, b"deltanet_recurrence_fused"))
    run_table(ctx, [rec(50, heads, tgs, [(i, 2 + i) for i in range(11)],
                        [(11, 0, d), (12, 1, f32bits(scale)), (13, 0, c), (14, 0, k), (15, 0, heads), (16, 1, f32bits(1e-6))])])
    st, cs, out = oracle.deltanet_recurrence_fused(t["state"], t["qkv"], t["b"], t["a"], t["a_log"], t["dt_bias"], t["conv_state"], t["conv_weight"], t["z"],
                                                   t["norm_w"], d, scale, c, k, heads, 1e-6, tgs)
    assert np.array_equal(read_slot(ctx, 9, (c, k)).view(np.uint16), cs.reshape(c, k).view(np.uint16))
    assert np.max(np.abs(read_slot(ctx, 2, (heads, d, d)).astype(F) - st.astype(F))) < 5e-4
    got = read_slot(ctx, 8, (heads, d)).astype(F)
    assert np.max(np.abs(got - out.astype(F))) < 2e-3 * np.max(np.abs(out.astype(F)))


@pytest.mark.gpu
@pytest.mark.parametrize("heads,d,k,n,tgs", [(16, 128, 4, 9, 128), (3, 64, 3, 5, 64), (2, 256, 4, 3, 256), (2, 96, 4, 4, 32)])
def test_fused_prefill_record(ctx, oracle, heads, d, k, n, tgs):
    t = fused_inputs(30 + d, heads, d, k, n)
    c, scale = 3 * heads * d, 1 / np.sqrt(d)
    load_slots(ctx, {2: t["state"], 3: t["conv_state"], 4: t["qkv"], 5: t["conv_weight"], 6: t["a_log"], 7: t["dt_bias"], 8: t["b"], 9: t["a"],
                     10: np.zeros((n, heads, d), np.float16)})
    ctx._check(ctx.lib.smelt_cuda_register_pipeline(ctx.h, 51, b"deltanet_recurrence_prefill"))
    run_table(ctx, [rec(51, heads, tgs, [(i, 2 + i) for i in range(9)],
                        [(9, 0, d), (10, 0, heads), (11, 0, n), (12, 0, c), (13, 0, k), (14, 1, f32bits(scale)), (15, 1, f32bits(1e-6))])])
    st, cs, x, out = oracle.deltanet_recurrence_prefill_fused(t["state"], t["conv_state"], t["qkv"], t["conv_weight"], t["a_log"], t["dt_bias"], t["b"], t["a"],
                                                              d, heads, n, c, k, scale, 1e-6, tgs)
    assert np.array_equal(read_slot(ctx, 3, (c, k)).view(np.uint16), cs.reshape(c, k).view(np.uint16))
    assert np.max(ulp_diff_f16(read_slot(ctx, 4, (n, c)), x)) <= 2
    assert np.max(np.abs(read_slot(ctx, 2, (heads, d, d)).astype(F) - st.astype(F))) < 2e-3
    got = read_slot(ctx, 10, (n, heads, d)).astype(F)
    assert np.max(np.abs(got - out.astype(F))) < 4e-3 * np.max(np.abs(out.astype(F)))


@pytest.mark.gpu
def test_step_records_refuse_bad_shapes(ctx):
    load_slots(ctx, {2: np.zeros(64, np.float16)})
    ctx._check(ctx.lib.smelt_cuda_register_pipeline(ctx.h, 52, b"state_decay"))
    tok = np.zeros(1, np.int32)
    r = rec(52, 4, 256, [(0, 2), (1, 2)], [(2, 0, 128)])  # four heads of 128 x 128 halves do not fit in 128 bytes
    st = ctx.lib.smelt_cuda_enqueue_decode(ctx.h, (capi.DispatchRecord * 1)(r), 1, tok.ctypes.data_as(C.c_void_p), 0)
    assert st == capi.OUT_OF_RANGE
    r = rec(52, 4, 256, [(0, 2)], [(2, 0, 4)])  # no gate binding
    st = ctx.lib.smelt_cuda_enqueue_decode(ctx.h, (capi.DispatchRecord * 1)(r), 1, tok.ctypes.data_as(C.c_void_p), 0)
    assert st == capi.BAD_ARGUMENT
