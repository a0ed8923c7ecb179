"""Hand-written dispatch records in the reference compiler's own shapes, replayed through the
interpreter and through the captured graph: the D256 split-K attention pair
(Sources/SmeltCompiler/AttentionPlugin.swift:865-918) and a table-mode RoPE record whose cos /
sin rows are bound at position-scaled offsets (offsetKind 1, Resources/Shaders/attention.metal:48-115)."""
import ctypes as C

import numpy as np
import pytest

from smelt_b200 import capi, synth
from helpers import INF_TOL, TWO_PASS_REL_TOL, inf_err, rel_err

pytestmark = pytest.mark.gpu

TOKEN_SLOT, POSITION_SLOT, ARGMAX_SLOT = 60, 61, 62


@pytest.fixture()
def ctx():
    c = capi.Context(0)
    yield c
    assert c.device_error() == 0
    c.close()


def configure(ctx, capacity):
    for slot in (TOKEN_SLOT, POSITION_SLOT, ARGMAX_SLOT):
        ctx.call("alloc_slot", slot, C.c_size_t(64))
    cfg = capi.RuntimeConfig(token_id_slot=TOKEN_SLOT, position_slot=POSITION_SLOT, weights_slot=30, argmax_slot=ARGMAX_SLOT, cur_slot=0,
                             alt_slot=1, cache_seq_capacity=capacity, context_limit=capacity, vocab_size=16, batch=1)
    ctx._check(ctx.lib.smelt_cuda_configure(ctx.h, C.byref(cfg)))


def put(ctx, slot, arr):
    arr = np.ascontiguousarray(arr)
    ctx.call("alloc_slot", slot, C.c_size_t(arr.nbytes))
    ctx.call("write_slot", slot, C.c_size_t(0), arr, C.c_size_t(arr.nbytes))


def get(ctx, slot, dtype, shape):
    out = np.empty(shape, dtype)
    ctx.call("read_slot", slot, C.c_size_t(0), out, C.c_size_t(out.nbytes))
    return out


def record(pipeline, buffers, constants, grid=(1, 1, 1)):
    r = capi.DispatchRecord()
    r.pipeline, r.buffer_count, r.constant_count = pipeline, len(buffers), len(constants)
    for i in range(3):
        r.grid[i] = grid[i]
    for i, (slot, binding, kind, offset) in enumerate(buffers):
        r.buf[i].slot, r.buf[i].binding_index, r.buf[i].offset_kind, r.buf[i].offset = slot, binding, kind, offset
    for i, (kind, binding, value) in enumerate(constants):
        r.con[i].kind, r.con[i].binding_index, r.con[i].value = kind, binding, value
    return r


TOK = np.array([0], np.int32).ctypes.data_as(C.c_void_p)


@pytest.mark.parametrize("seq_len", [1024, 1500, 4096])
def test_d256_two_pass_record_pair(ctx, oracle, seq_len):
    """The pair a reference-compiled head_dim-256 package emits from 1,024 keys on: record 1 fills the
    reference's partial / statistics buffers (fp16 [qHeads, 128, 256], fp32 [2][qHeads][128]),
    record 2 reduces them into the output slot.  Guarded by min position + 1 = 1024 as emitted."""
    n_q, n_kv, d, cap = 8, 2, 256, 4100
    Q, K, V, PART, STATS, OUT = 20, 40, 41, 50, 51, 23
    q = synth.activations(31, "q", n_q, d)
    k = synth.kv_cache(31, "k", 1, n_kv, cap, d)[0]
    v = synth.kv_cache(31, "v", 1, n_kv, cap, d)[0]
    configure(ctx, cap)
    put(ctx, Q, q); put(ctx, K, k); put(ctx, V, v)
    ctx.call("alloc_slot", PART, C.c_size_t(n_q * 128 * d * 2))
    ctx.call("alloc_slot", STATS, C.c_size_t(2 * n_q * 128 * 4))
    ctx.call("alloc_slot", OUT, C.c_size_t(n_q * d * 2))
    ctx.call("register_pipeline", 0, "attention_decode_mlx_vector_2pass_1_d256_b128")
    ctx.call("register_pipeline", 1, "attention_decode_mlx_vector_2pass_2_d256_b128")
    guard = (capi.CONST_SKIP_UNLESS_POS1_GE, 255, 1024)
    table = (capi.DispatchRecord * 2)(
        record(0, [(Q, 0, 0, 0), (K, 1, 0, 0), (V, 2, 0, 0), (PART, 3, 0, 0), (STATS, 4, 0, 0)],
               [(capi.CONST_POSITION_PLUS1, 5, 0), (capi.CONST_CACHE_SEQ_CAPACITY, 6, 0), (capi.CONST_LITERAL_U32, 7, n_q),
                (capi.CONST_LITERAL_U32, 8, n_kv), guard], grid=(n_kv, 1, 128)),
        record(1, [(PART, 0, 0, 0), (STATS, 1, 0, 0), (OUT, 2, 0, 0)], [(capi.CONST_LITERAL_U32, 3, n_q), guard], grid=(n_q, 1, 1)))
    ref = oracle.attention_decode(q, k, v, n_q, n_kv, d, cap, seq_len, scale=0.0625)
    ref_pair = oracle.attention_decode_mlx_2pass(q, k, v, n_q, n_kv, cap, seq_len)
    assert rel_err(ref_pair, ref) < TWO_PASS_REL_TOL  # the reference's own two formulations: fp16 partials cost this much

    def check():
        got = get(ctx, OUT, np.float16, (n_q, d))
        assert rel_err(got, ref) < TWO_PASS_REL_TOL and inf_err(got, ref) < INF_TOL
        assert rel_err(got, ref_pair) < 2 * TWO_PASS_REL_TOL  # two independent sets of fp16-rounded partials
        stats = get(ctx, STATS, np.float32, (2, n_q, 128))
        assert np.all(stats[0] >= 0) and np.all((stats[0] == 0) == (stats[1] <= -3e38))  # empty blocks are marked as the reference marks them
        assert np.all(np.sum(stats[0] > 0, axis=1) >= 1)

    ctx._check(ctx.lib.smelt_cuda_decode_step(ctx.h, table, 2, TOK, seq_len - 1, None))
    check()
    # below the guard nothing runs
    ctx.call("zero_slot", OUT)
    ctx._check(ctx.lib.smelt_cuda_decode_step(ctx.h, table, 2, TOK, 100, None))
    assert not get(ctx, OUT, np.uint16, (n_q, d)).any()
    # the captured graph resolves position + 1 and the guard on the device
    ctx._check(ctx.lib.smelt_cuda_graph_build(ctx.h, table, 2))
    ctx._check(ctx.lib.smelt_cuda_graph_seed(ctx.h, TOK, 100))
    ctx._check(ctx.lib.smelt_cuda_graph_decode(ctx.h, 1, None))
    ctx.synchronize()
    assert not get(ctx, OUT, np.uint16, (n_q, d)).any()
    ctx._check(ctx.lib.smelt_cuda_graph_seed(ctx.h, TOK, seq_len - 1))
    ctx._check(ctx.lib.smelt_cuda_graph_decode(ctx.h, 1, None))
    ctx.synchronize()
    check()


@pytest.mark.parametrize("layout", [0, 1])
def test_table_mode_rope_record_from_the_captured_graph(ctx, oracle, layout):
    """apply_rope and rope_kv_cache_update with cos / sin rows bound as position * rowBytes
    (offsetKind 1): the eager interpreter resolves the offset on the host, the captured graph on the
    device; both give the oracle's bits for the row of the seeded position."""
    heads, d, rope, positions, cap = 4, 128, 64, 40, 48
    DATA, COS, SIN, CACHE, NEW = 20, 32, 33, 40, 21
    qk = synth.ref_float16_vector(heads * d, float(synth.REGION_SEED_PRIMARY), 0.5, 0.1)
    cos = synth.ref_float16_vector(positions * rope, float(synth.REGION_SEED_SECONDARY), 0.9, phase=0.0237).reshape(positions, rope)
    sin = synth.ref_float16_vector(positions * rope, float(synth.REGION_SEED_TERTIARY), 0.9, phase=0.0193).reshape(positions, rope)
    configure(ctx, cap)
    put(ctx, COS, cos); put(ctx, SIN, sin); put(ctx, NEW, qk)
    ctx.call("alloc_slot", CACHE, C.c_size_t(heads * cap * d * 2))
    ctx.call("register_pipeline", 0, "apply_rope")
    ctx.call("register_pipeline", 1, "rope_kv_cache_update")
    row = rope * 2
    table = (capi.DispatchRecord * 2)(
        record(0, [(DATA, 0, 0, 0), (COS, 1, 1, row), (SIN, 2, 1, row)],
               [(capi.CONST_LITERAL_U32, 3, d), (capi.CONST_LITERAL_U32, 4, rope), (capi.CONST_LITERAL_U32, 5, heads), (capi.CONST_LITERAL_U32, 6, layout),
                (capi.CONST_POSITION, 7, 0), (capi.CONST_LITERAL_F32, 8, 0), (capi.CONST_LITERAL_U32, 9, 0)], grid=(heads, 1, 1)),
        record(1, [(CACHE, 0, 0, 0), (NEW, 1, 0, 0), (COS, 2, 1, row), (SIN, 3, 1, row)],
               [(capi.CONST_CACHE_SEQ_CAPACITY, 4, 0), (capi.CONST_LITERAL_U32, 5, d), (capi.CONST_POSITION, 6, 0), (capi.CONST_LITERAL_U32, 7, heads),
                (capi.CONST_LITERAL_U32, 8, rope), (capi.CONST_LITERAL_U32, 9, layout), (capi.CONST_LITERAL_F32, 10, 0), (capi.CONST_LITERAL_U32, 11, 0)],
               grid=(heads, 1, 1)))

    def check(position):
        want = oracle.apply_rope(qk, d, rope, heads, layout, position, math_mode=0, cos=cos[position], sin=sin[position])
        assert np.array_equal(get(ctx, DATA, np.uint16, (heads * d,)), want.view(np.uint16))
        cache = get(ctx, CACHE, np.uint16, (heads, cap, d))
        assert np.array_equal(cache[:, position, :].reshape(-1), want.view(np.uint16))

    put(ctx, DATA, qk)
    ctx._check(ctx.lib.smelt_cuda_decode_step(ctx.h, table, 2, TOK, 7, None))
    check(7)
    ctx._check(ctx.lib.smelt_cuda_graph_build(ctx.h, table, 2))
    for position in (5, 31, 0):
        ctx.call("write_slot", DATA, C.c_size_t(0), qk, C.c_size_t(qk.nbytes))
        ctx._check(ctx.lib.smelt_cuda_graph_seed(ctx.h, TOK, position))
        ctx._check(ctx.lib.smelt_cuda_graph_decode(ctx.h, 1, None))
        ctx.synchronize()
        check(position)


def test_graph_guards(ctx):
    """Graphs are dropped when a slot they captured is reallocated or resized, and a replay that
    would run past the cache capacity is refused before any launch."""
    cap = 16
    configure(ctx, cap)
    a = np.ones(32, np.float16)
    for slot in (0, 1, 2):
        put(ctx, slot, a)
    ctx.call("register_pipeline", 0, "elementwise_add")
    table = (capi.DispatchRecord * 1)(record(0, [(0, 0, 0, 0), (1, 1, 0, 0), (2, 2, 0, 0)], [(capi.CONST_LITERAL_U32, 3, 32)]))
    assert ctx.lib.smelt_cuda_graph_decode(ctx.h, 1, None) == capi.BAD_ARGUMENT  # nothing built
    ctx._check(ctx.lib.smelt_cuda_graph_build(ctx.h, table, 1))
    assert ctx.lib.smelt_cuda_graph_decode(ctx.h, 1, None) == capi.BAD_ARGUMENT and "seed" in ctx.last_error()
    ctx._check(ctx.lib.smelt_cuda_graph_seed(ctx.h, TOK, 10))
    assert ctx.lib.smelt_cuda_graph_decode(ctx.h, 7, None) == capi.OUT_OF_RANGE  # positions 10..16 pass capacity 16
    ctx._check(ctx.lib.smelt_cuda_graph_decode(ctx.h, 6, None))
    assert ctx.lib.smelt_cuda_graph_decode(ctx.h, 1, None) == capi.OUT_OF_RANGE  # the mirror advanced to 16
    ctx.synchronize()
    assert np.all(get(ctx, 2, np.float16, (32,)) == 2)
    ctx.call("resize_slot", 2, C.c_size_t(128), C.c_size_t(64))  # the graph's pointer to slot 2 is stale now
    out = np.zeros(1, np.int32)
    st = ctx.lib.smelt_cuda_graph_step(ctx.h, TOK, 3, out.ctypes.data_as(C.c_void_p))
    assert st == capi.BAD_ARGUMENT and "no graph" in ctx.last_error()
    ctx._check(ctx.lib.smelt_cuda_graph_build(ctx.h, table, 1))
    ctx._check(ctx.lib.smelt_cuda_graph_step(ctx.h, TOK, 3, out.ctypes.data_as(C.c_void_p)))
    ctx.call("alloc_slot", 1, C.c_size_t(64))  # allocating an existing slot again frees the old buffer
    assert ctx.lib.smelt_cuda_graph_step(ctx.h, TOK, 4, out.ctypes.data_as(C.c_void_p)) == capi.BAD_ARGUMENT
