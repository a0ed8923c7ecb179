"""Pins the CPU oracle against the known-answer vectors the reference's own tests hold for
the decode hot path.  Every expected value below is a vector stated in the cited reference
test; inputs are regenerated from the closed-form fixtures those tests define."""
import numpy as np
import pytest

from smelt_b200 import synth


def f16(*v):
    return np.array(v, dtype=np.float16)


# Tests/SmeltCompilerTests/SmeltAffineU4Tests.swift:67-80 — a single group [0..15] maps to
# nibbles 0..15, low nibble first; scale 1, bias 0 dequantises exactly.
def test_affine_u4_exact_packing_layout(oracle):
    w = np.arange(16, dtype=np.float32).reshape(1, 16)
    packed, scales, biases = oracle.affine_quantize(w, 16)
    assert packed.shape == (1, 8)
    for i in range(8):
        assert packed[0, i] & 0x0F == 2 * i
        assert packed[0, i] >> 4 == 2 * i + 1
        assert packed[0, i] == ((2 * i + 1) << 4 | 2 * i)
    assert np.array_equal(oracle.affine_dequantize(packed, scales, biases, 16, 16), w)


# Tests/SmeltCompilerTests/SmeltAffineU4Tests.swift:120-128 — a constant group uses scale 1,
# bias = value (through fp16), nibble 0.
def test_affine_u4_constant_group(oracle):
    w = np.full((1, 64), 0.123, np.float32)
    packed, scales, biases = oracle.affine_quantize(w, 64)
    assert np.all(packed == 0) and float(scales[0, 0]) == 1.0
    deq = oracle.affine_dequantize(packed, scales, biases, 64, 64)
    assert np.allclose(deq, float(np.float16(0.123)), atol=1e-6)


# Sources/SmeltCompiler/SmeltAffineU4.swift:141-161 — dequant is float(nibble)*scale + bias with
# fp16-read scale/bias; the fp16-stored form rounds that once.
def test_affine_u4_dequant_formula_bitexact(oracle):
    packed, scales, biases = synth.affine_u4(0, "dq", 8, 256, 64)
    deq = oracle.affine_dequantize(packed, scales, biases, 256, 64)
    nib = np.stack([packed & 0x0F, packed >> 4], axis=-1).reshape(8, 256).astype(np.float32)
    s = np.repeat(scales.astype(np.float32), 64, axis=1)
    b = np.repeat(biases.astype(np.float32), 64, axis=1)
    assert np.array_equal(deq, nib * s + b)
    assert np.array_equal(oracle.affine_dequantize_f16(packed, scales, biases, 8, 256, 64).view(np.uint16),
                          (nib * s + b).astype(np.float16).view(np.uint16))


# Tests/SmeltRuntimeTests/SmeltSignedQuantCodecTests.swift:6-14 — geometry helpers.
def test_signed_codec_geometry(oracle):
    assert oracle.signed_packed_byte_count(9, oracle.BINARY1) == 2
    assert oracle.signed_packed_byte_count(5, oracle.TERNARY2) == 2
    assert oracle.signed_groups_per_row(8, 4) == 2
    with pytest.raises(oracle.OracleError):
        oracle.signed_groups_per_row(7, 4)


# …:16-33 — binary byte 0b0101_1010, scales 0.5 / 2.
def test_signed_codec_binary_known_answer(oracle):
    out = oracle.signed_dequantize_row(oracle.BINARY1, np.array([0b01011010], np.uint8), f16(0.5, 2), 8, 8, 4)
    assert out.tolist() == [-0.5, 0.5, -0.5, 0.5, 2, -2, 2, -2]


# …:55-72 — ternary bytes 0b01_10_01_00, 0b10_00_01_10, scales 0.25 / 4.
def test_signed_codec_ternary_known_answer(oracle):
    out = oracle.signed_dequantize_row(oracle.TERNARY2, np.array([0b01100100, 0b10000110], np.uint8), f16(0.25, 4), 8, 8, 4)
    assert out.tolist() == [-0.25, 0, 0.25, 0, 4, 0, -4, 4]


# …:95-107 — the reserved ternary code 3 is rejected, naming logical index 0.
def test_signed_codec_rejects_code_three(oracle):
    rc, bad = oracle.signed_validate_codes(np.array([0b00011011], np.uint8), 4, oracle.TERNARY2)
    assert rc == oracle.INVALID_CODE and bad == 0
    with pytest.raises(oracle.OracleError) as e:
        oracle.signed_matvec(oracle.TERNARY2, np.full((1, 32), 0xFF, np.uint8), f16(1).reshape(1, 1), np.ones(128, np.float16), 1, 128)
    assert e.value.code == oracle.INVALID_CODE


def _mlx_ternary_fixture(rows, cols, batches, scale_unit):
    r = np.arange(rows)[:, None]
    c = np.arange(cols)[None, :]
    code = ((r * 13 + c * 7) % 3).astype(np.uint8)
    codes = synth.pack_codes(code, 2)
    groups = cols // 128
    scales = (np.float32(scale_unit) * ((np.arange(rows * groups) % 5) + 1).astype(np.float32)).astype(np.float16).reshape(rows, groups)
    i = np.arange(batches * cols)
    x = (((i * 17 + 3) % 31 - 15).astype(np.float32) / 16).astype(np.float16).reshape(batches, cols)
    return codes, scales, x


# Tests/SmeltCompilerTests/SignedQuantKernelTests.swift:87-106 — MLX v0.31.1 affine_qmv_fast
# fp16 bit patterns for the 9x512 ternary fixture.  All operands are dyadic, so a correct
# fp32-accumulated ternary matvec reproduces the bits whatever its summation order.
def test_ternary_matvec_matches_mlx_golden_bits_9x512(oracle):
    codes, scales, x = _mlx_ternary_fixture(9, 512, 1, 0.03125)
    got = oracle.signed_matvec(oracle.TERNARY2, codes, scales, x, 9, 512)
    expected = [0xb190, 0x3468, 0xb0b0, 0x2e20, 0xa580, 0x3370, 0xb518, 0x3498, 0xb170]
    assert got.view(np.uint16).reshape(-1).tolist() == expected


# …:143-164 — production width 9x5120, three batch rows.
def test_ternary_matvec_matches_mlx_golden_bits_9x5120x3(oracle):
    codes, scales, x = _mlx_ternary_fixture(9, 5120, 3, 0.00390625)
    got = oracle.signed_matvec(oracle.TERNARY2, codes, scales, x, 9, 5120)
    expected = [
        0xa160, 0x9dc0, 0x2420, 0xa160, 0x9dc0, 0x2420, 0xa160, 0x9dc0, 0x2420,
        0x2520, 0xa650, 0x1cc0, 0x2520, 0xa650, 0x1cc0, 0x2520, 0xa650, 0x1cc0,
        0x2280, 0x1700, 0xa360, 0x2280, 0x1700, 0xa360, 0x2280, 0x1700, 0xa360,
    ]
    assert got.view(np.uint16).reshape(-1).tolist() == expected


# Tests/SmeltCompilerTests/Helpers/MetalKernelTestSupport.swift:396-428 — the affine matvec
# oracle equals dequantise-then-dot up to fp32 reassociation, and the 4-row interleaved path
# is bit-identical to the one-row path (row tails 257 and 5 as in RegionExactnessTests).
def test_affine_matvec_oracle_consistency(oracle):
    rows, cols, g = 257, 512, 64
    w, s, b = synth.ref_affine_fixture(rows, cols, g, 3)
    x = synth.ref_float16_vector(cols, 3 * synth.REGION_SEED_PRIMARY, 0.5)
    y = oracle.affine_matvec(w, s, b, x, rows, cols, g, f32=True)[0]
    deq = oracle.affine_dequantize(w, s, b, cols, g).astype(np.float64)
    ref = deq @ x.astype(np.float64)
    assert np.max(np.abs(y - ref)) < 2e-4 * np.max(np.abs(ref))
    y5 = oracle.affine_matvec(w[:5], s[:5], b[:5], x, 5, cols, g, f32=True)[0]
    assert np.array_equal(y5[:4], y[:4]) and y5[4] == y[4]  # row 4: scalar path vs interleaved path


# Tests/SmeltCompilerTests/RegionExactnessTests.swift:1414-1475 — attention oracle against a
# float64 softmax on the reference's own fixture (seqLen 32 and 192, sliding window 8).
@pytest.mark.parametrize("seq_len,window", [(32, 0), (32, 8), (192, 0)])
def test_attention_oracle_matches_float64(oracle, seq_len, window):
    n_q, n_kv, d = 4, 2, 128
    cap = max(seq_len, 64)
    q, k, v = synth.ref_attention_inputs(n_q, n_kv, d, cap, 1)
    out = oracle.attention_decode(q, k, v, n_q, n_kv, d, cap, seq_len, sliding_window=window).astype(np.float64)
    start = seq_len - window if 0 < window < seq_len else 0
    for h in range(n_q):
        kk = k[h // 2, start:seq_len].astype(np.float64)
        vv = v[h // 2, start:seq_len].astype(np.float64)
        sc = kk @ q[h].astype(np.float64) / np.sqrt(d)
        p = np.exp(sc - sc.max())
        ref = (p / p.sum()) @ vv
        assert np.max(np.abs(out[h] - ref)) < 1e-3  # 1 fp16 ulp at |out| ~ 1
        assert np.max(np.abs(out[h])) > 1e-3


# Resources/Shaders/lut_matvec.metal:4045-4074 / Sources/SmeltRuntime/SmeltSelection.swift:165 —
# ties keep the lowest index; -0 and +0 compare equal.
def test_argmax_tie_rules(oracle):
    assert oracle.argmax_f16(f16(1, 3, 3, 2)) == 1
    assert oracle.argmax_f16(np.array([0x8000, 0x0000, 0x8000], np.uint16).view(np.float16)) == 0
    assert oracle.argmax_f16(np.array([0x0000, 0x8000], np.uint16).view(np.float16)) == 0
    assert oracle.argmax_f16(f16(-5, -2, -2)) == 1


# Tests/SmeltCompilerTests/RegionExactnessTests.swift:909-925 — KV append touches only [h, pos, :].
def test_kv_cache_update(oracle):
    heads, d, cap, pos = 2, 128, 16, 5
    cache = synth.ref_float16_vector(heads * cap * d, 11.0, 0.5).reshape(heads, cap, d)
    new = synth.ref_float16_vector(heads * d, 13.0, 0.5, 0.1).reshape(heads, d)
    out = oracle.kv_cache_update(cache, new, cap, d, pos, heads)
    exp = cache.copy()
    exp[:, pos, :] = new
    assert np.array_equal(out.view(np.uint16), exp.view(np.uint16))


# Resources/Shaders/attention.metal:48-115 — table-mode RoPE in the three layouts equals the
# closed form x0*c0 - x1*s0, x0*s1 + x1*c1 with the layout's pair indices.
@pytest.mark.parametrize("layout", [0, 1, 2])
def test_rope_table_mode_layouts(oracle, layout):
    heads, d, rope = 3, 128, 64
    qk = synth.ref_float16_vector(heads * d, float(synth.REGION_SEED_PRIMARY), 0.5, 0.1)
    cos = synth.ref_float16_vector(rope, float(synth.REGION_SEED_SECONDARY), 0.9, phase=0.0237)
    sin = synth.ref_float16_vector(rope, float(synth.REGION_SEED_TERTIARY), 0.9, phase=0.0193)
    out = oracle.apply_rope(qk, d, rope, heads, layout, 0, math_mode=0, cos=cos, sin=sin).reshape(heads, d)
    x = qk.reshape(heads, d).astype(np.float32)
    exp = qk.reshape(heads, d).copy()
    half = rope // 2
    for p in range(half):
        d0, d1, c0, c1 = {0: (2 * p, 2 * p + 1, 2 * p, 2 * p + 1), 1: (p, p + half, p, p + half), 2: (p, p + d // 2, p, p + half)}[layout]
        cf, sf = cos.astype(np.float32), sin.astype(np.float32)
        exp[:, d0] = (x[:, d0] * cf[c0] - x[:, d1] * sf[c0]).astype(np.float16)
        exp[:, d1] = (x[:, d0] * sf[c1] + x[:, d1] * cf[c1]).astype(np.float16)
    assert np.array_equal(out.view(np.uint16), exp.view(np.uint16))


# Tests/SmeltCompilerTests/Helpers/MetalKernelTestSupport.swift:227-243 vs norms.metal:58-63 —
# the one-rounding CPU form and the kernel's two-stage form agree within two fp16 ulp and are
# identical when the stored weight delta is zero.
def test_rms_norm_forms(oracle):
    x = synth.ref_float16_vector(2048, 6151.0, 0.5)
    w = synth.ref_float16_vector(2048, 4817.0, 0.5, 0.5, 0.0091)
    a = oracle.rms_norm_1pw(x, w, 1e-6, two_stage=False).astype(np.float32)
    b = oracle.rms_norm_1pw(x, w, 1e-6, two_stage=True).astype(np.float32)
    assert np.max(np.abs(a - b) / np.maximum(np.abs(a), 1e-3)) < 2e-3
    z = np.zeros(2048, np.float16)
    assert np.array_equal(oracle.rms_norm_1pw(x, z, 1e-6, False).view(np.uint16), oracle.rms_norm_1pw(x, z, 1e-6, True).view(np.uint16))


def test_two_pass_attention_restatement_agrees_with_the_decode_oracle(oracle):
    """The reference holds two formulations of single-token attention at head_dim 256: the generic
    oracle (RegionExactnessTests.swift:1414-1475) and the split-K record pair with 128 interleaved
    key blocks and fp16 partials (attention.metal:1071-1206).  Their restatements must agree within
    the bound the fp16 partials allow, for a context shorter than, equal to and longer than 128 blocks."""
    from helpers import INF_TOL, TWO_PASS_REL_TOL, inf_err, rel_err
    from smelt_b200 import synth

    n_q, n_kv, d, cap = 4, 2, 256, 1200
    q = synth.activations(5, "q2p", n_q, d)
    k = synth.kv_cache(5, "k2p", 1, n_kv, cap, d)[0]
    v = synth.kv_cache(5, "v2p", 1, n_kv, cap, d)[0]
    for seq_len in (1, 100, 128, 1100):
        ref = oracle.attention_decode(q, k, v, n_q, n_kv, d, cap, seq_len, scale=0.0625)
        two = oracle.attention_decode_mlx_2pass(q, k, v, n_q, n_kv, cap, seq_len)
        assert rel_err(two, ref) < TWO_PASS_REL_TOL and inf_err(two, ref) < INF_TOL, seq_len
