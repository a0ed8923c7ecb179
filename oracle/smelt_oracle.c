/*
 * smelt_oracle.c — CPU restatement of the reference's scalar oracles for the decode hot path.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the product library links, imports or executes this
 * file; only the test-suite, the smoke check and the CPU-baseline leg of the benchmark do.
 * The reference (Swift + Metal) cannot be compiled on Linux, so every function restates the
 * scalar Swift (or, where no Swift oracle exists, the Metal kernel's arithmetic) it cites, in
 * the same evaluation order, in fp32 with no fused multiply-add (build with
 * -ffp-contract=off).  The restatement is pinned against the reference's own known-answer
 * vectors in tests/test_oracle_golden.py.
 *
 * Conventions: fp16 values cross the ABI as uint16_t bit patterns; "f32" arrays are float.
 * All functions return 0 on success or a negative SO_ERR_* code.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define SO_OK 0
#define SO_ERR_GEOMETRY (-1)
#define SO_ERR_INVALID_CODE (-2)
#define SO_ERR_ALLOC (-3)

#define SO_API __attribute__((visibility("default")))

/* ───────────────────────── fp16 helpers ───────────────────────── */

static inline float h2f(uint16_t h) {
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float)v;
}
static inline uint16_t f2h(float f) {
    _Float16 v = (_Float16)f; /* round-to-nearest-even, as Swift's Float16(Float) */
    uint16_t h;
    memcpy(&h, &v, 2);
    return h;
}
static inline float round_h(float f) { return h2f(f2h(f)); }

SO_API int so_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
SO_API void so_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
SO_API void so_f16_to_f32(const uint16_t *in, float *out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = h2f(in[i]);
}
SO_API void so_f32_to_f16(const float *in, uint16_t *out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = f2h(in[i]);
}

/* ───────────────────────── affine u4 codec ─────────────────────────
 * Sources/SmeltCompiler/SmeltAffineU4.swift:94-161.  Two nibbles per byte, LOW nibble =
 * even column; scale = (max-min)/15 (1 when the range is below 1e-12), bias = min; the
 * dequantised value is float(nibble) * float(fp16 scale) + float(fp16 bias), a separate
 * multiply and add.
 */
SO_API int so_affine_u4_quantize_row(const float *values, int cols, int group, uint8_t *packed,
                                     uint16_t *scales, uint16_t *biases) {
    if (cols <= 0 || group <= 0) return SO_ERR_GEOMETRY;
    int groups = (cols + group - 1) / group;
    for (int g = 0; g < groups; ++g) {
        int c0 = g * group, c1 = c0 + group < cols ? c0 + group : cols;
        float lo = INFINITY, hi = -INFINITY;
        for (int c = c0; c < c1; ++c) {
            float v = values[c];
            if (v < lo) lo = v;
            if (v > hi) hi = v;
        }
        float range = hi - lo;
        float scale = range < 1e-12f ? 1.0f : range / 15.0f;
        scales[g] = f2h(scale);
        biases[g] = f2h(lo);
        float inv = 1.0f / scale;
        for (int c = c0; c < c1; ++c) {
            float n = (values[c] - lo) * inv;
            n = n < 0.0f ? 0.0f : (n > 15.0f ? 15.0f : n);
            uint8_t nib = (uint8_t)roundf(n); /* Swift .rounded(): half away from zero */
            if ((c & 1) == 0) packed[c >> 1] = nib;
            else packed[c >> 1] |= (uint8_t)(nib << 4);
        }
    }
    return SO_OK;
}

SO_API int so_affine_u4_dequantize_row(const uint8_t *packed, const uint16_t *scales,
                                       const uint16_t *biases, int cols, int group, float *out) {
    if (cols <= 0 || group <= 0) return SO_ERR_GEOMETRY;
    int groups = (cols + group - 1) / group;
    for (int g = 0; g < groups; ++g) {
        int c0 = g * group, c1 = c0 + group < cols ? c0 + group : cols;
        float scale = h2f(scales[g]), bias = h2f(biases[g]);
        for (int c = c0; c < c1; ++c) {
            uint8_t byte = packed[c >> 1];
            uint8_t nib = (c & 1) == 0 ? (byte & 0x0F) : (byte >> 4);
            out[c] = (float)nib * scale + bias;
        }
    }
    return SO_OK;
}

/* The on-device form of the same dequant, rounded to fp16 when stored
 * (Resources/Shaders/lut_matvec.metal:994-1025, affine_embedding_gather). */
SO_API int so_affine_u4_dequantize_rows_f16(const uint8_t *packed, const uint16_t *scales,
                                            const uint16_t *biases, int rows, int cols, int group,
                                            uint16_t *out) {
    if (cols <= 0 || group <= 0 || cols % 2) return SO_ERR_GEOMETRY;
    int groups = cols / group;
    if (groups * group != cols) return SO_ERR_GEOMETRY;
    for (int r = 0; r < rows; ++r) {
        const uint8_t *p = packed + (size_t)r * (cols / 2);
        for (int c = 0; c < cols; ++c) {
            uint8_t byte = p[c >> 1];
            uint8_t nib = (c & 1) == 0 ? (byte & 0x0F) : (byte >> 4);
            float s = h2f(scales[(size_t)r * groups + c / group]);
            float b = h2f(biases[(size_t)r * groups + c / group]);
            out[(size_t)r * cols + c] = f2h((float)nib * s + b);
        }
    }
    return SO_OK;
}

/* ───────────────────────── affine matvec ─────────────────────────
 * Tests/SmeltCompilerTests/Helpers/MetalKernelTestSupport.swift:396-428
 * (referenceAffineMatvecRow): per group, dot += float(nibble)*x and xsum += x in column
 * order; acc += scale*dot + bias*xsum; optional fp16 rounding of the row result.
 */
static inline float affine_row_acc(const uint8_t *w, const uint16_t *s, const uint16_t *b,
                                   const float *x, int cols, int group) {
    int groups = cols / group;
    float acc = 0.0f;
    for (int g = 0; g < groups; ++g) {
        float scale = h2f(s[g]), bias = h2f(b[g]);
        int base = g * group;
        float dot = 0.0f, xsum = 0.0f;
        for (int i = 0; i < group; ++i) {
            int col = base + i;
            uint8_t byte = w[col >> 1];
            uint8_t nib = (col & 1) == 0 ? (byte & 0x0F) : (byte >> 4);
            float xv = x[col];
            dot += (float)nib * xv;
            xsum += xv;
        }
        acc += scale * dot + bias * xsum;
    }
    return acc;
}

/* Four rows at once: the same per-row arithmetic in the same order as affine_row_acc, with
 * the four independent dependency chains interleaved so the CPU's add latency is hidden. */
static inline void affine_row_acc4(const uint8_t *w, size_t wstride, const uint16_t *s, const uint16_t *b,
                                   size_t sstride, const float *x, int cols, int group, float out[4]) {
    int groups = cols / group;
    float acc[4] = {0, 0, 0, 0};
    for (int g = 0; g < groups; ++g) {
        int base = g * group;
        float dot[4] = {0, 0, 0, 0}, xsum[4] = {0, 0, 0, 0};
        for (int i = 0; i < group; i += 2) {
            int col = base + i;
            float x0 = x[col], x1 = x[col + 1];
            for (int r = 0; r < 4; ++r) {
                uint8_t byte = w[r * wstride + (col >> 1)];
                dot[r] += (float)(byte & 0x0F) * x0;
                xsum[r] += x0;
                dot[r] += (float)(byte >> 4) * x1;
                xsum[r] += x1;
            }
        }
        for (int r = 0; r < 4; ++r)
            acc[r] += h2f(s[r * sstride + g]) * dot[r] + h2f(b[r * sstride + g]) * xsum[r];
    }
    for (int r = 0; r < 4; ++r) out[r] = acc[r];
}

static int affine_geometry_ok(int rows, int cols, int group, int batch) {
    return rows > 0 && cols > 0 && group > 0 && batch > 0 && cols % group == 0 && cols % 2 == 0;
}

/* y_f32[b*rows + r] = acc (not rounded).  x is fp16 [batch, cols]. */
static int affine_matvec_acc(const uint8_t *w, const uint16_t *s, const uint16_t *bz,
                             const uint16_t *x_f16, int rows, int cols, int group, int batch,
                             float *y) {
    if (!affine_geometry_ok(rows, cols, group, batch)) return SO_ERR_GEOMETRY;
    float *x = (float *)malloc(sizeof(float) * (size_t)batch * cols);
    if (!x) return SO_ERR_ALLOC;
    so_f16_to_f32(x_f16, x, (int64_t)batch * cols);
    int groups = cols / group;
    int blocks = (rows + 3) / 4;
#pragma omp parallel for schedule(static)
    for (int blk = 0; blk < blocks; ++blk) {
        int r0 = blk * 4;
        const uint8_t *wr = w + (size_t)r0 * (cols / 2);
        const uint16_t *sr = s + (size_t)r0 * groups, *br = bz + (size_t)r0 * groups;
        if (r0 + 4 <= rows && group % 2 == 0) {
            for (int b = 0; b < batch; ++b) {
                float out[4];
                affine_row_acc4(wr, (size_t)cols / 2, sr, br, (size_t)groups, x + (size_t)b * cols, cols, group, out);
                for (int r = 0; r < 4; ++r) y[(size_t)b * rows + r0 + r] = out[r];
            }
        } else {
            for (int r = r0; r < rows && r < r0 + 4; ++r)
                for (int b = 0; b < batch; ++b)
                    y[(size_t)b * rows + r] = affine_row_acc(w + (size_t)r * (cols / 2), s + (size_t)r * groups,
                                                             bz + (size_t)r * groups, x + (size_t)b * cols, cols, group);
        }
    }
    free(x);
    return SO_OK;
}

/* affine_matvec: y = half(acc).  Kernel contract: lut_matvec.metal:1157-1287. */
SO_API int so_affine_matvec(const uint8_t *w, const uint16_t *s, const uint16_t *b,
                            const uint16_t *x, int rows, int cols, int group, int batch,
                            uint16_t *y) {
    float *acc = (float *)malloc(sizeof(float) * (size_t)batch * rows);
    if (!acc) return SO_ERR_ALLOC;
    int rc = affine_matvec_acc(w, s, b, x, rows, cols, group, batch, acc);
    if (rc == SO_OK) so_f32_to_f16(acc, y, (int64_t)batch * rows);
    free(acc);
    return rc;
}

/* Unrounded fp32 accumulators, for error analysis in the tests. */
SO_API int so_affine_matvec_f32(const uint8_t *w, const uint16_t *s, const uint16_t *b,
                                const uint16_t *x, int rows, int cols, int group, int batch,
                                float *y) {
    return affine_matvec_acc(w, s, b, x, rows, cols, group, batch, y);
}

/* fused_affine_matvec_add (lut_matvec.metal:1718-1817): the matvec result is rounded to
 * fp16 first, then added to the fp16 residual with an fp16 add (:1802-1803). */
SO_API int so_affine_matvec_add(const uint8_t *w, const uint16_t *s, const uint16_t *b,
                                const uint16_t *x, const uint16_t *residual, int rows, int cols,
                                int group, int batch, uint16_t *y) {
    float *acc = (float *)malloc(sizeof(float) * (size_t)batch * rows);
    if (!acc) return SO_ERR_ALLOC;
    int rc = affine_matvec_acc(w, s, b, x, rows, cols, group, batch, acc);
    if (rc == SO_OK)
        for (int64_t i = 0; i < (int64_t)batch * rows; ++i)
            y[i] = f2h(round_h(acc[i]) + h2f(residual[i]));
    free(acc);
    return rc;
}

/* fused_affine_gate_up_swiglu.  round_gate_up = 0: gate and up stay fp32 into SiLU, one
 * rounding at the end (kernel lut_matvec.metal:2228; oracle
 * Tests/SmeltCompilerTests/RegionExactnessTests.swift:346-360).  round_gate_up = 1: gate and
 * up are each rounded to fp16 first (Tests/SmeltCompilerTests/PrefillKernelTests.swift:390-430). */
SO_API int so_affine_gate_up_swiglu(const uint8_t *gw, const uint16_t *gs, const uint16_t *gb,
                                    const uint8_t *uw, const uint16_t *us, const uint16_t *ub,
                                    const uint16_t *x, int rows, int cols, int group, int batch,
                                    int round_gate_up, uint16_t *y) {
    size_t n = (size_t)batch * rows;
    float *g = (float *)malloc(sizeof(float) * n), *u = (float *)malloc(sizeof(float) * n);
    if (!g || !u) { free(g); free(u); return SO_ERR_ALLOC; }
    int rc = affine_matvec_acc(gw, gs, gb, x, rows, cols, group, batch, g);
    if (rc == SO_OK) rc = affine_matvec_acc(uw, us, ub, x, rows, cols, group, batch, u);
    if (rc == SO_OK)
        for (size_t i = 0; i < n; ++i) {
            float gv = g[i], uv = u[i];
            if (round_gate_up) { gv = round_h(gv); uv = round_h(uv); }
            y[i] = f2h(gv / (1.0f + expf(-gv)) * uv);
        }
    free(g); free(u);
    return rc;
}

/* ───────────────────────── dense fp16 matvec ─────────────────────────
 * Resources/Shaders/lut_matvec.metal:799-834 (fp16_matvec): fp32 accumulation, clamp to
 * ±65504, fp16 out.  No Swift scalar twin exists; summation is in column order.
 */
SO_API int so_fp16_matvec(const uint16_t *w, const uint16_t *x_f16, int rows, int cols, int batch,
                          uint16_t *y) {
    if (rows <= 0 || cols <= 0 || batch <= 0) return SO_ERR_GEOMETRY;
    float *x = (float *)malloc(sizeof(float) * (size_t)batch * cols);
    if (!x) return SO_ERR_ALLOC;
    so_f16_to_f32(x_f16, x, (int64_t)batch * cols);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const uint16_t *wr = w + (size_t)r * cols;
        for (int b = 0; b < batch; ++b) {
            const float *xb = x + (size_t)b * cols;
            float acc = 0.0f;
            for (int c = 0; c < cols; ++c) acc += h2f(wr[c]) * xb[c];
            acc = acc < -65504.0f ? -65504.0f : (acc > 65504.0f ? 65504.0f : acc);
            y[(size_t)b * rows + r] = f2h(acc);
        }
    }
    free(x);
    return SO_OK;
}

/* ───────────────────────── binary1 / ternary2 codec ─────────────────────────
 * Sources/SmeltRuntime/SmeltSignedQuantCodec.swift:22-35 (semanticCode), :102-124 (code,
 * LSB-first), :219-257 (dequantizeRow).  format: 1 = binary1 (0 -> -1, 1 -> +1),
 * 2 = ternary2 (0 -> -1, 1 -> 0, 2 -> +1, 3 invalid).
 */
static inline int signed_bits(int format) { return format == 1 ? 1 : (format == 2 ? 2 : 0); }

SO_API int so_signed_packed_byte_count(int64_t logical_count, int format, int64_t *out) {
    int bits = signed_bits(format);
    if (!bits || logical_count < 0) return SO_ERR_GEOMETRY;
    *out = (logical_count * bits + 7) / 8;
    return SO_OK;
}

SO_API int so_signed_groups_per_row(int padded_cols, int group, int *out) {
    if (padded_cols <= 0 || group <= 0 || padded_cols % group != 0) return SO_ERR_GEOMETRY;
    *out = padded_cols / group;
    return SO_OK;
}

static inline uint8_t signed_code_at(const uint8_t *bytes, int64_t idx, int bits) {
    int64_t bit = idx * bits;
    return (uint8_t)((bytes[bit >> 3] >> (bit & 7)) & ((1u << bits) - 1u));
}

/* Returns SO_ERR_INVALID_CODE and the first offending logical index when a ternary code 3
 * is present (validateCodes, :127-147). */
SO_API int so_signed_validate_codes(const uint8_t *codes, int64_t byte_count, int64_t logical_count,
                                    int format, int64_t *bad_index) {
    int bits = signed_bits(format);
    if (!bits || logical_count < 0) return SO_ERR_GEOMETRY;
    if (byte_count < (logical_count * bits + 7) / 8) return SO_ERR_GEOMETRY;
    if (format != 2) return SO_OK;
    for (int64_t i = 0; i < logical_count; ++i)
        if (signed_code_at(codes, i, 2) == 3) {
            if (bad_index) *bad_index = i;
            return SO_ERR_INVALID_CODE;
        }
    return SO_OK;
}

SO_API int so_signed_dequantize_row(int format, const uint8_t *codes, int64_t code_bytes,
                                    const uint16_t *scales, int64_t scale_bytes, int cols,
                                    int padded_cols, int group, float *out) {
    int bits = signed_bits(format);
    if (!bits || cols <= 0 || cols > padded_cols) return SO_ERR_GEOMETRY;
    int groups;
    if (so_signed_groups_per_row(padded_cols, group, &groups)) return SO_ERR_GEOMETRY;
    if (code_bytes < ((int64_t)padded_cols * bits + 7) / 8) return SO_ERR_GEOMETRY;
    if (scale_bytes < (int64_t)groups * 2) return SO_ERR_GEOMETRY;
    int rc = so_signed_validate_codes(codes, code_bytes, padded_cols, format, NULL);
    if (rc) return rc;
    for (int c = 0; c < cols; ++c) {
        uint8_t code = signed_code_at(codes, c, bits);
        int sem = format == 1 ? (code == 0 ? -1 : 1) : (int)code - 1;
        out[c] = (float)sem * h2f(scales[c / group]);
    }
    return SO_OK;
}

/* ───────────────────────── binary / ternary matvec ─────────────────────────
 * Tests/SmeltCompilerTests/SignedQuantKernelTests.swift:1030-1045: one fp32 accumulator per
 * (batch,row), expected += x * semantic * scale in column order.  row_stride_bytes is the
 * packed row stride (padded_cols*bits/8).
 */
static int signed_matvec_acc(int format, const uint8_t *codes, const uint16_t *scales,
                             const uint16_t *x_f16, int rows, int cols, int group, int batch,
                             float *y) {
    int bits = signed_bits(format);
    if (!bits || rows <= 0 || cols <= 0 || group <= 0 || batch <= 0 || cols % group) return SO_ERR_GEOMETRY;
    int groups = cols / group;
    size_t row_bytes = (size_t)cols * bits / 8;
    float *x = (float *)malloc(sizeof(float) * (size_t)batch * cols);
    if (!x) return SO_ERR_ALLOC;
    so_f16_to_f32(x_f16, x, (int64_t)batch * cols);
    int bad = 0;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const uint8_t *cr = codes + (size_t)r * row_bytes;
        const uint16_t *sr = scales + (size_t)r * groups;
        for (int b = 0; b < batch; ++b) {
            const float *xb = x + (size_t)b * cols;
            float acc = 0.0f;
            for (int c = 0; c < cols; ++c) {
                uint8_t code = signed_code_at(cr, c, bits);
                float sem;
                if (format == 1) sem = code == 0 ? -1.0f : 1.0f;
                else {
                    if (code == 3) { bad = 1; sem = 0.0f; }
                    else sem = (float)((int)code - 1);
                }
                acc += xb[c] * sem * h2f(sr[c / group]);
            }
            y[(size_t)b * rows + r] = acc;
        }
    }
    free(x);
    return bad ? SO_ERR_INVALID_CODE : SO_OK;
}

SO_API int so_signed_matvec(int format, const uint8_t *codes, const uint16_t *scales,
                            const uint16_t *x, int rows, int cols, int group, int batch,
                            uint16_t *y) {
    float *acc = (float *)malloc(sizeof(float) * (size_t)batch * rows);
    if (!acc) return SO_ERR_ALLOC;
    int rc = signed_matvec_acc(format, codes, scales, x, rows, cols, group, batch, acc);
    if (rc == SO_OK) so_f32_to_f16(acc, y, (int64_t)batch * rows);
    free(acc);
    return rc;
}

SO_API int so_signed_matvec_f32(int format, const uint8_t *codes, const uint16_t *scales,
                                const uint16_t *x, int rows, int cols, int group, int batch,
                                float *y) {
    return signed_matvec_acc(format, codes, scales, x, rows, cols, group, batch, y);
}

/* signed_*_matvec_add (Resources/Shaders/signed_quant.metal:271-278): half(float(half(acc))
 * + float(residual)). */
SO_API int so_signed_matvec_add(int format, const uint8_t *codes, const uint16_t *scales,
                                const uint16_t *x, const uint16_t *residual, int rows, int cols,
                                int group, int batch, uint16_t *y) {
    float *acc = (float *)malloc(sizeof(float) * (size_t)batch * rows);
    if (!acc) return SO_ERR_ALLOC;
    int rc = signed_matvec_acc(format, codes, scales, x, rows, cols, group, batch, acc);
    if (rc == SO_OK)
        for (int64_t i = 0; i < (int64_t)batch * rows; ++i)
            y[i] = f2h(round_h(acc[i]) + h2f(residual[i]));
    free(acc);
    return rc;
}

/* Staged-fp16 SwiGLU shared by the signed kernels and swiglu_fused
 * (Resources/Shaders/signed_quant.metal:15-20, activations_precise.metal:9-22): every
 * intermediate is an fp16 value: tail = 1/(1+exp(|g|)), sigmoid = g<0 ? tail : 1-tail,
 * activated = g*sigmoid, out = activated*up. */
static inline uint16_t swiglu_staged_half(uint16_t gate, uint16_t up) {
    float g = h2f(gate);
    float e = round_h(expf(fabsf(g)));
    float denom = round_h(1.0f + e);
    float tail = round_h(1.0f / denom);
    float sig = g < 0.0f ? tail : round_h(1.0f - tail);
    float act = round_h(g * sig);
    return f2h(act * h2f(up));
}

SO_API void so_swiglu_staged(const uint16_t *gate, const uint16_t *up, int64_t n, uint16_t *y) {
    for (int64_t i = 0; i < n; ++i) y[i] = swiglu_staged_half(gate[i], up[i]);
}

/* signed_*_gate_up_swiglu.  staged = 1: the kernel's staged-fp16 chain (signed_quant.metal
 * :15-20).  staged = 0: the test oracle's form, gate and up rounded to fp16 then
 * half(clamp(g/(1+exp(-g))*u, ±65504)) (SignedQuantKernelTests.swift:1210-1226). */
SO_API int so_signed_gate_up_swiglu(int format, const uint8_t *gc, const uint16_t *gs,
                                    const uint8_t *uc, const uint16_t *us, const uint16_t *x,
                                    int rows, int cols, int group, int batch, int staged,
                                    uint16_t *y) {
    size_t n = (size_t)batch * rows;
    float *g = (float *)malloc(sizeof(float) * n), *u = (float *)malloc(sizeof(float) * n);
    if (!g || !u) { free(g); free(u); return SO_ERR_ALLOC; }
    int rc = signed_matvec_acc(format, gc, gs, x, rows, cols, group, batch, g);
    if (rc == SO_OK) rc = signed_matvec_acc(format, uc, us, x, rows, cols, group, batch, u);
    if (rc == SO_OK)
        for (size_t i = 0; i < n; ++i) {
            uint16_t gh = f2h(g[i]), uh = f2h(u[i]);
            if (staged) y[i] = swiglu_staged_half(gh, uh);
            else {
                float gv = h2f(gh), uv = h2f(uh);
                float v = gv / (1.0f + expf(-gv)) * uv;
                v = v < -65504.0f ? -65504.0f : (v > 65504.0f ? 65504.0f : v);
                y[i] = f2h(v);
            }
        }
    free(g); free(u);
    return rc;
}

/* ───────────────────────── glue ───────────────────────── */

/* rms_norm_1pw.  two_stage = 0: Tests/.../MetalKernelTestSupport.swift:227-243 (cpuRmsNorm1pw),
 * one rounding of x*invRms*(1+w).  two_stage = 1: the kernel's rounding points
 * (Resources/Shaders/norms.metal:58-63): half(x*rs) times half(1+w) as an fp16 product. */
SO_API int so_rms_norm_1pw(const uint16_t *x, const uint16_t *w, int dim, float eps, int two_stage,
                           uint16_t *y) {
    if (dim <= 0) return SO_ERR_GEOMETRY;
    float ss = 0.0f;
    for (int i = 0; i < dim; ++i) { float v = h2f(x[i]); ss += v * v; }
    float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    for (int i = 0; i < dim; ++i) {
        if (two_stage) {
            float n = round_h(h2f(x[i]) * inv);
            float dw = round_h(1.0f + h2f(w[i]));
            y[i] = f2h(dw * n);
        } else {
            y[i] = f2h(h2f(x[i]) * inv * (1.0f + h2f(w[i])));
        }
    }
    return SO_OK;
}

/* per_head_rms_norm with a direct weight (Resources/Shaders/attention_fused.metal:93-145):
 * weight * half(x*rs) as an fp16 product. */
SO_API int so_per_head_rms_norm(const uint16_t *x, const uint16_t *w, int heads, int head_dim,
                                float eps, uint16_t *y) {
    if (heads <= 0 || head_dim <= 0) return SO_ERR_GEOMETRY;
    for (int h = 0; h < heads; ++h) {
        const uint16_t *xh = x + (size_t)h * head_dim;
        float ss = 0.0f;
        for (int i = 0; i < head_dim; ++i) { float v = h2f(xh[i]); ss += v * v; }
        float inv = 1.0f / sqrtf(ss / (float)head_dim + eps);
        for (int i = 0; i < head_dim; ++i) {
            float n = round_h(h2f(xh[i]) * inv);
            y[(size_t)h * head_dim + i] = f2h(h2f(w[i]) * n);
        }
    }
    return SO_OK;
}

/* Metal's simd_sum over 32 lane values: a butterfly over lane distance 16, 8, 4, 2, 1 (the total as lane 0 sees it). */
static inline float simd_sum32(float *lane) {
    for (int off = 16; off > 0; off >>= 1)
        for (int l = 0; l < off; ++l) lane[l] += lane[l + off];
    return lane[0];
}

/* The per-head norms of Resources/Shaders/attention_fused.metal:38-330 with their reduction
 * topologies.  mode 0 per_head_rms_norm(_batched) (:93-145, :247-296): thread t squares its four
 * adjacent values 4 t .. 4 t + 3, every simdgroup sums its lanes, the simdgroups' sums are
 * themselves summed with simd_sum; y = w * half(x * rs) as an fp16 product.  mode 1
 * per_head_rms_norm_1pw(_batched) (:38-91, :188-245): thread t adds x[t]^2, x[t + tgs]^2, ...,
 * simdgroup sums, then added one after the other; y = half(x * rs * (1 + w)).  mode 2
 * per_head_rms_norm_noscale(_batched) (:147-186, :298-330): mode 1's reduction, y = half(x * rs).
 * The batched forms use tgs = min(head_dim, 256). */
SO_API int so_head_norm(int mode, const uint16_t *x, const uint16_t *w, int heads, int head_dim, float eps, int tgs, uint16_t *y) {
    if (heads <= 0 || head_dim <= 0 || head_dim > 1024 || mode < 0 || mode > 2 || tgs < 32 || tgs % 32 || tgs > 1024) return SO_ERR_GEOMETRY;
    for (int h = 0; h < heads; ++h) {
        const uint16_t *xh = x + (size_t)h * head_dim;
        float total;
        if (mode == 0) {
            float partial[32] = {0};
            for (int s = 0; s * 128 < head_dim; ++s) {
                float lane[32];
                for (int l = 0; l < 32; ++l) {
                    float p = 0.0f;
                    for (int i = 0; i < 4; ++i) {
                        const int e = s * 128 + 4 * l + i;
                        const float v = e < head_dim ? h2f(xh[e]) : 0.0f;
                        p += v * v;
                    }
                    lane[l] = p;
                }
                partial[s] = simd_sum32(lane);
            }
            total = simd_sum32(partial);
        } else {
            total = 0.0f;
            for (int s = 0; s < tgs / 32; ++s) {
                float lane[32];
                for (int l = 0; l < 32; ++l) {
                    float p = 0.0f;
                    for (int i = s * 32 + l; i < head_dim; i += tgs) p += h2f(xh[i]) * h2f(xh[i]);
                    lane[l] = p;
                }
                total += simd_sum32(lane);
            }
        }
        const float rs = 1.0f / sqrtf(total / (float)head_dim + eps);
        for (int i = 0; i < head_dim; ++i) {
            const float v = h2f(xh[i]);
            uint16_t o;
            if (mode == 0) o = f2h(h2f(w[i]) * round_h(v * rs));
            else if (mode == 1) o = f2h(v * rs * (1.0f + h2f(w[i])));
            else o = f2h(v * rs);
            y[(size_t)h * head_dim + i] = o;
        }
    }
    return SO_OK;
}

/* The row norms of Resources/Shaders/norms.metal beyond rms_norm_1pw, with their reduction
 * topologies and roundings.  One row of `dim` values per threadgroup.
 * topology 0 (rms_norm_1pw_batched, :1488-1550): thread t of tgs adds the squares of its four
 *   adjacent values in every tile of 4 tgs values; simdgroup sums; the sums summed by simd_sum.
 * topology 1 (the d1024 / d1536 / d2048 / d2560 kernels, :72-176, :262-575, :579-652, :727-990):
 *   dim / 8 threads, thread t takes values 4 t .. 4 t + 3 and 4 (t + dim / 8) ..: dot(x0, x0) +
 *   dot(x1, x1); simdgroup sums added one after the other.
 * topology 2 (rms_norm_scale_only(_precise), the d256 kernels, l2_normalize, :177-260, :991-1090,
 *   :1155-1190, :1436-1486): thread t adds x[t]^2, x[t + tgs]^2, ...; simdgroup sums added one
 *   after the other.
 * scale 0: rsqrt(total / dim + eps); 1 (l2_normalize): 1 / max(sqrt(total), eps).
 * value 0: none (the scale alone, to scale_out[row]); 1: half(1 + w) * half(x * rs) as an fp16
 *   product; 2: half(x * (rs * (1 + w))); 3: half(x * rs * (1 + w)); 4: half(x * rs).
 * pre (may be NULL): the row is half(x + pre), which is also written to y
 *   (residual_add_rms_norm_scale_only_precise, :1059-1090).  residual (may be NULL): y =
 *   half(y + residual) after the norm is rounded; scalar (may be NULL): y = half(float(y) *
 *   float(scalar[0])) after that (rms_norm_1pw_d256_add_scalar_weight). */
SO_API int so_row_norm(const uint16_t *x, const uint16_t *pre, const uint16_t *w, const uint16_t *residual, const uint16_t *scalar,
                       uint16_t *y, float *scale_out, int rows, int dim, float eps, int topology, int tgs, int value, int scale) {
    if (rows <= 0 || dim <= 0 || dim > 16384 || topology < 0 || topology > 2 || value < 0 || value > 4 || scale < 0 || scale > 1) return SO_ERR_GEOMETRY;
    if (topology == 1) { if (dim % 256) return SO_ERR_GEOMETRY; tgs = dim / 8; }
    if (tgs < 32 || tgs % 32 || tgs > 1024) return SO_ERR_GEOMETRY;
    float *v = (float *)malloc((size_t)dim * sizeof(float));
    if (!v) return SO_ERR_GEOMETRY;
    for (int r = 0; r < rows; ++r) {
        const uint16_t *xr = x + (size_t)r * dim;
        for (int i = 0; i < dim; ++i) {
            if (pre) {
                const uint16_t sum = f2h(h2f(xr[i]) + h2f(pre[(size_t)r * dim + i]));
                v[i] = h2f(sum);
                if (value == 0 && y) y[(size_t)r * dim + i] = sum;
            } else {
                v[i] = h2f(xr[i]);
            }
        }
        float total;
        if (topology == 0) {
            float partial[32] = {0};
            for (int s = 0; s < tgs / 32; ++s) {
                float lane[32];
                for (int l = 0; l < 32; ++l) {
                    const int t = 32 * s + l;
                    float p = 0.0f;
                    for (int tile = 0; tile < dim; tile += 4 * tgs)
                        for (int k = 0; k < 4; ++k) {
                            const int i = tile + 4 * t + k;
                            if (i < dim) p += v[i] * v[i];
                        }
                    lane[l] = p;
                }
                partial[s] = simd_sum32(lane);
            }
            total = simd_sum32(partial);
        } else {
            total = 0.0f;
            for (int s = 0; s < tgs / 32; ++s) {
                float lane[32];
                for (int l = 0; l < 32; ++l) {
                    const int t = 32 * s + l;
                    float p;
                    if (topology == 1) {
                        const float *a = v + 4 * t, *b = v + 4 * (t + tgs);
                        const float d0 = ((a[0] * a[0] + a[1] * a[1]) + a[2] * a[2]) + a[3] * a[3];
                        const float d1 = ((b[0] * b[0] + b[1] * b[1]) + b[2] * b[2]) + b[3] * b[3];
                        p = d0 + d1;
                    } else {
                        p = 0.0f;
                        for (int i = t; i < dim; i += tgs) p += v[i] * v[i];
                    }
                    lane[l] = p;
                }
                total += simd_sum32(lane);
            }
        }
        const float sqrt_total = sqrtf(total);
        const float rs = scale == 0 ? 1.0f / sqrtf(total / (float)dim + eps) : 1.0f / (sqrt_total > eps ? sqrt_total : eps);
        if (scale_out) scale_out[r] = rs;
        if (value == 0) continue;
        for (int i = 0; i < dim; ++i) {
            float o;
            const float wv = w ? h2f(w[i]) : 0.0f;
            if (value == 1) o = round_h(round_h(1.0f + wv) * round_h(v[i] * rs));
            else if (value == 2) o = round_h(v[i] * (rs * (1.0f + wv)));
            else if (value == 3) o = round_h(v[i] * rs * (1.0f + wv));
            else o = round_h(v[i] * rs);
            if (residual) o = round_h(o + h2f(residual[(size_t)r * dim + i]));
            if (scalar) o = round_h(o * h2f(scalar[0]));
            y[(size_t)r * dim + i] = f2h(o);
        }
    }
    free(v);
    return SO_OK;
}

/* gate_split (attention_fused.metal:11-27): [heads, 2 D] rows of query | gate -> query [heads, D], gate [heads, D]. */
SO_API void so_gate_split(const uint16_t *input, int heads, int head_dim, uint16_t *query, uint16_t *gate) {
    for (int h = 0; h < heads; ++h)
        for (int d = 0; d < head_dim; ++d) {
            query[(size_t)h * head_dim + d] = input[(size_t)h * head_dim * 2 + d];
            gate[(size_t)h * head_dim + d] = input[(size_t)h * head_dim * 2 + head_dim + d];
        }
}

/* The element-wise kernels of Resources/Shaders/activations.metal:4-210 and activations_precise.metal:22-35.
 * op 0 silu x / (1 + exp(-x)); 1 sigmoid 1 / (1 + exp(-x)); 2 softplus (x > 20 ? x : log(1 + exp(x)));
 * 3 buffer_copy; 4 scalar_mul half(x * scalar); 5 logit_cap half(cap * tanh(x / cap)); 6 elementwise_mul (fp16
 * product); 7 sigmoid_mul a * sigmoid(b) in half arithmetic; 8 geglu_fused half(clamp(gelu_tanh(a) * b)), b read
 * with its own row stride; 9 projection_bias_add_batched a[batch, rows] + b[rows].  a / y [batch, count]. */
SO_API int so_elementwise(int op, const uint16_t *a, const uint16_t *b, uint16_t *y, int count, int batch, int b_stride, float scalar) {
    if (count <= 0 || batch <= 0 || op < 0 || op > 9) return SO_ERR_GEOMETRY;
    for (int r = 0; r < batch; ++r)
        for (int i = 0; i < count; ++i) {
            const size_t idx = (size_t)r * count + i;
            const float x = h2f(a[idx]);
            uint16_t o;
            switch (op) {
                case 0: o = f2h(x / (1.0f + expf(-x))); break;
                case 1: o = f2h(1.0f / (1.0f + expf(-x))); break;
                case 2: o = f2h(x > 20.0f ? x : logf(1.0f + expf(x))); break;
                case 3: o = a[idx]; break;
                case 4: o = f2h(x * scalar); break;
                case 5: o = f2h(scalar * tanhf(x / scalar)); break;
                case 6: o = f2h(x * h2f(b[idx])); break;
                case 7: {
                    const float g = h2f(b[idx]);
                    const float tail = round_h(1.0f / round_h(1.0f + round_h(expf(fabsf(g)))));
                    const float sig = g < 0.0f ? tail : round_h(1.0f - tail);
                    o = f2h(x * sig);
                    break;
                }
                case 8: {
                    const float u = h2f(b[(size_t)r * b_stride + i]);
                    float inner = 0.7978845608f * (x + 0.044715f * (x * x * x));
                    inner = inner < -20.0f ? -20.0f : (inner > 20.0f ? 20.0f : inner);
                    float v = 0.5f * x * (1.0f + tanhf(inner)) * u;
                    v = v < -65504.0f ? -65504.0f : (v > 65504.0f ? 65504.0f : v);
                    o = f2h(v);
                    break;
                }
                default: o = f2h(x + h2f(b[i])); break;
            }
            y[idx] = o;
        }
    return SO_OK;
}

/* elementwise_add (Resources/Shaders/activations.metal:56-66): fp16 a + b. */
SO_API void so_elementwise_add(const uint16_t *a, const uint16_t *b, int64_t n, uint16_t *y) {
    for (int64_t i = 0; i < n; ++i) y[i] = f2h(h2f(a[i]) + h2f(b[i]));
}

/* embedding_gather (lut_matvec.metal:951-962): row copy. */
SO_API void so_embedding_gather(const uint16_t *table, int64_t token, int hidden, uint16_t *y) {
    memcpy(y, table + (size_t)token * hidden, (size_t)hidden * 2);
}

/* Argmax over fp16 logits: strictly-greater scan, so ties keep the lowest index and -0
 * equals +0 (Sources/SmeltRuntime/SmeltSelection.swift:165-204; key order
 * Resources/Shaders/lut_matvec.metal:4045-4074). */
SO_API int32_t so_argmax_f16(const uint16_t *logits, int64_t n) {
    float best = -INFINITY;
    int32_t idx = -1;
    for (int64_t i = 0; i < n; ++i) {
        float v = h2f(logits[i]);
        if (v > best) { best = v; idx = (int32_t)i; }
    }
    return idx;
}

/* ───────────────────────── RoPE + KV cache ─────────────────────────
 * Resources/Shaders/attention.metal:11-115.  layout: 0 adjacent pairs, 1 split-half,
 * 2 proportional split-half.  math_mode 1 (analytic): invFreq = exp2(-(pair/halfRope)*log2θ),
 * angle = float(position)*invFreq, fp32 cos/sin; math_mode 0: fp16 cos/sin table rows.
 * Results x0*c0 - x1*s0 and x0*s1 + x1*c1, rounded to fp16, in place.
 */
static inline void rope_pair_indices(int layout, int dim, int half_rope, int head_dim, int *d0, int *d1,
                                     int *c0, int *c1) {
    if (layout == 1) { *d0 = dim; *d1 = dim + half_rope; *c0 = *d0; *c1 = *d1; }
    else if (layout == 2) { *d0 = dim; *d1 = dim + head_dim / 2; *c0 = dim; *c1 = dim + half_rope; }
    else { *d0 = dim * 2; *d1 = *d0 + 1; *c0 = *d0; *c1 = *d1; }
}

static inline void rope_trig(int pair, int half_rope, uint32_t position, float base_log2, int math_mode,
                             const uint16_t *cos_t, const uint16_t *sin_t, int c0i, int c1i,
                             float *c0, float *s0, float *c1, float *s1) {
    if (math_mode == 1) {
        /* correctly rounded fp32 exp2 / cos / sin (evaluated in double, rounded once): Metal's
         * fast::cos / fast::sin are not reproducible off-device, and at large positions one ulp of
         * the frequency moves the phase by many fp16 ulps, so both sides pin the exact value. */
        float d = (float)pair / (float)half_rope;
        float inv_freq = (float)exp2((double)(-d * base_log2));
        float angle = (float)position * inv_freq;
        float c = (float)cos((double)angle), s = (float)sin((double)angle);
        *c0 = c; *s0 = s; *c1 = c; *s1 = s;
    } else {
        *c0 = h2f(cos_t[c0i]); *s0 = h2f(sin_t[c0i]);
        *c1 = h2f(cos_t[c1i]); *s1 = h2f(sin_t[c1i]);
    }
}

SO_API int so_apply_rope(uint16_t *qk, const uint16_t *cos_t, const uint16_t *sin_t, int head_dim,
                         int rope_dim, int heads, int layout, uint32_t position, float base_log2,
                         int math_mode) {
    if (head_dim <= 0 || rope_dim <= 0 || rope_dim > head_dim || heads <= 0) return SO_ERR_GEOMETRY;
    int half_rope = rope_dim / 2;
    for (int h = 0; h < heads; ++h) {
        uint16_t *v = qk + (size_t)h * head_dim;
        for (int dim = 0; dim < half_rope; ++dim) {
            int d0, d1, c0i, c1i;
            rope_pair_indices(layout, dim, half_rope, head_dim, &d0, &d1, &c0i, &c1i);
            float x0 = h2f(v[d0]), x1 = h2f(v[d1]);
            float c0, s0, c1, s1;
            rope_trig(dim, half_rope, position, base_log2, math_mode, cos_t, sin_t, c0i, c1i, &c0, &s0, &c1, &s1);
            v[d0] = f2h(x0 * c0 - x1 * s0);
            v[d1] = f2h(x0 * s1 + x1 * c1);
        }
    }
    return SO_OK;
}

/* kv_cache_update (attention.metal:122-139; Tests/.../RegionExactnessTests.swift:909-925):
 * cache[h, pos, :] = new[h, :], cache laid out [heads, capacity, head_dim]. */
SO_API int so_kv_cache_update(uint16_t *cache, const uint16_t *new_kv, int capacity, int head_dim,
                              int pos, int heads) {
    if (pos < 0 || pos >= capacity || head_dim <= 0 || heads <= 0) return SO_ERR_GEOMETRY;
    for (int h = 0; h < heads; ++h)
        memcpy(cache + ((size_t)h * capacity + pos) * head_dim, new_kv + (size_t)h * head_dim,
               (size_t)head_dim * 2);
    return SO_OK;
}

/* rope_kv_cache_update (attention.metal:141-209): rotate the new K row and write it at pos. */
SO_API int so_rope_kv_cache_update(uint16_t *cache, const uint16_t *new_kv, const uint16_t *cos_t,
                                   const uint16_t *sin_t, int capacity, int head_dim, int pos,
                                   int heads, int rope_dim, int layout, float base_log2,
                                   int math_mode) {
    if (pos < 0 || pos >= capacity || head_dim <= 0 || heads <= 0 || rope_dim > head_dim) return SO_ERR_GEOMETRY;
    uint16_t *tmp = (uint16_t *)malloc((size_t)heads * head_dim * 2);
    if (!tmp) return SO_ERR_ALLOC;
    memcpy(tmp, new_kv, (size_t)heads * head_dim * 2);
    int rc = so_apply_rope(tmp, cos_t, sin_t, head_dim, rope_dim, heads, layout, (uint32_t)pos, base_log2, math_mode);
    if (rc == SO_OK) rc = so_kv_cache_update(cache, tmp, capacity, head_dim, pos, heads);
    free(tmp);
    return rc;
}

/* ───────────────────────── attention decode ─────────────────────────
 * Tests/SmeltCompilerTests/RegionExactnessTests.swift:1414-1475
 * (referenceAttentionDecodeCPU): per q head, scores = (q·k)*scale over [seqStart, seqLen),
 * max, exp(score-max), invSum = 1/sum, out[d] = half(Σ_s (p_s*invSum) * v[s,d]).
 * K/V are [kv_heads, capacity, head_dim] fp16; GQA kvHead = qHead / (nQ/nKV).
 */
SO_API int so_attention_decode(const uint16_t *q, const uint16_t *k_cache, const uint16_t *v_cache,
                               int n_q, int n_kv, int head_dim, int capacity, int seq_len,
                               float scale, int sliding_window, uint16_t *out) {
    if (n_q <= 0 || n_kv <= 0 || n_q % n_kv || head_dim <= 0 || seq_len <= 0 || seq_len > capacity)
        return SO_ERR_GEOMETRY;
    int ratio = n_q / n_kv;
    size_t kv_stride = (size_t)capacity * head_dim;
    int seq_start = 0;
    if (sliding_window > 0 && sliding_window < seq_len) seq_start = seq_len - sliding_window;
    int n = seq_len - seq_start;
    int fail = 0;
#pragma omp parallel for schedule(static)
    for (int qh = 0; qh < n_q; ++qh) {
        int kvh = qh / ratio;
        float *qf = (float *)malloc(sizeof(float) * head_dim);
        float *scores = (float *)malloc(sizeof(float) * n);
        if (!qf || !scores) { fail = 1; free(qf); free(scores); continue; }
        for (int d = 0; d < head_dim; ++d) qf[d] = h2f(q[(size_t)qh * head_dim + d]);
        float mx = -INFINITY;
        for (int s = seq_start; s < seq_len; ++s) {
            const uint16_t *kr = k_cache + kvh * kv_stride + (size_t)s * head_dim;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; ++d) dot += qf[d] * h2f(kr[d]);
            float sc = dot * scale;
            scores[s - seq_start] = sc;
            if (sc > mx) mx = sc;
        }
        float sum = 0.0f;
        for (int i = 0; i < n; ++i) { scores[i] = expf(scores[i] - mx); sum += scores[i]; }
        float inv = 1.0f / sum;
        for (int d = 0; d < head_dim; ++d) {
            float acc = 0.0f;
            for (int s = seq_start; s < seq_len; ++s) {
                float w = scores[s - seq_start] * inv;
                acc += w * h2f(v_cache[kvh * kv_stride + (size_t)s * head_dim + d]);
            }
            out[(size_t)qh * head_dim + d] = f2h(acc);
        }
        free(qf); free(scores);
    }
    return fail ? SO_ERR_ALLOC : SO_OK;
}

/* The split-K pair a D256 package dispatches from 1,024 keys on
 * (Resources/Shaders/attention.metal:1071-1141 first pass, :1146-1206 second pass; emitted by
 * Sources/SmeltCompiler/AttentionPlugin.swift:865-918): head_dim 256, scale 1/16 folded into
 * the query, 128 key blocks that interleave the keys (block b owns keys b, b+128, ...), an
 * online softmax per block, partial outputs materialised as fp16 and (sum, max) kept in fp32;
 * the second pass weights block b by exp(max_b - max), adds blocks in index order and divides
 * by the weighted sum of the block sums.  partials [n_q,128,256] fp16 and stats [2][n_q][128]
 * fp32 are scratch the caller provides (their contents are the reference's intermediate buffers). */
SO_API int so_attention_decode_mlx_2pass(const uint16_t *q, const uint16_t *k_cache, const uint16_t *v_cache,
                                         int n_q, int n_kv, int capacity, int seq_len,
                                         uint16_t *partials, float *stats, uint16_t *out) {
    enum { D = 256, BLOCKS = 128 };
    if (n_q <= 0 || n_kv <= 0 || n_q % n_kv || seq_len <= 0 || seq_len > capacity || !partials || !stats)
        return SO_ERR_GEOMETRY;
    const float scale = 0.0625f;
    int gqa = n_q / n_kv;
#pragma omp parallel for schedule(static)
    for (int qh = 0; qh < n_q; ++qh) {
        int kvh = qh / gqa;
        float qv[D], ov[D];
        for (int d = 0; d < D; ++d) qv[d] = scale * h2f(q[(size_t)qh * D + d]);
        for (int block = 0; block < BLOCKS; ++block) {
            for (int d = 0; d < D; ++d) ov[d] = 0.0f;
            float mx = -3.402823466e+38f, sum = 0.0f;
            for (int key = block; key < seq_len; key += BLOCKS) {
                const uint16_t *kr = k_cache + ((size_t)kvh * capacity + key) * D;
                const uint16_t *vr = v_cache + ((size_t)kvh * capacity + key) * D;
                /* 32 lanes x 8 values, lane partials summed (simd_sum) */
                float score = 0.0f;
                for (int lane = 0; lane < 32; ++lane) {
                    float part = 0.0f;
                    for (int i = 0; i < 8; ++i) part += qv[lane * 8 + i] * h2f(kr[lane * 8 + i]);
                    score += part;
                }
                float nm = score > mx ? score : mx;
                float factor = expf(mx - nm), e = expf(score - nm);
                mx = nm;
                sum = sum * factor + e;
                for (int d = 0; d < D; ++d) ov[d] = ov[d] * factor + e * h2f(vr[d]);
            }
            stats[(size_t)qh * BLOCKS + block] = sum;
            stats[(size_t)n_q * BLOCKS + (size_t)qh * BLOCKS + block] = mx;
            for (int d = 0; d < D; ++d) partials[((size_t)qh * BLOCKS + block) * D + d] = f2h(ov[d]);
        }
        const float *sums = stats + (size_t)qh * BLOCKS;
        const float *maxs = stats + (size_t)n_q * BLOCKS + (size_t)qh * BLOCKS;
        float M = -3.402823466e+38f;
        for (int b = 0; b < BLOCKS; ++b) if (maxs[b] > M) M = maxs[b];
        float total = 0.0f;
        for (int b = 0; b < BLOCKS; ++b) total += expf(maxs[b] - M) * sums[b];
        for (int d = 0; d < D; ++d) {
            float acc = 0.0f;
            for (int b = 0; b < BLOCKS; ++b) acc += expf(maxs[b] - M) * h2f(partials[((size_t)qh * BLOCKS + b) * D + d]);
            out[(size_t)qh * D + d] = f2h(total == 0.0f ? acc : acc / total);
        }
    }
    return SO_OK;
}

/* the DeltaNet kernels are restated further down */
SO_API int so_conv1d_update_silu(uint16_t *state, const uint16_t *new_val, const uint16_t *weight, uint16_t *out, int channels, int kernel_size);
SO_API int so_rms_scale_qk(uint16_t *qkv, int head_dim, float eps, int qkv_dim, int qk_heads, int batch);
SO_API int so_deltanet_recurrence_decode(uint16_t *state, const uint16_t *qkv, const uint16_t *b_proj, const uint16_t *a_proj, const uint16_t *a_log,
                                         const uint16_t *dt_bias, uint16_t *out, int head_dim, int value_heads, int qk_heads);
SO_API int so_rms_norm_gated_tg(const uint16_t *input, const uint16_t *gate, const uint16_t *weight, uint16_t *out, int head_dim, float eps, int heads, int tgs);
SO_API int so_rms_norm_gated_d128(const uint16_t *input, const uint16_t *gate, const uint16_t *weight, uint16_t *out, int heads);

/* ───────────────────────── whole decoder ─────────────────────────
 * Structure: Sources/SmeltRuntime/Qwen3TTSTalker.swift:229-292 (forwardStep: norm → q/k/v →
 * RoPE → cache append → GQA attention → o → residual → norm → gate/up SwiGLU → down →
 * residual → final norm), with the per-dispatch fp16 rounding points of the Metal text path:
 * every inter-kernel buffer is fp16 (embedding row, two-stage rms_norm_1pw with a stored
 * weight delta, half(acc) after each projection, analytic-mode split-half RoPE, fp16 KV,
 * half attention output, fp16 residual add, one rounding after the fp32 SwiGLU, clamped fp16
 * logits, lowest-index argmax).
 */
typedef struct {
    const uint8_t *w;
    const uint16_t *s, *b;
} so_affine_t;

typedef struct {
    const uint16_t *input_norm, *post_norm; /* stored as weight-1 */
    so_affine_t q, k, v, o, gate, up, down;
    /* a DeltaNet layer (kind 1) replaces q / k / v / o by these (Sources/SmeltCompiler/DeltaNetPlugin.swift:60-420) */
    int kind;
    so_affine_t dqkv, dz, da, db, dout;
    const uint16_t *conv_w, *a_log, *dt_bias, *gnorm_w;
    uint16_t *conv_state, *rec_state;
} so_layer_t;

typedef struct {
    int layers, hidden, inter, n_q, n_kv, head_dim, vocab, group, capacity;
    float eps, rope_theta;
    const uint16_t *embedding;  /* [vocab, hidden] fp16 */
    const uint16_t *lm_head;    /* [vocab, hidden] fp16 */
    const uint16_t *final_norm; /* weight-1 */
    so_layer_t *layer;
    uint16_t **k_cache, **v_cache; /* per layer [n_kv, capacity, head_dim] */
    int d_value_heads, d_qk_heads, d_head_dim, d_conv_kernel; /* linear-attention geometry of the DeltaNet layers */
} so_model_t;

SO_API so_model_t *so_model_create(int layers, int hidden, int inter, int n_q, int n_kv, int head_dim,
                                   int vocab, int group, int capacity, float eps, float rope_theta) {
    so_model_t *m = (so_model_t *)calloc(1, sizeof(so_model_t));
    if (!m) return NULL;
    m->layers = layers; m->hidden = hidden; m->inter = inter; m->n_q = n_q; m->n_kv = n_kv;
    m->head_dim = head_dim; m->vocab = vocab; m->group = group; m->capacity = capacity;
    m->eps = eps; m->rope_theta = rope_theta;
    m->layer = (so_layer_t *)calloc((size_t)layers, sizeof(so_layer_t));
    m->k_cache = (uint16_t **)calloc((size_t)layers, sizeof(uint16_t *));
    m->v_cache = (uint16_t **)calloc((size_t)layers, sizeof(uint16_t *));
    size_t kv = (size_t)n_kv * capacity * head_dim;
    for (int l = 0; l < layers; ++l) {
        m->k_cache[l] = (uint16_t *)calloc(kv, 2);
        m->v_cache[l] = (uint16_t *)calloc(kv, 2);
    }
    return m;
}

SO_API void so_model_destroy(so_model_t *m) {
    if (!m) return;
    for (int l = 0; l < m->layers; ++l) { free(m->k_cache[l]); free(m->v_cache[l]); free(m->layer[l].conv_state); free(m->layer[l].rec_state); }
    free(m->k_cache); free(m->v_cache); free(m->layer); free(m);
}

SO_API void so_model_set_globals(so_model_t *m, const uint16_t *embedding, const uint16_t *lm_head,
                                 const uint16_t *final_norm) {
    m->embedding = embedding; m->lm_head = lm_head; m->final_norm = final_norm;
}

/* which: 0 q, 1 k, 2 v, 3 o, 4 gate, 5 up, 6 down */
SO_API int so_model_set_affine(so_model_t *m, int layer, int which, const uint8_t *w, const uint16_t *s,
                               const uint16_t *b) {
    if (layer < 0 || layer >= m->layers || which < 0 || which > 6) return SO_ERR_GEOMETRY;
    so_affine_t *t = &m->layer[layer].q + which;
    t->w = w; t->s = s; t->b = b;
    return SO_OK;
}

SO_API int so_model_set_norms(so_model_t *m, int layer, const uint16_t *input_norm, const uint16_t *post_norm) {
    if (layer < 0 || layer >= m->layers) return SO_ERR_GEOMETRY;
    m->layer[layer].input_norm = input_norm; m->layer[layer].post_norm = post_norm;
    return SO_OK;
}

/* Hybrid models: the geometry of the DeltaNet layers, then per DeltaNet layer its five projections (which: 0 qkv,
 * 1 z, 2 a, 3 b, 4 out) and its four small tensors.  Marking a layer allocates its zeroed states. */
SO_API int so_model_set_delta_geometry(so_model_t *m, int value_heads, int qk_heads, int head_dim, int conv_kernel) {
    if (value_heads <= 0 || qk_heads <= 0 || value_heads % qk_heads || head_dim <= 0 || head_dim % 32 || head_dim > 256 || conv_kernel <= 0 || conv_kernel > 8)
        return SO_ERR_GEOMETRY;
    m->d_value_heads = value_heads; m->d_qk_heads = qk_heads; m->d_head_dim = head_dim; m->d_conv_kernel = conv_kernel;
    return SO_OK;
}
SO_API int so_model_set_delta_affine(so_model_t *m, int layer, int which, const uint8_t *w, const uint16_t *s, const uint16_t *b) {
    if (layer < 0 || layer >= m->layers || which < 0 || which > 4 || !m->d_value_heads) return SO_ERR_GEOMETRY;
    so_affine_t *t = &m->layer[layer].dqkv + which;
    t->w = w; t->s = s; t->b = b;
    return SO_OK;
}
SO_API int so_model_set_delta_params(so_model_t *m, int layer, const uint16_t *conv_w, const uint16_t *a_log, const uint16_t *dt_bias,
                                     const uint16_t *norm_w) {
    if (layer < 0 || layer >= m->layers || !m->d_value_heads) return SO_ERR_GEOMETRY;
    so_layer_t *L = &m->layer[layer];
    L->kind = 1; L->conv_w = conv_w; L->a_log = a_log; L->dt_bias = dt_bias; L->gnorm_w = norm_w;
    const size_t dq = (size_t)(2 * m->d_qk_heads + m->d_value_heads) * m->d_head_dim;
    free(L->conv_state); free(L->rec_state);
    L->conv_state = (uint16_t *)calloc(dq * m->d_conv_kernel, 2);
    L->rec_state = (uint16_t *)calloc((size_t)m->d_value_heads * m->d_head_dim * m->d_head_dim, 2);
    return L->conv_state && L->rec_state ? SO_OK : SO_ERR_ALLOC;
}

SO_API void so_model_reset_cache(so_model_t *m) {
    size_t kv = (size_t)m->n_kv * m->capacity * m->head_dim;
    for (int l = 0; l < m->layers; ++l) {
        memset(m->k_cache[l], 0, kv * 2); memset(m->v_cache[l], 0, kv * 2);
        if (m->layer[l].kind == 1) {
            memset(m->layer[l].conv_state, 0, (size_t)(2 * m->d_qk_heads + m->d_value_heads) * m->d_head_dim * m->d_conv_kernel * 2);
            memset(m->layer[l].rec_state, 0, (size_t)m->d_value_heads * m->d_head_dim * m->d_head_dim * 2);
        }
    }
}

/* Benchmark support: loads rows [0, n_positions) of one layer's K and V caches from
 * [n_kv, n_positions, head_dim] fp16 arrays, so that a timed decode step can start at a long
 * context without decoding the prompt first (attention then walks n_positions + 1 keys as it
 * would after a real prompt of that length). */
SO_API int so_model_fill_kv(so_model_t *m, int layer, const uint16_t *k, const uint16_t *v, int n_positions) {
    if (layer < 0 || layer >= m->layers || n_positions < 0 || n_positions > m->capacity) return SO_ERR_GEOMETRY;
    for (int h = 0; h < m->n_kv; ++h) {
        memcpy(m->k_cache[layer] + (size_t)h * m->capacity * m->head_dim, k + (size_t)h * n_positions * m->head_dim, (size_t)n_positions * m->head_dim * 2);
        memcpy(m->v_cache[layer] + (size_t)h * m->capacity * m->head_dim, v + (size_t)h * n_positions * m->head_dim, (size_t)n_positions * m->head_dim * 2);
    }
    return SO_OK;
}

/* One decode step for one sequence.  Writes fp16 logits [vocab] when logits != NULL and
 * returns the greedy token through *out_token. */
SO_API int so_model_decode_step(so_model_t *m, int32_t token, int position, uint16_t *logits_out,
                                int32_t *out_token) {
    if (token < 0 || token >= m->vocab || position < 0 || position >= m->capacity) return SO_ERR_GEOMETRY;
    int H = m->hidden, I = m->inter, D = m->head_dim, qd = m->n_q * D, kvd = m->n_kv * D, G = m->group;
    const int DD = m->d_head_dim, Hv = m->d_value_heads, Hqk = m->d_qk_heads;
    const int dq = (2 * Hqk + Hv) * DD, dv = Hv * DD;
    size_t scratch = (size_t)H * 3 + qd * 2 + kvd * 2 + I + (size_t)dq + 2 * (size_t)dv + 2 * (size_t)Hv;
    uint16_t *buf = (uint16_t *)malloc(scratch * 2);
    uint16_t *logits = logits_out ? logits_out : (uint16_t *)malloc((size_t)m->vocab * 2);
    if (!buf || !logits) { free(buf); if (!logits_out) free(logits); return SO_ERR_ALLOC; }
    uint16_t *h = buf, *normed = h + H, *tmp = normed + H, *q = tmp + H, *attn = q + qd, *k = attn + qd,
             *v = k + kvd, *act = v + kvd;
    uint16_t *dqkv = act + I, *dz = dqkv + dq, *dout = dz + dv, *da = dout + dv, *db = da + Hv;
    int rc = SO_OK;
    float base_log2 = log2f(m->rope_theta);
    float scale = 1.0f / sqrtf((float)D);
    so_embedding_gather(m->embedding, token, H, h);
    for (int l = 0; l < m->layers && rc == SO_OK; ++l) {
        so_layer_t *L = &m->layer[l];
        rc = so_rms_norm_1pw(h, L->input_norm, H, m->eps, 1, normed);
        if (!rc && L->kind == 1) {
            /* DeltaNetPlugin.swift:60-420: QKV / Z / A / B projections, conv + SiLU in place, Q / K scaling, recurrence,
             * gated norm with Z (the d128 form when the head is 128 wide and eps is 1e-6, else a threadgroup of
             * min(head_dim, 256)), output projection + residual */
            rc = so_affine_matvec(L->dqkv.w, L->dqkv.s, L->dqkv.b, normed, dq, H, G, 1, dqkv);
            if (!rc) rc = so_affine_matvec(L->dz.w, L->dz.s, L->dz.b, normed, dv, H, G, 1, dz);
            if (!rc) rc = so_affine_matvec(L->da.w, L->da.s, L->da.b, normed, Hv, H, G, 1, da);
            if (!rc) rc = so_affine_matvec(L->db.w, L->db.s, L->db.b, normed, Hv, H, G, 1, db);
            if (!rc) rc = so_conv1d_update_silu(L->conv_state, dqkv, L->conv_w, dqkv, dq, m->d_conv_kernel);
            if (!rc) rc = so_rms_scale_qk(dqkv, DD, 1e-6f, dq, Hqk, 1);
            if (!rc) rc = so_deltanet_recurrence_decode(L->rec_state, dqkv, db, da, L->a_log, L->dt_bias, dout, DD, Hv, Hqk);
            if (!rc) rc = (DD == 128 && m->eps == 1e-6f) ? so_rms_norm_gated_d128(dout, dz, L->gnorm_w, dout, Hv)
                                                         : so_rms_norm_gated_tg(dout, dz, L->gnorm_w, dout, DD, m->eps, Hv, DD < 256 ? DD : 256);
            if (!rc) rc = so_affine_matvec(L->dout.w, L->dout.s, L->dout.b, dout, H, dv, G, 1, tmp);
            if (!rc) so_elementwise_add(h, tmp, H, h);
            if (!rc) rc = so_rms_norm_1pw(h, L->post_norm, H, m->eps, 1, normed);
            if (!rc) rc = so_affine_gate_up_swiglu(L->gate.w, L->gate.s, L->gate.b, L->up.w, L->up.s, L->up.b, normed, I, H, G, 1, 0, act);
            if (!rc) rc = so_affine_matvec(L->down.w, L->down.s, L->down.b, act, H, I, G, 1, tmp);
            if (!rc) so_elementwise_add(h, tmp, H, h);
            continue;
        }
        if (!rc) rc = so_affine_matvec(L->q.w, L->q.s, L->q.b, normed, qd, H, G, 1, q);
        if (!rc) rc = so_affine_matvec(L->k.w, L->k.s, L->k.b, normed, kvd, H, G, 1, k);
        if (!rc) rc = so_affine_matvec(L->v.w, L->v.s, L->v.b, normed, kvd, H, G, 1, v);
        if (!rc) rc = so_apply_rope(q, NULL, NULL, D, D, m->n_q, 1, (uint32_t)position, base_log2, 1);
        if (!rc) rc = so_rope_kv_cache_update(m->k_cache[l], k, NULL, NULL, m->capacity, D, position, m->n_kv, D, 1, base_log2, 1);
        if (!rc) rc = so_kv_cache_update(m->v_cache[l], v, m->capacity, D, position, m->n_kv);
        if (!rc) rc = so_attention_decode(q, m->k_cache[l], m->v_cache[l], m->n_q, m->n_kv, D, m->capacity,
                                          position + 1, scale, 0, attn);
        if (!rc) rc = so_affine_matvec(L->o.w, L->o.s, L->o.b, attn, H, qd, G, 1, tmp);
        if (!rc) so_elementwise_add(h, tmp, H, h);
        if (!rc) rc = so_rms_norm_1pw(h, L->post_norm, H, m->eps, 1, normed);
        if (!rc) rc = so_affine_gate_up_swiglu(L->gate.w, L->gate.s, L->gate.b, L->up.w, L->up.s, L->up.b,
                                               normed, I, H, G, 1, 0, act);
        if (!rc) rc = so_affine_matvec(L->down.w, L->down.s, L->down.b, act, H, I, G, 1, tmp);
        if (!rc) so_elementwise_add(h, tmp, H, h);
    }
    if (!rc) rc = so_rms_norm_1pw(h, m->final_norm, H, m->eps, 1, normed);
    if (!rc) rc = so_fp16_matvec(m->lm_head, normed, m->vocab, H, 1, logits);
    if (!rc && out_token) *out_token = so_argmax_f16(logits, m->vocab);
    free(buf);
    if (!logits_out) free(logits);
    return rc;
}

/* A prompt through the model `chunk` positions at a time, every layer over the whole chunk before the next layer,
 * as a prefill table runs it.  For attention layers this equals token-by-token decoding (each position sees the
 * cache rows before it); a DeltaNet layer takes the prompt-chunk kernels, whose recurrent rows stay in fp32 across
 * the chunk and are rounded to fp16 at its end (prefill_recurrence.metal:318-321), so the chunking is part of the
 * result.  Writes the logits of the last position and its greedy token. */
SO_API int so_conv1d_update_silu_prefill(uint16_t *state, uint16_t *qkv, const uint16_t *weight, int seq_len, int channels, int kernel_size, uint16_t *history);
SO_API int so_deltanet_recurrence_prefill(uint16_t *state, const uint16_t *qkv, const uint16_t *b_proj, const uint16_t *a_proj, const uint16_t *a_log,
                                          const uint16_t *dt_bias, uint16_t *out, int head_dim, int value_heads, int qk_heads, int seq_len, uint16_t *history);
SO_API int so_model_prefill(so_model_t *m, const int32_t *tokens, int n_tokens, int start_pos, int chunk, uint16_t *logits_out, int32_t *out_token) {
    if (n_tokens <= 0 || start_pos < 0 || start_pos + n_tokens > m->capacity || chunk <= 0) return SO_ERR_GEOMETRY;
    const int H = m->hidden, I = m->inter, D = m->head_dim, qd = m->n_q * D, kvd = m->n_kv * D, G = m->group;
    const int DD = m->d_head_dim, Hv = m->d_value_heads, Hqk = m->d_qk_heads;
    const int dq = (2 * Hqk + Hv) * DD, dv = Hv * DD;
    const size_t T = (size_t)(chunk < n_tokens ? chunk : n_tokens);
    const size_t per = (size_t)H * 3 + qd * 2 + kvd * 2 + I + (size_t)dq + 2 * (size_t)dv + 2 * (size_t)Hv;
    uint16_t *buf = (uint16_t *)malloc(per * T * 2);
    uint16_t *logits = logits_out ? logits_out : (uint16_t *)malloc((size_t)m->vocab * 2);
    if (!buf || !logits) { free(buf); if (!logits_out) free(logits); return SO_ERR_ALLOC; }
    uint16_t *hs = buf, *normed = hs + T * H, *tmp = normed + T * H, *q = tmp + T * H, *attn = q + T * qd, *k = attn + T * qd, *v = k + T * kvd,
             *act = v + T * kvd, *dqkv = act + T * I, *dz = dqkv + T * dq, *dout = dz + T * dv, *da = dout + T * dv, *db = da + T * Hv;
    const float base_log2 = log2f(m->rope_theta), scale = 1.0f / sqrtf((float)D);
    int rc = SO_OK;
    for (int t0 = 0; t0 < n_tokens && !rc; t0 += chunk) {
        const int n = n_tokens - t0 < chunk ? n_tokens - t0 : chunk, p0 = start_pos + t0;
        for (int t = 0; t < n; ++t) {
            if (tokens[t0 + t] < 0 || tokens[t0 + t] >= m->vocab) { rc = SO_ERR_GEOMETRY; break; }
            so_embedding_gather(m->embedding, tokens[t0 + t], H, hs + (size_t)t * H);
        }
        for (int l = 0; l < m->layers && !rc; ++l) {
            so_layer_t *L = &m->layer[l];
            for (int t = 0; t < n && !rc; ++t) rc = so_rms_norm_1pw(hs + (size_t)t * H, L->input_norm, H, m->eps, 1, normed + (size_t)t * H);
            if (!rc && L->kind == 1) {
                rc = so_affine_matvec(L->dqkv.w, L->dqkv.s, L->dqkv.b, normed, dq, H, G, n, dqkv);
                if (!rc) rc = so_affine_matvec(L->dz.w, L->dz.s, L->dz.b, normed, dv, H, G, n, dz);
                if (!rc) rc = so_affine_matvec(L->da.w, L->da.s, L->da.b, normed, Hv, H, G, n, da);
                if (!rc) rc = so_affine_matvec(L->db.w, L->db.s, L->db.b, normed, Hv, H, G, n, db);
                if (!rc) rc = so_conv1d_update_silu_prefill(L->conv_state, dqkv, L->conv_w, n, dq, m->d_conv_kernel, NULL);
                if (!rc) rc = so_rms_scale_qk(dqkv, DD, 1e-6f, dq, Hqk, n);
                if (!rc) rc = so_deltanet_recurrence_prefill(L->rec_state, dqkv, db, da, L->a_log, L->dt_bias, dout, DD, Hv, Hqk, n, NULL);
                if (!rc) rc = (DD == 128 && m->eps == 1e-6f) ? so_rms_norm_gated_d128(dout, dz, L->gnorm_w, dout, n * Hv)
                                                             : so_rms_norm_gated_tg(dout, dz, L->gnorm_w, dout, DD, m->eps, n * Hv, DD < 256 ? DD : 256);
                if (!rc) rc = so_affine_matvec(L->dout.w, L->dout.s, L->dout.b, dout, H, dv, G, n, tmp);
            } else if (!rc) {
                rc = so_affine_matvec(L->q.w, L->q.s, L->q.b, normed, qd, H, G, n, q);
                if (!rc) rc = so_affine_matvec(L->k.w, L->k.s, L->k.b, normed, kvd, H, G, n, k);
                if (!rc) rc = so_affine_matvec(L->v.w, L->v.s, L->v.b, normed, kvd, H, G, n, v);
                for (int t = 0; t < n && !rc; ++t) {
                    rc = so_apply_rope(q + (size_t)t * qd, NULL, NULL, D, D, m->n_q, 1, (uint32_t)(p0 + t), base_log2, 1);
                    if (!rc) rc = so_rope_kv_cache_update(m->k_cache[l], k + (size_t)t * kvd, NULL, NULL, m->capacity, D, p0 + t, m->n_kv, D, 1, base_log2, 1);
                    if (!rc) rc = so_kv_cache_update(m->v_cache[l], v + (size_t)t * kvd, m->capacity, D, p0 + t, m->n_kv);
                    if (!rc) rc = so_attention_decode(q + (size_t)t * qd, m->k_cache[l], m->v_cache[l], m->n_q, m->n_kv, D, m->capacity, p0 + t + 1, scale, 0,
                                                      attn + (size_t)t * qd);
                }
                if (!rc) rc = so_affine_matvec(L->o.w, L->o.s, L->o.b, attn, H, qd, G, n, tmp);
            }
            if (!rc) so_elementwise_add(hs, tmp, (int64_t)n * H, hs);
            for (int t = 0; t < n && !rc; ++t) rc = so_rms_norm_1pw(hs + (size_t)t * H, L->post_norm, H, m->eps, 1, normed + (size_t)t * H);
            if (!rc) rc = so_affine_gate_up_swiglu(L->gate.w, L->gate.s, L->gate.b, L->up.w, L->up.s, L->up.b, normed, I, H, G, n, 0, act);
            if (!rc) rc = so_affine_matvec(L->down.w, L->down.s, L->down.b, act, H, I, G, n, tmp);
            if (!rc) so_elementwise_add(hs, tmp, (int64_t)n * H, hs);
        }
        if (!rc && t0 + n >= n_tokens) {
            rc = so_rms_norm_1pw(hs + (size_t)(n - 1) * H, m->final_norm, H, m->eps, 1, normed);
            if (!rc) rc = so_fp16_matvec(m->lm_head, normed, m->vocab, H, 1, logits);
            if (!rc && out_token) *out_token = so_argmax_f16(logits, m->vocab);
        }
    }
    free(buf);
    if (!logits_out) free(logits);
    return rc;
}

/* Greedy generation: feed the prompt token by token (the reference does the same when a
 * package has no prefill table, Sources/SmeltRuntime/SmeltModel.swift:619-631), then
 * n_decode greedy steps.  out_tokens receives n_decode ids; margins (optional, n_decode
 * floats) receives top1-top2 logit gaps. */
SO_API int so_model_generate(so_model_t *m, const int32_t *prompt, int n_prompt, int n_decode,
                             int32_t *out_tokens, float *margins) {
    if (n_prompt <= 0 || n_prompt + n_decode > m->capacity) return SO_ERR_GEOMETRY;
    uint16_t *logits = (uint16_t *)malloc((size_t)m->vocab * 2);
    if (!logits) return SO_ERR_ALLOC;
    so_model_reset_cache(m);
    int32_t cur = -1;
    int rc = SO_OK, pos = 0;
    for (int i = 0; i < n_prompt && !rc; ++i, ++pos) rc = so_model_decode_step(m, prompt[i], pos, logits, &cur);
    for (int i = 0; i < n_decode && !rc; ++i, ++pos) {
        out_tokens[i] = cur;
        if (margins) {
            float best = -INFINITY, second = -INFINITY;
            for (int t = 0; t < m->vocab; ++t) {
                float v = h2f(logits[t]);
                if (v > best) { second = best; best = v; } else if (v > second) second = v;
            }
            margins[i] = best - second;
        }
        if (i + 1 < n_decode) rc = so_model_decode_step(m, cur, pos, logits, &cur);
    }
    free(logits);
    return rc;
}

/* ───────────────────── DeltaNet decode step (hybrid linear-attention layers) ─────────────────────
 * No scalar Swift oracle exists for these kernels beyond the float references inside the
 * reference's tests (PrefillKernelTests.swift:583-609, :4400-4441); the functions below restate
 * the Metal kernels' own arithmetic, including their staged fp16 roundings. */

/* smelt_silu_staged_half (Resources/Shaders/conv1d.metal:4-15): every intermediate an fp16
 * value; a result of either zero is +0. */
static inline uint16_t silu_staged_half(uint16_t xh) {
    float x = h2f(xh);
    float e = round_h(expf(fabsf(x)));
    float tail = round_h(1.0f / round_h(1.0f + e));
    float sig = x < 0.0f ? tail : round_h(1.0f - tail);
    uint16_t r = f2h(x * sig);
    return (r & 0x7fffu) == 0u ? (uint16_t)0 : r;
}

/* conv1d_update_silu (conv1d.metal:271-331): per channel, state [C, K] shifts left by one and
 * takes the new value; out = silu_staged(half(sum_k state[k] * weight[k])), taps added one at a
 * time from a float zero (conv1d.metal:20-27).  state is updated in place. */
SO_API int so_conv1d_update_silu(uint16_t *state, const uint16_t *new_val, const uint16_t *weight, uint16_t *out,
                                 int channels, int kernel_size) {
    if (channels <= 0 || kernel_size <= 0 || kernel_size > 8) return SO_ERR_GEOMETRY;
    for (int ch = 0; ch < channels; ++ch) {
        uint16_t *st = state + (size_t)ch * kernel_size;
        const uint16_t *w = weight + (size_t)ch * kernel_size;
        for (int k = 0; k + 1 < kernel_size; ++k) st[k] = st[k + 1];
        st[kernel_size - 1] = new_val[ch];
        float acc = 0.0f;
        for (int k = 0; k < kernel_size; ++k) acc += h2f(st[k]) * h2f(w[k]);
        out[ch] = silu_staged_half(f2h(acc));
    }
    return SO_OK;
}

/* rms_scale_qk (Resources/Shaders/norms.metal:1380-1431): for each of the qk_heads Q heads and
 * qk_heads K heads at the front of qkv [batch, qkv_dim]: x <- half(half(x * rsqrt(mean(x^2) +
 * eps)) * edge), edge = half(1 / head_dim) for Q, half(rsqrt(head_dim)) for K.  In place. */
SO_API int so_rms_scale_qk(uint16_t *qkv, int head_dim, float eps, int qkv_dim, int qk_heads, int batch) {
    if (head_dim <= 0 || head_dim > 512 || qk_heads <= 0 || 2 * qk_heads * head_dim > qkv_dim || batch <= 0) return SO_ERR_GEOMETRY;
    for (int b = 0; b < batch; ++b)
        for (int g = 0; g < 2 * qk_heads; ++g) {
            const int is_k = g >= qk_heads;
            uint16_t *x = qkv + (size_t)b * qkv_dim + (size_t)g * head_dim; /* K region follows the Q region */
            float sum = 0.0f;
            for (int i = 0; i < head_dim; ++i) sum += h2f(x[i]) * h2f(x[i]);
            const float scale = 1.0f / sqrtf(sum / (float)head_dim + eps);
            const float edge = is_k ? round_h(1.0f / sqrtf((float)head_dim)) : round_h(1.0f / (float)head_dim);
            for (int i = 0; i < head_dim; ++i) x[i] = f2h(round_h(h2f(x[i]) * scale) * edge);
        }
    return SO_OK;
}

/* smelt_decode_sigmoid_staged_half / smelt_decode_softplus_staged_half
 * (Resources/Shaders/recurrence.metal:4-21). */
static inline float sigmoid_staged_half(uint16_t xh) {
    float x = h2f(xh);
    float tail = round_h(1.0f / round_h(1.0f + round_h(expf(fabsf(x)))));
    return x < 0.0f ? tail : round_h(1.0f - tail);
}
static inline float decode_log1p(float x) {
    const float xp1 = 1.0f + x;
    if (xp1 == 1.0f) return x;
    return x * (logf(xp1) / (xp1 - 1.0f));
}
static inline float softplus_staged_half(uint16_t xh) {
    float x = h2f(xh);
    float mx = x > 0.0f ? x : 0.0f, mn = x < 0.0f ? x : 0.0f;
    return round_h(mx + decode_log1p(round_h(expf(round_h(mn - mx)))));
}

/* deltanet_recurrence_mlx_decode (recurrence.metal:511-588): per value head h and output row dv,
 * state row [Dk] *= decay; kv = state . k; delta = (v[dv] - kv) * beta; state += k * delta;
 * out = state . q; state written back as fp16.  beta = sigmoid_staged(b[h]); decay =
 * half(exp(-exp(a_log[h]) * softplus_staged(half(a[h] + dt_bias[h])))).  q / k heads are shared
 * by value_heads / qk_heads value heads; qkv = [q (Hqk, D) | k (Hqk, D) | v (Hv, D)].  The lane
 * partition of the Metal kernel (lane l holds dk = l * D/32 ...) fixes the summation order:
 * per-lane partial sums in dk order, then the 32 lane sums added pairwise as simd_sum does
 * (butterfly over lane distance 16, 8, 4, 2, 1). */
SO_API int so_deltanet_recurrence_decode(uint16_t *state, const uint16_t *qkv, const uint16_t *b_proj, const uint16_t *a_proj,
                                         const uint16_t *a_log, const uint16_t *dt_bias, uint16_t *out, int head_dim,
                                         int value_heads, int qk_heads) {
    if (head_dim <= 0 || head_dim % 32 || head_dim > 256 || qk_heads <= 0 || value_heads <= 0 || value_heads % qk_heads) return SO_ERR_GEOMETRY;
    const int D = head_dim, epl = D / 32, rep = value_heads / qk_heads;
    for (int h = 0; h < value_heads; ++h) {
        const int qh = h / rep;
        const uint16_t *q = qkv + (size_t)qh * D, *k = qkv + (size_t)(qk_heads + qh) * D, *v = qkv + (size_t)2 * qk_heads * D + (size_t)h * D;
        const float beta = sigmoid_staged_half(b_proj[h]);
        const uint16_t xh = f2h(h2f(a_proj[h]) + h2f(dt_bias[h]));
        const float decay = round_h(expf(-expf(h2f(a_log[h])) * softplus_staged_half(xh)));
        for (int dv = 0; dv < D; ++dv) {
            uint16_t *row = state + ((size_t)h * D + dv) * D;
            float st[256], lane[32];
            for (int l = 0; l < 32; ++l) {
                float p = 0.0f;
                for (int i = 0; i < epl; ++i) {
                    const int dk = l * epl + i;
                    st[dk] = h2f(row[dk]) * decay;
                    p += st[dk] * h2f(k[dk]);
                }
                lane[l] = p;
            }
            const float kv = simd_sum32(lane);
            const float delta = (h2f(v[dv]) - kv) * beta;
            for (int l = 0; l < 32; ++l) {
                float p = 0.0f;
                for (int i = 0; i < epl; ++i) {
                    const int dk = l * epl + i;
                    st[dk] += h2f(k[dk]) * delta;
                    p += st[dk] * h2f(q[dk]);
                }
                lane[l] = p;
            }
            out[(size_t)h * D + dv] = f2h(simd_sum32(lane));
            for (int dk = 0; dk < D; ++dk) row[dk] = f2h(st[dk]);
        }
    }
    return SO_OK;
}

/* conv1d_update_silu_prefill, conv1d_update_silu_c6144_k4_prefill and
 * conv1d_update_silu_prefill_checkpoint (conv1d.metal:129-268): one channel walks the prompt
 * chunk qkv [T, C] in place, keeping its taps in registers; state [C, K] is written once at the
 * end.  The taps are fp16 values throughout, their products with the fp16 weights are exact in
 * fp32, so the fused multiply-adds of the specialisation and the roundings of the checkpoint
 * variant change nothing: every variant equals T calls of so_conv1d_update_silu.  history (may
 * be NULL) [T + 1, C, K] receives the entry state and the state after every token. */
SO_API int so_conv1d_update_silu_prefill(uint16_t *state, uint16_t *qkv, const uint16_t *weight, int seq_len, int channels,
                                         int kernel_size, uint16_t *history) {
    if (channels <= 0 || kernel_size <= 0 || kernel_size > 8 || seq_len < 0) return SO_ERR_GEOMETRY;
    const size_t hs = (size_t)channels * kernel_size;
    for (int ch = 0; ch < channels; ++ch) {
        uint16_t *st = state + (size_t)ch * kernel_size;
        const uint16_t *w = weight + (size_t)ch * kernel_size;
        if (history) for (int k = 0; k < kernel_size; ++k) history[(size_t)ch * kernel_size + k] = st[k];
        for (int pos = 0; pos < seq_len; ++pos) {
            uint16_t *x = qkv + (size_t)pos * channels + ch;
            for (int k = 0; k + 1 < kernel_size; ++k) st[k] = st[k + 1];
            st[kernel_size - 1] = *x;
            float acc = 0.0f;
            for (int k = 0; k < kernel_size; ++k) acc += h2f(st[k]) * h2f(w[k]);
            *x = silu_staged_half(f2h(acc));
            if (history) for (int k = 0; k < kernel_size; ++k) history[(size_t)(pos + 1) * hs + (size_t)ch * kernel_size + k] = st[k];
        }
    }
    return SO_OK;
}

/* deltanet_recurrence_mlx_prefill and its _d128_h16 / _d128_h32_qk16 / _d128_h48_qk16
 * specialisations (Resources/Shaders/prefill_recurrence.metal:290-673): the decode step's
 * arithmetic over the T positions of qkv [T, (2 Hqk + Hv) D], b_proj / a_proj [T, Hv], with the
 * recurrent row held in fp32 across the whole chunk and rounded to fp16 only when it is
 * written back at the end ("keeps the recurrent state in FP32 registers across the entire
 * chunk", :318-321).  out [T, Hv, D].  With history != NULL it is
 * deltanet_recurrence_mlx_prefill_checkpoint (:675-775): history [T + 1, Hv, D, D] receives the
 * entry state and the fp16 state after every token, and the live row continues from that
 * rounded value, which makes the chunk equal to T decode steps. */
SO_API int so_deltanet_recurrence_prefill(uint16_t *state, const uint16_t *qkv, const uint16_t *b_proj, const uint16_t *a_proj,
                                          const uint16_t *a_log, const uint16_t *dt_bias, uint16_t *out, int head_dim,
                                          int value_heads, int qk_heads, int seq_len, uint16_t *history) {
    if (head_dim <= 0 || head_dim % 32 || head_dim > 256 || qk_heads <= 0 || value_heads <= 0 || value_heads % qk_heads || seq_len < 0)
        return SO_ERR_GEOMETRY;
    const int D = head_dim, epl = D / 32, rep = value_heads / qk_heads;
    const size_t stride = (size_t)(2 * qk_heads + value_heads) * D, hs = (size_t)value_heads * D * D;
    for (int h = 0; h < value_heads; ++h) {
        const int qh = h / rep;
        for (int dv = 0; dv < D; ++dv) {
            uint16_t *row = state + ((size_t)h * D + dv) * D;
            const size_t row_off = ((size_t)h * D + dv) * D;
            float st[256], lane[32];
            for (int dk = 0; dk < D; ++dk) st[dk] = h2f(row[dk]);
            if (history) for (int dk = 0; dk < D; ++dk) history[row_off + dk] = row[dk];
            for (int pos = 0; pos < seq_len; ++pos) {
                const uint16_t *x = qkv + (size_t)pos * stride;
                const uint16_t *q = x + (size_t)qh * D, *k = x + (size_t)(qk_heads + qh) * D, *v = x + (size_t)2 * qk_heads * D + (size_t)h * D;
                const float beta = sigmoid_staged_half(b_proj[(size_t)pos * value_heads + h]);
                const uint16_t xh = f2h(h2f(a_proj[(size_t)pos * value_heads + h]) + h2f(dt_bias[h]));
                const float decay = round_h(expf(-expf(h2f(a_log[h])) * softplus_staged_half(xh)));
                for (int l = 0; l < 32; ++l) {
                    float p = 0.0f;
                    for (int i = 0; i < epl; ++i) {
                        const int dk = l * epl + i;
                        st[dk] = st[dk] * decay;
                        p += st[dk] * h2f(k[dk]);
                    }
                    lane[l] = p;
                }
                const float kv = simd_sum32(lane);
                const float delta = (h2f(v[dv]) - kv) * beta;
                for (int l = 0; l < 32; ++l) {
                    float p = 0.0f;
                    for (int i = 0; i < epl; ++i) {
                        const int dk = l * epl + i;
                        st[dk] += h2f(k[dk]) * delta;
                        p += st[dk] * h2f(q[dk]);
                    }
                    lane[l] = p;
                }
                out[((size_t)pos * value_heads + h) * D + dv] = f2h(simd_sum32(lane));
                if (history)
                    for (int dk = 0; dk < D; ++dk) {
                        const uint16_t r = f2h(st[dk]);
                        history[(size_t)(pos + 1) * hs + row_off + dk] = r;
                        st[dk] = h2f(r);
                    }
            }
            for (int dk = 0; dk < D; ++dk) row[dk] = f2h(st[dk]);
        }
    }
    return SO_OK;
}

/* ── The DeltaNet step as separate launches (Resources/Shaders/recurrence.metal:44-302, :836-862) ──
 * The reference's kernel catalog still lists these pipelines (SmeltKernelCatalog.swift:655-696,
 * :847-893) although its emitters now dispatch the tiled forms above.  State here is
 * [H, Dk, Dv]: state[k * D + v].  The gates are plain fp32 (no staged roundings) and the sums
 * over k run one term at a time in k order.  The reference holds no test or scalar oracle for
 * them: parity unpinned beyond this restatement of the kernels' arithmetic. */
static inline void plain_gates(uint16_t b, uint16_t a, uint16_t a_log, uint16_t dt_bias, float *beta, float *g) {
    *beta = 1.0f / (1.0f + expf(-h2f(b)));
    const float x = h2f(a) + h2f(dt_bias);
    const float sp = x > 20.0f ? x : logf(1.0f + expf(x));
    *g = -expf(h2f(a_log)) * sp;
}

/* compute_gates (recurrence.metal:839-862): beta = half(sigmoid(b)), g = half(-exp(A_log) softplus(a + dt_bias)). */
SO_API int so_dn_compute_gates(const uint16_t *b_proj, const uint16_t *a_proj, const uint16_t *a_log, const uint16_t *dt_bias,
                               uint16_t *beta_out, uint16_t *g_out, int heads) {
    if (heads <= 0) return SO_ERR_GEOMETRY;
    for (int h = 0; h < heads; ++h) {
        float beta, g;
        plain_gates(b_proj[h], a_proj[h], a_log[h], dt_bias[h], &beta, &g);
        beta_out[h] = f2h(beta);
        g_out[h] = f2h(g);
    }
    return SO_OK;
}

/* state_decay (:48-63): state <- half(state * exp(g[h])). */
SO_API int so_dn_state_decay(uint16_t *state, const uint16_t *g_val, int head_dim, int heads) {
    if (head_dim <= 0 || heads <= 0) return SO_ERR_GEOMETRY;
    const size_t n = (size_t)head_dim * head_dim;
    for (int h = 0; h < heads; ++h) {
        const float decay = expf(h2f(g_val[h]));
        for (size_t i = 0; i < n; ++i) state[h * n + i] = f2h(h2f(state[h * n + i]) * decay);
    }
    return SO_OK;
}

/* kv_mem_readout (:70-90): kv_mem[h, v] = sum_k state[h, k, v] * key[h, k], fp32 out. */
SO_API int so_dn_kv_mem_readout(const uint16_t *state, const uint16_t *key, float *kv_mem, int head_dim, int heads) {
    if (head_dim <= 0 || heads <= 0) return SO_ERR_GEOMETRY;
    const int D = head_dim;
    for (int h = 0; h < heads; ++h)
        for (int v = 0; v < D; ++v) {
            float acc = 0.0f;
            for (int k = 0; k < D; ++k) acc += h2f(state[((size_t)h * D + k) * D + v]) * h2f(key[(size_t)h * D + k]);
            kv_mem[(size_t)h * D + v] = acc;
        }
    return SO_OK;
}

/* compute_delta (:95-108): delta = (value - kv_mem) * beta[h], fp32 out. */
SO_API int so_dn_compute_delta(const uint16_t *value, const float *kv_mem, const uint16_t *beta, float *delta, int head_dim, int heads) {
    if (head_dim <= 0 || heads <= 0) return SO_ERR_GEOMETRY;
    for (int i = 0; i < heads * head_dim; ++i) delta[i] = (h2f(value[i]) - kv_mem[i]) * h2f(beta[i / head_dim]);
    return SO_OK;
}

/* outer_product_update (:113-142) and, with g_val != NULL, state_decay_update (:246-276):
 * state[h, k, v] <- half(state (* exp(g[h])) + key[h, k] * delta[h, v]). */
SO_API int so_dn_outer_product_update(uint16_t *state, const uint16_t *g_val, const uint16_t *key, const float *delta, int head_dim, int heads) {
    if (head_dim <= 0 || heads <= 0) return SO_ERR_GEOMETRY;
    const int D = head_dim;
    for (int h = 0; h < heads; ++h) {
        const float decay = g_val ? expf(h2f(g_val[h])) : 1.0f;
        for (int k = 0; k < D; ++k)
            for (int v = 0; v < D; ++v) {
                uint16_t *s = state + ((size_t)h * D + k) * D + v;
                const float old = h2f(*s);
                const float upd = h2f(key[(size_t)h * D + k]) * delta[(size_t)h * D + v];
                *s = f2h(g_val ? old * decay + upd : old + upd);
            }
    }
    return SO_OK;
}

/* kv_readout_delta (:150-178) and, with b_proj != NULL, gates_kv_readout_delta (:186-239): the
 * readout of the un-decayed state times exp(g), then delta = (value - kv_mem) * beta.  The first
 * takes g and beta as fp16 inputs (g_val, beta); the second computes both in fp32 from b_proj,
 * a_proj, a_log, dt_bias and writes g_out[h] = half(g). */
SO_API int so_dn_kv_readout_delta(const uint16_t *state, const uint16_t *key, const uint16_t *value, const uint16_t *g_val,
                                  const uint16_t *beta_in, const uint16_t *b_proj, const uint16_t *a_proj, const uint16_t *a_log,
                                  const uint16_t *dt_bias, float *delta, uint16_t *g_out, int head_dim, int heads) {
    if (head_dim <= 0 || heads <= 0) return SO_ERR_GEOMETRY;
    const int D = head_dim;
    for (int h = 0; h < heads; ++h) {
        float decay, beta;
        if (b_proj) {
            float g;
            plain_gates(b_proj[h], a_proj[h], a_log[h], dt_bias[h], &beta, &g);
            decay = expf(g);
            g_out[h] = f2h(g);
        } else {
            decay = expf(h2f(g_val[h]));
            beta = h2f(beta_in[h]);
        }
        for (int v = 0; v < D; ++v) {
            float acc = 0.0f;
            for (int k = 0; k < D; ++k) acc += h2f(state[((size_t)h * D + k) * D + v]) * h2f(key[(size_t)h * D + k]);
            const float kv_mem = acc * decay;
            delta[(size_t)h * D + v] = (h2f(value[(size_t)h * D + v]) - kv_mem) * beta;
        }
    }
    return SO_OK;
}

/* query_readout (:282-302): out[h, v] = half(sum_k state[h, k, v] * (query[h, k] * scale)). */
SO_API int so_dn_query_readout(const uint16_t *state, const uint16_t *query, uint16_t *out, int head_dim, float scale, int heads) {
    if (head_dim <= 0 || heads <= 0) return SO_ERR_GEOMETRY;
    const int D = head_dim;
    for (int h = 0; h < heads; ++h)
        for (int v = 0; v < D; ++v) {
            float acc = 0.0f;
            for (int k = 0; k < D; ++k) {
                const float q = h2f(query[(size_t)h * D + k]) * scale;
                acc += h2f(state[((size_t)h * D + k) * D + v]) * q;
            }
            out[(size_t)h * D + v] = f2h(acc);
        }
    return SO_OK;
}

/* Sum of x[i]^2 over a head as a threadgroup of tgs threads forms it in these kernels: thread t
 * adds its elements t, t + tgs, ...; every simdgroup sums its 32 lanes (simd_sum); thread 0 adds
 * the simdgroups' sums one after the other. */
static float tg_sumsq(const float *x, int n, int tgs) {
    float total = 0.0f;
    for (int s = 0; s < tgs / 32; ++s) {
        float lane[32];
        for (int l = 0; l < 32; ++l) {
            float p = 0.0f;
            for (int i = s * 32 + l; i < n; i += tgs) p += x[i] * x[i];
            lane[l] = p;
        }
        total += simd_sum32(lane);
    }
    return total;
}

/* deltanet_recurrence_fused (recurrence.metal:310-503): one threadgroup of tgs threads per head
 * runs conv1d + SiLU (plain fp32, no fp16 staging) on the head's Q, K and V channels, L2-
 * normalises Q (times head_scale) and K, computes the gates in fp32, runs the recurrence on the
 * [H, Dv, Dk] state with lane l of a simdgroup holding dk = l, l + 32, ..., and applies the
 * gated RMS norm.  qkv = [Q (H, D) | K (H, D) | V (H, D)]; conv_state / conv_weight
 * [qkv_dim, conv_k]; z [H, D]; norm_weight [D]; out [H, D]. */
SO_API int so_deltanet_recurrence_fused(uint16_t *state, const uint16_t *qkv, const uint16_t *b_proj, const uint16_t *a_proj,
                                        const uint16_t *a_log, const uint16_t *dt_bias, uint16_t *out, uint16_t *conv_state,
                                        const uint16_t *conv_weight, const uint16_t *z_proj, const uint16_t *norm_weight, int head_dim,
                                        float head_scale, int qkv_dim, int conv_k, int heads, float rms_eps, int tgs) {
    if (head_dim <= 0 || head_dim % 32 || head_dim > 256 || heads <= 0 || conv_k <= 0 || conv_k > 8 || qkv_dim < 3 * heads * head_dim ||
        tgs <= 0 || tgs % 32 || tgs > 1024)
        return SO_ERR_GEOMETRY;
    const int D = head_dim, epl = D / 32;
    for (int h = 0; h < heads; ++h) {
        float q[256], k[256], v[256], raw[256];
        for (int i = 0; i < 3 * D; ++i) {
            const int part = i / D, local = i % D;
            const int ch = part * heads * D + h * D + local;
            uint16_t *st = conv_state + (size_t)ch * conv_k;
            const uint16_t *w = conv_weight + (size_t)ch * conv_k;
            for (int t = 0; t + 1 < conv_k; ++t) st[t] = st[t + 1];
            st[conv_k - 1] = qkv[ch];
            float acc = 0.0f;
            for (int t = 0; t < conv_k; ++t) acc += h2f(st[t]) * h2f(w[t]);
            const float act = acc / (1.0f + expf(-acc));
            (part == 0 ? q : part == 1 ? k : v)[local] = act;
        }
        const float q_scale = 1.0f / fmaxf(sqrtf(tg_sumsq(q, D, tgs)), 1e-6f);
        const float k_scale = 1.0f / fmaxf(sqrtf(tg_sumsq(k, D, tgs)), 1e-6f);
        float beta, g;
        plain_gates(b_proj[h], a_proj[h], a_log[h], dt_bias[h], &beta, &g);
        const float decay = expf(g);
        for (int i = 0; i < D; ++i) {
            q[i] *= q_scale * head_scale;
            k[i] *= k_scale;
        }
        for (int row = 0; row < D; ++row) {
            uint16_t *srow = state + ((size_t)h * D + row) * D;
            float st[256], lane[32];
            for (int l = 0; l < 32; ++l) {
                float p = 0.0f;
                for (int i = 0; i < epl; ++i) {
                    const int dk = i * 32 + l;
                    st[dk] = h2f(srow[dk]) * decay;
                    p += st[dk] * k[dk];
                }
                lane[l] = p;
            }
            const float kv_mem = simd_sum32(lane);
            const float delta = (v[row] - kv_mem) * beta;
            for (int l = 0; l < 32; ++l) {
                float p = 0.0f;
                for (int i = 0; i < epl; ++i) {
                    const int dk = i * 32 + l;
                    st[dk] += k[dk] * delta;
                    p += st[dk] * q[dk];
                    srow[dk] = f2h(st[dk]);
                }
                lane[l] = p;
            }
            raw[row] = simd_sum32(lane);
        }
        const float rs = 1.0f / sqrtf(tg_sumsq(raw, D, tgs) / (float)D + rms_eps);
        for (int i = 0; i < D; ++i) {
            const float z = h2f(z_proj[(size_t)h * D + i]);
            const float silu_z = z / (1.0f + expf(-z));
            out[(size_t)h * D + i] = f2h(raw[i] * rs * h2f(norm_weight[i]) * silu_z);
        }
    }
    return SO_OK;
}

/* deltanet_recurrence_prefill (Resources/Shaders/prefill_recurrence.metal:42-285): one threadgroup
 * of tgs threads per head walks the T positions of qkv [T, qkv_dim] = [Q | K | V] (H heads each):
 * conv1d + SiLU on the head's channels (written back as fp16), L2 norm of Q and of K in place
 * (scale = 1 / max(norm, l2_eps)), gates in fp32, then on the [H, Dv, Dk] state: decay (rounded
 * to fp16), kv_mem[v] = sum_k state[v, k] key[k], delta = (value - kv_mem) beta, state <-
 * half(state + delta[v] key[k]), out[v] = half(sum_k state[v, k] (q[k] head_scale)).  b / a
 * [T, H]; out [T, H, D]; conv_state [qkv_dim, conv_k] in place. */
SO_API int so_deltanet_recurrence_prefill_fused(uint16_t *state, uint16_t *conv_state, uint16_t *qkv, const uint16_t *conv_weight,
                                                const uint16_t *a_log, const uint16_t *dt_bias, const uint16_t *b_buf,
                                                const uint16_t *a_buf, uint16_t *out, int head_dim, int heads, int seq_len, int qkv_dim,
                                                int conv_k, float head_scale, float l2_eps, int tgs) {
    if (head_dim <= 0 || head_dim > 256 || heads <= 0 || conv_k <= 0 || conv_k > 8 || qkv_dim < 3 * heads * head_dim || seq_len < 0 ||
        tgs <= 0 || tgs % 32 || tgs > 1024)
        return SO_ERR_GEOMETRY;
    const int D = head_dim, HD = heads * head_dim;
    for (int h = 0; h < heads; ++h) {
        uint16_t *S = state + (size_t)h * D * D;
        for (int pos = 0; pos < seq_len; ++pos) {
            uint16_t *x = qkv + (size_t)pos * qkv_dim;
            for (int i = 0; i < 3 * D; ++i) {
                const int ch = (i / D) * HD + h * D + i % D;
                uint16_t *st = conv_state + (size_t)ch * conv_k;
                const uint16_t *w = conv_weight + (size_t)ch * conv_k;
                for (int t = 0; t + 1 < conv_k; ++t) st[t] = st[t + 1];
                st[conv_k - 1] = x[ch];
                float acc = 0.0f;
                for (int t = 0; t < conv_k; ++t) acc += h2f(st[t]) * h2f(w[t]);
                x[ch] = f2h(acc / (1.0f + expf(-acc)));
            }
            for (int part = 0; part < 2; ++part) {
                uint16_t *p = x + part * HD + h * D;
                float f[256];
                for (int i = 0; i < D; ++i) f[i] = h2f(p[i]);
                const float scale = 1.0f / fmaxf(sqrtf(tg_sumsq(f, D, tgs)), l2_eps);
                for (int i = 0; i < D; ++i) p[i] = f2h(f[i] * scale);
            }
            const uint16_t *q = x + h * D, *k = x + HD + h * D, *v = x + 2 * HD + h * D;
            float beta, g;
            plain_gates(b_buf[(size_t)pos * heads + h], a_buf[(size_t)pos * heads + h], a_log[h], dt_bias[h], &beta, &g);
            const float decay = expf(g);
            for (int vi = 0; vi < D; ++vi) {
                uint16_t *row = S + (size_t)vi * D;
                float acc = 0.0f;
                for (int kk = 0; kk < D; ++kk) {
                    row[kk] = f2h(h2f(row[kk]) * decay);
                    acc += h2f(row[kk]) * h2f(k[kk]);
                }
                const float delta = (h2f(v[vi]) - acc) * beta;
                float o = 0.0f;
                for (int kk = 0; kk < D; ++kk) {
                    row[kk] = f2h(h2f(row[kk]) + delta * h2f(k[kk]));
                    o += h2f(row[kk]) * (h2f(q[kk]) * head_scale);
                }
                out[((size_t)pos * heads + h) * D + vi] = f2h(o);
            }
        }
    }
    return SO_OK;
}

/* rms_norm_gated (norms.metal:1093-1143): per head, out = half(w * (x * rsqrt(mean(x^2) + eps)) *
 * silu(g)), silu(g) = g / (1 + exp(-g)) in fp32; weight [D] shared by the heads. */
SO_API int so_rms_norm_gated(const uint16_t *input, const uint16_t *gate, const uint16_t *weight, uint16_t *out, int head_dim,
                             float eps, int heads) {
    if (head_dim <= 0 || heads <= 0) return SO_ERR_GEOMETRY;
    for (int h = 0; h < heads; ++h) {
        const uint16_t *x = input + (size_t)h * head_dim, *g = gate + (size_t)h * head_dim;
        float sum = 0.0f;
        for (int i = 0; i < head_dim; ++i) sum += h2f(x[i]) * h2f(x[i]);
        const float rs = 1.0f / sqrtf(sum / (float)head_dim + eps);
        for (int i = 0; i < head_dim; ++i) {
            const float gv = h2f(g[i]);
            const float silu = gv / (1.0f + expf(-gv));
            out[(size_t)h * head_dim + i] = f2h(h2f(weight[i]) * (h2f(x[i]) * rs) * silu);
        }
    }
    return SO_OK;
}

/* rms_norm_gated with the threadgroup width the record dispatches it with (norms.metal:1093-1143):
 * thread t adds x[t]^2, x[t + tgs]^2, ... in that order, every simdgroup of 32 threads sums its
 * lanes (simd_sum), the simdgroups' partial sums are added one after the other.  tgs = 32 or 128
 * in the reference's tables. */
static float gated_norm_rs(const uint16_t *x, int head_dim, float eps, int tgs) {
    float total = 0.0f;
    for (int s = 0; s < tgs / 32; ++s) {
        float lane[32];
        for (int l = 0; l < 32; ++l) {
            float p = 0.0f;
            for (int i = s * 32 + l; i < head_dim; i += tgs) p += h2f(x[i]) * h2f(x[i]);
            lane[l] = p;
        }
        total += simd_sum32(lane);
    }
    return 1.0f / sqrtf(total / (float)head_dim + eps);
}
static inline uint16_t gated_norm_value(uint16_t x, uint16_t g, uint16_t w, float rs) {
    const float gv = h2f(g);
    const float silu = gv / (1.0f + expf(-gv));
    return f2h(h2f(w) * (h2f(x) * rs) * silu);
}
SO_API int so_rms_norm_gated_tg(const uint16_t *input, const uint16_t *gate, const uint16_t *weight, uint16_t *out, int head_dim,
                                float eps, int heads, int tgs) {
    if (head_dim <= 0 || heads <= 0 || tgs < 32 || tgs % 32 || tgs > 1024) return SO_ERR_GEOMETRY;
    for (int h = 0; h < heads; ++h) {
        const uint16_t *x = input + (size_t)h * head_dim, *g = gate + (size_t)h * head_dim;
        const float rs = gated_norm_rs(x, head_dim, eps, tgs);
        for (int i = 0; i < head_dim; ++i) out[(size_t)h * head_dim + i] = gated_norm_value(x[i], g[i], weight[i], rs);
    }
    return SO_OK;
}

/* rms_norm_gated_d128 and rms_norm_gated_d128_batched (Resources/Shaders/norms_gated_precise.metal:
 * 7-87): one simdgroup per head of 128, lane l adds the squares of its four adjacent values
 * 4 l .. 4 l + 3, simd_sum; value = half(float(w * half(x * rs)) * (g * sigmoid(g))) with the
 * norm materialised in fp16 (the half product w * half(..) included), the sigmoid in its stable
 * spelling (tail = 1 / (1 + exp(|g|))) and eps = 1e-6. */
static float gated_norm_d128_rs(const uint16_t *x) {
    float lane[32];
    for (int l = 0; l < 32; ++l) {
        float p = 0.0f;
        for (int i = 0; i < 4; ++i) p += h2f(x[4 * l + i]) * h2f(x[4 * l + i]);
        lane[l] = p;
    }
    return 1.0f / sqrtf(simd_sum32(lane) / 128.0f + 1e-6f);
}
static inline uint16_t gated_norm_d128_value(uint16_t x, uint16_t g, uint16_t w, float rs) {
    const float normalized = round_h(h2f(w) * round_h(h2f(x) * rs));
    const float gv = h2f(g);
    const float tail = 1.0f / (1.0f + expf(fabsf(gv)));
    const float sig = gv < 0.0f ? tail : 1.0f - tail;
    return f2h(normalized * (gv * sig));
}
SO_API int so_rms_norm_gated_d128(const uint16_t *input, const uint16_t *gate, const uint16_t *weight, uint16_t *out, int heads) {
    if (heads <= 0) return SO_ERR_GEOMETRY;
    for (int h = 0; h < heads; ++h) {
        const uint16_t *x = input + (size_t)h * 128, *g = gate + (size_t)h * 128;
        const float rs = gated_norm_d128_rs(x);
        for (int i = 0; i < 128; ++i) out[(size_t)h * 128 + i] = gated_norm_d128_value(x[i], g[i], weight[i], rs);
    }
    return SO_OK;
}

/* signed_binary_embedding_gather_g128 / signed_ternary_embedding_gather_g128
 * (Resources/Shaders/signed_quant.metal:690-745): out[b, c] = half(sem(code[row, c]) *
 * scale[row, c / 128]), row = token_ids[b]; binary bit 0 / 1 = -1 / +1 (LSB first), ternary
 * 2-bit code - 1. */
SO_API int so_signed_embedding_gather(int format, const uint8_t *codes, const uint16_t *scales, const int32_t *token_ids, uint16_t *out,
                                      int hidden, int batch) {
    if ((format != 1 && format != 2) || hidden <= 0 || hidden % 128 || batch <= 0) return SO_ERR_GEOMETRY;
    const size_t row_bytes = format == 2 ? (size_t)hidden / 4 : (size_t)hidden / 8;
    const int groups = hidden / 128;
    for (int b = 0; b < batch; ++b) {
        const size_t row = (size_t)token_ids[b];
        for (int c = 0; c < hidden; ++c) {
            float v;
            if (format == 2) v = (float)((int)((codes[row * row_bytes + c / 4] >> (2 * (c & 3))) & 3u) - 1);
            else v = ((codes[row * row_bytes + c / 8] >> (c & 7)) & 1u) ? 1.0f : -1.0f;
            out[(size_t)b * hidden + c] = f2h(v * h2f(scales[row * groups + c / 128]));
        }
    }
    return SO_OK;
}

/* ───────────────────── signed activation bit-planes (the Bonsai low-bit path) ─────────────────────
 * Producers turn 128 activations into a sign plane and PLANES-1 magnitude planes of a symmetric
 * integer quantisation plus one fp16 scale; consumers multiply the packed 1-bit / 2-bit weights
 * with the planes by popcount.  Restated from Resources/Shaders/signed_quant.metal:751-932
 * (producers) and :1300-1712, :1732-1822, :2054-2101 (consumers): the integer part is exact,
 * the fp32 accumulation follows the kernels' lane partition (lane l owns groups l, l + 32, ...)
 * and simd_sum's butterfly. */
static inline int bitplane_max_q(int planes) { return (1 << (planes - 1)) - 1; } /* i2 1, i3 3, i4 7, i5 15, i6 31 */

static int bitplane_group(const uint16_t *values, int planes, uint32_t *out_planes, uint16_t *out_scale) {
    /* signed_quant.metal:757-795 (i4), :797-834 (i2, i3 quantise with the unrounded scale; i5, i6 and i4
     * with the stored fp16 scale) */
    const int max_q = bitplane_max_q(planes);
    const int match_stored = planes >= 4;
    float max_abs = 0.0f;
    for (int i = 0; i < 128; ++i) max_abs = fmaxf(max_abs, fabsf(h2f(values[i])));
    const float producer_scale = max_abs > 0.0f ? max_abs / (float)max_q : 1.0f;
    const uint16_t stored = f2h(producer_scale);
    const float scale = match_stored ? h2f(stored) : producer_scale;
    *out_scale = stored;
    for (int p = 0; p < planes * 4; ++p) out_planes[p] = 0u;
    for (int w = 0; w < 4; ++w)
        for (int lane = 0; lane < 32; ++lane) {
            float v = h2f(values[w * 32 + lane]) / scale;
            v = v < -(float)max_q ? -(float)max_q : (v > (float)max_q ? (float)max_q : v);
            const int q = (int)roundf(v); /* round half away from zero, as Metal's round */
            const unsigned mag = (unsigned)abs(q);
            for (int p = 0; p < planes; ++p) {
                const unsigned bit = p == planes - 1 ? (q < 0 ? 1u : 0u) : ((mag >> p) & 1u);
                out_planes[p * 4 + w] |= bit << lane;
            }
        }
    return SO_OK;
}

/* signed_activation_bitplanes_i{2..6}_g128: planes [groups, PLANES, 4] words, scales [groups]. */
SO_API int so_signed_activation_bitplanes(const uint16_t *input, int cols, int planes, uint32_t *out_planes, uint16_t *out_scales) {
    if (cols <= 0 || cols % 128 || planes < 2 || planes > 6) return SO_ERR_GEOMETRY;
    for (int g = 0; g < cols / 128; ++g) bitplane_group(input + (size_t)g * 128, planes, out_planes + (size_t)g * planes * 4, out_scales + g);
    return SO_OK;
}

/* swiglu_signed_activation_bitplanes_i5_g128 (signed_quant.metal:876-916): the staged fp16 SwiGLU
 * of gate and up, then the i5 view. */
SO_API int so_swiglu_signed_activation_bitplanes_i5(const uint16_t *gate, const uint16_t *up, int cols, uint32_t *out_planes,
                                                    uint16_t *out_scales) {
    if (cols <= 0 || cols % 128) return SO_ERR_GEOMETRY;
    uint16_t v[128];
    for (int g = 0; g < cols / 128; ++g) {
        for (int i = 0; i < 128; ++i) v[i] = swiglu_staged_half(gate[(size_t)g * 128 + i], up[(size_t)g * 128 + i]);
        bitplane_group(v, 5, out_planes + (size_t)g * 20, out_scales + g);
    }
    return SO_OK;
}

/* sigmoid_mul_signed_activation_bitplanes_i6_g128 (signed_quant.metal:985-1031): the staged fp16
 * a * sigmoid(b) (tail = 1 / (1 + exp(|b|)) in half arithmetic), then the i6 view. */
SO_API int so_sigmoid_mul_signed_activation_bitplanes_i6(const uint16_t *a, const uint16_t *b, int cols, uint32_t *out_planes,
                                                         uint16_t *out_scales) {
    if (cols <= 0 || cols % 128) return SO_ERR_GEOMETRY;
    uint16_t v[128];
    for (int g = 0; g < cols / 128; ++g) {
        for (int i = 0; i < 128; ++i) {
            const float bv = h2f(b[(size_t)g * 128 + i]);
            const float tail = round_h(1.0f / round_h(1.0f + round_h(expf(fabsf(bv)))));
            const float sig = bv < 0.0f ? tail : round_h(1.0f - tail);
            v[i] = f2h(h2f(a[(size_t)g * 128 + i]) * sig);
        }
        bitplane_group(v, 6, out_planes + (size_t)g * 24, out_scales + g);
    }
    return SO_OK;
}

/* norm_scale_signed_activation_bitplanes_i{2..6}_g128 (signed_quant.metal:1175-1298): the value
 * rms_norm_1pw would write, half(half(x * rs) * half(1 + w)) with rs = norm_scale[0] computed
 * by an earlier dispatch, then the view. */
SO_API int so_norm_scale_signed_activation_bitplanes(const float *norm_scale, const uint16_t *input, const uint16_t *norm_weight, int cols,
                                                     int planes, uint32_t *out_planes, uint16_t *out_scales) {
    if (cols <= 0 || cols % 128 || planes < 2 || planes > 6) return SO_ERR_GEOMETRY;
    const float rs = norm_scale[0];
    uint16_t v[128];
    for (int g = 0; g < cols / 128; ++g) {
        for (int i = 0; i < 128; ++i) {
            const size_t c = (size_t)g * 128 + i;
            v[i] = f2h(round_h(h2f(input[c]) * rs) * round_h(1.0f + h2f(norm_weight[c])));
        }
        bitplane_group(v, planes, out_planes + (size_t)g * planes * 4, out_scales + g);
    }
    return SO_OK;
}

/* rms_norm_gated_d128_signed_activation_bitplanes_i6_g128 (signed_quant.metal:1040-1173): the
 * gated norm of a head of 128 and its i6 view in one dispatch.  A threadgroup of 32 threads takes
 * rms_norm_gated_d128's arithmetic, any other width rms_norm_gated's (the fused record keeps the
 * norm's dispatch, Sources/SmeltCompiler/SmeltFusionPlanner.swift:1239-1280). */
SO_API int so_rms_norm_gated_d128_signed_activation_bitplanes_i6(const uint16_t *input, const uint16_t *gate, const uint16_t *weight,
                                                                 int heads, float eps, int tgs, uint32_t *out_planes, uint16_t *out_scales) {
    if (heads <= 0 || tgs < 32 || tgs % 32 || tgs > 1024) return SO_ERR_GEOMETRY;
    uint16_t v[128];
    for (int h = 0; h < heads; ++h) {
        const uint16_t *x = input + (size_t)h * 128, *g = gate + (size_t)h * 128;
        if (tgs == 32) {
            /* the fused kernel passes eps to the precise arithmetic (signed_quant.metal:1083-1085) */
            float lane[32];
            for (int l = 0; l < 32; ++l) {
                float p = 0.0f;
                for (int i = 0; i < 4; ++i) p += h2f(x[4 * l + i]) * h2f(x[4 * l + i]);
                lane[l] = p;
            }
            const float rs = 1.0f / sqrtf(simd_sum32(lane) / 128.0f + eps);
            for (int i = 0; i < 128; ++i) v[i] = gated_norm_d128_value(x[i], g[i], weight[i], rs);
        } else {
            const float rs = gated_norm_rs(x, 128, eps, tgs);
            for (int i = 0; i < 128; ++i) v[i] = gated_norm_value(x[i], g[i], weight[i], rs);
        }
        bitplane_group(v, 6, out_planes + (size_t)h * 24, out_scales + h);
    }
    return SO_OK;
}

static inline int popc32(uint32_t v) { return __builtin_popcount(v); }

/* Integer dot of one weight group with the planes: sum_bit 2^bit * (2 * agreements - active). */
static inline int bitplane_group_dot(int format, const uint8_t *codes, const uint32_t *planes_g, int planes) {
    uint32_t pos[4], neg[4];
    if (format == 1) { /* binary: bit 1 = +1, bit 0 = -1; LSB first, 16 bytes per group */
        memcpy(pos, codes, 16);
        for (int w = 0; w < 4; ++w) neg[w] = ~pos[w];
    } else { /* ternary: 2-bit codes 0 / 1 / 2 = -1 / 0 / +1, 32 bytes per group (signed_quant.metal:50-79) */
        for (int w = 0; w < 4; ++w) {
            pos[w] = neg[w] = 0u;
            for (int i = 0; i < 32; ++i) {
                const int idx = w * 32 + i;
                const unsigned code = (codes[idx >> 2] >> ((idx & 3) * 2)) & 3u;
                if (code == 2u) pos[w] |= 1u << i;
                if (code == 0u) neg[w] |= 1u << i;
            }
        }
    }
    const uint32_t *sign = planes_g + (size_t)(planes - 1) * 4;
    int dot = 0;
    for (int bit = 0; bit + 1 < planes; ++bit) {
        const uint32_t *mag = planes_g + (size_t)bit * 4;
        int agree = 0, active = 0;
        for (int w = 0; w < 4; ++w) {
            agree += popc32(((pos[w] & ~sign[w]) | (neg[w] & sign[w])) & mag[w]);
            active += popc32((pos[w] | neg[w]) & mag[w]);
        }
        dot += (1 << bit) * (2 * agree - active);
    }
    return dot;
}

static float bitplane_row_acc(int format, const uint8_t *row_codes, const uint16_t *row_scales, const uint32_t *planes_all,
                              const uint16_t *act_scales, int groups, int planes) {
    const int group_bytes = format == 1 ? 16 : 32;
    float lane[32];
    for (int l = 0; l < 32; ++l) {
        float acc = 0.0f;
        for (int g = l; g < groups; g += 32) {
            const int dot = bitplane_group_dot(format, row_codes + (size_t)g * group_bytes, planes_all + (size_t)g * planes * 4, planes);
            acc += (float)dot * h2f(act_scales[g]) * h2f(row_scales[g]);
        }
        lane[l] = acc;
    }
    return simd_sum32(lane);
}

/* signed_{binary,ternary}_bitplane_i{P}_matvec[_add]_g128_rows8: y[r] = half(acc), with a residual
 * half(float(half(acc)) + residual[r]) (signed_quant.metal:1697-1710). */
SO_API int so_signed_bitplane_matvec(int format, const uint8_t *codes, const uint16_t *weight_scales, const uint32_t *planes_all,
                                     const uint16_t *act_scales, const uint16_t *residual, int rows, int cols, int planes, uint16_t *out) {
    if ((format != 1 && format != 2) || rows <= 0 || cols <= 0 || cols % 128 || planes < 2 || planes > 6) return SO_ERR_GEOMETRY;
    const int groups = cols / 128;
    const size_t row_bytes = format == 1 ? (size_t)cols / 8 : (size_t)cols / 4;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const float acc = bitplane_row_acc(format, codes + (size_t)r * row_bytes, weight_scales + (size_t)r * groups, planes_all, act_scales, groups, planes);
        out[r] = residual ? f2h(round_h(acc) + h2f(residual[r])) : f2h(acc);
    }
    return SO_OK;
}

/* signed_binary_bitplane_i{P}_gate_up_swiglu_g128_rows8 (signed_quant.metal:1732-1822). */
SO_API int so_signed_bitplane_gate_up_swiglu(int format, const uint8_t *gate_codes, const uint16_t *gate_scales, const uint8_t *up_codes,
                                             const uint16_t *up_scales, const uint32_t *planes_all, const uint16_t *act_scales, int rows,
                                             int cols, int planes, uint16_t *out) {
    if ((format != 1 && format != 2) || rows <= 0 || cols <= 0 || cols % 128 || planes < 2 || planes > 6) return SO_ERR_GEOMETRY;
    const int groups = cols / 128;
    const size_t row_bytes = format == 1 ? (size_t)cols / 8 : (size_t)cols / 4;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const float g = bitplane_row_acc(format, gate_codes + (size_t)r * row_bytes, gate_scales + (size_t)r * groups, planes_all, act_scales, groups, planes);
        const float u = bitplane_row_acc(format, up_codes + (size_t)r * row_bytes, up_scales + (size_t)r * groups, planes_all, act_scales, groups, planes);
        out[r] = swiglu_staged_half(f2h(g), f2h(u));
    }
    return SO_OK;
}
