// Signed activation bit-planes: the low-bit activation view of the Bonsai-class packages and the
// popcount consumers that multiply it with packed binary (1-bit) and ternary (2-bit) weights.
//
// Producers (Resources/Shaders/signed_quant.metal:751-932): per group of 128 activations one fp16
// scale = max|x| / maxQ and a symmetric integer q = round(clamp(x / scale)), stored as PLANES - 1
// magnitude bit-planes plus a sign plane, four 32-bit words each, word w bit l = column
// 32 w + l: signed_activation_bitplanes_i{2..6}_g128 and, with the staged fp16 SwiGLU of gate
// and up in front, swiglu_signed_activation_bitplanes_i5_g128.  One warp per group: a warp
// ballot IS the packed word.
// Consumers (signed_quant.metal:1300-1712, :1732-1822, :2054-2101):
// signed_binary_bitplane_i{P}_matvec[_add]_g128_rows8, ..._gate_up_swiglu_g128_rows8 and
// signed_ternary_bitplane_i{P}_matvec_g128_rows8: per weight group an exact integer dot
// sum_bit 2^bit (2 popc(agree & magnitude) - popc(nonzero & magnitude)), scaled by the
// activation scale and the weight scale in fp32.  A warp owns four weight rows; lane l owns
// groups l, l + 32, ... (the reference's partition, which fixes the fp32 order) and the lanes'
// sums meet in simd_sum's butterfly.  The planes of a row of 5120 activations are 3 KB: they
// stay in L1 / L2 while the 1-bit weights stream from HBM once.
#include <string>

#include "common.cuh"
#include "glue.h"
#include "runtime.h"

namespace smelt {

namespace {


// The view of one group held by one warp: v[w] is the fp16 value of column 32 w + lane.
template <int PLANES>
__device__ __forceinline__ void pack_group(const float (&v)[4], uint32_t* out, __half* scale_out, int lane) {
    constexpr int kMaxQ = (1 << (PLANES - 1)) - 1;
    constexpr bool kMatchStored = PLANES >= 4;
    float max_abs = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) max_abs = fmaxf(max_abs, __shfl_xor_sync(0xffffffffu, max_abs, off));
    const float producer_scale = max_abs > 0.0f ? __fdiv_rn(max_abs, (float)kMaxQ) : 1.0f;
    const __half stored = __float2half_rn(producer_scale);
    const float scale = kMatchStored ? __half2float(stored) : producer_scale;
    if (lane == 0) *scale_out = stored;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const float c = fminf(fmaxf(__fdiv_rn(v[w], scale), -(float)kMaxQ), (float)kMaxQ);
        const int q = (int)roundf(c);  // half away from zero, as Metal's round
        const unsigned mag = (unsigned)abs(q);
#pragma unroll
        for (int p = 0; p < PLANES; ++p) {
            const bool bit = p == PLANES - 1 ? q < 0 : ((mag >> p) & 1u) != 0u;
            const uint32_t word = __ballot_sync(0xffffffffu, bit);
            if (lane == 0) out[p * 4 + w] = word;
        }
    }
}

// One warp per (group, batch row).  SWIGLU: the values are swiglu_staged(gate, up) instead of x.
template <int PLANES, bool SWIGLU>
__global__ void __launch_bounds__(128) bitplane_producer_kernel(const __half* x, const __half* up, uint32_t* planes, __half* scales, int cols,
                                                                DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int groups = cols / 128, lane = threadIdx.x & 31;
    const int group = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (group >= groups) return;
    const size_t row = blockIdx.y;
    const size_t base = row * cols + (size_t)group * 128;
    float v[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        __half h = x[base + w * 32 + lane];
        if (SWIGLU) h = swiglu_staged(h, up[base + w * 32 + lane]);
        v[w] = __half2float(h);
    }
    pack_group<PLANES>(v, planes + (row * groups + group) * (PLANES * 4), scales + row * groups + group, lane);
}

// Producers with another kernel's arithmetic in front (signed_quant.metal:985-1298): every lane
// makes the fp16 values the staged kernel would have written, then the view is the same.
//   FRONT 2  a * sigmoid(b) in half arithmetic (sigmoid_mul), i6
//   FRONT 3  half(half(x * rs) * half(1 + w)), rs = norm_scale[0] from an earlier dispatch (rms_norm_1pw), i2..i6
//   FRONT 4  the gated RMS norm of a head of 128 = one group: a threadgroup of 32 threads takes
//            rms_norm_gated_d128's arithmetic, any other width rms_norm_gated's, i6
template <int PLANES, int FRONT>
__global__ void __launch_bounds__(128) bitplane_fused_producer_kernel(const __half* a, const __half* b, const __half* c, const float* norm_scale,
                                                                      uint32_t* planes, __half* scales, int cols, float eps, int tgs, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int groups = cols / 128, lane = threadIdx.x & 31;
    const int group = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (group >= groups) return;
    const size_t base = (size_t)group * 128;
    float v[4];
    if (FRONT == 2) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const size_t col = base + w * 32 + lane;
            const __half bv = b[col];
            const __half tail = __hdiv(__float2half_rn(1.0f), __hadd(__float2half_rn(1.0f), __float2half_rn(expf(fabsf(__half2float(bv))))));
            const __half sig = __half2float(bv) < 0.0f ? tail : __hsub(__float2half_rn(1.0f), tail);
            v[w] = __half2float(__hmul(a[col], sig));
        }
    } else if (FRONT == 3) {
        const float rs = norm_scale[0];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const size_t col = base + w * 32 + lane;
            const __half normalized = __float2half_rn(__fmul_rn(__half2float(a[col]), rs));
            const __half direct = __float2half_rn(__fadd_rn(1.0f, __half2float(c[col])));
            v[w] = __half2float(__hmul(normalized, direct));
        }
    } else {
        const bool precise = tgs == 32;
        const float rs = precise ? gated_norm_d128_rs(a + base, eps, lane) : gated_norm_rs(a + base, 128, eps, tgs, lane);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const int i = w * 32 + lane;
            v[w] = __half2float(precise ? gated_norm_d128_value(a[base + i], b[base + i], c[i], rs) : gated_norm_value(a[base + i], b[base + i], c[i], rs));
        }
    }
    pack_group<PLANES>(v, planes + (size_t)group * (PLANES * 4), scales + group, lane);
}

// signed_binary_embedding_gather_g128 / signed_ternary_embedding_gather_g128 (signed_quant.metal:690-745):
// out[b, c] = half(sem(code[row, c]) * scale[row, c / 128]), row = token_ids[b].  One thread per eight columns.
template <bool TERNARY>
__global__ void __launch_bounds__(128) signed_embedding_gather_kernel(const uint8_t* codes, const __half* scales, const int32_t* token_ids, __half* out,
                                                                      int hidden, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int c8 = blockIdx.x * blockDim.x + threadIdx.x;
    if (c8 * 8 >= hidden) return;
    const size_t row = (size_t)token_ids[blockIdx.y];
    const size_t row_bytes = TERNARY ? (size_t)hidden / 4 : (size_t)hidden / 8;
    const float scale = __half2float(scales[row * (hidden / 128) + c8 / 16]);
    const uint8_t* src = codes + row * row_bytes + (TERNARY ? c8 * 2 : c8);
    const uint32_t bits = TERNARY ? (uint32_t)src[0] | ((uint32_t)src[1] << 8) : (uint32_t)src[0];
    __half* dst = out + (size_t)blockIdx.y * hidden + (size_t)c8 * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float v = TERNARY ? (float)((int)((bits >> (2 * i)) & 3u) - 1) : (((bits >> i) & 1u) ? 1.0f : -1.0f);
        dst[i] = __float2half_rn(__fmul_rn(v, scale));
    }
}

// 32 two-bit codes (0 / 1 / 2 = -1 / 0 / +1) in a 64-bit word -> positive and negative masks
__device__ __forceinline__ uint32_t compact_even_bits(uint32_t v) {
    v &= 0x55555555u;
    v = (v | (v >> 1)) & 0x33333333u;
    v = (v | (v >> 2)) & 0x0f0f0f0fu;
    v = (v | (v >> 4)) & 0x00ff00ffu;
    v = (v | (v >> 8)) & 0x0000ffffu;
    return v;
}
__device__ __forceinline__ void ternary_masks32(uint32_t w0, uint32_t w1, uint32_t& pos, uint32_t& neg) {
    const uint32_t l0 = w0 & 0x55555555u, h0 = (w0 >> 1) & 0x55555555u;
    const uint32_t l1 = w1 & 0x55555555u, h1 = (w1 >> 1) & 0x55555555u;
    pos = compact_even_bits(h0 & ~l0) | (compact_even_bits(h1 & ~l1) << 16);
    neg = compact_even_bits(~(h0 | l0)) | (compact_even_bits(~(h1 | l1)) << 16);
}


// MODE 0 plain, 1 + residual, 2 gate/up + SwiGLU.  ROWS weight rows per warp.
template <int PLANES, bool TERNARY, int MODE, int ROWS, int U>
__global__ void __launch_bounds__(256) bitplane_matvec_kernel(const uint8_t* __restrict__ codes, const __half* __restrict__ wscales,
                                                              const uint8_t* __restrict__ codes2, const __half* __restrict__ wscales2,
                                                              const uint32_t* __restrict__ planes, const __half* __restrict__ ascales,
                                                              const __half* residual, __half* out, int rows, int cols, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    constexpr int NM = MODE == 2 ? 2 : 1;
    const int lane = threadIdx.x & 31;
    const int row0 = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * ROWS;
    if (row0 >= rows) return;
    const int groups = cols / 128;
    const size_t row_bytes = TERNARY ? (size_t)cols / 4 : (size_t)cols / 8;
    const size_t b = blockIdx.y;  // batch row: its own planes, scales and outputs
    planes += b * (size_t)groups * PLANES * 4;
    ascales += b * (size_t)groups;
    float acc[NM][ROWS];
#pragma unroll
    for (int m = 0; m < NM; ++m)
#pragma unroll
        for (int t = 0; t < ROWS; ++t) acc[m][t] = 0.0f;
    // U of the lane's groups per round: every load of the round is requested before any is used;
    // the sums still take the groups in ascending order.
    for (int g0 = lane; g0 < groups; g0 += 32 * U) {
        uint4 pl[U][PLANES], wa[U][NM][ROWS], wb[U][NM][ROWS];
        float as[U], ws[U][NM][ROWS];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int g = g0 + 32 * u;
            if (g >= groups) continue;
#pragma unroll
            for (int p = 0; p < PLANES; ++p) pl[u][p] = *reinterpret_cast<const uint4*>(planes + ((size_t)g * PLANES + p) * 4);
            as[u] = __half2float(ascales[g]);
#pragma unroll
            for (int m = 0; m < NM; ++m) {
                const uint8_t* cm = m == 0 ? codes : codes2;
                const __half* sm = m == 0 ? wscales : wscales2;
#pragma unroll
                for (int t = 0; t < ROWS; ++t) {
                    const int row = row0 + t;
                    if (row >= rows) continue;
                    const uint8_t* src = cm + row * row_bytes + (size_t)g * (TERNARY ? 32 : 16);
                    wa[u][m][t] = *reinterpret_cast<const uint4*>(src);
                    if (TERNARY) wb[u][m][t] = *reinterpret_cast<const uint4*>(src + 16);
                    ws[u][m][t] = __half2float(sm[(size_t)row * groups + g]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int g = g0 + 32 * u;
            if (g >= groups) continue;
            const uint4 sign = pl[u][PLANES - 1];
#pragma unroll
            for (int m = 0; m < NM; ++m)
#pragma unroll
                for (int t = 0; t < ROWS; ++t) {
                    if (row0 + t >= rows) continue;
                    uint4 pos, neg;
                    if (TERNARY) {
                        const uint4 a = wa[u][m][t], c = wb[u][m][t];
                        ternary_masks32(a.x, a.y, pos.x, neg.x); ternary_masks32(a.z, a.w, pos.y, neg.y);
                        ternary_masks32(c.x, c.y, pos.z, neg.z); ternary_masks32(c.z, c.w, pos.w, neg.w);
                    } else {
                        pos = wa[u][m][t];
                        neg = make_uint4(~pos.x, ~pos.y, ~pos.z, ~pos.w);
                    }
                    const uint4 agree = make_uint4((pos.x & ~sign.x) | (neg.x & sign.x), (pos.y & ~sign.y) | (neg.y & sign.y),
                                                   (pos.z & ~sign.z) | (neg.z & sign.z), (pos.w & ~sign.w) | (neg.w & sign.w));
                    int dot = 0;
#pragma unroll
                    for (int bit = 0; bit < PLANES - 1; ++bit) {
                        const uint4 mag = pl[u][bit];
                        const int ag = __popc(agree.x & mag.x) + __popc(agree.y & mag.y) + __popc(agree.z & mag.z) + __popc(agree.w & mag.w);
                        int active;
                        if (TERNARY) active = __popc((pos.x | neg.x) & mag.x) + __popc((pos.y | neg.y) & mag.y) + __popc((pos.z | neg.z) & mag.z) + __popc((pos.w | neg.w) & mag.w);
                        else active = __popc(mag.x) + __popc(mag.y) + __popc(mag.z) + __popc(mag.w);
                        dot += (2 * ag - active) << bit;
                    }
                    acc[m][t] = __fadd_rn(acc[m][t], __fmul_rn(__fmul_rn((float)dot, as[u]), ws[u][m][t]));
                }
        }
    }
#pragma unroll
    for (int m = 0; m < NM; ++m)
#pragma unroll
        for (int t = 0; t < ROWS; ++t) acc[m][t] = simd_sum_lane0(acc[m][t]);
    if (lane == 0) {
#pragma unroll
        for (int t = 0; t < ROWS; ++t) {
            const int row = row0 + t;
            if (row >= rows) continue;
            const size_t o = b * rows + row;
            if (MODE == 0) out[o] = __float2half_rn(acc[0][t]);
            else if (MODE == 1) out[o] = __float2half_rn(__half2float(__float2half_rn(acc[0][t])) + __half2float(residual[o]));
            else out[o] = swiglu_staged(__float2half_rn(acc[0][t]), __float2half_rn(acc[NM - 1][t]));
        }
    }
}

// Prompt rows (signed_quant.metal:1346-1436, the batched_b4 / b8 / b16 tiles): a warp takes ROWS weight rows and BT
// activation rows, reads each weight group once and walks the BT rows' planes against it.  Every (weight row,
// activation row) pair adds the same terms in the same order as the matvec above, so the tile is bit-identical to
// independent rows, which is what the reference asserts of its own tiles.  Binary weights, plain output.
template <int PLANES, int ROWS, int BT>
__global__ void __launch_bounds__(256) bitplane_matvec_tile_kernel(const uint8_t* __restrict__ codes, const __half* __restrict__ wscales,
                                                                   const uint32_t* __restrict__ planes, const __half* __restrict__ ascales,
                                                                   __half* out, int rows, int cols, int batch, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int lane = threadIdx.x & 31;
    const int row0 = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * ROWS;
    if (row0 >= rows) return;
    const int groups = cols / 128;
    const size_t row_bytes = (size_t)cols / 8;
    const int b0 = blockIdx.y * BT;
    float acc[ROWS][BT];
#pragma unroll
    for (int t = 0; t < ROWS; ++t)
#pragma unroll
        for (int b = 0; b < BT; ++b) acc[t][b] = 0.0f;
    for (int g = lane; g < groups; g += 32) {
        uint4 w[ROWS];
        float ws[ROWS];
#pragma unroll
        for (int t = 0; t < ROWS; ++t) {
            const int row = row0 + t < rows ? row0 + t : rows - 1;  // a ragged last tile repeats its last row; the copy is not stored
            w[t] = *reinterpret_cast<const uint4*>(codes + row * row_bytes + (size_t)g * 16);
            ws[t] = __half2float(wscales[(size_t)row * groups + g]);
        }
#pragma unroll
        for (int b = 0; b < BT; ++b) {
            if (b0 + b >= batch) break;
            const uint32_t* pb = planes + ((size_t)(b0 + b) * groups + g) * (PLANES * 4);
            uint4 pl[PLANES];
#pragma unroll
            for (int p = 0; p < PLANES; ++p) pl[p] = *reinterpret_cast<const uint4*>(pb + p * 4);
            const float as = __half2float(ascales[(size_t)(b0 + b) * groups + g]);
            const uint4 sign = pl[PLANES - 1];
            int active[PLANES - 1];
#pragma unroll
            for (int bit = 0; bit < PLANES - 1; ++bit) active[bit] = __popc(pl[bit].x) + __popc(pl[bit].y) + __popc(pl[bit].z) + __popc(pl[bit].w);
#pragma unroll
            for (int t = 0; t < ROWS; ++t) {
                // agree = weight bit where the activation is positive, its complement where it is negative
                const uint4 agree = make_uint4(w[t].x ^ sign.x, w[t].y ^ sign.y, w[t].z ^ sign.z, w[t].w ^ sign.w);
                int dot = 0;
#pragma unroll
                for (int bit = 0; bit < PLANES - 1; ++bit) {
                    const uint4 mag = pl[bit];
                    const int ag = __popc(agree.x & mag.x) + __popc(agree.y & mag.y) + __popc(agree.z & mag.z) + __popc(agree.w & mag.w);
                    dot += (2 * ag - active[bit]) << bit;
                }
                acc[t][b] = __fadd_rn(acc[t][b], __fmul_rn(__fmul_rn((float)dot, as), ws[t]));
            }
        }
    }
#pragma unroll
    for (int t = 0; t < ROWS; ++t)
#pragma unroll
        for (int b = 0; b < BT; ++b) acc[t][b] = simd_sum_lane0(acc[t][b]);
    if (lane == 0) {
#pragma unroll
        for (int t = 0; t < ROWS; ++t)
#pragma unroll
            for (int b = 0; b < BT; ++b)
                if (row0 + t < rows && b0 + b < batch) out[(size_t)(b0 + b) * rows + row0 + t] = __float2half_rn(acc[t][b]);
    }
}

cudaError_t cfg_launch(const Launch& l, cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, dim3 grid, dim3 block) {
    cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = l.stream;
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = l.pdl ? 1 : 0;
    return cudaSuccess;
}

template <int PLANES, bool SWIGLU>
cudaError_t launch_producer_t(const Launch& l, const __half* x, const __half* up, uint32_t* planes, __half* scales, int cols, int batch) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3((cols / 128 + 3) / 4, batch), dim3(128));
    auto k = bitplane_producer_kernel<PLANES, SWIGLU>;
    prefer_max_shared(k);
    return cudaLaunchKernelEx(&cfg, k, x, up, planes, scales, cols, dev_dyn(l));
}

template <int PLANES, bool TERNARY, int MODE, int ROWS, int U>
cudaError_t launch_consumer_r(const Launch& l, const BitplaneArgs& a) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    const int warps = (a.rows + ROWS - 1) / ROWS;
    cfg_launch(l, cfg, attr, dim3((warps + 7) / 8, a.batch), dim3(256));
    auto k = bitplane_matvec_kernel<PLANES, TERNARY, MODE, ROWS, U>;
    prefer_max_shared(k);
    return cudaLaunchKernelEx(&cfg, k, a.codes, a.wscales, a.codes2, a.wscales2, a.planes, a.ascales, a.residual, a.out, a.rows, a.cols, dev_dyn(l));
}

// A row's arithmetic does not depend on how many rows share a warp (lane l owns the row's groups
// l, l + 32, ... either way).  Short rows (up to 64 groups) of binary weights: four rows per warp
// share the plane loads, which outweigh the 16 bytes of weights per group; long rows: one row per
// warp and two groups in flight per lane (measured 13.2 against 22.0 us at 5120 x 17408).
template <int PLANES>
cudaError_t launch_consumer_tile(const Launch& l, const BitplaneArgs& a) {
    constexpr int ROWS = 4, BT = 4;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    const int warps = (a.rows + ROWS - 1) / ROWS;
    cfg_launch(l, cfg, attr, dim3((warps + 7) / 8, (a.batch + BT - 1) / BT), dim3(256));
    auto k = bitplane_matvec_tile_kernel<PLANES, ROWS, BT>;
    prefer_max_shared(k);
    return cudaLaunchKernelEx(&cfg, k, a.codes, a.wscales, a.planes, a.ascales, a.out, a.rows, a.cols, a.batch, dev_dyn(l));
}

template <int PLANES, bool TERNARY, int MODE>
cudaError_t launch_consumer_t(const Launch& l, const BitplaneArgs& a) {
    if (!TERNARY && MODE == 0 && a.batch >= 2) return launch_consumer_tile<PLANES>(l, a);  // prompt rows: weights read once per four rows
    if (TERNARY) return launch_consumer_r<PLANES, true, MODE, 1, 1>(l, a);
    if (a.cols / 128 <= 64) return launch_consumer_r<PLANES, false, MODE, 4, 1>(l, a);
    return launch_consumer_r<PLANES, false, MODE, 1, 2>(l, a);
}

template <bool TERNARY, int MODE>
cudaError_t launch_consumer_p(const Launch& l, const BitplaneArgs& a) {
    switch (a.n_planes) {
        case 2: return launch_consumer_t<2, TERNARY, MODE>(l, a);
        case 3: return launch_consumer_t<3, TERNARY, MODE>(l, a);
        case 4: return launch_consumer_t<4, TERNARY, MODE>(l, a);
        case 5: return launch_consumer_t<5, TERNARY, MODE>(l, a);
        case 6: return launch_consumer_t<6, TERNARY, MODE>(l, a);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

cudaError_t launch_bitplane_producer(const Launch& l, const __half* x, const __half* up, uint32_t* planes, __half* scales, int cols, int n_planes,
                                     int batch) {
    if (cols <= 0 || cols % 128 || batch <= 0) return cudaErrorInvalidValue;
    if (up) return n_planes == 5 ? launch_producer_t<5, true>(l, x, up, planes, scales, cols, batch) : cudaErrorInvalidValue;
    switch (n_planes) {
        case 2: return launch_producer_t<2, false>(l, x, nullptr, planes, scales, cols, batch);
        case 3: return launch_producer_t<3, false>(l, x, nullptr, planes, scales, cols, batch);
        case 4: return launch_producer_t<4, false>(l, x, nullptr, planes, scales, cols, batch);
        case 5: return launch_producer_t<5, false>(l, x, nullptr, planes, scales, cols, batch);
        case 6: return launch_producer_t<6, false>(l, x, nullptr, planes, scales, cols, batch);
        default: return cudaErrorInvalidValue;
    }
}

template <int PLANES, int FRONT>
cudaError_t launch_fused_producer_t(const Launch& l, const __half* a, const __half* b, const __half* c, const float* norm_scale, uint32_t* planes,
                                    __half* scales, int cols, float eps, int tgs) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3((cols / 128 + 3) / 4, 1), dim3(128));
    auto k = bitplane_fused_producer_kernel<PLANES, FRONT>;
    prefer_max_shared(k);
    return cudaLaunchKernelEx(&cfg, k, a, b, c, norm_scale, planes, scales, cols, eps, tgs, dev_dyn(l));
}

cudaError_t launch_bitplane_fused_producer(const Launch& l, int front, const __half* a, const __half* b, const __half* c, const float* norm_scale,
                                           uint32_t* planes, __half* scales, int cols, int n_planes, float eps, int tgs) {
    if (cols <= 0 || cols % 128) return cudaErrorInvalidValue;
    if (front == 2) return n_planes == 6 && a && b ? launch_fused_producer_t<6, 2>(l, a, b, nullptr, nullptr, planes, scales, cols, eps, 32) : cudaErrorInvalidValue;
    if (front == 4) {
        if (n_planes != 6 || !a || !b || !c || tgs < 32 || tgs % 32 || tgs > 1024) return cudaErrorInvalidValue;
        return launch_fused_producer_t<6, 4>(l, a, b, c, nullptr, planes, scales, cols, eps, tgs);
    }
    if (front != 3 || !a || !c || !norm_scale) return cudaErrorInvalidValue;
    switch (n_planes) {
        case 2: return launch_fused_producer_t<2, 3>(l, a, nullptr, c, norm_scale, planes, scales, cols, eps, 32);
        case 3: return launch_fused_producer_t<3, 3>(l, a, nullptr, c, norm_scale, planes, scales, cols, eps, 32);
        case 4: return launch_fused_producer_t<4, 3>(l, a, nullptr, c, norm_scale, planes, scales, cols, eps, 32);
        case 5: return launch_fused_producer_t<5, 3>(l, a, nullptr, c, norm_scale, planes, scales, cols, eps, 32);
        case 6: return launch_fused_producer_t<6, 3>(l, a, nullptr, c, norm_scale, planes, scales, cols, eps, 32);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_signed_embedding_gather(const Launch& l, int format, const uint8_t* codes, const __half* scales, const int32_t* token_ids, __half* out,
                                           int hidden, int batch) {
    if ((format != 1 && format != 2) || hidden <= 0 || hidden % 128 || batch <= 0) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3((hidden / 8 + 127) / 128, batch), dim3(128));
    if (format == 2) {
        prefer_max_shared(signed_embedding_gather_kernel<true>);
        return cudaLaunchKernelEx(&cfg, signed_embedding_gather_kernel<true>, codes, scales, token_ids, out, hidden, dev_dyn(l));
    }
    prefer_max_shared(signed_embedding_gather_kernel<false>);
    return cudaLaunchKernelEx(&cfg, signed_embedding_gather_kernel<false>, codes, scales, token_ids, out, hidden, dev_dyn(l));
}

cudaError_t launch_bitplane_matvec(const Launch& l, const BitplaneArgs& a) {
    if (a.rows <= 0 || a.cols <= 0 || a.cols % 128 || a.batch <= 0 || (a.format != 1 && a.format != 2)) return cudaErrorInvalidValue;
    if (a.mode == 2 && (!a.codes2 || !a.wscales2)) return cudaErrorInvalidValue;
    if (a.mode == 1 && !a.residual) return cudaErrorInvalidValue;
    const bool t = a.format == 2;
    switch (a.mode) {
        case 0: return t ? launch_consumer_p<true, 0>(l, a) : launch_consumer_p<false, 0>(l, a);
        case 1: return t ? launch_consumer_p<true, 1>(l, a) : launch_consumer_p<false, 1>(l, a);
        case 2: return t ? launch_consumer_p<true, 2>(l, a) : launch_consumer_p<false, 2>(l, a);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace smelt

using namespace smelt;

namespace {
Launch typed(smelt_cuda_ctx* ctx) {
    Launch l;
    l.stream = ctx->stream;
    l.pdl = ctx->capturing && ctx->pdl;
    return l;
}
}  // namespace

extern "C" {

smelt_status smelt_cuda_signed_activation_bitplanes(smelt_cuda_ctx* ctx, const void* x, const void* up_or_null, void* planes, void* scales,
                                                    int cols, int n_planes, int batch) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!x || !planes || !scales || cols <= 0 || cols % 128 || batch <= 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "activation bit-planes: cols a multiple of 128");
    if (n_planes < 2 || n_planes > 6 || (up_or_null && n_planes != 5)) return fail(ctx, SMELT_ERR_UNSUPPORTED, "activation bit-planes: 2..6 planes (the SwiGLU producer: 5)");
    return check_cuda(ctx, launch_bitplane_producer(typed(ctx), (const __half*)x, (const __half*)up_or_null, (uint32_t*)planes, (__half*)scales, cols, n_planes, batch), "activation bit-planes");
}

smelt_status smelt_cuda_fused_activation_bitplanes(smelt_cuda_ctx* ctx, int front, const void* a, const void* b, const void* c, const void* norm_scale,
                                                   void* planes, void* scales, int cols, int n_planes, float eps, int threadgroup_width) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!planes || !scales || cols <= 0 || cols % 128) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "fused activation bit-planes: cols a multiple of 128");
    const bool ok = (front == SMELT_BITPLANE_FRONT_SIGMOID_MUL && a && b && n_planes == 6) ||
                    (front == SMELT_BITPLANE_FRONT_NORM_SCALE && a && c && norm_scale && n_planes >= 2 && n_planes <= 6) ||
                    (front == SMELT_BITPLANE_FRONT_GATED_NORM_D128 && a && b && c && n_planes == 6 && threadgroup_width >= 32 && threadgroup_width % 32 == 0 &&
                     threadgroup_width <= 1024);
    if (!ok) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "fused activation bit-planes: operands or plane count do not fit the front end");
    return check_cuda(ctx, launch_bitplane_fused_producer(typed(ctx), front, (const __half*)a, (const __half*)b, (const __half*)c, (const float*)norm_scale,
                                                          (uint32_t*)planes, (__half*)scales, cols, n_planes, eps, threadgroup_width),
                      "fused activation bit-planes");
}

smelt_status smelt_cuda_signed_embedding_gather(smelt_cuda_ctx* ctx, int format, const void* codes, const void* scales, const void* token_ids, void* out,
                                                int hidden, int batch) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!codes || !scales || !token_ids || !out || hidden <= 0 || hidden % 128 || batch <= 0 || (format != 1 && format != 2))
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "signed embedding gather: bad arguments");
    return check_cuda(ctx, launch_signed_embedding_gather(typed(ctx), format, (const uint8_t*)codes, (const __half*)scales, (const int32_t*)token_ids, (__half*)out, hidden, batch),
                      "signed embedding gather");
}

smelt_status smelt_cuda_signed_bitplane_matvec(smelt_cuda_ctx* ctx, int format, int mode, const void* codes, const void* weight_scales,
                                               const void* codes2, const void* weight_scales2, const void* planes, const void* act_scales,
                                               const void* residual, void* out, int rows, int cols, int n_planes, int batch) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!codes || !weight_scales || !planes || !act_scales || !out || rows <= 0 || cols <= 0 || cols % 128 || batch <= 0 || (format != 1 && format != 2) ||
        mode < 0 || mode > 2 || (mode == 2 && (!codes2 || !weight_scales2)) || (mode == 1 && !residual))
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "bit-plane matvec: bad arguments");
    if (n_planes < 2 || n_planes > 6) return fail(ctx, SMELT_ERR_UNSUPPORTED, "bit-plane matvec: 2..6 planes");
    if ((reinterpret_cast<uintptr_t>(codes) | reinterpret_cast<uintptr_t>(codes2) | reinterpret_cast<uintptr_t>(planes)) & 15u)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "bit-plane matvec: codes and planes must be 16-byte aligned");
    BitplaneArgs a = {};
    a.format = format; a.mode = mode; a.codes = (const uint8_t*)codes; a.wscales = (const __half*)weight_scales; a.codes2 = (const uint8_t*)codes2;
    a.wscales2 = (const __half*)weight_scales2; a.planes = (const uint32_t*)planes; a.ascales = (const __half*)act_scales;
    a.residual = (const __half*)residual; a.out = (__half*)out; a.rows = rows; a.cols = cols; a.n_planes = n_planes; a.batch = batch;
    return check_cuda(ctx, launch_bitplane_matvec(typed(ctx), a), "bit-plane matvec");
}

}  // extern "C"
