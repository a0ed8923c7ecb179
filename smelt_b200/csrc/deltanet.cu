// The decode step of a DeltaNet (gated linear-attention) layer: the four kernels the reference's
// emitter dispatches between the layer's input projections and its output projection
// (Sources/SmeltCompiler/DeltaNetPlugin.swift:196-318):
//   conv1d_update_silu   Resources/Shaders/conv1d.metal:271-331   depthwise conv state shift + SiLU
//   rms_scale_qk         Resources/Shaders/norms.metal:1380-1431  Q / K RMS scaling with their edge scales
//   deltanet_recurrence_mlx_decode (and its _d128_h16 / _d128_h32_qk16 / _d128_h48_qk16
//                        specialisations) Resources/Shaders/recurrence.metal:511-836
//   rms_norm_gated (and rms_norm_gated_d128) Resources/Shaders/norms.metal:1093-1143
// and their prompt-chunk forms (conv1d.metal:129-268, prefill_recurrence.metal:290-775).
// The arithmetic, including every staged fp16 rounding of the Metal kernels, is kept; the thread
// mapping is CUDA's.  The recurrent state [Hv, Dv, Dk] fp16 is read and written once per step
// (32 KB per head at D = 128): one warp per (head, output row) with the row's Dk values in
// registers, lane l holding dk = l * D/32 ..., exactly the reference's partition, so that the two
// warp sums run over the same operands in the same order.
#include <string>

#include "common.cuh"
#include "glue.h"
#include "runtime.h"

namespace smelt {

namespace {

__device__ __forceinline__ __half exp_half(__half x) { return __float2half_rn(expf(__half2float(x))); }

// smelt_silu_staged_half (conv1d.metal:4-15): every intermediate an fp16 value; zero results are +0
__device__ __forceinline__ __half silu_staged_half(__half x) {
    const float xf = __half2float(x);
    const __half e = __float2half_rn(expf(fabsf(xf)));
    const __half tail = __float2half_rn(1.0f / __half2float(__float2half_rn(1.0f + __half2float(e))));
    const __half sig = xf < 0.0f ? tail : __float2half_rn(1.0f - __half2float(tail));
    const __half r = __float2half_rn(xf * __half2float(sig));
    return (__half_as_ushort(r) & 0x7fffu) == 0u ? __ushort_as_half(0) : r;
}

__global__ void conv1d_update_silu_kernel(__half* state, const __half* new_val, const __half* weight, __half* out, int channels,
                                          int kernel_size, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= channels) return;
    __half* st = state + (size_t)ch * kernel_size;
    const __half* w = weight + (size_t)ch * kernel_size;
    __half cached[8];
    for (int k = 0; k + 1 < kernel_size; ++k) cached[k] = st[k + 1];
    cached[kernel_size - 1] = new_val[ch];
    float acc = 0.0f;  // one tap at a time from a float zero (conv1d.metal:20-27)
    for (int k = 0; k < kernel_size; ++k) {
        st[k] = cached[k];
        acc = __fadd_rn(acc, __fmul_rn(__half2float(cached[k]), __half2float(w[k])));
    }
    out[ch] = silu_staged_half(__float2half_rn(acc));
}

// One warp per (batch row, Q or K head): x <- half(half(x * rsqrt(mean(x^2) + eps)) * edge).
__global__ void rms_scale_qk_kernel(__half* qkv, int head_dim, float eps, int qkv_dim, int qk_heads, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int g = blockIdx.x, lane = threadIdx.x;
    const bool is_k = g >= qk_heads;
    __half* x = qkv + (size_t)blockIdx.y * qkv_dim + (size_t)g * head_dim;
    float sum = 0.0f;
    for (int i = lane; i < head_dim; i += 32) {
        const float v = __half2float(x[i]);
        sum += v * v;
    }
    sum = warp_sum(sum);
    const float scale = __frcp_rn(__fsqrt_rn(sum / (float)head_dim + eps));
    const __half edge = is_k ? __float2half_rn(__frcp_rn(__fsqrt_rn((float)head_dim))) : __float2half_rn(1.0f / (float)head_dim);
    for (int i = lane; i < head_dim; i += 32) {
        const __half n = __float2half_rn(__half2float(x[i]) * scale);
        x[i] = __hmul(n, edge);
    }
}

__device__ __forceinline__ float sigmoid_staged_half(__half x) {
    const float xf = __half2float(x);
    const __half e = __float2half_rn(expf(fabsf(xf)));
    const __half tail = __float2half_rn(1.0f / __half2float(__float2half_rn(1.0f + __half2float(e))));
    return xf < 0.0f ? __half2float(tail) : __half2float(__float2half_rn(1.0f - __half2float(tail)));
}
__device__ __forceinline__ float decode_log1p(float x) {
    const float xp1 = 1.0f + x;
    if (xp1 == 1.0f) return x;
    return x * (logf(xp1) / (xp1 - 1.0f));
}
__device__ __forceinline__ float softplus_staged_half(__half x) {
    const float xf = __half2float(x);
    const float mx = fmaxf(xf, 0.0f), mn = fminf(xf, 0.0f);
    const __half d = __float2half_rn(mn - mx);
    return __half2float(__float2half_rn(mx + decode_log1p(__half2float(exp_half(d)))));
}

template <int EPL>
__global__ void __launch_bounds__(256) deltanet_recurrence_decode_kernel(__half* state, const __half* qkv, const __half* b_proj,
                                                                         const __half* a_proj, const __half* a_log, const __half* dt_bias,
                                                                         __half* out, int value_heads, int qk_heads, DevDyn dyn) {
    constexpr int D = EPL * 32;
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int head = blockIdx.y, dv = blockIdx.x * (blockDim.x >> 5) + warp;
    if (dv >= D) return;
    const int qh = head / (value_heads / qk_heads);
    const __half* q = qkv + (size_t)qh * D + lane * EPL;
    const __half* k = qkv + (size_t)(qk_heads + qh) * D + lane * EPL;
    __half* row = state + ((size_t)head * D + dv) * D + lane * EPL;
    float st[EPL], kr[EPL], qr[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) { st[i] = __half2float(row[i]); kr[i] = __half2float(k[i]); qr[i] = __half2float(q[i]); }
    const float beta = sigmoid_staged_half(b_proj[head]);
    const __half xh = __hadd(a_proj[head], dt_bias[head]);
    const float decay = __half2float(__float2half_rn(expf(-expf(__half2float(a_log[head])) * softplus_staged_half(xh))));
    float kv = 0.0f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        st[i] = __fmul_rn(st[i], decay);
        kv = __fadd_rn(kv, __fmul_rn(st[i], kr[i]));
    }
    kv = __shfl_sync(0xffffffffu, simd_sum_lane0(kv), 0);
    const float delta = __fmul_rn(__fsub_rn(__half2float(qkv[(size_t)2 * qk_heads * D + (size_t)head * D + dv]), kv), beta);
    float o = 0.0f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        st[i] = __fadd_rn(st[i], __fmul_rn(kr[i], delta));
        o = __fadd_rn(o, __fmul_rn(st[i], qr[i]));
    }
    o = simd_sum_lane0(o);
    if (lane == 0) out[(size_t)head * D + dv] = __float2half_rn(o);
#pragma unroll
    for (int i = 0; i < EPL; ++i) row[i] = __float2half_rn(st[i]);
}

// Prompt chunk of the depthwise convolution (conv1d.metal:129-268): one thread per channel walks
// the T rows of qkv [T, C] in place with its taps in registers; neighbouring threads read
// neighbouring channels, so every row access is coalesced.  The taps are fp16 values and their
// products with fp16 weights are exact in fp32, which makes the fused multiply-adds of the
// c6144_k4 specialisation and the per-token rounding of the checkpoint variant equal to the
// generic kernel; one body serves the three names.  history (may be null) [T + 1, C, K].
template <int K>
__global__ void __launch_bounds__(128) conv1d_update_silu_prefill_kernel(__half* state, __half* qkv, const __half* weight, int seq_len,
                                                                         int channels, int kernel_size, __half* history, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= channels) return;
    const int ks = K > 0 ? K : kernel_size;
    __half* st = state + (size_t)ch * ks;
    const size_t hs = (size_t)channels * ks;
    __half cached[8];
    float w[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)
        if (k < ks) {
            cached[k] = st[k];
            w[k] = __half2float(weight[(size_t)ch * ks + k]);
            if (history) history[(size_t)ch * ks + k] = cached[k];
        }
    __half x = seq_len > 0 ? qkv[ch] : __ushort_as_half(0);
    for (int pos = 0; pos < seq_len; ++pos) {
        const __half next = pos + 1 < seq_len ? qkv[(size_t)(pos + 1) * channels + ch] : __ushort_as_half(0);
#pragma unroll
        for (int k = 0; k < 7; ++k)
            if (k + 1 < ks) cached[k] = cached[k + 1];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (k == ks - 1) cached[k] = x;
        float acc = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (k < ks) acc = __fadd_rn(acc, __fmul_rn(__half2float(cached[k]), w[k]));
        qkv[(size_t)pos * channels + ch] = silu_staged_half(__float2half_rn(acc));
        if (history) {
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (k < ks) history[(size_t)(pos + 1) * hs + (size_t)ch * ks + k] = cached[k];
        }
        x = next;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k)
        if (k < ks) st[k] = cached[k];
}

// Prompt chunk of the recurrence (prefill_recurrence.metal:290-775).  The loop over positions
// is a dependent chain per row (decay, warp sum, rank-one update, warp sum) and the kernel is
// bound by instruction issue along it, not by bytes.  Measured at 512 positions of 32 heads x
// 128 x 128: 435 us with one row per warp, operands loaded and converted by every warp and two
// warp sums per position; 230 us in this form (one row per warp with operands shared as floats
// ran 275 us, four rows per warp 395 us):
//  * a warp carries two rows of one head; the two rows sit in the halves of packed fp32x2
//    registers, so every multiply and add of the reference's scalar code is one packed
//    instruction for both rows, each half rounded as the scalar instruction would
//    (mul.rn.f32x2 / add.rn.f32x2; nothing is contracted into a fused multiply-add); the
//    position's k and q are read and converted once for both rows;
//  * the warp sums share their shuffles: at lane distance 16 and 8 the lanes swap halves of the
//    value set instead of adding every value everywhere, which leaves one value per lane for the
//    last three steps.  The additions pair the same lanes in the same order as a butterfly per
//    value, so the bits are those of simd_sum;
//  * the read-out sums of position t (state . q) do not feed the state, so they ride along with
//    the state . k sums of position t + 1 in that one four-value reduction (one chain of five
//    shuffle steps per position instead of two) and leave in one store per stage;
//  * the CTA's eight warps share a head: k, q and the CTA's slice of v for blocks of
//    kDnPosPerStage positions come through a ring of cp.async stages in shared memory, requested
//    two stages ahead; the gates of up to kDnGateBlock positions are computed once per CTA.
// The rows stay in fp32 registers across all T positions with one fp16 rounding when they are
// written back; CHECKPOINT rounds after every position and records the rows in history
// [T + 1, Hv, D, D] (prefill_recurrence.metal:675-775).
constexpr int kDnGateBlock = 1024;
constexpr int kDnRows = 2;
constexpr int kDnWarps = 8;
constexpr int kDnPosPerStage = 8;
constexpr int kDnStages = 3;

__host__ __device__ constexpr int dn_pos_halves(int d) { return 2 * d + kDnWarps * kDnRows; }  // k | q | the CTA's v values
__host__ __device__ constexpr int dn_smem_bytes(int d) { return kDnStages * kDnPosPerStage * dn_pos_halves(d) * 2 + kDnGateBlock * 8; }

// Sum of each of four per-lane values over the warp in simd_sum's order; the total of value j
// ends up in the eight lanes 8 j .. 8 j + 7.
__device__ __forceinline__ float simd_sum4_grouped(float v0, float v1, float v2, float v3, int lane) {
    const bool up16 = lane & 16, up8 = lane & 8;
    const float k0 = up16 ? v2 : v0, k1 = up16 ? v3 : v1;
    const float s0 = up16 ? v0 : v2, s1 = up16 ? v1 : v3;
    const float a0 = __fadd_rn(k0, __shfl_xor_sync(0xffffffffu, s0, 16));
    const float a1 = __fadd_rn(k1, __shfl_xor_sync(0xffffffffu, s1, 16));
    float b = __fadd_rn(up8 ? a1 : a0, __shfl_xor_sync(0xffffffffu, up8 ? a0 : a1, 8));
    b = __fadd_rn(b, __shfl_xor_sync(0xffffffffu, b, 4));
    b = __fadd_rn(b, __shfl_xor_sync(0xffffffffu, b, 2));
    b = __fadd_rn(b, __shfl_xor_sync(0xffffffffu, b, 1));
    return b;
}

template <int N>
__device__ __forceinline__ void load_halves(const __half* p, __half (&dst)[N], bool vec) {
    if constexpr (N == 8 || N == 4 || N == 2) {
        if (vec) {
            uint32_t w[N / 2];
            if constexpr (N == 8) {
                const uint4 u = *reinterpret_cast<const uint4*>(p);
                w[0] = u.x; w[1] = u.y; w[2] = u.z; w[3] = u.w;
            } else if constexpr (N == 4) {
                const uint2 u = *reinterpret_cast<const uint2*>(p);
                w[0] = u.x; w[1] = u.y;
            } else {
                w[0] = *reinterpret_cast<const uint32_t*>(p);
            }
#pragma unroll
            for (int i = 0; i < N; ++i) dst[i] = __ushort_as_half((unsigned short)(w[i >> 1] >> (16 * (i & 1))));
            return;
        }
    }
#pragma unroll
    for (int i = 0; i < N; ++i) dst[i] = p[i];
}

template <int EPL, bool CHECKPOINT>
__global__ void __launch_bounds__(kDnWarps * 32) deltanet_recurrence_prefill_kernel(__half* state, const __half* qkv, const __half* b_proj,
                                                                                    const __half* a_proj, const __half* a_log,
                                                                                    const __half* dt_bias, __half* out, int value_heads,
                                                                                    int qk_heads, int seq_len, __half* history, int vec, DevDyn dyn) {
    constexpr int D = EPL * 32, R = kDnRows, PB = kDnPosPerStage, NS = kDnStages, PH = dn_pos_halves(D);
    constexpr int CH = D / 4 + kDnWarps * R / 8;  // 16-byte pieces per position: k, q, v slice
    static_assert(R == 2 && PB == 8, "two rows per packed register; a stage's sums leave through sixteen lanes");
    extern __shared__ __align__(16) uint8_t dn_smem[];
    __half* ring = reinterpret_cast<__half*>(dn_smem);  // [NS][PB][PH]
    float2* s_gate = reinterpret_cast<float2*>(dn_smem + NS * PB * PH * 2);  // [kDnGateBlock] {decay, beta}
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int head = blockIdx.y, dv_cta = blockIdx.x * (kDnWarps * R), dv0 = dv_cta + warp * R;  // D is a multiple of 32 = twice a CTA's rows
    const int qh = head / (value_heads / qk_heads);
    const size_t stride = (size_t)(2 * qk_heads + value_heads) * D;
    const size_t hs = (size_t)value_heads * D * D;
    const size_t row_off = ((size_t)head * D + dv0) * D + lane * EPL;  // row r of the warp: + r * D
    const __half* q_src = qkv + (size_t)qh * D;
    const __half* k_src = qkv + (size_t)(qk_heads + qh) * D;
    const __half* v_src = qkv + (size_t)2 * qk_heads * D + (size_t)head * D + dv_cta;
    const bool vq = vec != 0;
    const int n_stages = (seq_len + PB - 1) / PB;

    // stage g of the ring: positions g PB .. g PB + PB - 1; always one commit, so the group count is uniform
    auto fill = [&](int g) {
        if (g < n_stages) {
            __half* dst0 = ring + (size_t)(g % NS) * PB * PH;
            for (int c = tid; c < PB * CH; c += kDnWarps * 32) {
                const int pp = c / CH, cc = c % CH, pos = g * PB + pp;
                if (pos >= seq_len) continue;
                const __half* src = (cc < D / 8 ? k_src + cc * 8 : (cc < D / 4 ? q_src + (cc - D / 8) * 8 : v_src + (cc - D / 4) * 8)) + (size_t)pos * stride;
                __half* dst = dst0 + pp * PH + cc * 8;
                if (vq) {
                    cp_async16(dst, src);
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) dst[e] = src[e];
                }
            }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int g = 0; g < NS - 1; ++g) fill(g);

    float2 st[EPL];  // .x: row dv0, .y: row dv0 + 1
    {
        __half h0[EPL], h1[EPL];
        load_halves<EPL>(state + row_off, h0, vq);
        load_halves<EPL>(state + row_off + D, h1, vq);
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            st[i] = make_float2(__half2float(h0[i]), __half2float(h1[i]));
            if (CHECKPOINT) { history[row_off + i] = h0[i]; history[row_off + D + i] = h1[i]; }
        }
    }
    const float ea = expf(__half2float(a_log[head]));
    const __half dtb = dt_bias[head];
    float2 o_prev = make_float2(0.0f, 0.0f);  // state . q of the previous position, before its warp sum

    for (int g = 0; g < n_stages; ++g) {
        cp_async_wait<NS - 2>();
        __syncthreads();  // stage g has landed for every thread; every warp is done with stage g - 1
        fill(g + NS - 1);  // into the buffer stage g - 1 used
        const int p0 = g * PB;
        if (p0 % kDnGateBlock == 0) {
            // every warp passed the barrier above, so nobody reads the previous block's gates any more
            const int nb = min(kDnGateBlock, seq_len - p0);
            for (int t = tid; t < nb; t += kDnWarps * 32) {
                const size_t pi = (size_t)(p0 + t) * value_heads + head;
                const __half xh = __hadd(a_proj[pi], dtb);
                s_gate[t] = make_float2(__half2float(__float2half_rn(expf(-ea * softplus_staged_half(xh)))), sigmoid_staged_half(b_proj[pi]));
            }
            __syncthreads();
        }
        const __half* stage = ring + (size_t)(g % NS) * PB * PH;
        const float2* gates = s_gate + p0 % kDnGateBlock;
        const int np = min(PB, seq_len - p0);
        // One position.  After the reduction lanes 16-23 hold the first row's read-out sum of the position before it
        // and lanes 24-31 the second row's; lane 16 + pp and lane 24 + pp keep them, and the stage's sums leave in one
        // store after the loop.
        float keep = 0.0f;
        auto step = [&](int pp) {
            const __half* row = stage + pp * PH;
            __half kh[EPL], qh16[EPL], vh[R];
            load_halves<EPL>(row + lane * EPL, kh, true);
            load_halves<EPL>(row + D + lane * EPL, qh16, true);
            load_halves<R>(row + 2 * D + warp * R, vh, true);
            float2 kk[EPL], qq[EPL];
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                const float kf = __half2float(kh[i]), qf = __half2float(qh16[i]);
                kk[i] = make_float2(kf, kf);
                qq[i] = make_float2(qf, qf);
            }
            const float2 gate = gates[pp];
            const float2 dd = make_float2(gate.x, gate.x);
            float2 kv = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                st[i] = __fmul2_rn(st[i], dd);
                kv = __fadd2_rn(kv, __fmul2_rn(st[i], kk[i]));
            }
            const float red = simd_sum4_grouped(kv.x, kv.y, o_prev.x, o_prev.y, lane);
            keep = (lane & 7) == pp ? red : keep;
            const float2 neg_kv = make_float2(-__shfl_sync(0xffffffffu, red, 0), -__shfl_sync(0xffffffffu, red, 8));
            const float2 delta = __fmul2_rn(__fadd2_rn(make_float2(__half2float(vh[0]), __half2float(vh[1])), neg_kv), make_float2(gate.y, gate.y));
            float2 o = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                st[i] = __fadd2_rn(st[i], __fmul2_rn(kk[i], delta));
                o = __fadd2_rn(o, __fmul2_rn(st[i], qq[i]));
            }
            o_prev = o;
            if (CHECKPOINT) {
#pragma unroll
                for (int i = 0; i < EPL; ++i) {
                    const __half h0 = __float2half_rn(st[i].x), h1 = __float2half_rn(st[i].y);
                    history[(size_t)(p0 + pp + 1) * hs + row_off + i] = h0;
                    history[(size_t)(p0 + pp + 1) * hs + row_off + D + i] = h1;
                    st[i] = make_float2(__half2float(h0), __half2float(h1));
                }
            }
        };
        if (np == PB) {
#pragma unroll
            for (int pp = 0; pp < PB; ++pp) step(pp);
        } else {
            for (int pp = 0; pp < np; ++pp) step(pp);
        }
        {
            const int prev = p0 + (lane & 7) - 1;  // the position whose sums lanes 16 + pp and 24 + pp kept
            if (lane >= 16 && (lane & 7) < np && prev >= 0) out[((size_t)prev * value_heads + head) * D + dv0 + ((lane >> 3) & 1)] = __float2half_rn(keep);
        }
    }
    cp_async_wait<0>();  // nothing of this CTA's may still be in flight when its shared memory retires
    if (seq_len > 0) {
        const float red = simd_sum4_grouped(o_prev.x, o_prev.y, 0.0f, 0.0f, lane);
        if ((lane & 7) == 0 && lane < 16) out[((size_t)(seq_len - 1) * value_heads + head) * D + dv0 + (lane >> 3)] = __float2half_rn(red);
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        state[row_off + i] = __float2half_rn(st[i].x);
        state[row_off + D + i] = __float2half_rn(st[i].y);
    }
}

// One warp per head; may run in place.  tgs: the threadgroup width whose summation order the sum of
// squares follows (rms_norm_gated); precise: rms_norm_gated_d128's arithmetic (head_dim 128).
__global__ void rms_norm_gated_kernel(const __half* input, const __half* gate, const __half* weight, __half* out, int head_dim, float eps,
                                      int tgs, int precise, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int lane = threadIdx.x;
    const size_t off = (size_t)blockIdx.x * head_dim;
    const float rs = precise ? gated_norm_d128_rs(input + off, eps, lane) : gated_norm_rs(input + off, head_dim, eps, tgs, lane);
    for (int i = lane; i < head_dim; i += 32)
        out[off + i] = precise ? gated_norm_d128_value(input[off + i], gate[off + i], weight[i], rs)
                               : gated_norm_value(input[off + i], gate[off + i], weight[i], rs);
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

}  // namespace

cudaError_t launch_conv1d_update_silu(const Launch& l, __half* state, const __half* new_val, const __half* weight, __half* out, int channels,
                                      int kernel_size) {
    if (channels <= 0 || kernel_size <= 0 || kernel_size > 8) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3((channels + 255) / 256), dim3(256));
    prefer_max_shared(conv1d_update_silu_kernel);
    return cudaLaunchKernelEx(&cfg, conv1d_update_silu_kernel, state, new_val, weight, out, channels, kernel_size, dev_dyn(l));
}

cudaError_t launch_rms_scale_qk(const Launch& l, __half* qkv, int head_dim, float eps, int qkv_dim, int qk_heads, int batch) {
    if (head_dim <= 0 || qk_heads <= 0 || batch <= 0 || 2 * qk_heads * head_dim > qkv_dim) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3(2 * qk_heads, batch), dim3(32));
    prefer_max_shared(rms_scale_qk_kernel);
    return cudaLaunchKernelEx(&cfg, rms_scale_qk_kernel, qkv, head_dim, eps, qkv_dim, qk_heads, dev_dyn(l));
}

cudaError_t launch_deltanet_recurrence_decode(const Launch& l, __half* state, const __half* qkv, const __half* b_proj, const __half* a_proj,
                                              const __half* a_log, const __half* dt_bias, __half* out, int head_dim, int value_heads,
                                              int qk_heads) {
    if (head_dim <= 0 || head_dim % 32 || head_dim > 256 || value_heads <= 0 || qk_heads <= 0 || value_heads % qk_heads) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3((head_dim + 7) / 8, value_heads), dim3(256));
#define SMELT_DN_CASE(E)                                                                                                                     \
    case E:                                                                                                                                  \
        prefer_max_shared(deltanet_recurrence_decode_kernel<E>);                                                                             \
        return cudaLaunchKernelEx(&cfg, deltanet_recurrence_decode_kernel<E>, state, qkv, b_proj, a_proj, a_log, dt_bias, out, value_heads, \
                                  qk_heads, dev_dyn(l));
    switch (head_dim / 32) {
        SMELT_DN_CASE(1) SMELT_DN_CASE(2) SMELT_DN_CASE(3) SMELT_DN_CASE(4) SMELT_DN_CASE(5) SMELT_DN_CASE(6) SMELT_DN_CASE(7) SMELT_DN_CASE(8)
        default: return cudaErrorInvalidValue;
    }
#undef SMELT_DN_CASE
}

cudaError_t launch_conv1d_update_silu_prefill(const Launch& l, __half* state, __half* qkv, const __half* weight, int seq_len, int channels,
                                              int kernel_size, __half* history) {
    if (channels <= 0 || kernel_size <= 0 || kernel_size > 8 || seq_len < 0) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3((channels + 127) / 128), dim3(128));
    if (kernel_size == 4) {
        prefer_max_shared(conv1d_update_silu_prefill_kernel<4>);
        return cudaLaunchKernelEx(&cfg, conv1d_update_silu_prefill_kernel<4>, state, qkv, weight, seq_len, channels, kernel_size, history, dev_dyn(l));
    }
    prefer_max_shared(conv1d_update_silu_prefill_kernel<0>);
    return cudaLaunchKernelEx(&cfg, conv1d_update_silu_prefill_kernel<0>, state, qkv, weight, seq_len, channels, kernel_size, history, dev_dyn(l));
}

cudaError_t launch_deltanet_recurrence_prefill(const Launch& l, __half* state, const __half* qkv, const __half* b_proj, const __half* a_proj,
                                               const __half* a_log, const __half* dt_bias, __half* out, int head_dim, int value_heads,
                                               int qk_heads, int seq_len, __half* history) {
    if (head_dim <= 0 || head_dim % 32 || head_dim > 256 || value_heads <= 0 || qk_heads <= 0 || value_heads % qk_heads || seq_len < 0)
        return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3(head_dim / (kDnWarps * kDnRows), value_heads), dim3(kDnWarps * 32));
    cfg.dynamicSmemBytes = dn_smem_bytes(head_dim);  // at most 33.5 KB: below the limit that needs an opt-in
    // 16-byte aligned operands take vector loads (every row offset is a multiple of 64 bytes)
    const int vec = ((reinterpret_cast<uintptr_t>(state) | reinterpret_cast<uintptr_t>(qkv)) & 15u) == 0;
#define SMELT_DN_CASE(E)                                                                                                                   \
    case E:                                                                                                                                \
        if (history) {                                                                                                                     \
            prefer_max_shared(deltanet_recurrence_prefill_kernel<E, true>);                                                                \
            return cudaLaunchKernelEx(&cfg, deltanet_recurrence_prefill_kernel<E, true>, state, qkv, b_proj, a_proj, a_log, dt_bias, out, \
                                      value_heads, qk_heads, seq_len, history, vec, dev_dyn(l));                                          \
        }                                                                                                                                  \
        prefer_max_shared(deltanet_recurrence_prefill_kernel<E, false>);                                                                   \
        return cudaLaunchKernelEx(&cfg, deltanet_recurrence_prefill_kernel<E, false>, state, qkv, b_proj, a_proj, a_log, dt_bias, out,    \
                                  value_heads, qk_heads, seq_len, history, vec, dev_dyn(l));
    switch (head_dim / 32) {
        SMELT_DN_CASE(1) SMELT_DN_CASE(2) SMELT_DN_CASE(3) SMELT_DN_CASE(4) SMELT_DN_CASE(5) SMELT_DN_CASE(6) SMELT_DN_CASE(7) SMELT_DN_CASE(8)
        default: return cudaErrorInvalidValue;
    }
#undef SMELT_DN_CASE
}

cudaError_t launch_rms_norm_gated(const Launch& l, const __half* input, const __half* gate, const __half* weight, __half* out, int head_dim,
                                  float eps, int heads, int tgs, bool precise_d128) {
    if (head_dim <= 0 || heads <= 0 || tgs < 32 || tgs % 32 || tgs > 1024 || (precise_d128 && head_dim != 128)) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3(heads), dim3(32));
    prefer_max_shared(rms_norm_gated_kernel);
    return cudaLaunchKernelEx(&cfg, rms_norm_gated_kernel, input, gate, weight, out, head_dim, eps, tgs, precise_d128 ? 1 : 0, dev_dyn(l));
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

smelt_status smelt_cuda_conv1d_update_silu(smelt_cuda_ctx* ctx, void* state, const void* new_val, const void* weight, void* out, int channels,
                                           int kernel_size) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!state || !new_val || !weight || !out || channels <= 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "conv1d update: bad arguments");
    if (kernel_size <= 0 || kernel_size > 8) return fail(ctx, SMELT_ERR_UNSUPPORTED, "conv1d update: kernel size in 1..8");
    return check_cuda(ctx, launch_conv1d_update_silu(typed(ctx), (__half*)state, (const __half*)new_val, (const __half*)weight, (__half*)out, channels, kernel_size), "conv1d update");
}

smelt_status smelt_cuda_rms_scale_qk(smelt_cuda_ctx* ctx, void* qkv, int head_dim, float eps, int qkv_dim, int qk_heads, int batch) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!qkv || head_dim <= 0 || qk_heads <= 0 || batch <= 0 || 2 * qk_heads * head_dim > qkv_dim) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "rms scale q / k: bad arguments");
    return check_cuda(ctx, launch_rms_scale_qk(typed(ctx), (__half*)qkv, head_dim, eps, qkv_dim, qk_heads, batch), "rms scale q / k");
}

smelt_status smelt_cuda_deltanet_recurrence_decode(smelt_cuda_ctx* ctx, void* state, const void* qkv, const void* b_proj, const void* a_proj,
                                                   const void* a_log, const void* dt_bias, void* out, int head_dim, int value_heads,
                                                   int qk_heads) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!state || !qkv || !b_proj || !a_proj || !a_log || !dt_bias || !out || value_heads <= 0 || qk_heads <= 0 || value_heads % qk_heads)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "deltanet recurrence: bad arguments");
    if (head_dim <= 0 || head_dim % 32 || head_dim > 256) return fail(ctx, SMELT_ERR_UNSUPPORTED, "deltanet recurrence: head_dim a multiple of 32, at most 256");
    return check_cuda(ctx, launch_deltanet_recurrence_decode(typed(ctx), (__half*)state, (const __half*)qkv, (const __half*)b_proj, (const __half*)a_proj,
                                                             (const __half*)a_log, (const __half*)dt_bias, (__half*)out, head_dim, value_heads, qk_heads),
                      "deltanet recurrence");
}

smelt_status smelt_cuda_conv1d_update_silu_prefill(smelt_cuda_ctx* ctx, void* state, void* qkv, const void* weight, int seq_len, int channels,
                                                   int kernel_size, void* history) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!state || !qkv || !weight || channels <= 0 || seq_len < 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "conv1d prefill: bad arguments");
    if (kernel_size <= 0 || kernel_size > 8) return fail(ctx, SMELT_ERR_UNSUPPORTED, "conv1d prefill: kernel size in 1..8");
    return check_cuda(ctx, launch_conv1d_update_silu_prefill(typed(ctx), (__half*)state, (__half*)qkv, (const __half*)weight, seq_len, channels, kernel_size, (__half*)history),
                      "conv1d prefill");
}

smelt_status smelt_cuda_deltanet_recurrence_prefill(smelt_cuda_ctx* ctx, void* state, const void* qkv, const void* b_proj, const void* a_proj,
                                                    const void* a_log, const void* dt_bias, void* out, int head_dim, int value_heads,
                                                    int qk_heads, int seq_len, void* history) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!state || !qkv || !b_proj || !a_proj || !a_log || !dt_bias || !out || value_heads <= 0 || qk_heads <= 0 || value_heads % qk_heads || seq_len < 0)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "deltanet prefill recurrence: bad arguments");
    if (head_dim <= 0 || head_dim % 32 || head_dim > 256) return fail(ctx, SMELT_ERR_UNSUPPORTED, "deltanet prefill recurrence: head_dim a multiple of 32, at most 256");
    return check_cuda(ctx, launch_deltanet_recurrence_prefill(typed(ctx), (__half*)state, (const __half*)qkv, (const __half*)b_proj, (const __half*)a_proj,
                                                              (const __half*)a_log, (const __half*)dt_bias, (__half*)out, head_dim, value_heads, qk_heads,
                                                              seq_len, (__half*)history),
                      "deltanet prefill recurrence");
}

smelt_status smelt_cuda_rms_norm_gated(smelt_cuda_ctx* ctx, const void* input, const void* gate, const void* weight, void* out, int head_dim,
                                       float eps, int heads) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!input || !gate || !weight || !out || head_dim <= 0 || heads <= 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "gated rms norm: bad arguments");
    return check_cuda(ctx, launch_rms_norm_gated(typed(ctx), (const __half*)input, (const __half*)gate, (const __half*)weight, (__half*)out, head_dim, eps, heads, 32, false), "gated rms norm");
}

smelt_status smelt_cuda_rms_norm_gated_ex(smelt_cuda_ctx* ctx, const void* input, const void* gate, const void* weight, void* out, int head_dim,
                                          float eps, int heads, int threadgroup_width, int precise_d128) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!input || !gate || !weight || !out || head_dim <= 0 || heads <= 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "gated rms norm: bad arguments");
    if (threadgroup_width < 32 || threadgroup_width % 32 || threadgroup_width > 1024) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "gated rms norm: threadgroup width a multiple of 32 up to 1024");
    if (precise_d128 && head_dim != 128) return fail(ctx, SMELT_ERR_UNSUPPORTED, "gated rms norm: the precise form is for heads of 128");
    return check_cuda(ctx, launch_rms_norm_gated(typed(ctx), (const __half*)input, (const __half*)gate, (const __half*)weight, (__half*)out, head_dim, eps, heads,
                                                 threadgroup_width, precise_d128 != 0), "gated rms norm");
}

}  // extern "C"
