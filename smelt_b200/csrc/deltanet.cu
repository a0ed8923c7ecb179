// The decode step of a DeltaNet (gated linear-attention) layer: the four kernels the reference's
// emitter dispatches between the layer's input projections and its output projection
// (Sources/SmeltCompiler/DeltaNetPlugin.swift:196-318):
//   conv1d_update_silu   Resources/Shaders/conv1d.metal:271-331   depthwise conv state shift + SiLU
//   rms_scale_qk         Resources/Shaders/norms.metal:1380-1431  Q / K RMS scaling with their edge scales
//   deltanet_recurrence_mlx_decode (and its _d128_h16 / _d128_h32_qk16 / _d128_h48_qk16
//                        specialisations) Resources/Shaders/recurrence.metal:511-836
//   rms_norm_gated (and rms_norm_gated_d128) Resources/Shaders/norms.metal:1093-1143
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

// One warp per head: out = half(w * (x * rsqrt(mean(x^2) + eps)) * silu(g)); may run in place.
__global__ void rms_norm_gated_kernel(const __half* input, const __half* gate, const __half* weight, __half* out, int head_dim, float eps,
                                      DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int lane = threadIdx.x;
    const size_t off = (size_t)blockIdx.x * head_dim;
    float sum = 0.0f;
    for (int i = lane; i < head_dim; i += 32) {
        const float v = __half2float(input[off + i]);
        sum += v * v;
    }
    sum = warp_sum(sum);
    const float rs = __frcp_rn(__fsqrt_rn(sum / (float)head_dim + eps));
    for (int i = lane; i < head_dim; i += 32) {
        const float x = __half2float(input[off + i]), g = __half2float(gate[off + i]);
        const float silu = g / (1.0f + expf(-g));
        out[off + i] = __float2half_rn(__half2float(weight[i]) * (x * rs) * silu);
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

cudaError_t launch_rms_norm_gated(const Launch& l, const __half* input, const __half* gate, const __half* weight, __half* out, int head_dim,
                                  float eps, int heads) {
    if (head_dim <= 0 || heads <= 0) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3(heads), dim3(32));
    prefer_max_shared(rms_norm_gated_kernel);
    return cudaLaunchKernelEx(&cfg, rms_norm_gated_kernel, input, gate, weight, out, head_dim, eps, dev_dyn(l));
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

smelt_status smelt_cuda_rms_norm_gated(smelt_cuda_ctx* ctx, const void* input, const void* gate, const void* weight, void* out, int head_dim,
                                       float eps, int heads) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!input || !gate || !weight || !out || head_dim <= 0 || heads <= 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "gated rms norm: bad arguments");
    return check_cuda(ctx, launch_rms_norm_gated(typed(ctx), (const __half*)input, (const __half*)gate, (const __half*)weight, (__half*)out, head_dim, eps, heads), "gated rms norm");
}

}  // extern "C"
