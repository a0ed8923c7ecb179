// The small kernels between the projections of a layer: element-wise activations and products,
// the per-head RMS norms with their reduction topologies, the gate split of a gated attention
// layer.  They move a few kilobytes each; what matters is that a package that names them runs and
// that their arithmetic, fp16 roundings included, is the reference's.
//   Resources/Shaders/activations.metal:4-210        silu, sigmoid_kernel, softplus, buffer_copy,
//                                                     projection_bias_add_batched, elementwise_mul, scalar_mul,
//                                                     scalar_mul_weight, geglu_fused(_strided_batched), logit_cap
//   Resources/Shaders/activations_precise.metal:22-35 sigmoid_mul (half arithmetic)
//   Resources/Shaders/attention_fused.metal:11-330    gate_split, per_head_rms_norm[_1pw | _noscale][_batched]
//   Resources/Shaders/norms.metal:72-1090, :1155-1550 the shape-specialised and batched rms_norm_1pw forms, the
//                                                     scale-only norms, l2_normalize
#include <string>

#include "common.cuh"
#include "glue.h"
#include "runtime.h"

namespace smelt {

namespace {

// a / y [batch, count]; b per op: [batch, count] (mul, sigmoid_mul), rows of b_stride (geglu), [count] (bias add),
// one fp16 value (scalar_mul_weight passes it as `scalar_dev`).
template <int OP>
__global__ void __launch_bounds__(256) elementwise_kernel(const __half* a, const __half* b, __half* y, int count, int b_stride, float scalar,
                                                          const __half* scalar_dev, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const size_t idx = (size_t)blockIdx.y * count + i;
    const float x = __half2float(a[idx]);
    __half o;
    if (OP == kEwSilu) o = __float2half_rn(__fdiv_rn(x, __fadd_rn(1.0f, expf(-x))));
    else if (OP == kEwSigmoid) o = __float2half_rn(__fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))));
    else if (OP == kEwSoftplus) o = __float2half_rn(x > 20.0f ? x : logf(__fadd_rn(1.0f, expf(x))));
    else if (OP == kEwCopy) o = a[idx];
    else if (OP == kEwScalarMul) o = __float2half_rn(__fmul_rn(x, scalar_dev ? __half2float(scalar_dev[0]) : scalar));
    else if (OP == kEwLogitCap) o = __float2half_rn(__fmul_rn(scalar, tanhf(__fdiv_rn(x, scalar))));
    else if (OP == kEwMul) o = __hmul(a[idx], b[idx]);
    else if (OP == kEwSigmoidMul) {
        const __half g = b[idx];
        const __half one = __float2half_rn(1.0f);
        const __half tail = __hdiv(one, __hadd(one, __float2half_rn(expf(fabsf(__half2float(g))))));
        o = __hmul(a[idx], __half2float(g) < 0.0f ? tail : __hsub(one, tail));
    } else if (OP == kEwGeglu) {
        const float u = __half2float(b[(size_t)blockIdx.y * b_stride + i]);
        float inner = __fmul_rn(0.7978845608f, __fadd_rn(x, __fmul_rn(0.044715f, __fmul_rn(__fmul_rn(x, x), x))));
        inner = fminf(fmaxf(inner, -20.0f), 20.0f);
        const float gelu = __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, tanhf(inner)));
        o = __float2half_rn(fminf(fmaxf(__fmul_rn(gelu, u), -65504.0f), 65504.0f));
    } else {
        o = __hadd(a[idx], b[i]);
    }
    y[idx] = o;
}

__global__ void __launch_bounds__(256) gate_split_kernel(const __half* in, __half* query, __half* gate, int head_dim, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= head_dim) return;
    const size_t head = blockIdx.y;
    query[head * head_dim + d] = in[head * head_dim * 2 + d];
    gate[head * head_dim + d] = in[head * head_dim * 2 + head_dim + d];
}

// One warp per head.  MODE 0: four adjacent squares per thread, a simdgroup per 128 values, the simdgroups' sums
// summed by simd_sum; y = w * half(x * rs).  MODE 1 / 2: thread t of a threadgroup of tgs adds x[t]^2, x[t + tgs]^2,
// ..., simdgroup sums added in order; y = half(x * rs * (1 + w)) / half(x * rs).  May run in place: every value is
// read before the first is written (a warp holds a head of up to 1024 values in registers).
template <int MODE>
__global__ void __launch_bounds__(32) head_norm_kernel(const __half* x, const __half* w, __half* y, int head_dim, float eps, int tgs, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int lane = threadIdx.x;
    const __half* xh = x + (size_t)blockIdx.x * head_dim;
    __half* yh = y + (size_t)blockIdx.x * head_dim;
    float total;
    if (MODE == 0) {
        float mine = 0.0f;  // lane s ends up with simdgroup s's sum
        for (int s = 0; s * 128 < head_dim; ++s) {
            float p = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int e = s * 128 + 4 * lane + i;
                const float v = e < head_dim ? __half2float(xh[e]) : 0.0f;
                p = __fadd_rn(p, __fmul_rn(v, v));
            }
            const float part = __shfl_sync(0xffffffffu, simd_sum_lane0(p), 0);
            if (lane == s) mine = part;
        }
        total = __shfl_sync(0xffffffffu, simd_sum_lane0(mine), 0);
    } else {
        total = 0.0f;
        for (int s = 0; s < tgs / 32; ++s) {
            float p = 0.0f;
            for (int i = s * 32 + lane; i < head_dim; i += tgs) {
                const float v = __half2float(xh[i]);
                p = __fadd_rn(p, __fmul_rn(v, v));
            }
            total = __fadd_rn(total, __shfl_sync(0xffffffffu, simd_sum_lane0(p), 0));
        }
    }
    const float rs = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)head_dim), eps)));
    __half vals[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) {
        const int i = lane + 32 * k;
        vals[k] = i < head_dim ? xh[i] : __ushort_as_half(0);
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 32; ++k) {
        const int i = lane + 32 * k;
        if (i >= head_dim) break;
        const float v = __half2float(vals[k]);
        if (MODE == 0) yh[i] = __hmul(w[i], __float2half_rn(__fmul_rn(v, rs)));
        else if (MODE == 1) yh[i] = __float2half_rn(__fmul_rn(__fmul_rn(v, rs), __fadd_rn(1.0f, __half2float(w[i]))));
        else yh[i] = __float2half_rn(__fmul_rn(v, rs));
    }
}

// The row norms of norms.metal beyond rms_norm_1pw (norms.metal:72-1090, :1155-1190, :1436-1550): one warp per
// row plays the threadgroup, simdgroup after simdgroup, so that the sum of squares is added in the kernel's own
// order.  topology 0: thread t of tgs adds its four adjacent values of every tile of 4 tgs; the simdgroups' sums
// are summed by simd_sum.  1: dim / 8 threads, thread t takes dot(x0, x0) + dot(x1, x1) of the quads t and
// t + dim / 8; simdgroup sums added in order.  2: thread t adds x[t]^2, x[t + tgs]^2, ...; sums added in order.
// scale 0: rsqrt(total / dim + eps); 1: 1 / max(sqrt(total), eps).  value 0: the scale only; 1: half(1 + w) *
// half(x * rs); 2: half(x * (rs * (1 + w))); 3: half(x * rs * (1 + w)); 4: half(x * rs).  pre: the row is
// half(x + pre), also written to y when value is 0.  residual / scalar: applied to the rounded norm.
struct RowNormArgs {
    const __half* x; const __half* pre; const __half* w; const __half* residual; const __half* scalar;
    __half* y; float* scale_out;
    int dim, tgs, topology, value, scale;
    float eps;
    int group_rows, group_stride;  // rows come in groups of group_rows adjacent rows, group_stride values apart (0: all rows adjacent)
};

__global__ void __launch_bounds__(32) row_norm_kernel(const RowNormArgs a, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int lane = threadIdx.x;
    const size_t off = a.group_rows ? (size_t)(blockIdx.x / a.group_rows) * a.group_stride + (size_t)(blockIdx.x % a.group_rows) * a.dim : (size_t)blockIdx.x * a.dim;
    const __half* x = a.x + off;
    auto val = [&](int i) -> float {
        if (a.pre) return __half2float(__hadd(x[i], a.pre[off + i]));
        return __half2float(x[i]);
    };
    float total = 0.0f, mine = 0.0f;
    for (int s = 0; s < a.tgs / 32; ++s) {
        const int t = 32 * s + lane;
        float p = 0.0f;
        if (a.topology == 0) {
            for (int tile = 0; tile < a.dim; tile += 4 * a.tgs)
                for (int k = 0; k < 4; ++k) {
                    const int i = tile + 4 * t + k;
                    if (i < a.dim) { const float v = val(i); p = __fadd_rn(p, __fmul_rn(v, v)); }
                }
        } else if (a.topology == 1) {
            float d[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int b = 4 * (t + h * a.tgs);
                const float v0 = val(b), v1 = val(b + 1), v2 = val(b + 2), v3 = val(b + 3);
                d[h] = __fadd_rn(__fadd_rn(__fadd_rn(__fmul_rn(v0, v0), __fmul_rn(v1, v1)), __fmul_rn(v2, v2)), __fmul_rn(v3, v3));
            }
            p = __fadd_rn(d[0], d[1]);
        } else {
            for (int i = t; i < a.dim; i += a.tgs) { const float v = val(i); p = __fadd_rn(p, __fmul_rn(v, v)); }
        }
        const float part = __shfl_sync(0xffffffffu, simd_sum_lane0(p), 0);
        if (a.topology == 0) { if (lane == s) mine = part; }
        else total = __fadd_rn(total, part);
    }
    if (a.topology == 0) total = __shfl_sync(0xffffffffu, simd_sum_lane0(mine), 0);
    const float rs = a.scale == 0 ? __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)a.dim), a.eps))) : __frcp_rn(fmaxf(__fsqrt_rn(total), a.eps));
    if (lane == 0 && a.scale_out) a.scale_out[blockIdx.x] = rs;
    if (a.value == 0) {
        if (a.pre && a.y)
            for (int i = lane; i < a.dim; i += 32) a.y[off + i] = __hadd(x[i], a.pre[off + i]);
        return;
    }
    // in place is allowed: position i is read and written by the same lane, after the whole row was summed
    __syncwarp();
    for (int i = lane; i < a.dim; i += 32) {
        const float v = val(i);
        const float wv = a.w ? __half2float(a.w[i]) : 0.0f;
        __half o;
        if (a.value == 1) o = __hmul(__float2half_rn(__fadd_rn(1.0f, wv)), __float2half_rn(__fmul_rn(v, rs)));
        else if (a.value == 2) o = __float2half_rn(__fmul_rn(v, __fmul_rn(rs, __fadd_rn(1.0f, wv))));
        else if (a.value == 3) o = __float2half_rn(__fmul_rn(__fmul_rn(v, rs), __fadd_rn(1.0f, wv)));
        else o = __float2half_rn(__fmul_rn(v, rs));
        if (a.residual) o = __hadd(o, a.residual[off + i]);
        if (a.scalar) o = __float2half_rn(__fmul_rn(__half2float(o), __half2float(a.scalar[0])));
        a.y[off + i] = o;
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

template <int OP>
cudaError_t launch_ew(const Launch& l, const __half* a, const __half* b, __half* y, int count, int batch, int b_stride, float scalar, const __half* scalar_dev) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3((count + 255) / 256, batch), dim3(256));
    prefer_max_shared(elementwise_kernel<OP>);
    return cudaLaunchKernelEx(&cfg, elementwise_kernel<OP>, a, b, y, count, b_stride, scalar, scalar_dev, dev_dyn(l));
}

}  // namespace

cudaError_t launch_elementwise(const Launch& l, int op, const __half* a, const __half* b, __half* y, int count, int batch, int b_stride, float scalar,
                               const __half* scalar_dev) {
    if (count <= 0 || batch <= 0 || !a || !y) return cudaErrorInvalidValue;
    const bool needs_b = op == kEwMul || op == kEwSigmoidMul || op == kEwGeglu || op == kEwBiasAdd;
    if (needs_b && !b) return cudaErrorInvalidValue;
    switch (op) {
        case kEwSilu: return launch_ew<kEwSilu>(l, a, b, y, count, batch, b_stride, scalar, scalar_dev);
        case kEwSigmoid: return launch_ew<kEwSigmoid>(l, a, b, y, count, batch, b_stride, scalar, scalar_dev);
        case kEwSoftplus: return launch_ew<kEwSoftplus>(l, a, b, y, count, batch, b_stride, scalar, scalar_dev);
        case kEwCopy: return launch_ew<kEwCopy>(l, a, b, y, count, batch, b_stride, scalar, scalar_dev);
        case kEwScalarMul: return launch_ew<kEwScalarMul>(l, a, b, y, count, batch, b_stride, scalar, scalar_dev);
        case kEwLogitCap: return launch_ew<kEwLogitCap>(l, a, b, y, count, batch, b_stride, scalar, scalar_dev);
        case kEwMul: return launch_ew<kEwMul>(l, a, b, y, count, batch, b_stride, scalar, scalar_dev);
        case kEwSigmoidMul: return launch_ew<kEwSigmoidMul>(l, a, b, y, count, batch, b_stride, scalar, scalar_dev);
        case kEwGeglu: return launch_ew<kEwGeglu>(l, a, b, y, count, batch, b_stride, scalar, scalar_dev);
        case kEwBiasAdd: return launch_ew<kEwBiasAdd>(l, a, b, y, count, batch, b_stride, scalar, scalar_dev);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_gate_split(const Launch& l, const __half* in, __half* query, __half* gate, int heads, int head_dim) {
    if (heads <= 0 || head_dim <= 0) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3((head_dim + 255) / 256, heads), dim3(256));
    prefer_max_shared(gate_split_kernel);
    return cudaLaunchKernelEx(&cfg, gate_split_kernel, in, query, gate, head_dim, dev_dyn(l));
}

cudaError_t launch_head_norm(const Launch& l, int mode, const __half* x, const __half* w, __half* y, int heads, int head_dim, float eps, int tgs) {
    if (heads <= 0 || head_dim <= 0 || head_dim > 1024 || tgs < 32 || tgs % 32 || tgs > 1024 || (mode != kHeadNormNoScale && !w)) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3(heads), dim3(32));
    switch (mode) {
        case kHeadNormDirect: prefer_max_shared(head_norm_kernel<0>); return cudaLaunchKernelEx(&cfg, head_norm_kernel<0>, x, w, y, head_dim, eps, tgs, dev_dyn(l));
        case kHeadNorm1pw: prefer_max_shared(head_norm_kernel<1>); return cudaLaunchKernelEx(&cfg, head_norm_kernel<1>, x, w, y, head_dim, eps, tgs, dev_dyn(l));
        case kHeadNormNoScale: prefer_max_shared(head_norm_kernel<2>); return cudaLaunchKernelEx(&cfg, head_norm_kernel<2>, x, w, y, head_dim, eps, tgs, dev_dyn(l));
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_row_norm(const Launch& l, const __half* x, const __half* pre, const __half* w, const __half* residual, const __half* scalar, __half* y,
                            float* scale_out, int rows, int dim, float eps, int topology, int tgs, int value, int scale, int group_rows, int group_stride) {
    if (rows <= 0 || dim <= 0 || !x || topology < 0 || topology > 2 || value < 0 || value > 4 || scale < 0 || scale > 1) return cudaErrorInvalidValue;
    if (topology == 1) {
        if (dim % 256) return cudaErrorInvalidValue;
        tgs = dim / 8;
    }
    if (tgs < 32 || tgs % 32 || tgs > 1024 || (value && !y) || (!value && !scale_out && !pre)) return cudaErrorInvalidValue;
    if ((value == 1 || value == 2 || value == 3) && !w) return cudaErrorInvalidValue;
    if (group_rows < 0 || (group_rows > 0 && (group_stride < group_rows * dim || rows % group_rows))) return cudaErrorInvalidValue;
    RowNormArgs a = {x, pre, w, residual, scalar, y, scale_out, dim, tgs, topology, value, scale, eps, group_rows, group_stride};
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3(rows), dim3(32));
    prefer_max_shared(row_norm_kernel);
    return cudaLaunchKernelEx(&cfg, row_norm_kernel, a, dev_dyn(l));
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

smelt_status smelt_cuda_elementwise(smelt_cuda_ctx* ctx, int op, const void* a, const void* b, void* y, int count, int batch, int b_stride, float scalar) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!a || !y || count <= 0 || batch <= 0 || op < 0 || op > SMELT_EW_SCALAR_MUL_WEIGHT) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "elementwise: bad arguments");
    const bool needs_b = op == SMELT_EW_MUL || op == SMELT_EW_SIGMOID_MUL || op == SMELT_EW_GEGLU || op == SMELT_EW_BIAS_ADD || op == SMELT_EW_SCALAR_MUL_WEIGHT;
    if (needs_b && !b) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "elementwise: the second operand is missing");
    if (op == SMELT_EW_SCALAR_MUL_WEIGHT)
        return check_cuda(ctx, launch_elementwise(typed(ctx), kEwScalarMul, (const __half*)a, nullptr, (__half*)y, count, batch, count, 0.0f, (const __half*)b), "elementwise");
    return check_cuda(ctx, launch_elementwise(typed(ctx), op, (const __half*)a, (const __half*)b, (__half*)y, count, batch, b_stride > 0 ? b_stride : count, scalar, nullptr), "elementwise");
}

smelt_status smelt_cuda_gate_split(smelt_cuda_ctx* ctx, const void* input, void* query, void* gate, int heads, int head_dim) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!input || !query || !gate || heads <= 0 || head_dim <= 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "gate split: bad arguments");
    return check_cuda(ctx, launch_gate_split(typed(ctx), (const __half*)input, (__half*)query, (__half*)gate, heads, head_dim), "gate split");
}

smelt_status smelt_cuda_head_norm(smelt_cuda_ctx* ctx, int mode, const void* x, const void* w, void* y, int heads, int head_dim, float eps,
                                  int threadgroup_width) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!x || !y || heads <= 0 || head_dim <= 0 || mode < 0 || mode > 2 || (mode != SMELT_HEAD_NORM_NOSCALE && !w)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "head norm: bad arguments");
    if (head_dim > 1024) return fail(ctx, SMELT_ERR_UNSUPPORTED, "head norm: heads of up to 1024 values");
    if (threadgroup_width < 32 || threadgroup_width % 32 || threadgroup_width > 1024) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "head norm: threadgroup width a multiple of 32 up to 1024");
    return check_cuda(ctx, launch_head_norm(typed(ctx), mode, (const __half*)x, (const __half*)w, (__half*)y, heads, head_dim, eps, threadgroup_width), "head norm");
}

smelt_status smelt_cuda_row_norm(smelt_cuda_ctx* ctx, const void* x, const void* pre, const void* w, const void* residual, const void* scalar, void* y,
                                 void* scale_out, int rows, int dim, float eps, int topology, int threadgroup_width, int value, int scale) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!x || rows <= 0 || dim <= 0 || topology < 0 || topology > 2 || value < 0 || value > 4 || scale < 0 || scale > 1 || (value && !y) ||
        ((value == 1 || value == 2 || value == 3) && !w) || (!value && !scale_out && !pre))
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "row norm: bad arguments");
    if (topology == 1 && dim % 256) return fail(ctx, SMELT_ERR_UNSUPPORTED, "row norm: the two-quads-per-thread form needs a multiple of 256 values");
    if (topology != 1 && (threadgroup_width < 32 || threadgroup_width % 32 || threadgroup_width > 1024)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "row norm: threadgroup width a multiple of 32 up to 1024");
    if (scale_out && (reinterpret_cast<uintptr_t>(scale_out) & 3u)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "row norm: the scale output must be 4-byte aligned");
    return check_cuda(ctx, launch_row_norm(typed(ctx), (const __half*)x, (const __half*)pre, (const __half*)w, (const __half*)residual, (const __half*)scalar, (__half*)y,
                                           (float*)scale_out, rows, dim, eps, topology, threadgroup_width, value, scale, 0, 0), "row norm");
}

}  // extern "C"
