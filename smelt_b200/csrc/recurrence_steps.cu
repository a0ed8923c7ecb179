// The DeltaNet step as the reference's older pipelines cut it
// (Resources/Shaders/recurrence.metal:44-503, :836-862; Resources/Shaders/prefill_recurrence.metal:42-285):
//   compute_gates, state_decay, kv_mem_readout, compute_delta, outer_product_update, query_readout
//   kv_readout_delta, gates_kv_readout_delta, state_decay_update        (pairs of the above in one pass)
//   deltanet_recurrence_fused       conv1d + SiLU, L2 norms, gates, recurrence, gated RMS norm: one decode step
//   deltanet_recurrence_prefill     conv1d + SiLU, L2 norms, gates, recurrence over the positions of a prompt chunk
// The reference's kernel catalog still lists them (Sources/SmeltCompiler/SmeltKernelCatalog.swift:655-696, :829-925)
// while its emitters dispatch the tiled forms of deltanet.cu, so these are here for packages compiled
// before that change; they are written for correctness, one CTA per head as the Metal kernels run.
// The separate-launch kernels keep the state as [H, Dk, Dv] (state[k * D + v]); the two fused ones as
// [H, Dv, Dk].  Gates are plain fp32 (no staged fp16 roundings), sums over k run one term at a time in k
// order, and every product feeding a sum is rounded on its own (no fused multiply-add), as the CPU
// restatement of these kernels does.
#include <string>

#include "common.cuh"
#include "glue.h"
#include "runtime.h"

namespace smelt {

namespace {

__device__ __forceinline__ void plain_gates(__half b, __half a, __half a_log, __half dt_bias, float& beta, float& g) {
    beta = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-__half2float(b))));
    const float x = __fadd_rn(__half2float(a), __half2float(dt_bias));
    const float sp = x > 20.0f ? x : logf(__fadd_rn(1.0f, expf(x)));
    g = __fmul_rn(-expf(__half2float(a_log)), sp);
}

__device__ __forceinline__ float silu_f32(float x) { return __fdiv_rn(x, __fadd_rn(1.0f, expf(-x))); }

__global__ void dn_compute_gates_kernel(const __half* b_proj, const __half* a_proj, const __half* a_log, const __half* dt_bias,
                                        __half* beta_out, __half* g_out, int heads, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int h = blockIdx.x * blockDim.x + threadIdx.x;
    if (h >= heads) return;
    float beta, g;
    plain_gates(b_proj[h], a_proj[h], a_log[h], dt_bias[h], beta, g);
    beta_out[h] = __float2half_rn(beta);
    g_out[h] = __float2half_rn(g);
}

// state_decay (key == null), outer_product_update (g_val == null) and state_decay_update (both):
// grid (chunks of 1024 elements, heads).
__global__ void __launch_bounds__(256) dn_state_update_kernel(__half* state, const __half* g_val, const __half* key, const float* delta,
                                                              int head_dim, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int D = head_dim, head = blockIdx.y, n = D * D;
    const float decay = g_val ? expf(__half2float(g_val[head])) : 1.0f;
    __half* s = state + (size_t)head * n;
    for (int i = 0; i < 4; ++i) {
        const int idx = blockIdx.x * 1024 + i * 256 + threadIdx.x;
        if (idx >= n) break;
        const float old = __half2float(s[idx]);
        float v = g_val ? __fmul_rn(old, decay) : old;
        if (key) v = __fadd_rn(v, __fmul_rn(__half2float(key[(size_t)head * D + idx / D]), delta[(size_t)head * D + idx % D]));
        s[idx] = __float2half_rn(v);
    }
}

enum { kReadoutKvMem = 0, kReadoutDelta = 1, kReadoutGatesDelta = 2, kReadoutQuery = 3 };

struct ReadoutArgs {
    const __half* state;   // [H, Dk, Dv]
    const __half* vec;     // key or query [H, D]
    const __half* value;   // [H, D]
    const __half* g_val;   // [H]   (delta form)
    const __half* beta;    // [H]   (delta form)
    const __half* b_proj;  // [H]   (gates form) ...
    const __half* a_proj;
    const __half* a_log;
    const __half* dt_bias;
    float* out_f32;        // kv_mem or delta [H, D]
    __half* out_f16;       // query readout [H, D]
    __half* g_out;         // [H]   (gates form)
    int head_dim;
    float scale;           // query readout
};

// One CTA per head, thread v sums column v of the head's state over k.
template <int MODE>
__global__ void __launch_bounds__(256) dn_readout_kernel(const ReadoutArgs a, DevDyn dyn) {
    __shared__ float s_vec[256];
    __shared__ float s_gate[2];
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int D = a.head_dim, head = blockIdx.x, v = threadIdx.x;
    if (v < D) {
        const float x = __half2float(a.vec[(size_t)head * D + v]);
        s_vec[v] = MODE == kReadoutQuery ? __fmul_rn(x, a.scale) : x;
    }
    if (MODE == kReadoutGatesDelta && v == 0) {
        float beta, g;
        plain_gates(a.b_proj[head], a.a_proj[head], a.a_log[head], a.dt_bias[head], beta, g);
        s_gate[0] = expf(g);
        s_gate[1] = beta;
        a.g_out[head] = __float2half_rn(g);
    }
    __syncthreads();
    if (v >= D) return;
    const __half* col = a.state + (size_t)head * D * D + v;
    float acc = 0.0f;
#pragma unroll 8
    for (int k = 0; k < D; ++k) acc = __fadd_rn(acc, __fmul_rn(__half2float(col[(size_t)k * D]), s_vec[k]));
    const size_t o = (size_t)head * D + v;
    if (MODE == kReadoutKvMem) {
        a.out_f32[o] = acc;
    } else if (MODE == kReadoutQuery) {
        a.out_f16[o] = __float2half_rn(acc);
    } else {
        const float decay = MODE == kReadoutGatesDelta ? s_gate[0] : expf(__half2float(a.g_val[head]));
        const float beta = MODE == kReadoutGatesDelta ? s_gate[1] : __half2float(a.beta[head]);
        a.out_f32[o] = __fmul_rn(__fsub_rn(__half2float(a.value[o]), __fmul_rn(acc, decay)), beta);
    }
}

__global__ void dn_compute_delta_kernel(const __half* value, const float* kv_mem, const __half* beta, float* delta, int head_dim, int total,
                                        DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    delta[i] = __fmul_rn(__fsub_rn(__half2float(value[i]), kv_mem[i]), __half2float(beta[i / head_dim]));
}

// Sum over a head of x[i]^2 as a threadgroup of blockDim.x threads forms it in the fused kernels:
// thread t adds its elements t, t + tgs, ..., every warp sums its lanes as simd_sum does, thread 0
// adds the warps' sums one after the other.  The total is returned to every thread.  part: 33 floats.
__device__ __forceinline__ float cta_sumsq(const float* x, int n, float* part) {
    float p = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) p = __fadd_rn(p, __fmul_rn(x[i], x[i]));
    p = simd_sum_lane0(p);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = p;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int s = 0; s < (int)(blockDim.x >> 5); ++s) total = __fadd_rn(total, part[s]);
        part[32] = total;
    }
    __syncthreads();
    const float total = part[32];
    __syncthreads();  // part is reused by the next sum
    return total;
}

struct FusedArgs {
    __half* state;            // [H, Dv, Dk]
    const __half* qkv;        // decode: [qkv_dim]
    __half* qkv_rw;           // prefill: [T, qkv_dim], rewritten with the conv output and the normalised Q, K
    const __half* b_proj;     // [H] or [T, H]
    const __half* a_proj;
    const __half* a_log;      // [H]
    const __half* dt_bias;    // [H]
    __half* out;              // [H, D] or [T, H, D]
    __half* conv_state;       // [qkv_dim, conv_k]
    const __half* conv_weight;
    const __half* z_proj;     // decode: [H, D]
    const __half* norm_weight;  // decode: [D]
    int head_dim, heads, qkv_dim, conv_k, seq_len;
    float head_scale, eps;    // eps: rms epsilon (decode), L2 floor (prefill)
};

// Depthwise convolution step of channel ch: shifts its taps, appends x, returns silu(sum taps * weights).
__device__ __forceinline__ float conv_step(__half* st, const __half* w, int conv_k, __half x) {
    float acc = 0.0f;
    for (int t = 0; t < conv_k; ++t) {
        const __half c = t + 1 < conv_k ? st[t + 1] : x;
        st[t] = c;
        acc = __fadd_rn(acc, __fmul_rn(__half2float(c), __half2float(w[t])));
    }
    return silu_f32(acc);
}

// deltanet_recurrence_fused: one CTA of tgs threads per head; a warp owns one output row of the
// state at a time, lane l holding dk = l, l + 32, ...
__global__ void __launch_bounds__(1024) dn_fused_decode_kernel(const FusedArgs a, DevDyn dyn) {
    __shared__ float s_q[256], s_k[256], s_v[256], s_raw[256], s_part[33], s_gate[2];
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int D = a.head_dim, H = a.heads, head = blockIdx.x, tid = threadIdx.x, tgs = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, warps = tgs >> 5, epl = D / 32;
    for (int i = tid; i < 3 * D; i += tgs) {
        const int part = i / D, local = i - part * D;
        const int ch = part * H * D + head * D + local;
        const float act = conv_step(a.conv_state + (size_t)ch * a.conv_k, a.conv_weight + (size_t)ch * a.conv_k, a.conv_k, a.qkv[ch]);
        (part == 0 ? s_q : part == 1 ? s_k : s_v)[local] = act;
    }
    if (tid == 0) {
        float beta, g;
        plain_gates(a.b_proj[head], a.a_proj[head], a.a_log[head], a.dt_bias[head], beta, g);
        s_gate[0] = expf(g);
        s_gate[1] = beta;
    }
    __syncthreads();
    const float q_scale = __fdiv_rn(1.0f, fmaxf(__fsqrt_rn(cta_sumsq(s_q, D, s_part)), 1e-6f));
    const float k_scale = __fdiv_rn(1.0f, fmaxf(__fsqrt_rn(cta_sumsq(s_k, D, s_part)), 1e-6f));
    const float qs = __fmul_rn(q_scale, a.head_scale);
    for (int i = tid; i < D; i += tgs) {
        s_q[i] = __fmul_rn(s_q[i], qs);
        s_k[i] = __fmul_rn(s_k[i], k_scale);
    }
    __syncthreads();
    const float decay = s_gate[0], beta = s_gate[1];
    float kr[8], qr[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (i < epl) { kr[i] = s_k[i * 32 + lane]; qr[i] = s_q[i * 32 + lane]; }
    for (int row = warp; row < D; row += warps) {
        __half* srow = a.state + ((size_t)head * D + row) * D;
        float st[8];
        float kv = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i < epl) {
                st[i] = __fmul_rn(__half2float(srow[i * 32 + lane]), decay);
                kv = __fadd_rn(kv, __fmul_rn(st[i], kr[i]));
            }
        kv = __shfl_sync(0xffffffffu, simd_sum_lane0(kv), 0);
        const float delta = __fmul_rn(__fsub_rn(s_v[row], kv), beta);
        float o = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i < epl) {
                st[i] = __fadd_rn(st[i], __fmul_rn(kr[i], delta));
                o = __fadd_rn(o, __fmul_rn(st[i], qr[i]));
                srow[i * 32 + lane] = __float2half_rn(st[i]);
            }
        o = simd_sum_lane0(o);
        if (lane == 0) s_raw[row] = o;
    }
    __syncthreads();
    const float total = cta_sumsq(s_raw, D, s_part);
    const float rs = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)D), a.eps)));
    for (int i = tid; i < D; i += tgs) {
        const float z = __half2float(a.z_proj[(size_t)head * D + i]);
        a.out[(size_t)head * D + i] = __float2half_rn(__fmul_rn(__fmul_rn(__fmul_rn(s_raw[i], rs), __half2float(a.norm_weight[i])), silu_f32(z)));
    }
}

// deltanet_recurrence_prefill: one CTA per head walks the chunk's positions with the head's state
// [Dv, Dk] in shared memory (rows padded by two halves: a thread owns whole rows and neighbouring
// threads' rows fall into different banks).  Dynamic shared memory: D * (D + 2) halves.
__global__ void __launch_bounds__(1024) dn_fused_prefill_kernel(const FusedArgs a, DevDyn dyn) {
    extern __shared__ __align__(16) unsigned char dn_smem[];
    __shared__ float s_key[256], s_qs[256], s_x[256], s_part[33], s_gate[2];
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int D = a.head_dim, H = a.heads, HD = H * D, C = a.qkv_dim, head = blockIdx.x, tid = threadIdx.x, tgs = blockDim.x;
    const int pitch = D + 2;
    __half* S = reinterpret_cast<__half*>(dn_smem);
    __half* gstate = a.state + (size_t)head * D * D;
    for (int i = tid; i < D * D; i += tgs) S[(i / D) * pitch + i % D] = gstate[i];
    __syncthreads();
    for (int pos = 0; pos < a.seq_len; ++pos) {
        __half* x = a.qkv_rw + (size_t)pos * C;
        for (int i = tid; i < 3 * D; i += tgs) {
            const int part = i / D, local = i - part * D;
            const int ch = part * HD + head * D + local;
            x[ch] = __float2half_rn(conv_step(a.conv_state + (size_t)ch * a.conv_k, a.conv_weight + (size_t)ch * a.conv_k, a.conv_k, x[ch]));
        }
        if (tid == 0) {
            float beta, g;
            plain_gates(a.b_proj[(size_t)pos * H + head], a.a_proj[(size_t)pos * H + head], a.a_log[head], a.dt_bias[head], beta, g);
            s_gate[0] = expf(g);
            s_gate[1] = beta;
        }
        __syncthreads();
        for (int part = 0; part < 2; ++part) {  // L2 norm of Q, then of K, in place
            __half* p = x + part * HD + head * D;
            for (int i = tid; i < D; i += tgs) s_x[i] = __half2float(p[i]);
            __syncthreads();
            const float scale = __fdiv_rn(1.0f, fmaxf(__fsqrt_rn(cta_sumsq(s_x, D, s_part)), a.eps));
            for (int i = tid; i < D; i += tgs) {
                const __half r = __float2half_rn(__fmul_rn(s_x[i], scale));
                p[i] = r;
                if (part == 0) s_qs[i] = __fmul_rn(__half2float(r), a.head_scale);
                else s_key[i] = __half2float(r);
            }
            __syncthreads();
        }
        const float decay = s_gate[0], beta = s_gate[1];
        for (int v = tid; v < D; v += tgs) {
            __half* row = S + v * pitch;
            float acc = 0.0f;
            for (int k = 0; k < D; ++k) {
                const __half s = __float2half_rn(__fmul_rn(__half2float(row[k]), decay));
                row[k] = s;
                acc = __fadd_rn(acc, __fmul_rn(__half2float(s), s_key[k]));
            }
            const float delta = __fmul_rn(__fsub_rn(__half2float(x[2 * HD + head * D + v]), acc), beta);
            float o = 0.0f;
            for (int k = 0; k < D; ++k) {
                const __half s = __float2half_rn(__fadd_rn(__half2float(row[k]), __fmul_rn(delta, s_key[k])));
                row[k] = s;
                o = __fadd_rn(o, __fmul_rn(__half2float(s), s_qs[k]));
            }
            a.out[((size_t)pos * H + head) * D + v] = __float2half_rn(o);
        }
        __syncthreads();  // s_key, s_qs and s_gate are rewritten by the next position
    }
    for (int i = tid; i < D * D; i += tgs) gstate[i] = S[(i / D) * pitch + i % D];
}

void cfg_launch(const Launch& l, cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, dim3 grid, dim3 block) {
    cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = l.stream;
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = l.pdl ? 1 : 0;
}

}  // namespace

cudaError_t launch_dn_compute_gates(const Launch& l, const __half* b_proj, const __half* a_proj, const __half* a_log, const __half* dt_bias,
                                    __half* beta_out, __half* g_out, int heads) {
    if (heads <= 0) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3((heads + 127) / 128), dim3(128));
    prefer_max_shared(dn_compute_gates_kernel);
    return cudaLaunchKernelEx(&cfg, dn_compute_gates_kernel, b_proj, a_proj, a_log, dt_bias, beta_out, g_out, heads, dev_dyn(l));
}

cudaError_t launch_dn_state_update(const Launch& l, __half* state, const __half* g_val, const __half* key, const float* delta, int head_dim,
                                   int heads) {
    if (head_dim <= 0 || heads <= 0 || (!g_val && !key) || (key && !delta)) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3((head_dim * head_dim + 1023) / 1024, heads), dim3(256));
    prefer_max_shared(dn_state_update_kernel);
    return cudaLaunchKernelEx(&cfg, dn_state_update_kernel, state, g_val, key, delta, head_dim, dev_dyn(l));
}

cudaError_t launch_dn_readout(const Launch& l, int mode, const __half* state, const __half* vec, const __half* value, const __half* g_val,
                              const __half* beta, const __half* b_proj, const __half* a_proj, const __half* a_log, const __half* dt_bias,
                              float* out_f32, __half* out_f16, __half* g_out, int head_dim, float scale, int heads) {
    if (head_dim <= 0 || head_dim > 256 || heads <= 0) return cudaErrorInvalidValue;
    ReadoutArgs a = {state, vec, value, g_val, beta, b_proj, a_proj, a_log, dt_bias, out_f32, out_f16, g_out, head_dim, scale};
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3(heads), dim3((head_dim + 31) / 32 * 32));
#define SMELT_DN_READOUT(M)                              \
    case M:                                              \
        prefer_max_shared(dn_readout_kernel<M>);         \
        return cudaLaunchKernelEx(&cfg, dn_readout_kernel<M>, a, dev_dyn(l));
    switch (mode) {
        SMELT_DN_READOUT(kReadoutKvMem) SMELT_DN_READOUT(kReadoutDelta) SMELT_DN_READOUT(kReadoutGatesDelta) SMELT_DN_READOUT(kReadoutQuery)
        default: return cudaErrorInvalidValue;
    }
#undef SMELT_DN_READOUT
}

cudaError_t launch_dn_compute_delta(const Launch& l, const __half* value, const float* kv_mem, const __half* beta, float* delta, int head_dim,
                                    int heads) {
    if (head_dim <= 0 || heads <= 0) return cudaErrorInvalidValue;
    const int total = head_dim * heads;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3((total + 255) / 256), dim3(256));
    prefer_max_shared(dn_compute_delta_kernel);
    return cudaLaunchKernelEx(&cfg, dn_compute_delta_kernel, value, kv_mem, beta, delta, head_dim, total, dev_dyn(l));
}

cudaError_t launch_dn_fused_decode(const Launch& l, __half* state, const __half* qkv, const __half* b_proj, const __half* a_proj,
                                   const __half* a_log, const __half* dt_bias, __half* out, __half* conv_state, const __half* conv_weight,
                                   const __half* z_proj, const __half* norm_weight, int head_dim, float head_scale, int qkv_dim, int conv_k,
                                   int heads, float rms_eps, int tgs) {
    if (head_dim <= 0 || head_dim % 32 || head_dim > 256 || heads <= 0 || conv_k <= 0 || conv_k > 8 || qkv_dim < 3 * heads * head_dim ||
        tgs < 32 || tgs % 32 || tgs > 1024)
        return cudaErrorInvalidValue;
    FusedArgs a = {};
    a.state = state; a.qkv = qkv; a.b_proj = b_proj; a.a_proj = a_proj; a.a_log = a_log; a.dt_bias = dt_bias; a.out = out;
    a.conv_state = conv_state; a.conv_weight = conv_weight; a.z_proj = z_proj; a.norm_weight = norm_weight;
    a.head_dim = head_dim; a.heads = heads; a.qkv_dim = qkv_dim; a.conv_k = conv_k; a.head_scale = head_scale; a.eps = rms_eps;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3(heads), dim3(tgs));
    prefer_max_shared(dn_fused_decode_kernel);
    return cudaLaunchKernelEx(&cfg, dn_fused_decode_kernel, a, dev_dyn(l));
}

cudaError_t launch_dn_fused_prefill(const Launch& l, __half* state, __half* conv_state, __half* qkv, const __half* conv_weight,
                                    const __half* a_log, const __half* dt_bias, const __half* b_buf, const __half* a_buf, __half* out,
                                    int head_dim, int heads, int seq_len, int qkv_dim, int conv_k, float head_scale, float l2_eps, int tgs) {
    if (head_dim <= 0 || head_dim > 256 || heads <= 0 || conv_k <= 0 || conv_k > 8 || qkv_dim < 3 * heads * head_dim || seq_len < 0 ||
        tgs < 32 || tgs % 32 || tgs > 1024)
        return cudaErrorInvalidValue;
    FusedArgs a = {};
    a.state = state; a.qkv_rw = qkv; a.b_proj = b_buf; a.a_proj = a_buf; a.a_log = a_log; a.dt_bias = dt_bias; a.out = out;
    a.conv_state = conv_state; a.conv_weight = conv_weight;
    a.head_dim = head_dim; a.heads = heads; a.qkv_dim = qkv_dim; a.conv_k = conv_k; a.seq_len = seq_len; a.head_scale = head_scale; a.eps = l2_eps;
    const size_t smem = (size_t)head_dim * (head_dim + 2) * sizeof(__half);
    cudaError_t e = cudaFuncSetAttribute(dn_fused_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cfg_launch(l, cfg, attr, dim3(heads), dim3(tgs));
    cfg.dynamicSmemBytes = smem;
    prefer_max_shared(dn_fused_prefill_kernel);
    return cudaLaunchKernelEx(&cfg, dn_fused_prefill_kernel, a, dev_dyn(l));
}

}  // namespace smelt
