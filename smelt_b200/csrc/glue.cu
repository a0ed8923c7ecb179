// Small per-token kernels around the matvecs: norms, residual add, SwiGLU, embedding gathers,
// RoPE, KV-cache append, argmax, the on-device u4 dequant probe and the dense fp16 matvec
// used as LM head.  Each kernel cites the reference kernel whose arithmetic and rounding
// points it keeps.
#include "glue.h"
#include "rope.cuh"

namespace smelt {

namespace {

__device__ __forceinline__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < nw; ++w) tot += scratch[w];  // fixed order
    __syncthreads();
    return tot;
}

// rms_norm_1pw (Resources/Shaders/norms.metal:9-67): y = half(1 + w) * half(x * rsqrt(mean x^2 + eps)),
// the weight being stored as a delta from one.  One CTA per batch row.
__global__ void rms_norm_1pw_kernel(const __half* __restrict__ x, const __half* __restrict__ w, __half* __restrict__ y,
                                    int dim, float eps, DevDyn dyn) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const __half* xr = x + (size_t)blockIdx.x * dim;
    __half* yr = y + (size_t)blockIdx.x * dim;
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = __half2float(xr[i]);
        ss += v * v;
    }
    const float tot = block_sum(ss, scratch);
    const float rs = __frcp_rn(__fsqrt_rn(tot / (float)dim + eps));
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const __half n = __float2half_rn(__half2float(xr[i]) * rs);
        const __half dw = __float2half_rn(1.0f + __half2float(w[i]));
        yr[i] = __hmul(dw, n);
    }
}

// The same norm for rows of 8k elements at 16-byte alignment: 256 threads, 16-byte loads and
// stores, and the reduction order the matvec kernels with a folded norm use, so that a folded
// norm and this kernel give the same bits.
__global__ void __launch_bounds__(256) rms_norm_1pw_vec_kernel(const __half* __restrict__ x, const __half* __restrict__ w,
                                                               __half* __restrict__ y, int dim, float eps, DevDyn dyn) {
    __shared__ float scratch[8];
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const __half* xr = x + (size_t)blockIdx.x * dim;
    __half* yr = y + (size_t)blockIdx.x * dim;
    const float tot = cta256_sumsq_f16(xr, dim, scratch);
    const float rs = __frcp_rn(__fsqrt_rn(tot / (float)dim + eps));
    for (int c8 = threadIdx.x; c8 < dim / 8; c8 += 256) {
        uint4 v = *reinterpret_cast<const uint4*>(xr + c8 * 8);
        const uint4 wv = *reinterpret_cast<const uint4*>(w + c8 * 8);
        v.x = rms_norm_1pw_pair(v.x, wv.x, rs); v.y = rms_norm_1pw_pair(v.y, wv.y, rs);
        v.z = rms_norm_1pw_pair(v.z, wv.z, rs); v.w = rms_norm_1pw_pair(v.w, wv.w, rs);
        *reinterpret_cast<uint4*>(yr + c8 * 8) = v;
    }
}

// elementwise_add (Resources/Shaders/activations.metal:56-66): fp16 add.
__global__ void elementwise_add_kernel(const __half* a, const __half* b, __half* y, int64_t n, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __hadd(a[i], b[i]);
}


__global__ void swiglu_fused_kernel(const __half* gate, const __half* up, __half* y, int64_t n, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = swiglu_staged(gate[i], up[i]);
}

// embedding_gather (Resources/Shaders/lut_matvec.metal:951-962): row copy; the token id is
// read from device memory (a slot, or the context's dynamic state).
__global__ void embedding_gather_kernel(const __half* __restrict__ table, const int32_t* __restrict__ token,
                                        __half* __restrict__ y, int hidden, int token_stride, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int64_t row = token[(size_t)blockIdx.y * token_stride];
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < hidden) y[(size_t)blockIdx.y * hidden + i] = table[row * hidden + i];
}

// affine_embedding_gather (Resources/Shaders/lut_matvec.metal:994-1025):
// half(float(nibble) * scale + bias), multiply and add kept separate.
__global__ void affine_embedding_gather_kernel(const uint8_t* __restrict__ w, const __half* __restrict__ s,
                                               const __half* __restrict__ b, const int32_t* __restrict__ token,
                                               __half* __restrict__ y, int cols, int group, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= cols / 2) return;
    const int64_t row = token[blockIdx.y];  // grid.y: the rows of affine_embedding_gather_batched (lut_matvec.metal:1081-1116)
    y += (size_t)blockIdx.y * cols;
    const int groups = cols / group;
    const uint8_t p = w[row * (cols / 2) + i];
    const int c0 = 2 * i, c1 = c0 + 1;
    const float s0 = __half2float(s[row * groups + c0 / group]), b0 = __half2float(b[row * groups + c0 / group]);
    const float s1 = __half2float(s[row * groups + c1 / group]), b1 = __half2float(b[row * groups + c1 / group]);
    y[c0] = __float2half_rn(__fadd_rn(__fmul_rn((float)(p & 0xF), s0), b0));
    y[c1] = __float2half_rn(__fadd_rn(__fmul_rn((float)(p >> 4), s1), b1));
}

// Dequantise whole rows (the parity probe for the bit-exact unpack requirement):
// out_f32 = float(nibble)*scale + bias (Sources/SmeltCompiler/SmeltAffineU4.swift:141-161),
// out_f16 = the same value rounded once.
__global__ void affine_dequant_kernel(const uint8_t* __restrict__ w, const __half* __restrict__ s,
                                      const __half* __restrict__ b, float* out32, __half* out16, int rows, int cols,
                                      int group) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)rows * cols) return;
    const int64_t r = i / cols;
    const int c = (int)(i % cols);
    const uint8_t p = w[r * (cols / 2) + c / 2];
    const uint32_t nib = (c & 1) ? (p >> 4) : (p & 0xF);
    const int groups = cols / group;
    const float v = __fadd_rn(__fmul_rn((float)nib, __half2float(s[r * groups + c / group])),
                              __half2float(b[r * groups + c / group]));
    if (out32) out32[i] = v;
    if (out16) out16[i] = __float2half_rn(v);
}

// binary1 / ternary2 row dequant (Sources/SmeltRuntime/SmeltSignedQuantCodec.swift:219-257):
// float(semantic) * float(fp16 scale); an invalid ternary code 3 sets *bad.
__global__ void signed_dequant_kernel(const uint8_t* __restrict__ codes, const __half* __restrict__ s, float* out,
                                      int rows, int cols, int bits, int group, int* bad) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)rows * cols) return;
    const int64_t r = i / cols;
    const int c = (int)(i % cols);
    const size_t row_bytes = (size_t)cols * bits / 8;
    const int bit = c * bits;
    const uint32_t code = (codes[r * row_bytes + (bit >> 3)] >> (bit & 7)) & ((1u << bits) - 1u);
    float sem;
    if (bits == 1) sem = code ? 1.f : -1.f;
    else {
        if (code == 3) { atomicExch(bad, 1); sem = 0.f; }
        else sem = (float)((int)code - 1);
    }
    out[i] = sem * __half2float(s[r * (cols / group) + c / group]);
}

// apply_rope (attention.metal:48-115), in place; grid.y = batch row (position + row when
// rows are consecutive positions is NOT implied: every row uses the same position unless
// pos_per_row is set, for independent sequences the positions are equal).
__global__ void apply_rope_kernel(__half* qk, const __half* cos_t, const __half* sin_t, int head_dim, int rope_dim,
                                  int heads, int layout, float base_log2, int math_mode, size_t table_stride,
                                  DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int tid = blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= heads * head_dim) return;
    const int head = tid / head_dim, dim = tid % head_dim, half_rope = rope_dim / 2;
    if (dim >= half_rope) return;
    const uint32_t position = dyn_arg_position(dyn);
    __half* v = qk + ((size_t)blockIdx.y * heads + head) * head_dim;
    if (cos_t) { cos_t += (size_t)position * table_stride; sin_t += (size_t)position * table_stride; }
    int d0, d1, c0i, c1i;
    rope_indices(layout, dim, half_rope, head_dim, d0, d1, c0i, c1i);
    const float x0 = __half2float(v[d0]), x1 = __half2float(v[d1]);
    float c0, s0, c1, s1;
    rope_trig(dim, half_rope, position, base_log2, math_mode, cos_t, sin_t, c0i, c1i, c0, s0, c1, s1);
    v[d0] = __float2half_rn(__fsub_rn(__fmul_rn(x0, c0), __fmul_rn(x1, s0)));
    v[d1] = __float2half_rn(__fadd_rn(__fmul_rn(x0, s1), __fmul_rn(x1, c1)));
}

// kv_cache_update / rope_kv_cache_update (attention.metal:122-209):
// cache[(seq) h, pos, :] = (rotated) new[h, :]; grid.y = sequence, caches seq_stride elements apart.
__global__ void kv_cache_update_kernel(__half* cache, const __half* new_kv, const __half* cos_t, const __half* sin_t,
                                       uint32_t capacity, int head_dim, int heads, int rope_dim, int layout,
                                       float base_log2, int math_mode, int do_rope, size_t table_stride,
                                       size_t seq_stride, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int tid = blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= heads * head_dim) return;
    const uint32_t pos = dyn_arg_position(dyn);
    if (pos >= capacity) return;  // host validates; never write outside the cache
    const int head = tid / head_dim, dim = tid % head_dim;
    const __half* src = new_kv + ((size_t)blockIdx.y * heads + head) * head_dim;
    __half* dst = cache + (size_t)blockIdx.y * seq_stride + ((size_t)head * capacity + pos) * head_dim;
    if (!do_rope) { dst[dim] = src[dim]; return; }
    const int half_rope = rope_dim / 2;
    if (cos_t) { cos_t += (size_t)pos * table_stride; sin_t += (size_t)pos * table_stride; }
    if (dim < half_rope) {
        int d0, d1, c0i, c1i;
        rope_indices(layout, dim, half_rope, head_dim, d0, d1, c0i, c1i);
        const float x0 = __half2float(src[d0]), x1 = __half2float(src[d1]);
        float c0, s0, c1, s1;
        rope_trig(dim, half_rope, pos, base_log2, math_mode, cos_t, sin_t, c0i, c1i, c0, s0, c1, s1);
        dst[d0] = __float2half_rn(__fsub_rn(__fmul_rn(x0, c0), __fmul_rn(x1, s0)));
        dst[d1] = __float2half_rn(__fadd_rn(__fmul_rn(x1, c1), __fmul_rn(x0, s1)));
        return;
    }
    bool rotated_second;
    if (layout == 2) rotated_second = dim >= head_dim / 2 && dim < head_dim / 2 + half_rope;
    else if (layout == 1) rotated_second = dim < rope_dim;
    else rotated_second = dim < rope_dim;
    if (!rotated_second) dst[dim] = src[dim];
}

// RoPE on Q (in place), RoPE on the new K row written into the K cache, and the new V row
// copied into the V cache, in one launch: the work of apply_rope + rope_kv_cache_update +
// kv_cache_update (attention.metal:48-209) for full-head rotation (ropeDim == headDim,
// adjacent or split-half pairs, analytic trig).  One thread per pair.
__global__ void rope_qkv_append_kernel(__half* q, const __half* k_new, const __half* v_new, __half* k_cache,
                                       __half* v_cache, uint32_t capacity, int head_dim, int n_q, int n_kv, int layout,
                                       float base_log2, size_t seq_stride, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const uint32_t pos = dyn_arg_position(dyn);
    if (pos >= capacity) return;
    const int half = head_dim / 2;
    const int item = blockIdx.x * blockDim.x + threadIdx.x;
    const int total = (n_q + 2 * n_kv) * half;
    if (item >= total) return;
    const int head = item / half, p = item % half, b = blockIdx.y;
    if (head >= n_q + n_kv) {  // V: copy two elements
        const int h = head - n_q - n_kv;
        const __half2 v = reinterpret_cast<const __half2*>(v_new + ((size_t)b * n_kv + h) * head_dim)[p];
        reinterpret_cast<__half2*>(v_cache + (size_t)b * seq_stride + ((size_t)h * capacity + pos) * head_dim)[p] = v;
        return;
    }
    int d0, d1, c0i, c1i;
    rope_indices(layout, p, half, head_dim, d0, d1, c0i, c1i);
    float c0, s0, c1, s1;
    rope_trig(p, half, pos, base_log2, 1, nullptr, nullptr, c0i, c1i, c0, s0, c1, s1);
    if (head < n_q) {
        __half* v = q + ((size_t)b * n_q + head) * head_dim;
        const float x0 = __half2float(v[d0]), x1 = __half2float(v[d1]);
        v[d0] = __float2half_rn(__fsub_rn(__fmul_rn(x0, c0), __fmul_rn(x1, s0)));
        v[d1] = __float2half_rn(__fadd_rn(__fmul_rn(x0, s1), __fmul_rn(x1, c1)));
    } else {
        const int h = head - n_q;
        const __half* src = k_new + ((size_t)b * n_kv + h) * head_dim;
        __half* dst = k_cache + (size_t)b * seq_stride + ((size_t)h * capacity + pos) * head_dim;
        const float x0 = __half2float(src[d0]), x1 = __half2float(src[d1]);
        dst[d0] = __float2half_rn(__fsub_rn(__fmul_rn(x0, c0), __fmul_rn(x1, s0)));
        dst[d1] = __float2half_rn(__fadd_rn(__fmul_rn(x1, c1), __fmul_rn(x0, s1)));
    }
}

// Argmax over fp16 logits with the reference's ordered key
// (Resources/Shaders/lut_matvec.metal:4045-4074): ties keep the lowest index, -0 == +0.
__device__ __forceinline__ uint64_t argmax_key(__half v, uint32_t index) {
    uint32_t bits = __half_as_ushort(v);
    if ((bits & 0x7FFFu) == 0u) bits = 0u;
    const uint32_t ordered = (bits & 0x8000u) ? (0xFFFFu - bits) : (bits ^ 0x8000u);
    return ((uint64_t)ordered << 32) | (uint64_t)(0xFFFFFFFFu - index);
}

__global__ void argmax_partials_kernel(const __half* __restrict__ logits, uint64_t* __restrict__ partials, int vocab,
                                       int chunk, DevDyn dyn) {
    __shared__ uint64_t sbest[32];
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const __half* lg = logits + (size_t)blockIdx.y * vocab;
    const int start = blockIdx.x * chunk, end = min(start + chunk, vocab);
    uint64_t best = 0;
    for (int i = start + threadIdx.x; i < end; i += blockDim.x) {
        const uint64_t k = argmax_key(lg[i], (uint32_t)i);
        best = k > best ? k : best;
    }
    for (int o = 16; o > 0; o >>= 1) {
        const uint64_t other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if ((threadIdx.x & 31) == 0) sbest[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) best = sbest[w] > best ? sbest[w] : best;
        partials[(size_t)blockIdx.y * gridDim.x + blockIdx.x] = best;
    }
}

__global__ void argmax_reduce_kernel(const uint64_t* __restrict__ partials, int32_t* __restrict__ out, int n,
                                     int out_stride, DevDyn dyn) {
    __shared__ uint64_t sbest[32];
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const uint64_t* p = partials + (size_t)blockIdx.x * n;
    uint64_t best = 0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) best = p[i] > best ? p[i] : best;
    for (int o = 16; o > 0; o >>= 1) {
        const uint64_t other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if ((threadIdx.x & 31) == 0) sbest[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) best = sbest[w] > best ? sbest[w] : best;
        out[(size_t)blockIdx.x * out_stride] = (int32_t)(0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFu));
    }
}

// Dense fp16 matvec (Resources/Shaders/lut_matvec.metal:799-834, fp16_matvec): fp32
// accumulation, clamp to ±65504, fp16 out.  One warp per output row, 16-byte loads along the
// row (512 contiguous bytes per warp instruction), activations staged in shared memory,
// up to NB batch rows per pass.
template <int NB>
__global__ void __launch_bounds__(256) fp16_matvec_kernel(const __half* __restrict__ w, const __half* __restrict__ x,
                                                          __half* __restrict__ y, int rows, int cols, int batch,
                                                          DevDyn dyn) {
    extern __shared__ __align__(16) uint8_t smem[];
    __half* sx = reinterpret_cast<__half*>(smem);
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    for (int i = threadIdx.x; i < batch * cols / 8; i += blockDim.x)
        reinterpret_cast<uint4*>(sx)[i] = reinterpret_cast<const uint4*>(x)[i];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows_per_cta = (rows + gridDim.x - 1) / gridDim.x;
    const int r_begin = blockIdx.x * rows_per_cta, r_end = min(rows, r_begin + rows_per_cta);
    for (int r = r_begin + warp; r < r_end; r += 8) {
        const uint4* wr = reinterpret_cast<const uint4*>(w + (size_t)r * cols);
        float acc[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) acc[b] = 0.f;
        for (int c = lane; c < cols / 8; c += 32) {
            const uint4 wv = __ldg(wr + c);
            const float2 w0 = __half22float2(u32_as_h2(wv.x)), w1 = __half22float2(u32_as_h2(wv.y));
            const float2 w2 = __half22float2(u32_as_h2(wv.z)), w3 = __half22float2(u32_as_h2(wv.w));
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                if (b < batch) {
                    const uint4 xv = reinterpret_cast<const uint4*>(sx + (size_t)b * cols)[c];
                    const float2 x0 = __half22float2(u32_as_h2(xv.x)), x1 = __half22float2(u32_as_h2(xv.y));
                    const float2 x2 = __half22float2(u32_as_h2(xv.z)), x3 = __half22float2(u32_as_h2(xv.w));
                    acc[b] += w0.x * x0.x + w0.y * x0.y + w1.x * x1.x + w1.y * x1.y + w2.x * x2.x + w2.y * x2.y +
                              w3.x * x3.x + w3.y * x3.y;
                }
            }
        }
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            const float v = warp_sum(acc[b]);
            if (lane == 0 && b < batch) y[(size_t)b * rows + r] = __float2half_rn(fminf(fmaxf(v, -65504.f), 65504.f));
        }
    }
}

cudaError_t launch_cfg(const Launch& l, cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, dim3 grid, dim3 block,
                       size_t smem) {
    cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = l.stream;
    cfg.numAttrs = 0;
    cfg.attrs = attr;
    if (l.pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 1;
    }
    return cudaSuccess;
}

#define SMELT_LAUNCH(kernel, grid, block, smem, ...)                 \
    do {                                                             \
        cudaLaunchConfig_t cfg;                                      \
        cudaLaunchAttribute attr[1];                                 \
        cudaError_t ce = launch_cfg(l, cfg, attr, grid, block, smem); \
        if (ce != cudaSuccess) return ce;                            \
        prefer_max_shared(kernel);                                   \
        return cudaLaunchKernelEx(&cfg, kernel, __VA_ARGS__);        \
    } while (0)

}  // namespace

cudaError_t launch_rms_norm_1pw(const Launch& l, const __half* x, const __half* w, __half* y, int dim, float eps,
                                int batch) {
    if (dim % 8 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0) {
        SMELT_LAUNCH(rms_norm_1pw_vec_kernel, dim3(batch), dim3(256), 0, x, w, y, dim, eps, dev_dyn(l));
    }
    int threads = dim >= 4096 ? 1024 : (dim >= 1024 ? 512 : 256);
    SMELT_LAUNCH(rms_norm_1pw_kernel, dim3(batch), dim3(threads), 0, x, w, y, dim, eps, dev_dyn(l));
}

cudaError_t launch_per_head_rms_norm(const Launch& l, const __half* x, const __half* w, __half* y, int heads,
                                     int head_dim, float eps) {
    return launch_head_norm(l, kHeadNormDirect, x, w, y, heads, head_dim, eps, 32);  // elementwise.cu: the kernel's own reduction topology
}

cudaError_t launch_elementwise_add(const Launch& l, const __half* a, const __half* b, __half* y, int64_t n) {
    SMELT_LAUNCH(elementwise_add_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, a, b, y, n, dev_dyn(l));
}

cudaError_t launch_swiglu_fused(const Launch& l, const __half* gate, const __half* up, __half* y, int64_t n) {
    SMELT_LAUNCH(swiglu_fused_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, gate, up, y, n, dev_dyn(l));
}

cudaError_t launch_embedding_gather(const Launch& l, const __half* table, const int32_t* token, __half* y, int hidden,
                                    int batch, int token_stride) {
    SMELT_LAUNCH(embedding_gather_kernel, dim3((hidden + 255) / 256, batch), dim3(256), 0, table, token, y, hidden,
                 token_stride, dev_dyn(l));
}

cudaError_t launch_affine_embedding_gather(const Launch& l, const uint8_t* w, const __half* s, const __half* b,
                                           const int32_t* token, __half* y, int cols, int group, int batch) {
    SMELT_LAUNCH(affine_embedding_gather_kernel, dim3((cols / 2 + 255) / 256, batch), dim3(256), 0, w, s, b, token, y, cols,
                 group, dev_dyn(l));
}

cudaError_t launch_affine_dequant(const Launch& l, const uint8_t* w, const __half* s, const __half* b, float* out32,
                                  __half* out16, int rows, int cols, int group) {
    const int64_t n = (int64_t)rows * cols;
    affine_dequant_kernel<<<(unsigned)((n + 255) / 256), 256, 0, l.stream>>>(w, s, b, out32, out16, rows, cols, group);
    return cudaGetLastError();
}

cudaError_t launch_signed_dequant(const Launch& l, const uint8_t* codes, const __half* s, float* out, int rows,
                                  int cols, int bits, int group, int* bad) {
    const int64_t n = (int64_t)rows * cols;
    signed_dequant_kernel<<<(unsigned)((n + 255) / 256), 256, 0, l.stream>>>(codes, s, out, rows, cols, bits, group, bad);
    return cudaGetLastError();
}

cudaError_t launch_apply_rope(const Launch& l, __half* qk, const __half* cos_t, const __half* sin_t, int head_dim,
                              int rope_dim, int heads, int layout, float base_log2, int math_mode, size_t table_stride,
                              int batch) {
    SMELT_LAUNCH(apply_rope_kernel, dim3((heads * head_dim + 127) / 128, batch), dim3(128), 0, qk, cos_t, sin_t,
                 head_dim, rope_dim, heads, layout, base_log2, math_mode, table_stride, dev_dyn(l));
}

cudaError_t launch_kv_cache_update(const Launch& l, __half* cache, const __half* new_kv, const __half* cos_t,
                                   const __half* sin_t, uint32_t capacity, int head_dim, int heads, int rope_dim,
                                   int layout, float base_log2, int math_mode, int do_rope, size_t table_stride,
                                   int batch, size_t seq_stride) {
    SMELT_LAUNCH(kv_cache_update_kernel, dim3((heads * head_dim + 127) / 128, batch), dim3(128), 0, cache, new_kv,
                 cos_t, sin_t, capacity, head_dim, heads, rope_dim, layout, base_log2, math_mode, do_rope,
                 table_stride, seq_stride, dev_dyn(l));
}

cudaError_t launch_rope_qkv_append(const Launch& l, __half* q, const __half* k_new, const __half* v_new, __half* k_cache,
                                   __half* v_cache, uint32_t capacity, int head_dim, int n_q, int n_kv, int layout,
                                   float base_log2, int batch, size_t seq_stride) {
    if (layout == 2 || head_dim % 2) return cudaErrorInvalidValue;
    const int total = (n_q + 2 * n_kv) * head_dim / 2;
    SMELT_LAUNCH(rope_qkv_append_kernel, dim3((total + 127) / 128, batch), dim3(128), 0, q, k_new, v_new, k_cache, v_cache,
                 capacity, head_dim, n_q, n_kv, layout, base_log2, seq_stride, dev_dyn(l));
}

cudaError_t launch_argmax_partials(const Launch& l, const __half* logits, uint64_t* partials, int vocab, int chunk,
                                   int batch) {
    SMELT_LAUNCH(argmax_partials_kernel, dim3((vocab + chunk - 1) / chunk, batch), dim3(256), 0, logits, partials,
                 vocab, chunk, dev_dyn(l));
}

cudaError_t launch_argmax_reduce(const Launch& l, const uint64_t* partials, int32_t* out, int n, int batch,
                                 int out_stride) {
    SMELT_LAUNCH(argmax_reduce_kernel, dim3(batch), dim3(256), 0, partials, out, n, out_stride, dev_dyn(l));
}

cudaError_t launch_fp16_matvec(const Launch& l, const __half* w, const __half* x, __half* y, int rows, int cols,
                               int batch, int sm_count) {
    if (cols % 8 != 0 || batch <= 0) return cudaErrorInvalidValue;
    for (int b0 = 0; b0 < batch; b0 += 8) {
        const int nb = batch - b0 < 8 ? batch - b0 : 8;
        const size_t smem = (size_t)nb * cols * 2;
        if (smem > 200 * 1024) return cudaErrorInvalidValue;
        // As many CTAs as can be resident at once (eight of 256 threads per SM), no fewer: a smaller
        // grid launched programmatically behind a kernel that still holds most SMs piles up to
        // eight CTAs on each of the few SMs that are free and leaves the others without work.
        int grid = sm_count * 8;
        if (grid > (rows + 7) / 8) grid = (rows + 7) / 8;
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[1];
        launch_cfg(l, cfg, attr, dim3(grid), dim3(256), smem);
        cudaError_t e;
        if (nb == 1) {
            e = cudaFuncSetAttribute(fp16_matvec_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            prefer_max_shared(fp16_matvec_kernel<1>);
            if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, fp16_matvec_kernel<1>, w, x + (size_t)b0 * cols, y + (size_t)b0 * rows, rows, cols, nb, dev_dyn(l));
        } else {
            e = cudaFuncSetAttribute(fp16_matvec_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            prefer_max_shared(fp16_matvec_kernel<8>);
            if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, fp16_matvec_kernel<8>, w, x + (size_t)b0 * cols, y + (size_t)b0 * rows, rows, cols, nb, dev_dyn(l));
        }
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace smelt
