// Shared device/host helpers for the libsmelt_cuda kernels (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace smelt {

// Per-launch dynamic state shared by every kernel the dispatch interpreter launches.
// `dyn` points at the context's device-resident {token, position} pair so that a captured
// CUDA graph can be replayed for every token without re-recording kernel parameters; when it
// is null the literal position is used.  The guard fields mirror the reference's
// "skip unless position+1 < / >= literal" constants
// (Sources/SmeltSchema/SmeltDispatchTable.swift:80-83): a guarded kernel returns at once when
// its condition is false.
struct DynState {
    int32_t token;
    uint32_t position;
};

struct Launch {
    cudaStream_t stream = nullptr;
    const DynState* dyn = nullptr;  // device pointer or null
    uint32_t position = 0;          // used when dyn == null
    uint32_t guard_lt = 0;          // 0 = no guard; else run only if position+1 <  guard_lt
    uint32_t guard_ge = 0;          // 0 = no guard; else run only if position+1 >= guard_ge
    uint32_t arg_pos = 0;           // literal position argument of the kernel, when arg_pos_valid
    uint32_t arg_pos_valid = 0;
    bool pdl = false;               // launch with programmatic stream serialization
};

struct DevDyn {
    const DynState* dyn;
    uint32_t position;
    uint32_t guard_lt;
    uint32_t guard_ge;
    uint32_t arg_pos;
    uint32_t arg_pos_valid;
};

inline DevDyn dev_dyn(const Launch& l) {
    return DevDyn{l.dyn, l.position, l.guard_lt, l.guard_ge, l.arg_pos, l.arg_pos_valid};
}

// The token position of the step being decoded (drives guards and "position" constants).
__device__ __forceinline__ uint32_t dyn_position(const DevDyn& d) { return d.dyn ? d.dyn->position : d.position; }
// The kernel's own position argument: a literal from the record when one was bound, else the
// step position.
__device__ __forceinline__ uint32_t dyn_arg_position(const DevDyn& d) {
    return d.arg_pos_valid ? d.arg_pos : dyn_position(d);
}

// True when the launch must be skipped.  Only valid after the grid dependency has resolved
// (the position may be written by the preceding kernel in the stream).
__device__ __forceinline__ bool dyn_skip(const DevDyn& d) {
    if (d.guard_lt == 0 && d.guard_ge == 0) return false;
    uint32_t p1 = dyn_position(d) + 1u;
    if (d.guard_lt != 0 && !(p1 < d.guard_lt)) return true;
    if (d.guard_ge != 0 && !(p1 >= d.guard_ge)) return true;
    return false;
}

// Programmatic dependent launch: wait for the upstream grid (and its memory) / allow the
// downstream grid to start its prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h);
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u);

// Sum of squares of one fp16 row (cols a multiple of 8, 16-byte aligned) by the first 256
// threads of a CTA (of 256 threads or more), in a fixed order, so that every kernel that norms a row gets the same bits:
// thread t folds the 8-element chunks t, t + 256, ... into one FMA chain, lanes combine by
// xor-shuffle, the eight warp sums are added in warp order.  scratch: 8 floats of shared
// memory that no thread reads or writes around the call.
__device__ __forceinline__ float cta256_sumsq_f16(const __half* xr, int cols, float* scratch);

// rms_norm_1pw's element step (Resources/Shaders/norms.metal:58-63) on two lanes:
// half(x * rs) times half(1 + w) as an fp16 product.
__device__ __forceinline__ uint32_t rms_norm_1pw_pair(uint32_t x2, uint32_t w2, float rs);

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// mma.sync m16n8k16, fp16 operands, fp32 accumulate.
__device__ __forceinline__ void mma16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Same with a zero accumulator input (starts a fresh sum without clearing registers first).
__device__ __forceinline__ void mma16816_zero(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// (a & b) | c in one LOP3.
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// One 16-byte word (eight fp16 values) folded into a running sum of squares, as an FMA chain.
__device__ __forceinline__ float sumsq8(float ss, const uint4& v) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(u32_as_h2(u[j]));
        ss = __fmaf_rn(f.x, f.x, ss);
        ss = __fmaf_rn(f.y, f.y, ss);
    }
    return ss;
}

// The per-thread sums of the first 256 threads combined: lanes by xor-shuffle, then the eight
// warp sums in warp order.  Every thread of the CTA must call it (two barriers inside).
__device__ __forceinline__ float cta256_sum_finish(float ss, float* scratch) {
    ss = warp_sum(ss);
    __syncthreads();
    if ((threadIdx.x & 31) == 0 && threadIdx.x < 256) scratch[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot = __fadd_rn(tot, scratch[w]);
    return tot;
}

__device__ __forceinline__ float cta256_sumsq_f16(const __half* xr, int cols, float* scratch) {
    float ss = 0.f;
    for (int c8 = threadIdx.x < 256 ? (int)threadIdx.x : cols; c8 < cols / 8; c8 += 256)  // threads past 255 only join the barriers
        ss = sumsq8(ss, *reinterpret_cast<const uint4*>(xr + c8 * 8));
    return cta256_sum_finish(ss, scratch);
}

__device__ __forceinline__ uint32_t rms_norm_1pw_pair(uint32_t x2, uint32_t w2, float rs) {
    const float2 xf = __half22float2(u32_as_h2(x2)), wf = __half22float2(u32_as_h2(w2));
    const __half2 n = __floats2half2_rn(__fmul_rn(xf.x, rs), __fmul_rn(xf.y, rs));
    const __half2 dw = __floats2half2_rn(__fadd_rn(1.0f, wf.x), __fadd_rn(1.0f, wf.y));
    return h2_as_u32(__hmul2(dw, n));
}

// ── mbarrier + bulk async copy (TMA, untiled) ───────────────────────────────
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2^22 polls (each poll itself blocks for a hardware-defined
// time slice) and reports failure instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 22); ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// Global -> shared bulk copy; dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// 16-byte asynchronous global -> shared copy that bypasses L1 (streamed weights are used once).
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src_gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// 4- and 8-byte asynchronous global -> shared copies (scales and biases beside streamed weights).
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async8(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}

// D = A (u8, 16 x 32) * B (s8, 32 x 8) + C; C may name one register four times.
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1, int c0, int c1, int c2, int c3) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
}

// Largest |v| of the eight fp16 values in a 16-byte word, as a float.
__device__ __forceinline__ float amax8(const uint4& v) {
    const __half2 m = __hmax2(__hmax2(__habs2(u32_as_h2(v.x)), __habs2(u32_as_h2(v.y))),
                              __hmax2(__habs2(u32_as_h2(v.z)), __habs2(u32_as_h2(v.w))));
    const float2 f = __half22float2(m);
    return fmaxf(f.x, f.y);
}

// The staged fp16 SwiGLU of the reference (Resources/Shaders/activations_precise.metal:9-22,
// signed_quant.metal:15-20): tail = 1 / (1 + exp(|g|)), sigmoid = g < 0 ? tail : 1 - tail,
// out = (g * sigmoid) * up, every intermediate an fp16 value; the fp16 exp is half(expf(float)).
__device__ __forceinline__ __half swiglu_staged(__half gate, __half up) {
    const float gf = __half2float(gate);
    const __half e = __float2half_rn(expf(fabsf(gf)));
    const __half denom = __hadd(__float2half_rn(1.0f), e);
    const __half tail = __hdiv(__float2half_rn(1.0f), denom);
    const __half sig = gf < 0.f ? tail : __hsub(__float2half_rn(1.0f), tail);
    return __hmul(__hmul(gate, sig), up);
}

// Metal's simd_sum as a butterfly over lane distance 16, 8, 4, 2, 1; the total is in lane 0.
__device__ __forceinline__ float simd_sum_lane0(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
    return v;
}

// Gated RMS norm of one head by one warp (Resources/Shaders/norms.metal:1093-1143,
// norms_gated_precise.metal:7-52).  rs as a threadgroup of tgs threads sums it: thread t adds
// x[t]^2, x[t + tgs]^2, ..., each simdgroup sums its lanes, the simdgroups' sums are added in
// order; the d128 kernel's lanes add four adjacent squares each.  The total is the same in
// every lane.
__device__ __forceinline__ float gated_norm_rs(const __half* x, int head_dim, float eps, int tgs, int lane) {
    float total = 0.0f;
    for (int s = 0; s < tgs / 32; ++s) {
        float p = 0.0f;
        for (int i = s * 32 + lane; i < head_dim; i += tgs) {
            const float v = __half2float(x[i]);
            p = __fadd_rn(p, __fmul_rn(v, v));
        }
        total = __fadd_rn(total, __shfl_sync(0xffffffffu, simd_sum_lane0(p), 0));
    }
    return __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)head_dim), eps)));
}
__device__ __forceinline__ float gated_norm_d128_rs(const __half* x, float eps, int lane) {
    float p = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float v = __half2float(x[4 * lane + i]);
        p = __fadd_rn(p, __fmul_rn(v, v));
    }
    const float total = __shfl_sync(0xffffffffu, simd_sum_lane0(p), 0);
    return __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(total, 128.0f), eps)));
}
// half(w * (x * rs) * silu(g)), silu in fp32
__device__ __forceinline__ __half gated_norm_value(__half x, __half g, __half w, float rs) {
    const float gf = __half2float(g);
    const float silu = __fdiv_rn(gf, __fadd_rn(1.0f, expf(-gf)));
    return __float2half_rn(__fmul_rn(__fmul_rn(__half2float(w), __fmul_rn(__half2float(x), rs)), silu));
}
// half(float(w * half(x * rs)) * (g * sigmoid(g))): the norm materialised in fp16, the stable sigmoid in fp32
__device__ __forceinline__ __half gated_norm_d128_value(__half x, __half g, __half w, float rs) {
    const __half normalized = __hmul(w, __float2half_rn(__fmul_rn(__half2float(x), rs)));
    const float gf = __half2float(g);
    const float tail = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(fabsf(gf))));
    const float sig = gf < 0.0f ? tail : __fsub_rn(1.0f, tail);
    return __float2half_rn(__fmul_rn(__half2float(normalized), __fmul_rn(gf, sig)));
}

// Error word shared by all kernels of a context: 0 = ok; kernels OR in a code when a bounded
// wait gives up so the host can report it instead of hanging.
enum : uint32_t { KERR_BARRIER_TIMEOUT = 1u, KERR_FLAG_TIMEOUT = 2u };

// Every kernel of a decode step asks for the same shared-memory carve-out (the largest): an SM
// drains before it changes its L1 / shared-memory split, so kernels that prefer different
// splits can neither overlap nor follow each other without a gap.
template <typename Kernel>
inline cudaError_t prefer_max_shared(Kernel kernel) {
    return cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel), cudaFuncAttributePreferredSharedMemoryCarveout,
                                (int)cudaSharedmemCarveoutMaxShared);
}

}  // namespace smelt
