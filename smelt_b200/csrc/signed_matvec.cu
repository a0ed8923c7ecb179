// binary1 / ternary2 low-bit matvec (group 128) for sm_100a.
//
// Replaces the reference's signed_* family (Resources/Shaders/signed_quant.metal:81-138
// signed_binary_matvec_g128_rows8, :223-286 the fused residual add, :140-221 the gate/up
// SwiGLU, :288-332 signed_ternary_matvec_g128_rows8; Resources/Shaders/signed_quant_precise.metal
// :41-108 the ternary affine form).  Semantics follow the scalar oracle
// (Sources/SmeltRuntime/SmeltSignedQuantCodec.swift:219-257 and
// Tests/SmeltCompilerTests/SignedQuantKernelTests.swift:1030-1045):
//   y[b,r] = sum_g scale[r,g] * sum_{k in g} sem(code[r,k]) * x[b,k],
// binary sem = {-1,+1}, ternary sem = {-1,0,+1}; codes are LSB-first in the row.
//
// One warp owns one output row; a lane consumes one 32-bit word of codes per step (32 binary
// or 16 ternary weights), applies the sign by flipping the activation's sign bit (binary) or
// by a masked add/subtract (ternary), accumulates the word's partial in fp32 and folds it in
// with the group scale.  Activations are staged in shared memory as fp32.
#include "glue.h"

namespace smelt {

namespace {

constexpr int kGroup = 128;


template <int BITS>
__device__ __forceinline__ float word_dot(uint32_t w, const float* __restrict__ xs) {
    float acc = 0.f;
    if (BITS == 1) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            // bit 1 -> +x, bit 0 -> -x : flip the sign bit when the code bit is clear
            const uint32_t flip = (~(w >> i) & 1u) << 31;
            acc += __uint_as_float(__float_as_uint(xs[i]) ^ flip);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int code = (int)((w >> (2 * i)) & 3u);
            acc += (float)(code - 1) * xs[i];
        }
    }
    return acc;
}

template <int BITS, int MODE, int NB>
__global__ void __launch_bounds__(256) signed_matvec_kernel(SignedArgs a, DevDyn dyn) {
    constexpr int NW = MODE == kSignedGateUp ? 2 : 1;
    constexpr int CPW = 32 / BITS;  // columns per 32-bit word
    extern __shared__ __align__(16) float sxf[];  // [NB][cols]
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int b0 = blockIdx.y * NB;
    const int nb = min(NB, a.batch - b0);
    for (int i = threadIdx.x; i < nb * a.cols; i += blockDim.x)
        sxf[i] = __half2float(a.x[(size_t)b0 * a.cols + i]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + warp;
    if (row >= a.rows) return;
    const int words = a.cols / CPW, groups = a.cols / kGroup;
    float acc[NW][NB];
#pragma unroll
    for (int s = 0; s < NW; ++s)
#pragma unroll
        for (int b = 0; b < NB; ++b) acc[s][b] = 0.f;
    for (int wi = lane; wi < words; wi += 32) {
        const int col = wi * CPW;
#pragma unroll
        for (int s = 0; s < NW; ++s) {
            const uint32_t w = reinterpret_cast<const uint32_t*>(a.codes[s] + (size_t)row * (a.cols * BITS / 8))[wi];
            const float sc = __half2float(a.scales[s][(size_t)row * groups + col / kGroup]);
#pragma unroll
            for (int b = 0; b < NB; ++b)
                if (b < nb) acc[s][b] += sc * word_dot<BITS>(w, sxf + (size_t)b * a.cols + col);
        }
    }
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        float v0 = warp_sum(acc[0][b]);
        float v1 = NW == 2 ? warp_sum(acc[NW - 1][b]) : 0.f;
        if (lane != 0 || b >= nb) continue;
        const size_t o = (size_t)(b0 + b) * a.rows + row;
        if (MODE == kSignedPlain) a.y[o] = __float2half_rn(v0);
        else if (MODE == kSignedAdd)  // signed_quant.metal:271-278: half(float(half(acc)) + float(residual))
            a.y[o] = __float2half_rn(__half2float(__float2half_rn(v0)) + __half2float(a.residual[o]));
        else a.y[o] = swiglu_staged(__float2half_rn(v0), __float2half_rn(v1));
    }
}

template <int BITS, int MODE, int NB>
cudaError_t launch_nb(const Launch& l, const SignedArgs& a) {
    const size_t smem = (size_t)NB * a.cols * sizeof(float);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    auto kern = signed_matvec_kernel<BITS, MODE, NB>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((a.rows + 7) / 8, (a.batch + NB - 1) / NB);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = l.pdl ? 1 : 0;
    prefer_max_shared(kern);
    return cudaLaunchKernelEx(&cfg, kern, a, dev_dyn(l));
}

template <int BITS, int MODE>
cudaError_t launch_mode(const Launch& l, const SignedArgs& a) {
    // batch rows per pass: as many as fit next to the fp32 activation stage in shared memory
    const size_t per_row = (size_t)a.cols * sizeof(float);
    if (a.batch >= 4 && 4 * per_row <= 200 * 1024) return launch_nb<BITS, MODE, 4>(l, a);
    if (a.batch >= 2 && 2 * per_row <= 200 * 1024) return launch_nb<BITS, MODE, 2>(l, a);
    return launch_nb<BITS, MODE, 1>(l, a);
}

template <int BITS>
cudaError_t launch_bits(const Launch& l, int mode, const SignedArgs& a) {
    switch (mode) {
        case kSignedPlain: return launch_mode<BITS, kSignedPlain>(l, a);
        case kSignedAdd: return launch_mode<BITS, kSignedAdd>(l, a);
        case kSignedGateUp: return launch_mode<BITS, kSignedGateUp>(l, a);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

cudaError_t launch_signed(const Launch& l, int mode, const SignedArgs& a) {
    if (a.rows <= 0 || a.cols <= 0 || a.batch <= 0 || a.cols % kGroup != 0) return cudaErrorInvalidValue;
    {
        bool handled = false;
        cudaError_t e = launch_signed_imma(l, mode, a, 0, &handled);  // batch 1 and 2, cols % 512 == 0
        if (handled || e != cudaSuccess) return e;
    }
    if (a.bits == 1) return launch_bits<1>(l, mode, a);
    if (a.bits == 2) return launch_bits<2>(l, mode, a);
    return cudaErrorInvalidValue;
}

}  // namespace smelt
