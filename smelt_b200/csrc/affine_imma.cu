// Integer-tensor-core form of the group-64 affine u4 matvec for batch 1 and 2.
//
// Same reference kernels as affine_matvec.cu (Resources/Shaders/lut_matvec.metal:1157-1287,
// :1718-1817, :2152-2233, :1824-1908): y[r] = sum_g (scale[r,g] * sum_c q[r,c] x[c] + bias[r,g] *
// sum_c x[c]).  The nibbles never become fp16.  A nibble pair is split with two ANDs into a
// byte holding n (even column) and a byte holding 16 n (odd column) and fed to
// mma.sync.m16n8k32.u8.s8 as the A operand.  The activations are turned, once per CTA, into
// signed base-128 digit planes of a per-row fixed-point value X = x * 2^26 / S (S a power of
// two >= max |x|; odd columns carry X / 16 to undo the 16 n): four planes per batch row are the
// B operand's columns, so one MMA yields sum q * digit for every plane and the exact integer
// results are recombined in fp32 as ((C3 * 128 + C2) * 128 + C1) * 128 + C0.  The fixed-point
// step is 2^-26 (2^-22 for odd columns) of the row's largest activation, below the fp32
// accumulation error of the reference kernels.
//
// The int32 accumulators start at the bit pattern of 1.5 * 2^23, so that reinterpreted as
// floats they read 12582912 + C and one FADD recovers C; no integer-to-float conversion runs.
//
// One persistent CTA per SM walks 16-row tiles.  Inside a tile warp w owns a contiguous K
// range and streams it through its own ring of cp.async stages (two or four groups each: 16
// rows x 64 or 128 bytes of nibbles, swizzled so that the fragment loads are conflict free,
// plus the groups' scales and biases).  A warp only waits for its own copies, so the main
// loop has no CTA-wide barrier; the rings keep running across tiles.  The K-partials of a
// tile are added in warp order through shared memory (one barrier per tile), so results are
// bit-reproducible.  Shared memory and registers are sized so that the CTAs of the next
// launch fit beside this one: with programmatic dependent launch they become resident while
// this launch still computes and fill their rings (weights do not depend on the previous
// kernel) before they wait for it.
#include <cstdlib>

#include "affine_imma.cuh"

namespace smelt {

namespace {

using namespace imma;

template <int MODE, int DEPTH, int WARPS, int GPS, int TG>
__global__ void __launch_bounds__(WARPS * 32, 1) affine_imma_kernel(const AffineArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    affine_imma_body<MODE, DEPTH, WARPS, GPS, TG>(a, smem, PdlSync());
}

template <int MODE, int DEPTH, int WARPS, int GPS, int TG>
cudaError_t launch_imma_t(const Launch& l, AffineArgs a) {
    using G = Geo<WARPS, GPS>;
    constexpr int NW = (MODE == kAffineGateUp || MODE == kAffineDual) ? 2 : 1;
    const ImmaLayout L = imma_layout(NW, DEPTH, WARPS, G::kSetBytes, a.cols, a.batch, TG);
    if (L.total > 226u * 1024u) return cudaErrorNotSupported;  // digit planes too large to stay resident
    a.dyn = dev_dyn(l);
    auto kern = affine_imma_kernel<MODE, DEPTH, WARPS, GPS, TG>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L.total);
    if (e != cudaSuccess) return e;
    if (NW == 1 && a.nseg <= 1) {
        a.nseg = 1;
        a.seg[0].w = a.w[0]; a.seg[0].s = a.s[0]; a.seg[0].b = a.b[0]; a.seg[0].y = a.y; a.seg[0].rows = a.rows;
    }
    int tiles = 0;
    if (NW == 1) for (int i = 0; i < a.nseg; ++i) tiles += (a.seg[i].rows + kTileRows - 1) / kTileRows;
    else tiles = (a.rows + kTileRows - 1) / kTileRows;
    a.ks = tiles;
    const int sm = a.sm_count > 0 ? a.sm_count : 148;
    cudaLaunchConfig_t cfg = {};
    const int want = (tiles + TG - 1) / TG;
    cfg.gridDim = dim3(want < sm ? want : sm, 1, 1);
    cfg.blockDim = dim3(G::kThreads, 1, 1);
    cfg.dynamicSmemBytes = L.total;
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = l.pdl ? 1 : 0;
    prefer_max_shared(kern);
    return cudaLaunchKernelEx(&cfg, kern, a);
}

// Eight warps on one tile, four groups (256 columns) per ring stage; when the columns are a
// multiple of 128 only, sixteen warps with two groups per stage.  Ring depth = stages each warp
// keeps in flight + 1: four (measured against three, five, six and eight: an SM keeps about
// 100 KB of copies outstanding, deeper rings only move waiting from the loop to the requests),
// three when the digit planes of a long row leave no room for four.
template <int MODE, int WARPS, int GPS>
cudaError_t launch_imma_depth(const Launch& l, const AffineArgs& a) {
    constexpr int NW = (MODE == kAffineGateUp || MODE == kAffineDual) ? 2 : 1;
    using G = Geo<WARPS, GPS>;
    if (imma_layout(NW, 4, WARPS, G::kSetBytes, a.cols, a.batch, 1).total <= 226u * 1024u) return launch_imma_t<MODE, 4, WARPS, GPS, 1>(l, a);
    return launch_imma_t<MODE, 3, WARPS, GPS, 1>(l, a);
}

template <int MODE>
cudaError_t launch_imma_mode(const Launch& l, const AffineArgs& a, bool* handled) {
    const cudaError_t e = a.cols % 256 != 0 ? launch_imma_depth<MODE, 16, 2>(l, a) : launch_imma_depth<MODE, 8, 4>(l, a);
    if (e == cudaErrorNotSupported) return cudaSuccess;  // not handled: the caller falls back
    *handled = true;
    return e;
}

}  // namespace

// Launches the integer-MMA kernel when the shape is eligible (group 64, batch <= 2, cols a
// multiple of 128, 16-byte aligned operands, every segment but the last a multiple of 16
// rows, digit planes small enough to stay resident); *handled tells the caller whether it did.
cudaError_t launch_affine_imma(const Launch& l, int mode, const AffineArgs& a, int group, bool* handled) {
    *handled = false;
    if (group != kGroup || a.batch > 2 || a.cols % 128 != 0) return cudaSuccess;
    const int nw = (mode == kAffineGateUp || mode == kAffineDual) ? 2 : 1;
    if (a.nseg > 1) {
        if (nw != 1 || a.nseg > 3 || mode != kAffinePlain) return cudaErrorInvalidValue;
        for (int i = 0; i < a.nseg; ++i) {
            if ((reinterpret_cast<uintptr_t>(a.seg[i].w) | reinterpret_cast<uintptr_t>(a.seg[i].s) | reinterpret_cast<uintptr_t>(a.seg[i].b)) & 15u) return cudaSuccess;
            if (i + 1 < a.nseg && a.seg[i].rows % kTileRows != 0) return cudaSuccess;
        }
    } else {
        for (int s = 0; s < nw; ++s)
            if ((reinterpret_cast<uintptr_t>(a.w[s]) | reinterpret_cast<uintptr_t>(a.s[s]) | reinterpret_cast<uintptr_t>(a.b[s])) & 15u) return cudaSuccess;
    }
    if (a.norm_w && (reinterpret_cast<uintptr_t>(a.norm_w) & 15u)) return cudaSuccess;
    if (reinterpret_cast<uintptr_t>(a.x) & 15u) return cudaSuccess;
    switch (mode) {
        case kAffinePlain: return launch_imma_mode<kAffinePlain>(l, a, handled);
        case kAffineAdd: return launch_imma_mode<kAffineAdd>(l, a, handled);
        case kAffineGateUp: return launch_imma_mode<kAffineGateUp>(l, a, handled);
        case kAffineDual: return launch_imma_mode<kAffineDual>(l, a, handled);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace smelt
