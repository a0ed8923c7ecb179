// Group-wise affine u4 matvec / small-batch matmul for sm_100a.
//
// Replaces the reference's affine_matvec family (Resources/Shaders/lut_matvec.metal:1157-1287
// affine_matvec, :1718-1817 fused_affine_matvec_add, :2152-2233 fused_affine_gate_up_swiglu,
// :1824-1908 fused_dual_affine_matvec, :3238-3461 the batched / ext forms) with ONE kernel
// template that serves batch 1..16:
//
//   y[b, r] = sum_g ( s[r,g] * sum_{k in g} q[r,k] * x[b,k]  +  b[r,g] * sum_{k in g} x[b,k] )
//
// Data path.  A CTA owns 16 output rows and one K-slice.  Its whole packed weight tile is
// fetched with 16-byte cp.async copies (512 contiguous bytes per warp instruction, L1
// bypassed) committed as four K-quarter groups, so compute on the first quarter starts while
// the rest is in flight; the copies and the scale / bias loads are issued before the
// programmatic-dependent-launch wait and therefore overlap the tail of the kernel that
// produces x.  Eight warps split the slice's groups; a warp dequantises a 16-row x
// GROUP-column block in registers (two LOP3 and two HFMA2 per eight nibbles give exact fp16
// integers 0..15) and multiplies it with up to 8 (or 16) activation rows by
// mma.sync.m16n8k16 with fp32 accumulators: the tensor pipe is used as a wide FMA unit so the
// CUDA cores only pay for the unpack.  The k order inside an MMA is permuted (nibbles i and
// i+4 of a word share a half2) and the activations are staged in shared memory in the same
// permuted order.  After every group the fp32 block sum is folded into the running row sums
// with the group's scale, and the bias term uses per-group activation sums computed once per
// CTA.  Warp partials are reduced through shared memory in a fixed order; K-slices of one row
// tile form a thread-block cluster and are reduced through distributed shared memory in rank
// order, so results are bit-reproducible.
#include "affine_matvec.h"

#include <cooperative_groups.h>

#include <cstdlib>

namespace cg = cooperative_groups;

namespace smelt {

namespace {

constexpr int kRows = 16;  // rows per CTA (one m16 tile)
constexpr int kQuarters = 4;  // cp.async commit groups per weight tile

struct SmemLayout {
    uint32_t bars, w, sb, xs, xsum, red, total;
    uint32_t pitch_w, pitch_sb, pitch_x;
};

template <int GROUP>
__host__ __device__ inline SmemLayout make_layout(int nw, int nb, int ks, int batch_rows, int kWarps) {
    SmemLayout L;
    const int gs = ks / GROUP;
    L.pitch_w = (uint32_t)(ks / 2 + GROUP / 2);          // ≡ GROUP/2 (mod 128): conflict-free row stride
    L.pitch_sb = (uint32_t)((gs | 1) * 4);               // odd number of fp16 {scale,bias} pairs per row
    L.pitch_x = (uint32_t)(ks * 2 + 16);                 // ≡ 16 (mod 128)
    uint32_t off = 0;
    L.bars = off; off += 256;  // a block of zeros (B operand of threads past the batch)
    L.w = off; off += (uint32_t)nw * kRows * L.pitch_w;
    off = (off + 15u) & ~15u;
    L.sb = off; off += (uint32_t)nw * kRows * L.pitch_sb;
    off = (off + 15u) & ~15u;
    L.xs = off; off += (uint32_t)batch_rows * L.pitch_x;
    off = (off + 15u) & ~15u;
    L.xsum = off; off += (uint32_t)gs * nb * 4;
    off = (off + 15u) & ~15u;
    L.red = L.w;  // the reduction buffer reuses the weight tile once every warp is done with it
    {
        const uint32_t red_bytes = (uint32_t)kWarps * 32 * 4 * (nb / 8) * nw * 4;
        if (L.w + red_bytes > off) off = L.w + red_bytes;
    }
    L.total = off;
    return L;
}

// Eight nibbles of one packed word -> four half2 of exact integers:
// {n0,n4} {n1,n5} {n2,n6} {n3,n7}.
__device__ __forceinline__ void dequant8(uint32_t w, uint32_t p[4]) {
    const uint32_t kMagic = 0x64006400u;  // half2(1024, 1024)
    const __half2 k1024 = u32_as_h2(0x64006400u);
    const __half2 k16th = u32_as_h2(0x2C002C00u);   // half2(1/16)
    const __half2 km64 = u32_as_h2(0xD400D400u);    // half2(-64)
    uint32_t lo = lop3_and_or(w, 0x000F000Fu, kMagic);
    uint32_t hi = lop3_and_or(w, 0x00F000F0u, kMagic);
    uint32_t w2 = w >> 8;
    uint32_t lo2 = lop3_and_or(w2, 0x000F000Fu, kMagic);
    uint32_t hi2 = lop3_and_or(w2, 0x00F000F0u, kMagic);
    p[0] = h2_as_u32(__hsub2(u32_as_h2(lo), k1024));
    p[1] = h2_as_u32(__hfma2(u32_as_h2(hi), k16th, km64));
    p[2] = h2_as_u32(__hsub2(u32_as_h2(lo2), k1024));
    p[3] = h2_as_u32(__hfma2(u32_as_h2(hi2), k16th, km64));
}

template <int N>
struct WordLoad;
template <>
struct WordLoad<1> {
    static __device__ __forceinline__ void ld(const uint8_t* p, uint32_t w[1]) { w[0] = *reinterpret_cast<const uint32_t*>(p); }
};
template <>
struct WordLoad<2> {
    static __device__ __forceinline__ void ld(const uint8_t* p, uint32_t w[2]) {
        uint2 v = *reinterpret_cast<const uint2*>(p);
        w[0] = v.x; w[1] = v.y;
    }
};
template <>
struct WordLoad<4> {
    static __device__ __forceinline__ void ld(const uint8_t* p, uint32_t w[4]) {
        uint4 v = *reinterpret_cast<const uint4*>(p);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    }
};

template <int MODE, int GROUP, int NBT, int kWarps>
__global__ void __launch_bounds__(kWarps * 32, kWarps == 16 ? 2 : 3) affine_mma_kernel(const AffineArgs a) {
    constexpr int kThreads = kWarps * 32;
    constexpr int NW = (MODE == kAffineGateUp || MODE == kAffineDual) ? 2 : 1;
    constexpr int NB = NBT * 8;
    constexpr int WPT = GROUP / 32;  // packed words per thread per row per group

    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * kRows;
    const int k0 = blockIdx.y * a.ks;                       // first column of this CTA's slice
    const int ks = min(a.ks, a.cols - k0);                  // columns in this slice
    const int gs = ks / GROUP;                              // groups in this slice
    const int groups_total = a.cols / GROUP;
    const SmemLayout L = make_layout<GROUP>(NW, NB, a.ks, a.batch, kWarps);
    uint8_t* szero = smem + L.bars;
    uint8_t* sw = smem + L.w;
    uint32_t* ssb = reinterpret_cast<uint32_t*>(smem + L.sb);
    uint8_t* sx = smem + L.xs;
    float* sxsum = reinterpret_cast<float*>(smem + L.xsum);
    float* sred = reinterpret_cast<float*>(smem + L.red);

    const int gq = (gs + kQuarters - 1) / kQuarters;        // groups per K-quarter

    // ── weight prefetch: independent of the upstream kernel, issued before the PDL wait ──
    // A warp copies one row segment at a time, 512 contiguous bytes per instruction.
    for (int q = 0; q < kQuarters; ++q) {
        const int c0 = min(q * gq, gs) * (GROUP / 32), c1 = min((q + 1) * gq, gs) * (GROUP / 32);  // 16-byte chunks
#pragma unroll
        for (int rr = warp; rr < NW * kRows; rr += kWarps) {  // rr = set * 16 + row
            const int set = rr / kRows, r = rr % kRows;
            if (row0 + r < a.rows) {
                const uint8_t* src = a.w[set] + (size_t)(row0 + r) * (a.cols / 2) + k0 / 2;
                uint8_t* dst = sw + (size_t)rr * L.pitch_w;
                for (int c = c0 + lane; c < c1; c += 32) cp_async16(dst + c * 16, src + c * 16);
            }
        }
        cp_async_commit();
    }
    // {scale, bias} of every (row, group) of the slice as fp16 pairs: one 32-bit read per row in
    // the main loop.
    {
        const bool vec = ((groups_total * 2) % 16 == 0) && ((k0 / GROUP * 2) % 16 == 0) && (gs % 8 == 0) &&
                         ((reinterpret_cast<uintptr_t>(a.s[0]) | reinterpret_cast<uintptr_t>(a.b[0]) |
                           reinterpret_cast<uintptr_t>(a.s[NW - 1]) | reinterpret_cast<uintptr_t>(a.b[NW - 1])) & 15u) == 0;
#pragma unroll
        for (int rr = warp; rr < NW * kRows; rr += kWarps) {
            const int set = rr / kRows, r = rr % kRows;
            uint32_t* dst = ssb + (size_t)rr * (L.pitch_sb / 4);
            const bool valid = row0 + r < a.rows;
            const size_t base = (size_t)(row0 + r) * groups_total + k0 / GROUP;
            if (vec) {
                for (int c = lane; c < gs / 8; c += 32) {  // 8 groups = 16 bytes of scales
                    uint4 sv = make_uint4(0, 0, 0, 0), bv = make_uint4(0, 0, 0, 0);
                    if (valid) {
                        sv = __ldg(reinterpret_cast<const uint4*>(a.s[set] + base + c * 8));
                        bv = __ldg(reinterpret_cast<const uint4*>(a.b[set] + base + c * 8));
                    }
                    const uint32_t sw4[4] = {sv.x, sv.y, sv.z, sv.w}, bw4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        dst[c * 8 + 2 * j] = __byte_perm(sw4[j], bw4[j], 0x5410);      // {scale, bias} of group 2j
                        dst[c * 8 + 2 * j + 1] = __byte_perm(sw4[j], bw4[j], 0x7632);  // group 2j+1
                    }
                }
            } else {
                for (int gi = lane; gi < gs; gi += 32)
                    dst[gi] = valid ? ((uint32_t)__half_as_ushort(a.s[set][base + gi]) | ((uint32_t)__half_as_ushort(a.b[set][base + gi]) << 16)) : 0u;
            }
        }
    }

    pdl_trigger();
    pdl_wait();
    if (dyn_skip(a.dyn)) {
        cp_async_wait<0>();  // copies in flight must land before the CTA's shared memory retires
        return;
    }

    // ── activations: permuted copy into shared memory + per-group sums ──
    {
        const int chunks = ks / 8;  // 8-column chunks per batch row
        constexpr int CPG = GROUP / 8;  // chunks per group
        for (int b = 0; b < a.batch; ++b) {
            const __half* xr = a.x + (size_t)b * a.cols + k0;
            uint8_t* xd = sx + (size_t)b * L.pitch_x;
            for (int base = 0; base < chunks; base += kThreads) {
                const int c8 = base + tid;
                float sum = 0.f;
                if (c8 < chunks) {
                    const uint4 v = *reinterpret_cast<const uint4*>(xr + c8 * 8);
                    const float2 f0 = __half22float2(u32_as_h2(v.x)), f1 = __half22float2(u32_as_h2(v.y));
                    const float2 f2 = __half22float2(u32_as_h2(v.z)), f3 = __half22float2(u32_as_h2(v.w));
                    sum = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
                    uint4 o;  // x0 x4 | x1 x5 | x2 x6 | x3 x7
                    o.x = __byte_perm(v.x, v.z, 0x5410);
                    o.y = __byte_perm(v.x, v.z, 0x7632);
                    o.z = __byte_perm(v.y, v.w, 0x5410);
                    o.w = __byte_perm(v.y, v.w, 0x7632);
                    *reinterpret_cast<uint4*>(xd + c8 * 16) = o;
                }
#pragma unroll
                for (int o = 1; o < CPG; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                if (c8 < chunks && (c8 % CPG) == 0) sxsum[(c8 / CPG) * NB + b] = sum;
            }
        }
        for (int i = tid; i < gs * NB; i += kThreads)
            if ((i % NB) >= a.batch) sxsum[i] = 0.f;
        if (tid < GROUP / 8) reinterpret_cast<uint4*>(szero)[tid] = make_uint4(0, 0, 0, 0);  // read by threads past the batch
    }

    // ── main loop: this warp's groups, quarter by quarter ──
    float acc[NW][NBT][4];
#pragma unroll
    for (int s = 0; s < NW; ++s)
#pragma unroll
        for (int n = 0; n < NBT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[s][n][i] = 0.f;

    // Per-thread base pointers; inside the loop everything advances by compile-time strides.
    const uint8_t* pw_base[NW];
    const uint32_t* psb_base[NW];
#pragma unroll
    for (int s = 0; s < NW; ++s) {
        pw_base[s] = sw + (size_t)(s * kRows + g) * L.pitch_w + t * (GROUP / 8);
        psb_base[s] = ssb + (size_t)(s * kRows + g) * (L.pitch_sb / 4);
    }
    const size_t w_row8 = 8 * (size_t)L.pitch_w;        // rows g -> g+8
    const size_t sb_row8 = 8 * (size_t)(L.pitch_sb / 4);
    // Batch rows this thread feeds as the B operand; threads past the batch read a row of zeros.
    const uint8_t* px_base[NBT];
    int px_stride[NBT];
#pragma unroll
    for (int n = 0; n < NBT; ++n) {
        const int b = n * 8 + g;
        px_base[n] = b < a.batch ? sx + (size_t)b * L.pitch_x + t * (GROUP / 2) : szero;
        px_stride[n] = b < a.batch ? GROUP * 2 : 0;
    }
    const float* pxs_base = sxsum + 2 * t;

    for (int q = 0; q < kQuarters; ++q) {
        // Quarter q is complete once every thread has waited for its own copies of the first
        // q+1 commit groups and the CTA has synchronised (which also publishes x and the scales).
        if (q == 0) cp_async_wait<3>();
        else if (q == 1) cp_async_wait<2>();
        else if (q == 2) cp_async_wait<1>();
        else cp_async_wait<0>();
        __syncthreads();
        const int g_hi = min((q + 1) * gq, gs);
#pragma unroll 1
        for (int gi = min(q * gq, gs) + warp; gi < g_hi; gi += kWarps) {
            uint32_t xb[NBT][WPT * 4];
#pragma unroll
            for (int n = 0; n < NBT; ++n) {
                const uint8_t* px = px_base[n] + gi * px_stride[n];
#pragma unroll
                for (int j = 0; j < WPT; ++j) {
                    const uint4 v = *reinterpret_cast<const uint4*>(px + j * 16);
                    xb[n][4 * j + 0] = v.x; xb[n][4 * j + 1] = v.y; xb[n][4 * j + 2] = v.z; xb[n][4 * j + 3] = v.w;
                }
            }
            float2 xs[NBT];
#pragma unroll
            for (int n = 0; n < NBT; ++n) xs[n] = *reinterpret_cast<const float2*>(pxs_base + gi * NB + n * 8);
#pragma unroll
            for (int s = 0; s < NW; ++s) {
                uint32_t wa[WPT], wb[WPT];
                const uint8_t* pw = pw_base[s] + (size_t)gi * (GROUP / 2);
                WordLoad<WPT>::ld(pw, wa);
                WordLoad<WPT>::ld(pw + w_row8, wb);
                const float2 f0 = __half22float2(u32_as_h2(psb_base[s][gi]));            // {scale, bias}, row g
                const float2 f1 = __half22float2(u32_as_h2(psb_base[s][gi + sb_row8]));  // row g+8
                float c[NBT][4];
#pragma unroll
                for (int j = 0; j < WPT; ++j) {
                    uint32_t pa[4], pb[4];
                    dequant8(wa[j], pa);
                    dequant8(wb[j], pb);
#pragma unroll
                    for (int n = 0; n < NBT; ++n) {
                        if (j == 0) mma16816_zero(c[n], pa[0], pb[0], pa[1], pb[1], xb[n][0], xb[n][1]);
                        else mma16816(c[n], pa[0], pb[0], pa[1], pb[1], xb[n][4 * j + 0], xb[n][4 * j + 1]);
                        mma16816(c[n], pa[2], pb[2], pa[3], pb[3], xb[n][4 * j + 2], xb[n][4 * j + 3]);
                    }
                }
#pragma unroll
                for (int n = 0; n < NBT; ++n) {
                    acc[s][n][0] = fmaf(f0.x, c[n][0], acc[s][n][0]); acc[s][n][0] = fmaf(f0.y, xs[n].x, acc[s][n][0]);
                    acc[s][n][1] = fmaf(f0.x, c[n][1], acc[s][n][1]); acc[s][n][1] = fmaf(f0.y, xs[n].y, acc[s][n][1]);
                    acc[s][n][2] = fmaf(f1.x, c[n][2], acc[s][n][2]); acc[s][n][2] = fmaf(f1.y, xs[n].x, acc[s][n][2]);
                    acc[s][n][3] = fmaf(f1.x, c[n][3], acc[s][n][3]); acc[s][n][3] = fmaf(f1.y, xs[n].y, acc[s][n][3]);
                }
            }
        }
    }

    // ── fixed-order reduction across the CTA's warps ──
    constexpr int VPT = NW * NBT * 4;  // values per thread
    __syncthreads();  // sred aliases the weight tile: wait until no warp reads weights any more
    {
        float* dst = sred + (size_t)(warp * 32 + lane) * VPT;
#pragma unroll
        for (int s = 0; s < NW; ++s)
#pragma unroll
            for (int n = 0; n < NBT; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) dst[(s * NBT + n) * 4 + i] = acc[s][n][i];
    }
    __syncthreads();
    float tot[VPT];
    if (warp == 0) {
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) sum += sred[(size_t)(w * 32 + lane) * VPT + v];
            tot[v] = sum;
        }
    }

    // ── fixed-order reduction across the K-slices (cluster ranks) through distributed smem ──
    if (a.nsplit > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        const unsigned rank = cluster.block_rank();
        cluster.sync();  // every CTA of the cluster is done reading its own sred
        if (warp == 0 && rank != 0) {
            float* remote = cluster.map_shared_rank(sred, 0);
#pragma unroll
            for (int v = 0; v < VPT; ++v) remote[(size_t)(rank * 32 + lane) * VPT + v] = tot[v];
        }
        cluster.sync();
        if (rank != 0) return;
        if (warp == 0) {
            for (int r = 1; r < a.nsplit; ++r)
#pragma unroll
                for (int v = 0; v < VPT; ++v) tot[v] += sred[(size_t)(r * 32 + lane) * VPT + v];
        }
    }
    if (warp != 0) return;

    // ── epilogue: thread (g,t) owns rows g, g+8 and batch columns 2t, 2t+1 of every n-tile ──
#pragma unroll
    for (int n = 0; n < NBT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = row0 + g + (i >> 1) * 8;
            const int b = n * 8 + 2 * t + (i & 1);
            if (row >= a.rows || b >= a.batch) continue;
            const size_t o = (size_t)b * a.rows + row;
            const float v0 = tot[(0 * NBT + n) * 4 + i];
            if (MODE == kAffinePlain) {
                a.y[o] = __float2half_rn(v0);
            } else if (MODE == kAffineAdd) {
                // half(acc) first, then an fp16 add with the residual (lut_matvec.metal:1802-1803)
                a.y[o] = __hadd(__float2half_rn(v0), a.residual[o]);
            } else if (MODE == kAffineGateUp) {
                const float v1 = tot[(1 * NBT + n) * 4 + i];
                a.y[o] = __float2half_rn(v0 / (1.0f + expf(-v0)) * v1);  // lut_matvec.metal:2228
            } else {
                a.y[o] = __float2half_rn(v0);
                a.y2[o] = __float2half_rn(tot[(1 * NBT + n) * 4 + i]);
            }
        }
}

// Largest K-slice a CTA stages (columns).  Smaller slices mean smaller tiles, more resident
// CTAs per SM and more of them per matrix.
constexpr int kMaxSliceCols = 4096;

template <int MODE, int GROUP, int NBT, int WARPS>
cudaError_t launch_t(const Launch& l, AffineArgs a) {
    constexpr int NW = (MODE == kAffineGateUp || MODE == kAffineDual) ? 2 : 1;
    // K-slice: an equal number of groups per slice, at most max_slice_cols() columns, shrunk
    // further until the tile fits in shared memory.
    const int groups = a.cols / GROUP;
    int max_gs = kMaxSliceCols / GROUP, nsplit = 1;
    if (max_gs < 1) max_gs = 1;
    SmemLayout L;
    for (;; max_gs /= 2) {
        if (max_gs == 0) return cudaErrorInvalidValue;
        nsplit = (groups + max_gs - 1) / max_gs;
        if (nsplit > 8) return cudaErrorInvalidValue;
        const int gs = (groups + nsplit - 1) / nsplit;
        nsplit = (groups + gs - 1) / gs;
        a.ks = gs * GROUP;
        L = make_layout<GROUP>(NW, NBT * 8, a.ks, a.batch, WARPS);
        if (L.total <= 200u * 1024u) break;
    }
    a.nsplit = nsplit;
    a.dyn = dev_dyn(l);
    auto kern = affine_mma_kernel<MODE, GROUP, NBT, WARPS>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L.total);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((a.rows + kRows - 1) / kRows, nsplit, 1);
    cfg.blockDim = dim3(WARPS * 32, 1, 1);
    cfg.dynamicSmemBytes = L.total;
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (nsplit > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = nsplit;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (l.pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    prefer_max_shared(kern);
    return cudaLaunchKernelEx(&cfg, kern, a);
}

template <int MODE, int GROUP>
cudaError_t launch_nb(const Launch& l, const AffineArgs& a) {
    if (a.batch <= 8) return launch_t<MODE, GROUP, 1, 16>(l, a);
    if (a.batch <= 16) return launch_t<MODE, GROUP, 2, 8>(l, a);
    return cudaErrorInvalidValue;
}

template <int MODE>
cudaError_t launch_group(const Launch& l, const AffineArgs& a, int group) {
    switch (group) {
        case 32: return launch_nb<MODE, 32>(l, a);
        case 64: return launch_nb<MODE, 64>(l, a);
        case 128: return launch_nb<MODE, 128>(l, a);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

cudaError_t launch_affine(const Launch& l, int mode, const AffineArgs& args, int group) {
    if (args.rows <= 0 || args.cols <= 0 || args.batch <= 0 || args.cols % group != 0) return cudaErrorInvalidValue;
    if (args.batch > 64) {  // tcgen05 QMM, wide form: the weights are expanded once per 512 batch rows
        bool handled = false;
        cudaError_t e = launch_affine_qmm_wide(l, mode, args, group, &handled);
        if (handled || e != cudaSuccess) return e;
    }
    if (args.batch >= 17) {  // tcgen05 QMM: the weights cross HBM once per 64 batch rows
        bool handled = false;
        cudaError_t e = launch_affine_qmm(l, mode, args, group, &handled);
        if (handled || e != cudaSuccess) return e;
    }
    // Batches beyond 16 rows are processed in passes of 16 (weights re-streamed per pass).
    if (args.batch > 16) {
        for (int b0 = 0; b0 < args.batch; b0 += 16) {
            AffineArgs s = args;
            s.batch = args.batch - b0 < 16 ? args.batch - b0 : 16;
            s.x = args.x + (size_t)b0 * args.cols;
            s.y = args.y + (size_t)b0 * args.rows;
            if (args.y2) s.y2 = args.y2 + (size_t)b0 * args.rows;
            if (args.residual) s.residual = args.residual + (size_t)b0 * args.rows;
            for (int i = 0; i < args.nseg && i < 3; ++i) s.seg[i].y = args.seg[i].y + (size_t)b0 * args.seg[i].rows;
            cudaError_t e = launch_affine(l, mode, s, group);
            if (e != cudaSuccess) return e;
        }
        return cudaSuccess;
    }
    {
        bool handled = false;
        cudaError_t e = launch_affine_imma(l, mode, args, group, &handled);  // batch 1 and 2
        if (handled || e != cudaSuccess) return e;
        e = launch_affine_stream(l, mode, args, group, &handled);
        if (handled || e != cudaSuccess) return e;
        if (args.norm_w || args.nseg > 1) return cudaErrorNotSupported;  // only the streaming kernel fuses these
    }
    switch (mode) {
        case kAffinePlain: return launch_group<kAffinePlain>(l, args, group);
        case kAffineAdd: return launch_group<kAffineAdd>(l, args, group);
        case kAffineGateUp: return launch_group<kAffineGateUp>(l, args, group);
        case kAffineDual: return launch_group<kAffineDual>(l, args, group);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace smelt
