// Streaming (persistent, multistage) form of the group-64 affine u4 matvec for batch <= 16
// (eight batch rows per pass).
//
// Same arithmetic and the same reference kernels as affine_matvec.cu
// (Resources/Shaders/lut_matvec.metal:1157-1287, :1718-1817, :2152-2233, :1824-1908); what
// changes is how the weight stream is organised, because at B200 bandwidth the per-tile fixed
// work of the one-tile-per-CTA kernel (activation staging, barriers, load/compute phases that
// line up across the CTAs of an SM) costs more than the arithmetic.
//
// A persistent CTA of eight warps walks 16-row tiles (tile index = blockIdx.x + i * gridDim.x).
// The packed weights, scales and biases of a tile arrive as a continuous sequence of stages of
// 1024 columns through a ring of cp.async buffers (16-byte copies, 512 contiguous bytes per
// row); the ring keeps running across tile boundaries, so HBM requests are always in flight
// while the tensor pipe works on the oldest stage.  The activations are staged once per CTA
// (permuted for the MMA operand order, with their per-group sums), not once per tile.  Warp
// wk owns groups 2wk, 2wk+1 of every stage; its fp32 row sums live in registers for the whole
// K loop and the eight K-partials of a tile are added in a fixed order through shared memory,
// so results are bit-reproducible.  The first stages are
// requested before the programmatic-dependent-launch wait: weight traffic overlaps the tail
// of the kernel that produces x.
#include <cstdlib>

#include "affine_matvec.h"

namespace smelt {

namespace {

constexpr int kGroup = 64;
constexpr int kTileRows = 16;
constexpr int kStageCols = 1024;                      // 16 groups, two per warp
constexpr int kRowBytes = kStageCols / 2;             // 512 packed bytes per row per stage
constexpr int kPitchW = kRowBytes + 32;               // ≡ 32 (mod 128): conflict-free LDS.64 across rows
constexpr int kSetW = kTileRows * kPitchW;            // 8704
constexpr int kSetS = kTileRows * 32;                 // 16 fp16 scales per row
constexpr int kSetBytes = kSetW + 2 * kSetS;          // 9728: [W | scales | biases]

struct StreamLayout {
    uint32_t zero, ring, xs, xsum, red, total, pitch_x, stage_bytes;
};

__host__ __device__ inline StreamLayout stream_layout(int nw, int stages, int cols, int batch, int warps = 8) {
    StreamLayout L;
    L.stage_bytes = (uint32_t)nw * kSetBytes;
    L.pitch_x = (uint32_t)cols * 2 + 16;              // ≡ 16 (mod 128)
    uint32_t off = 0;
    L.zero = off; off += 256;
    L.ring = off; off += (uint32_t)stages * L.stage_bytes;
    L.xs = off; off += (uint32_t)batch * L.pitch_x;
    off = (off + 15u) & ~15u;
    L.xsum = off; off += (uint32_t)(cols / kGroup) * 8 * 4;
    L.red = off; off += (uint32_t)warps * 32u * (uint32_t)(4 * nw) * 4u;
    L.total = off;
    return L;
}

__device__ __forceinline__ void dequant8s(uint32_t w, uint32_t p[4]) {
    const uint32_t kMagic = 0x64006400u;              // half2(1024, 1024)
    const __half2 k1024 = u32_as_h2(0x64006400u);
    const __half2 k16th = u32_as_h2(0x2C002C00u);     // half2(1/16)
    const __half2 km64 = u32_as_h2(0xD400D400u);      // half2(-64)
    const uint32_t lo = lop3_and_or(w, 0x000F000Fu, kMagic);
    const uint32_t hi = lop3_and_or(w, 0x00F000F0u, kMagic);
    const uint32_t w2 = w >> 8;
    const uint32_t lo2 = lop3_and_or(w2, 0x000F000Fu, kMagic);
    const uint32_t hi2 = lop3_and_or(w2, 0x00F000F0u, kMagic);
    p[0] = h2_as_u32(__hsub2(u32_as_h2(lo), k1024));          // {n0, n4}
    p[1] = h2_as_u32(__hfma2(u32_as_h2(hi), k16th, km64));    // {n1, n5}
    p[2] = h2_as_u32(__hsub2(u32_as_h2(lo2), k1024));         // {n2, n6}
    p[3] = h2_as_u32(__hfma2(u32_as_h2(hi2), k16th, km64));   // {n3, n7}
}

// Eight warps: warp wk owns groups 2wk, 2wk+1 of every stage and up to three CTAs share an SM.
template <int MODE, int STAGES, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 16 ? 1 : (STAGES == 3 ? 3 : 2)) affine_stream_kernel(const AffineArgs a) {
    constexpr int NW = (MODE == kAffineGateUp || MODE == kAffineDual) ? 2 : 1;
    constexpr int kThreads = WARPS * 32;
    constexpr int GPW = 16 / WARPS;  // groups of a stage per warp (2 or 1)
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int wk = warp;  // this warp's share of every stage: groups GPW * wk ...
    const StreamLayout L = stream_layout(NW, STAGES, a.cols, a.batch, WARPS);
    uint8_t* ring = smem + L.ring;
    uint8_t* sx = smem + L.xs;
    float* sxsum = reinterpret_cast<float*>(smem + L.xsum);
    float* sred = reinterpret_cast<float*>(smem + L.red);

    const int tiles_total = a.nseg > 1 ? a.ks : (a.rows + kTileRows - 1) / kTileRows;  // ks carries the tile count of a multi-segment launch
    const int spt = a.cols / kStageCols;  // stages per tile
    const int my_tiles = blockIdx.x < tiles_total ? (tiles_total - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int total_stages = my_tiles * spt;
    const int groups_total = a.cols / kGroup;

    // Plain mode may cover up to three tensors (segments) that share x; a tile belongs to one.
    const int seg_end0 = (a.seg[0].rows + kTileRows - 1) / kTileRows;
    const int seg_end1 = seg_end0 + (a.nseg > 1 ? (a.seg[1].rows + kTileRows - 1) / kTileRows : 0);
    auto seg_of = [&](int tile, int& first_tile) {
        const int sg = (a.nseg > 1 && tile >= seg_end0) + (a.nseg > 2 && tile >= seg_end1);
        first_tile = sg == 0 ? 0 : (sg == 1 ? seg_end0 : seg_end1);
        return sg;
    };

    // ── producer side: every thread copies a fixed part of each stage ──
    const int ld_chunk = tid & 31, ld_row = tid >> 5;  // 16-byte chunk ld_chunk of row ld_row (and of row ld_row + 8 with eight warps)
    int f_tile = blockIdx.x, f_ks = 0, f_n = 0;        // next stage to request
    auto fetch = [&]() {
        if (f_n < total_stages) {
            uint8_t* st = ring + (size_t)(f_n % STAGES) * L.stage_bytes;
            int row0 = f_tile * kTileRows, rows = a.rows;
            const uint8_t* wsrc[NW];
            const __half* ssrc[NW];
            const __half* bsrc[NW];
            if (NW == 1) {
                int first;
                const int sg = seg_of(f_tile, first);
                row0 = (f_tile - first) * kTileRows;
                rows = sg == 0 ? a.seg[0].rows : (sg == 1 ? a.seg[1].rows : a.seg[2].rows);
                wsrc[0] = sg == 0 ? a.seg[0].w : (sg == 1 ? a.seg[1].w : a.seg[2].w);
                ssrc[0] = sg == 0 ? a.seg[0].s : (sg == 1 ? a.seg[1].s : a.seg[2].s);
                bsrc[0] = sg == 0 ? a.seg[0].b : (sg == 1 ? a.seg[1].b : a.seg[2].b);
            } else {
#pragma unroll
                for (int s = 0; s < NW; ++s) { wsrc[s] = a.w[s]; ssrc[s] = a.s[s]; bsrc[s] = a.b[s]; }
            }
#pragma unroll
            for (int s = 0; s < NW; ++s) {
                uint8_t* dst = st + s * kSetBytes;
#pragma unroll
                for (int h = 0; h < GPW; ++h) {
                    const int r = ld_row + 8 * h;
                    if (row0 + r < rows)
                        cp_async16(dst + r * kPitchW + ld_chunk * 16,
                                   wsrc[s] + (size_t)(row0 + r) * (a.cols / 2) + (size_t)f_ks * kRowBytes + ld_chunk * 16);
                }
                if (warp < 2 && row0 + (lane >> 1) < rows) {  // warp 0: scales, warp 1: biases; two 16-byte chunks per row
                    const __half* src = (warp == 0 ? ssrc[s] : bsrc[s]) + (size_t)(row0 + (lane >> 1)) * groups_total + f_ks * 16 + (lane & 1) * 8;
                    cp_async16(dst + kSetW + warp * kSetS + lane * 16, src);
                }
            }
            ++f_n;
            if (++f_ks == spt) { f_ks = 0; f_tile += gridDim.x; }
        }
        cp_async_commit();  // always commit so that group counting stays uniform
    };
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) fetch();

    uint64_t* xbar = reinterpret_cast<uint64_t*>(smem + L.zero + 64);  // past the 32 zero bytes the MMA reads
    if (tid == 0) { mbar_init(xbar, 1); mbar_fence_init(); }
    __syncthreads();

    pdl_trigger();
    pdl_wait();
    if (dyn_skip(a.dyn)) {
        cp_async_wait<0>();  // copies in flight must land before the CTA's shared memory retires
        return;
    }

    // ── activations: permuted copy into shared memory + per-group sums, once per CTA ──
    {
        const int chunks = a.cols / 8;
        // Raw copy of every batch row first, everything in flight at once (one load latency for
        // the whole block instead of one per row and pass); the permutation below stays inside a
        // 16-byte chunk, so it is done in place.
        // One bulk copy per row, tracked by an mbarrier of their own, so the wait does not also
        // wait for the weight stages requested above.
        if (tid == 0) {
            mbar_arrive_expect_tx(xbar, (uint32_t)a.batch * (uint32_t)a.cols * 2u);
            for (int b = 0; b < a.batch; ++b)
                bulk_g2s(sx + (size_t)b * L.pitch_x, a.x + (size_t)b * a.cols, (uint32_t)a.cols * 2u, xbar);
        }
        if (!mbar_wait_bounded(xbar, 0)) {  // gave up: report, let the weight copies land, leave
            if (tid == 0 && a.err) atomicOr(a.err, KERR_BARRIER_TIMEOUT);
            cp_async_wait<0>();
            return;
        }
        for (int b = 0; b < a.batch; ++b) {
            uint8_t* xd = sx + (size_t)b * L.pitch_x;
            float rs = 0.f;
            if (a.norm_w) {
                // rms_norm_1pw (Resources/Shaders/norms.metal:9-67) folded into the staging pass
                // sred is free here: no tile has been reduced yet
                const float tot = cta256_sumsq_f16(reinterpret_cast<const __half*>(xd), a.cols, sred);
                rs = __frcp_rn(__fsqrt_rn(tot / (float)a.cols + a.norm_eps));
            }
            for (int base = 0; base < chunks; base += kThreads) {
                const int c8 = base + tid;
                float sum = 0.f;
                if (c8 < chunks) {
                    uint4 v = *reinterpret_cast<const uint4*>(xd + c8 * 16);
                    if (a.norm_w) {
                        const uint4 wv = *reinterpret_cast<const uint4*>(a.norm_w + c8 * 8);
                        v.x = rms_norm_1pw_pair(v.x, wv.x, rs); v.y = rms_norm_1pw_pair(v.y, wv.y, rs);
                        v.z = rms_norm_1pw_pair(v.z, wv.z, rs); v.w = rms_norm_1pw_pair(v.w, wv.w, rs);
                    }
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
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                if (c8 < chunks && (c8 & 7) == 0) sxsum[(c8 >> 3) * 8 + b] = sum;
            }
        }
        for (int i = tid; i < groups_total * 8; i += kThreads)
            if ((i & 7) >= a.batch) sxsum[i] = 0.f;
        if (tid < 2) reinterpret_cast<uint4*>(smem + L.zero)[tid] = make_uint4(0, 0, 0, 0);
    }

    // ── consumer side ──
    // B operand: batch row g of x, or a block of zeros for threads past the batch.
    const uint8_t* px_base = g < a.batch ? sx + (size_t)g * L.pitch_x + t * 32 : smem + L.zero;
    const int px_stride = g < a.batch ? kGroup * 2 : 0;
    const float* pxs_base = sxsum + 2 * t;
    const int w_off = g * kPitchW + wk * (GPW * 32) + t * 8;  // this thread's first word in a set's W block
    const int s_off = kSetW + g * 32 + wk * (GPW * 2);  // its scale(s); biases kSetS later

    float acc[NW][4];
#pragma unroll
    for (int s = 0; s < NW; ++s) acc[s][0] = acc[s][1] = acc[s][2] = acc[s][3] = 0.f;

    int c_tile = blockIdx.x, c_ks = 0;
    for (int n = 0; n < total_stages; ++n) {
        cp_async_wait<STAGES - 2>();  // this thread's copies of stage n have landed
        __syncthreads();              // ... everyone's have, and everyone is done with stage n-1
        fetch();                      // refill the buffer stage n-1 used
        const uint8_t* st = ring + (size_t)(n % STAGES) * L.stage_bytes;
        float2 sa[NW], ba[NW], sb[NW], bb[NW];  // {first, second group of this warp}: scale / bias of row g (a) and row g+8 (b)
#pragma unroll
        for (int s = 0; s < NW; ++s) {
            const uint8_t* base = st + s * kSetBytes + s_off;
            if (GPW == 2) {
                sa[s] = __half22float2(u32_as_h2(*reinterpret_cast<const uint32_t*>(base)));
                ba[s] = __half22float2(u32_as_h2(*reinterpret_cast<const uint32_t*>(base + kSetS)));
                sb[s] = __half22float2(u32_as_h2(*reinterpret_cast<const uint32_t*>(base + 8 * 32)));
                bb[s] = __half22float2(u32_as_h2(*reinterpret_cast<const uint32_t*>(base + kSetS + 8 * 32)));
            } else {
                sa[s] = make_float2(__half2float(*reinterpret_cast<const __half*>(base)), 0.f);
                ba[s] = make_float2(__half2float(*reinterpret_cast<const __half*>(base + kSetS)), 0.f);
                sb[s] = make_float2(__half2float(*reinterpret_cast<const __half*>(base + 8 * 32)), 0.f);
                bb[s] = make_float2(__half2float(*reinterpret_cast<const __half*>(base + kSetS + 8 * 32)), 0.f);
            }
        }
#pragma unroll
        for (int gg = 0; gg < GPW; ++gg) {
            const int gi = c_ks * 16 + wk * GPW + gg;  // group index within the row
            const uint8_t* px = px_base + gi * px_stride;
            const uint4 x0 = *reinterpret_cast<const uint4*>(px), x1 = *reinterpret_cast<const uint4*>(px + 16);
            const float2 xs = *reinterpret_cast<const float2*>(pxs_base + gi * 8);
#pragma unroll
            for (int s = 0; s < NW; ++s) {
                const uint8_t* base = st + s * kSetBytes;
                const uint2 wa = *reinterpret_cast<const uint2*>(base + w_off + gg * 32);
                const uint2 wb = *reinterpret_cast<const uint2*>(base + w_off + gg * 32 + 8 * kPitchW);
                uint32_t pa[4], pb[4];
                float c[4];
                dequant8s(wa.x, pa); dequant8s(wb.x, pb);
                mma16816_zero(c, pa[0], pb[0], pa[1], pb[1], x0.x, x0.y);
                mma16816(c, pa[2], pb[2], pa[3], pb[3], x0.z, x0.w);
                dequant8s(wa.y, pa); dequant8s(wb.y, pb);
                mma16816(c, pa[0], pb[0], pa[1], pb[1], x1.x, x1.y);
                mma16816(c, pa[2], pb[2], pa[3], pb[3], x1.z, x1.w);
                const float s0 = gg ? sa[s].y : sa[s].x, b0 = gg ? ba[s].y : ba[s].x, s1 = gg ? sb[s].y : sb[s].x, b1 = gg ? bb[s].y : bb[s].x;
                acc[s][0] = fmaf(s0, c[0], acc[s][0]); acc[s][0] = fmaf(b0, xs.x, acc[s][0]);
                acc[s][1] = fmaf(s0, c[1], acc[s][1]); acc[s][1] = fmaf(b0, xs.y, acc[s][1]);
                acc[s][2] = fmaf(s1, c[2], acc[s][2]); acc[s][2] = fmaf(b1, xs.x, acc[s][2]);
                acc[s][3] = fmaf(s1, c[3], acc[s][3]); acc[s][3] = fmaf(b1, xs.y, acc[s][3]);
            }
        }
        if (++c_ks == spt) {
            // ── tile done: add the warps' K-partials in a fixed order, write out ──
            float* dst = sred + (size_t)(wk * 32 + lane) * (4 * NW);
#pragma unroll
            for (int s = 0; s < NW; ++s)
#pragma unroll
                for (int i = 0; i < 4; ++i) { dst[s * 4 + i] = acc[s][i]; acc[s][i] = 0.f; }
            __syncthreads();
            if (wk == 0) {
                float tot[NW][4];
#pragma unroll
                for (int s = 0; s < NW; ++s)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float v = 0.f;
#pragma unroll
                        for (int k = 0; k < WARPS; ++k) v += sred[(size_t)(k * 32 + lane) * (4 * NW) + s * 4 + i];
                        tot[s][i] = v;
                    }
                int first = 0, rows = a.rows;
                __half* yout = a.y;
                if (NW == 1) {
                    const int sg = seg_of(c_tile, first);
                    rows = sg == 0 ? a.seg[0].rows : (sg == 1 ? a.seg[1].rows : a.seg[2].rows);
                    yout = sg == 0 ? a.seg[0].y : (sg == 1 ? a.seg[1].y : a.seg[2].y);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = (c_tile - first) * kTileRows + g + (i >> 1) * 8;
                    const int b = 2 * t + (i & 1);
                    if (row >= rows || b >= a.batch) continue;
                    const size_t o = (size_t)b * rows + row;
                    const float v0 = tot[0][i];
                    if (MODE == kAffinePlain) yout[o] = __float2half_rn(v0);
                    else if (MODE == kAffineAdd) yout[o] = __hadd(__float2half_rn(v0), a.residual[o]);  // lut_matvec.metal:1802-1803
                    else if (MODE == kAffineGateUp) a.y[o] = __float2half_rn(v0 / (1.0f + expf(-v0)) * tot[NW - 1][i]);  // :2228
                    else { a.y[o] = __float2half_rn(v0); a.y2[o] = __float2half_rn(tot[NW - 1][i]); }
                }
            }
            c_ks = 0;
            c_tile += gridDim.x;
        }
    }
    cp_async_wait<0>();
}

template <int MODE, int STAGES, int WARPS>
cudaError_t launch_stream_t(const Launch& l, AffineArgs a, int ctas_per_sm) {
    constexpr int NW = (MODE == kAffineGateUp || MODE == kAffineDual) ? 2 : 1;
    const StreamLayout L = stream_layout(NW, STAGES, a.cols, a.batch, WARPS);
    a.dyn = dev_dyn(l);
    auto kern = affine_stream_kernel<MODE, STAGES, WARPS>;
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
    int grid = sm * ctas_per_sm;
    if (grid > tiles) grid = tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(WARPS * 32, 1, 1);
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

template <int MODE>
cudaError_t launch_stream_mode(const Launch& l, const AffineArgs& a, bool* handled) {
    constexpr int NW = (MODE == kAffineGateUp || MODE == kAffineDual) ? 2 : 1;
    // Ring depth: the preferred one if two CTAs per SM fit beside it (about 113 KB each), else a
    // shallower one that lets them; when the activations leave room for one CTA only, the deepest
    // ring that fits (the ring then is all that hides the HBM latency).
    const uint32_t budget3 = 75u * 1024u, budget2 = 113u * 1024u, budget1 = 226u * 1024u;
    const int order[2][3] = {{NW == 2 ? 4 : 6, 4, 3}, {6, 4, 3}};
    for (int pass = 0; pass < 2; ++pass)
        for (int i = 0; i < 3; ++i) {
            const int st = order[pass][i];
            const uint32_t total = stream_layout(NW, st, a.cols, a.batch, 8).total;
            if (total > (pass == 0 ? budget2 : budget1)) continue;
            *handled = true;
            const int per_sm = (st == 3 && total <= budget3) ? 3 : (total <= budget2 ? 2 : 1);
            if (st == 6) return launch_stream_t<MODE, 6, 8>(l, a, per_sm);
            if (st == 4) return launch_stream_t<MODE, 4, 8>(l, a, per_sm);
            return launch_stream_t<MODE, 3, 8>(l, a, per_sm);
        }
    *handled = false;
    return cudaSuccess;
}

}  // namespace

// Launches the streaming kernel when the shape is eligible (group 64, batch <= 16, cols a
// multiple of 1024, 16-byte aligned operands; up to eight batch rows per pass, fewer when the
// activations would not stay resident);
// *handled tells the caller whether it did.
cudaError_t launch_affine_stream(const Launch& l, int mode, const AffineArgs& a, int group, bool* handled) {
    *handled = false;
    if (group != kGroup || a.batch > 16 || a.cols % kStageCols != 0) return cudaSuccess;
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
    // Rows of the batch that fit in shared memory beside the shallowest ring go in one pass;
    // a larger batch (or very wide activations) takes up to four passes over the same weights,
    // which the later passes find in L2 for the matrices of a decoder layer.
    int bmax = a.batch < 8 ? a.batch : 8;
    while (bmax > 0 && stream_layout(nw, 3, a.cols, bmax, 8).total > 226u * 1024u) --bmax;
    if (bmax == 0) return cudaSuccess;
    const int passes = (a.batch + bmax - 1) / bmax;
    if (passes > 4) return cudaSuccess;
    // Eight rows or fewer that need two passes: the general kernel's K split over a cluster is as fast.
    if (passes > 1 && a.batch <= 8 && !a.norm_w && a.nseg <= 1) return cudaSuccess;
    const int per_pass = (a.batch + passes - 1) / passes;
    for (int b0 = 0; b0 < a.batch; b0 += per_pass) {
        AffineArgs p = a;
        p.batch = a.batch - b0 < per_pass ? a.batch - b0 : per_pass;
        p.x = a.x + (size_t)b0 * a.cols;
        if (a.y) p.y = a.y + (size_t)b0 * a.rows;
        if (a.y2) p.y2 = a.y2 + (size_t)b0 * a.rows;
        if (a.residual) p.residual = a.residual + (size_t)b0 * a.rows;
        for (int i = 0; i < a.nseg && i < 3; ++i) p.seg[i].y = a.seg[i].y + (size_t)b0 * a.seg[i].rows;
        cudaError_t e;
        switch (mode) {
            case kAffinePlain: e = launch_stream_mode<kAffinePlain>(l, p, handled); break;
            case kAffineAdd: e = launch_stream_mode<kAffineAdd>(l, p, handled); break;
            case kAffineGateUp: e = launch_stream_mode<kAffineGateUp>(l, p, handled); break;
            case kAffineDual: e = launch_stream_mode<kAffineDual>(l, p, handled); break;
            default: return cudaErrorInvalidValue;
        }
        if (e != cudaSuccess || !*handled) return e;
    }
    return cudaSuccess;
}

}  // namespace smelt
