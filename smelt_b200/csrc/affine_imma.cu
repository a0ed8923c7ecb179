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
// One persistent CTA of 16 warps per SM walks 16-row tiles.  Inside a tile warp w owns a
// contiguous K range and streams it through its own ring of cp.async stages (128 columns
// each: 16 rows x 64 bytes of nibbles, swizzled so that the fragment loads are conflict free,
// plus the two groups' scales and biases).  A warp only waits for its own copies, so the main
// loop has no CTA-wide barrier; the rings keep running across tiles.  The 16 K-partials of a
// tile are added in warp order through shared memory (one barrier per tile), so results are
// bit-reproducible.  Shared memory and registers are sized so that the CTAs of the next
// launch fit beside this one: with programmatic dependent launch they become resident while
// this launch still computes and fill their rings (weights do not depend on the previous
// kernel) before they wait for it.
#include <cstdlib>

#include "affine_matvec.h"

namespace smelt {

namespace {

constexpr int kGroup = 64;
constexpr int kTileRows = 16;
constexpr int kChunkCols = 128;                        // two groups per ring stage
constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kSetW = kTileRows * (kChunkCols / 2);    // 1024 bytes of nibbles
constexpr int kSetS = kTileRows * 4;                   // 2 fp16 scales per row
constexpr int kSetBytes = kSetW + 2 * kSetS;           // 1152: [W | scales | biases]
constexpr int kDigits = 4;
constexpr uint32_t kMagic = 0x4B400000u;               // float 12582912 = 1.5 * 2^23
constexpr float kMagicF = 12582912.0f;

struct ImmaLayout {
    uint32_t zero, xq, pitch_x, xsum, xscale, red, ring, stage_bytes, total;
};

__host__ __device__ inline ImmaLayout imma_layout(int nw, int depth, int cols, int batch) {
    ImmaLayout L;
    L.stage_bytes = (uint32_t)nw * kSetBytes;
    L.pitch_x = (uint32_t)cols + 64u;                  // one byte per column per plane; ≡ 64 (mod 128)
    uint32_t off = 0;
    L.zero = off; off += 64;
    L.xq = off; off += (uint32_t)(kDigits * batch) * L.pitch_x;
    L.xsum = off; off += (uint32_t)(cols / kGroup) * 2u * 4u;       // [group][batch slot 0/1]
    L.xscale = off; off += 16;
    L.red = off; off += 2u * (uint32_t)nw * 2u * kTileRows * kWarps * 4u;  // [buffer][set][batch][row][warp]
    off = (off + 127u) & ~127u;
    L.ring = off; off += (uint32_t)kWarps * depth * L.stage_bytes;
    L.total = off;
    return L;
}

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}

// Largest |v| of the eight fp16 values in a 16-byte word, as a float.
__device__ __forceinline__ float amax8(const uint4& v) {
    const __half2 m = __hmax2(__hmax2(__habs2(u32_as_h2(v.x)), __habs2(u32_as_h2(v.y))),
                              __hmax2(__habs2(u32_as_h2(v.z)), __habs2(u32_as_h2(v.w))));
    const float2 f = __half22float2(m);
    return fmaxf(f.x, f.y);
}

// Four signed base-128 digits of X (|X| < 2^27), least significant first, each in [-64, 63]
// except the last, which takes what remains.
__device__ __forceinline__ void digits128(int X, int (&d)[4]) {
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        d[k] = ((X + 64) & 127) - 64;
        X = (X - d[k]) >> 7;
    }
    d[3] = X;
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

template <int MODE, int DEPTH>
__global__ void __launch_bounds__(kThreads, 2) affine_imma_kernel(const AffineArgs a) {
    constexpr int NW = (MODE == kAffineGateUp || MODE == kAffineDual) ? 2 : 1;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const ImmaLayout L = imma_layout(NW, DEPTH, a.cols, a.batch);
    uint8_t* xq = smem + L.xq;
    float* sxsum = reinterpret_cast<float*>(smem + L.xsum);
    float* sxscale = reinterpret_cast<float*>(smem + L.xscale);
    float* sred = reinterpret_cast<float*>(smem + L.red);
    uint8_t* ring = smem + L.ring + (size_t)warp * DEPTH * L.stage_bytes;

    const int tiles_total = a.ks;  // filled by the launcher
    const int nchunks = a.cols / kChunkCols;
    const int cpw = (nchunks + kWarps - 1) / kWarps;  // chunks per warp: a contiguous K range
    const int c_begin = min(warp * cpw, nchunks);
    const int cnt = min(c_begin + cpw, nchunks) - c_begin;
    const int my_tiles = (int)blockIdx.x < tiles_total ? (tiles_total - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int total_stages = my_tiles * cnt;
    const int groups_total = a.cols / kGroup;

    // Plain mode may cover up to three tensors (segments) that share x; a tile belongs to one.
    const int seg_end0 = (a.seg[0].rows + kTileRows - 1) / kTileRows;
    const int seg_end1 = seg_end0 + (a.nseg > 1 ? (a.seg[1].rows + kTileRows - 1) / kTileRows : 0);
    auto seg_of = [&](int tile, int& first_tile) {
        const int sg = (a.nseg > 1 && tile >= seg_end0) + (a.nseg > 2 && tile >= seg_end1);
        first_tile = sg == 0 ? 0 : (sg == 1 ? seg_end0 : seg_end1);
        return sg;
    };

    // ── producer side: each warp copies the stages it will consume ──
    const int sw = ((g >> 1) & 1) << 1;  // 16-byte chunk swizzle of rows g and g + 8
    int f_tile = blockIdx.x, f_j = 0, f_n = 0, f_slot = 0;
    auto fetch = [&]() {
        if (f_n < total_stages) {
            uint8_t* st = ring + (size_t)f_slot * L.stage_bytes;
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
            const int ch = c_begin + f_j;
#pragma unroll
            for (int s = 0; s < NW; ++s) {
                uint8_t* dst = st + s * kSetBytes;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int r = g + 8 * h;
                    if (row0 + r < rows)
                        cp_async16(dst + r * 64 + ((t ^ sw) * 16),
                                   wsrc[s] + (size_t)(row0 + r) * (a.cols / 2) + (size_t)ch * 64 + t * 16);
                }
                const int r = lane & 15;  // lanes 0-15: the rows' two scales; lanes 16-31: their two biases
                if (row0 + r < rows) {
                    const __half* src = (lane < 16 ? ssrc[s] : bsrc[s]) + (size_t)(row0 + r) * groups_total + ch * 2;
                    cp_async4(dst + kSetW + (lane >> 4) * kSetS + r * 4, src);
                }
            }
            ++f_n;
            f_slot = f_slot + 1 == DEPTH ? 0 : f_slot + 1;
            if (++f_j == cnt) { f_j = 0; f_tile += gridDim.x; }
        }
        cp_async_commit();  // always commit so that group counting stays uniform
    };
#pragma unroll
    for (int i = 0; i < DEPTH - 1; ++i) fetch();

    pdl_trigger();
    pdl_wait();
    if (dyn_skip(a.dyn)) {
        cp_async_wait<0>();  // copies in flight must land before the CTA's shared memory retires
        return;
    }

    // ── activations: digit planes + per-group sums, once per CTA ──
    {
        const int chunks = a.cols / 8;
        if (tid < 4) reinterpret_cast<uint4*>(smem + L.zero)[tid] = make_uint4(0, 0, 0, 0);
        if (a.batch == 1)
            for (int i = tid; i < groups_total; i += kThreads) sxsum[i * 2 + 1] = 0.f;
        for (int b = 0; b < a.batch; ++b) {
            const __half* xr = a.x + (size_t)b * a.cols;
            float rs = 0.f;
            if (a.norm_w) {
                // rms_norm_1pw (Resources/Shaders/norms.metal:9-67) folded into the staging pass;
                // sred is free here: no tile has been reduced yet
                const float tot = cta256_sumsq_f16(xr, a.cols, sred);
                rs = __frcp_rn(__fsqrt_rn(tot / (float)a.cols + a.norm_eps));
            }
            auto load8 = [&](int c8) {
                uint4 v = *reinterpret_cast<const uint4*>(xr + c8 * 8);
                if (a.norm_w) {
                    const uint4 wv = *reinterpret_cast<const uint4*>(a.norm_w + c8 * 8);
                    v.x = rms_norm_1pw_pair(v.x, wv.x, rs); v.y = rms_norm_1pw_pair(v.y, wv.y, rs);
                    v.z = rms_norm_1pw_pair(v.z, wv.z, rs); v.w = rms_norm_1pw_pair(v.w, wv.w, rs);
                }
                return v;
            };
            float m = 0.f;
            for (int c8 = tid; c8 < chunks; c8 += kThreads) m = fmaxf(m, amax8(load8(c8)));
            m = warp_max(m);
            __syncthreads();
            if (lane == 0) sred[16 + warp] = m;
            __syncthreads();
            float mx = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) mx = fmaxf(mx, sred[16 + w]);
            // S = 2^(e-126) > mx; X = x * 2^26 / S; results are scaled back by S / 2^26
            const uint32_t e = (__float_as_uint(mx) >> 23) & 0xFFu;
            const bool live = e >= 26u && e < 255u;
            const float inv = live ? __uint_as_float((279u - e) << 23) : 0.f;
            const float inv16 = inv * 0.0625f;
            if (tid == 0) sxscale[b] = live ? __uint_as_float((e - 25u) << 23) : 0.f;
            for (int base = 0; base < chunks; base += kThreads) {
                const int c8 = base + tid;
                float sum = 0.f;
                if (c8 < chunks) {
                    const uint4 v = load8(c8);
                    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
                    int de[4][4], dq[4][4];  // [pair][digit]: even / odd column of each pair
                    float fs[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __half22float2(u32_as_h2(u[j]));
                        fs[j] = f.x + f.y;
                        digits128(__float2int_rn(f.x * inv), de[j]);
                        digits128(__float2int_rn(f.y * inv16), dq[j]);
                    }
                    sum = (fs[0] + fs[1]) + (fs[2] + fs[3]);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        uint2 o;
                        o.x = pack4(de[0][k], de[1][k], de[2][k], de[3][k]);
                        o.y = pack4(dq[0][k], dq[1][k], dq[2][k], dq[3][k]);
                        *reinterpret_cast<uint2*>(xq + (size_t)(4 * b + 3 - k) * L.pitch_x + (size_t)c8 * 8) = o;
                    }
                }
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                if (c8 < chunks && (c8 & 7) == 0) sxsum[(c8 >> 3) * 2 + b] = sum;
            }
        }
        __syncthreads();
    }

    // ── consumer side ──
    // B operand: digit plane g (batch g / 4, digit 3 - g % 4), or zeros past the batch.
    const bool bvalid = g < kDigits * a.batch;
    const uint8_t* pb_base = bvalid ? xq + (size_t)g * L.pitch_x + t * 16 : smem + L.zero + t * 16;
    const int pb_stride = bvalid ? kGroup : 0;
    const float* pxs = sxsum + (t >> 1);  // this lane's columns belong to batch row t / 2
    const int w_off0 = g * 64 + (((t >> 1) ^ sw) * 16) + (t & 1) * 8;        // group 0 of the stage, row g
    const int w_off1 = g * 64 + (((2 + (t >> 1)) ^ sw) * 16) + (t & 1) * 8;  // group 1
    const int s_off = kSetW + g * 4;
    const int b_off = kSetW + kSetS + g * 4 + (t & 1) * 2;  // the bias product of group t & 1 is this lane's

    int c_tile = blockIdx.x, slot = 0;
    for (int ti = 0; ti < my_tiles; ++ti) {
        float acc[NW][2], bacc[NW][2];
#pragma unroll
        for (int s = 0; s < NW; ++s) acc[s][0] = acc[s][1] = bacc[s][0] = bacc[s][1] = 0.f;
        for (int j = 0; j < cnt; ++j) {
            cp_async_wait<DEPTH - 2>();  // this lane's copies of the stage have landed
            __syncwarp();                // ... every lane's have, and every lane is done with the previous stage
            fetch();                     // refill the buffer the previous stage used
            const uint8_t* st = ring + (size_t)slot * L.stage_bytes;
            slot = slot + 1 == DEPTH ? 0 : slot + 1;
            const int grp0 = (c_begin + j) * 2;
            const float xs = pxs[(grp0 + (t & 1)) * 2];
#pragma unroll
            for (int s = 0; s < NW; ++s) {
                const uint8_t* base = st + s * kSetBytes;
                bacc[s][0] = fmaf(__half2float(*reinterpret_cast<const __half*>(base + b_off)), xs, bacc[s][0]);
                bacc[s][1] = fmaf(__half2float(*reinterpret_cast<const __half*>(base + b_off + 32)), xs, bacc[s][1]);
            }
#pragma unroll
            for (int gg = 0; gg < 2; ++gg) {
                const uint4 xb = *reinterpret_cast<const uint4*>(pb_base + (grp0 + gg) * pb_stride);
#pragma unroll
                for (int s = 0; s < NW; ++s) {
                    const uint8_t* base = st + s * kSetBytes;
                    const uint2 wa = *reinterpret_cast<const uint2*>(base + (gg ? w_off1 : w_off0));
                    const uint2 wb = *reinterpret_cast<const uint2*>(base + (gg ? w_off1 : w_off0) + 8 * 64);
                    int c[4] = {(int)kMagic, (int)kMagic, (int)kMagic, (int)kMagic};
                    mma_u8s8(c, wa.x & 0x0F0F0F0Fu, wb.x & 0x0F0F0F0Fu, wa.x & 0xF0F0F0F0u, wb.x & 0xF0F0F0F0u, xb.x, xb.y);
                    mma_u8s8(c, wa.y & 0x0F0F0F0Fu, wb.y & 0x0F0F0F0Fu, wa.y & 0xF0F0F0F0u, wb.y & 0xF0F0F0F0u, xb.z, xb.w);
                    const float2 sa = __half22float2(u32_as_h2(*reinterpret_cast<const uint32_t*>(base + s_off)));
                    const float2 sb = __half22float2(u32_as_h2(*reinterpret_cast<const uint32_t*>(base + s_off + 32)));
                    // columns 2t, 2t+1 hold neighbouring digit planes: 128 * high + low
                    const float va = fmaf(__int_as_float(c[0]) - kMagicF, 128.f, __int_as_float(c[1]) - kMagicF);
                    const float vb = fmaf(__int_as_float(c[2]) - kMagicF, 128.f, __int_as_float(c[3]) - kMagicF);
                    acc[s][0] = fmaf(gg ? sa.y : sa.x, va, acc[s][0]);
                    acc[s][1] = fmaf(gg ? sb.y : sb.x, vb, acc[s][1]);
                }
            }
        }
        // ── tile done: lanes t = 0,1 (2,3) hold the upper and lower digit pairs of batch row 0 (1) ──
        const int buf = ti & 1;
        const float xscale = sxscale[t >> 1];
#pragma unroll
        for (int s = 0; s < NW; ++s)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float mine = acc[s][h], other = __shfl_xor_sync(0xffffffffu, mine, 1);
                const float tot = (t & 1) ? fmaf(other, 16384.f, mine) : fmaf(mine, 16384.f, other);
                const float bs = bacc[s][h] + __shfl_xor_sync(0xffffffffu, bacc[s][h], 1);
                if ((t & 1) == 0)
                    sred[((((buf * NW + s) * 2 + (t >> 1)) * kTileRows) + g + 8 * h) * kWarps + warp] = fmaf(tot, xscale, bs);
            }
        __syncthreads();
        if (warp == (ti & (kWarps - 1))) {
            // add the 16 K-partials in warp order, write out: lane -> (batch row, tile row)
            const int b = lane >> 4, r = lane & 15;
            float tot[NW];
#pragma unroll
            for (int s = 0; s < NW; ++s) {
                const float4* p = reinterpret_cast<const float4*>(sred + ((((buf * NW + s) * 2 + b) * kTileRows) + r) * kWarps);
                float v = 0.f;
#pragma unroll
                for (int q = 0; q < kWarps / 4; ++q) {
                    const float4 f = p[q];
                    v += f.x; v += f.y; v += f.z; v += f.w;
                }
                tot[s] = v;
            }
            int first = 0, rows = a.rows;
            __half* yout = a.y;
            if (NW == 1) {
                const int sg = seg_of(c_tile, first);
                rows = sg == 0 ? a.seg[0].rows : (sg == 1 ? a.seg[1].rows : a.seg[2].rows);
                yout = sg == 0 ? a.seg[0].y : (sg == 1 ? a.seg[1].y : a.seg[2].y);
            }
            const int row = (c_tile - first) * kTileRows + r;
            if (row < rows && b < a.batch) {
                const size_t o = (size_t)b * rows + row;
                const float v0 = tot[0];
                if (MODE == kAffinePlain) yout[o] = __float2half_rn(v0);
                else if (MODE == kAffineAdd) yout[o] = __hadd(__float2half_rn(v0), a.residual[o]);  // lut_matvec.metal:1802-1803
                else if (MODE == kAffineGateUp) a.y[o] = __float2half_rn(v0 / (1.0f + expf(-v0)) * tot[NW - 1]);  // :2228
                else { a.y[o] = __float2half_rn(v0); a.y2[o] = __float2half_rn(tot[NW - 1]); }
            }
        }
        c_tile += gridDim.x;
    }
    cp_async_wait<0>();
}

int env_int(const char* name, int dflt) {
    const char* e = getenv(name);
    return e ? atoi(e) : dflt;
}

template <int MODE, int DEPTH>
cudaError_t launch_imma_t(const Launch& l, AffineArgs a) {
    constexpr int NW = (MODE == kAffineGateUp || MODE == kAffineDual) ? 2 : 1;
    const ImmaLayout L = imma_layout(NW, DEPTH, a.cols, a.batch);
    a.dyn = dev_dyn(l);
    auto kern = affine_imma_kernel<MODE, DEPTH>;
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
    cfg.gridDim = dim3(tiles < sm ? tiles : sm, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = L.total;
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = l.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, a);
}

template <int MODE>
cudaError_t launch_imma_mode(const Launch& l, const AffineArgs& a, bool* handled) {
    constexpr int NW = (MODE == kAffineGateUp || MODE == kAffineDual) ? 2 : 1;
    static const int forced = env_int("SMELT_IMMA_DEPTH", 0);
    const int depth = forced ? forced : (NW == 2 ? 3 : 4);
    if (depth != 3 && depth != 4 && depth != 6) return cudaErrorInvalidValue;
    if (imma_layout(NW, depth, a.cols, a.batch).total > 226u * 1024u) return cudaSuccess;  // activations too large to stay resident
    *handled = true;
    if (depth == 3) return launch_imma_t<MODE, 3>(l, a);
    if (depth == 4) return launch_imma_t<MODE, 4>(l, a);
    return launch_imma_t<MODE, 6>(l, a);
}

}  // namespace

// Launches the integer-MMA kernel when the shape is eligible (group 64, batch <= 2, cols a
// multiple of 128, 16-byte aligned operands, every segment but the last a multiple of 16
// rows, digit planes small enough to stay resident); *handled tells the caller whether it did.
cudaError_t launch_affine_imma(const Launch& l, int mode, const AffineArgs& a, int group, bool* handled) {
    *handled = false;
    static const int disabled = env_int("SMELT_AFFINE_NO_IMMA", 0);
    if (disabled || group != kGroup || a.batch > 2 || a.cols % kChunkCols != 0) return cudaSuccess;
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
