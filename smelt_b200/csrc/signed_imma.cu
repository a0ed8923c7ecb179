// Integer-tensor-core form of the binary1 / ternary2 (group 128) matvec for batch 1 and 2.
//
// Same reference kernels and semantics as signed_matvec.cu (Resources/Shaders/signed_quant.metal
// :81-138, :223-286, :140-221, :288-332; oracle Tests/SmeltCompilerTests/SignedQuantKernelTests.swift
// :1030-1045):  y[r] = sum_g scale[r,g] * sum_{c in g} sem(code[r,c]) * x[c].
//
// The codes are never unpacked with shifts.  A 32-bit word of codes ANDed with the byte mask
// 0x01010101 << p (binary, p = 0..7) or 0x03030303 << 2p (ternary, p = 0..3) is already four
// u8 values 2^p * bit or 4^p * code, one per byte, and goes straight into
// mma.sync.m16n8k32.u8.s8 as the A operand.  The power of two is undone on the other side:
// the activations become, once per CTA, signed base-128 digit planes of the fixed-point value
// X * 2^(7-p) (binary) or X * 4^(3-p) (ternary), X = x * 2^19 / S or x * 2^20 / S with S a
// power of two above the row's largest |x|, laid out in the k order the masks produce.  Every
// product is then 128 * bit * X (64 * code * X): exact integers, recombined in fp32 from the four
// planes.  With bit = (sem + 1) / 2 and code = sem + 1 the result is
// sum sem * x = scale_back * C - sum x, and the second term uses the per-group sums of x.
//
// Structure (persistent CTA, per-warp cp.async rings over a contiguous K range, teams of
// warps that each walk their own 16-row tiles, K-partials added in warp order) is that of
// affine_imma.cu.
#include <cstdlib>

#include "glue.h"

namespace smelt {

namespace {

constexpr int kGroup = 128;
constexpr int kTileRows = 16;
constexpr int kDigits = 4;
constexpr int kWarps = 8;
constexpr int kTeams = 2;
constexpr int kWG = kWarps / kTeams;                  // warps per team
constexpr int kThreads = kWarps * 32;
constexpr int kGPS = 4;                               // groups per ring stage (512 columns)
constexpr int kDepth = 4;
constexpr float kMagicF = 12582912.0f;                // 1.5 * 2^23, bit pattern 0x4B400000

template <int BITS>
struct Geo {
    static constexpr int kPitch = kGPS * kGroup * BITS / 8;  // code bytes per row per stage: 64 or 128
    static constexpr int kSetW = kTileRows * kPitch;
    static constexpr int kRowS = kGPS * 2;                   // bytes of scales per row per stage
    static constexpr int kSetS = kTileRows * kRowS;          // 128
    static constexpr int kSetBytes = kSetW + kSetS;          // a multiple of 128
};

struct SignedLayout {
    uint32_t zero, xq, pitch_x, xsum, xscale, red, ring, stage_bytes, total;
};

__host__ __device__ inline SignedLayout signed_layout(int nw, int set_bytes, int cols, int batch) {
    SignedLayout L;
    L.stage_bytes = (uint32_t)nw * set_bytes;
    L.pitch_x = (uint32_t)cols + 16u;                 // one byte per column per plane; ≡ 16 (mod 128)
    uint32_t off = 0;
    L.zero = off; off += 128;
    L.xq = off; off += (uint32_t)(kDigits * batch) * L.pitch_x;
    off = (off + 15u) & ~15u;
    L.xsum = off; off += (uint32_t)(cols / kGroup) * 2u * 4u;   // [group][batch slot 0/1]
    L.xscale = off; off += 16;
    L.red = off; off += (uint32_t)kTeams * 2u * (uint32_t)nw * 2u * kTileRows * 4u * 4u;  // [team][buffer][set][batch][row][warp slot, 4]
    off = (off + 127u) & ~127u;
    L.ring = off; off += (uint32_t)kWarps * kDepth * L.stage_bytes;
    L.total = off;
    return L;
}

// Four signed base-128 digits of X (|X| < 2^27), least significant first.
__device__ __forceinline__ void digits128(int X, int (&d)[4]) {
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        d[k] = ((X + 64) & 127) - 64;
        X = (X - d[k]) >> 7;
    }
    d[3] = X;
}


template <int BITS, int MODE>
__global__ void __launch_bounds__(kThreads, 1) signed_imma_kernel(const SignedArgs a, int tiles_total, DevDyn dyn) {
    using G = Geo<BITS>;
    constexpr int NW = MODE == kSignedGateUp ? 2 : 1;
    constexpr int LPR = G::kPitch / 16;   // lanes that copy one row of a stage (4 or 8)
    constexpr int RPI = 32 / LPR;         // rows per copy instruction (8 or 4)
    constexpr int NI = kTileRows / RPI;   // copy instructions per set and stage (2 or 4)
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int team = warp / kWG, wl = warp % kWG;
    const SignedLayout L = signed_layout(NW, G::kSetBytes, a.cols, a.batch);
    uint8_t* xq = smem + L.xq;
    float* sxsum = reinterpret_cast<float*>(smem + L.xsum);
    float* sxscale = reinterpret_cast<float*>(smem + L.xscale);
    float* sred0 = reinterpret_cast<float*>(smem + L.red);
    float* sred = sred0 + (size_t)team * (2 * NW * 2 * kTileRows * 4);
    uint8_t* ring = smem + L.ring + (size_t)warp * kDepth * L.stage_bytes;

    // K split over the team's warps: contiguous ranges of stages, sizes differing by at most one
    const int nst = a.cols / (kGPS * kGroup);
    const int base_cnt = nst / kWG, extra = nst % kWG;
    const int c_begin = wl * base_cnt + min(wl, extra);
    const int cnt = base_cnt + (wl < extra ? 1 : 0);
    const int tile0 = (int)blockIdx.x * kTeams + team, tile_step = (int)gridDim.x * kTeams;
    const int my_tiles = tile0 < tiles_total ? (tiles_total - 1 - tile0) / tile_step + 1 : 0;
    const int total_stages = my_tiles * cnt;
    const int groups_total = a.cols / kGroup;
    const uint32_t row_bytes = (uint32_t)a.cols * BITS / 8;

    // ── producer side: each warp copies the stages it will consume ──
    const int fr = lane / LPR, fc = lane % LPR;
    const int fsw = BITS == 1 ? (fr >> 1) & 3 : (fr & 3) << 1;  // 16-byte chunk swizzle of this lane's rows
    const uint32_t f_dst = fr * G::kPitch + ((fc ^ fsw) * 16);
    const uint32_t f_sdst = G::kSetW + (lane & 15) * G::kRowS;
    int f_tile = tile0, f_j = 0, f_n = 0, f_slot = 0;
    uint32_t f_woff = 0, f_soff = 0, f_rows_ok = 0;
    auto fetch_tile = [&]() {
        const int row0 = f_tile * kTileRows;
        f_woff = (uint32_t)(row0 + fr) * row_bytes + (uint32_t)c_begin * G::kPitch + fc * 16;
        f_soff = ((uint32_t)(row0 + (lane & 15)) * (uint32_t)groups_total + (uint32_t)c_begin * kGPS) * 2u;
        f_rows_ok = 0;
#pragma unroll
        for (int h = 0; h < NI; ++h) f_rows_ok |= (row0 + fr + RPI * h < a.rows ? 1u : 0u) << h;
        f_rows_ok |= (lane < 16 && row0 + lane < a.rows ? 1u : 0u) << 8;
    };
    if (total_stages > 0) fetch_tile();
    auto fetch = [&]() {
        if (f_n < total_stages) {
            uint8_t* st = ring + (size_t)f_slot * L.stage_bytes;
            const uint32_t woff = f_woff + (uint32_t)f_j * G::kPitch;
            const uint32_t soff = f_soff + (uint32_t)f_j * G::kRowS;
#pragma unroll
            for (int s = 0; s < NW; ++s) {
                uint8_t* dst = st + s * G::kSetBytes;
#pragma unroll
                for (int h = 0; h < NI; ++h)
                    if (f_rows_ok & (1u << h))
                        cp_async16(dst + f_dst + h * RPI * G::kPitch, a.codes[s] + woff + (uint32_t)(h * RPI) * row_bytes);
                if (f_rows_ok & 0x100u) cp_async8(dst + f_sdst, reinterpret_cast<const uint8_t*>(a.scales[s]) + soff);
            }
            ++f_n;
            f_slot = f_slot + 1 == kDepth ? 0 : f_slot + 1;
            if (++f_j == cnt) {
                f_j = 0;
                f_tile += tile_step;
                if (f_n < total_stages) fetch_tile();
            }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int i = 0; i < kDepth - 1; ++i) fetch();

    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) {
        cp_async_wait<0>();
        return;
    }

    // ── activations: scaled digit planes in the k order of the masks + per-group sums, once per CTA ──
    {
        const int chunks = a.cols / 8;
        if (tid < 8) reinterpret_cast<uint4*>(smem + L.zero)[tid] = make_uint4(0, 0, 0, 0);
        if (a.batch == 1)
            for (int i = tid; i < groups_total; i += kThreads) sxsum[i * 2 + 1] = 0.f;
        for (int b = 0; b < a.batch; ++b) {
            const __half* xr = a.x + (size_t)b * a.cols;
            float m = 0.f;
            for (int c8 = tid; c8 < chunks; c8 += kThreads) m = fmaxf(m, amax8(*reinterpret_cast<const uint4*>(xr + c8 * 8)));
            m = warp_max(m);
            __syncthreads();
            if (lane == 0) sred0[warp] = m;
            __syncthreads();
            float mx = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) mx = fmaxf(mx, sred0[w]);
            // S = 2^(e-126) > mx.  binary: X = x 2^19 / S, sum sem x = C S 2^-25 - sum x;
            // ternary: X = x 2^20 / S, sum sem x = C S 2^-26 - sum x.
            const uint32_t e = (__float_as_uint(mx) >> 23) & 0xFFu;
            const bool live = e >= 26u && e < 255u;
            const float inv = live ? __uint_as_float(((BITS == 1 ? 272u : 273u) - e) << 23) : 0.f;
            if (tid == 0) sxscale[b] = live ? __uint_as_float((e - (BITS == 1 ? 24u : 25u)) << 23) : 0.f;
            for (int base = 0; base < chunks; base += kThreads) {
                const int c8 = base + tid;
                float sum = 0.f;
                if (c8 < chunks) {
                    const uint4 v = *reinterpret_cast<const uint4*>(xr + c8 * 8);
                    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
                    float f[8];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 p = __half22float2(u32_as_h2(u[j]));
                        f[2 * j] = p.x; f[2 * j + 1] = p.y;
                    }
                    sum = ((f[0] + f[1]) + (f[2] + f[3])) + ((f[4] + f[5]) + (f[6] + f[7]));
                    const int m4 = c8 & 3;  // which 8 columns of the lane's 32-column slice
                    uint8_t* dst = xq + (size_t)(4 * b) * L.pitch_x + (size_t)(c8 >> 2) * 32;
#pragma unroll
                    for (int el = 0; el < 8; ++el) {
                        int shift, bi;
                        if (BITS == 1) {
                            shift = 7 - el;
                            bi = (el >> 1) * 8 + (el & 1) * 4 + m4;
                        } else {
                            const int p = el & 3;
                            shift = 2 * (3 - p);
                            bi = ((m4 >> 1) * 2 + (p >> 1)) * 8 + (p & 1) * 4 + 2 * (m4 & 1) + (el >> 2);
                        }
                        int d[4];
                        digits128(__float2int_rn(f[el] * inv) * (1 << shift), d);
#pragma unroll
                        for (int k = 0; k < 4; ++k) dst[(size_t)(3 - k) * L.pitch_x + bi] = (uint8_t)d[k];
                    }
                }
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                sum += __shfl_xor_sync(0xffffffffu, sum, 8);
                if (c8 < chunks && (c8 & 15) == 0) sxsum[(c8 >> 4) * 2 + b] = sum;
            }
        }
        __syncthreads();
    }

    // ── consumer side ──
    // B operand: digit plane g (batch g / 4, digit 3 - g % 4), or zeros past the batch.
    const bool bvalid = g < kDigits * a.batch;
    const uint8_t* pb_base = bvalid ? xq + (size_t)g * L.pitch_x + t * 32 : smem + L.zero + t * 32;
    const int pb_stride = bvalid ? kGroup : 0;
    const float* pxs = sxsum + (t >> 1);  // this lane's columns belong to batch row t / 2
    const int csw = BITS == 1 ? (g >> 1) & 3 : (g & 3) << 1;
    int w_off[kGPS];
#pragma unroll
    for (int gg = 0; gg < kGPS; ++gg)
        w_off[gg] = BITS == 1 ? g * G::kPitch + ((gg ^ csw) * 16) + t * 4
                              : g * G::kPitch + (((2 * gg + (t >> 1)) ^ csw) * 16) + (t & 1) * 8;
    const int s_off = G::kSetW + g * G::kRowS;
    const int bias_g0 = (t & 1) * (kGPS / 2);  // the sum-of-x terms of these two groups of a stage are this lane's
    const int magic = 0x4B400000;

    int c_tile = tile0, slot = 0;
    for (int ti = 0; ti < my_tiles; ++ti) {
        float acc[NW][2], bacc[NW][2];
#pragma unroll
        for (int s = 0; s < NW; ++s) acc[s][0] = acc[s][1] = bacc[s][0] = bacc[s][1] = 0.f;
        for (int j = 0; j < cnt; ++j) {
            cp_async_wait<kDepth - 2>();
            __syncwarp();
            fetch();
            const uint8_t* st = ring + (size_t)slot * L.stage_bytes;
            slot = slot + 1 == kDepth ? 0 : slot + 1;
            const int grp0 = (c_begin + j) * kGPS;
            float sc[NW][2][kGPS];  // [set][row g / g + 8][group of the stage]
#pragma unroll
            for (int s = 0; s < NW; ++s)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(st + s * G::kSetBytes + s_off + h * 8 * G::kRowS);
                    const float2 lo = __half22float2(u32_as_h2(raw.x)), hi = __half22float2(u32_as_h2(raw.y));
                    sc[s][h][0] = lo.x; sc[s][h][1] = lo.y; sc[s][h][2] = hi.x; sc[s][h][3] = hi.y;
                }
#pragma unroll
            for (int q = 0; q < kGPS / 2; ++q) {
                const float xs = pxs[(grp0 + bias_g0 + q) * 2];
#pragma unroll
                for (int s = 0; s < NW; ++s) {
                    bacc[s][0] = fmaf((t & 1) ? sc[s][0][2 + q] : sc[s][0][q], xs, bacc[s][0]);
                    bacc[s][1] = fmaf((t & 1) ? sc[s][1][2 + q] : sc[s][1][q], xs, bacc[s][1]);
                }
            }
#pragma unroll
            for (int gg = 0; gg < kGPS; ++gg) {
                const uint4 x0 = *reinterpret_cast<const uint4*>(pb_base + (grp0 + gg) * pb_stride);
                const uint4 x1 = *reinterpret_cast<const uint4*>(pb_base + (grp0 + gg) * pb_stride + 16);
#pragma unroll
                for (int s = 0; s < NW; ++s) {
                    const uint8_t* base = st + s * G::kSetBytes;
                    int c[4];
                    if (BITS == 1) {
                        const uint32_t wa = *reinterpret_cast<const uint32_t*>(base + w_off[gg]);
                        const uint32_t wb = *reinterpret_cast<const uint32_t*>(base + w_off[gg] + 8 * G::kPitch);
                        mma_u8s8(c, wa & 0x01010101u, wb & 0x01010101u, wa & 0x02020202u, wb & 0x02020202u, x0.x, x0.y, magic, magic, magic, magic);
                        mma_u8s8(c, wa & 0x04040404u, wb & 0x04040404u, wa & 0x08080808u, wb & 0x08080808u, x0.z, x0.w, c[0], c[1], c[2], c[3]);
                        mma_u8s8(c, wa & 0x10101010u, wb & 0x10101010u, wa & 0x20202020u, wb & 0x20202020u, x1.x, x1.y, c[0], c[1], c[2], c[3]);
                        mma_u8s8(c, wa & 0x40404040u, wb & 0x40404040u, wa & 0x80808080u, wb & 0x80808080u, x1.z, x1.w, c[0], c[1], c[2], c[3]);
                    } else {
                        const uint2 wa = *reinterpret_cast<const uint2*>(base + w_off[gg]);
                        const uint2 wb = *reinterpret_cast<const uint2*>(base + w_off[gg] + 8 * G::kPitch);
                        mma_u8s8(c, wa.x & 0x03030303u, wb.x & 0x03030303u, wa.x & 0x0C0C0C0Cu, wb.x & 0x0C0C0C0Cu, x0.x, x0.y, magic, magic, magic, magic);
                        mma_u8s8(c, wa.x & 0x30303030u, wb.x & 0x30303030u, wa.x & 0xC0C0C0C0u, wb.x & 0xC0C0C0C0u, x0.z, x0.w, c[0], c[1], c[2], c[3]);
                        mma_u8s8(c, wa.y & 0x03030303u, wb.y & 0x03030303u, wa.y & 0x0C0C0C0Cu, wb.y & 0x0C0C0C0Cu, x1.x, x1.y, c[0], c[1], c[2], c[3]);
                        mma_u8s8(c, wa.y & 0x30303030u, wb.y & 0x30303030u, wa.y & 0xC0C0C0C0u, wb.y & 0xC0C0C0C0u, x1.z, x1.w, c[0], c[1], c[2], c[3]);
                    }
                    // columns 2t, 2t+1 hold neighbouring digit planes: 128 * high + low
                    const float va = fmaf(__int_as_float(c[0]) - kMagicF, 128.f, __int_as_float(c[1]) - kMagicF);
                    const float vb = fmaf(__int_as_float(c[2]) - kMagicF, 128.f, __int_as_float(c[3]) - kMagicF);
                    acc[s][0] = fmaf(sc[s][0][gg], va, acc[s][0]);
                    acc[s][1] = fmaf(sc[s][1][gg], vb, acc[s][1]);
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
                    sred[((((buf * NW + s) * 2 + (t >> 1)) * kTileRows) + g + 8 * h) * 4 + wl] = fmaf(tot, xscale, -bs);
            }
        asm volatile("bar.sync %0, %1;" ::"r"(1 + team), "r"(kWG * 32) : "memory");
        if (wl == (ti % kWG)) {
            const int b = lane >> 4, r = lane & 15;
            float tot[NW];
#pragma unroll
            for (int s = 0; s < NW; ++s) {
                const float4 f = *reinterpret_cast<const float4*>(sred + ((((buf * NW + s) * 2 + b) * kTileRows) + r) * 4);
                tot[s] = ((f.x + f.y) + f.z) + f.w;
            }
            const int row = c_tile * kTileRows + r;
            if (row < a.rows && b < a.batch) {
                const size_t o = (size_t)b * a.rows + row;
                const float v0 = tot[0];
                if (MODE == kSignedPlain) a.y[o] = __float2half_rn(v0);
                else if (MODE == kSignedAdd)  // signed_quant.metal:271-278: half(float(half(acc)) + float(residual))
                    a.y[o] = __float2half_rn(__half2float(__float2half_rn(v0)) + __half2float(a.residual[o]));
                else a.y[o] = swiglu_staged(__float2half_rn(v0), __float2half_rn(tot[NW - 1]));
            }
        }
        c_tile += tile_step;
    }
    cp_async_wait<0>();
}

template <int BITS, int MODE>
cudaError_t launch_signed_imma_t(const Launch& l, const SignedArgs& a, int sm_count, bool* handled) {
    using G = Geo<BITS>;
    constexpr int NW = MODE == kSignedGateUp ? 2 : 1;
    const SignedLayout L = signed_layout(NW, G::kSetBytes, a.cols, a.batch);
    if (L.total > 226u * 1024u) return cudaSuccess;  // digit planes too large to stay resident: not handled
    *handled = true;
    auto kern = signed_imma_kernel<BITS, MODE>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L.total);
    if (e != cudaSuccess) return e;
    const int tiles = (a.rows + kTileRows - 1) / kTileRows;
    const int sm = sm_count > 0 ? sm_count : 148;
    const int want = (tiles + kTeams - 1) / kTeams;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(want < sm ? want : sm, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = L.total;
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = l.pdl ? 1 : 0;
    prefer_max_shared(kern);
    return cudaLaunchKernelEx(&cfg, kern, a, tiles, dev_dyn(l));
}

template <int BITS>
cudaError_t launch_signed_imma_bits(const Launch& l, int mode, const SignedArgs& a, int sm_count, bool* handled) {
    switch (mode) {
        case kSignedPlain: return launch_signed_imma_t<BITS, kSignedPlain>(l, a, sm_count, handled);
        case kSignedAdd: return launch_signed_imma_t<BITS, kSignedAdd>(l, a, sm_count, handled);
        case kSignedGateUp: return launch_signed_imma_t<BITS, kSignedGateUp>(l, a, sm_count, handled);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

// Launches the integer-MMA kernel when the shape is eligible (batch <= 2, cols a multiple of
// 512, 16-byte aligned operands, digit planes small enough to stay resident); *handled tells
// the caller whether it did.
cudaError_t launch_signed_imma(const Launch& l, int mode, const SignedArgs& a, int sm_count, bool* handled) {
    *handled = false;
    if (a.batch > 2 || a.cols % (kGPS * kGroup) != 0 || (a.bits != 1 && a.bits != 2)) return cudaSuccess;
    const int nw = mode == kSignedGateUp ? 2 : 1;
    for (int s = 0; s < nw; ++s)
        if ((reinterpret_cast<uintptr_t>(a.codes[s]) | reinterpret_cast<uintptr_t>(a.scales[s])) & 15u) return cudaSuccess;
    if (reinterpret_cast<uintptr_t>(a.x) & 15u) return cudaSuccess;
    return a.bits == 1 ? launch_signed_imma_bits<1>(l, mode, a, sm_count, handled) : launch_signed_imma_bits<2>(l, mode, a, sm_count, handled);
}

}  // namespace smelt
