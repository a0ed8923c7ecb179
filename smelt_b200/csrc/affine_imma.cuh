// Device side of the integer-MMA affine u4 matvec (see affine_imma.cu for the description).
#pragma once
#include "affine_matvec.h"

namespace smelt {
namespace imma {

constexpr int kGroup = 64;
constexpr int kTileRows = 16;
constexpr int kDigits = 4;
constexpr float kMagicF = 12582912.0f;                 // 1.5 * 2^23, bit pattern 0x4B400000

// Geometry of one variant: WARPS warps per CTA, GPS groups (of 64 columns) per ring stage.
template <int WARPS, int GPS>
struct Geo {
    static constexpr int kThreads = WARPS * 32;
    static constexpr int kStageCols = GPS * kGroup;
    static constexpr int kPitch = GPS * 32;                 // packed bytes per row per stage (64 or 128)
    static constexpr int kSetW = kTileRows * kPitch;
    static constexpr int kRowS = GPS * 2;                   // bytes of scales (or biases) per row per stage
    static constexpr int kSetS = kTileRows * kRowS;
    static constexpr int kSetBytes = kSetW + 2 * kSetS;     // [W | scales | biases]; a multiple of 128
};

struct ImmaLayout {
    uint32_t zero, xq, pitch_x, xsum, gscale, red, ring, stage_bytes, total;
};

__host__ __device__ inline ImmaLayout imma_layout(int nw, int depth, int warps, int set_bytes, int cols, int batch, int teams) {
    ImmaLayout L;
    L.stage_bytes = (uint32_t)nw * set_bytes;
    L.pitch_x = (uint32_t)cols + 64u;                  // one byte per column per plane; ≡ 64 (mod 128)
    uint32_t off = 0;
    L.zero = off; off += 64;
    L.xq = off; off += (uint32_t)(kDigits * batch) * L.pitch_x;
    L.xsum = off; off += (uint32_t)(cols / kGroup) * 2u * 4u;       // [group][batch slot 0/1]
    L.gscale = off; off += (uint32_t)(cols / kGroup) * 2u * 4u;     // [group][batch slot 0/1]: 2^-26 of the group's fixed-point unit
    L.red = off; off += (uint32_t)teams * 2u * (uint32_t)nw * 2u * kTileRows * 16u * 4u;  // [team][buffer][set][batch][row][warp slot, 16]
    off = (off + 127u) & ~127u;
    L.ring = off; off += (uint32_t)warps * depth * L.stage_bytes;
    L.total = off;
    return L;
}

// X (|X| < 2^27) as four base-128 digits packed one per byte, least significant first: the low
// three are the 7-bit fields of the two's-complement value (0..127), the top one is X >> 21
// (signed).  Every byte is a valid s8 and X = sum digit_k * 128^k.
__device__ __forceinline__ uint32_t digit_bytes(int X) {
    const uint32_t u = (uint32_t)X;
    return (u & 0x7Fu) | ((u << 1) & 0x7F00u) | ((u << 2) & 0x7F0000u) | ((uint32_t)(X >> 21) << 24);
}

// Four words of digit bytes (one value each) -> four words holding one digit of all four values.
__device__ __forceinline__ void transpose4x4(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t (&o)[4]) {
    const uint32_t ab_lo = __byte_perm(a, b, 0x5140), ab_hi = __byte_perm(a, b, 0x7362);  // (a0 b0 a1 b1), (a2 b2 a3 b3)
    const uint32_t cd_lo = __byte_perm(c, d, 0x5140), cd_hi = __byte_perm(c, d, 0x7362);
    o[0] = __byte_perm(ab_lo, cd_lo, 0x5410);  // a0 b0 c0 d0
    o[1] = __byte_perm(ab_lo, cd_lo, 0x7632);  // a1 b1 c1 d1
    o[2] = __byte_perm(ab_hi, cd_hi, 0x5410);
    o[3] = __byte_perm(ab_hi, cd_hi, 0x7632);
}

// TG tile groups per CTA: the CTA's warps form TG teams of WARPS / TG warps; each team walks its
// own tiles (splitting K among its warps) and only synchronises with itself.
// Sync is called once, by every thread of every CTA, between the first weight requests and the
// first read of the activations: the programmatic-dependent-launch wait of a stand-alone
// launch.
template <int MODE, int DEPTH, int WARPS, int GPS, int TG, class Sync>
__device__ __forceinline__ void affine_imma_body(const AffineArgs& a, uint8_t* smem, Sync sync) {
    using G = Geo<WARPS, GPS>;
    constexpr int NW = (MODE == kAffineGateUp || MODE == kAffineDual) ? 2 : 1;
    constexpr int kThreads = G::kThreads;
    constexpr int LPR = G::kPitch / 16;   // lanes that copy one row of a stage (4 or 8)
    constexpr int RPI = 32 / LPR;         // rows per copy instruction (8 or 4)
    constexpr int NI = kTileRows / RPI;   // copy instructions per set and stage (2 or 4)
    constexpr int WG = WARPS / TG;        // warps per team
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int team = warp / WG, wl = warp % WG;
    const ImmaLayout L = imma_layout(NW, DEPTH, WARPS, G::kSetBytes, a.cols, a.batch, TG);
    uint8_t* xq = smem + L.xq;
    float* sxsum = reinterpret_cast<float*>(smem + L.xsum);
    float* sgscale = reinterpret_cast<float*>(smem + L.gscale);
    float* sred0 = reinterpret_cast<float*>(smem + L.red);                      // staging scratch (whole CTA)
    float* sred = sred0 + (size_t)team * (2 * NW * 2 * kTileRows * 16);          // this team's K-partials
    uint8_t* ring = smem + L.ring + (size_t)warp * DEPTH * L.stage_bytes;

    const int tiles_total = a.ks;  // filled by the launcher
    const int nchunks = a.cols / G::kStageCols;
    const int cpw = (nchunks + WG - 1) / WG;  // stages per warp and tile: a contiguous K range
    const int c_begin = min(wl * cpw, nchunks);
    const int cnt = min(c_begin + cpw, nchunks) - c_begin;
    const int tile0 = (int)blockIdx.x * TG + team, tile_step = (int)gridDim.x * TG;
    const int my_tiles = tile0 < tiles_total ? (tiles_total - 1 - tile0) / tile_step + 1 : 0;
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
    const int fr = lane / LPR, fc = lane % LPR;
    const int fsw = GPS == 2 ? ((fr >> 1) & 1) << 1 : (fr & 3) << 1;  // 16-byte chunk swizzle of this lane's rows
    const uint32_t f_dst = fr * G::kPitch + ((fc ^ fsw) * 16);
    const uint32_t f_sdst = G::kSetW + (lane >> 4) * G::kSetS + (lane & 15) * G::kRowS;
    int f_tile = tile0, f_j = 0, f_n = 0, f_slot = 0;
    // per tile: the tensors and this lane's byte offsets into them (stage 0 of the warp's K range)
    const uint8_t* f_w[NW];
    const __half* f_sb[NW];
    uint32_t f_woff = 0, f_soff = 0, f_rows_ok = 0;  // bit h: copy row fr + RPI * h; bit 8: copy the scale piece
    auto fetch_tile = [&]() {
        int row0 = f_tile * kTileRows, rows = a.rows;
        if (NW == 1) {
            int first;
            const int sg = seg_of(f_tile, first);
            row0 = (f_tile - first) * kTileRows;
            rows = sg == 0 ? a.seg[0].rows : (sg == 1 ? a.seg[1].rows : a.seg[2].rows);
            f_w[0] = sg == 0 ? a.seg[0].w : (sg == 1 ? a.seg[1].w : a.seg[2].w);
            const __half* ss = sg == 0 ? a.seg[0].s : (sg == 1 ? a.seg[1].s : a.seg[2].s);
            const __half* bb = sg == 0 ? a.seg[0].b : (sg == 1 ? a.seg[1].b : a.seg[2].b);
            f_sb[0] = lane < 16 ? ss : bb;
        } else {
#pragma unroll
            for (int s = 0; s < NW; ++s) { f_w[s] = a.w[s]; f_sb[s] = lane < 16 ? a.s[s] : a.b[s]; }
        }
        f_woff = (uint32_t)(row0 + fr) * (uint32_t)(a.cols / 2) + (uint32_t)c_begin * G::kPitch + fc * 16;
        f_soff = ((uint32_t)(row0 + (lane & 15)) * (uint32_t)groups_total + (uint32_t)c_begin * GPS) * 2u;
        f_rows_ok = 0;
#pragma unroll
        for (int h = 0; h < NI; ++h) f_rows_ok |= (row0 + fr + RPI * h < rows ? 1u : 0u) << h;
        f_rows_ok |= (row0 + (lane & 15) < rows ? 1u : 0u) << 8;
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
                        cp_async16(dst + f_dst + h * RPI * G::kPitch, f_w[s] + woff + (uint32_t)(h * RPI) * (uint32_t)(a.cols / 2));
                if (f_rows_ok & 0x100u) {
                    const uint8_t* src = reinterpret_cast<const uint8_t*>(f_sb[s]) + soff;
                    if (GPS == 2) cp_async4(dst + f_sdst, src); else cp_async8(dst + f_sdst, src);
                }
            }
            ++f_n;
            f_slot = f_slot + 1 == DEPTH ? 0 : f_slot + 1;
            if (++f_j == cnt) {
                f_j = 0;
                f_tile += tile_step;
                if (f_n < total_stages) fetch_tile();
            }
        }
        cp_async_commit();  // always commit so that group counting stays uniform
    };
#pragma unroll
    for (int i = 0; i < DEPTH - 1; ++i) fetch();

    // The norm weights are weights too: requested before the wait, like the first stages.
    uint4 nwv[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    const bool nw_pre = a.norm_w && kThreads == 256 && a.cols / 8 <= 2 * 256;
    if (nw_pre) {
#pragma unroll
        for (int i = 0; i < 2; ++i)
            if (tid + 256 * i < a.cols / 8) nwv[i] = *reinterpret_cast<const uint4*>(a.norm_w + (tid + 256 * i) * 8);
    }

    sync();
    if (dyn_skip(a.dyn)) {
        cp_async_wait<0>();  // copies in flight must land before the CTA's shared memory retires
        return;
    }

    // ── activations: digit planes, per-group scales and per-group sums, once per CTA ──
    // Each group of 64 activations gets its own fixed-point scale: S = the power of two above the
    // group's largest |x|, X = x * 2^26 / S (odd columns X / 16), so no pass over the whole row
    // and no CTA-wide reduction comes before the digits.  A thread keeps its 16-byte chunks
    // (tid, tid + threads, ...) in registers from the one global read to the end.
    {
        constexpr int XC = 6;  // chunks a thread caches: rows of up to 6 * 8 * threads activations
        const int chunks = a.cols / 8;
        if (tid < 4) reinterpret_cast<uint4*>(smem + L.zero)[tid] = make_uint4(0, 0, 0, 0);
        if (a.batch == 1)
            for (int i = tid; i < groups_total; i += kThreads) sxsum[i * 2 + 1] = sgscale[i * 2 + 1] = 0.f;
        const bool cached = chunks <= XC * kThreads;
        for (int b = 0; b < a.batch; ++b) {
            const __half* xr = a.x + (size_t)b * a.cols;
            uint4 xc[XC];
            if (cached) {
#pragma unroll
                for (int i = 0; i < XC; ++i)
                    xc[i] = tid + kThreads * i < chunks ? *reinterpret_cast<const uint4*>(xr + (size_t)(tid + kThreads * i) * 8) : make_uint4(0, 0, 0, 0);
            }
            float rs = 0.f;
            if (a.norm_w) {
                // rms_norm_1pw (Resources/Shaders/norms.metal:9-67) folded into the staging pass, with
                // the summation order of cta256_sumsq_f16: thread t folds chunks t, t + 256, ... in one chain
                float tot;
                if (cached && kThreads == 256) {
                    float ss = 0.f;
#pragma unroll
                    for (int i = 0; i < XC; ++i)
                        if (tid + kThreads * i < chunks) ss = sumsq8(ss, xc[i]);
                    tot = cta256_sum_finish(ss, sred0);
                } else {
                    tot = cta256_sumsq_f16(xr, a.cols, sred0);
                }
                rs = __frcp_rn(__fsqrt_rn(tot / (float)a.cols + a.norm_eps));
            }
            auto normed = [&](uint4 v, const uint4& wv) {
                v.x = rms_norm_1pw_pair(v.x, wv.x, rs); v.y = rms_norm_1pw_pair(v.y, wv.y, rs);
                v.z = rms_norm_1pw_pair(v.z, wv.z, rs); v.w = rms_norm_1pw_pair(v.w, wv.w, rs);
                return v;
            };
            auto stage_chunk = [&](int c8, uint4 v) {  // called by all 32 lanes together; c8 >= chunks: lane idles
                const bool on = c8 < chunks;
                float m = on ? amax8(v) : 0.f;
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));  // the group's eight chunks sit in eight neighbouring lanes
                // S = 2^(e-126) > m; X = x * 2^26 / S; results are scaled back by S / 2^26
                const uint32_t e = (__float_as_uint(m) >> 23) & 0xFFu;
                const bool live = e >= 26u && e < 255u;
                const float inv = live ? __uint_as_float((279u - e) << 23) : 0.f;
                const float inv16 = inv * 0.0625f;
                float sum = 0.f;
                if (on) {
                    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
                    uint32_t de[4], dq[4];  // digit bytes of the even / odd column of each pair
                    float fs[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __half22float2(u32_as_h2(u[j]));
                        fs[j] = f.x + f.y;
                        de[j] = digit_bytes(__float2int_rn(f.x * inv));
                        dq[j] = digit_bytes(__float2int_rn(f.y * inv16));
                    }
                    sum = (fs[0] + fs[1]) + (fs[2] + fs[3]);
                    uint32_t pe[4], pq[4];
                    transpose4x4(de[0], de[1], de[2], de[3], pe);
                    transpose4x4(dq[0], dq[1], dq[2], dq[3], pq);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        *reinterpret_cast<uint2*>(xq + (size_t)(4 * b + 3 - k) * L.pitch_x + (size_t)c8 * 8) = make_uint2(pe[k], pq[k]);
                }
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                if (on && (c8 & 7) == 0) {
                    sxsum[(c8 >> 3) * 2 + b] = sum;
                    sgscale[(c8 >> 3) * 2 + b] = live ? __uint_as_float((e - 25u) << 23) : 0.f;
                }
            };
            if (cached) {
#pragma unroll
                for (int i = 0; i < XC; ++i) {
                    if (kThreads * i >= chunks) break;  // uniform: the whole CTA is past the row
                    const int c8 = tid + kThreads * i;
                    uint4 v = xc[i];
                    if (a.norm_w && c8 < chunks) v = normed(v, (nw_pre && i < 2) ? nwv[i] : *reinterpret_cast<const uint4*>(a.norm_w + (size_t)c8 * 8));
                    stage_chunk(c8, v);
                }
            } else {
                for (int base = 0; base < chunks; base += kThreads) {
                    const int c8 = base + tid;
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (c8 < chunks) {
                        v = *reinterpret_cast<const uint4*>(xr + (size_t)c8 * 8);
                        if (a.norm_w) v = normed(v, *reinterpret_cast<const uint4*>(a.norm_w + (size_t)c8 * 8));
                    }
                    stage_chunk(c8, v);
                }
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
    const float* pgs = sgscale + (t >> 1);
    const int csw = GPS == 2 ? ((g >> 1) & 1) << 1 : (g & 3) << 1;
    int w_off[GPS];
#pragma unroll
    for (int gg = 0; gg < GPS; ++gg) w_off[gg] = g * G::kPitch + (((2 * gg + (t >> 1)) ^ csw) * 16) + (t & 1) * 8;
    const int s_off = G::kSetW + g * G::kRowS;
    // the bias products of groups (t & 1) * GPS / 2 ... of a stage are this lane's
    const int bias_g0 = (t & 1) * (GPS / 2);
    const int b_off = G::kSetW + G::kSetS + g * G::kRowS + bias_g0 * 2;
    const int magic = 0x4B400000;

    int c_tile = tile0, slot = 0;
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
            const int grp0 = (c_begin + j) * GPS;
#pragma unroll
            for (int q = 0; q < GPS / 2; ++q) {
                const float xs = pxs[(grp0 + bias_g0 + q) * 2];
#pragma unroll
                for (int s = 0; s < NW; ++s) {
                    const uint8_t* base = st + s * G::kSetBytes + b_off + q * 2;
                    bacc[s][0] = fmaf(__half2float(*reinterpret_cast<const __half*>(base)), xs, bacc[s][0]);
                    bacc[s][1] = fmaf(__half2float(*reinterpret_cast<const __half*>(base + 8 * G::kRowS)), xs, bacc[s][1]);
                }
            }
#pragma unroll
            for (int gg = 0; gg < GPS; ++gg) {
                const uint4 xb = *reinterpret_cast<const uint4*>(pb_base + (grp0 + gg) * pb_stride);
                const float gsv = pgs[(grp0 + gg) * 2];  // the group's fixed-point unit
#pragma unroll
                for (int s = 0; s < NW; ++s) {
                    const uint8_t* base = st + s * G::kSetBytes;
                    const uint2 wa = *reinterpret_cast<const uint2*>(base + w_off[gg]);
                    const uint2 wb = *reinterpret_cast<const uint2*>(base + w_off[gg] + 8 * G::kPitch);
                    int c[4];
                    mma_u8s8(c, wa.x & 0x0F0F0F0Fu, wb.x & 0x0F0F0F0Fu, wa.x & 0xF0F0F0F0u, wb.x & 0xF0F0F0F0u, xb.x, xb.y,
                             magic, magic, magic, magic);
                    mma_u8s8(c, wa.y & 0x0F0F0F0Fu, wb.y & 0x0F0F0F0Fu, wa.y & 0xF0F0F0F0u, wb.y & 0xF0F0F0F0u, xb.z, xb.w,
                             c[0], c[1], c[2], c[3]);
                    const float sa = __half2float(*reinterpret_cast<const __half*>(base + s_off + gg * 2));
                    const float sb = __half2float(*reinterpret_cast<const __half*>(base + s_off + 8 * G::kRowS + gg * 2));
                    // columns 2t, 2t+1 hold neighbouring digit planes: 128 * high + low
                    const float va = fmaf(__int_as_float(c[0]) - kMagicF, 128.f, __int_as_float(c[1]) - kMagicF);
                    const float vb = fmaf(__int_as_float(c[2]) - kMagicF, 128.f, __int_as_float(c[3]) - kMagicF);
                    acc[s][0] = fmaf(sa * gsv, va, acc[s][0]);
                    acc[s][1] = fmaf(sb * gsv, vb, acc[s][1]);
                }
            }
        }
        // ── tile done: lanes t = 0,1 (2,3) hold the upper and lower digit pairs of batch row 0 (1) ──
        const int buf = ti & 1;
#pragma unroll
        for (int s = 0; s < NW; ++s)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float mine = acc[s][h], other = __shfl_xor_sync(0xffffffffu, mine, 1);
                const float tot = (t & 1) ? fmaf(other, 16384.f, mine) : fmaf(mine, 16384.f, other);
                const float bs = bacc[s][h] + __shfl_xor_sync(0xffffffffu, bacc[s][h], 1);
                if ((t & 1) == 0)
                    sred[((((buf * NW + s) * 2 + (t >> 1)) * kTileRows) + g + 8 * h) * 16 + wl] = tot + bs;
            }
        if (TG == 1) __syncthreads();
        else asm volatile("bar.sync %0, %1;" ::"r"(1 + team), "r"(WG * 32) : "memory");
        if (wl == (ti % WG)) {
            // add the K-partials in warp order, write out: lane -> (batch row, tile row)
            const int b = lane >> 4, r = lane & 15;
            float tot[NW];
#pragma unroll
            for (int s = 0; s < NW; ++s) {
                const float4* p = reinterpret_cast<const float4*>(sred + ((((buf * NW + s) * 2 + b) * kTileRows) + r) * 16);
                float v = 0.f;
#pragma unroll
                for (int q = 0; q < WG / 4; ++q) {
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
        c_tile += tile_step;
    }
    cp_async_wait<0>();
}

struct PdlSync {
    __device__ __forceinline__ void operator()() const {
        pdl_trigger();
        pdl_wait();
    }
};

}  // namespace imma
}  // namespace smelt
