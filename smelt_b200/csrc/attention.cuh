// Device side of the flash-decode attention kernel (see attention.cu for the description).
#pragma once
#include <cooperative_groups.h>

#include "glue.h"
#include "rope.cuh"

namespace smelt {
namespace attn {

namespace cg = cooperative_groups;


constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = 8;
constexpr int kMaxSplits = 64;
constexpr int kMlxBlocks = 128;  // key blocks of the reference's two-pass pair (attention_decode_mlx_vector_2pass_*_d256_b128)
constexpr float kNegBig = -1.0e30f;

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// out = sum_s exp2(m_s - M) O_s / sum_s exp2(m_s - M) l_s over the splits of `heads` consecutive
// query heads starting at qh0, splits in index order.  The (max, sum) pairs are staged in shared
// memory first (smem: 2 * heads * nsplits floats), so the loop over the splits carries no load
// that depends on another: sixteen partial rows are in flight per thread.
template <int D>
__device__ __forceinline__ void merge_partials(const AttnDev& p, float* smem, size_t qh0, int heads, int tid, int nthreads) {
    const int ns = p.nsplits;
    float* s_m = smem;
    float* s_l = smem + heads * ns;
    for (int i = tid; i < heads * ns; i += nthreads) {
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml) + qh0 * ns + i);
        s_m[i] = ml.x; s_l[i] = ml.y;
    }
    __syncthreads();
    for (int idx = tid; idx < heads * D; idx += nthreads) {
        const int h = idx / D, d = idx % D;
        const float* hm = s_m + h * ns;
        const float* hl = s_l + h * ns;
        float mstar = kNegBig;
        for (int s2 = 0; s2 < ns; ++s2) mstar = fmaxf(mstar, hm[s2]);
        const float* po = p.part_o + (qh0 + h) * ns * D + d;
        float acc = 0.f, lsum = 0.f;
        int s2 = 0;
        for (; s2 + 16 <= ns; s2 += 16) {
            float v[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) v[u] = __ldcg(po + (size_t)(s2 + u) * D);
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const float f = exp2f(hm[s2 + u] - mstar);
                acc += v[u] * f;
                lsum += hl[s2 + u] * f;
            }
        }
        for (; s2 < ns; ++s2) {
            const float f = exp2f(hm[s2] - mstar);
            acc += __ldcg(po + (size_t)s2 * D) * f;
            lsum += hl[s2] * f;
        }
        p.a.out[(qh0 + h) * D + d] = __float2half_rn(acc / lsum);
    }
}

__device__ __forceinline__ void key_range(const AttnDev& p, uint32_t& seq_start, uint32_t& seq_len) {
    seq_len = p.a.seq_from_pos ? dyn_position(p.dyn) + 1u : p.a.seq_len;
    if (seq_len > p.a.capacity) seq_len = p.a.capacity;
    seq_start = 0;
    if (p.a.sliding_window > 0 && p.a.sliding_window < seq_len) seq_start = seq_len - p.a.sliding_window;
}

// One (split, KV head, sequence) work item by one CTA of kAttnThreads threads.  Sync is called
// once by every thread before the first read of q or the caches (see affine_imma.cuh).
// One 16-key tile, first half: S^T = K . Q^T from the K unit's pieces (ku: piece p of lane l at
// p * 512 + l * 16, already offset to this lane), then the online softmax of the tile's columns.
// valid_a / valid_b: this thread's keys g and g + 8 of the tile take part.  Leaves P^T as fp16
// high and low parts in B-operand layout (pb0, pb1, pl0, pl1) and rescales m_run, l_run, o.
template <int D, int NH>
__device__ __forceinline__ void tile_scores_softmax(const unsigned char* ku, const uint32_t (&qf)[NH][D / 8], bool valid_a, bool valid_b,
                                                    float scale2, float (&m_run)[NH][2], float (&l_run)[NH][2], float (&o)[NH][D / 16][4],
                                                    uint32_t (&pb0)[NH], uint32_t (&pb1)[NH], uint32_t (&pl0)[NH], uint32_t (&pl1)[NH]) {
    constexpr int MT = D / 16, KJ = D / 32;
    // ── S^T = K · Q^T ──
    float s[NH][4];
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) s[nh][0] = s[nh][1] = s[nh][2] = s[nh][3] = 0.f;
#pragma unroll
    for (int j = 0; j < KJ; ++j) {
        const uint4 ka = *reinterpret_cast<const uint4*>(ku + (2 * j) * 512), kb = *reinterpret_cast<const uint4*>(ku + (2 * j + 1) * 512);
#pragma unroll
        for (int nh = 0; nh < NH; ++nh) {
            mma16816(s[nh], ka.x, kb.x, ka.y, kb.y, qf[nh][4 * j + 0], qf[nh][4 * j + 1]);
            mma16816(s[nh], ka.z, kb.z, ka.w, kb.w, qf[nh][4 * j + 2], qf[nh][4 * j + 3]);
        }
    }

    // ── online softmax per query head (columns 2t, 2t+1 of the tile) ──
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
        float v0 = valid_a ? s[nh][0] * scale2 : kNegBig, v1 = valid_a ? s[nh][1] * scale2 : kNegBig;
        float v2 = valid_b ? s[nh][2] * scale2 : kNegBig, v3 = valid_b ? s[nh][3] * scale2 : kNegBig;
        float mx0 = fmaxf(v0, v2), mx1 = fmaxf(v1, v3);
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
        }
        const float mn0 = fmaxf(m_run[nh][0], mx0), mn1 = fmaxf(m_run[nh][1], mx1);
        const float c0 = exp2f(m_run[nh][0] - mn0), c1 = exp2f(m_run[nh][1] - mn1);
        m_run[nh][0] = mn0; m_run[nh][1] = mn1;
        // p = hi + lo with both halves fp16: the tensor pipe sees 22 significant bits of p
        const float p0 = valid_a ? exp2f(v0 - mn0) : 0.f, p1 = valid_a ? exp2f(v1 - mn1) : 0.f;
        const float p2 = valid_b ? exp2f(v2 - mn0) : 0.f, p3 = valid_b ? exp2f(v3 - mn1) : 0.f;
        const __half2 pa = __floats2half2_rn(p0, p1), pb = __floats2half2_rn(p2, p3);
        const float2 paf = __half22float2(pa), pbf = __half22float2(pb);
        const __half2 pa_lo = __floats2half2_rn(p0 - paf.x, p1 - paf.y), pb_lo = __floats2half2_rn(p2 - pbf.x, p3 - pbf.y);
        l_run[nh][0] = l_run[nh][0] * c0 + (p0 + p2);
        l_run[nh][1] = l_run[nh][1] * c1 + (p1 + p3);
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            o[nh][i][0] *= c0; o[nh][i][2] *= c0;
            o[nh][i][1] *= c1; o[nh][i][3] *= c1;
        }
        pb0[nh] = movmatrix_trans(h2_as_u32(pa));  // {P[key 2t][head g], P[key 2t+1][head g]}
        pb1[nh] = movmatrix_trans(h2_as_u32(pb));  // keys 2t+8, 2t+9
        pl0[nh] = movmatrix_trans(h2_as_u32(pa_lo));
        pl1[nh] = movmatrix_trans(h2_as_u32(pb_lo));
    }

}

// Second half: O^T += V^T . P^T from the V unit's pieces (vu, same addressing).
template <int D, int NH>
__device__ __forceinline__ void tile_weighted_sum(const unsigned char* vu, float (&o)[NH][D / 16][4], const uint32_t (&pb0)[NH],
                                                  const uint32_t (&pb1)[NH], const uint32_t (&pl0)[NH], const uint32_t (&pl1)[NH]) {
    constexpr int VC = D / 64;
#pragma unroll
    for (int c = 0; c < VC; ++c) {
        const uint4 v0 = *reinterpret_cast<const uint4*>(vu + (4 * c + 0) * 512), v1 = *reinterpret_cast<const uint4*>(vu + (4 * c + 1) * 512);
        const uint4 v2 = *reinterpret_cast<const uint4*>(vu + (4 * c + 2) * 512), v3 = *reinterpret_cast<const uint4*>(vu + (4 * c + 3) * 512);
        const uint32_t r0[4] = {v0.x, v0.y, v0.z, v0.w};
        const uint32_t r1[4] = {v1.x, v1.y, v1.z, v1.w};
        const uint32_t r2[4] = {v2.x, v2.y, v2.z, v2.w};
        const uint32_t r3[4] = {v3.x, v3.y, v3.z, v3.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t a0 = __byte_perm(r0[e], r1[e], 0x5410), a1 = __byte_perm(r0[e], r1[e], 0x7632);
            const uint32_t a2 = __byte_perm(r2[e], r3[e], 0x5410), a3 = __byte_perm(r2[e], r3[e], 0x7632);
#pragma unroll
            for (int nh = 0; nh < NH; ++nh) {
                mma16816(o[nh][4 * c + e], a0, a1, a2, a3, pb0[nh], pb1[nh]);
                mma16816(o[nh][4 * c + e], a0, a1, a2, a3, pl0[nh], pl1[nh]);
            }
        }
    }
}

template <int D, int NU>
__host__ __device__ constexpr size_t attn_ring_bytes() {
    return (size_t)kAttnWarps * NU * (D / 16) * 512;
}

// Shared memory of a CTA: the rings plus the RoPE prologue's scratch (up to 16 rotated query heads)
// during the key loop and the warps' merge area [8][heads][D + 2] afterwards, in the same bytes;
// behind both, where no phase of this CTA ever writes, the area the other ranks of a cluster push
// their merged states into: [8 ranks][slice] values (16 D + 8 floats cover every split count),
// then [8 ranks][16 heads][2].
template <int D, int NH, int NU>
__host__ __device__ constexpr size_t attn_recv_offset() {
    const size_t loop = attn_ring_bytes<D, NU>() + (size_t)16 * D * sizeof(__half);
    const size_t merge = (size_t)kAttnWarps * NH * 8 * (D + 2) * sizeof(float);
    return ((loop > merge ? loop : merge) + 15) & ~(size_t)15;
}
__host__ __device__ constexpr int kRecvMlOffset(int D) { return 16 * D + 8; }
template <int D, int NH, int NU>
__host__ __device__ constexpr size_t attn_smem_bytes() {
    return attn_recv_offset<D, NH, NU>() + ((size_t)16 * D + 8 + 8 * 16 * 2) * sizeof(float);
}


template <int D, int NH, int NU, class Sync>
__device__ __forceinline__ void attn_decode_body(const AttnDev& p, float* smem_f, int split, int kvh, int b, Sync sync) {
    constexpr int MT = D / 16;  // m-tiles of O^T
    constexpr int KJ = D / 32;  // 16-byte chunks per thread per K row
    constexpr int VC = D / 64;  // 16-byte chunks per thread per V row
    const AttnArgs& a = p.a;
    // Cache rows below seq_len - 1 that were written before this token's launches began may be
    // requested before the wait for the previous launch; everything else is read after it.
    const bool early = a.kv_rows_stable && a.k_new;
    if (!early) sync();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int ratio = a.n_q / a.n_kv;

    uint32_t seq_start, seq_len;
    key_range(p, seq_start, seq_len);
    const uint32_t n = seq_len - seq_start;
    uint32_t per = (n + p.nsplits - 1) / p.nsplits;
    per = (per + 15u) & ~15u;
    const uint32_t k_begin = min(seq_len, seq_start + (uint32_t)split * per);
    const uint32_t k_end = min(seq_len, k_begin + per);

    const __half* Kb = a.k_cache + (size_t)b * a.seq_stride + (size_t)kvh * a.capacity * D;
    const __half* Vb = a.v_cache + (size_t)b * a.seq_stride + (size_t)kvh * a.capacity * D;

    // One tile = 16 keys.  Its K half (rows g and g + 8: 16-byte pieces that are A fragments as
    // they come) and its V half (the four rows this thread contracts over) are one ring unit
    // each: D / 16 pieces of 16 bytes per thread, copied with cp.async into this warp's ring of
    // NU units and read back by the thread that copied them, so a unit needs no barrier, only
    // this thread's cp.async group count.  NU - 1 units are in flight while one is consumed.
    constexpr int CH = D / 16;  // 16-byte pieces per thread and unit
    unsigned char* ring = reinterpret_cast<unsigned char*>(smem_f) + (size_t)warp * NU * CH * 512 + lane * 16;
    const uint32_t kt0 = k_begin + warp * 16;
    const uint32_t k_off = (uint32_t)g * D + 8 * t, v_off = (uint32_t)(2 * t) * D + 8 * g;  // this thread's first piece of a full tile
    auto issue_unit = [&](int u) {  // unit u of this warp: K (even) or V (odd) of its tile u / 2
        const uint32_t kt = kt0 + (uint32_t)(u >> 1) * (kAttnWarps * 16);
        if (kt < k_end) {
            unsigned char* dst = ring + (size_t)(u % NU) * CH * 512;
            if (kt + 16 <= k_end) {  // a full tile: rows g, g + 8 of K; rows 2t, 2t+1, 2t+8, 2t+9 of V
                if ((u & 1) == 0) {
                    const __half* kp = Kb + (size_t)kt * D + k_off;
#pragma unroll
                    for (int j = 0; j < KJ; ++j) {
                        cp_async16(dst + (2 * j) * 512, kp + 32 * j);
                        cp_async16(dst + (2 * j + 1) * 512, kp + 8 * D + 32 * j);
                    }
                } else {
                    const __half* vp = Vb + (size_t)kt * D + v_off;
#pragma unroll
                    for (int c = 0; c < VC; ++c) {
                        cp_async16(dst + (4 * c + 0) * 512, vp + 64 * c);
                        cp_async16(dst + (4 * c + 1) * 512, vp + D + 64 * c);
                        cp_async16(dst + (4 * c + 2) * 512, vp + 8 * D + 64 * c);
                        cp_async16(dst + (4 * c + 3) * 512, vp + 9 * D + 64 * c);
                    }
                }
            } else {  // the ragged last tile: rows past the end repeat the last key (their scores are masked)
                const uint32_t last = k_end - 1;
                if ((u & 1) == 0) {
                    const __half* ka_p = Kb + (size_t)min(kt + g, last) * D + 8 * t;
                    const __half* kb_p = Kb + (size_t)min(kt + g + 8, last) * D + 8 * t;
#pragma unroll
                    for (int j = 0; j < KJ; ++j) {
                        cp_async16(dst + (2 * j) * 512, ka_p + 32 * j);
                        cp_async16(dst + (2 * j + 1) * 512, kb_p + 32 * j);
                    }
                } else {
                    const uint32_t kv[4] = {min(kt + 2 * t, last), min(kt + 2 * t + 1, last), min(kt + 2 * t + 8, last), min(kt + 2 * t + 9, last)};
#pragma unroll
                    for (int c = 0; c < VC; ++c)
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            cp_async16(dst + (4 * c + kk) * 512, Vb + (size_t)kv[kk] * D + 64 * c + 8 * g);
                }
            }
        }
        cp_async_commit();  // always: the group count stays uniform past the last tile
    };
    // Units are requested before the RoPE prologue, whose own round trips they then overlap,
    // up to the tile that holds the new token's row, which this CTA is about to write.
    int issued = 0;
    for (; issued < NU - 1; ++issued) {
        const uint32_t kt = kt0 + (uint32_t)(issued >> 1) * (kAttnWarps * 16);
        if (a.k_new && kt < k_end && kt + 16 > seq_len - 1u) break;
        issue_unit(issued);
    }
    if (early) sync();
    if (dyn_skip(p.dyn)) {
        cp_async_wait<0>();  // copies in flight must land before the CTA's shared memory retires
        return;
    }

    // ── folded RoPE / KV append (apply_rope, rope_kv_cache_update, kv_cache_update of
    // Resources/Shaders/attention.metal:48-209, full-head analytic mode): the new token is key
    // seq_len - 1.  cos / sin of the position once per CTA, the group's query heads rotated
    // into shared memory, and the CTA whose key range holds the new key writes its K and V rows.
    const __half* q_src = a.q + ((size_t)b * a.n_q + (size_t)kvh * ratio) * D;
    int q_pitch = D;
    if (a.k_new) {
        constexpr int HALF = D / 2;
        constexpr int QI = (16 * HALF + kAttnThreads - 1) / kAttnThreads;  // rotated pairs per thread at the largest group (16 heads)
        __half* s_q = reinterpret_cast<__half*>(smem_f + attn_ring_bytes<D, NU>() / sizeof(float));  // behind the rings, which are already filling
        const uint32_t pos = seq_len - 1u;
        const bool owner = k_begin <= pos && pos < k_end && pos < a.capacity && tid < HALF;  // this thread rotates a pair of the new key
        const __half* kn = a.k_new + ((size_t)b * a.n_kv + kvh) * D;
        const __half* vn = a.v_new + ((size_t)b * a.n_kv + kvh) * D;
        // Every global read of the prologue is requested before any of them is used: the cos / sin
        // pair of each of this thread's query pairs (from the per-token table when there is one),
        // the query values, and the new key / value pair: one round trip, not three.
        float qc[QI], qs[QI];
        __half qx0[QI], qx1[QI];
        int qd0[QI], qd1[QI], qh[QI];
#pragma unroll
        for (int i = 0; i < QI; ++i) {
            const int idx = tid + kAttnThreads * i;
            qh[i] = -1;
            if (idx < ratio * HALF) {
                const int h = idx / HALF, pr = idx % HALF;
                int c0i, c1i;
                rope_indices(a.rope_layout, pr, HALF, D, qd0[i], qd1[i], c0i, c1i);
                qh[i] = h;
                if (a.rope_table) { qc[i] = a.rope_table[pr]; qs[i] = a.rope_table[HALF + pr]; }
                qx0[i] = q_src[h * D + qd0[i]]; qx1[i] = q_src[h * D + qd1[i]];
            }
        }
        float kc = 0.f, ks = 0.f;
        __half kx0 = __half(), kx1 = __half();
        __half2 vpair = __half2();
        int kd0 = 0, kd1 = 0;
        if (owner) {
            int c0i, c1i;
            rope_indices(a.rope_layout, tid, HALF, D, kd0, kd1, c0i, c1i);
            if (a.rope_table) { kc = a.rope_table[tid]; ks = a.rope_table[HALF + tid]; }
            kx0 = kn[kd0]; kx1 = kn[kd1];
            vpair = reinterpret_cast<const __half2*>(vn)[tid];
        }
        if (!a.rope_table) {  // no table: cos / sin of the position from the base, per pair
#pragma unroll
            for (int i = 0; i < QI; ++i)
                if (qh[i] >= 0) {
                    float c1, s1;
                    rope_trig((tid + kAttnThreads * i) % HALF, HALF, pos, a.rope_base_log2, 1, nullptr, nullptr, 0, 0, qc[i], qs[i], c1, s1);
                }
            if (owner) {
                float c1, s1;
                rope_trig(tid, HALF, pos, a.rope_base_log2, 1, nullptr, nullptr, 0, 0, kc, ks, c1, s1);
            }
        }
#pragma unroll
        for (int i = 0; i < QI; ++i)
            if (qh[i] >= 0) {
                const float x0 = __half2float(qx0[i]), x1 = __half2float(qx1[i]);
                s_q[qh[i] * D + qd0[i]] = __float2half_rn(__fsub_rn(__fmul_rn(x0, qc[i]), __fmul_rn(x1, qs[i])));
                s_q[qh[i] * D + qd1[i]] = __float2half_rn(__fadd_rn(__fmul_rn(x0, qs[i]), __fmul_rn(x1, qc[i])));
            }
        if (owner) {
            __half* kd = const_cast<__half*>(Kb) + (size_t)pos * D;
            __half* vd = const_cast<__half*>(Vb) + (size_t)pos * D;
            const float x0 = __half2float(kx0), x1 = __half2float(kx1);
            kd[kd0] = __float2half_rn(__fsub_rn(__fmul_rn(x0, kc), __fmul_rn(x1, ks)));
            kd[kd1] = __float2half_rn(__fadd_rn(__fmul_rn(x1, kc), __fmul_rn(x0, ks)));
            reinterpret_cast<__half2*>(vd)[tid] = vpair;
            __threadfence_block();
        }
        __syncthreads();  // rotated q and the new cache rows are visible to the whole CTA
        q_src = s_q;
    }

    // Q^T fragments: thread (g,t) keeps head g's dims [32j + 8t, +8) for every j.
    uint32_t qf[NH][D / 8];
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
        const int hl = nh * 8 + g;
        if (hl < ratio) {
            const __half* qh = q_src + (size_t)hl * q_pitch;
#pragma unroll
            for (int j = 0; j < KJ; ++j) {
                const uint4 v = *reinterpret_cast<const uint4*>(qh + 32 * j + 8 * t);
                qf[nh][4 * j + 0] = v.x; qf[nh][4 * j + 1] = v.y; qf[nh][4 * j + 2] = v.z; qf[nh][4 * j + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < D / 8; ++j) qf[nh][j] = 0u;
        }
    }
    for (; issued < NU - 1; ++issued) issue_unit(issued);
    const float scale2 = a.scale * 1.4426950408889634f;

    float m_run[NH][2], l_run[NH][2], o[NH][MT][4];
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
        m_run[nh][0] = m_run[nh][1] = kNegBig;
        l_run[nh][0] = l_run[nh][1] = 0.f;
#pragma unroll
        for (int i = 0; i < MT; ++i) o[nh][i][0] = o[nh][i][1] = o[nh][i][2] = o[nh][i][3] = 0.f;
    }

    int unit = 0;
    for (uint32_t kt = kt0; kt < k_end; kt += kAttnWarps * 16, unit += 2) {
        const bool valid_a = kt + g < k_end, valid_b = kt + g + 8 < k_end;
        issue_unit(unit + NU - 1);
        cp_async_wait<NU - 1>();  // this thread's pieces of the K unit have landed
        const unsigned char* ku = ring + (size_t)(unit % NU) * CH * 512;

        uint32_t pb0[NH], pb1[NH], pl0[NH], pl1[NH];
        tile_scores_softmax<D, NH>(ku, qf, valid_a, valid_b, scale2, m_run, l_run, o, pb0, pb1, pl0, pl1);

        // ── O^T += V^T · P^T ──
        issue_unit(unit + NU);
        cp_async_wait<NU - 1>();  // the V unit has landed
        const unsigned char* vu = ring + (size_t)((unit + 1) % NU) * CH * 512;
        tile_weighted_sum<D, NH>(vu, o, pb0, pb1, pl0, pl1);
    }

    // per-thread partial denominators cover keys g, g+8 only: finish the sum over g
#pragma unroll
    for (int nh = 0; nh < NH; ++nh)
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            l_run[nh][0] += __shfl_xor_sync(0xffffffffu, l_run[nh][0], off);
            l_run[nh][1] += __shfl_xor_sync(0xffffffffu, l_run[nh][1], off);
        }

    // ── merge the warps through shared memory, which the rings no longer need ──
    cp_async_wait<0>();
    __syncthreads();
    constexpr int HN = NH * 8;
    float* s_o = smem_f;                                  // [warps][HN][D]
    float* s_ml = smem_f + kAttnWarps * HN * D;           // [warps][HN][2]
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
        if (g == 0) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                s_ml[((warp * HN) + nh * 8 + 2 * t + c) * 2 + 0] = m_run[nh][c];
                s_ml[((warp * HN) + nh * 8 + 2 * t + c) * 2 + 1] = l_run[nh][c];
            }
        }
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int head = nh * 8 + 2 * t + (c & 1);
                const int j = 2 * i + (c >> 1);                      // index among this thread's dims
                const int dim = 64 * (j >> 3) + 8 * g + (j & 7);
                s_o[(size_t)(warp * HN + head) * D + dim] = o[nh][i][c];
            }
    }
    __syncthreads();
    for (int idx = tid; idx < ratio * D; idx += kAttnThreads) {
        const int h = idx / D, d = idx % D;
        float mstar = kNegBig;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) mstar = fmaxf(mstar, s_ml[(w * HN + h) * 2]);
        float acc = 0.f, lsum = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float f = exp2f(s_ml[(w * HN + h) * 2] - mstar);
            acc += s_o[(size_t)(w * HN + h) * D + d] * f;
            lsum += s_ml[(w * HN + h) * 2 + 1] * f;
        }
        const size_t qh = (size_t)b * a.n_q + (size_t)kvh * ratio + h;
        if (a.mlx_partials) {
            // First half of the reference's two-pass pair (Resources/Shaders/attention.metal:1071-1141):
            // block `split` of this head in the reference's buffers: fp16 partial [n_q, 128, D],
            // fp32 stats [2][n_q][128] = sum of exp(score - max), then max, in natural-log units.
            a.mlx_partials[(qh * kMlxBlocks + split) * D + d] = __float2half_rn(acc);
            if (d == 0) {
                a.mlx_stats[qh * kMlxBlocks + split] = lsum;
                a.mlx_stats[(size_t)a.n_q * kMlxBlocks + qh * kMlxBlocks + split] = lsum > 0.f ? mstar * 0.6931471805599453f : -3.402823466e+38f;
            }
        } else if (p.nsplits == 1) {
            a.out[qh * D + d] = __float2half_rn(acc / lsum);
        } else if (p.cluster) {
            // Pushed, not pulled: this CTA's merged value goes straight into the shared memory of the
            // rank that finishes the item ([source rank][item of the owner's slice]), its (max, sum)
            // pairs to every rank; a remote store needs no reply, a remote load is a round trip.
            cg::cluster_group cluster = cg::this_cluster();
            float* recv = smem_f + attn_recv_offset<D, NH, NU>() / sizeof(float);  // [8 ranks][slice] values, then [8 ranks][16 heads][2]
            const int items = ratio * D, per_rank = (items + p.nsplits - 1) / p.nsplits;
            const int owner = idx / per_rank;
            cluster.map_shared_rank(recv, owner)[split * per_rank + (idx - owner * per_rank)] = acc;
            if (d == 0) {
                for (int s2 = 0; s2 < p.nsplits; ++s2) {
                    float* ml = cluster.map_shared_rank(recv, s2) + kRecvMlOffset(D) + (split * 16 + h) * 2;
                    ml[0] = mstar; ml[1] = lsum;
                }
            }
        } else {
            p.part_o[(qh * p.nsplits + split) * D + d] = acc;
            if (d == 0) {
                p.part_ml[(qh * p.nsplits + split) * 2 + 0] = mstar;
                p.part_ml[(qh * p.nsplits + split) * 2 + 1] = lsum;
            }
        }
    }
    if (a.mlx_partials) {
        // blocks no split owns are empty: sum 0, max -FLT_MAX, as a block without keys leaves them
        for (int idx = tid; idx < ratio * kMlxBlocks; idx += kAttnThreads) {
            const int h = idx / kMlxBlocks, j = idx % kMlxBlocks;
            if (j >= p.nsplits && j % p.nsplits == split) {
                const size_t qh = (size_t)b * a.n_q + (size_t)kvh * ratio + h;
                a.mlx_stats[qh * kMlxBlocks + j] = 0.f;
                a.mlx_stats[(size_t)a.n_q * kMlxBlocks + qh * kMlxBlocks + j] = -3.402823466e+38f;
            }
        }
        return;
    }
    if (p.nsplits > 1 && p.cluster) {
        // ── merge across the cluster: rank r finishes a slice of the (head, dim) outputs from the
        // values every rank pushed into its shared memory, in rank order (the arithmetic of
        // attn_merge_kernel).  One cluster barrier: after it nobody touches another CTA's memory. ──
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        const float* recv = smem_f + attn_recv_offset<D, NH, NU>() / sizeof(float);
        const int items = ratio * D, per_rank = (items + p.nsplits - 1) / p.nsplits;
        const int hi = min(items, (split + 1) * per_rank);
        for (int idx = split * per_rank + tid; idx < hi; idx += kAttnThreads) {
            const int h = idx / D, d = idx % D, local = idx - split * per_rank;
            float mstar = kNegBig;
            for (int s2 = 0; s2 < p.nsplits; ++s2) mstar = fmaxf(mstar, recv[kRecvMlOffset(D) + (s2 * 16 + h) * 2]);
            float acc = 0.f, lsum = 0.f;
            for (int s2 = 0; s2 < p.nsplits; ++s2) {
                const float f = exp2f(recv[kRecvMlOffset(D) + (s2 * 16 + h) * 2] - mstar);
                acc += recv[s2 * per_rank + local] * f;
                lsum += recv[kRecvMlOffset(D) + (s2 * 16 + h) * 2 + 1] * f;
            }
            a.out[((size_t)b * a.n_q + (size_t)kvh * ratio + h) * D + d] = __float2half_rn(acc / lsum);
        }
        return;
    }
    if (p.nsplits == 1 || !a.counters) return;

    // ── the last split of this (sequence, KV head) to arrive merges the partials in split
    // order (the arithmetic of attn_merge_kernel) and leaves the counter at zero ──
    __threadfence();
    __syncthreads();
    int* counter = a.counters + (size_t)b * a.n_kv + kvh;
    int* s_ticket = reinterpret_cast<int*>(smem_f);
    if (tid == 0) *s_ticket = atomicAdd(counter, 1);
    __syncthreads();
    if (*s_ticket != p.nsplits - 1) return;
    if (tid == 0) *counter = 0;
    __threadfence();
    merge_partials<D>(p, smem_f + 4, (size_t)b * a.n_q + (size_t)kvh * ratio, ratio, tid, kAttnThreads);  // + 4: clear of the ticket word
}

}  // namespace attn
}  // namespace smelt
