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

__device__ __forceinline__ void key_range(const AttnDev& p, uint32_t& seq_start, uint32_t& seq_len) {
    seq_len = p.a.seq_from_pos ? dyn_position(p.dyn) + 1u : p.a.seq_len;
    if (seq_len > p.a.capacity) seq_len = p.a.capacity;
    seq_start = 0;
    if (p.a.sliding_window > 0 && p.a.sliding_window < seq_len) seq_start = seq_len - p.a.sliding_window;
}

// One (split, KV head, sequence) work item by one CTA of kAttnThreads threads.  Sync is called
// once by every thread before the first read of q or the caches (see affine_imma.cuh).
template <int D, int NH, class Sync>
__device__ __forceinline__ void attn_decode_body(const AttnDev& p, float* smem_f, int split, int kvh, int b, Sync sync) {
    constexpr int MT = D / 16;  // m-tiles of O^T
    constexpr int KJ = D / 32;  // 16-byte chunks per thread per K row
    constexpr int VC = D / 64;  // 16-byte chunks per thread per V row
    sync();
    if (dyn_skip(p.dyn)) return;

    const AttnArgs& a = p.a;
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

    // One tile = 16 keys: K rows g and g + 8 (16-byte pieces that are A fragments as they come)
    // and the four V rows this thread contracts over.
    uint4 tka[KJ], tkb[KJ], vv[VC][4];
    auto tile_loads = [&](uint32_t kt) {
        const uint32_t last = k_end - 1;
        const __half* ka_p = Kb + (size_t)min(kt + g, last) * D + 8 * t;
        const __half* kb_p = Kb + (size_t)min(kt + g + 8, last) * D + 8 * t;
#pragma unroll
        for (int j = 0; j < KJ; ++j) {
            tka[j] = *reinterpret_cast<const uint4*>(ka_p + 32 * j);
            tkb[j] = *reinterpret_cast<const uint4*>(kb_p + 32 * j);
        }
        // V rows: k-slots 2t, 2t+1, 2t+8, 2t+9 of the tile
        const uint32_t kv[4] = {min(kt + 2 * t, last), min(kt + 2 * t + 1, last), min(kt + 2 * t + 8, last), min(kt + 2 * t + 9, last)};
#pragma unroll
        for (int c = 0; c < VC; ++c)
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
                vv[c][kk] = *reinterpret_cast<const uint4*>(Vb + (size_t)kv[kk] * D + 64 * c + 8 * g);
    };
    // The first tile of every warp is requested before the RoPE prologue, whose own round trips
    // it then overlaps, unless it holds the new token's row, which this CTA is about to write.
    const uint32_t kt0 = k_begin + warp * 16;
    const bool preloaded = D <= 128 && kt0 < k_end && (!a.k_new || kt0 + 16 <= seq_len - 1u);
    if (preloaded) tile_loads(kt0);

    // ── folded RoPE / KV append (apply_rope, rope_kv_cache_update, kv_cache_update of
    // Resources/Shaders/attention.metal:48-209, full-head analytic mode): the new token is key
    // seq_len - 1.  cos / sin of the position once per CTA, the group's query heads rotated
    // into shared memory, and the CTA whose key range holds the new key writes its K and V rows.
    const __half* q_src = a.q + ((size_t)b * a.n_q + (size_t)kvh * ratio) * D;
    int q_pitch = D;
    if (a.k_new) {
        constexpr int HALF = D / 2;
        float* s_cos = smem_f;
        float* s_sin = smem_f + HALF;
        __half* s_q = reinterpret_cast<__half*>(smem_f + 2 * HALF);
        const uint32_t pos = seq_len - 1u;
        if (tid < HALF) {
            if (a.rope_table) {  // cos | sin of this token's position, computed once per token
                s_cos[tid] = a.rope_table[tid]; s_sin[tid] = a.rope_table[HALF + tid];
            } else {
                int d0, d1, c0i, c1i;
                float c0, s0, c1, s1;
                rope_indices(a.rope_layout, tid, HALF, D, d0, d1, c0i, c1i);
                rope_trig(tid, HALF, pos, a.rope_base_log2, 1, nullptr, nullptr, c0i, c1i, c0, s0, c1, s1);
                s_cos[tid] = c0; s_sin[tid] = s0;
            }
        }
        __syncthreads();
        for (int idx = tid; idx < ratio * HALF; idx += kAttnThreads) {
            const int h = idx / HALF, pr = idx % HALF;
            int d0, d1, c0i, c1i;
            rope_indices(a.rope_layout, pr, HALF, D, d0, d1, c0i, c1i);
            const float c = s_cos[pr], sn = s_sin[pr];
            const float x0 = __half2float(q_src[h * D + d0]), x1 = __half2float(q_src[h * D + d1]);
            s_q[h * D + d0] = __float2half_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn)));
            s_q[h * D + d1] = __float2half_rn(__fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c)));
        }
        if (k_begin <= pos && pos < k_end && pos < a.capacity) {
            const __half* kn = a.k_new + ((size_t)b * a.n_kv + kvh) * D;
            const __half* vn = a.v_new + ((size_t)b * a.n_kv + kvh) * D;
            __half* kd = const_cast<__half*>(Kb) + (size_t)pos * D;
            __half* vd = const_cast<__half*>(Vb) + (size_t)pos * D;
            for (int pr = tid; pr < HALF; pr += kAttnThreads) {
                int d0, d1, c0i, c1i;
                rope_indices(a.rope_layout, pr, HALF, D, d0, d1, c0i, c1i);
                const float c = s_cos[pr], sn = s_sin[pr];
                const float x0 = __half2float(kn[d0]), x1 = __half2float(kn[d1]);
                kd[d0] = __float2half_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn)));
                kd[d1] = __float2half_rn(__fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, sn)));
                reinterpret_cast<__half2*>(vd)[pr] = reinterpret_cast<const __half2*>(vn)[pr];
            }
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
    if (a.k_new) __syncthreads();  // the rotated q lives where the warps later exchange their states
    const float scale2 = a.scale * 1.4426950408889634f;

    float m_run[NH][2], l_run[NH][2], o[NH][MT][4];
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
        m_run[nh][0] = m_run[nh][1] = kNegBig;
        l_run[nh][0] = l_run[nh][1] = 0.f;
#pragma unroll
        for (int i = 0; i < MT; ++i) o[nh][i][0] = o[nh][i][1] = o[nh][i][2] = o[nh][i][3] = 0.f;
    }

    for (uint32_t kt = k_begin + warp * 16; kt < k_end; kt += kAttnWarps * 16) {
        const bool valid_a = kt + g < k_end, valid_b = kt + g + 8 < k_end;
        // every load of the tile is issued before any arithmetic: one memory round trip per tile
        if (!(preloaded && kt == kt0)) tile_loads(kt);

        // ── S^T = K · Q^T ──
        float s[NH][4];
#pragma unroll
        for (int nh = 0; nh < NH; ++nh) s[nh][0] = s[nh][1] = s[nh][2] = s[nh][3] = 0.f;
#pragma unroll
        for (int j = 0; j < KJ; ++j) {
            const uint4 ka = tka[j], kb = tkb[j];
#pragma unroll
            for (int nh = 0; nh < NH; ++nh) {
                mma16816(s[nh], ka.x, kb.x, ka.y, kb.y, qf[nh][4 * j + 0], qf[nh][4 * j + 1]);
                mma16816(s[nh], ka.z, kb.z, ka.w, kb.w, qf[nh][4 * j + 2], qf[nh][4 * j + 3]);
            }
        }

        // ── online softmax per query head (columns 2t, 2t+1 of the tile) ──
        uint32_t pb0[NH], pb1[NH], pl0[NH], pl1[NH];
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

        // ── O^T += V^T · P^T ──
#pragma unroll
        for (int c = 0; c < VC; ++c) {
            const uint32_t r0[4] = {vv[c][0].x, vv[c][0].y, vv[c][0].z, vv[c][0].w};
            const uint32_t r1[4] = {vv[c][1].x, vv[c][1].y, vv[c][1].z, vv[c][1].w};
            const uint32_t r2[4] = {vv[c][2].x, vv[c][2].y, vv[c][2].z, vv[c][2].w};
            const uint32_t r3[4] = {vv[c][3].x, vv[c][3].y, vv[c][3].z, vv[c][3].w};
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

    // per-thread partial denominators cover keys g, g+8 only: finish the sum over g
#pragma unroll
    for (int nh = 0; nh < NH; ++nh)
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            l_run[nh][0] += __shfl_xor_sync(0xffffffffu, l_run[nh][0], off);
            l_run[nh][1] += __shfl_xor_sync(0xffffffffu, l_run[nh][1], off);
        }

    // ── merge the four warps through shared memory ──
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
            float* c_o = smem_f + kAttnWarps * HN * (D + 2);  // [16][D] then [16][2]
            c_o[idx] = acc;
            if (d == 0) { c_o[16 * D + 2 * h] = mstar; c_o[16 * D + 2 * h + 1] = lsum; }
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
        // ── merge across the cluster: rank r finishes a slice of the (head, dim) outputs from
        // every rank's partials, in rank order (the arithmetic of attn_merge_kernel) ──
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        float* c_o = smem_f + kAttnWarps * HN * (D + 2);
        const int items = ratio * D, per_rank = (items + p.nsplits - 1) / p.nsplits;
        const int hi = min(items, (split + 1) * per_rank);
        for (int idx = split * per_rank + tid; idx < hi; idx += kAttnThreads) {
            const int h = idx / D, d = idx % D;
            float mstar = kNegBig;
            for (int s2 = 0; s2 < p.nsplits; ++s2) mstar = fmaxf(mstar, cluster.map_shared_rank(c_o, s2)[16 * D + 2 * h]);
            float acc = 0.f, lsum = 0.f;
            for (int s2 = 0; s2 < p.nsplits; ++s2) {
                const float* rc = cluster.map_shared_rank(c_o, s2);
                const float f = exp2f(rc[16 * D + 2 * h] - mstar);
                acc += rc[idx] * f;
                lsum += rc[16 * D + 2 * h + 1] * f;
            }
            a.out[((size_t)b * a.n_q + (size_t)kvh * ratio + h) * D + d] = __float2half_rn(acc / lsum);
        }
        cluster.sync();  // nobody leaves while a peer still reads its shared memory
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
    for (int idx = tid; idx < ratio * D; idx += kAttnThreads) {
        const int h = idx / D, d = idx % D;
        const size_t qh = (size_t)b * a.n_q + (size_t)kvh * ratio + h;
        float mstar = kNegBig;
        for (int s2 = 0; s2 < p.nsplits; ++s2) mstar = fmaxf(mstar, __ldcg(p.part_ml + (qh * p.nsplits + s2) * 2));
        float acc = 0.f, lsum = 0.f;
        for (int s2 = 0; s2 < p.nsplits; ++s2) {
            const float f = exp2f(__ldcg(p.part_ml + (qh * p.nsplits + s2) * 2) - mstar);
            acc += __ldcg(p.part_o + (qh * p.nsplits + s2) * D + d) * f;
            lsum += __ldcg(p.part_ml + (qh * p.nsplits + s2) * 2 + 1) * f;
        }
        a.out[qh * D + d] = __float2half_rn(acc / lsum);
    }
}

template <int D, int NH>
__host__ __device__ constexpr size_t attn_smem_bytes() {
    return ((size_t)kAttnWarps * NH * 8 + 16) * (D + 2) * sizeof(float);
}

}  // namespace attn
}  // namespace smelt
