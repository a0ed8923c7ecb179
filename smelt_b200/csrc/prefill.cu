// Prefill: a chunk of prompt positions through the decoder at once instead of one decode step
// per token.
//
// Kernels.  rope_kv_prefill_kernel is rope_and_kv_cache_prefill
// (Resources/Shaders/prefill_rope_kv.metal:64-187): RoPE in place on the chunk's queries
// [T, qHeads, headDim] and keys [T, kvHeads, headDim] at positions startPos + t, then the
// rotated keys and the values written to cache rows startPos + t.  attn_prefill_kernel is
// attention_prefill (Resources/Shaders/prefill_attention.metal:14-413): query position t attends
// causally to keys [seqStart, startPos + t], seqStart from the sliding window, softmax in fp32,
// fp16 out [T, qHeads, headDim].  The matmuls of the chunk are the batched affine kernels
// (agent_affine_qmm_fixed_batched_full, Resources/Shaders/agent_affine_qmm.h:107-316), which
// from seventeen rows on run on the tensor-memory QMM (affine_qmm.cu).
//
// attn_prefill_kernel: one CTA per (eight consecutive query positions, KV head); warp w owns
// position 8 * block + w with all query heads that share the KV head, on the decode kernel's
// tile arithmetic (attention.cuh: S^T = K.Q^T and O^T = V^T.P^T on mma.sync, P as fp16 high +
// low parts).  The CTA walks the 16-key tiles up to its last position's causal limit; a tile's
// K and V halves are copied once per CTA with cp.async into one of two buffers, in the
// piece-per-lane layout the tile functions read, and every warp masks the keys beyond its own
// position.  No split over keys and no merge: a prompt chunk has positions enough to fill the GPU.
//
// smelt_cuda_prefill drives a plain attention decoder (the descriptor smelt_cuda_build_decoder
// takes, one sequence, one GPU) chunk by chunk and leaves the KV caches and the argmax of the
// last position behind, so that decoding continues from the prompt's end.
#include <algorithm>
#include <cmath>
#include <string>

#include "affine_matvec.h"
#include "attention.cuh"
#include "runtime.h"

namespace smelt {

namespace {

using namespace attn;

__global__ void __launch_bounds__(128) rope_kv_prefill_kernel(__half* q, __half* k, const __half* v, const __half* cos_t,
                                                              const __half* sin_t, __half* k_cache, __half* v_cache, int head_dim,
                                                              int rope_dim, int q_heads, int kv_heads, uint32_t start_pos,
                                                              uint32_t capacity, int layout, float base_log2, int math_mode,
                                                              size_t table_stride) {
    pdl_trigger();
    pdl_wait();
    const uint32_t t = blockIdx.x, pos = start_pos + t;
    if (pos >= capacity) return;  // the host validates; never write outside the cache
    const int half_rope = rope_dim / 2;
    if (cos_t) { cos_t += (size_t)pos * table_stride; sin_t += (size_t)pos * table_stride; }
    __half* qrow = q + (size_t)t * q_heads * head_dim;
    __half* krow = k + (size_t)t * kv_heads * head_dim;
    for (int pair = threadIdx.x; pair < half_rope; pair += blockDim.x) {
        int d0, d1, c0i, c1i;
        rope_indices(layout, pair, half_rope, head_dim, d0, d1, c0i, c1i);
        float c0, s0, c1, s1;  // once per (position, pair), shared by every head
        rope_trig(pair, half_rope, pos, base_log2, math_mode, cos_t, sin_t, c0i, c1i, c0, s0, c1, s1);
        for (int h = 0; h < q_heads + kv_heads; ++h) {
            __half* row = h < q_heads ? qrow + (size_t)h * head_dim : krow + (size_t)(h - q_heads) * head_dim;
            const float x0 = __half2float(row[d0]), x1 = __half2float(row[d1]);
            row[d0] = __float2half_rn(__fsub_rn(__fmul_rn(x0, c0), __fmul_rn(x1, s0)));
            row[d1] = __float2half_rn(__fadd_rn(__fmul_rn(x1, c1), __fmul_rn(x0, s1)));
        }
    }
    __syncthreads();  // the rotated keys are complete before they are copied
    const __half* vrow = v + (size_t)t * kv_heads * head_dim;
    for (int i = threadIdx.x; i < kv_heads * head_dim / 2; i += blockDim.x) {
        const int h = (2 * i) / head_dim, d = (2 * i) % head_dim;
        const size_t dst = ((size_t)h * capacity + pos) * head_dim + d;
        *reinterpret_cast<__half2*>(k_cache + dst) = *reinterpret_cast<const __half2*>(krow + 2 * i);
        *reinterpret_cast<__half2*>(v_cache + dst) = *reinterpret_cast<const __half2*>(vrow + 2 * i);
    }
}

template <int D, int NH>
__global__ void __launch_bounds__(kAttnThreads) attn_prefill_kernel(const __half* __restrict__ q, const __half* __restrict__ k_cache,
                                                                    const __half* __restrict__ v_cache, __half* __restrict__ out, int n_q,
                                                                    int n_kv, uint32_t n_pos, uint32_t start_pos, uint32_t capacity,
                                                                    float scale, uint32_t window) {
    constexpr int MT = D / 16, KJ = D / 32, CH = D / 16;
    constexpr int kUnit = CH * 512;  // bytes of a tile's K half (and of its V half)
    __shared__ __align__(16) unsigned char tiles[2][2][kUnit];  // [buffer][K | V]
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int kvh = blockIdx.y, ratio = n_q / n_kv;
    const uint32_t p_first = blockIdx.x * kAttnWarps, p = p_first + warp;
    const bool active = p < n_pos;
    const uint32_t p_last = min(n_pos, p_first + kAttnWarps) - 1u;
    // this warp's keys: [w_lo, w_hi); the CTA's tiles: from the first position's window start to the last position's limit
    const uint32_t w_hi = start_pos + p + 1u, w_lo = (window > 0 && window < w_hi) ? w_hi - window : 0u;
    const uint32_t c_hi = start_pos + p_last + 1u, first_hi = start_pos + p_first + 1u;
    const uint32_t c_lo = ((window > 0 && window < first_hi) ? first_hi - window : 0u) & ~15u;
    const __half* Kb = k_cache + (size_t)kvh * capacity * D;
    const __half* Vb = v_cache + (size_t)kvh * capacity * D;

    auto issue_tile = [&](uint32_t kt, int buf) {
        const uint32_t last = c_hi - 1u;
        for (int i = tid; i < CH * 32; i += kAttnThreads) {
            const int c = i >> 5, ln = i & 31, gg = ln >> 2, tt = ln & 3;
            // K piece c of lane ln: row gg (+8 for odd c), halves [32 (c / 2) + 8 tt, +8)
            const uint32_t krow = min(kt + gg + 8u * (c & 1), last);
            cp_async16(&tiles[buf][0][i * 16], Kb + (size_t)krow * D + 32 * (c >> 1) + 8 * tt);
            // V piece c = 4 cc + kk of lane ln: row 2 tt + (kk & 1) + 8 (kk / 2), halves [64 cc + 8 gg, +8)
            const int kk = c & 3;
            const uint32_t vrow = min(kt + 2u * tt + (kk & 1) + 8u * (kk >> 1), last);
            cp_async16(&tiles[buf][1][i * 16], Vb + (size_t)vrow * D + 64 * (c >> 2) + 8 * gg);
        }
        cp_async_commit();
    };
    issue_tile(c_lo, 0);

    // Q^T fragments of this warp's position: thread (g,t) keeps head g's dims [32j + 8t, +8)
    uint32_t qf[NH][D / 8];
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
        const int hl = nh * 8 + g;
        if (active && hl < ratio) {
            const __half* qh = q + ((size_t)p * n_q + (size_t)kvh * ratio + hl) * D;
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
    const float scale2 = scale * 1.4426950408889634f;
    float m_run[NH][2], l_run[NH][2], o[NH][MT][4];
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
        m_run[nh][0] = m_run[nh][1] = kNegBig;
        l_run[nh][0] = l_run[nh][1] = 0.f;
#pragma unroll
        for (int i = 0; i < MT; ++i) o[nh][i][0] = o[nh][i][1] = o[nh][i][2] = o[nh][i][3] = 0.f;
    }

    int buf = 0;
    for (uint32_t kt = c_lo; kt < c_hi; kt += 16, buf ^= 1) {
        if (kt + 16 < c_hi) issue_tile(kt + 16, buf ^ 1);
        else cp_async_commit();  // the group count stays uniform
        cp_async_wait<1>();
        __syncthreads();  // every thread's pieces of this tile have landed
        if (active && kt < w_hi && kt + 16 > w_lo) {
            const uint32_t ka = kt + g, kb = kt + g + 8;
            const bool valid_a = ka < w_hi && ka >= w_lo, valid_b = kb < w_hi && kb >= w_lo;
            uint32_t pb0[NH], pb1[NH], pl0[NH], pl1[NH];
            tile_scores_softmax<D, NH>(&tiles[buf][0][lane * 16], qf, valid_a, valid_b, scale2, m_run, l_run, o, pb0, pb1, pl0, pl1);
            tile_weighted_sum<D, NH>(&tiles[buf][1][lane * 16], o, pb0, pb1, pl0, pl1);
        }
        __syncthreads();  // the buffer may be refilled
    }
    cp_async_wait<0>();
    if (!active) return;
    // per-thread partial denominators cover keys g, g + 8 only: finish the sum over g
#pragma unroll
    for (int nh = 0; nh < NH; ++nh)
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            l_run[nh][0] += __shfl_xor_sync(0xffffffffu, l_run[nh][0], off);
            l_run[nh][1] += __shfl_xor_sync(0xffffffffu, l_run[nh][1], off);
        }
#pragma unroll
    for (int nh = 0; nh < NH; ++nh)
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int head = nh * 8 + 2 * t + (c & 1);
                if (head >= ratio) continue;
                const int j = 2 * i + (c >> 1);
                const int dim = 64 * (j >> 3) + 8 * g + (j & 7);
                out[((size_t)p * n_q + (size_t)kvh * ratio + head) * D + dim] = __float2half_rn(o[nh][i][c] / l_run[nh][c & 1]);
            }
}

template <int D, int NH>
cudaError_t launch_prefill_attention_t(const Launch& l, const __half* q, const __half* kc, const __half* vc, __half* out, int n_q, int n_kv,
                                       uint32_t n_pos, uint32_t start_pos, uint32_t capacity, float scale, uint32_t window) {
    auto kern = attn_prefill_kernel<D, NH>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((n_pos + kAttnWarps - 1) / kAttnWarps, n_kv);
    cfg.blockDim = dim3(kAttnThreads);
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = l.pdl ? 1 : 0;
    prefer_max_shared(kern);
    return cudaLaunchKernelEx(&cfg, kern, q, kc, vc, out, n_q, n_kv, n_pos, start_pos, capacity, scale, window);
}

Launch lch(smelt_cuda_ctx* ctx) {  // chunk launches chain with programmatic dependent launch, as a decode table's do
    Launch l;
    l.stream = ctx->stream;
    l.pdl = ctx->pdl;
    return l;
}

}  // namespace

cudaError_t launch_rope_kv_prefill(const Launch& l, __half* q, __half* k, const __half* v, const __half* cos_t, const __half* sin_t,
                                   __half* k_cache, __half* v_cache, int head_dim, int rope_dim, int q_heads, int kv_heads, uint32_t n_pos,
                                   uint32_t start_pos, uint32_t capacity, int layout, float base_log2, int math_mode, size_t table_stride) {
    if (n_pos == 0) return cudaSuccess;
    if (head_dim <= 0 || head_dim % 2 || rope_dim <= 0 || rope_dim > head_dim || rope_dim % 2 || q_heads < 0 || kv_heads < 0 ||
        (uint64_t)start_pos + n_pos > capacity)
        return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_pos);
    cfg.blockDim = dim3(128);
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = l.pdl ? 1 : 0;
    prefer_max_shared(rope_kv_prefill_kernel);
    return cudaLaunchKernelEx(&cfg, rope_kv_prefill_kernel, q, k, v, cos_t, sin_t, k_cache, v_cache, head_dim, rope_dim, q_heads, kv_heads,
                              start_pos, capacity, layout, base_log2, math_mode, table_stride);
}

cudaError_t launch_attention_prefill(const Launch& l, const __half* q, const __half* k_cache, const __half* v_cache, __half* out, int n_q,
                                     int n_kv, int head_dim, uint32_t n_pos, uint32_t start_pos, uint32_t capacity, float scale,
                                     uint32_t window) {
    if (n_pos == 0) return cudaSuccess;
    if (n_q <= 0 || n_kv <= 0 || n_q % n_kv || n_q / n_kv > 16 || (uint64_t)start_pos + n_pos > capacity) return cudaErrorInvalidValue;
    const int nh = n_q / n_kv > 8 ? 2 : 1;
#define SMELT_PREFILL_CASE(DD)                                                                                                           \
    case DD:                                                                                                                             \
        return nh == 1 ? launch_prefill_attention_t<DD, 1>(l, q, k_cache, v_cache, out, n_q, n_kv, n_pos, start_pos, capacity, scale, window) \
                       : launch_prefill_attention_t<DD, 2>(l, q, k_cache, v_cache, out, n_q, n_kv, n_pos, start_pos, capacity, scale, window);
    switch (head_dim) {
        SMELT_PREFILL_CASE(64)
        SMELT_PREFILL_CASE(128)
        SMELT_PREFILL_CASE(256)
        default: return cudaErrorInvalidValue;
    }
#undef SMELT_PREFILL_CASE
}

}  // namespace smelt

using namespace smelt;

extern "C" {

smelt_status smelt_cuda_rope_kv_prefill(smelt_cuda_ctx* ctx, void* q, void* k, const void* v, const void* cos_t, const void* sin_t,
                                        void* k_cache, void* v_cache, int head_dim, int rope_dim, int q_heads, int kv_heads,
                                        uint32_t n_pos, uint32_t start_pos, uint32_t capacity, int layout, float base_log2,
                                        int math_mode) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!q || !k || !v || !k_cache || !v_cache || (math_mode != 1 && (!cos_t || !sin_t)) || layout < 0 || layout > 2)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "rope / kv prefill: bad arguments");
    if ((uint64_t)start_pos + n_pos > capacity)
        return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "rope / kv prefill: positions " + std::to_string(start_pos) + " .. +" + std::to_string(n_pos) + " pass the cache capacity " + std::to_string(capacity));
    Launch l;
    l.stream = ctx->stream;
    l.pdl = ctx->capturing && ctx->pdl;
    return check_cuda(ctx, launch_rope_kv_prefill(l, (__half*)q, (__half*)k, (const __half*)v, (const __half*)cos_t, (const __half*)sin_t,
                                                  (__half*)k_cache, (__half*)v_cache, head_dim, rope_dim, q_heads, kv_heads, n_pos, start_pos,
                                                  capacity, layout, base_log2, math_mode, (size_t)rope_dim),
                      "rope / kv prefill");
}

smelt_status smelt_cuda_attention_prefill(smelt_cuda_ctx* ctx, const void* q, const void* k_cache, const void* v_cache, void* out, int n_q,
                                          int n_kv, int head_dim, uint32_t n_pos, uint32_t start_pos, uint32_t capacity, float scale,
                                          uint32_t sliding_window) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!q || !k_cache || !v_cache || !out || n_q <= 0 || n_kv <= 0 || n_q % n_kv)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "attention prefill: bad arguments");
    if (n_q / n_kv > 16 || (head_dim != 64 && head_dim != 128 && head_dim != 256))
        return fail(ctx, SMELT_ERR_UNSUPPORTED, "attention prefill: head_dim in {64,128,256}, GQA ratio <= 16");
    if ((uint64_t)start_pos + n_pos > capacity)
        return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "attention prefill: positions pass the cache capacity");
    Launch l;
    l.stream = ctx->stream;
    l.pdl = ctx->capturing && ctx->pdl;
    return check_cuda(ctx, launch_attention_prefill(l, (const __half*)q, (const __half*)k_cache, (const __half*)v_cache, (__half*)out, n_q, n_kv,
                                                    head_dim, n_pos, start_pos, capacity, scale, sliding_window),
                      "attention prefill");
}

smelt_status smelt_cuda_prefill(smelt_cuda_ctx* ctx, const smelt_decoder_desc* d, const smelt_layer_ref* layers, const int32_t* tokens,
                                int n_tokens, int32_t start_pos, int chunk, int32_t* out_token) {
    if (!ctx || !d || !layers || !tokens || n_tokens <= 0 || start_pos < 0) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (ctx->capturing) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "prefill: a stream capture is open");
    if (!ctx->configured || ctx->cfg.batch != 1) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "prefill: build the decoder for one sequence first (smelt_cuda_build_decoder, batch 1)");
    if (d->tp_world > 1) return fail(ctx, SMELT_ERR_UNSUPPORTED, "prefill: one GPU only");
    const int H = d->hidden, I = d->inter, D = d->head_dim, G = d->group, L = d->layers, V = d->vocab;
    const int qd = d->n_q * D, kvd = d->n_kv * D;
    const uint32_t cap = ctx->cfg.cache_seq_capacity;
    if ((uint64_t)start_pos + (uint64_t)n_tokens > cap || (uint64_t)start_pos + (uint64_t)n_tokens > ctx->cfg.context_limit)
        return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "prefill: " + std::to_string(n_tokens) + " tokens from position " + std::to_string(start_pos) + " pass the limit of " + std::to_string(cap) + " positions");
    for (int i = 0; i < n_tokens; ++i)
        if (tokens[i] < 0 || (uint32_t)tokens[i] >= ctx->cfg.vocab_size)
            return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "tokenId out of range [0, " + std::to_string(ctx->cfg.vocab_size) + ")");
    constexpr int kKvBase = 40, kLogits = 16, kArgmax = 17, kArgmaxScratch = 35;  // the slots smelt_cuda_build_decoder allocates
    const Slot& ws = ctx->slots[ctx->cfg.weights_slot];
    if (!ws.ptr || kKvBase + 2 * L > (int)ctx->slots.size() || !ctx->slots[kLogits].ptr || !ctx->slots[kArgmaxScratch].ptr)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "prefill: the decoder's slots are missing");
    for (int l = 0; l < 2 * L; ++l)
        if (!ctx->slots[kKvBase + l].ptr || ctx->slots[kKvBase + l].bytes < (size_t)d->n_kv * cap * D * 2)
            return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "prefill: KV cache slot " + std::to_string(kKvBase + l) + " is missing or too small");
    if (chunk <= 0) chunk = 512;
    if (chunk > (int)ctx->h_pinned_count / 2) chunk = (int)ctx->h_pinned_count / 2;
    const int T = std::min(chunk, n_tokens);
    // activation scratch for one chunk, owned by the context and kept for the next call
    const size_t per_row = (size_t)2 * (3 * H + 2 * qd + 2 * kvd + I) + 4;
    const size_t need = per_row * T + 4096;
    if (ctx->prefill_scratch_bytes < need) {
        if (ctx->prefill_scratch) cudaFree(ctx->prefill_scratch);
        ctx->prefill_scratch = nullptr;
        ctx->prefill_scratch_bytes = 0;
        cudaError_t e = cudaMalloc(&ctx->prefill_scratch, need);
        if (e != cudaSuccess) return fail(ctx, SMELT_ERR_ALLOC, std::string("prefill scratch: ") + cudaGetErrorString(e));
        ctx->prefill_scratch_bytes = need;
    }
    uint8_t* base = (uint8_t*)ctx->prefill_scratch;
    auto carve = [&](size_t bytes) { uint8_t* p = base; base += (bytes + 255) & ~(size_t)255; return p; };
    int32_t* tok_dev = (int32_t*)carve((size_t)T * 4);
    __half* x0 = (__half*)carve((size_t)T * H * 2);
    __half* x1 = (__half*)carve((size_t)T * H * 2);
    __half* xn = (__half*)carve((size_t)T * H * 2);
    __half* qb = (__half*)carve((size_t)T * qd * 2);
    __half* kb = (__half*)carve((size_t)T * kvd * 2);
    __half* vb = (__half*)carve((size_t)T * kvd * 2);
    __half* ab = (__half*)carve((size_t)T * qd * 2);
    __half* hb = (__half*)carve((size_t)T * I * 2);
    if ((size_t)(base - (uint8_t*)ctx->prefill_scratch) > ctx->prefill_scratch_bytes) return fail(ctx, SMELT_ERR_ALLOC, "prefill scratch: carve overflow");

    const uint8_t* W = (const uint8_t*)ws.ptr;
    auto affine = [&](int mode, const smelt_affine_ref& w0, const smelt_affine_ref* w1, const __half* x, __half* y, __half* y2, const __half* res,
                      int rows, int cols, int n) {
        AffineArgs a = {};
        a.w[0] = W + w0.packed; a.s[0] = (const __half*)(W + w0.scales); a.b[0] = (const __half*)(W + w0.biases);
        if (w1) { a.w[1] = W + w1->packed; a.s[1] = (const __half*)(W + w1->scales); a.b[1] = (const __half*)(W + w1->biases); }
        a.x = x; a.y = y; a.y2 = y2; a.residual = res; a.rows = rows; a.cols = cols; a.batch = n; a.nseg = 1;
        a.sm_count = ctx->sm_count; a.err = ctx->err_dev;
        a.part_scratch = ctx->qmm_scratch; a.part_scratch_bytes = ctx->qmm_scratch_bytes; a.part_counters = ctx->qmm_counters;
        return launch_affine(lch(ctx), mode, a, G);
    };
    const float log2_theta = log2f(d->rope_theta), scale = 1.0f / sqrtf((float)D);
    size_t launches = 0;
#define PF(call, what)                                        \
    do {                                                      \
        smelt_status s_ = check_cuda(ctx, (call), what);      \
        if (s_) return s_;                                    \
        ++launches;                                           \
    } while (0)
    for (int t0 = 0; t0 < n_tokens; t0 += T) {
        const int n = std::min(T, n_tokens - t0);
        const uint32_t p0 = (uint32_t)start_pos + (uint32_t)t0;
        // the previous chunk's copy of its token ids must have been consumed before the staging area is reused
        smelt_status s = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "prefill: chunk boundary");
        if (s) return s;
        for (int i = 0; i < n; ++i) ctx->h_pinned[256 + i] = tokens[t0 + i];
        s = check_cuda(ctx, cudaMemcpyAsync(tok_dev, ctx->h_pinned + 256, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream), "prefill: token ids");
        if (s) return s;
        const Launch l = lch(ctx);
        PF(launch_embedding_gather(l, (const __half*)(W + d->embedding), tok_dev, x0, H, n, 1), "prefill: embedding gather");
        for (int li = 0; li < L; ++li) {
            const smelt_layer_ref& w = layers[li];
            __half* kc = (__half*)ctx->slots[kKvBase + li].ptr;
            __half* vc = (__half*)ctx->slots[kKvBase + L + li].ptr;
            PF(launch_rms_norm_1pw(l, x0, (const __half*)(W + w.input_norm), xn, H, d->eps, n), "prefill: input norm");
            PF(affine(kAffinePlain, w.q, nullptr, xn, qb, nullptr, nullptr, qd, H, n), "prefill: Q projection");
            PF(affine(kAffineDual, w.k, &w.v, xn, kb, vb, nullptr, kvd, H, n), "prefill: K | V projection");
            PF(launch_rope_kv_prefill(l, qb, kb, vb, nullptr, nullptr, kc, vc, D, D, d->n_q, d->n_kv, (uint32_t)n, p0, cap, 1, log2_theta, 1, 0), "prefill: rope + kv write");
            PF(launch_attention_prefill(l, qb, kc, vc, ab, d->n_q, d->n_kv, D, (uint32_t)n, p0, cap, scale, 0), "prefill: attention");
            PF(affine(kAffineAdd, w.o, nullptr, ab, x1, nullptr, x0, H, qd, n), "prefill: O projection + residual");
            PF(launch_rms_norm_1pw(l, x1, (const __half*)(W + w.post_norm), xn, H, d->eps, n), "prefill: post norm");
            PF(affine(kAffineGateUp, w.gate, &w.up, xn, hb, nullptr, nullptr, I, H, n), "prefill: gate / up + SwiGLU");
            PF(affine(kAffineAdd, w.down, nullptr, hb, x0, nullptr, x1, H, I, n), "prefill: down projection + residual");
        }
        if (t0 + n == n_tokens) {
            // the last position only: final norm, LM head, argmax (the decode table's tail)
            const __half* last = x0 + (size_t)(n - 1) * H;
            __half* logits = (__half*)ctx->slots[kLogits].ptr;
            const int achunk = 2048, parts = (V + achunk - 1) / achunk;
            PF(launch_rms_norm_1pw(l, last, (const __half*)(W + d->final_norm), xn, H, d->eps, 1), "prefill: final norm");
            PF(launch_fp16_matvec(l, (const __half*)(W + d->lm_head), xn, logits, V, H, 1, ctx->sm_count), "prefill: LM head");
            PF(launch_argmax_partials(l, logits, (uint64_t*)ctx->slots[kArgmaxScratch].ptr, V, achunk, 1), "prefill: argmax partials");
            PF(launch_argmax_reduce(l, (const uint64_t*)ctx->slots[kArgmaxScratch].ptr, (int32_t*)ctx->slots[kArgmax].ptr, parts, 1, 1), "prefill: argmax");
        }
    }
#undef PF
    ctx->launch_count = launches;
    cudaMemcpyAsync(ctx->h_pinned + 128, ctx->slots[kArgmax].ptr, 4, cudaMemcpyDeviceToHost, ctx->stream);
    smelt_status s = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "prefill");
    if (s) return s;
    if (out_token) *out_token = ctx->h_pinned[128];
    return SMELT_OK;
}

}  // extern "C"
