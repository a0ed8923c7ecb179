// Single-token GQA attention over an fp16 KV cache: split-K flash-decode for sm_100a.
//
// Replaces the reference's attention_decode family (Resources/Shaders/attention.metal:217-314
// generic three-pass kernel, :981-1065 one-pass online softmax, :1071-1206 two-pass split-K,
// :1211-1309 D128 sdpa) with one kernel pair.  Semantics follow the reference oracle
// (Tests/SmeltCompilerTests/RegionExactnessTests.swift:1414-1475): scores = (q.k) * scale over
// keys [seqStart, seqLen), softmax in fp32, output rounded to fp16 once; K and V are laid out
// [n_kv, capacity, head_dim] per sequence and GQA maps query head h to KV head h / (n_q/n_kv).
//
// Data path.  Grid = (splits, n_kv, batch); a CTA of four warps owns a contiguous key range
// of one KV head and all query heads that share it, so K and V are read from HBM exactly
// once.  A warp walks 16-key tiles.  S^T = K·Q^T and O^T = V^T·P^T both run on
// mma.sync.m16n8k16 (keys or head dims on M, the <= 8 grouped query heads on N), which keeps
// the CUDA cores free for loads and the online softmax; K fragments are 16-byte loads used
// directly as the A operand (the contraction order over head_dim is permuted consistently in
// Q), V is loaded 16 bytes per key and paired across keys with byte permutes, and P is
// transposed into B-operand layout with movmatrix.  Each probability enters the tensor pipe
// as an fp16 high part plus an fp16 low part (two MMAs), so the weighted sum keeps about 22
// significant bits of p and stays within fp32-accumulation error of the oracle.  Warp states are merged in shared memory; splits write fp32 partial
// (max, sum, O) triples to a scratch buffer that a second kernel merges in split order.
#include <cstdlib>

#include "affine_imma.cuh"
#include "attention.cuh"

namespace smelt {

namespace {

using namespace attn;

template <int D, int NH, int NU>
__global__ void __launch_bounds__(kAttnThreads, D <= 128 ? 2 : 1) attn_decode_kernel(const AttnDev p) {
    extern __shared__ __align__(16) float smem_f[];
    attn_decode_body<D, NH, NU>(p, smem_f, blockIdx.x, blockIdx.y, blockIdx.z, imma::PdlSync());
}

// Ring units per warp: K and V of one tile when no warp gets a second tile; else three (two in
// flight while one is consumed).  The kernel is bound by the latency of a warp's chain through a
// tile (scores, softmax, weighted sum), not by copies in flight, so up to head_dim 128 the rings
// stay under half the shared memory and two CTAs (sixteen warps) share an SM.
template <int D>
constexpr int ring_units(bool deep) { return !deep ? 2 : D == 64 ? 6 : 3; }
constexpr int ctas_per_sm(int head_dim) { return head_dim <= 128 ? 2 : 1; }

// cos | sin of the current position for the half pairs of a head (analytic full-head RoPE),
// once per token; the attention launches of every layer read it.
__global__ void rope_table_kernel(float* table, int half, float base_log2, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    const int p = threadIdx.x;
    if (p >= half) return;
    int d0, d1, c0i, c1i;
    float c0, s0, c1, s1;
    rope_indices(1, p, half, 2 * half, d0, d1, c0i, c1i);
    rope_trig(p, half, dyn_position(dyn), base_log2, 1, nullptr, nullptr, c0i, c1i, c0, s0, c1, s1);
    table[p] = c0; table[half + p] = s0;
}

// Merge the per-split partials of one (sequence, query head) in split order.
template <int D>
__global__ void attn_merge_kernel(const AttnDev p) {
    __shared__ float s_ml[2 * kMaxSplits];
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(p.dyn)) return;
    merge_partials<D>(p, s_ml, blockIdx.x, 1, threadIdx.x, blockDim.x);
}

// attention_decode_mlx_vector_2pass_2_d256_b128 (Resources/Shaders/attention.metal:1146-1206):
// out = sum_b exp(max_b - M) partial_b / sum_b exp(max_b - M) sum_b over the 128 key blocks of
// one query head, M the largest block maximum; blocks in index order; a head whose total is
// zero keeps the unnormalised sum, as the reference does.
__global__ void attn_mlx_reduce_kernel(const __half* partials, const float* stats, __half* out, int n_q, int D, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int qh = blockIdx.x;
    const float* sums = stats + (size_t)qh * kMlxBlocks;
    const float* maxs = stats + (size_t)n_q * kMlxBlocks + (size_t)qh * kMlxBlocks;
    float M = -3.402823466e+38f;
    for (int b = 0; b < kMlxBlocks; ++b) M = fmaxf(M, maxs[b]);
    float total = 0.f;
    for (int b = 0; b < kMlxBlocks; ++b)
        if (sums[b] != 0.f) total += expf(maxs[b] - M) * sums[b];
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.f;
        for (int b = 0; b < kMlxBlocks; ++b)
            if (sums[b] != 0.f) acc += expf(maxs[b] - M) * __half2float(partials[((size_t)qh * kMlxBlocks + b) * D + d]);
        out[(size_t)qh * D + d] = __float2half_rn(total == 0.f ? acc : acc / total);
    }
}

template <int D, int NH, int NU>
cudaError_t launch_decode_t(const Launch& l, const AttnDev& p) {
    const size_t smem = attn_smem_bytes<D, NH, NU>();
    auto kern = attn_decode_kernel<D, NH, NU>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.nsplits, p.a.n_kv, p.a.batch);
    cfg.blockDim = dim3(kAttnThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (l.pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (p.cluster) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = p.nsplits;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    prefer_max_shared(kern);
    return cudaLaunchKernelEx(&cfg, kern, p);
}

}  // namespace

int attention_max_splits() { return kMaxSplits; }

size_t attention_scratch_bytes(int n_q, int head_dim, int batch, int max_splits) {
    return (size_t)batch * n_q * max_splits * (head_dim + 2) * sizeof(float);
}

cudaError_t launch_rope_table(const Launch& l, float* table, int half, float base_log2) {
    if (half <= 0 || half > 128) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(128);
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = l.pdl ? 1 : 0;
    prefer_max_shared(rope_table_kernel);
    return cudaLaunchKernelEx(&cfg, rope_table_kernel, table, half, base_log2, dev_dyn(l));
}

cudaError_t launch_attention_decode(const Launch& l, const AttnArgs& a) {
    if (a.n_q <= 0 || a.n_kv <= 0 || a.n_q % a.n_kv != 0 || a.batch <= 0) return cudaErrorInvalidValue;
    const int ratio = a.n_q / a.n_kv;
    if (ratio > 16 || (a.head_dim != 64 && a.head_dim != 128 && a.head_dim != 256)) return cudaErrorInvalidValue;
    const uint32_t n_max = a.seq_from_pos ? a.capacity : (a.seq_len < a.capacity ? a.seq_len : a.capacity);
    if (n_max == 0) return cudaErrorInvalidValue;
    const int sm = a.sm_count > 0 ? a.sm_count : 148;
    const int by_len = (int)((n_max + 127u) / 128u);  // at least one 16-key tile per warp and split
    // The grid runs in waves of as many CTAs as are resident at once: the smallest split count
    // within 2 % of the best-filled last wave.
    const int base = a.n_kv * a.batch;
    const long slots = (long)sm * ctas_per_sm(a.head_dim);
    int cap = by_len < kMaxSplits ? by_len : kMaxSplits;
    if (a.mlx_partials) {
        // two-pass pair: the partials go to the record's own buffers, the second record merges
        if (a.batch != 1 || !a.mlx_stats) return cudaErrorInvalidValue;
    } else {
        while (cap > 1 && attention_scratch_bytes(a.n_q, a.head_dim, a.batch, cap) > a.scratch_bytes) --cap;
    }
    auto fill = [&](int n) { const long ctas = (long)n * base; return (double)ctas / (double)(((ctas + slots - 1) / slots) * slots); };
    double best = 0.0;
    for (int n = 1; n <= cap; ++n) best = fill(n) > best ? fill(n) : best;
    int nsplits = 1;
    while (nsplits < cap && fill(nsplits) < best - 0.02) ++nsplits;
    // Short contexts are latency bound: up to 4096 keys, eight splits of a KV head run as one
    // thread-block cluster and merge through distributed shared memory, with no partials in
    // global memory (measured against one tile per warp and the ticket merge: 11.2 against
    // 13.9 us at 4096 keys, batch 1).  Always eight: the key ranges are cut from the live
    // length, so with a fixed split count the summation order, and with it every output bit,
    // is the same whatever capacity the cache was given or has grown to.
    const bool cluster = n_max <= 4096 && by_len >= 2 && !a.mlx_partials;
    if (cluster) nsplits = 8;
    AttnDev p;
    p.a = a;
    p.nsplits = nsplits;
    p.cluster = cluster ? 1 : 0;
    p.part_o = reinterpret_cast<float*>(a.scratch);
    p.part_ml = p.part_o ? p.part_o + (size_t)a.batch * a.n_q * nsplits * a.head_dim : nullptr;
    p.dyn = dev_dyn(l);
    cudaError_t e = cudaSuccess;
    const int nh = ratio > 8 ? 2 : 1;
    const bool deep = (n_max + (uint32_t)nsplits - 1) / (uint32_t)nsplits > (uint32_t)kAttnWarps * 16u;  // some warp walks two tiles or more
#define SMELT_ATTN_CASE(DD)                                                                                             \
    case DD:                                                                                                            \
        e = nh == 1 ? (deep ? launch_decode_t<DD, 1, ring_units<DD>(true)>(l, p) : launch_decode_t<DD, 1, 2>(l, p))     \
                    : (deep ? launch_decode_t<DD, 2, ring_units<DD>(true)>(l, p) : launch_decode_t<DD, 2, 2>(l, p));    \
        break;
    switch (a.head_dim) {
        SMELT_ATTN_CASE(64)
        SMELT_ATTN_CASE(128)
        SMELT_ATTN_CASE(256)
        default: return cudaErrorInvalidValue;
    }
#undef SMELT_ATTN_CASE
    if (e != cudaSuccess || nsplits == 1 || a.counters || cluster || a.mlx_partials) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.batch * a.n_q);
    cfg.blockDim = dim3(a.head_dim < 128 ? 64 : 128);
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = l.pdl ? 1 : 0;
    auto merge = a.head_dim == 64 ? attn_merge_kernel<64> : a.head_dim == 128 ? attn_merge_kernel<128> : attn_merge_kernel<256>;
    prefer_max_shared(merge);
    return cudaLaunchKernelEx(&cfg, merge, p);
}

cudaError_t launch_attention_mlx_reduce(const Launch& l, const __half* partials, const float* stats, __half* out, int n_q, int head_dim) {
    if (n_q <= 0 || head_dim <= 0) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_q);
    cfg.blockDim = dim3(head_dim < 256 ? 128 : 256);
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = l.pdl ? 1 : 0;
    prefer_max_shared(attn_mlx_reduce_kernel);
    return cudaLaunchKernelEx(&cfg, attn_mlx_reduce_kernel, partials, stats, out, n_q, head_dim, dev_dyn(l));
}

}  // namespace smelt
