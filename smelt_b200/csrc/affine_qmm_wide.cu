// Quantised matrix-matrix product for wide batches (prompt chunks; more than 64 rows of X):
// Y[M, R] = X[M, K] . W[R, K]^T with W affine u4, group 64, every K step accumulated in tensor
// memory, so that the packed weights are expanded once per CTA for up to 512 rows of X.
//
// Same reference kernels as affine_qmm.cu (agent_affine_qmm_fixed_batched_full,
// Resources/Shaders/agent_affine_qmm.h:107-316, :360-742).  affine_qmm.cu keeps one accumulator
// slot per quantisation group and applies scale and bias in fp32 when it drains the slot; that
// drain costs one FMA per weight per 64 rows of X and caps the batch a CTA can serve at 64.
// Here the tensor core multiplies the dequantised weight itself, w = scale * q + bias, as TWO
// fp16 operands: hi = half(w) and lo = half(w - hi), w evaluated in fp32 with one FMA.  hi + lo
// carries 22 significant bits of w, so D += A_hi . B + A_lo . B in the fp32 accumulator is within
// 2^-22 of the factored form the matvec family computes, and the accumulator of a (row, batch
// row) pair lives in tensor memory across the whole K loop: 128 lanes x up to 512 columns.
//
// Mapping.  One CTA = 128 weight rows (for the paired forms 64 rows of each matrix: gate | up or
// K | V, so that the SwiGLU epilogue finds both halves in the CTA) x all M <= 512 batch rows, in
// chunks of up to 256 (the MMA's N limit).  Per 64-column block:
//   * warps 0-7: thread (row r, half h) turns its 32 nibbles into hi / lo fp16 and stores them in
//     the K-major, 128-byte-swizzled A_hi / A_lo tiles (two stages); the same threads copy the
//     block's activations, chunk by chunk, from registers loaded one unit ahead into a ring of
//     three swizzled B tiles;
//   * warp 8: one lane waits for the tiles (mbarriers), issues per chunk four K = 16 MMAs with
//     A_hi and four with A_lo into the chunk's columns and commits them to the barriers that
//     free the tiles.
// After the last block the producers read their row's columns with tcgen05.ld and write the
// epilogue (plain, + residual, SwiGLU of the gate | up halves through shared memory, dual).
// Matrices with few row tiles split K over gridDim.y CTAs (fp32 partials, ticket, ordered sum).
// Every wait is bounded: on expiry the CTA sets bit 10 of the error word, drains its copies,
// frees its tensor memory and returns.
//
// What bounds it (ncu at M = 512, gate/up 12288 x 4096: tensor pipe 38 % busy, 59 % while a wave
// runs): shared-memory bandwidth.  Per 64-column block the MMAs read A_hi + A_lo once per chunk and
// the B tile once for hi and once for lo, 192 KB, and the producers store 96 KB: about 137 bytes
// per clock against the SM's 128.  A two-CTA MMA (cta_group::2) would halve the B traffic per SM.
#include "affine_matvec.h"
#include "tcgen05.cuh"

namespace smelt {

namespace {

constexpr int kRows = 128;
constexpr int kBlockCols = 64;
constexpr int kStageCols = 256;
constexpr int kProducers = 256;                          // eight warps (sixteen measured 364 / 217 / 90 us against 334 / 262 / 78 at M = 512: no clear gain)
constexpr int kThreads = kProducers + 32;
constexpr int kRawSliceBytes = 64 + 8 + 8;               // per producer thread and stage: 64 packed bytes + 4 scales + 4 biases
constexpr int kRawStageBytes = kProducers * kRawSliceBytes;
constexpr int kRawStages = 2;
constexpr int kATileBytes = kRows * kBlockCols * 2;      // 16 KB; hi and lo per stage
constexpr int kAStages = 2;
constexpr int kChunk = 256;                              // batch rows per MMA (N)
constexpr int kBTileBytes = kChunk * kBlockCols * 2;     // 32 KB
constexpr int kBSlots = 3;
constexpr int kMaxBatch = 512;

struct WideLayout {
    uint32_t a_tiles, b_tiles, raw, bars, total;
};
__host__ __device__ inline WideLayout wide_layout() {
    WideLayout L;
    uint32_t off = 0;
    L.a_tiles = off; off += kAStages * 2 * kATileBytes;
    L.b_tiles = off; off += kBSlots * kBTileBytes;
    L.raw = off; off += kRawStages * kRawStageBytes;
    L.bars = off; off += 128;
    L.total = off + 1024;  // slack to align the dynamic base to 1024 bytes (the swizzle atom)
    return L;
}

// Eight nibbles of a packed word -> eight weights w = sc * q + bi as fp16 hi / lo pairs in column order.
__device__ __forceinline__ void dequant8(uint32_t word, float sc, float bi, uint32_t (&hi)[4], uint32_t (&lo)[4]) {
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const float q0 = __uint_as_float(((word >> (8 * p)) & 15u) | 0x4B000000u) - 8388608.0f;
        const float q1 = __uint_as_float(((word >> (8 * p + 4)) & 15u) | 0x4B000000u) - 8388608.0f;
        const float w0 = fmaf(q0, sc, bi), w1 = fmaf(q1, sc, bi);
        const __half2 h = __floats2half2_rn(w0, w1);
        const float2 hf = __half22float2(h);
        hi[p] = h2_as_u32(h);
        lo[p] = h2_as_u32(__floats2half2_rn(w0 - hf.x, w1 - hf.y));
    }
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1) affine_qmm_wide_kernel(const AffineArgs a, const int m_pad) {
    constexpr bool kPaired = MODE == kAffineGateUp || MODE == kAffineDual;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const WideLayout L = wide_layout();
    uint64_t* full_a = reinterpret_cast<uint64_t*>(smem + L.bars);  // [2] producers -> issuer
    uint64_t* done_a = full_a + kAStages;                            // [2] tensor core -> producers
    uint64_t* full_b = done_a + kAStages;                            // [3]
    uint64_t* done_b = full_b + kBSlots;                             // [3]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_b + kBSlots);
    uint32_t* s_dead = tmem_slot + 2;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ksplit = (int)gridDim.y, stages_total = a.cols / kStageCols;
    const int st0 = (int)blockIdx.y * stages_total / ksplit, nstages = ((int)blockIdx.y + 1) * stages_total / ksplit - st0;
    const int kb0 = st0 * 4, nblocks = nstages * 4;
    const int groups_total = a.cols / 64;
    const int nchunks = (m_pad + kChunk - 1) / kChunk;           // 1 or 2
    const uint32_t tmem_cols = m_pad <= 32 ? 32u : m_pad <= 64 ? 64u : m_pad <= 128 ? 128u : m_pad <= 256 ? 256u : 512u;

    if (tid == 0) {
        for (int i = 0; i < kAStages; ++i) { mbar_init(&full_a[i], kProducers / 32); mbar_init(&done_a[i], 1); }
        for (int i = 0; i < kBSlots; ++i) { mbar_init(&full_b[i], kProducers / 32); mbar_init(&done_b[i], 1); }
        *s_dead = 0u;
        mbar_fence_init();
    }
    if (warp == kProducers / 32) tmem_alloc(tmem_slot, tmem_cols);

    // this thread's weight row: rows 0-63 of the tile come from matrix 0, rows 64-127 from matrix 1 in the paired forms
    const int r = tid & (kRows - 1), h = (tid >> 7) & 1;
    const bool producer = tid < kProducers;
    const int mat = kPaired ? (r >> 6) : 0;
    const int grow = kPaired ? (int)blockIdx.x * 64 + (r & 63) : (int)blockIdx.x * kRows + r;
    const bool row_ok = producer && grow < a.rows;
    uint8_t* raw_row = smem + L.raw + (size_t)(h * kRows + r) * kRawSliceBytes;
    auto request_stage = [&](int st) {
        if (st < nstages && row_ok) {
            uint8_t* dst = raw_row + (size_t)(st % kRawStages) * kRawStageBytes;
            const uint8_t* src = a.w[mat] + (size_t)grow * (a.cols / 2) + (size_t)(st0 + st) * (kStageCols / 2) + h * 16;
#pragma unroll
            for (int c = 0; c < 4; ++c) cp_async16(dst + c * 16, src + c * 32);
            const size_t g0 = (size_t)grow * groups_total + (size_t)(st0 + st) * 4;
            cp_async8(dst + 64, a.s[mat] + g0);
            cp_async8(dst + 72, a.b[mat] + g0);
        }
        cp_async_commit();
    };
    if (producer) request_stage(0);

    pdl_trigger();
    pdl_wait();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const bool skip = dyn_skip(a.dyn);
    bool dead = false;
    const int units = nblocks * nchunks;

    if (producer && !skip) {
        // B-tile pieces of this thread: piece q -> (batch row n of the chunk, 16-byte piece c of the block)
        uint4 xreg[8];  // one unit ahead (two units ahead measured slower: 389 against 343 us at M = 512)
        auto load_x = [&](int u, uint4 (&dst)[8]) {
            const int kb = u / nchunks, ch = u % nchunks;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int q = tid + kProducers * i, n = ch * kChunk + (q >> 3), c = q & 7;
                dst[i] = (u < units && n < a.batch)
                             ? *reinterpret_cast<const uint4*>(a.x + (size_t)n * a.cols + (size_t)(kb0 + kb) * kBlockCols + c * 8)
                             : make_uint4(0, 0, 0, 0);
            }
        };
        load_x(0, xreg);
        for (int kb = 0; kb < nblocks && !dead; ++kb) {
            const int st = kb >> 2, sub = kb & 3, abuf = kb & 1;
            if (sub == 0) {
                cp_async_wait<0>();  // this thread's copies of stage st have landed
                request_stage(st + 1);
            }
            // ── A_hi / A_lo of the block: wait until the MMAs of block kb - 2 have read the buffer ──
            if (kb >= 2 && !mbar_poll_bounded(&done_a[abuf], (uint32_t)(((kb >> 1) - 1) & 1))) { dead = true; break; }
            {
                const uint8_t* src = raw_row + (size_t)(st % kRawStages) * kRawStageBytes;
                uint4 pw = make_uint4(0, 0, 0, 0);
                float sc = 0.f, bi = 0.f;
                if (row_ok) {
                    pw = *reinterpret_cast<const uint4*>(src + sub * 16);
                    sc = __half2float(*reinterpret_cast<const __half*>(src + 64 + sub * 2));
                    bi = __half2float(*reinterpret_cast<const __half*>(src + 72 + sub * 2));
                }
                uint8_t* a_hi = smem + L.a_tiles + (size_t)(abuf * 2) * kATileBytes + (r >> 3) * 1024 + (r & 7) * 128;
                uint8_t* a_lo = a_hi + kATileBytes;
                const uint32_t words[4] = {pw.x, pw.y, pw.z, pw.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {  // eight columns -> one 16-byte piece of the row in each tile
                    uint32_t hi[4], lo[4];
                    dequant8(words[q], sc, bi, hi, lo);
                    const int piece = ((h * 4 + q) ^ (r & 7)) << 4;
                    *reinterpret_cast<uint4*>(a_hi + piece) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<uint4*>(a_lo + piece) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                }
            }
            // ── the block's activations, chunk by chunk, into the B ring ──
            for (int ch = 0; ch < nchunks && !dead; ++ch) {
                const int u = kb * nchunks + ch, slot = u % kBSlots, use = u / kBSlots;
                if (use >= 1 && !mbar_poll_bounded(&done_b[slot], (uint32_t)((use - 1) & 1))) { dead = true; break; }
                uint8_t* b_tile = smem + L.b_tiles + (size_t)slot * kBTileBytes;
                const int n_cols = min(kChunk, m_pad - ch * kChunk);  // rows of the tile the MMA reads
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int q = tid + kProducers * i, n = q >> 3, c = q & 7;
                    if (n < n_cols) *reinterpret_cast<uint4*>(b_tile + (n >> 3) * 1024 + (n & 7) * 128 + ((c ^ (n & 7)) << 4)) = xreg[i];
                }
                load_x(u + 1, xreg);
                fence_async_smem();  // generic-proxy stores -> visible to the tensor core's async-proxy reads
                __syncwarp();
                if (lane == 0) {
                    if (ch == 0) mbar_arrive(&full_a[abuf]);
                    mbar_arrive(&full_b[slot]);
                }
            }
        }
        // ── every MMA has completed once the last block's commit has arrived ──
        if (!dead && !mbar_poll_bounded(&done_a[(nblocks - 1) & 1], (uint32_t)(((nblocks - 1) >> 1) & 1))) dead = true;
        cp_async_wait<0>();
        // a wait that gave up in one thread stops the whole CTA: the barriers below need every producer
        if (dead) atomicOr(s_dead, 1u);
        asm volatile("bar.sync 1, %0;" ::"r"(kProducers) : "memory");
        dead = *reinterpret_cast<volatile uint32_t*>(s_dead) != 0u;
        tc_fence_after();
        const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const int half_cols = m_pad / 2;                    // this thread's batch rows: [h * half_cols, +half_cols)
        bool finish = !dead;
        if (ksplit > 1 && !dead) {
            float* mine = a.part_scratch + ((size_t)blockIdx.x * ksplit + blockIdx.y) * ((size_t)m_pad * kRows);
            for (int c0 = 0; c0 < half_cols; c0 += 8) {
                uint32_t v[8];
                tmem_ld8(lane_base + (uint32_t)(h * half_cols + c0), v);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 8; ++j) __stcg(mine + (size_t)(h * half_cols + c0 + j) * kRows + r, __uint_as_float(v[j]));
            }
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"r"(kProducers) : "memory");
            if (tid == 0) *tmem_slot = (uint32_t)atomicAdd(a.part_counters + blockIdx.x, 1);  // the allocation address has been read by everyone
            asm volatile("bar.sync 1, %0;" ::"r"(kProducers) : "memory");
            finish = (int)*tmem_slot == ksplit - 1;
            if (finish) {
                __threadfence();
                if (tid == 0) a.part_counters[blockIdx.x] = 0;
            }
        }
        if (finish) {
            float* ex = reinterpret_cast<float*>(smem + L.a_tiles);  // [h][64 rows][8] exchange of the up / second half, after all MMAs
            for (int c0 = 0; c0 < half_cols; c0 += 8) {
                float v[8];
                if (ksplit > 1) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = 0.f;
                    for (int z = 0; z < ksplit; ++z) {
                        const float* p = a.part_scratch + ((size_t)blockIdx.x * ksplit + z) * ((size_t)m_pad * kRows);
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[j] += __ldcg(p + (size_t)(h * half_cols + c0 + j) * kRows + r);
                    }
                } else {
                    uint32_t u[8];
                    tmem_ld8(lane_base + (uint32_t)(h * half_cols + c0), u);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(u[j]);
                }
                if (MODE == kAffineGateUp) {
                    if (r >= 64) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) ex[(h * 64 + (r - 64)) * 8 + j] = v[j];
                    }
                    asm volatile("bar.sync 1, %0;" ::"r"(kProducers) : "memory");
                    if (r < 64 && grow < a.rows) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const int n = h * half_cols + c0 + j;
                            if (n < a.batch) {
                                const float g = v[j], up = ex[(h * 64 + r) * 8 + j];
                                a.y[(size_t)n * a.rows + grow] = __float2half_rn(g / (1.0f + expf(-g)) * up);  // lut_matvec.metal:2228
                            }
                        }
                    }
                    asm volatile("bar.sync 1, %0;" ::"r"(kProducers) : "memory");
                } else if (grow < a.rows) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int n = h * half_cols + c0 + j;
                        if (n >= a.batch) continue;
                        const size_t o = (size_t)n * a.rows + grow;
                        if (MODE == kAffinePlain) a.y[o] = __float2half_rn(v[j]);
                        else if (MODE == kAffineAdd) a.y[o] = __hadd(__float2half_rn(v[j]), a.residual[o]);  // lut_matvec.metal:1802-1803
                        else (mat == 0 ? a.y : a.y2)[o] = __float2half_rn(v[j]);
                    }
                }
            }
        }
    } else if (warp == kProducers / 32 && !skip) {
        // ── issuer: one lane feeds the tensor core ──
        if (lane == 0) {
            for (int kb = 0; kb < nblocks && !dead; ++kb) {
                const int abuf = kb & 1;
                if (!mbar_poll_bounded(&full_a[abuf], (uint32_t)((kb >> 1) & 1))) { dead = true; break; }
                const uint32_t a_hi = smem_u32(smem + L.a_tiles + (size_t)(abuf * 2) * kATileBytes), a_lo = a_hi + kATileBytes;
                for (int ch = 0; ch < nchunks; ++ch) {
                    const int u = kb * nchunks + ch, slot = u % kBSlots, use = u / kBSlots;
                    if (!mbar_poll_bounded(&full_b[slot], (uint32_t)(use & 1))) { dead = true; break; }
                    tc_fence_after();
                    const int n_cols = min(kChunk, m_pad - ch * kChunk);  // a multiple of 16
                    const uint32_t idesc = (1u << 4) | ((uint32_t)(n_cols >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);  // f32 accumulate, f16 x f16, K-major both
                    const uint32_t b_addr = smem_u32(smem + L.b_tiles + (size_t)slot * kBTileBytes);
                    const uint32_t d = tmem_base + (uint32_t)(ch * kChunk);
#pragma unroll
                    for (int k = 0; k < kBlockCols / 16; ++k) {
                        umma_f16(d, smem_desc_sw128(a_hi + k * 32), smem_desc_sw128(b_addr + k * 32), idesc, (kb != 0 || k != 0) ? 1u : 0u);
                        umma_f16(d, smem_desc_sw128(a_lo + k * 32), smem_desc_sw128(b_addr + k * 32), idesc, 1u);
                    }
                    umma_commit(&done_b[slot]);  // arrives when the MMAs above are complete: the B slot is free
                }
                if (!dead) umma_commit(&done_a[abuf]);
            }
        }
        dead = __shfl_sync(0xffffffffu, dead ? 1 : 0, 0) != 0;
    }
    if (dead && a.err && lane == 0) atomicOr(a.err, 0x400u);
    cp_async_wait<0>();
    tc_fence_before();
    __syncthreads();
    if (warp == kProducers / 32) {
        tc_fence_after();
        tmem_dealloc(tmem_base, tmem_cols);
    }
}

template <int MODE>
cudaError_t launch_wide_t(const Launch& l, AffineArgs a) {
    constexpr bool kPaired = MODE == kAffineGateUp || MODE == kAffineDual;
    const WideLayout L = wide_layout();
    a.dyn = dev_dyn(l);
    auto kern = affine_qmm_wide_kernel<MODE>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L.total);
    if (e != cudaSuccess) return e;
    const int m_pad = (a.batch + 31) & ~31;  // a multiple of 32: each half of the columns a multiple of 16 (the MMA's N step) and of 8 (the epilogue's)
    const int tiles = kPaired ? (a.rows + 63) / 64 : (a.rows + kRows - 1) / kRows, stages = a.cols / kStageCols;
    const int sm = a.sm_count > 0 ? a.sm_count : 148;
    int ksplit = sm / tiles;
    if (ksplit > stages / 2) ksplit = stages / 2;
    if (ksplit < 1 || !a.part_scratch || !a.part_counters || tiles > 4096) ksplit = 1;
    while (ksplit > 1 && (size_t)tiles * ksplit * m_pad * kRows * sizeof(float) > a.part_scratch_bytes) --ksplit;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles, ksplit, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = L.total;
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = l.pdl ? 1 : 0;
    prefer_max_shared(kern);
    return cudaLaunchKernelEx(&cfg, kern, a, m_pad);
}

}  // namespace

// Launches the wide QMM when the shape is eligible (group 64, more than 64 batch rows, cols a
// multiple of 256, 16-byte aligned operands, one tensor per matrix, no folded norm, paired forms
// with a multiple of 64 rows); batches beyond 512 rows run as passes of 512.
cudaError_t launch_affine_qmm_wide(const Launch& l, int mode, const AffineArgs& a, int group, bool* handled) {
    *handled = false;
    if (group != 64 || a.batch <= 64 || a.cols % kStageCols != 0 || a.norm_w || a.nseg > 1) return cudaSuccess;
    if (wide_layout().total > 227u * 1024u) return cudaSuccess;
    const int nw = (mode == kAffineGateUp || mode == kAffineDual) ? 2 : 1;
    if (nw == 2 && a.rows % 64 != 0) return cudaSuccess;
    for (int s = 0; s < nw; ++s)
        if ((reinterpret_cast<uintptr_t>(a.w[s]) & 15u) || (reinterpret_cast<uintptr_t>(a.s[s]) & 7u) || (reinterpret_cast<uintptr_t>(a.b[s]) & 7u)) return cudaSuccess;
    if (reinterpret_cast<uintptr_t>(a.x) & 15u) return cudaSuccess;
    if (((size_t)(a.cols / 64) * 2) % 8 != 0) return cudaSuccess;  // a row's scales start 8-byte aligned
    for (int b0 = 0; b0 < a.batch; b0 += kMaxBatch) {
        AffineArgs p = a;
        p.batch = a.batch - b0 < kMaxBatch ? a.batch - b0 : kMaxBatch;
        p.x = a.x + (size_t)b0 * a.cols;
        p.y = a.y + (size_t)b0 * a.rows;
        if (a.y2) p.y2 = a.y2 + (size_t)b0 * a.rows;
        if (a.residual) p.residual = a.residual + (size_t)b0 * a.rows;
        cudaError_t e;
        switch (mode) {
            case kAffinePlain: e = launch_wide_t<kAffinePlain>(l, p); break;
            case kAffineAdd: e = launch_wide_t<kAffineAdd>(l, p); break;
            case kAffineGateUp: e = launch_wide_t<kAffineGateUp>(l, p); break;
            case kAffineDual: e = launch_wide_t<kAffineDual>(l, p); break;
            default: return cudaErrorInvalidValue;
        }
        if (e != cudaSuccess) return e;
    }
    *handled = true;
    return cudaSuccess;
}

}  // namespace smelt
