// Quantised matrix-matrix product for batches of seventeen rows and more (decode at large batch,
// prompt chunks; up to sixteen rows the mma.sync streaming kernels measure as fast or faster): Y[M, R] = X[M, K] . W[R, K]^T with W affine u4, group 64, on the fifth-generation
// tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// Replaces agent_affine_qmm_fixed_batched_full and its fused gate/up form
// (Resources/Shaders/agent_affine_qmm.h:107-316, :360-742; wrappers
// Resources/Shaders/lut_matvec.metal:6519-6545, :6615-6635): a tile GEMM over the packed weights
// with fp16 activations and fp32 accumulation.  The arithmetic is the matvec family's factored
// form (Tests/SmeltCompilerTests/Helpers/MetalKernelTestSupport.swift:396-428): per group of 64
// columns acc += scale * sum(nibble * x) + bias * sum(x).  The tensor core multiplies the exact
// nibble values (fp16 integers) with the activations, one group per accumulator slot; scale
// and bias are applied in fp32 when the slot is drained, so no weight is ever rounded to fp16.
// The epilogues are those of the matvec family: half(acc), half(acc) + residual,
// half(silu(gate) * up) with fp32 gate / up (lut_matvec.metal:1802-1803, :2228), and the dual form.
//
// Mapping.  The weight rows are the MMA's M (128 rows per CTA), the batch its N (16, 32 or 64), so a
// 128 x N fp32 accumulator per group and matrix lives in tensor memory (four slots rotate)
// and the 4-bit weights, by far the larger operand, cross HBM once per 64 batch rows.
//   * Warps 0-7 produce and drain.  Thread (row r, half h) owns half a weight row: it copies its
//     own 64 packed bytes of every 256-column stage (and the row's scales / biases) with
//     cp.async into a ring, so it only ever waits for its own copies; turns 32 nibbles per
//     64-column block into fp16 integers and stores them as the K-major, 128-byte-swizzled A
//     tile the tensor core reads.  The activations of the block (B tile, X rows K-major) and
//     their per-row sums are staged by the same threads from registers loaded one block ahead.
//     Then the thread drains the previous block's accumulator slot: tensor-memory lane r is
//     weight row r, so scale and bias are per-thread scalars.
//   * Warp 8 issues.  One lane waits for a block's tiles (mbarrier), issues the four K = 16
//     tcgen05.mma of the block per matrix into the block's slot and commits them to the
//     barrier the drain waits on.
// Every wait is bounded: a barrier that does not complete sets bit 10 of the error word and
// the CTA drains its copies, frees its tensor memory and leaves.
#include "affine_matvec.h"
#include "tcgen05.cuh"

namespace smelt {

namespace {

constexpr int kRowsPerCta = 128;
constexpr int kBlockCols = 64;                 // one quantisation group = one A / B tile along K
constexpr int kStageCols = 256;                // packed columns per cp.async stage
__host__ __device__ constexpr int raw_stages(int nw) { return nw == 2 ? 3 : 4; }  // cp.async ring depth (all but one in flight), as shared memory allows
constexpr int kTileStages = 2;                 // A / B tile buffers
constexpr int kProducers = 256;                // eight warps: two threads per weight row (sixteen warps measured slower: the loop is bound by instruction issue)
constexpr int kThreads = kProducers + 32;
// Raw stage of one matrix: one 80-byte slice per producer thread (row r, half h), at (h * 128 + r) * 80:
// its 64 packed bytes (the 16-byte pieces it unpacks, block by block) + the row's 4 scales + 4 biases.
constexpr int kRawSliceBytes = 64 + 8 + 8;
constexpr int kRawStageBytes = kProducers * kRawSliceBytes;
constexpr int kATileBytes = kRowsPerCta * kBlockCols * 2;                // 16 KB

struct QmmLayout {
    uint32_t a_tiles, b_tiles, raw, xsum, bars, total;
};

__host__ __device__ inline QmmLayout qmm_layout(int nw, int nb) {
    QmmLayout L;
    uint32_t off = 0;
    L.a_tiles = off; off += (uint32_t)(kTileStages * nw * kATileBytes);
    L.b_tiles = off; off += (uint32_t)(kTileStages * nb * kBlockCols * 2);
    L.raw = off; off += (uint32_t)(raw_stages(nw) * nw * kRawStageBytes);
    L.xsum = off; off += 8u * (uint32_t)nb * 4u;   // [block & 7][batch row]
    L.bars = off; off += 128;
    L.total = off + 1024;  // slack to align the dynamic base to 1024 bytes (the swizzle atom)
    return L;
}

// Eight nibbles of a packed word (columns c .. c+7, low nibble first) as four half2 of exact
// integers in column order {c, c+1}, {c+2, c+3}, {c+4, c+5}, {c+6, c+7}.
__device__ __forceinline__ void nibbles_to_half(uint32_t w, uint32_t (&p)[4]) {
    const uint32_t kMagic = 0x64006400u;                       // half2(1024, 1024)
    const __half2 k1024 = u32_as_h2(0x64006400u), k16th = u32_as_h2(0x2C002C00u), km64 = u32_as_h2(0xD400D400u);
    const uint32_t w2 = w >> 8;
    const uint32_t n04 = h2_as_u32(__hsub2(u32_as_h2(lop3_and_or(w, 0x000F000Fu, kMagic)), k1024));          // {n0, n4}
    const uint32_t n15 = h2_as_u32(__hfma2(u32_as_h2(lop3_and_or(w, 0x00F000F0u, kMagic)), k16th, km64));    // {n1, n5}
    const uint32_t n26 = h2_as_u32(__hsub2(u32_as_h2(lop3_and_or(w2, 0x000F000Fu, kMagic)), k1024));         // {n2, n6}
    const uint32_t n37 = h2_as_u32(__hfma2(u32_as_h2(lop3_and_or(w2, 0x00F000F0u, kMagic)), k16th, km64));   // {n3, n7}
    p[0] = __byte_perm(n04, n15, 0x5410);  // {n0, n1}
    p[1] = __byte_perm(n26, n37, 0x5410);  // {n2, n3}
    p[2] = __byte_perm(n04, n15, 0x7632);  // {n4, n5}
    p[3] = __byte_perm(n26, n37, 0x7632);  // {n6, n7}
}

template <int MODE, int NB>
__global__ void __launch_bounds__(kThreads, 1) affine_qmm_kernel(const AffineArgs a) {
    constexpr int NW = (MODE == kAffineGateUp || MODE == kAffineDual) ? 2 : 1;
    constexpr int kRawStages = raw_stages(NW);
    constexpr int XCH = (NB * 8 + kProducers - 1) / kProducers;  // 16-byte chunks of the B tile per producer thread
    constexpr int CPT = NB / 2;                                   // accumulator columns (batch rows) a thread drains
    constexpr uint32_t kSlotCols = NW * NB;
    constexpr uint32_t kTmemCols = 4 * kSlotCols < 32 ? 32 : 4 * kSlotCols;  // four slots; a power of two, at most 512
    constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(kRowsPerCta >> 4) << 24);  // f32 accumulate, f16 x f16, K-major both
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const QmmLayout L = qmm_layout(NW, NB);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L.bars);      // [2]: producers -> issuer (tiles of a block are written)
    uint64_t* done_bar = full_bar + kTileStages;                          // [2]: tensor core -> producers (the block's MMAs are complete)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + kTileStages);
    uint32_t* s_dead = tmem_slot + 2;
    float* xsum = reinterpret_cast<float*>(smem + L.xsum);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row0 = (int)blockIdx.x * kRowsPerCta;
    // K is split across gridDim.y CTAs at raw-stage (256-column) granularity: this CTA owns stages
    // [st0, st0 + nstages), i.e. blocks kb0 ... of the row; lb counts its own blocks from zero.
    const int ksplit = (int)gridDim.y, stages_total = a.cols / kStageCols;
    const int st0 = (int)blockIdx.y * stages_total / ksplit, nstages = ((int)blockIdx.y + 1) * stages_total / ksplit - st0;
    const int kb0 = st0 * 4, nblocks = nstages * 4;
    const int groups_total = a.cols / 64;

    if (tid == 0) {
        for (int i = 0; i < kTileStages; ++i) { mbar_init(&full_bar[i], kProducers / 32); mbar_init(&done_bar[i], 1); }
        *s_dead = 0u;
        mbar_fence_init();
    }
    if (warp == kProducers / 32) {  // the issuing warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    // ── producers: request the first raw stages before anything depends on the previous kernel ──
    const int r = tid & (kRowsPerCta - 1), h = (tid >> 7) & 1;
    const bool producer = tid < kProducers;
    const bool row_ok = producer && row0 + r < a.rows;
    uint8_t* raw_row = smem + L.raw + (size_t)(h * kRowsPerCta + r) * kRawSliceBytes;  // + (stage * NW + s) * kRawStageBytes
    auto request_stage = [&](int st) {
        if (st < nstages && row_ok) {
            uint8_t* dst = raw_row + (size_t)((st % kRawStages) * NW) * kRawStageBytes;
#pragma unroll
            for (int s = 0; s < NW; ++s) {
                // block c of the stage: this thread's 16 packed bytes (32 columns) are bytes c * 32 + h * 16 of the row's 128
                const uint8_t* src = a.w[s] + (size_t)(row0 + r) * (a.cols / 2) + (size_t)(st0 + st) * (kStageCols / 2) + h * 16;
#pragma unroll
                for (int c = 0; c < 4; ++c) cp_async16(dst + s * kRawStageBytes + c * 16, src + c * 32);
                const size_t g0 = (size_t)(row0 + r) * groups_total + (size_t)(st0 + st) * 4;  // the row's four groups of this stage
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst + s * kRawStageBytes + 64)), "l"(a.s[s] + g0) : "memory");
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst + s * kRawStageBytes + 72)), "l"(a.b[s] + g0) : "memory");
            }
        }
        cp_async_commit();
    };
    if (producer) {
#pragma unroll
        for (int i = 0; i < kRawStages - 1; ++i) request_stage(i);
    }

    pdl_trigger();
    pdl_wait();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const bool skip = dyn_skip(a.dyn);
    bool dead = false;  // a bounded wait gave up: stop waiting, drain the copies, free, leave

    if (producer && !skip) {
        float acc[NW][CPT];
#pragma unroll
        for (int s = 0; s < NW; ++s)
#pragma unroll
            for (int j = 0; j < CPT; ++j) acc[s][j] = 0.f;
        float sc_hist[2][NW], bi_hist[2][NW];  // scale / bias of this thread's row for blocks kb - 1 and kb - 2
#pragma unroll
        for (int s = 0; s < NW; ++s) sc_hist[0][s] = sc_hist[1][s] = bi_hist[0][s] = bi_hist[1][s] = 0.f;
        const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        // Adds block kb's accumulator slot into the registers: acc += scale * dot + bias * xsum.
        // The caller has seen done_bar of block kb complete.
        auto drain = [&](int kb, const float (&scv)[NW], const float (&biv)[NW]) {
            tc_fence_after();
            const float* xs = xsum + (kb & 7) * NB + h * CPT;
            constexpr int CW = CPT < 8 ? 4 : 8;  // columns per tensor-memory load
#pragma unroll
            for (int c0 = 0; c0 < CPT; c0 += CW) {
                uint32_t v[NW][8];
#pragma unroll
                for (int s = 0; s < NW; ++s) {
                    const uint32_t taddr = lane_base + (uint32_t)((kb & 3) * kSlotCols + s * NB + h * CPT + c0);
                    if (CW == 8) tmem_ld8(taddr, v[s]);
                    else asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v[s][0]), "=r"(v[s][1]), "=r"(v[s][2]), "=r"(v[s][3]) : "r"(taddr) : "memory");
                }
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < CW; ++j) {
                    const float x = xs[c0 + j];
#pragma unroll
                    for (int s = 0; s < NW; ++s) acc[s][c0 + j] = fmaf(biv[s], x, fmaf(scv[s], __uint_as_float(v[s][j]), acc[s][c0 + j]));
                }
            }
            tc_fence_before();
        };
        auto wait_done = [&](int kb) {
            if (!mbar_poll_bounded(&done_bar[kb & 1], (uint32_t)((kb >> 1) & 1))) dead = true;
        };
        // B tile chunks of this thread: chunk q -> (batch row n, 16-byte chunk c of the block)
        uint4 xreg[XCH];
        auto load_x = [&](int kb) {
#pragma unroll
            for (int i = 0; i < XCH; ++i) {
                const int q = tid + kProducers * i, n = q >> 3, c = q & 7;
                xreg[i] = (q < NB * 8 && n < a.batch && kb < nblocks)
                              ? *reinterpret_cast<const uint4*>(a.x + (size_t)n * a.cols + (size_t)(kb0 + kb) * kBlockCols + c * 8)
                              : make_uint4(0, 0, 0, 0);
            }
        };
        load_x(0);
        for (int kb = 0; kb < nblocks && !dead; ++kb) {
            const int st = kb >> 2, sub = kb & 3;  // raw stage and block within it
            if (sub == 0) {
                cp_async_wait<kRawStages - 2>();  // this thread's copies of stage st have landed
                request_stage(st + kRawStages - 1);
            }
            const int buf = kb & 1;
            if (kb >= 2) { wait_done(kb - 2); if (dead) break; }  // block kb - 2 has read these tile buffers; its slot is drained below
            // ── this thread's 32 columns of the block as fp16 integers into the A tile(s) ──
            const uint8_t* src = raw_row + (size_t)((st % kRawStages) * NW) * kRawStageBytes;
            uint8_t* a_row = smem + L.a_tiles + (size_t)(buf * NW) * kATileBytes + (r >> 3) * 1024 + (r & 7) * 128;
            float sc[NW], bi[NW];
#pragma unroll
            for (int s = 0; s < NW; ++s) {
                uint4 pw = make_uint4(0, 0, 0, 0);
                sc[s] = bi[s] = 0.f;
                if (row_ok) {
                    pw = *reinterpret_cast<const uint4*>(src + s * kRawStageBytes + sub * 16);
                    sc[s] = __half2float(*reinterpret_cast<const __half*>(src + s * kRawStageBytes + 64 + sub * 2));
                    bi[s] = __half2float(*reinterpret_cast<const __half*>(src + s * kRawStageBytes + 72 + sub * 2));
                }
                const uint32_t words[4] = {pw.x, pw.y, pw.z, pw.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {  // eight columns -> one 16-byte chunk of the row
                    uint32_t p[4];
                    nibbles_to_half(words[q], p);
                    const int chunk = h * 4 + q;
                    *reinterpret_cast<uint4*>(a_row + s * kATileBytes + ((chunk ^ (r & 7)) << 4)) = make_uint4(p[0], p[1], p[2], p[3]);
                }
            }
            // ── the block's activations into the B tile, their sums per batch row beside it ──
            uint8_t* b_tile = smem + L.b_tiles + (size_t)buf * (NB * kBlockCols * 2);
            if (warp * 32 < NB * 8)  // the warps that hold B-tile chunks (warp-uniform)
#pragma unroll
            for (int i = 0; i < XCH; ++i) {
                const int q = tid + kProducers * i, n = q >> 3, c = q & 7;
                const uint32_t u[4] = {xreg[i].x, xreg[i].y, xreg[i].z, xreg[i].w};
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(u32_as_h2(u[j]));
                    sum += f.x + f.y;
                }
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                if (q < NB * 8) {
                    *reinterpret_cast<uint4*>(b_tile + (n >> 3) * 1024 + (n & 7) * 128 + ((c ^ (n & 7)) << 4)) = xreg[i];
                    if (c == 0) xsum[(kb & 7) * NB + n] = sum;
                }
            }
            if (warp * 32 < NB * 8) load_x(kb + 1);
            fence_async_smem();  // generic-proxy stores above -> visible to the tensor core's async-proxy reads
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_bar[buf]);
            if (kb >= 2) drain(kb - 2, sc_hist[1], bi_hist[1]);  // a whole block behind the tensor core: no stall
#pragma unroll
            for (int s = 0; s < NW; ++s) { sc_hist[1][s] = sc_hist[0][s]; bi_hist[1][s] = bi_hist[0][s]; sc_hist[0][s] = sc[s]; bi_hist[0][s] = bi[s]; }
        }
        if (!dead && nblocks >= 2) { wait_done(nblocks - 2); if (!dead) drain(nblocks - 2, sc_hist[1], bi_hist[1]); }
        if (!dead) { wait_done(nblocks - 1); if (!dead) drain(nblocks - 1, sc_hist[0], bi_hist[0]); }
        cp_async_wait<0>();
        // a wait that gave up in one thread stops the whole CTA: the barriers below need every producer
        if (dead) atomicOr(s_dead, 1u);
        asm volatile("bar.sync 1, %0;" ::"r"(kProducers) : "memory");
        dead = *reinterpret_cast<volatile uint32_t*>(s_dead) != 0u;
        // ── epilogue: this thread holds row r, batch rows h * CPT ... ──
        const int row = row0 + r;
        bool finish = !dead;
        if (ksplit > 1 && !dead) {
            // K split across CTAs: every CTA leaves its fp32 sums in the scratch, the last one of
            // the row tile to arrive (ticket) adds them in split order and writes the tile
            float* mine = a.part_scratch + (((size_t)blockIdx.x * ksplit + blockIdx.y) * NW) * (NB * kRowsPerCta);
#pragma unroll
            for (int s = 0; s < NW; ++s)
#pragma unroll
                for (int j = 0; j < CPT; ++j) __stcg(mine + ((size_t)s * NB + h * CPT + j) * kRowsPerCta + r, acc[s][j]);
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"r"(kProducers) : "memory");  // the producer warps only
            if (tid == 0) *tmem_slot = (uint32_t)atomicAdd(a.part_counters + blockIdx.x, 1);  // the allocation address has been read by everyone
            asm volatile("bar.sync 1, %0;" ::"r"(kProducers) : "memory");
            finish = (int)*tmem_slot == ksplit - 1;
            if (finish) {
                __threadfence();
                if (tid == 0) a.part_counters[blockIdx.x] = 0;  // the next launch finds every counter at zero
#pragma unroll
                for (int s = 0; s < NW; ++s)
#pragma unroll
                    for (int j = 0; j < CPT; ++j) acc[s][j] = 0.f;
                for (int z = 0; z < ksplit; ++z) {
                    const float* p = a.part_scratch + (((size_t)blockIdx.x * ksplit + z) * NW) * (NB * kRowsPerCta);
#pragma unroll
                    for (int s = 0; s < NW; ++s)
#pragma unroll
                        for (int j = 0; j < CPT; ++j) acc[s][j] += __ldcg(p + ((size_t)s * NB + h * CPT + j) * kRowsPerCta + r);
                }
            }
        }
        if (finish && row < a.rows) {
#pragma unroll
            for (int j = 0; j < CPT; ++j) {
                const int n = h * CPT + j;
                if (n < a.batch) {
                    const size_t o = (size_t)n * a.rows + row;
                    const float x0 = acc[0][j];
                    if (MODE == kAffinePlain) a.y[o] = __float2half_rn(x0);
                    else if (MODE == kAffineAdd) a.y[o] = __hadd(__float2half_rn(x0), a.residual[o]);
                    else if (MODE == kAffineGateUp) a.y[o] = __float2half_rn(x0 / (1.0f + expf(-x0)) * acc[NW - 1][j]);
                    else { a.y[o] = __float2half_rn(x0); a.y2[o] = __float2half_rn(acc[NW - 1][j]); }
                }
            }
        }
    } else if (warp == kProducers / 32 && !skip) {
        // ── issuer: one lane feeds the tensor core ──
        if (lane == 0) {
            for (int kb = 0; kb < nblocks; ++kb) {
                const int buf = kb & 1;
                // every producer warp has arrived: the tiles are written, and slot kb & 3 was drained of block kb - 4
                if (!mbar_poll_bounded(&full_bar[buf], (uint32_t)((kb >> 1) & 1))) { dead = true; break; }
                tc_fence_after();
                const uint32_t b_addr = smem_u32(smem + L.b_tiles + (size_t)buf * (NB * kBlockCols * 2));
#pragma unroll
                for (int s = 0; s < NW; ++s) {
                    const uint32_t a_addr = smem_u32(smem + L.a_tiles + (size_t)(buf * NW + s) * kATileBytes);
#pragma unroll
                    for (int k = 0; k < kBlockCols / 16; ++k)
                        umma_f16(tmem_base + (uint32_t)((kb & 3) * kSlotCols + s * NB), smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), kIdesc,
                                 k != 0 ? 1u : 0u);
                }
                umma_commit(&done_bar[buf]);  // arrives when the MMAs above are complete
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

template <int MODE, int NB>
cudaError_t launch_qmm_t(const Launch& l, AffineArgs a) {
    constexpr int NW = (MODE == kAffineGateUp || MODE == kAffineDual) ? 2 : 1;
    const QmmLayout L = qmm_layout(NW, NB);
    if (L.total > 227u * 1024u) return cudaErrorNotSupported;
    a.dyn = dev_dyn(l);
    auto kern = affine_qmm_kernel<MODE, NB>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L.total);
    if (e != cudaSuccess) return e;
    // Row tiles rarely fill the GPU (a 2048-row matrix has 16): K is split across CTAs so that about
    // every SM gets one, as far as the hand-over scratch allows and at least two stages per CTA.
    const int tiles = (a.rows + kRowsPerCta - 1) / kRowsPerCta, stages = a.cols / kStageCols;
    const int sm = a.sm_count > 0 ? a.sm_count : 148;
    int ksplit = sm / tiles;
    if (ksplit > stages / 2) ksplit = stages / 2;
    if (ksplit < 1 || !a.part_scratch || !a.part_counters || tiles > 4096) ksplit = 1;
    while (ksplit > 1 && (size_t)tiles * ksplit * NW * NB * kRowsPerCta * sizeof(float) > a.part_scratch_bytes) --ksplit;
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
    return cudaLaunchKernelEx(&cfg, kern, a);
}

template <int MODE>
cudaError_t launch_qmm_mode(const Launch& l, const AffineArgs& a) {
    if (a.batch <= 16) return launch_qmm_t<MODE, 16>(l, a);
    if (a.batch <= 32) return launch_qmm_t<MODE, 32>(l, a);
    return launch_qmm_t<MODE, 64>(l, a);
}

}  // namespace

// Launches the tensor-memory QMM when the shape is eligible (group 64, batch >= 17, cols a multiple
// of 256, 16-byte aligned operands, one tensor per matrix, no folded norm); batches beyond 64 rows
// run as passes of 64.  *handled tells the caller whether it did.
cudaError_t launch_affine_qmm(const Launch& l, int mode, const AffineArgs& a, int group, bool* handled) {
    *handled = false;
    if (group != 64 || a.batch < 17 || a.cols % kStageCols != 0 || a.norm_w || a.nseg > 1) return cudaSuccess;
    const int nw = (mode == kAffineGateUp || mode == kAffineDual) ? 2 : 1;
    for (int s = 0; s < nw; ++s)
        if ((reinterpret_cast<uintptr_t>(a.w[s]) & 15u) || (reinterpret_cast<uintptr_t>(a.s[s]) & 7u) || (reinterpret_cast<uintptr_t>(a.b[s]) & 7u)) return cudaSuccess;
    if (reinterpret_cast<uintptr_t>(a.x) & 15u) return cudaSuccess;
    if (((size_t)(a.cols / 64) * 2) % 8 != 0) return cudaSuccess;  // a row's scales start 8-byte aligned
    for (int b0 = 0; b0 < a.batch; b0 += 64) {
        AffineArgs p = a;
        p.batch = a.batch - b0 < 64 ? a.batch - b0 : 64;
        p.x = a.x + (size_t)b0 * a.cols;
        p.y = a.y + (size_t)b0 * a.rows;
        if (a.y2) p.y2 = a.y2 + (size_t)b0 * a.rows;
        if (a.residual) p.residual = a.residual + (size_t)b0 * a.rows;
        cudaError_t e;
        switch (mode) {
            case kAffinePlain: e = launch_qmm_mode<kAffinePlain>(l, p); break;
            case kAffineAdd: e = launch_qmm_mode<kAffineAdd>(l, p); break;
            case kAffineGateUp: e = launch_qmm_mode<kAffineGateUp>(l, p); break;
            case kAffineDual: e = launch_qmm_mode<kAffineDual>(l, p); break;
            default: return cudaErrorInvalidValue;
        }
        if (e == cudaErrorNotSupported) return b0 == 0 ? cudaSuccess : e;
        if (e != cudaSuccess) return e;
    }
    *handled = true;
    return cudaSuccess;
}

}  // namespace smelt
