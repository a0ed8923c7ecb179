// Tensor-parallel communicator: NCCL over NVLink, one process per GPU.
//
// The reference is single-device (one MTLDevice, one command queue,
// Sources/SmeltRuntime/SmeltRuntime.swift:522-523), so this file has no counterpart there.
// NCCL is bound at run time with dlopen so that single-GPU users carry no NCCL dependency;
// when a process has already loaded NCCL (for example through torch) the same copy is reused.
#include <dlfcn.h>

#include <cstring>
#include <new>

#include "runtime.h"

namespace smelt {

namespace {

typedef struct { char internal[128]; } nccl_unique_id;
static_assert(sizeof(nccl_unique_id) == SMELT_TP_ID_BYTES, "ncclUniqueId is 128 bytes");
typedef void* nccl_comm_t;
enum { kNcclFloat16 = 6, kNcclSum = 0 };

struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(nccl_unique_id*) = nullptr;
    int (*CommInitRank)(nccl_comm_t*, int, nccl_unique_id, int) = nullptr;
    int (*CommDestroy)(nccl_comm_t) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
};

NcclApi& api() {
    static NcclApi a;
    if (a.handle) return a;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        a.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (a.handle) break;
    }
    if (!a.handle) return a;
    a.GetUniqueId = (int (*)(nccl_unique_id*))dlsym(a.handle, "ncclGetUniqueId");
    a.CommInitRank = (int (*)(nccl_comm_t*, int, nccl_unique_id, int))dlsym(a.handle, "ncclCommInitRank");
    a.CommDestroy = (int (*)(nccl_comm_t))dlsym(a.handle, "ncclCommDestroy");
    a.AllReduce = (int (*)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t))dlsym(a.handle, "ncclAllReduce");
    a.GetErrorString = (const char* (*)(int))dlsym(a.handle, "ncclGetErrorString");
    a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllReduce && a.GetErrorString;
    return a;
}

}  // namespace

smelt_status tp_all_reduce_f16(smelt_cuda_ctx* ctx, void* data, size_t count, cudaStream_t stream) {
    if (ctx->tp_world <= 1) return SMELT_OK;
    NcclApi& a = api();
    if (!a.ok || !ctx->nccl_comm) return fail(ctx, SMELT_ERR_COMM, "tensor-parallel communicator is not initialised");
    const int rc = a.AllReduce(data, data, count, kNcclFloat16, kNcclSum, (nccl_comm_t)ctx->nccl_comm, stream);
    if (rc != 0) return fail(ctx, SMELT_ERR_COMM, std::string("ncclAllReduce: ") + a.GetErrorString(rc));
    return SMELT_OK;
}

// ── all-reduce + residual add over peer memory ──────────────────────────────
// Every rank owns an exchange buffer that its peers can write (CUDA IPC mapping over NVLink):
//   ll [2 buffers][world sources][kTpMaxCount / 2] of {two fp16 values, sequence number}
// One launch per reduction and rank.  A thread pushes one word of its partial into slot [rank] of
// every rank's buffer as 8-byte stores that carry four bytes of data and the reduction's
// sequence number together (no fence and no separate flag: a word is valid as soon as its
// number matches, the way NCCL's low-latency protocol packs data and flag); nothing is loaded
// across NVLink.  It then polls its own buffer (bounded), adds the world's
// partials in rank order in fp32, rounds once to fp16 and adds the residual as elementwise_add
// does.  Every rank adds the same values in the same order, so the replicated hidden state
// stays bit-identical across ranks.  Two buffers alternate: a rank cannot be more than one
// reduction ahead of a peer, because it cannot finish reduction k + 1 before every peer has
// pushed k + 1, which the peer does after it has finished reading k.
constexpr int kTpMaxWorld = 8;
constexpr int kTpMaxCount = 8 * 8192;            // elements per reduction (batch 8 x hidden 8192)
constexpr uint32_t kTpSpinLimit = 1u << 21;      // about a second of polling per word, then give up with an error flag

struct TpExchange {
    uint2* ll[kTpMaxWorld];   // every rank's buffer, as mapped into this process
    uint32_t* seq;            // this rank's reduction counter (device memory)
    uint32_t* ticket;         // CTAs of the running reduction that have finished (zero between launches)
    int rank, world;
};

__host__ __device__ inline size_t tp_ll_index(int buf, int src, int world) { return ((size_t)buf * world + src) * (kTpMaxCount / 2); }

__device__ __forceinline__ void st_volatile_v2(uint2* p, uint32_t a, uint32_t b) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint2 ld_volatile_v2(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

// One thread per packed word.  The pushes go out first; then the thread requests its word from
// every source's slot at once (independent loads, one round trip for all of them) and re-requests
// only the slots whose sequence number has not arrived yet.  The last CTA to finish (ticket)
// advances the reduction counter: every thread of the launch has read it by then.
__global__ void __launch_bounds__(256) tp_reduce_add_kernel(TpExchange ex, const __half* partial, const __half* residual, __half* out,
                                                            int count, uint32_t* err, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t seq = *ex.seq + 1u;
    const int buf = (int)(seq & 1u);
    const int words = count / 2;
    if (i < words) {
        const uint32_t mine = reinterpret_cast<const uint32_t*>(partial)[i];
#pragma unroll
        for (int r = 0; r < kTpMaxWorld; ++r)
            if (r < ex.world) st_volatile_v2(ex.ll[r] + tp_ll_index(buf, ex.rank, ex.world) + i, mine, seq);
        const uint2* base = ex.ll[ex.rank] + tp_ll_index(buf, 0, ex.world) + i;
        const size_t stride = kTpMaxCount / 2;  // words between two sources' slots
        uint2 v[kTpMaxWorld];
#pragma unroll
        for (int r = 0; r < kTpMaxWorld; ++r) v[r] = r < ex.world ? ld_volatile_v2(base + r * stride) : make_uint2(0u, seq);
        uint32_t spins = 0;
        for (;;) {
            uint32_t pending = 0;
#pragma unroll
            for (int r = 0; r < kTpMaxWorld; ++r) pending |= (v[r].y != seq ? 1u : 0u) << r;
            if (!pending) break;
            if (++spins >= kTpSpinLimit) {  // a peer never arrived: results are not valid
                if (err) atomicOr(err, 0x100u);
                break;
            }
#pragma unroll
            for (int r = 0; r < kTpMaxWorld; ++r)
                if (pending & (1u << r)) v[r] = ld_volatile_v2(base + r * stride);
        }
        float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
        for (int r = 0; r < kTpMaxWorld; ++r)
            if (r < ex.world) {
                const float2 f = __half22float2(u32_as_h2(v[r].x));
                acc0 += f.x; acc1 += f.y;
            }
        // half(sum) + residual as an fp16 add (activations.metal elementwise_add)
        const uint32_t rv = reinterpret_cast<const uint32_t*>(residual)[i];
        reinterpret_cast<uint32_t*>(out)[i] = h2_as_u32(__hadd2(__floats2half2_rn(acc0, acc1), u32_as_h2(rv)));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(ex.ticket, 1u) == gridDim.x - 1u) {
            *ex.ticket = 0u;
            *ex.seq = seq;
        }
    }
}

// Vocab-parallel argmax: every rank holds the ordered keys (lut_matvec.metal:4045-4074) of its
// slice of the logits; the best local key, with the slice's offset folded into its index half,
// goes to every rank through the same packed words, and every rank takes the largest.
__global__ void __launch_bounds__(256) tp_argmax_kernel(TpExchange ex, uint2* const* regions, const uint64_t* partials, int32_t* out,
                                                        int n, uint32_t offset, int batch, uint32_t* err, DevDyn dyn) {
    __shared__ uint64_t sbest[8];
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    const int tid = threadIdx.x;
    const uint32_t seq = *ex.seq + 1u;
    __syncthreads();
    const int buf = (int)(seq & 1u);
    for (int b = 0; b < batch; ++b) {
        uint64_t best = 0;
        for (int i = tid; i < n; i += blockDim.x) { const uint64_t k = partials[(size_t)b * n + i]; best = k > best ? k : best; }
        for (int o = 16; o > 0; o >>= 1) { const uint64_t other = __shfl_xor_sync(0xffffffffu, best, o); best = other > best ? other : best; }
        if ((tid & 31) == 0) sbest[tid >> 5] = best;
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < 8; ++w) best = sbest[w] > best ? sbest[w] : best;
            best -= offset;  // index half is 0xFFFFFFFF - index: the slice's first row is global row `offset`
            for (int r = 0; r < ex.world; ++r) {
                uint2* dst = regions[r] + ((size_t)(buf * ex.world + ex.rank) * 8 + b) * 2;
                st_volatile_v2(dst, (uint32_t)best, seq);
                st_volatile_v2(dst + 1, (uint32_t)(best >> 32), seq);
            }
            uint64_t top = 0;
            bool gave_up = false;
            for (int r = 0; r < ex.world; ++r) {
                const uint2* src = regions[ex.rank] + ((size_t)(buf * ex.world + r) * 8 + b) * 2;
                uint2 lo = ld_volatile_v2(src), hi = ld_volatile_v2(src + 1);
                uint32_t spins = 0;
                while ((lo.y != seq || hi.y != seq) && !gave_up && ++spins < kTpSpinLimit) { lo = ld_volatile_v2(src); hi = ld_volatile_v2(src + 1); }
                gave_up |= lo.y != seq || hi.y != seq;
                const uint64_t k = ((uint64_t)hi.x << 32) | lo.x;
                top = k > top ? k : top;
            }
            if (gave_up && err) atomicOr(err, 0x100u);
            out[b] = (int32_t)(0xFFFFFFFFu - (uint32_t)top);
        }
        __syncthreads();
    }
    if (tid == 0) *ex.seq = seq;
}

struct TpPeerState {
    void* local = nullptr;               // this rank's exchange buffer
    void* mapped[kTpMaxWorld] = {};      // every rank's buffer as mapped here ([rank] = local)
    uint32_t* seq = nullptr;
    uint2** argmax_regions = nullptr;    // device array: every rank's argmax words, as mapped here
    bool open = false;
    bool loopback = false;               // diagnostic set-up: every buffer is a local allocation
};

constexpr size_t kTpArgmaxBytes = (size_t)2 * kTpMaxWorld * 8 * 2 * sizeof(uint2);  // [buffer][source][sequence, 8][2 words]

size_t tp_ll_bytes(int world) { return (size_t)2 * world * (kTpMaxCount / 2) * sizeof(uint2); }
size_t tp_exchange_bytes(int world) { return tp_ll_bytes(world) + kTpArgmaxBytes; }

// Fused all-reduce + residual add when the exchange buffers are open and the shape fits;
// *handled tells the caller whether it ran.
smelt_status tp_reduce_add(smelt_cuda_ctx* ctx, const Launch& l, const void* partial, const void* residual, void* out,
                           size_t count, bool* handled) {
    *handled = false;
    TpPeerState* st = (TpPeerState*)ctx->tp_peer;
    if (!st || !st->open || count == 0 || count % 2 || count > (size_t)kTpMaxCount) return SMELT_OK;
    if ((reinterpret_cast<uintptr_t>(partial) | reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(out)) & 3u) return SMELT_OK;
    TpExchange ex = {};
    for (int r = 0; r < ctx->tp_world; ++r) ex.ll[r] = (uint2*)st->mapped[r];
    ex.seq = st->seq; ex.ticket = st->seq + 1; ex.rank = ctx->tp_rank; ex.world = ctx->tp_world;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((count / 2 + 255) / 256));
    cfg.blockDim = dim3(256);
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = l.pdl ? 1 : 0;
    prefer_max_shared(tp_reduce_add_kernel);
    *handled = true;
    return check_cuda(ctx, cudaLaunchKernelEx(&cfg, tp_reduce_add_kernel, ex, (const __half*)partial, (const __half*)residual, (__half*)out,
                                              (int)count, ctx->err_dev, dev_dyn(l)), "tp reduce add");
}

// Cross-rank argmax over vocab slices (see tp_argmax_kernel); needs the open exchange.
smelt_status tp_argmax(smelt_cuda_ctx* ctx, const Launch& l, const void* partials, void* out, int n, uint32_t offset, int batch) {
    TpPeerState* st = (TpPeerState*)ctx->tp_peer;
    if (!st || !st->open) return fail(ctx, SMELT_ERR_UNSUPPORTED, "smelt_tp_argmax: the peer exchange is not open (smelt_cuda_tp_exchange_open)");
    if (batch <= 0 || batch > 8 || n <= 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "smelt_tp_argmax: batch 1..8");
    TpExchange ex = {};
    for (int r = 0; r < ctx->tp_world; ++r) ex.ll[r] = (uint2*)st->mapped[r];
    ex.seq = st->seq; ex.rank = ctx->tp_rank; ex.world = ctx->tp_world;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(256);
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = l.pdl ? 1 : 0;
    prefer_max_shared(tp_argmax_kernel);
    return check_cuda(ctx, cudaLaunchKernelEx(&cfg, tp_argmax_kernel, ex, (uint2* const*)st->argmax_regions, (const uint64_t*)partials,
                                              (int32_t*)out, n, offset, batch, ctx->err_dev, dev_dyn(l)), "tp argmax");
}

void tp_destroy(smelt_cuda_ctx* ctx) {
    if (TpPeerState* st = (TpPeerState*)ctx->tp_peer) {
        cudaFree(st->argmax_regions);
        for (int r = 0; r < ctx->tp_world && r < kTpMaxWorld; ++r)
            if (st->mapped[r] && st->mapped[r] != st->local) { if (st->loopback) cudaFree(st->mapped[r]); else cudaIpcCloseMemHandle(st->mapped[r]); }
        cudaFree(st->local);
        cudaFree(st->seq);
        delete st;
        ctx->tp_peer = nullptr;
    }
    if (ctx->nccl_comm && api().ok) api().CommDestroy((nccl_comm_t)ctx->nccl_comm);
    ctx->nccl_comm = nullptr;
}

}  // namespace smelt

using namespace smelt;

extern "C" {

smelt_status smelt_cuda_tp_unique_id(uint8_t id[SMELT_TP_ID_BYTES]) {
    if (!id) return SMELT_ERR_BAD_ARGUMENT;
    NcclApi& a = api();
    if (!a.ok) return SMELT_ERR_COMM;
    nccl_unique_id u;
    if (a.GetUniqueId(&u) != 0) return SMELT_ERR_COMM;
    memcpy(id, &u, SMELT_TP_ID_BYTES);
    return SMELT_OK;
}

smelt_status smelt_cuda_tp_init(smelt_cuda_ctx* ctx, int rank, int world, const uint8_t id[SMELT_TP_ID_BYTES]) {
    if (!ctx || !id || world < 1 || rank < 0 || rank >= world) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    ctx->tp_rank = rank;
    ctx->tp_world = world;
    if (world == 1) return SMELT_OK;
    NcclApi& a = api();
    if (!a.ok) return fail(ctx, SMELT_ERR_COMM, "libnccl.so.2 could not be loaded");
    nccl_unique_id u;
    memcpy(&u, id, SMELT_TP_ID_BYTES);
    nccl_comm_t comm = nullptr;
    const int rc = a.CommInitRank(&comm, world, u, rank);
    if (rc != 0) return fail(ctx, SMELT_ERR_COMM, std::string("ncclCommInitRank: ") + a.GetErrorString(rc));
    ctx->nccl_comm = comm;
    return SMELT_OK;
}

smelt_status smelt_cuda_tp_exchange_handle(smelt_cuda_ctx* ctx, uint8_t handle[SMELT_TP_HANDLE_BYTES]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == SMELT_TP_HANDLE_BYTES, "cudaIpcMemHandle_t is 64 bytes");
    if (!ctx || !handle) return SMELT_ERR_BAD_ARGUMENT;
    if (ctx->tp_world < 2 || ctx->tp_world > kTpMaxWorld) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "tp exchange: call smelt_cuda_tp_init with 2..8 ranks first");
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    TpPeerState* st = (TpPeerState*)ctx->tp_peer;
    if (!st) {
        st = new (std::nothrow) TpPeerState();
        if (!st) return SMELT_ERR_ALLOC;
        const size_t bytes = tp_exchange_bytes(ctx->tp_world);
        bool ok = cudaMalloc(&st->local, bytes) == cudaSuccess && cudaMemset(st->local, 0, bytes) == cudaSuccess;
        ok = ok && cudaMalloc((void**)&st->seq, 2 * sizeof(uint32_t)) == cudaSuccess && cudaMemset(st->seq, 0, 2 * sizeof(uint32_t)) == cudaSuccess;
        ok = ok && cudaDeviceSynchronize() == cudaSuccess;
        if (!ok) { cudaFree(st->local); cudaFree(st->seq); delete st; return fail(ctx, SMELT_ERR_ALLOC, "tp exchange: allocation failed"); }
        ctx->tp_peer = st;
    }
    cudaIpcMemHandle_t h;
    smelt_status s = check_cuda(ctx, cudaIpcGetMemHandle(&h, st->local), "cudaIpcGetMemHandle");
    if (!s) memcpy(handle, &h, SMELT_TP_HANDLE_BYTES);
    return s;
}

smelt_status smelt_cuda_tp_exchange_open(smelt_cuda_ctx* ctx, const uint8_t* handles) {
    if (!ctx || !handles) return SMELT_ERR_BAD_ARGUMENT;
    TpPeerState* st = (TpPeerState*)ctx->tp_peer;
    if (!st) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "tp exchange: call smelt_cuda_tp_exchange_handle first");
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    for (int r = 0; r < ctx->tp_world; ++r) {
        if (r == ctx->tp_rank) { st->mapped[r] = st->local; continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)r * SMELT_TP_HANDLE_BYTES, SMELT_TP_HANDLE_BYTES);
        smelt_status s = check_cuda(ctx, cudaIpcOpenMemHandle(&st->mapped[r], h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
        if (s) return s;
    }
    // the argmax words sit behind the reduction words of every rank's buffer
    uint2* regions[kTpMaxWorld] = {};
    for (int r = 0; r < ctx->tp_world; ++r) regions[r] = (uint2*)((char*)st->mapped[r] + tp_ll_bytes(ctx->tp_world));
    if (!st->argmax_regions && cudaMalloc((void**)&st->argmax_regions, sizeof(regions)) != cudaSuccess) return fail(ctx, SMELT_ERR_ALLOC, "tp exchange: allocation failed");
    smelt_status s2 = check_cuda(ctx, cudaMemcpy(st->argmax_regions, regions, sizeof(regions), cudaMemcpyHostToDevice), "tp exchange: upload");
    if (s2) return s2;
    st->open = true;
    return SMELT_OK;
}

smelt_status smelt_cuda_tp_exchange_open_loopback(smelt_cuda_ctx* ctx, int world) {
    if (!ctx || world < 2 || world > kTpMaxWorld) return SMELT_ERR_BAD_ARGUMENT;
    if (ctx->tp_peer) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "tp exchange: already set up");
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    TpPeerState* st = new (std::nothrow) TpPeerState();
    if (!st) return SMELT_ERR_ALLOC;
    const size_t bytes = tp_exchange_bytes(world);
    bool ok = cudaMalloc((void**)&st->seq, 2 * sizeof(uint32_t)) == cudaSuccess && cudaMemset(st->seq, 0, 2 * sizeof(uint32_t)) == cudaSuccess;
    for (int r = 0; r < world && ok; ++r) ok = cudaMalloc(&st->mapped[r], bytes) == cudaSuccess && cudaMemset(st->mapped[r], 0, bytes) == cudaSuccess;
    uint2* regions[kTpMaxWorld] = {};
    for (int r = 0; r < world; ++r) regions[r] = (uint2*)((char*)st->mapped[r] + tp_ll_bytes(world));
    ok = ok && cudaMalloc((void**)&st->argmax_regions, sizeof(regions)) == cudaSuccess &&
         cudaMemcpy(st->argmax_regions, regions, sizeof(regions), cudaMemcpyHostToDevice) == cudaSuccess;
    st->local = st->mapped[0];
    st->loopback = true;
    st->open = ok;
    ctx->tp_peer = st;
    ctx->tp_world = world;
    ctx->tp_rank = 0;
    return ok ? SMELT_OK : fail(ctx, SMELT_ERR_ALLOC, "tp exchange: allocation failed");
}

smelt_status smelt_cuda_tp_reduce_add(smelt_cuda_ctx* ctx, const void* partial, const void* residual, void* out, size_t count) {
    if (!ctx || !partial || !residual || !out) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    Launch l;
    l.stream = ctx->stream;
    bool handled = false;
    smelt_status s = tp_reduce_add(ctx, l, partial, residual, out, count, &handled);
    if (!s && !handled) return fail(ctx, SMELT_ERR_UNSUPPORTED, "tp reduce add: the exchange is not open, or count is odd / too large");
    return s;
}

smelt_status smelt_cuda_tp_all_reduce_f16(smelt_cuda_ctx* ctx, void* data_dev, size_t count) {
    if (!ctx || !data_dev) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    return tp_all_reduce_f16(ctx, data_dev, count, ctx->stream);
}

}  // extern "C"
