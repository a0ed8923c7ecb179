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
//   data  [2 buffers][world sources][kTpMaxCount fp16]   partial row-parallel outputs
//   flags [2 buffers][world sources] uint32               sequence number of the data beside it
// One launch per reduction, one CTA per rank: the CTA pushes its partial into slot [rank] of
// every peer's buffer (plain remote stores, no loads cross NVLink), fences, publishes the
// reduction's sequence number in every peer's flag, waits (bounded) until all of its own
// flags carry that number, then adds the world's partials in rank order in fp32, rounds once
// to fp16 and adds the residual as elementwise_add does.  Every rank adds the same values in
// the same order, so the replicated hidden state stays bit-identical across ranks.  Two
// buffers alternate: a rank cannot be more than one reduction ahead of a peer, because it
// cannot finish reduction k + 1 before every peer has published k + 1.
constexpr int kTpMaxWorld = 8;
constexpr int kTpMaxCount = 8 * 8192;            // elements per reduction (batch 8 x hidden 8192)
constexpr uint32_t kTpSpinLimit = 1u << 21;      // about a second of polling, then give up with an error flag

struct TpExchange {
    __half* data[kTpMaxWorld];      // data region of every rank's buffer, as mapped into this process
    uint32_t* flags[kTpMaxWorld];   // flag region of every rank's buffer
    uint32_t* seq;                  // this rank's reduction counter (device memory)
    int rank, world;
};

__host__ __device__ inline size_t tp_data_index(int buf, int src, int world) { return ((size_t)buf * world + src) * kTpMaxCount; }

__global__ void __launch_bounds__(1024) tp_reduce_add_kernel(TpExchange ex, const __half* partial, const __half* residual, __half* out,
                                                             int count, uint32_t* err, DevDyn dyn) {
    pdl_trigger();
    pdl_wait();
    if (dyn_skip(dyn)) return;
    __shared__ uint32_t s_seq;
    const int tid = threadIdx.x;
    if (tid == 0) s_seq = *ex.seq + 1u;
    __syncthreads();
    const uint32_t seq = s_seq;
    const int buf = (int)(seq & 1u);
    // push this rank's partial into every rank's buffer (its own included)
    const int chunks = count / 8;
    for (int r = 0; r < ex.world; ++r) {
        uint4* dst = reinterpret_cast<uint4*>(ex.data[r] + tp_data_index(buf, ex.rank, ex.world));
        for (int i = tid; i < chunks; i += blockDim.x) dst[i] = reinterpret_cast<const uint4*>(partial)[i];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < ex.world) {
        volatile uint32_t* f = ex.flags[tid] + buf * ex.world + ex.rank;
        *f = seq;  // tells rank tid that this rank's data for this reduction has landed
    }
    // wait for every source's flag in this rank's own buffer
    if (tid < ex.world) {
        volatile uint32_t* f = ex.flags[ex.rank] + buf * ex.world + tid;
        uint32_t spins = 0;
        while ((int32_t)(*f - seq) < 0 && ++spins < kTpSpinLimit) {}
        if (spins >= kTpSpinLimit && err) atomicOr(err, 0x100u);  // peer never arrived: results are not valid
    }
    __syncthreads();
    __threadfence_system();
    const __half* mine = ex.data[ex.rank];
    for (int i = tid; i < chunks; i += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int r = 0; r < ex.world; ++r) {
            const uint4 v = __ldcv(reinterpret_cast<const uint4*>(mine + tp_data_index(buf, r, ex.world)) + i);
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(u32_as_h2(u[j]));
                acc[2 * j] += f.x; acc[2 * j + 1] += f.y;
            }
        }
        const uint4 rv = reinterpret_cast<const uint4*>(residual)[i];
        const uint32_t ru[4] = {rv.x, rv.y, rv.z, rv.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)  // half(sum) + residual as an fp16 add (activations.metal elementwise_add)
            o[j] = h2_as_u32(__hadd2(__floats2half2_rn(acc[2 * j], acc[2 * j + 1]), u32_as_h2(ru[j])));
        reinterpret_cast<uint4*>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    if (tid == 0) *ex.seq = seq;
}

struct TpPeerState {
    void* local = nullptr;               // this rank's exchange buffer
    void* mapped[kTpMaxWorld] = {};      // every rank's buffer as mapped here ([rank] = local)
    uint32_t* seq = nullptr;
    bool open = false;
};

size_t tp_exchange_bytes(int world) { return (size_t)2 * world * kTpMaxCount * sizeof(__half) + 2 * world * sizeof(uint32_t) + 256; }

// Fused all-reduce + residual add when the exchange buffers are open and the shape fits;
// *handled tells the caller whether it ran.
smelt_status tp_reduce_add(smelt_cuda_ctx* ctx, const Launch& l, const void* partial, const void* residual, void* out,
                           size_t count, bool* handled) {
    *handled = false;
    TpPeerState* st = (TpPeerState*)ctx->tp_peer;
    if (!st || !st->open || count == 0 || count % 8 || count > (size_t)kTpMaxCount) return SMELT_OK;
    if ((reinterpret_cast<uintptr_t>(partial) | reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(out)) & 15u) return SMELT_OK;
    if (cudaError_t fe = flush_phases(l)) return check_cuda(ctx, fe, "multi-phase launch");
    TpExchange ex = {};
    const size_t data_bytes = (size_t)2 * ctx->tp_world * kTpMaxCount * sizeof(__half);
    for (int r = 0; r < ctx->tp_world; ++r) {
        ex.data[r] = (__half*)st->mapped[r];
        ex.flags[r] = (uint32_t*)((char*)st->mapped[r] + data_bytes);
    }
    ex.seq = st->seq; ex.rank = ctx->tp_rank; ex.world = ctx->tp_world;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(1024);
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

void tp_destroy(smelt_cuda_ctx* ctx) {
    if (TpPeerState* st = (TpPeerState*)ctx->tp_peer) {
        for (int r = 0; r < ctx->tp_world && r < kTpMaxWorld; ++r)
            if (st->mapped[r] && st->mapped[r] != st->local) cudaIpcCloseMemHandle(st->mapped[r]);
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
        ok = ok && cudaMalloc((void**)&st->seq, sizeof(uint32_t)) == cudaSuccess && cudaMemset(st->seq, 0, sizeof(uint32_t)) == cudaSuccess;
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
    st->open = true;
    return SMELT_OK;
}

smelt_status smelt_cuda_tp_all_reduce_f16(smelt_cuda_ctx* ctx, void* data_dev, size_t count) {
    if (!ctx || !data_dev) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    return tp_all_reduce_f16(ctx, data_dev, count, ctx->stream);
}

}  // extern "C"
