// Tensor-parallel communicator: NCCL over NVLink, one process per GPU.
//
// The reference is single-device (one MTLDevice, one command queue,
// Sources/SmeltRuntime/SmeltRuntime.swift:522-523), so this file has no counterpart there.
// NCCL is bound at run time with dlopen so that single-GPU users carry no NCCL dependency;
// when a process has already loaded NCCL (for example through torch) the same copy is reused.
#include <dlfcn.h>

#include <cstring>

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

void tp_destroy(smelt_cuda_ctx* ctx) {
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

smelt_status smelt_cuda_tp_all_reduce_f16(smelt_cuda_ctx* ctx, void* data_dev, size_t count) {
    if (!ctx || !data_dev) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    return tp_all_reduce_f16(ctx, data_dev, count, ctx->stream);
}

}  // extern "C"
