// smelt_cuda_attention_decode_static: attention_decode with the split partials in a fixed
// device array instead of the context's allocation.
//
// The entry point makes no device allocation on any call, and no host allocation on a call
// that succeeds (a refusal builds its message): the scratch is a file-scope __device__ array,
// and its address is looked up once per device with cudaGetSymbolAddress on the first call
// for that device (that lookup may load the module, so make the first call before any stream
// capture begins).  Nothing in the scratch has to
// start at zero: every partial the merge kernel reads is written by the decode kernel of the
// same call first, so the array is never cleared.  All calls on one device share the array:
// two calls that overlap in time (different contexts or streams) race on it.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "glue.h"
#include "runtime.h"

namespace smelt {
namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB: batch * n_q * (head_dim + 2) <= 32768
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_attn_static_scratch[kStaticScratchBytes];

std::mutex g_mu;
void* g_scratch_addr[kMaxDevices] = {};

cudaError_t static_scratch(int device, void** out) {
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_addr[device]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_attn_static_scratch);
        if (e != cudaSuccess) return e;
        g_scratch_addr[device] = p;
    }
    *out = g_scratch_addr[device];
    return cudaSuccess;
}

}  // namespace
}  // namespace smelt

using namespace smelt;

extern "C" smelt_status smelt_cuda_attention_decode_static(smelt_cuda_ctx* ctx, const void* q, const void* k_cache,
                                                           const void* v_cache, void* out, int n_q, int n_kv,
                                                           int head_dim, uint32_t capacity, uint32_t seq_len, float scale,
                                                           uint32_t sliding_window, int batch, size_t kv_seq_stride) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    if (ctx->device < 0 || ctx->device >= kMaxDevices)
        return fail(ctx, SMELT_ERR_UNSUPPORTED, "attention decode (static scratch): device ordinal beyond 63");
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e != cudaSuccess) return check_cuda(ctx, e, "cudaSetDevice");
    if (!q || !k_cache || !v_cache || !out || n_q <= 0 || n_kv <= 0 || n_q % n_kv || batch <= 0 || seq_len == 0 ||
        seq_len > capacity)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "attention decode (static scratch): bad geometry (1 <= seq_len <= capacity, n_q % n_kv == 0)");
    if (n_q / n_kv > 16 || (head_dim != 64 && head_dim != 128 && head_dim != 256))
        return fail(ctx, SMELT_ERR_UNSUPPORTED, "attention decode (static scratch): head_dim in {64,128,256}, GQA ratio <= 16");
    // Room for the largest split count the launcher may pick, so that the split (and with it
    // every bit of the result) is the one smelt_cuda_attention_decode chooses.
    const size_t need = attention_scratch_bytes(n_q, head_dim, batch, attention_max_splits());
    if (need > kStaticScratchBytes)
        return fail(ctx, SMELT_ERR_OUT_OF_RANGE,
                    "attention decode (static scratch): batch * n_q * (head_dim + 2) = " +
                        std::to_string((size_t)batch * n_q * (head_dim + 2)) +
                        " exceeds 32768, the most the 8 MiB static scratch holds; use smelt_cuda_attention_decode");
    void* scratch = nullptr;
    e = static_scratch(ctx->device, &scratch);
    if (e != cudaSuccess) return check_cuda(ctx, e, "cudaGetSymbolAddress(static attention scratch)");
    AttnArgs a = {};
    a.q = (const __half*)q; a.k_cache = (const __half*)k_cache; a.v_cache = (const __half*)v_cache; a.out = (__half*)out;
    a.n_q = n_q; a.n_kv = n_kv; a.head_dim = head_dim; a.batch = batch; a.capacity = capacity; a.seq_len = seq_len;
    a.seq_from_pos = 0; a.scale = scale; a.sliding_window = sliding_window;
    a.seq_stride = kv_seq_stride ? kv_seq_stride : (size_t)n_kv * capacity * head_dim;
    a.scratch = scratch; a.scratch_bytes = kStaticScratchBytes; a.sm_count = ctx->sm_count;
    Launch l;
    l.stream = ctx->stream;
    l.pdl = false;
    return check_cuda(ctx, launch_attention_decode(l, a), "attention decode (static scratch) launch");
}
