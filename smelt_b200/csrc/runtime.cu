// Context, buffer slots and the typed launchers of the libsmelt_cuda C ABI.
#include "runtime.h"

#include <cstdio>
#include <cstring>

#include "affine_matvec.h"
#include "glue.h"

using namespace smelt;

namespace smelt {

smelt_status fail(smelt_cuda_ctx* ctx, smelt_status code, const std::string& msg) {
    if (ctx) ctx->err = msg;
    return code;
}

smelt_status check_cuda(smelt_cuda_ctx* ctx, cudaError_t e, const char* what) {
    if (e == cudaSuccess) return SMELT_OK;
    return fail(ctx, SMELT_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

namespace {

__global__ void kv_regrow_kernel(const __half* src, __half* dst, int heads, int head_dim, uint32_t old_cap,
                                 uint32_t new_cap, uint32_t live) {
    const size_t per_head = (size_t)live * head_dim;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= per_head * heads) return;
    const size_t h = i / per_head, r = i % per_head;
    dst[h * (size_t)new_cap * head_dim + r] = src[h * (size_t)old_cap * head_dim + r];
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace smelt

#define CTX_OR_FAIL()                                \
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;         \
    {                                                \
        cudaError_t _e = cudaSetDevice(ctx->device); \
        if (_e != cudaSuccess) return check_cuda(ctx, _e, "cudaSetDevice"); \
    }

void smelt::destroy_decode_graphs(smelt_cuda_ctx* ctx) {
    if (ctx->graph_exec) cudaGraphExecDestroy(ctx->graph_exec);
    if (ctx->graph) cudaGraphDestroy(ctx->graph);
    if (ctx->graph_burst_exec) cudaGraphExecDestroy(ctx->graph_burst_exec);
    if (ctx->graph_burst) cudaGraphDestroy(ctx->graph_burst);
    ctx->graph_exec = ctx->graph_burst_exec = nullptr;
    ctx->graph = ctx->graph_burst = nullptr;
}

extern "C" {

smelt_status smelt_cuda_create(int device_ordinal, smelt_cuda_ctx** out_ctx) {
    if (!out_ctx) return SMELT_ERR_BAD_ARGUMENT;
    *out_ctx = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0 || device_ordinal < 0 || device_ordinal >= n) return SMELT_ERR_CUDA;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device_ordinal) != cudaSuccess) return SMELT_ERR_CUDA;
    if (prop.major < 10) return SMELT_ERR_UNSUPPORTED;  // kernels are built for sm_100a only
    if (cudaSetDevice(device_ordinal) != cudaSuccess) return SMELT_ERR_CUDA;
    smelt_cuda_ctx* ctx = new (std::nothrow) smelt_cuda_ctx();
    if (!ctx) return SMELT_ERR_ALLOC;
    ctx->device = device_ordinal;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->slots.resize(256);
    bool ok = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaMalloc(&ctx->dyn_dev, sizeof(DynState)) == cudaSuccess;
    ok = ok && cudaMalloc(&ctx->err_dev, sizeof(uint32_t)) == cudaSuccess;
    ok = ok && cudaMemset(ctx->dyn_dev, 0, sizeof(DynState)) == cudaSuccess;
    ok = ok && cudaMemset(ctx->err_dev, 0, sizeof(uint32_t)) == cudaSuccess;
    ctx->h_pinned_count = 4096;
    ok = ok && cudaMallocHost(&ctx->h_pinned, ctx->h_pinned_count * sizeof(int32_t)) == cudaSuccess;
    // Split-K attention partials: sized for the largest supported decode shape at creation so
    // no launch ever allocates (64 splits x 64 heads x batch 8 x (256+2) floats = 34 MB).
    ctx->attn_scratch_bytes = attention_scratch_bytes(64, 256, 8, attention_max_splits());
    ok = ok && cudaMalloc(&ctx->attn_scratch, ctx->attn_scratch_bytes) == cudaSuccess;
    ok = ok && cudaMalloc(&ctx->rope_table, 256 * sizeof(float)) == cudaSuccess;
    ctx->qmm_scratch_bytes = (size_t)40 << 20;  // 148 CTAs x 512 batch rows x 128 rows of fp32 (the wide QMM's split-K partials), with room to spare
    ok = ok && cudaMalloc(&ctx->qmm_scratch, ctx->qmm_scratch_bytes) == cudaSuccess;
    ok = ok && cudaMalloc(&ctx->qmm_counters, 4096 * sizeof(int)) == cudaSuccess;
    ok = ok && cudaMemset(ctx->qmm_counters, 0, 4096 * sizeof(int)) == cudaSuccess;
    ok = ok && cudaMalloc(&ctx->attn_counters, 4096 * sizeof(int)) == cudaSuccess;
    ok = ok && cudaMemset(ctx->attn_counters, 0, 4096 * sizeof(int)) == cudaSuccess;
    ctx->argmax_scratch_bytes = 64 * 1024 * sizeof(uint64_t);
    ok = ok && cudaMalloc(&ctx->argmax_scratch, ctx->argmax_scratch_bytes) == cudaSuccess;
    ok = ok && cudaEventCreate(&ctx->ev_start) == cudaSuccess && cudaEventCreate(&ctx->ev_stop) == cudaSuccess;
    if (!ok) {
        smelt_cuda_destroy(ctx);
        return SMELT_ERR_ALLOC;
    }
    *out_ctx = ctx;
    return SMELT_OK;
}

void smelt_cuda_destroy(smelt_cuda_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    if (ctx->user_graph_exec) cudaGraphExecDestroy(ctx->user_graph_exec);
    ctx->user_graph_exec = nullptr;
    // Graphs first: a communicator waits for every graph that captured one of its collectives
    // to be released before ncclCommDestroy returns.
    destroy_decode_graphs(ctx);
    tp_destroy(ctx);
    package_destroy(ctx);
    for (auto& s : ctx->slots)
        if (s.ptr) cudaFree(s.ptr);
    cudaFree(ctx->dyn_dev);
    cudaFree(ctx->err_dev);
    cudaFree(ctx->attn_scratch);
    cudaFree(ctx->attn_counters);
    cudaFree(ctx->qmm_scratch);
    if (ctx->prefill_scratch) cudaFree(ctx->prefill_scratch);
    cudaFree(ctx->qmm_counters);
    cudaFree(ctx->rope_table);
    cudaFree(ctx->argmax_scratch);
    cudaFree(ctx->gen_ring);
    cudaFree(ctx->gen_count);
    if (ctx->ev_start) cudaEventDestroy(ctx->ev_start);
    if (ctx->ev_stop) cudaEventDestroy(ctx->ev_stop);
    if (ctx->h_pinned) cudaFreeHost(ctx->h_pinned);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

const char* smelt_cuda_last_error(const smelt_cuda_ctx* ctx) { return ctx ? ctx->err.c_str() : "null context"; }

smelt_status smelt_cuda_synchronize(smelt_cuda_ctx* ctx) {
    CTX_OR_FAIL();
    return check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
}

void* smelt_cuda_stream(smelt_cuda_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

int smelt_cuda_sm_count(const smelt_cuda_ctx* ctx) { return ctx ? ctx->sm_count : 0; }

smelt_status smelt_cuda_device_error(smelt_cuda_ctx* ctx, uint32_t* out_flags) {
    CTX_OR_FAIL();
    if (!out_flags) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "out_flags is null");
    smelt_status s = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
    if (s) return s;
    s = check_cuda(ctx, cudaMemcpy(out_flags, ctx->err_dev, 4, cudaMemcpyDeviceToHost), "read error word");
    if (s) return s;
    if (*out_flags) {
        cudaMemset(ctx->err_dev, 0, 4);
        return fail(ctx, SMELT_ERR_DEVICE_TIMEOUT, "a kernel's bounded wait gave up (flags " + std::to_string(*out_flags) + ")");
    }
    return SMELT_OK;
}

smelt_status smelt_cuda_clear_device_error(smelt_cuda_ctx* ctx) {
    CTX_OR_FAIL();
    smelt_status s = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
    if (!s) s = check_cuda(ctx, cudaMemset(ctx->err_dev, 0, sizeof(uint32_t)), "clear error word");
    return s;
}

smelt_status smelt_cuda_capture_begin(smelt_cuda_ctx* ctx) {
    CTX_OR_FAIL();
    if (ctx->capturing) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "capture_begin: a capture is already open");
    if (ctx->user_graph_exec) { cudaGraphExecDestroy(ctx->user_graph_exec); ctx->user_graph_exec = nullptr; }
    smelt_status s = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "capture_begin: sync");
    if (s) return s;
    s = check_cuda(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
    if (!s) ctx->capturing = true;
    return s;
}

smelt_status smelt_cuda_capture_end(smelt_cuda_ctx* ctx) {
    CTX_OR_FAIL();
    if (!ctx->capturing) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "capture_end: no capture is open");
    ctx->capturing = false;
    cudaGraph_t g = nullptr;
    smelt_status s = check_cuda(ctx, cudaStreamEndCapture(ctx->stream, &g), "cudaStreamEndCapture");
    if (s) return s;
    s = check_cuda(ctx, cudaGraphInstantiate(&ctx->user_graph_exec, g, 0), "cudaGraphInstantiate");
    cudaGraphDestroy(g);
    return s;
}

smelt_status smelt_cuda_capture_replay(smelt_cuda_ctx* ctx, int warmup, int reps, float* out_ms) {
    CTX_OR_FAIL();
    if (!ctx->user_graph_exec || reps <= 0 || warmup < 0 || !out_ms) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "capture_replay: nothing recorded, or bad counts");
    smelt_status s = SMELT_OK;
    for (int i = 0; i < warmup && !s; ++i) s = check_cuda(ctx, cudaGraphLaunch(ctx->user_graph_exec, ctx->stream), "cudaGraphLaunch");
    if (!s) s = check_cuda(ctx, cudaEventRecord(ctx->ev_start, ctx->stream), "capture_replay: start event");
    for (int i = 0; i < reps && !s; ++i) s = check_cuda(ctx, cudaGraphLaunch(ctx->user_graph_exec, ctx->stream), "cudaGraphLaunch");
    if (!s) s = check_cuda(ctx, cudaEventRecord(ctx->ev_stop, ctx->stream), "capture_replay: stop event");
    if (!s) s = check_cuda(ctx, cudaEventSynchronize(ctx->ev_stop), "capture_replay: sync");
    float ms = 0.f;
    if (!s) s = check_cuda(ctx, cudaEventElapsedTime(&ms, ctx->ev_start, ctx->ev_stop), "capture_replay: elapsed");
    if (!s) *out_ms = ms / (float)reps;
    return s;
}

smelt_status smelt_cuda_timer_start(smelt_cuda_ctx* ctx) {
    CTX_OR_FAIL();
    return check_cuda(ctx, cudaEventRecord(ctx->ev_start, ctx->stream), "timer start");
}
smelt_status smelt_cuda_timer_stop(smelt_cuda_ctx* ctx, float* out_ms) {
    CTX_OR_FAIL();
    if (!out_ms) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "out_ms is null");
    smelt_status s = check_cuda(ctx, cudaEventRecord(ctx->ev_stop, ctx->stream), "timer stop");
    if (!s) s = check_cuda(ctx, cudaEventSynchronize(ctx->ev_stop), "timer sync");
    if (!s) s = check_cuda(ctx, cudaEventElapsedTime(out_ms, ctx->ev_start, ctx->ev_stop), "timer elapsed");
    return s;
}

smelt_status smelt_cuda_malloc(smelt_cuda_ctx* ctx, size_t bytes, void** out_dev) {
    CTX_OR_FAIL();
    if (!out_dev) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "out_dev is null");
    cudaError_t e = cudaMalloc(out_dev, bytes ? bytes : 16);
    if (e != cudaSuccess) return fail(ctx, SMELT_ERR_ALLOC, std::string("cudaMalloc: ") + cudaGetErrorString(e));
    return SMELT_OK;
}
smelt_status smelt_cuda_free(smelt_cuda_ctx* ctx, void* dev) {
    CTX_OR_FAIL();
    return check_cuda(ctx, cudaFree(dev), "cudaFree");
}
smelt_status smelt_cuda_memcpy_h2d(smelt_cuda_ctx* ctx, void* dst_dev, const void* src, size_t bytes) {
    CTX_OR_FAIL();
    smelt_status s = check_cuda(ctx, cudaMemcpyAsync(dst_dev, src, bytes, cudaMemcpyHostToDevice, ctx->stream), "memcpy h2d");
    return s ? s : check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "memcpy h2d sync");
}
smelt_status smelt_cuda_memcpy_d2h(smelt_cuda_ctx* ctx, void* dst, const void* src_dev, size_t bytes) {
    CTX_OR_FAIL();
    smelt_status s = check_cuda(ctx, cudaMemcpyAsync(dst, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream), "memcpy d2h");
    return s ? s : check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "memcpy d2h sync");
}
smelt_status smelt_cuda_memset(smelt_cuda_ctx* ctx, void* dst_dev, int value, size_t bytes) {
    CTX_OR_FAIL();
    return check_cuda(ctx, cudaMemsetAsync(dst_dev, value, bytes, ctx->stream), "memset");
}

// ── slots ───────────────────────────────────────────────────────────────────
// A captured graph holds the device pointers of the slots as they were at capture.  When a
// slot's allocation is about to be replaced or freed, every graph of the context is dropped, so
// that a later replay reports "no graph has been built" instead of touching freed memory
// (the reference's rule that a buffer handle cached across a grow is stale,
// SmeltRuntime.swift:5101-5103).  Refused while a capture is open.
static smelt_status drop_graphs_for_slot_change(smelt_cuda_ctx* ctx, const char* what) {
    if (ctx->capturing) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, std::string(what) + ": a slot cannot change while a capture is open");
    if (!ctx->graph_exec && !ctx->graph && !ctx->user_graph_exec) return SMELT_OK;
    smelt_status s = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), what);
    if (ctx->user_graph_exec) { cudaGraphExecDestroy(ctx->user_graph_exec); ctx->user_graph_exec = nullptr; }
    destroy_decode_graphs(ctx);
    return s;
}

static smelt_status slot_ok(smelt_cuda_ctx* ctx, int slot, bool must_exist) {
    if (slot < 0 || slot >= (int)ctx->slots.size()) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "slot index " + std::to_string(slot) + " out of range");
    if (must_exist && !ctx->slots[slot].ptr) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "slot " + std::to_string(slot) + " is not allocated");
    return SMELT_OK;
}

smelt_status smelt_cuda_alloc_slot(smelt_cuda_ctx* ctx, int slot, size_t bytes) {
    CTX_OR_FAIL();
    smelt_status s = slot_ok(ctx, slot, false);
    if (s) return s;
    Slot& sl = ctx->slots[slot];
    if (sl.ptr) {
        s = drop_graphs_for_slot_change(ctx, "alloc_slot");
        if (s) return s;
        cudaStreamSynchronize(ctx->stream);
        cudaFree(sl.ptr);
        sl = Slot();
    }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes ? bytes : 16);
    if (e != cudaSuccess) return fail(ctx, SMELT_ERR_ALLOC, "slot " + std::to_string(slot) + ": " + cudaGetErrorString(e));
    sl.ptr = p;
    sl.bytes = bytes;
    return check_cuda(ctx, cudaMemsetAsync(p, 0, bytes ? bytes : 16, ctx->stream), "zero slot");
}

smelt_status smelt_cuda_resize_slot(smelt_cuda_ctx* ctx, int slot, size_t bytes, size_t preserve_bytes) {
    CTX_OR_FAIL();
    smelt_status s = slot_ok(ctx, slot, true);
    if (s) return s;
    Slot& sl = ctx->slots[slot];
    s = drop_graphs_for_slot_change(ctx, "resize_slot");
    if (s) return s;
    if (preserve_bytes > sl.bytes) preserve_bytes = sl.bytes;
    if (preserve_bytes > bytes) preserve_bytes = bytes;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes ? bytes : 16);
    if (e != cudaSuccess) return fail(ctx, SMELT_ERR_ALLOC, std::string("resize slot: ") + cudaGetErrorString(e));
    cudaMemsetAsync(p, 0, bytes ? bytes : 16, ctx->stream);
    if (preserve_bytes) cudaMemcpyAsync(p, sl.ptr, preserve_bytes, cudaMemcpyDeviceToDevice, ctx->stream);
    s = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "resize slot");
    cudaFree(sl.ptr);
    sl.ptr = p;
    sl.bytes = bytes;
    return s;
}

smelt_status smelt_cuda_resize_kv_slot(smelt_cuda_ctx* ctx, int slot, int heads, int head_dim, uint32_t old_capacity,
                                       uint32_t new_capacity, uint32_t live_len) {
    CTX_OR_FAIL();
    smelt_status s = slot_ok(ctx, slot, true);
    if (s) return s;
    Slot& sl = ctx->slots[slot];
    if (heads <= 0 || head_dim <= 0 || live_len > old_capacity || live_len > new_capacity ||
        (size_t)heads * old_capacity * head_dim * 2 > sl.bytes)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "resize_kv_slot: geometry does not match the slot");
    s = drop_graphs_for_slot_change(ctx, "resize_kv_slot");
    if (s) return s;
    const size_t bytes = (size_t)heads * new_capacity * head_dim * 2;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes ? bytes : 16);
    if (e != cudaSuccess) return fail(ctx, SMELT_ERR_ALLOC, std::string("resize kv slot: ") + cudaGetErrorString(e));
    cudaMemsetAsync(p, 0, bytes ? bytes : 16, ctx->stream);
    const size_t n = (size_t)heads * live_len * head_dim;
    if (n) kv_regrow_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>((const __half*)sl.ptr, (__half*)p, heads, head_dim, old_capacity, new_capacity, live_len);
    s = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "resize kv slot");
    cudaFree(sl.ptr);
    sl.ptr = p;
    sl.bytes = bytes;
    return s;
}

smelt_status smelt_cuda_slot_ptr(smelt_cuda_ctx* ctx, int slot, void** out_dev, size_t* out_bytes) {
    if (!ctx) return SMELT_ERR_BAD_ARGUMENT;
    smelt_status s = slot_ok(ctx, slot, true);
    if (s) return s;
    if (out_dev) *out_dev = ctx->slots[slot].ptr;
    if (out_bytes) *out_bytes = ctx->slots[slot].bytes;
    return SMELT_OK;
}

smelt_status smelt_cuda_write_slot(smelt_cuda_ctx* ctx, int slot, size_t offset, const void* src, size_t bytes) {
    CTX_OR_FAIL();
    smelt_status s = slot_ok(ctx, slot, true);
    if (s) return s;
    if (offset + bytes > ctx->slots[slot].bytes) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "write_slot beyond the slot's size");
    return smelt_cuda_memcpy_h2d(ctx, (uint8_t*)ctx->slots[slot].ptr + offset, src, bytes);
}

smelt_status smelt_cuda_read_slot(smelt_cuda_ctx* ctx, int slot, size_t offset, void* dst, size_t bytes) {
    CTX_OR_FAIL();
    smelt_status s = slot_ok(ctx, slot, true);
    if (s) return s;
    if (offset + bytes > ctx->slots[slot].bytes) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "read_slot beyond the slot's size");
    return smelt_cuda_memcpy_d2h(ctx, dst, (const uint8_t*)ctx->slots[slot].ptr + offset, bytes);
}

smelt_status smelt_cuda_zero_slot(smelt_cuda_ctx* ctx, int slot) {
    CTX_OR_FAIL();
    smelt_status s = slot_ok(ctx, slot, true);
    if (s) return s;
    return check_cuda(ctx, cudaMemsetAsync(ctx->slots[slot].ptr, 0, ctx->slots[slot].bytes, ctx->stream), "zero slot");
}

smelt_status smelt_cuda_upload_weights(smelt_cuda_ctx* ctx, int slot, const void* image, size_t bytes) {
    smelt_status s = smelt_cuda_alloc_slot(ctx, slot, bytes);
    if (s) return s;
    return smelt_cuda_write_slot(ctx, slot, 0, image, bytes);
}

smelt_status smelt_cuda_configure(smelt_cuda_ctx* ctx, const smelt_cuda_runtime_config* cfg) {
    if (!ctx || !cfg) return SMELT_ERR_BAD_ARGUMENT;
    if (cfg->batch == 0 || cfg->batch > 64) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "batch must be in 1..64");
    ctx->cfg = *cfg;
    ctx->configured = true;
    return SMELT_OK;
}

// ── typed launchers ─────────────────────────────────────────────────────────
static Launch typed_launch(smelt_cuda_ctx* ctx) {
    Launch l;
    l.stream = ctx->stream;
    l.pdl = ctx->capturing && ctx->pdl;  // inside a capture the launches chain like a decode table's
    return l;
}

static smelt_status affine_common(smelt_cuda_ctx* ctx, int mode, const void* w0, const void* s0, const void* b0,
                                  const void* w1, const void* s1, const void* b1, const void* x, void* y, void* y2,
                                  const void* residual, int rows, int cols, int group, int batch) {
    CTX_OR_FAIL();
    if (!w0 || !s0 || !b0 || !x || !y) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "affine matvec: null pointer");
    if (rows <= 0 || cols <= 0 || batch <= 0 || (group != 32 && group != 64 && group != 128) || cols % group != 0)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "affine matvec: rows/cols/batch must be positive, group in {32,64,128} dividing cols");
    if (!aligned16(w0) || !aligned16(x) || (w1 && !aligned16(w1)))
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "affine matvec: weight and activation pointers must be 16-byte aligned");
    AffineArgs a = {};
    a.w[0] = (const uint8_t*)w0; a.s[0] = (const __half*)s0; a.b[0] = (const __half*)b0;
    a.w[1] = (const uint8_t*)w1; a.s[1] = (const __half*)s1; a.b[1] = (const __half*)b1;
    a.x = (const __half*)x; a.y = (__half*)y; a.y2 = (__half*)y2; a.residual = (const __half*)residual;
    a.rows = rows; a.cols = cols; a.batch = batch; a.err = ctx->err_dev; a.sm_count = ctx->sm_count; a.part_scratch = ctx->qmm_scratch; a.part_scratch_bytes = ctx->qmm_scratch_bytes; a.part_counters = ctx->qmm_counters;
    return check_cuda(ctx, launch_affine(typed_launch(ctx), mode, a, group), "affine matvec launch");
}

smelt_status smelt_cuda_affine_matvec(smelt_cuda_ctx* ctx, const void* w, const void* s, const void* b, const void* x,
                                      void* y, int rows, int cols, int group, int batch) {
    return affine_common(ctx, kAffinePlain, w, s, b, nullptr, nullptr, nullptr, x, y, nullptr, nullptr, rows, cols, group, batch);
}
smelt_status smelt_cuda_affine_matvec_add(smelt_cuda_ctx* ctx, const void* w, const void* s, const void* b,
                                          const void* x, const void* residual, void* y, int rows, int cols, int group,
                                          int batch) {
    if (!residual) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "affine matvec add: null residual");
    return affine_common(ctx, kAffineAdd, w, s, b, nullptr, nullptr, nullptr, x, y, nullptr, residual, rows, cols, group, batch);
}
smelt_status smelt_cuda_affine_gate_up_swiglu(smelt_cuda_ctx* ctx, const void* gw, const void* gs, const void* gb,
                                              const void* uw, const void* us, const void* ub, const void* x, void* y,
                                              int rows, int cols, int group, int batch) {
    if (!uw || !us || !ub) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "gate/up: null pointer");
    return affine_common(ctx, kAffineGateUp, gw, gs, gb, uw, us, ub, x, y, nullptr, nullptr, rows, cols, group, batch);
}
smelt_status smelt_cuda_affine_dual_matvec(smelt_cuda_ctx* ctx, const void* w0, const void* s0, const void* b0,
                                           const void* w1, const void* s1, const void* b1, const void* x, void* y0,
                                           void* y1, int rows, int cols, int group, int batch) {
    if (!w1 || !s1 || !b1 || !y1) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "dual matvec: null pointer");
    return affine_common(ctx, kAffineDual, w0, s0, b0, w1, s1, b1, x, y0, y1, nullptr, rows, cols, group, batch);
}

smelt_status smelt_cuda_affine_multi_matvec(smelt_cuda_ctx* ctx, const smelt_affine_tensor* tensors, int n_tensors, const void* x,
                                            const void* norm_w, float eps, int cols, int group, int batch) {
    CTX_OR_FAIL();
    if (!tensors || n_tensors < 1 || n_tensors > 3 || !x || cols <= 0 || batch <= 0)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "affine multi matvec: 1..3 tensors, positive cols and batch");
    AffineArgs a = {};
    a.nseg = n_tensors;
    for (int i = 0; i < n_tensors; ++i) {
        const smelt_affine_tensor& t = tensors[i];
        if (!t.w_dev || !t.scales_dev || !t.biases_dev || !t.y_dev || t.rows <= 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "affine multi matvec: null tensor field");
        a.seg[i].w = (const uint8_t*)t.w_dev; a.seg[i].s = (const __half*)t.scales_dev; a.seg[i].b = (const __half*)t.biases_dev;
        a.seg[i].y = (__half*)t.y_dev; a.seg[i].rows = t.rows;
        a.rows += t.rows;
    }
    a.w[0] = a.seg[0].w; a.s[0] = a.seg[0].s; a.b[0] = a.seg[0].b; a.y = a.seg[0].y;
    a.x = (const __half*)x; a.norm_w = (const __half*)norm_w; a.norm_eps = eps;
    a.cols = cols; a.batch = batch; a.err = ctx->err_dev; a.sm_count = ctx->sm_count; a.part_scratch = ctx->qmm_scratch; a.part_scratch_bytes = ctx->qmm_scratch_bytes; a.part_counters = ctx->qmm_counters;
    if (n_tensors == 1 && !norm_w) a.nseg = 0;
    cudaError_t e = launch_affine(typed_launch(ctx), kAffinePlain, a, group);
    if (e == cudaErrorNotSupported) return fail(ctx, SMELT_ERR_UNSUPPORTED, "affine multi matvec: needs group 64, cols % 1024 == 0, 16-byte aligned operands, rows % 16 == 0 for all but the last tensor");
    return check_cuda(ctx, e, "affine multi matvec launch");
}

smelt_status smelt_cuda_rmsnorm_affine_gate_up_swiglu(smelt_cuda_ctx* ctx, const void* gw, const void* gs, const void* gb, const void* uw,
                                                      const void* us, const void* ub, const void* x, const void* norm_w, float eps,
                                                      void* y, int rows, int cols, int group, int batch) {
    CTX_OR_FAIL();
    if (!gw || !gs || !gb || !uw || !us || !ub || !x || !norm_w || !y || rows <= 0 || cols <= 0 || batch <= 0)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "rmsnorm gate/up: null pointer or bad shape");
    AffineArgs a = {};
    a.w[0] = (const uint8_t*)gw; a.s[0] = (const __half*)gs; a.b[0] = (const __half*)gb;
    a.w[1] = (const uint8_t*)uw; a.s[1] = (const __half*)us; a.b[1] = (const __half*)ub;
    a.x = (const __half*)x; a.y = (__half*)y; a.norm_w = (const __half*)norm_w; a.norm_eps = eps;
    a.rows = rows; a.cols = cols; a.batch = batch; a.err = ctx->err_dev; a.sm_count = ctx->sm_count; a.part_scratch = ctx->qmm_scratch; a.part_scratch_bytes = ctx->qmm_scratch_bytes; a.part_counters = ctx->qmm_counters;
    cudaError_t e = launch_affine(typed_launch(ctx), kAffineGateUp, a, group);
    if (e == cudaErrorNotSupported) return fail(ctx, SMELT_ERR_UNSUPPORTED, "rmsnorm gate/up: needs group 64, cols % 1024 == 0, 16-byte aligned operands");
    return check_cuda(ctx, e, "rmsnorm gate/up launch");
}

smelt_status smelt_cuda_rope_qkv_append(smelt_cuda_ctx* ctx, void* q, const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                                        uint32_t capacity, int head_dim, int n_q, int n_kv, int layout, uint32_t position,
                                        float base_log2, int batch, size_t kv_seq_stride) {
    CTX_OR_FAIL();
    if (!q || !k_new || !v_new || !k_cache || !v_cache || head_dim <= 0 || head_dim % 2 || n_q <= 0 || n_kv <= 0 || batch <= 0 || (layout != 0 && layout != 1))
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "rope qkv append: bad arguments (layout 0 or 1, even head_dim)");
    if (position >= capacity) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "rope qkv append: position must be below capacity");
    Launch l = typed_launch(ctx);
    l.position = position;
    return check_cuda(ctx, launch_rope_qkv_append(l, (__half*)q, (const __half*)k_new, (const __half*)v_new, (__half*)k_cache, (__half*)v_cache, capacity, head_dim, n_q, n_kv, layout, base_log2, batch, kv_seq_stride ? kv_seq_stride : (size_t)n_kv * capacity * head_dim), "rope qkv append");
}

smelt_status smelt_cuda_affine_dequantize(smelt_cuda_ctx* ctx, const void* w, const void* s, const void* b,
                                          void* out_f32, void* out_f16, int rows, int cols, int group) {
    CTX_OR_FAIL();
    if (!w || !s || !b || rows <= 0 || cols <= 0 || group <= 0 || cols % group || cols % 2)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "affine dequantize: bad geometry");
    return check_cuda(ctx, launch_affine_dequant(typed_launch(ctx), (const uint8_t*)w, (const __half*)s, (const __half*)b, (float*)out_f32, (__half*)out_f16, rows, cols, group), "affine dequantize");
}

smelt_status smelt_cuda_fp16_matvec(smelt_cuda_ctx* ctx, const void* w, const void* x, void* y, int rows, int cols,
                                    int batch) {
    CTX_OR_FAIL();
    if (!w || !x || !y || rows <= 0 || cols <= 0 || cols % 8 || batch <= 0 || !aligned16(w) || !aligned16(x))
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "fp16 matvec: cols must be a multiple of 8 and pointers 16-byte aligned");
    return check_cuda(ctx, launch_fp16_matvec(typed_launch(ctx), (const __half*)w, (const __half*)x, (__half*)y, rows, cols, batch, ctx->sm_count), "fp16 matvec");
}

static smelt_status signed_common(smelt_cuda_ctx* ctx, int mode, int format, const void* c0, const void* s0,
                                  const void* c1, const void* s1, const void* x, const void* residual, void* y,
                                  int rows, int cols, int batch) {
    CTX_OR_FAIL();
    if ((format != 1 && format != 2) || !c0 || !s0 || !x || !y || rows <= 0 || cols <= 0 || cols % 128 || batch <= 0)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "signed matvec: format in {1,2}, cols a positive multiple of 128");
    SignedArgs a = {};
    a.codes[0] = (const uint8_t*)c0; a.scales[0] = (const __half*)s0;
    a.codes[1] = (const uint8_t*)c1; a.scales[1] = (const __half*)s1;
    a.x = (const __half*)x; a.y = (__half*)y; a.residual = (const __half*)residual;
    a.rows = rows; a.cols = cols; a.batch = batch; a.bits = format;
    return check_cuda(ctx, launch_signed(typed_launch(ctx), mode, a), "signed matvec launch");
}
smelt_status smelt_cuda_signed_matvec(smelt_cuda_ctx* ctx, int format, const void* codes, const void* scales,
                                      const void* x, void* y, int rows, int cols, int batch) {
    return signed_common(ctx, kSignedPlain, format, codes, scales, nullptr, nullptr, x, nullptr, y, rows, cols, batch);
}
smelt_status smelt_cuda_signed_matvec_add(smelt_cuda_ctx* ctx, int format, const void* codes, const void* scales,
                                          const void* x, const void* residual, void* y, int rows, int cols, int batch) {
    if (!residual) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "signed matvec add: null residual");
    return signed_common(ctx, kSignedAdd, format, codes, scales, nullptr, nullptr, x, residual, y, rows, cols, batch);
}
smelt_status smelt_cuda_signed_gate_up_swiglu(smelt_cuda_ctx* ctx, int format, const void* gc, const void* gs,
                                              const void* uc, const void* us, const void* x, void* y, int rows,
                                              int cols, int batch) {
    if (!uc || !us) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "signed gate/up: null pointer");
    return signed_common(ctx, kSignedGateUp, format, gc, gs, uc, us, x, nullptr, y, rows, cols, batch);
}
smelt_status smelt_cuda_signed_dequantize(smelt_cuda_ctx* ctx, int format, const void* codes, const void* scales,
                                          void* out_f32, int rows, int cols, int* out_invalid) {
    CTX_OR_FAIL();
    if ((format != 1 && format != 2) || !codes || !scales || !out_f32 || rows <= 0 || cols <= 0 || cols % 128)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "signed dequantize: bad geometry");
    int* bad = nullptr;
    if (cudaMalloc(&bad, sizeof(int)) != cudaSuccess) return fail(ctx, SMELT_ERR_ALLOC, "signed dequantize: flag");
    cudaMemsetAsync(bad, 0, sizeof(int), ctx->stream);
    smelt_status s = check_cuda(ctx, launch_signed_dequant(typed_launch(ctx), (const uint8_t*)codes, (const __half*)scales, (float*)out_f32, rows, cols, format, 128, bad), "signed dequantize");
    int h = 0;
    if (!s) s = check_cuda(ctx, cudaMemcpyAsync(&h, bad, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream), "signed dequantize flag");
    if (!s) s = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "signed dequantize sync");
    cudaFree(bad);
    if (out_invalid) *out_invalid = h;
    return s;
}

smelt_status smelt_cuda_attention_decode(smelt_cuda_ctx* ctx, const void* q, const void* k_cache, const void* v_cache,
                                         void* out, int n_q, int n_kv, int head_dim, uint32_t capacity,
                                         uint32_t seq_len, float scale, uint32_t sliding_window, int batch,
                                         size_t kv_seq_stride) {
    CTX_OR_FAIL();
    if (!q || !k_cache || !v_cache || !out || n_q <= 0 || n_kv <= 0 || n_q % n_kv || batch <= 0 || seq_len == 0 ||
        seq_len > capacity)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "attention decode: bad geometry (1 <= seq_len <= capacity, n_q % n_kv == 0)");
    if (n_q / n_kv > 16 || (head_dim != 64 && head_dim != 128 && head_dim != 256))
        return fail(ctx, SMELT_ERR_UNSUPPORTED, "attention decode: head_dim in {64,128,256}, GQA ratio <= 16");
    AttnArgs a = {};
    a.q = (const __half*)q; a.k_cache = (const __half*)k_cache; a.v_cache = (const __half*)v_cache; a.out = (__half*)out;
    a.n_q = n_q; a.n_kv = n_kv; a.head_dim = head_dim; a.batch = batch; a.capacity = capacity; a.seq_len = seq_len;
    a.seq_from_pos = 0; a.scale = scale; a.sliding_window = sliding_window;
    a.seq_stride = kv_seq_stride ? kv_seq_stride : (size_t)n_kv * capacity * head_dim;
    a.scratch = ctx->attn_scratch; a.scratch_bytes = ctx->attn_scratch_bytes; a.sm_count = ctx->sm_count;
    if ((size_t)batch * n_kv <= 4096) a.counters = ctx->attn_counters;
    return check_cuda(ctx, launch_attention_decode(typed_launch(ctx), a), "attention decode launch");
}

smelt_status smelt_cuda_rope_attention_decode(smelt_cuda_ctx* ctx, const void* q, const void* k_new, const void* v_new, void* k_cache,
                                              void* v_cache, void* out, int n_q, int n_kv, int head_dim, uint32_t capacity,
                                              uint32_t position, float scale, uint32_t sliding_window, int layout,
                                              float base_log2, int batch, size_t kv_seq_stride) {
    CTX_OR_FAIL();
    if (!q || !k_new || !v_new || !k_cache || !v_cache || !out || n_q <= 0 || n_kv <= 0 || n_q % n_kv || batch <= 0 || (layout != 0 && layout != 1))
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "rope attention decode: bad arguments (layout 0 or 1, n_q % n_kv == 0)");
    if (position >= capacity) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "rope attention decode: position must be below capacity");
    if (n_q / n_kv > 16 || (head_dim != 64 && head_dim != 128 && head_dim != 256) || (size_t)batch * n_kv > 4096)
        return fail(ctx, SMELT_ERR_UNSUPPORTED, "rope attention decode: head_dim in {64,128,256}, GQA ratio <= 16");
    AttnArgs a = {};
    a.q = (const __half*)q; a.k_cache = (const __half*)k_cache; a.v_cache = (const __half*)v_cache; a.out = (__half*)out;
    a.k_new = (const __half*)k_new; a.v_new = (const __half*)v_new; a.rope_layout = layout; a.rope_base_log2 = base_log2;
    a.n_q = n_q; a.n_kv = n_kv; a.head_dim = head_dim; a.batch = batch; a.capacity = capacity; a.seq_len = position + 1;
    a.seq_from_pos = 0; a.scale = scale; a.sliding_window = sliding_window;
    a.seq_stride = kv_seq_stride ? kv_seq_stride : (size_t)n_kv * capacity * head_dim;
    a.scratch = ctx->attn_scratch; a.scratch_bytes = ctx->attn_scratch_bytes; a.sm_count = ctx->sm_count;
    a.counters = ctx->attn_counters;
    return check_cuda(ctx, launch_attention_decode(typed_launch(ctx), a), "rope attention decode launch");
}

smelt_status smelt_cuda_kv_cache_update(smelt_cuda_ctx* ctx, void* cache, const void* new_kv, uint32_t capacity,
                                        int head_dim, uint32_t position, int heads, int batch, size_t kv_seq_stride) {
    CTX_OR_FAIL();
    if (!cache || !new_kv || position >= capacity || head_dim <= 0 || heads <= 0 || batch <= 0)
        return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "kv cache update: position must be below capacity");
    Launch l = typed_launch(ctx);
    l.position = position;
    return check_cuda(ctx, launch_kv_cache_update(l, (__half*)cache, (const __half*)new_kv, nullptr, nullptr, capacity, head_dim, heads, 0, 0, 0.f, 0, 0, 0, batch, kv_seq_stride ? kv_seq_stride : (size_t)heads * capacity * head_dim), "kv cache update");
}

smelt_status smelt_cuda_rope_kv_cache_update(smelt_cuda_ctx* ctx, void* cache, const void* new_kv, const void* cos_t,
                                             const void* sin_t, uint32_t capacity, int head_dim, uint32_t position,
                                             int heads, int rope_dim, int layout, float base_log2, int math_mode,
                                             int batch, size_t kv_seq_stride) {
    CTX_OR_FAIL();
    if (!cache || !new_kv || position >= capacity || head_dim <= 0 || heads <= 0 || batch <= 0 || rope_dim > head_dim ||
        (math_mode != 1 && (!cos_t || !sin_t)))
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "rope kv cache update: bad arguments");
    Launch l = typed_launch(ctx);
    l.position = position;
    return check_cuda(ctx, launch_kv_cache_update(l, (__half*)cache, (const __half*)new_kv, (const __half*)cos_t, (const __half*)sin_t, capacity, head_dim, heads, rope_dim, layout, base_log2, math_mode, 1, 0, batch, kv_seq_stride ? kv_seq_stride : (size_t)heads * capacity * head_dim), "rope kv cache update");
}

smelt_status smelt_cuda_apply_rope(smelt_cuda_ctx* ctx, void* qk, const void* cos_t, const void* sin_t, int head_dim,
                                   int rope_dim, int heads, int layout, uint32_t position, float base_log2,
                                   int math_mode, int batch) {
    CTX_OR_FAIL();
    if (!qk || head_dim <= 0 || heads <= 0 || rope_dim > head_dim || batch <= 0 || (math_mode != 1 && (!cos_t || !sin_t)))
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "apply rope: bad arguments");
    Launch l = typed_launch(ctx);
    l.position = position;
    return check_cuda(ctx, launch_apply_rope(l, (__half*)qk, (const __half*)cos_t, (const __half*)sin_t, head_dim, rope_dim, heads, layout, base_log2, math_mode, 0, batch), "apply rope");
}

smelt_status smelt_cuda_rms_norm_1pw(smelt_cuda_ctx* ctx, const void* x, const void* w, void* y, int dim, float eps,
                                     int batch) {
    CTX_OR_FAIL();
    if (!x || !w || !y || dim <= 0 || batch <= 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "rms norm: bad arguments");
    return check_cuda(ctx, launch_rms_norm_1pw(typed_launch(ctx), (const __half*)x, (const __half*)w, (__half*)y, dim, eps, batch), "rms norm");
}
smelt_status smelt_cuda_per_head_rms_norm(smelt_cuda_ctx* ctx, const void* x, const void* w, void* y, int heads,
                                          int head_dim, float eps) {
    CTX_OR_FAIL();
    if (!x || !w || !y || heads <= 0 || head_dim <= 0 || head_dim > 1024) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "per-head rms norm: bad arguments");
    return check_cuda(ctx, launch_per_head_rms_norm(typed_launch(ctx), (const __half*)x, (const __half*)w, (__half*)y, heads, head_dim, eps), "per-head rms norm");
}
smelt_status smelt_cuda_elementwise_add(smelt_cuda_ctx* ctx, const void* a, const void* b, void* y, size_t count) {
    CTX_OR_FAIL();
    if (!a || !b || !y) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "elementwise add: null pointer");
    if (count == 0) return SMELT_OK;
    return check_cuda(ctx, launch_elementwise_add(typed_launch(ctx), (const __half*)a, (const __half*)b, (__half*)y, (int64_t)count), "elementwise add");
}
smelt_status smelt_cuda_swiglu_fused(smelt_cuda_ctx* ctx, const void* gate, const void* up, void* y, size_t count) {
    CTX_OR_FAIL();
    if (!gate || !up || !y) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "swiglu: null pointer");
    if (count == 0) return SMELT_OK;
    return check_cuda(ctx, launch_swiglu_fused(typed_launch(ctx), (const __half*)gate, (const __half*)up, (__half*)y, (int64_t)count), "swiglu");
}
smelt_status smelt_cuda_embedding_gather(smelt_cuda_ctx* ctx, const void* table, const void* token, void* y,
                                         int hidden, int batch) {
    CTX_OR_FAIL();
    if (!table || !token || !y || hidden <= 0 || batch <= 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "embedding gather: bad arguments");
    return check_cuda(ctx, launch_embedding_gather(typed_launch(ctx), (const __half*)table, (const int32_t*)token, (__half*)y, hidden, batch, 1), "embedding gather");
}
smelt_status smelt_cuda_affine_embedding_gather(smelt_cuda_ctx* ctx, const void* w, const void* s, const void* b,
                                                const void* token, void* y, int cols, int group) {
    CTX_OR_FAIL();
    if (!w || !s || !b || !token || !y || cols <= 0 || group <= 0 || cols % group || cols % 2)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "affine embedding gather: bad arguments");
    return check_cuda(ctx, launch_affine_embedding_gather(typed_launch(ctx), (const uint8_t*)w, (const __half*)s, (const __half*)b, (const int32_t*)token, (__half*)y, cols, group), "affine embedding gather");
}
smelt_status smelt_cuda_argmax_f16(smelt_cuda_ctx* ctx, const void* logits, void* out, int vocab, int batch) {
    CTX_OR_FAIL();
    if (!logits || !out || vocab <= 0 || batch <= 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "argmax: bad arguments");
    const int chunk = 2048, parts = (vocab + chunk - 1) / chunk;
    if ((size_t)parts * batch * sizeof(uint64_t) > ctx->argmax_scratch_bytes) return fail(ctx, SMELT_ERR_UNSUPPORTED, "argmax: vocab * batch too large for the scratch buffer");
    smelt_status s = check_cuda(ctx, launch_argmax_partials(typed_launch(ctx), (const __half*)logits, ctx->argmax_scratch, vocab, chunk, batch), "argmax partials");
    if (s) return s;
    return check_cuda(ctx, launch_argmax_reduce(typed_launch(ctx), ctx->argmax_scratch, (int32_t*)out, parts, batch, 1), "argmax reduce");
}

}  // extern "C"
