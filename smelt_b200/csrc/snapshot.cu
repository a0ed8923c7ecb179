// Prompt-state snapshots: the live prefix of every KV-cache slot and the whole of every other
// state slot copied into private device buffers and back, or out to host bytes.
//
// Follows SmeltRuntime.captureDevicePromptSnapshot / restoreDevicePromptSnapshot
// (Sources/SmeltRuntime/SmeltRuntime.swift:1385-1553) and, for the host form and the partial
// restore, capturePromptSnapshot / restorePromptSnapshot(_:length:) (:1254-1383): a cache slot
// is laid out [rows, capacity, head_dim] (rows = KV heads x sequences); the snapshot keeps the
// first `captured_length` positions of every row compactly ([rows, captured_length, head_dim]),
// the restore writes the first min(length, captured, destination capacity) positions of every
// row at the destination's own stride, which it derives from the slot's current size as the
// reference does (:1514-1519), so a snapshot survives a capacity change in between.  Opaque
// state slots (recurrent / convolutional state) are copied whole and cannot be rewound: a
// restore shorter than the capture is refused when the snapshot holds any (:1338-1345).
//
// All slots of a snapshot move in one launch per 32 slots: a grid of 16-byte copies driven by
// a descriptor table in the kernel's arguments (the reference issues one blit per head).
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"
#include "runtime.h"

struct smelt_cuda_snapshot {
    struct Part {
        int32_t slot;
        int32_t rows;         // cache: KV heads x sequences; whole slot: 1
        int32_t head_dim;     // cache only
        uint32_t length;      // cache: positions kept per row; whole slot: 0
        uint64_t bytes;       // bytes held for this slot
        uint64_t offset;      // into the snapshot's device buffer (256-byte aligned)
        int32_t whole;
    };
    int device = 0;
    uint32_t captured_length = 0;
    uint32_t prompt_length = 0;
    int32_t next_token = 0;
    std::vector<Part> parts;
    void* data = nullptr;
    size_t data_bytes = 0;
    bool has_opaque = false;
};

namespace smelt {
namespace {

constexpr int kCopiesPerLaunch = 32;
constexpr uint32_t kBlobMagic = 0x50534D53u;  // "SMSP"
constexpr uint32_t kBlobVersion = 1;

// rows of row_bytes bytes each, source and destination with their own pitch; all multiples of 16
struct RowCopy {
    const uint8_t* src;
    uint8_t* dst;
    uint64_t src_pitch, dst_pitch, row_bytes;
    uint32_t rows;
};
struct RowCopyBatch {
    RowCopy c[kCopiesPerLaunch];
    int n;
};

__global__ void __launch_bounds__(256) row_copy_kernel(const RowCopyBatch b) {
    const RowCopy& c = b.c[blockIdx.y];
    const uint64_t per_row = c.row_bytes / 16, total = per_row * c.rows;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = i / per_row, k = i % per_row;
        const uint4 v = __ldcs(reinterpret_cast<const uint4*>(c.src + r * c.src_pitch) + k);
        __stcs(reinterpret_cast<uint4*>(c.dst + r * c.dst_pitch) + k, v);
    }
}

smelt_status run_copies(smelt_cuda_ctx* ctx, const std::vector<RowCopy>& copies, const char* what) {
    for (size_t i0 = 0; i0 < copies.size(); i0 += kCopiesPerLaunch) {
        RowCopyBatch b = {};
        b.n = (int)std::min<size_t>(kCopiesPerLaunch, copies.size() - i0);
        uint64_t most = 0;
        for (int i = 0; i < b.n; ++i) {
            b.c[i] = copies[i0 + i];
            const uint64_t units = b.c[i].row_bytes / 16 * b.c[i].rows;
            most = units > most ? units : most;
        }
        if (most == 0) continue;
        const int sm = ctx->sm_count > 0 ? ctx->sm_count : 148;
        uint64_t gx = (most + 255) / 256;
        const uint64_t cap = (uint64_t)(8 * sm + b.n - 1) / b.n;  // about eight resident CTAs per SM over all slots
        if (gx > cap) gx = cap;
        if (gx < 1) gx = 1;
        prefer_max_shared(row_copy_kernel);
        row_copy_kernel<<<dim3((unsigned)gx, (unsigned)b.n), 256, 0, ctx->stream>>>(b);
        smelt_status s = check_cuda(ctx, cudaGetLastError(), what);
        if (s) return s;
    }
    return SMELT_OK;
}

size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

}  // namespace
}  // namespace smelt

using namespace smelt;

extern "C" {

smelt_status smelt_cuda_snapshot_capture(smelt_cuda_ctx* ctx, const smelt_cuda_kv_slot* kv_slots, int n_kv,
                                         const int32_t* state_slots, int n_state, uint32_t captured_length,
                                         uint32_t prompt_length, int32_t next_token, smelt_cuda_snapshot** out) {
    if (!ctx || !out || n_kv < 0 || n_state < 0 || (n_kv && !kv_slots) || (n_state && !state_slots)) return SMELT_ERR_BAD_ARGUMENT;
    *out = nullptr;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (ctx->capturing) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "snapshot capture: a stream capture is open");
    const uint32_t limit = ctx->configured ? ctx->cfg.context_limit : 0xFFFFFFFFu;
    const uint32_t length = captured_length < limit ? captured_length : limit;  // clamped as the reference clamps (:1260)
    auto snap = new smelt_cuda_snapshot();
    snap->device = ctx->device;
    snap->captured_length = length;
    snap->prompt_length = prompt_length < limit ? prompt_length : limit;
    snap->next_token = next_token;
    std::vector<RowCopy> copies;
    size_t off = 0;
    auto bad = [&](smelt_status code, const std::string& msg) {
        delete snap;
        return fail(ctx, code, msg);
    };
    for (int i = 0; i < n_kv; ++i) {
        const smelt_cuda_kv_slot& k = kv_slots[i];
        if (k.slot < 0 || k.slot >= (int)ctx->slots.size() || !ctx->slots[k.slot].ptr) continue;  // absent slots are skipped (:1484-1487)
        if (k.rows <= 0 || k.head_dim <= 0 || (k.head_dim * 2) % 16 != 0)
            return bad(SMELT_ERR_BAD_ARGUMENT, "snapshot capture: cache slot " + std::to_string(k.slot) + " needs rows > 0 and head_dim a multiple of 8");
        const Slot& sl = ctx->slots[k.slot];
        const size_t pos_bytes = (size_t)k.head_dim * 2;
        const size_t stride = sl.bytes / ((size_t)k.rows * pos_bytes);  // positions per row now (:1437-1441)
        if (stride == 0) return bad(SMELT_ERR_BAD_ARGUMENT, "snapshot capture: cache slot " + std::to_string(k.slot) + " is smaller than one position per row");
        const uint32_t live = length < stride ? length : (uint32_t)stride;
        smelt_cuda_snapshot::Part p = {};
        p.slot = k.slot; p.rows = k.rows; p.head_dim = k.head_dim; p.length = live; p.whole = 0;
        p.bytes = (uint64_t)k.rows * live * pos_bytes;
        p.offset = off;
        off += align256(p.bytes);
        snap->parts.push_back(p);
    }
    for (int i = 0; i < n_state; ++i) {
        const int s = state_slots[i];
        if (s < 0 || s >= (int)ctx->slots.size() || !ctx->slots[s].ptr || ctx->slots[s].bytes == 0) continue;
        if (ctx->slots[s].bytes % 16 != 0) return bad(SMELT_ERR_BAD_ARGUMENT, "snapshot capture: state slot " + std::to_string(s) + " is not a multiple of 16 bytes");
        smelt_cuda_snapshot::Part p = {};
        p.slot = s; p.rows = 1; p.whole = 1; p.bytes = ctx->slots[s].bytes; p.offset = off;
        off += align256(p.bytes);
        snap->parts.push_back(p);
        snap->has_opaque = true;
    }
    snap->data_bytes = off;
    if (off) {
        cudaError_t e = cudaMalloc(&snap->data, off);
        if (e != cudaSuccess) return bad(SMELT_ERR_ALLOC, "snapshot capture: could not allocate " + std::to_string(off) + " bytes (" + cudaGetErrorString(e) + ")");
    }
    for (const auto& p : snap->parts) {
        const Slot& sl = ctx->slots[p.slot];
        RowCopy c = {};
        c.src = (const uint8_t*)sl.ptr;
        c.dst = (uint8_t*)snap->data + p.offset;
        if (p.whole) {
            c.rows = 1; c.row_bytes = p.bytes; c.src_pitch = c.dst_pitch = p.bytes;
        } else {
            const size_t pos_bytes = (size_t)p.head_dim * 2;
            c.rows = (uint32_t)p.rows;
            c.row_bytes = (uint64_t)p.length * pos_bytes;
            c.src_pitch = sl.bytes / ((size_t)p.rows * pos_bytes) * pos_bytes;
            c.dst_pitch = c.row_bytes;
        }
        copies.push_back(c);
    }
    smelt_status s = run_copies(ctx, copies, "snapshot capture");
    if (!s) s = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "snapshot capture");
    if (s) {
        cudaFree(snap->data);
        delete snap;
        return s;
    }
    *out = snap;
    return SMELT_OK;
}

smelt_status smelt_cuda_snapshot_restore(smelt_cuda_ctx* ctx, const smelt_cuda_snapshot* snap, uint32_t length) {
    if (!ctx || !snap) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (ctx->capturing) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "snapshot restore: a stream capture is open");
    if (snap->device != ctx->device) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "snapshot restore: the snapshot lives on another device");
    if (length > snap->captured_length)
        return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "restore length " + std::to_string(length) + " outside [0, " + std::to_string(snap->captured_length) + "]");
    if (length < snap->captured_length && snap->has_opaque)
        return fail(ctx, SMELT_ERR_UNSUPPORTED, "partial restore (length " + std::to_string(length) + " < captured " + std::to_string(snap->captured_length) +
                                                    ") of a snapshot that holds position-less state slots");
    std::vector<RowCopy> copies;
    for (const auto& p : snap->parts) {
        if (p.slot < 0 || p.slot >= (int)ctx->slots.size() || !ctx->slots[p.slot].ptr) continue;  // (:1488-1490)
        const Slot& sl = ctx->slots[p.slot];
        RowCopy c = {};
        c.src = (const uint8_t*)snap->data + p.offset;
        c.dst = (uint8_t*)sl.ptr;
        if (p.whole) {
            const uint64_t n = (p.bytes < sl.bytes ? p.bytes : (uint64_t)sl.bytes) & ~(uint64_t)15;
            c.rows = 1; c.row_bytes = n; c.src_pitch = c.dst_pitch = n;
        } else {
            const size_t pos_bytes = (size_t)p.head_dim * 2;
            const size_t dst_stride = sl.bytes / ((size_t)p.rows * pos_bytes);
            if (dst_stride == 0) continue;
            uint32_t live = length < p.length ? length : p.length;
            if (live > dst_stride) live = (uint32_t)dst_stride;  // the caller grows the cache first when it wants the whole prefix (:1348-1355)
            c.rows = (uint32_t)p.rows;
            c.row_bytes = (uint64_t)live * pos_bytes;
            c.src_pitch = (uint64_t)p.length * pos_bytes;
            c.dst_pitch = (uint64_t)dst_stride * pos_bytes;
        }
        copies.push_back(c);
    }
    smelt_status s = run_copies(ctx, copies, "snapshot restore");
    return s ? s : check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "snapshot restore");
}

smelt_status smelt_cuda_snapshot_info(const smelt_cuda_snapshot* snap, smelt_cuda_snapshot_info_t* out) {
    if (!snap || !out) return SMELT_ERR_BAD_ARGUMENT;
    out->captured_length = snap->captured_length;
    out->prompt_length = snap->prompt_length;
    out->next_token = snap->next_token;
    out->n_slots = (uint32_t)snap->parts.size();
    uint64_t total = 0;
    for (const auto& p : snap->parts) total += p.bytes;
    out->byte_count = total;
    // blob: header (8 words) + one 40-byte record per slot, padded to 16, then each slot's bytes padded to 16
    uint64_t blob = 32 + (uint64_t)snap->parts.size() * 40;
    blob = (blob + 15) & ~(uint64_t)15;
    for (const auto& p : snap->parts) blob += (p.bytes + 15) & ~(uint64_t)15;
    out->blob_bytes = blob;
    return SMELT_OK;
}

smelt_status smelt_cuda_snapshot_export(smelt_cuda_ctx* ctx, const smelt_cuda_snapshot* snap, void* dst, size_t dst_bytes) {
    if (!ctx || !snap || !dst) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    smelt_cuda_snapshot_info_t info;
    smelt_cuda_snapshot_info(snap, &info);
    if (dst_bytes < info.blob_bytes) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "snapshot export: " + std::to_string(info.blob_bytes) + " bytes are needed");
    uint8_t* o = (uint8_t*)dst;
    const uint32_t head[8] = {kBlobMagic, kBlobVersion, snap->captured_length, snap->prompt_length, (uint32_t)snap->next_token,
                              (uint32_t)snap->parts.size(), 0u, 0u};
    std::memcpy(o, head, 32);
    size_t at = 32;
    for (const auto& p : snap->parts) {
        const uint32_t rec[10] = {(uint32_t)p.slot, (uint32_t)p.rows, (uint32_t)p.head_dim, p.length, (uint32_t)p.whole, 0u,
                                  (uint32_t)(p.bytes & 0xFFFFFFFFu), (uint32_t)(p.bytes >> 32), 0u, 0u};
        std::memcpy(o + at, rec, 40);
        at += 40;
    }
    at = (at + 15) & ~(size_t)15;
    for (const auto& p : snap->parts) {
        if (p.bytes) {
            cudaError_t e = cudaMemcpyAsync(o + at, (const uint8_t*)snap->data + p.offset, p.bytes, cudaMemcpyDeviceToHost, ctx->stream);
            if (e != cudaSuccess) return check_cuda(ctx, e, "snapshot export");
        }
        at += (p.bytes + 15) & ~(size_t)15;
    }
    return check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "snapshot export");
}

smelt_status smelt_cuda_snapshot_import(smelt_cuda_ctx* ctx, const void* src, size_t src_bytes, smelt_cuda_snapshot** out) {
    if (!ctx || !src || !out) return SMELT_ERR_BAD_ARGUMENT;
    *out = nullptr;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    const uint8_t* in = (const uint8_t*)src;
    uint32_t head[8];
    if (src_bytes < 32) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "snapshot import: truncated header");
    std::memcpy(head, in, 32);
    if (head[0] != kBlobMagic || head[1] != kBlobVersion) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "snapshot import: not a snapshot of this library (magic / version)");
    const uint32_t n = head[5];
    if (n > 65536 || src_bytes < 32 + (size_t)n * 40) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "snapshot import: truncated slot table");
    auto snap = new smelt_cuda_snapshot();
    snap->device = ctx->device;
    snap->captured_length = head[2]; snap->prompt_length = head[3]; snap->next_token = (int32_t)head[4];
    size_t at = 32, off = 0;
    for (uint32_t i = 0; i < n; ++i) {
        uint32_t rec[10];
        std::memcpy(rec, in + at, 40);
        at += 40;
        smelt_cuda_snapshot::Part p = {};
        p.slot = (int32_t)rec[0]; p.rows = (int32_t)rec[1]; p.head_dim = (int32_t)rec[2]; p.length = rec[3]; p.whole = (int32_t)rec[4];
        p.bytes = (uint64_t)rec[6] | ((uint64_t)rec[7] << 32);
        const bool cache_ok = !p.whole && p.rows > 0 && p.head_dim > 0 && (p.head_dim * 2) % 16 == 0 && p.length <= snap->captured_length &&
                              p.bytes == (uint64_t)p.rows * p.length * p.head_dim * 2;
        const bool whole_ok = p.whole == 1 && p.bytes % 16 == 0;
        if (!cache_ok && !whole_ok) {
            delete snap;
            return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "snapshot import: slot record " + std::to_string(i) + " is inconsistent");
        }
        p.offset = off;
        off += align256(p.bytes);
        snap->has_opaque = snap->has_opaque || p.whole;
        snap->parts.push_back(p);
    }
    at = (at + 15) & ~(size_t)15;
    size_t need = at;
    for (const auto& p : snap->parts) need += (p.bytes + 15) & ~(size_t)15;
    if (src_bytes < need) {
        delete snap;
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "snapshot import: " + std::to_string(need) + " bytes expected, " + std::to_string(src_bytes) + " given");
    }
    snap->data_bytes = off;
    if (off && cudaMalloc(&snap->data, off) != cudaSuccess) {
        delete snap;
        return fail(ctx, SMELT_ERR_ALLOC, "snapshot import: could not allocate " + std::to_string(off) + " bytes");
    }
    for (const auto& p : snap->parts) {
        if (p.bytes) cudaMemcpyAsync((uint8_t*)snap->data + p.offset, in + at, p.bytes, cudaMemcpyHostToDevice, ctx->stream);
        at += (p.bytes + 15) & ~(size_t)15;
    }
    smelt_status s = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "snapshot import");
    if (s) {
        cudaFree(snap->data);
        delete snap;
        return s;
    }
    *out = snap;
    return SMELT_OK;
}

void smelt_cuda_snapshot_destroy(smelt_cuda_snapshot* snap) {
    if (!snap) return;
    cudaSetDevice(snap->device);
    if (snap->data) cudaFree(snap->data);
    delete snap;
}

}  // extern "C"
