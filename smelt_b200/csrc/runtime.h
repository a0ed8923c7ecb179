// Internal state of a libsmelt_cuda context (host side).
#pragma once

#include <string>
#include <vector>

#include "../../include/smelt_cuda.h"
#include "common.cuh"

namespace smelt {

struct Slot {
    void* ptr = nullptr;
    size_t bytes = 0;
};

enum PipeKind : int {
    PK_NONE = 0,
    PK_AFFINE_MATVEC,
    PK_AFFINE_ADD,
    PK_AFFINE_GATEUP,
    PK_AFFINE_DUAL,
    PK_FP16_MATVEC,
    PK_EMBEDDING_GATHER,
    PK_AFFINE_EMBEDDING_GATHER,
    PK_ARGMAX_PARTIALS,
    PK_ARGMAX_REDUCE,
    PK_ARGMAX_SINGLE,
    PK_SIGNED_MATVEC,
    PK_SIGNED_ADD,
    PK_SIGNED_GATEUP,
    PK_SIGNED_TERNARY_AFFINE,
    PK_KV_UPDATE,
    PK_APPLY_ROPE,
    PK_ROPE_KV_UPDATE,
    PK_ATTN_GENERIC,
    PK_ATTN_INPLACE,
    PK_ATTN_MLX_2PASS_1,
    PK_ATTN_MLX_2PASS_2,
    PK_RMS_NORM,
    PK_PER_HEAD_NORM,
    PK_ADD,
    PK_SWIGLU,
    PK_TP_ALL_REDUCE,
    PK_FUSED_NORM_QKV,
    PK_FUSED_NORM_GATEUP,
    PK_ROPE_QKV_APPEND,
    PK_ATTN_ROPE,
    PK_TP_REDUCE_ADD,
    PK_TP_ARGMAX,
    PK_CONV1D_SILU,
    PK_RMS_SCALE_QK,
    PK_DELTANET_DECODE,
    PK_RMS_NORM_GATED,
    PK_CONV1D_SILU_PREFILL,
    PK_DELTANET_PREFILL,
    PK_BITPLANE_PRODUCER,
    PK_BITPLANE_SWIGLU_PRODUCER,
    PK_BITPLANE_SIGMOID_MUL_PRODUCER,
    PK_BITPLANE_NORM_SCALE_PRODUCER,
    PK_BITPLANE_GATED_NORM_PRODUCER,
    PK_SIGNED_EMBEDDING_GATHER,
    PK_SIGNED_BANK,
    PK_SIGNED_TERNARY_AFFINE_ADD,
    PK_SIGNED_TERNARY_AFFINE_GATEUP,
    PK_ELEMENTWISE,
    PK_GATE_SPLIT,
    PK_HEAD_NORM,
    PK_ROW_NORM,
    PK_ROPE_KV_PREFILL,
    PK_ATTN_PREFILL,
    PK_EMBEDDING_GATHER_BATCHED,
    PK_AFFINE_EMBEDDING_GATHER_BATCHED,
    PK_BITPLANE_BANK4,
    PK_BITPLANE_MATVEC,
    PK_BITPLANE_ADD,
    PK_BITPLANE_GATEUP,
    PK_DN_GATES,
    PK_DN_STATE_UPDATE,
    PK_DN_READOUT,
    PK_DN_DELTA,
    PK_DN_FUSED_DECODE,
    PK_DN_FUSED_PREFILL,
};

struct Pipeline {
    PipeKind kind = PK_NONE;
    std::string name;
    int cols = 0, rows = 0, group = 0;  // from "name:cols:group" or "_c{C}_r{R}_g{G}"
    bool fixed_shape = false;            // rows come from the name, no numRows constant
    bool batched = false;                // x is [B, C], an actualBatch constant is bound
    int bits = 0;                        // signed kernels: 1 or 2
    int planes = 0;                      // activation bit-plane kernels: planes of the view (2..6)
    int n_q = 0, n_kv = 0, head_dim = 0; // shape-specialised attention names
};

// Parses a manifest pipeline entry; returns false when the kernel is not implemented.
bool parse_pipeline(const char* entry, Pipeline* out);

}  // namespace smelt

struct smelt_package_state;

struct smelt_cuda_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    std::string err;
    std::vector<smelt::Slot> slots;
    std::vector<smelt::Pipeline> pipelines;
    smelt_cuda_runtime_config cfg = {};
    bool configured = false;
    bool pdl = true;

    smelt::DynState* dyn_dev = nullptr;  // {token, position} read by graph-replayed kernels
    uint32_t* err_dev = nullptr;         // device error word
    void* attn_scratch = nullptr;
    size_t attn_scratch_bytes = 0;
    float* rope_table = nullptr;   // cos | sin of the current position (256 floats), written once per interpretation
    float* qmm_scratch = nullptr;  // tensor-memory QMM: fp32 sums of CTAs that split a row tile's K (affine_qmm.cu)
    size_t qmm_scratch_bytes = 0;
    void* prefill_scratch = nullptr;  // activations of one prompt chunk (prefill.cu), grown on demand
    size_t prefill_scratch_bytes = 0;
    int* qmm_counters = nullptr;   // ... and their arrival counters (4096), zero between launches
    int* attn_counters = nullptr;  // one zeroed int per (sequence, KV head): in-kernel merge of attention splits
    uint64_t* argmax_scratch = nullptr;
    size_t argmax_scratch_bytes = 0;

    int32_t* h_pinned = nullptr;  // pinned staging: tokens in, tokens out
    size_t h_pinned_count = 0;

    // graph replay
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t graph_exec = nullptr;
    cudaGraph_t graph_burst = nullptr;            // kGraphBurst tokens per launch
    cudaGraphExec_t graph_burst_exec = nullptr;
    cudaGraphExec_t user_graph_exec = nullptr;  // smelt_cuda_capture_begin / _end / _replay
    int32_t* gen_ring = nullptr;   // device: generated ids, step-major
    uint32_t* gen_count = nullptr; // device: steps written
    uint32_t gen_capacity = 0;
    int launch_count = 0;
    uint32_t graph_next_pos = 0;   // host mirror of the device position the next replay decodes at
    bool graph_pos_known = false;  // set by graph_seed / graph_step
    bool capturing = false;
    cudaEvent_t ev_start = nullptr, ev_stop = nullptr;

    // tensor parallel
    void* nccl_comm = nullptr;
    void* tp_peer = nullptr;   // peer-memory exchange state (tp.cu)
    int tp_rank = 0, tp_world = 1;
    smelt_package_state* package = nullptr;  // decode table of the open .smeltpkg (package_reader.cu)
};

namespace smelt {
constexpr int kGraphBurst = 8;  // tokens per launch of the multi-token decode graph
void destroy_decode_graphs(smelt_cuda_ctx* ctx);  // the single-token and the multi-token graph
smelt_status fail(smelt_cuda_ctx* ctx, smelt_status code, const std::string& msg);
smelt_status check_cuda(smelt_cuda_ctx* ctx, cudaError_t e, const char* what);
smelt_status tp_all_reduce_f16(smelt_cuda_ctx* ctx, void* data, size_t count, cudaStream_t stream);
void tp_destroy(smelt_cuda_ctx* ctx);
void package_destroy(smelt_cuda_ctx* ctx);
smelt_status tp_argmax(smelt_cuda_ctx* ctx, const Launch& l, const void* partials, void* out, int n, uint32_t offset, int batch);
smelt_status tp_reduce_add(smelt_cuda_ctx* ctx, const Launch& l, const void* partial, const void* residual, void* out, size_t count,
                           bool* handled);
}  // namespace smelt
