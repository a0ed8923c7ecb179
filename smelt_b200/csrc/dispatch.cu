// Pipeline registry, SmeltDispatchRecord interpreter, per-token decode step and CUDA-graph replay.
//
// The interpreter keeps the contract of SmeltRuntime.emitDecodeDispatchRecord
// (Sources/SmeltRuntime/SmeltRuntime.swift:3187-3247): buffers are bound by binding index from
// slot-indexed allocations at literal or position-scaled byte offsets, constants are resolved
// by kind, guard constants may skip the dispatch, swap records exchange cur and alt.  What a
// kernel name means (which binding is which operand) follows the Metal kernel signatures the
// handlers cite.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "affine_matvec.h"
#include "glue.h"
#include "runtime.h"

using namespace smelt;

static_assert(sizeof(smelt_buffer_record) == 16, "SmeltBufferRecord is 16 bytes");
static_assert(sizeof(smelt_constant_record) == 8, "SmeltConstantRecord is 8 bytes");
static_assert(sizeof(smelt_dispatch_record) == 360, "SmeltDispatchRecord is 360 bytes");
static_assert(offsetof(smelt_dispatch_record, pipeline) == 2 && offsetof(smelt_dispatch_record, style) == 4 &&
                  offsetof(smelt_dispatch_record, buffer_count) == 5 && offsetof(smelt_dispatch_record, constant_count) == 6 &&
                  offsetof(smelt_dispatch_record, min_seq_len) == 8 && offsetof(smelt_dispatch_record, grid) == 12 &&
                  offsetof(smelt_dispatch_record, threadgroup) == 24 && offsetof(smelt_dispatch_record, buf) == 40 &&
                  offsetof(smelt_dispatch_record, con) == 296,
              "SmeltDispatchRecord field offsets");

namespace smelt {

namespace {

bool starts_with(const std::string& s, const char* p) { return s.rfind(p, 0) == 0; }

// Consumes "_c{C}_r{R}_g{G}" at the front of `rest`.
bool parse_shape(std::string& rest, Pipeline* p) {
    int c = 0, r = 0, g = 0, n = 0;
    if (sscanf(rest.c_str(), "_c%d_r%d_g%d%n", &c, &r, &g, &n) == 3 && n > 0) {
        p->cols = c; p->rows = r; p->group = g; p->fixed_shape = true;
        rest = rest.substr(n);
        return true;
    }
    return false;
}

// The row norms of norms.metal beyond rms_norm_1pw.  form = the binding layout:
//   0: 0 in, 1 weight, 2 out, 3 dim, 4 eps (rows = grid.x)          1: 0 in, 1 weight, 2 out
//   2: 0 in, 1 weight, 2 residual, 3 out                            3: 0 in, 1 weight, 2 residual, 3 scalar, 4 out
//   4: 0 in, 1 scale out, 2 dim, 3 eps                              5: 0 in, 1 scale out
//   6: 0 a, 1 b, 2 out (a + b), 3 scale out, 4 dim, 5 eps           7: 0 data (in place), 1 headDim, 2 eps (rows = grid.x)
//   8: 0 data (in place)
//   9: 0 qkv (in place), 1 headDim, 2 eps, 3 qkvDim, 4 qkHeads; grid (qkHeads, positions); dim < 0: the K heads, which follow the Q heads
//  10: 0 qkv (in place) with headDim 128, qkvDim 6144, 16 heads fixed; grid (16, positions)
struct RowNormName { const char* name; int dim, topology, value, scale, form; float eps; bool batched; };
constexpr int kT4 = SMELT_ROW_NORM_TILES4, kQ2 = SMELT_ROW_NORM_QUADS2, kST = SMELT_ROW_NORM_STRIDED;
const RowNormName kRowNorms[] = {
    {"rms_norm_1pw_batched", 0, kT4, 1, 0, 0, 0.0f, true},
    {"rms_norm_1pw_d2048", 2048, kQ2, 2, 0, 1, 1e-6f, false},
    {"rms_norm_1pw_d1024", 1024, kQ2, 2, 0, 1, 1e-6f, false},
    {"rms_norm_1pw_d1024_batched", 1024, kQ2, 2, 0, 1, 1e-6f, true},
    {"rms_norm_1pw_d1536", 1536, kQ2, 2, 0, 1, 1e-6f, false},
    {"rms_norm_1pw_d1536_add", 1536, kQ2, 2, 0, 2, 1e-6f, false},
    {"rms_norm_1pw_d1536_batched", 1536, kQ2, 2, 0, 1, 1e-6f, true},
    {"rms_norm_1pw_d1536_add_batched", 1536, kQ2, 2, 0, 2, 1e-6f, true},
    {"rms_norm_1pw_d2560", 2560, kQ2, 2, 0, 1, 1e-6f, false},
    {"rms_norm_1pw_d2560_add", 2560, kQ2, 2, 0, 2, 1e-6f, false},
    {"rms_norm_1pw_d2560_batched", 2560, kQ2, 2, 0, 1, 1e-6f, true},
    {"rms_norm_1pw_d2560_add_batched", 2560, kQ2, 2, 0, 2, 1e-6f, true},
    {"rms_norm_1pw_d256_add", 256, kST, 3, 0, 2, 1e-6f, false},
    {"rms_norm_1pw_d256_add_scalar_weight", 256, kST, 3, 0, 3, 1e-6f, false},
    {"rms_norm_scale_only", 0, kST, 0, 0, 4, 0.0f, false},
    {"rms_norm_scale_only_precise", 0, kST, 0, 0, 4, 0.0f, false},
    {"rms_norm_scale_only_d1536", 1536, kQ2, 0, 0, 5, 1e-6f, false},
    {"rms_norm_scale_only_d2560", 2560, kQ2, 0, 0, 5, 1e-6f, false},
    {"rms_norm_scale_only_d1024_batched", 1024, kQ2, 0, 0, 5, 1e-6f, true},
    {"rms_norm_scale_only_d2048_batched", 2048, kST, 0, 0, 5, 1e-6f, true},
    {"rms_norm_scale_only_d2048_eps1e5_batched", 2048, kST, 0, 0, 5, 1e-5f, true},
    {"rms_norm_scale_only_d2560_batched", 2560, kST, 0, 0, 5, 1e-6f, true},
    {"rms_norm_scale_only_d3072_eps1e5_batched", 3072, kST, 0, 0, 5, 1e-5f, true},
    {"residual_add_rms_norm_scale_only_precise", 0, kST, 0, 0, 6, 0.0f, false},
    {"l2_normalize", 0, kST, 4, 1, 7, 0.0f, true},
    {"l2_normalize_d128", 128, kST, 4, 1, 8, 1e-6f, true},
    // the Q / K heads of a prompt chunk's qkv rows (norms.metal:1192-1378)
    {"l2_normalize_q_prefill", 0, kST, 4, 1, 9, 0.0f, true},
    {"l2_normalize_k_prefill", -1, kST, 4, 1, 9, 0.0f, true},
    {"l2_normalize_q_d128_c6144_h16_prefill", 128, kST, 4, 1, 10, 1e-6f, true},
    {"l2_normalize_k_d128_c6144_h16_prefill", -128, kST, 4, 1, 10, 1e-6f, true},
};
constexpr int kRowNormCount = (int)(sizeof(kRowNorms) / sizeof(kRowNorms[0]));

bool parse_affine(const std::string& name, const char* base, PipeKind kind, Pipeline* p) {
    if (!starts_with(name, base)) return false;
    std::string rest = name.substr(strlen(base));
    if (!rest.empty() && rest[0] != '_') return false;
    Pipeline q = *p;
    q.kind = kind;
    if (!rest.empty()) {
        if (!parse_shape(rest, &q)) return false;
        if (starts_with(rest, "_rows4_sg1")) rest = rest.substr(10);  // row-tile forms of the same kernel (lut_matvec.metal:7727-7742, :8701-8738)
        else if (starts_with(rest, "_rows4") || starts_with(rest, "_rows8")) rest = rest.substr(6);
        if (starts_with(rest, "_batched")) { q.batched = true; rest.clear(); }  // _batched, _batched_full, _batched_tile3, _batched_sg4_bt5, _batched_ext_b5 ...
        if (!rest.empty()) return false;
    }
    *p = q;
    return true;
}

}  // namespace

bool parse_pipeline(const char* entry, Pipeline* out) {
    if (!entry || !out) return false;
    Pipeline p;
    std::string e(entry);
    std::string name = e;
    size_t colon = e.find(':');
    if (colon != std::string::npos) {
        name = e.substr(0, colon);
        int c = 0, g = 0;
        if (sscanf(e.c_str() + colon, ":%d:%d", &c, &g) != 2 || c <= 0 || g <= 0) return false;
        p.cols = c; p.group = g;
    }
    p.name = name;
    // Longest prefixes first.
    if (parse_affine(name, "fused_affine_gate_up_swiglu", PK_AFFINE_GATEUP, &p) ||
        parse_affine(name, "fused_affine_matvec_add", PK_AFFINE_ADD, &p) ||
        parse_affine(name, "fused_dual_affine_matvec", PK_AFFINE_DUAL, &p) ||
        parse_affine(name, "affine_matvec", PK_AFFINE_MATVEC, &p)) {
        if (p.cols <= 0 || (p.group != 32 && p.group != 64 && p.group != 128) || p.cols % p.group) return false;
        *out = p;
        return true;
    }
    // Fused extension kernels emitted by the decoder builder's fused table (group 64 only).
    if (name == "smelt_rmsnorm_affine_qkv" || name == "smelt_rmsnorm_affine_gate_up_swiglu") {
        if (p.cols <= 0 || p.group != 64 || p.cols % 1024) return false;
        p.kind = name == "smelt_rmsnorm_affine_qkv" ? PK_FUSED_NORM_QKV : PK_FUSED_NORM_GATEUP;
        *out = p;
        return true;
    }
    struct Simple { const char* name; PipeKind kind; int bits; bool batched; };
    static const Simple table[] = {
        {"fp16_matvec", PK_FP16_MATVEC, 0, false},
        {"embedding_gather", PK_EMBEDDING_GATHER, 0, false},
        {"affine_embedding_gather", PK_AFFINE_EMBEDDING_GATHER, 0, false},
        {"argmax_fp16_partials", PK_ARGMAX_PARTIALS, 0, false},
        {"argmax_key_reduce", PK_ARGMAX_REDUCE, 0, false},
        {"argmax_fp16", PK_ARGMAX_SINGLE, 0, false},
        {"signed_binary_matvec_g128_rows8", PK_SIGNED_MATVEC, 1, false},
        {"signed_binary_matvec_g128_rows8_batched_b4", PK_SIGNED_MATVEC, 1, true},
        {"signed_ternary_matvec_g128_rows8", PK_SIGNED_MATVEC, 2, false},
        {"signed_ternary_matvec_g128_rows8_batched_b4", PK_SIGNED_MATVEC, 2, true},
        {"signed_binary_matvec_add_g128_rows8", PK_SIGNED_ADD, 1, false},
        {"signed_binary_gate_up_swiglu_g128_rows8", PK_SIGNED_GATEUP, 1, false},
        {"signed_binary_gate_up_swiglu_g128_rows8_batched_b4", PK_SIGNED_GATEUP, 1, true},
        {"signed_ternary_affine_matvec_g128_rows8", PK_SIGNED_TERNARY_AFFINE, 2, false},
        // the other MLX-affine ternary forms (signed_quant_precise.metal:113-420): the bias scales repeat the scales, so they
        // are the ternary kernels with one more binding
        {"signed_ternary_affine_matvec_add_g128_rows8", PK_SIGNED_TERNARY_AFFINE_ADD, 2, false},
        {"signed_ternary_affine_gate_up_swiglu_g128_rows8", PK_SIGNED_TERNARY_AFFINE_GATEUP, 2, false},
        {"signed_ternary_affine_qmm_g128_bm32_bn32_bk32", PK_SIGNED_TERNARY_AFFINE, 2, true},
        {"signed_ternary_affine_bank4_matvec_g128_rows8", PK_SIGNED_BANK, 3, false},
        // projection banks: the standalone matvec over a larger row space, outputs handed to their consumers
        // (signed_quant.metal:2634-2960); bits = layout: 0 two weight tensors, 1 one slab and two outputs, 2 one slab and four
        {"signed_binary_dual_matvec_g128_rows8", PK_SIGNED_BANK, 0, false},
        {"signed_binary_virtual_bank_matvec_g128_rows8", PK_SIGNED_BANK, 0, false},
        {"signed_binary_packed_bank_matvec_g128_rows8", PK_SIGNED_BANK, 1, false},
        {"signed_binary_packed_bank4_matvec_g128_rows8", PK_SIGNED_BANK, 2, false},
        {"signed_binary_embedding_gather_g128", PK_SIGNED_EMBEDDING_GATHER, 1, false},
        {"signed_ternary_embedding_gather_g128", PK_SIGNED_EMBEDDING_GATHER, 2, false},
        // element-wise kernels (activations.metal:4-210, activations_precise.metal:22-35): bits = the operation
        {"silu", PK_ELEMENTWISE, kEwSilu, false},
        {"sigmoid_kernel", PK_ELEMENTWISE, kEwSigmoid, false},
        {"softplus", PK_ELEMENTWISE, kEwSoftplus, false},
        {"buffer_copy", PK_ELEMENTWISE, kEwCopy, false},
        {"scalar_mul", PK_ELEMENTWISE, kEwScalarMul, false},
        {"scalar_mul_weight", PK_ELEMENTWISE, kEwScalarMul, true},
        {"logit_cap", PK_ELEMENTWISE, kEwLogitCap, false},
        {"elementwise_mul", PK_ELEMENTWISE, kEwMul, false},
        {"sigmoid_mul", PK_ELEMENTWISE, kEwSigmoidMul, false},
        {"geglu_fused", PK_ELEMENTWISE, kEwGeglu, false},
        {"geglu_fused_strided_batched", PK_ELEMENTWISE, kEwGeglu, true},
        {"projection_bias_add_batched", PK_ELEMENTWISE, kEwBiasAdd, true},
        {"gate_split", PK_GATE_SPLIT, 0, false},
        // per-head norms (attention_fused.metal:38-330): bits = the form
        {"per_head_rms_norm_1pw", PK_HEAD_NORM, kHeadNorm1pw, false},
        {"per_head_rms_norm_noscale", PK_HEAD_NORM, kHeadNormNoScale, false},
        {"per_head_rms_norm_batched", PK_HEAD_NORM, kHeadNormDirect, true},
        {"per_head_rms_norm_1pw_batched", PK_HEAD_NORM, kHeadNorm1pw, true},
        {"per_head_rms_norm_noscale_batched", PK_HEAD_NORM, kHeadNormNoScale, true},
        {"embedding_gather_batched", PK_EMBEDDING_GATHER_BATCHED, 0, true},
        {"affine_embedding_gather_batched", PK_AFFINE_EMBEDDING_GATHER_BATCHED, 0, true},
        // prompt chunks (prefill_rope_kv.metal:64-187, prefill_rope_kv_precise.metal:8-60, prefill_attention.metal:14-413): bits 1 = analytic RoPE
        {"rope_and_kv_cache_prefill", PK_ROPE_KV_PREFILL, 0, true},
        {"rope_and_kv_cache_prefill_analytic", PK_ROPE_KV_PREFILL, 1, true},
        {"attention_prefill", PK_ATTN_PREFILL, 0, true},
        {"kv_cache_update", PK_KV_UPDATE, 0, false},
        {"apply_rope", PK_APPLY_ROPE, 0, false},
        {"rope_kv_cache_update", PK_ROPE_KV_UPDATE, 0, false},
        {"attention_decode", PK_ATTN_GENERIC, 0, false},
        {"rms_norm_1pw", PK_RMS_NORM, 0, false},
        {"per_head_rms_norm", PK_PER_HEAD_NORM, 0, false},
        {"elementwise_add", PK_ADD, 0, false},
        {"swiglu_fused", PK_SWIGLU, 0, false},
        {"smelt_tp_all_reduce", PK_TP_ALL_REDUCE, 0, false},
        {"smelt_tp_reduce_add", PK_TP_REDUCE_ADD, 0, false},
        {"smelt_tp_argmax", PK_TP_ARGMAX, 0, false},
        {"smelt_rope_qkv_append", PK_ROPE_QKV_APPEND, 0, false},
        {"smelt_rope_attention_decode", PK_ATTN_ROPE, 0, false},
        {"conv1d_update_silu", PK_CONV1D_SILU, 0, false},
        {"rms_scale_qk", PK_RMS_SCALE_QK, 0, false},
        {"deltanet_recurrence_mlx_decode", PK_DELTANET_DECODE, 0, false},
        {"rms_norm_gated", PK_RMS_NORM_GATED, 0, false},
        {"conv1d_update_silu_prefill", PK_CONV1D_SILU_PREFILL, 0, false},
        {"conv1d_update_silu_prefill_checkpoint", PK_CONV1D_SILU_PREFILL, 1, false},
        {"deltanet_recurrence_mlx_prefill", PK_DELTANET_PREFILL, 0, false},
        {"deltanet_recurrence_mlx_prefill_checkpoint", PK_DELTANET_PREFILL, 1, false},
        // the DeltaNet step as separate launches and the one-CTA-per-head fused forms (recurrence.metal:44-503, :836-862,
        // prefill_recurrence.metal:42-285); bits = which of a family
        {"compute_gates", PK_DN_GATES, 0, false},
        {"state_decay", PK_DN_STATE_UPDATE, 0, false},
        {"outer_product_update", PK_DN_STATE_UPDATE, 1, false},
        {"state_decay_update", PK_DN_STATE_UPDATE, 2, false},
        {"kv_mem_readout", PK_DN_READOUT, 0, false},
        {"kv_readout_delta", PK_DN_READOUT, 1, false},
        {"gates_kv_readout_delta", PK_DN_READOUT, 2, false},
        {"query_readout", PK_DN_READOUT, 3, false},
        {"compute_delta", PK_DN_DELTA, 0, false},
        {"deltanet_recurrence_fused", PK_DN_FUSED_DECODE, 0, false},
        {"deltanet_recurrence_prefill", PK_DN_FUSED_PREFILL, 0, false},
    };
    // Activation bit-plane producers and consumers (Resources/Shaders/signed_quant.metal:751-2245):
    // the plane count is part of the name.
    {
        int planes = 0, n = 0;
        if (sscanf(name.c_str(), "signed_activation_bitplanes_i%d_g128%n", &planes, &n) == 1 && planes >= 2 && planes <= 6) {
            const std::string rest = name.substr(n);
            if (rest.empty() || rest == "_batched") {
                p.kind = PK_BITPLANE_PRODUCER; p.planes = planes; p.batched = !rest.empty();
                *out = p;
                return true;
            }
        }
        if (name == "swiglu_signed_activation_bitplanes_i5_g128") {
            p.kind = PK_BITPLANE_SWIGLU_PRODUCER; p.planes = 5;
            *out = p;
            return true;
        }
        // producers with another kernel's arithmetic in front (signed_quant.metal:985-1298)
        if (name == "sigmoid_mul_signed_activation_bitplanes_i6_g128") {
            p.kind = PK_BITPLANE_SIGMOID_MUL_PRODUCER; p.planes = 6;
            *out = p;
            return true;
        }
        if (name == "rms_norm_gated_d128_signed_activation_bitplanes_i6_g128") {
            p.kind = PK_BITPLANE_GATED_NORM_PRODUCER; p.planes = 6;
            *out = p;
            return true;
        }
        if (sscanf(name.c_str(), "norm_scale_signed_activation_bitplanes_i%d_g128%n", &planes, &n) == 1 && planes >= 2 && planes <= 6 && name.substr(n).empty()) {
            p.kind = PK_BITPLANE_NORM_SCALE_PRODUCER; p.planes = planes;
            *out = p;
            return true;
        }
        char kind[16] = {0};
        if (sscanf(name.c_str(), "signed_%15[a-z]_bitplane_i%d_%n", kind, &planes, &n) == 2 && planes >= 2 && planes <= 6) {
            const std::string fam = kind, rest = name.substr(n);
            const int bits = fam == "binary" ? 1 : (fam == "ternary" ? 2 : 0);
            PipeKind k = PK_NONE;
            bool batched = false;
            if (rest == "matvec_g128_rows8" || (bits == 2 && rest == "matvec_g128_rows2_wide")) k = PK_BITPLANE_MATVEC;
            else if (bits == 1 && (rest == "matvec_g128_rows8_batched_b4" || rest == "matvec_g128_rows8_batched_b8" || rest == "matvec_g128_rows8_batched_b16")) {
                k = PK_BITPLANE_MATVEC; batched = true;  // the prompt-row tiles compute every (row, batch row) as the matvec does (signed_quant.metal:1346-1436)
            }
            else if (rest == "bank4_matvec_g128_rows8") k = PK_BITPLANE_BANK4;
            else if (rest == "matvec_add_g128_rows8" && bits == 1) k = PK_BITPLANE_ADD;
            else if (rest == "gate_up_swiglu_g128_rows8") k = PK_BITPLANE_GATEUP;
            if (bits && k != PK_NONE) {
                p.kind = k; p.bits = bits; p.planes = planes; p.batched = batched;
                *out = p;
                return true;
            }
        }
    }
    // The row norms of norms.metal beyond rms_norm_1pw: each name fixes a reduction topology, a value formula and its bindings.
    for (int i = 0; i < kRowNormCount; ++i)
        if (name == kRowNorms[i].name) {
            p.kind = PK_ROW_NORM; p.planes = i;
            *out = p;
            return true;
        }
    // Shape-specialised DeltaNet names carry their constants in the name
    // (Resources/Shaders/recurrence.metal:590-836, norms_gated_precise.metal:20-52).
    {
        struct Fixed { const char* name; PipeKind kind; int d, hv, hqk; };
        static const Fixed fixed[] = {
            {"deltanet_recurrence_mlx_decode_d128_h16", PK_DELTANET_DECODE, 128, 16, 16},
            {"deltanet_recurrence_mlx_decode_d128_h32_qk16", PK_DELTANET_DECODE, 128, 32, 16},
            {"deltanet_recurrence_mlx_decode_d128_h48_qk16", PK_DELTANET_DECODE, 128, 48, 16},
            {"rms_norm_gated_d128", PK_RMS_NORM_GATED, 128, 0, 0},
            {"rms_norm_gated_d128_batched", PK_RMS_NORM_GATED, 128, 0, 1},  // hqk field: 1 = the batched form (grid.y rows of numHeads heads)
            // prompt-chunk forms (Resources/Shaders/prefill_recurrence.metal:290-578, conv1d.metal:129-171): d = channels, hv = taps for the conv
            {"deltanet_recurrence_mlx_prefill_d128_h16", PK_DELTANET_PREFILL, 128, 16, 16},
            {"deltanet_recurrence_mlx_prefill_d128_h32_qk16", PK_DELTANET_PREFILL, 128, 32, 16},
            {"deltanet_recurrence_mlx_prefill_d128_h48_qk16", PK_DELTANET_PREFILL, 128, 48, 16},
            {"conv1d_update_silu_c6144_k4_prefill", PK_CONV1D_SILU_PREFILL, 6144, 4, 0},
            {"conv1d_update_silu_c6144_k4", PK_CONV1D_SILU, 6144, 4, 0},
            // + l2_normalize_d128 on the 32 Q / K heads of the output (conv1d.metal:69-127; the reference asserts equality with the staged pair)
            {"conv1d_update_silu_l2_qk_c6144_k4_d128_h16", PK_CONV1D_SILU, 6144, 4, 32},  // conv1d.metal:34-67: the taps' products are exact in fp32, so its fused multiply-adds equal the generic kernel
        };
        for (const Fixed& f : fixed)
            if (name == f.name) {
                p.kind = f.kind; p.head_dim = f.d; p.n_q = f.hv; p.n_kv = f.hqk; p.fixed_shape = true;
                *out = p;
                return true;
            }
    }
    for (const Simple& s : table)
        if (name == s.name) {
            p.kind = s.kind; p.bits = s.bits; p.batched = s.batched;
            *out = p;
            return true;
        }
    // In-place shape-specialised decode attention:
    // attention_decode_d{D}_h{H}_kv{KV}[_sdpa] (Resources/Shaders/attention.metal:422-977, :1211-1309)
    // and attention_decode_mlx_vector_d256 (:981-1065, head counts bound as constants 5 and 6).
    {
        int d = 0, h = 0, kv = 0, n = 0;
        if (sscanf(name.c_str(), "attention_decode_d%d_h%d_kv%d%n", &d, &h, &kv, &n) == 3) {
            std::string rest = name.substr(n);
            if ((rest.empty() || rest == "_sdpa") && (d == 64 || d == 128 || d == 256) && kv > 0 && h % kv == 0 && h / kv <= 16) {
                p.kind = PK_ATTN_INPLACE; p.head_dim = d; p.n_q = h; p.n_kv = kv;
                *out = p;
                return true;
            }
            return false;
        }
        // The split-K record pair a D256 package emits from 1,024 keys on
        // (Resources/Shaders/attention.metal:1071-1206; Sources/SmeltCompiler/AttentionPlugin.swift:865-918).
        if (name == "attention_decode_mlx_vector_2pass_1_d256_b128" || name == "attention_decode_mlx_vector_2pass_2_d256_b128") {
            p.kind = name.find("2pass_1") != std::string::npos ? PK_ATTN_MLX_2PASS_1 : PK_ATTN_MLX_2PASS_2; p.head_dim = 256;
            *out = p;
            return true;
        }
        if (name == "attention_decode_mlx_vector_d256") {
            p.kind = PK_ATTN_INPLACE; p.head_dim = 256;
            *out = p;
            return true;
        }
    }
    return false;
}

namespace {

struct RBuf {
    bool present = false;
    uint8_t* ptr = nullptr;   // base + resolved offset (literal, or position * stride when known on the host)
    size_t avail = 0;         // bytes from ptr to the end of the slot
    bool pos_strided = false; // offset is position * stride and position is only known on the device
    uint64_t stride = 0;
};
struct RConst {
    bool present = false;
    uint8_t kind = 0;
    uint32_t value = 0;
};

struct Resolved {
    RBuf buf[32];
    RConst con[32];
    uint32_t guard_lt = 0, guard_ge = 0;
    bool skip = false;
};

struct Interp {
    smelt_cuda_ctx* ctx;
    bool device_pos;    // graph capture: position lives on the device
    uint32_t position;  // host copy (valid when !device_pos)
    int cur, alt;
    int launches = 0;
    bool prefill = false;    // a prompt chunk: seq_len positions from start_pos (position == start_pos; SmeltRuntime.swift:1217-1250)
    uint32_t seq_len = 0, start_pos = 0;
    int rope_half = 0;       // the position's cos | sin table holds this many pairs ...
    float rope_base = 0.f;   // ... for this log2(theta); 0 pairs = not written in this interpretation
};

smelt_status resolve(Interp& in, const smelt_dispatch_record& rec, Resolved* out) {
    smelt_cuda_ctx* ctx = in.ctx;
    if (rec.buffer_count > 16 || rec.constant_count > 8) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "record: buffer/constant count out of range");
    for (int i = 0; i < rec.buffer_count; ++i) {
        const smelt_buffer_record& b = rec.buf[i];
        int slot = b.slot == SMELT_SLOT_CUR ? in.cur : (b.slot == SMELT_SLOT_ALT ? in.alt : b.slot);
        if (slot < 0 || slot >= (int)ctx->slots.size() || !ctx->slots[slot].ptr)
            return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "record binds slot " + std::to_string(slot) + " which is not allocated");
        if (b.binding_index >= 32) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "record: buffer binding index out of range");
        RBuf& r = out->buf[b.binding_index];
        r.present = true;
        uint64_t off = b.offset;
        if (b.offset_kind == 1) {
            if (in.device_pos) { r.pos_strided = true; r.stride = b.offset; off = 0; }
            else off = (uint64_t)in.position * b.offset;
        } else if (b.offset_kind >= 2 && b.offset_kind <= 4) {
            // the prompt-chunk offsets (resolveDispatchBufferOffset, SmeltRuntime.swift:6160-6185)
            if (!in.prefill) return fail(ctx, SMELT_ERR_UNSUPPORTED, "record: prefill offset kinds are outside the decode path");
            const uint64_t lo = b.offset & 0xFFFFFFFFull, hi = b.offset >> 32;
            if (b.offset_kind == 2) off = (uint64_t)in.start_pos * lo + hi;
            else if (b.offset_kind == 3) off = (uint64_t)(in.seq_len - 1) * b.offset;
            else off = ((uint64_t)in.seq_len / (hi ? hi : 1)) * lo;
        } else if (b.offset_kind != 0) {
            return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "record: unknown offset kind " + std::to_string(b.offset_kind));
        }
        if (off > ctx->slots[slot].bytes)
            return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "record: offset " + std::to_string(off) + " is outside slot " + std::to_string(slot));
        r.ptr = (uint8_t*)ctx->slots[slot].ptr + off;
        r.avail = ctx->slots[slot].bytes - off;
    }
    for (int i = 0; i < rec.constant_count; ++i) {
        const smelt_constant_record& c = rec.con[i];
        switch (c.kind) {
            case SMELT_CONST_SKIP_UNLESS_POS1_LT:
                if (in.device_pos) out->guard_lt = c.value;
                else if (!(in.position + 1u < c.value)) out->skip = true;
                break;
            case SMELT_CONST_SKIP_UNLESS_POS1_GE:
                if (in.device_pos) out->guard_ge = c.value;
                else if (!(in.position + 1u >= c.value)) out->skip = true;
                break;
            case SMELT_CONST_LITERAL_U32: case SMELT_CONST_LITERAL_F32: case SMELT_CONST_POSITION:
            case SMELT_CONST_POSITION_PLUS1: case SMELT_CONST_CACHE_SEQ_CAPACITY:
                break;
            case SMELT_CONST_SEQ_LEN: case SMELT_CONST_START_POS: case SMELT_CONST_START_POS_PLUS: case SMELT_CONST_SEQ_LEN_MUL:
            case SMELT_CONST_SEQ_LEN_MOD: case SMELT_CONST_SEQ_LEN_MOD_SKIP_IF_ZERO: case SMELT_CONST_SKIP_UNLESS_SEQ_LEN_LT:
                if (!in.prefill) return fail(ctx, SMELT_ERR_UNSUPPORTED, "record: constant kind " + std::to_string(c.kind) + " is outside the decode path");
                break;
            default:
                return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "record: unknown constant kind " + std::to_string(c.kind));
        }
        uint8_t kind = c.kind;
        uint32_t value = c.value;
        if (in.prefill) {
            // resolvePrefillConstant (SmeltRuntime.swift:1217-1250): every run-time kind becomes a plain value here
            switch (c.kind) {
                case SMELT_CONST_SEQ_LEN: value = in.seq_len; kind = SMELT_CONST_LITERAL_U32; break;
                case SMELT_CONST_START_POS: value = in.start_pos; kind = SMELT_CONST_LITERAL_U32; break;
                case SMELT_CONST_START_POS_PLUS: value = in.start_pos + c.value; kind = SMELT_CONST_LITERAL_U32; break;
                case SMELT_CONST_SEQ_LEN_MUL: value = in.seq_len * c.value; kind = SMELT_CONST_LITERAL_U32; break;
                case SMELT_CONST_SEQ_LEN_MOD: value = c.value ? in.seq_len % c.value : 0u; kind = SMELT_CONST_LITERAL_U32; break;
                case SMELT_CONST_SEQ_LEN_MOD_SKIP_IF_ZERO:
                    value = c.value ? in.seq_len % c.value : 0u; kind = SMELT_CONST_LITERAL_U32;
                    if (value == 0) out->skip = true;
                    break;
                case SMELT_CONST_SKIP_UNLESS_SEQ_LEN_LT:
                    value = in.seq_len < c.value ? 1u : 0u; kind = SMELT_CONST_LITERAL_U32;
                    if (value == 0) out->skip = true;
                    break;
                default: break;
            }
        }
        if (c.binding_index != 255) {
            if (c.binding_index >= 32) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "record: constant binding index out of range");
            RConst& r = out->con[c.binding_index];
            r.present = true; r.kind = kind; r.value = value;
        }
    }
    return SMELT_OK;
}

// A constant that must be known on the host (shapes, counts).
bool host_u32(const Interp& in, const Resolved& r, int idx, uint32_t* v) {
    const RConst& c = r.con[idx];
    if (!c.present) return false;
    switch (c.kind) {
        case SMELT_CONST_LITERAL_U32: case SMELT_CONST_LITERAL_F32:
        case SMELT_CONST_SKIP_UNLESS_POS1_LT: case SMELT_CONST_SKIP_UNLESS_POS1_GE:
            *v = c.value; return true;
        case SMELT_CONST_CACHE_SEQ_CAPACITY: *v = in.ctx->cfg.cache_seq_capacity; return true;
        case SMELT_CONST_POSITION: if (in.device_pos) return false; *v = in.position; return true;
        case SMELT_CONST_POSITION_PLUS1: if (in.device_pos) return false; *v = in.position + 1u; return true;
        default: return false;
    }
}
float as_f32(uint32_t bits) { float f; memcpy(&f, &bits, 4); return f; }

Launch make_launch(const Interp& in, const Resolved& r) {
    Launch l;
    l.stream = in.ctx->stream;
    l.pdl = in.ctx->pdl;
    if (in.device_pos) {
        l.dyn = in.ctx->dyn_dev;
        l.guard_lt = r.guard_lt;
        l.guard_ge = r.guard_ge;
    } else {
        l.position = in.position;
    }
    return l;
}

// Binds a "position"-valued kernel argument: the step position when the constant is dynamic,
// else the literal.
bool bind_pos_arg(const Interp& in, const Resolved& r, int idx, Launch* l) {
    const RConst& c = r.con[idx];
    if (!c.present) return false;
    if (c.kind == SMELT_CONST_POSITION) return true;
    uint32_t v;
    if (!host_u32(in, r, idx, &v)) return false;
    l->arg_pos = v;
    l->arg_pos_valid = 1;
    return true;
}

#define NEED_BUF(i)                                                                                        \
    if (!r.buf[i].present) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": buffer binding " #i " is missing"); \
    if (r.buf[i].pos_strided) return fail(ctx, SMELT_ERR_UNSUPPORTED, p.name + ": position-scaled offset on binding " #i " cannot be captured")
#define NEED_U32(i, var)                                                                                   \
    uint32_t var = 0;                                                                                      \
    if (!host_u32(in, r, i, &var)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": constant binding " #i " is missing or not host-resolvable")
#define NEED_BYTES(i, n)                                                                                   \
    if (r.buf[i].avail < (size_t)(n)) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, p.name + ": binding " #i " needs " + std::to_string((size_t)(n)) + " bytes, slot has " + std::to_string(r.buf[i].avail))

int batch_of(const smelt_dispatch_record& rec) { return rec.grid[1] > 0 ? (int)rec.grid[1] : 1; }

smelt_status run_affine(Interp& in, const Pipeline& p, const smelt_dispatch_record& rec, const Resolved& r) {
    smelt_cuda_ctx* ctx = in.ctx;
    // binding layouts: lut_matvec.metal:1157-1165 (matvec), :1718-1727 (add), :2152-2163 (gate/up), :1824-1836 (dual)
    int ix, iy, iy2 = -1, ires = -1, icount;
    int nw = 1;
    switch (p.kind) {
        case PK_AFFINE_MATVEC: ix = 3; iy = 4; icount = 5; break;
        case PK_AFFINE_ADD: ix = 3; iy = 4; ires = 5; icount = 6; break;
        case PK_AFFINE_GATEUP: nw = 2; ix = 6; iy = 7; icount = 8; break;
        default: nw = 2; ix = 6; iy = 7; iy2 = 8; icount = 9; break;
    }
    int rows = p.rows, batch = 1;
    if (!p.fixed_shape) { NEED_U32(icount, nrows); rows = (int)nrows; }
    else if (p.batched) { NEED_U32(icount, nb); batch = (int)nb; }
    if (rows <= 0 || batch <= 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": rows and batch must be positive");
    const int groups = p.cols / p.group;
    AffineArgs a = {};
    for (int s = 0; s < nw; ++s) {
        const int b0 = 3 * s;
        if (!r.buf[b0].present || !r.buf[b0 + 1].present || !r.buf[b0 + 2].present)
            return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": weight bindings are missing");
        if (r.buf[b0].avail < (size_t)rows * p.cols / 2 || r.buf[b0 + 1].avail < (size_t)rows * groups * 2 || r.buf[b0 + 2].avail < (size_t)rows * groups * 2)
            return fail(ctx, SMELT_ERR_OUT_OF_RANGE, p.name + ": weight tensor extends past the weights slot");
        a.w[s] = r.buf[b0].ptr; a.s[s] = (const __half*)r.buf[b0 + 1].ptr; a.b[s] = (const __half*)r.buf[b0 + 2].ptr;
        if ((uintptr_t)a.w[s] & 15u) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": packed weights must be 16-byte aligned");
    }
    NEED_BUF(ix); NEED_BUF(iy);
    NEED_BYTES(ix, (size_t)batch * p.cols * 2); NEED_BYTES(iy, (size_t)batch * rows * 2);
    a.x = (const __half*)r.buf[ix].ptr; a.y = (__half*)r.buf[iy].ptr;
    if (iy2 >= 0) { NEED_BUF(iy2); NEED_BYTES(iy2, (size_t)batch * rows * 2); a.y2 = (__half*)r.buf[iy2].ptr; }
    if (ires >= 0) { NEED_BUF(ires); NEED_BYTES(ires, (size_t)batch * rows * 2); a.residual = (const __half*)r.buf[ires].ptr; }
    a.rows = rows; a.cols = p.cols; a.batch = batch; a.err = ctx->err_dev; a.sm_count = ctx->sm_count; a.part_scratch = ctx->qmm_scratch; a.part_scratch_bytes = ctx->qmm_scratch_bytes; a.part_counters = ctx->qmm_counters;
    const int mode = p.kind == PK_AFFINE_MATVEC ? kAffinePlain : p.kind == PK_AFFINE_ADD ? kAffineAdd : p.kind == PK_AFFINE_GATEUP ? kAffineGateUp : kAffineDual;
    in.launches += (batch + 15) / 16;
    return check_cuda(ctx, launch_affine(make_launch(in, r), mode, a, p.group), p.name.c_str());
}

smelt_status run_signed(Interp& in, const Pipeline& p, const smelt_dispatch_record& rec, const Resolved& r) {
    smelt_cuda_ctx* ctx = in.ctx;
    // signed_quant.metal:574-583 (matvec), :662-672 (add), :625-636 (gate/up); signed_quant_precise.metal:41-50
    SignedArgs a = {};
    int ix, iy, irows, ires = -1, mode = kSignedPlain;
    int icodes2 = 2;  // gate / up: where the second matrix's codes are bound
    if (p.kind == PK_SIGNED_MATVEC) { ix = 2; iy = 3; irows = 4; }
    else if (p.kind == PK_SIGNED_ADD) { ix = 2; iy = 3; ires = 4; irows = 5; mode = kSignedAdd; }
    else if (p.kind == PK_SIGNED_GATEUP) { ix = 4; iy = 5; irows = 6; mode = kSignedGateUp; }
    else if (p.kind == PK_SIGNED_TERNARY_AFFINE_ADD) { ix = 3; iy = 4; ires = 5; irows = 6; mode = kSignedAdd; }  // signed_quant_precise.metal:113-121
    else if (p.kind == PK_SIGNED_TERNARY_AFFINE_GATEUP) { ix = 6; iy = 7; irows = 8; icodes2 = 3; mode = kSignedGateUp; }  // :268-278
    else { ix = 3; iy = 4; irows = 5; }  // ternary affine: binding 2 repeats the scales as the bias source
    NEED_U32(irows, rows); NEED_U32(irows + 1, cols);
    int batch = batch_of(rec);
    if (p.batched) { NEED_U32(irows + 2, nb); batch = (int)nb; }
    if (cols == 0 || cols % 128 || rows == 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": cols must be a positive multiple of 128");
    const size_t code_bytes = (size_t)rows * cols * p.bits / 8, scale_bytes = (size_t)rows * (cols / 128) * 2;
    NEED_BUF(0); NEED_BUF(1); NEED_BYTES(0, code_bytes); NEED_BYTES(1, scale_bytes);
    a.codes[0] = r.buf[0].ptr; a.scales[0] = (const __half*)r.buf[1].ptr;
    if (mode == kSignedGateUp) {
        NEED_BUF(icodes2); NEED_BUF(icodes2 + 1); NEED_BYTES(icodes2, code_bytes); NEED_BYTES(icodes2 + 1, scale_bytes);
        a.codes[1] = r.buf[icodes2].ptr; a.scales[1] = (const __half*)r.buf[icodes2 + 1].ptr;
    }
    NEED_BUF(ix); NEED_BUF(iy);
    NEED_BYTES(ix, (size_t)batch * cols * 2); NEED_BYTES(iy, (size_t)batch * rows * 2);
    a.x = (const __half*)r.buf[ix].ptr; a.y = (__half*)r.buf[iy].ptr;
    if (ires >= 0) { NEED_BUF(ires); NEED_BYTES(ires, (size_t)batch * rows * 2); a.residual = (const __half*)r.buf[ires].ptr; }
    a.rows = (int)rows; a.cols = (int)cols; a.batch = batch; a.bits = p.bits;
    in.launches += 1;
    return check_cuda(ctx, launch_signed(make_launch(in, r), mode, a), p.name.c_str());
}

smelt_status run_attention(Interp& in, const Pipeline& p, const smelt_dispatch_record& rec, const Resolved& r) {
    smelt_cuda_ctx* ctx = in.ctx;
    AttnArgs a = {};
    int iseq;
    NEED_BUF(0); NEED_BUF(1); NEED_BUF(2);
    a.batch = batch_of(rec);
    a.k_cache = (const __half*)r.buf[1].ptr; a.v_cache = (const __half*)r.buf[2].ptr;
    a.q = (const __half*)r.buf[0].ptr;
    if (p.kind == PK_ATTN_GENERIC || p.kind == PK_ATTN_ROPE) {
        // attention.metal:217-229: 0 q, 1 K, 2 V, 3 mask (unused), 4 out, 5 headDim, 6 capacity, 7 seqLen,
        // 8 numKVHeads, 9 scale, 10 slidingWindow; numQHeads = threadgroups in x.
        NEED_BUF(4);
        NEED_U32(5, d); NEED_U32(6, cap); NEED_U32(8, nkv); NEED_U32(9, scale_bits);
        uint32_t window = 0;
        (void)host_u32(in, r, 10, &window);
        a.out = (__half*)r.buf[4].ptr; a.head_dim = (int)d; a.capacity = cap; a.n_kv = (int)nkv; a.n_q = (int)rec.grid[0];
        a.scale = as_f32(scale_bits); a.sliding_window = window;
        iseq = 7;
        if (p.kind == PK_ATTN_ROPE) {
            // the generic bindings plus 11 new K, 12 new V, 13 pair layout, 14 log2(theta)
            NEED_BUF(11); NEED_BUF(12); NEED_U32(13, layout); NEED_U32(14, base_bits);
            if (layout > 1) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": layout must be 0 or 1");
            a.k_new = (const __half*)r.buf[11].ptr; a.v_new = (const __half*)r.buf[12].ptr;
            a.rope_layout = (int)layout; a.rope_base_log2 = as_f32(base_bits);
            if (d / 2 <= 128 && r.con[7].present && r.con[7].kind == SMELT_CONST_POSITION_PLUS1) {
                // the new token sits at the step position in every layer: cos | sin once per token
                if (in.rope_half != (int)d / 2 || in.rope_base != a.rope_base_log2) {
                    Launch lt = make_launch(in, r);
                    lt.guard_lt = lt.guard_ge = 0;
                    smelt_status st = check_cuda(ctx, launch_rope_table(lt, ctx->rope_table, (int)d / 2, a.rope_base_log2), "rope table");
                    if (st) return st;
                    in.rope_half = (int)d / 2; in.rope_base = a.rope_base_log2;
                    in.launches += 1;
                }
                a.rope_table = ctx->rope_table;
                // a decode table appends one row per token to this cache and nothing else writes it:
                // the rows of earlier tokens are final before this token's first launch
                a.kv_rows_stable = 1;
            }
            NEED_BYTES(11, (size_t)a.batch * nkv * d * 2); NEED_BYTES(12, (size_t)a.batch * nkv * d * 2);
        }
    } else if (p.kind == PK_ATTN_MLX_2PASS_1) {
        // attention.metal:1071-1083: 0 q, 1 K, 2 V, 3 partials (fp16 [qHeads, 128, 256]), 4 stats
        // (fp32 [2][qHeads][128]), 5 seqLen, 6 capacity, 7 qHeads, 8 kvHeads; scale 1/16 is fixed.
        NEED_BUF(3); NEED_BUF(4);
        NEED_U32(6, cap); NEED_U32(7, nq); NEED_U32(8, nkv);
        if (a.batch != 1) return fail(ctx, SMELT_ERR_UNSUPPORTED, p.name + ": one sequence per record");
        a.head_dim = 256; a.capacity = cap; a.n_q = (int)nq; a.n_kv = (int)nkv; a.scale = 0.0625f;
        NEED_BYTES(3, (size_t)nq * 128 * 256 * 2); NEED_BYTES(4, (size_t)2 * nq * 128 * 4);
        a.mlx_partials = (__half*)r.buf[3].ptr; a.mlx_stats = (float*)r.buf[4].ptr;
        a.out = nullptr;
        iseq = 5;
    } else {
        // in place: 0 q/out, 1 K, 2 V, 3 seqLen, 4 capacity (attention.metal:422-431, :1211-1218);
        // the mlx_vector form adds 5 qHeads, 6 kvHeads (:981-989).
        NEED_U32(4, cap);
        a.out = (__half*)r.buf[0].ptr; a.head_dim = p.head_dim; a.capacity = cap; a.n_q = p.n_q; a.n_kv = p.n_kv;
        if (p.n_q == 0) { NEED_U32(5, nq); NEED_U32(6, nkv); a.n_q = (int)nq; a.n_kv = (int)nkv; }
        a.scale = 1.0f / sqrtf((float)p.head_dim);
        iseq = 3;
    }
    const RConst& cs = r.con[iseq];
    if (!cs.present) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": seqLen constant is missing");
    if (cs.kind == SMELT_CONST_POSITION_PLUS1 && in.device_pos) a.seq_from_pos = 1;
    else {
        NEED_U32(iseq, sl);
        a.seq_len = sl;
        if (sl == 0 || sl > a.capacity) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, p.name + ": seqLen must be in 1..capacity");
    }
    if (a.n_kv <= 0 || a.n_q <= 0 || a.n_q % a.n_kv || a.n_q / a.n_kv > 16 || (a.head_dim != 64 && a.head_dim != 128 && a.head_dim != 256))
        return fail(ctx, SMELT_ERR_UNSUPPORTED, p.name + ": head_dim in {64,128,256}, GQA ratio <= 16");
    a.seq_stride = (size_t)a.n_kv * a.capacity * a.head_dim;
    NEED_BYTES(1, a.seq_stride * 2 * a.batch); NEED_BYTES(2, a.seq_stride * 2 * a.batch);
    NEED_BYTES(0, (size_t)a.batch * a.n_q * a.head_dim * 2);
    a.scratch = ctx->attn_scratch; a.scratch_bytes = ctx->attn_scratch_bytes; a.sm_count = ctx->sm_count;
    if ((size_t)a.batch * a.n_kv <= 4096 && !a.mlx_partials) a.counters = ctx->attn_counters;
    if (p.kind == PK_ATTN_ROPE && !a.counters) return fail(ctx, SMELT_ERR_UNSUPPORTED, p.name + ": too many (sequence, KV head) pairs");
    in.launches += 1;
    return check_cuda(ctx, launch_attention_decode(make_launch(in, r), a), p.name.c_str());
}

smelt_status run_record(Interp& in, const smelt_dispatch_record& rec_in) {
    smelt_cuda_ctx* ctx = in.ctx;
    smelt_dispatch_record rec = rec_in;
    if (in.prefill) {
        // minSeqLen guard and the grid dimensions that follow the chunk length (SmeltDispatchTable.swift:163-222,
        // resolvePrefillGrid, SmeltRuntime.swift:6187-6207): handlers read the resolved grid
        if (rec.min_seq_len && in.seq_len < rec.min_seq_len) return SMELT_OK;
        for (int d = 0; d < 3; ++d) {
            const uint32_t kind = (rec.style >> (2 + 2 * d)) & 3u, lit = rec.grid[d];
            if (kind == 1) rec.grid[d] = in.seq_len;
            else if (kind == 2) rec.grid[d] = in.seq_len * lit;
            else if (kind == 3) {
                const uint32_t div = (lit & 0x7FFFFFFFu) ? (lit & 0x7FFFFFFFu) : 1u;
                rec.grid[d] = (lit & 0x80000000u) ? in.seq_len / div : (in.seq_len + div - 1) / div;
            }
        }
    } else if (rec.style >> 2) {
        return fail(ctx, SMELT_ERR_UNSUPPORTED, "record: prefill grid kinds are outside the decode path");
    }
    if (rec.pipeline >= ctx->pipelines.size() || ctx->pipelines[rec.pipeline].kind == PK_NONE)
        return fail(ctx, SMELT_ERR_UNKNOWN_PIPELINE, "record names pipeline index " + std::to_string(rec.pipeline) + " which is not registered");
    const Pipeline& p = ctx->pipelines[rec.pipeline];
    Resolved r;
    smelt_status s = resolve(in, rec, &r);
    if (s) return s;
    if (r.skip) return SMELT_OK;
    Launch l = make_launch(in, r);
    switch (p.kind) {
        case PK_AFFINE_MATVEC: case PK_AFFINE_ADD: case PK_AFFINE_GATEUP: case PK_AFFINE_DUAL:
            return run_affine(in, p, rec, r);
        case PK_SIGNED_MATVEC: case PK_SIGNED_ADD: case PK_SIGNED_GATEUP: case PK_SIGNED_TERNARY_AFFINE:
        case PK_SIGNED_TERNARY_AFFINE_ADD: case PK_SIGNED_TERNARY_AFFINE_GATEUP:
            return run_signed(in, p, rec, r);
        case PK_ATTN_GENERIC: case PK_ATTN_INPLACE: case PK_ATTN_ROPE: case PK_ATTN_MLX_2PASS_1:
            return run_attention(in, p, rec, r);
        case PK_ATTN_MLX_2PASS_2: {
            // attention.metal:1146-1153: 0 partials, 1 stats, 2 out, 3 qHeads.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_U32(3, nq);
            if (nq == 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": qHeads must be positive");
            NEED_BYTES(0, (size_t)nq * 128 * 256 * 2); NEED_BYTES(1, (size_t)2 * nq * 128 * 4); NEED_BYTES(2, (size_t)nq * 256 * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_attention_mlx_reduce(l, (const __half*)r.buf[0].ptr, (const float*)r.buf[1].ptr, (__half*)r.buf[2].ptr, (int)nq, 256), p.name.c_str());
        }
        case PK_FP16_MATVEC: {
            // lut_matvec.metal:799-803: 0 W, 1 x, 2 y, 3 cols; one threadgroup per row.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_U32(3, cols);
            const int rows = (int)rec.grid[0], batch = batch_of(rec);
            if (rows <= 0 || cols == 0 || cols % 8) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "fp16_matvec: cols must be a positive multiple of 8");
            NEED_BYTES(0, (size_t)rows * cols * 2); NEED_BYTES(1, (size_t)batch * cols * 2); NEED_BYTES(2, (size_t)batch * rows * 2);
            in.launches += (batch + 7) / 8;
            return check_cuda(ctx, launch_fp16_matvec(l, (const __half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, (__half*)r.buf[2].ptr, rows, (int)cols, batch, ctx->sm_count), "fp16_matvec");
        }
        case PK_EMBEDDING_GATHER: {
            // lut_matvec.metal:951-956: 0 table, 1 token id, 2 out, 3 hidden.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_U32(3, hidden);
            const int batch = batch_of(rec);
            NEED_BYTES(1, (size_t)batch * 4); NEED_BYTES(2, (size_t)batch * hidden * 2);
            NEED_BYTES(0, (size_t)ctx->cfg.vocab_size * hidden * 2);  // token ids are checked against vocab_size when they are written
            in.launches += 1;
            return check_cuda(ctx, launch_embedding_gather(l, (const __half*)r.buf[0].ptr, (const int32_t*)r.buf[1].ptr, (__half*)r.buf[2].ptr, (int)hidden, batch, 1), "embedding_gather");
        }
        case PK_AFFINE_EMBEDDING_GATHER: {
            // lut_matvec.metal:994-1002: 0 W, 1 scales, 2 biases, 3 token id, 4 out, 5 cols, 6 groupSize.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_BUF(3); NEED_BUF(4); NEED_U32(5, cols); NEED_U32(6, group);
            if (cols == 0 || group == 0 || cols % group || cols % 2) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "affine_embedding_gather: bad cols/group");
            NEED_BYTES(4, (size_t)cols * 2);
            NEED_BYTES(0, (size_t)ctx->cfg.vocab_size * cols / 2); NEED_BYTES(1, (size_t)ctx->cfg.vocab_size * (cols / group) * 2); NEED_BYTES(2, (size_t)ctx->cfg.vocab_size * (cols / group) * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_affine_embedding_gather(l, r.buf[0].ptr, (const __half*)r.buf[1].ptr, (const __half*)r.buf[2].ptr, (const int32_t*)r.buf[3].ptr, (__half*)r.buf[4].ptr, (int)cols, (int)group), "affine_embedding_gather");
        }
        case PK_ARGMAX_PARTIALS: {
            // lut_matvec.metal:8901-8906: 0 logits, 1 partials, 2 vocab, 3 chunk.
            NEED_BUF(0); NEED_BUF(1); NEED_U32(2, vocab); NEED_U32(3, chunk);
            const int batch = batch_of(rec);
            if (vocab == 0 || chunk == 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "argmax_fp16_partials: vocab and chunk must be positive");
            const size_t parts = (vocab + chunk - 1) / chunk;
            NEED_BYTES(0, (size_t)batch * vocab * 2); NEED_BYTES(1, parts * batch * 8);
            in.launches += 1;
            return check_cuda(ctx, launch_argmax_partials(l, (const __half*)r.buf[0].ptr, (uint64_t*)r.buf[1].ptr, (int)vocab, (int)chunk, batch), "argmax_fp16_partials");
        }
        case PK_ARGMAX_REDUCE: {
            // lut_matvec.metal:8938-8942: 0 partials, 1 out, 2 numPartials.
            NEED_BUF(0); NEED_BUF(1); NEED_U32(2, parts);
            const int batch = batch_of(rec);
            NEED_BYTES(0, (size_t)parts * batch * 8); NEED_BYTES(1, (size_t)batch * 4);
            in.launches += 1;
            return check_cuda(ctx, launch_argmax_reduce(l, (const uint64_t*)r.buf[0].ptr, (int32_t*)r.buf[1].ptr, (int)parts, batch, 1), "argmax_key_reduce");
        }
        case PK_ARGMAX_SINGLE: {
            // single-threadgroup argmax_fp16: 0 logits, 1 out, 2 vocab.
            NEED_BUF(0); NEED_BUF(1); NEED_U32(2, vocab);
            const int batch = batch_of(rec);
            const int chunk = 2048;
            const size_t parts = (vocab + chunk - 1) / chunk;
            if (parts * batch * 8 > ctx->argmax_scratch_bytes) return fail(ctx, SMELT_ERR_UNSUPPORTED, "argmax_fp16: vocab too large");
            in.launches += 2;
            s = check_cuda(ctx, launch_argmax_partials(l, (const __half*)r.buf[0].ptr, ctx->argmax_scratch, (int)vocab, chunk, batch), "argmax_fp16");
            if (s) return s;
            return check_cuda(ctx, launch_argmax_reduce(l, ctx->argmax_scratch, (int32_t*)r.buf[1].ptr, (int)parts, batch, 1), "argmax_fp16");
        }
        case PK_KV_UPDATE: {
            // attention.metal:122-129: 0 cache, 1 new, 2 capacity, 3 headDim, 4 pos, 5 numHeads.
            NEED_BUF(0); NEED_BUF(1); NEED_U32(2, cap); NEED_U32(3, d); NEED_U32(5, heads);
            if (!bind_pos_arg(in, r, 4, &l)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "kv_cache_update: position constant is missing");
            const int batch = batch_of(rec);
            const size_t seq = (size_t)heads * cap * d;
            NEED_BYTES(0, seq * 2 * batch); NEED_BYTES(1, (size_t)batch * heads * d * 2);
            if (!in.device_pos && (l.arg_pos_valid ? l.arg_pos : in.position) >= cap) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "kv_cache_update: position beyond the cache capacity");
            in.launches += 1;
            return check_cuda(ctx, launch_kv_cache_update(l, (__half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, nullptr, nullptr, cap, (int)d, (int)heads, 0, 0, 0.f, 0, 0, 0, batch, seq), "kv_cache_update");
        }
        case PK_APPLY_ROPE: {
            // attention.metal:48-59: 0 data, 1 cos, 2 sin, 3 headDim, 4 ropeDim, 5 numHeads, 6 layout,
            // 7 position, 8 log2(theta) f32, 9 mathMode.
            NEED_BUF(0); NEED_U32(3, d); NEED_U32(4, rope); NEED_U32(5, heads); NEED_U32(6, layout);
            uint32_t mode = 0, base_bits = 0;
            (void)host_u32(in, r, 9, &mode); (void)host_u32(in, r, 8, &base_bits);
            if (!bind_pos_arg(in, r, 7, &l)) { if (mode == 1) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "apply_rope: position constant is missing"); l.arg_pos = 0; l.arg_pos_valid = 1; }
            const int batch = batch_of(rec);
            NEED_BYTES(0, (size_t)batch * heads * d * 2);
            const __half *cos_t = nullptr, *sin_t = nullptr;
            size_t stride = 0;
            if (mode != 1) {
                if (!r.buf[1].present || !r.buf[2].present) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "apply_rope: table mode needs cos/sin bindings");
                cos_t = (const __half*)r.buf[1].ptr; sin_t = (const __half*)r.buf[2].ptr;
                if (r.buf[1].pos_strided) stride = r.buf[1].stride / 2;  // table row per position, resolved on the device
            }
            if (rope > d || d == 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "apply_rope: ropeDim must not exceed headDim");
            in.launches += 1;
            return check_cuda(ctx, launch_apply_rope(l, (__half*)r.buf[0].ptr, cos_t, sin_t, (int)d, (int)rope, (int)heads, (int)layout, as_f32(base_bits), (int)mode, stride, batch), "apply_rope");
        }
        case PK_ROPE_KV_UPDATE: {
            // attention.metal:141-154: 0 cache, 1 new, 2 cos, 3 sin, 4 capacity, 5 headDim, 6 pos, 7 numHeads,
            // 8 ropeDim, 9 layout, 10 log2(theta), 11 mathMode.
            NEED_BUF(0); NEED_BUF(1); NEED_U32(4, cap); NEED_U32(5, d); NEED_U32(7, heads); NEED_U32(8, rope); NEED_U32(9, layout);
            uint32_t mode = 0, base_bits = 0;
            (void)host_u32(in, r, 11, &mode); (void)host_u32(in, r, 10, &base_bits);
            if (!bind_pos_arg(in, r, 6, &l)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "rope_kv_cache_update: position constant is missing");
            const int batch = batch_of(rec);
            const size_t seq = (size_t)heads * cap * d;
            NEED_BYTES(0, seq * 2 * batch); NEED_BYTES(1, (size_t)batch * heads * d * 2);
            if (!in.device_pos && (l.arg_pos_valid ? l.arg_pos : in.position) >= cap) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "rope_kv_cache_update: position beyond the cache capacity");
            const __half *cos_t = nullptr, *sin_t = nullptr;
            size_t stride = 0;
            if (mode != 1) {
                if (!r.buf[2].present || !r.buf[3].present) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "rope_kv_cache_update: table mode needs cos/sin bindings");
                cos_t = (const __half*)r.buf[2].ptr; sin_t = (const __half*)r.buf[3].ptr;
                if (r.buf[2].pos_strided) stride = r.buf[2].stride / 2;
            }
            in.launches += 1;
            return check_cuda(ctx, launch_kv_cache_update(l, (__half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, cos_t, sin_t, cap, (int)d, (int)heads, (int)rope, (int)layout, as_f32(base_bits), (int)mode, 1, stride, batch, seq), "rope_kv_cache_update");
        }
        case PK_RMS_NORM: {
            // norms.metal:9-14: 0 in, 1 weight, 2 out, 3 dim, 4 eps; one threadgroup per row.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_U32(3, dim); NEED_U32(4, eps_bits);
            const int batch = rec.grid[0] > 0 ? (int)rec.grid[0] : 1;
            NEED_BYTES(0, (size_t)batch * dim * 2); NEED_BYTES(1, (size_t)dim * 2); NEED_BYTES(2, (size_t)batch * dim * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_rms_norm_1pw(l, (const __half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, (__half*)r.buf[2].ptr, (int)dim, as_f32(eps_bits), batch), "rms_norm_1pw");
        }
        case PK_PER_HEAD_NORM: {
            // attention_fused.metal:93-98: 0 in, 1 weight, 2 out, 3 headDim, 4 eps; one threadgroup per head.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_U32(3, d); NEED_U32(4, eps_bits);
            const int heads = (int)rec.grid[0];
            if (heads <= 0 || d == 0 || d > 1024) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "per_head_rms_norm: bad shape");
            NEED_BYTES(0, (size_t)heads * d * 2); NEED_BYTES(2, (size_t)heads * d * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_per_head_rms_norm(l, (const __half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, (__half*)r.buf[2].ptr, heads, (int)d, as_f32(eps_bits)), "per_head_rms_norm");
        }
        case PK_ELEMENTWISE: {
            // activations.metal: unary kernels bind 0 in, 1 out, 2 count (scalar_mul: 2 scalar, 3 count; logit_cap: 3 cap);
            // binary kernels 0 a, 1 b, 2 out, 3 count (scalar_mul_weight: 1 = one fp16 value; geglu_fused_strided_batched:
            // 4 upStride, grid.y rows; projection_bias_add_batched: 1 bias [rows], 3 rows, grid.y rows).
            const int op = p.bits;
            const bool binary = op == kEwMul || op == kEwSigmoidMul || op == kEwGeglu || op == kEwBiasAdd || (op == kEwScalarMul && p.batched);
            const int iout = binary ? 2 : 1;
            NEED_BUF(0); NEED_BUF(iout);
            uint32_t count = 0, scalar_bits = 0, b_stride = 0;
            int batch = 1;
            if (binary) {
                NEED_BUF(1);
                if (!host_u32(in, r, 3, &count)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": the count constant is missing");
                if ((op == kEwGeglu || op == kEwBiasAdd) && p.batched) batch = batch_of(rec);
                b_stride = count;
                if (op == kEwGeglu && p.batched && !host_u32(in, r, 4, &b_stride)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": the up stride constant is missing");
            } else if (op == kEwScalarMul) {
                if (!host_u32(in, r, 2, &scalar_bits) || !host_u32(in, r, 3, &count)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": scalar / count constants are missing");
            } else {
                if (!host_u32(in, r, 2, &count)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": the count constant is missing");
                if (op == kEwLogitCap && !host_u32(in, r, 3, &scalar_bits)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": the cap constant is missing");
            }
            if (count == 0 || b_stride > 0x7fffffffu) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": count must be positive");
            const size_t n = (size_t)batch * count * 2;
            NEED_BYTES(0, n); NEED_BYTES(iout, n);
            const __half* b = nullptr;
            const __half* scalar_dev = nullptr;
            if (binary) {
                const size_t need = op == kEwBiasAdd ? (size_t)count * 2 : (op == kEwScalarMul ? 2 : (op == kEwGeglu ? ((size_t)(batch - 1) * b_stride + count) * 2 : n));
                NEED_BYTES(1, need);
                if (op == kEwScalarMul) scalar_dev = (const __half*)r.buf[1].ptr; else b = (const __half*)r.buf[1].ptr;
            }
            in.launches += 1;
            return check_cuda(ctx, launch_elementwise(l, op, (const __half*)r.buf[0].ptr, b, (__half*)r.buf[iout].ptr, (int)count, batch, (int)b_stride, as_f32(scalar_bits), scalar_dev), p.name.c_str());
        }
        case PK_GATE_SPLIT: {
            // attention_fused.metal:11-18: 0 input [H, 2 D], 1 query, 2 gate, 3 nHeads, 4 headDim.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_U32(3, heads); NEED_U32(4, d);
            if (heads == 0 || d == 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "gate_split: bad shape");
            NEED_BYTES(0, (size_t)heads * d * 4); NEED_BYTES(1, (size_t)heads * d * 2); NEED_BYTES(2, (size_t)heads * d * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_gate_split(l, (const __half*)r.buf[0].ptr, (__half*)r.buf[1].ptr, (__half*)r.buf[2].ptr, (int)heads, (int)d), "gate_split");
        }
        case PK_HEAD_NORM: {
            // attention_fused.metal:38-48 (1pw: 0 in, 1 weight, 2 out, 3 headDim, 4 eps), :147-151 (noscale: 0 data, 1 headDim,
            // 2 eps), :188-196 and :247-255 (batched: 3 nHeads, 4 headDim, 5 eps; grid (nHeads, rows)), :298-303 (noscale
            // batched: 1 nHeads, 2 headDim, 3 eps).  The threadgroup width of the record fixes the order of the sum of
            // squares; the batched kernels fix it at min(headDim, 256).
            const int mode = p.bits;
            const bool noscale = mode == kHeadNormNoScale;
            const int iout = noscale ? 0 : 2, ic = noscale ? 1 : 3;
            NEED_BUF(0); NEED_BUF(iout);
            if (!noscale) { NEED_BUF(1); }
            uint32_t d = 0, eps_bits = 0, nheads = rec.grid[0];
            if (p.batched) {
                if (!host_u32(in, r, ic, &nheads) || !host_u32(in, r, ic + 1, &d) || !host_u32(in, r, ic + 2, &eps_bits)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": nHeads / headDim / eps constants are missing");
            } else {
                if (!host_u32(in, r, ic, &d) || !host_u32(in, r, ic + 1, &eps_bits)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": headDim / eps constants are missing");
            }
            const int heads = (int)nheads * (p.batched ? batch_of(rec) : 1);
            if (heads <= 0 || d == 0 || d > 1024) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": bad shape");
            int tgs = p.batched ? (int)(d < 256 ? d : 256) : (rec.threadgroup[0] ? (int)rec.threadgroup[0] : 32);
            tgs = (tgs + 31) / 32 * 32;
            if (tgs > 1024) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": bad threadgroup width");
            NEED_BYTES(0, (size_t)heads * d * 2); NEED_BYTES(iout, (size_t)heads * d * 2);
            if (!noscale) { NEED_BYTES(1, (size_t)d * 2); }
            in.launches += 1;
            return check_cuda(ctx, launch_head_norm(l, mode, (const __half*)r.buf[0].ptr, noscale ? nullptr : (const __half*)r.buf[1].ptr, (__half*)r.buf[iout].ptr, heads, (int)d, as_f32(eps_bits), tgs), p.name.c_str());
        }
        case PK_ROW_NORM: {
            const RowNormName& n = kRowNorms[p.planes];
            uint32_t dim = (uint32_t)n.dim, eps_bits = 0;
            float eps = n.eps;
            int ix = 0, ipre = -1, iw = -1, ires = -1, iscalar = -1, iy = -1, iscale = -1;
            switch (n.form) {
                case 0: iw = 1; iy = 2; if (!host_u32(in, r, 3, &dim) || !host_u32(in, r, 4, &eps_bits)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": dim / eps constants are missing"); eps = as_f32(eps_bits); break;
                case 1: iw = 1; iy = 2; break;
                case 2: iw = 1; ires = 2; iy = 3; break;
                case 3: iw = 1; ires = 2; iscalar = 3; iy = 4; break;
                case 4: iscale = 1; if (!host_u32(in, r, 2, &dim) || !host_u32(in, r, 3, &eps_bits)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": dim / eps constants are missing"); eps = as_f32(eps_bits); break;
                case 5: iscale = 1; break;
                case 6: ipre = 1; iy = 2; iscale = 3; if (!host_u32(in, r, 4, &dim) || !host_u32(in, r, 5, &eps_bits)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": dim / eps constants are missing"); eps = as_f32(eps_bits); break;
                case 7: iy = 0; if (!host_u32(in, r, 1, &dim) || !host_u32(in, r, 2, &eps_bits)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": headDim / eps constants are missing"); eps = as_f32(eps_bits); break;
                default: iy = 0; break;
            }
            int rows = n.batched ? (int)rec.grid[0] : 1;
            int group_rows = 0, group_stride = 0;
            size_t base = 0;  // first value of the first row inside binding 0
            if (n.form == 9 || n.form == 10) {
                uint32_t qkv_dim = 6144, heads = 16;
                iy = 0;
                if (n.form == 9) {
                    if (!host_u32(in, r, 1, &dim) || !host_u32(in, r, 2, &eps_bits) || !host_u32(in, r, 3, &qkv_dim) || !host_u32(in, r, 4, &heads))
                        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": headDim / eps / qkvDim / qkHeads constants are missing");
                    eps = as_f32(eps_bits);
                } else {
                    dim = 128;
                }
                const bool k_heads = n.dim < 0;
                const int positions = batch_of(rec);
                if (heads == 0 || dim == 0 || (uint64_t)2 * heads * dim > qkv_dim || positions <= 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": bad head layout");
                group_rows = (int)heads; group_stride = (int)qkv_dim; rows = (int)heads * positions;
                base = k_heads ? (size_t)heads * dim : 0;
            }
            int tgs = (n.form == 8 || n.form == 10) ? 128 : (n.dim == 256 ? 256 : (rec.threadgroup[0] ? (int)rec.threadgroup[0] : 256));
            if (n.topology == kQ2) tgs = (int)dim / 8;
            if (rows <= 0 || dim == 0 || dim > 16384 || tgs < 32 || tgs % 32 || tgs > 1024 || (n.topology == kQ2 && dim % 256)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": bad rows, dim or threadgroup width");
            if (group_rows) {
                NEED_BUF(0);
                NEED_BYTES(0, ((size_t)(rows / group_rows - 1) * group_stride + base + (size_t)group_rows * dim) * 2);
                __half* data = (__half*)r.buf[0].ptr + base;
                in.launches += 1;
                return check_cuda(ctx, launch_row_norm(l, data, nullptr, nullptr, nullptr, nullptr, data, nullptr, rows, (int)dim, eps, n.topology, tgs, n.value, n.scale, group_rows, group_stride), p.name.c_str());
            }
            const size_t row_bytes = (size_t)rows * dim * 2;
            const int bufs[] = {ix, ipre, ires, iy};
            for (int b : bufs)
                if (b >= 0) {
                    if (!r.buf[b].present || r.buf[b].pos_strided) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": a buffer binding is missing");
                    if (r.buf[b].avail < row_bytes) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, p.name + ": a binding is smaller than the rows need");
                }
            if (iw >= 0) { NEED_BUF(iw); NEED_BYTES(iw, (size_t)dim * 2); }
            if (iscalar >= 0) { NEED_BUF(iscalar); NEED_BYTES(iscalar, 2); }
            if (iscale >= 0) {
                NEED_BUF(iscale); NEED_BYTES(iscale, (size_t)rows * 4);
                if (reinterpret_cast<uintptr_t>(r.buf[iscale].ptr) & 3u) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": the scale output must be 4-byte aligned");
            }
            auto hp = [&](int i) { return i >= 0 ? (const __half*)r.buf[i].ptr : (const __half*)nullptr; };
            in.launches += 1;
            return check_cuda(ctx, launch_row_norm(l, hp(ix), hp(ipre), hp(iw), hp(ires), hp(iscalar), iy >= 0 ? (__half*)r.buf[iy].ptr : nullptr,
                                                   iscale >= 0 ? (float*)r.buf[iscale].ptr : nullptr, rows, (int)dim, eps, n.topology, tgs, n.value, n.scale), p.name.c_str());
        }
        case PK_ROPE_KV_PREFILL: {
            // prefill_rope_kv.metal:64-79: 0 q [T, Hq, D] and 1 k [T, Hkv, D] (rotated in place), 2 v, 3 cos and 4 sin tables
            // [maxSeq, ropeDim], 5 K cache, 6 V cache, 7 headDim, 8 ropeDim, 9 qHeads, 10 kvHeads, 11 seqLen, 12 startPos,
            // 13 cacheSeqCapacity, 14 ropeLayout.  prefill_rope_kv_precise.metal:8-21 (analytic): 3 K cache, 4 V cache,
            // 5 headDim | ropeDim << 16, 6 qHeads | kvHeads << 16, 7 seqLen, 8 startPos, 9 cacheSeqCapacity, 10 ropeLayout, 11 log2(theta).
            const bool analytic = p.bits == 1;
            const int ikc = analytic ? 3 : 5, ic = analytic ? 5 : 7;
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_BUF(ikc); NEED_BUF(ikc + 1);
            uint32_t d = 0, rope = 0, hq = 0, hkv = 0, t = 0, start = 0, cap = 0, layout = 0, base_bits = 0;
            if (analytic) {
                uint32_t dims = 0, heads = 0;
                if (!host_u32(in, r, 5, &dims) || !host_u32(in, r, 6, &heads) || !host_u32(in, r, 7, &t) || !host_u32(in, r, 8, &start) || !host_u32(in, r, 9, &cap) ||
                    !host_u32(in, r, 10, &layout) || !host_u32(in, r, 11, &base_bits))
                    return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": a constant binding is missing");
                d = dims & 0xffffu; rope = dims >> 16; hq = heads & 0xffffu; hkv = heads >> 16;
            } else {
                NEED_BUF(3); NEED_BUF(4);
                if (!host_u32(in, r, ic, &d) || !host_u32(in, r, ic + 1, &rope) || !host_u32(in, r, ic + 2, &hq) || !host_u32(in, r, ic + 3, &hkv) || !host_u32(in, r, ic + 4, &t) ||
                    !host_u32(in, r, ic + 5, &start) || !host_u32(in, r, ic + 6, &cap) || !host_u32(in, r, ic + 7, &layout))
                    return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": a constant binding is missing");
            }
            if (d == 0 || d % 2 || rope == 0 || rope > d || rope % 2 || layout > 2 || (uint64_t)start + t > cap) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": bad shape, layout or positions past the cache capacity");
            NEED_BYTES(0, (size_t)t * hq * d * 2); NEED_BYTES(1, (size_t)t * hkv * d * 2); NEED_BYTES(2, (size_t)t * hkv * d * 2);
            NEED_BYTES(ikc, (size_t)hkv * cap * d * 2); NEED_BYTES(ikc + 1, (size_t)hkv * cap * d * 2);
            if (!analytic) { NEED_BYTES(3, ((size_t)start + t) * rope * 2); NEED_BYTES(4, ((size_t)start + t) * rope * 2); }
            in.launches += 1;
            return check_cuda(ctx, launch_rope_kv_prefill(l, (__half*)r.buf[0].ptr, (__half*)r.buf[1].ptr, (const __half*)r.buf[2].ptr, analytic ? nullptr : (const __half*)r.buf[3].ptr,
                                                          analytic ? nullptr : (const __half*)r.buf[4].ptr, (__half*)r.buf[ikc].ptr, (__half*)r.buf[ikc + 1].ptr, (int)d, (int)rope, (int)hq, (int)hkv,
                                                          t, start, cap, (int)layout, analytic ? as_f32(base_bits) : 0.0f, analytic ? 1 : 0, (size_t)rope), p.name.c_str());
        }
        case PK_ATTN_PREFILL: {
            // prefill_attention.metal:14-25: 0 q [T, Hq, D], 1 K cache, 2 V cache, 3 out, 4 headDim, 5 seqLen, 6 startPos,
            // 7 cacheSeqCapacity, 8 numKVHeads, 9 scale, 10 slidingWindow; grid (numQHeads, seqLen).
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_BUF(3); NEED_U32(4, d); NEED_U32(5, t); NEED_U32(6, start); NEED_U32(7, cap); NEED_U32(8, hkv); NEED_U32(9, scale_bits);
            uint32_t window = 0;
            (void)host_u32(in, r, 10, &window);
            const int hq = (int)rec.grid[0];
            if (hq <= 0 || hkv == 0 || hq % (int)hkv || hq / (int)hkv > 16 || (d != 64 && d != 128 && d != 256) || (uint64_t)start + t > cap)
                return fail(ctx, SMELT_ERR_UNSUPPORTED, p.name + ": head_dim 64 / 128 / 256, up to 16 query heads per KV head, positions inside the cache");
            NEED_BYTES(0, (size_t)t * hq * d * 2); NEED_BYTES(3, (size_t)t * hq * d * 2); NEED_BYTES(1, (size_t)hkv * cap * d * 2); NEED_BYTES(2, (size_t)hkv * cap * d * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_attention_prefill(l, (const __half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, (const __half*)r.buf[2].ptr, (__half*)r.buf[3].ptr, hq, (int)hkv, (int)d,
                                                            t, start, cap, as_f32(scale_bits), window), p.name.c_str());
        }
        case PK_EMBEDDING_GATHER_BATCHED: {
            // lut_matvec.metal:1121-1134: 0 table, 1 token ids [B], 2 out [B, hidden], 3 hidden, 4 batchSize.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_U32(3, hidden); NEED_U32(4, batch);
            if (hidden == 0 || batch == 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": bad shape");
            NEED_BYTES(1, (size_t)batch * 4); NEED_BYTES(2, (size_t)batch * hidden * 2);
            NEED_BYTES(0, (size_t)ctx->cfg.vocab_size * hidden * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_embedding_gather(l, (const __half*)r.buf[0].ptr, (const int32_t*)r.buf[1].ptr, (__half*)r.buf[2].ptr, (int)hidden, (int)batch, 1), p.name.c_str());
        }
        case PK_AFFINE_EMBEDDING_GATHER_BATCHED: {
            // lut_matvec.metal:1081-1116: 0 W, 1 scales, 2 biases, 3 token ids [B], 4 out [B, cols], 5 cols, 6 batchSize, 7 groupSize.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_BUF(3); NEED_BUF(4); NEED_U32(5, cols); NEED_U32(6, batch); NEED_U32(7, group);
            if (cols == 0 || group == 0 || cols % group || cols % 2 || batch == 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": bad cols / group / batch");
            NEED_BYTES(3, (size_t)batch * 4); NEED_BYTES(4, (size_t)batch * cols * 2);
            NEED_BYTES(0, (size_t)ctx->cfg.vocab_size * cols / 2); NEED_BYTES(1, (size_t)ctx->cfg.vocab_size * (cols / group) * 2); NEED_BYTES(2, (size_t)ctx->cfg.vocab_size * (cols / group) * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_affine_embedding_gather(l, (const uint8_t*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, (const __half*)r.buf[2].ptr, (const int32_t*)r.buf[3].ptr, (__half*)r.buf[4].ptr, (int)cols, (int)group, (int)batch), p.name.c_str());
        }
        case PK_BITPLANE_PRODUCER: {
            // signed_quant.metal:757-762: 0 input [B, cols], 1 planes, 2 activation scales, 3 cols; one threadgroup per
            // group, grid.y = rows of the batched form.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_U32(3, cols);
            const int rows = p.batched ? batch_of(rec) : 1;
            if (cols == 0 || cols % 128) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": cols must be a multiple of 128");
            NEED_BYTES(0, (size_t)rows * cols * 2); NEED_BYTES(1, (size_t)rows * (cols / 128) * p.planes * 16); NEED_BYTES(2, (size_t)rows * (cols / 128) * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_bitplane_producer(l, (const __half*)r.buf[0].ptr, nullptr, (uint32_t*)r.buf[1].ptr, (__half*)r.buf[2].ptr, (int)cols, p.planes, rows), p.name.c_str());
        }
        case PK_BITPLANE_SWIGLU_PRODUCER: {
            // signed_quant.metal:876-883: 0 gate, 1 up, 2 planes, 3 activation scales, 4 cols.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_BUF(3); NEED_U32(4, cols);
            if (cols == 0 || cols % 128) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": cols must be a multiple of 128");
            NEED_BYTES(0, (size_t)cols * 2); NEED_BYTES(1, (size_t)cols * 2); NEED_BYTES(2, (size_t)(cols / 128) * 5 * 16); NEED_BYTES(3, (size_t)(cols / 128) * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_bitplane_producer(l, (const __half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, (uint32_t*)r.buf[2].ptr, (__half*)r.buf[3].ptr, (int)cols, 5, 1), p.name.c_str());
        }
        case PK_BITPLANE_SIGMOID_MUL_PRODUCER: {
            // signed_quant.metal:985-992: 0 a, 1 b, 2 planes, 3 activation scales, 4 cols.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_BUF(3); NEED_U32(4, cols);
            if (cols == 0 || cols % 128) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": cols must be a multiple of 128");
            NEED_BYTES(0, (size_t)cols * 2); NEED_BYTES(1, (size_t)cols * 2); NEED_BYTES(2, (size_t)(cols / 128) * 6 * 16); NEED_BYTES(3, (size_t)(cols / 128) * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_bitplane_fused_producer(l, SMELT_BITPLANE_FRONT_SIGMOID_MUL, (const __half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, nullptr, nullptr,
                                                                  (uint32_t*)r.buf[2].ptr, (__half*)r.buf[3].ptr, (int)cols, 6, 0.0f, 32), p.name.c_str());
        }
        case PK_BITPLANE_NORM_SCALE_PRODUCER: {
            // signed_quant.metal:1225-1234: 0 norm scale (one float), 1 input, 2 norm weight, 3 planes, 4 activation scales, 5 cols.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_BUF(3); NEED_BUF(4); NEED_U32(5, cols);
            if (cols == 0 || cols % 128) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": cols must be a multiple of 128");
            NEED_BYTES(0, 4); NEED_BYTES(1, (size_t)cols * 2); NEED_BYTES(2, (size_t)cols * 2); NEED_BYTES(3, (size_t)(cols / 128) * p.planes * 16); NEED_BYTES(4, (size_t)(cols / 128) * 2);
            if (reinterpret_cast<uintptr_t>(r.buf[0].ptr) & 3u) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": the norm scale must be 4-byte aligned");
            in.launches += 1;
            return check_cuda(ctx, launch_bitplane_fused_producer(l, SMELT_BITPLANE_FRONT_NORM_SCALE, (const __half*)r.buf[1].ptr, nullptr, (const __half*)r.buf[2].ptr, (const float*)r.buf[0].ptr,
                                                                  (uint32_t*)r.buf[3].ptr, (__half*)r.buf[4].ptr, (int)cols, p.planes, 0.0f, 32), p.name.c_str());
        }
        case PK_BITPLANE_GATED_NORM_PRODUCER: {
            // signed_quant.metal:1149-1162: 0 input [H, 128], 1 gate, 2 weight [128], 3 planes, 4 activation scales, 5 headDim, 6 eps;
            // one threadgroup per head, whose width (32 or 128: the norm's own dispatch) selects the arithmetic.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_BUF(3); NEED_BUF(4); NEED_U32(5, d); NEED_U32(6, eps_bits);
            if (d != 128) return fail(ctx, SMELT_ERR_UNSUPPORTED, p.name + ": heads of 128");
            const int heads = (int)rec.grid[0];
            const int tgs = rec.threadgroup[0] ? (int)rec.threadgroup[0] : 32;
            if (heads <= 0 || tgs % 32 || tgs > 1024) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": bad grid or threadgroup width");
            NEED_BYTES(0, (size_t)heads * 256); NEED_BYTES(1, (size_t)heads * 256); NEED_BYTES(2, 256); NEED_BYTES(3, (size_t)heads * 6 * 16); NEED_BYTES(4, (size_t)heads * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_bitplane_fused_producer(l, SMELT_BITPLANE_FRONT_GATED_NORM_D128, (const __half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, (const __half*)r.buf[2].ptr, nullptr,
                                                                  (uint32_t*)r.buf[3].ptr, (__half*)r.buf[4].ptr, heads * 128, 6, as_f32(eps_bits), tgs), p.name.c_str());
        }
        case PK_SIGNED_EMBEDDING_GATHER: {
            // signed_quant.metal:722-745: 0 codes, 1 scales, 2 token ids, 3 out, 4 hidden; grid.y = tokens.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_BUF(3); NEED_U32(4, hidden);
            const int batch = batch_of(rec);
            if (hidden == 0 || hidden % 128) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": hidden must be a multiple of 128");
            NEED_BYTES(2, (size_t)batch * 4); NEED_BYTES(3, (size_t)batch * hidden * 2);
            // token ids are checked against vocab_size when they are written: the table must hold that many rows
            NEED_BYTES(0, (size_t)ctx->cfg.vocab_size * hidden * p.bits / 8); NEED_BYTES(1, (size_t)ctx->cfg.vocab_size * (hidden / 128) * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_signed_embedding_gather(l, p.bits, (const uint8_t*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, (const int32_t*)r.buf[2].ptr, (__half*)r.buf[3].ptr, (int)hidden, batch), p.name.c_str());
        }
        case PK_BITPLANE_MATVEC: case PK_BITPLANE_ADD: case PK_BITPLANE_GATEUP: {
            // signed_quant.metal:1564-1572 (matvec: 0 codes, 1 weight scales, 2 planes, 3 activation scales, 4 out, 5 rows,
            // 6 cols), :2246-2255 (add: 5 residual, 6 rows, 7 cols), :1823-1833 (gate/up: 0 gate codes, 1 gate scales,
            // 2 up codes, 3 up scales, 4 planes, 5 activation scales, 6 out, 7 rows, 8 cols).
            BitplaneArgs a = {};
            a.format = p.bits; a.n_planes = p.planes; a.batch = 1;
            int irows;
            if (p.kind == PK_BITPLANE_GATEUP) {
                for (int i = 0; i <= 6; ++i) if (!r.buf[i].present || r.buf[i].pos_strided) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": buffer bindings 0..6 are required");
                a.mode = 2; a.codes = (const uint8_t*)r.buf[0].ptr; a.wscales = (const __half*)r.buf[1].ptr; a.codes2 = (const uint8_t*)r.buf[2].ptr; a.wscales2 = (const __half*)r.buf[3].ptr;
                a.planes = (const uint32_t*)r.buf[4].ptr; a.ascales = (const __half*)r.buf[5].ptr; a.out = (__half*)r.buf[6].ptr;
                irows = 7;
            } else {
                const int nb = p.kind == PK_BITPLANE_ADD ? 5 : 4;
                for (int i = 0; i <= nb; ++i) if (!r.buf[i].present || r.buf[i].pos_strided) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": a buffer binding is missing");
                a.mode = p.kind == PK_BITPLANE_ADD ? 1 : 0;
                a.codes = (const uint8_t*)r.buf[0].ptr; a.wscales = (const __half*)r.buf[1].ptr; a.planes = (const uint32_t*)r.buf[2].ptr; a.ascales = (const __half*)r.buf[3].ptr;
                a.out = (__half*)r.buf[4].ptr;
                if (a.mode == 1) a.residual = (const __half*)r.buf[5].ptr;
                irows = nb + 1;
            }
            uint32_t rows = 0, cols = 0;
            if (!host_u32(in, r, irows, &rows) || !host_u32(in, r, irows + 1, &cols)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": rows / cols constants are missing");
            if (rows == 0 || cols == 0 || cols % 128) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": cols must be a multiple of 128");
            a.rows = (int)rows; a.cols = (int)cols;
            if (p.batched) {  // the prompt-row tiles bind the number of rows in use after cols (signed_quant.metal:1438-1452)
                uint32_t nb = 0;
                if (!host_u32(in, r, irows + 2, &nb) || nb == 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": the batch constant is missing");
                a.batch = (int)nb;
            }
            const size_t nbat = (size_t)a.batch;
            const size_t wbytes = (size_t)rows * cols / (p.bits == 1 ? 8 : 4), sbytes = (size_t)rows * (cols / 128) * 2;
            const int iplanes = a.mode == 2 ? 4 : 2;
            if (r.buf[0].avail < wbytes || r.buf[1].avail < sbytes || (a.mode == 2 && (r.buf[2].avail < wbytes || r.buf[3].avail < sbytes)) ||
                r.buf[iplanes].avail < nbat * (cols / 128) * p.planes * 16 || r.buf[iplanes + 1].avail < nbat * (cols / 128) * 2 || r.buf[iplanes + 2].avail < nbat * rows * 2 ||
                (a.mode == 1 && r.buf[5].avail < (size_t)rows * 2))
                return fail(ctx, SMELT_ERR_OUT_OF_RANGE, p.name + ": a binding is smaller than the shape needs");
            if ((reinterpret_cast<uintptr_t>(a.codes) | reinterpret_cast<uintptr_t>(a.codes2) | reinterpret_cast<uintptr_t>(a.planes)) & 15u)
                return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": codes and planes must be 16-byte aligned");
            in.launches += 1;
            return check_cuda(ctx, launch_bitplane_matvec(l, a), p.name.c_str());
        }
        case PK_BITPLANE_BANK4: {
            // signed_quant.metal:2475-2497, :2602-2632: 0 codes and 1 weight scales of the members stacked by rows, 2 planes,
            // 3 activation scales, 4..7 the members' outputs, 8..11 their row counts (trailing members may be empty), 12 cols.
            // Every row is the standalone matvec's arithmetic, so the members run as that kernel over their row ranges.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_BUF(3); NEED_U32(12, cols);
            if (cols == 0 || cols % 128) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": cols must be a multiple of 128");
            const size_t row_bytes = (size_t)cols / (p.bits == 1 ? 8 : 4), groups = cols / 128;
            NEED_BYTES(2, groups * p.planes * 16); NEED_BYTES(3, groups * 2);
            if ((reinterpret_cast<uintptr_t>(r.buf[0].ptr) | reinterpret_cast<uintptr_t>(r.buf[2].ptr)) & 15u) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": codes and planes must be 16-byte aligned");
            size_t first = 0;
            for (int m = 0; m < 4; ++m) {
                uint32_t rows = 0;
                if (!host_u32(in, r, 8 + m, &rows)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": a row count is missing");
                if (rows == 0) continue;
                if (!r.buf[4 + m].present || r.buf[4 + m].pos_strided || r.buf[4 + m].avail < (size_t)rows * 2) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": a member's output binding is missing or too small");
                if (r.buf[0].avail < (first + rows) * row_bytes || r.buf[1].avail < (first + rows) * groups * 2) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, p.name + ": the stacked weights are smaller than the members need");
                BitplaneArgs a = {};
                a.format = p.bits; a.n_planes = p.planes; a.batch = 1; a.mode = 0;
                a.codes = (const uint8_t*)r.buf[0].ptr + first * row_bytes; a.wscales = (const __half*)r.buf[1].ptr + first * groups;
                a.planes = (const uint32_t*)r.buf[2].ptr; a.ascales = (const __half*)r.buf[3].ptr; a.out = (__half*)r.buf[4 + m].ptr;
                a.rows = (int)rows; a.cols = (int)cols;
                in.launches += 1;
                const smelt_status st = check_cuda(ctx, launch_bitplane_matvec(l, a), p.name.c_str());
                if (st) return st;
                first += rows;
            }
            return SMELT_OK;
        }
        case PK_SIGNED_BANK: {
            // signed_quant.metal:2638-2650 (dual, virtual bank: 0 / 1 first codes and scales, 2 / 3 second, 4 input, 5 / 6 outputs,
            // 7 / 8 row counts, 9 cols), :2802-2813 (packed bank: 0 codes, 1 scales, 2 input, 3 / 4 outputs, 5 / 6 row counts,
            // 7 cols), :2867-2882 (packed bank of four: 3..6 outputs, 7..10 row counts, 11 cols).  Exact lowerings of the
            // standalone binary matvec: the members run as that kernel.
            // signed_quant_precise.metal:186-199 (ternary-affine bank of four: 0 codes, 1 scales, 2 bias scales, 3 input, 4..7 outputs,
            // 8..11 row counts, 12 cols) is layout 3.
            const int layout = p.bits;
            const int n_members = layout >= 2 ? 4 : 2;
            const int ix = layout == 0 ? 4 : (layout == 3 ? 3 : 2), iout = ix + 1, irows = iout + n_members, icols = irows + n_members;
            const int wbits = layout == 3 ? 2 : 1;
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(ix);
            uint32_t cols = 0;
            if (!host_u32(in, r, icols, &cols) || cols == 0 || cols % 128) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": cols must be a positive multiple of 128");
            const size_t row_bytes = (size_t)cols * wbits / 8, groups = cols / 128;
            NEED_BYTES(ix, (size_t)cols * 2);
            size_t first = 0;
            for (int m = 0; m < n_members; ++m) {
                uint32_t rows = 0;
                if (!host_u32(in, r, irows + m, &rows)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": a row count is missing");
                if (rows == 0) continue;
                const int ic = layout == 0 ? 2 * m : 0, is = ic + 1;
                if (!r.buf[ic].present || !r.buf[is].present || r.buf[ic].pos_strided || r.buf[is].pos_strided) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": a member's weights are missing");
                const size_t off = layout == 0 ? 0 : first;
                if (r.buf[ic].avail < (off + rows) * row_bytes || r.buf[is].avail < (off + rows) * groups * 2) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, p.name + ": the weights are smaller than the members need");
                if (!r.buf[iout + m].present || r.buf[iout + m].pos_strided || r.buf[iout + m].avail < (size_t)rows * 2) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": a member's output binding is missing or too small");
                SignedArgs a = {};
                a.codes[0] = (const uint8_t*)r.buf[ic].ptr + off * row_bytes; a.scales[0] = (const __half*)r.buf[is].ptr + off * groups;
                a.x = (const __half*)r.buf[ix].ptr; a.y = (__half*)r.buf[iout + m].ptr;
                a.rows = (int)rows; a.cols = (int)cols; a.batch = 1; a.bits = wbits;
                in.launches += 1;
                const smelt_status st = check_cuda(ctx, launch_signed(l, kSignedPlain, a), p.name.c_str());
                if (st) return st;
                first += rows;
            }
            return SMELT_OK;
        }
        case PK_CONV1D_SILU: {
            // conv1d.metal:271-278: 0 state [C, K] (in place), 1 new value [C], 2 weight [C, K], 3 out [C], 4 channels, 5 kernel size.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_BUF(3);
            uint32_t channels = (uint32_t)p.head_dim, ksize = (uint32_t)p.n_q;
            if (!p.fixed_shape) {
                NEED_U32(4, c_); NEED_U32(5, k_);
                channels = c_; ksize = k_;
            }
            if (channels == 0 || ksize == 0 || ksize > 8) return fail(ctx, SMELT_ERR_UNSUPPORTED, "conv1d_update_silu: kernel size in 1..8");
            NEED_BYTES(0, (size_t)channels * ksize * 2); NEED_BYTES(1, (size_t)channels * 2); NEED_BYTES(2, (size_t)channels * ksize * 2); NEED_BYTES(3, (size_t)channels * 2);
            in.launches += 1;
            {
                const smelt_status st = check_cuda(ctx, launch_conv1d_update_silu(l, (__half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, (const __half*)r.buf[2].ptr, (__half*)r.buf[3].ptr, (int)channels, (int)ksize), p.name.c_str());
                if (st || !(p.fixed_shape && p.n_kv > 0)) return st;
            }
            in.launches += 1;  // the fused name: its Q / K heads of 128, L2-normalised in place in the output
            return check_cuda(ctx, launch_row_norm(l, (const __half*)r.buf[3].ptr, nullptr, nullptr, nullptr, nullptr, (__half*)r.buf[3].ptr, nullptr, p.n_kv, 128, 1e-6f, SMELT_ROW_NORM_STRIDED, 128, 4, 1), p.name.c_str());
        }
        case PK_RMS_SCALE_QK: {
            // norms.metal:1380-1386: 0 qkv (in place), 1 headDim, 2 eps, 3 qkvDim, 4 qkHeads; grid.y = rows of qkv.
            NEED_BUF(0); NEED_U32(1, d); NEED_U32(2, eps_bits); NEED_U32(3, qkv_dim); NEED_U32(4, qk_heads);
            const int rows = batch_of(rec);
            if (d == 0 || qk_heads == 0 || (uint64_t)2 * qk_heads * d > qkv_dim) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "rms_scale_qk: bad shape");
            NEED_BYTES(0, (size_t)rows * qkv_dim * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_rms_scale_qk(l, (__half*)r.buf[0].ptr, (int)d, as_f32(eps_bits), (int)qkv_dim, (int)qk_heads, rows), "rms_scale_qk");
        }
        case PK_DELTANET_DECODE: {
            // recurrence.metal:511-522: 0 state [Hv, D, D] (in place), 1 qkv, 2 b, 3 a, 4 A_log, 5 dt_bias, 6 out [Hv, D],
            // 7 headDim, 8 headScale (unused by the kernel: q arrives scaled), 9 valueHeads, 10 qkHeads; the
            // specialised names fix 7, 9 and 10.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_BUF(3); NEED_BUF(4); NEED_BUF(5); NEED_BUF(6);
            uint32_t d = (uint32_t)p.head_dim, hv = (uint32_t)p.n_q, hqk = (uint32_t)p.n_kv;
            if (!p.fixed_shape) {
                NEED_U32(7, d_); NEED_U32(9, hv_); NEED_U32(10, hqk_);
                d = d_; hv = hv_; hqk = hqk_;
            }
            if (d == 0 || d % 32 || d > 256 || hv == 0 || hqk == 0 || hv % hqk) return fail(ctx, SMELT_ERR_UNSUPPORTED, p.name + ": head_dim a multiple of 32 up to 256, value heads a multiple of q/k heads");
            NEED_BYTES(0, (size_t)hv * d * d * 2); NEED_BYTES(1, ((size_t)2 * hqk + hv) * d * 2); NEED_BYTES(2, (size_t)hv * 2); NEED_BYTES(3, (size_t)hv * 2);
            NEED_BYTES(4, (size_t)hv * 2); NEED_BYTES(5, (size_t)hv * 2); NEED_BYTES(6, (size_t)hv * d * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_deltanet_recurrence_decode(l, (__half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, (const __half*)r.buf[2].ptr, (const __half*)r.buf[3].ptr,
                                                                     (const __half*)r.buf[4].ptr, (const __half*)r.buf[5].ptr, (__half*)r.buf[6].ptr, (int)d, (int)hv, (int)hqk), p.name.c_str());
        }
        case PK_CONV1D_SILU_PREFILL: {
            // conv1d.metal:129-225: 0 state [C, K] (in place), 1 qkv [T, C] (in place), 2 weight [C, K], 3 seqLen, 4 channels,
            // 5 kernel size (the c6144_k4 name fixes 4 and 5), 6 history [T + 1, C, K] (the checkpoint name only).
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_U32(3, seq_len);
            uint32_t channels = (uint32_t)p.head_dim, ksize = (uint32_t)p.n_q;
            if (!p.fixed_shape) {
                NEED_U32(4, c_); NEED_U32(5, k_);
                channels = c_; ksize = k_;
            }
            if (channels == 0 || ksize == 0 || ksize > 8) return fail(ctx, SMELT_ERR_UNSUPPORTED, p.name + ": kernel size in 1..8");
            NEED_BYTES(0, (size_t)channels * ksize * 2); NEED_BYTES(1, (size_t)seq_len * channels * 2); NEED_BYTES(2, (size_t)channels * ksize * 2);
            __half* history = nullptr;
            if (p.bits == 1) {
                NEED_BUF(6); NEED_BYTES(6, ((size_t)seq_len + 1) * channels * ksize * 2);
                history = (__half*)r.buf[6].ptr;
            }
            in.launches += 1;
            return check_cuda(ctx, launch_conv1d_update_silu_prefill(l, (__half*)r.buf[0].ptr, (__half*)r.buf[1].ptr, (const __half*)r.buf[2].ptr, (int)seq_len, (int)channels, (int)ksize, history), p.name.c_str());
        }
        case PK_DELTANET_PREFILL: {
            // prefill_recurrence.metal:580-592: 0 state [Hv, D, D] (in place), 1 qkv [T, (2 Hqk + Hv) D], 2 b [T, Hv], 3 a [T, Hv],
            // 4 A_log, 5 dt_bias, 6 out [T, Hv, D], 7 headDim, 8 valueHeads, 9 qkHeads, 10 seqLen, 11 history [T + 1, Hv, D, D]
            // (the checkpoint name only); the specialised names fix the shape and bind seqLen at 7 (:290-299).
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_BUF(3); NEED_BUF(4); NEED_BUF(5); NEED_BUF(6);
            uint32_t d = (uint32_t)p.head_dim, hv = (uint32_t)p.n_q, hqk = (uint32_t)p.n_kv, seq_len = 0;
            if (p.fixed_shape) {
                NEED_U32(7, t_);
                seq_len = t_;
            } else {
                NEED_U32(7, d_); NEED_U32(8, hv_); NEED_U32(9, hqk_); NEED_U32(10, t_);
                d = d_; hv = hv_; hqk = hqk_; seq_len = t_;
            }
            if (d == 0 || d % 32 || d > 256 || hv == 0 || hqk == 0 || hv % hqk) return fail(ctx, SMELT_ERR_UNSUPPORTED, p.name + ": head_dim a multiple of 32 up to 256, value heads a multiple of q/k heads");
            NEED_BYTES(0, (size_t)hv * d * d * 2); NEED_BYTES(1, (size_t)seq_len * ((size_t)2 * hqk + hv) * d * 2); NEED_BYTES(2, (size_t)seq_len * hv * 2); NEED_BYTES(3, (size_t)seq_len * hv * 2);
            NEED_BYTES(4, (size_t)hv * 2); NEED_BYTES(5, (size_t)hv * 2); NEED_BYTES(6, (size_t)seq_len * hv * d * 2);
            __half* history = nullptr;
            if (p.bits == 1) {
                NEED_BUF(11); NEED_BYTES(11, ((size_t)seq_len + 1) * hv * d * d * 2);
                history = (__half*)r.buf[11].ptr;
            }
            in.launches += 1;
            return check_cuda(ctx, launch_deltanet_recurrence_prefill(l, (__half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, (const __half*)r.buf[2].ptr, (const __half*)r.buf[3].ptr,
                                                                      (const __half*)r.buf[4].ptr, (const __half*)r.buf[5].ptr, (__half*)r.buf[6].ptr, (int)d, (int)hv, (int)hqk, (int)seq_len, history), p.name.c_str());
        }
        case PK_DN_GATES: {
            // recurrence.metal:839-847: 0 b, 1 a, 2 A_log, 3 dt_bias, 4 beta out, 5 g out, 6 numHeads.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_BUF(3); NEED_BUF(4); NEED_BUF(5); NEED_U32(6, heads);
            if (heads == 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "compute_gates: no heads");
            for (int i = 0; i < 6; ++i)
                if (r.buf[i].avail < (size_t)heads * 2) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "compute_gates: a binding is shorter than numHeads halves");
            in.launches += 1;
            return check_cuda(ctx, launch_dn_compute_gates(l, (const __half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, (const __half*)r.buf[2].ptr, (const __half*)r.buf[3].ptr,
                                                           (__half*)r.buf[4].ptr, (__half*)r.buf[5].ptr, (int)heads), "compute_gates");
        }
        case PK_DN_STATE_UPDATE: {
            // state_decay (recurrence.metal:48-55): 0 state, 1 g, 2 headDim.  outer_product_update (:113-121): 0 state, 1 key,
            // 2 delta (fp32), 3 headDim.  state_decay_update (:246-255): 0 state, 1 g, 2 key, 3 delta, 4 headDim.  One
            // threadgroup per head: grid.x heads (state_decay dispatched by threads: grid.x = heads * D * D).
            const int form = p.bits, ig = form == 1 ? -1 : 1, ikey = form == 0 ? -1 : (form == 1 ? 1 : 2), idelta = ikey < 0 ? -1 : ikey + 1;
            const int id = form == 0 ? 2 : (form == 1 ? 3 : 4);
            NEED_BUF(0);
            uint32_t d = 0;
            if (!host_u32(in, r, id, &d) || d == 0 || d > 1024) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": headDim constant is missing or out of range");
            uint32_t heads = rec.grid[0];
            if ((rec.style & 3) == 1) {
                if (heads % (d * d)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": a grid of threads must hold heads * headDim^2");
                heads /= d * d;
            }
            if (heads == 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": no heads in the grid");
            NEED_BYTES(0, (size_t)heads * d * d * 2);
            const __half *g = nullptr, *key = nullptr;
            const float* delta = nullptr;
            if (ig >= 0) {
                if (!r.buf[ig].present || r.buf[ig].avail < (size_t)heads * 2) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": the gate binding is missing or short");
                g = (const __half*)r.buf[ig].ptr;
            }
            if (ikey >= 0) {
                if (!r.buf[ikey].present || r.buf[ikey].avail < (size_t)heads * d * 2 || !r.buf[idelta].present || r.buf[idelta].avail < (size_t)heads * d * 4)
                    return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": the key or delta binding is missing or short");
                key = (const __half*)r.buf[ikey].ptr;
                delta = (const float*)r.buf[idelta].ptr;
            }
            in.launches += 1;
            return check_cuda(ctx, launch_dn_state_update(l, (__half*)r.buf[0].ptr, g, key, delta, (int)d, (int)heads), p.name.c_str());
        }
        case PK_DN_READOUT: {
            // kv_mem_readout (recurrence.metal:70-77): 0 state, 1 key, 2 kv_mem (fp32), 3 headDim.  kv_readout_delta (:150-160):
            // 0 state, 1 key, 2 value, 3 g, 4 beta, 5 delta (fp32), 6 headDim.  gates_kv_readout_delta (:186-199): 0 state, 1 key,
            // 2 value, 3 b, 4 a, 5 A_log, 6 dt_bias, 7 delta, 8 g out, 9 headDim.  query_readout (:282-290): 0 state, 1 query,
            // 2 out, 3 headDim, 4 scale.  grid.x = heads.
            const int mode = p.bits;
            const int nbuf = mode == 0 ? 3 : (mode == 1 ? 6 : (mode == 2 ? 9 : 3));
            for (int i = 0; i < nbuf; ++i)
                if (!r.buf[i].present || r.buf[i].pos_strided) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": a buffer binding is missing");
            uint32_t d = 0, scale_bits = 0;
            if (!host_u32(in, r, nbuf, &d) || d == 0 || d > 256) return fail(ctx, SMELT_ERR_UNSUPPORTED, p.name + ": headDim constant missing or above 256");
            if (mode == 3 && !host_u32(in, r, 4, &scale_bits)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": the scale constant is missing");
            const uint32_t heads = rec.grid[0];
            if (heads == 0) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": no heads in the grid");
            const size_t vec = (size_t)heads * d * 2, hb = (size_t)heads * 2;
            NEED_BYTES(0, (size_t)heads * d * d * 2); NEED_BYTES(1, vec);
            const __half *value = nullptr, *g = nullptr, *beta = nullptr, *b = nullptr, *a = nullptr, *al = nullptr, *dt = nullptr;
            float* out32 = nullptr;
            __half *out16 = nullptr, *g_out = nullptr;
            if (mode == 0) {
                NEED_BYTES(2, vec * 2);
                out32 = (float*)r.buf[2].ptr;
            } else if (mode == 1) {
                NEED_BYTES(2, vec); NEED_BYTES(3, hb); NEED_BYTES(4, hb); NEED_BYTES(5, vec * 2);
                value = (const __half*)r.buf[2].ptr; g = (const __half*)r.buf[3].ptr; beta = (const __half*)r.buf[4].ptr; out32 = (float*)r.buf[5].ptr;
            } else if (mode == 2) {
                NEED_BYTES(2, vec); NEED_BYTES(3, hb); NEED_BYTES(4, hb); NEED_BYTES(5, hb); NEED_BYTES(6, hb); NEED_BYTES(7, vec * 2); NEED_BYTES(8, hb);
                value = (const __half*)r.buf[2].ptr; b = (const __half*)r.buf[3].ptr; a = (const __half*)r.buf[4].ptr; al = (const __half*)r.buf[5].ptr;
                dt = (const __half*)r.buf[6].ptr; out32 = (float*)r.buf[7].ptr; g_out = (__half*)r.buf[8].ptr;
            } else {
                NEED_BYTES(2, vec);
                out16 = (__half*)r.buf[2].ptr;
            }
            in.launches += 1;
            return check_cuda(ctx, launch_dn_readout(l, mode, (const __half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, value, g, beta, b, a, al, dt, out32, out16, g_out,
                                                     (int)d, as_f32(scale_bits), (int)heads), p.name.c_str());
        }
        case PK_DN_DELTA: {
            // recurrence.metal:95-102: 0 value, 1 kv_mem (fp32), 2 beta, 3 delta (fp32), 4 headDim; one thread per element.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_BUF(3); NEED_U32(4, d);
            const uint64_t total = (rec.style & 3) == 1 ? rec.grid[0] : (uint64_t)rec.grid[0] * (rec.threadgroup[0] ? rec.threadgroup[0] : 1);
            if (d == 0 || total == 0 || total % d || total > (1u << 30)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "compute_delta: the grid must hold heads * headDim threads");
            const uint32_t heads = (uint32_t)(total / d);
            NEED_BYTES(0, total * 2); NEED_BYTES(1, total * 4); NEED_BYTES(2, (size_t)heads * 2); NEED_BYTES(3, total * 4);
            in.launches += 1;
            return check_cuda(ctx, launch_dn_compute_delta(l, (const __half*)r.buf[0].ptr, (const float*)r.buf[1].ptr, (const __half*)r.buf[2].ptr, (float*)r.buf[3].ptr, (int)d, (int)heads), "compute_delta");
        }
        case PK_DN_FUSED_DECODE: {
            // recurrence.metal:310-333: 0 state [H, Dv, Dk], 1 qkv, 2 b, 3 a, 4 A_log, 5 dt_bias, 6 out, 7 conv state, 8 conv weight,
            // 9 z, 10 norm weight, 11 headDim, 12 headScale, 13 qkvDim, 14 convK, 15 numHeads, 16 rmsEps; one threadgroup per head,
            // whose width fixes the order of the three sums of squares.
            for (int i = 0; i <= 10; ++i)
                if (!r.buf[i].present || r.buf[i].pos_strided) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "deltanet_recurrence_fused: a buffer binding is missing");
            NEED_U32(11, d); NEED_U32(12, scale_bits); NEED_U32(13, qkv_dim); NEED_U32(14, conv_k); NEED_U32(15, heads); NEED_U32(16, eps_bits);
            const int tgs = rec.threadgroup[0] ? (int)rec.threadgroup[0] : 256;
            if (d == 0 || d % 32 || d > 256 || heads == 0 || conv_k == 0 || conv_k > 8 || (uint64_t)3 * heads * d > qkv_dim || tgs % 32 || tgs > 1024)
                return fail(ctx, SMELT_ERR_UNSUPPORTED, "deltanet_recurrence_fused: head_dim a multiple of 32 up to 256, conv kernel up to 8, threadgroup a multiple of 32");
            const size_t hb = (size_t)heads * 2, hd = (size_t)heads * d * 2, cs = (size_t)qkv_dim * conv_k * 2;
            NEED_BYTES(0, hd * d); NEED_BYTES(1, (size_t)qkv_dim * 2); NEED_BYTES(2, hb); NEED_BYTES(3, hb); NEED_BYTES(4, hb); NEED_BYTES(5, hb); NEED_BYTES(6, hd);
            NEED_BYTES(7, cs); NEED_BYTES(8, cs); NEED_BYTES(9, hd); NEED_BYTES(10, (size_t)d * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_dn_fused_decode(l, (__half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, (const __half*)r.buf[2].ptr, (const __half*)r.buf[3].ptr,
                                                          (const __half*)r.buf[4].ptr, (const __half*)r.buf[5].ptr, (__half*)r.buf[6].ptr, (__half*)r.buf[7].ptr,
                                                          (const __half*)r.buf[8].ptr, (const __half*)r.buf[9].ptr, (const __half*)r.buf[10].ptr, (int)d, as_f32(scale_bits),
                                                          (int)qkv_dim, (int)conv_k, (int)heads, as_f32(eps_bits), tgs), "deltanet_recurrence_fused");
        }
        case PK_DN_FUSED_PREFILL: {
            // prefill_recurrence.metal:42-62: 0 state [H, Dv, Dk], 1 conv state, 2 qkv [T, C] (in place), 3 conv weight, 4 A_log,
            // 5 dt_bias, 6 b [T, H], 7 a [T, H], 8 out [T, H, D], 9 headDim, 10 numHeads, 11 seqLen, 12 qkvDim, 13 convKernel,
            // 14 headScale, 15 l2Eps; one threadgroup of headDim threads per head.
            for (int i = 0; i <= 8; ++i)
                if (!r.buf[i].present || r.buf[i].pos_strided) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "deltanet_recurrence_prefill: a buffer binding is missing");
            NEED_U32(9, d); NEED_U32(10, heads); NEED_U32(11, seq_len); NEED_U32(12, qkv_dim); NEED_U32(13, conv_k); NEED_U32(14, scale_bits); NEED_U32(15, eps_bits);
            const int tgs = rec.threadgroup[0] ? (int)rec.threadgroup[0] : (int)((d + 31) / 32 * 32);
            if (d == 0 || d > 256 || heads == 0 || conv_k == 0 || conv_k > 8 || (uint64_t)3 * heads * d > qkv_dim || tgs % 32 || tgs > 1024)
                return fail(ctx, SMELT_ERR_UNSUPPORTED, "deltanet_recurrence_prefill: head_dim up to 256, conv kernel up to 8, threadgroup a multiple of 32");
            const size_t hb = (size_t)heads * 2, cs = (size_t)qkv_dim * conv_k * 2;
            NEED_BYTES(0, (size_t)heads * d * d * 2); NEED_BYTES(1, cs); NEED_BYTES(2, (size_t)seq_len * qkv_dim * 2); NEED_BYTES(3, cs); NEED_BYTES(4, hb); NEED_BYTES(5, hb);
            NEED_BYTES(6, (size_t)seq_len * hb); NEED_BYTES(7, (size_t)seq_len * hb); NEED_BYTES(8, (size_t)seq_len * heads * d * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_dn_fused_prefill(l, (__half*)r.buf[0].ptr, (__half*)r.buf[1].ptr, (__half*)r.buf[2].ptr, (const __half*)r.buf[3].ptr,
                                                           (const __half*)r.buf[4].ptr, (const __half*)r.buf[5].ptr, (const __half*)r.buf[6].ptr, (const __half*)r.buf[7].ptr,
                                                           (__half*)r.buf[8].ptr, (int)d, (int)heads, (int)seq_len, (int)qkv_dim, (int)conv_k, as_f32(scale_bits), as_f32(eps_bits), tgs),
                              "deltanet_recurrence_prefill");
        }
        case PK_RMS_NORM_GATED: {
            // norms.metal:1093-1099: 0 in [H, D], 1 gate [H, D], 2 weight [D], 3 out, 4 headDim, 5 eps; one threadgroup per
            // head, whose width fixes the order of the sum of squares.  rms_norm_gated_d128 (norms_gated_precise.metal:20-52)
            // fixes headDim 128 and eps 1e-6 and materialises the norm in fp16; its _batched form binds numHeads at 4 and
            // takes grid.y rows of heads (:54-87).
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_BUF(3);
            uint32_t d = (uint32_t)p.head_dim;
            float eps = 1e-6f;
            int heads = (int)rec.grid[0];
            if (!p.fixed_shape) {
                NEED_U32(4, d_); NEED_U32(5, eps_bits);
                d = d_; eps = as_f32(eps_bits);
            } else if (p.n_kv == 1) {
                NEED_U32(4, num_heads);
                if (num_heads != rec.grid[0]) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": numHeads must equal grid.x");
                heads = (int)num_heads * batch_of(rec);
            }
            const int tgs = !p.fixed_shape && rec.threadgroup[0] ? (int)rec.threadgroup[0] : 32;
            if (heads <= 0 || d == 0 || tgs % 32 || tgs > 1024) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": bad shape");
            NEED_BYTES(0, (size_t)heads * d * 2); NEED_BYTES(1, (size_t)heads * d * 2); NEED_BYTES(2, (size_t)d * 2); NEED_BYTES(3, (size_t)heads * d * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_rms_norm_gated(l, (const __half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, (const __half*)r.buf[2].ptr, (__half*)r.buf[3].ptr, (int)d, eps, heads, tgs, p.fixed_shape), p.name.c_str());
        }
        case PK_ADD: {
            // activations.metal:56-61: 0 a, 1 b, 2 out, 3 count.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_U32(3, count);
            NEED_BYTES(0, (size_t)count * 2); NEED_BYTES(1, (size_t)count * 2); NEED_BYTES(2, (size_t)count * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_elementwise_add(l, (const __half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, (__half*)r.buf[2].ptr, (int64_t)count), "elementwise_add");
        }
        case PK_SWIGLU: {
            // activations_precise.metal:9-14: 0 gate, 1 up, 2 out, 3 count.
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_U32(3, count);
            NEED_BYTES(0, (size_t)count * 2); NEED_BYTES(1, (size_t)count * 2); NEED_BYTES(2, (size_t)count * 2);
            in.launches += 1;
            return check_cuda(ctx, launch_swiglu_fused(l, (const __half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, (__half*)r.buf[2].ptr, (int64_t)count), "swiglu_fused");
        }
        case PK_FUSED_NORM_QKV: {
            // 0-2 Q, 3-5 K, 6-8 V (W, scales, biases), 9 x, 10 norm weight, 11-13 outputs;
            // constants 14 rows of Q, 15 rows of K and of V, 16 eps, 17 batch.
            for (int i = 0; i <= 13; ++i)
                if (!r.buf[i].present || r.buf[i].pos_strided) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": buffer binding missing");
            NEED_U32(14, rows_q); NEED_U32(15, rows_kv); NEED_U32(16, eps_bits); NEED_U32(17, nb);
            if (rows_q == 0 || rows_kv == 0 || nb == 0 || nb > 64) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": bad rows / batch");
            AffineArgs a = {};
            const uint32_t rows[3] = {rows_q, rows_kv, rows_kv};
            const int groups = p.cols / p.group;
            a.nseg = 3;
            for (int i = 0; i < 3; ++i) {
                if (r.buf[3 * i].avail < (size_t)rows[i] * p.cols / 2 || r.buf[3 * i + 1].avail < (size_t)rows[i] * groups * 2 || r.buf[3 * i + 2].avail < (size_t)rows[i] * groups * 2)
                    return fail(ctx, SMELT_ERR_OUT_OF_RANGE, p.name + ": weight tensor extends past the weights slot");
                if (r.buf[11 + i].avail < (size_t)nb * rows[i] * 2) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, p.name + ": output slot too small");
                a.seg[i].w = r.buf[3 * i].ptr; a.seg[i].s = (const __half*)r.buf[3 * i + 1].ptr; a.seg[i].b = (const __half*)r.buf[3 * i + 2].ptr;
                a.seg[i].y = (__half*)r.buf[11 + i].ptr; a.seg[i].rows = (int)rows[i];
                a.rows += (int)rows[i];
            }
            NEED_BYTES(9, (size_t)nb * p.cols * 2); NEED_BYTES(10, (size_t)p.cols * 2);
            a.w[0] = a.seg[0].w; a.s[0] = a.seg[0].s; a.b[0] = a.seg[0].b; a.y = a.seg[0].y;
            a.x = (const __half*)r.buf[9].ptr; a.norm_w = (const __half*)r.buf[10].ptr; a.norm_eps = as_f32(eps_bits);
            a.cols = p.cols; a.batch = (int)nb; a.err = ctx->err_dev; a.sm_count = ctx->sm_count; a.part_scratch = ctx->qmm_scratch; a.part_scratch_bytes = ctx->qmm_scratch_bytes; a.part_counters = ctx->qmm_counters;
            in.launches += 1;
            cudaError_t e = launch_affine(l, kAffinePlain, a, p.group);
            if (e == cudaErrorNotSupported) return fail(ctx, SMELT_ERR_UNSUPPORTED, p.name + ": shape not eligible for the fused kernel");
            return check_cuda(ctx, e, p.name.c_str());
        }
        case PK_FUSED_NORM_GATEUP: {
            // 0-2 gate, 3-5 up, 6 x, 7 y, 9 norm weight; constants 8 rows, 10 eps, 11 batch.
            for (int i = 0; i <= 7; ++i)
                if (!r.buf[i].present || r.buf[i].pos_strided) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": buffer binding missing");
            NEED_BUF(9); NEED_U32(8, rows); NEED_U32(10, eps_bits); NEED_U32(11, nb);
            if (rows == 0 || nb == 0 || nb > 64) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, p.name + ": bad rows / batch");
            const int groups = p.cols / p.group;
            AffineArgs a = {};
            for (int s2 = 0; s2 < 2; ++s2) {
                if (r.buf[3 * s2].avail < (size_t)rows * p.cols / 2 || r.buf[3 * s2 + 1].avail < (size_t)rows * groups * 2 || r.buf[3 * s2 + 2].avail < (size_t)rows * groups * 2)
                    return fail(ctx, SMELT_ERR_OUT_OF_RANGE, p.name + ": weight tensor extends past the weights slot");
                a.w[s2] = r.buf[3 * s2].ptr; a.s[s2] = (const __half*)r.buf[3 * s2 + 1].ptr; a.b[s2] = (const __half*)r.buf[3 * s2 + 2].ptr;
            }
            NEED_BYTES(6, (size_t)nb * p.cols * 2); NEED_BYTES(7, (size_t)nb * rows * 2); NEED_BYTES(9, (size_t)p.cols * 2);
            a.x = (const __half*)r.buf[6].ptr; a.y = (__half*)r.buf[7].ptr; a.norm_w = (const __half*)r.buf[9].ptr; a.norm_eps = as_f32(eps_bits);
            a.rows = (int)rows; a.cols = p.cols; a.batch = (int)nb; a.err = ctx->err_dev; a.sm_count = ctx->sm_count; a.part_scratch = ctx->qmm_scratch; a.part_scratch_bytes = ctx->qmm_scratch_bytes; a.part_counters = ctx->qmm_counters;
            in.launches += 1;
            cudaError_t e = launch_affine(l, kAffineGateUp, a, p.group);
            if (e == cudaErrorNotSupported) return fail(ctx, SMELT_ERR_UNSUPPORTED, p.name + ": shape not eligible for the fused kernel");
            return check_cuda(ctx, e, p.name.c_str());
        }
        case PK_ROPE_QKV_APPEND: {
            // 0 q (in place), 1 new K, 2 new V, 3 K cache, 4 V cache; constants 7 headDim, 8 q heads,
            // 9 kv heads, 10 capacity, 11 position, 12 layout, 13 log2(theta).
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_BUF(3); NEED_BUF(4);
            NEED_U32(7, d); NEED_U32(8, nq); NEED_U32(9, nkv); NEED_U32(10, cap); NEED_U32(12, layout); NEED_U32(13, base_bits);
            if (!bind_pos_arg(in, r, 11, &l)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "smelt_rope_qkv_append: position constant is missing");
            if (d == 0 || d % 2 || nq == 0 || nkv == 0 || layout > 1) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "smelt_rope_qkv_append: bad shape or layout");
            const int batch = batch_of(rec);
            const size_t seq = (size_t)nkv * cap * d;
            NEED_BYTES(0, (size_t)batch * nq * d * 2); NEED_BYTES(1, (size_t)batch * nkv * d * 2); NEED_BYTES(2, (size_t)batch * nkv * d * 2);
            NEED_BYTES(3, seq * 2 * batch); NEED_BYTES(4, seq * 2 * batch);
            if (!in.device_pos && (l.arg_pos_valid ? l.arg_pos : in.position) >= cap) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "smelt_rope_qkv_append: position beyond the cache capacity");
            in.launches += 1;
            return check_cuda(ctx, launch_rope_qkv_append(l, (__half*)r.buf[0].ptr, (const __half*)r.buf[1].ptr, (const __half*)r.buf[2].ptr, (__half*)r.buf[3].ptr, (__half*)r.buf[4].ptr, cap, (int)d, (int)nq, (int)nkv, (int)layout, as_f32(base_bits), batch, seq), "smelt_rope_qkv_append");
        }
        case PK_TP_ALL_REDUCE: {
            NEED_BUF(0); NEED_U32(1, count);
            NEED_BYTES(0, (size_t)count * 2);
            if (ctx->tp_world <= 1) return SMELT_OK;
            in.launches += 1;
            return tp_all_reduce_f16(ctx, r.buf[0].ptr, count, ctx->stream);
        }
        case PK_TP_ARGMAX: {
            // 0 this rank's partial keys (argmax_fp16_partials over its vocab slice), 1 out token ids;
            // 2 partials per sequence, 3 first vocab row of the slice
            NEED_BUF(0); NEED_BUF(1); NEED_U32(2, parts); NEED_U32(3, offset);
            const int batch = batch_of(rec);
            NEED_BYTES(0, (size_t)batch * parts * 8); NEED_BYTES(1, (size_t)batch * 4);
            in.launches += 1;
            return tp_argmax(ctx, l, r.buf[0].ptr, r.buf[1].ptr, (int)parts, offset, batch);
        }
        case PK_TP_REDUCE_ADD: {
            // 0 this rank's partial (reduced in place on the fallback path), 1 residual, 2 out, 3 count
            NEED_BUF(0); NEED_BUF(1); NEED_BUF(2); NEED_U32(3, count);
            NEED_BYTES(0, (size_t)count * 2); NEED_BYTES(1, (size_t)count * 2); NEED_BYTES(2, (size_t)count * 2);
            if (ctx->tp_world > 1) {
                bool handled = false;
                smelt_status st = tp_reduce_add(ctx, l, r.buf[0].ptr, r.buf[1].ptr, r.buf[2].ptr, count, &handled);
                if (st || handled) { in.launches += 1; return st; }
                st = tp_all_reduce_f16(ctx, r.buf[0].ptr, count, ctx->stream);
                if (st) return st;
                in.launches += 1;
            }
            in.launches += 1;
            return check_cuda(ctx, launch_elementwise_add(l, (const __half*)r.buf[1].ptr, (const __half*)r.buf[0].ptr, (__half*)r.buf[2].ptr, (int64_t)count), "smelt_tp_reduce_add");
        }
        default:
            return fail(ctx, SMELT_ERR_UNKNOWN_PIPELINE, p.name + ": no handler");
    }
}

// full_first: the first record's launches take a full dependency on the work in front of them
// instead of a programmatic one (a token inside a multi-token graph starts only when the token
// before it has completed, as a separate graph launch would).
smelt_status interpret(smelt_cuda_ctx* ctx, const smelt_dispatch_record* table, size_t n, bool device_pos, uint32_t position, bool full_first = false) {
    Interp in;
    in.ctx = ctx; in.device_pos = device_pos; in.position = position;
    in.cur = ctx->cfg.cur_slot; in.alt = ctx->cfg.alt_slot;
    bool first = true;
    for (size_t i = 0; i < n; ++i) {
        const smelt_dispatch_record& rec = table[i];
        if (rec.op_kind == SMELT_OP_SWAP) { int t = in.cur; in.cur = in.alt; in.alt = t; continue; }
        if (rec.op_kind != SMELT_OP_DISPATCH) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "record " + std::to_string(i) + ": unknown op kind");
        const bool pdl = ctx->pdl;
        if (first && full_first) ctx->pdl = false;
        smelt_status s = run_record(in, rec);
        ctx->pdl = pdl;
        first = false;
        if (s) { ctx->err = "record " + std::to_string(i) + ": " + ctx->err; return s; }
    }
    ctx->launch_count = in.launches;
    return SMELT_OK;
}

smelt_status check_step(smelt_cuda_ctx* ctx, const int32_t* tokens, int32_t position) {
    if (!ctx->configured) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "context is not configured");
    // SmeltRuntime.swift:3176-3183: position in [0, contextLimit), token in [0, vocabSize)
    if (position < 0 || (uint32_t)position >= ctx->cfg.context_limit || (uint32_t)position >= ctx->cfg.cache_seq_capacity)
        return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "position out of range [0, " + std::to_string(ctx->cfg.context_limit) + ")");
    if (tokens)
        for (uint32_t b = 0; b < ctx->cfg.batch; ++b)
            if (tokens[b] < 0 || (uint32_t)tokens[b] >= ctx->cfg.vocab_size)
                return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "tokenId out of range [0, " + std::to_string(ctx->cfg.vocab_size) + ")");
    return SMELT_OK;
}

struct TokenPack {
    int32_t t[64];
};

__global__ void set_dynamic_kernel(TokenPack pack, int32_t position, int batch, int32_t* token_slot,
                                   int32_t* position_slot, DynState* dyn) {
    if (threadIdx.x < batch) token_slot[threadIdx.x] = pack.t[threadIdx.x];
    if (threadIdx.x == 0) {
        position_slot[0] = position;
        dyn->token = pack.t[0];
        dyn->position = (uint32_t)position;
    }
}

// Writes token ids and position into their slots (prepareDecodeDynamicState,
// SmeltRuntime.swift:3171-3184) and into the device dynamic state.  The values travel as
// kernel parameters, so no host staging buffer has to outlive the call.
smelt_status write_dynamic(smelt_cuda_ctx* ctx, const int32_t* tokens, int32_t position) {
    const uint32_t B = ctx->cfg.batch;
    Slot& ts = ctx->slots[ctx->cfg.token_id_slot];
    Slot& ps = ctx->slots[ctx->cfg.position_slot];
    if (!ts.ptr || ts.bytes < B * 4 || !ps.ptr || ps.bytes < 4) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "token / position slots are missing or too small");
    TokenPack pack = {};
    for (uint32_t b = 0; b < B; ++b) pack.t[b] = tokens[b];
    prefer_max_shared(set_dynamic_kernel);
    set_dynamic_kernel<<<1, 64, 0, ctx->stream>>>(pack, position, (int)B, (int32_t*)ts.ptr, (int32_t*)ps.ptr, ctx->dyn_dev);
    return check_cuda(ctx, cudaGetLastError(), "write dynamic state");
}

// Tail of a captured token: feed argmax back as the next token, advance the position and
// append the ids to the generated ring.
__global__ void advance_kernel(const int32_t* argmax, int32_t* token_slot, int32_t* position_slot, DynState* dyn,
                               int32_t* ring, uint32_t* count, uint32_t capacity, int batch) {
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x == 0) {
        const uint32_t step = *count;
        for (int b = 0; b < batch; ++b) {
            const int32_t t = argmax[b];
            token_slot[b] = t;
            if (step < capacity) ring[(size_t)step * batch + b] = t;
        }
        dyn->token = argmax[0];
        dyn->position += 1u;
        position_slot[0] = (int32_t)dyn->position;
        *count = step + 1u;
    }
}

}  // namespace
}  // namespace smelt

extern "C" {

int smelt_cuda_pipeline_supported(const char* name) {
    Pipeline p;
    std::string e(name ? name : "");
    if (parse_pipeline(e.c_str(), &p)) return 1;
    // generic affine names need the ":cols:group" suffix to be launchable; accept the bare name too
    if (e.find(':') == std::string::npos && parse_pipeline((e + ":64:64").c_str(), &p)) return 1;
    return 0;
}

smelt_status smelt_cuda_register_pipeline(smelt_cuda_ctx* ctx, int index, const char* name) {
    if (!ctx || !name || index < 0 || index > 65535) return SMELT_ERR_BAD_ARGUMENT;
    Pipeline p;
    if (!parse_pipeline(name, &p))
        return fail(ctx, SMELT_ERR_UNKNOWN_PIPELINE, std::string("pipeline '") + name + "' is not an implemented kernel");
    if ((size_t)index >= ctx->pipelines.size()) ctx->pipelines.resize(index + 1);
    ctx->pipelines[index] = p;
    return SMELT_OK;
}

smelt_status smelt_cuda_enqueue_decode(smelt_cuda_ctx* ctx, const smelt_dispatch_record* table, size_t n_records,
                                       const int32_t* tokens, int32_t position) {
    if (!ctx || !table || !tokens) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    smelt_status s = check_step(ctx, tokens, position);
    if (s) return s;
    s = write_dynamic(ctx, tokens, position);
    if (s) return s;
    return interpret(ctx, table, n_records, false, (uint32_t)position);
}

// A prompt chunk through a prefill table: seq_len token ids into the token slot, then every record with seqLen /
// startPos resolved on the host (resolvePrefillConstant, resolveDispatchBufferOffset, resolvePrefillGrid;
// SmeltRuntime.swift:1217-1250, :6160-6207).  Eager only: a prefill table's shapes change with the chunk.
smelt_status smelt_cuda_enqueue_prefill(smelt_cuda_ctx* ctx, const smelt_dispatch_record* table, size_t n_records, const int32_t* tokens,
                                        int32_t seq_len, int32_t start_pos) {
    if (!ctx || !table || !tokens) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!ctx->configured) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "context is not configured");
    if (ctx->capturing) return fail(ctx, SMELT_ERR_UNSUPPORTED, "prefill tables are interpreted eagerly, not captured");
    const uint64_t limit = ctx->cfg.context_limit < ctx->cfg.cache_seq_capacity ? ctx->cfg.context_limit : ctx->cfg.cache_seq_capacity;
    if (seq_len <= 0 || start_pos < 0 || (uint64_t)start_pos + (uint64_t)seq_len > limit)
        return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "prefill: positions [" + std::to_string(start_pos) + ", " + std::to_string((int64_t)start_pos + seq_len) + ") are outside [0, " + std::to_string(limit) + ")");
    if ((size_t)seq_len > ctx->h_pinned_count - 256) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "prefill: at most " + std::to_string(ctx->h_pinned_count - 256) + " positions per chunk");
    for (int32_t i = 0; i < seq_len; ++i)
        if (tokens[i] < 0 || (uint32_t)tokens[i] >= ctx->cfg.vocab_size) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "tokenId out of range [0, " + std::to_string(ctx->cfg.vocab_size) + ")");
    Slot& ts = ctx->slots[ctx->cfg.token_id_slot];
    if (!ts.ptr || ts.bytes < (size_t)seq_len * 4) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "prefill: the token slot holds fewer than seq_len ids");
    // the staging area may still feed an earlier chunk's copy
    smelt_status s = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "prefill: chunk boundary");
    if (s) return s;
    for (int32_t i = 0; i < seq_len; ++i) ctx->h_pinned[256 + i] = tokens[i];
    s = check_cuda(ctx, cudaMemcpyAsync(ts.ptr, ctx->h_pinned + 256, (size_t)seq_len * 4, cudaMemcpyHostToDevice, ctx->stream), "prefill: token ids");
    if (s) return s;
    Interp in;
    in.ctx = ctx; in.device_pos = false; in.position = (uint32_t)start_pos;
    in.prefill = true; in.seq_len = (uint32_t)seq_len; in.start_pos = (uint32_t)start_pos;
    in.cur = ctx->cfg.cur_slot; in.alt = ctx->cfg.alt_slot;
    for (size_t i = 0; i < n_records; ++i) {
        const smelt_dispatch_record& rec = table[i];
        if (rec.op_kind == SMELT_OP_SWAP) { int t = in.cur; in.cur = in.alt; in.alt = t; continue; }
        if (rec.op_kind != SMELT_OP_DISPATCH) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "record " + std::to_string(i) + ": unknown op kind");
        s = run_record(in, rec);
        if (s) { ctx->err = "record " + std::to_string(i) + ": " + ctx->err; return s; }
    }
    ctx->launch_count = in.launches;
    return SMELT_OK;
}

smelt_status smelt_cuda_decode_step(smelt_cuda_ctx* ctx, const smelt_dispatch_record* table, size_t n_records,
                                    const int32_t* tokens, int32_t position, int32_t* out_tokens) {
    smelt_status s = smelt_cuda_enqueue_decode(ctx, table, n_records, tokens, position);
    if (s) return s;
    const uint32_t B = ctx->cfg.batch;
    Slot& as = ctx->slots[ctx->cfg.argmax_slot];
    if (!as.ptr || as.bytes < B * 4) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "argmax slot is missing or too small");
    cudaMemcpyAsync(ctx->h_pinned + 128, as.ptr, B * 4, cudaMemcpyDeviceToHost, ctx->stream);
    s = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "decode step");
    if (s) return s;
    if (out_tokens)
        for (uint32_t b = 0; b < B; ++b) out_tokens[b] = ctx->h_pinned[128 + b];
    return SMELT_OK;
}

// Captures n_tokens decode steps (the table, then the advance kernel, per token) into one graph.
static smelt_status capture_tokens(smelt_cuda_ctx* ctx, const smelt_dispatch_record* table, size_t n_records, int n_tokens,
                                   cudaGraph_t* graph, cudaGraphExec_t* exec) {
    const uint32_t B = ctx->cfg.batch;
    Slot& as = ctx->slots[ctx->cfg.argmax_slot];
    Slot& ts = ctx->slots[ctx->cfg.token_id_slot];
    Slot& ps = ctx->slots[ctx->cfg.position_slot];
    smelt_status s = check_cuda(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
    if (s) return s;
    ctx->capturing = true;
    size_t launches = 0;
    for (int t = 0; t < n_tokens && !s; ++t) {
        s = interpret(ctx, table, n_records, true, 0, t > 0);
        if (s) break;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1); cfg.blockDim = dim3(32); cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = ctx->pdl ? 1 : 0;
        prefer_max_shared(advance_kernel);
        s = check_cuda(ctx, cudaLaunchKernelEx(&cfg, advance_kernel, (const int32_t*)as.ptr, (int32_t*)ts.ptr, (int32_t*)ps.ptr, ctx->dyn_dev, ctx->gen_ring, ctx->gen_count, ctx->gen_capacity, (int)B), "advance kernel");
        ctx->launch_count += 1;
        launches = ctx->launch_count;
    }
    ctx->launch_count = launches;  // launches of one token
    ctx->capturing = false;
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
    if (s) { if (g) cudaGraphDestroy(g); return s; }
    s = check_cuda(ctx, e, "cudaStreamEndCapture");
    if (s) return s;
    *graph = g;
    s = check_cuda(ctx, cudaGraphInstantiate(exec, g, 0), "cudaGraphInstantiate");
    if (s) return s;
    // Upload now: otherwise the first launch of the graph pays for it (about a millisecond for
    // the eight-token graph's two thousand nodes), inside whatever the caller is timing.
    return check_cuda(ctx, cudaGraphUpload(*exec, ctx->stream), "cudaGraphUpload");
}

smelt_status smelt_cuda_graph_build(smelt_cuda_ctx* ctx, const smelt_dispatch_record* table, size_t n_records) {
    if (!ctx || !table) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!ctx->configured) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "context is not configured");
    destroy_decode_graphs(ctx);
    if (!ctx->gen_ring) {
        ctx->gen_capacity = 65536;
        if (cudaMalloc(&ctx->gen_ring, (size_t)ctx->gen_capacity * 64 * 4) != cudaSuccess || cudaMalloc(&ctx->gen_count, 4) != cudaSuccess)
            return fail(ctx, SMELT_ERR_ALLOC, "graph: generated-token ring");
        cudaMemset(ctx->gen_count, 0, 4);
    }
    Slot& as = ctx->slots[ctx->cfg.argmax_slot];
    Slot& ts = ctx->slots[ctx->cfg.token_id_slot];
    Slot& ps = ctx->slots[ctx->cfg.position_slot];
    if (!as.ptr || !ts.ptr || !ps.ptr) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "graph: argmax / token / position slots are not allocated");
    smelt_status s = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "graph: pre-capture sync");
    if (s) return s;
    ctx->graph_pos_known = false;
    // One graph of a single token, and one of kGraphBurst tokens that smelt_cuda_graph_decode uses
    // for runs of that many steps: fewer graph launches, each of which costs the GPU a gap.
    s = capture_tokens(ctx, table, n_records, 1, &ctx->graph, &ctx->graph_exec);
    if (s) return s;
    s = capture_tokens(ctx, table, n_records, kGraphBurst, &ctx->graph_burst, &ctx->graph_burst_exec);
    if (s) destroy_decode_graphs(ctx);
    return s;
}

smelt_status smelt_cuda_graph_seed(smelt_cuda_ctx* ctx, const int32_t* tokens, int32_t position) {
    if (!ctx || !tokens) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    smelt_status s = check_step(ctx, tokens, position);
    if (s) return s;
    s = write_dynamic(ctx, tokens, position);
    if (s) return s;
    if (ctx->gen_count) cudaMemsetAsync(ctx->gen_count, 0, 4, ctx->stream);
    ctx->graph_next_pos = (uint32_t)position;
    ctx->graph_pos_known = true;
    return check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "graph seed");
}

smelt_status smelt_cuda_graph_decode(smelt_cuda_ctx* ctx, int n_steps, int32_t* out_tokens) {
    if (!ctx || n_steps <= 0) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!ctx->graph_exec) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "no graph has been built");
    const uint32_t B = ctx->cfg.batch;
    // The position advances on the device; the host mirrors it so that a run past the context
    // limit or the cache capacity is refused (SmeltRuntime.swift:3176-3183) instead of clamped.
    if (!ctx->graph_pos_known) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "graph decode: seed the graph first (smelt_cuda_graph_seed)");
    const uint32_t limit = ctx->cfg.context_limit < ctx->cfg.cache_seq_capacity ? ctx->cfg.context_limit : ctx->cfg.cache_seq_capacity;
    if ((uint64_t)ctx->graph_next_pos + (uint64_t)n_steps > (uint64_t)limit)
        return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "graph decode: " + std::to_string(n_steps) + " steps from position " + std::to_string(ctx->graph_next_pos) + " pass the limit of " + std::to_string(limit) + " positions");
    ctx->graph_next_pos += (uint32_t)n_steps;
    if (out_tokens) cudaMemsetAsync(ctx->gen_count, 0, 4, ctx->stream);
    if (out_tokens && (uint32_t)n_steps > ctx->gen_capacity) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "graph decode: too many steps for one readback");
    for (int i = 0; i < n_steps;) {
        const bool burst = ctx->graph_burst_exec && n_steps - i >= kGraphBurst;
        smelt_status s = check_cuda(ctx, cudaGraphLaunch(burst ? ctx->graph_burst_exec : ctx->graph_exec, ctx->stream), "cudaGraphLaunch");
        if (s) return s;
        i += burst ? kGraphBurst : 1;
    }
    if (!out_tokens) return SMELT_OK;
    smelt_status s = check_cuda(ctx, cudaMemcpyAsync(out_tokens, ctx->gen_ring, (size_t)n_steps * B * 4, cudaMemcpyDeviceToHost, ctx->stream), "graph readback");
    if (s) return s;
    return check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "graph decode");
}

smelt_status smelt_cuda_graph_generated(smelt_cuda_ctx* ctx, int n_steps, int32_t* out_tokens) {
    if (!ctx || n_steps <= 0 || !out_tokens) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!ctx->gen_ring) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "no graph has been built");
    uint32_t count = 0;
    smelt_status s = check_cuda(ctx, cudaMemcpyAsync(&count, ctx->gen_count, 4, cudaMemcpyDeviceToHost, ctx->stream), "graph generated: count");
    if (!s) s = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "graph generated: sync");
    if (s) return s;
    if (count > ctx->gen_capacity) count = ctx->gen_capacity;
    if ((uint32_t)n_steps > count) return fail(ctx, SMELT_ERR_OUT_OF_RANGE, "graph generated: only " + std::to_string(count) + " steps were replayed since the last seed");
    const uint32_t B = ctx->cfg.batch;
    s = check_cuda(ctx, cudaMemcpyAsync(out_tokens, ctx->gen_ring + (size_t)(count - (uint32_t)n_steps) * B, (size_t)n_steps * B * 4, cudaMemcpyDeviceToHost, ctx->stream), "graph generated: readback");
    return s ? s : check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "graph generated: sync");
}

smelt_status smelt_cuda_graph_step(smelt_cuda_ctx* ctx, const int32_t* tokens, int32_t position, int32_t* out_tokens) {
    if (!ctx || !tokens) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    if (!ctx->graph_exec) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "no graph has been built");
    smelt_status s = check_step(ctx, tokens, position);
    if (s) return s;
    s = write_dynamic(ctx, tokens, position);
    if (s) return s;
    s = check_cuda(ctx, cudaGraphLaunch(ctx->graph_exec, ctx->stream), "cudaGraphLaunch");
    if (s) return s;
    ctx->graph_next_pos = (uint32_t)position + 1u;
    ctx->graph_pos_known = true;
    const uint32_t B = ctx->cfg.batch;
    Slot& as = ctx->slots[ctx->cfg.argmax_slot];
    cudaMemcpyAsync(ctx->h_pinned + 128, as.ptr, B * 4, cudaMemcpyDeviceToHost, ctx->stream);
    s = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "graph step");
    if (s) return s;
    if (out_tokens)
        for (uint32_t b = 0; b < B; ++b) out_tokens[b] = ctx->h_pinned[128 + b];
    return SMELT_OK;
}

int smelt_cuda_last_launch_count(const smelt_cuda_ctx* ctx) { return ctx ? ctx->launch_count : 0; }

}  // extern "C"
