// Launchers of the glue, attention and low-bit kernels (glue.cu, attention.cu, signed_matvec.cu).
#pragma once
#include "common.cuh"

namespace smelt {

cudaError_t launch_rms_norm_1pw(const Launch& l, const __half* x, const __half* w, __half* y, int dim, float eps, int batch);
cudaError_t launch_per_head_rms_norm(const Launch& l, const __half* x, const __half* w, __half* y, int heads, int head_dim, float eps);
cudaError_t launch_elementwise_add(const Launch& l, const __half* a, const __half* b, __half* y, int64_t n);
cudaError_t launch_swiglu_fused(const Launch& l, const __half* gate, const __half* up, __half* y, int64_t n);
cudaError_t launch_embedding_gather(const Launch& l, const __half* table, const int32_t* token, __half* y, int hidden, int batch, int token_stride);
cudaError_t launch_affine_embedding_gather(const Launch& l, const uint8_t* w, const __half* s, const __half* b, const int32_t* token, __half* y, int cols, int group, int batch = 1);
cudaError_t launch_affine_dequant(const Launch& l, const uint8_t* w, const __half* s, const __half* b, float* out32, __half* out16, int rows, int cols, int group);
cudaError_t launch_signed_dequant(const Launch& l, const uint8_t* codes, const __half* s, float* out, int rows, int cols, int bits, int group, int* bad);
cudaError_t launch_apply_rope(const Launch& l, __half* qk, const __half* cos_t, const __half* sin_t, int head_dim, int rope_dim, int heads, int layout, float base_log2, int math_mode, size_t table_stride, int batch);
cudaError_t launch_kv_cache_update(const Launch& l, __half* cache, const __half* new_kv, const __half* cos_t, const __half* sin_t, uint32_t capacity, int head_dim, int heads, int rope_dim, int layout, float base_log2, int math_mode, int do_rope, size_t table_stride, int batch, size_t seq_stride);
cudaError_t launch_rope_qkv_append(const Launch& l, __half* q, const __half* k_new, const __half* v_new, __half* k_cache, __half* v_cache, uint32_t capacity, int head_dim, int n_q, int n_kv, int layout, float base_log2, int batch, size_t seq_stride);
cudaError_t launch_argmax_partials(const Launch& l, const __half* logits, uint64_t* partials, int vocab, int chunk, int batch);
cudaError_t launch_argmax_reduce(const Launch& l, const uint64_t* partials, int32_t* out, int n, int batch, int out_stride);
// Signed activation bit-planes (bitplane.cu)
struct BitplaneArgs {
    int format;              // 1 binary, 2 ternary
    int mode;                // 0 plain, 1 + residual, 2 gate/up + SwiGLU
    const uint8_t* codes;    // [rows, cols/8] or [rows, cols/4]
    const __half* wscales;   // [rows, cols/128]
    const uint8_t* codes2;   // mode 2: the up matrix
    const __half* wscales2;
    const uint32_t* planes;  // [batch, cols/128, n_planes, 4]
    const __half* ascales;   // [batch, cols/128]
    const __half* residual;  // mode 1: [batch, rows]
    __half* out;             // [batch, rows]
    int rows, cols, n_planes, batch;
};
cudaError_t launch_bitplane_producer(const Launch& l, const __half* x, const __half* up, uint32_t* planes, __half* scales, int cols, int n_planes, int batch);
// front 2: a * sigmoid(b) (i6); 3: rms_norm_1pw value from norm_scale[0], a = x, c = norm weight (i2..i6); 4: gated norm of heads of 128, a = x, b = gate, c = weight (i6)
cudaError_t launch_bitplane_fused_producer(const Launch& l, int front, const __half* a, const __half* b, const __half* c, const float* norm_scale, uint32_t* planes, __half* scales, int cols, int n_planes, float eps, int tgs);
enum { kEwSilu = 0, kEwSigmoid, kEwSoftplus, kEwCopy, kEwScalarMul, kEwLogitCap, kEwMul, kEwSigmoidMul, kEwGeglu, kEwBiasAdd };
enum { kHeadNormDirect = 0, kHeadNorm1pw = 1, kHeadNormNoScale = 2 };
cudaError_t launch_elementwise(const Launch& l, int op, const __half* a, const __half* b, __half* y, int count, int batch, int b_stride, float scalar, const __half* scalar_dev);
cudaError_t launch_row_norm(const Launch& l, const __half* x, const __half* pre, const __half* w, const __half* residual, const __half* scalar, __half* y, float* scale_out, int rows, int dim, float eps, int topology, int tgs, int value, int scale, int group_rows = 0, int group_stride = 0);
// prompt-chunk RoPE + KV write and causal attention (prefill.cu)
cudaError_t launch_rope_kv_prefill(const Launch& l, __half* q, __half* k, const __half* v, const __half* cos_t, const __half* sin_t, __half* k_cache, __half* v_cache, int head_dim, int rope_dim, int q_heads, int kv_heads, uint32_t n_pos, uint32_t start_pos, uint32_t capacity, int layout, float base_log2, int math_mode, size_t table_stride);
cudaError_t launch_attention_prefill(const Launch& l, const __half* q, const __half* k_cache, const __half* v_cache, __half* out, int n_q, int n_kv, int head_dim, uint32_t n_pos, uint32_t start_pos, uint32_t capacity, float scale, uint32_t window);
cudaError_t launch_gate_split(const Launch& l, const __half* in, __half* query, __half* gate, int heads, int head_dim);
cudaError_t launch_head_norm(const Launch& l, int mode, const __half* x, const __half* w, __half* y, int heads, int head_dim, float eps, int tgs);
cudaError_t launch_signed_embedding_gather(const Launch& l, int format, const uint8_t* codes, const __half* scales, const int32_t* token_ids, __half* out, int hidden, int batch);
cudaError_t launch_bitplane_matvec(const Launch& l, const BitplaneArgs& a);
// DeltaNet decode step (deltanet.cu)
cudaError_t launch_conv1d_update_silu(const Launch& l, __half* state, const __half* new_val, const __half* weight, __half* out, int channels, int kernel_size);
cudaError_t launch_rms_scale_qk(const Launch& l, __half* qkv, int head_dim, float eps, int qkv_dim, int qk_heads, int batch);
cudaError_t launch_conv1d_update_silu_prefill(const Launch& l, __half* state, __half* qkv, const __half* weight, int seq_len, int channels, int kernel_size, __half* history);
cudaError_t launch_deltanet_recurrence_prefill(const Launch& l, __half* state, const __half* qkv, const __half* b_proj, const __half* a_proj, const __half* a_log, const __half* dt_bias, __half* out, int head_dim, int value_heads, int qk_heads, int seq_len, __half* history);
cudaError_t launch_deltanet_recurrence_decode(const Launch& l, __half* state, const __half* qkv, const __half* b_proj, const __half* a_proj, const __half* a_log, const __half* dt_bias, __half* out, int head_dim, int value_heads, int qk_heads);
cudaError_t launch_rms_norm_gated(const Launch& l, const __half* input, const __half* gate, const __half* weight, __half* out, int head_dim, float eps, int heads, int tgs, bool precise_d128);
// The DeltaNet step as separate launches and its two one-CTA-per-head fused forms (recurrence_steps.cu).
// launch_dn_state_update: state_decay (key null), outer_product_update (g_val null), state_decay_update (both).
// launch_dn_readout mode: 0 kv_mem_readout, 1 kv_readout_delta, 2 gates_kv_readout_delta, 3 query_readout.
cudaError_t launch_dn_compute_gates(const Launch& l, const __half* b_proj, const __half* a_proj, const __half* a_log, const __half* dt_bias, __half* beta_out, __half* g_out, int heads);
cudaError_t launch_dn_state_update(const Launch& l, __half* state, const __half* g_val, const __half* key, const float* delta, int head_dim, int heads);
cudaError_t launch_dn_readout(const Launch& l, int mode, const __half* state, const __half* vec, const __half* value, const __half* g_val, const __half* beta, const __half* b_proj, const __half* a_proj, const __half* a_log, const __half* dt_bias, float* out_f32, __half* out_f16, __half* g_out, int head_dim, float scale, int heads);
cudaError_t launch_dn_compute_delta(const Launch& l, const __half* value, const float* kv_mem, const __half* beta, float* delta, int head_dim, int heads);
cudaError_t launch_dn_fused_decode(const Launch& l, __half* state, const __half* qkv, const __half* b_proj, const __half* a_proj, const __half* a_log, const __half* dt_bias, __half* out, __half* conv_state, const __half* conv_weight, const __half* z_proj, const __half* norm_weight, int head_dim, float head_scale, int qkv_dim, int conv_k, int heads, float rms_eps, int tgs);
cudaError_t launch_dn_fused_prefill(const Launch& l, __half* state, __half* conv_state, __half* qkv, const __half* conv_weight, const __half* a_log, const __half* dt_bias, const __half* b_buf, const __half* a_buf, __half* out, int head_dim, int heads, int seq_len, int qkv_dim, int conv_k, float head_scale, float l2_eps, int tgs);
cudaError_t launch_fp16_matvec(const Launch& l, const __half* w, const __half* x, __half* y, int rows, int cols, int batch, int sm_count);

// attention.cu — split-K flash-decode.  scratch holds fp32 partials; see attention_scratch_bytes.
struct AttnArgs {
    const __half* q;        // [batch, n_q, head_dim]
    const __half* k_cache;  // [batch][n_kv, capacity, head_dim]
    const __half* v_cache;
    __half* out;            // [batch, n_q, head_dim]; may alias q
    int n_q, n_kv, head_dim, batch;
    uint32_t capacity;
    uint32_t seq_len;       // used when seq_from_pos == 0
    int seq_from_pos;       // 1: seq_len = position + 1 (read through the dynamic state)
    float scale;
    uint32_t sliding_window;
    size_t seq_stride;      // elements between consecutive sequences' caches
    void* scratch;
    size_t scratch_bytes;
    int sm_count;
    // Optional.  counters != null: one zeroed int per (sequence, KV head); the last split of a
    // head to finish merges the partials itself (no merge launch) and leaves its counter at zero.
    int* counters;
    // k_new != null: RoPE on q, RoPE + append of the new K row and append of the new V row
    // (apply_rope + rope_kv_cache_update + kv_cache_update, full-head analytic mode) happen
    // inside the kernel; the new token sits at key index seq_len - 1.
    const __half* k_new;    // [batch, n_kv, head_dim]
    const __half* v_new;
    int rope_layout;        // 0 adjacent pairs, 1 split-half
    float rope_base_log2;
    const float* rope_table;  // optional: cos[half] | sin[half] of the position (launch_rope_table)
    // 1 (with k_new): every cache row below seq_len - 1 was written before the launch sequence of
    // this token began (tokens never overlap: a token's graph launch, or its eager step, starts
    // after the previous one has completed), so the kernel requests those rows before it waits
    // for the launch in front of it.
    int kv_rows_stable;
    // mlx_partials != null (batch 1): the launch is the first half of the reference's two-pass
    // pair; every split writes its state as one of the 128 key blocks of the reference's
    // buffers (fp16 partials [n_q, 128, head_dim], fp32 stats [2][n_q][128]) and nothing merges.
    __half* mlx_partials;
    float* mlx_stats;
};
// What one attention launch works from.
struct AttnDev {
    AttnArgs a;
    int nsplits;
    int cluster;     // 1: the splits of a KV head are one thread-block cluster and merge through distributed shared memory
    float* part_o;   // [batch*n_q, nsplits, head_dim]
    float* part_ml;  // [batch*n_q, nsplits, 2]
    DevDyn dyn;
};
size_t attention_scratch_bytes(int n_q, int head_dim, int batch, int max_splits);
int attention_max_splits();
cudaError_t launch_attention_decode(const Launch& l, const AttnArgs& a);
cudaError_t launch_rope_table(const Launch& l, float* table, int half, float base_log2);
// Second half of the two-pass pair: out[n_q, head_dim] from the 128 blocks of partials / stats.
cudaError_t launch_attention_mlx_reduce(const Launch& l, const __half* partials, const float* stats, __half* out, int n_q, int head_dim);

// signed_matvec.cu — binary1 / ternary2, group 128.
enum SignedMode : int { kSignedPlain = 0, kSignedAdd = 1, kSignedGateUp = 2 };
struct SignedArgs {
    const uint8_t* codes[2];
    const __half* scales[2];
    const __half* x;
    __half* y;
    const __half* residual;
    int rows, cols, batch, bits;
};
cudaError_t launch_signed(const Launch& l, int mode, const SignedArgs& a);
cudaError_t launch_signed_imma(const Launch& l, int mode, const SignedArgs& a, int sm_count, bool* handled);

}  // namespace smelt
