// Decoder table builder: writes the per-token SmeltDispatchRecord sequence the reference
// compiler emits for a plain attention decoder (Sources/SmeltCompiler/TopLevelEmitter.swift
// :89-930 generatePlanned; Sources/SmeltCompiler/AttentionPlugin.swift:105-560 emitLayer;
// record encoding Sources/SmeltCompiler/SmeltCodeEmitter.swift:348 toRecord), allocates the
// slots it binds (numbers follow SmeltFixedSlot, Sources/SmeltCompiler/SmeltBufferPlan.swift
// :129-198) and registers the pipeline names.  It stands in for the build-time Swift
// compiler, which is outside the decode path.
#include <cmath>
#include <cstring>
#include <map>
#include <vector>

#include "runtime.h"

using namespace smelt;

namespace {

enum FixedSlot : int {
    kHiddenA = 0, kHiddenB = 1, kNormOut = 8, kFfnInt = 13, kFfnDown = 14, kLogits = 16, kArgmax = 17,
    kAttnQ = 20, kAttnK = 21, kAttnV = 22, kAttnOut = 23, kWeights = 30,
    kTokenId = 33, kPosition = 34, kArgmaxScratch = 35, kKvBase = 40,
};

uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

struct Emitter {
    smelt_cuda_ctx* ctx;
    smelt_dispatch_record* out;
    size_t cap, n = 0;
    std::map<std::string, int> pipes;
    smelt_status status = SMELT_OK;
    int base = 0;  // first pipeline index this table may register (a prefill table comes after the decode table's)

    int pipe(const std::string& name) {
        auto it = pipes.find(name);
        if (it != pipes.end()) return it->second;
        const int idx = base + (int)pipes.size();
        if (ctx) {
            smelt_status s = smelt_cuda_register_pipeline(ctx, idx, name.c_str());
            if (s && !status) status = s;
        }
        pipes[name] = idx;
        return idx;
    }
    smelt_dispatch_record* next() {
        static smelt_dispatch_record scratch;
        smelt_dispatch_record* r = (out && n < cap) ? &out[n] : &scratch;
        memset(r, 0, sizeof(*r));
        ++n;
        return r;
    }
    void swap() { next()->op_kind = SMELT_OP_SWAP; }
};

struct Rec {
    smelt_dispatch_record* r;
    Rec(Emitter& e, const std::string& name, uint32_t gx = 1, uint32_t gy = 1) : r(e.next()) {
        r->op_kind = SMELT_OP_DISPATCH;
        r->pipeline = (uint16_t)e.pipe(name);
        r->grid[0] = gx; r->grid[1] = gy; r->grid[2] = 1;
        r->threadgroup[0] = 64; r->threadgroup[1] = 1; r->threadgroup[2] = 1;
    }
    Rec& buf(int binding, int slot, uint64_t offset = 0) {
        smelt_buffer_record& b = r->buf[r->buffer_count++];
        b.slot = (int16_t)slot; b.binding_index = (uint8_t)binding; b.offset_kind = 0; b.offset = offset;
        return *this;
    }
    Rec& con(int binding, uint8_t kind, uint32_t value = 0) {
        smelt_constant_record& c = r->con[r->constant_count++];
        c.kind = kind; c.binding_index = (uint8_t)binding; c.value = value;
        return *this;
    }
    Rec& u32(int binding, uint32_t v) { return con(binding, SMELT_CONST_LITERAL_U32, v); }
    // grid dimension `dim` follows the chunk length: kind 1 seqLen, 2 seqLen * literal, 3 ceil(seqLen / literal) (SmeltDispatchTable.swift:163-222)
    Rec& grid_kind(int dim, uint8_t kind) { r->style = (uint8_t)(r->style | (kind << (2 + 2 * dim))); return *this; }
    Rec& buf_kind(int binding, int slot, uint8_t kind, uint64_t offset) {
        buf(binding, slot, offset);
        r->buf[r->buffer_count - 1].offset_kind = kind;
        return *this;
    }
    Rec& tg(uint32_t w) { r->threadgroup[0] = w; return *this; }
    Rec& f32(int binding, float v) { return con(binding, SMELT_CONST_LITERAL_F32, f32_bits(v)); }
    Rec& affine(int first, const smelt_affine_ref& w) {
        return buf(first, kWeights, w.packed).buf(first + 1, kWeights, w.scales).buf(first + 2, kWeights, w.biases);
    }
};

std::string shaped(const char* base, int cols, int rows, int group, bool batched) {
    return std::string(base) + "_c" + std::to_string(cols) + "_r" + std::to_string(rows) + "_g" + std::to_string(group) + (batched ? "_batched" : "");
}

}  // namespace

struct Hybrid {
    const smelt_delta_desc* dd;
    const smelt_delta_ref* refs;
    const uint8_t* kinds;
};
enum DeltaSlot : int { kDeltaQkv = 24, kDeltaZ = 25, kDeltaA = 26, kDeltaB = 27, kDeltaOut = 28 };

static smelt_status build_decoder_impl(smelt_cuda_ctx* ctx, const smelt_decoder_desc* d, const smelt_layer_ref* layers,
                                       uint32_t capacity, uint32_t batch, smelt_dispatch_record* records,
                                       size_t* n_records, std::vector<std::string>* names, const Hybrid* hy = nullptr) {
    if (!d || !layers || !n_records) return SMELT_ERR_BAD_ARGUMENT;
    if (hy) {
        const smelt_delta_desc* dd = hy->dd;
        if (!dd || !hy->refs || !hy->kinds || dd->value_heads <= 0 || dd->qk_heads <= 0 || dd->value_heads % dd->qk_heads || dd->head_dim <= 0 || dd->head_dim % 32 ||
            dd->head_dim > 256 || dd->conv_kernel <= 0 || dd->conv_kernel > 8 || batch != 1 || d->tp_world > 1)
            return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "build_hybrid_decoder: bad linear-attention geometry (one GPU, batch 1)");
    }
    if (d->layers <= 0 || d->hidden <= 0 || d->inter <= 0 || d->n_q <= 0 || d->n_kv <= 0 || d->n_q % d->n_kv || d->head_dim <= 0 ||
        d->vocab <= 0 || batch == 0 || batch > 64 || capacity == 0 || d->layers > 100)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "build_decoder: bad model description");
    // With a null context nothing is allocated or registered: the call only writes (or counts)
    // the records, which lets host-side tooling and CPU tests inspect the table.
    const bool dry = ctx == nullptr;
    const int H = d->hidden, I = d->inter, D = d->head_dim, G = d->group, B = (int)batch;
    const int qd = d->n_q * D, kvd = d->n_kv * D, L = d->layers, V = d->vocab;
    const bool tp = d->tp_world > 1;
    const bool fuse = (d->fuse_residual & 1) && !tp;
    // bit 1: fold the norms into the projections (one QKV launch, one gate/up launch) and RoPE /
    // KV append into one launch; needs the shapes the streaming matvec kernel accepts.
    const bool fuse_tp = (d->fuse_residual & 4) != 0;  // bit 2: all-reduce and residual add in one launch over peer memory
    const bool fuse2 = (d->fuse_residual & 2) && G == 64 && H % 1024 == 0 && qd % 16 == 0 && kvd % 16 == 0 && B <= 8 && D % 2 == 0;
    const bool bt = B > 1;  // batched kernel names bind actualBatch instead of numRows

    if (!dry) {
        if (!records) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "build_decoder: a context needs a record buffer (query the count with a null context)");
        if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
        if (kKvBase + 2 * L > (int)ctx->slots.size()) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "build_decoder: too many layers for the slot table");
        if (!ctx->slots[kWeights].ptr) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "build_decoder: upload the weights image to slot 30 first");
        const int chunk = 2048, parts = (V + chunk - 1) / chunk;
        struct { int slot; size_t bytes; } plan[] = {
            {kHiddenA, (size_t)B * H * 2}, {kHiddenB, (size_t)B * H * 2}, {kNormOut, (size_t)B * H * 2},
            {kFfnInt, (size_t)B * I * 2}, {kFfnDown, (size_t)B * H * 2}, {kLogits, (size_t)B * V * 2},
            {kArgmax, (size_t)B * 4 < 8 ? 8 : (size_t)B * 4}, {kAttnQ, (size_t)B * qd * 2}, {kAttnK, (size_t)B * kvd * 2},
            {kAttnV, (size_t)B * kvd * 2}, {kAttnOut, (size_t)B * qd * 2}, {kTokenId, (size_t)B * 4},
            {kPosition, 8}, {kArgmaxScratch, (size_t)parts * B * 8},
        };
        for (auto& p : plan) {
            smelt_status s = smelt_cuda_alloc_slot(ctx, p.slot, p.bytes);
            if (s) return s;
        }
        const size_t kv_bytes = (size_t)B * d->n_kv * capacity * D * 2;  // heads * capacity * headDim * 2 per sequence
        for (int l = 0; l < 2 * L; ++l) {
            if (hy && hy->kinds[l % L]) continue;  // a DeltaNet layer keeps no KV cache
            smelt_status s = smelt_cuda_alloc_slot(ctx, kKvBase + l, kv_bytes);
            if (s) return s;
        }
        if (hy) {
            const smelt_delta_desc* dd = hy->dd;
            const size_t dq = (size_t)(2 * dd->qk_heads + dd->value_heads) * dd->head_dim, dv = (size_t)dd->value_heads * dd->head_dim;
            if (kKvBase + 4 * L > (int)ctx->slots.size()) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "build_hybrid_decoder: too many layers for the slot table");
            struct { int slot; size_t bytes; } dplan[] = {{kDeltaQkv, dq * 2}, {kDeltaZ, dv * 2}, {kDeltaA, (size_t)dd->value_heads * 2 < 16 ? 16 : (size_t)dd->value_heads * 2},
                                                          {kDeltaB, (size_t)dd->value_heads * 2 < 16 ? 16 : (size_t)dd->value_heads * 2}, {kDeltaOut, dv * 2}};
            for (auto& p : dplan) {
                smelt_status s = smelt_cuda_alloc_slot(ctx, p.slot, p.bytes);
                if (s) return s;
            }
            for (int l = 0; l < L; ++l)
                if (hy->kinds[l]) {
                    smelt_status s = smelt_cuda_alloc_slot(ctx, kKvBase + 2 * L + l, dq * dd->conv_kernel * 2);
                    if (!s) s = smelt_cuda_alloc_slot(ctx, kKvBase + 3 * L + l, (size_t)dd->value_heads * dd->head_dim * dd->head_dim * 2);
                    if (s) return s;
                }
        }
        smelt_cuda_runtime_config cfg = {};
        cfg.token_id_slot = kTokenId; cfg.position_slot = kPosition; cfg.weights_slot = kWeights; cfg.argmax_slot = kArgmax;
        cfg.cur_slot = kHiddenA; cfg.alt_slot = kHiddenB; cfg.cache_seq_capacity = capacity; cfg.context_limit = capacity;
        cfg.vocab_size = (uint32_t)V; cfg.batch = batch;
        smelt_status s = smelt_cuda_configure(ctx, &cfg);
        if (s) return s;
        ctx->pipelines.clear();
    }

    Emitter e{ctx, records, records ? *n_records : 0};
    const float log2_theta = log2f(d->rope_theta);
    const float scale = 1.0f / sqrtf((float)D);
    auto matvec_name = [&](int cols, int rows) {
        return bt ? shaped("affine_matvec", cols, rows, G, true) : "affine_matvec:" + std::to_string(cols) + ":" + std::to_string(G);
    };
    auto count_const = [&](Rec& r, int binding, int rows) { r.u32(binding, bt ? (uint32_t)B : (uint32_t)rows); };

    // embedding gather -> hiddenA (TopLevelEmitter.swift:164-228)
    Rec(e, "embedding_gather", (H + 63) / 64, B).buf(0, kWeights, d->embedding).buf(1, kTokenId).buf(2, SMELT_SLOT_CUR).u32(3, H);

    for (int l = 0; l < L; ++l) {
        const smelt_layer_ref& w = layers[l];
        const int kslot = kKvBase + l, vslot = kKvBase + L + l;
        const bool is_delta = hy && hy->kinds[l];
        if (is_delta) {
            // DeltaNetPlugin.swift:60-420: projections of the normed hidden state, convolution, Q / K scaling, recurrence, gated norm
            const smelt_delta_desc* dd = hy->dd;
            const smelt_delta_ref& x = hy->refs[l];
            const int DD = dd->head_dim, Hv = dd->value_heads, Hqk = dd->qk_heads;
            const int dq = (2 * Hqk + Hv) * DD, dv = Hv * DD;
            const int conv_slot = kKvBase + 2 * L + l, rec_slot = kKvBase + 3 * L + l;
            Rec(e, "rms_norm_1pw", 1).buf(0, SMELT_SLOT_CUR).buf(1, kWeights, w.input_norm).buf(2, kNormOut).u32(3, H).f32(4, d->eps);
            { Rec r(e, matvec_name(H, dq), (dq + 7) / 8); r.affine(0, x.qkv).buf(3, kNormOut).buf(4, kDeltaQkv); count_const(r, 5, dq); }
            { Rec r(e, matvec_name(H, dv), (dv + 7) / 8); r.affine(0, x.z).buf(3, kNormOut).buf(4, kDeltaZ); count_const(r, 5, dv); }
            { Rec r(e, matvec_name(H, Hv), (Hv + 7) / 8); r.affine(0, x.a).buf(3, kNormOut).buf(4, kDeltaA); count_const(r, 5, Hv); }
            { Rec r(e, matvec_name(H, Hv), (Hv + 7) / 8); r.affine(0, x.b).buf(3, kNormOut).buf(4, kDeltaB); count_const(r, 5, Hv); }
            Rec(e, "conv1d_update_silu", (dq + 255) / 256).tg(256).buf(0, conv_slot).buf(1, kDeltaQkv).buf(2, kWeights, x.conv_weight).buf(3, kDeltaQkv)
                .u32(4, dq).u32(5, dd->conv_kernel);
            Rec(e, "rms_scale_qk", 2 * Hqk).tg(32u * (uint32_t)((DD + 127) / 128)).buf(0, kDeltaQkv).u32(1, DD).f32(2, 1e-6f).u32(3, dq).u32(4, Hqk);
            Rec(e, "deltanet_recurrence_mlx_decode", 32, DD).tg(32).buf(0, rec_slot).buf(1, kDeltaQkv).buf(2, kDeltaB).buf(3, kDeltaA).buf(4, kWeights, x.a_log)
                .buf(5, kWeights, x.dt_bias).buf(6, kDeltaOut).u32(7, DD).f32(8, 1.0f / sqrtf((float)DD)).u32(9, Hv).u32(10, Hqk);
            if (DD == 128 && d->eps == 1e-6f)
                Rec(e, "rms_norm_gated_d128", Hv).tg(32).buf(0, kDeltaOut).buf(1, kDeltaZ).buf(2, kWeights, x.norm_weight).buf(3, kDeltaOut);
            else
                Rec(e, "rms_norm_gated", Hv).tg((uint32_t)(DD < 256 ? DD : 256)).buf(0, kDeltaOut).buf(1, kDeltaZ).buf(2, kWeights, x.norm_weight).buf(3, kDeltaOut)
                    .u32(4, DD).f32(5, d->eps);
            if (fuse) {
                Rec r(e, "fused_affine_matvec_add:" + std::to_string(dv) + ":" + std::to_string(G), (H + 7) / 8);
                r.affine(0, x.out).buf(3, kDeltaOut).buf(4, SMELT_SLOT_ALT).buf(5, SMELT_SLOT_CUR);
                count_const(r, 6, H);
            } else {
                { Rec r(e, matvec_name(dv, H), (H + 7) / 8); r.affine(0, x.out).buf(3, kDeltaOut).buf(4, kNormOut); count_const(r, 5, H); }
                Rec(e, "elementwise_add", (H + 63) / 64).buf(0, SMELT_SLOT_CUR).buf(1, kNormOut).buf(2, SMELT_SLOT_ALT).u32(3, (uint32_t)H);
            }
        } else {
        if (fuse2) {
            Rec r(e, "smelt_rmsnorm_affine_qkv:" + std::to_string(H) + ":64", ((qd + 2 * kvd) + 15) / 16);
            r.affine(0, w.q).affine(3, w.k).affine(6, w.v).buf(9, SMELT_SLOT_CUR).buf(10, kWeights, w.input_norm)
                .buf(11, kAttnQ).buf(12, kAttnK).buf(13, kAttnV).u32(14, qd).u32(15, kvd).f32(16, d->eps).u32(17, B);
            // RoPE, K/V append and attention in one launch
            Rec(e, "smelt_rope_attention_decode", d->n_q, B).buf(0, kAttnQ).buf(1, kslot).buf(2, vslot).buf(4, kAttnOut).buf(11, kAttnK).buf(12, kAttnV)
                .u32(5, D).con(6, SMELT_CONST_CACHE_SEQ_CAPACITY).con(7, SMELT_CONST_POSITION_PLUS1).u32(8, d->n_kv).f32(9, scale).u32(10, 0)
                .u32(13, 1).f32(14, log2_theta);
        } else {
        // input norm (TopLevelEmitter.swift:316-326)
        Rec(e, "rms_norm_1pw", B).buf(0, SMELT_SLOT_CUR).buf(1, kWeights, w.input_norm).buf(2, kNormOut).u32(3, H).f32(4, d->eps);
        // Q projection; fused dual K/V projection (AttentionPlugin.swift:105-300)
        { Rec r(e, matvec_name(H, qd), (qd + 7) / 8); r.affine(0, w.q).buf(3, kNormOut).buf(4, kAttnQ); count_const(r, 5, qd); }
        {
            Rec r(e, bt ? shaped("fused_dual_affine_matvec", H, kvd, G, true) : "fused_dual_affine_matvec:" + std::to_string(H) + ":" + std::to_string(G), (kvd + 7) / 8);
            r.affine(0, w.k).affine(3, w.v).buf(6, kNormOut).buf(7, kAttnK).buf(8, kAttnV);
            count_const(r, 9, kvd);
        }
        // RoPE on Q, fused RoPE + K append, V append (AttentionPlugin.swift:300-560; analytic mode :344-346)
        Rec(e, "apply_rope", (qd + 63) / 64, B).buf(0, kAttnQ).buf(1, kAttnQ).buf(2, kAttnQ)
            .u32(3, D).u32(4, D).u32(5, d->n_q).u32(6, 1).con(7, SMELT_CONST_POSITION).f32(8, log2_theta).u32(9, 1);
        {
            Rec r(e, "rope_kv_cache_update", (kvd + 63) / 64, B);
            r.buf(0, kslot).buf(1, kAttnK).buf(2, kAttnK).buf(3, kAttnK).con(4, SMELT_CONST_CACHE_SEQ_CAPACITY).u32(5, D)
                .con(6, SMELT_CONST_POSITION).u32(7, d->n_kv);
            // split-half layout over the full head, analytic trig: exactly the eight constants a record holds
            r.u32(8, D).u32(9, 1).f32(10, log2_theta).u32(11, 1);
        }
        Rec(e, "kv_cache_update", (kvd + 63) / 64, B).buf(0, vslot).buf(1, kAttnV).con(2, SMELT_CONST_CACHE_SEQ_CAPACITY).u32(3, D)
            .con(4, SMELT_CONST_POSITION).u32(5, d->n_kv);
        // attention decode (AttentionPlugin.swift:738-984): one threadgroup per query head
        Rec(e, "attention_decode", d->n_q, B).buf(0, kAttnQ).buf(1, kslot).buf(2, vslot).buf(3, kAttnQ).buf(4, kAttnOut)
            .u32(5, D).con(6, SMELT_CONST_CACHE_SEQ_CAPACITY).con(7, SMELT_CONST_POSITION_PLUS1).u32(8, d->n_kv).f32(9, scale).u32(10, 0);
        }
        // O projection + residual (TopLevelEmitter.swift:417-429)
        if (fuse) {
            Rec r(e, bt ? shaped("fused_affine_matvec_add", qd, H, G, true) : "fused_affine_matvec_add:" + std::to_string(qd) + ":" + std::to_string(G), (H + 7) / 8);
            r.affine(0, w.o).buf(3, kAttnOut).buf(4, SMELT_SLOT_ALT).buf(5, SMELT_SLOT_CUR);
            count_const(r, 6, H);
        } else {
            { Rec r(e, matvec_name(qd, H), (H + 7) / 8); r.affine(0, w.o).buf(3, kAttnOut).buf(4, kNormOut); count_const(r, 5, H); }
            if (tp && fuse_tp) Rec(e, "smelt_tp_reduce_add").buf(0, kNormOut).buf(1, SMELT_SLOT_CUR).buf(2, SMELT_SLOT_ALT).u32(3, (uint32_t)(B * H));
            else {
            if (tp) Rec(e, "smelt_tp_all_reduce").buf(0, kNormOut).u32(1, (uint32_t)(B * H));
            Rec(e, "elementwise_add", (B * H + 63) / 64).buf(0, SMELT_SLOT_CUR).buf(1, kNormOut).buf(2, SMELT_SLOT_ALT).u32(3, (uint32_t)(B * H));
            }
        }
        }  // attention mixer
        e.swap();
        // post-attention norm + FFN (TopLevelEmitter.swift:1021-1322 emitSwiGLU)
        if (fuse2) {
            Rec r(e, "smelt_rmsnorm_affine_gate_up_swiglu:" + std::to_string(H) + ":64", (I + 15) / 16);
            r.affine(0, w.gate).affine(3, w.up).buf(6, SMELT_SLOT_CUR).buf(7, kFfnInt).u32(8, I).buf(9, kWeights, w.post_norm).f32(10, d->eps).u32(11, B);
        } else {
        Rec(e, "rms_norm_1pw", B).buf(0, SMELT_SLOT_CUR).buf(1, kWeights, w.post_norm).buf(2, kNormOut).u32(3, H).f32(4, d->eps);
        {
            Rec r(e, bt ? shaped("fused_affine_gate_up_swiglu", H, I, G, true) : "fused_affine_gate_up_swiglu:" + std::to_string(H) + ":" + std::to_string(G), (I + 7) / 8);
            r.affine(0, w.gate).affine(3, w.up).buf(6, kNormOut).buf(7, kFfnInt);
            count_const(r, 8, I);
        }
        }
        if (fuse) {
            Rec r(e, bt ? shaped("fused_affine_matvec_add", I, H, G, true) : "fused_affine_matvec_add:" + std::to_string(I) + ":" + std::to_string(G), (H + 7) / 8);
            r.affine(0, w.down).buf(3, kFfnInt).buf(4, SMELT_SLOT_ALT).buf(5, SMELT_SLOT_CUR);
            count_const(r, 6, H);
        } else {
            { Rec r(e, matvec_name(I, H), (H + 7) / 8); r.affine(0, w.down).buf(3, kFfnInt).buf(4, kFfnDown); count_const(r, 5, H); }
            if (tp && fuse_tp) Rec(e, "smelt_tp_reduce_add").buf(0, kFfnDown).buf(1, SMELT_SLOT_CUR).buf(2, SMELT_SLOT_ALT).u32(3, (uint32_t)(B * H));
            else {
            if (tp) Rec(e, "smelt_tp_all_reduce").buf(0, kFfnDown).u32(1, (uint32_t)(B * H));
            Rec(e, "elementwise_add", (B * H + 63) / 64).buf(0, SMELT_SLOT_CUR).buf(1, kFfnDown).buf(2, SMELT_SLOT_ALT).u32(3, (uint32_t)(B * H));
            }
        }
        e.swap();
    }
    // final norm, LM head, argmax (TopLevelEmitter.swift:657-930)
    Rec(e, "rms_norm_1pw", B).buf(0, SMELT_SLOT_CUR).buf(1, kWeights, d->final_norm).buf(2, kNormOut).u32(3, H).f32(4, d->eps);
    // bit 3 (tp_world > 1): the LM head is split by vocab rows (lm_head addresses this rank's
    // slice), logits hold the slice, and the ranks exchange their best keys
    const bool vocab_par = tp && (d->fuse_residual & 8) && V % d->tp_world == 0;
    const int Vl = vocab_par ? V / d->tp_world : V;
    Rec(e, "fp16_matvec", Vl, B).buf(0, kWeights, d->lm_head).buf(1, kNormOut).buf(2, kLogits).u32(3, H);
    const int chunk = 2048, parts = (Vl + chunk - 1) / chunk;
    Rec(e, "argmax_fp16_partials", parts, B).buf(0, kLogits).buf(1, kArgmaxScratch).u32(2, Vl).u32(3, chunk);
    if (vocab_par) Rec(e, "smelt_tp_argmax", 1, B).buf(0, kArgmaxScratch).buf(1, kArgmax).u32(2, parts).u32(3, (uint32_t)(d->tp_rank * Vl));
    else Rec(e, "argmax_key_reduce", 1, B).buf(0, kArgmaxScratch).buf(1, kArgmax).u32(2, parts);

    const size_t need = e.n;
    if (records && need > *n_records) {
        *n_records = need;
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "build_decoder: record buffer too small");
    }
    *n_records = need;
    if (names) {
        names->assign(e.pipes.size(), std::string());
        for (auto& kv : e.pipes) (*names)[kv.second] = kv.first;
    }
    return e.status;
}

extern "C" smelt_status smelt_cuda_build_decoder(smelt_cuda_ctx* ctx, const smelt_decoder_desc* d,
                                                 const smelt_layer_ref* layers, uint32_t capacity, uint32_t batch,
                                                 smelt_dispatch_record* records, size_t* n_records) {
    return build_decoder_impl(ctx, d, layers, capacity, batch, records, n_records, nullptr);
}

// The prompt-chunk table of the same decoder, in the reference's prefill record shapes
// (Sources/SmeltCompiler/PrefillEmitter.swift: batched gathers and norms, *_batched projections with actualBatch =
// seqLen, rope_and_kv_cache_prefill_analytic, attention_prefill, last-row offset for the LM head): chunk length and
// start position are run-time constants, so one table serves every chunk up to max_chunk positions.
enum PrefillSlot : int { kPfX0 = 2, kPfX1 = 3, kPfNorm = 4, kPfQ = 5, kPfK = 6, kPfV = 7, kPfAttn = 9, kPfFfn = 10 };

enum PrefillDeltaSlot : int { kPfDeltaQkv = 11, kPfDeltaZ = 12, kPfDeltaA = 15, kPfDeltaB = 18, kPfDeltaOut = 19 };

static smelt_status build_prefill_impl(smelt_cuda_ctx* ctx, const smelt_decoder_desc* d, const smelt_layer_ref* layers, uint32_t max_chunk,
                                       smelt_dispatch_record* records, size_t* n_records, std::vector<std::string>* names, const Hybrid* hy = nullptr) {
    if (!d || !layers || !n_records) return SMELT_ERR_BAD_ARGUMENT;
    if (hy) {
        const smelt_delta_desc* dd = hy->dd;
        if (!dd || !hy->refs || !hy->kinds || dd->value_heads <= 0 || dd->qk_heads <= 0 || dd->value_heads % dd->qk_heads || dd->head_dim <= 0 || dd->head_dim % 32 ||
            dd->head_dim > 256 || dd->conv_kernel <= 0 || dd->conv_kernel > 8)
            return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "build_hybrid_prefill_table: bad linear-attention geometry");
    }
    if (d->layers <= 0 || d->layers > 100 || d->hidden <= 0 || d->inter <= 0 || d->n_q <= 0 || d->n_kv <= 0 || d->n_q % d->n_kv || d->head_dim <= 0 || d->vocab <= 0 ||
        max_chunk == 0 || d->tp_world > 1)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "build_prefill_table: bad model description (one GPU, batch 1)");
    const int H = d->hidden, I = d->inter, D = d->head_dim, G = d->group, L = d->layers, V = d->vocab;
    const int qd = d->n_q * D, kvd = d->n_kv * D;
    const size_t T = max_chunk;
    Emitter e{ctx, records, records ? *n_records : 0};
    if (ctx) {
        if (!records) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "build_prefill_table: a context needs a record buffer (query the count with a null context)");
        if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
        if (!ctx->configured || ctx->cfg.batch != 1 || !ctx->slots[kWeights].ptr)
            return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "build_prefill_table: build the decoder (batch 1) first");
        if (hy) {
            const smelt_delta_desc* dd = hy->dd;
            const size_t dq = (size_t)(2 * dd->qk_heads + dd->value_heads) * dd->head_dim, dv = (size_t)dd->value_heads * dd->head_dim;
            struct { int slot; size_t bytes; } dplan[] = {{kPfDeltaQkv, T * dq * 2}, {kPfDeltaZ, T * dv * 2}, {kPfDeltaA, T * dd->value_heads * 2 + 16},
                                                          {kPfDeltaB, T * dd->value_heads * 2 + 16}, {kPfDeltaOut, T * dv * 2}};
            for (auto& p : dplan) {
                smelt_status s = smelt_cuda_alloc_slot(ctx, p.slot, p.bytes);
                if (s) return s;
            }
        }
        struct { int slot; size_t bytes; } plan[] = {
            {kPfX0, T * H * 2}, {kPfX1, T * H * 2}, {kPfNorm, T * H * 2}, {kPfQ, T * qd * 2}, {kPfK, T * kvd * 2}, {kPfV, T * kvd * 2},
            {kPfAttn, T * qd * 2}, {kPfFfn, T * I * 2},
        };
        for (auto& p : plan) {
            smelt_status s = smelt_cuda_alloc_slot(ctx, p.slot, p.bytes);
            if (s) return s;
        }
        if (ctx->slots[kTokenId].bytes < T * 4) {  // a chunk's token ids (dropping any captured graph: rebuild it afterwards)
            smelt_status s = smelt_cuda_alloc_slot(ctx, kTokenId, T * 4);
            if (s) return s;
        }
        e.base = (int)ctx->pipelines.size();
    }
    const float log2_theta = log2f(d->rope_theta), scale = 1.0f / sqrtf((float)D);
    const uint8_t kSeq = SMELT_CONST_SEQ_LEN, kStart = SMELT_CONST_START_POS;
    Rec(e, "embedding_gather_batched", (H + 63) / 64, 1).grid_kind(1, 1).buf(0, kWeights, d->embedding).buf(1, kTokenId).buf(2, kPfX0).u32(3, H).con(4, kSeq);
    for (int l = 0; l < L; ++l) {
        const smelt_layer_ref& w = layers[l];
        const int kslot = kKvBase + l, vslot = kKvBase + L + l;
        Rec(e, "rms_norm_1pw_batched", 1).grid_kind(0, 1).tg(256).buf(0, kPfX0).buf(1, kWeights, w.input_norm).buf(2, kPfNorm).u32(3, H).f32(4, d->eps);
        if (hy && hy->kinds[l]) {
            // the DeltaNet mixer over the chunk: batched projections, the prompt-chunk convolution and recurrence, gated norm per (position, head)
            const smelt_delta_desc* dd = hy->dd;
            const smelt_delta_ref& x = hy->refs[l];
            const int DD = dd->head_dim, Hv = dd->value_heads, Hqk = dd->qk_heads;
            const int dq = (2 * Hqk + Hv) * DD, dv = Hv * DD;
            const int conv_slot = kKvBase + 2 * L + l, rec_slot = kKvBase + 3 * L + l;
            auto proj = [&](const smelt_affine_ref& wt, int rows, int out_slot) {
                Rec r(e, shaped("affine_matvec", H, rows, G, true) + "_full", (rows + 31) / 32, 1);
                r.grid_kind(1, 3).r->grid[1] = 8;
                r.affine(0, wt).buf(3, kPfNorm).buf(4, out_slot).con(5, kSeq);
            };
            proj(x.qkv, dq, kPfDeltaQkv); proj(x.z, dv, kPfDeltaZ); proj(x.a, Hv, kPfDeltaA); proj(x.b, Hv, kPfDeltaB);
            Rec(e, "conv1d_update_silu_prefill", (dq + 255) / 256).tg(256).buf(0, conv_slot).buf(1, kPfDeltaQkv).buf(2, kWeights, x.conv_weight).con(3, kSeq).u32(4, dq).u32(5, dd->conv_kernel);
            Rec(e, "rms_scale_qk", 2 * Hqk, 1).grid_kind(1, 1).tg(32u * (uint32_t)((DD + 127) / 128)).buf(0, kPfDeltaQkv).u32(1, DD).f32(2, 1e-6f).u32(3, dq).u32(4, Hqk);
            Rec(e, "deltanet_recurrence_mlx_prefill", 32, DD).tg(32).buf(0, rec_slot).buf(1, kPfDeltaQkv).buf(2, kPfDeltaB).buf(3, kPfDeltaA).buf(4, kWeights, x.a_log)
                .buf(5, kWeights, x.dt_bias).buf(6, kPfDeltaOut).u32(7, DD).u32(8, Hv).u32(9, Hqk).con(10, kSeq);
            if (DD == 128 && d->eps == 1e-6f)
                Rec(e, "rms_norm_gated_d128_batched", Hv, 1).grid_kind(1, 1).tg(32).buf(0, kPfDeltaOut).buf(1, kPfDeltaZ).buf(2, kWeights, x.norm_weight).buf(3, kPfDeltaOut).u32(4, Hv);
            else
                Rec(e, "rms_norm_gated", Hv).grid_kind(0, 2).tg((uint32_t)(DD < 256 ? DD : 256)).buf(0, kPfDeltaOut).buf(1, kPfDeltaZ).buf(2, kWeights, x.norm_weight).buf(3, kPfDeltaOut)
                    .u32(4, DD).f32(5, d->eps);
            { Rec r(e, shaped("fused_affine_matvec_add", dv, H, G, true), (H + 7) / 8, 1); r.grid_kind(1, 3).r->grid[1] = 4; r.affine(0, x.out).buf(3, kPfDeltaOut).buf(4, kPfX1).buf(5, kPfX0).con(6, kSeq); }
        } else {
        { Rec r(e, shaped("affine_matvec", H, qd, G, true) + "_full", (qd + 31) / 32, 1); r.grid_kind(1, 3).r->grid[1] = 8; r.affine(0, w.q).buf(3, kPfNorm).buf(4, kPfQ).con(5, kSeq); }
        { Rec r(e, shaped("fused_dual_affine_matvec", H, kvd, G, true), (kvd + 7) / 8, 1); r.grid_kind(1, 3).r->grid[1] = 4; r.affine(0, w.k).affine(3, w.v).buf(6, kPfNorm).buf(7, kPfK).buf(8, kPfV).con(9, kSeq); }
        Rec(e, "rope_and_kv_cache_prefill_analytic", 1, (uint32_t)(d->n_q > d->n_kv ? d->n_q : d->n_kv)).grid_kind(0, 1).buf(0, kPfQ).buf(1, kPfK).buf(2, kPfV).buf(3, kslot).buf(4, vslot)
            .u32(5, (uint32_t)D | ((uint32_t)D << 16)).u32(6, (uint32_t)d->n_q | ((uint32_t)d->n_kv << 16)).con(7, kSeq).con(8, kStart)
            .con(9, SMELT_CONST_CACHE_SEQ_CAPACITY).u32(10, 1).f32(11, log2_theta);
        {
            Rec r(e, "attention_prefill", d->n_q, 1);
            r.grid_kind(1, 1).buf(0, kPfQ).buf(1, kslot).buf(2, vslot).buf(3, kPfAttn).u32(4, D).con(5, kSeq).con(6, kStart).con(7, SMELT_CONST_CACHE_SEQ_CAPACITY);
            // a record holds eight constants: numKVHeads and scale follow, the sliding window (none) stays unbound
            r.u32(8, d->n_kv).f32(9, scale);
        }
        { Rec r(e, shaped("fused_affine_matvec_add", qd, H, G, true), (H + 7) / 8, 1); r.grid_kind(1, 3).r->grid[1] = 4; r.affine(0, w.o).buf(3, kPfAttn).buf(4, kPfX1).buf(5, kPfX0).con(6, kSeq); }
        }  // attention mixer
        Rec(e, "rms_norm_1pw_batched", 1).grid_kind(0, 1).tg(256).buf(0, kPfX1).buf(1, kWeights, w.post_norm).buf(2, kPfNorm).u32(3, H).f32(4, d->eps);
        { Rec r(e, shaped("fused_affine_gate_up_swiglu", H, I, G, true), (I + 7) / 8, 1); r.grid_kind(1, 3).r->grid[1] = 4; r.affine(0, w.gate).affine(3, w.up).buf(6, kPfNorm).buf(7, kPfFfn).con(8, kSeq); }
        { Rec r(e, shaped("fused_affine_matvec_add", I, H, G, true), (H + 7) / 8, 1); r.grid_kind(1, 3).r->grid[1] = 4; r.affine(0, w.down).buf(3, kPfFfn).buf(4, kPfX0).buf(5, kPfX1).con(6, kSeq); }
    }
    // the last position only: final norm, LM head, argmax (offset kind 3: (seqLen - 1) * row bytes)
    Rec(e, "rms_norm_1pw", 1).buf_kind(0, kPfX0, 3, (uint64_t)H * 2).buf(1, kWeights, d->final_norm).buf(2, kNormOut).u32(3, H).f32(4, d->eps);
    Rec(e, "fp16_matvec", V, 1).buf(0, kWeights, d->lm_head).buf(1, kNormOut).buf(2, kLogits).u32(3, H);
    const int chunk = 2048, parts = (V + chunk - 1) / chunk;
    Rec(e, "argmax_fp16_partials", parts, 1).buf(0, kLogits).buf(1, kArgmaxScratch).u32(2, V).u32(3, chunk);
    Rec(e, "argmax_key_reduce", 1, 1).buf(0, kArgmaxScratch).buf(1, kArgmax).u32(2, parts);
    const size_t need = e.n;
    if (records && need > *n_records) {
        *n_records = need;
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "build_prefill_table: record buffer too small");
    }
    *n_records = need;
    if (names) {
        names->assign(e.pipes.size(), std::string());
        for (auto& kv : e.pipes) (*names)[kv.second - e.base] = kv.first;
    }
    return e.status;
}

extern "C" smelt_status smelt_cuda_build_prefill_table(smelt_cuda_ctx* ctx, const smelt_decoder_desc* d, const smelt_layer_ref* layers,
                                                       uint32_t max_chunk, smelt_dispatch_record* records, size_t* n_records) {
    return build_prefill_impl(ctx, d, layers, max_chunk, records, n_records, nullptr);
}

extern "C" smelt_status smelt_cuda_build_hybrid_prefill_table(smelt_cuda_ctx* ctx, const smelt_decoder_desc* d, const smelt_layer_ref* layers,
                                                              const smelt_delta_desc* delta_desc, const smelt_delta_ref* delta, const uint8_t* kinds,
                                                              uint32_t max_chunk, smelt_dispatch_record* records, size_t* n_records) {
    const Hybrid hy{delta_desc, delta, kinds};
    return build_prefill_impl(ctx, d, layers, max_chunk, records, n_records, nullptr, &hy);
}

extern "C" smelt_status smelt_cuda_prefill_pipelines(const smelt_decoder_desc* d, char* out, size_t out_bytes, size_t* needed_bytes) {
    if (!d || !needed_bytes) return SMELT_ERR_BAD_ARGUMENT;
    std::vector<smelt_layer_ref> layers(d->layers > 0 && d->layers <= 100 ? d->layers : 1);
    std::vector<std::string> names;
    size_t n = 0;
    smelt_status s = build_prefill_impl(nullptr, d, layers.data(), 1, nullptr, &n, &names);
    if (s) return s;
    std::string joined;
    for (size_t i = 0; i < names.size(); ++i) joined += names[i] + "\n";
    *needed_bytes = joined.size() + 1;
    if (out && out_bytes >= joined.size() + 1) memcpy(out, joined.c_str(), joined.size() + 1);
    return SMELT_OK;
}

extern "C" smelt_status smelt_cuda_build_hybrid_decoder(smelt_cuda_ctx* ctx, const smelt_decoder_desc* d, const smelt_layer_ref* layers,
                                                        const smelt_delta_desc* delta_desc, const smelt_delta_ref* delta, const uint8_t* kinds,
                                                        uint32_t capacity, smelt_dispatch_record* records, size_t* n_records) {
    const Hybrid hy{delta_desc, delta, kinds};
    return build_decoder_impl(ctx, d, layers, capacity, 1, records, n_records, nullptr, &hy);
}

extern "C" smelt_status smelt_cuda_decoder_pipelines(const smelt_decoder_desc* d, uint32_t batch, char* out, size_t out_bytes,
                                                     size_t* needed_bytes) {
    if (!d || !needed_bytes) return SMELT_ERR_BAD_ARGUMENT;
    std::vector<smelt_layer_ref> layers(d->layers > 0 && d->layers <= 100 ? d->layers : 1);
    std::vector<std::string> names;
    size_t n = 0;
    smelt_status s = build_decoder_impl(nullptr, d, layers.data(), 1, batch, nullptr, &n, &names);
    if (s) return s;
    std::string joined;
    for (size_t i = 0; i < names.size(); ++i) joined += names[i] + "\n";
    *needed_bytes = joined.size() + 1;
    if (out && out_bytes >= joined.size() + 1) memcpy(out, joined.c_str(), joined.size() + 1);
    return SMELT_OK;
}
