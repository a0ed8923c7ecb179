/*
 * smelt_cuda.h — C ABI of libsmelt_cuda: the sm_100a (B200) replacement for the Metal kernels
 * behind SmeltRuntime's decode dispatch surface.
 *
 * What it replaces.  In the reference, Sources/SmeltRuntime/SmeltRuntime.swift interprets a
 * table of fixed-width SmeltDispatchRecord values (Sources/SmeltSchema/SmeltDispatchTable.swift
 * :21-165) into Metal compute commands: it resolves a pipeline by name, binds slot-indexed
 * buffers at byte offsets, resolves up to eight constants and dispatches
 * (SmeltRuntime.swift:3187-3247, emitDecodeDispatchRecord).  This library keeps that surface —
 * the same 360-byte records, the same kernel names, buffer binding indices and constant
 * binding indices, the same packed-weight layout — and launches hand-written CUDA kernels.
 * A Metal grid / threadgroup size in a record is advisory; launch geometry is derived from the
 * kernel name, constants and shapes.
 *
 * Conventions.  Every function returns a smelt_status (0 = ok) and never aborts; the text of
 * the last failure is available from smelt_cuda_last_error().  A context is bound to one CUDA
 * device and one stream and is not thread-safe (the reference runtime is single-threaded per
 * instance, SmeltRuntime.swift:1950).  Pointers named *_dev are device pointers, everything
 * else is host memory.  fp16 data is IEEE binary16 stored as uint16_t.  There is no CPU
 * fallback anywhere: when no CUDA device is usable, smelt_cuda_create fails.
 */
#ifndef SMELT_CUDA_H
#define SMELT_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SMELT_CUDA_API __attribute__((visibility("default")))

typedef int32_t smelt_status;
enum {
    SMELT_OK = 0,
    SMELT_ERR_BAD_ARGUMENT = 1,     /* shape / alignment / null-pointer violation */
    SMELT_ERR_UNKNOWN_PIPELINE = 2, /* kernel name not implemented (no silent default) */
    SMELT_ERR_OUT_OF_RANGE = 3,     /* token, position, slot or weight offset out of range */
    SMELT_ERR_CUDA = 4,             /* a CUDA runtime call failed */
    SMELT_ERR_ALLOC = 5,            /* device or host allocation failed */
    SMELT_ERR_UNSUPPORTED = 6,      /* valid request outside the implemented hot path */
    SMELT_ERR_COMM = 7,             /* tensor-parallel communicator failure */
    SMELT_ERR_DEVICE_TIMEOUT = 8    /* a bounded device-side wait gave up */
};

typedef struct smelt_cuda_ctx smelt_cuda_ctx;

/* ── SmeltDispatchRecord, byte for byte (Sources/SmeltSchema/SmeltDispatchTable.swift:21-165;
 *    sizes 16 / 8 / 360 pinned by Tests/SmeltCompilerTests/DispatchTableTests.swift:12-30) ── */
typedef struct {
    int16_t slot;         /* >= 0 literal slot, -1 = cur, -2 = alt */
    uint8_t binding_index;
    uint8_t offset_kind;  /* 0 literal byte offset, 1 position * offset */
    uint32_t _pad;
    uint64_t offset;
} smelt_buffer_record;

typedef struct {
    uint8_t kind;           /* SMELT_CONST_* */
    uint8_t binding_index;  /* 255 = guard only, not bound */
    uint16_t pad;
    uint32_t value;
} smelt_constant_record;

typedef struct {
    uint8_t op_kind; /* 0 dispatch, 1 swap cur/alt */
    uint8_t _pad0;
    uint16_t pipeline;
    uint8_t style;
    uint8_t buffer_count;
    uint8_t constant_count;
    uint8_t _pad1;
    uint16_t min_seq_len;
    uint16_t _pad2;
    uint32_t grid[3];
    uint32_t threadgroup[3];
    uint32_t _pad3;
    smelt_buffer_record buf[16];
    smelt_constant_record con[8];
} smelt_dispatch_record;

enum {
    SMELT_CONST_LITERAL_U32 = 0,
    SMELT_CONST_LITERAL_F32 = 1,
    SMELT_CONST_POSITION = 2,
    SMELT_CONST_POSITION_PLUS1 = 3,
    /* prompt chunks only (smelt_cuda_enqueue_prefill): seqLen, startPos, startPos + value, seqLen * value, seqLen % value,
     * the same with the dispatch skipped when it is zero (SmeltDispatchTable.swift:68-79) */
    SMELT_CONST_SEQ_LEN = 4,
    SMELT_CONST_START_POS = 5,
    SMELT_CONST_START_POS_PLUS = 6,
    SMELT_CONST_SEQ_LEN_MUL = 7,
    SMELT_CONST_SEQ_LEN_MOD = 8,
    SMELT_CONST_SEQ_LEN_MOD_SKIP_IF_ZERO = 9,
    SMELT_CONST_SKIP_UNLESS_POS1_LT = 10,
    SMELT_CONST_SKIP_UNLESS_POS1_GE = 11,
    SMELT_CONST_CACHE_SEQ_CAPACITY = 12,
    SMELT_CONST_SKIP_UNLESS_SEQ_LEN_LT = 13 /* prompt chunks only: the dispatch runs only while seqLen < value */
};
enum { SMELT_OP_DISPATCH = 0, SMELT_OP_SWAP = 1 };
enum { SMELT_SLOT_CUR = -1, SMELT_SLOT_ALT = -2 };

/* ── context ─────────────────────────────────────────────────────────────────
 * Replaces the MTLDevice / MTLCommandQueue set-up of SmeltRuntime.init
 * (SmeltRuntime.swift:695-712). */
SMELT_CUDA_API smelt_status smelt_cuda_create(int device_ordinal, smelt_cuda_ctx** out_ctx);
SMELT_CUDA_API void smelt_cuda_destroy(smelt_cuda_ctx* ctx);
SMELT_CUDA_API const char* smelt_cuda_last_error(const smelt_cuda_ctx* ctx);
SMELT_CUDA_API smelt_status smelt_cuda_synchronize(smelt_cuda_ctx* ctx);
/* The context's cudaStream_t, for callers that enqueue their own work around the library's. */
SMELT_CUDA_API void* smelt_cuda_stream(smelt_cuda_ctx* ctx);
/* Reads and clears the device error word that kernels set when a bounded wait gives up.
 * Synchronises the stream.  *out_flags == 0 means no kernel reported a problem. */
SMELT_CUDA_API smelt_status smelt_cuda_device_error(smelt_cuda_ctx* ctx, uint32_t* out_flags);
SMELT_CUDA_API int smelt_cuda_sm_count(const smelt_cuda_ctx* ctx);

/* Raw device memory for callers that drive the typed launchers directly (tests, benchmarks). */
SMELT_CUDA_API smelt_status smelt_cuda_malloc(smelt_cuda_ctx* ctx, size_t bytes, void** out_dev);
SMELT_CUDA_API smelt_status smelt_cuda_free(smelt_cuda_ctx* ctx, void* dev);
SMELT_CUDA_API smelt_status smelt_cuda_memcpy_h2d(smelt_cuda_ctx* ctx, void* dst_dev, const void* src, size_t bytes);
SMELT_CUDA_API smelt_status smelt_cuda_memcpy_d2h(smelt_cuda_ctx* ctx, void* dst, const void* src_dev, size_t bytes);
SMELT_CUDA_API smelt_status smelt_cuda_memset(smelt_cuda_ctx* ctx, void* dst_dev, int value, size_t bytes);

/* ── buffer slots ────────────────────────────────────────────────────────────
 * The slot-indexed buffer array of SmeltRuntime (allocation and zero fill
 * SmeltRuntime.swift:922-979; request-scoped growth :6803-6913; KV sizing
 * heads * capacity * head_dim * 2 bytes :6891-6913).  Slots are zero-filled at creation. */
SMELT_CUDA_API smelt_status smelt_cuda_alloc_slot(smelt_cuda_ctx* ctx, int slot, size_t bytes);
/* Grow (or shrink) a slot, keeping the first preserve_bytes bytes and zero-filling the rest.
 * Any device pointer obtained earlier for the slot is stale afterwards
 * (SmeltRuntime.swift:5101-5103). */
SMELT_CUDA_API smelt_status smelt_cuda_resize_slot(smelt_cuda_ctx* ctx, int slot, size_t bytes, size_t preserve_bytes);
/* Grow a KV-cache slot laid out [heads, capacity, head_dim] fp16 from old_capacity to
 * new_capacity positions, keeping the first live_len positions of every head in place
 * (contents are preserved across growth, SmeltRuntime.swift:6957-6959). */
SMELT_CUDA_API smelt_status smelt_cuda_resize_kv_slot(smelt_cuda_ctx* ctx, int slot, int heads, int head_dim,
                                                      uint32_t old_capacity, uint32_t new_capacity, uint32_t live_len);
SMELT_CUDA_API smelt_status smelt_cuda_slot_ptr(smelt_cuda_ctx* ctx, int slot, void** out_dev, size_t* out_bytes);
SMELT_CUDA_API smelt_status smelt_cuda_write_slot(smelt_cuda_ctx* ctx, int slot, size_t offset, const void* src, size_t bytes);
SMELT_CUDA_API smelt_status smelt_cuda_read_slot(smelt_cuda_ctx* ctx, int slot, size_t offset, void* dst, size_t bytes);
SMELT_CUDA_API smelt_status smelt_cuda_zero_slot(smelt_cuda_ctx* ctx, int slot);
/* The whole weights.bin image into one device allocation bound to `slot`; record offsets into
 * that slot index the image exactly as bindBuffer does (SmeltRuntime.swift:3153-3169). */
SMELT_CUDA_API smelt_status smelt_cuda_upload_weights(smelt_cuda_ctx* ctx, int slot, const void* image, size_t bytes);

/* Runtime configuration a package's manifest provides (slot layout and limits,
 * Sources/SmeltSchema/SmeltManifest.swift:806-817; bounds checks SmeltRuntime.swift:3176-3183). */
typedef struct {
    int32_t token_id_slot;      /* int32 token id(s), one per sequence */
    int32_t position_slot;      /* int32 position */
    int32_t weights_slot;
    int32_t argmax_slot;        /* int32 result(s) read back by smelt_cuda_decode_step */
    int32_t cur_slot, alt_slot; /* initial double-buffer pair (0 and 1 in the reference) */
    uint32_t cache_seq_capacity;
    uint32_t context_limit;
    uint32_t vocab_size;
    uint32_t batch;             /* independent sequences decoded together (1 in the reference) */
} smelt_cuda_runtime_config;
SMELT_CUDA_API smelt_status smelt_cuda_configure(smelt_cuda_ctx* ctx, const smelt_cuda_runtime_config* cfg);

/* ── pipelines and dispatch ──────────────────────────────────────────────────
 * manifest.pipelines[index] = "name" or "name:cols:groupSize" (function constants 0/1,
 * SmeltRuntime.swift:6229-6263).  Unknown names are an error, mirroring the reference's
 * total kernel table (Sources/SmeltCompiler/MatvecKernelTable.swift:258-270). */
SMELT_CUDA_API smelt_status smelt_cuda_register_pipeline(smelt_cuda_ctx* ctx, int index, const char* name);
/* 1 when `name` (with or without the :cols:group suffix) is an implemented kernel. */
SMELT_CUDA_API int smelt_cuda_pipeline_supported(const char* name);

/* One decoded token, synchronously: writes token / position into their slots, interprets the
 * table, waits, reads the argmax slot (SmeltRuntime.decodeStep, SmeltRuntime.swift:1573-1641).
 * tokens / out_tokens hold config.batch entries. */
/* A prompt chunk through a prefill dispatch table (encodeTrunkPrefill, SmeltRuntime.swift:5062-5091): writes seq_len
 * token ids to the token slot and interprets the records with the prompt-chunk kinds resolved on the host: constants
 * seqLen / startPos / startPos + v / seqLen * v / seqLen % v (4..9) and the seqLen < v guard (13), position kinds as
 * startPos, buffer offsets startPos * stride + addend / (seqLen - 1) * stride / floor(seqLen / d) * stride (2..4), grid
 * dimensions that follow seqLen (style bits 2..7) and the record's minSeqLen guard.  Enqueue only; eager (not captured);
 * start_pos + seq_len must stay inside min(context_limit, cache_seq_capacity). */
SMELT_CUDA_API smelt_status smelt_cuda_enqueue_prefill(smelt_cuda_ctx* ctx, const smelt_dispatch_record* table, size_t n_records,
                                                       const int32_t* tokens_host, int32_t seq_len, int32_t start_pos);
SMELT_CUDA_API smelt_status smelt_cuda_decode_step(smelt_cuda_ctx* ctx, const smelt_dispatch_record* table, size_t n_records,
                                                   const int32_t* tokens, int32_t position, int32_t* out_tokens);
/* Enqueue-only form (encodeTrunkDecode, SmeltRuntime.swift:5029-5091): no wait, no readback.
 * Capacity must have been ensured before the call. */
SMELT_CUDA_API smelt_status smelt_cuda_enqueue_decode(smelt_cuda_ctx* ctx, const smelt_dispatch_record* table, size_t n_records,
                                                      const int32_t* tokens, int32_t position);
/* Capture the table once into a CUDA graph whose kernels read token and position from device
 * memory; each replay decodes one token and feeds the argmax result back as the next token
 * on the device, so a run of greedy steps needs no host round trip.  Allocating an existing
 * slot again or resizing a slot drops every graph of the context (their kernels hold the old
 * device pointers): graph_step / graph_decode / capture_replay then fail with
 * SMELT_ERR_BAD_ARGUMENT until the graph is built again. */
SMELT_CUDA_API smelt_status smelt_cuda_graph_build(smelt_cuda_ctx* ctx, const smelt_dispatch_record* table, size_t n_records);
/* Set the device-resident token(s) and position the next replay starts from. */
SMELT_CUDA_API smelt_status smelt_cuda_graph_seed(smelt_cuda_ctx* ctx, const int32_t* tokens, int32_t position);
/* Replay n_steps tokens.  When out_tokens != NULL, waits and returns the n_steps * batch
 * generated ids (step-major).  Needs a graph_seed (or graph_step) first; a run that would pass
 * min(context_limit, cache_seq_capacity) is refused with SMELT_ERR_OUT_OF_RANGE before any replay
 * (positions are bounds-checked as in SmeltRuntime.swift:3176-3183). */
SMELT_CUDA_API smelt_status smelt_cuda_graph_decode(smelt_cuda_ctx* ctx, int n_steps, int32_t* out_tokens);
/* The ids of the last n_steps replays since the last graph_seed (step-major, n_steps * batch),
 * read from the device ring without replaying anything: what a run of
 * smelt_cuda_graph_decode(ctx, n, NULL) calls generated.  Waits for the stream.  (The reference
 * reads each token back per step, SmeltRuntime.swift:1630-1641; this is the batched form.) */
SMELT_CUDA_API smelt_status smelt_cuda_graph_generated(smelt_cuda_ctx* ctx, int n_steps, int32_t* out_tokens);
/* One token through the captured graph with host buffers: tokens and position travel in,
 * the graph is replayed once, the argmax ids are read back and the call waits — the
 * graph-backed equivalent of smelt_cuda_decode_step. */
SMELT_CUDA_API smelt_status smelt_cuda_graph_step(smelt_cuda_ctx* ctx, const int32_t* tokens, int32_t position, int32_t* out_tokens);
/* Device-side stopwatch on the context's stream (the gpuStartTime / gpuEndTime pair of
 * profileDecodeStep, SmeltRuntime.swift:3279-3318): start records an event, stop records a
 * second one, waits for it and returns the elapsed milliseconds between the two. */
SMELT_CUDA_API smelt_status smelt_cuda_timer_start(smelt_cuda_ctx* ctx);
SMELT_CUDA_API smelt_status smelt_cuda_timer_stop(smelt_cuda_ctx* ctx, float* out_ms);
/* Caller-driven capture: every launch made through this context between capture_begin and
 * capture_end (typed launchers, smelt_cuda_enqueue_decode) is recorded instead of run, the way
 * encodeTrunkDecode records into a caller-owned encoder without committing it
 * (SmeltRuntime.swift:5029-5091).  capture_replay runs the recorded sequence `warmup` times
 * untimed, then `reps` times between two events, and returns the mean device time of one
 * replay in milliseconds.  Nothing may allocate or synchronise between begin and end; a new
 * capture_begin discards the previous recording. */
SMELT_CUDA_API smelt_status smelt_cuda_capture_begin(smelt_cuda_ctx* ctx);
SMELT_CUDA_API smelt_status smelt_cuda_capture_end(smelt_cuda_ctx* ctx);
SMELT_CUDA_API smelt_status smelt_cuda_capture_replay(smelt_cuda_ctx* ctx, int warmup, int reps, float* out_ms_per_replay);
/* Number of kernel launches one interpretation of the last built / enqueued table issues. */
SMELT_CUDA_API int smelt_cuda_last_launch_count(const smelt_cuda_ctx* ctx);

/* ── decoder table builder ───────────────────────────────────────────────────
 * Emits, for a plain decoder-only model, the per-token record sequence the reference
 * compiler emits (Sources/SmeltCompiler/TopLevelEmitter.swift:89-930, AttentionPlugin.swift
 * :105-560): embedding gather, per layer rms_norm_1pw -> Q/K/V projections -> RoPE ->
 * KV append -> attention decode -> O projection -> residual add -> rms_norm_1pw ->
 * fused gate/up SwiGLU -> down projection -> residual add, final norm, LM head, argmax.
 * Weight offsets address the weights slot; the slot numbers follow SmeltFixedSlot
 * (Sources/SmeltCompiler/SmeltBufferPlan.swift:129-198). */
typedef struct {
    uint64_t packed, scales, biases; /* byte offsets into the weights image */
} smelt_affine_ref;
typedef struct {
    uint64_t input_norm, post_norm;  /* fp16 [hidden], stored as weight - 1 */
    smelt_affine_ref q, k, v, o, gate, up, down;
} smelt_layer_ref;
typedef struct {
    int32_t layers, hidden, inter, n_q, n_kv, head_dim, vocab, group;
    float eps, rope_theta;
    uint64_t embedding, lm_head, final_norm;
    int32_t tp_world;   /* 1 = single GPU; >1 inserts an all-reduce after the O and down projections */
    int32_t tp_rank;
    int32_t fuse_residual; /* bit 0: emit fused_affine_matvec_add instead of matvec + elementwise_add (tp_world == 1 only);
                              bit 1: fold each RMS norm into the projection that follows it (one Q/K/V launch, one
                              gate/up launch) and RoPE + KV append + attention into one launch (the smelt_*
                              extension kernels); bit 2 (tp_world > 1): all-reduce + residual add as one
                              smelt_tp_reduce_add record; bit 3 (tp_world > 1): lm_head addresses this rank's
                              vocab / tp_world rows and the ranks exchange their best keys (smelt_tp_argmax) */
} smelt_decoder_desc;
/* Allocates the activation / KV / scratch slots for `desc` at `capacity` positions and
 * `batch` sequences, registers the pipelines, configures the context and writes the table.
 * With ctx == NULL nothing is allocated: the call only writes the records (or, with
 * records == NULL, returns their count through *n_records); pipeline indices are
 * assigned in order of first use and listed by smelt_cuda_decoder_pipelines. */
SMELT_CUDA_API smelt_status smelt_cuda_build_decoder(smelt_cuda_ctx* ctx, const smelt_decoder_desc* desc,
                                                     const smelt_layer_ref* layers, uint32_t capacity, uint32_t batch,
                                                     smelt_dispatch_record* records, size_t* n_records);
/* A hybrid decoder: layers whose token mixer is a DeltaNet (gated linear-attention) block instead of attention, as the
 * reference's DeltaNetPlugin emits them (Sources/SmeltCompiler/DeltaNetPlugin.swift:60-420): input norm, the QKV / Z / A / B
 * projections of the normed hidden state, conv1d_update_silu on the QKV row, rms_scale_qk, deltanet_recurrence_mlx_decode,
 * rms_norm_gated with Z, the output projection + residual; then the same feed-forward half as an attention layer.
 * kinds[l] = 0 attention (layers[l] complete), 1 DeltaNet (layers[l] supplies the norms and the feed-forward tensors,
 * delta[l] the mixer's).  Per DeltaNet layer two state slots are allocated after the KV slots: the convolution taps
 * [qkv_dim, conv_kernel] at 40 + 2 L + l and the recurrent matrix [value_heads, head_dim, head_dim] at 40 + 3 L + l
 * (fp16, zero at start).  One GPU, batch 1; the norm + projection fusions apply to the feed-forward half only. */
typedef struct {
    int32_t value_heads, qk_heads, head_dim, conv_kernel;
} smelt_delta_desc;
typedef struct {
    smelt_affine_ref qkv, z, a, b, out;                   /* [(2 qk_heads + value_heads) D, H], [value_heads D, H], [value_heads, H] x 2, [H, value_heads D] */
    uint64_t conv_weight, a_log, dt_bias, norm_weight;    /* fp16 [qkv_dim, conv_kernel], [value_heads], [value_heads], [D] */
} smelt_delta_ref;
SMELT_CUDA_API smelt_status smelt_cuda_build_hybrid_decoder(smelt_cuda_ctx* ctx, const smelt_decoder_desc* desc,
                                                            const smelt_layer_ref* layers, const smelt_delta_desc* delta_desc,
                                                            const smelt_delta_ref* delta, const uint8_t* kinds, uint32_t capacity,
                                                            smelt_dispatch_record* records, size_t* n_records);
/* The same for a hybrid decoder (smelt_cuda_build_hybrid_decoder): a DeltaNet layer runs its batched projections,
 * conv1d_update_silu_prefill, rms_scale_qk over the chunk's rows, deltanet_recurrence_mlx_prefill and the gated norm per
 * (position, head).  The recurrent rows stay in fp32 across a chunk and are rounded at its end, as the reference's
 * prompt-chunk kernel does, so the chunking is part of the result.  Adds the chunk slots 11, 12, 15, 18, 19. */
SMELT_CUDA_API smelt_status smelt_cuda_build_hybrid_prefill_table(smelt_cuda_ctx* ctx, const smelt_decoder_desc* desc,
                                                                  const smelt_layer_ref* layers, const smelt_delta_desc* delta_desc,
                                                                  const smelt_delta_ref* delta, const uint8_t* kinds, uint32_t max_chunk,
                                                                  smelt_dispatch_record* records, size_t* n_records);

/* The prompt-chunk table of the decoder smelt_cuda_build_decoder built (same descriptor and layer references; one
 * GPU, batch 1), in the reference's prefill record shapes (Sources/SmeltCompiler/PrefillEmitter.swift): chunk length
 * and start position are run-time constants, so one table serves every chunk of up to max_chunk positions through
 * smelt_cuda_enqueue_prefill.  Allocates the chunk's activation slots (2..7, 9, 10), grows the token slot to
 * max_chunk ids (call it before smelt_cuda_graph_build: growing a slot drops a captured graph) and registers the
 * table's pipelines after the decode table's.  Null ctx / records: counts only. */
SMELT_CUDA_API smelt_status smelt_cuda_build_prefill_table(smelt_cuda_ctx* ctx, const smelt_decoder_desc* desc,
                                                           const smelt_layer_ref* layers, uint32_t max_chunk,
                                                           smelt_dispatch_record* records, size_t* n_records);

/* The pipeline names of the table smelt_cuda_build_prefill_table writes, in the order of the indices a table built
 * without a context carries (0, 1, ...): newline separated, as smelt_cuda_decoder_pipelines reports the decode table's. */
SMELT_CUDA_API smelt_status smelt_cuda_prefill_pipelines(const smelt_decoder_desc* desc, char* out, size_t out_bytes, size_t* needed_bytes);

/* The manifest.pipelines array matching the table smelt_cuda_build_decoder writes for `desc`
 * and `batch`: names in index order, newline separated.  *needed_bytes receives the size of
 * the text including its terminator; out may be NULL to query it. */
SMELT_CUDA_API smelt_status smelt_cuda_decoder_pipelines(const smelt_decoder_desc* desc, uint32_t batch, char* out,
                                                         size_t out_bytes, size_t* needed_bytes);

/* ── package reader ──────────────────────────────────────────────────────────
 * The part of SmeltRuntime.init between a .smeltpkg directory and the first decoded token
 * (Sources/SmeltRuntime/SmeltRuntime.swift:668-998): manifest.json (pipelines, buffers.slots,
 * slotLayout, config.vocabSize, weights.entries: Sources/SmeltSchema/SmeltManifest.swift:26-98,
 * :806-817, :1649-1768), weights.bin, dispatches.bin and, when present, prefill_dispatches.bin
 * (SmeltRuntime.swift:842-853).  model.metallib, checksums, the verify tables and prepared-prefix
 * snapshots are not read. */
typedef struct {
    uint32_t context_capacity; /* positions every KV cache slot holds; 0 = the capacity the slots were compiled for */
    uint32_t context_limit;    /* 0 = context_capacity */
} smelt_package_options;
typedef struct {
    uint32_t n_records, n_pipelines, n_pipelines_used, n_slots, n_weight_entries;
    uint32_t vocab_size, hidden_size, num_layers, cache_seq_capacity;
    int32_t token_id_slot, position_slot, weights_slot, argmax_slot, logits_slot;
    uint64_t weights_bytes;
    uint32_t n_prefill_records; /* records of prefill_dispatches.bin when the package has one and every kernel it names is bound; else 0 */
    uint32_t _pad;
} smelt_package_info;
/* Host only (no device needed): parses and validates a package the way the loader does and
 * reports the first problem in err: manifest fields missing, a weight entry outside weights.bin
 * (SMELT_ERR_OUT_OF_RANGE), dispatches.bin not a multiple of the 360-byte record stride
 * (SmeltRuntime.swift:6332-6338), a record naming a pipeline index the manifest does not list or
 * a kernel that is not implemented (SMELT_ERR_UNKNOWN_PIPELINE). */
SMELT_CUDA_API smelt_status smelt_cuda_inspect_package(const char* package_dir, smelt_package_info* out_info, char* err, size_t err_bytes);
/* Loads the package into the context: weights.bin into the weights slot, one zero-filled buffer
 * per manifest slot (KV caches keyCache_<n> / valCache_<n> of shape [heads, capacity, head_dim]
 * sized for context_capacity, SmeltRuntime.swift:6891-6913), the pipelines the decode table uses
 * registered under their manifest indices, the runtime configured (token / position / weights
 * slots from slotLayout, argmax in fixed slot 17, hiddenA / hiddenB = slots 0 / 1 as the double
 * buffer, SmeltRuntimeConfig.swift:104-150), dispatches.bin kept as the context's decode table. */
SMELT_CUDA_API smelt_status smelt_cuda_open_package(smelt_cuda_ctx* ctx, const char* package_dir, const smelt_package_options* options,
                                                    smelt_package_info* out_info);
/* The decode table of the open package (owned by the context; valid until the next open or destroy):
 * pass it to smelt_cuda_decode_step / smelt_cuda_enqueue_decode / smelt_cuda_graph_build. */
SMELT_CUDA_API smelt_status smelt_cuda_package_table(smelt_cuda_ctx* ctx, const smelt_dispatch_record** out_table, size_t* out_n);
/* The prompt-chunk table of the open package for smelt_cuda_enqueue_prefill.  A package without
 * prefill_dispatches.bin, or whose prefill table names a kernel that is not bound, still opens and decodes; this call
 * then fails with the reason (SMELT_ERR_UNSUPPORTED / SMELT_ERR_UNKNOWN_PIPELINE) and the prompt goes through decode steps. */
SMELT_CUDA_API smelt_status smelt_cuda_package_prefill_table(smelt_cuda_ctx* ctx, const smelt_dispatch_record** out_table, size_t* out_n);

/* ── tensor parallelism (no counterpart in the reference, which is single-device) ──
 * One process per GPU.  Rank 0 creates an id, the caller ships it to the other ranks, every
 * rank calls init.  The record interpreter then accepts the pipeline name
 * "smelt_tp_all_reduce" (buffer 0 in/out fp16, constant 1 = element count). */
#define SMELT_TP_ID_BYTES 128
SMELT_CUDA_API smelt_status smelt_cuda_tp_unique_id(uint8_t id[SMELT_TP_ID_BYTES]);
SMELT_CUDA_API smelt_status smelt_cuda_tp_init(smelt_cuda_ctx* ctx, int rank, int world, const uint8_t id[SMELT_TP_ID_BYTES]);
SMELT_CUDA_API smelt_status smelt_cuda_tp_all_reduce_f16(smelt_cuda_ctx* ctx, void* data_dev, size_t count);
/* Peer-memory exchange for the fused all-reduce + residual add ("smelt_tp_reduce_add": buffer 0
 * this rank's partial, 1 residual, 2 out, constant 3 = element count): every rank publishes the
 * IPC handle of its exchange buffer (exchange_handle), the caller gathers the handles of all
 * ranks in rank order and every rank maps them (exchange_open).  A reduction is then one launch
 * per rank: partials are pushed into the peers' buffers over NVLink in 8-byte stores that carry
 * their sequence number (no fence, no separate flag),
 * each rank adds the partials in rank order in fp32, rounds once to fp16 and adds the residual.
 * Waits are bounded (about a second); a peer that never arrives sets bit 8 of the device error
 * word (smelt_cuda_device_error), so the ranks must be aligned (a barrier on the host) between
 * their set-up and the first exchange.  Without open exchange buffers the record falls back to
 * ncclAllReduce followed by elementwise_add. */
#define SMELT_TP_HANDLE_BYTES 64
SMELT_CUDA_API smelt_status smelt_cuda_tp_exchange_handle(smelt_cuda_ctx* ctx, uint8_t handle[SMELT_TP_HANDLE_BYTES]);
SMELT_CUDA_API smelt_status smelt_cuda_tp_exchange_open(smelt_cuda_ctx* ctx, const uint8_t* handles_in_rank_order);
/* Diagnostic: makes this context rank 0 of `world` ranks whose other exchange buffers are local
 * allocations that nobody ever writes.  A smelt_tp_reduce_add or smelt_tp_argmax launched
 * afterwards therefore runs into its bounded wait, sets bit 8 of the device error word and
 * returns, leaving the context usable: the way to exercise the give-up path on one GPU without
 * a peer that fails.  smelt_cuda_tp_reduce_add is the typed form of the record. */
SMELT_CUDA_API smelt_status smelt_cuda_tp_exchange_open_loopback(smelt_cuda_ctx* ctx, int world);
SMELT_CUDA_API smelt_status smelt_cuda_tp_reduce_add(smelt_cuda_ctx* ctx, const void* partial_dev, const void* residual_dev,
                                                     void* out_dev, size_t count);
/* Clears the device error word (after smelt_cuda_device_error has been read). */
SMELT_CUDA_API smelt_status smelt_cuda_clear_device_error(smelt_cuda_ctx* ctx);

/* ── typed launchers (asynchronous on the context's stream) ──────────────────
 * Packed-weight layouts are the package's: affine u4 = two nibbles per byte, low nibble =
 * even column, scales / biases fp16 [rows, cols/group]
 * (Sources/SmeltCompiler/SmeltAffineU4.swift:5-10); binary1 / ternary2 = LSB-first codes,
 * scales fp16 [rows, cols/128] (Sources/SmeltRuntime/SmeltSignedQuantCodec.swift:102-124).
 * Activations x are fp16 [batch, cols]; outputs y fp16 [batch, rows]. */

/* affine_matvec (Resources/Shaders/lut_matvec.metal:1157-1287) and its batched forms (:3238-3461). */
SMELT_CUDA_API smelt_status smelt_cuda_affine_matvec(smelt_cuda_ctx* ctx, const void* w_dev, const void* scales_dev,
                                                     const void* biases_dev, const void* x_dev, void* y_dev, int rows,
                                                     int cols, int group, int batch);
/* fused_affine_matvec_add (lut_matvec.metal:1718-1817): y = half(acc) + residual; y may alias residual. */
SMELT_CUDA_API smelt_status smelt_cuda_affine_matvec_add(smelt_cuda_ctx* ctx, const void* w_dev, const void* scales_dev,
                                                         const void* biases_dev, const void* x_dev,
                                                         const void* residual_dev, void* y_dev, int rows, int cols,
                                                         int group, int batch);
/* fused_affine_gate_up_swiglu (lut_matvec.metal:2152-2233): y = half(silu(gate) * up), fp32 gate / up. */
SMELT_CUDA_API smelt_status smelt_cuda_affine_gate_up_swiglu(smelt_cuda_ctx* ctx, const void* gw_dev, const void* gs_dev,
                                                             const void* gb_dev, const void* uw_dev, const void* us_dev,
                                                             const void* ub_dev, const void* x_dev, void* y_dev,
                                                             int rows, int cols, int group, int batch);
/* fused_dual_affine_matvec (lut_matvec.metal:1824-1908): two same-shape matvecs sharing x. */
SMELT_CUDA_API smelt_status smelt_cuda_affine_dual_matvec(smelt_cuda_ctx* ctx, const void* w0_dev, const void* s0_dev,
                                                          const void* b0_dev, const void* w1_dev, const void* s1_dev,
                                                          const void* b1_dev, const void* x_dev, void* y0_dev,
                                                          void* y1_dev, int rows, int cols, int group, int batch);
/* Fused forms used by the decoder builder's fused table (no single counterpart in the
 * reference; each is the composition of the reference kernels it names, with the same
 * rounding points).
 * affine_multi_matvec: rms_norm_1pw (norms.metal:9-67; skipped when norm_w_dev is NULL)
 * followed by up to three affine_matvec launches that share x (for example the Q, K and V
 * projections) in one kernel.  Needs group 64, cols a multiple of 1024, every tensor but the
 * last with rows a multiple of 16.  More than eight batch rows run as several passes over the
 * weights. */
typedef struct {
    const void* w_dev;
    const void* scales_dev;
    const void* biases_dev;
    void* y_dev; /* [batch, rows] */
    int32_t rows;
} smelt_affine_tensor;
SMELT_CUDA_API smelt_status smelt_cuda_affine_multi_matvec(smelt_cuda_ctx* ctx, const smelt_affine_tensor* tensors, int n_tensors,
                                                           const void* x_dev, const void* norm_w_dev, float eps, int cols,
                                                           int group, int batch);
/* rms_norm_1pw followed by fused_affine_gate_up_swiglu in one kernel. */
SMELT_CUDA_API smelt_status smelt_cuda_rmsnorm_affine_gate_up_swiglu(smelt_cuda_ctx* ctx, const void* gw_dev, const void* gs_dev,
                                                                     const void* gb_dev, const void* uw_dev, const void* us_dev,
                                                                     const void* ub_dev, const void* x_dev, const void* norm_w_dev,
                                                                     float eps, void* y_dev, int rows, int cols, int group, int batch);
/* apply_rope on Q + rope_kv_cache_update on K + kv_cache_update on V (attention.metal:48-209)
 * in one kernel; analytic trig, ropeDim == headDim, layout 0 (adjacent) or 1 (split-half). */
SMELT_CUDA_API smelt_status smelt_cuda_rope_qkv_append(smelt_cuda_ctx* ctx, void* q_dev, const void* k_new_dev, const void* v_new_dev,
                                                       void* k_cache_dev, void* v_cache_dev, uint32_t capacity, int head_dim,
                                                       int n_q, int n_kv, int layout, uint32_t position, float base_log2, int batch,
                                                       size_t kv_seq_stride);

/* Whole-tensor dequant probe: out_f32[rows*cols] and/or out_f16 (either may be NULL) —
 * SmeltAffineU4.dequantizeRow (SmeltAffineU4.swift:141-161), bit-exact. */
SMELT_CUDA_API smelt_status smelt_cuda_affine_dequantize(smelt_cuda_ctx* ctx, const void* w_dev, const void* scales_dev,
                                                         const void* biases_dev, void* out_f32_dev, void* out_f16_dev,
                                                         int rows, int cols, int group);
/* fp16_matvec (lut_matvec.metal:799-834): dense fp16 [rows, cols], clamp to +-65504. */
SMELT_CUDA_API smelt_status smelt_cuda_fp16_matvec(smelt_cuda_ctx* ctx, const void* w_dev, const void* x_dev, void* y_dev,
                                                   int rows, int cols, int batch);

/* signed_binary_matvec_g128_rows8 / signed_ternary_matvec_g128_rows8
 * (Resources/Shaders/signed_quant.metal:81-138, :288-332); format 1 = binary1, 2 = ternary2. */
SMELT_CUDA_API smelt_status smelt_cuda_signed_matvec(smelt_cuda_ctx* ctx, int format, const void* codes_dev,
                                                     const void* scales_dev, const void* x_dev, void* y_dev, int rows,
                                                     int cols, int batch);
/* signed_*_matvec_add (signed_quant.metal:223-286). */
SMELT_CUDA_API smelt_status smelt_cuda_signed_matvec_add(smelt_cuda_ctx* ctx, int format, const void* codes_dev,
                                                         const void* scales_dev, const void* x_dev,
                                                         const void* residual_dev, void* y_dev, int rows, int cols,
                                                         int batch);
/* signed_*_gate_up_swiglu (signed_quant.metal:140-221): gate and up rounded to fp16, staged-fp16 SwiGLU. */
SMELT_CUDA_API smelt_status smelt_cuda_signed_gate_up_swiglu(smelt_cuda_ctx* ctx, int format, const void* gc_dev,
                                                             const void* gs_dev, const void* uc_dev, const void* us_dev,
                                                             const void* x_dev, void* y_dev, int rows, int cols,
                                                             int batch);
/* SmeltSignedQuantCodec.dequantizeRow (SmeltSignedQuantCodec.swift:219-257) for whole tensors;
 * *out_invalid = 1 when a ternary code 3 is present (the codec's invalidCode error). */
SMELT_CUDA_API smelt_status smelt_cuda_signed_dequantize(smelt_cuda_ctx* ctx, int format, const void* codes_dev,
                                                         const void* scales_dev, void* out_f32_dev, int rows, int cols,
                                                         int* out_invalid);

/* attention_decode (Resources/Shaders/attention.metal:217-314) and its specialisations:
 * q, out fp16 [batch, n_q, head_dim] (may alias); caches fp16 [n_kv, capacity, head_dim] per
 * sequence, kv_seq_stride elements apart; keys [seqStart, seq_len) with seqStart from the
 * sliding window (0 = full causal). */
SMELT_CUDA_API smelt_status smelt_cuda_attention_decode(smelt_cuda_ctx* ctx, const void* q_dev, const void* k_cache_dev,
                                                        const void* v_cache_dev, void* out_dev, int n_q, int n_kv,
                                                        int head_dim, uint32_t capacity, uint32_t seq_len, float scale,
                                                        uint32_t sliding_window, int batch, size_t kv_seq_stride);
/* Extension (no single reference kernel): apply_rope on q, rope_kv_cache_update of the new K
 * row, kv_cache_update of the new V row (attention.metal:48-209, full-head analytic mode,
 * layout 0 adjacent / 1 split-half) and attention_decode over keys [.., position] in one
 * launch, with the rounding points of the four kernels.  q is not modified; out may alias q. */
SMELT_CUDA_API smelt_status smelt_cuda_rope_attention_decode(smelt_cuda_ctx* ctx, const void* q_dev, const void* k_new_dev,
                                                             const void* v_new_dev, void* k_cache_dev, void* v_cache_dev,
                                                             void* out_dev, int n_q, int n_kv, int head_dim, uint32_t capacity,
                                                             uint32_t position, float scale, uint32_t sliding_window, int layout,
                                                             float base_log2, int batch, size_t kv_seq_stride);
/* smelt_cuda_attention_decode with the split partials in a fixed 8 MiB device array instead of
 * the context's allocation; same arguments, same results bit for bit.  This entry point has
 * no counterpart in the reference.  It makes no device allocation on any call: the address of
 * the array is looked up once per device on the first call (make that call before any stream
 * capture begins).  Accepts batch * n_q * (head_dim + 2) <= 32768 and returns
 * SMELT_ERR_OUT_OF_RANGE beyond that.  Nothing in the array has to start at zero, so it is
 * never cleared.  All calls on one device share the array: calls that overlap in time race. */
SMELT_CUDA_API smelt_status smelt_cuda_attention_decode_static(smelt_cuda_ctx* ctx, const void* q_dev, const void* k_cache_dev,
                                                               const void* v_cache_dev, void* out_dev, int n_q, int n_kv,
                                                               int head_dim, uint32_t capacity, uint32_t seq_len, float scale,
                                                               uint32_t sliding_window, int batch, size_t kv_seq_stride);
/* kv_cache_update / rope_kv_cache_update (attention.metal:122-209). cos/sin may be NULL in analytic mode. */
SMELT_CUDA_API smelt_status smelt_cuda_kv_cache_update(smelt_cuda_ctx* ctx, void* cache_dev, const void* new_kv_dev,
                                                       uint32_t capacity, int head_dim, uint32_t position, int heads,
                                                       int batch, size_t kv_seq_stride);
SMELT_CUDA_API smelt_status smelt_cuda_rope_kv_cache_update(smelt_cuda_ctx* ctx, void* cache_dev, const void* new_kv_dev,
                                                            const void* cos_dev, const void* sin_dev, uint32_t capacity,
                                                            int head_dim, uint32_t position, int heads, int rope_dim,
                                                            int layout, float base_log2, int math_mode, int batch,
                                                            size_t kv_seq_stride);
/* apply_rope (attention.metal:48-115), in place on [batch, heads, head_dim]. */
SMELT_CUDA_API smelt_status smelt_cuda_apply_rope(smelt_cuda_ctx* ctx, void* qk_dev, const void* cos_dev, const void* sin_dev,
                                                  int head_dim, int rope_dim, int heads, int layout, uint32_t position,
                                                  float base_log2, int math_mode, int batch);

/* rms_norm_1pw (Resources/Shaders/norms.metal:9-67); weight stored as a delta from one. */
SMELT_CUDA_API smelt_status smelt_cuda_rms_norm_1pw(smelt_cuda_ctx* ctx, const void* x_dev, const void* w_dev, void* y_dev,
                                                    int dim, float eps, int batch);
/* The element-wise kernels of Resources/Shaders/activations.metal:4-210 and activations_precise.metal:22-35.
 * a / y [batch, count] fp16; b: [batch, count] (MUL, SIGMOID_MUL), rows of b_stride values (GEGLU: geglu_fused and
 * geglu_fused_strided_batched), [count] (BIAS_ADD: projection_bias_add_batched), one fp16 value on the device
 * (SCALAR_MUL_WEIGHT: scalar_mul_weight); scalar: SCALAR_MUL's factor, LOGIT_CAP's cap. */
enum {
    SMELT_EW_SILU = 0, SMELT_EW_SIGMOID = 1, SMELT_EW_SOFTPLUS = 2, SMELT_EW_COPY = 3, SMELT_EW_SCALAR_MUL = 4, SMELT_EW_LOGIT_CAP = 5,
    SMELT_EW_MUL = 6, SMELT_EW_SIGMOID_MUL = 7, SMELT_EW_GEGLU = 8, SMELT_EW_BIAS_ADD = 9, SMELT_EW_SCALAR_MUL_WEIGHT = 10
};
SMELT_CUDA_API smelt_status smelt_cuda_elementwise(smelt_cuda_ctx* ctx, int op, const void* a_dev, const void* b_dev, void* y_dev, int count,
                                                   int batch, int b_stride, float scalar);
/* The row norms of Resources/Shaders/norms.metal beyond rms_norm_1pw, each with the reduction topology and the
 * roundings of its kernel; x / y [rows, dim] fp16 (y may be x), scale_out (may be NULL) [rows] fp32.
 * topology SMELT_ROW_NORM_TILES4: rms_norm_1pw_batched (:1488-1550): four adjacent values per thread and tile of
 *   4 x threadgroup_width; SMELT_ROW_NORM_QUADS2: the d1024 / d1536 / d2048 / d2560 kernels (:72-176, :262-990): dim / 8
 *   threads, two quads each; SMELT_ROW_NORM_STRIDED: rms_norm_scale_only(_precise), the d256 kernels, l2_normalize
 *   (:177-260, :991-1090, :1155-1190, :1436-1486): thread t adds x[t], x[t + width], ...
 * value 0: the scale only; 1: half(1 + w) * half(x * rs); 2: half(x * (rs * (1 + w))) (the dXXXX kernels);
 *   3: half(x * rs * (1 + w)) (d256); 4: half(x * rs) (l2_normalize).
 * scale 0: rsqrt(mean(x^2) + eps); 1: 1 / max(sqrt(sum x^2), eps).
 * pre_dev (may be NULL): the row is half(x + pre) and, with value 0, is written to y
 *   (residual_add_rms_norm_scale_only_precise, :1059-1090); residual_dev / scalar_dev (may be NULL): the _add kernels'
 *   half(norm + residual) and rms_norm_1pw_d256_add_scalar_weight's final product. */
enum { SMELT_ROW_NORM_TILES4 = 0, SMELT_ROW_NORM_QUADS2 = 1, SMELT_ROW_NORM_STRIDED = 2 };
SMELT_CUDA_API smelt_status smelt_cuda_row_norm(smelt_cuda_ctx* ctx, const void* x_dev, const void* pre_dev, const void* w_dev,
                                                const void* residual_dev, const void* scalar_dev, void* y_dev, void* scale_out_dev,
                                                int rows, int dim, float eps, int topology, int threadgroup_width, int value, int scale);
/* gate_split (Resources/Shaders/attention_fused.metal:11-27): [heads, 2 head_dim] rows of query | gate. */
SMELT_CUDA_API smelt_status smelt_cuda_gate_split(smelt_cuda_ctx* ctx, const void* input_dev, void* query_dev, void* gate_dev, int heads,
                                                  int head_dim);
/* The per-head norms of Resources/Shaders/attention_fused.metal:38-330 with their reduction topologies: DIRECT
 * per_head_rms_norm(_batched) (four adjacent values per thread, y = w * half(x * rs)), ONE_PLUS_W per_head_rms_norm_1pw(_batched)
 * and NOSCALE per_head_rms_norm_noscale(_batched) (thread t of a threadgroup of threadgroup_width adds x[t]^2,
 * x[t + width]^2, ...; the batched forms use min(head_dim, 256)).  heads counts every head of every row; may run in place. */
enum { SMELT_HEAD_NORM_DIRECT = 0, SMELT_HEAD_NORM_ONE_PLUS_W = 1, SMELT_HEAD_NORM_NOSCALE = 2 };
SMELT_CUDA_API smelt_status smelt_cuda_head_norm(smelt_cuda_ctx* ctx, int mode, const void* x_dev, const void* w_dev, void* y_dev, int heads,
                                                 int head_dim, float eps, int threadgroup_width);
/* per_head_rms_norm (Resources/Shaders/attention_fused.metal:93-145); direct weight. */
SMELT_CUDA_API smelt_status smelt_cuda_per_head_rms_norm(smelt_cuda_ctx* ctx, const void* x_dev, const void* w_dev,
                                                         void* y_dev, int heads, int head_dim, float eps);
/* elementwise_add (Resources/Shaders/activations.metal:56-66). */
SMELT_CUDA_API smelt_status smelt_cuda_elementwise_add(smelt_cuda_ctx* ctx, const void* a_dev, const void* b_dev,
                                                       void* y_dev, size_t count);
/* swiglu_fused (Resources/Shaders/activations_precise.metal:9-22). */
SMELT_CUDA_API smelt_status smelt_cuda_swiglu_fused(smelt_cuda_ctx* ctx, const void* gate_dev, const void* up_dev,
                                                    void* y_dev, size_t count);
/* embedding_gather / affine_embedding_gather (lut_matvec.metal:951-962, :994-1025); token ids int32 on device. */
SMELT_CUDA_API smelt_status smelt_cuda_embedding_gather(smelt_cuda_ctx* ctx, const void* table_dev, const void* token_dev,
                                                        void* y_dev, int hidden, int batch);
SMELT_CUDA_API smelt_status smelt_cuda_affine_embedding_gather(smelt_cuda_ctx* ctx, const void* w_dev, const void* scales_dev,
                                                               const void* biases_dev, const void* token_dev,
                                                               void* y_dev, int cols, int group);
/* argmax_fp16_partials + argmax_key_reduce (lut_matvec.metal:8901-8966): lowest index on ties,
 * -0 == +0.  out_dev receives `batch` int32 ids. */
SMELT_CUDA_API smelt_status smelt_cuda_argmax_f16(smelt_cuda_ctx* ctx, const void* logits_dev, void* out_dev, int vocab,
                                                  int batch);

/* ── prefill ─────────────────────────────────────────────────────────────────
 * A chunk of prompt positions at once.  rope_kv_prefill = rope_and_kv_cache_prefill
 * (Resources/Shaders/prefill_rope_kv.metal:64-187): RoPE in place on q [n_pos, q_heads, head_dim]
 * and k [n_pos, kv_heads, head_dim] at positions start_pos + t (tables [maxSeq, rope_dim] when
 * math_mode == 0, analytic from base_log2 when 1; layout 0 adjacent pairs, 1 split-half,
 * 2 proportional split-half), then the rotated keys and v written to cache rows start_pos + t of
 * [kv_heads, capacity, head_dim].  attention_prefill = attention_prefill
 * (Resources/Shaders/prefill_attention.metal:14-413): position t attends causally to keys
 * [seqStart, start_pos + t] (seqStart from sliding_window, 0 = full), out [n_pos, n_q, head_dim]. */
SMELT_CUDA_API smelt_status smelt_cuda_rope_kv_prefill(smelt_cuda_ctx* ctx, void* q_dev, void* k_dev, const void* v_dev,
                                                       const void* cos_dev, const void* sin_dev, void* k_cache_dev,
                                                       void* v_cache_dev, int head_dim, int rope_dim, int q_heads, int kv_heads,
                                                       uint32_t n_pos, uint32_t start_pos, uint32_t capacity, int layout,
                                                       float base_log2, int math_mode);
SMELT_CUDA_API smelt_status smelt_cuda_attention_prefill(smelt_cuda_ctx* ctx, const void* q_dev, const void* k_cache_dev,
                                                         const void* v_cache_dev, void* out_dev, int n_q, int n_kv, int head_dim,
                                                         uint32_t n_pos, uint32_t start_pos, uint32_t capacity, float scale,
                                                         uint32_t sliding_window);
/* Prompt tokens [start_pos, start_pos + n_tokens) of one sequence through the decoder that
 * smelt_cuda_build_decoder was given (same descriptor and layer references, batch 1, one GPU),
 * `chunk` positions at a time (0 = 512): batched projections (tensor-memory QMM from 17 rows),
 * rope_kv_prefill, attention_prefill; LM head and argmax for the last position only.  Leaves
 * the KV caches filled, the last logits in the logits slot and *out_token (optional) = the
 * argmax after the last prompt token, so decoding continues with smelt_cuda_graph_seed /
 * smelt_cuda_decode_step at position start_pos + n_tokens.  The reference decodes a prompt
 * token by token when a package has no prefill table (Sources/SmeltRuntime/SmeltModel.swift
 * :619-631); this is the batched alternative, same arithmetic per position. */
SMELT_CUDA_API smelt_status smelt_cuda_prefill(smelt_cuda_ctx* ctx, const smelt_decoder_desc* desc, const smelt_layer_ref* layers,
                                               const int32_t* tokens, int n_tokens, int32_t start_pos, int chunk,
                                               int32_t* out_token);

/* ── signed activation bit-planes (the Bonsai low-bit path) ──────────────────
 * Producers (Resources/Shaders/signed_quant.metal:751-932): per group of 128 activations one fp16
 * scale and a symmetric integer of n_planes bits as magnitude planes + a sign plane:
 * planes uint32 [batch, cols/128, n_planes, 4], scales fp16 [batch, cols/128].  up_or_null != null
 * (n_planes 5 only) is swiglu_signed_activation_bitplanes_i5_g128: x is the gate, the view is taken
 * of the staged fp16 SwiGLU.  Consumers (:1300-1712, :1732-1822, :2054-2101): packed binary
 * (format 1) or ternary (format 2) weights times the planes by popcount, exact integer dot per
 * group scaled by activation scale and weight scale; mode 0 y = half(acc), 1 y = half(half(acc)
 * + residual), 2 y = staged SwiGLU of the gate (codes) and up (codes2) results. */
SMELT_CUDA_API smelt_status smelt_cuda_signed_activation_bitplanes(smelt_cuda_ctx* ctx, const void* x_dev, const void* up_or_null_dev,
                                                                   void* planes_dev, void* scales_dev, int cols, int n_planes,
                                                                   int batch);
/* Producers with another kernel's arithmetic in front (Resources/Shaders/signed_quant.metal:985-1298):
 * the fp16 values the staged kernel would have written, then the same view.
 *   SMELT_BITPLANE_FRONT_SIGMOID_MUL      sigmoid_mul_signed_activation_bitplanes_i6_g128: a * sigmoid(b); n_planes 6
 *   SMELT_BITPLANE_FRONT_NORM_SCALE       norm_scale_signed_activation_bitplanes_i{2..6}_g128: a = x, c = norm weight,
 *                                         norm_scale_dev = one float, the row's rsqrt(mean(x^2) + eps) from an earlier dispatch
 *   SMELT_BITPLANE_FRONT_GATED_NORM_D128  rms_norm_gated_d128_signed_activation_bitplanes_i6_g128: a = x, b = gate [cols],
 *                                         c = weight [128]; cols = heads * 128; a threadgroup width of 32 selects
 *                                         rms_norm_gated_d128's arithmetic, any other width rms_norm_gated's */
enum { SMELT_BITPLANE_FRONT_SIGMOID_MUL = 2, SMELT_BITPLANE_FRONT_NORM_SCALE = 3, SMELT_BITPLANE_FRONT_GATED_NORM_D128 = 4 };
SMELT_CUDA_API smelt_status smelt_cuda_fused_activation_bitplanes(smelt_cuda_ctx* ctx, int front, const void* a_dev, const void* b_dev,
                                                                  const void* c_dev, const void* norm_scale_dev, void* planes_dev,
                                                                  void* scales_dev, int cols, int n_planes, float eps,
                                                                  int threadgroup_width);
/* signed_binary_embedding_gather_g128 / signed_ternary_embedding_gather_g128
 * (Resources/Shaders/signed_quant.metal:690-745): out [batch, hidden] = sem(code) * scale of rows token_ids[b];
 * format 1 binary, 2 ternary. */
SMELT_CUDA_API smelt_status smelt_cuda_signed_embedding_gather(smelt_cuda_ctx* ctx, int format, const void* codes_dev,
                                                               const void* scales_dev, const void* token_ids_dev, void* out_dev,
                                                               int hidden, int batch);
SMELT_CUDA_API smelt_status smelt_cuda_signed_bitplane_matvec(smelt_cuda_ctx* ctx, int format, int mode, const void* codes_dev,
                                                              const void* weight_scales_dev, const void* codes2_dev,
                                                              const void* weight_scales2_dev, const void* planes_dev,
                                                              const void* act_scales_dev, const void* residual_dev, void* out_dev,
                                                              int rows, int cols, int n_planes, int batch);

/* ── DeltaNet decode step (hybrid linear-attention layers) ───────────────────
 * The four kernels between a DeltaNet layer's input projections and its output projection
 * (Sources/SmeltCompiler/DeltaNetPlugin.swift:196-318), also accepted as records under the
 * reference's pipeline names with its bindings.
 * conv1d_update_silu (Resources/Shaders/conv1d.metal:271-331): state [C, K] shifts left by one,
 *   takes new_val [C]; out [C] = staged-fp16 SiLU of the K-tap dot product with weight [C, K].
 * rms_scale_qk (Resources/Shaders/norms.metal:1380-1431): in place on the qk_heads Q heads and
 *   qk_heads K heads at the front of each qkv row: RMS normalisation times 1/head_dim (Q) or
 *   rsqrt(head_dim) (K).
 * deltanet_recurrence_decode (Resources/Shaders/recurrence.metal:511-588 and the d128
 *   specialisations :590-836): per value head, state [Dv, Dk] fp16 decays, takes the rank-one
 *   update k x (v - state.k) * beta and is read out with q; state in place, out [Hv, D].
 * rms_norm_gated (Resources/Shaders/norms.metal:1093-1143): per head RMS norm times weight [D]
 *   times silu(gate). */
SMELT_CUDA_API smelt_status smelt_cuda_conv1d_update_silu(smelt_cuda_ctx* ctx, void* state_dev, const void* new_val_dev,
                                                          const void* weight_dev, void* out_dev, int channels, int kernel_size);
SMELT_CUDA_API smelt_status smelt_cuda_rms_scale_qk(smelt_cuda_ctx* ctx, void* qkv_dev, int head_dim, float eps, int qkv_dim,
                                                    int qk_heads, int batch);
SMELT_CUDA_API smelt_status smelt_cuda_deltanet_recurrence_decode(smelt_cuda_ctx* ctx, void* state_dev, const void* qkv_dev,
                                                                  const void* b_proj_dev, const void* a_proj_dev,
                                                                  const void* a_log_dev, const void* dt_bias_dev, void* out_dev,
                                                                  int head_dim, int value_heads, int qk_heads);
SMELT_CUDA_API smelt_status smelt_cuda_rms_norm_gated(smelt_cuda_ctx* ctx, const void* input_dev, const void* gate_dev,
                                                      const void* weight_dev, void* out_dev, int head_dim, float eps, int heads);
/* rms_norm_gated as a threadgroup of threadgroup_width threads sums it (the width of the record that dispatches it:
 * 32 or 128 in the reference's tables), or, with precise_d128 != 0, rms_norm_gated_d128 / rms_norm_gated_d128_batched
 * (Resources/Shaders/norms_gated_precise.metal:7-87): the norm materialised in fp16 before the fp32 gate. */
SMELT_CUDA_API smelt_status smelt_cuda_rms_norm_gated_ex(smelt_cuda_ctx* ctx, const void* input_dev, const void* gate_dev,
                                                         const void* weight_dev, void* out_dev, int head_dim, float eps, int heads,
                                                         int threadgroup_width, int precise_d128);
/* Prompt-chunk forms (the DeltaNet layers of a prefill table).
 * conv1d_update_silu_prefill (Resources/Shaders/conv1d.metal:129-268: conv1d_update_silu_prefill,
 *   conv1d_update_silu_c6144_k4_prefill, conv1d_update_silu_prefill_checkpoint): qkv [seq_len,
 *   channels] is convolved and activated in place, position after position; state [channels,
 *   kernel_size] is written once at the end.  history_dev (may be NULL) [seq_len + 1, channels,
 *   kernel_size] receives the entry state and the state after every position.
 * deltanet_recurrence_prefill (Resources/Shaders/prefill_recurrence.metal:290-673:
 *   deltanet_recurrence_mlx_prefill and its d128 specialisations): qkv [seq_len, (2 qk_heads +
 *   value_heads) head_dim], b_proj / a_proj [seq_len, value_heads], out [seq_len, value_heads,
 *   head_dim]; the recurrent rows stay in fp32 across the chunk and are rounded to fp16 once, at
 *   the end, as the reference's kernels do.  With history_dev != NULL it is
 *   deltanet_recurrence_mlx_prefill_checkpoint (:675-775): history [seq_len + 1, value_heads,
 *   head_dim, head_dim] receives the entry state and the fp16 state after every position, and the
 *   rows continue from those rounded values, which makes the chunk equal to seq_len decode steps. */
SMELT_CUDA_API smelt_status smelt_cuda_conv1d_update_silu_prefill(smelt_cuda_ctx* ctx, void* state_dev, void* qkv_dev,
                                                                  const void* weight_dev, int seq_len, int channels,
                                                                  int kernel_size, void* history_dev);
SMELT_CUDA_API smelt_status smelt_cuda_deltanet_recurrence_prefill(smelt_cuda_ctx* ctx, void* state_dev, const void* qkv_dev,
                                                                   const void* b_proj_dev, const void* a_proj_dev,
                                                                   const void* a_log_dev, const void* dt_bias_dev, void* out_dev,
                                                                   int head_dim, int value_heads, int qk_heads, int seq_len,
                                                                   void* history_dev);

/* ── prompt-state snapshots ──────────────────────────────────────────────────
 * SmeltRuntime.captureDevicePromptSnapshot / restoreDevicePromptSnapshot
 * (Sources/SmeltRuntime/SmeltRuntime.swift:1385-1553) and the host form with a partial restore,
 * capturePromptSnapshot / restorePromptSnapshot(_:length:) (:1254-1383).  A KV-cache slot is laid
 * out [rows, capacity, head_dim] fp16 (rows = KV heads x sequences): the snapshot keeps the first
 * captured_length positions of every row compactly in a private device buffer; state slots
 * (recurrent / convolutional state) are copied whole.  Restore writes the first
 * min(length, captured, destination capacity) positions of every row at the destination's own
 * stride, derived from the slot's current size as the reference derives it, so the cache may have
 * been grown in between (grow it first, smelt_cuda_resize_kv_slot, when the whole prefix is
 * wanted).  length < captured_length is refused (SMELT_ERR_UNSUPPORTED) when the snapshot holds
 * state slots, which have no positions to rewind to (:1338-1345); length > captured_length is
 * SMELT_ERR_OUT_OF_RANGE (:1333-1337).  Slots that do not exist are skipped on both sides.  The
 * caller seeds position and token afterwards (smelt_cuda_graph_seed / decode_step) from
 * prompt_length / next_token, which the snapshot only carries. */
typedef struct smelt_cuda_snapshot smelt_cuda_snapshot;
typedef struct {
    int32_t slot;
    int32_t rows;      /* KV heads x sequences */
    int32_t head_dim;  /* a multiple of 8 */
} smelt_cuda_kv_slot;
typedef struct {
    uint32_t captured_length, prompt_length;
    int32_t next_token;
    uint32_t n_slots;
    uint64_t byte_count;  /* payload bytes held (SmeltPromptSnapshot.byteCount) */
    uint64_t blob_bytes;  /* size smelt_cuda_snapshot_export needs */
} smelt_cuda_snapshot_info_t;
SMELT_CUDA_API smelt_status smelt_cuda_snapshot_capture(smelt_cuda_ctx* ctx, const smelt_cuda_kv_slot* kv_slots, int n_kv,
                                                        const int32_t* state_slots, int n_state, uint32_t captured_length,
                                                        uint32_t prompt_length, int32_t next_token,
                                                        smelt_cuda_snapshot** out);
SMELT_CUDA_API smelt_status smelt_cuda_snapshot_restore(smelt_cuda_ctx* ctx, const smelt_cuda_snapshot* snap, uint32_t length);
SMELT_CUDA_API smelt_status smelt_cuda_snapshot_info(const smelt_cuda_snapshot* snap, smelt_cuda_snapshot_info_t* out);
/* Host form (the serialisable SmeltPromptSnapshot): a self-describing blob of this library's own
 * layout (header, one record per slot, then the payloads), importable on any context. */
SMELT_CUDA_API smelt_status smelt_cuda_snapshot_export(smelt_cuda_ctx* ctx, const smelt_cuda_snapshot* snap, void* dst, size_t dst_bytes);
SMELT_CUDA_API smelt_status smelt_cuda_snapshot_import(smelt_cuda_ctx* ctx, const void* src, size_t src_bytes, smelt_cuda_snapshot** out);
SMELT_CUDA_API void smelt_cuda_snapshot_destroy(smelt_cuda_snapshot* snap);

#ifdef __cplusplus
}
#endif
#endif /* SMELT_CUDA_H */
