// .smeltpkg reader: the part of SmeltRuntime.init that stands between a package directory and
// the first decoded token (Sources/SmeltRuntime/SmeltRuntime.swift:668-998): manifest.json
// (Sources/SmeltSchema/SmeltManifest.swift:26-98; slot layout :806-817; weight entries
// :1649-1725; buffer slots :1739-1768), weights.bin into the weights slot, one zero-filled
// buffer per manifest slot with the KV caches sized for the requested context
// (contextScopedSize, SmeltRuntime.swift:6891-6913), the pipelines the decode table names
// resolved by name (:6229-6263, unknown names are an error), dispatches.bin as an array of
// 360-byte records whose size must be a multiple of the record stride (:6322-6350), and the
// runtime configuration (Sources/SmeltSchema/SmeltRuntimeConfig.swift:104-150; argmax result
// in fixed slot 17, double buffer hiddenA / hiddenB in slots 0 / 1).
// Prefill tables, the metallib, checksums and prepared-prefix snapshots are outside the decode path.
#include <sys/stat.h>

#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "runtime.h"

using namespace smelt;

namespace {

// ── a small JSON reader (objects, arrays, strings, numbers, true / false / null) ──
struct JVal {
    enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
    bool b = false;
    double num = 0;
    std::string str;
    std::vector<JVal> arr;
    std::vector<std::pair<std::string, JVal>> obj;
    const JVal* get(const char* key) const {
        if (kind != Obj) return nullptr;
        for (auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool is_num() const { return kind == Num; }
};

struct JParser {
    const char* p;
    const char* end;
    std::string err;
    int depth = 0;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool fail(const char* what) { if (err.empty()) err = std::string(what) + " at byte " + std::to_string(p - start); return false; }
    const char* start;
    bool parse_string(std::string& out) {
        if (p >= end || *p != '"') return fail("expected a string");
        ++p;
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) return fail("unterminated escape");
                switch (*p) {
                    case 'n': out += '\n'; break; case 't': out += '\t'; break; case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break; case 'f': out += '\f'; break;
                    case 'u': {
                        if (end - p < 5) return fail("short \\u escape");
                        unsigned cp = 0;
                        for (int i = 1; i <= 4; ++i) {
                            const char c = p[i];
                            cp = cp * 16 + (c >= '0' && c <= '9' ? c - '0' : (c >= 'a' && c <= 'f' ? c - 'a' + 10 : (c >= 'A' && c <= 'F' ? c - 'A' + 10 : 0)));
                        }
                        p += 4;
                        if (cp < 0x80) out += (char)cp;
                        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
                        else { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
                        break;
                    }
                    default: out += *p;
                }
                ++p;
            } else {
                out += *p++;
            }
        }
        if (p >= end) return fail("unterminated string");
        ++p;
        return true;
    }
    bool parse(JVal& v) {
        if (++depth > 64) return fail("nesting too deep");
        ws();
        if (p >= end) return fail("unexpected end");
        bool ok = true;
        if (*p == '{') {
            v.kind = JVal::Obj;
            ++p; ws();
            if (p < end && *p == '}') { ++p; --depth; return true; }
            for (;;) {
                ws();
                std::string key;
                if (!parse_string(key)) return false;
                ws();
                if (p >= end || *p != ':') return fail("expected ':'");
                ++p;
                v.obj.emplace_back(key, JVal());
                if (!parse(v.obj.back().second)) return false;
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == '}') { ++p; break; }
                return fail("expected ',' or '}'");
            }
        } else if (*p == '[') {
            v.kind = JVal::Arr;
            ++p; ws();
            if (p < end && *p == ']') { ++p; --depth; return true; }
            for (;;) {
                v.arr.emplace_back();
                if (!parse(v.arr.back())) return false;
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == ']') { ++p; break; }
                return fail("expected ',' or ']'");
            }
        } else if (*p == '"') {
            v.kind = JVal::Str;
            ok = parse_string(v.str);
        } else if (end - p >= 4 && !strncmp(p, "true", 4)) { v.kind = JVal::Bool; v.b = true; p += 4; }
        else if (end - p >= 5 && !strncmp(p, "false", 5)) { v.kind = JVal::Bool; v.b = false; p += 5; }
        else if (end - p >= 4 && !strncmp(p, "null", 4)) { v.kind = JVal::Null; p += 4; }
        else {
            char* e = nullptr;
            std::string tmp(p, (size_t)std::min<ptrdiff_t>(end - p, 64));
            v.num = strtod(tmp.c_str(), &e);
            if (e == tmp.c_str()) return fail("unexpected character");
            v.kind = JVal::Num;
            p += e - tmp.c_str();
        }
        --depth;
        return ok;
    }
};

bool read_file(const std::string& path, std::vector<uint8_t>& out) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return false;
    fseek(f, 0, SEEK_END);
    const long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    out.resize(n > 0 ? (size_t)n : 0);
    const size_t got = out.empty() ? 0 : fread(out.data(), 1, out.size(), f);
    fclose(f);
    return got == out.size();
}

bool file_size(const std::string& path, uint64_t* bytes) {
    struct stat st;
    if (stat(path.c_str(), &st) != 0) return false;
    *bytes = (uint64_t)st.st_size;
    return true;
}

struct SlotSpec {
    int index = -1;
    std::string name, dtype;
    uint64_t size_bytes = 0;
    std::vector<int64_t> shape;
};

struct Package {
    std::vector<smelt_dispatch_record> prefill_table;   // prefill_dispatches.bin, when present and runnable
    std::vector<int> prefill_pipelines;                 // manifest indices its records name
    std::string prefill_problem;                        // why the prompt-chunk table is not available (empty = it is)
    smelt_status prefill_status = SMELT_ERR_UNSUPPORTED;
    std::vector<std::string> pipelines;
    std::vector<SlotSpec> slots;
    int token_id_slot = -1, position_slot = -1, weights_slot = -1, key_base = -1, val_base = -1;
    uint32_t vocab = 0, hidden = 0, layers = 0;
    uint64_t weights_total = 0, weights_file = 0;
    uint32_t n_weight_entries = 0;
    std::vector<smelt_dispatch_record> table;
    std::vector<int> used_pipelines;
};

bool get_int(const JVal* obj, const char* key, int64_t* out) {
    const JVal* v = obj ? obj->get(key) : nullptr;
    if (!v || !v->is_num()) return false;
    *out = (int64_t)v->num;
    return true;
}

int dtype_bytes(const std::string& d) {
    if (d == "fp16" || d == "float16" || d == "bf16") return 2;
    if (d == "fp32" || d == "float32" || d == "int32") return 4;
    return 1;
}

bool is_kv_slot(const SlotSpec& s) { return s.name.rfind("keyCache_", 0) == 0 || s.name.rfind("valCache_", 0) == 0; }

// Parses and validates the host-visible part of a package.  err receives the first problem.
smelt_status load_package(const std::string& dir, Package& pk, std::string& err) {
    std::vector<uint8_t> text;
    if (!read_file(dir + "/manifest.json", text)) { err = "cannot read " + dir + "/manifest.json"; return SMELT_ERR_BAD_ARGUMENT; }
    JVal root;
    JParser jp{(const char*)text.data(), (const char*)text.data() + text.size()};
    jp.start = jp.p;
    if (!jp.parse(root) || root.kind != JVal::Obj) { err = "manifest.json: " + (jp.err.empty() ? std::string("not a JSON object") : jp.err); return SMELT_ERR_BAD_ARGUMENT; }

    const JVal* pipes = root.get("pipelines");
    if (!pipes || pipes->kind != JVal::Arr) { err = "manifest.json: 'pipelines' is missing"; return SMELT_ERR_BAD_ARGUMENT; }
    for (auto& p : pipes->arr) {
        if (p.kind != JVal::Str) { err = "manifest.json: a pipeline entry is not a string"; return SMELT_ERR_BAD_ARGUMENT; }
        pk.pipelines.push_back(p.str);
    }
    const JVal* layout = root.get("slotLayout");
    int64_t v = 0;
    if (!get_int(layout, "tokenIdSlot", &v)) { err = "manifest.json: slotLayout.tokenIdSlot is missing"; return SMELT_ERR_BAD_ARGUMENT; }
    pk.token_id_slot = (int)v;
    if (!get_int(layout, "positionSlot", &v)) { err = "manifest.json: slotLayout.positionSlot is missing"; return SMELT_ERR_BAD_ARGUMENT; }
    pk.position_slot = (int)v;
    if (!get_int(layout, "weightsSlot", &v)) { err = "manifest.json: slotLayout.weightsSlot is missing"; return SMELT_ERR_BAD_ARGUMENT; }
    pk.weights_slot = (int)v;
    if (get_int(layout, "keyCacheBaseSlot", &v)) pk.key_base = (int)v;
    if (get_int(layout, "valCacheBaseSlot", &v)) pk.val_base = (int)v;
    const JVal* config = root.get("config");
    if (!get_int(config, "vocabSize", &v) || v <= 0) { err = "manifest.json: config.vocabSize is missing"; return SMELT_ERR_BAD_ARGUMENT; }
    pk.vocab = (uint32_t)v;
    if (get_int(config, "hiddenSize", &v)) pk.hidden = (uint32_t)v;
    if (get_int(config, "numLayers", &v)) pk.layers = (uint32_t)v;

    const JVal* buffers = root.get("buffers");
    const JVal* slots = buffers ? buffers->get("slots") : nullptr;
    if (!slots || slots->kind != JVal::Arr) { err = "manifest.json: buffers.slots is missing"; return SMELT_ERR_BAD_ARGUMENT; }
    for (auto& s : slots->arr) {
        SlotSpec sp;
        int64_t idx = -1, bytes = 0;
        if (!get_int(&s, "index", &idx) || !get_int(&s, "size_bytes", &bytes) || idx < 0 || idx >= 256 || bytes < 0) {
            err = "manifest.json: a buffer slot lacks index / size_bytes, or its index is outside 0..255"; return SMELT_ERR_BAD_ARGUMENT;
        }
        sp.index = (int)idx; sp.size_bytes = (uint64_t)bytes;
        if (const JVal* n = s.get("name")) sp.name = n->str;
        if (const JVal* d = s.get("dtype")) sp.dtype = d->str;
        if (const JVal* sh = s.get("shape"))
            for (auto& e : sh->arr) sp.shape.push_back((int64_t)e.num);
        pk.slots.push_back(sp);
    }

    // weights: every entry must lie inside weights.bin (bindBuffer's bound, SmeltRuntime.swift:3153-3169)
    const JVal* weights = root.get("weights");
    if (!get_int(weights, "total_bytes", &v) || v < 0) { err = "manifest.json: weights.total_bytes is missing"; return SMELT_ERR_BAD_ARGUMENT; }
    pk.weights_total = (uint64_t)v;
    if (!file_size(dir + "/weights.bin", &pk.weights_file)) { err = "cannot read " + dir + "/weights.bin"; return SMELT_ERR_BAD_ARGUMENT; }
    if (pk.weights_file < pk.weights_total) {
        err = "weights.bin holds " + std::to_string(pk.weights_file) + " bytes, the manifest declares " + std::to_string(pk.weights_total);
        return SMELT_ERR_OUT_OF_RANGE;
    }
    if (const JVal* entries = weights->get("entries")) {
        for (auto& e : entries->arr) {
            ++pk.n_weight_entries;
            static const char* const regions[][2] = {{"offset", "size_bytes"}, {"scales_offset", "scales_size_bytes"}, {"biases_offset", "biases_size_bytes"}};
            for (auto& r : regions) {
                int64_t off = 0, size = 0;
                if (!get_int(&e, r[0], &off)) continue;
                get_int(&e, r[1], &size);
                if (off < 0 || size < 0 || (uint64_t)off + (uint64_t)size > pk.weights_file) {
                    const JVal* n = e.get("name");
                    err = "weight entry '" + (n ? n->str : std::string("?")) + "': " + r[0] + " " + std::to_string(off) + " + " + std::to_string(size) + " bytes lies outside weights.bin";
                    return SMELT_ERR_OUT_OF_RANGE;
                }
            }
        }
    }

    // dispatches.bin: an array of records, nothing else
    std::vector<uint8_t> raw;
    if (!read_file(dir + "/dispatches.bin", raw)) { err = "cannot read " + dir + "/dispatches.bin"; return SMELT_ERR_BAD_ARGUMENT; }
    if (raw.size() % sizeof(smelt_dispatch_record) != 0) {
        err = "dispatches.bin size " + std::to_string(raw.size()) + " is not a multiple of dispatch stride " + std::to_string(sizeof(smelt_dispatch_record));
        return SMELT_ERR_BAD_ARGUMENT;
    }
    pk.table.resize(raw.size() / sizeof(smelt_dispatch_record));
    if (!raw.empty()) memcpy(pk.table.data(), raw.data(), raw.size());
    std::vector<bool> used(pk.pipelines.size(), false);
    for (size_t i = 0; i < pk.table.size(); ++i) {
        const smelt_dispatch_record& r = pk.table[i];
        if (r.op_kind == SMELT_OP_SWAP) continue;
        if (r.op_kind != SMELT_OP_DISPATCH) { err = "dispatches.bin record " + std::to_string(i) + ": unknown op kind " + std::to_string(r.op_kind); return SMELT_ERR_BAD_ARGUMENT; }
        if (r.pipeline >= pk.pipelines.size()) {
            err = "dispatches.bin record " + std::to_string(i) + " names pipeline " + std::to_string(r.pipeline) + ", the manifest lists " + std::to_string(pk.pipelines.size());
            return SMELT_ERR_UNKNOWN_PIPELINE;
        }
        used[r.pipeline] = true;
    }
    // only the pipelines the decode table can dispatch are materialised (SmeltRuntime.swift:884-905)
    for (size_t i = 0; i < used.size(); ++i)
        if (used[i]) {
            Pipeline p;
            if (!parse_pipeline(pk.pipelines[i].c_str(), &p)) {
                err = "pipeline " + std::to_string(i) + " '" + pk.pipelines[i] + "' is used by dispatches.bin and is not an implemented kernel";
                return SMELT_ERR_UNKNOWN_PIPELINE;
            }
            pk.used_pipelines.push_back((int)i);
        }
    // prefill_dispatches.bin is optional (SmeltRuntime.swift:842-853); a table this library cannot run does not
    // stop the package from decoding
    std::vector<uint8_t> praw;
    if (!read_file(dir + "/prefill_dispatches.bin", praw)) {
        pk.prefill_problem = "the package has no prefill_dispatches.bin";
        return SMELT_OK;
    }
    if (praw.empty() || praw.size() % sizeof(smelt_dispatch_record) != 0) {
        pk.prefill_problem = "prefill_dispatches.bin size " + std::to_string(praw.size()) + " is not a positive multiple of dispatch stride " + std::to_string(sizeof(smelt_dispatch_record));
        pk.prefill_status = SMELT_ERR_BAD_ARGUMENT;
        return SMELT_OK;
    }
    std::vector<smelt_dispatch_record> pt(praw.size() / sizeof(smelt_dispatch_record));
    memcpy(pt.data(), praw.data(), praw.size());
    std::vector<bool> pused(pk.pipelines.size(), false);
    for (size_t i = 0; i < pt.size(); ++i) {
        const smelt_dispatch_record& r = pt[i];
        if (r.op_kind == SMELT_OP_SWAP) continue;
        if (r.op_kind != SMELT_OP_DISPATCH || r.pipeline >= pk.pipelines.size()) {
            pk.prefill_problem = "prefill_dispatches.bin record " + std::to_string(i) + ": unknown op kind or pipeline index";
            pk.prefill_status = SMELT_ERR_BAD_ARGUMENT;
            return SMELT_OK;
        }
        pused[r.pipeline] = true;
    }
    for (size_t i = 0; i < pused.size(); ++i)
        if (pused[i]) {
            Pipeline p;
            if (!parse_pipeline(pk.pipelines[i].c_str(), &p)) {
                pk.prefill_problem = "pipeline " + std::to_string(i) + " '" + pk.pipelines[i] + "' is used by prefill_dispatches.bin and is not an implemented kernel";
                pk.prefill_status = SMELT_ERR_UNKNOWN_PIPELINE;
                pk.prefill_pipelines.clear();
                return SMELT_OK;
            }
            pk.prefill_pipelines.push_back((int)i);
        }
    pk.prefill_table.swap(pt);
    pk.prefill_status = SMELT_OK;
    return SMELT_OK;
}

void fill_info(const Package& pk, uint32_t capacity, smelt_package_info* info) {
    if (!info) return;
    memset(info, 0, sizeof(*info));
    info->n_records = (uint32_t)pk.table.size();
    info->n_pipelines = (uint32_t)pk.pipelines.size();
    info->n_pipelines_used = (uint32_t)pk.used_pipelines.size();
    info->n_slots = (uint32_t)pk.slots.size();
    info->n_weight_entries = pk.n_weight_entries;
    info->vocab_size = pk.vocab; info->hidden_size = pk.hidden; info->num_layers = pk.layers;
    info->cache_seq_capacity = capacity;
    info->token_id_slot = pk.token_id_slot; info->position_slot = pk.position_slot; info->weights_slot = pk.weights_slot;
    info->argmax_slot = 17; info->logits_slot = 16;
    info->weights_bytes = pk.weights_file;
    info->n_prefill_records = (uint32_t)pk.prefill_table.size();
}

void copy_err(const std::string& e, char* out, size_t n) {
    if (!out || n == 0) return;
    const size_t k = e.size() < n - 1 ? e.size() : n - 1;
    memcpy(out, e.c_str(), k);
    out[k] = 0;
}

}  // namespace

struct smelt_package_state {
    std::vector<smelt_dispatch_record> table;
    std::vector<smelt_dispatch_record> prefill_table;
    std::string prefill_problem;
    smelt_status prefill_status = SMELT_ERR_UNSUPPORTED;
};

extern "C" {

smelt_status smelt_cuda_inspect_package(const char* package_dir, smelt_package_info* out_info, char* err, size_t err_bytes) {
    if (!package_dir) return SMELT_ERR_BAD_ARGUMENT;
    Package pk;
    std::string e;
    const smelt_status s = load_package(package_dir, pk, e);
    copy_err(e, err, err_bytes);
    if (!s) fill_info(pk, 0, out_info);
    return s;
}

smelt_status smelt_cuda_open_package(smelt_cuda_ctx* ctx, const char* package_dir, const smelt_package_options* options,
                                     smelt_package_info* out_info) {
    if (!ctx || !package_dir) return SMELT_ERR_BAD_ARGUMENT;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, SMELT_ERR_CUDA, "cudaSetDevice");
    Package pk;
    std::string e;
    smelt_status s = load_package(package_dir, pk, e);
    if (s) return fail(ctx, s, e);
    if (pk.weights_slot < 0 || pk.weights_slot >= (int)ctx->slots.size() || pk.token_id_slot < 0 || pk.position_slot < 0)
        return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "manifest.json: slot layout outside the slot table");
    // context capacity: as asked, else what the KV slots were compiled for
    uint32_t capacity = options ? options->context_capacity : 0;
    for (const SlotSpec& sp : pk.slots)
        if (!capacity && is_kv_slot(sp) && sp.shape.size() >= 3 && sp.shape[1] > 0) capacity = (uint32_t)sp.shape[1];
    if (!capacity) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "open_package: no context capacity given and no KV cache slot to take it from");
    // weights.bin -> the weights slot (one device allocation; record offsets index it)
    {
        std::vector<uint8_t> image;
        if (!read_file(std::string(package_dir) + "/weights.bin", image)) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "cannot read weights.bin");
        s = smelt_cuda_upload_weights(ctx, pk.weights_slot, image.data(), image.size());
        if (s) return s;
    }
    // one zero-filled buffer per slot; KV caches [heads, capacity, head_dim] scale with the context
    for (const SlotSpec& sp : pk.slots) {
        if (sp.index == pk.weights_slot) continue;
        uint64_t bytes = sp.size_bytes;
        if (is_kv_slot(sp) && sp.shape.size() >= 3) bytes = (uint64_t)sp.shape[0] * capacity * (uint64_t)sp.shape[2] * dtype_bytes(sp.dtype);
        if (bytes < 16) bytes = 16;
        s = smelt_cuda_alloc_slot(ctx, sp.index, (size_t)bytes);
        if (s) return s;
    }
    ctx->pipelines.clear();
    for (int idx : pk.used_pipelines) {
        s = smelt_cuda_register_pipeline(ctx, idx, pk.pipelines[idx].c_str());
        if (s) return s;
    }
    for (int idx : pk.prefill_pipelines) {
        s = smelt_cuda_register_pipeline(ctx, idx, pk.pipelines[idx].c_str());
        if (s) return s;
    }
    smelt_cuda_runtime_config cfg = {};
    cfg.token_id_slot = pk.token_id_slot; cfg.position_slot = pk.position_slot; cfg.weights_slot = pk.weights_slot;
    cfg.argmax_slot = 17; cfg.cur_slot = 0; cfg.alt_slot = 1;
    cfg.cache_seq_capacity = capacity;
    cfg.context_limit = options && options->context_limit ? options->context_limit : capacity;
    cfg.vocab_size = pk.vocab; cfg.batch = 1;
    s = smelt_cuda_configure(ctx, &cfg);
    if (s) return s;
    if (!ctx->package) ctx->package = new (std::nothrow) smelt_package_state();
    if (!ctx->package) return fail(ctx, SMELT_ERR_ALLOC, "open_package: out of host memory");
    ctx->package->table.swap(pk.table);
    fill_info(pk, capacity, out_info);
    ctx->package->prefill_table.swap(pk.prefill_table);
    ctx->package->prefill_problem = pk.prefill_problem;
    ctx->package->prefill_status = pk.prefill_status;
    if (out_info) out_info->n_records = (uint32_t)ctx->package->table.size();
    return SMELT_OK;
}

smelt_status smelt_cuda_package_table(smelt_cuda_ctx* ctx, const smelt_dispatch_record** out_table, size_t* out_n) {
    if (!ctx || !out_table || !out_n) return SMELT_ERR_BAD_ARGUMENT;
    if (!ctx->package) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "no package is open");
    *out_table = ctx->package->table.data();
    *out_n = ctx->package->table.size();
    return SMELT_OK;
}

smelt_status smelt_cuda_package_prefill_table(smelt_cuda_ctx* ctx, const smelt_dispatch_record** out_table, size_t* out_n) {
    if (!ctx || !out_table || !out_n) return SMELT_ERR_BAD_ARGUMENT;
    if (!ctx->package) return fail(ctx, SMELT_ERR_BAD_ARGUMENT, "no package is open");
    if (ctx->package->prefill_status != SMELT_OK) return fail(ctx, ctx->package->prefill_status, ctx->package->prefill_problem);
    *out_table = ctx->package->prefill_table.data();
    *out_n = ctx->package->prefill_table.size();
    return SMELT_OK;
}

}  // extern "C"

namespace smelt {
void package_destroy(smelt_cuda_ctx* ctx) {
    delete ctx->package;
    ctx->package = nullptr;
}
}  // namespace smelt
