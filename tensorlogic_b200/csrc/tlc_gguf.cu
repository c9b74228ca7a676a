// GGUF container reader and the name -> tensor map behind load_model /
// get_tensor.
//
// Follows the header walk of MmapGGUFLoader (src/model/formats/mmap_gguf.rs:
// 187-275, :301-379) and the name/shape conventions of GGUFLoader::load
// (src/model/formats/gguf.rs:256-464): dims of rank >= 2 tensors are reversed so
// that weights are [out, in]; tensor data starts at the aligned end of the
// header.  Two things differ from the reference on purpose, following the GGUF
// specification instead: 1-byte and 2-byte metadata values are skipped by their
// real size (the reference consumes 4 bytes for them, mmap_gguf.rs:329-336) and
// the data alignment honours the general.alignment key (the reference always
// uses 32).  Quantized tensors are uploaded verbatim; nothing is dequantized.
#include <cerrno>
#include <climits>
#include <cstdint>
#include <cstring>
#include <fstream>
#include <memory>

#include "tlc_internal.h"

struct GGUFTensor {
    std::string name;
    int32_t type;
    int64_t rows, cols;   // reversed dims: [prod(dims[1..]), dims[0]]
    int32_t n_dims;
    uint64_t offset;      // absolute file offset of the data
    uint64_t nbytes;
};

// MmapGGUFLoader (src/model/formats/mmap_gguf.rs:101-275): the parsed header
// of one file; pure host state, no device needed.
struct tlc_gguf {
    std::string path;
    uint32_t version = 0;
    uint64_t alignment = 32, data_start = 0, file_size = 0;
    std::vector<GGUFTensor> tensors;
    std::map<std::string, double> meta_num;
    std::map<std::string, std::string> meta_str;
};

struct tlc_model {
    tlc_ctx *ctx;
    std::map<std::string, tlc_qtensor *> tensors;
    std::vector<std::string> order;
    std::map<std::string, double> meta_num;       // numeric / bool metadata
    std::map<std::string, std::string> meta_str;  // string metadata
    int tp_rank = 0, tp_size = 1;
};

namespace {

struct Reader {
    std::ifstream f;
    uint64_t size = 0;
    bool ok = true;
    template <typename T>
    T get() {
        T v{};
        f.read(reinterpret_cast<char *>(&v), sizeof(T));
        if (!f) ok = false;
        return v;
    }
    std::string str() {
        uint64_t n = get<uint64_t>();
        if (!ok || n > left()) {
            ok = false;
            return {};
        }
        std::string s(n, '\0');
        f.read(&s[0], (std::streamsize)n);
        if (!f) ok = false;
        return s;
    }
    // Bytes left in the file; a length field larger than this is corrupt, whatever it multiplies to.
    uint64_t left() {
        const uint64_t p = pos();
        return p <= size ? size - p : 0;
    }
    void skip(uint64_t n) {
        if (!ok || n > left()) {
            ok = false;
            return;
        }
        f.seekg((std::streamoff)n, std::ios::cur);
        if (!f) ok = false;
    }
    uint64_t pos() {
        const std::streamoff p = f.tellg();
        return p < 0 ? UINT64_MAX : (uint64_t)p;
    }
};

// GGUF metadata value types.
enum { GT_U8, GT_I8, GT_U16, GT_I16, GT_U32, GT_I32, GT_F32, GT_BOOL, GT_STR, GT_ARR, GT_U64, GT_I64, GT_F64 };

size_t scalar_size(uint32_t t) {
    switch (t) {
        case GT_U8: case GT_I8: case GT_BOOL: return 1;
        case GT_U16: case GT_I16: return 2;
        case GT_U32: case GT_I32: case GT_F32: return 4;
        case GT_U64: case GT_I64: case GT_F64: return 8;
        default: return 0;
    }
}

bool read_scalar(Reader &r, uint32_t t, double *out) {
    switch (t) {
        case GT_U8: *out = r.get<uint8_t>(); return true;
        case GT_I8: *out = r.get<int8_t>(); return true;
        case GT_BOOL: *out = r.get<uint8_t>() != 0; return true;
        case GT_U16: *out = r.get<uint16_t>(); return true;
        case GT_I16: *out = r.get<int16_t>(); return true;
        case GT_U32: *out = r.get<uint32_t>(); return true;
        case GT_I32: *out = r.get<int32_t>(); return true;
        case GT_F32: *out = r.get<float>(); return true;
        case GT_U64: *out = (double)r.get<uint64_t>(); return true;
        case GT_I64: *out = (double)r.get<int64_t>(); return true;
        case GT_F64: *out = r.get<double>(); return true;
        default: return false;
    }
}

bool skip_value(Reader &r, uint32_t t, int depth = 0) {
    if (t == GT_STR) {
        uint64_t n = r.get<uint64_t>();
        r.skip(n);
        return r.ok;
    }
    if (t == GT_ARR) {
        if (depth > 4) return false;
        uint32_t et = r.get<uint32_t>();
        uint64_t n = r.get<uint64_t>();
        if (!r.ok) return false;
        if (size_t s = scalar_size(et)) {
            uint64_t total = 0;
            if (__builtin_mul_overflow(n, (uint64_t)s, &total)) return false;
            r.skip(total);
            return r.ok;
        }
        if (n > r.left()) return false;  // every element takes at least one byte
        for (uint64_t i = 0; i < n && r.ok; i++)
            if (!skip_value(r, et, depth + 1)) return false;
        return r.ok;
    }
    size_t s = scalar_size(t);
    if (!s) return false;
    r.skip(s);
    return r.ok;
}

struct TensorInfo {
    std::string name;
    std::vector<uint64_t> dims;  // file order (fastest first)
    uint32_t type;
    uint64_t offset;
};

// How a tensor is split across tensor-parallel ranks, by its GGUF name
// (column-parallel q/k/v/gate/up/lm_head keep whole rows, row-parallel o/down
// keep a slice of every row; embeddings and norms are replicated).
int split_for(const std::string &name) {
    auto ends = [&](const char *s) {
        size_t n = strlen(s);
        return name.size() >= n && name.compare(name.size() - n, n, s) == 0;
    };
    if (ends("attn_q.weight") || ends("attn_k.weight") || ends("attn_v.weight") || ends("ffn_gate.weight") ||
        ends("ffn_up.weight") || name == "output.weight")
        return TLC_SPLIT_ROWS;
    if (ends("attn_output.weight") || ends("ffn_down.weight")) return TLC_SPLIT_COLS;
    return TLC_SPLIT_NONE;
}

}  // namespace

extern "C" int32_t tlc_model_create(tlc_ctx *ctx, tlc_model **out) {
    TLC_REQUIRE(ctx && out, TLC_ERR_INVALID_OPERATION, "model_create: null pointer");
    *out = new tlc_model();
    (*out)->ctx = ctx;
    return TLC_OK;
}

extern "C" int32_t tlc_model_destroy(tlc_model *m) {
    if (!m) return TLC_OK;
    for (auto &kv : m->tensors) tlc_qtensor_destroy(kv.second);
    delete m;
    return TLC_OK;
}

extern "C" int32_t tlc_model_add(tlc_model *m, const char *name, tlc_qtensor *qt) {
    TLC_REQUIRE(m && name && qt, TLC_ERR_INVALID_OPERATION, "model_add: null pointer");
    auto it = m->tensors.find(name);
    if (it != m->tensors.end()) {
        tlc_qtensor_destroy(it->second);
        it->second = qt;
    } else {
        m->tensors[name] = qt;
        m->order.push_back(name);
    }
    return TLC_OK;
}

// get_tensor(model, name) (src/interpreter/builtin_model.rs:203-246): the
// returned handle stays owned by the model.
extern "C" int32_t tlc_model_get(tlc_model *m, const char *name, tlc_qtensor **out) {
    TLC_REQUIRE(m && name && out, TLC_ERR_INVALID_OPERATION, "model_get: null pointer");
    auto it = m->tensors.find(name);
    TLC_REQUIRE(it != m->tensors.end(), TLC_ERR_LOAD, "Tensor '%s' not found in model", name);
    *out = it->second;
    return TLC_OK;
}

extern "C" int32_t tlc_model_tensor_count(tlc_model *m) { return m ? (int32_t)m->order.size() : 0; }

extern "C" const char *tlc_model_tensor_name(tlc_model *m, int32_t i) {
    if (!m || i < 0 || i >= (int32_t)m->order.size()) return nullptr;
    return m->order[(size_t)i].c_str();
}

extern "C" int32_t tlc_model_meta_num(tlc_model *m, const char *key, double *out) {
    TLC_REQUIRE(m && key && out, TLC_ERR_INVALID_OPERATION, "model_meta_num: null pointer");
    auto it = m->meta_num.find(key);
    TLC_REQUIRE(it != m->meta_num.end(), TLC_ERR_LOAD, "metadata key '%s' not found", key);
    *out = it->second;
    return TLC_OK;
}

extern "C" const char *tlc_model_meta_str(tlc_model *m, const char *key) {
    if (!m || !key) return nullptr;
    auto it = m->meta_str.find(key);
    return it == m->meta_str.end() ? nullptr : it->second.c_str();
}

static int32_t parse_gguf(const char *path, tlc_gguf *g) {
    Reader r;
    r.f.open(path, std::ios::binary);
    TLC_REQUIRE(r.f.good(), TLC_ERR_LOAD, "Failed to open GGUF file '%s': %s", path, strerror(errno));
    r.f.seekg(0, std::ios::end);
    r.size = (uint64_t)r.f.tellg();
    r.f.seekg(0);
    g->path = path;
    g->file_size = r.size;

    const uint32_t magic = r.get<uint32_t>();
    TLC_REQUIRE(r.ok && magic == 0x46554747u, TLC_ERR_LOAD, "Invalid GGUF magic: 0x%08x (expected 0x46554747)", magic);
    g->version = r.get<uint32_t>();
    TLC_REQUIRE(r.ok && (g->version == 2 || g->version == 3), TLC_ERR_LOAD,
                "Unsupported GGUF version: %u (only v2 and v3 supported)", g->version);
    const uint64_t n_tensors = r.get<uint64_t>();
    const uint64_t n_kv = r.get<uint64_t>();
    TLC_REQUIRE(r.ok && n_tensors < (1u << 24) && n_kv < (1u << 24), TLC_ERR_LOAD, "GGUF header is truncated or corrupt");

    for (uint64_t i = 0; i < n_kv; i++) {
        std::string key = r.str();
        const uint32_t vt = r.get<uint32_t>();
        TLC_REQUIRE(r.ok, TLC_ERR_LOAD, "GGUF metadata is truncated (key %llu of %llu)", (unsigned long long)i,
                    (unsigned long long)n_kv);
        if (vt == GT_STR) {
            g->meta_str[key] = r.str();
        } else if (vt == GT_ARR) {
            // Arrays (tokenizer vocabularies) are not needed on this path; only the length is kept.
            const uint64_t at = r.pos();
            const uint32_t et = r.get<uint32_t>();
            const uint64_t n = r.get<uint64_t>();
            (void)et;
            g->meta_num[key + ".length"] = (double)n;
            r.f.seekg((std::streamoff)at);
            TLC_REQUIRE(skip_value(r, GT_ARR), TLC_ERR_LOAD, "GGUF metadata array '%s' is corrupt", key.c_str());
        } else {
            double v = 0;
            TLC_REQUIRE(read_scalar(r, vt, &v), TLC_ERR_LOAD, "GGUF metadata key '%s' has unknown type %u",
                        key.c_str(), vt);
            g->meta_num[key] = v;
        }
        TLC_REQUIRE(r.ok, TLC_ERR_LOAD, "GGUF metadata is truncated at key '%s'", key.c_str());
    }
    if (g->meta_num.count("general.alignment")) g->alignment = (uint64_t)g->meta_num["general.alignment"];
    TLC_REQUIRE(g->alignment >= 1 && (g->alignment & (g->alignment - 1)) == 0, TLC_ERR_LOAD,
                "bad general.alignment %llu", (unsigned long long)g->alignment);

    std::vector<TensorInfo> infos(n_tensors);
    for (auto &ti : infos) {
        ti.name = r.str();
        const uint32_t nd = r.get<uint32_t>();
        TLC_REQUIRE(r.ok && nd >= 1 && nd <= 4, TLC_ERR_LOAD, "tensor '%s' has %u dimensions", ti.name.c_str(), nd);
        ti.dims.resize(nd);
        for (auto &d : ti.dims) d = r.get<uint64_t>();
        ti.type = r.get<uint32_t>();
        ti.offset = r.get<uint64_t>();
        TLC_REQUIRE(r.ok, TLC_ERR_LOAD, "GGUF tensor table is truncated at '%s'", ti.name.c_str());
    }
    g->data_start = (r.pos() + g->alignment - 1) / g->alignment * g->alignment;

    for (const auto &ti : infos) {
        GGUFTensor t;
        t.name = ti.name;
        t.type = (int32_t)ti.type;
        t.n_dims = (int32_t)ti.dims.size();
        // Reversed dims: file order is fastest-first; [rows, cols] = [prod(dims[1..]), dims[0]].
        // The header comes from an untrusted file: every product is checked for overflow, so
        // that a wrapped size can never pass the end-of-file test below.
        uint64_t rows = 1, elems = 0;
        bool ok = ti.dims[0] >= 1 && ti.dims[0] <= (uint64_t)INT64_MAX;
        for (size_t i = 1; ok && i < ti.dims.size(); i++)
            ok = ti.dims[i] >= 1 && !__builtin_mul_overflow(rows, ti.dims[i], &rows);
        ok = ok && rows <= (uint64_t)INT64_MAX && !__builtin_mul_overflow(rows, ti.dims[0], &elems);
        TLC_REQUIRE(ok, TLC_ERR_LOAD, "tensor '%s' has a zero or overflowing shape", ti.name.c_str());
        t.cols = (int64_t)ti.dims[0];
        t.rows = (int64_t)rows;
        uint64_t units = 0, unit_bytes = 0;  // nbytes = units * unit_bytes
        if (t.type == TLC_TYPE_F32) { units = elems; unit_bytes = 4; }
        else if (t.type == TLC_TYPE_F16) { units = elems; unit_bytes = 2; }
        else if (t.type == TLC_TYPE_Q4_0 || t.type == TLC_TYPE_Q8_0) {
            TLC_REQUIRE(t.cols % 32 == 0, TLC_ERR_LOAD, "tensor '%s': %lld columns are not a multiple of 32",
                        t.name.c_str(), (long long)t.cols);
            units = elems / 32;
            unit_bytes = tlc_block_bytes(t.type);
        } else if (t.type == TLC_TYPE_Q6_K) {
            TLC_REQUIRE(t.cols % 256 == 0, TLC_ERR_LOAD, "tensor '%s': %lld columns are not a multiple of 256",
                        t.name.c_str(), (long long)t.cols);
            units = elems / 256;
            unit_bytes = 210;
        }  // else unsupported type: listed with 0 bytes, cannot be uploaded
        TLC_REQUIRE(!__builtin_mul_overflow(units, unit_bytes, &t.nbytes), TLC_ERR_LOAD,
                    "tensor '%s' has an overflowing byte size", ti.name.c_str());
        TLC_REQUIRE(!__builtin_add_overflow(g->data_start, ti.offset, &t.offset) && t.offset <= g->file_size,
                    TLC_ERR_LOAD, "tensor '%s' starts past the end of the file (offset %llu, file has %llu)",
                    ti.name.c_str(), (unsigned long long)ti.offset, (unsigned long long)g->file_size);
        TLC_REQUIRE(t.nbytes <= g->file_size - t.offset, TLC_ERR_LOAD,
                    "tensor '%s' runs past the end of the file (%llu bytes at offset %llu, file has %llu)",
                    t.name.c_str(), (unsigned long long)t.nbytes, (unsigned long long)t.offset,
                    (unsigned long long)g->file_size);
        g->tensors.push_back(std::move(t));
    }
    return TLC_OK;
}

// MmapGGUFLoader::new (src/model/formats/mmap_gguf.rs:120): parse only.
extern "C" int32_t tlc_gguf_open(const char *path, tlc_gguf **out) {
    TLC_REQUIRE(path && out, TLC_ERR_INVALID_OPERATION, "gguf_open: null pointer");
    *out = nullptr;
    std::unique_ptr<tlc_gguf> g(new tlc_gguf());
    if (int32_t rc = parse_gguf(path, g.get())) return rc;
    *out = g.release();
    return TLC_OK;
}

extern "C" int32_t tlc_gguf_close(tlc_gguf *g) {
    delete g;
    return TLC_OK;
}

extern "C" int32_t tlc_gguf_tensor_count(tlc_gguf *g) { return g ? (int32_t)g->tensors.size() : 0; }

extern "C" int32_t tlc_gguf_tensor_info(tlc_gguf *g, int32_t index, const char **name, int32_t *type, int64_t *rows,
                                        int64_t *cols, uint64_t *file_offset, uint64_t *nbytes) {
    TLC_REQUIRE(g && index >= 0 && index < (int32_t)g->tensors.size(), TLC_ERR_INDEX,
                "Index out of bounds: index %d, size %d", index, g ? (int)g->tensors.size() : 0);
    const GGUFTensor &t = g->tensors[(size_t)index];
    if (name) *name = t.name.c_str();
    if (type) *type = t.type;
    if (rows) *rows = t.rows;
    if (cols) *cols = t.cols;
    if (file_offset) *file_offset = t.offset;
    if (nbytes) *nbytes = t.nbytes;
    return TLC_OK;
}

extern "C" int32_t tlc_gguf_meta_num(tlc_gguf *g, const char *key, double *out) {
    TLC_REQUIRE(g && key && out, TLC_ERR_INVALID_OPERATION, "gguf_meta_num: null pointer");
    auto it = g->meta_num.find(key);
    TLC_REQUIRE(it != g->meta_num.end(), TLC_ERR_LOAD, "metadata key '%s' not found", key);
    *out = it->second;
    return TLC_OK;
}

extern "C" const char *tlc_gguf_meta_str(tlc_gguf *g, const char *key) {
    if (!g || !key) return nullptr;
    auto it = g->meta_str.find(key);
    return it == g->meta_str.end() ? nullptr : it->second.c_str();
}

extern "C" uint64_t tlc_gguf_data_start(tlc_gguf *g) { return g ? g->data_start : 0; }

// load_model(path) (src/interpreter/builtin_model.rs:106-131 -> Model::load,
// src/model/mod.rs:165-184 -> GGUFLoader::load, gguf.rs:256).
extern "C" int32_t tlc_model_load_gguf(tlc_ctx *ctx, const char *path, int32_t tp_rank, int32_t tp_size,
                                       tlc_model **out) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(path && out, TLC_ERR_INVALID_OPERATION, "load_gguf: null pointer");
    *out = nullptr;
    TLC_REQUIRE(tp_size >= 1 && tp_rank >= 0 && tp_rank < tp_size, TLC_ERR_INVALID_OPERATION,
                "bad tensor-parallel rank %d of %d", tp_rank, tp_size);
    tlc_gguf g;
    if (int32_t rc = parse_gguf(path, &g)) return rc;
    std::unique_ptr<tlc_model, int32_t (*)(tlc_model *)> model(new tlc_model(), tlc_model_destroy);
    model->ctx = ctx;
    model->tp_rank = tp_rank;
    model->tp_size = tp_size;
    model->meta_num = g.meta_num;
    model->meta_str = g.meta_str;
    std::ifstream f(path, std::ios::binary);
    TLC_REQUIRE(f.good(), TLC_ERR_LOAD, "Failed to open GGUF file '%s': %s", path, strerror(errno));
    std::vector<char> host;
    for (const auto &t : g.tensors) {
        TLC_REQUIRE(t.type == TLC_TYPE_F32 || t.type == TLC_TYPE_F16 || t.type == TLC_TYPE_Q4_0 ||
                        t.type == TLC_TYPE_Q8_0 || t.type == TLC_TYPE_Q6_K,
                    TLC_ERR_LOAD, "tensor '%s' has unsupported GGUF type %d (supported: F32, F16, Q4_0, Q8_0, Q6_K)",
                    t.name.c_str(), t.type);
        host.resize(t.nbytes);
        f.seekg((std::streamoff)t.offset);
        f.read(host.data(), (std::streamsize)t.nbytes);
        TLC_REQUIRE((bool)f, TLC_ERR_LOAD, "short read on tensor '%s'", t.name.c_str());
        const int split = tp_size > 1 && t.n_dims >= 2 ? split_for(t.name) : TLC_SPLIT_NONE;
        tlc_qtensor *qt = nullptr;
        if (int32_t rc = tlc_qtensor_create(ctx, t.type, t.rows, t.cols, host.data(), t.nbytes, tp_rank, tp_size, split, &qt))
            return rc;
        // The embedding gather reads f16 rows: a quantized table is dequantized once, here
        // (the reference dequantizes every tensor at load time).
        if (t.name == "token_embd.weight" && qt->type != TLC_TYPE_F16) {
            tlc_qtensor *dense = nullptr;
            if (int32_t rc = tlc_qtensor_to_f16(ctx, qt, &dense)) {
                tlc_qtensor_destroy(qt);
                return rc;
            }
            tlc_qtensor_destroy(qt);
            qt = dense;
        }
        tlc_model_add(model.get(), t.name.c_str(), qt);
    }
    *out = model.release();
    return TLC_OK;
}

// ---------------------------------------------------------------------------
// Lazy weight cache: GGUFWeightCache (src/model/gguf_weight_cache.rs:45-262,
// :418-441; builtins load_weight_cache_gguf_f16/_f32 and get_weight,
// src/interpreter/builtin_model.rs:330-414).  The file's tensor table is read
// once; a tensor is read from the file and uploaded on its first get_weight and
// then kept under an LRU policy with a capacity counted in tensors, as upstream.
// Unlike upstream the cached tensors stay quantized (Q4_0 / Q8_0 blocks) in
// device memory, and an evicted tensor is freed once the caller's work on the
// stream has been waited for.
// ---------------------------------------------------------------------------
#include <list>

struct tlc_weight_cache {
    tlc_ctx *ctx;
    tlc_gguf file;
    size_t capacity;
    std::list<std::string> lru;  // most recently used first
    std::map<std::string, std::pair<tlc_qtensor *, std::list<std::string>::iterator>> entries;
    uint64_t hits = 0, misses = 0, evictions = 0;
};

extern "C" int32_t tlc_weight_cache_open(tlc_ctx *ctx, const char *path, int64_t capacity, tlc_weight_cache **out) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(path && out, TLC_ERR_INVALID_OPERATION, "weight_cache_open: null pointer");
    *out = nullptr;
    // LruCache::new(NonZeroUsize::new(capacity).unwrap()) panics on 0 upstream
    TLC_REQUIRE(capacity >= 1, TLC_ERR_INVALID_OPERATION, "cache capacity must be at least 1 (got %lld)",
                (long long)capacity);
    std::unique_ptr<tlc_weight_cache> c(new tlc_weight_cache());
    c->ctx = ctx;
    c->capacity = (size_t)capacity;
    if (int32_t rc = parse_gguf(path, &c->file)) return rc;
    *out = c.release();
    return TLC_OK;
}

extern "C" int32_t tlc_weight_cache_clear(tlc_weight_cache *c) {
    if (!c) return TLC_OK;
    cudaSetDevice(c->ctx->device);
    cudaStreamSynchronize(c->ctx->stream);  // kernels may still read the cached weights
    for (auto &e : c->entries) tlc_qtensor_destroy(e.second.first);
    c->entries.clear();
    c->lru.clear();
    return TLC_OK;
}

extern "C" int32_t tlc_weight_cache_close(tlc_weight_cache *c) {
    if (!c) return TLC_OK;
    tlc_weight_cache_clear(c);
    delete c;
    return TLC_OK;
}

extern "C" int32_t tlc_weight_cache_contains(tlc_weight_cache *c, const char *name) {
    if (!c || !name) return 0;
    for (const auto &t : c->file.tensors)
        if (t.name == name) return 1;
    return 0;
}

// cache_stats(): (tensors held, capacity); plus hit / miss / eviction counters.
extern "C" int32_t tlc_weight_cache_stats(tlc_weight_cache *c, int64_t *len, int64_t *capacity, uint64_t *hits,
                                          uint64_t *misses, uint64_t *evictions) {
    TLC_REQUIRE(c, TLC_ERR_INVALID_OPERATION, "weight_cache_stats: null pointer");
    if (len) *len = (int64_t)c->entries.size();
    if (capacity) *capacity = (int64_t)c->capacity;
    if (hits) *hits = c->hits;
    if (misses) *misses = c->misses;
    if (evictions) *evictions = c->evictions;
    return TLC_OK;
}

// get_weight(name): the tensor stays owned by the cache and valid until it is
// evicted (capacity further get_weight calls for other names) or the cache is
// cleared / closed.
extern "C" int32_t tlc_weight_cache_get(tlc_weight_cache *c, const char *name, tlc_qtensor **out) {
    TLC_REQUIRE(c && name && out, TLC_ERR_INVALID_OPERATION, "weight_cache_get: null pointer");
    if (int32_t rc = tlc_enter(c->ctx)) return rc;
    *out = nullptr;
    auto hit = c->entries.find(name);
    if (hit != c->entries.end()) {
        c->hits++;
        c->lru.splice(c->lru.begin(), c->lru, hit->second.second);
        *out = hit->second.first;
        return TLC_OK;
    }
    const GGUFTensor *t = nullptr;
    for (const auto &cand : c->file.tensors)
        if (cand.name == name) t = &cand;
    TLC_REQUIRE(t, TLC_ERR_LOAD, "Weight not found: %s", name);
    TLC_REQUIRE(t->nbytes > 0, TLC_ERR_LOAD, "Unsupported quantization type: %d", t->type);
    c->misses++;
    std::ifstream f(c->file.path, std::ios::binary);
    TLC_REQUIRE(f.good(), TLC_ERR_LOAD, "Failed to open GGUF file '%s': %s", c->file.path.c_str(), strerror(errno));
    std::vector<char> host(t->nbytes);
    f.seekg((std::streamoff)t->offset);
    f.read(host.data(), (std::streamsize)t->nbytes);
    TLC_REQUIRE((bool)f, TLC_ERR_LOAD, "Failed to load tensor data: short read on '%s'", name);
    tlc_qtensor *qt = nullptr;
    if (int32_t rc = tlc_qtensor_create(c->ctx, t->type, t->rows, t->cols, host.data(), t->nbytes, 0, 1, TLC_SPLIT_NONE, &qt))
        return rc;
    if (c->entries.size() >= c->capacity) {
        // evict the least recently used tensor, once nothing on the stream can still read it
        cudaStreamSynchronize(c->ctx->stream);
        const std::string victim = c->lru.back();
        c->lru.pop_back();
        tlc_qtensor_destroy(c->entries[victim].first);
        c->entries.erase(victim);
        c->evictions++;
    }
    c->lru.push_front(name);
    c->entries[name] = {qt, c->lru.begin()};
    *out = qt;
    return TLC_OK;
}
