// GGUF reader (host only): maps every shard of a model file, indexes its tensors by name and keeps the first shard's
// metadata.  The counterpart of the reference's reader (engine/src/gguf.hpp:47-95, gguf.cpp): read-only, the tensor
// data stays in the mapping; the loader (model_load.cu) slices it and copies it to the GPU.
//
// The container, version 2 or 3, little endian: "GGUF", u32 version, u64 tensors, u64 keys; the keys (string key, u32
// type, value); the tensor records (string name, u32 dims, u64 extent per dim, u32 type, u64 offset into the data
// section); the data section, starting at the next multiple of general.alignment (32 when the key is absent).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "fnx_common.cuh"
#include "iq3s_grid.h"

namespace fnxb {

struct GgufType {
    int block, bytes;
};

// elements and bytes per block of the ggml tensor types (0 bytes: a type this reader cannot size)
static GgufType gguf_type(uint32_t t) {
    switch (t) {
        case 0: return {1, 4};        // F32
        case 1: return {1, 2};        // F16
        case 2: return {32, 18};      // Q4_0
        case 3: return {32, 20};      // Q4_1
        case 6: return {32, 22};      // Q5_0
        case 7: return {32, 24};      // Q5_1
        case 8: return {32, 34};      // Q8_0
        case 9: return {32, 36};      // Q8_1
        case 10: return {256, 84};    // Q2_K
        case 11: return {256, 110};   // Q3_K
        case 12: return {256, 144};   // Q4_K
        case 13: return {256, 176};   // Q5_K
        case 14: return {256, 210};   // Q6_K
        case 15: return {256, 292};   // Q8_K
        case 16: return {256, 66};    // IQ2_XXS
        case 17: return {256, 74};    // IQ2_XS
        case 18: return {256, 98};    // IQ3_XXS
        case 19: return {256, 50};    // IQ1_S
        case 20: return {32, 18};     // IQ4_NL
        case 21: return {256, 110};   // IQ3_S
        case 22: return {256, 82};    // IQ2_S
        case 23: return {256, 136};   // IQ4_XS
        case 24: return {1, 1};       // I8
        case 25: return {1, 2};       // I16
        case 26: return {1, 4};       // I32
        case 27: return {1, 8};       // I64
        case 28: return {1, 8};       // F64
        case 29: return {256, 56};    // IQ1_M
        case 30: return {1, 2};       // BF16
        default: return {1, 0};
    }
}

struct GgufTensor {
    std::string name;
    uint32_t type = 0;
    int n_dims = 0;
    int64_t ne[4] = {1, 1, 1, 1};
    const uint8_t* data = nullptr;
    size_t bytes = 0;
    int shard = 0;
    uint64_t offset = 0;   // in its shard's file
};

struct GgufMap {
    void* base = nullptr;
    size_t size = 0;
    int fd = -1;
    std::string path;
};

}  // namespace fnxb

struct fnx_gguf {
    std::vector<fnxb::GgufMap> maps;
    std::vector<fnxb::GgufTensor> tensors;
    std::map<std::string, int> by_name;
    std::map<std::string, double> nums;
    std::map<std::string, bool> num_is_int;
    std::map<std::string, std::string> strs;
    std::map<std::string, std::vector<int64_t>> int_arrays;
    std::map<std::string, uint32_t> key_types;
};

namespace fnxb {

// a bounds-checked cursor over one mapped shard
struct Cursor {
    const uint8_t* p;
    size_t n, at = 0;
    bool ok = true;
    bool take(void* dst, size_t k) {
        if (!ok || k > n - at) {
            ok = false;
            return false;
        }
        memcpy(dst, p + at, k);
        at += k;
        return true;
    }
    template <typename T>
    T get() {
        T v{};
        take(&v, sizeof(T));
        return v;
    }
    std::string str() {
        const uint64_t len = get<uint64_t>();
        if (!ok || len > n - at || len > (1u << 20)) {
            ok = false;
            return {};
        }
        std::string s((const char*) p + at, (size_t) len);
        at += (size_t) len;
        return s;
    }
    void skip(size_t k) {
        if (!ok || k > n - at) ok = false;
        else at += k;
    }
};

static size_t scalar_bytes(uint32_t vt) {
    switch (vt) {
        case 0: case 1: case 7: return 1;
        case 2: case 3: return 2;
        case 4: case 5: case 6: return 4;
        case 10: case 11: case 12: return 8;
        default: return 0;
    }
}

// one scalar of metadata type vt as a double (and whether it is an integer type)
static bool scalar_value(Cursor& c, uint32_t vt, double& v, bool& is_int) {
    is_int = true;
    switch (vt) {
        case 0: v = c.get<uint8_t>(); break;
        case 1: v = c.get<int8_t>(); break;
        case 2: v = c.get<uint16_t>(); break;
        case 3: v = c.get<int16_t>(); break;
        case 4: v = c.get<uint32_t>(); break;
        case 5: v = c.get<int32_t>(); break;
        case 6: v = c.get<float>(); is_int = false; break;
        case 7: v = c.get<uint8_t>() != 0; break;
        case 10: v = (double) c.get<uint64_t>(); break;
        case 11: v = (double) c.get<int64_t>(); break;
        case 12: v = c.get<double>(); is_int = false; break;
        default: return false;
    }
    return c.ok;
}

static int load_shard(fnx_gguf* g, const std::string& path, bool meta) {
    GgufMap m;
    m.path = path;
    m.fd = ::open(path.c_str(), O_RDONLY);
    if (m.fd < 0) return fail(FNX_E_ARG, "gguf: cannot open %s", path.c_str());
    struct stat sb;
    if (fstat(m.fd, &sb) != 0 || sb.st_size < 24) {
        ::close(m.fd);
        return fail(FNX_E_ARG, "gguf: %s is too short to be a GGUF file", path.c_str());
    }
    m.size = (size_t) sb.st_size;
    m.base = mmap(nullptr, m.size, PROT_READ, MAP_PRIVATE, m.fd, 0);
    if (m.base == MAP_FAILED) {
        ::close(m.fd);
        return fail(FNX_E_ARG, "gguf: cannot map %s", path.c_str());
    }
    const int shard = (int) g->maps.size();
    g->maps.push_back(m);
    Cursor c{(const uint8_t*) m.base, m.size};
    const uint32_t magic = c.get<uint32_t>(), version = c.get<uint32_t>();
    if (magic != 0x46554747u) return fail(FNX_E_ARG, "gguf: %s does not start with GGUF", path.c_str());
    if (version != 2 && version != 3) return fail(FNX_E_ARG, "gguf: %s is version %u (2 and 3 are read)", path.c_str(), version);
    const uint64_t n_tensors = c.get<uint64_t>(), n_keys = c.get<uint64_t>();
    if (n_tensors > (1u << 24) || n_keys > (1u << 24)) return fail(FNX_E_ARG, "gguf: %s: implausible counts", path.c_str());
    size_t alignment = 32;
    for (uint64_t k = 0; k < n_keys && c.ok; ++k) {
        const std::string key = c.str();
        const uint32_t vt = c.get<uint32_t>();
        if (!c.ok) break;
        if (vt == 8) {
            const std::string v = c.str();
            if (meta) g->strs[key] = v;
        } else if (vt == 9) {
            const uint32_t et = c.get<uint32_t>();
            const uint64_t cnt = c.get<uint64_t>();
            if (et == 8) {   // strings (a tokenizer's vocabulary): skipped, the engine takes token ids
                for (uint64_t i = 0; i < cnt && c.ok; ++i) c.skip((size_t) c.get<uint64_t>());
            } else if (scalar_bytes(et) == 0) {
                return fail(FNX_E_ARG, "gguf: %s: key %s is an array of type %u", path.c_str(), key.c_str(), et);
            } else if (et == 6 || et == 12 || cnt > (1u << 22)) {
                c.skip((size_t) cnt * scalar_bytes(et));
            } else {
                std::vector<int64_t> a;
                a.reserve((size_t) cnt);
                for (uint64_t i = 0; i < cnt && c.ok; ++i) {
                    double v;
                    bool is_int;
                    if (!scalar_value(c, et, v, is_int)) break;
                    a.push_back((int64_t) v);
                }
                if (meta) g->int_arrays[key] = std::move(a);
            }
        } else {
            double v;
            bool is_int;
            if (!scalar_value(c, vt, v, is_int)) return fail(FNX_E_ARG, "gguf: %s: key %s has the unknown type %u", path.c_str(), key.c_str(), vt);
            if (meta) {
                g->nums[key] = v;
                g->num_is_int[key] = is_int;
            }
            if (key == "general.alignment") alignment = (size_t) v;
        }
        if (meta) g->key_types[key] = vt;
    }
    if (!c.ok) return fail(FNX_E_ARG, "gguf: %s ends inside its metadata", path.c_str());
    if (alignment == 0 || (alignment & (alignment - 1))) return fail(FNX_E_ARG, "gguf: %s: alignment %zu is not a power of two", path.c_str(), alignment);
    const size_t first = g->tensors.size();
    for (uint64_t i = 0; i < n_tensors && c.ok; ++i) {
        GgufTensor t;
        t.name = c.str();
        t.n_dims = (int) c.get<uint32_t>();
        if (!c.ok || t.n_dims < 1 || t.n_dims > 4) return fail(FNX_E_ARG, "gguf: %s: tensor %s has %d dimensions", path.c_str(), t.name.c_str(), t.n_dims);
        for (int d = 0; d < t.n_dims; ++d) t.ne[d] = (int64_t) c.get<uint64_t>();
        t.type = c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        t.shard = shard;
        const GgufType ti = gguf_type(t.type);
        if (ti.bytes == 0) return fail(FNX_E_ARG, "gguf: %s: tensor %s has the unknown type %u", path.c_str(), t.name.c_str(), t.type);
        for (int d = 0; d < t.n_dims; ++d)
            if (t.ne[d] < 0 || t.ne[d] > ((int64_t) 1 << 40)) return fail(FNX_E_ARG, "gguf: %s: tensor %s has a bad extent", path.c_str(), t.name.c_str());
        if (t.ne[0] % ti.block) return fail(FNX_E_ARG, "gguf: %s: tensor %s: %lld columns are not whole blocks of %d", path.c_str(), t.name.c_str(), (long long) t.ne[0], ti.block);
        t.bytes = (size_t) (t.ne[0] / ti.block) * ti.bytes * (size_t) (t.ne[1] * t.ne[2] * t.ne[3]);
        g->tensors.push_back(std::move(t));
    }
    if (!c.ok) return fail(FNX_E_ARG, "gguf: %s ends inside its tensor records", path.c_str());
    const size_t data0 = (c.at + alignment - 1) / alignment * alignment;
    for (size_t i = first; i < g->tensors.size(); ++i) {
        GgufTensor& t = g->tensors[i];
        if (t.offset % alignment) return fail(FNX_E_ARG, "gguf: %s: tensor %s starts off the alignment of %zu", path.c_str(), t.name.c_str(), alignment);
        t.offset += data0;
        if (t.offset > m.size || t.bytes > m.size - t.offset)
            return fail(FNX_E_ARG, "gguf: %s: tensor %s runs past the end of the file", path.c_str(), t.name.c_str());
        t.data = (const uint8_t*) m.base + t.offset;
        if (!g->by_name.emplace(t.name, (int) i).second) return fail(FNX_E_ARG, "gguf: tensor %s appears twice", t.name.c_str());
    }
    return FNX_OK;
}

// "<stem>-00001-of-0000N.gguf": the N shard paths; anything else: the path alone
static std::vector<std::string> shard_paths(const std::string& first) {
    std::vector<std::string> out{first};
    const size_t ext = first.rfind(".gguf");
    if (ext == std::string::npos || ext + 5 != first.size() || ext < 15) return out;
    const std::string tag = first.substr(ext - 15, 15);   // -00001-of-0000N
    int a = 0, n = 0;
    if (tag[0] != '-' || tag.substr(6, 4) != "-of-" || std::sscanf(tag.c_str(), "-%5d-of-%5d", &a, &n) != 2 || a != 1 || n < 2) return out;
    for (int s = 2; s <= n; ++s) {
        char buf[32];
        std::snprintf(buf, sizeof buf, "-%05d-of-%05d.gguf", s, n);
        out.push_back(first.substr(0, ext - 15) + buf);
    }
    return out;
}

static inline float half_bits_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t) (h & 0x8000u) << 16, ex = (h >> 10) & 31u, man = h & 1023u;
    uint32_t u;
    if (ex == 0) {
        if (man == 0) u = sign;
        else {   // subnormal: man * 2^-24
            const float f = (float) man * (1.0f / 16777216.0f);
            uint32_t b;
            memcpy(&b, &f, 4);
            u = b | sign;
        }
    } else if (ex == 31) u = sign | 0x7f800000u | (man << 13);
    else u = sign | ((ex + 112u) << 23) | (man << 13);
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static const uint32_t iq3s_grid_host[512] = {FNX_IQ3S_GRID_VALUES};

// one block_iq3_s (110 bytes: d f16, qs[64], qh[8], signs[32], scales[4]) to 256 floats
static void iq3s_block_to_f32(const uint8_t* b, float* out) {
    uint16_t dh;
    memcpy(&dh, b, 2);
    const float d = half_bits_to_float(dh);
    const uint8_t *qs = b + 2, *qh = b + 66, *signs = b + 74, *scales = b + 106;
    for (int ib = 0; ib < 8; ++ib) {   // 32 weights each
        const int nib = (scales[ib / 2] >> (4 * (ib & 1))) & 15;
        const float db = d * (float) (1 + 2 * nib);
        for (int l = 0; l < 8; ++l) {   // 4 weights each
            const int idx = qs[ib * 8 + l] | (((qh[ib] >> l) & 1) << 8);
            const uint32_t gv = iq3s_grid_host[idx];
            const uint8_t sg = signs[ib * 4 + l / 2];
            for (int j = 0; j < 4; ++j) {
                const float mag = (float) ((gv >> (8 * j)) & 255u);
                const bool neg = (sg >> ((l & 1) * 4 + j)) & 1;
                out[ib * 32 + l * 4 + j] = db * (neg ? -mag : mag);
            }
        }
    }
}

}  // namespace fnxb

using namespace fnxb;

extern "C" int fnx_gguf_open(const char* path, fnx_gguf** out) {
    FNX_REQUIRE(path && out, "fnx_gguf_open: null argument");
    *out = nullptr;
    fnx_gguf* g = new fnx_gguf();
    const std::vector<std::string> paths = shard_paths(path);
    int rc = FNX_OK;
    for (size_t s = 0; s < paths.size() && rc == FNX_OK; ++s) rc = load_shard(g, paths[s], s == 0);
    if (rc != FNX_OK) {
        fnx_gguf_close(g);
        return rc;
    }
    *out = g;
    return FNX_OK;
}

extern "C" void fnx_gguf_close(fnx_gguf* g) {
    if (!g) return;
    for (GgufMap& m : g->maps) {
        if (m.base && m.base != MAP_FAILED) munmap(m.base, m.size);
        if (m.fd >= 0) ::close(m.fd);
    }
    delete g;
}

extern "C" int fnx_gguf_count(const fnx_gguf* g) { return g ? (int) g->tensors.size() : 0; }
extern "C" int fnx_gguf_shards(const fnx_gguf* g) { return g ? (int) g->maps.size() : 0; }

static void export_tensor(const GgufTensor& t, fnx_gguf_tensor* out) {
    out->name = t.name.c_str();
    out->type = t.type;
    out->n_dims = t.n_dims;
    for (int d = 0; d < 4; ++d) out->ne[d] = t.ne[d];
    out->data = t.data;
    out->bytes = t.bytes;
    out->shard = t.shard;
    out->offset = t.offset;
}

extern "C" int fnx_gguf_tensor_at(const fnx_gguf* g, int i, fnx_gguf_tensor* out) {
    FNX_REQUIRE(g && out && i >= 0 && i < (int) g->tensors.size(), "fnx_gguf_tensor_at: tensor %d of %d", i, g ? (int) g->tensors.size() : 0);
    export_tensor(g->tensors[(size_t) i], out);
    return FNX_OK;
}

extern "C" int fnx_gguf_find(const fnx_gguf* g, const char* name, fnx_gguf_tensor* out) {
    if (!g || !name) return 0;
    auto it = g->by_name.find(name);
    if (it == g->by_name.end()) return 0;
    if (out) export_tensor(g->tensors[(size_t) it->second], out);
    return 1;
}

extern "C" int fnx_gguf_num(const fnx_gguf* g, const char* key, double* out) {
    if (!g || !key) return 0;
    auto it = g->nums.find(key);
    if (it == g->nums.end()) return 0;
    if (out) *out = it->second;
    return 1;
}

extern "C" int fnx_gguf_str(const fnx_gguf* g, const char* key, char* buf, size_t cap) {
    if (!g || !key) return 0;
    auto it = g->strs.find(key);
    if (it == g->strs.end()) return 0;
    if (buf && cap) {
        const size_t n = it->second.size() < cap - 1 ? it->second.size() : cap - 1;
        memcpy(buf, it->second.data(), n);
        buf[n] = 0;
    }
    return 1;
}

extern "C" int fnx_gguf_int_array(const fnx_gguf* g, const char* key, int64_t* out, size_t cap, size_t* n) {
    if (n) *n = 0;
    if (!g || !key) return 0;
    auto it = g->int_arrays.find(key);
    if (it == g->int_arrays.end()) return 0;
    if (n) *n = it->second.size();
    if (out)
        for (size_t i = 0; i < it->second.size() && i < cap; ++i) out[i] = it->second[i];
    return 1;
}

extern "C" int fnx_gguf_rows_f32(const fnx_gguf_tensor* t, int64_t row0, int64_t n_rows, float* out) {
    FNX_REQUIRE(t && out && t->data, "fnx_gguf_rows_f32: null argument");
    const int64_t rows = t->ne[1] * t->ne[2] * t->ne[3], cols = t->ne[0];
    FNX_REQUIRE(row0 >= 0 && n_rows >= 0 && row0 + n_rows <= rows, "fnx_gguf_rows_f32: rows [%lld, %lld) of %lld in %s", (long long) row0,
                (long long) (row0 + n_rows), (long long) rows, t->name);
    const GgufType ti = gguf_type(t->type);
    const size_t row_bytes = (size_t) (cols / ti.block) * ti.bytes;
    const uint8_t* src = (const uint8_t*) t->data + (size_t) row0 * row_bytes;
    const size_t n = (size_t) n_rows * (size_t) cols;
    switch (t->type) {
        case 0: memcpy(out, src, n * 4); break;
        case 1:
            for (size_t i = 0; i < n; ++i) {
                uint16_t h;
                memcpy(&h, src + 2 * i, 2);
                out[i] = half_bits_to_float(h);
            }
            break;
        case 30:
            for (size_t i = 0; i < n; ++i) {
                uint16_t h;
                memcpy(&h, src + 2 * i, 2);
                const uint32_t u = (uint32_t) h << 16;
                memcpy(out + i, &u, 4);
            }
            break;
        case 8:   // Q8_0: d f16, 32 int8
            for (size_t b = 0; b < n / 32; ++b) {
                const uint8_t* q = src + b * 34;
                uint16_t h;
                memcpy(&h, q, 2);
                const float d = half_bits_to_float(h);
                for (int j = 0; j < 32; ++j) out[b * 32 + j] = d * (float) (int8_t) q[2 + j];
            }
            break;
        case 21:
            for (size_t b = 0; b < n / 256; ++b) iq3s_block_to_f32(src + b * 110, out + b * 256);
            break;
        default:
            return fail(FNX_E_UNAVAILABLE, "fnx_gguf_rows_f32: tensor %s has type %u; F32, F16, BF16, Q8_0 and IQ3_S are converted", t->name, t->type);
    }
    return FNX_OK;
}

// the architecture's fields of the model configuration from the metadata (the keys the reference checks,
// engine/src/model.cpp:1481-1506); the caller's run-time fields (max_ctx, max_rows, n_seq, ep_rank, ep_size) stay
extern "C" int fnx_gguf_model_config(const fnx_gguf* g, fnx_model_config* cfg) {
    FNX_REQUIRE(g && cfg, "fnx_gguf_model_config: null argument");
    auto it = g->strs.find("general.architecture");
    FNX_REQUIRE(it != g->strs.end(), "gguf: no general.architecture");
    const std::string p = it->second + ".";
    bool missing = false;
    std::string first_missing;
    auto num = [&](const char* k, double dflt, bool required) {
        auto f = g->nums.find(p + k);
        if (f != g->nums.end()) return f->second;
        if (required && !missing) {
            missing = true;
            first_missing = p + k;
        }
        return dflt;
    };
    const int nextn = (int) num("nextn_predict_layers", 0, false);
    FNX_REQUIRE(nextn == 1, "gguf: %snextn_predict_layers = %d: the verify path drafts with one next-token layer", p.c_str(), nextn);
    cfg->n_layer = (int) num("block_count", 0, true) - nextn;
    cfg->hidden = (int) num("embedding_length", 0, true);
    cfg->n_expert = (int) num("expert_count", 0, true);
    cfg->top_k = (int) num("expert_used_count", 0, true);
    cfg->ffn = (int) num("expert_feed_forward_length", 0, true);
    cfg->n_q_head = (int) num("attention.head_count", 0, true);
    cfg->n_kv_head = (int) num("attention.head_count_kv", 0, true);
    cfg->head_dim = (int) num("attention.key_length", 0, true);
    cfg->n_rot = (int) num("rope.dimension_count", 0, true);
    cfg->gdn_k_head = (int) num("ssm.group_count", 0, true);
    cfg->gdn_v_head = (int) num("ssm.time_step_rank", 0, true);
    cfg->gdn_head_dim = (int) num("ssm.state_size", 0, true);
    cfg->attn_every = (int) num("full_attention_interval", 4, false);
    cfg->eps = (float) num("attention.layer_norm_rms_epsilon", 1e-6, false);
    cfg->rope_base = (float) num("rope.freq_base", 1e7, false);
    FNX_REQUIRE(!missing, "gguf: no key %s", first_missing.c_str());
    FNX_REQUIRE((int) num("attention.value_length", cfg->head_dim, false) == cfg->head_dim, "gguf: key and value heads differ in length");
    FNX_REQUIRE((int) num("ssm.conv_kernel", 4, false) == 4, "gguf: %sssm.conv_kernel is not 4", p.c_str());
    auto emb = g->by_name.find("token_embd.weight");
    FNX_REQUIRE(emb != g->by_name.end(), "gguf: no token_embd.weight");
    cfg->vocab = (int) g->tensors[(size_t) emb->second].ne[1];
    char name[96];
    std::snprintf(name, sizeof name, "blk.%d.nextn.draft_vocab", cfg->n_layer);
    auto dv = g->by_name.find(name);
    cfg->draft_vocab = dv == g->by_name.end() ? 0 : (int) g->tensors[(size_t) dv->second].ne[0];
    return FNX_OK;
}
