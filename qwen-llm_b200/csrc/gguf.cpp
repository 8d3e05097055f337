// GGUF reader: maps a .gguf file and exposes its tensors as a dfl_tensor table (pointers into the mapping) and its
// metadata through typed getters, plus the two derived structures the step needs - the target's dfl_arch and the
// drafter's dfl_dflash_config (reference: crates/qwen-llm/src/gguf.rs - GgufFile::open :154, find :474, typed getters
// :514-729, header validation :1135-1300; crates/qwen-llm/src/loader.rs - build_arch_from_metadata :1331-1656, the
// DFlash key sets and config extraction :860-1060).  Single-file models only: a split.count above 1 is refused.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/dflash_b200.h"

namespace dfl {
dfl_status fail(dfl_status st, const std::string& msg);
}
using dfl::fail;

namespace {
constexpr uint32_t GGUF_MAGIC = 0x46554747;   // "GGUF"
constexpr uint64_t MAX_TENSORS = 1000000, MAX_KV = 1000000, MAX_KEY_LEN = 1024, MAX_ALIGNMENT = 65536;   // gguf.rs:46, :1303-1306
constexpr uint64_t MAX_ARCH_DIM = 1u << 24, MAX_ARCH_LAYERS = 4096;
enum VType : uint32_t { T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 };

struct Value {
    uint32_t type = 0, elem_type = 0;
    uint64_t count = 0;          // array length
    const uint8_t* p = nullptr;  // scalar bytes / string bytes / first array element
    uint64_t len = 0;            // string length
};

// (elements per block, bytes per block) of a ggml type; false when the type is not known here
bool storage_layout(int32_t t, uint64_t* el, uint64_t* nb) {
    static const struct { int32_t t; uint32_t el, nb; } k[] = {
        {0, 1, 4},    {1, 1, 2},     {2, 32, 18},   {3, 32, 20},   {6, 32, 22},   {7, 32, 24},   {8, 32, 34},  {9, 32, 36},
        {10, 256, 84}, {11, 256, 110}, {12, 256, 144}, {13, 256, 176}, {14, 256, 210}, {15, 256, 292}, {24, 1, 1},  {25, 1, 2},
        {26, 1, 4},   {27, 1, 8},    {28, 1, 8},    {30, 1, 2}};
    for (auto& e : k)
        if (e.t == t) { *el = e.el; *nb = e.nb; return true; }
    return false;
}
size_t scalar_size(uint32_t t) {
    switch (t) {
        case T_U8: case T_I8: case T_BOOL: return 1;
        case T_U16: case T_I16: return 2;
        case T_U32: case T_I32: case T_F32: return 4;
        case T_U64: case T_I64: case T_F64: return 8;
        default: return 0;
    }
}
template <typename T> T rd(const uint8_t* p) { T v; memcpy(&v, p, sizeof(T)); return v; }
bool scalar_u64(uint32_t t, const uint8_t* p, uint64_t* out) {   // value_as_u64, gguf.rs:1255: any non-negative integer
    int64_t s;
    switch (t) {
        case T_U8: *out = rd<uint8_t>(p); return true;
        case T_U16: *out = rd<uint16_t>(p); return true;
        case T_U32: *out = rd<uint32_t>(p); return true;
        case T_U64: *out = rd<uint64_t>(p); return true;
        case T_I8: s = rd<int8_t>(p); break;
        case T_I16: s = rd<int16_t>(p); break;
        case T_I32: s = rd<int32_t>(p); break;
        case T_I64: s = rd<int64_t>(p); break;
        default: return false;
    }
    if (s < 0) return false;
    *out = (uint64_t)s;
    return true;
}
}  // namespace

struct dfl_gguf {
    int fd = -1;
    const uint8_t* map = nullptr;
    uint64_t size = 0, data_start = 0, alignment = 32;
    uint32_t version = 0;
    std::map<std::string, Value> kv;
    std::vector<std::string> names;       // owned copies (NUL-terminated) of the tensor names
    std::vector<dfl_tensor> tensors;
    std::vector<std::string> alias_names; // canonical drafter names
    std::vector<dfl_tensor> drafter_tensors;
    std::map<std::string, size_t> index;

    const Value* get(const char* key) const {
        auto it = kv.find(key);
        return it == kv.end() ? nullptr : &it->second;
    }
    bool u64(const std::string& key, uint64_t* out) const {
        const Value* v = get(key.c_str());
        return v && v->type != T_ARR && v->type != T_STR && scalar_u64(v->type, v->p, out);
    }
    bool f64(const std::string& key, double* out) const {   // gguf.rs:524 / :697: f32 or f64 (integers too)
        const Value* v = get(key.c_str());
        if (!v) return false;
        if (v->type == T_F32) { *out = rd<float>(v->p); return true; }
        if (v->type == T_F64) { *out = rd<double>(v->p); return true; }
        uint64_t u;
        if (v->type != T_ARR && v->type != T_STR && v->type != T_BOOL && scalar_u64(v->type, v->p, &u)) { *out = (double)u; return true; }
        return false;
    }
    std::string str(const std::string& key) const {
        const Value* v = get(key.c_str());
        return v && v->type == T_STR ? std::string((const char*)v->p, v->len) : std::string();
    }
};

namespace {
struct Cursor {
    const uint8_t* base;
    uint64_t size, off = 0;
    bool ok = true;
    bool need(uint64_t n) { if (!ok || n > size - off) { ok = false; return false; } return true; }
    template <typename T> T get() { if (!need(sizeof(T))) return T(); T v = rd<T>(base + off); off += sizeof(T); return v; }
    bool str(const uint8_t** p, uint64_t* len, uint64_t cap) {
        *len = get<uint64_t>();
        if (!ok || *len > cap || !need(*len)) { ok = false; return false; }
        *p = base + off;
        off += *len;
        return true;
    }
};

dfl_status parse(dfl_gguf* g) {
    Cursor c{g->map, g->size};
    if (g->size < 24 || c.get<uint32_t>() != GGUF_MAGIC) return fail(DFL_ERR_BAD_ARG, "gguf: bad magic");
    g->version = c.get<uint32_t>();
    if (g->version != 2 && g->version != 3) return fail(DFL_ERR_UNSUPPORTED, "gguf: unsupported version " + std::to_string(g->version));
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    if (n_tensors > MAX_TENSORS || n_kv > MAX_KV) return fail(DFL_ERR_BAD_SHAPE, "gguf: tensor or metadata count exceeds the cap");
    for (uint64_t i = 0; i < n_kv; ++i) {
        const uint8_t* kp;
        uint64_t kl;
        if (!c.str(&kp, &kl, MAX_KEY_LEN)) return fail(DFL_ERR_BAD_SHAPE, "gguf: truncated or oversized metadata key");
        Value v;
        v.type = c.get<uint32_t>();
        if (v.type == T_STR) {
            if (!c.str(&v.p, &v.len, g->size)) return fail(DFL_ERR_BAD_SHAPE, "gguf: truncated metadata string");
        } else if (v.type == T_ARR) {
            v.elem_type = c.get<uint32_t>();
            v.count = c.get<uint64_t>();
            v.p = g->map + c.off;
            if (v.elem_type == T_STR) {
                for (uint64_t e = 0; e < v.count; ++e) {
                    const uint8_t* sp;
                    uint64_t sl;
                    if (!c.str(&sp, &sl, g->size)) return fail(DFL_ERR_BAD_SHAPE, "gguf: truncated string array");
                }
            } else {
                const size_t es = scalar_size(v.elem_type);
                if (!es || v.count > g->size / es || !c.need(v.count * es)) return fail(DFL_ERR_BAD_SHAPE, "gguf: bad metadata array");
                c.off += v.count * es;
            }
        } else {
            const size_t es = scalar_size(v.type);
            if (!es || !c.need(es)) return fail(DFL_ERR_BAD_SHAPE, "gguf: bad metadata value type");
            v.p = g->map + c.off;
            c.off += es;
        }
        if (!c.ok) return fail(DFL_ERR_BAD_SHAPE, "gguf: truncated metadata");
        g->kv[std::string((const char*)kp, kl)] = v;
    }
    uint64_t split = 0;
    if (g->u64("split.count", &split) && split > 1) return fail(DFL_ERR_UNSUPPORTED, "gguf: split files are not supported (split.count > 1)");
    uint64_t al = 32;
    if (g->get("general.alignment") && !g->u64("general.alignment", &al)) return fail(DFL_ERR_BAD_SHAPE, "gguf: general.alignment is not an integer");
    if (al == 0 || al > MAX_ALIGNMENT || (al & (al - 1))) return fail(DFL_ERR_BAD_SHAPE, "gguf: general.alignment must be a power of two up to 65536");
    g->alignment = al;
    struct Info { uint64_t off; };
    std::vector<uint64_t> offs(n_tensors);
    g->names.reserve(n_tensors);
    g->tensors.resize(n_tensors);
    for (uint64_t i = 0; i < n_tensors; ++i) {
        const uint8_t* np;
        uint64_t nl;
        if (!c.str(&np, &nl, MAX_KEY_LEN)) return fail(DFL_ERR_BAD_SHAPE, "gguf: truncated or oversized tensor name");
        dfl_tensor& t = g->tensors[i];
        memset(&t, 0, sizeof(t));
        const uint32_t nd = c.get<uint32_t>();
        if (!c.ok || nd < 1 || nd > 4) return fail(DFL_ERR_BAD_SHAPE, "gguf: tensor rank must be 1..4");
        t.n_dims = (int32_t)nd;
        for (uint32_t d = 0; d < nd; ++d) t.shape[d] = c.get<uint64_t>();
        t.dtype = (int32_t)c.get<uint32_t>();
        offs[i] = c.get<uint64_t>();
        if (!c.ok) return fail(DFL_ERR_BAD_SHAPE, "gguf: truncated tensor table");
        g->names.emplace_back((const char*)np, nl);
        if (!g->index.emplace(g->names.back(), i).second) return fail(DFL_ERR_BAD_SHAPE, "gguf: duplicate tensor name " + g->names.back());
    }
    g->data_start = (c.off + al - 1) / al * al;
    if (n_tensors && g->data_start > g->size) return fail(DFL_ERR_BAD_SHAPE, "gguf: tensor data section starts beyond the file");
    for (uint64_t i = 0; i < n_tensors; ++i) {
        dfl_tensor& t = g->tensors[i];
        t.name = g->names[i].c_str();
        uint64_t n_el = 1;
        for (int d = 0; d < t.n_dims; ++d) {
            if (t.shape[d] && n_el > UINT64_MAX / t.shape[d]) return fail(DFL_ERR_BAD_SHAPE, "gguf: tensor element count overflows: " + g->names[i]);
            n_el *= t.shape[d];
        }
        uint64_t el, nb;
        if (!storage_layout(t.dtype, &el, &nb)) return fail(DFL_ERR_UNSUPPORTED, "gguf: tensor " + g->names[i] + " has an unknown ggml type " + std::to_string(t.dtype));
        if (t.shape[0] % el) return fail(DFL_ERR_BAD_SHAPE, "gguf: tensor " + g->names[i] + " row length is not a multiple of its block size");
        t.n_bytes = n_el / el * nb;   // validate_tensor_storage_size, gguf.rs:1094
        if (offs[i] % al) return fail(DFL_ERR_BAD_SHAPE, "gguf: tensor " + g->names[i] + " is not aligned");
        if (offs[i] > g->size - g->data_start || t.n_bytes > g->size - g->data_start - offs[i])
            return fail(DFL_ERR_BAD_SHAPE, "gguf: tensor " + g->names[i] + " extends beyond the file");
        t.data = g->map + g->data_start + offs[i];
    }
    return DFL_OK;
}

dfl_status need_u32(const dfl_gguf* g, const std::string& key, uint32_t* out, uint64_t cap, bool nonzero) {
    uint64_t v;
    if (!g->u64(key, &v)) return fail(DFL_ERR_BAD_ARG, "gguf: missing or non-integer metadata " + key);
    if (v > cap) return fail(DFL_ERR_BAD_SHAPE, "gguf: metadata " + key + " exceeds its cap");
    if (nonzero && v == 0) return fail(DFL_ERR_BAD_SHAPE, "gguf: metadata " + key + " must be nonzero");
    *out = (uint32_t)v;
    return DFL_OK;
}
}  // namespace

#define G_CHECK(expr)                   \
    do {                                \
        dfl_status _s = (expr);         \
        if (_s != DFL_OK) return _s;    \
    } while (0)

extern "C" {

dfl_status dfl_gguf_open(const char* path, dfl_gguf** out) {
    if (!path || !out) return fail(DFL_ERR_BAD_ARG, "gguf_open: null argument");
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(DFL_ERR_BAD_ARG, std::string("gguf_open: cannot open ") + path);
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size <= 0) { close(fd); return fail(DFL_ERR_BAD_ARG, std::string("gguf_open: empty or unreadable file ") + path); }
    void* m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (m == MAP_FAILED) { close(fd); return fail(DFL_ERR_OOM, std::string("gguf_open: mmap failed for ") + path); }
    auto* g = new dfl_gguf();
    g->fd = fd;
    g->map = (const uint8_t*)m;
    g->size = (uint64_t)st.st_size;
    const dfl_status s = parse(g);
    if (s != DFL_OK) { dfl_gguf_close(g); return s; }
    *out = g;
    return DFL_OK;
}

void dfl_gguf_close(dfl_gguf* g) {
    if (!g) return;
    if (g->map) munmap((void*)g->map, (size_t)g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

uint64_t dfl_gguf_tensor_count(const dfl_gguf* g) { return g ? g->tensors.size() : 0; }
const dfl_tensor* dfl_gguf_tensors(const dfl_gguf* g) { return g && !g->tensors.empty() ? g->tensors.data() : nullptr; }

dfl_status dfl_gguf_find(const dfl_gguf* g, const char* name, dfl_tensor* out) {
    if (!g || !name || !out) return fail(DFL_ERR_BAD_ARG, "gguf_find: null argument");
    auto it = g->index.find(name);
    if (it == g->index.end()) return fail(DFL_ERR_MISSING_TENSOR, std::string("gguf: no tensor named ") + name);
    *out = g->tensors[it->second];
    return DFL_OK;
}

dfl_status dfl_gguf_get_u64(const dfl_gguf* g, const char* key, uint64_t* out, int32_t* found) {
    if (!g || !key || !out || !found) return fail(DFL_ERR_BAD_ARG, "gguf_get_u64: null argument");
    *found = g->u64(key, out) ? 1 : 0;
    return DFL_OK;
}
dfl_status dfl_gguf_get_f64(const dfl_gguf* g, const char* key, double* out, int32_t* found) {
    if (!g || !key || !out || !found) return fail(DFL_ERR_BAD_ARG, "gguf_get_f64: null argument");
    *found = g->f64(key, out) ? 1 : 0;
    return DFL_OK;
}
dfl_status dfl_gguf_get_bool(const dfl_gguf* g, const char* key, int32_t* out, int32_t* found) {
    if (!g || !key || !out || !found) return fail(DFL_ERR_BAD_ARG, "gguf_get_bool: null argument");
    const Value* v = g->get(key);
    *found = 0;
    if (!v) return DFL_OK;
    if (v->type != T_BOOL) return fail(DFL_ERR_BAD_SHAPE, std::string("gguf: metadata ") + key + " is not a bool");   // gguf.rs:535-544
    *out = v->p[0] != 0;
    *found = 1;
    return DFL_OK;
}
dfl_status dfl_gguf_get_str(const dfl_gguf* g, const char* key, char* buf, uint64_t cap, int32_t* found) {
    if (!g || !key || !buf || !found || cap == 0) return fail(DFL_ERR_BAD_ARG, "gguf_get_str: null argument");
    const Value* v = g->get(key);
    *found = 0;
    if (!v || v->type != T_STR) return DFL_OK;
    if (v->len + 1 > cap) return fail(DFL_ERR_BAD_SHAPE, std::string("gguf: metadata string ") + key + " does not fit the buffer");
    memcpy(buf, v->p, v->len);
    buf[v->len] = 0;
    *found = 1;
    return DFL_OK;
}
// integer or bool arrays, widened to u64 (get_u64_array :613, get_bool_array :679)
dfl_status dfl_gguf_get_u64_array(const dfl_gguf* g, const char* key, uint64_t* out, uint64_t cap, uint64_t* count, int32_t* found) {
    if (!g || !key || !count || !found) return fail(DFL_ERR_BAD_ARG, "gguf_get_u64_array: null argument");
    const Value* v = g->get(key);
    *found = 0;
    *count = 0;
    if (!v) return DFL_OK;
    if (v->type != T_ARR || v->elem_type == T_STR || v->elem_type == T_F32 || v->elem_type == T_F64 || v->elem_type == T_ARR)
        return fail(DFL_ERR_BAD_SHAPE, std::string("gguf: metadata ") + key + " is not an integer array");
    *count = v->count;
    *found = 1;
    if (!out) return DFL_OK;
    if (v->count > cap) return fail(DFL_ERR_BAD_SHAPE, std::string("gguf: metadata array ") + key + " does not fit the buffer");
    const size_t es = scalar_size(v->elem_type);
    for (uint64_t i = 0; i < v->count; ++i) {
        if (v->elem_type == T_BOOL) out[i] = v->p[i] != 0;
        else if (!scalar_u64(v->elem_type, v->p + i * es, &out[i])) return fail(DFL_ERR_BAD_SHAPE, std::string("gguf: negative element in ") + key);
    }
    return DFL_OK;
}

// build_arch_from_metadata  loader.rs:1331-1656
dfl_status dfl_gguf_arch(const dfl_gguf* g, dfl_arch* out) {
    if (!g || !out) return fail(DFL_ERR_BAD_ARG, "gguf_arch: null argument");
    memset(out, 0, sizeof(*out));
    const std::string p = g->str("general.architecture");
    const bool moe = p == "qwen35moe";
    if (p != "qwen35" && !moe) return fail(DFL_ERR_UNSUPPORTED, "gguf: unsupported architecture '" + p + "'");
    uint32_t blocks = 0, nextn = 0;
    G_CHECK(need_u32(g, p + ".block_count", &blocks, MAX_ARCH_LAYERS + MAX_ARCH_LAYERS, true));
    uint64_t nn = 0;
    if (g->u64(p + ".nextn_predict_layers", &nn)) nextn = (uint32_t)std::min<uint64_t>(nn, blocks);
    if (blocks - nextn == 0 || blocks - nextn > MAX_ARCH_LAYERS) return fail(DFL_ERR_BAD_SHAPE, "gguf: block_count - nextn_predict_layers out of range");
    out->n_layer = blocks - nextn;   // trailing next-token-prediction layers are not part of the main forward
    G_CHECK(need_u32(g, p + ".embedding_length", &out->hidden_size, MAX_ARCH_DIM, true));
    uint64_t ff = 0;
    if (g->u64(p + ".feed_forward_length", &ff)) {
        if (ff > MAX_ARCH_DIM) return fail(DFL_ERR_BAD_SHAPE, "gguf: feed_forward_length exceeds its cap");
        out->intermediate_size = (uint32_t)ff;
    }
    if (!moe && out->intermediate_size == 0) return fail(DFL_ERR_BAD_SHAPE, "gguf: feed_forward_length must be nonzero on a dense model");
    G_CHECK(need_u32(g, p + ".attention.head_count", &out->n_q_heads, MAX_ARCH_DIM, true));
    G_CHECK(need_u32(g, p + ".attention.head_count_kv", &out->n_kv_heads, MAX_ARCH_DIM, true));
    if (out->n_q_heads % out->n_kv_heads) return fail(DFL_ERR_BAD_SHAPE, "gguf: attention.head_count is not a multiple of attention.head_count_kv");
    G_CHECK(need_u32(g, p + ".attention.key_length", &out->attn_head_dim, MAX_ARCH_DIM, true));
    uint64_t fai = 4;
    g->u64(p + ".full_attention_interval", &fai);
    if (fai == 0 || fai > MAX_ARCH_LAYERS) return fail(DFL_ERR_BAD_SHAPE, "gguf: full_attention_interval out of range");
    out->full_attention_interval = (uint32_t)fai;
    G_CHECK(need_u32(g, p + ".ssm.state_size", &out->gdn_head_dim, MAX_ARCH_DIM, true));
    G_CHECK(need_u32(g, p + ".ssm.time_step_rank", &out->gdn_n_v_heads, MAX_ARCH_DIM, true));
    G_CHECK(need_u32(g, p + ".ssm.group_count", &out->gdn_n_k_heads, MAX_ARCH_DIM, true));
    G_CHECK(need_u32(g, p + ".ssm.conv_kernel", &out->gdn_conv_kernel, 16, true));
    if (moe) {
        G_CHECK(need_u32(g, p + ".expert_count", &out->expert_count, MAX_ARCH_DIM, true));
        G_CHECK(need_u32(g, p + ".expert_used_count", &out->expert_used_count, MAX_ARCH_DIM, true));
        if (out->expert_used_count > out->expert_count) return fail(DFL_ERR_BAD_SHAPE, "gguf: expert_used_count exceeds expert_count");
        G_CHECK(need_u32(g, p + ".expert_feed_forward_length", &out->expert_feed_forward_length, MAX_ARCH_DIM, true));
        G_CHECK(need_u32(g, p + ".expert_shared_feed_forward_length", &out->expert_shared_feed_forward_length, MAX_ARCH_DIM, true));
    }
    auto it = g->index.find("token_embd.weight");   // vocab from the embedding's shape, the metadata key may be absent
    if (it == g->index.end() || g->tensors[it->second].n_dims < 2) return fail(DFL_ERR_MISSING_TENSOR, "gguf: token_embd.weight is missing or not 2-D");
    const uint64_t vocab = g->tensors[it->second].shape[1];
    if (vocab == 0 || vocab > MAX_ARCH_DIM) return fail(DFL_ERR_BAD_SHAPE, "gguf: vocabulary size out of range");
    out->vocab_size = (uint32_t)vocab;
    double theta = 10000000.0;
    g->f64(p + ".rope.freq_base", &theta);
    out->rope_theta = (float)theta;
    out->partial_rotary_factor = 0.25f;
    return DFL_OK;
}

// DFlashConfig from a drafter file  loader.rs:860-1060 (key sets "dflash-draft" and "dflash")
dfl_status dfl_gguf_dflash_config(const dfl_gguf* g, const dfl_arch* target, dfl_dflash_config* out) {
    if (!g || !target || !out) return fail(DFL_ERR_BAD_ARG, "gguf_dflash_config: null argument");
    memset(out, 0, sizeof(*out));
    const std::string a = g->str("general.architecture");
    const bool v2 = a == "dflash";
    if (a != "dflash-draft" && !v2) return fail(DFL_ERR_UNSUPPORTED, "gguf: unsupported drafter architecture '" + a + "'");
    const std::string p = a + ".";
    G_CHECK(need_u32(g, p + "block_count", &out->n_layer, DFL_MAX_DRAFTER_LAYERS, true));
    G_CHECK(need_u32(g, p + "embedding_length", &out->hidden_size, MAX_ARCH_DIM, true));
    G_CHECK(need_u32(g, p + "feed_forward_length", &out->intermediate_size, MAX_ARCH_DIM, true));
    G_CHECK(need_u32(g, p + "attention.head_count", &out->n_q_heads, MAX_ARCH_DIM, true));
    G_CHECK(need_u32(g, p + "attention.head_count_kv", &out->n_kv_heads, MAX_ARCH_DIM, true));
    G_CHECK(need_u32(g, p + "attention.key_length", &out->head_dim, MAX_ARCH_DIM, true));
    double theta = 10000000.0, eps = 1e-6;
    g->f64(p + "rope.freq_base", &theta);
    out->rope_theta = (float)theta;
    if (g->get((p + "attention.layer_norm_rms_epsilon").c_str()) && !g->f64(p + "attention.layer_norm_rms_epsilon", &eps))
        return fail(DFL_ERR_BAD_SHAPE, "gguf: bad metadata " + p + "attention.layer_norm_rms_epsilon");
    if (!std::isfinite(eps) || eps <= 0.0 || (float)eps == 0.0f) return fail(DFL_ERR_BAD_SHAPE, "gguf: bad metadata " + p + "attention.layer_norm_rms_epsilon");
    out->rms_norm_eps = (float)eps;
    int32_t causal = 1, found = 0;
    G_CHECK(dfl_gguf_get_bool(g, (p + "attention.causal").c_str(), &causal, &found));
    out->causal = found ? (uint32_t)causal : 1u;
    uint64_t win = 0;
    g->u64(p + "attention.sliding_window", &win);
    if (win > UINT32_MAX) return fail(DFL_ERR_BAD_SHAPE, "gguf: sliding_window out of range");
    out->swa_window = (uint32_t)win;
    G_CHECK(need_u32(g, v2 ? "dflash.block_size" : "dflash-draft.dflash.block_size", &out->block_size, DFL_MAX_BLOCK, true));
    uint32_t mask = 0;
    G_CHECK(need_u32(g, v2 ? "tokenizer.ggml.mask_token_id" : "dflash-draft.dflash.mask_token_id", &mask, INT32_MAX, false));
    if (mask >= target->vocab_size) return fail(DFL_ERR_BAD_SHAPE, "gguf: mask_token_id is outside the target vocabulary");
    out->mask_token_id = (int32_t)mask;
    const char* ids_key = v2 ? "dflash.target_layers" : "dflash-draft.dflash.target_layer_ids";
    uint64_t ids[DFL_MAX_TARGET_LAYERS], n_ids = 0;
    G_CHECK(dfl_gguf_get_u64_array(g, ids_key, ids, DFL_MAX_TARGET_LAYERS, &n_ids, &found));
    if (!found || n_ids == 0) return fail(DFL_ERR_BAD_ARG, std::string("gguf: missing metadata ") + ids_key);
    out->n_target_layers = (uint32_t)n_ids;
    for (uint64_t i = 0; i < n_ids; ++i) {
        uint64_t id = ids[i];
        if (v2) {   // the "dflash" format stores layer-input indices (post-block index + 1), loader.rs:1009-1023
            if (id == 0) return fail(DFL_ERR_BAD_SHAPE, "gguf: dflash.target_layers cannot capture layer input 0 as a post-block state");
            --id;
        }
        if (id >= target->n_layer) return fail(DFL_ERR_BAD_SHAPE, "gguf: target layer id is outside the target model");
        out->target_layer_ids[i] = (uint32_t)id;
    }
    uint64_t pat[DFL_MAX_DRAFTER_LAYERS], n_pat = 0;
    G_CHECK(dfl_gguf_get_u64_array(g, (p + "attention.sliding_window_pattern").c_str(), pat, DFL_MAX_DRAFTER_LAYERS, &n_pat, &found));
    if (!found) return fail(DFL_ERR_BAD_ARG, "gguf: missing metadata " + p + "attention.sliding_window_pattern");
    if (n_pat != out->n_layer) return fail(DFL_ERR_BAD_SHAPE, "gguf: sliding_window_pattern length differs from block_count");
    for (uint64_t i = 0; i < n_pat; ++i) out->layer_is_swa[i] = pat[i] ? 1 : 0;
    if (v2 && g->index.count("selector_hidden.weight")) {   // DFlash 2, presence-gated (loader.rs:1025-1060)
        G_CHECK(need_u32(g, "dflash.selector_rank", &out->selector_rank, MAX_ARCH_DIM, true));
        G_CHECK(need_u32(g, "dflash.selector_top_k", &out->selector_top_k, 64, true));
    }
    return DFL_OK;
}

// The drafter file's tensors under the names dfl_drafter_create expects: the "dflash" format's fc.weight,
// enc.output_norm.weight and blk.N.ffn_norm.weight are the "dflash-draft" format's dflash_fc.weight,
// dflash_hidden_norm.weight and blk.N.post_attention_norm.weight (loader.rs:876-912).
dfl_status dfl_gguf_drafter_tensors(dfl_gguf* g, const dfl_tensor** table, uint64_t* count) {
    if (!g || !table || !count) return fail(DFL_ERR_BAD_ARG, "gguf_drafter_tensors: null argument");
    if (g->drafter_tensors.empty()) {
        const bool v2 = g->str("general.architecture") == "dflash";
        g->alias_names.reserve(g->tensors.size());
        for (size_t i = 0; i < g->tensors.size(); ++i) {
            std::string n = g->names[i];
            if (v2) {
                if (n == "fc.weight") n = "dflash_fc.weight";
                else if (n == "enc.output_norm.weight") n = "dflash_hidden_norm.weight";
                else if (n.rfind("blk.", 0) == 0 && n.size() > 16 && n.compare(n.size() - 16, 16, ".ffn_norm.weight") == 0)
                    n = n.substr(0, n.size() - 16) + ".post_attention_norm.weight";
            }
            g->alias_names.push_back(n);
        }
        g->drafter_tensors = g->tensors;
        for (size_t i = 0; i < g->tensors.size(); ++i) g->drafter_tensors[i].name = g->alias_names[i].c_str();
    }
    *table = g->drafter_tensors.data();
    *count = g->drafter_tensors.size();
    return DFL_OK;
}

}  // extern "C"
