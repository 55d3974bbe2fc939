// Read-only GGUF access for the MoE tensors: maps the file (or every shard of a split model),
// indexes tensor name -> {ggml type, shape, bytes}, keeps the scalar and string metadata, and
// hands the eight `blk.N.ffn_*` tensors of a layer to qkm_upload_layer.
//
// What is kept from the reference's reader (src/gguf.h:54-198) is the file format handling:
// GGUF v2/v3 little-endian, `general.alignment` (default 32) for the start of the data section,
// llama-gguf-split shards named "<prefix>-00001-of-000NN.gguf" merged into one directory with
// the metadata taken from the first shard; and from loadMoeT (src/main.cpp:1265-1308) the tensor
// names, the accepted types and where the dimensions come from.  Unlike the reference, every
// length read from the file is checked against the mapping, and errors are returned, not fatal.
// Host-only code.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <new>
#include <string>
#include <vector>

#include "../../include/qk_moe.h"

namespace {

struct Tensor {
    uint32_t type = 0;
    uint64_t ne[4] = {1, 1, 1, 1};
    const uint8_t* data = nullptr;
    uint64_t nbytes = 0;   // bytes available from `data` to the end of its shard
};

struct Shard { const uint8_t* base; size_t size; };

// cursor over one mapped shard; every read is bounds-checked
struct Cursor {
    const uint8_t* base;
    size_t size, pos;
    bool ok = true;
    template <typename T> T rd() {
        T v{};
        if (!ok || size - pos < sizeof(T)) { ok = false; return v; }
        memcpy(&v, base + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t n = rd<uint64_t>();
        if (!ok || n > size - pos) { ok = false; return {}; }
        std::string s(reinterpret_cast<const char*>(base + pos), (size_t)n);
        pos += (size_t)n;
        return s;
    }
};

}  // namespace

struct qkm_gguf {
    std::vector<Shard> shards;
    std::map<std::string, Tensor> tensors;
    std::map<std::string, uint64_t> kv_int;
    std::map<std::string, std::string> kv_str;
    std::string error;

    ~qkm_gguf() {
        for (auto& s : shards) munmap(const_cast<uint8_t*>(s.base), s.size);
    }

    bool fail(const char* fmt, ...) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        error = buf;
        return false;
    }

    // value of a metadata entry of type t; scalars come back as u64 (floats are skipped)
    bool value(Cursor& c, uint32_t t, uint64_t* out, int depth) {
        *out = 0;
        switch (t) {
            case 0: case 1: case 7: *out = c.rd<uint8_t>(); return c.ok;
            case 2: case 3: *out = c.rd<uint16_t>(); return c.ok;
            case 4: case 5: *out = c.rd<uint32_t>(); return c.ok;
            case 6: c.rd<uint32_t>(); return c.ok;               // f32
            case 8: c.str(); return c.ok;
            case 9: {
                if (depth > 2) return false;
                const uint32_t et = c.rd<uint32_t>();
                const uint64_t n = c.rd<uint64_t>();
                if (!c.ok) return false;
                static const int fixed[13] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};
                if (et < 13 && fixed[et]) {                       // fixed-size elements: skip in one step
                    if (n > (c.size - c.pos) / fixed[et]) return false;
                    c.pos += (size_t)n * fixed[et];
                    return true;
                }
                uint64_t dummy;
                for (uint64_t i = 0; i < n; ++i)
                    if (!value(c, et, &dummy, depth + 1)) return false;
                return true;
            }
            case 10: case 11: *out = c.rd<uint64_t>(); return c.ok;
            case 12: c.rd<uint64_t>(); return c.ok;               // f64
            default: return false;
        }
    }

    bool open_one(const std::string& path, bool first, uint64_t* split_count) {
        const int fd = ::open(path.c_str(), O_RDONLY);
        if (fd < 0) return fail("cannot open %s", path.c_str());
        struct stat st;
        if (fstat(fd, &st) != 0 || st.st_size < 24) { ::close(fd); return fail("%s: not a GGUF file", path.c_str()); }
        const size_t size = (size_t)st.st_size;
        void* m = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
        ::close(fd);
        if (m == MAP_FAILED) return fail("%s: mmap failed", path.c_str());
        shards.push_back({static_cast<const uint8_t*>(m), size});
        Cursor c{static_cast<const uint8_t*>(m), size, 0};
        if (memcmp(c.base, "GGUF", 4) != 0) return fail("%s: not a GGUF file", path.c_str());
        c.pos = 4;
        const uint32_t ver = c.rd<uint32_t>();
        if (ver < 2) return fail("%s: GGUF version %u is not supported", path.c_str(), ver);
        const uint64_t n_tensors = c.rd<uint64_t>(), n_kv = c.rd<uint64_t>();
        if (!c.ok || n_tensors > size / 24 || n_kv > size / 12) return fail("%s: corrupt header", path.c_str());
        uint64_t alignment = 32;
        for (uint64_t i = 0; i < n_kv; ++i) {
            const std::string key = c.str();
            const uint32_t t = c.rd<uint32_t>();
            if (!c.ok) return fail("%s: truncated metadata", path.c_str());
            if (t == 8) {
                const std::string v = c.str();
                if (!c.ok) return fail("%s: truncated metadata", path.c_str());
                if (first) kv_str[key] = v;
                continue;
            }
            uint64_t v = 0;
            if (!value(c, t, &v, 0)) return fail("%s: bad metadata entry '%s'", path.c_str(), key.c_str());
            const bool is_int = t <= 5 || t == 7 || t == 10 || t == 11;
            if (is_int && first) kv_int[key] = v;
            if (is_int && key == "general.alignment" && v) alignment = v;
            if (is_int && key == "split.count" && split_count) *split_count = v;
        }
        if (alignment == 0 || alignment > (1u << 20) || (alignment & (alignment - 1))) return fail("%s: bad alignment", path.c_str());
        struct Info { std::string name; Tensor t; uint64_t off; };
        std::vector<Info> infos((size_t)n_tensors);
        for (auto& inf : infos) {
            inf.name = c.str();
            const uint32_t nd = c.rd<uint32_t>();
            if (!c.ok || nd > 4) return fail("%s: bad tensor entry", path.c_str());
            for (uint32_t d = 0; d < nd; ++d) inf.t.ne[d] = c.rd<uint64_t>();
            inf.t.type = c.rd<uint32_t>();
            inf.off = c.rd<uint64_t>();
            if (!c.ok) return fail("%s: truncated tensor directory", path.c_str());
        }
        const uint64_t data_start = (c.pos + alignment - 1) / alignment * alignment;
        for (auto& inf : infos) {
            if (data_start > size || inf.off > size - data_start) return fail("%s: tensor '%s' lies outside the file", path.c_str(), inf.name.c_str());
            inf.t.data = c.base + data_start + inf.off;
            inf.t.nbytes = size - data_start - inf.off;
            tensors[inf.name] = inf.t;
        }
        return true;
    }

    bool open(const std::string& path) {
        uint64_t split = 0;
        if (!open_one(path, true, &split)) return false;
        if (split > 1) {
            // "<prefix>-00001-of-000NN.gguf": the sibling shards follow from the name
            const char* marker = "-00001-of-";
            const size_t tp = path.rfind(marker);
            if (split > 99999 || tp == std::string::npos || path.size() != tp + 20 || path.compare(path.size() - 5, 5, ".gguf") != 0)
                return fail("split.count=%llu but %s is not a -00001-of-NNNNN.gguf first shard", (unsigned long long)split, path.c_str());
            const std::string prefix = path.substr(0, tp);
            for (uint64_t i = 2; i <= split; ++i) {
                char name[64];
                snprintf(name, sizeof name, "-%05u-of-%05u.gguf", (unsigned)i, (unsigned)split);
                if (!open_one(prefix + name, false, nullptr)) return false;
            }
        }
        return true;
    }
};

extern "C" QKM_API qkm_gguf* qkm_gguf_open(const char* path, char* err, size_t err_len) {
    if (err && err_len) err[0] = 0;
    if (!path) { if (err && err_len) snprintf(err, err_len, "NULL path"); return nullptr; }
    qkm_gguf* g = new (std::nothrow) qkm_gguf();
    if (!g) return nullptr;
    if (!g->open(path)) {
        if (err && err_len) snprintf(err, err_len, "%s", g->error.c_str());
        delete g;
        return nullptr;
    }
    return g;
}

extern "C" QKM_API void qkm_gguf_close(qkm_gguf* g) { delete g; }

extern "C" QKM_API const char* qkm_gguf_last_error(const qkm_gguf* g) { return g ? g->error.c_str() : "NULL file"; }

extern "C" QKM_API uint64_t qkm_gguf_tensor_count(const qkm_gguf* g) { return g ? g->tensors.size() : 0; }

extern "C" QKM_API int qkm_gguf_find(const qkm_gguf* g, const char* name, uint32_t* type, uint64_t ne[4],
                                     const void** data, uint64_t* nbytes) {
    if (!g || !name) return QKM_ERR_ARG;
    const auto it = g->tensors.find(name);
    if (it == g->tensors.end()) return QKM_ERR_BOUNDS;
    if (type) *type = it->second.type;
    if (ne) for (int i = 0; i < 4; ++i) ne[i] = it->second.ne[i];
    if (data) *data = it->second.data;
    if (nbytes) *nbytes = it->second.nbytes;
    return QKM_OK;
}

extern "C" QKM_API uint64_t qkm_gguf_kv_u64(const qkm_gguf* g, const char* key, uint64_t def) {
    if (!g || !key) return def;
    const auto it = g->kv_int.find(key);
    return it == g->kv_int.end() ? def : it->second;
}

extern "C" QKM_API int qkm_gguf_kv_str(const qkm_gguf* g, const char* key, char* out, size_t out_len) {
    if (!g || !key || !out || !out_len) return QKM_ERR_ARG;
    const auto it = g->kv_str.find(key);
    if (it == g->kv_str.end()) { out[0] = 0; return QKM_ERR_BOUNDS; }
    snprintf(out, out_len, "%s", it->second.c_str());
    return QKM_OK;
}

// The eight MoE tensors of `blk.<layer>` with the checks loadMoeT makes: all present, router and
// shared gate F32 (F16 router also taken), gate/up both IQ3_XXS or both IQ4_XS, down IQ4_XS or
// Q6_K, shared expert Q8_0, top-k from "<arch>.expert_used_count" (default 8) in 1..16; plus
// what the reference leaves to luck: shapes consistent and every tensor's bytes inside the file.
extern "C" QKM_API int qkm_gguf_moe_layer(qkm_gguf* g, uint32_t layer, qkm_dims* dims, qkm_layer_weights* w) {
    if (!g || !dims || !w) return QKM_ERR_ARG;
    static const char* suffix[8] = {"ffn_gate_inp.weight", "ffn_gate_inp_shexp.weight", "ffn_gate_exps.weight",
                                    "ffn_up_exps.weight", "ffn_down_exps.weight", "ffn_gate_shexp.weight",
                                    "ffn_up_shexp.weight", "ffn_down_shexp.weight"};
    const Tensor* t[8];
    for (int i = 0; i < 8; ++i) {
        char name[128];
        snprintf(name, sizeof name, "blk.%u.%s", layer, suffix[i]);
        const auto it = g->tensors.find(name);
        if (it == g->tensors.end()) { g->fail("layer %u: missing tensor %s", layer, name); return QKM_ERR_BOUNDS; }
        t[i] = &it->second;
    }
    const bool gu3 = t[2]->type == QKM_TYPE_IQ3_XXS && t[3]->type == QKM_TYPE_IQ3_XXS;
    const bool gu4 = t[2]->type == QKM_TYPE_IQ4_XS && t[3]->type == QKM_TYPE_IQ4_XS;
    if ((t[0]->type != QKM_TYPE_F32 && t[0]->type != QKM_TYPE_F16) || t[1]->type != QKM_TYPE_F32 || (!gu3 && !gu4) ||
        (t[4]->type != QKM_TYPE_IQ4_XS && t[4]->type != QKM_TYPE_Q6_K) || t[5]->type != QKM_TYPE_Q8_0 ||
        t[6]->type != QKM_TYPE_Q8_0 || t[7]->type != QKM_TYPE_Q8_0) {
        g->fail("layer %u: unexpected MoE tensor types", layer);
        return QKM_ERR_TYPE;
    }
    // Dimensions are range-checked as 64-bit values before anything is narrowed or multiplied:
    // a crafted header must not wrap a size computation (limits: what qkm_open accepts, with
    // rows of at most 2^20 elements).
    const uint64_t kMaxDim = 1u << 20;
    if (t[2]->ne[0] < 256 || t[2]->ne[0] > kMaxDim || t[2]->ne[0] % 256 || t[2]->ne[1] < 256 || t[2]->ne[1] > kMaxDim ||
        t[2]->ne[1] % 256 || t[2]->ne[2] < 1 || t[2]->ne[2] > 512) {
        g->fail("layer %u: MoE tensor dims out of range (n_embd, n_ff multiples of 256 up to 2^20; at most 512 experts)", layer);
        return QKM_ERR_BOUNDS;
    }
    qkm_dims d;
    d.n_embd = (uint32_t)t[2]->ne[0];
    d.n_ff = (uint32_t)t[2]->ne[1];
    d.n_expert = (uint32_t)t[2]->ne[2];
    const auto arch = g->kv_str.find("general.architecture");
    const std::string key = (arch == g->kv_str.end() ? std::string() : arch->second) + ".expert_used_count";
    d.n_used = (uint32_t)qkm_gguf_kv_u64(g, key.c_str(), 8);
    if (d.n_used < 1 || d.n_used > 16 || d.n_used > d.n_expert) { g->fail("layer %u: expert_used_count %u unsupported", layer, d.n_used); return QKM_ERR_BOUNDS; }
    auto shape = [&](int i, uint64_t a, uint64_t b, uint64_t c) {
        return t[i]->ne[0] == a && t[i]->ne[1] == b && t[i]->ne[2] == c && t[i]->ne[3] == 1;
    };
    if (!shape(0, d.n_embd, d.n_expert, 1) || !shape(1, d.n_embd, 1, 1) || !shape(2, d.n_embd, d.n_ff, d.n_expert) ||
        !shape(3, d.n_embd, d.n_ff, d.n_expert) || !shape(4, d.n_ff, d.n_embd, d.n_expert) || !shape(5, d.n_embd, d.n_ff, 1) ||
        !shape(6, d.n_embd, d.n_ff, 1) || !shape(7, d.n_ff, d.n_embd, 1)) {
        g->fail("layer %u: inconsistent MoE tensor shapes", layer);
        return QKM_ERR_BOUNDS;
    }
    // every extent is now <= 2^20 (ne[2] <= 512), so rb * ne[1] * ne[2] < 2^23 * 2^20 * 2^9 = 2^52
    for (int i = 0; i < 8; ++i) {
        const size_t rb = qkm_row_bytes(t[i]->type, t[i]->ne[0]);
        const uint64_t need = (uint64_t)rb * t[i]->ne[1] * t[i]->ne[2];
        if (rb == 0 || need > t[i]->nbytes) { g->fail("layer %u: tensor %s is truncated", layer, suffix[i]); return QKM_ERR_BOUNDS; }
    }
    *dims = d;
    memset(w, 0, sizeof *w);
    w->router_type = t[0]->type;
    w->gateup_type = t[2]->type;
    w->down_type = t[4]->type;
    w->router = t[0]->data;
    w->gate_inp_shexp = reinterpret_cast<const float*>(t[1]->data);
    w->gate_exps = t[2]->data; w->up_exps = t[3]->data; w->down_exps = t[4]->data;
    w->gate_shexp = t[5]->data; w->up_shexp = t[6]->data; w->down_shexp = t[7]->data;
    return QKM_OK;
}

// Layer `file_layer` of the file into slot `layer` of the context.  A sharded context
// (expert_first / expert_count at open) takes its slice of the three expert tensors.
extern "C" QKM_API int qkm_upload_layer_gguf(qkm_ctx* c, uint32_t layer, qkm_gguf* g, uint32_t file_layer) {
    if (!c || !g) return QKM_ERR_ARG;
    qkm_dims d;
    qkm_layer_weights w;
    if (int rc = qkm_gguf_moe_layer(g, file_layer, &d, &w)) return rc;
    if (d.n_embd != qkm_n_embd(c) || d.n_ff != qkm_n_ff(c) || d.n_expert != qkm_n_expert(c) || d.n_used != qkm_n_used(c)) {
        g->fail("layer %u: file dims %u/%u/%u/%u differ from the context's", file_layer, d.n_embd, d.n_ff, d.n_expert, d.n_used);
        return QKM_ERR_BOUNDS;
    }
    uint32_t first = 0, count = 0;
    qkm_expert_range(c, &first, &count);
    const size_t gu = (size_t)d.n_ff * qkm_row_bytes(w.gateup_type, d.n_embd), dn = (size_t)d.n_embd * qkm_row_bytes(w.down_type, d.n_ff);
    w.gate_exps = static_cast<const uint8_t*>(w.gate_exps) + (size_t)first * gu;
    w.up_exps = static_cast<const uint8_t*>(w.up_exps) + (size_t)first * gu;
    w.down_exps = static_cast<const uint8_t*>(w.down_exps) + (size_t)first * dn;
    return qkm_upload_layer(c, layer, &w);
}
