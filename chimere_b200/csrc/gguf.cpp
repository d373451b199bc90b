// GGUF tensor directory and the MoE tensors of one layer: what the reference's loader does for this path
// (src/gguf_loader.rs:286-455 parses the header, the metadata and the tensor infos; compute_graph.rs:992-999 and
// :1400-1500 pick blk.{L}.ffn_gate_inp / ffn_{gate,up,down}_exps / ffn_*_shexp / ffn_gate_inp_shexp and upload their
// bytes untouched).  Host code only: the file is parsed with buffered reads, tensor bytes are read with pread() into
// the caller's (pinned) buffer; packing for the kernels is chimere_b200_moe_pack_*'s job.
//
// File layout (GGUF v2/v3, little endian): "GGUF", u32 version, u64 n_tensors, u64 n_kv; n_kv x { string key, u32 type,
// value }; n_tensors x { string name, u32 n_dims, u64 dims[n_dims] (innermost first), u32 ggml type, u64 offset };
// padding to general.alignment (default 32); tensor data, offsets relative to that point.
#include <fcntl.h>
#include <unistd.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/chimere_b200_moe.h"

namespace {

enum { kErrArg = -1, kErrShape = -2, kErrIo = -9, kErrFormat = -10, kErrMissing = -11 };

struct TypeInfo { int block, bytes; };
// block size and bytes per block by ggml type id (gguf_loader.rs:159-193); {0,0} = not known here
TypeInfo type_info(int t) {
    switch (t) {
        case 0: return {1, 4};      // F32
        case 1: return {1, 2};      // F16
        case 2: return {32, 18};    // Q4_0
        case 3: return {32, 20};    // Q4_1
        case 6: return {32, 22};    // Q5_0
        case 7: return {32, 24};    // Q5_1
        case 8: return {32, 34};    // Q8_0
        case 10: return {256, 84};  // Q2_K
        case 11: return {256, 110}; // Q3_K
        case 12: return {256, 144}; // Q4_K
        case 13: return {256, 176}; // Q5_K
        case 14: return {256, 210}; // Q6_K
        case 16: return {256, 66};  // IQ2_XXS
        case 17: return {256, 74};  // IQ2_XS
        case 18: return {256, 98};  // IQ3_XXS
        case 19: return {256, 50};  // IQ1_S
        case 20: return {32, 18};   // IQ4_NL
        case 21: return {256, 110}; // IQ3_S
        case 22: return {256, 82};  // IQ2_S
        case 23: return {256, 136}; // IQ4_XS
        case 24: return {1, 1};     // I8
        case 25: return {1, 2};     // I16
        case 26: return {1, 4};     // I32
        case 27: return {1, 8};     // I64
        case 28: return {1, 8};     // F64
        case 29: return {256, 56};  // IQ1_M
        case 30: return {1, 2};     // BF16
        default: return {0, 0};
    }
}

struct Reader {
    FILE* f;
    bool ok = true;
    template <typename T> T get() {
        T v{};
        if (ok && fread(&v, sizeof(T), 1, f) != 1) ok = false;
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (!ok || n > (1u << 20)) { ok = false; return {}; }
        std::string s(n, '\0');
        if (n && fread(&s[0], 1, n, f) != n) ok = false;
        return s;
    }
    void skip(uint64_t n) { if (ok && fseeko(f, (off_t)n, SEEK_CUR) != 0) ok = false; }
};

int scalar_size(uint32_t t) {
    switch (t) {
        case 0: case 1: case 7: return 1;   // u8, i8, bool
        case 2: case 3: return 2;           // u16, i16
        case 4: case 5: case 6: return 4;   // u32, i32, f32
        case 10: case 11: case 12: return 8; // u64, i64, f64
        default: return 0;
    }
}

}  // namespace

struct chimere_gguf {
    int fd = -1;
    uint32_t version = 0;
    uint64_t alignment = 32;
    int64_t data_start = 0, file_size = 0;
    std::vector<std::string> names;
    std::vector<chimere_gguf_tensor> tensors;
    std::unordered_map<std::string, size_t> index;
    std::unordered_map<std::string, uint64_t> int_meta;     // every integer-valued key
    std::unordered_map<std::string, std::string> str_meta;  // every string-valued key
};

extern "C" {

int chimere_b200_gguf_open(const char* path, chimere_gguf** out) {
    if (!path || !out) return kErrArg;
    *out = nullptr;
    FILE* f = fopen(path, "rb");
    if (!f) return kErrIo;
    Reader r{f};
    chimere_gguf* g = new chimere_gguf();
    auto fail = [&](int code) { fclose(f); delete g; return code; };
    char magic[4] = {};
    if (fread(magic, 1, 4, f) != 4 || memcmp(magic, "GGUF", 4) != 0) return fail(kErrFormat);
    g->version = r.get<uint32_t>();
    if (g->version < 2 || g->version > 3) return fail(kErrFormat);
    const uint64_t n_tensors = r.get<uint64_t>(), n_kv = r.get<uint64_t>();
    if (!r.ok || n_tensors > (1u << 24) || n_kv > (1u << 24)) return fail(kErrFormat);
    for (uint64_t i = 0; i < n_kv && r.ok; ++i) {
        const std::string key = r.str();
        const uint32_t t = r.get<uint32_t>();
        if (t == 8) { g->str_meta[key] = r.str(); continue; }
        if (t == 9) {   // array: element type, count, elements
            const uint32_t et = r.get<uint32_t>();
            const uint64_t n = r.get<uint64_t>();
            if (et == 8) { for (uint64_t k = 0; k < n && r.ok; ++k) r.skip(r.get<uint64_t>()); }
            else if (scalar_size(et)) r.skip(n * scalar_size(et));
            else r.ok = false;
            continue;
        }
        const int sz = scalar_size(t);
        if (!sz) { r.ok = false; break; }
        uint64_t raw = 0;
        if (fread(&raw, 1, sz, f) != (size_t)sz) { r.ok = false; break; }
        if (t == 1) raw = (uint64_t)(int64_t)(int8_t)raw;
        else if (t == 3) raw = (uint64_t)(int64_t)(int16_t)raw;
        else if (t == 5) raw = (uint64_t)(int64_t)(int32_t)raw;
        if (t != 6 && t != 12) g->int_meta[key] = raw;
    }
    if (!r.ok) return fail(kErrFormat);
    auto al = g->int_meta.find("general.alignment");
    if (al != g->int_meta.end() && al->second > 0) g->alignment = al->second;
    g->names.reserve(n_tensors);
    g->tensors.reserve(n_tensors);
    for (uint64_t i = 0; i < n_tensors && r.ok; ++i) {
        std::string name = r.str();
        chimere_gguf_tensor t{};
        const uint32_t nd = r.get<uint32_t>();
        if (!r.ok || nd > 4) { r.ok = false; break; }
        t.n_dims = (int32_t)nd;
        int64_t n_el = 1;
        for (int d = 0; d < 4; ++d) t.dims[d] = 1;
        for (uint32_t d = 0; d < nd; ++d) {
            t.dims[d] = (int64_t)r.get<uint64_t>();
            if (t.dims[d] < 0 || __builtin_mul_overflow(n_el, t.dims[d], &n_el)) r.ok = false;   // (a foreign or damaged file)
        }
        if (!r.ok) break;
        t.ggml_type = (int32_t)r.get<uint32_t>();
        t.file_offset = (int64_t)r.get<uint64_t>();   // relative for now
        const TypeInfo ti = type_info(t.ggml_type);
        t.nbytes = ti.block ? n_el / ti.block * ti.bytes : -1;
        if (ti.block && (t.dims[0] % ti.block)) r.ok = false;
        g->index[name] = g->tensors.size();
        g->names.push_back(std::move(name));
        g->tensors.push_back(t);
    }
    if (!r.ok) return fail(kErrFormat);
    const int64_t header_end = (int64_t)ftello(f);
    g->data_start = (header_end + (int64_t)g->alignment - 1) / (int64_t)g->alignment * (int64_t)g->alignment;
    fseeko(f, 0, SEEK_END);
    g->file_size = (int64_t)ftello(f);
    fclose(f);
    for (auto& t : g->tensors) {
        t.file_offset += g->data_start;
        if (t.nbytes >= 0 && t.file_offset + t.nbytes > g->file_size) { delete g; return kErrFormat; }
    }
    g->fd = open(path, O_RDONLY);
    if (g->fd < 0) { delete g; return kErrIo; }
    *out = g;
    return 0;
}

void chimere_b200_gguf_close(chimere_gguf* g) {
    if (!g) return;
    if (g->fd >= 0) close(g->fd);
    delete g;
}

int64_t chimere_b200_gguf_n_tensors(const chimere_gguf* g) { return g ? (int64_t)g->tensors.size() : kErrArg; }

int chimere_b200_gguf_tensor_name(const chimere_gguf* g, int64_t i, char* buf, int buflen) {
    if (!g || !buf || buflen <= 0 || i < 0 || i >= (int64_t)g->names.size()) return kErrArg;
    snprintf(buf, (size_t)buflen, "%s", g->names[(size_t)i].c_str());
    return (int)g->names[(size_t)i].size();
}

int chimere_b200_gguf_find(const chimere_gguf* g, const char* name, chimere_gguf_tensor* out) {
    if (!g || !name || !out) return kErrArg;
    auto it = g->index.find(name);
    if (it == g->index.end()) return kErrMissing;
    *out = g->tensors[it->second];
    return 0;
}

int chimere_b200_gguf_read(const chimere_gguf* g, const chimere_gguf_tensor* t, void* dst, int64_t dst_bytes) {
    if (!g || !t || !dst || t->nbytes < 0) return kErrArg;
    if (dst_bytes < t->nbytes) return kErrShape;
    int64_t done = 0;
    while (done < t->nbytes) {
        const ssize_t n = pread(g->fd, (char*)dst + done, (size_t)(t->nbytes - done), (off_t)(t->file_offset + done));
        if (n <= 0) return kErrIo;
        done += n;
    }
    return 0;
}

int chimere_b200_gguf_meta_u64(const chimere_gguf* g, const char* key, uint64_t* out) {
    if (!g || !key || !out) return kErrArg;
    auto it = g->int_meta.find(key);
    if (it == g->int_meta.end()) return kErrMissing;
    *out = it->second;
    return 0;
}

int chimere_b200_gguf_meta_str(const chimere_gguf* g, const char* key, char* buf, int buflen) {
    if (!g || !key || !buf || buflen <= 0) return kErrArg;
    auto it = g->str_meta.find(key);
    if (it == g->str_meta.end()) return kErrMissing;
    snprintf(buf, (size_t)buflen, "%s", it->second.c_str());
    return (int)it->second.size();
}

// The MoE tensors of layer `layer`, shapes checked against each other:
//   router  blk.L.ffn_gate_inp.weight        F32  [H, E]
//   experts blk.L.ffn_{gate,up}_exps.weight  [H, F, E],  blk.L.ffn_down_exps.weight [F, H, E]   (gate absent: ungated experts)
//   shared  blk.L.ffn_{gate,up}_shexp.weight [H, F_s], blk.L.ffn_down_shexp.weight [F_s, H], blk.L.ffn_gate_inp_shexp.weight F32 [H]
int chimere_b200_gguf_moe_layer(const chimere_gguf* g, int layer, chimere_gguf_moe_layer* out) {
    if (!g || !out || layer < 0) return kErrArg;
    memset(out, 0, sizeof(*out));
    auto find = [&](const char* what, chimere_gguf_tensor* t) {
        char name[96];
        snprintf(name, sizeof(name), "blk.%d.%s.weight", layer, what);
        return chimere_b200_gguf_find(g, name, t) == 0;
    };
    if (!find("ffn_gate_inp", &out->router) || !find("ffn_up_exps", &out->up_exps) || !find("ffn_down_exps", &out->down_exps)) return kErrMissing;
    out->has_gate = find("ffn_gate_exps", &out->gate_exps) ? 1 : 0;
    const chimere_gguf_tensor &r = out->router, &u = out->up_exps, &d = out->down_exps;
    if (r.ggml_type != 0 || r.n_dims != 2 || u.n_dims != 3 || d.n_dims != 3) return kErrShape;
    out->H = (int)r.dims[0]; out->E = (int)r.dims[1]; out->F = (int)u.dims[1];
    if (u.dims[0] != out->H || u.dims[2] != out->E || d.dims[0] != out->F || d.dims[1] != out->H || d.dims[2] != out->E) return kErrShape;
    if (out->has_gate) {
        const chimere_gguf_tensor& ga = out->gate_exps;
        if (ga.n_dims != 3 || ga.dims[0] != u.dims[0] || ga.dims[1] != u.dims[1] || ga.dims[2] != u.dims[2] || ga.ggml_type != u.ggml_type) return kErrShape;
    }
    out->has_shared = find("ffn_up_shexp", &out->sh_up) ? 1 : 0;
    if (out->has_shared) {
        if (!find("ffn_down_shexp", &out->sh_down)) return kErrMissing;
        out->has_shared_gate = find("ffn_gate_shexp", &out->sh_gate) ? 1 : 0;
        out->has_shared_gate_proj = find("ffn_gate_inp_shexp", &out->sh_gate_proj) ? 1 : 0;
        out->F_s = (int)out->sh_up.dims[1];
        if (out->sh_up.dims[0] != out->H || out->sh_down.dims[0] != out->F_s || out->sh_down.dims[1] != out->H) return kErrShape;
        if (out->has_shared_gate && (out->sh_gate.dims[0] != out->H || out->sh_gate.dims[1] != out->F_s)) return kErrShape;
        if (out->has_shared_gate_proj && (out->sh_gate_proj.ggml_type != 0 || out->sh_gate_proj.dims[0] != out->H)) return kErrShape;
    }
    return 0;
}

}  // extern "C"
