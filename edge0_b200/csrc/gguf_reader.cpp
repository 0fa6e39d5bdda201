// Reader for GGUF model files (version 2 and 3), the container edge0-infer loads its weights from through ggml's gguf API
// (edge0-infer/src/model/asset_index.cpp; format: third_party/ggml/docs/gguf.md, written by third_party/ggml/src/gguf.cpp).
// Host code only.  The file is mapped read-only; a tensor is handed out as a pointer into the mapping, in ggml's block layout -
// which is the layout the kernels read, so loading a layer is a copy per tensor and no repacking.
//
//   header   : magic "GGUF", u32 version, u64 tensor count, u64 key/value count
//   metadata : key (string = u64 length + bytes), u32 value type, value (scalars, string, or array = u32 type + u64 count + items)
//   tensors  : name (string), u32 n_dims, u64 ne[n_dims], u32 ggml type, u64 offset into the data section
//   data     : starts at the next multiple of general.alignment (default 32) behind the tensor table
#include "../../include/edge0_b200_moe.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

namespace {

struct TensorInfo {
    int32_t type = 0;
    int64_t ne[4] = {1, 1, 1, 1};
    uint64_t offset = 0;     // from the start of the data section
    uint64_t nbytes = 0;
};

// block size (values) and block bytes of the ggml types this library reads; 0 = a type it has no use for
bool type_traits(int32_t type, int64_t & blck, int64_t & bytes) {
    switch (type) {
        case 0:  blck = 1;   bytes = 4;   return true;   // F32
        case 1:  blck = 1;   bytes = 2;   return true;   // F16
        case 30: blck = 1;   bytes = 2;   return true;   // BF16
        case 8:  blck = 32;  bytes = 34;  return true;   // Q8_0
        case 11: blck = 256; bytes = 110; return true;   // Q3_K
        case 40: blck = 64;  bytes = 36;  return true;   // NVFP4
        case 24: blck = 1;   bytes = 1;   return true;   // I8
        case 26: blck = 1;   bytes = 4;   return true;   // I32
        default: return false;
    }
}

struct Cursor {
    const uint8_t * p;
    const uint8_t * end;
    bool ok = true;
    template <typename T>
    T get() {
        T v{};
        if (!ok || (size_t) (end - p) < sizeof(T)) { ok = false; return v; }
        memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (!ok || (uint64_t) (end - p) < n) { ok = false; return {}; }
        std::string s(reinterpret_cast<const char *>(p), (size_t) n);
        p += n;
        return s;
    }
    void skip(uint64_t n) {
        if (!ok || (uint64_t) (end - p) < n) { ok = false; return; }
        p += n;
    }
};

size_t scalar_size(uint32_t t) {
    switch (t) {
        case 0: case 1: case 7: return 1;     // u8, i8, bool
        case 2: case 3: return 2;             // u16, i16
        case 4: case 5: case 6: return 4;     // u32, i32, f32
        case 10: case 11: case 12: return 8;  // u64, i64, f64
        default: return 0;
    }
}

}  // namespace

struct b200moe_gguf {
    int fd = -1;
    const uint8_t * base = nullptr;
    size_t size = 0;
    uint64_t data_start = 0;
    uint32_t version = 0;
    std::map<std::string, TensorInfo> tensors;
    std::map<std::string, uint64_t> u_values;      // unsigned / signed integer metadata
    std::map<std::string, std::string> s_values;   // string metadata
};

namespace {

int fail(char * err, size_t err_len, int code, const char * fmt, ...) {
    if (err && err_len) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(err, err_len, fmt, ap);
        va_end(ap);
    }
    return code;
}

void skip_value(Cursor & c, uint32_t type, b200moe_gguf * g, const std::string * key) {
    if (type == 8) {                       // string
        std::string s = c.str();
        if (key) g->s_values[*key] = s;
    } else if (type == 9) {                // array
        const uint32_t it = c.get<uint32_t>();
        const uint64_t n = c.get<uint64_t>();
        if (it == 8) { for (uint64_t i = 0; i < n && c.ok; ++i) c.str(); }
        else if (scalar_size(it)) c.skip(n * scalar_size(it));
        else c.ok = false;                 // nested arrays do not occur in model files
    } else if (const size_t sz = scalar_size(type)) {
        uint64_t v = 0;
        if (c.ok && (size_t) (c.end - c.p) >= sz) memcpy(&v, c.p, sz);
        c.skip(sz);
        if (key && type != 6 && type != 12) g->u_values[*key] = v;
    } else {
        c.ok = false;
    }
}

}  // namespace

extern "C" {

int b200moe_gguf_open(const char * path, b200moe_gguf ** out, char * err, size_t err_len) {
    if (!out) return B200MOE_ERR_INVALID_ARG;
    *out = nullptr;
    if (!path) return fail(err, err_len, B200MOE_ERR_INVALID_ARG, "null path");
    b200moe_gguf * g = new b200moe_gguf();
    auto bail = [&](int code, const char * what) {
        const int rc = fail(err, err_len, code, "%s: %s", path, what);
        b200moe_gguf_close(g);
        return rc;
    };
    g->fd = open(path, O_RDONLY);
    if (g->fd < 0) return bail(B200MOE_ERR_INVALID_ARG, "cannot open");
    struct stat st;
    if (fstat(g->fd, &st) != 0 || st.st_size < 24) return bail(B200MOE_ERR_INVALID_ARG, "not a GGUF file (too short)");
    g->size = (size_t) st.st_size;
    void * m = mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (m == MAP_FAILED) return bail(B200MOE_ERR_ALLOC, "cannot map");
    g->base = static_cast<const uint8_t *>(m);
    Cursor c{ g->base, g->base + g->size };
    if (memcmp(c.p, "GGUF", 4) != 0) return bail(B200MOE_ERR_INVALID_ARG, "not a GGUF file (magic)");
    c.skip(4);
    g->version = c.get<uint32_t>();
    if (g->version != 2 && g->version != 3) return bail(B200MOE_ERR_UNSUPPORTED, "unsupported GGUF version");
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    if (!c.ok || n_tensors > (1u << 24) || n_kv > (1u << 24)) return bail(B200MOE_ERR_INVALID_ARG, "implausible header");
    for (uint64_t i = 0; i < n_kv && c.ok; ++i) {
        const std::string key = c.str();
        const uint32_t type = c.get<uint32_t>();
        skip_value(c, type, g, &key);
    }
    if (!c.ok) return bail(B200MOE_ERR_INVALID_ARG, "truncated or malformed metadata");
    for (uint64_t i = 0; i < n_tensors && c.ok; ++i) {
        const std::string name = c.str();
        TensorInfo t;
        const uint32_t nd = c.get<uint32_t>();
        if (nd > 4) { c.ok = false; break; }
        for (uint32_t d = 0; d < nd; ++d) t.ne[d] = (int64_t) c.get<uint64_t>();
        t.type = (int32_t) c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        int64_t blck = 0, bytes = 0;
        if (type_traits(t.type, blck, bytes) && t.ne[0] > 0 && t.ne[0] % blck == 0)
            t.nbytes = (uint64_t) (t.ne[0] / blck * bytes) * (uint64_t) t.ne[1] * (uint64_t) t.ne[2] * (uint64_t) t.ne[3];
        g->tensors[name] = t;            // nbytes stays 0 for types this library does not read
    }
    if (!c.ok) return bail(B200MOE_ERR_INVALID_ARG, "truncated or malformed tensor table");
    uint64_t align = 32;
    auto a = g->u_values.find("general.alignment");
    if (a != g->u_values.end() && a->second > 0) align = a->second;
    const uint64_t pos = (uint64_t) (c.p - g->base);
    g->data_start = (pos + align - 1) / align * align;
    for (auto & kv : g->tensors)
        if (kv.second.nbytes && (g->data_start + kv.second.offset + kv.second.nbytes > g->size || kv.second.offset % align))
            return bail(B200MOE_ERR_INVALID_ARG, "tensor data outside the file or misaligned");
    *out = g;
    return B200MOE_OK;
}

void b200moe_gguf_close(b200moe_gguf * g) {
    if (!g) return;
    if (g->base) munmap(const_cast<uint8_t *>(g->base), g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

int64_t b200moe_gguf_n_tensors(const b200moe_gguf * g) { return g ? (int64_t) g->tensors.size() : -1; }

int b200moe_gguf_tensor(const b200moe_gguf * g, const char * name, int32_t * type, int64_t ne[4], const void ** data, uint64_t * nbytes) {
    if (!g || !name) return B200MOE_ERR_INVALID_ARG;
    auto it = g->tensors.find(name);
    if (it == g->tensors.end()) return B200MOE_ERR_INVALID_ARG;
    const TensorInfo & t = it->second;
    if (type) *type = t.type;
    if (ne) memcpy(ne, t.ne, sizeof t.ne);
    if (nbytes) *nbytes = t.nbytes;
    if (data) *data = t.nbytes ? g->base + g->data_start + t.offset : nullptr;
    return t.nbytes ? B200MOE_OK : B200MOE_ERR_UNSUPPORTED;
}

int b200moe_gguf_metadata_u64(const b200moe_gguf * g, const char * key, uint64_t * value) {
    if (!g || !key || !value) return B200MOE_ERR_INVALID_ARG;
    auto it = g->u_values.find(key);
    if (it == g->u_values.end()) return B200MOE_ERR_INVALID_ARG;
    *value = it->second;
    return B200MOE_OK;
}

int b200moe_gguf_moe_layer(const b200moe_gguf * g, int32_t layer, int32_t n_expert_used, b200moe_layer * out, char * err, size_t err_len) {
    if (!g || !out || layer < 0) return fail(err, err_len, B200MOE_ERR_INVALID_ARG, "null argument or negative layer");
    memset(out, 0, sizeof *out);
    const std::string prefix = "blk." + std::to_string(layer) + ".";
    struct Got { int32_t type; int64_t ne[4]; const void * data; uint64_t nbytes; };
    auto find = [&](const char * suffix, Got & t) {
        return b200moe_gguf_tensor(g, (prefix + suffix).c_str(), &t.type, t.ne, &t.data, &t.nbytes);
    };
    Got router{}, gate{}, up{}, down{};
    if (find("ffn_gate_inp.weight", router) || find("ffn_gate_exps.weight", gate) || find("ffn_up_exps.weight", up) || find("ffn_down_exps.weight", down))
        return fail(err, err_len, B200MOE_ERR_INVALID_ARG, "block %d lacks ffn_gate_inp / ffn_gate_exps / ffn_up_exps / ffn_down_exps (or holds a type without a kernel)", layer);
    if (router.type != B200MOE_TYPE_F32) return fail(err, err_len, B200MOE_ERR_UNSUPPORTED, "router of block %d is not F32", layer);
    const int64_t n_embd = gate.ne[0], n_ff = gate.ne[1], n_expert = gate.ne[2];
    if (gate.type != up.type || gate.type != down.type || up.ne[0] != n_embd || up.ne[1] != n_ff || up.ne[2] != n_expert || down.ne[0] != n_ff ||
        down.ne[1] != n_embd || down.ne[2] != n_expert || router.ne[0] != n_embd || router.ne[1] != n_expert)
        return fail(err, err_len, B200MOE_ERR_INVALID_ARG, "expert tensors of block %d disagree in type or shape", layer);
    if (n_expert_used <= 0) {           // <architecture>.expert_used_count, as edge0-infer reads it (models/edge0_35b/assets.cpp:63-66)
        auto arch = g->s_values.find("general.architecture");
        uint64_t v = 0;
        if (arch == g->s_values.end() || b200moe_gguf_metadata_u64(g, (arch->second + ".expert_used_count").c_str(), &v) || v == 0)
            return fail(err, err_len, B200MOE_ERR_INVALID_ARG, "n_expert_used not given and no <architecture>.expert_used_count in the file");
        n_expert_used = (int32_t) v;
    }
    out->n_embd = (int32_t) n_embd; out->n_expert = (int32_t) n_expert; out->n_expert_used = n_expert_used; out->n_ff = (int32_t) n_ff;
    out->wtype = gate.type;
    out->router_w = static_cast<const float *>(router.data);
    out->gate = gate.data; out->up = up.data; out->down = down.data;
    Got bias{};
    if (!find("exp_probs_b.bias", bias) && bias.type == B200MOE_TYPE_F32 && bias.ne[0] == n_expert) out->router_bias = static_cast<const float *>(bias.data);
    // shared expert with its gate (forward.cpp:312-314): all four tensors or none
    Got sg{}, su{}, sd{}, si{};
    const int have = (find("ffn_gate_shexp.weight", sg) == 0) + (find("ffn_up_shexp.weight", su) == 0) + (find("ffn_down_shexp.weight", sd) == 0) +
                     (find("ffn_gate_inp_shexp.weight", si) == 0);
    if (have == 4 && sg.type == gate.type && su.type == gate.type && sd.type == gate.type && si.type == B200MOE_TYPE_F32 && sg.ne[0] == n_embd &&
        su.ne[0] == n_embd && su.ne[1] == sg.ne[1] && sd.ne[0] == sg.ne[1] && sd.ne[1] == n_embd && si.ne[0] == n_embd) {
        out->gate_shexp = sg.data; out->up_shexp = su.data; out->down_shexp = sd.data;
        out->gate_inp_shexp = static_cast<const float *>(si.data);
        out->n_ff_shexp = (int32_t) sg.ne[1];
    }
    return B200MOE_OK;
}

}  // extern "C"
