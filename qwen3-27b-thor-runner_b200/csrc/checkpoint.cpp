// Host-side NVFP4 checkpoint ingestion (include/nvfp4_checkpoint.h): safetensors reader and
// writer, row merges, tensor-parallel shard rule.  Plain C++17, no CUDA.
//
// A safetensors file is an 8-byte little-endian header length, a JSON object
//   { "name": {"dtype": "...", "shape": [...], "data_offsets": [begin, end]}, ..., "__metadata__": {...} }
// and the raw tensor bytes; offsets are relative to the end of the header.  The header is read
// with a small recursive-descent JSON reader (strings with escapes, numbers, nested objects and
// arrays), so nested or unordered metadata does not confuse it.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/nvfp4_checkpoint.h"

namespace {

struct Entry {
    std::string dtype;
    std::vector<long long> shape;
    unsigned long long begin = 0, end = 0;
};

// ---- JSON reader over [p, e): just enough structure to walk the header.
struct Json {
    const char* p;
    const char* e;
    bool ok = true;

    void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool eat(char c) { ws(); if (p < e && *p == c) { ++p; return true; } return false; }
    bool peek(char c) { ws(); return p < e && *p == c; }

    std::string string() {
        std::string s;
        if (!eat('"')) { ok = false; return s; }
        while (p < e && *p != '"') {
            if (*p == '\\' && p + 1 < e) {
                ++p;
                switch (*p) {
                    case 'n': s += '\n'; break;
                    case 't': s += '\t'; break;
                    case 'r': s += '\r'; break;
                    case 'b': s += '\b'; break;
                    case 'f': s += '\f'; break;
                    case 'u': s += '?'; p += (e - p > 4 ? 4 : e - p - 1); break;   // names are ASCII; keep the length sane
                    default: s += *p;
                }
                ++p;
            } else {
                s += *p++;
            }
        }
        if (!eat('"')) ok = false;
        return s;
    }
    long long integer() {
        ws();
        bool neg = false;
        if (p < e && *p == '-') { neg = true; ++p; }
        if (p >= e || *p < '0' || *p > '9') { ok = false; return 0; }
        long long v = 0;
        while (p < e && *p >= '0' && *p <= '9') v = v * 10 + (*p++ - '0');
        return neg ? -v : v;
    }
    void skip_value() {   // any JSON value
        ws();
        if (p >= e) { ok = false; return; }
        if (*p == '"') { string(); return; }
        if (*p == '{') {
            ++p;
            if (eat('}')) return;
            do { string(); if (!eat(':')) { ok = false; return; } skip_value(); } while (ok && eat(','));
            if (!eat('}')) ok = false;
            return;
        }
        if (*p == '[') {
            ++p;
            if (eat(']')) return;
            do { skip_value(); } while (ok && eat(','));
            if (!eat(']')) ok = false;
            return;
        }
        while (p < e && *p != ',' && *p != '}' && *p != ']' && *p != ' ' && *p != '\n') ++p;   // number / true / false / null
    }
    std::vector<long long> int_array() {
        std::vector<long long> v;
        if (!eat('[')) { ok = false; return v; }
        if (eat(']')) return v;
        do { v.push_back(integer()); } while (ok && eat(','));
        if (!eat(']')) ok = false;
        return v;
    }
};

bool parse_header(const char* json, size_t len, std::map<std::string, Entry>& out, std::vector<std::string>& order) {
    Json j{json, json + len};
    if (!j.eat('{')) return false;
    if (j.eat('}')) return true;
    do {
        const std::string name = j.string();
        if (!j.ok || !j.eat(':')) return false;
        if (name == "__metadata__") { j.skip_value(); continue; }
        if (!j.eat('{')) return false;
        Entry en;
        bool have_off = false;
        if (!j.peek('}')) {
            do {
                const std::string key = j.string();
                if (!j.ok || !j.eat(':')) return false;
                if (key == "dtype") en.dtype = j.string();
                else if (key == "shape") en.shape = j.int_array();
                else if (key == "data_offsets") {
                    const std::vector<long long> o = j.int_array();
                    if (o.size() != 2 || o[0] < 0 || o[1] < o[0]) return false;
                    en.begin = (unsigned long long)o[0];
                    en.end = (unsigned long long)o[1];
                    have_off = true;
                } else j.skip_value();
            } while (j.ok && j.eat(','));
        }
        if (!j.ok || !j.eat('}') || !have_off || en.dtype.empty() || en.shape.size() > 8) return false;
        if (out.emplace(name, en).second) order.push_back(name);
    } while (j.ok && j.eat(','));
    return j.ok && j.eat('}');
}

int dtype_bytes(const std::string& d) {
    if (d == "U8" || d == "I8" || d == "F8_E4M3" || d == "F8_E5M2" || d == "BOOL") return 1;
    if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
    if (d == "F32" || d == "I32" || d == "U32") return 4;
    if (d == "F64" || d == "I64" || d == "U64") return 8;
    return 0;   // unknown (e.g. sub-byte types): size is not checked
}

}  // namespace

struct nvfp4_ckpt {
    int fd = -1;
    const unsigned char* base = nullptr;
    size_t size = 0;
    size_t data_off = 0;
    std::map<std::string, Entry> entries;
    std::vector<std::string> order;
};

extern "C" {

const char* nvfp4_ckpt_status_string(int s) {
    switch (s) {
        case NVFP4_CKPT_OK: return "ok";
        case NVFP4_CKPT_E_NULL: return "null argument";
        case NVFP4_CKPT_E_IO: return "cannot open, map or write the file";
        case NVFP4_CKPT_E_FORMAT: return "not a well-formed safetensors file";
        case NVFP4_CKPT_E_MISSING: return "no tensor of that name";
        case NVFP4_CKPT_E_TYPE: return "tensor of the wrong dtype or rank";
        case NVFP4_CKPT_E_SHAPE: return "shapes do not agree";
        case NVFP4_CKPT_E_SCALE: return "parts of a merge carry different global scales";
        default: return "unknown status";
    }
}

int nvfp4_ckpt_close(nvfp4_ckpt* c) {
    if (!c) return NVFP4_CKPT_E_NULL;
    if (c->base) munmap(const_cast<unsigned char*>(c->base), c->size);
    if (c->fd >= 0) close(c->fd);
    delete c;
    return NVFP4_CKPT_OK;
}

int nvfp4_ckpt_open(const char* path, nvfp4_ckpt** out) {
    if (!path || !out) return NVFP4_CKPT_E_NULL;
    *out = nullptr;
    nvfp4_ckpt* c = new nvfp4_ckpt();
    c->fd = open(path, O_RDONLY);
    struct stat st {};
    if (c->fd < 0 || fstat(c->fd, &st) != 0 || st.st_size < 10) { nvfp4_ckpt_close(c); return NVFP4_CKPT_E_IO; }
    c->size = (size_t)st.st_size;
    void* m = mmap(nullptr, c->size, PROT_READ, MAP_PRIVATE, c->fd, 0);
    if (m == MAP_FAILED) { nvfp4_ckpt_close(c); return NVFP4_CKPT_E_IO; }
    c->base = static_cast<const unsigned char*>(m);
    unsigned long long hlen = 0;
    std::memcpy(&hlen, c->base, 8);
    if (hlen < 2 || hlen > c->size - 8) { nvfp4_ckpt_close(c); return NVFP4_CKPT_E_FORMAT; }
    c->data_off = 8 + (size_t)hlen;
    if (!parse_header(reinterpret_cast<const char*>(c->base + 8), (size_t)hlen, c->entries, c->order)) {
        nvfp4_ckpt_close(c);
        return NVFP4_CKPT_E_FORMAT;
    }
    for (const auto& kv : c->entries) {   // every tensor inside the file, sizes consistent with dtype x shape
        const Entry& e = kv.second;
        if (e.end > c->size - c->data_off) { nvfp4_ckpt_close(c); return NVFP4_CKPT_E_FORMAT; }
        unsigned long long n = 1;
        for (long long d : e.shape) { if (d < 0) { nvfp4_ckpt_close(c); return NVFP4_CKPT_E_FORMAT; } n *= (unsigned long long)d; }
        const int b = dtype_bytes(e.dtype);
        if (b && n * (unsigned long long)b != e.end - e.begin) { nvfp4_ckpt_close(c); return NVFP4_CKPT_E_FORMAT; }
    }
    *out = c;
    return NVFP4_CKPT_OK;
}

int nvfp4_ckpt_count(const nvfp4_ckpt* c) { return c ? (int)c->order.size() : NVFP4_CKPT_E_NULL; }

const char* nvfp4_ckpt_name(const nvfp4_ckpt* c, int i) {
    return (c && i >= 0 && i < (int)c->order.size()) ? c->order[(size_t)i].c_str() : nullptr;
}

int nvfp4_ckpt_get(const nvfp4_ckpt* c, const char* name, nvfp4_ckpt_tensor* out) {
    if (!c || !name || !out) return NVFP4_CKPT_E_NULL;
    const auto it = c->entries.find(name);
    if (it == c->entries.end()) return NVFP4_CKPT_E_MISSING;
    const Entry& e = it->second;
    std::memset(out, 0, sizeof *out);
    out->data = c->base + c->data_off + e.begin;
    out->nbytes = (size_t)(e.end - e.begin);
    std::snprintf(out->dtype, sizeof out->dtype, "%s", e.dtype.c_str());
    out->rank = (int)e.shape.size();
    for (size_t i = 0; i < e.shape.size(); ++i) out->shape[i] = e.shape[i];
    return NVFP4_CKPT_OK;
}

int nvfp4_ckpt_linear(const nvfp4_ckpt* c, const char* prefix, nvfp4_host_weight* out) {
    if (!c || !prefix || !out) return NVFP4_CKPT_E_NULL;
    std::memset(out, 0, sizeof *out);
    const std::string p(prefix);
    nvfp4_ckpt_tensor pk, sc, gs, is;
    if (int e = nvfp4_ckpt_get(c, (p + ".weight_packed").c_str(), &pk)) return e;
    if (int e = nvfp4_ckpt_get(c, (p + ".weight_scale").c_str(), &sc)) return e;
    if (int e = nvfp4_ckpt_get(c, (p + ".weight_global_scale").c_str(), &gs)) return e;
    if (std::strcmp(pk.dtype, "U8") != 0 || pk.rank != 2) return NVFP4_CKPT_E_TYPE;
    if ((std::strcmp(sc.dtype, "F8_E4M3") != 0 && std::strcmp(sc.dtype, "U8") != 0) || sc.rank != 2) return NVFP4_CKPT_E_TYPE;
    if (std::strcmp(gs.dtype, "F32") != 0 || gs.nbytes != 4) return NVFP4_CKPT_E_TYPE;
    const long long N = pk.shape[0], K = pk.shape[1] * 2;
    if (N <= 0 || K <= 0 || (K % 16) != 0 || N > 0x7fffffff || K > 0x7fffffff) return NVFP4_CKPT_E_SHAPE;
    if (sc.shape[0] != N || sc.shape[1] != K / 16) return NVFP4_CKPT_E_SHAPE;
    out->packed = static_cast<const uint8_t*>(pk.data);
    out->scale = static_cast<const uint8_t*>(sc.data);
    std::memcpy(&out->global_scale, gs.data, 4);
    if (nvfp4_ckpt_get(c, (p + ".input_global_scale").c_str(), &is) == NVFP4_CKPT_OK) {
        if (std::strcmp(is.dtype, "F32") != 0 || is.nbytes != 4) return NVFP4_CKPT_E_TYPE;
        std::memcpy(&out->input_scale, is.data, 4);
    }
    out->N = (int)N;
    out->K = (int)K;
    return NVFP4_CKPT_OK;
}

int nvfp4_merge_rows(const nvfp4_host_weight* parts, int n, uint8_t* packed_out, uint8_t* scale_out,
                     nvfp4_host_weight* merged) {
    return nvfp4_merge_rows_ex(parts, n, packed_out, scale_out, merged, 0);
}

int nvfp4_merge_rows_ex(const nvfp4_host_weight* parts, int n, uint8_t* packed_out, uint8_t* scale_out,
                        nvfp4_host_weight* merged, int take_first_scale) {
    if (!parts || !packed_out || !scale_out || !merged || n < 1) return NVFP4_CKPT_E_NULL;
    const int K = parts[0].K;
    long long rows = 0;
    for (int i = 0; i < n; ++i) {
        if (!parts[i].packed || !parts[i].scale) return NVFP4_CKPT_E_NULL;
        if (parts[i].K != K || parts[i].N <= 0) return NVFP4_CKPT_E_SHAPE;
        if (!take_first_scale && parts[i].global_scale != parts[0].global_scale) return NVFP4_CKPT_E_SCALE;
        rows += parts[i].N;
    }
    if (rows > 0x7fffffff) return NVFP4_CKPT_E_SHAPE;
    size_t po = 0, so = 0;
    for (int i = 0; i < n; ++i) {
        const size_t pb = (size_t)parts[i].N * (size_t)(K / 2), sb = (size_t)parts[i].N * (size_t)(K / 16);
        std::memcpy(packed_out + po, parts[i].packed, pb);
        std::memcpy(scale_out + so, parts[i].scale, sb);
        po += pb;
        so += sb;
    }
    *merged = parts[0];
    merged->packed = packed_out;
    merged->scale = scale_out;
    merged->N = (int)rows;
    return NVFP4_CKPT_OK;
}

int nvfp4_tp_shard_down_k(int I, int world) {
    if (I <= 0 || world < 1 || (I % (16 * world)) != 0) return NVFP4_CKPT_E_SHAPE;
    return (I / world + 255) / 256 * 256;
}

int nvfp4_tp_shard_gate_up(const nvfp4_host_weight* m, int rank, int world, uint8_t* packed_out, uint8_t* scale_out,
                           nvfp4_host_weight* shard) {
    if (!m || !m->packed || !m->scale || !packed_out || !scale_out || !shard) return NVFP4_CKPT_E_NULL;
    if (world < 1 || rank < 0 || rank >= world || (m->N % 2) != 0) return NVFP4_CKPT_E_SHAPE;
    const int I = m->N / 2;
    if ((I % (16 * world)) != 0) return NVFP4_CKPT_E_SHAPE;
    const size_t ip = (size_t)(I / world), prow = (size_t)m->K / 2, srow = (size_t)m->K / 16;
    // gate rows [r*ip, (r+1)*ip) then up rows I + [r*ip, (r+1)*ip)
    std::memcpy(packed_out, m->packed + (size_t)rank * ip * prow, ip * prow);
    std::memcpy(packed_out + ip * prow, m->packed + ((size_t)I + (size_t)rank * ip) * prow, ip * prow);
    std::memcpy(scale_out, m->scale + (size_t)rank * ip * srow, ip * srow);
    std::memcpy(scale_out + ip * srow, m->scale + ((size_t)I + (size_t)rank * ip) * srow, ip * srow);
    *shard = *m;
    shard->packed = packed_out;
    shard->scale = scale_out;
    shard->N = (int)(2 * ip);
    return NVFP4_CKPT_OK;
}

int nvfp4_tp_shard_down(const nvfp4_host_weight* d, int rank, int world, uint8_t* packed_out, uint8_t* scale_out,
                        nvfp4_host_weight* shard) {
    if (!d || !d->packed || !d->scale || !packed_out || !scale_out || !shard) return NVFP4_CKPT_E_NULL;
    if (world < 1 || rank < 0 || rank >= world) return NVFP4_CKPT_E_SHAPE;
    const int kp = nvfp4_tp_shard_down_k(d->K, world);
    if (kp < 0) return kp;
    const size_t ip = (size_t)(d->K / world);
    const size_t prow_in = (size_t)d->K / 2, srow_in = (size_t)d->K / 16, prow = (size_t)kp / 2, srow = (size_t)kp / 16;
    std::memset(packed_out, 0, (size_t)d->N * prow);   // zero codes and zero scales in the K padding
    std::memset(scale_out, 0, (size_t)d->N * srow);
    for (int n = 0; n < d->N; ++n) {
        std::memcpy(packed_out + (size_t)n * prow, d->packed + (size_t)n * prow_in + (size_t)rank * ip / 2, ip / 2);
        std::memcpy(scale_out + (size_t)n * srow, d->scale + (size_t)n * srow_in + (size_t)rank * ip / 16, ip / 16);
    }
    *shard = *d;
    shard->packed = packed_out;
    shard->scale = scale_out;
    shard->K = kp;
    return NVFP4_CKPT_OK;
}

int nvfp4_interleave_gate_up(const nvfp4_host_weight* m, uint8_t* packed_out, uint8_t* scale_out, nvfp4_host_weight* out) {
    if (!m || !m->packed || !m->scale || !packed_out || !scale_out || !out) return NVFP4_CKPT_E_NULL;
    if ((m->N % 16) != 0) return NVFP4_CKPT_E_SHAPE;
    const size_t I = (size_t)m->N / 2, prow = (size_t)m->K / 2, srow = (size_t)m->K / 16;
    for (size_t s = 0; s < I / 8; ++s) {          // slab s: 8 gate rows, then their 8 up rows
        std::memcpy(packed_out + (16 * s) * prow, m->packed + (8 * s) * prow, 8 * prow);
        std::memcpy(packed_out + (16 * s + 8) * prow, m->packed + (I + 8 * s) * prow, 8 * prow);
        std::memcpy(scale_out + (16 * s) * srow, m->scale + (8 * s) * srow, 8 * srow);
        std::memcpy(scale_out + (16 * s + 8) * srow, m->scale + (I + 8 * s) * srow, 8 * srow);
    }
    *out = *m;
    out->packed = packed_out;
    out->scale = scale_out;
    return NVFP4_CKPT_OK;
}

int nvfp4_tp_shard_qkv_rows(int q_rows, int kv_rows, int n_kv_heads, int world) {
    if (q_rows <= 0 || kv_rows <= 0 || n_kv_heads <= 0 || world < 1) return NVFP4_CKPT_E_SHAPE;
    if ((q_rows % (8 * world)) != 0 || (kv_rows % n_kv_heads) != 0) return NVFP4_CKPT_E_SHAPE;
    if (world <= n_kv_heads ? (n_kv_heads % world) != 0 : (world % n_kv_heads) != 0) return NVFP4_CKPT_E_SHAPE;
    const int kv_local = world <= n_kv_heads ? kv_rows / world : kv_rows / n_kv_heads;
    if ((kv_local % 8) != 0) return NVFP4_CKPT_E_SHAPE;
    return q_rows / world + 2 * kv_local;
}

int nvfp4_tp_shard_qkv(const nvfp4_host_weight* m, int q_rows, int kv_rows, int n_kv_heads, int rank, int world,
                       uint8_t* packed_out, uint8_t* scale_out, nvfp4_host_weight* shard) {
    if (!m || !m->packed || !m->scale || !packed_out || !scale_out || !shard) return NVFP4_CKPT_E_NULL;
    const int rows = nvfp4_tp_shard_qkv_rows(q_rows, kv_rows, n_kv_heads, world);
    if (rows < 0) return rows;
    if (rank < 0 || rank >= world || m->N != q_rows + 2 * kv_rows) return NVFP4_CKPT_E_SHAPE;
    const int head = kv_rows / n_kv_heads;
    const size_t q_local = (size_t)(q_rows / world);
    const size_t kv_local = world <= n_kv_heads ? (size_t)(kv_rows / world) : (size_t)head;
    const size_t kv_first = world <= n_kv_heads ? (size_t)rank * kv_local : (size_t)(rank / (world / n_kv_heads)) * head;
    const size_t prow = (size_t)m->K / 2, srow = (size_t)m->K / 16;
    const size_t src[3] = {(size_t)rank * q_local, (size_t)q_rows + kv_first, (size_t)q_rows + kv_rows + kv_first};
    const size_t cnt[3] = {q_local, kv_local, kv_local};
    size_t dst = 0;
    for (int b = 0; b < 3; ++b) {           // q, k, v: three contiguous row blocks
        std::memcpy(packed_out + dst * prow, m->packed + src[b] * prow, cnt[b] * prow);
        std::memcpy(scale_out + dst * srow, m->scale + src[b] * srow, cnt[b] * srow);
        dst += cnt[b];
    }
    *shard = *m;
    shard->packed = packed_out;
    shard->scale = scale_out;
    shard->N = rows;
    return NVFP4_CKPT_OK;
}

int nvfp4_ckpt_write(const char* path, const char* const* names, const nvfp4_ckpt_tensor* t, int n) {
    if (!path || !names || !t || n < 0) return NVFP4_CKPT_E_NULL;
    std::string h = "{";
    unsigned long long off = 0;
    for (int i = 0; i < n; ++i) {
        if (!names[i] || (!t[i].data && t[i].nbytes) || t[i].rank < 0 || t[i].rank > 8) return NVFP4_CKPT_E_NULL;
        if (i) h += ",";
        h += "\"";
        for (const char* q = names[i]; *q; ++q) { if (*q == '"' || *q == '\\') h += '\\'; h += *q; }
        h += "\":{\"dtype\":\"" + std::string(t[i].dtype) + "\",\"shape\":[";
        for (int d = 0; d < t[i].rank; ++d) h += (d ? "," : "") + std::to_string(t[i].shape[d]);
        h += "],\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + t[i].nbytes) + "]}";
        off += t[i].nbytes;
    }
    h += "}";
    while ((h.size() + 8) % 8) h += ' ';     // data starts on an 8-byte boundary
    FILE* f = std::fopen(path, "wb");
    if (!f) return NVFP4_CKPT_E_IO;
    const unsigned long long hlen = h.size();
    bool ok = std::fwrite(&hlen, 8, 1, f) == 1 && std::fwrite(h.data(), 1, h.size(), f) == h.size();
    for (int i = 0; ok && i < n; ++i) ok = t[i].nbytes == 0 || std::fwrite(t[i].data, 1, t[i].nbytes, f) == t[i].nbytes;
    ok = (std::fclose(f) == 0) && ok;
    return ok ? NVFP4_CKPT_OK : NVFP4_CKPT_E_IO;
}

}  // extern "C"
