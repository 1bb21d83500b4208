// GGUF files -> one device blob: the data format on the input side of the GEMV path (the raw block
// stream a tensor has on disk IS what the kernels read; nothing is repacked).  Host code only.
//
// What the reference's loader does for this path (src/model/gguf.{h,cpp}; the device blob of
// src/backend/weight_store.h:28-62), restated as a C interface: parse header, metadata and tensor
// table of a file (or of all shards of a split file "...-00001-of-0000N.gguf"), keep the files
// mapped, say where every tensor will sit in ONE device allocation the caller owns, and copy the
// data sections there.  A tensor of dims [K][N] is N rows of K values: b200q_seg.w = blob +
// blob_offset, K = dims[0], n_rows = dims[1]; expert banks [K][N][E] are E planes of N rows, plane
// e at blob_offset + e * N * row_bytes.  Files are untrusted input: every read is bounds-checked.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace b200q {
namespace {

struct TypeSize {
    uint32_t block, bytes; // values per block, bytes per block (ggml's public type table)
};
bool type_size(uint32_t t, TypeSize & ts) {
    switch (t) {
    case 0: ts = {1, 4}; return true;      // F32
    case 1: ts = {1, 2}; return true;      // F16
    case 2: ts = {32, 18}; return true;    // Q4_0
    case 3: ts = {32, 20}; return true;    // Q4_1
    case 6: ts = {32, 22}; return true;    // Q5_0
    case 7: ts = {32, 24}; return true;    // Q5_1
    case 8: ts = {32, 34}; return true;    // Q8_0
    case 9: ts = {32, 36}; return true;    // Q8_1
    case 10: ts = {256, 84}; return true;  // Q2_K
    case 11: ts = {256, 110}; return true; // Q3_K
    case 12: ts = {256, 144}; return true; // Q4_K
    case 13: ts = {256, 176}; return true; // Q5_K
    case 14: ts = {256, 210}; return true; // Q6_K
    case 15: ts = {256, 292}; return true; // Q8_K
    case 16: ts = {256, 66}; return true;  // IQ2_XXS
    case 17: ts = {256, 74}; return true;  // IQ2_XS
    case 18: ts = {256, 98}; return true;  // IQ3_XXS
    case 19: ts = {256, 50}; return true;  // IQ1_S
    case 20: ts = {32, 18}; return true;   // IQ4_NL
    case 21: ts = {256, 110}; return true; // IQ3_S
    case 22: ts = {256, 82}; return true;  // IQ2_S
    case 23: ts = {256, 136}; return true; // IQ4_XS
    case 24: ts = {1, 1}; return true;     // I8
    case 25: ts = {1, 2}; return true;     // I16
    case 26: ts = {1, 4}; return true;     // I32
    case 27: ts = {1, 8}; return true;     // I64
    case 28: ts = {1, 8}; return true;     // F64
    case 29: ts = {256, 56}; return true;  // IQ1_M
    case 30: ts = {1, 2}; return true;     // BF16
    default: return false;
    }
}

struct Meta {
    uint32_t type = 0;      // GGUF value type 0..12
    uint64_t u = 0;         // integers and bool
    double f = 0;           // floats
    std::string s;          // string
    uint32_t elem_type = 0; // arrays
    uint64_t count = 0;
    const uint8_t * raw = nullptr;        // first element of a fixed-size array inside the mapping
    std::vector<std::string> strs;        // a string array's elements
};

struct Shard {
    int fd = -1;
    const uint8_t * base = nullptr;
    size_t size = 0, data_offset = 0, data_bytes = 0;
    uint64_t slot = 0; // where its data section starts in the device blob
};

struct Tensor {
    std::string name;
    uint32_t type = 0, n_dims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};
    uint64_t n_rows = 0, row_bytes = 0, nbytes = 0, offset = 0, blob_offset = 0;
    int shard = 0;
};

// bounds-checked little-endian reader over one mapping
struct Cursor {
    const uint8_t *p, *end;
    bool ok = true;
    template <class T> T get() {
        T v{};
        if (!ok || (size_t)(end - p) < sizeof(T)) {
            ok = false;
            return v;
        }
        memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (!ok || n > (uint64_t)(end - p)) {
            ok = false;
            return {};
        }
        std::string s(reinterpret_cast<const char *>(p), (size_t)n);
        p += n;
        return s;
    }
};

uint32_t scalar_bytes(uint32_t t) {
    switch (t) {
    case 0: case 1: case 7: return 1;
    case 2: case 3: return 2;
    case 4: case 5: case 6: return 4;
    case 10: case 11: case 12: return 8;
    default: return 0;
    }
}

bool read_scalar(Cursor & c, uint32_t t, Meta & m) {
    switch (t) {
    case 0: m.u = c.get<uint8_t>(); m.f = (double)m.u; break;
    case 1: { const int8_t v = c.get<int8_t>(); m.u = (uint64_t)(int64_t)v; m.f = v; } break;
    case 2: m.u = c.get<uint16_t>(); m.f = (double)m.u; break;
    case 3: { const int16_t v = c.get<int16_t>(); m.u = (uint64_t)(int64_t)v; m.f = v; } break;
    case 4: m.u = c.get<uint32_t>(); m.f = (double)m.u; break;
    case 5: { const int32_t v = c.get<int32_t>(); m.u = (uint64_t)(int64_t)v; m.f = v; } break;
    case 6: { const float v = c.get<float>(); m.f = v; m.u = (uint64_t)(int64_t)v; } break;
    case 7: m.u = c.get<uint8_t>() ? 1 : 0; m.f = (double)m.u; break;
    case 10: m.u = c.get<uint64_t>(); m.f = (double)m.u; break;
    case 11: { const int64_t v = c.get<int64_t>(); m.u = (uint64_t)v; m.f = (double)v; } break;
    case 12: m.f = c.get<double>(); m.u = (uint64_t)(int64_t)m.f; break;
    default: return false;
    }
    return c.ok;
}

bool read_meta(Cursor & c, Meta & m) {
    m.type = c.get<uint32_t>();
    if (!c.ok) {
        return false;
    }
    if (m.type == 8) {
        m.s = c.str();
        return c.ok;
    }
    if (m.type != 9) {
        return read_scalar(c, m.type, m);
    }
    m.elem_type = c.get<uint32_t>();
    m.count = c.get<uint64_t>();
    if (!c.ok) {
        return false;
    }
    if (m.elem_type == 8) {
        if (m.count > (uint64_t)(c.end - c.p) / 8) { // every string needs its 8-byte length at least
            return false;
        }
        m.strs.reserve((size_t)m.count);
        for (uint64_t i = 0; i < m.count; i++) {
            m.strs.push_back(c.str());
            if (!c.ok) {
                return false;
            }
        }
        return true;
    }
    const uint32_t w = scalar_bytes(m.elem_type);
    if (w == 0 || m.count > (uint64_t)(c.end - c.p) / w) { // nested arrays are not part of any model file
        return false;
    }
    m.raw = c.p;
    c.p += m.count * w;
    return true;
}

} // namespace
} // namespace b200q

using namespace b200q;

struct b200q_gguf {
    std::vector<Shard> shards;
    std::vector<Tensor> tensors;
    std::unordered_map<std::string, int> index;
    std::unordered_map<std::string, Meta> meta;
    uint32_t version = 0, alignment = 32;
    uint64_t blob_bytes = 0;
    ~b200q_gguf() {
        for (Shard & s : shards) {
            if (s.base) {
                munmap(const_cast<uint8_t *>(s.base), s.size);
            }
            if (s.fd >= 0) {
                close(s.fd);
            }
        }
    }
};

namespace {

// "...-00002-of-00004.gguf" -> all shard paths in order (the count comes from the name, as in the
// reference, src/model/gguf.cpp:302-341); anything else: the path itself
std::vector<std::string> shard_names(const std::string & path) {
    const size_t n = path.size();
    // <stem>-DDDDD-of-DDDDD.gguf : 5 + 4 + 5 + 5 characters behind the dash
    if (n < 1 + 5 + 4 + 5 + 5 || path.compare(n - 5, 5, ".gguf") != 0 || path.compare(n - 14, 4, "-of-") != 0 ||
        path[n - 20] != '-') {
        return {path};
    }
    for (size_t i : {n - 19, n - 18, n - 17, n - 16, n - 15, n - 10, n - 9, n - 8, n - 7, n - 6}) {
        if (path[i] < '0' || path[i] > '9') {
            return {path};
        }
    }
    const int count = atoi(path.substr(n - 10, 5).c_str());
    if (count <= 1) {
        return {path};
    }
    std::vector<std::string> out;
    for (int i = 1; i <= count; i++) {
        char idx[16];
        snprintf(idx, sizeof(idx), "%05d", i);
        out.push_back(path.substr(0, n - 19) + idx + path.substr(n - 14));
    }
    return out;
}

int fail(b200q_gguf * g, int code, const char * fmt, const std::string & what) {
    set_error(fmt, what.c_str());
    delete g;
    return code;
}

} // namespace

extern "C" {

static int gguf_open_impl(const char * path, b200q_gguf * g);

int b200q_gguf_open(const char * path, b200q_gguf ** out) {
    if (!path || !out) {
        set_error("b200q_gguf_open: path and out must be non-null");
        return B200Q_EINVAL;
    }
    *out = nullptr;
    b200q_gguf * g = nullptr;
    try { // no exception may cross the C boundary (allocation failure on a hostile file)
        g = new b200q_gguf();
        const int rc = gguf_open_impl(path, g);
        if (rc == B200Q_OK) {
            *out = g;
        }
        return rc;
    } catch (...) {
        delete g;
        set_error("b200q_gguf_open: out of memory while parsing %s", path);
        return B200Q_EINVAL;
    }
}

// parses into g; on failure g has been deleted
static int gguf_open_impl(const char * path, b200q_gguf * g) {
    const std::vector<std::string> names = shard_names(path);
    for (size_t si = 0; si < names.size(); si++) {
        Shard sh;
        sh.fd = open(names[si].c_str(), O_RDONLY);
        struct stat st;
        if (sh.fd < 0 || fstat(sh.fd, &st) != 0 || st.st_size < 24) {
            if (sh.fd >= 0) {
                close(sh.fd);
            }
            return fail(g, B200Q_EINVAL, "b200q_gguf_open: cannot open %s (or shorter than a header)", names[si]);
        }
        sh.size = (size_t)st.st_size;
        void * m = mmap(nullptr, sh.size, PROT_READ, MAP_PRIVATE, sh.fd, 0);
        if (m == MAP_FAILED) {
            close(sh.fd);
            return fail(g, B200Q_EINVAL, "b200q_gguf_open: cannot map %s", names[si]);
        }
        sh.base = static_cast<const uint8_t *>(m);
        g->shards.push_back(sh);
        Shard & s = g->shards.back();
        Cursor c{s.base, s.base + s.size};
        if (c.get<uint32_t>() != 0x46554747u) { // "GGUF"
            return fail(g, B200Q_EINVAL, "b200q_gguf_open: %s is not a GGUF file", names[si]);
        }
        const uint32_t version = c.get<uint32_t>();
        const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
        if (!c.ok || version < 2 || version > 3 || n_tensors > s.size / 24 || n_kv > s.size / 12) {
            return fail(g, B200Q_EUNSUPPORTED, "b200q_gguf_open: %s: unsupported version or impossible counts", names[si]);
        }
        if (si == 0) {
            g->version = version;
        }
        uint32_t alignment = 32;
        for (uint64_t i = 0; i < n_kv; i++) {
            const std::string key = c.str();
            Meta m;
            if (!c.ok || !read_meta(c, m)) {
                return fail(g, B200Q_EINVAL, "b200q_gguf_open: %s: metadata runs past the end of the file", names[si]);
            }
            if (key == "general.alignment" && m.type != 8 && m.type != 9) {
                alignment = (uint32_t)m.u;
            }
            if (si == 0 || !g->meta.count(key)) { // the first shard's metadata describes the model
                g->meta[key] = std::move(m);
            }
        }
        if (alignment == 0 || (alignment & (alignment - 1))) {
            return fail(g, B200Q_EINVAL, "b200q_gguf_open: %s: general.alignment is not a power of two", names[si]);
        }
        if (si == 0) {
            g->alignment = alignment;
        }
        const size_t first = g->tensors.size();
        for (uint64_t i = 0; i < n_tensors; i++) {
            Tensor t;
            t.name = c.str();
            t.n_dims = c.get<uint32_t>();
            if (!c.ok || t.n_dims < 1 || t.n_dims > 4) {
                return fail(g, B200Q_EINVAL, "b200q_gguf_open: %s: bad tensor table", names[si]);
            }
            for (uint32_t d = 0; d < t.n_dims; d++) {
                t.dims[d] = c.get<uint64_t>();
            }
            t.type = c.get<uint32_t>();
            t.offset = c.get<uint64_t>();
            t.shard = (int)si;
            TypeSize ts;
            if (!c.ok) {
                return fail(g, B200Q_EINVAL, "b200q_gguf_open: %s: tensor table runs past the end of the file", names[si]);
            }
            if (!type_size(t.type, ts)) {
                return fail(g, B200Q_EUNSUPPORTED, "b200q_gguf_open: tensor %s has a type this library cannot size", t.name);
            }
            if (t.dims[0] == 0 || t.dims[0] % ts.block) {
                return fail(g, B200Q_EINVAL, "b200q_gguf_open: tensor %s: row length is not a whole number of blocks", t.name);
            }
            t.row_bytes = t.dims[0] / ts.block * ts.bytes;
            t.n_rows = 1;
            for (uint32_t d = 1; d < t.n_dims; d++) {
                if (t.dims[d] == 0 || t.n_rows > (1ull << 40) / t.dims[d]) {
                    return fail(g, B200Q_EINVAL, "b200q_gguf_open: tensor %s: impossible shape", t.name);
                }
                t.n_rows *= t.dims[d];
            }
            if (t.row_bytes > (1ull << 40) || t.n_rows * t.row_bytes > (1ull << 46)) {
                return fail(g, B200Q_EINVAL, "b200q_gguf_open: tensor %s: impossible size", t.name);
            }
            t.nbytes = t.n_rows * t.row_bytes;
            if (g->index.count(t.name)) {
                return fail(g, B200Q_EINVAL, "b200q_gguf_open: tensor %s appears twice", t.name);
            }
            g->index[t.name] = (int)g->tensors.size();
            g->tensors.push_back(std::move(t));
        }
        const size_t pos = (size_t)(c.p - s.base);
        s.data_offset = (pos + alignment - 1) / alignment * alignment;
        if (s.data_offset > s.size) {
            if (n_tensors > 0) {
                return fail(g, B200Q_EINVAL, "b200q_gguf_open: %s: no data section", names[si]);
            }
            s.data_offset = s.size; // a metadata-only shard may end with its header
        }
        s.data_bytes = s.size - s.data_offset;
        s.slot = g->blob_bytes;
        g->blob_bytes = (g->blob_bytes + s.data_bytes + 255) / 256 * 256;
        for (size_t i = first; i < g->tensors.size(); i++) {
            Tensor & t = g->tensors[i];
            if (t.offset % alignment || t.offset > s.data_bytes || t.nbytes > s.data_bytes - t.offset) {
                return fail(g, B200Q_EINVAL, "b200q_gguf_open: tensor %s lies outside its file's data section", t.name);
            }
            t.blob_offset = s.slot + t.offset;
        }
    }
    return B200Q_OK;
}

void b200q_gguf_close(b200q_gguf * g) {
    delete g;
}

int b200q_gguf_n_tensors(const b200q_gguf * g) {
    return g ? (int)g->tensors.size() : 0;
}
int b200q_gguf_n_shards(const b200q_gguf * g) {
    return g ? (int)g->shards.size() : 0;
}
uint32_t b200q_gguf_version(const b200q_gguf * g) {
    return g ? g->version : 0;
}
uint64_t b200q_gguf_blob_bytes(const b200q_gguf * g) {
    return g ? g->blob_bytes : 0;
}

int b200q_gguf_tensor_at(const b200q_gguf * g, int i, b200q_gguf_tensor * out) {
    if (!g || !out || i < 0 || i >= (int)g->tensors.size()) {
        set_error("b200q_gguf_tensor_at: bad handle, index or output");
        return B200Q_EINVAL;
    }
    const Tensor & t = g->tensors[(size_t)i];
    out->name = t.name.c_str();
    out->type = t.type;
    out->n_dims = t.n_dims;
    for (int d = 0; d < 4; d++) {
        out->dims[d] = t.dims[d];
    }
    out->n_rows = t.n_rows;
    out->row_bytes = t.row_bytes;
    out->nbytes = t.nbytes;
    out->blob_offset = t.blob_offset;
    out->shard = t.shard;
    out->host_data = g->shards[(size_t)t.shard].base + g->shards[(size_t)t.shard].data_offset + t.offset;
    return B200Q_OK;
}

int b200q_gguf_find(const b200q_gguf * g, const char * name) {
    if (!g || !name) {
        return -1;
    }
    const auto it = g->index.find(name);
    return it == g->index.end() ? -1 : it->second;
}

int b200q_gguf_upload(const b200q_gguf * g, void * blob, void * stream) {
    if (!g || !blob || (reinterpret_cast<uintptr_t>(blob) & 255)) {
        set_error("b200q_gguf_upload: handle and a 256-byte aligned device blob required");
        return B200Q_EINVAL;
    }
    for (const Shard & s : g->shards) {
        if (s.data_bytes) {
            B200Q_CUDA_OK(cudaMemcpyAsync(static_cast<uint8_t *>(blob) + s.slot, s.base + s.data_offset, s.data_bytes,
                                          cudaMemcpyHostToDevice, (cudaStream_t)stream));
        }
    }
    return B200Q_OK;
}

// ---- metadata: type (-1 = absent), then the value in the form asked for
int b200q_gguf_meta_type(const b200q_gguf * g, const char * key) {
    if (!g || !key) {
        return -1;
    }
    const auto it = g->meta.find(key);
    return it == g->meta.end() ? -1 : (int)it->second.type;
}
static const Meta * meta_of(const b200q_gguf * g, const char * key) {
    if (!g || !key) {
        return nullptr;
    }
    const auto it = g->meta.find(key);
    return it == g->meta.end() ? nullptr : &it->second;
}
int b200q_gguf_meta_u64(const b200q_gguf * g, const char * key, uint64_t * out) {
    const Meta * m = meta_of(g, key);
    if (!m || !out || m->type == 8 || m->type == 9) {
        return B200Q_EINVAL;
    }
    *out = m->u;
    return B200Q_OK;
}
int b200q_gguf_meta_f64(const b200q_gguf * g, const char * key, double * out) {
    const Meta * m = meta_of(g, key);
    if (!m || !out || m->type == 8 || m->type == 9) {
        return B200Q_EINVAL;
    }
    *out = m->f;
    return B200Q_OK;
}
const char * b200q_gguf_meta_str(const b200q_gguf * g, const char * key) {
    const Meta * m = meta_of(g, key);
    return m && m->type == 8 ? m->s.c_str() : nullptr;
}
int b200q_gguf_meta_arr(const b200q_gguf * g, const char * key, uint32_t * elem_type, uint64_t * count) {
    const Meta * m = meta_of(g, key);
    if (!m || m->type != 9 || !elem_type || !count) {
        return B200Q_EINVAL;
    }
    *elem_type = m->elem_type;
    *count = m->count;
    return B200Q_OK;
}
const char * b200q_gguf_meta_arr_str(const b200q_gguf * g, const char * key, uint64_t i) {
    const Meta * m = meta_of(g, key);
    return m && m->type == 9 && m->elem_type == 8 && i < m->count ? m->strs[(size_t)i].c_str() : nullptr;
}
const void * b200q_gguf_meta_arr_data(const b200q_gguf * g, const char * key) {
    const Meta * m = meta_of(g, key);
    return m && m->type == 9 && m->elem_type != 8 ? m->raw : nullptr;
}

} // extern "C"
