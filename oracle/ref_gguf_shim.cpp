// TEST INFRASTRUCTURE ONLY.
// Thin extern "C" surface over the reference's own GGUF loader (src/model/gguf.{h,cpp} of the
// reference project), compiled together with that unmodified source file into _ref/libsigguf.so
// (see Makefile).  Nothing of the reference is copied here; the functions only forward.  The
// tests use it to check that files written by this repository's writer mean to the reference's
// loader what they mean to this repository's loader.
#include <cstdint>
#include <cstring>
#include <string>

#include "gguf.h"

extern "C" {

void * sigguf_load(const char * path) {
    gguf_file * f = new gguf_file();
    try {
        f->load(path);
    } catch (...) {
        delete f;
        return nullptr;
    }
    return f;
}
void sigguf_close(void * h) {
    delete static_cast<gguf_file *>(h);
}
int sigguf_n_tensors(void * h) {
    return (int)static_cast<gguf_file *>(h)->tensors.size();
}
int sigguf_n_shards(void * h) {
    const gguf_file * f = static_cast<gguf_file *>(h);
    return f->shards.empty() ? 1 : (int)f->shards.size();
}
uint32_t sigguf_version(void * h) {
    return static_cast<gguf_file *>(h)->version;
}
// name into buf (cap bytes), dims[4] (unused = 1), type, n_dims, nbytes, and the tensor's data pointer
int sigguf_tensor(void * h, int i, char * buf, int cap, uint64_t * dims, uint32_t * type, uint32_t * n_dims,
                  uint64_t * nbytes, const void ** data) {
    const gguf_file * f = static_cast<gguf_file *>(h);
    if (i < 0 || i >= (int)f->tensors.size()) {
        return -1;
    }
    const gguf_tensor_info & t = f->tensors[(size_t)i];
    snprintf(buf, (size_t)cap, "%s", t.name.c_str());
    for (int d = 0; d < 4; d++) {
        dims[d] = d < (int)t.dims.size() ? t.dims[(size_t)d] : 1;
    }
    *type = t.type;
    *n_dims = (uint32_t)t.dims.size();
    *nbytes = (uint64_t)t.nbytes();
    *data = t.data;
    return 0;
}
int sigguf_has(void * h, const char * key) {
    return static_cast<gguf_file *>(h)->meta(key) ? 1 : 0;
}
uint32_t sigguf_u32(void * h, const char * key) {
    return static_cast<gguf_file *>(h)->get_u32(key, 0);
}
float sigguf_f32(void * h, const char * key) {
    return static_cast<gguf_file *>(h)->get_f32(key, 0.f);
}
const char * sigguf_str(void * h, const char * key) {
    const std::string * s = static_cast<gguf_file *>(h)->get_str(key);
    return s ? s->c_str() : nullptr;
}
int sigguf_arr_len(void * h, const char * key) {
    const gguf_kv * v = static_cast<gguf_file *>(h)->meta(key);
    return v && v->is_arr() ? (int)v->arr.size() : -1;
}
const char * sigguf_arr_str(void * h, const char * key, int i) {
    const gguf_kv * v = static_cast<gguf_file *>(h)->meta(key);
    return v && v->is_arr() && i >= 0 && i < (int)v->arr.size() ? v->arr[(size_t)i].str.c_str() : nullptr;
}
long long sigguf_arr_i64(void * h, const char * key, int i) {
    const gguf_kv * v = static_cast<gguf_file *>(h)->meta(key);
    return v && v->is_arr() && i >= 0 && i < (int)v->arr.size() ? (long long)v->arr[(size_t)i].i64 : 0;
}

} // extern "C"
