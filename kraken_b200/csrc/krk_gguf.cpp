// GGUF v2 / v3 container reader for the quantized-weight path: header, key/value block and tensor
// directory of a .gguf file, tensors handed to the backend as the unmodified bytes of the file (what
// Backend::upload receives is what the kernels read, include/krk/backend.hpp:8-10, 720). Replaces, for
// this path, krk::Gguf (include/krk/gguf.hpp, src/gguf.cpp): a single file, mapped read-only, never
// copied on the host. Split models, the reference's repacking loader and its model graph are not here.
//
// Layout read (the public GGUF specification): magic "GGUF", u32 version, u64 tensor count, u64 key/value
// count; key/values (string key, u32 type, value; strings are u64 length + bytes; arrays are u32 element
// type + u64 count + elements); tensor infos (string name, u32 n_dims, u64 dims, u32 type, u64 offset into
// the data section); the data section starts at the next multiple of general.alignment (default 32).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <utility>
#include <vector>

#include "krk_cuda.h"

namespace {

enum : uint32_t { kU8 = 0, kI8, kU16, kI16, kU32, kI32, kF32, kBool, kString, kArray, kU64, kI64, kF64 };

struct Value {
    uint32_t type = kU32;
    uint64_t u = 0;
    int64_t i = 0;
    double f = 0.0;
    std::string str;
    uint32_t elem = kU8;        // arrays: element type, count and where the elements lie in the file
    uint64_t count = 0;
    size_t array_off = 0;
};

struct Tensor {
    std::string name;
    uint32_t type_id = 0;
    int n_dims = 0;
    uint64_t ne[4] = {1, 1, 1, 1};
    uint64_t offset = 0;
    const uint8_t *data = nullptr;
    size_t n_bytes = 0;         // 0 when the type is not one this library sizes
};

struct File {
    int fd = -1;
    const uint8_t *base = nullptr;
    size_t size = 0;
    uint32_t version = 0;
    size_t data_off = 0;
    std::vector<std::pair<std::string, Value>> kvs;
    std::vector<Tensor> tensors;
    ~File() {
        if (base) munmap(const_cast<uint8_t *>(base), size);
        if (fd >= 0) close(fd);
    }
};

// bytes of one row of n values: the block formats of this library, plus plain f32 / f16 / bf16 / i8 / i32
size_t type_row_bytes(uint32_t type_id, uint64_t n) {
    switch (type_id) {
    case 0: return (size_t)n * 4;     // F32
    case 1: return (size_t)n * 2;     // F16
    case 30: return (size_t)n * 2;    // BF16
    case 24: return (size_t)n;        // I8
    case 26: return (size_t)n * 4;    // I32
    default: break;
    }
    if (!krk_cuda_dtype_ok((int)type_id)) return 0;
    if (n % (uint64_t)krk_cuda_block_size((int)type_id) != 0) return 0;
    return krk_cuda_row_bytes((int)type_id, (int64_t)n);
}

struct Cursor {
    const uint8_t *p, *end;
    bool ok = true;
    template <class T> T get() {
        T v{};
        if (!ok || (size_t)(end - p) < sizeof(T)) {
            ok = false;
            return v;
        }
        std::memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (!ok || n > (uint64_t)(end - p)) {
            ok = false;
            return std::string();
        }
        std::string s(reinterpret_cast<const char *>(p), (size_t)n);
        p += n;
        return s;
    }
    void skip(uint64_t n) {
        if (!ok || n > (uint64_t)(end - p)) ok = false;
        else p += n;
    }
};

size_t scalar_size(uint32_t t) {
    switch (t) {
    case kU8: case kI8: case kBool: return 1;
    case kU16: case kI16: return 2;
    case kU32: case kI32: case kF32: return 4;
    case kU64: case kI64: case kF64: return 8;
    default: return 0;
    }
}

bool read_scalar(Cursor &c, uint32_t t, Value &v) {
    switch (t) {
    case kU8: v.u = c.get<uint8_t>(); v.i = (int64_t)v.u; break;
    case kI8: v.i = c.get<int8_t>(); v.u = (uint64_t)v.i; break;
    case kU16: v.u = c.get<uint16_t>(); v.i = (int64_t)v.u; break;
    case kI16: v.i = c.get<int16_t>(); v.u = (uint64_t)v.i; break;
    case kU32: v.u = c.get<uint32_t>(); v.i = (int64_t)v.u; break;
    case kI32: v.i = c.get<int32_t>(); v.u = (uint64_t)v.i; break;
    case kU64: v.u = c.get<uint64_t>(); v.i = (int64_t)v.u; break;
    case kI64: v.i = c.get<int64_t>(); v.u = (uint64_t)v.i; break;
    case kF32: v.f = c.get<float>(); v.i = (int64_t)v.f; break;
    case kF64: v.f = c.get<double>(); v.i = (int64_t)v.f; break;
    case kBool: v.u = c.get<uint8_t>() != 0; v.i = (int64_t)v.u; break;
    default: return false;
    }
    if (t != kF32 && t != kF64) v.f = (double)v.i;
    return c.ok;
}

bool parse(File &f, std::string &err) {
    Cursor c{f.base, f.base + f.size};
    if (c.get<uint32_t>() != 0x46554747u) { err = "not a GGUF file (bad magic)"; return false; }
    f.version = c.get<uint32_t>();
    if (f.version != 2 && f.version != 3) { err = "unsupported GGUF version " + std::to_string(f.version); return false; }
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    // (a tensor entry takes at least 24 bytes of the file and a key/value at least 13: no count can exceed that)
    if (!c.ok || n_tensors > (1u << 24) || n_kv > (1u << 24) || n_tensors > f.size / 24 || n_kv > f.size / 13) {
        err = "truncated or implausible header";
        return false;
    }
    uint64_t alignment = 32;
    for (uint64_t k = 0; k < n_kv; k++) {
        std::string key = c.str();
        Value v;
        v.type = c.get<uint32_t>();
        if (v.type == kString) {
            v.str = c.str();
        } else if (v.type == kArray) {
            v.elem = c.get<uint32_t>();
            v.count = c.get<uint64_t>();
            v.array_off = (size_t)(c.p - f.base);
            if (v.elem == kString) {
                for (uint64_t j = 0; j < v.count && c.ok; j++) c.skip(c.get<uint64_t>());
            } else {
                const size_t es = scalar_size(v.elem);
                if (es == 0 || (v.count && v.count > (uint64_t)(c.end - c.p) / es)) { err = "bad array in key " + key; return false; }
                c.skip(v.count * es);
            }
        } else if (!read_scalar(c, v.type, v)) {
            err = "bad value type in key " + key;
            return false;
        }
        if (!c.ok) { err = "truncated key/value block at " + key; return false; }
        if (key == "general.alignment" && v.type != kString && v.type != kArray && v.u > 0) alignment = v.u;
        f.kvs.emplace_back(std::move(key), std::move(v));
    }
    if (alignment == 0 || (alignment & (alignment - 1)) != 0 || alignment > (1u << 20)) {
        err = "general.alignment is not a power of two up to 1 MiB";
        return false;
    }
    f.tensors.resize((size_t)n_tensors);
    for (Tensor &t : f.tensors) {
        t.name = c.str();
        const uint32_t nd = c.get<uint32_t>();
        if (!c.ok || nd > 4) { err = "tensor " + t.name + ": more than 4 dimensions"; return false; }
        t.n_dims = (int)nd;
        for (uint32_t d = 0; d < nd; d++) t.ne[d] = c.get<uint64_t>();
        t.type_id = c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        if (!c.ok) { err = "truncated tensor directory"; return false; }
    }
    const size_t dir_end = (size_t)(c.p - f.base);
    f.data_off = (dir_end + alignment - 1) / alignment * alignment;
    if (f.data_off > f.size) { err = "file ends before the tensor data section"; return false; }
    for (Tensor &t : f.tensors) {
        if (t.offset % alignment != 0) { err = "tensor " + t.name + ": offset not aligned"; return false; }
        const size_t rb = type_row_bytes(t.type_id, t.ne[0]);
        uint64_t rows = 1, total = 0;
        bool overflow = false;
        for (int d = 1; d < 4; d++) overflow |= __builtin_mul_overflow(rows, t.ne[d], &rows);
        overflow |= __builtin_mul_overflow((uint64_t)rb, rows, &total);
        if (overflow) { err = "tensor " + t.name + ": implausible shape"; return false; }
        t.n_bytes = (size_t)total;
        if (t.offset > f.size - f.data_off || t.n_bytes > f.size - f.data_off - t.offset) {
            err = "tensor " + t.name + ": data runs past the end of the file";
            return false;
        }
        t.data = f.base + f.data_off + t.offset;
    }
    return true;
}

const Value *find(const File *f, const char *key) {
    for (const auto &kv : f->kvs)
        if (kv.first == key) return &kv.second;
    return nullptr;
}

void set_err(char *err, size_t n, const std::string &msg) {
    if (err && n) {
        std::strncpy(err, msg.c_str(), n - 1);
        err[n - 1] = 0;
    }
}

} // namespace

extern "C" {

void *krk_gguf_open(const char *path, char *err, size_t err_len) {
    if (!path) { set_err(err, err_len, "null path"); return nullptr; }
    File *f = new File();
    f->fd = open(path, O_RDONLY);
    struct stat st;
    if (f->fd < 0 || fstat(f->fd, &st) != 0 || st.st_size < 24) {
        set_err(err, err_len, std::string("cannot open ") + path);
        delete f;
        return nullptr;
    }
    f->size = (size_t)st.st_size;
    void *m = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
    if (m == MAP_FAILED) {
        set_err(err, err_len, std::string("cannot map ") + path);
        delete f;
        return nullptr;
    }
    f->base = static_cast<const uint8_t *>(m);
    std::string msg;
    if (!parse(*f, msg)) {
        set_err(err, err_len, msg);
        delete f;
        return nullptr;
    }
    return f;
}

void krk_gguf_close(void *g) { delete static_cast<File *>(g); }
int krk_gguf_version(void *g) { return g ? (int)static_cast<File *>(g)->version : 0; }
int64_t krk_gguf_tensor_count(void *g) { return g ? (int64_t)static_cast<File *>(g)->tensors.size() : 0; }
int64_t krk_gguf_kv_count(void *g) { return g ? (int64_t)static_cast<File *>(g)->kvs.size() : 0; }

int64_t krk_gguf_find_tensor(void *g, const char *name) {
    if (!g || !name) return -1;
    const File *f = static_cast<File *>(g);
    for (size_t i = 0; i < f->tensors.size(); i++)
        if (f->tensors[i].name == name) return (int64_t)i;
    return -1;
}

int krk_gguf_tensor_info(void *g, int64_t index, struct krk_gguf_tensor *out) {
    if (!g || !out) return KRK_CUDA_ENULL;
    const File *f = static_cast<File *>(g);
    if (index < 0 || (size_t)index >= f->tensors.size()) return KRK_CUDA_EARG;
    const Tensor &t = f->tensors[(size_t)index];
    out->name = t.name.c_str();
    out->type_id = (int)t.type_id;
    out->supported = krk_cuda_dtype_ok((int)t.type_id);
    out->n_dims = t.n_dims;
    for (int d = 0; d < 4; d++) out->ne[d] = (int64_t)t.ne[d];
    out->host_data = t.data;
    out->n_bytes = t.n_bytes;
    return KRK_CUDA_OK;
}

int krk_gguf_get_i64(void *g, const char *key, int64_t *out) {
    const Value *v = g && key ? find(static_cast<File *>(g), key) : nullptr;
    if (!v || v->type == kString || v->type == kArray || !out) return KRK_CUDA_EARG;
    *out = v->i;
    return KRK_CUDA_OK;
}

int krk_gguf_get_f64(void *g, const char *key, double *out) {
    const Value *v = g && key ? find(static_cast<File *>(g), key) : nullptr;
    if (!v || v->type == kString || v->type == kArray || !out) return KRK_CUDA_EARG;
    *out = v->f;
    return KRK_CUDA_OK;
}

int64_t krk_gguf_get_str(void *g, const char *key, char *buf, size_t buf_len) {
    const Value *v = g && key ? find(static_cast<File *>(g), key) : nullptr;
    if (!v || v->type != kString) return -1;
    if (buf && buf_len) {
        std::strncpy(buf, v->str.c_str(), buf_len - 1);
        buf[buf_len - 1] = 0;
    }
    return (int64_t)v->str.size();
}

int64_t krk_gguf_get_array_count(void *g, const char *key, int *elem_type) {
    const Value *v = g && key ? find(static_cast<File *>(g), key) : nullptr;
    if (!v || v->type != kArray) return -1;
    if (elem_type) *elem_type = (int)v->elem;
    return (int64_t)v->count;
}

void *krk_gguf_upload_tensor(void *g, int64_t index, void *backend) {
    // The tensor's bytes as they lie in the file, into memory from the backend's alloc(): the upload
    // contract of Backend::upload (include/krk/backend.hpp:720). NULL for a type this library does not size.
    if (!g || !backend) return nullptr;
    const File *f = static_cast<File *>(g);
    if (index < 0 || (size_t)index >= f->tensors.size()) return nullptr;
    const Tensor &t = f->tensors[(size_t)index];
    if (t.n_bytes == 0) return nullptr;
    void *dev = krk_cuda_backend_alloc(backend, t.n_bytes);
    if (!dev) return nullptr;
    krk_cuda_backend_upload(backend, dev, t.data, t.n_bytes, 0);
    return dev;
}

} // extern "C"
