// GGUF v2/v3 container reader: enough of GgufFile (src/gguf/container.rs:152-384) to find token_embd.weight, the
// norm weights and the biases of a checkpoint and hand their bytes to the gather and the norms.
//
// Same walk as the reference: magic, version (big-endian and anything but v2/v3 refused), tensor and KV counts,
// metadata values (scalars widened to u64 / i64 / f64, arrays of strings / ints / floats), tensor infos (name,
// n_dims 1..4, ne[] fastest first, type id, offset relative to the data section), data section at the next
// multiple of general.alignment (default 32), every tensor range bounds-checked against the file, dims reversed
// to row-major, duplicate names refused, row length checked against the block size. Tensor types this library
// cannot decode are collected over the whole file and reported in ONE error with counts and an example tensor
// each (container.rs:190-245), not raised at the first one. The file is mapped read-only; tensor data pointers
// point into the mapping and live until lokal_gguf_close.
//
// Host code only; the one device entry point, lokal_cuda_gguf_upload, copies a tensor's bytes into a fresh device
// allocation.
#include "common.cuh"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstdarg>
#include <cstring>
#include <exception>
#include <map>
#include <new>
#include <string>
#include <unordered_map>
#include <vector>

struct lokal_gguf {
    enum Kind { U64, I64, F64, BOOL, STR, ARR_STR, ARR_I64, ARR_F64 };
    struct Value {
        Kind kind;
        uint64_t u = 0;
        int64_t i = 0;
        double f = 0.0;
        std::string s;
        std::vector<std::string> arr_s;
        std::vector<const char*> arr_s_ptrs;
        std::vector<int64_t> arr_i;
        std::vector<double> arr_f;
    };
    struct Info {
        std::string name;
        std::vector<uint64_t> dims;  // row-major
        int type;
        uint64_t start, nbytes;
    };
    const unsigned char* map = nullptr;
    size_t len = 0;
    uint32_t version = 0;
    uint64_t data_start = 0;
    std::unordered_map<std::string, Value> kv;
    std::vector<Info> infos;
    std::unordered_map<std::string, size_t> by_name;
    std::string err;
};

namespace {

const char* kind_name(lokal_gguf::Kind k) {
    switch (k) {
        case lokal_gguf::U64: return "uint";
        case lokal_gguf::I64: return "int";
        case lokal_gguf::F64: return "float";
        case lokal_gguf::BOOL: return "bool";
        case lokal_gguf::STR: return "string";
        case lokal_gguf::ARR_STR: return "string array";
        case lokal_gguf::ARR_I64: return "int array";
        default: return "float array";
    }
}

// ggml type id -> name, for the types this library does not decode (ggml.h enum ggml_type; src/gguf/dequant.rs:46-78).
const char* unsupported_type_name(uint32_t id) {
    switch (id) {
        case 3: return "Q4_1";
        case 7: return "Q5_1";
        case 9: return "Q8_1";
        case 15: return "Q8_K";
        case 16: return "IQ2_XXS";
        case 17: return "IQ2_XS";
        case 18: return "IQ3_XXS";
        case 19: return "IQ1_S";
        case 21: return "IQ3_S";
        case 22: return "IQ2_S";
        case 24: case 25: case 26: case 27: return "integer tensor";
        case 28: return "F64";
        case 29: return "IQ1_M";
        default: return "unknown ggml type";
    }
}

std::string fmt(const char* f, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, f);
    vsnprintf(buf, sizeof buf, f, ap);
    va_end(ap);
    return buf;
}

// Bounds-checked little-endian cursor (container.rs:49-77). Every read either succeeds or sets `err`.
struct Cursor {
    const unsigned char* b;
    size_t len, p = 0;
    std::string err;
    bool take(size_t n, const unsigned char** out) {
        if (!err.empty()) return false;
        if (n > len || p > len - n) {
            err = fmt("GGUF truncated: need %zu bytes at offset %zu, file has %zu", n, p, len);
            return false;
        }
        *out = b + p;
        p += n;
        return true;
    }
    template <typename T>
    bool num(T* v) {
        const unsigned char* s;
        if (!take(sizeof(T), &s)) return false;
        std::memcpy(v, s, sizeof(T));  // the host is little-endian, like the file
        return true;
    }
    bool str(std::string* out) {
        uint64_t n;
        if (!num(&n)) return false;
        if (n > (1ull << 24)) {
            err = fmt("GGUF string of %llu bytes at offset %zu: corrupt length", (unsigned long long)n, p);
            return false;
        }
        const unsigned char* s;
        if (!take(static_cast<size_t>(n), &s)) return false;
        out->assign(reinterpret_cast<const char*>(s), static_cast<size_t>(n));
        return true;
    }
    // Scalars of GGUF value type `ty` (0..7, 10..12) widened the way the reference widens them.
    bool scalar(uint32_t ty, lokal_gguf::Value* v) {
        switch (ty) {
            case 0: { uint8_t x; if (!num(&x)) return false; v->kind = lokal_gguf::U64; v->u = x; return true; }
            case 1: { int8_t x; if (!num(&x)) return false; v->kind = lokal_gguf::I64; v->i = x; return true; }
            case 2: { uint16_t x; if (!num(&x)) return false; v->kind = lokal_gguf::U64; v->u = x; return true; }
            case 3: { int16_t x; if (!num(&x)) return false; v->kind = lokal_gguf::I64; v->i = x; return true; }
            case 4: { uint32_t x; if (!num(&x)) return false; v->kind = lokal_gguf::U64; v->u = x; return true; }
            case 5: { int32_t x; if (!num(&x)) return false; v->kind = lokal_gguf::I64; v->i = x; return true; }
            case 6: { float x; if (!num(&x)) return false; v->kind = lokal_gguf::F64; v->f = x; return true; }
            case 7: { uint8_t x; if (!num(&x)) return false; v->kind = lokal_gguf::BOOL; v->u = x != 0; return true; }
            case 10: { uint64_t x; if (!num(&x)) return false; v->kind = lokal_gguf::U64; v->u = x; return true; }
            case 11: { int64_t x; if (!num(&x)) return false; v->kind = lokal_gguf::I64; v->i = x; return true; }
            case 12: { double x; if (!num(&x)) return false; v->kind = lokal_gguf::F64; v->f = x; return true; }
            default: return false;
        }
    }
    bool value(uint32_t ty, const std::string& key, lokal_gguf::Value* v) {
        if (ty == 8) {
            v->kind = lokal_gguf::STR;
            return str(&v->s);
        }
        if (ty != 9) {
            if (ty > 12) {
                err = fmt("GGUF key %s: value type %u unsupported", key.c_str(), ty);
                return false;
            }
            return scalar(ty, v);
        }
        uint32_t et;
        uint64_t n;
        if (!num(&et) || !num(&n)) return false;
        if (n > (1ull << 26)) {
            err = fmt("GGUF array %s: %llu entries: corrupt length", key.c_str(), (unsigned long long)n);
            return false;
        }
        // Nothing is reserved for entries the file cannot hold: every entry takes at least its scalar size (a string at
        // least its 8-byte length), so a count beyond the bytes that are left is a damaged header, refused before any
        // allocation is made for it.
        static const unsigned char kMinBytes[13] = {1, 1, 2, 2, 4, 4, 4, 1, 8, 0, 8, 8, 8};
        const size_t each = et <= 12 ? kMinBytes[et] : 0;
        if (each != 0 && n > (len - p) / each) {
            err = fmt("GGUF array %s: %llu entries of at least %zu bytes, %zu bytes left in the file", key.c_str(), (unsigned long long)n,
                      each, len - p);
            return false;
        }
        if (et == 8) {
            v->kind = lokal_gguf::ARR_STR;
            v->arr_s.resize(static_cast<size_t>(n));
            for (auto& s : v->arr_s)
                if (!str(&s)) return false;
            return true;
        }
        if (et == 6 || et == 12) {
            v->kind = lokal_gguf::ARR_F64;
            v->arr_f.resize(static_cast<size_t>(n));
            for (auto& x : v->arr_f) {
                lokal_gguf::Value e;
                if (!scalar(et, &e)) return false;
                x = e.f;
            }
            return true;
        }
        if (et <= 5 || et == 7 || et == 10 || et == 11) {  // bools ride the int rail as 0 / 1
            v->kind = lokal_gguf::ARR_I64;
            v->arr_i.resize(static_cast<size_t>(n));
            for (auto& x : v->arr_i) {
                lokal_gguf::Value e;
                if (!scalar(et, &e)) return false;
                x = e.kind == lokal_gguf::I64 ? e.i : static_cast<int64_t>(e.u);
            }
            return true;
        }
        err = fmt("GGUF array %s: element type %u unsupported", key.c_str(), et);
        return false;
    }
};

int fail_open(std::string msg, char* err, size_t err_len, lokal_gguf* g, int code) {
    if (err && err_len) snprintf(err, err_len, "%s", msg.c_str());
    if (g) {
        if (g->map) munmap(const_cast<unsigned char*>(g->map), g->len);
        delete g;
    }
    return code;
}

int fail(const lokal_gguf* g, int code, std::string msg) {
    const_cast<lokal_gguf*>(g)->err = std::move(msg);
    return code;
}

const lokal_gguf::Value* find_kv(const lokal_gguf* g, const char* key, int* rc) {
    if (!g || !key) {
        *rc = LOKAL_ERR_BAD_ARG;
        return nullptr;
    }
    auto it = g->kv.find(key);
    if (it == g->kv.end()) {
        *rc = fail(g, LOKAL_ERR_NOT_FOUND, fmt("GGUF metadata key %s is missing", key));
        return nullptr;
    }
    *rc = LOKAL_OK;
    return &it->second;
}

void fill_tensor(const lokal_gguf* g, const lokal_gguf::Info& i, lokal_gguf_tensor* out) {
    out->name = i.name.c_str();
    out->n_dims = static_cast<uint32_t>(i.dims.size());
    for (size_t d = 0; d < 4; d++) out->dims[d] = d < i.dims.size() ? i.dims[d] : 1;
    out->ggml_type = i.type;
    out->file_offset = i.start;
    out->data_offset = i.start - g->data_start;
    out->nbytes = i.nbytes;
    out->data = g->map + i.start;
}

}  // namespace

extern "C" {

static int gguf_open_impl(const char* path, lokal_gguf** out, char* err, size_t err_len, lokal_gguf** partial);

// A damaged header must come back as an error code, never as an exception crossing the C boundary: allocation
// failures (and anything else the containers may throw) are caught here and the half-built handle is released.
int lokal_gguf_open(const char* path, lokal_gguf** out, char* err, size_t err_len) {
    lokal_gguf* partial = nullptr;
    try {
        return gguf_open_impl(path, out, err, err_len, &partial);
    } catch (const std::bad_alloc&) {
        if (out) *out = nullptr;
        return fail_open("out of memory while reading the GGUF header", err, err_len, partial, LOKAL_ERR_FORMAT);
    } catch (const std::exception& e) {
        if (out) *out = nullptr;
        return fail_open(fmt("GGUF header could not be read: %s", e.what()), err, err_len, partial, LOKAL_ERR_FORMAT);
    }
}

static int gguf_open_impl(const char* path, lokal_gguf** out, char* err, size_t err_len, lokal_gguf** partial) {
    // every failure below releases the handle through fail_open and returns; `partial` is read on the exception path only
    if (!path || !out) return fail_open("lokal_gguf_open: path and out must be non-null", err, err_len, nullptr, LOKAL_ERR_BAD_ARG);
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail_open(fmt("cannot open %s: %s", path, strerror(errno)), err, err_len, nullptr, LOKAL_ERR_IO);
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size <= 0) {
        close(fd);
        return fail_open(fmt("cannot map %s: empty or unreadable", path), err, err_len, nullptr, LOKAL_ERR_IO);
    }
    void* m = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (m == MAP_FAILED) return fail_open(fmt("cannot map %s: %s", path, strerror(errno)), err, err_len, nullptr, LOKAL_ERR_IO);
    lokal_gguf* g = new (std::nothrow) lokal_gguf();
    if (!g) {
        munmap(m, static_cast<size_t>(st.st_size));
        return fail_open("out of memory", err, err_len, nullptr, LOKAL_ERR_IO);
    }
    *partial = g;
    g->map = static_cast<const unsigned char*>(m);
    g->len = static_cast<size_t>(st.st_size);
    Cursor rd{g->map, g->len};

    const unsigned char* magic;
    if (!rd.take(4, &magic)) return fail_open(rd.err, err, err_len, g, LOKAL_ERR_FORMAT);
    if (std::memcmp(magic, "GGUF", 4) != 0) return fail_open(fmt("%s is not a GGUF file (bad magic)", path), err, err_len, g, LOKAL_ERR_FORMAT);
    uint32_t version;
    if (!rd.num(&version)) return fail_open(rd.err, err, err_len, g, LOKAL_ERR_FORMAT);
    const uint32_t swapped = __builtin_bswap32(version);
    if (swapped == 2 || swapped == 3)
        return fail_open("big-endian GGUF files are not supported: re-export little-endian", err, err_len, g, LOKAL_ERR_FORMAT);
    if (version < 2 || version > 3) return fail_open(fmt("GGUF version %u unsupported (v2 and v3 only)", version), err, err_len, g, LOKAL_ERR_FORMAT);
    g->version = version;
    uint64_t n_tensors, n_kv;
    if (!rd.num(&n_tensors) || !rd.num(&n_kv)) return fail_open(rd.err, err, err_len, g, LOKAL_ERR_FORMAT);

    for (uint64_t k = 0; k < n_kv; k++) {
        std::string key;
        uint32_t ty;
        lokal_gguf::Value v;
        if (!rd.str(&key) || !rd.num(&ty) || !rd.value(ty, key, &v)) return fail_open(rd.err, err, err_len, g, LOKAL_ERR_FORMAT);
        v.arr_s_ptrs.assign(v.arr_s.size(), nullptr);
        g->kv[key] = std::move(v);
    }
    for (auto& e : g->kv) {  // stable pointers for the string-array accessor, taken after the map stopped moving values
        auto& v = e.second;
        for (size_t i = 0; i < v.arr_s.size(); i++) v.arr_s_ptrs[i] = v.arr_s[i].c_str();
    }

    struct Raw {
        std::string name;
        std::vector<uint64_t> ne;
        int type;
        uint64_t offset;
    };
    std::vector<Raw> raw;
    std::map<std::string, std::pair<size_t, std::string>> unsupported;  // type name -> (count, first tensor)
    for (uint64_t t = 0; t < n_tensors; t++) {
        Raw r;
        uint32_t n_dims, ty_id;
        if (!rd.str(&r.name) || !rd.num(&n_dims)) return fail_open(rd.err, err, err_len, g, LOKAL_ERR_FORMAT);
        if (n_dims == 0 || n_dims > 4) return fail_open(fmt("tensor %s: %u dimensions", r.name.c_str(), n_dims), err, err_len, g, LOKAL_ERR_FORMAT);
        r.ne.resize(n_dims);
        for (auto& d : r.ne)
            if (!rd.num(&d)) return fail_open(rd.err, err, err_len, g, LOKAL_ERR_FORMAT);
        if (!rd.num(&ty_id) || !rd.num(&r.offset)) return fail_open(rd.err, err, err_len, g, LOKAL_ERR_FORMAT);
        const size_t be = ty_id <= 0x7fffffffu ? lokal_cuda_blk_elems(static_cast<int>(ty_id)) : 0;
        if (be == 0) {  // collected, not raised: every field of this tensor has been read, the walk stays in sync
            auto& slot = unsupported[unsupported_type_name(ty_id)];
            if (slot.first++ == 0) slot.second = r.name;
            continue;
        }
        if (r.ne[0] % be != 0)
            return fail_open(fmt("tensor %s: row length %llu is not a whole number of %zu-element blocks (type %u)", r.name.c_str(),
                                 (unsigned long long)r.ne[0], be, ty_id), err, err_len, g, LOKAL_ERR_FORMAT);
        r.type = static_cast<int>(ty_id);
        raw.push_back(std::move(r));
    }
    if (!unsupported.empty()) {
        size_t total = 0;
        std::string detail;
        for (auto& u : unsupported) {
            total += u.second.first;
            if (!detail.empty()) detail += ", ";
            detail += fmt("%s (%zu %s, e.g. %s)", u.first.c_str(), u.second.first, u.second.first == 1 ? "tensor" : "tensors", u.second.second.c_str());
        }
        return fail_open(fmt("this checkpoint uses %zu quantization type(s) this library does not decode, across %zu of %llu tensors: ",
                             unsupported.size(), total, (unsigned long long)n_tensors) + detail, err, err_len, g, LOKAL_ERR_UNSUPPORTED);
    }

    uint64_t align = 32;
    auto al = g->kv.find("general.alignment");
    if (al != g->kv.end()) {
        const auto& v = al->second;
        if (v.kind != lokal_gguf::U64 || v.u == 0 || (v.u & (v.u - 1)) != 0)
            return fail_open(fmt("general.alignment is invalid (%s)", kind_name(v.kind)), err, err_len, g, LOKAL_ERR_FORMAT);
        align = v.u;
    }
    g->data_start = (rd.p + align - 1) / align * align;

    for (auto& r : raw) {
        unsigned __int128 elems = 1;
        for (auto d : r.ne) {
            elems *= d;
            if (elems >= (static_cast<unsigned __int128>(1) << 62)) return fail_open(fmt("tensor %s: element count overflow", r.name.c_str()), err, err_len, g, LOKAL_ERR_FORMAT);
        }
        // bytes in 128-bit arithmetic: elems / block elements * block bytes must itself fit the file
        const unsigned __int128 wide = elems / lokal_cuda_blk_elems(r.type) * lokal_cuda_blk_bytes(r.type);
        if (wide > g->len) return fail_open(fmt("tensor %s: its bytes run past the file", r.name.c_str()), err, err_len, g, LOKAL_ERR_FORMAT);
        const uint64_t nbytes = static_cast<uint64_t>(wide);
        const uint64_t start = g->data_start + r.offset;
        if (start < g->data_start) return fail_open(fmt("tensor %s: offset overflow", r.name.c_str()), err, err_len, g, LOKAL_ERR_FORMAT);
        if (nbytes > g->len || start > g->len - nbytes)
            return fail_open(fmt("tensor %s: %llu bytes at data offset %llu run past the file", r.name.c_str(), (unsigned long long)nbytes,
                                 (unsigned long long)r.offset), err, err_len, g, LOKAL_ERR_FORMAT);
        lokal_gguf::Info info;
        info.name = r.name;
        info.dims.assign(r.ne.rbegin(), r.ne.rend());  // fastest-first -> row-major
        info.type = r.type;
        info.start = start;
        info.nbytes = nbytes;
        if (!g->by_name.emplace(info.name, g->infos.size()).second)
            return fail_open(fmt("tensor %s appears twice", r.name.c_str()), err, err_len, g, LOKAL_ERR_FORMAT);
        g->infos.push_back(std::move(info));
    }
    *out = g;
    return LOKAL_OK;
}

void lokal_gguf_close(lokal_gguf* g) {
    if (!g) return;
    if (g->map) munmap(const_cast<unsigned char*>(g->map), g->len);
    delete g;
}

const char* lokal_gguf_last_error(const lokal_gguf* g) { return g ? g->err.c_str() : "null GGUF handle"; }
uint32_t lokal_gguf_version(const lokal_gguf* g) { return g ? g->version : 0; }
size_t lokal_gguf_n_tensors(const lokal_gguf* g) { return g ? g->infos.size() : 0; }
uint64_t lokal_gguf_data_start(const lokal_gguf* g) { return g ? g->data_start : 0; }

int lokal_gguf_tensor_at(const lokal_gguf* g, size_t i, lokal_gguf_tensor* out) {
    if (!g || !out) return LOKAL_ERR_BAD_ARG;
    if (i >= g->infos.size()) return fail(g, LOKAL_ERR_NOT_FOUND, fmt("tensor index %zu out of %zu", i, g->infos.size()));
    fill_tensor(g, g->infos[i], out);
    return LOKAL_OK;
}

int lokal_gguf_find_tensor(const lokal_gguf* g, const char* name, lokal_gguf_tensor* out) {
    if (!g || !name || !out) return LOKAL_ERR_BAD_ARG;
    auto it = g->by_name.find(name);
    if (it == g->by_name.end()) return fail(g, LOKAL_ERR_NOT_FOUND, fmt("tensor %s not in the GGUF file", name));
    fill_tensor(g, g->infos[it->second], out);
    return LOKAL_OK;
}

int lokal_gguf_has_key(const lokal_gguf* g, const char* key) { return g && key && g->kv.count(key) ? 1 : 0; }

int lokal_gguf_get_u64(const lokal_gguf* g, const char* key, uint64_t* out) {
    int rc;
    const auto* v = find_kv(g, key, &rc);
    if (!v) return rc;
    if (!out) return LOKAL_ERR_BAD_ARG;
    if (v->kind == lokal_gguf::U64) *out = v->u;
    else if (v->kind == lokal_gguf::I64 && v->i >= 0) *out = static_cast<uint64_t>(v->i);
    else return fail(g, LOKAL_ERR_BAD_ARG, fmt("GGUF key %s is a %s, expected an integer", key, kind_name(v->kind)));
    return LOKAL_OK;
}

int lokal_gguf_get_f32(const lokal_gguf* g, const char* key, float* out) {
    int rc;
    const auto* v = find_kv(g, key, &rc);
    if (!v) return rc;
    if (!out) return LOKAL_ERR_BAD_ARG;
    if (v->kind != lokal_gguf::F64) return fail(g, LOKAL_ERR_BAD_ARG, fmt("GGUF key %s is a %s, expected a float", key, kind_name(v->kind)));
    *out = static_cast<float>(v->f);
    return LOKAL_OK;
}

int lokal_gguf_get_str(const lokal_gguf* g, const char* key, const char** out, size_t* len) {
    int rc;
    const auto* v = find_kv(g, key, &rc);
    if (!v) return rc;
    if (!out) return LOKAL_ERR_BAD_ARG;
    if (v->kind != lokal_gguf::STR) return fail(g, LOKAL_ERR_BAD_ARG, fmt("GGUF key %s is a %s, expected a string", key, kind_name(v->kind)));
    *out = v->s.c_str();
    if (len) *len = v->s.size();
    return LOKAL_OK;
}

int lokal_gguf_get_arr_i64(const lokal_gguf* g, const char* key, const int64_t** out, size_t* n) {
    int rc;
    const auto* v = find_kv(g, key, &rc);
    if (!v) return rc;
    if (!out || !n) return LOKAL_ERR_BAD_ARG;
    if (v->kind != lokal_gguf::ARR_I64) return fail(g, LOKAL_ERR_BAD_ARG, fmt("GGUF key %s is a %s, expected an int array", key, kind_name(v->kind)));
    *out = v->arr_i.data();
    *n = v->arr_i.size();
    return LOKAL_OK;
}

int lokal_gguf_get_arr_str(const lokal_gguf* g, const char* key, const char* const** out, size_t* n) {
    int rc;
    const auto* v = find_kv(g, key, &rc);
    if (!v) return rc;
    if (!out || !n) return LOKAL_ERR_BAD_ARG;
    if (v->kind != lokal_gguf::ARR_STR) return fail(g, LOKAL_ERR_BAD_ARG, fmt("GGUF key %s is a %s, expected a string array", key, kind_name(v->kind)));
    *out = v->arr_s_ptrs.data();
    *n = v->arr_s_ptrs.size();
    return LOKAL_OK;
}

int lokal_cuda_gguf_upload(lokal_cuda_ctx* ctx, lokal_cuda_stream s, const lokal_gguf* g, const char* name, void** dptr, lokal_gguf_tensor* info) {
    if (!ctx) return LOKAL_ERR_BAD_ARG;
    lokal::DeviceGuard guard(ctx->device);
    if (!guard.ok) return ctx->fail(LOKAL_ERR_CUDA, "cannot select device %d", ctx->device);
    if (!g || !name || !dptr) return ctx->fail(LOKAL_ERR_BAD_ARG, "gguf_upload: file, name and dptr must be non-null");
    lokal_gguf_tensor t;
    const int rc = lokal_gguf_find_tensor(g, name, &t);
    if (rc != LOKAL_OK) return ctx->fail(rc, "gguf_upload: %s", lokal_gguf_last_error(g));
    void* d = nullptr;
    LOKAL_CUDA_TRY(ctx, cudaMalloc(&d, t.nbytes ? t.nbytes : 1));
    cudaStream_t st = static_cast<cudaStream_t>(s);
    // The mapping is pageable memory: the copy is staged by the driver and has left the mapping when the call
    // returns, so the file may be closed right after.
    cudaError_t e = cudaMemcpyAsync(d, t.data, t.nbytes, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) {
        cudaFree(d);
        return ctx->fail(LOKAL_ERR_CUDA, "gguf_upload: copy of %s failed: %s", name, cudaGetErrorString(e));
    }
    *dptr = d;
    if (info) *info = t;
    return LOKAL_OK;
}

}  // extern "C"
