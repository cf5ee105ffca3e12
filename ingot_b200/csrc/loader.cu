// Host side of the weight loader: a safetensors file mapped read-only, its header parsed into a tensor table, and the
// two byte-level transforms the reference applies while building device layouts (lossless 4 -> 8-bit widening).
// No CUDA here: the functions run on any host; the caller uploads the bytes.
//
// Mirrors Loader/Safetensors.swift:46-148 (MappedFile, SafetensorsStore.parseHeader / info / bytes) and
// Layers/Linear.swift:599-610 (widen4to8Words), :170-175 (scales of a widened piece divided by 16).
#include <errno.h>
#include <fcntl.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <new>
#include <string>
#include <vector>

#include "../../include/ingot_qmm.h"

namespace {

thread_local char g_st_error[320] = {0};

int32_t st_fail(int32_t code, const char* fmt, const char* a = "", const char* b = "") {
    snprintf(g_st_error, sizeof(g_st_error), fmt, a, b);
    return code;
}

struct Entry {
    std::string name;
    int32_t dtype;
    std::vector<int64_t> shape;
    uint64_t begin, end;  // data_offsets, relative to the end of the header
};

// A cursor over the header's JSON. The grammar needed is small: an object of objects whose members are strings, integers
// and arrays of integers; anything else (the free-form "__metadata__") is skipped as a generic value.
struct Json {
    const char* p;
    const char* e;
    void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++; }
    bool eat(char c) { ws(); if (p < e && *p == c) { p++; return true; } return false; }
    bool string(std::string* out) {
        ws();
        if (p >= e || *p != '"') return false;
        p++;
        std::string s;
        while (p < e && *p != '"') {
            if (*p == '\\') {
                if (p + 1 >= e) return false;
                const char c = p[1];
                if (c == 'u') {  // \uXXXX: kept verbatim (tensor names are ASCII; exactness only matters for lookups)
                    if (p + 6 > e) return false;
                    s.append(p, 6);
                    p += 6;
                    continue;
                }
                s.push_back(c == 'n' ? '\n' : c == 't' ? '\t' : c == 'r' ? '\r' : c == 'b' ? '\b' : c == 'f' ? '\f' : c);
                p += 2;
            } else {
                s.push_back(*p++);
            }
        }
        if (p >= e) return false;
        p++;
        if (out) *out = s;
        return true;
    }
    bool integer(int64_t* out) {
        ws();
        const char* q = p;
        bool neg = false;
        if (q < e && *q == '-') { neg = true; q++; }
        if (q >= e || *q < '0' || *q > '9') return false;
        int64_t v = 0;
        while (q < e && *q >= '0' && *q <= '9') {
            if (v > (INT64_MAX - 9) / 10) return false;
            v = v * 10 + (*q++ - '0');
        }
        if (q < e && (*q == '.' || *q == 'e' || *q == 'E')) return false;  // not an integer
        p = q;
        *out = neg ? -v : v;
        return true;
    }
    bool skip_value(int depth = 0) {
        if (depth > 64) return false;
        ws();
        if (p >= e) return false;
        if (*p == '"') return string(nullptr);
        if (*p == '{' || *p == '[') {
            const char close = *p == '{' ? '}' : ']';
            const bool obj = *p == '{';
            p++;
            if (eat(close)) return true;
            for (;;) {
                if (obj) {
                    if (!string(nullptr) || !eat(':')) return false;
                }
                if (!skip_value(depth + 1)) return false;
                if (eat(',')) continue;
                return eat(close);
            }
        }
        // number, true, false, null
        const char* q = p;
        while (q < e && *q != ',' && *q != '}' && *q != ']' && *q != ' ' && *q != '\n' && *q != '\t' && *q != '\r') q++;
        if (q == p) return false;
        p = q;
        return true;
    }
};

int32_t dtype_of(const std::string& s, int* size) {
    struct { const char* n; int32_t id; int size; } t[] = {{"BF16", IQ_ST_BF16, 2}, {"F16", IQ_ST_F16, 2}, {"F32", IQ_ST_F32, 4},
                                                             {"U32", IQ_ST_U32, 4}, {"I32", IQ_ST_I32, 4}, {"U8", IQ_ST_U8, 1}};
    for (auto& x : t)
        if (s == x.n) { *size = x.size; return x.id; }
    return -1;
}

}  // namespace

struct iq_st {
    std::string path;
    void* base = nullptr;
    size_t file_size = 0, mapped = 0;
    uint64_t data_start = 0;
    std::vector<Entry> entries;
};

extern "C" const char* iq_st_last_error(void) { return g_st_error; }

extern "C" void iq_st_close(iq_st* f) {
    if (f == nullptr) return;
    if (f->base != nullptr) munmap(f->base, f->mapped);
    delete f;
}

extern "C" int32_t iq_st_open(const char* path, iq_st** out) {
    if (path == nullptr || out == nullptr) return st_fail(IQ_ERR_INVALID_ARG, "st_open: null argument");
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return st_fail(IQ_ERR_IO, "I/O: cannot open %s", path);
    struct stat sb;
    if (fstat(fd, &sb) != 0) { close(fd); return st_fail(IQ_ERR_IO, "I/O: fstat %s", path); }
    iq_st* f = new (std::nothrow) iq_st();
    if (f == nullptr) { close(fd); return st_fail(IQ_ERR_IO, "I/O: out of memory"); }
    f->path = path;
    f->file_size = (size_t)sb.st_size;
    if (f->file_size < 8) { close(fd); delete f; return st_fail(IQ_ERR_FORMAT, "format: %s too short", path); }
    const size_t page = (size_t)getpagesize();
    f->mapped = (f->file_size + page - 1) / page * page;
    void* m = mmap(nullptr, f->mapped, PROT_READ, MAP_PRIVATE, fd, 0);  // the pages stay the system cache's
    close(fd);
    if (m == MAP_FAILED) { delete f; return st_fail(IQ_ERR_IO, "I/O: mmap %s", path); }
    f->base = m;
    // header: little-endian u64 with the length N, N bytes of JSON, then the data
    uint64_t n = 0;
    memcpy(&n, m, 8);
    if (n > f->file_size - 8) { iq_st_close(f); return st_fail(IQ_ERR_FORMAT, "format: header out of range in %s", path); }
    f->data_start = 8 + n;
    Json j{static_cast<const char*>(m) + 8, static_cast<const char*>(m) + 8 + n};
    if (!j.eat('{')) { iq_st_close(f); return st_fail(IQ_ERR_FORMAT, "format: header of %s is not a JSON object", path); }
    if (!j.eat('}')) {
        for (;;) {
            Entry en;
            if (!j.string(&en.name) || !j.eat(':')) { iq_st_close(f); return st_fail(IQ_ERR_FORMAT, "format: malformed header in %s", path); }
            if (en.name == "__metadata__") {
                if (!j.skip_value()) { iq_st_close(f); return st_fail(IQ_ERR_FORMAT, "format: malformed __metadata__ in %s", path); }
            } else {
                std::string dt;
                bool have_dt = false, have_shape = false, have_off = false, ok = j.eat('{');
                while (ok) {
                    std::string key;
                    if (!j.string(&key) || !j.eat(':')) { ok = false; break; }
                    if (key == "dtype") {
                        ok = j.string(&dt);
                        have_dt = ok;
                    } else if (key == "shape" || key == "data_offsets") {
                        std::vector<int64_t> v;
                        ok = j.eat('[');
                        if (ok && !j.eat(']')) {
                            for (;;) {
                                int64_t x;
                                if (!j.integer(&x) || x < 0) { ok = false; break; }
                                v.push_back(x);
                                if (j.eat(',')) continue;
                                ok = j.eat(']');
                                break;
                            }
                        }
                        if (ok && key == "shape") { en.shape = v; have_shape = true; }
                        if (ok && key == "data_offsets") {
                            if (v.size() != 2) ok = false;
                            else { en.begin = (uint64_t)v[0]; en.end = (uint64_t)v[1]; have_off = true; }
                        }
                    } else {
                        ok = j.skip_value();
                    }
                    if (!ok) break;
                    if (j.eat(',')) continue;
                    ok = j.eat('}');
                    break;
                }
                int esz = 0;
                en.dtype = ok && have_dt ? dtype_of(dt, &esz) : -1;
                if (!ok || !have_dt || !have_shape || !have_off || en.dtype < 0 || en.shape.size() > 8) {
                    const std::string nm = en.name;
                    iq_st_close(f);
                    return st_fail(IQ_ERR_FORMAT, "format: malformed entry: %s", nm.c_str());
                }
                // element count times element size, refused when the product leaves 64 bits (the reference's Swift
                // multiplication traps there): a wrapped product must not pass the size check below
                uint64_t count = 1;
                bool overflow = false;
                for (int64_t d : en.shape)
                    overflow = overflow || d < 0 || __builtin_mul_overflow(count, (uint64_t)d, &count);
                uint64_t want_bytes = 0;
                overflow = overflow || __builtin_mul_overflow(count, (uint64_t)esz, &want_bytes);
                if (overflow || en.end < en.begin || en.end - en.begin != want_bytes || f->data_start + en.end > f->file_size) {
                    const std::string nm = en.name;
                    iq_st_close(f);
                    return st_fail(IQ_ERR_FORMAT, "format: inconsistent size in %s", nm.c_str());
                }
                f->entries.push_back(en);
            }
            if (j.eat(',')) continue;
            if (!j.eat('}')) { iq_st_close(f); return st_fail(IQ_ERR_FORMAT, "format: malformed header in %s", path); }
            break;
        }
    }
    *out = f;
    return IQ_OK;
}

extern "C" int32_t iq_st_count(const iq_st* f) { return f == nullptr ? 0 : (int32_t)f->entries.size(); }

static void fill(const iq_st* f, const Entry& en, iq_st_tensor* t) {
    t->name = en.name.c_str();
    t->dtype = en.dtype;
    t->rank = (int32_t)en.shape.size();
    for (int i = 0; i < 8; i++) t->shape[i] = i < (int)en.shape.size() ? en.shape[i] : 0;
    t->file_offset = f->data_start + en.begin;
    t->bytes = en.end - en.begin;
    t->data = static_cast<const unsigned char*>(f->base) + t->file_offset;
}

extern "C" int32_t iq_st_entry(const iq_st* f, int32_t index, iq_st_tensor* out) {
    if (f == nullptr || out == nullptr || index < 0 || index >= (int32_t)f->entries.size())
        return st_fail(IQ_ERR_INVALID_ARG, "st_entry: index out of range");
    fill(f, f->entries[index], out);
    return IQ_OK;
}

extern "C" int32_t iq_st_find(const iq_st* f, const char* name, iq_st_tensor* out) {
    if (f == nullptr || name == nullptr || out == nullptr) return st_fail(IQ_ERR_INVALID_ARG, "st_find: null argument");
    for (const Entry& en : f->entries)
        if (en.name == name) { fill(f, en, out); return IQ_OK; }
    return st_fail(IQ_ERR_MISSING, "no such tensor %s", name);
}

// Packed MLX 4-bit words (8 values each, low nibble first) to 8-bit words with each value times 16; src may be
// unaligned (straight from the mapping). Linear.swift:599-610.
extern "C" void iq_widen4to8_words(const void* src, void* dst, size_t source_words) {
    const unsigned char* s = static_cast<const unsigned char*>(src);
    uint32_t* d = static_cast<uint32_t*>(dst);
    for (size_t i = 0; i < source_words; i++) {
        uint32_t x;
        memcpy(&x, s + 4 * i, 4);
        uint32_t lo = 0, hi = 0;
        for (int j = 0; j < 4; j++) {
            lo |= ((x >> (4 * j)) & 0xFu) << (8 * j + 4);
            hi |= ((x >> (4 * j + 16)) & 0xFu) << (8 * j + 4);
        }
        d[2 * i] = lo;
        d[2 * i + 1] = hi;
    }
}

// bf16 scales of a piece widened from 4 to 8 bits: divided by 16, which is exact in bf16 (Linear.swift:170-175).
extern "C" void iq_scales_div16_bf16(const void* src, void* dst, size_t count) {
    const unsigned char* s = static_cast<const unsigned char*>(src);
    uint16_t* d = static_cast<uint16_t*>(dst);
    for (size_t i = 0; i < count; i++) {
        uint16_t v;
        memcpy(&v, s + 2 * i, 2);
        uint32_t u = (uint32_t)v << 16;
        float f;
        memcpy(&f, &u, 4);
        f /= 16.0f;
        memcpy(&u, &f, 4);
        d[i] = (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);  // round to nearest even (Quant.swift:121-125)
    }
}
