// GGUF container reader and ggml element decoders (host code; the host compiler runs with floating-point contraction
// off, so a product followed by a difference rounds twice, as the reference's decoders do).
#include "it_gguf.h"
#include "it_internal.h"
#include <cstring>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

bool it_gg_block(uint32_t type, size_t* be, size_t* bb) {
    switch (type) {
        case GG_F32: *be = 1; *bb = 4; return true;
        case GG_F16: case GG_BF16: *be = 1; *bb = 2; return true;
        case GG_Q8_0: *be = 32; *bb = 34; return true;
        case GG_Q4_K: *be = 256; *bb = 144; return true;
        case GG_Q6_K: *be = 256; *bb = 210; return true;
        case GG_PQ2_0: *be = 128; *bb = 34; return true;
        case GG_PTQ1_0: *be = 128; *bb = 28; return true;
    }
    return false;
}
const char* it_gg_type_name(uint32_t type) {
    switch (type) {
        case GG_F32: return "F32"; case GG_F16: return "F16"; case GG_BF16: return "BF16"; case GG_Q8_0: return "Q8_0";
        case GG_Q4_K: return "Q4_K"; case GG_Q6_K: return "Q6_K"; case GG_PQ2_0: return "PQ2_0"; case GG_PTQ1_0: return "PTQ1_0";
    }
    return "unknown";
}

bool it_gguf_value::as_u64(uint64_t* v) const {
    if (!is_int()) return false;
    if (type == GV_U8 || type == GV_U16 || type == GV_U32 || type == GV_U64) { *v = u; return true; }
    if (i < 0) return false;
    *v = (uint64_t)i; return true;
}
bool it_gguf_value::as_f32(float* v) const { if (type != GV_F32 && type != GV_F64) return false; *v = (float)f; return true; }
bool it_gguf_value::as_bool(bool* v) const { if (type != GV_BOOL) return false; *v = u != 0; return true; }

namespace {
// A cursor over the mapping; every read is bounds-checked and a short file turns into `ok = false`.
struct Cursor {
    const uint8_t* b; size_t n, p; bool ok;
    const uint8_t* take(size_t k) { if (!ok || k > n - p) { ok = false; return nullptr; } const uint8_t* r = b + p; p += k; return r; }
    template <typename T> T le() { T v{}; const uint8_t* s = take(sizeof(T)); if (s) memcpy(&v, s, sizeof(T)); return v; }
    bool str(std::string* out) { const uint64_t k = le<uint64_t>(); if (!ok || k > n - p) { ok = false; return false; } out->assign((const char*)b + p, (size_t)k); p += (size_t)k; return true; }
};
size_t scalar_bytes(uint32_t t) {
    switch (t) { case GV_U8: case GV_I8: case GV_BOOL: return 1; case GV_U16: case GV_I16: return 2; case GV_U32: case GV_I32: case GV_F32: return 4;
                 case GV_U64: case GV_I64: case GV_F64: return 8; }
    return 0;
}
// one scalar of kind t into v (u / i / f by kind)
bool read_scalar(Cursor& c, uint32_t t, it_gguf_value* v) {
    switch (t) {
        case GV_U8: v->u = c.le<uint8_t>(); break; case GV_I8: v->i = c.le<int8_t>(); break;
        case GV_U16: v->u = c.le<uint16_t>(); break; case GV_I16: v->i = c.le<int16_t>(); break;
        case GV_U32: v->u = c.le<uint32_t>(); break; case GV_I32: v->i = c.le<int32_t>(); break;
        case GV_F32: v->f = c.le<float>(); break; case GV_BOOL: v->u = c.le<uint8_t>() != 0; break;
        case GV_U64: v->u = c.le<uint64_t>(); break; case GV_I64: v->i = c.le<int64_t>(); break; case GV_F64: v->f = c.le<double>(); break;
        default: return false;
    }
    return c.ok;
}
}  // namespace

it_gguf::~it_gguf() { if (base_) munmap((void*)base_, len_); }

int it_gguf::open(const char* path) {
    if (!path || !*path) return it_fail(IT_EINVAL, "gguf: empty path");
    if (base_) return it_fail(IT_ESTATE, "gguf: already open");
    path_ = path;
    const int fd = ::open(path, O_RDONLY);
    if (fd < 0) return it_fail(IT_EFORMAT, "gguf: cannot open %s: %s", path, strerror(errno));
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 24) { ::close(fd); return it_fail(IT_EFORMAT, "gguf: %s is not a GGUF file (too short)", path); }
    void* m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED) return it_fail(IT_EFORMAT, "gguf: cannot map %s: %s", path, strerror(errno));
    base_ = (const uint8_t*)m; len_ = (size_t)st.st_size;
    Cursor c{ base_, len_, 0, true };
    const uint8_t* magic = c.take(4);
    if (!magic || memcmp(magic, "GGUF", 4) != 0) return it_fail(IT_EFORMAT, "gguf: %s is not a GGUF file (bad magic)", path);
    version_ = c.le<uint32_t>();
    if (version_ < 2 || version_ > 3) return it_fail(IT_EFORMAT, "gguf: unsupported container version %u", version_);
    const uint64_t nt = c.le<uint64_t>(), nkv = c.le<uint64_t>();
    if (!c.ok || nt > len_ || nkv > len_) return it_fail(IT_EFORMAT, "gguf: implausible tensor or metadata count");
    for (uint64_t k = 0; k < nkv; k++) {
        std::string key; it_gguf_value v;
        if (!c.str(&key)) return it_fail(IT_EFORMAT, "gguf: unexpected end of file in the metadata");
        v.raw_off = c.p; v.type = c.le<uint32_t>();
        if (v.type == GV_STR) { c.str(&v.s); }
        else if (v.type == GV_ARR) {
            v.elem_type = c.le<uint32_t>(); v.count = c.le<uint64_t>();
            if (!c.ok || v.elem_type == GV_ARR || v.elem_type > GV_F64 || v.count > len_ - c.p) return it_fail(IT_EFORMAT, "gguf: bad array type or length for key %s", key.c_str());
            const bool keep = key.compare(0, 10, "tokenizer.") != 0;
            if (v.elem_type == GV_STR) {
                std::string s;
                for (uint64_t j = 0; j < v.count && c.ok; j++) { c.str(&s); if (keep) v.strs.push_back(s); }
            } else if (!keep) { c.take((size_t)v.count * scalar_bytes(v.elem_type)); }
            else {
                it_gguf_value el; el.type = v.elem_type;
                const bool fl = v.elem_type == GV_F32 || v.elem_type == GV_F64;
                for (uint64_t j = 0; j < v.count && c.ok; j++) {
                    read_scalar(c, v.elem_type, &el);
                    if (fl) v.floats.push_back(el.f);
                    else { uint64_t uu; v.ints.push_back(el.as_u64(&uu) ? (int64_t)uu : el.i); }
                }
            }
        } else if (!read_scalar(c, v.type, &v)) {
            if (c.ok) return it_fail(IT_EFORMAT, "gguf: bad value type %u for key %s", v.type, key.c_str());
        }
        if (!c.ok) return it_fail(IT_EFORMAT, "gguf: unexpected end of file in the metadata");
        v.raw_len = c.p - v.raw_off;
        if (!kv_.emplace(key, std::move(v)).second) return it_fail(IT_EFORMAT, "gguf: duplicate metadata key %s", key.c_str());
    }
    tensors_.reserve((size_t)nt);
    for (uint64_t k = 0; k < nt; k++) {
        it_gguf_tensor t;
        if (!c.str(&t.name)) return it_fail(IT_EFORMAT, "gguf: unexpected end of file in the tensor directory");
        const uint32_t nd = c.le<uint32_t>();
        if (!c.ok || nd < 1 || nd > 4) return it_fail(IT_EFORMAT, "gguf: tensor %s has rank %u", t.name.c_str(), nd);
        t.nelem = 1;
        for (uint32_t d = 0; d < nd; d++) {
            const uint64_t e = c.le<uint64_t>(); t.dims.push_back(e);
            if (e == 0 || (t.nelem != 0 && e > UINT64_MAX / t.nelem)) return it_fail(IT_EFORMAT, "gguf: tensor %s has bad dimensions", t.name.c_str());
            t.nelem *= e;
        }
        t.type = c.le<uint32_t>(); t.offset = c.le<uint64_t>(); t.nbytes = 0;
        if (!c.ok) return it_fail(IT_EFORMAT, "gguf: unexpected end of file in the tensor directory");
        if (!index_.emplace(t.name, tensors_.size()).second) return it_fail(IT_EFORMAT, "gguf: duplicate tensor name %s", t.name.c_str());
        tensors_.push_back(std::move(t));
    }
    uint64_t align = 32;
    if (const it_gguf_value* a = get("general.alignment")) if (!a->as_u64(&align)) align = 0;
    if (align == 0 || (align & (align - 1)) != 0 || align > 65536) return it_fail(IT_EFORMAT, "gguf: bad general.alignment");
    data_off_ = (c.p + (size_t)align - 1) / (size_t)align * (size_t)align;
    if (data_off_ > len_) return it_fail(IT_EFORMAT, "gguf: unexpected end of file before the tensor data");
    for (it_gguf_tensor& t : tensors_) {
        size_t be, bb;
        if (!it_gg_block(t.type, &be, &bb)) continue;                 // a type this library never reads: bounds unknown
        if (t.dims[0] % be) return it_fail(IT_EFORMAT, "gguf: tensor %s: row length %llu is not a multiple of the %s block", t.name.c_str(), (unsigned long long)t.dims[0], it_gg_type_name(t.type));
        const uint64_t blocks = t.nelem / be;
        if (blocks > (UINT64_MAX - t.offset) / bb) return it_fail(IT_EFORMAT, "gguf: tensor %s: size overflow", t.name.c_str());
        t.nbytes = blocks * bb;
        if (t.offset > len_ - data_off_ || t.nbytes > len_ - data_off_ - t.offset) return it_fail(IT_EFORMAT, "gguf: tensor %s lies outside the file", t.name.c_str());
    }
    return IT_OK;
}

const it_gguf_value* it_gguf::get(const std::string& key) const { auto it = kv_.find(key); return it == kv_.end() ? nullptr : &it->second; }
int it_gguf::u(const std::string& key, uint64_t* v) const {
    const it_gguf_value* x = get(key);
    if (!x || !x->as_u64(v)) return it_fail(IT_EFORMAT, "gguf: missing key %s", key.c_str());
    return IT_OK;
}
int it_gguf::f(const std::string& key, float* v) const {
    const it_gguf_value* x = get(key);
    if (!x || !x->as_f32(v)) return it_fail(IT_EFORMAT, "gguf: missing key %s", key.c_str());
    return IT_OK;
}
std::vector<std::string> it_gguf::strings(const std::string& key) const {
    const it_gguf_value* x = get(key);
    return x && x->type == GV_ARR && x->elem_type == GV_STR ? x->strs : std::vector<std::string>();
}
const it_gguf_tensor* it_gguf::tensor(const std::string& name) const { auto it = index_.find(name); return it == index_.end() ? nullptr : &tensors_[it->second]; }
int it_gguf::need(const std::string& name, const it_gguf_tensor** t) const {
    *t = tensor(name);
    if (!*t) return it_fail(IT_EFORMAT, "gguf: missing tensor %s", name.c_str());
    size_t be, bb;
    if (!it_gg_block((*t)->type, &be, &bb)) return it_fail(IT_EUNSUPPORTED, "gguf: tensor %s has ggml type %u, which this library does not read", name.c_str(), (*t)->type);
    return IT_OK;
}

// ---------------------------------------------------------------- element decoders
namespace {
inline float f16_at(const uint8_t* p) { unsigned short b = (unsigned short)(p[0] | (p[1] << 8)); __half h; memcpy(&h, &b, 2); return __half2float(h); }
inline float bf16_at(const uint8_t* p) { const uint32_t u = ((uint32_t)p[0] | ((uint32_t)p[1] << 8)) << 16; float f; memcpy(&f, &u, 4); return f; }
// base-3 digit n of a PTQ1_0 byte: the byte times 3^n (mod 256), then the top "trit" of the result
inline uint8_t trit(uint8_t byte, int n) { static const uint8_t pow3[5] = { 1, 3, 9, 27, 81 }; const uint8_t q = (uint8_t)(byte * pow3[n]); return (uint8_t)(((unsigned)q * 3) >> 8); }
// the 128 codes (value = code - 1) of a PTQ1_0 block in element order: runs of 32, 16 and 8 bytes holding five digits
// each, digit-major inside a run, then two bytes holding four digits each
void ptq1_codes(const uint8_t* b, uint8_t* codes) {
    static const int runs[3] = { 32, 16, 8 };
    int o = 0, j = 0;
    for (int s = 0; s < 3; s++) {
        const int c = runs[s];
        while (j + c <= 24) { for (int n = 0; n < 5; n++) for (int m = 0; m < c; m++) codes[o++] = trit(b[j + m], n); j += c; }
    }
    for (int n = 0; n < 4; n++) for (int h = 0; h < 2; h++) codes[o++] = trit(b[24 + h], n);
}
inline void k4_scale_min(int j, const uint8_t* q, uint8_t* sc, uint8_t* mn) {
    if (j < 4) { *sc = q[j] & 63; *mn = q[j + 4] & 63; }
    else { *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4)); *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4)); }
}
}  // namespace

void it_gg_ptq1_to_pq2(const uint8_t* src, size_t nblocks, uint8_t* dst) {
    uint8_t codes[128];
    for (size_t i = 0; i < nblocks; i++) {
        const uint8_t* b = src + i * 28; uint8_t* o = dst + i * 34;
        ptq1_codes(b, codes);
        o[0] = b[26]; o[1] = b[27];
        for (int w = 0; w < 32; w++) o[2 + w] = (uint8_t)(codes[4 * w] | (codes[4 * w + 1] << 2) | (codes[4 * w + 2] << 4) | (codes[4 * w + 3] << 6));
    }
}

int it_gg_dequant(uint32_t type, const uint8_t* src, size_t n, float* out) {
    size_t be, bb;
    if (!it_gg_block(type, &be, &bb)) return it_fail(IT_EUNSUPPORTED, "gguf: cannot decode ggml type %u", type);
    if (n % be) return it_fail(IT_EINVAL, "gguf: %zu elements is not a multiple of the %s block", n, it_gg_type_name(type));
    const size_t nb = n / be;
    switch (type) {
        case GG_F32: memcpy(out, src, n * 4); break;
        case GG_F16: for (size_t i = 0; i < n; i++) out[i] = f16_at(src + 2 * i); break;
        case GG_BF16: for (size_t i = 0; i < n; i++) out[i] = bf16_at(src + 2 * i); break;
        case GG_Q8_0:
            for (size_t i = 0; i < nb; i++) { const uint8_t* b = src + i * 34; const float d = f16_at(b); for (int j = 0; j < 32; j++) out[i * 32 + j] = (float)(int8_t)b[2 + j] * d; }
            break;
        case GG_PQ2_0:
            for (size_t i = 0; i < nb; i++) { const uint8_t* b = src + i * 34; const float d = f16_at(b);
                for (int j = 0; j < 128; j++) out[i * 128 + j] = (float)((int)((b[2 + j / 4] >> ((j % 4) * 2)) & 3) - 1) * d; }
            break;
        case GG_PTQ1_0: {
            uint8_t codes[128];
            for (size_t i = 0; i < nb; i++) { const uint8_t* b = src + i * 28; const float d = f16_at(b + 26); ptq1_codes(b, codes);
                for (int j = 0; j < 128; j++) out[i * 128 + j] = (float)((int)codes[j] - 1) * d; }
            break; }
        case GG_Q4_K:   // d, dmin (f16), 12 bytes of packed 6-bit scales and mins, 128 bytes of nibbles; 8 sub-blocks of 32
            for (size_t i = 0; i < nb; i++) {
                const uint8_t* b = src + i * 144; const float d = f16_at(b), mn = f16_at(b + 2); const uint8_t* sc = b + 4; const uint8_t* q = b + 16; float* y = out + i * 256;
                for (int k = 0; k < 4; k++) {
                    uint8_t s1, m1, s2, m2; k4_scale_min(2 * k, sc, &s1, &m1); k4_scale_min(2 * k + 1, sc, &s2, &m2);
                    const float d1 = d * (float)s1, mm1 = mn * (float)m1, d2 = d * (float)s2, mm2 = mn * (float)m2;
                    const uint8_t* qq = q + k * 32;
                    for (int l = 0; l < 32; l++) y[k * 64 + l] = d1 * (float)(qq[l] & 0xF) - mm1;
                    for (int l = 0; l < 32; l++) y[k * 64 + 32 + l] = d2 * (float)(qq[l] >> 4) - mm2;
                }
            }
            break;
        case GG_Q6_K:   // 128 low nibbles, 64 bytes of high bit pairs, 16 int8 scales, d (f16); value = d * scale * (q - 32)
            for (size_t i = 0; i < nb; i++) {
                const uint8_t* b = src + i * 210; const float d = f16_at(b + 208); float* y = out + i * 256;
                for (int h = 0; h < 2; h++) {
                    const uint8_t* ql = b + h * 64; const uint8_t* qh = b + 128 + h * 32; const int8_t* sc = (const int8_t*)b + 192 + h * 8;
                    for (int l = 0; l < 32; l++) {
                        const int is = l / 16;
                        const int q1 = (int)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32, q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                        const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32, q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                        y[h * 128 + l] = d * (float)sc[is] * (float)q1; y[h * 128 + l + 32] = d * (float)sc[is + 2] * (float)q2;
                        y[h * 128 + l + 64] = d * (float)sc[is + 4] * (float)q3; y[h * 128 + l + 96] = d * (float)sc[is + 6] * (float)q4;
                    }
                }
            }
            break;
    }
    return IT_OK;
}
