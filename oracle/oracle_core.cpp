// CPU oracle for the IronTimber ternary hot path.  TEST INFRASTRUCTURE ONLY.
//
// This file restates, in plain C++, the arithmetic of the reference's CPU path so that
// the CUDA kernels can be checked against it.  Nothing in the product may link or call
// it; only tests, the smoke check and the benchmark's CPU-baseline leg do.
//
// Parity status: the weight decode, the Packed2 / Q8G16 repacks, the k-quant decodes, the
// Walsh-Hadamard transform, the argmax tie rule and the speculative loop are pinned by the
// reference's own golden vectors and known-answer tests (see tests/test_oracle_golden.py).
// The q8k integer dot product and Q8G16::dot have no fixture in the reference; for those
// this restatement is cross-checked against an independent numpy implementation.
//
// Build: g++ -O3 -march=x86-64-v3 -ffp-contract=off -fopenmp (no fused multiply-add: the
// reference is Rust, which never contracts a*b+c).
//
// Each function cites the reference file:line it follows (paths inside the reference
// project).
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <algorithm>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int QK = 128;        // src/quant.rs:5
constexpr int PQ2_BYTES = 34;  // src/quant.rs:6
constexpr int PTQ1_BYTES = 28; // src/quant.rs:7
constexpr int QK_K = 256;      // src/quant.rs:8

// IEEE binary16 -> binary32 (what half::f16::to_f32 does; src/quant.rs:10).
inline float f16_to_f32(uint8_t lo, uint8_t hi) {
    uint32_t h = (uint32_t)lo | ((uint32_t)hi << 8);
    uint32_t sign = (h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ff;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {  // subnormal: normalise
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ff) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
    else bits = sign | ((exp + 112) << 23) | (man << 13);
    float f; std::memcpy(&f, &bits, 4); return f;
}

// src/quant.rs:21
inline uint8_t pq2_code(const uint8_t* qs, int j) { return (qs[j / 4] >> ((j % 4) * 2)) & 3; }

// src/quant.rs:24-29
inline float pq2_block_codes(const uint8_t* b, uint8_t* codes) {
    float d = f16_to_f32(b[0], b[1]);
    const uint8_t* qs = b + 2;
    for (int j = 0; j < QK; j++) codes[j] = pq2_code(qs, j);
    return d;
}

// src/quant.rs:31-49: radix-3 PTQ1_0 block (qs[24], qh[2], d f16), ggml element order.
inline uint8_t trit(uint8_t byte, int n) {
    static const uint8_t POW3[6] = {1, 3, 9, 27, 81, 243};
    uint8_t q = (uint8_t)(byte * POW3[n]);
    return (uint8_t)(((uint16_t)q * 3) >> 8);
}
inline float ptq1_block_codes(const uint8_t* b, uint8_t* codes) {
    const uint8_t* qs = b; const uint8_t* qh = b + 24; float d = f16_to_f32(b[26], b[27]);
    static const int STAGES[3] = {32, 16, 8};
    int o = 0, j = 0;
    for (int c : STAGES) {
        while (j + c <= 24) {
            for (int n = 0; n < 5; n++) for (int m = 0; m < c; m++) codes[o++] = trit(qs[j + m], n);
            j += c;
        }
    }
    for (int n = 0; n < 4; n++) for (int h = 0; h < 2; h++) codes[o++] = trit(qh[h], n);
    return d;
}

// src/quant.rs:64: ggml nearest_int = round half to even.
inline int nearest_int(float x) { return (int)std::nearbyintf(x); }

}  // namespace

// ---------------------------------------------------------------- weight decode
// src/quant.rs:51-57
ORC_API void orc_dequant_pq2_0(const uint8_t* src, int64_t nblocks, float* out) {
    uint8_t c[QK];
    for (int64_t i = 0; i < nblocks; i++) {
        float d = pq2_block_codes(src + i * PQ2_BYTES, c);
        for (int j = 0; j < QK; j++) out[i * QK + j] = (float)((int)c[j] - 1) * d;
    }
}
// src/quant.rs:58-64
ORC_API void orc_dequant_ptq1_0(const uint8_t* src, int64_t nblocks, float* out) {
    uint8_t c[QK];
    for (int64_t i = 0; i < nblocks; i++) {
        float d = ptq1_block_codes(src + i * PTQ1_BYTES, c);
        for (int j = 0; j < QK; j++) out[i * QK + j] = (float)((int)c[j] - 1) * d;
    }
}
// src/quant.rs:188-191
ORC_API void orc_dequant_q8_0(const uint8_t* src, int64_t nblocks, float* out) {
    for (int64_t i = 0; i < nblocks; i++) {
        const uint8_t* b = src + i * 34; float d = f16_to_f32(b[0], b[1]);
        for (int j = 0; j < 32; j++) out[i * 32 + j] = (float)(int8_t)b[2 + j] * d;
    }
}
// src/quant.rs:192-211
ORC_API void orc_dequant_q6_k(const uint8_t* src, int64_t nblocks, float* out) {
    for (int64_t i = 0; i < nblocks; i++) {
        const uint8_t* b = src + i * 210; float d = f16_to_f32(b[208], b[209]); float* y = out + i * 256;
        for (int n = 0; n < 2; n++) {
            const uint8_t* ql = b + n * 64; const uint8_t* qh = b + 128 + n * 32; const uint8_t* sc = b + 192 + n * 8;
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int q1 = (int)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32;
                int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                y[n * 128 + l]      = d * (float)(int8_t)sc[is]     * (float)q1;
                y[n * 128 + l + 32] = d * (float)(int8_t)sc[is + 2] * (float)q2;
                y[n * 128 + l + 64] = d * (float)(int8_t)sc[is + 4] * (float)q3;
                y[n * 128 + l + 96] = d * (float)(int8_t)sc[is + 6] * (float)q4;
            }
        }
    }
}
// src/quant.rs:212-228
static inline void scale_min_k4(int j, const uint8_t* q, uint8_t* s, uint8_t* m) {
    if (j < 4) { *s = q[j] & 63; *m = q[j + 4] & 63; }
    else { *s = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}
ORC_API void orc_dequant_q4_k(const uint8_t* src, int64_t nblocks, float* out) {
    for (int64_t i = 0; i < nblocks; i++) {
        const uint8_t* b = src + i * 144; float d = f16_to_f32(b[0], b[1]); float mn = f16_to_f32(b[2], b[3]);
        const uint8_t* sc = b + 4; const uint8_t* q = b + 16; float* y = out + i * 256;
        for (int jj = 0; jj < 4; jj++) {
            int is = 2 * jj; uint8_t s1, m1, s2, m2;
            scale_min_k4(is, sc, &s1, &m1); scale_min_k4(is + 1, sc, &s2, &m2);
            float d1 = d * (float)s1, mm1 = mn * (float)m1, d2 = d * (float)s2, mm2 = mn * (float)m2;
            const uint8_t* qq = q + jj * 32;
            for (int l = 0; l < 32; l++) y[jj * 64 + l] = d1 * (float)(qq[l] & 0xF) - mm1;
            for (int l = 0; l < 32; l++) y[jj * 64 + 32 + l] = d2 * (float)(qq[l] >> 4) - mm2;
        }
    }
}

// ---------------------------------------------------------------- Packed2 (src/quant.rs:92-162)
// type: 0 = PQ2_0, 1 = PTQ1_0.  words[rows*cols/16], scales[rows*cols/128].
ORC_API void orc_packed2_from_ggml(int type, const uint8_t* data, int64_t rows, int64_t cols, uint32_t* words, float* scales) {
    int64_t nblk = rows * cols / QK; int bs = type == 0 ? PQ2_BYTES : PTQ1_BYTES;
    uint8_t c[QK];
    for (int64_t i = 0; i < nblk; i++) {
        scales[i] = type == 0 ? pq2_block_codes(data + i * bs, c) : ptq1_block_codes(data + i * bs, c);
        for (int w = 0; w < 8; w++) {
            uint32_t v = 0;
            for (int k = 0; k < 16; k++) v |= (uint32_t)c[w * 16 + k] << (2 * k);
            words[i * 8 + w] = v;
        }
    }
}
// src/quant.rs:121-127
ORC_API void orc_packed2_row_f32(const uint32_t* words, const float* scales, int64_t cols, int64_t r, float* out) {
    int64_t wpr = cols / 16, bpr = cols / QK;
    for (int64_t j = 0; j < cols; j++) {
        uint32_t c = (words[r * wpr + j / 16] >> (2 * (j % 16))) & 3;
        out[j] = (float)((int)c - 1) * scales[r * bpr + j / QK];
    }
}

// ---------------------------------------------------------------- Q8_K activations (src/quant.rs:66-90)
// d[n/256], qs[n], sum128[n/128]
ORC_API void orc_quantize_q8k(const float* x, int64_t n, float* d, int8_t* qs, int32_t* sum128) {
    int64_t nb = n / QK_K;
    for (int64_t i = 0; i < nb; i++) {
        const float* xb = x + i * QK_K;
        float amax = 0.f, mx = 0.f;
        for (int j = 0; j < QK_K; j++) { float v = xb[j]; if (std::fabs(v) > amax) { amax = std::fabs(v); mx = v; } }
        d[i] = 0.f;
        if (amax == 0.f) { for (int j = 0; j < QK_K; j++) qs[i * QK_K + j] = 0; continue; }
        float iscale = -127.0f / mx;
        for (int j = 0; j < QK_K; j++) qs[i * QK_K + j] = (int8_t)std::min(nearest_int(iscale * xb[j]), 127);
        d[i] = 1.0f / iscale;
    }
    for (int64_t b = 0; b < n / QK; b++) { int32_t s = 0; for (int j = 0; j < QK; j++) s += qs[b * QK + j]; sum128[b] = s; }
}

// src/quant.rs:130-148 (Packed2::dot_q8k)
ORC_API float orc_packed2_dot_q8k(const uint32_t* words, const float* scales, int64_t cols, int64_t r,
                                  const float* yd, const int8_t* yqs, const int32_t* ysum128) {
    int64_t wpr = cols / 16, bpr = cols / QK; const uint32_t* w = words + r * wpr;
    float sumf = 0.f;
    for (int64_t b = 0; b < bpr; b++) {
        const int8_t* q8 = yqs + b * QK; int32_t s = 0;
        for (int k = 0; k < 8; k++) { uint32_t word = w[b * 8 + k]; const int8_t* q = q8 + k * 16;
            for (int e = 0; e < 16; e++) s += (int32_t)((word >> (2 * e)) & 3) * (int32_t)q[e]; }
        int32_t sumi = s - ysum128[b];
        sumf += (scales[r * bpr + b] * yd[b / 2]) * (float)sumi;
    }
    return sumf;
}
// src/quant.rs:150-161 (Packed2::dot_f32)
ORC_API float orc_packed2_dot_f32(const uint32_t* words, const float* scales, int64_t cols, int64_t r, const float* x) {
    int64_t wpr = cols / 16, bpr = cols / QK; const uint32_t* w = words + r * wpr;
    float sum = 0.f;
    for (int64_t b = 0; b < bpr; b++) {
        float s = 0.f;
        for (int k = 0; k < 8; k++) { uint32_t word = w[b * 8 + k]; const float* xb = x + b * QK + k * 16;
            for (int e = 0; e < 16; e++) s += ((float)((word >> (2 * e)) & 3) - 1.0f) * xb[e]; }
        sum += s * scales[r * bpr + b];
    }
    return sum;
}

// ---------------------------------------------------------------- cpu::matvec, ternary arm (src/cpu.rs:25-35, :48-73)
// type: 0 = PQ2_0, 1 = PTQ1_0.  numerics: 0 = Ggml (q8k integer dot), 1 = F32.
// Rows run in parallel in chunks of >= 64 rows like the reference's rayon with_min_len(64);
// every row is an independent sequential computation, so the thread count never changes a result.
// If sumi_out != NULL (Ggml only) it receives the integer accumulators (s - sum128) per (row, block).
ORC_API void orc_matvec_ternary(int type, const uint8_t* data, int64_t rows, int64_t cols, const float* x,
                                int numerics, float* y, int nthreads, int32_t* sumi_out) {
    int bs = type == 0 ? PQ2_BYTES : PTQ1_BYTES; int64_t bpr = cols / QK; int64_t rb = bpr * bs;
    std::vector<float> qd; std::vector<int8_t> qq; std::vector<int32_t> qs;
    if (numerics == 0) { qd.resize(cols / QK_K); qq.resize(cols); qs.resize(bpr); orc_quantize_q8k(x, cols, qd.data(), qq.data(), qs.data()); }
    (void)nthreads;
#ifdef _OPENMP
    #pragma omp parallel for schedule(dynamic, 64) num_threads(nthreads > 0 ? nthreads : omp_get_max_threads())
#endif
    for (int64_t r = 0; r < rows; r++) {
        const uint8_t* row = data + r * rb; uint8_t c[QK]; float sum = 0.f;
        for (int64_t b = 0; b < bpr; b++) {
            float d = type == 0 ? pq2_block_codes(row + b * bs, c) : ptq1_block_codes(row + b * bs, c);
            if (numerics == 0) {
                const int8_t* q8 = qq.data() + b * QK; int32_t s = 0;
                for (int j = 0; j < QK; j++) s += (int32_t)c[j] * (int32_t)q8[j];
                int32_t sumi = s - qs[b];
                if (sumi_out) sumi_out[r * bpr + b] = sumi;
                sum += (d * qd[b / 2]) * (float)sumi;
            } else {
                const float* xb = x + b * QK; float s = 0.f;
                for (int j = 0; j < QK; j++) s += ((float)c[j] - 1.0f) * xb[j];
                sum += s * d;
            }
        }
        y[r] = sum;
    }
}

// ---------------------------------------------------------------- Q8G16 (src/quant.rs:230-271)
// type: 0 = Q8_0, 1 = Q6_K.  words[rows*cols/4], scales[rows*cols/16].
ORC_API void orc_q8g16_from_ggml(int type, const uint8_t* data, int64_t rows, int64_t cols, uint32_t* words, float* scales) {
    int64_t n = rows * cols; std::vector<int8_t> q(n);
    if (type == 0) {
        for (int64_t i = 0; i < n / 32; i++) { const uint8_t* b = data + i * 34; float d = f16_to_f32(b[0], b[1]);
            scales[2 * i] = d; scales[2 * i + 1] = d; for (int j = 0; j < 32; j++) q[i * 32 + j] = (int8_t)b[2 + j]; }
    } else {
        for (int64_t i = 0; i < n / 256; i++) { const uint8_t* b = data + i * 210; float d = f16_to_f32(b[208], b[209]);
            for (int g = 0; g < 16; g++) scales[i * 16 + g] = d * (float)(int8_t)b[192 + g];
            for (int nn = 0; nn < 2; nn++) { const uint8_t* ql = b + nn * 64; const uint8_t* qh = b + 128 + nn * 32; int64_t o = i * 256 + nn * 128;
                for (int l = 0; l < 32; l++) {
                    q[o + l]      = (int8_t)((int)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32);
                    q[o + l + 32] = (int8_t)((int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32);
                    q[o + l + 64] = (int8_t)((int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32);
                    q[o + l + 96] = (int8_t)((int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32);
                } } }
    }
    for (int64_t i = 0; i < n / 4; i++)
        words[i] = (uint32_t)(uint8_t)q[4 * i] | ((uint32_t)(uint8_t)q[4 * i + 1] << 8) | ((uint32_t)(uint8_t)q[4 * i + 2] << 16) | ((uint32_t)(uint8_t)q[4 * i + 3] << 24);
}
static inline int8_t q8g16_q(const uint32_t* words, int64_t i) { return (int8_t)(uint8_t)(words[i / 4] >> (8 * (i % 4))); }
ORC_API void orc_q8g16_row_f32(const uint32_t* words, const float* scales, int64_t cols, int64_t r, float* out) {
    for (int64_t j = 0; j < cols; j++) { int64_t i = r * cols + j; out[j] = scales[i / 16] * (float)q8g16_q(words, i); }
}
// src/quant.rs:266-270 (Q8G16::dot) applied to every row: src/mtp.rs:93 (mv)
ORC_API void orc_mvq(const uint32_t* words, const float* scales, int64_t rows, int64_t cols, const float* x, float* y, int nthreads) {
    (void)nthreads;
#ifdef _OPENMP
    #pragma omp parallel for schedule(static) num_threads(nthreads > 0 ? nthreads : omp_get_max_threads())
#endif
    for (int64_t r = 0; r < rows; r++) {
        float s = 0.f;
        for (int64_t g = 0; g < cols / 16; g++) { int64_t b = r * cols + g * 16; float t = 0.f;
            for (int j = 0; j < 16; j++) t += (float)q8g16_q(words, b + j) * x[g * 16 + j];
            s += t * scales[b / 16]; }
        y[r] = s;
    }
}

// ---------------------------------------------------------------- Hadamard (src/hadamard.rs:7-46)
ORC_API void orc_fwht_blocks(float* x, int64_t n, int64_t block) {
    float scale = 1.0f / std::sqrt((float)block);
    for (int64_t c0 = 0; c0 < n; c0 += block) {
        float* c = x + c0;
        for (int64_t h = 1; h < block; h *= 2)
            for (int64_t i = 0; i < block; i += h * 2)
                for (int64_t j = i; j < i + h; j++) { float a = c[j], b = c[j + h]; c[j] = a + b; c[j + h] = a - b; }
        for (int64_t j = 0; j < block; j++) c[j] *= scale;
    }
}
// src/hadamard.rs:23-29: tiled [hd, nk, rep] -> grouped [hd, rep, nk]
ORC_API void orc_gdn_group_perm(const float* x, float* o, int64_t hd, int64_t nk, int64_t rep) {
    for (int64_t k = 0; k < nk; k++) for (int64_t r = 0; r < rep; r++) for (int64_t i = 0; i < hd; i++)
        o[i + hd * (r + rep * k)] = x[i + hd * (k + nk * r)];
}
// src/hadamard.rs:35-40 with the optional permutation of src/cpu.rs:239 applied first.  signs may be NULL.
ORC_API void orc_hadamard_forward(const float* x, float* y, int64_t n, int64_t block, const float* signs, int64_t hd, int64_t nk, int64_t rep) {
    if (hd > 0) orc_gdn_group_perm(x, y, hd, nk, rep); else std::memcpy(y, x, n * sizeof(float));
    if (signs) for (int64_t i = 0; i < n; i++) y[i] *= signs[i];
    orc_fwht_blocks(y, n, block);
}
// src/hadamard.rs:41-46
ORC_API void orc_hadamard_inverse(const float* z, float* y, int64_t n, int64_t block, const float* signs) {
    std::memcpy(y, z, n * sizeof(float));
    orc_fwht_blocks(y, n, block);
    if (signs) for (int64_t i = 0; i < n; i++) y[i] *= signs[i];
}

// ---------------------------------------------------------------- argmax (src/sampling.rs:50)
ORC_API uint32_t orc_argmax(const float* v, int64_t n) { int64_t b = 0; for (int64_t i = 1; i < n; i++) if (v[i] > v[b]) b = i; return (uint32_t)b; }

// ---------------------------------------------------------------- greedy_mtp (src/mtp.rs:166-204)
// The backend is a table of C callbacks so that tests can script it.  Stats layout (int64):
// drafted, accepted, steps, draft_calls, verify_calls, single_forwards, timed_decode_forwards, rejected, terminal_rollbacks
struct OrcMtpBackend {
    void* user;
    uint32_t (*prefill)(void*, const uint32_t*, int64_t);
    uint32_t (*single)(void*, uint32_t);
    uint32_t (*draft)(void*, const uint32_t*, int64_t);
    void (*verify)(void*, uint32_t, uint32_t, uint32_t*, uint32_t*);
    void (*reject)(void*);
    void (*reset_all)(void*);
};
ORC_API int64_t orc_greedy_mtp(const OrcMtpBackend* b, const uint32_t* prompt, int64_t np, int64_t n,
                               int (*is_eog)(void*, uint32_t), int (*on_tok)(void*, uint32_t), void* cb_user,
                               uint32_t* out, int64_t* stats) {
    for (int i = 0; i < 9; i++) stats[i] = 0;
    int64_t no = 0;
    auto emit = [&](uint32_t t) -> bool { out[no++] = t; bool go = on_tok(cb_user, t) != 0; return go && !is_eog(cb_user, t) && no < n; };
    if (n == 0) return 0;
    if (np <= 0) return -1;
    uint32_t x = b->prefill(b->user, prompt, np);
    if (!emit(x)) return no;
    std::vector<uint32_t> pending{ x };
    for (;;) {
        if (n - no == 1) { uint32_t a = b->single(b->user, x); stats[5]++; stats[6]++; emit(a); break; }
        uint32_t d = b->draft(b->user, pending.data(), (int64_t)pending.size()); stats[3]++;
        uint32_t a0, a1; b->verify(b->user, x, d, &a0, &a1);
        stats[0]++; stats[2]++; stats[4]++; stats[6] += 2;
        if (a0 == d) {
            stats[1]++;
            if (!emit(d)) { b->reject(b->user); stats[8]++; break; }
            if (!emit(a1)) break;
            x = a1; pending = { a0, a1 };
        } else {
            b->reject(b->user); stats[7]++;
            if (!emit(a0)) break;
            x = a0; pending = { a0 };
        }
    }
    return no;
}

ORC_API int orc_max_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
