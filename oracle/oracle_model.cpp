// CPU oracle, part 2: the decoder forward pass and the MTP head.  TEST INFRASTRUCTURE ONLY.
//
// Restates src/cpu.rs:14-22, :118-274 (rmsnorm, rope, l2norm, forward_token, gdn, attn) and
// src/mtp.rs:93-137 (mv, cpu_step) of the reference, on synthetic or uploaded weights held in host memory.
//
// Two summation/function modes:
//   mode 0 "reference order": exactly the reference's CPU arithmetic - sequential f32 sums everywhere,
//          f64 accumulation for dense f32 weights, the C library's expf/logf/sinf/cosf.
//   mode 1 "device order":    identical except for three documented choices the CUDA kernels make,
//          reproduced here bit for bit: (a) the width-n_embd rmsnorm adds its squares in a fixed
//          256-lane / 32-lane-tree order, (b) dense f32 rows (ssm_beta/alpha) and the int8-group rows of the
//          MTP head are summed lane-strided with a butterfly tree, (c) exp/log/sin/cos come from
//          irontimber_b200/csrc/it_math.h instead of libm.
// Everything else (ternary matvec, Hadamard, q8k, conv, delta rule, attention, rope recurrence) is
// sequential and identical in both modes.  Mode 0 is the ground truth; mode 1 is what the GPU must match
// bit for bit; tests bound the distance between the two.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <algorithm>
#include "../irontimber_b200/csrc/it_math.h"

#define ORC_API extern "C" __attribute__((visibility("default")))

extern "C" {
void orc_quantize_q8k(const float* x, int64_t n, float* d, int8_t* qs, int32_t* sum128);
void orc_matvec_ternary(int type, const uint8_t* data, int64_t rows, int64_t cols, const float* x, int numerics, float* y, int nthreads, int32_t* sumi_out);
void orc_hadamard_forward(const float* x, float* y, int64_t n, int64_t block, const float* signs, int64_t hd, int64_t nk, int64_t rep);
uint32_t orc_argmax(const float* v, int64_t n);
}

namespace {

struct Config {   // mirrors it_model_config of include/irontimber_cuda.h field for field
    int32_t n_layer, n_embd, n_ff, n_vocab, n_head, n_head_kv, head_dim, n_rot;
    float rope_base; int32_t rope_sections[4]; float eps;
    int32_t conv_k, ssm_state, ssm_groups, ssm_vheads, ssm_inner, full_attn_interval, gdn_v_grouped, ctx_len;
    bool recurrent(int il) const { return (il + 1) % full_attn_interval != 0; }     // src/model.rs:40
    int qk_dim() const { return ssm_state * ssm_groups; }                             // src/model.rs:41
    int conv_dim() const { return 2 * qk_dim() + ssm_inner; }                         // src/model.rs:42
    int head_v_dim() const { return ssm_inner / ssm_vheads; }                         // src/model.rs:43
};

enum Tensor {   // same numbering as IT_T_* in include/irontimber_cuda.h
    T_ATTN_NORM = 0, T_POST_NORM, T_FFN_GATE, T_FFN_UP, T_FFN_DOWN,
    T_QKV, T_GATE, T_CONV, T_DT, T_A, T_BETA, T_ALPHA, T_SSM_NORM, T_SSM_OUT,
    T_Q, T_K, T_V, T_O, T_Q_NORM, T_K_NORM,
    T_TOK_EMBD, T_OUTPUT_NORM, T_OUTPUT,
    T_MTP_EH, T_MTP_Q, T_MTP_K, T_MTP_V, T_MTP_O, T_MTP_GATE, T_MTP_UP, T_MTP_DOWN,
    T_MTP_ENORM, T_MTP_HNORM, T_MTP_ATTN_NORM, T_MTP_POST_NORM, T_MTP_Q_NORM, T_MTP_K_NORM, T_MTP_HEAD_NORM,
    T_MTP_EMBD,   // the head's own embedding table; empty = the trunk's (MtpHead::embed, src/mtp.rs:101)
    T_COUNT
};

struct Blob { std::vector<uint8_t> bytes; const float* f() const { return reinterpret_cast<const float*>(bytes.data()); } };

struct Model {
    Config c;
    std::vector<std::vector<Blob>> layer;    // [n_layer][T_COUNT]
    std::vector<Blob> global;                // [T_COUNT] (embedding, output, MTP head)
    std::vector<std::vector<float>> signs;   // by width (index = width / 1024)
    int nthreads;
};

struct State {   // src/cpu.rs:124-135
    int pos;
    std::vector<float> h;
    std::vector<std::vector<float>> conv, ssm, k, v;
};
struct MtpState { std::vector<float> k, v; };   // src/mtp.rs:96

// ---- scalar helpers ------------------------------------------------------------------------
inline float f16r(float x) { return (float)(_Float16)x; }   // half::f16::from_f32(x).to_f32(): IEEE round to nearest even (src/cpu.rs:22)
inline float fexp(float x, int mode) { return mode ? it_expf(x) : std::exp(x); }
inline float silu(float x, int mode) { return mode ? it_silu(x) : x / (1.0f + std::exp(-x)); }                       // src/cpu.rs:19
inline float sigmoid(float x, int mode) { return mode ? it_sigmoid(x) : 1.0f / (1.0f + std::exp(-x)); }              // src/cpu.rs:20
inline float softplus(float x, int mode) { return mode ? it_softplus(x) : (x > 20.0f ? x : std::log(1.0f + std::exp(x))); }   // src/cpu.rs:21

// Sum of squares of a width-n vector.  Reference: sequential.  Device order: lane i of 256 adds the squares of
// x[i], x[i+256], ... in ascending order; each run of 32 lanes is folded with a butterfly (offsets 16, 8, 4, 2, 1);
// the eight results are added in ascending order.
float sum_squares(const float* x, int n, int mode, bool wide) {
    if (!mode || !wide) { float s = 0.f; for (int i = 0; i < n; i++) s += x[i] * x[i]; return s; }
    float p[256];
    for (int i = 0; i < 256; i++) { float s = 0.f; for (int j = i; j < n; j += 256) s = it_add(s, it_mul(x[j], x[j])); p[i] = s; }
    for (int m = 16; m >= 1; m >>= 1) { float q[256]; for (int i = 0; i < 256; i++) q[i] = it_add(p[i], p[i ^ m]); std::memcpy(p, q, sizeof p); }
    float t = p[0]; for (int w = 1; w < 8; w++) t = it_add(t, p[32 * w]); return t;
}
// src/cpu.rs:14-18.  `wide` marks the width-n_embd norms, the only ones the device sums in tree order.
void rmsnorm(const float* x, const float* w, int n, float eps, float* out, int mode, bool wide) {
    float ss = sum_squares(x, n, mode, wide) / (float)n;
    float s = 1.0f / std::sqrt(ss + eps);
    for (int i = 0; i < n; i++) out[i] = x[i] * s * w[i];
}
// src/cpu.rs:164
void l2norm(float* x, int n, float eps) { float s = 0.f; for (int i = 0; i < n; i++) s += x[i] * x[i]; float sc = 1.0f / std::max(std::sqrt(s), eps); for (int i = 0; i < n; i++) x[i] *= sc; }

// src/cpu.rs:145-162: neox-style (I)MRoPE for text positions.
void rope(float* x, int nheads, int head_dim, int n_rot, int pos, float base, const int32_t* sections, int mode) {
    int half = n_rot / 2; float theta_scale = std::pow(base, -2.0f / (float)n_rot);
    int sect = sections[0] + sections[1] + sections[2] + sections[3];
    for (int hh = 0; hh < nheads; hh++) {
        float* h = x + (size_t)hh * head_dim; float theta = (float)pos;
        for (int i = 0; i < half; i++) {
            int sector = sect > 0 ? i % sect : 0;
            bool use_e = sect > 0 && !((sector % 3 == 1 && sector < 3 * sections[1]) || (sector % 3 == 2 && sector < 3 * sections[2]) || (sector % 3 == 0 && sector < 3 * sections[0]));
            float th = use_e ? 0.0f : theta, s, c;
            if (mode) it_sincosf(th, &s, &c); else { s = std::sin(th); c = std::cos(th); }
            float x0 = h[i], x1 = h[i + half];
            h[i] = x0 * c - x1 * s; h[i + half] = x0 * s + x1 * c;
            theta *= theta_scale;
        }
    }
}

// Hadamard-rotate (Model::prep, src/cpu.rs:115-117; every ternary matrix of the synthetic model is folded) and
// multiply by a ternary matrix (src/cpu.rs:25-35).
void tmatvec(const Model& m, const Blob& w, int rows, int cols, const float* x, float* y, int hd = 0, int nk = 0, int rep = 0) {
    std::vector<float> hx(cols);
    const std::vector<float>& sg = m.signs[cols / 1024];
    orc_hadamard_forward(x, hx.data(), cols, 1024, sg.empty() ? nullptr : sg.data(), hd, nk, rep);
    orc_matvec_ternary(0, w.bytes.data(), rows, cols, hx.data(), 0, y, m.nthreads, nullptr);
}
// Dense f32 rows (ssm_beta / ssm_alpha): src/cpu.rs:36-43 with Numerics::Ggml on an F32 weight - f32 products, f64 sum.
void dense_matvec(const float* w, int rows, int cols, const float* x, float* y, int mode) {
    for (int r = 0; r < rows; r++) {
        const float* row = w + (size_t)r * cols;
        if (!mode) { double s = 0; for (int i = 0; i < cols; i++) s += (double)(row[i] * x[i]); y[r] = (float)s; continue; }
        double p[256];   // device order: thread i of 256 adds the products i, i+256, ...; warp butterflies; eight warp sums in order
        for (int l = 0; l < 256; l++) { double s = 0; for (int i = l; i < cols; i += 256) s += (double)it_mul(row[i], x[i]); p[l] = s; }
        for (int mm = 16; mm >= 1; mm >>= 1) { double q[256]; for (int l = 0; l < 256; l++) q[l] = p[l] + p[l ^ mm]; std::memcpy(p, q, sizeof p); }
        double t = p[0]; for (int w = 1; w < 8; w++) t += p[32 * w];
        y[r] = (float)t;
    }
}
// Int8-group rows of the MTP head on raw Q8_0 blocks.  Reference order: Q8G16::dot (src/quant.rs:266-270).  Device order:
// lane l takes the 16-groups g = l, l+32, ...; inside a group a fused multiply-add chain over the 16 products, then
// acc = fma(t, scale, acc); the 32 lane sums are folded with a butterfly (offsets 16 .. 1).
void mvq(const Blob& w, int rows, int cols, const float* x, float* y, int mode) {
    const uint8_t* raw = w.bytes.data(); int bpr = cols / 32;
    // a blob of rows*cols int8 values followed by rows*cols/16 f32 scales is the 16-weight-group form (Q6_K source,
    // Q8G16::from_ggml, src/quant.rs:245-257); anything else is raw Q8_0 blocks
    const bool g16 = w.bytes.size() == (size_t)rows * cols / 16 * 20;
    const float* s16 = reinterpret_cast<const float*>(raw + (size_t)rows * cols);
    for (int r = 0; r < rows; r++) {
        const uint8_t* rowb = raw + (size_t)r * bpr * 34;
        auto scale8 = [&](int g) { const uint8_t* b = rowb + (g / 2) * 34; uint16_t hb = (uint16_t)(b[0] | (b[1] << 8)); uint32_t sign = (hb & 0x8000u) << 16, e = (hb >> 10) & 31, mm = hb & 0x3ff, bits;
            if (e == 0) { if (!mm) bits = sign; else { int k = -1; do { mm <<= 1; k++; } while (!(mm & 0x400)); bits = sign | ((uint32_t)(127 - 15 - k) << 23) | ((mm & 0x3ff) << 13); } }
            else if (e == 31) bits = sign | 0x7f800000u | (mm << 13); else bits = sign | ((e + 112) << 23) | (mm << 13);
            float f; std::memcpy(&f, &bits, 4); return f; };
        auto scale = [&](int g) { return g16 ? s16[(size_t)r * (cols / 16) + g] : scale8(g); };
        auto q = [&](int j) { return g16 ? (float)(int8_t)raw[(size_t)r * cols + j] : (float)(int8_t)rowb[(j / 32) * 34 + 2 + (j % 32)]; };
        if (!mode) { float s = 0.f; for (int g = 0; g < cols / 16; g++) { float t = 0.f; for (int j = 0; j < 16; j++) t += q(g * 16 + j) * x[g * 16 + j]; s += t * scale(g); } y[r] = s; continue; }
        float p[32];
        for (int l = 0; l < 32; l++) { float acc = 0.f; for (int g = l; g < cols / 16; g += 32) { float t = 0.f; for (int j = 0; j < 16; j++) t = it_fma(q(g * 16 + j), x[g * 16 + j], t); acc = it_fma(t, scale(g), acc); } p[l] = acc; }
        for (int mm = 16; mm >= 1; mm >>= 1) { float qq[32]; for (int l = 0; l < 32; l++) qq[l] = it_add(p[l], p[l ^ mm]); std::memcpy(p, qq, sizeof p); }
        y[r] = p[0];
    }
}

}  // namespace
#include "oracle_model_forward.inc"
