// Fused Hadamard rotation + q8k activation quantisation, and the plain f32 transform.
//
// One CTA of 256 threads per (1024-element block, activation row).  Thread `tid` owns elements
// 4*tid .. 4*tid+3.  The ten radix-2 stages run in the reference's order h = 1, 2, ..., 512 on the
// pairs (j, j+h) with new[j] = a + b, new[j+h] = a - b (src/hadamard.rs:12-17; shaders/hadamard.comp:20-25):
// stages 1-2 inside the thread, 4-64 by lane exchange, 128-512 through shared memory.  Every
// output is produced by the same sequence of rounded additions as on the CPU, so the f32 result
// is bit-identical; the scale 1/32 is exact.
//
// Quantisation follows quantize_row_q8_K_ref as restated in src/quant.rs:75-90: per 256 elements
// (two warps) the signed value of the FIRST element of maximum magnitude gives iscale = -127/max;
// q = min(round_half_even(iscale*x), 127); d = 1/iscale; per-128 sums of q (one warp each).
// Algorithmic traffic per row: 4n bytes in, n + 4n/256 + 4n/128 bytes out.
#include "it_internal.h"
#include "it_math.h"
#include "it_support.h"

namespace {

struct Best { float amax; float val; unsigned idx; };
__device__ __forceinline__ Best better(Best a, Best b) {
    // b replaces a when strictly larger, or equal magnitude with a lower index
    bool take = (b.amax > a.amax) || (b.amax == a.amax && b.idx < a.idx);
    return take ? b : a;
}

template <bool QUANT>
__global__ void __launch_bounds__(256)
k_hadamard(const float* arena_in, size_t in_off, size_t in_stride,
           float* f32_out, size_t out_off, size_t out_stride,
           const float* __restrict__ signs, int rotate, int inverse,
           unsigned perm_hd, unsigned perm_nk, unsigned perm_rep,
           int8_t* __restrict__ qs, float* __restrict__ qd, int32_t* __restrict__ qsum, size_t q_stride, it_had_prologue pro) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    __shared__ float4 xch[256];
    __shared__ float wsum[8];
    __shared__ float s_amax[8]; __shared__ float s_val[8]; __shared__ unsigned s_idx[8];
    const unsigned tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned blk = blockIdx.x; const size_t tok = blockIdx.y;
    const unsigned g0 = blk * 1024u + 4u * tid;      // index of this thread's first element inside the row
    const float* x = arena_in + in_off + tok * in_stride;

    float v[4];
    if (pro.mode == 2) {
        // rmsnorm of the whole row first (src/cpu.rs:14-18), in the order of k_rmsnorm_wide: thread i adds x[i]^2,
        // x[i+256]^2, ...; warp butterflies; eight warp sums in ascending order.  Every CTA of the row repeats it.
        float xv[32];
#pragma unroll
        for (int k = 0; k < 32; k++) { const unsigned j = tid + 256u * k; xv[k] = j < pro.n ? x[j] : 0.f; }
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < 32; k++) if (tid + 256u * k < pro.n) s = it_add(s, it_mul(xv[k], xv[k]));
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) s = it_add(s, __shfl_xor_sync(0xffffffffu, s, m));
        if (lane == 0) wsum[warp] = s;
        __syncthreads();
        float tot = wsum[0];
#pragma unroll
        for (int k = 1; k < 8; k++) tot = it_add(tot, wsum[k]);
        const float sc = it_div(1.0f, it_sqrt(it_add(it_div(tot, (float)pro.n), pro.eps)));
        const float4 t = *reinterpret_cast<const float4*>(x + g0), w4 = *reinterpret_cast<const float4*>(pro.w + g0);
        v[0] = it_mul(it_mul(t.x, sc), w4.x); v[1] = it_mul(it_mul(t.y, sc), w4.y); v[2] = it_mul(it_mul(t.z, sc), w4.z); v[3] = it_mul(it_mul(t.w, sc), w4.w);
        if (pro.xn_out) *reinterpret_cast<float4*>(pro.xn_out + tok * pro.xn_stride + g0) = make_float4(v[0], v[1], v[2], v[3]);
    } else if (pro.mode == 1) {
        // silu(a) * b (src/cpu.rs:183) computed on the way in
        const float4 a = *reinterpret_cast<const float4*>(x + g0), b = *reinterpret_cast<const float4*>(pro.b + tok * pro.b_stride + g0);
        v[0] = it_mul(it_silu(a.x), b.x); v[1] = it_mul(it_silu(a.y), b.y); v[2] = it_mul(it_silu(a.z), b.z); v[3] = it_mul(it_silu(a.w), b.w);
    } else if (perm_hd == 0) {
        float4 t = *reinterpret_cast<const float4*>(x + g0);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
#pragma unroll
        for (int e = 0; e < 4; e++) {   // grouped [hd, rep, nk] position g reads tiled [hd, nk, rep] source
            unsigned g = g0 + e, i0 = g % perm_hd, q = g / perm_hd, r = q % perm_rep, k = q / perm_rep;
            v[e] = x[i0 + perm_hd * (k + perm_nk * r)];
        }
    }
    if (signs && !inverse) {
        float4 s = *reinterpret_cast<const float4*>(signs + g0);
        v[0] *= s.x; v[1] *= s.y; v[2] *= s.z; v[3] *= s.w;
    }
    if (rotate) {
        float a, b;
        a = v[0]; b = v[1]; v[0] = a + b; v[1] = a - b;      // h = 1
        a = v[2]; b = v[3]; v[2] = a + b; v[3] = a - b;
        a = v[0]; b = v[2]; v[0] = a + b; v[2] = a - b;      // h = 2
        a = v[1]; b = v[3]; v[1] = a + b; v[3] = a - b;
#pragma unroll
        for (unsigned m = 1; m < 32; m <<= 1) {              // h = 4*m: partner lane differs in bit m
            const bool upper = lane & m;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float o = __shfl_xor_sync(0xffffffffu, v[e], m);
                v[e] = upper ? (o - v[e]) : (v[e] + o);
            }
        }
#pragma unroll
        for (unsigned m = 32; m < 256; m <<= 1) {            // h = 4*m: partner thread differs in bit m
            xch[tid] = make_float4(v[0], v[1], v[2], v[3]);
            __syncthreads();
            float4 o = xch[tid ^ m];
            __syncthreads();
            if (tid & m) { v[0] = o.x - v[0]; v[1] = o.y - v[1]; v[2] = o.z - v[2]; v[3] = o.w - v[3]; }
            else         { v[0] = v[0] + o.x; v[1] = v[1] + o.y; v[2] = v[2] + o.z; v[3] = v[3] + o.w; }
        }
#pragma unroll
        for (int e = 0; e < 4; e++) v[e] *= 0.03125f;
    }
    if (signs && inverse) {
        float4 s = *reinterpret_cast<const float4*>(signs + g0);
        v[0] *= s.x; v[1] *= s.y; v[2] *= s.z; v[3] *= s.w;
    }
    if (!QUANT) {
        *reinterpret_cast<float4*>(f32_out + out_off + tok * out_stride + g0) = make_float4(v[0], v[1], v[2], v[3]);
        return;
    }
    // ---- q8k: first element of maximum magnitude in each 256-element block (threads 64*q .. 64*q+63)
    Best best{0.f, 0.f, 0xffffffffu};
#pragma unroll
    for (int e = 0; e < 4; e++) { float a = fabsf(v[e]); if (a > best.amax) { best.amax = a; best.val = v[e]; best.idx = 4 * tid + e; } }
#pragma unroll
    for (unsigned m = 1; m < 32; m <<= 1) {
        Best o{ __shfl_xor_sync(0xffffffffu, best.amax, m), __shfl_xor_sync(0xffffffffu, best.val, m), __shfl_xor_sync(0xffffffffu, best.idx, m) };
        best = better(best, o);
    }
    if (lane == 0) { s_amax[warp] = best.amax; s_val[warp] = best.val; s_idx[warp] = best.idx; }
    __syncthreads();
    { Best o{ s_amax[warp ^ 1], s_val[warp ^ 1], s_idx[warp ^ 1] }; best = better(best, o); }

    int q[4] = {0, 0, 0, 0}; float d = 0.f;
    if (best.amax != 0.f) {
        const float iscale = __fdiv_rn(-127.0f, best.val);
#pragma unroll
        for (int e = 0; e < 4; e++) q[e] = min(__float2int_rn(__fmul_rn(iscale, v[e])), 127);
        d = __fdiv_rn(1.0f, iscale);
    }
    const size_t row_q = tok * q_stride;
    uint32_t packed = (uint32_t)(uint8_t)q[0] | ((uint32_t)(uint8_t)q[1] << 8) | ((uint32_t)(uint8_t)q[2] << 16) | ((uint32_t)(uint8_t)q[3] << 24);
    *reinterpret_cast<uint32_t*>(qs + row_q + g0) = packed;
    int s = q[0] + q[1] + q[2] + q[3];
#pragma unroll
    for (unsigned m = 16; m > 0; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
    if (lane == 0) qsum[tok * (q_stride / 128) + blk * 8 + warp] = s;
    if ((tid & 63) == 0) qd[tok * (q_stride / 256) + blk * 4 + (tid >> 6)] = d;
}

int check_common(it_ctx* c, size_t n, size_t ntok, size_t in_off, size_t in_stride, int use_signs,
                 size_t hd, size_t nk, size_t rep, const float** signs, const char* who) {
    IT_CHECK_ARG(c, "%s: null context", who);
    IT_CHECK_ARG(n > 0 && n % 1024 == 0, "%s: width %zu is not a multiple of the 1024 Hadamard block", who, n);
    IT_CHECK_ARG(ntok > 0 && ntok <= 65535, "%s: bad row count %zu", who, ntok);
    IT_CHECK_ARG(in_off % 4 == 0 && (ntok == 1 || in_stride % 4 == 0), "%s: activation offsets must be 4-float aligned", who);
    IT_CHECK_ARG(in_off <= c->arena_floats && (ntok - 1) * in_stride + n <= c->arena_floats - in_off, "%s: input rows fall outside the arena", who);
    if (hd) IT_CHECK_ARG(nk > 0 && rep > 0 && hd * nk * rep == n, "%s: permutation (%zu,%zu,%zu) does not cover width %zu", who, hd, nk, rep, n);
    *signs = nullptr;
    if (use_signs) {
        auto it = c->signs.find(n);
        IT_CHECK_ARG(it != c->signs.end(), "%s: no sign vector registered for width %zu", who, n);
        *signs = it->second;
    }
    return IT_OK;
}

}  // namespace

IT_API int it_hadamard_q8(it_ctx* c, size_t n, size_t ntok, size_t x_off, size_t x_stride, int rotate, int use_signs,
                          size_t hd, size_t nk, size_t rep, it_q8* out) {
    const float* signs; int r = check_common(c, n, ntok, x_off, x_stride, use_signs, hd, nk, rep, &signs, "it_hadamard_q8"); if (r) return r;
    IT_CHECK_ARG(out && out->ctx == c, "it_hadamard_q8: q8 buffer is null or belongs to another context");
    IT_CHECK_ARG(n <= out->max_n && ntok <= out->max_tok, "it_hadamard_q8: %zu rows of %zu do not fit the q8 buffer (%zu x %zu)", ntok, n, out->max_tok, out->max_n);
    it_note_op(c);
    dim3 grid((unsigned)(n / 1024), (unsigned)ntok);
    it_pdl(k_hadamard<true>, dim3(grid), dim3(256), 0, c->stream, c->arena, x_off, x_stride, nullptr, 0, 0, signs, rotate, 0,
        (unsigned)hd, (unsigned)nk, (unsigned)rep, out->qs, out->d, out->sum128, out->max_n, it_had_prologue{});
    IT_LAUNCH_CHECK("hadamard_q8");
    out->n = n;
    return IT_OK;
}

IT_API int it_hadamard_f32(it_ctx* c, size_t n, size_t ntok, size_t in_off, size_t in_stride, size_t out_off, size_t out_stride,
                           int use_signs, size_t hd, size_t nk, size_t rep, int inverse) {
    const float* signs; int r = check_common(c, n, ntok, in_off, in_stride, use_signs, hd, nk, rep, &signs, "it_hadamard_f32"); if (r) return r;
    IT_CHECK_ARG(!(inverse && hd), "it_hadamard_f32: the inverse transform takes no permutation");
    IT_CHECK_ARG(!(hd && in_off == out_off), "it_hadamard_f32: a permuted transform cannot run in place");
    IT_CHECK_ARG(out_off % 4 == 0 && (ntok == 1 || out_stride % 4 == 0), "it_hadamard_f32: output offsets must be 4-float aligned");
    IT_CHECK_ARG(out_off <= c->arena_floats && (ntok - 1) * out_stride + n <= c->arena_floats - out_off, "it_hadamard_f32: output rows fall outside the arena");
    it_note_op(c);
    dim3 grid((unsigned)(n / 1024), (unsigned)ntok);
    it_pdl(k_hadamard<false>, dim3(grid), dim3(256), 0, c->stream, c->arena, in_off, in_stride, c->arena, out_off, out_stride, signs, 1, inverse,
        (unsigned)hd, (unsigned)nk, (unsigned)rep, nullptr, nullptr, nullptr, 0, it_had_prologue{});
    IT_LAUNCH_CHECK("hadamard_f32");
    return IT_OK;
}

// Engine-internal: the forward transform + q8k with an elementwise prologue (see it_had_prologue in it_support.h).
int it_sup_hadamard_q8_fused(it_ctx* c, size_t n, size_t ntok, size_t x_off, size_t x_stride, it_q8* out, const it_had_prologue& pro) {
    const float* signs; int r = check_common(c, n, ntok, x_off, x_stride, 1, 0, 0, 0, &signs, "hadamard_q8_fused"); if (r) return r;
    IT_CHECK_ARG(out && out->ctx == c && n <= out->max_n && ntok <= out->max_tok && (pro.mode != 2 || (n <= 8192 && pro.n == n)), "hadamard_q8_fused: bad q8 buffer or width");
    it_note_op(c);
    dim3 grid((unsigned)(n / 1024), (unsigned)ntok);
    it_pdl(k_hadamard<true>, dim3(grid), dim3(256), 0, c->stream, c->arena, x_off, x_stride, nullptr, 0, 0, signs, 1, 0, 0u, 0u, 0u, out->qs, out->d, out->sum128, out->max_n, pro);
    IT_LAUNCH_CHECK("hadamard_q8_fused");
    out->n = n;
    return IT_OK;
}
