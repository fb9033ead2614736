// The Hadamard + q8k block transform as a device function (one 1024-element block by 256 threads), used by k_hadamard.
#pragma once
#include "it_internal.h"
#include "it_math.h"
#include "it_support.h"

namespace {

// Shared memory of one Hadamard block (one CTA of 256 threads).
struct it_had_smem { float4 xch[256]; float wsum[8]; float s_amax[8]; float s_val[8]; unsigned s_idx[8]; };

// The 256 threads of a block synchronise on named barrier 2, so callers may have other warps that do not take part.
__device__ __forceinline__ void it_had_sync() { asm volatile("bar.sync 2, 256;" ::: "memory"); }

struct Best { float amax; float val; unsigned idx; };
__device__ __forceinline__ Best better(Best a, Best b) {
    // b replaces a when strictly larger, or equal magnitude with a lower index
    bool take = (b.amax > a.amax) || (b.amax == a.amax && b.idx < a.idx);
    return take ? b : a;
}

// One 1024-element block of one activation row by 256 threads (tid = 0..255): optional prologue, signs, the ten
// butterfly stages, and either the f32 store or q8k quantisation.  Called by k_hadamard (one CTA per block); the
// barriers are named so that a caller with more warps can use it too.
template <bool QUANT>
__device__ __forceinline__ void it_hadamard_block(it_had_smem& sm, const unsigned tid, const unsigned blk, const size_t tok,
           const float* arena_in, size_t in_off, size_t in_stride,
           float* f32_out, size_t out_off, size_t out_stride,
           const float* __restrict__ signs, int rotate, int inverse,
           unsigned perm_hd, unsigned perm_nk, unsigned perm_rep,
           int8_t* __restrict__ qs, float* __restrict__ qd, int32_t* __restrict__ qsum, size_t q_stride, const it_had_prologue& pro) {
    float4* xch = sm.xch; float* wsum = sm.wsum; float* s_amax = sm.s_amax; float* s_val = sm.s_val; unsigned* s_idx = sm.s_idx;
    const unsigned lane = tid & 31, warp = tid >> 5;
    const unsigned g0 = blk * 1024u + 4u * tid;      // index of this thread's first element inside the row
    const float* x = arena_in + in_off + tok * in_stride;

    // loads that depend on nothing computed here are issued first, so that their latency overlaps the row reduction
    float4 sg = make_float4(1.f, 1.f, 1.f, 1.f);
    if (signs) sg = *reinterpret_cast<const float4*>(signs + g0);
    float4 own = make_float4(0.f, 0.f, 0.f, 0.f), w4 = own;
    if (pro.mode == 2) { own = *reinterpret_cast<const float4*>(x + g0); w4 = *reinterpret_cast<const float4*>(pro.w + g0); }
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
        it_had_sync();
        float tot = wsum[0];
#pragma unroll
        for (int k = 1; k < 8; k++) tot = it_add(tot, wsum[k]);
        const float sc = it_div(1.0f, it_sqrt(it_add(it_div(tot, (float)pro.n), pro.eps)));
        const float4 t = own;
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
    if (signs && !inverse) { v[0] *= sg.x; v[1] *= sg.y; v[2] *= sg.z; v[3] *= sg.w; }
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
            it_had_sync();
            float4 o = xch[tid ^ m];
            it_had_sync();
            if (tid & m) { v[0] = o.x - v[0]; v[1] = o.y - v[1]; v[2] = o.z - v[2]; v[3] = o.w - v[3]; }
            else         { v[0] = v[0] + o.x; v[1] = v[1] + o.y; v[2] = v[2] + o.z; v[3] = v[3] + o.w; }
        }
#pragma unroll
        for (int e = 0; e < 4; e++) v[e] *= 0.03125f;
    }
    if (signs && inverse) { v[0] *= sg.x; v[1] *= sg.y; v[2] *= sg.z; v[3] *= sg.w; }
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
    it_had_sync();
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

}  // namespace
