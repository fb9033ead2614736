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
#include "it_hadamard.cuh"

namespace {

template <bool QUANT>
__global__ void __launch_bounds__(256)
k_hadamard(const float* arena_in, size_t in_off, size_t in_stride,
           float* f32_out, size_t out_off, size_t out_stride,
           const float* __restrict__ signs, int rotate, int inverse,
           unsigned perm_hd, unsigned perm_nk, unsigned perm_rep,
           int8_t* __restrict__ qs, float* __restrict__ qd, int32_t* __restrict__ qsum, size_t q_stride, it_had_prologue pro) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    __shared__ it_had_smem sm;
    it_hadamard_block<QUANT>(sm, threadIdx.x, blockIdx.x, blockIdx.y, arena_in, in_off, in_stride, f32_out, out_off, out_stride, signs, rotate, inverse,
                             perm_hd, perm_nk, perm_rep, qs, qd, qsum, q_stride, pro);
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
