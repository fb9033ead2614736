// Ternary GEMV / small-M GEMM on q8k activations (decode, MTP verification, short prompts).
//
// Arithmetic (bit-exact with cpu::matvec's ternary arm under Numerics::Ggml, src/cpu.rs:48-63):
//     y[t, r] = sum over blocks b ascending of  (d_w[r,b] * d_x[t,b/2]) * float(S[t,r,b] - sum128[t,b])
// with S = sum_j code(r, 128b+j) * q(t, 128b+j) an exact integer, every product and the running sum
// rounded separately to f32.
//
// Mapping.  One CTA per 32-row group; its warps split the 128-column blocks of the row group into
// contiguous ranges and stream the tile layout of it_internal.h front to back with 128-bit loads,
// several tiles in flight per warp; each warp stages its slice of the q8 activation rows into shared
// memory with cp.async while the weight loads are in flight.
// Per tile a warp issues eight mma.sync.m16n8k32 (u8 x s8 -> s32): the A operand is produced from
// the packed 2-bit words by one AND per register (codes scaled by 1, 4, 16, 64 for the four rows a
// word holds; the accumulators are shifted back, which is exact), the B operand is the q8 row of
// token n in column n, so up to eight activation rows share every weight load.  The per-block terms
// (d_w*d_x)*float(S - sum128) go to shared memory; after a CTA barrier one thread per (row, token)
// adds them in ascending block order.  No float partial sums are ever combined out of order, and
// K is split across warps only at the level of exact integers.
//
// Algorithmic bytes per launch: rows*cols/128*34 (codes + f16 scales) + ntok*(cols + 4*cols/256)
// + 4*ntok*rows (x2 when accumulating).  The kernel is HBM-bound.
#include "it_internal.h"

namespace {

constexpr int TERM_PAD = 4;       // floats of padding between token planes in shared memory
constexpr int XROW_PAD = 16;      // bytes of padding between staged activation rows

struct Stage {
    uint4 wa, wb;                 // 32 bytes of packed codes
    uint2 sc;                     // four f16 scales (rows g, g+8, g+16, g+24)
    float dx0, dx1;               // q8k scale of tokens 2t, 2t+1 for this block
    int s0, s1;                   // sum128 of tokens 2t, 2t+1 for this block
};

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream2(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MT: activation rows per launch (columns of the mma B operand in use); WARPS: warps per CTA, which
// split the blocks of the row group; PIPE: tiles each warp keeps in flight; MINB: CTAs per SM the
// register budget is set for.
template <int MT, int WARPS, int PIPE, int MINB, bool SUMI>
__global__ void __launch_bounds__(WARPS * 32, MINB)
k_matvec_t2(const uint8_t* __restrict__ tiles, int nb, int rows,
            const int8_t* __restrict__ xq, const float* __restrict__ xd, const int32_t* __restrict__ xs128, int x_stride, int ntok,
            float* y, size_t y_stride, int accum, int32_t* __restrict__ sumi_out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int plane = nb * 32 + TERM_PAD;
    const int xrow = nb * 128 + XROW_PAD;
    float* terms = reinterpret_cast<float*>(smem_raw);                                   // [MT][plane]
    int8_t* xs = reinterpret_cast<int8_t*>(smem_raw) + (SUMI ? 0 : (size_t)MT * plane * 4);   // [MT][xrow]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int rg = blockIdx.x;
    const int b0 = (warp * nb) / WARPS, b1 = ((warp + 1) * nb) / WARPS, nblk = b1 - b0;
    const uint8_t* tp = tiles + ((size_t)rg * nb) * IT_TILE_BYTES;
    const bool x_lane = g < ntok && g < MT;          // this lane feeds column g of the B operand
    const int c0 = 2 * t, c1 = 2 * t + 1;            // token columns this lane receives from the mma
    const bool v0 = c0 < MT && c0 < ntok, v1 = c1 < MT && c1 < ntok;
    const int dstride = x_stride / 256, sstride = x_stride / 128;

    Stage st[PIPE];
    auto load = [&](Stage& s, int b) {
        const uint8_t* tile = tp + (size_t)b * IT_TILE_BYTES;
        s.wa = ldg_stream(tile + 16 * lane);
        s.wb = ldg_stream(tile + 512 + 16 * lane);
        s.sc = ldg_stream2(tile + 1024 + 8 * g);
        s.dx0 = v0 ? __ldg(xd + c0 * dstride + (b >> 1)) : 0.f; s.s0 = v0 ? __ldg(xs128 + c0 * sstride + b) : 0;
        if (MT > 1) { s.dx1 = v1 ? __ldg(xd + c1 * dstride + (b >> 1)) : 0.f; s.s1 = v1 ? __ldg(xs128 + c1 * sstride + b) : 0; }
    };
    auto compute = [&](const Stage& s, int b) {
        int cx[4] = {0, 0, 0, 0}, cy[4] = {0, 0, 0, 0};
        const uint32_t w[8] = { s.wa.x, s.wa.y, s.wa.z, s.wa.w, s.wb.x, s.wb.y, s.wb.z, s.wb.w };
        uint4 xa = make_uint4(0, 0, 0, 0), xb4 = make_uint4(0, 0, 0, 0);
        if (x_lane) {
            const uint4* xp = reinterpret_cast<const uint4*>(xs + g * xrow + 128 * b + 32 * t);
            xa = xp[0]; xb4 = xp[1];
        }
        const uint32_t xb[8] = { xa.x, xa.y, xa.z, xa.w, xb4.x, xb4.y, xb4.z, xb4.w };
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t lo = w[2 * j], hi = w[2 * j + 1];
            mma_u8s8(cx, lo & 0x03030303u, lo & 0x0c0c0c0cu, hi & 0x03030303u, hi & 0x0c0c0c0cu, xb[2 * j], xb[2 * j + 1]);
            mma_u8s8(cy, lo & 0x30303030u, lo & 0xc0c0c0c0u, hi & 0x30303030u, hi & 0xc0c0c0c0u, xb[2 * j], xb[2 * j + 1]);
        }
        // rows g, g+8, g+16, g+24 of the tile; accumulators carry the factors 1, 4, 16, 64
        const int S0[4] = { cx[0], cx[2] >> 2, cy[0] >> 4, cy[2] >> 6 };   // token c0
        const int S1[4] = { cx[1], cx[3] >> 2, cy[1] >> 4, cy[3] >> 6 };   // token c1
        const __half2 h01 = *reinterpret_cast<const __half2*>(&s.sc.x), h23 = *reinterpret_cast<const __half2*>(&s.sc.y);
        const float dw[4] = { __low2float(h01), __high2float(h01), __low2float(h23), __high2float(h23) };
        if (v0) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int sumi = S0[i] - s.s0;
                if (SUMI) { const int row = rg * 32 + g + 8 * i; if (row < rows) sumi_out[((size_t)c0 * rows + row) * nb + b] = sumi; }
                else terms[c0 * plane + b * 32 + g + 8 * i] = __fmul_rn(__fmul_rn(dw[i], s.dx0), (float)sumi);
            }
        }
        if (MT > 1 && v1) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int sumi = S1[i] - s.s1;
                if (SUMI) { const int row = rg * 32 + g + 8 * i; if (row < rows) sumi_out[((size_t)c1 * rows + row) * nb + b] = sumi; }
                else terms[c1 * plane + b * 32 + g + 8 * i] = __fmul_rn(__fmul_rn(dw[i], s.dx1), (float)sumi);
            }
        }
    };

    // weights first (they come from HBM), then this warp's slice of the activation rows into shared memory
#pragma unroll
    for (int p = 0; p < PIPE; p++) if (p < nblk) load(st[p], b0 + p);
    {
        const int chunks = nblk * 8;                 // 16-byte pieces per activation row in this warp's range
        for (int m = 0; m < MT; m++) {
            if (m < ntok) {
                const int8_t* src = xq + (size_t)m * x_stride + 128 * b0;
                int8_t* dst = xs + m * xrow + 128 * b0;
                for (int ch = lane; ch < chunks; ch += 32) cp_async16(dst + 16 * ch, src + 16 * ch);
            }
        }
        cp_async_wait_all();
        __syncwarp();
    }
    for (int i = 0; i < nblk; i += PIPE) {
#pragma unroll
        for (int p = 0; p < PIPE; p++) {
            if (i + p < nblk) {
                compute(st[p], b0 + i + p);
                if (i + p + PIPE < nblk) load(st[p], b0 + i + p + PIPE);
            }
        }
    }
    if (SUMI) return;
    __syncthreads();
    // ordered f32 accumulation: thread (row r, token c) walks the blocks front to back
    for (int idx = tid; idx < 32 * MT; idx += WARPS * 32) {
        const int c = idx >> 5, r = idx & 31, row = rg * 32 + r;
        if (c < ntok && row < rows) {
            const float* tcol = terms + c * plane + r;
            float sum = 0.f;
#pragma unroll 8
            for (int b = 0; b < nb; b++) sum = __fadd_rn(sum, tcol[b * 32]);
            float* dst = y + (size_t)c * y_stride + row;
            *dst = accum ? __fadd_rn(*dst, sum) : sum;
        }
    }
}

template <int MT>
size_t smem_bytes(int nb, bool sumi) { return (sumi ? 0 : (size_t)MT * (nb * 32 + TERM_PAD) * 4) + (size_t)MT * (nb * 128 + XROW_PAD); }

template <int MT, int WARPS, int PIPE, int MINB, bool SUMI>
int launch_cfg(it_ctx* c, const it_mat* w, int ntok, const it_q8* x, size_t xrow0, float* y, size_t y_stride, int accum, int32_t* sumi) {
    const int nb = (int)(w->cols / 128);
    const size_t smem = smem_bytes<MT>(nb, SUMI);
    auto kern = k_matvec_t2<MT, WARPS, PIPE, MINB, SUMI>;
    if (smem > 48 * 1024) IT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<(unsigned)w->row_groups, WARPS * 32, smem, c->stream>>>(w->tiles, nb, (int)w->rows,
        x->qs + xrow0 * x->max_n, x->d + xrow0 * (x->max_n / 256), x->sum128 + xrow0 * (x->max_n / 128), (int)x->max_n, ntok,
        y, y_stride, accum, sumi);
    IT_LAUNCH_CHECK("matvec_t2");
    return IT_OK;
}

// Shape policy: few blocks per row group -> small CTAs, several per SM, so that a whole matrix of the
// model's wide-output shapes is resident in one wave; many blocks per row group (the long-K shapes have
// few rows) -> 32 warps per CTA to keep enough bytes in flight.
template <int MT, bool SUMI>
int launch(it_ctx* c, const it_mat* w, int ntok, const it_q8* x, size_t xrow0, float* y, size_t y_stride, int accum, int32_t* sumi) {
    const int nb = (int)(w->cols / 128);
    if (MT == 1 && nb <= 48) return launch_cfg<MT, 8, 3, 4, SUMI>(c, w, ntok, x, xrow0, y, y_stride, accum, sumi);
    if (nb <= 48) return launch_cfg<MT, 16, 3, 2, SUMI>(c, w, ntok, x, xrow0, y, y_stride, accum, sumi);
    return launch_cfg<MT, 32, 3, 1, SUMI>(c, w, ntok, x, xrow0, y, y_stride, accum, sumi);
}

template <bool SUMI>
int dispatch(it_ctx* c, const it_mat* w, size_t ntok, const it_q8* x, float* y, size_t y_stride, int accum, int32_t* sumi) {
    // activation rows are processed in groups of up to eight (one mma N tile); wide matrices use smaller
    // groups so that the staged rows and the per-block terms fit in shared memory
    const int nb = (int)(w->cols / 128);
    size_t group = 8;
    while (group > 1 && (group == 8 ? smem_bytes<8>(nb, SUMI) : group == 4 ? smem_bytes<4>(nb, SUMI) : smem_bytes<2>(nb, SUMI)) > 160 * 1024) group /= 2;
    if (smem_bytes<1>(nb, SUMI) > 200 * 1024) return it_fail(IT_EINVAL, "it_matvec_t2: %zu columns exceed the shared-memory budget", w->cols);
    for (size_t t0 = 0; t0 < ntok; t0 += group) {
        const int nt = (int)((ntok - t0) < group ? (ntok - t0) : group);
        float* yy = y ? y + t0 * y_stride : nullptr;
        int32_t* ss = sumi ? sumi + t0 * w->rows * (w->cols / 128) : nullptr;
        int r;
        if (nt == 1) r = launch<1, SUMI>(c, w, nt, x, t0, yy, y_stride, accum, ss);
        else if (nt == 2) r = launch<2, SUMI>(c, w, nt, x, t0, yy, y_stride, accum, ss);
        else if (nt <= 4) r = launch<4, SUMI>(c, w, nt, x, t0, yy, y_stride, accum, ss);
        else r = launch<8, SUMI>(c, w, nt, x, t0, yy, y_stride, accum, ss);
        if (r) return r;
    }
    return IT_OK;
}

int check(it_ctx* c, const it_mat* w, size_t ntok, const it_q8* x, const char* who) {
    IT_CHECK_ARG(c && w && x, "%s: null argument", who);
    IT_CHECK_ARG(w->ctx == c && x->ctx == c, "%s: matrix or q8 buffer belongs to another context", who);
    IT_CHECK_ARG(w->cols % 256 == 0, "%s: cols %zu is not a multiple of the 256-element q8k block", who, w->cols);
    IT_CHECK_ARG(x->n == w->cols, "%s: activation width %zu does not match the matrix (%zu columns)", who, x->n, w->cols);
    IT_CHECK_ARG(ntok > 0 && ntok <= x->max_tok, "%s: bad row count %zu (buffer holds %zu)", who, ntok, x->max_tok);
    return IT_OK;
}

}  // namespace

IT_API int it_matvec_t2(it_ctx* c, const it_mat* w, size_t ntok, const it_q8* x, size_t y_off, size_t y_stride, int accum) {
    int r = check(c, w, ntok, x, "it_matvec_t2"); if (r) return r;
    IT_CHECK_ARG(ntok == 1 || y_stride >= w->rows, "it_matvec_t2: output stride %zu is shorter than a row of %zu results", y_stride, w->rows);
    IT_CHECK_ARG(y_off <= c->arena_floats && (ntok - 1) * y_stride + w->rows <= c->arena_floats - y_off, "it_matvec_t2: output rows fall outside the arena");
    return dispatch<false>(c, w, ntok, x, c->arena + y_off, y_stride, accum, nullptr);
}

IT_API int it_matvec_t2_sumi(it_ctx* c, const it_mat* w, size_t ntok, const it_q8* x, int32_t* sumi_dev) {
    int r = check(c, w, ntok, x, "it_matvec_t2_sumi"); if (r) return r;
    IT_CHECK_ARG(sumi_dev, "it_matvec_t2_sumi: null output");
    return dispatch<true>(c, w, ntok, x, nullptr, 0, 0, sumi_dev);
}
