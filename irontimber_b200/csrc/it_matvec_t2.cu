// Ternary GEMV / small-M GEMM on q8k activations (decode, MTP verification, short prompts).
//
// Arithmetic (bit-exact with cpu::matvec's ternary arm under Numerics::Ggml, src/cpu.rs:48-63):
//     y[t, r] = sum over blocks b ascending of  (d_w[r,b] * d_x[t,b/2]) * float(S[t,r,b] - sum128[t,b])
// with S = sum_j code(r, 128b+j) * q(t, 128b+j) an exact integer, every product and the running sum
// rounded separately to f32.
//
// Mapping.  In the tile layout of it_internal.h a 32-row group is one contiguous run of bytes.  A
// persistent grid of a few CTAs per SM shares out the row groups round robin (CTA i takes i, i+grid,
// ...).  In each CTA a producer thread streams its row groups, chunk by chunk (eight 128-column tiles),
// into a shared-memory ring with bulk asynchronous copies (cp.async.bulk, completion counted on an
// mbarrier), as far ahead as the ring is deep and across row-group boundaries, so the HBM request
// stream does not drain between row groups.  Consumer warps, in groups of eight, take one tile each
// per chunk.  Per tile a warp issues eight mma.sync.m16n8k32 (u8 x s8 -> s32): the A operand comes
// from the packed 2-bit words by one AND per register (codes scaled by 1, 4, 16, 64 for the four rows
// a word holds; the accumulators are shifted back, which is exact), the B operand is the q8 row of
// token n in column n, so up to eight activation rows share every weight load.  The q8 rows, their
// scales and block sums are staged in shared memory once per CTA.
//
// The per-block terms (d_w*d_x)*float(S - sum128) go to a shared array; after a barrier per row group
// one thread per (row, token) adds them in ascending block order while the other warps go on with the
// next row group (second terms buffer).  Float partial sums are never combined out of order; K is
// split across warps only at the level of exact integers, and never across CTAs.
//
// Every wait on an mbarrier is bounded; when one runs out the CTA raises a flag that the host reads
// after the stream is synchronised (IT_ETIMEOUT), drains its copies and leaves.
//
// Algorithmic bytes per launch: rows*cols/128*34 (codes + f16 scales) + ntok*(cols + 4*cols/256)
// + 4*ntok*rows (x2 when accumulating).  The kernel is HBM-bound.
#include "it_internal.h"
#include "it_pipe.cuh"
#include <algorithm>

namespace {

constexpr int CWARPS = 8;                         // warps per consumer group = tiles per chunk
constexpr int TERM_PAD = 4;                       // floats of padding between token planes
constexpr int XROW_PAD = 16;                      // bytes of padding between staged activation rows
constexpr int SM_SMEM = 227 * 1024;               // shared memory one SM can give to CTAs

struct Smem {   // byte offsets into dynamic shared memory
    int ring, x, dx, s128, terms, wsc, bars, flag, total, plane, xrow;
};
__host__ __device__ inline Smem smem_layout(int MT, int nb, int slots, int nbuf, int cw = CWARPS) {
    Smem L; int o = 0;
    L.plane = nb * 32 + TERM_PAD; L.xrow = nb * 128 + XROW_PAD;
    L.ring = o; o += slots * cw * IT_TILE_BYTES;
    L.x = o; o += MT * L.xrow;
    L.dx = o; o += MT * (nb / 2) * 4;
    L.s128 = o; o += MT * nb * 4;
    L.terms = o; o += nbuf * MT * L.plane * 4;
    o = (o + 15) & ~15;
    L.wsc = o; o += nbuf * nb * 64;                 // copies of the tiles' f16 scales (see LATE)
    L.bars = o; o += 2 * slots * 8;
    L.flag = o; o += 16;
    L.total = o;
    return L;
}

// MT: activation rows per launch (columns of the mma B operand in use).  CW: consumer warps per group = tiles per
// chunk.  NG: consumer groups of CW warps; group j takes the chunks k of the CTA's stream with k % NG == j.  MINB: CTAs per SM the
// register budget allows.  nbuf: terms buffers (0 for the integer-accumulator variant, 1 when every CTA
// has a single row group, else 2).
template <int MT, int NG, int MINB, bool SUMI, int CW = CWARPS>
__global__ void __launch_bounds__((NG * CW + 1) * 32, MINB)
k_matvec_t2(const uint8_t* __restrict__ tiles, int nb, int rows, int row_groups, int slots, int nbuf,
            const int8_t* __restrict__ xq, const float* __restrict__ xd, const int32_t* __restrict__ xs128, int x_stride, int ntok,
            float* arena, size_t y_off, size_t y_stride, int accum, int32_t* __restrict__ sumi_out, int* error_flag, int wait_early,
            const it_peers* peers, const it_rowmap map, int ll_mode, int out_rows) {
    constexpr int NCONS = NG * CW, CHUNK = CW * IT_TILE_BYTES;   // consumer warps; bytes of one ring slot (CW tiles)
    extern __shared__ __align__(128) unsigned char smem[];
    const Smem L = smem_layout(MT, nb, slots, nbuf, CW);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.flag);
    const unsigned bars = smem_u32(smem + L.bars);             // full[s] at bars + 8*s, empty[s] at bars + 8*(slots + s)
    const int cpr = (nb + CW - 1) / CW;                 // chunks per row group
    const int my_rgs = row_groups > (int)blockIdx.x ? (row_groups - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < slots; s++) { mbar_init(bars + 8 * s, 1); mbar_init(bars + 8 * (slots + s), CW); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == NCONS) {
        // ---------------- producer: one thread keeps the ring full
        if (lane == 0) {
            int issued = 0, s = 0; unsigned ph = 0;
            for (int i = 0; i < my_rgs && !*abort_flag; i++) {
                const uint8_t* src = tiles + ((size_t)((int)blockIdx.x + i * (int)gridDim.x) * nb) * IT_TILE_BYTES;
                for (int cq = 0; cq < cpr; cq++) {
                    if (!mbar_wait(bars + 8 * (slots + s), ph ^ 1u, abort_flag, error_flag)) break;
                    const int ntile = min(CW, nb - cq * CW);
                    const unsigned bytes = (unsigned)ntile * IT_TILE_BYTES;
                    mbar_expect_tx(bars + 8 * s, bytes);
                    bulk_load(smem_u32(smem + L.ring + s * CHUNK), src + (size_t)cq * CHUNK, bytes, bars + 8 * s);
                    issued++;
                    if (++s == slots) { s = 0; ph ^= 1u; }
                }
            }
            if (*abort_flag) {
                // leave only after every copy this thread started has landed (each wait bounded by the clock limit)
                const int first = issued > slots ? issued - slots : 0;
                for (int k = first; k < issued; k++) {
                    const long long t0 = clock64();
                    while (!mbar_test(bars + 8 * (k % slots), (unsigned)(k / slots) & 1u) && clock64() - t0 < WAIT_CLOCKS) { }
                }
            }
        }
        return;
    }

    // ---------------- consumers
    // Programmatic dependent launch.  The weights never depend on an earlier kernel, so the producer warp above
    // requests them without waiting (and never triggers: its exit counts as done).  When the kernel before this one
    // produced our activation rows (wait_early) the consumers wait for it here, and only then let the next kernel
    // start: a kernel that follows us may read the same rows without waiting, so they must be complete by the time
    // it is allowed to run.  Otherwise the rows are known to be complete already and the only wait is the one in
    // front of the store of y.
    if (wait_early) asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int g = lane >> 2, t = lane & 3;
    int8_t* xs = reinterpret_cast<int8_t*>(smem + L.x);
    float* dxs = reinterpret_cast<float*>(smem + L.dx);
    int* sss = reinterpret_cast<int*>(smem + L.s128);
    float* terms = reinterpret_cast<float*>(smem + L.terms);
    // LATE: a tile only leaves its integer block sums and its 32 scales in shared memory; the warp that adds the terms
    // of an activation row in block order also forms them, one matrix row per lane, instead of every tile's warp doing
    // it with a quarter of its lanes.  Same operations on the same values, 15 % fewer instructions at one row.
    constexpr bool LATE = !SUMI;
    {   // stage the activation rows, their q8k scales and block sums once per CTA
        const int pieces = nb * 8;
        for (int m = 0; m < MT; m++) {
            if (m < ntok) {
                const int8_t* src = xq + (size_t)m * x_stride;
                for (int ch = tid; ch < pieces; ch += NCONS * 32) cp_async16(xs + m * L.xrow + 16 * ch, src + 16 * ch);
                for (int i = tid; i < nb / 2; i += NCONS * 32) dxs[m * (nb / 2) + i] = xd[m * (x_stride / 256) + i];
                for (int i = tid; i < nb; i += NCONS * 32) sss[m * nb + i] = xs128[m * (x_stride / 128) + i];
            }
        }
        cp_async_wait_all();
        consumer_barrier<NCONS * 32>();
    }
    const bool x_lane = g < ntok && g < MT;          // this lane feeds column g of the B operand
    const int c0 = 2 * t, c1 = 2 * t + 1;            // token columns this lane receives from the mma
    const bool v0 = c0 < MT && c0 < ntok, v1 = c1 < MT && c1 < ntok;
    const int group = warp / CW, wi = warp % CW;   // consumer group and tile index inside a chunk

    int s = 0; unsigned ph = 0; int kg = 0;           // ring slot, its phase, and (chunk index) % NG
    for (int i = 0; i < my_rgs; i++) {
        const int rg = (int)blockIdx.x + i * (int)gridDim.x;
        float* tbuf = terms + (size_t)(nbuf > 1 ? (i & 1) : 0) * MT * L.plane;
        uint2* wsc = reinterpret_cast<uint2*>(smem + L.wsc + (nbuf > 1 ? (i & 1) : 0) * nb * 64);
        for (int cq = 0; cq < cpr; cq++) {
            const bool mine = NG == 1 || kg == group;
            const int cs = s; const unsigned cph = ph;
            if (++s == slots) { s = 0; ph ^= 1u; }
            if (NG > 1 && ++kg == NG) kg = 0;
            if (!mine) continue;
            const int b = cq * CW + wi;
            const bool ready = mbar_wait(bars + 8 * cs, cph, abort_flag, error_flag);
            if (ready && b < nb) {
                const unsigned char* tile = smem + L.ring + cs * CHUNK + wi * IT_TILE_BYTES;
                const uint4 wa = *reinterpret_cast<const uint4*>(tile + 16 * lane);
                const uint4 wb = *reinterpret_cast<const uint4*>(tile + 512 + 16 * lane);
                const uint2 sc = *reinterpret_cast<const uint2*>(tile + 1024 + 8 * g);
                // B column g is activation row g; a lane whose column holds no row reads row 0 instead of zeros: the
                // mma results of such a column are never looked at (v0 / v1), and the load needs no predicate
                const uint4* xp = reinterpret_cast<const uint4*>(xs + (x_lane ? g : 0) * L.xrow + 128 * b + 32 * t);
                const uint4 xa = xp[0], xb4 = xp[1];
                int cx[4] = {0, 0, 0, 0}, cy[4] = {0, 0, 0, 0};
                const uint32_t w[8] = { wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w };
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
                const __half2 h01 = *reinterpret_cast<const __half2*>(&sc.x), h23 = *reinterpret_cast<const __half2*>(&sc.y);
                const float dw[4] = { __low2float(h01), __high2float(h01), __low2float(h23), __high2float(h23) };
                if (LATE) {
                    if (v0) {
                        // rows g, g + 8, g + 16, g + 24 side by side: one 16-byte store; row L of the tile sits at 4 * (L & 7) + (L >> 3)
                        *reinterpret_cast<int4*>(reinterpret_cast<int*>(tbuf) + c0 * L.plane + b * 32 + 4 * g) = make_int4(cx[0], cx[2], cy[0], cy[2]);   // still carrying 1, 4, 16, 64
                        if (t == 0) wsc[b * 8 + g] = sc;
                    }
                    if (MT > 1 && v1) {
                        *reinterpret_cast<int4*>(reinterpret_cast<int*>(tbuf) + c1 * L.plane + b * 32 + 4 * g) = make_int4(cx[1], cx[3], cy[1], cy[3]);
                    }
                } else if (v0) {
                    const float dx = dxs[c0 * (nb / 2) + (b >> 1)]; const int s128 = sss[c0 * nb + b];
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        const int sumi = S0[r] - s128;
                        if (SUMI) { const int row = rg * 32 + g + 8 * r; if (row < rows) sumi_out[((size_t)c0 * rows + row) * nb + b] = sumi; }
                        else tbuf[c0 * L.plane + b * 32 + g + 8 * r] = __fmul_rn(__fmul_rn(dw[r], dx), (float)sumi);
                    }
                }
                if (!LATE && MT > 1 && v1) {
                    const float dx = dxs[c1 * (nb / 2) + (b >> 1)]; const int s128 = sss[c1 * nb + b];
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        const int sumi = S1[r] - s128;
                        if (SUMI) { const int row = rg * 32 + g + 8 * r; if (row < rows) sumi_out[((size_t)c1 * rows + row) * nb + b] = sumi; }
                        else tbuf[c1 * L.plane + b * 32 + g + 8 * r] = __fmul_rn(__fmul_rn(dw[r], dx), (float)sumi);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + 8 * (slots + cs));     // the slot may be refilled
        }
        if (SUMI) continue;
        consumer_barrier<NCONS * 32>();                              // every term of this row group is in shared memory
        // ordered f32 accumulation: warp c (token c), lane r (row r) walks the blocks front to back while the
        // remaining warps go on with the next row group (whose terms go to the other buffer)
        if (warp < MT && warp < ntok) {
            const int row = rg * 32 + lane;
            if (row < rows) {
                const float* tcol = tbuf + warp * L.plane + lane;
                // y may be read or written by the kernel before us; a sharded launch waits before the additions so
                // that the load of the epoch counter overlaps them
                unsigned epoch = 0;
                if (peers && ll_mode) {
                    if (!wait_early) asm volatile("griddepcontrol.wait;" ::: "memory");
                    epoch = *reinterpret_cast<volatile unsigned*>(peers->epoch) + 1u;
                }
                float sum = 0.f;
                if (LATE) {
                    const int* icol = reinterpret_cast<const int*>(tbuf + warp * L.plane) + 4 * (lane & 7) + (lane >> 3);
                    const __half* hs = reinterpret_cast<const __half*>(wsc) + 4 * (lane & 7) + (lane >> 3);   // row g + 8 j: half j of group g
                    const float* dxr = dxs + warp * (nb / 2); const int* ssr = sss + warp * nb;
                    const int sh = 2 * (lane >> 3);            // the factor 4^j the tile's warp left on the sums of rows g + 8 j
#pragma unroll 8
                    for (int b = 0; b < nb; b++)
                        sum = __fadd_rn(sum, __fmul_rn(__fmul_rn(__half2float(hs[b * 32]), dxr[b >> 1]), (float)((icol[b * 32] >> sh) - ssr[b])));
                } else {
#pragma unroll 8
                    for (int b = 0; b < nb; b++) sum = __fadd_rn(sum, tcol[b * 32]);
                }
                if (!wait_early && !(peers && ll_mode)) asm volatile("griddepcontrol.wait;" ::: "memory");
                int shift; const int grow = it_map_row(map, row, &shift);
                if (peers && ll_mode) it_result_exchange_ll(peers, arena, y_off + (size_t)warp * y_stride, (size_t)warp * out_rows, grow, shift, sum, accum, epoch, error_flag);
                else it_result_store(peers, arena, y_off + (size_t)warp * y_stride + grow, sum, accum);
            }
        }
    }
    if (!SUMI && peers) {
        // sharded launch: count the CTA as done; without the slot protocol first make its pushes visible system-wide
        if (!ll_mode) __threadfence_system();
        consumer_barrier<NCONS * 32>();
        if (tid == 0) { if (ll_mode) it_shard_finish_ll(peers, gridDim.x); else it_shard_finish(peers, gridDim.x, error_flag); }
    }
}

template <int MT, int NG, int MINB, bool SUMI, int CW = CWARPS>
int launch_cfg(it_ctx* c, const it_mat* w, int ntok, const it_q8* x, size_t xrow0, float* y, size_t y_stride, int accum, int32_t* sumi,
               int slots, int nbuf, int grid) {
    const int nb = (int)(w->cols / 128);
    const Smem L = smem_layout(MT, nb, slots, nbuf, CW);
    auto kern = k_matvec_t2<MT, NG, MINB, SUMI, CW>;
    static bool attr_set[16] = {};
    if (!attr_set[c->device & 15]) { IT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_SMEM - 1024)); attr_set[c->device & 15] = true; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3((NG * CW + 1) * 32); cfg.dynamicSmemBytes = (size_t)L.total; cfg.stream = c->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    // the activation rows are safe to read without waiting only if the previous op was a matvec on the same rows
    const int wait_early = (SUMI || c->pdl_safe_q8 != x) ? 1 : 0;
    const int nb_ = nb, rows_ = (int)w->rows, rgs_ = (int)w->row_groups, xs_ = (int)x->max_n;
    IT_CUDA(cudaLaunchKernelEx(&cfg, kern, (const uint8_t*)w->tiles, nb_, rows_, rgs_, slots, nbuf,
        (const int8_t*)(x->qs + xrow0 * x->max_n), (const float*)(x->d + xrow0 * (x->max_n / 256)), (const int32_t*)(x->sum128 + xrow0 * (x->max_n / 128)), xs_, ntok,
        c->arena, y ? (size_t)(y - c->arena) : (size_t)0, y_stride, accum, sumi, c->error_flag_dev, wait_early,
        (const it_peers*)(w->sharded ? c->peers_dev : nullptr), w->map,
        (w->sharded && (size_t)ntok * w->out_rows <= c->ll_slots) ? 1 : 0, (int)w->out_rows));
    c->pdl_safe_q8 = x;
    return IT_OK;
}

// Largest ring (up to `want` chunks) that fits `per_cta` bytes of shared memory; 0 if not even `need` fit.
int ring_slots(int MT, int nb, int nbuf, int per_cta, int want, int need, int cw = CWARPS) {
    int slots = want;
    while (slots >= need && smem_layout(MT, nb, slots, nbuf, cw).total > per_cta) slots--;
    return slots >= need ? slots : 0;
}

// Shape policy: a persistent grid with a producer warp and one consumer group per CTA, as many CTAs per SM as the
// staged activation rows, the terms and a ring of at least four chunks leave room for: four for short rows (K <= 8192;
// 17408 x 5120: 6.0 us against 6.6 us for one CTA per row group that requests its whole row group at once), three
// for long rows (the 160 row groups of a 5120 x 17408 matrix then have a CTA each: 5.2 us against 8.4 us with one
// three-group CTA per SM, where twelve CTAs had to take a second row group).  Three consumer groups only when a
// single CTA fits an SM and the rows are long, so that the per-warp chain stays short.
template <int MT, bool SUMI>
int launch(it_ctx* c, const it_mat* w, int ntok, const it_q8* x, size_t xrow0, float* y, size_t y_stride, int accum, int32_t* sumi) {
    const int nb = (int)(w->cols / 128), cpr = (nb + CWARPS - 1) / CWARPS, rgs = (int)w->row_groups;
    const bool long_rows = nb > 64;
    // Short rows, one to four activation rows, enough row groups for two CTAs per SM: CTAs of four consumer warps and a
    // small ring, up to eight per SM.  Two consecutive launches then fit an SM side by side, so the CTAs of the next
    // matvec are resident and filling their rings while this one drains, and its first chunks are in shared memory
    // when its turn comes (17408 x 5120 in a back-to-back sweep: 5.98 us with the eight-warp CTAs below).
    static const bool small_ctas = !getenv("IT_MV_CW4") || atoi(getenv("IT_MV_CW4")) != 0;
    if (small_ctas && !SUMI && MT <= 4 && !long_rows && rgs >= 2 * c->sm_count) {
        // as many of these CTAs per SM as their footprint allows (eight at one activation row, six at two: every row
        // adds its staged bytes and its block sums), and only when every row group gets a CTA of its own in one wave:
        // with fewer than four per SM, or with CTAs that loop over row groups, the eight-warp CTAs below do better
        // (34816 x 5120 at two rows: 13.8 us against 12.1 us)
        constexpr int CW = 4, MAX_PER_SM = 8;
        const int cpr4 = (nb + CW - 1) / CW, slots = cpr4 < 3 ? cpr4 : 3;
        const int per_sm = std::min(MAX_PER_SM, SM_SMEM / (smem_layout(MT, nb, slots, 1, CW).total + 1024));
        if (per_sm >= 4 && rgs <= per_sm * c->sm_count)
            return launch_cfg<MT, 1, MAX_PER_SM, false, CW>(c, w, ntok, x, xrow0, y, y_stride, accum, nullptr, slots, 1, rgs);
    }
    for (int per_sm = long_rows ? 3 : 4; per_sm >= 1; per_sm--) {
        const int grid = rgs < per_sm * c->sm_count ? rgs : per_sm * c->sm_count;
        const int nbuf = SUMI ? 0 : (grid == rgs ? 1 : 2);
        const int want = long_rows ? 16 : (per_sm == 4 ? 6 : (cpr + 2 > 4 ? cpr + 2 : 4));
        const int slots = ring_slots(MT, nb, nbuf, SM_SMEM / per_sm - 1024, want, cpr < 4 ? cpr : 4);
        if (!slots) continue;
        if (SUMI) return launch_cfg<MT, 1, 1, SUMI>(c, w, ntok, x, xrow0, y, y_stride, accum, sumi, slots, nbuf, grid);
        if (per_sm == 4) return launch_cfg<MT, 1, 4, false>(c, w, ntok, x, xrow0, y, y_stride, accum, nullptr, slots, nbuf, grid);
        if (per_sm == 3) return launch_cfg<MT, 1, 3, false>(c, w, ntok, x, xrow0, y, y_stride, accum, nullptr, slots, nbuf, grid);
        if (per_sm == 2) return launch_cfg<MT, 1, 2, false>(c, w, ntok, x, xrow0, y, y_stride, accum, nullptr, slots, nbuf, grid);
        // a single CTA per SM: long rows get three consumer groups so that the per-warp chain stays short
        if (long_rows) return launch_cfg<MT, 3, 1, false>(c, w, ntok, x, xrow0, y, y_stride, accum, nullptr, slots, nbuf, grid);
        return launch_cfg<MT, 1, 1, false>(c, w, ntok, x, xrow0, y, y_stride, accum, nullptr, slots, nbuf, grid);
    }
    return it_fail(IT_EINVAL, "it_matvec_t2: %d rows of width %zu exceed the shared-memory budget", MT, w->cols);
}

template <bool SUMI>
int dispatch(it_ctx* c, const it_mat* w, size_t ntok, const it_q8* x, float* y, size_t y_stride, int accum, int32_t* sumi) {
    // activation rows are processed in groups of up to eight (one mma N tile); wide matrices use smaller
    // groups so that the staged rows, the per-block terms and a ring of at least four chunks fit one SM
    const int nb = (int)(w->cols / 128);
    // more than one mma N tile of activation rows: the tile kernel reads the weights once per 64 rows
    if (!SUMI && ntok > 8) return it_matmul_t2_launch(c, w, (int)ntok, x, y, y_stride, accum);
    size_t group = 8;
    while (group > 1 && smem_layout((int)group, nb, 4, SUMI ? 0 : 2).total > SM_SMEM - 1024) group /= 2;
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
    IT_CHECK_ARG(ntok == 1 || y_stride >= w->out_rows, "it_matvec_t2: output stride %zu is shorter than a row of %zu results", y_stride, w->out_rows);
    IT_CHECK_ARG(y_off <= c->arena_floats && (ntok - 1) * y_stride + w->out_rows <= c->arena_floats - y_off, "it_matvec_t2: output rows fall outside the arena");
    if (w->sharded && !c->peers_dev) return it_fail(IT_ESTATE, "it_matvec_t2: the matrix is a row shard but no peers are attached to the context");
    return dispatch<false>(c, w, ntok, x, c->arena + y_off, y_stride, accum, nullptr);
}

IT_API int it_matvec_t2_sumi(it_ctx* c, const it_mat* w, size_t ntok, const it_q8* x, int32_t* sumi_dev) {
    int r = check(c, w, ntok, x, "it_matvec_t2_sumi"); if (r) return r;
    IT_CHECK_ARG(sumi_dev, "it_matvec_t2_sumi: null output");
    return dispatch<true>(c, w, ntok, x, nullptr, 0, 0, sumi_dev);
}
