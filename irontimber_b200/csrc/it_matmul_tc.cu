// Ternary GEMM on q8k activations with the 5th-generation tensor cores: tcgen05.mma kind::i8, accumulators in tensor
// memory.  Same function and the same bits as k_matmul_t2 (it_matmul_t2.cu) and cpu::matvec's ternary arm
// (src/cpu.rs:48-63); it takes the place of the 64x64 tile kernels VkEngine::mv selects for prompt chunks
// (src/vk/mod.rs:655-677).
//
// A CTA owns 128 matrix rows (four 32-row groups) x 64 activation rows (x 128 when the launch has more than 64: one
// expanded tile and one issue sequence then feed twice the columns) and walks the 128-column blocks in order.
//   warp 24  producer: per block one stage = four weight tiles (bulk copies) + the 64 x 128 int8 activations as one
//            box of a tiled tensor map with the 128-byte swizzle, i.e. already in the K-major layout the MMA reads
//   warps 16-23 expanders (two sets of four, alternating blocks): turn the packed 2-bit codes of a stage into a 128 x 128 tile of unsigned bytes (codes 0..3)
//            in the same K-major 128-byte-swizzled layout (row r at 128 r, 16-byte piece p at (p ^ (r & 7)) * 16),
//            and the f16 block scales of the 128 rows into f32
//   warp 25  one thread issues four tcgen05.mma (M 128, N 64, K 32, u8 x s8 -> s32) per block into one of eight
//            64-column accumulators in tensor memory and commits them to mbarriers (accumulator ready; A tile and
//            stage free again)
//   warps 0-15 epilogue, four groups of four warps: group q owns activation rows 16 q .. 16 q + 15, its thread r reads
//            those columns of row r of the accumulator (tcgen05.ld 32x32b; warp w may touch lanes 32 (w % 4) ..), forms
//            (d_w * d_x) * float(S - sum128) for each and adds it to an f32 accumulator it keeps in registers for the
//            whole row of blocks: ascending block order, one thread per (row, activation row) pair - the CPU's order,
//            bit for bit.  The MMA of block b + 1 runs while block b is folded.
// Integer block sums are exact whatever the hardware's summation order, so only the f32 epilogue decides the bits.
//
// Every wait is bounded; when one runs out the CTA raises the context's error flag (IT_ETIMEOUT), every role leaves
// its loop, the producer waits (bounded) for its copies in flight, and the tensor memory is released before the CTA exits.
#include "it_internal.h"
#include "it_pipe.cuh"

namespace {

constexpr int TC_ROWS = 128;                     // matrix rows per CTA (M of the MMA)
constexpr int TC_A_BYTES = TC_ROWS * 128;        // one expanded weight tile
constexpr int TC_KB = 4;                         // blocks per weight stage: one bulk copy per row group and stage (issuing a bulk copy costs a
                                                 // thread some 250 cycles, so four small copies per block made the producer the bottleneck)
constexpr int TC_W_BYTES = 4 * TC_KB * IT_TILE_BYTES;   // four row groups x TC_KB consecutive tiles
constexpr int TC_NA = 2;                         // expanded tiles in flight
constexpr int TC_NDW = 16;                       // ring of per-block row scales (expanders run at most TC_NA + ND blocks ahead of the epilogue)
constexpr int TC_SMEM_MAX = 226 * 1024;
constexpr unsigned TC_TMEM_COLS = 512;           // all of it: ND accumulators x TOK columns
constexpr int TC_EPI_GROUPS = 4, TC_EPI_WARPS = 4 * TC_EPI_GROUPS;   // epilogue warps 0..15
// NH: 64-row halves of the CTA's activation tile.  NH = 1: 64 activation rows per CTA (prompt passes of up to 64 rows).
// NH = 2: 128 rows: one expanded weight tile and one issue sequence feed twice the columns, which is what the kernel is
// bound by (the tensor pipe is 8 % busy at 64 rows); the epilogue then folds 32 values per thread and block.
template <int NH> struct Tc {
    static constexpr int TOK = 64 * NH;                  // activation rows per CTA (N of the MMA)
    static constexpr int X_BYTES = TOK * 128;            // the activation tile of one block: NH boxes of the tensor map, one under the other
    static constexpr int XS = NH == 1 ? 6 : 3;           // activation tiles in flight (they come from L2)
    static constexpr int ND = 512 / TOK;                 // accumulators in tensor memory: the MMA -> read-out -> release loop is long, so many are in flight
    static constexpr int EPI_TOK = TOK / TC_EPI_GROUPS;  // activation rows per epilogue thread
    static constexpr int ESETS = NH == 1 ? 2 : 1;        // sets of four expander warps; set e expands the blocks b with b % ESETS == e
    static constexpr int EXP_WARPS = 4 * ESETS;
    static constexpr int THREADS = (TC_EPI_WARPS + EXP_WARPS + 3) * 32;   // + weight producer, MMA issuer, activation producer
    // kind::i8 instruction descriptor: D s32, A unsigned 8 bit, B signed 8 bit, both K-major, N = TOK, M = 128
    static constexpr unsigned IDESC = (2u << 4) | (0u << 7) | (1u << 10) | ((unsigned)(TOK >> 3) << 17) | ((unsigned)(TC_ROWS >> 4) << 24);
};

// Weight stages and activation boxes have rings of their own: the weights come from HBM (a deep ring, about 70 KB in
// flight per SM, hides its latency), the boxes from L2.
struct TcSmem { int x, a, w, dx, s128, dw, bars, tmem, flag, total; };
template <int NH> __host__ __device__ inline TcSmem tc_layout(int nb, int wstages) {
    constexpr int TC_XS = Tc<NH>::XS, TC_X_BYTES = Tc<NH>::X_BYTES, TC_TOK = Tc<NH>::TOK, TC_ND = Tc<NH>::ND;
    TcSmem L; int o = 0;
    L.x = o; o += TC_XS * TC_X_BYTES;              // 1024-byte aligned (128-byte swizzle)
    L.a = o; o += TC_NA * TC_A_BYTES;              // 1024-byte aligned
    L.w = o; o += wstages * TC_W_BYTES;
    L.dx = o; o += (nb / 2) * TC_TOK * 4;
    L.s128 = o; o += nb * TC_TOK * 4;
    L.dw = o; o += TC_NDW * TC_ROWS * 4;
    o = (o + 15) & ~15;
    L.bars = o; o += (2 * wstages + TC_XS + TC_NA + 2 * TC_ND) * 8;
    L.tmem = o; o += 16;
    L.flag = o; o += 16;
    L.total = o;
    return L;
}

// K-major operand tile with 128-byte rows and the 128-byte swizzle: start address in 16-byte units, 8-row groups 1024
// bytes apart (stride byte offset), descriptor version 1, layout type 2 (128-byte swizzle).
__device__ __forceinline__ unsigned long long tc_smem_desc(unsigned addr) {
    return (unsigned long long)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((unsigned long long)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
template <bool ACC>
__device__ __forceinline__ void tc_mma(unsigned d_tmem, unsigned long long adesc, unsigned long long bdesc, unsigned idesc) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
                 :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "n"(ACC ? 1 : 0), "r"(0u) : "memory");
}
__device__ __forceinline__ void tc_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld16(unsigned taddr, int (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]),
                   "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr) : "memory");
}

// v + 0x4B400000 (the bit pattern of 1.5 * 2^23 plus an integer of magnitude below 2^22) as the float v, exactly; the block's
// -sum128 and the constant are one shared-memory word, so the conversion costs one integer and one float addition
__device__ __forceinline__ float tc_biased_to_float(int biased) { return __fsub_rn(__int_as_float(biased), 12582912.0f); }

template <int NH>
__global__ void __launch_bounds__(Tc<NH>::THREADS, 1)
k_matmul_tc(const __grid_constant__ CUtensorMap xmap, const uint8_t* __restrict__ tiles, int nb, int rows, int row_groups, int wstages,
            const float* __restrict__ xd, const int32_t* __restrict__ xs128, int x_stride, int ntok,
            float* arena, size_t y_off, size_t y_stride, int accum, int* error_flag, const it_peers* peers, const it_rowmap map) {
    constexpr int TC_TOK = Tc<NH>::TOK, TC_X_BYTES = Tc<NH>::X_BYTES, TC_XS = Tc<NH>::XS, TC_ND = Tc<NH>::ND, TC_EPI_TOK = Tc<NH>::EPI_TOK,
                  TC_ESETS = Tc<NH>::ESETS, TC_EXP_WARPS = Tc<NH>::EXP_WARPS;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const TcSmem L = tc_layout<NH>(nb, wstages);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.flag);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(smem + L.tmem);
    const unsigned bars = smem_u32(smem + L.bars);
    // barrier addresses: weight stages (full / empty), activation boxes landed, expanded tiles ready, accumulators (full / empty).
    // "Accumulator d full" is the one commit of a block: it also tells the expanders and the activation producer that the
    // tile and the box that block read may be reused.
    const unsigned wfull0 = bars, wempty0 = wfull0 + 8 * wstages, xfull0 = wempty0 + 8 * wstages,
                   afull0 = xfull0 + 8 * TC_XS, dfull0 = afull0 + 8 * TC_NA, dempty0 = dfull0 + 8 * TC_ND;
    const int rg0 = (int)blockIdx.x * 4, tok0 = (int)blockIdx.y * TC_TOK;
    const int ntv = min(TC_TOK, ntok - tok0), nrg = min(4, row_groups - rg0);

    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < wstages; s++) { mbar_init(wfull0 + 8 * s, 1); mbar_init(wempty0 + 8 * s, 4 * TC_KB); }
        for (int s = 0; s < TC_XS; s++) mbar_init(xfull0 + 8 * s, 1);
        for (int a = 0; a < TC_NA; a++) mbar_init(afull0 + 8 * a, 128);
        for (int d = 0; d < TC_ND; d++) { mbar_init(dfull0 + 8 * d, 1); mbar_init(dempty0 + 8 * d, TC_EPI_WARPS * 32); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {   // tensor memory for the accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(tmem_slot)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *tmem_slot;

    if (warp == TC_EPI_WARPS + TC_EXP_WARPS) {
        // ---------------- weight producer: the weights depend on no earlier kernel, so it neither waits for one nor triggers.
        // Lane i < 4 copies the TC_KB consecutive tiles of row group i; lane 0 announces the bytes of the stage first.
        const int nst = (nb + TC_KB - 1) / TC_KB;
        int s = 0, issued = 0; unsigned ph = 0;
        for (int q = 0; q < nst; q++) {
            bool ok = true;
            if (lane == 0) ok = mbar_wait(wempty0 + 8 * s, ph ^ 1u, abort_flag, error_flag, 11);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            const int kb = min(TC_KB, nb - q * TC_KB);
            unsigned char* st = smem + L.w + s * TC_W_BYTES;
            if (lane == 0) mbar_expect_tx(wfull0 + 8 * s, (unsigned)(nrg * kb * IT_TILE_BYTES));
            __syncwarp();
            if (lane < nrg) bulk_load(smem_u32(st + lane * TC_KB * IT_TILE_BYTES), tiles + ((size_t)(rg0 + lane) * nb + (size_t)q * TC_KB) * IT_TILE_BYTES,
                                      (unsigned)(kb * IT_TILE_BYTES), wfull0 + 8 * s);
            issued++;
            if (++s == wstages) { s = 0; ph ^= 1u; }
        }
        if (*abort_flag && lane == 0) {   // leave only after every copy this warp started has landed (bounded)
            const int first = issued > wstages ? issued - wstages : 0;
            for (int k = first; k < issued; k++) {
                const long long t0 = clock64();
                while (!mbar_test(wfull0 + 8 * (k % wstages), (unsigned)(k / wstages) & 1u) && clock64() - t0 < WAIT_CLOCKS) { }
            }
        }
    } else if (warp == TC_EPI_WARPS + TC_EXP_WARPS + 2) {
        // ---------------- activation producer: the rows come from the kernel before this one
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            int s = 0, issued = 0;
            for (int b = 0; b < nb; b++) {
                // the box slot was last read by block b - TC_XS: wait for that block's commit
                if (b >= TC_XS && !mbar_wait(dfull0 + 8 * ((b - TC_XS) % TC_ND), (unsigned)((b - TC_XS) / TC_ND) & 1u, abort_flag, error_flag, 19)) break;
                mbar_expect_tx(xfull0 + 8 * s, (unsigned)TC_X_BYTES);
#pragma unroll
                for (int hh = 0; hh < NH; hh++)     // 64 rows per box; the boxes of a block lie one under the other like one box of TOK rows
                    tma_load_2d(smem_u32(smem + L.x + s * TC_X_BYTES + hh * 64 * 128), &xmap, b * 128, tok0 + 64 * hh, xfull0 + 8 * s);
                issued++;
                if (++s == TC_XS) s = 0;
            }
            if (*abort_flag) {
                const int first = issued > TC_XS ? issued - TC_XS : 0;
                for (int k = first; k < issued; k++) {
                    const long long t0 = clock64();
                    while (!mbar_test(xfull0 + 8 * (k % TC_XS), (unsigned)(k / TC_XS) & 1u) && clock64() - t0 < WAIT_CLOCKS) { }
                }
            }
        }
    } else if (warp == TC_EPI_WARPS + TC_EXP_WARPS + 1) {
        // ---------------- MMA issuer.  Its loop is the critical path of the CTA (one thread, three barrier waits and seven
        // asynchronous instructions per block), so the waits try the non-blocking test first.
        if (lane == 0) {
            int s = 0, a = 0, d = 0; unsigned aph = 0;
            const unsigned long long adesc0 = tc_smem_desc(smem_u32(smem + L.a)), bdesc0 = tc_smem_desc(smem_u32(smem + L.x));
            for (int b = 0; b < nb; b++) {
                // one wait per block: the expanders arrive only when the tile is expanded, the activation box has landed and the
                // accumulator has been read out (this thread's loop is the critical path of the CTA)
                if (!mbar_wait(afull0 + 8 * a, aph, abort_flag, error_flag, 12)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // descriptors differ from the first tile's only in the start-address field (16-byte units): + tile index, + 2 per K step of 32
                const unsigned long long ad = adesc0 + (unsigned)(a * (TC_A_BYTES >> 4)), bd = bdesc0 + (unsigned)(s * (TC_X_BYTES >> 4));
                const unsigned dt = tmem_base + (unsigned)(d * TC_TOK);
                tc_mma<false>(dt, ad, bd, Tc<NH>::IDESC);
                tc_mma<true>(dt, ad + 2, bd + 2, Tc<NH>::IDESC);
                tc_mma<true>(dt, ad + 4, bd + 4, Tc<NH>::IDESC);
                tc_mma<true>(dt, ad + 6, bd + 6, Tc<NH>::IDESC);
                tc_commit(dfull0 + 8 * d);        // accumulator complete; tile and box of this block may be reused
                if (++s == TC_XS) s = 0;
                if (++a == TC_NA) { a = 0; aph ^= 1u; }
                if (++d == TC_ND) d = 0;
            }
        }
    } else if (warp >= TC_EPI_WARPS) {
        // ---------------- expanders: warp 16 + 4 e + i expands row group i of the blocks b with b % TC_ESETS == e
        // (one warp per row group could not keep up: a single warp issues its hundred dependent instructions per block slowly)
        const int eset = (warp - TC_EPI_WARPS) >> 2, rgl = (warp - TC_EPI_WARPS) & 3, g = lane >> 2, t = lane & 3;
        float* dws = reinterpret_cast<float*>(smem + L.dw);
        for (int b = eset; b < nb; b += TC_ESETS) {
            const int q = b / TC_KB, s = q % wstages, a = b % TC_NA;
            const unsigned sph = (unsigned)(q / wstages) & 1u;
            if (!mbar_wait(wfull0 + 8 * s, sph, abort_flag, error_flag, 15)) break;
            // the tile buffer was last read by block b - TC_NA: wait for that block's commit
            if (b >= TC_NA && !mbar_wait(dfull0 + 8 * ((b - TC_NA) % TC_ND), (unsigned)((b - TC_NA) / TC_ND) & 1u, abort_flag, error_flag, 16)) break;
            const unsigned char* tile = smem + L.w + s * TC_W_BYTES + (rgl * TC_KB + b % TC_KB) * IT_TILE_BYTES;
            const uint4 wa = *reinterpret_cast<const uint4*>(tile + 16 * lane);
            const uint4 wb = *reinterpret_cast<const uint4*>(tile + 512 + 16 * lane);
            unsigned char* at = smem + L.a + a * TC_A_BYTES;
#pragma unroll
            for (int i = 0; i < 4; i++) {         // bit pair i of every byte: matrix row g + 8 i of the group
                const int r = rgl * 32 + g + 8 * i;
                const uint4 lo = make_uint4((wa.x >> (2 * i)) & 0x03030303u, (wa.y >> (2 * i)) & 0x03030303u, (wa.z >> (2 * i)) & 0x03030303u, (wa.w >> (2 * i)) & 0x03030303u);
                const uint4 hi = make_uint4((wb.x >> (2 * i)) & 0x03030303u, (wb.y >> (2 * i)) & 0x03030303u, (wb.z >> (2 * i)) & 0x03030303u, (wb.w >> (2 * i)) & 0x03030303u);
                *reinterpret_cast<uint4*>(at + r * 128 + (((2 * t) ^ g) << 4)) = lo;       // columns 32 t .. 32 t + 15
                *reinterpret_cast<uint4*>(at + r * 128 + (((2 * t + 1) ^ g) << 4)) = hi;   // columns 32 t + 16 .. 32 t + 31
            }
            if (t == 0) {
                const uint2 sc = *reinterpret_cast<const uint2*>(tile + 1024 + 8 * g);
                const __half2 h01 = *reinterpret_cast<const __half2*>(&sc.x), h23 = *reinterpret_cast<const __half2*>(&sc.y);
                float* dw = dws + (b % TC_NDW) * TC_ROWS + rgl * 32 + g;
                dw[0] = __low2float(h01); dw[8] = __high2float(h01); dw[16] = __low2float(h23); dw[24] = __high2float(h23);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy stores before the MMA's async-proxy reads
            // the other two conditions of the block's MMA, checked here so that the issuing thread has a single wait
            if (!mbar_wait(xfull0 + 8 * (b % TC_XS), (unsigned)(b / TC_XS) & 1u, abort_flag, error_flag, 13)) break;
            if (!mbar_wait(dempty0 + 8 * (b % TC_ND), ((unsigned)(b / TC_ND) & 1u) ^ 1u, abort_flag, error_flag, 14)) break;
            mbar_arrive(afull0 + 8 * a);
            __syncwarp();
            if (lane == 0) mbar_arrive(wempty0 + 8 * s);                     // this warp has read its tile: one of the 4 * TC_KB arrivals that free the stage
        }
    } else {
        // ---------------- epilogue: group q = warp / 4 owns activation rows 16 q ..; thread r = 32 * (warp % 4) + lane owns matrix row r
        float* dxs = reinterpret_cast<float*>(smem + L.dx);
        int* sss = reinterpret_cast<int*>(smem + L.s128);
        const float* dws = reinterpret_cast<const float*>(smem + L.dw);
        constexpr int NEPI = TC_EPI_WARPS * 32;
        asm volatile("griddepcontrol.wait;" ::: "memory");            // q8 scales, block sums and (when accumulating) y come from earlier kernels
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        for (int i = tid; i < (nb / 2) * TC_TOK; i += NEPI) { const int m = i % TC_TOK, bb = i / TC_TOK; dxs[i] = m < ntv ? xd[(size_t)(tok0 + m) * (x_stride / 256) + bb] : 0.f; }
        for (int i = tid; i < nb * TC_TOK; i += NEPI) { const int m = i % TC_TOK, bb = i / TC_TOK; sss[i] = 0x4B400000 - (m < ntv ? xs128[(size_t)(tok0 + m) * (x_stride / 128) + bb] : 0); }   // ready to be added to the integer block sum: see tc_int_to_float
        asm volatile("bar.sync 1, %0;" :: "n"(NEPI) : "memory");
        const int grp = warp >> 2, r = 32 * (warp & 3) + lane, m0 = grp * TC_EPI_TOK;
        const bool active = m0 < ntv;              // groups past the last activation row only release the accumulators
        float acc[TC_EPI_TOK];
#pragma unroll
        for (int m = 0; m < TC_EPI_TOK; m++) acc[m] = 0.f;
        int d = 0; unsigned dph = 0;
        bool ok = true;
        for (int b = 0; b < nb; b++) {
            if (!mbar_wait(dfull0 + 8 * d, dph, abort_flag, error_flag, 17)) { ok = false; break; }
            int S[TC_EPI_TOK];
            if (active) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int cch = 0; cch < TC_EPI_TOK / 16; cch++)
                    tc_ld16(tmem_base + ((unsigned)((warp & 3) * 32) << 16) + (unsigned)(d * TC_TOK + m0 + 16 * cch), *reinterpret_cast<int (*)[16]>(&S[16 * cch]));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
            mbar_arrive(dempty0 + 8 * d);          // the next MMA may overwrite this accumulator
            if (active) {
                // row scales of this block: stored by the expanders before they released the tile to the MMA whose completion we just saw
                const float dw = dws[(b % TC_NDW) * TC_ROWS + r];
                const float4* dx4 = reinterpret_cast<const float4*>(dxs + (b >> 1) * TC_TOK + m0);
                const int4* s4 = reinterpret_cast<const int4*>(sss + b * TC_TOK + m0);
#pragma unroll
                for (int q = 0; q < TC_EPI_TOK / 4; q++) {
                    const float4 dx = dx4[q]; const int4 sb = s4[q];
                    acc[4 * q + 0] = __fadd_rn(acc[4 * q + 0], __fmul_rn(__fmul_rn(dw, dx.x), tc_biased_to_float(S[4 * q + 0] + sb.x)));
                    acc[4 * q + 1] = __fadd_rn(acc[4 * q + 1], __fmul_rn(__fmul_rn(dw, dx.y), tc_biased_to_float(S[4 * q + 1] + sb.y)));
                    acc[4 * q + 2] = __fadd_rn(acc[4 * q + 2], __fmul_rn(__fmul_rn(dw, dx.z), tc_biased_to_float(S[4 * q + 2] + sb.z)));
                    acc[4 * q + 3] = __fadd_rn(acc[4 * q + 3], __fmul_rn(__fmul_rn(dw, dx.w), tc_biased_to_float(S[4 * q + 3] + sb.w)));
                }
            }
            if (++d == TC_ND) { d = 0; dph ^= 1u; }
        }
        const int row = rg0 * 32 + r;
        if (ok && active && !*abort_flag && row < rows) {
            const int grow = it_map_row(map, row);
#pragma unroll
            for (int m = 0; m < TC_EPI_TOK; m++)
                if (m0 + m < ntv) it_result_store(peers, arena, y_off + (size_t)(tok0 + m0 + m) * y_stride + grow, acc[m], accum);
        }
        if (peers) __threadfence_system();
    }
    // ---------------- common end: every role arrives here, also after a wait that ran out
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
    }
    if (peers && tid == 0) it_shard_finish(peers, gridDim.x * gridDim.y, error_flag);
}

}  // namespace

template <int NH>
static int tc_launch(it_ctx* c, const it_mat* w, int ntok, const it_q8* x, float* y, size_t y_stride, int accum) {
    const int nb = (int)(w->cols / 128);
    int stages = 5;                        // weight stages of TC_KB blocks: as deep as shared memory allows (about 70 KB in flight)
    while (stages > 2 && tc_layout<NH>(nb, stages).total + 1024 > TC_SMEM_MAX) stages--;
    const TcSmem L = tc_layout<NH>(nb, stages);
    if (L.total + 1024 > TC_SMEM_MAX) return 1;
    static bool attr_set[16] = {};
    if (!attr_set[c->device & 15]) { IT_CUDA(cudaFuncSetAttribute(k_matmul_tc<NH>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_MAX)); attr_set[c->device & 15] = true; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((w->row_groups + 3) / 4), (unsigned)((ntok + Tc<NH>::TOK - 1) / Tc<NH>::TOK));
    cfg.blockDim = dim3(Tc<NH>::THREADS); cfg.dynamicSmemBytes = (size_t)L.total + 1024; cfg.stream = c->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    IT_CUDA(cudaLaunchKernelEx(&cfg, k_matmul_tc<NH>, x->tmap, (const uint8_t*)w->tiles, nb, (int)w->rows, (int)w->row_groups, stages,
        (const float*)x->d, (const int32_t*)x->sum128, (int)x->max_n, ntok, c->arena, (size_t)(y - c->arena), y_stride, accum, c->error_flag_dev,
        (const it_peers*)(w->sharded ? c->peers_dev : nullptr), w->map));
    c->pdl_safe_q8 = x;
    return IT_OK;
}

// Returns IT_OK after launching, or a positive value when the shape does not suit this kernel (the caller then uses k_matmul_t2).
// More than 64 activation rows go to the 128-row variant when its buffers fit (rows of up to about 12,000 columns).
int it_matmul_tc_launch(it_ctx* c, const it_mat* w, int ntok, const it_q8* x, float* y, size_t y_stride, int accum) {
    static const bool wide = []{ const char* v = getenv("IT_MATMUL_WIDE"); return !v || atoi(v) != 0; }();
    if (wide && ntok > 64) { const int r = tc_launch<2>(c, w, ntok, x, y, y_stride, accum); if (r != 1) return r; }
    return tc_launch<1>(c, w, ntok, x, y, y_stride, accum);
}
