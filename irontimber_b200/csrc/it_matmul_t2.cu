// Ternary GEMM on q8k activations for many activation rows (prompt chunks, wide verification passes): the role of
// the 64x64 tile kernels that VkEngine::mv selects once ntok >= tile_min (src/vk/mod.rs:655-677), with the
// arithmetic of cpu::matvec's ternary arm (src/cpu.rs:48-63):
//     y[t, r] = sum over blocks b ascending of  (d_w[r,b] * d_x[t,b/2]) * float(S[t,r,b] - sum128[t,b]).
//
// A CTA owns WR row groups (32 rows each) x 64 activation rows and walks the 128-column blocks front to back.
// A producer thread fills a ring of stages: per block the WR weight tiles (1088 bytes each, one bulk copy each) and
// the 128 int8 of all 64 activation rows as one box of a tiled tensor map (cp.async.bulk.tensor, 128-byte swizzle, so
// that the 16-byte fragment loads of a quarter warp fall on distinct banks; rows past the end of the buffer read as
// zero).  Many small bulk copies instead of the box cost about 60 cycles each.  The consumer warps are laid out
// WR x WT: a warp owns one row group and NT = 8/WT column tiles of eight activation rows.  Per block it forms the
// A operands from the packed 2-bit words by one AND per register, issues 8*NT mma.sync.m16n8k32 (u8 x s8 -> s32)
// and folds the exact block sums into f32 accumulators that stay in registers for the whole row of blocks: one
// thread adds the terms of one (row, activation row) pair in ascending block order, which is the CPU's order, so
// the result is bit-identical and no partial float sums are ever combined.  Weights cross HBM once per 64
// activation rows.
//
// Every mbarrier wait is bounded; a wait that runs out raises the context's error flag (IT_ETIMEOUT), the producer
// waits (again bounded) for its copies in flight and the CTA leaves.
#include "it_internal.h"
#include "it_pipe.cuh"

namespace {

constexpr int MM_TOK = 64;                 // activation rows per CTA
constexpr int MM_X_BYTES = MM_TOK * 128;   // one box of the activation tensor map
constexpr int MM_SMEM_MAX = 226 * 1024;

struct MmSmem { int stage, stage_bytes, dx, s128, bars, flag, total; };
__host__ __device__ inline MmSmem mm_layout(int WR, int nb, int stages) {
    MmSmem L; int o = 0;
    L.stage_bytes = (MM_X_BYTES + WR * IT_TILE_BYTES + 1023) & ~1023;   // the swizzled box needs 1024-byte alignment
    L.stage = o; o += stages * L.stage_bytes;
    L.dx = o; o += (nb / 2) * MM_TOK * 4;          // [block pair][activation row]
    L.s128 = o; o += nb * MM_TOK * 4;              // [block][activation row]
    L.bars = o; o += 2 * stages * 8;
    L.flag = o; o += 16;
    L.total = o;
    return L;
}

// exact int -> float for |v| < 2^22 without the conversion pipe: 1.5 * 2^23 + v is representable, then subtract
__device__ __forceinline__ float small_int_to_float(int v) { return __fsub_rn(__int_as_float(0x4B400000 + v), 12582912.0f); }

template <int WR, int WT>
__global__ void __launch_bounds__((WR * WT + 1) * 32, 1)
k_matmul_t2(const __grid_constant__ CUtensorMap xmap, const uint8_t* __restrict__ tiles, int nb, int rows, int row_groups, int stages,
            const float* __restrict__ xd, const int32_t* __restrict__ xs128, int x_stride, int ntok,
            float* arena, size_t y_off, size_t y_stride, int accum, int* error_flag, const it_peers* peers, const it_rowmap map) {
    constexpr int NCW = WR * WT, NT = MM_TOK / (8 * WT);   // consumer warps; mma column tiles (8 activation rows) per warp
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const MmSmem L = mm_layout(WR, nb, stages);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.flag);
    const unsigned bars = smem_u32(smem + L.bars);               // full[s] at bars + 8*s, empty[s] at bars + 8*(stages + s)
    const int rg0 = (int)blockIdx.x * WR, tok0 = (int)blockIdx.y * MM_TOK;
    const int ntv = min(MM_TOK, ntok - tok0);                    // activation rows this CTA really has
    const int nrg = min(WR, row_groups - rg0);                   // row groups this CTA really has

    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < stages; s++) { mbar_init(bars + 8 * s, 1); mbar_init(bars + 8 * (stages + s), NCW); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // the activation rows come from the kernel before this one
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == NCW) {
        // ---------------- producer: one thread keeps the ring full
        int s = 0, issued = 0; unsigned ph = 0;
        const unsigned stage_tx = (unsigned)(nrg * IT_TILE_BYTES + MM_X_BYTES);
        if (lane == 0) for (int b = 0; b < nb; b++) {
            if (!mbar_wait(bars + 8 * (stages + s), ph ^ 1u, abort_flag, error_flag)) break;
            unsigned char* st = smem + L.stage + s * L.stage_bytes;
            mbar_expect_tx(bars + 8 * s, stage_tx);
            tma_load_2d(smem_u32(st), &xmap, b * 128, tok0, bars + 8 * s);
            for (int i = 0; i < nrg; i++)
                bulk_load(smem_u32(st + MM_X_BYTES + i * IT_TILE_BYTES), tiles + ((size_t)(rg0 + i) * nb + b) * IT_TILE_BYTES, IT_TILE_BYTES, bars + 8 * s);
            issued++;
            if (++s == stages) { s = 0; ph ^= 1u; }
        }
        if (*abort_flag && lane == 0) {
            // leave only after every copy this warp started has landed (each wait bounded by the clock limit)
            const int first = issued > stages ? issued - stages : 0;
            for (int k = first; k < issued; k++) {
                const long long t0 = clock64();
                while (!mbar_test(bars + 8 * (k % stages), (unsigned)(k / stages) & 1u) && clock64() - t0 < WAIT_CLOCKS) { }
            }
        }
        return;
    }

    // ---------------- consumers
    float* dxs = reinterpret_cast<float*>(smem + L.dx);
    int* sss = reinterpret_cast<int*>(smem + L.s128);
    for (int i = tid; i < (nb / 2) * MM_TOK; i += NCW * 32) { const int m = i % MM_TOK, bb = i / MM_TOK; dxs[i] = m < ntv ? xd[(size_t)(tok0 + m) * (x_stride / 256) + bb] : 0.f; }
    for (int i = tid; i < nb * MM_TOK; i += NCW * 32) { const int m = i % MM_TOK, bb = i / MM_TOK; sss[i] = m < ntv ? xs128[(size_t)(tok0 + m) * (x_stride / 128) + bb] : 0; }
    consumer_barrier<NCW * 32>();

    const int g = lane >> 2, t = lane & 3;
    const int wr = warp / WT, wt = warp % WT;
    const int tb = wt * NT * 8;                                  // first activation row of this warp inside the CTA tile
    const bool rg_valid = wr < nrg;
    float acc[NT][4][2];
#pragma unroll
    for (int n = 0; n < NT; n++)
#pragma unroll
        for (int r = 0; r < 4; r++) { acc[n][r][0] = 0.f; acc[n][r][1] = 0.f; }

    int s = 0; unsigned ph = 0;
    for (int b = 0; b < nb; b++) {
        const bool ready = mbar_wait(bars + 8 * s, ph, abort_flag, error_flag);
        if (ready && rg_valid && tb < ntv) {
            const unsigned char* st = smem + L.stage + s * L.stage_bytes;
            const unsigned char* tile = st + MM_X_BYTES + wr * IT_TILE_BYTES;
            const uint4 wa = *reinterpret_cast<const uint4*>(tile + 16 * lane);
            const uint4 wb = *reinterpret_cast<const uint4*>(tile + 512 + 16 * lane);
            const uint2 sc = *reinterpret_cast<const uint2*>(tile + 1024 + 8 * g);
            const uint32_t w[8] = { wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w };
            uint32_t a[8][4];
#pragma unroll
            for (int j = 0; j < 8; j++) { a[j][0] = w[j] & 0x03030303u; a[j][1] = w[j] & 0x0c0c0c0cu; a[j][2] = w[j] & 0x30303030u; a[j][3] = w[j] & 0xc0c0c0c0u; }
            const __half2 h01 = *reinterpret_cast<const __half2*>(&sc.x), h23 = *reinterpret_cast<const __half2*>(&sc.y);
            const float dw[4] = { __low2float(h01), __high2float(h01), __low2float(h23), __high2float(h23) };
#pragma unroll
            for (int n = 0; n < NT; n++) {
                {   // column tiles past the last activation row work on zeros or on rows nobody stores
                    // row tb + 8n + g of the box; its 16-byte pieces are stored at piece index ^ (row % 8)
                    const unsigned char* xrow = st + (tb + 8 * n + g) * 128;
                    const uint4 xa = *reinterpret_cast<const uint4*>(xrow + (((2 * t) ^ g) << 4));
                    const uint4 xb4 = *reinterpret_cast<const uint4*>(xrow + (((2 * t + 1) ^ g) << 4));
                    const uint32_t xb[8] = { xa.x, xa.y, xa.z, xa.w, xb4.x, xb4.y, xb4.z, xb4.w };
                    int cx[4] = {0, 0, 0, 0}, cy[4] = {0, 0, 0, 0};
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        mma_u8s8(cx, a[2 * j][0], a[2 * j][1], a[2 * j + 1][0], a[2 * j + 1][1], xb[2 * j], xb[2 * j + 1]);
                        mma_u8s8(cy, a[2 * j][2], a[2 * j][3], a[2 * j + 1][2], a[2 * j + 1][3], xb[2 * j], xb[2 * j + 1]);
                    }
                    const int c0 = tb + 8 * n + 2 * t;               // activation rows c0, c0 + 1 land in this lane
                    const float2 dx = *reinterpret_cast<const float2*>(dxs + (b >> 1) * MM_TOK + c0);
                    const int2 s2 = *reinterpret_cast<const int2*>(sss + b * MM_TOK + c0);
                    const int S0[4] = { cx[0], cx[2] >> 2, cy[0] >> 4, cy[2] >> 6 };
                    const int S1[4] = { cx[1], cx[3] >> 2, cy[1] >> 4, cy[3] >> 6 };
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        acc[n][r][0] = __fadd_rn(acc[n][r][0], __fmul_rn(__fmul_rn(dw[r], dx.x), small_int_to_float(S0[r] - s2.x)));
                        acc[n][r][1] = __fadd_rn(acc[n][r][1], __fmul_rn(__fmul_rn(dw[r], dx.y), small_int_to_float(S1[r] - s2.y)));
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + 8 * (stages + s));     // the stage may be refilled
        if (++s == stages) { s = 0; ph ^= 1u; }
    }
    if (!*abort_flag && rg_valid) {
#pragma unroll
        for (int n = 0; n < NT; n++)
#pragma unroll
            for (int cc = 0; cc < 2; cc++) {
                const int m = tb + 8 * n + 2 * t + cc;
                if (m < ntv) {
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        const int row = (rg0 + wr) * 32 + g + 8 * r;
                        if (row < rows) it_result_store(peers, arena, y_off + (size_t)(tok0 + m) * y_stride + it_map_row(map, row), acc[n][r][cc], accum);
                    }
                }
            }
    }
    if (peers) {
        // sharded launch: make this CTA's pushes visible system-wide, then count the CTA as done
        __threadfence_system();
        consumer_barrier<NCW * 32>();
        if (tid == 0) it_shard_finish(peers, gridDim.x * gridDim.y, error_flag);
    }
}

template <int WR, int WT>
int mm_launch(it_ctx* c, const it_mat* w, int ntok, const it_q8* x, float* y, size_t y_stride, int accum) {
    const int nb = (int)(w->cols / 128);
    // the smaller tiles run two CTAs per SM when a ring of at least three stages fits half the shared memory
    int stages = 6;
    const int half = MM_SMEM_MAX / 2 - 1024;
    if (WR * WT <= 8 && mm_layout(WR, nb, 3).total + 1024 <= half) { while (mm_layout(WR, nb, stages).total + 1024 > half) stages--; }
    else while (stages > 2 && mm_layout(WR, nb, stages).total + 1024 > MM_SMEM_MAX) stages--;
    const MmSmem L = mm_layout(WR, nb, stages);
    if (L.total + 1024 > MM_SMEM_MAX) return it_fail(IT_EINVAL, "it_matvec_t2: rows of width %zu exceed the shared-memory budget of the tile kernel", w->cols);
    auto kern = k_matmul_t2<WR, WT>;
    static bool attr_set[16] = {};
    if (!attr_set[c->device & 15]) { IT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, MM_SMEM_MAX)); attr_set[c->device & 15] = true; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((w->row_groups + WR - 1) / WR), (unsigned)((ntok + MM_TOK - 1) / MM_TOK));
    cfg.blockDim = dim3((WR * WT + 1) * 32); cfg.dynamicSmemBytes = (size_t)L.total + 1024; cfg.stream = c->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    IT_CUDA(cudaLaunchKernelEx(&cfg, kern, x->tmap, (const uint8_t*)w->tiles, nb, (int)w->rows, (int)w->row_groups, stages,
        (const float*)x->d, (const int32_t*)x->sum128, (int)x->max_n, ntok, c->arena, (size_t)(y - c->arena), y_stride, accum, c->error_flag_dev,
        (const it_peers*)(w->sharded ? c->peers_dev : nullptr), w->map));
    c->pdl_safe_q8 = x;     // this kernel waits for its predecessor before it lets its successor start
    return IT_OK;
}

}  // namespace

// Tile policy: 128-row tiles with sixteen consumer warps when that still gives the grid at least 0.6 CTAs per SM, else
// 64-row tiles (eight warps, two CTAs per SM), else 32-row tiles.
int it_matmul_t2_launch(it_ctx* c, const it_mat* w, int ntok, const it_q8* x, float* y, size_t y_stride, int accum) {
    const long tok_tiles = (ntok + MM_TOK - 1) / MM_TOK;
    const long want = (long)c->sm_count * 6 / 10;
    // The tensor-memory kernel (it_matmul_tc.cu) works on 128-row tiles: it takes the shapes that give such tiles to
    // most SMs; smaller matrices keep the finer tiles of the kernel in this file.  IT_MATMUL=legacy / tc forces one.
    const char* fv = getenv("IT_MATMUL");      // read on every call so that a test can exercise both kernels on one shape
    const int force = !fv ? 0 : !strcmp(fv, "legacy") ? 1 : !strcmp(fv, "tc") ? 2 : 0;
    if (force != 1 && (force == 2 || (long)((w->row_groups + 3) / 4) * tok_tiles >= want)) {
        const int r = it_matmul_tc_launch(c, w, ntok, x, y, y_stride, accum); if (r <= 0) return r;
    }
    if ((long)((w->row_groups + 3) / 4) * tok_tiles >= want) return mm_launch<4, 4>(c, w, ntok, x, y, y_stride, accum);
    if ((long)((w->row_groups + 1) / 2) * tok_tiles >= want) return mm_launch<2, 4>(c, w, ntok, x, y, y_stride, accum);
    return mm_launch<1, 8>(c, w, ntok, x, y, y_stride, accum);
}
