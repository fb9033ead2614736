// Internal declarations shared by the translation units of libirontimber_cuda.so.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>
#include <cstdlib>
#include <map>
#include <string>
#include "../../include/irontimber_cuda.h"

#define IT_API extern "C" __attribute__((visibility("default")))

// ---- error plumbing -------------------------------------------------------------------------
int it_fail(int code, const char* fmt, ...);
#define IT_CHECK_ARG(cond, ...) do { if (!(cond)) return it_fail(IT_EINVAL, __VA_ARGS__); } while (0)
#define IT_CUDA(expr) do { cudaError_t e__ = (expr); if (e__ != cudaSuccess) \
    return it_fail(e__ == cudaErrorMemoryAllocation ? IT_ENOMEM : IT_ECUDA, "%s: %s", #expr, cudaGetErrorString(e__)); } while (0)
#define IT_LAUNCH_CHECK(name) do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) \
    return it_fail(IT_ECUDA, "launch %s: %s", name, cudaGetErrorString(e__)); } while (0)

// ---- device layout of a ternary matrix ----------------------------------------------------------
// Rows are grouped by 32 and columns by 128 (one PQ2_0 block).  Tile (rg, b) covers rows
// 32*rg .. 32*rg+31 and columns 128*b .. 128*b+127 and is IT_TILE_BYTES long; tiles of one row
// group are contiguous in ascending b, so a warp streams a row group front to back.
//
// Inside a tile, with lane = 4*g + t (g = 0..7, t = 0..3) as in the mma.m16n8k32 fragments:
//   bytes [ 16*lane      , +16): words (j=0,h=0) (0,1) (1,0) (1,1)
//   bytes [ 512 + 16*lane, +16): words (j=2,h=0) (2,1) (3,0) (3,1)
//   word (j,h), byte c, bit pair i holds the 2-bit code of row 32*rg + g + 8*i, column
//   128*b + 32*t + 8*j + 4*h + c.  Masking a word with 0x03030303 << 2*i therefore yields the
//   four int8 operands (scaled by 4^i) of matrix row g + 8*i for one mma A register.
//   bytes [1024 + 8*g, +8): f16 scales of rows g, g+8, g+16, g+24 (block b).
// 32 bytes of codes + 2 bytes of scale per 128 weights: the density of PQ2_0 itself.
#define IT_TILE_ROWS 32
#define IT_TILE_BYTES 1088

// ---- row sharding over several GPUs -----------------------------------------------------------------------------
// A matrix may hold only some rows of a logical matrix; its results land at the rows' positions in the full output and
// are pushed into the arena of every attached peer (one process per GPU, arenas mapped through CUDA IPC).
#define IT_MAX_PEERS 8
struct it_peers {                       // lives in device memory, one per attached context
    float* arena[IT_MAX_PEERS];         // every rank's arena as mapped into this process (own arena at [rank])
    unsigned* flags[IT_MAX_PEERS];      // every rank's flag words: flags[p][r] is written by rank r and read by rank p
    int rank, world;
    unsigned* done;                     // CTAs of the running sharded kernel that have finished their stores
    unsigned* epoch;                    // sharded ops completed so far (the same sequence on every rank)
    // low-latency exchange: every rank's buffer of 8-byte (value, epoch) slots, two halves of ll_slots slots used by
    // even and odd epochs; a slot is complete as soon as its epoch tag matches, no fence or flag needed
    unsigned long long* ll[IT_MAX_PEERS];
    size_t ll_slots;
    long long wait_clocks;              // how long a kernel waits for a peer's results before it gives up (SM clock cycles)
};
// Local row r belongs to the last segment with start[s] <= r and lands at output row r + delta[s].
struct it_rowmap { int nseg; int start[4]; int delta[4]; int shift[4]; };   // shift[s]: how far segment s moves from one rank to the next
__host__ __device__ static inline int it_map_row(const it_rowmap& m, int r, int* shift = nullptr) {
    int d = 0, sh = 0;
#pragma unroll
    for (int s = 0; s < 4; s++) if (s < m.nseg && r >= m.start[s]) { d = m.delta[s]; sh = m.shift[s]; }
    if (shift) *shift = sh;
    return r + d;
}

struct it_mat {
    it_ctx* ctx;
    size_t rows, cols;      // logical shape
    size_t row_groups;      // ceil(rows / 32)
    uint8_t* tiles;         // [row_groups][cols/128][IT_TILE_BYTES]
    size_t bytes;
    bool owns_tiles;        // false for a view into a larger allocation (stacked matrices)
    bool sharded;           // rows of a larger logical matrix: results are pushed to every peer
    it_rowmap map;          // where the local rows land in the full output (identity when nseg == 0)
    size_t out_rows;        // rows of the full output (== rows unless sharded)
};

// Int8-group matrix: row-major int8 q[rows][cols] and f16 d[rows][cols/32] (Q8_0 density).
struct it_qmat {
    it_ctx* ctx;
    size_t rows, cols;
    int8_t* q;
    __half* d;                             // one f16 scale per 32 weights (Q8_0 source), or null
    float* s16;                            // one f32 scale per 16 weights (Q6_K source: d * sub-block scale), or null
    size_t bytes;
    bool sharded; size_t row0, out_rows;   // rows [row0, row0 + rows) of a logical matrix of out_rows rows (see it_mat)
};

struct it_q8 {
    it_ctx* ctx;
    size_t max_n, max_tok;
    size_t n;               // width of the rows currently held
    int8_t* qs;             // [max_tok][max_n]  (row stride max_n whatever the current width)
    float* d;               // [max_tok][max_n/256]
    int32_t* sum128;        // [max_tok][max_n/128]
    CUtensorMap tmap;       // qs as a 2-D byte tensor [rows][max_n], box 128 x 64, 128-byte swizzle (tile kernel)
};

struct it_graph { it_ctx* ctx; cudaGraph_t graph; cudaGraphExec_t exec; };

struct it_ctx {
    int device;
    cudaStream_t stream;
    float* arena;
    size_t arena_floats;
    std::map<size_t, float*> signs;   // width -> device sign vector
    // argmax scratch: per-block partial (value, index) pairs + a completion counter
    unsigned long long* argmax_partials;
    unsigned int* argmax_counter;
    int sm_count;
    bool capturing;
    // raised by a kernel whose bounded wait ran out; lives in mapped host memory so that reading it
    // costs nothing on the normal path
    int* error_flag_host;
    int* error_flag_dev;
    // words of the grid-wide barrier of persistent kernels: [0] arrivals so far, [1] arrivals at the end of the last
    // launch, [2] abort word (set by a CTA whose wait ran out; cleared by the host together with the error flag)
    unsigned* grid_sync;
    // Programmatic-dependent-launch bookkeeping: the q8 buffer whose contents are known to be complete by the
    // time the most recently enqueued kernel lets its dependents start (null after any op that is not a matvec).
    const it_q8* pdl_safe_q8;
    // peers (null / world 1 until it_ctx_attach_peers): device copy of the table, the mapped peer allocations, own flag words
    it_peers* peers_dev;
    void* peer_base[IT_MAX_PEERS];
    int rank, world;
    size_t ll_slots;
};
// The arena allocation continues with IT_ARENA_TAIL bytes of flag words ([0, IT_MAX_PEERS) arrival flags, [8] done
// counter, [9] epoch) and the low-latency exchange buffer of 2 * ll_slots 8-byte slots.
#define IT_ARENA_TAIL 256
#define IT_LL_MAX_SLOTS ((size_t)1 << 21)
// Every entry point that enqueues device work other than the ternary matvec calls this.
static inline void it_note_op(it_ctx* c) { c->pdl_safe_q8 = nullptr; }

// bytes of split-K terms per slot: enough for 8 activation rows of width 17408 (8 * 136 blocks * 32 rows * 4)
int it_check_device_error(it_ctx* ctx, const char* who);

#define IT_ARGMAX_MAX_BLOCKS 1024

// ---- programmatic dependent launch -----------------------------------------------------------------------------
// The ternary matvec and tile kernels are launched with programmatic stream serialization: their weight requests do not
// depend on the kernel before them, so they start while it still runs and wait (IT_PDL_WAIT) only in front of the first
// access to memory it may have written.  Every other kernel of the decode path triggers its dependents at once
// (IT_PDL_TRIGGER) so that a matvec behind it can start early, but is itself launched the plain way: measured, launching
// the small support kernels early made a decode step 3-9 % slower (IT_PDL_SUPPORT=1 turns it on for experiments).
// Completion is transitive: a kernel only finishes after its own wait has returned.
#define IT_PDL_TRIGGER() asm volatile("griddepcontrol.launch_dependents;" ::: "memory")
#define IT_PDL_WAIT() asm volatile("griddepcontrol.wait;" ::: "memory")
template <typename... KArgs, typename... Args>
static inline cudaError_t it_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[0].val.programmaticStreamSerializationAllowed = 1;
    static const int pdl_on = []{ const char* v = getenv("IT_PDL_SUPPORT"); return v ? atoi(v) : 0; }();
    cfg.attrs = attr; cfg.numAttrs = pdl_on ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ---- synthetic data: hash(seed, i) is the i-th output of splitmix64 seeded with `seed` (src/sampling.rs:43) ----
__host__ __device__ static inline uint64_t it_mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull; z = (z ^ (z >> 27)) * 0x94d049bb133111ebull; return z ^ (z >> 31);
}
__host__ __device__ static inline uint64_t it_hash(uint64_t seed, uint64_t i) { return it_mix64(seed + 0x9e3779b97f4a7c15ull * (i + 1)); }

// ---- launchers implemented in the kernel translation units ------------------------------------------
int it_launch_repack_pq2(it_ctx* ctx, const uint8_t* raw_dev, size_t rows, size_t cols, uint8_t* tiles);
int it_launch_repack_packed2(it_ctx* ctx, const uint32_t* words_dev, const float* scales_dev, size_t rows, size_t cols, uint8_t* tiles);
int it_launch_unpack_pq2(it_ctx* ctx, const uint8_t* tiles, size_t rows, size_t cols, uint8_t* raw_dev);
// rows [row0, row0 + rows) of the synthetic matrix with this seed and column count
int it_launch_synth_pq2(it_ctx* ctx, uint64_t seed, size_t rows, size_t cols, int four_codes, uint8_t* raw_dev, size_t row0 = 0);
// A synthetic matrix generated into caller-owned tile storage (rows must be a multiple of 32 when matrices are stacked);
// the returned it_mat is a view that does not free the tiles.
int it_matrix_synth_view(it_ctx* ctx, uint64_t seed, size_t rows, size_t cols, uint8_t* tiles, it_mat** out, size_t row0 = 0);
// A view over `row_groups` consecutive row groups starting at `tiles` (e.g. several stacked matrices seen as one).
int it_matrix_view(it_ctx* ctx, size_t rows, size_t cols, uint8_t* tiles, it_mat** out);
// Tile kernel for more than eight activation rows (it_matmul_t2.cu); same arithmetic as the matvec kernel.
int it_matmul_t2_launch(it_ctx* ctx, const it_mat* w, int ntok, const it_q8* x, float* y, size_t y_stride, int accum);
// tcgen05 version of the tile kernel (it_matmul_tc.cu); returns a positive value when the shape does not fit it.
int it_matmul_tc_launch(it_ctx* ctx, const it_mat* w, int ntok, const it_q8* x, float* y, size_t y_stride, int accum);
int it_launch_synth_q8_0(it_ctx* ctx, uint64_t seed, size_t rows, size_t cols, int8_t* q, __half* d, size_t row0 = 0);
