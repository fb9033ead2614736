// Greedy argmax over the logits and the int8-group matvec of the MTP head.
#include "it_internal.h"
#include "it_pipe.cuh"

namespace {

// ---------------------------------------------------------------- argmax
// First index of the maximum (src/sampling.rs:50: strict '>' scan from index 0; shaders/argmax.comp:
// ties resolve to the lowest index).  Two levels: every CTA scans a contiguous slice and publishes
// its (value, index); the CTA that finishes last folds the partials and resets the counter, so the
// scratch is ready for the next launch.  NaN never wins a comparison, as in the reference shader.
// Algorithmic traffic: 4n bytes.
struct Pick { float v; unsigned i; };
__device__ __forceinline__ Pick pick_better(Pick a, Pick b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }
__device__ __forceinline__ unsigned long long pick_pack(Pick p) { return ((unsigned long long)__float_as_uint(p.v) << 32) | p.i; }
__device__ __forceinline__ Pick pick_unpack(unsigned long long u) { return Pick{ __uint_as_float((unsigned)(u >> 32)), (unsigned)u }; }

__device__ __forceinline__ Pick block_reduce(Pick p, Pick* sh) {
    const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (unsigned m = 16; m > 0; m >>= 1) { Pick o{ __shfl_xor_sync(0xffffffffu, p.v, m), __shfl_xor_sync(0xffffffffu, p.i, m) }; p = pick_better(p, o); }
    if (lane == 0) sh[warp] = p;
    __syncthreads();
    if (warp == 0) {
        p = lane < (blockDim.x >> 5) ? sh[lane] : Pick{ -INFINITY, 0xffffffffu };
#pragma unroll
        for (unsigned m = 16; m > 0; m >>= 1) { Pick o{ __shfl_xor_sync(0xffffffffu, p.v, m), __shfl_xor_sync(0xffffffffu, p.i, m) }; p = pick_better(p, o); }
    }
    return p;   // valid in warp 0
}

__global__ void __launch_bounds__(256)
k_argmax(const float* __restrict__ v, unsigned n, unsigned per_block, unsigned long long* partials, unsigned* counter, float* dst) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    __shared__ Pick sh[8];
    __shared__ bool is_last;
    const unsigned begin = blockIdx.x * per_block, end = min(n, begin + per_block);   // per_block % 4 == 0
    Pick p{ -INFINITY, 0xffffffffu };
    for (unsigned i = begin + 4 * threadIdx.x; i < end; i += 4 * blockDim.x) {
        if (i + 4 <= end) {
            float4 x = *reinterpret_cast<const float4*>(v + i);
            p = pick_better(p, Pick{ x.x, i }); p = pick_better(p, Pick{ x.y, i + 1 }); p = pick_better(p, Pick{ x.z, i + 2 }); p = pick_better(p, Pick{ x.w, i + 3 });
        } else {
            for (unsigned k = i; k < end; k++) p = pick_better(p, Pick{ v[k], k });
        }
    }
    p = block_reduce(p, sh);
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = pick_pack(p);
        __threadfence();
        is_last = atomicAdd(counter, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    Pick q{ -INFINITY, 0xffffffffu };
    for (unsigned b = threadIdx.x; b < gridDim.x; b += blockDim.x) q = pick_better(q, pick_unpack(__ldcg(partials + b)));
    __syncthreads();
    q = block_reduce(q, sh);
    if (threadIdx.x == 0) { *dst = __uint_as_float(q.i == 0xffffffffu ? 0u : q.i); *counter = 0; }
}

// ---------------------------------------------------------------- int8-group matvec (f32 activations)
// y[t, r] (+)= sum_g d[r, g/2] * (sum_{j<16} q[r,16g+j] * x[t,16g+j])   (src/quant.rs:266-270, shaders/matvec_q8.comp)
// One warp per four rows: a lane takes 16 weights of each row per step (one 128-bit load per row) and
// reuses its 16 activations for the four rows.  HBM-bound: rows*cols*(1 + 2/32) bytes of weights (Q8_0 source: one f16
// scale per 32 weights) or rows*cols*(1 + 4/16) (G16, Q6_K source: one f32 scale per 16 weights).
constexpr int QROWS = 4;
// Byte k of w (bytes already offset by 128: w = raw ^ 0x80808080) as a float, exactly: the byte becomes the low mantissa
// bits of 2^23, and 2^23 + 128 is subtracted.  One permute and one addition on the main pipes instead of a shift and an
// integer-to-float conversion, which shares the slow special-function pipe (72 % busy in this kernel before the change).
__device__ __forceinline__ float q8_to_float(uint32_t w_off, int k) {
    return __fadd_rn(__uint_as_float(__byte_perm(w_off, 0x4B000000u, 0x7650u + (unsigned)k)), -8388736.0f);
}
template <int NT, bool G16>
__global__ void __launch_bounds__(256)
k_matvec_q8(const int8_t* __restrict__ wq, const __half* __restrict__ wd, const float* __restrict__ ws, int rows, int cols,
            const float* x, size_t x_stride, float* arena, size_t y_off, size_t y_stride, int ntok, int accum,
            const it_peers* peers, int row_off, int* error_flag) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r0 = (blockIdx.x * 8 + warp) * QROWS;
    const int groups = r0 < rows ? cols / 16 : 0;      // warps past the last row only take part in the end-of-kernel handshake
    float acc[QROWS][NT];
#pragma unroll
    for (int r = 0; r < QROWS; r++)
#pragma unroll
        for (int t = 0; t < NT; t++) acc[r][t] = 0.f;
    // the weights and scales of the next group are requested before this group's arithmetic starts: twice the bytes in flight
    uint4 wn[QROWS]; float dn[QROWS];
    auto fetch = [&](int g) {
#pragma unroll
        for (int r = 0; r < QROWS; r++) {
            const int row = min(r0 + r, rows - 1);
            asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(wn[r].x), "=r"(wn[r].y), "=r"(wn[r].z), "=r"(wn[r].w)
                         : "l"(wq + (size_t)row * cols + 16 * g));
            dn[r] = G16 ? ws[(size_t)row * (cols / 16) + g] : __half2float(wd[(size_t)row * (cols / 32) + (g >> 1)]);
        }
    };
    if (lane < groups) fetch(lane);
    for (int g = lane; g < groups; g += 32) {
        uint4 w[QROWS]; float d[QROWS];
#pragma unroll
        for (int r = 0; r < QROWS; r++) { w[r] = wn[r]; d[r] = dn[r]; }
        if (g + 32 < groups) fetch(g + 32);
#pragma unroll
        for (int t = 0; t < NT; t++) {
            if (t < ntok) {
                const float4* xp = reinterpret_cast<const float4*>(x + t * x_stride + 16 * g);
                const float4 x0 = xp[0], x1 = xp[1], x2 = xp[2], x3 = xp[3];
                const float xv[16] = { x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w, x2.x, x2.y, x2.z, x2.w, x3.x, x3.y, x3.z, x3.w };
#pragma unroll
                for (int r = 0; r < QROWS; r++) {
                    const uint32_t ww[4] = { w[r].x ^ 0x80808080u, w[r].y ^ 0x80808080u, w[r].z ^ 0x80808080u, w[r].w ^ 0x80808080u };
                    float s = 0.f;
#pragma unroll
                    for (int k = 0; k < 16; k++) s = fmaf(q8_to_float(ww[k >> 2], k & 3), xv[k], s);
                    acc[r][t] = fmaf(s, d[r], acc[r][t]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < QROWS; r++)
#pragma unroll
        for (int t = 0; t < NT; t++) {
            float s = acc[r][t];
#pragma unroll
            for (unsigned m = 16; m > 0; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
            if (lane == 0 && t < ntok && r0 + r < rows) {
                // a row shard writes at its rows' place in the full output, into every rank's arena (the old value of an
                // accumulating call is added with a plain f32 addition, as before)
                const size_t off = y_off + t * y_stride + row_off + r0 + r;
                if (accum) s = arena[off] + s;
                it_result_store(peers, arena, off, s, 0);
            }
        }
    if (peers) {
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) it_shard_finish(peers, gridDim.x, error_flag);
    }
}

}  // namespace

IT_API int it_argmax(it_ctx* c, size_t logits_off, size_t n, size_t dst_off) {
    IT_CHECK_ARG(c, "it_argmax: null context");
    IT_CHECK_ARG(n > 0 && n < 0xffffffffull, "it_argmax: bad length %zu", n);
    IT_CHECK_ARG(logits_off % 4 == 0, "it_argmax: logits offset must be 4-float aligned");
    IT_CHECK_ARG(logits_off <= c->arena_floats && n <= c->arena_floats - logits_off && dst_off < c->arena_floats, "it_argmax: range outside the arena");
    IT_CHECK_ARG(dst_off < logits_off || dst_off >= logits_off + n, "it_argmax: the result slot overlaps the logits");
    it_note_op(c);
    unsigned blocks = (unsigned)((n + 4095) / 4096);
    const unsigned cap = (unsigned)(c->sm_count * 2 < IT_ARGMAX_MAX_BLOCKS ? c->sm_count * 2 : IT_ARGMAX_MAX_BLOCKS);
    if (blocks > cap) blocks = cap;
    unsigned per_block = (unsigned)((n + blocks - 1) / blocks); per_block = (per_block + 3) & ~3u;
    blocks = (unsigned)((n + per_block - 1) / per_block);
    it_pdl(k_argmax, dim3(blocks), dim3(256), 0, c->stream, c->arena + logits_off, (unsigned)n, per_block, c->argmax_partials, c->argmax_counter, c->arena + dst_off);
    IT_LAUNCH_CHECK("argmax");
    return IT_OK;
}

IT_API int it_matvec_q8(it_ctx* c, const it_qmat* w, size_t ntok, size_t x_off, size_t x_stride, size_t y_off, size_t y_stride, int accum) {
    IT_CHECK_ARG(c && w, "it_matvec_q8: null argument");
    IT_CHECK_ARG(w->ctx == c, "it_matvec_q8: matrix belongs to another context");
    IT_CHECK_ARG(ntok > 0 && ntok <= 65535, "it_matvec_q8: bad row count %zu", ntok);
    IT_CHECK_ARG(x_off % 4 == 0 && (ntok == 1 || x_stride % 4 == 0), "it_matvec_q8: activation offsets must be 4-float aligned");
    IT_CHECK_ARG(x_off <= c->arena_floats && (ntok - 1) * x_stride + w->cols <= c->arena_floats - x_off, "it_matvec_q8: input rows fall outside the arena");
    IT_CHECK_ARG(ntok == 1 || y_stride >= w->out_rows, "it_matvec_q8: output stride shorter than a row of results");
    IT_CHECK_ARG(y_off <= c->arena_floats && (ntok - 1) * y_stride + w->out_rows <= c->arena_floats - y_off, "it_matvec_q8: output rows fall outside the arena");
    if (w->sharded && !c->peers_dev) return it_fail(IT_ESTATE, "it_matvec_q8: the matrix is a row shard but no peers are attached to the context");
    it_note_op(c);
    const unsigned grid = (unsigned)((w->rows + 8 * QROWS - 1) / (8 * QROWS));
    const it_peers* peers = w->sharded ? c->peers_dev : nullptr;
    for (size_t t0 = 0; t0 < ntok; t0 += 4) {
        const int nt = (int)((ntok - t0) < 4 ? (ntok - t0) : 4);
        const float* x = c->arena + x_off + t0 * x_stride; const size_t yo = y_off + t0 * y_stride;
#define IT_Q8_LAUNCH(NT, G) it_pdl(k_matvec_q8<NT, G>, dim3(grid), dim3(256), 0, c->stream, w->q, w->d, w->s16, (int)w->rows, (int)w->cols, x, x_stride, c->arena, yo, y_stride, nt, accum, peers, (int)w->row0, c->error_flag_dev)
        if (w->s16) { if (nt == 1) IT_Q8_LAUNCH(1, true); else if (nt == 2) IT_Q8_LAUNCH(2, true); else IT_Q8_LAUNCH(4, true); }
        else { if (nt == 1) IT_Q8_LAUNCH(1, false); else if (nt == 2) IT_Q8_LAUNCH(2, false); else IT_Q8_LAUNCH(4, false); }
#undef IT_Q8_LAUNCH
        IT_LAUNCH_CHECK("matvec_q8");
    }
    return IT_OK;
}

// ---------------------------------------------------------------- argmax without any allocation
// Scratch of it_argmax_static: the per-CTA (value, index) partials followed by the arrival counter.  It is
// part of the library image, so every GPU that loads the library carries these bytes until the process ends.
#define IT_ARGMAX_STATIC_MAX_N (1u << 24)
#define IT_ARGMAX_STATIC_MAX_DEVICES 64
static __device__ __align__(256) unsigned long long g_argmax_static_scratch[IT_ARGMAX_MAX_BLOCKS + 32];
// Device address of the array above, one per GPU.  The array's name is only a host-side handle in host code;
// the address a kernel can use has to be asked for, on each device, with that device current.
static unsigned long long* g_argmax_static_ptr[IT_ARGMAX_STATIC_MAX_DEVICES] = {};
static int g_argmax_static_sms[IT_ARGMAX_STATIC_MAX_DEVICES] = {};

IT_API int it_argmax_static(void* stream, const float* logits_dev, size_t n, uint32_t* index_dev) {
    IT_CHECK_ARG(logits_dev && index_dev, "it_argmax_static: null pointer");
    IT_CHECK_ARG(((uintptr_t)logits_dev & 15) == 0 && ((uintptr_t)index_dev & 3) == 0, "it_argmax_static: logits must be 16-byte aligned, the result 4-byte aligned");
    IT_CHECK_ARG(n > 0, "it_argmax_static: empty input");
    IT_CHECK_ARG(n <= IT_ARGMAX_STATIC_MAX_N, "it_argmax_static: %zu logits exceed the built-in scratch limit of %u", n, IT_ARGMAX_STATIC_MAX_N);
    int dev = -1;
    IT_CUDA(cudaGetDevice(&dev));
    IT_CHECK_ARG(dev >= 0 && dev < IT_ARGMAX_STATIC_MAX_DEVICES, "it_argmax_static: device index %d not supported", dev);
    if (!g_argmax_static_ptr[dev]) {
        // first call on this device: resolve the scratch address and the SM count (no allocation involved)
        unsigned long long* p = nullptr;
        IT_CUDA(cudaGetSymbolAddress((void**)&p, g_argmax_static_scratch));
        int sms = 0;
        IT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        g_argmax_static_sms[dev] = sms;
        g_argmax_static_ptr[dev] = p;
    }
    unsigned long long* partials = g_argmax_static_ptr[dev];
    unsigned* counter = reinterpret_cast<unsigned*>(partials + IT_ARGMAX_MAX_BLOCKS);
    cudaStream_t st = (cudaStream_t)stream;
    {   // the scratch resolved above belongs to the current device: a stream of another GPU is refused here, not at the launch
        int sdev = dev;
        if (st && st != cudaStreamLegacy && st != cudaStreamPerThread && cudaStreamGetDevice(st, &sdev) != cudaSuccess) { cudaGetLastError(); sdev = dev; }
        IT_CHECK_ARG(sdev == dev, "it_argmax_static: the stream belongs to device %d but device %d is current", sdev, dev);
    }
    // the counter must start at zero; the kernel leaves it at zero, but a launch that failed earlier may not have
    IT_CUDA(cudaMemsetAsync(counter, 0, sizeof(unsigned), st));
    unsigned blocks = (unsigned)((n + 4095) / 4096);
    const unsigned cap = (unsigned)(g_argmax_static_sms[dev] * 2 < IT_ARGMAX_MAX_BLOCKS ? g_argmax_static_sms[dev] * 2 : IT_ARGMAX_MAX_BLOCKS);
    if (blocks > cap) blocks = cap;
    unsigned per_block = (unsigned)((n + blocks - 1) / blocks); per_block = (per_block + 3) & ~3u;
    blocks = (unsigned)((n + per_block - 1) / per_block);
    k_argmax<<<blocks, 256, 0, st>>>(logits_dev, (unsigned)n, per_block, partials, counter, reinterpret_cast<float*>(index_dev));
    IT_LAUNCH_CHECK("argmax_static");
    return IT_OK;
}
