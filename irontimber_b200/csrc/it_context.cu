// Context, arena, weight upload / repack and q8 activation buffers of libirontimber_cuda.so.
#include "it_internal.h"
#include <cstddef>
#include <cstring>
#include <vector>

static thread_local char g_err[512] = "";

int it_fail(int code, const char* fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(g_err, sizeof g_err, fmt, ap); va_end(ap);
    return code;
}
IT_API const char* it_last_error(void) { return g_err; }
IT_API int it_version(void) { return 1; }

// ---------------------------------------------------------------- synthetic data rule
// hash(seed, i) is the i-th output of splitmix64 seeded with `seed` (the reference's RNG family,
// src/sampling.rs:43).  Codes: one hash per two elements, 32 bits each, code = v % 3 (or v % 4).
// Scales: u = top 24 bits of hash(seed ^ 0x5ca1e5, block) / 2^24, d = f16(0.01 + 0.04*u) with
// separately rounded multiply and add.
__global__ void k_synth_pq2(uint64_t seed, size_t rows, size_t cols, int four, uint8_t* raw, size_t row0) {
    size_t bpr = cols / 128, nblk = rows * bpr;
    for (size_t lblk = blockIdx.x * (size_t)blockDim.x + threadIdx.x; lblk < nblk; lblk += (size_t)gridDim.x * blockDim.x) {
        unsigned short* o = reinterpret_cast<unsigned short*>(raw + lblk * 34);   // 34-byte blocks are 2-byte aligned
        const size_t blk = lblk + row0 * bpr;                                     // block index in the full matrix
        const uint64_t hs = it_hash(seed ^ 0x5ca1e5ull, blk);
        const float u = __fmul_rn((float)(uint32_t)(hs >> 40), 1.0f / 16777216.0f);
        o[0] = __half_as_ushort(__float2half_rn(__fadd_rn(0.01f, __fmul_rn(0.04f, u))));
        size_t e0 = blk * 128;   // global element index of the block's first element (row-major)
        for (int q = 0; q < 16; q++) {   // 8 elements = 2 code bytes per step
            uint32_t packed = 0;
            for (int p = 0; p < 4; p++) {
                const uint64_t h = it_hash(seed, (e0 + 8 * q) / 2 + p);
                const uint32_t lo = (uint32_t)h, hi = (uint32_t)(h >> 32);
                packed |= (four ? (lo & 3u) : (lo % 3u)) << (4 * p);
                packed |= (four ? (hi & 3u) : (hi % 3u)) << (4 * p + 2);
            }
            o[1 + q] = (unsigned short)packed;
        }
    }
}
int it_launch_synth_pq2(it_ctx* ctx, uint64_t seed, size_t rows, size_t cols, int four_codes, uint8_t* raw_dev, size_t row0) {
    k_synth_pq2<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(seed, rows, cols, four_codes, raw_dev, row0);
    IT_LAUNCH_CHECK("synth_pq2"); return IT_OK;
}

// Q8_0 synthetic rule: q = (hash(seed, e/2) 32-bit half) % 255 - 127, d = f16(0.002 + 0.004*u) per 32-block.
__global__ void k_synth_q8_0(uint64_t seed, size_t rows, size_t cols, int8_t* q, __half* d, size_t row0) {
    size_t n = rows * cols;
    for (size_t lp = blockIdx.x * (size_t)blockDim.x + threadIdx.x; lp < n / 2; lp += (size_t)gridDim.x * blockDim.x) {
        const size_t p = lp + row0 * cols / 2;            // pair index in the full matrix (cols is a multiple of 32)
        uint64_t h = it_hash(seed, p);
        q[2 * lp] = (int8_t)((int)((uint32_t)h % 255u) - 127);
        q[2 * lp + 1] = (int8_t)((int)((uint32_t)(h >> 32) % 255u) - 127);
        if (p % 16 == 0) {
            float u = (float)(it_hash(seed ^ 0x5ca1e5ull, p / 16) >> 40) * (1.0f / 16777216.0f);
            d[lp / 16] = __float2half_rn(__fadd_rn(0.002f, __fmul_rn(0.004f, u)));
        }
    }
}
int it_launch_synth_q8_0(it_ctx* ctx, uint64_t seed, size_t rows, size_t cols, int8_t* q, __half* d, size_t row0) {
    k_synth_q8_0<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(seed, rows, cols, q, d, row0);
    IT_LAUNCH_CHECK("synth_q8_0"); return IT_OK;
}

// ---------------------------------------------------------------- PQ2_0 <-> tile layout
// One thread per 32-bit code word of the tile layout (see it_internal.h).
__global__ void k_repack_pq2(const uint8_t* __restrict__ raw, size_t rows, size_t cols, uint8_t* __restrict__ tiles) {
    size_t nb = cols / 128, rgs = (rows + 31) / 32;
    size_t nwords = rgs * nb * 256;   // 8 words per lane, 32 lanes
    for (size_t w = blockIdx.x * (size_t)blockDim.x + threadIdx.x; w < nwords; w += (size_t)gridDim.x * blockDim.x) {
        size_t tile = w / 256; int r = (int)(w % 256);
        int half = r / 128, lane = (r % 128) / 4, slot = r % 4;     // byte offset = 512*half + 16*lane + 4*slot
        int j = half * 2 + slot / 2, h = slot % 2, g = lane >> 2, t = lane & 3;
        size_t rg = tile / nb, b = tile % nb;
        uint32_t word = 0;
        for (int i = 0; i < 4; i++) {
            size_t row = rg * 32 + g + 8 * i;
            if (row >= rows) { word |= 0x01010101u << (2 * i); continue; }   // padding rows decode to 0
            const uint8_t* qs = raw + (row * nb + b) * 34 + 2;
            int k0 = 32 * t + 8 * j + 4 * h;                                   // k0 % 4 == 0: one source byte
            uint32_t src = qs[k0 / 4];
            for (int c = 0; c < 4; c++) word |= ((src >> (2 * c)) & 3u) << (8 * c + 2 * i);
        }
        *(uint32_t*)(tiles + tile * IT_TILE_BYTES + 512 * half + 16 * lane + 4 * slot) = word;
        if (r < 32) {   // 32 threads of the tile also copy the 32 scales
            int gg = r >> 2, ii = r & 3; size_t row = rg * 32 + gg + 8 * ii;
            unsigned short sb = 0;
            if (row < rows) { const uint8_t* blk = raw + (row * nb + b) * 34; sb = (unsigned short)(blk[0] | (blk[1] << 8)); }
            *(unsigned short*)(tiles + tile * IT_TILE_BYTES + 1024 + 8 * gg + 2 * ii) = sb;
        }
    }
}
int it_launch_repack_pq2(it_ctx* ctx, const uint8_t* raw_dev, size_t rows, size_t cols, uint8_t* tiles) {
    k_repack_pq2<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(raw_dev, rows, cols, tiles);
    IT_LAUNCH_CHECK("repack_pq2"); return IT_OK;
}

// One thread per raw PQ2_0 block: gathers its 128 codes back out of the tile layout.
__global__ void k_unpack_pq2(const uint8_t* __restrict__ tiles, size_t rows, size_t cols, uint8_t* __restrict__ raw) {
    size_t nb = cols / 128, nblk = rows * nb;
    for (size_t blk = blockIdx.x * (size_t)blockDim.x + threadIdx.x; blk < nblk; blk += (size_t)gridDim.x * blockDim.x) {
        size_t row = blk / nb, b = blk % nb, rg = row / 32; int rr = (int)(row % 32), g = rr % 8, i = rr / 8;
        const uint8_t* tile = tiles + (rg * nb + b) * IT_TILE_BYTES;
        uint8_t* o = raw + blk * 34;
        unsigned short sb = *(const unsigned short*)(tile + 1024 + 8 * g + 2 * i);
        o[0] = (uint8_t)(sb & 0xff); o[1] = (uint8_t)(sb >> 8);
        for (int q = 0; q < 32; q++) {          // source byte q holds columns 4q..4q+3
            int k0 = 4 * q, t = k0 / 32, j = (k0 % 32) / 8, h = (k0 % 8) / 4, lane = 4 * g + t;
            uint32_t word = *(const uint32_t*)(tile + 512 * (j / 2) + 16 * lane + 4 * ((j % 2) * 2 + h));
            uint8_t byte = 0;
            for (int c = 0; c < 4; c++) byte |= (uint8_t)(((word >> (8 * c + 2 * i)) & 3u) << (2 * c));
            o[2 + q] = byte;
        }
    }
}
int it_launch_unpack_pq2(it_ctx* ctx, const uint8_t* tiles, size_t rows, size_t cols, uint8_t* raw_dev) {
    k_unpack_pq2<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(tiles, rows, cols, raw_dev);
    IT_LAUNCH_CHECK("unpack_pq2"); return IT_OK;
}

// ---------------------------------------------------------------- context
IT_API int it_ctx_create(int device, size_t arena_floats, it_ctx** out) {
    IT_CHECK_ARG(out != nullptr, "it_ctx_create: out is null");
    *out = nullptr;
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0) return it_fail(IT_ECUDA, "no CUDA device is visible: %s", cudaGetErrorString(e));
    IT_CHECK_ARG(device >= 0 && device < ndev, "it_ctx_create: device %d out of range (%d visible)", device, ndev);
    IT_CHECK_ARG(arena_floats > 0 && arena_floats % 64 == 0, "it_ctx_create: arena size must be a positive multiple of 64 floats");
    IT_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop; IT_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return it_fail(IT_ESTATE, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
    it_ctx* c = new it_ctx(); c->device = device; c->arena = nullptr; c->arena_floats = arena_floats; c->sm_count = prop.multiProcessorCount;
    c->argmax_partials = nullptr; c->argmax_counter = nullptr; c->stream = nullptr; c->capturing = false;
    c->peers_dev = nullptr; c->rank = 0; c->world = 1; for (int i = 0; i < IT_MAX_PEERS; i++) c->peer_base[i] = nullptr;
    c->pdl_safe_q8 = nullptr; c->error_flag_host = nullptr; c->error_flag_dev = nullptr; c->grid_sync = nullptr;
    cudaError_t e1 = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    c->ll_slots = arena_floats < IT_LL_MAX_SLOTS ? arena_floats : IT_LL_MAX_SLOTS;
    const size_t arena_bytes = arena_floats * sizeof(float) + IT_ARENA_TAIL + 2 * c->ll_slots * 8;
    cudaError_t e2 = e1 == cudaSuccess ? cudaMalloc(&c->arena, arena_bytes) : e1;
    cudaError_t e3 = e2 == cudaSuccess ? cudaMalloc(&c->argmax_partials, IT_ARGMAX_MAX_BLOCKS * sizeof(unsigned long long)) : e2;
    cudaError_t e4 = e3 == cudaSuccess ? cudaMalloc(&c->argmax_counter, 256) : e3;
    if (e4 == cudaSuccess) e4 = cudaMalloc(&c->grid_sync, 256);
    if (e4 == cudaSuccess) e4 = cudaMemsetAsync(c->grid_sync, 0, 256, c->stream);
    if (e4 == cudaSuccess) e4 = cudaHostAlloc(&c->error_flag_host, sizeof(int), cudaHostAllocMapped);
    if (e4 == cudaSuccess) { *c->error_flag_host = 0; e4 = cudaHostGetDevicePointer(&c->error_flag_dev, c->error_flag_host, 0); }
    if (e4 != cudaSuccess) { it_ctx_destroy(c); return it_fail(e4 == cudaErrorMemoryAllocation ? IT_ENOMEM : IT_ECUDA, "it_ctx_create: %s", cudaGetErrorString(e4)); }
    cudaMemsetAsync(c->arena, 0, arena_bytes, c->stream);
    cudaMemsetAsync(c->argmax_counter, 0, 256, c->stream);
    IT_CUDA(cudaStreamSynchronize(c->stream));
    *out = c; return IT_OK;
}
IT_API void it_ctx_destroy(it_ctx* c) {
    if (!c) return;
    cudaSetDevice(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    for (int i = 0; i < IT_MAX_PEERS; i++) if (c->peer_base[i]) cudaIpcCloseMemHandle(c->peer_base[i]);
    if (c->peers_dev) cudaFree(c->peers_dev);
    for (auto& kv : c->signs) cudaFree(kv.second);
    if (c->error_flag_host) cudaFreeHost(c->error_flag_host);
    if (c->grid_sync) cudaFree(c->grid_sync);
    if (c->argmax_counter) cudaFree(c->argmax_counter);
    if (c->argmax_partials) cudaFree(c->argmax_partials);
    if (c->arena) cudaFree(c->arena);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
}
// ---------------------------------------------------------------- peers (one process per GPU)
IT_API int it_ctx_ipc_handle(it_ctx* c, void* handle64) {
    IT_CHECK_ARG(c && handle64, "it_ctx_ipc_handle: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are exchanged as 64-byte blobs");
    IT_CUDA(cudaSetDevice(c->device));
    IT_CUDA(cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle64), c->arena));
    return IT_OK;
}
// Common part of the two attach calls: bases[p] is rank p's arena allocation as this process sees it (own arena at [rank]).
static int attach_common(it_ctx* c, int rank, int world, char* const* bases) {
    it_peers P; memset(&P, 0, sizeof P);
    P.rank = rank; P.world = world;
    const size_t tail = c->arena_floats * sizeof(float);
    for (int p = 0; p < world; p++) {
        P.arena[p] = reinterpret_cast<float*>(bases[p]);
        P.flags[p] = reinterpret_cast<unsigned*>(bases[p] + tail);
        P.ll[p] = reinterpret_cast<unsigned long long*>(bases[p] + tail + IT_ARENA_TAIL);
    }
    P.ll_slots = c->ll_slots;
    P.wait_clocks = 1ll << 33;             // about four seconds: another process may be a little behind
    P.done = P.flags[rank] + IT_MAX_PEERS; P.epoch = P.flags[rank] + IT_MAX_PEERS + 1;
    IT_CUDA(cudaMalloc(&c->peers_dev, sizeof P));
    IT_CUDA(cudaMemcpyAsync(c->peers_dev, &P, sizeof P, cudaMemcpyHostToDevice, c->stream));
    IT_CUDA(cudaStreamSynchronize(c->stream));
    c->rank = rank; c->world = world;
    return IT_OK;
}
IT_API int it_ctx_attach_peers(it_ctx* c, int rank, int world, const void* handles) {
    IT_CHECK_ARG(c && handles, "it_ctx_attach_peers: null argument");
    IT_CHECK_ARG(world >= 1 && world <= IT_MAX_PEERS && rank >= 0 && rank < world, "it_ctx_attach_peers: bad rank %d of %d", rank, world);
    if (c->peers_dev) return it_fail(IT_ESTATE, "it_ctx_attach_peers: peers are already attached");
    if (c->capturing) return it_fail(IT_ESTATE, "it_ctx_attach_peers: not allowed while recording a graph");
    IT_CUDA(cudaSetDevice(c->device));
    char* bases[IT_MAX_PEERS] = {};
    for (int p = 0; p < world; p++) {
        bases[p] = reinterpret_cast<char*>(c->arena);
        if (p != rank) {
            cudaIpcMemHandle_t h; memcpy(&h, static_cast<const char*>(handles) + 64 * p, 64);
            void* mapped = nullptr;
            cudaError_t e = cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) {
                for (int q = 0; q < p; q++) if (c->peer_base[q]) { cudaIpcCloseMemHandle(c->peer_base[q]); c->peer_base[q] = nullptr; }
                return it_fail(IT_ECUDA, "it_ctx_attach_peers: cannot map the arena of rank %d: %s", p, cudaGetErrorString(e));
            }
            c->peer_base[p] = mapped; bases[p] = static_cast<char*>(mapped);
        }
    }
    return attach_common(c, rank, world, bases);
}
// The same for contexts that live in ONE process (a single-process host that drives several GPUs, or two contexts on one
// GPU): the arenas are addressed directly, with peer access enabled between different devices.
IT_API int it_ctx_attach_peers_local(it_ctx* c, int rank, int world, it_ctx* const* all) {
    IT_CHECK_ARG(c && all, "it_ctx_attach_peers_local: null argument");
    IT_CHECK_ARG(world >= 1 && world <= IT_MAX_PEERS && rank >= 0 && rank < world, "it_ctx_attach_peers_local: bad rank %d of %d", rank, world);
    if (c->peers_dev) return it_fail(IT_ESTATE, "it_ctx_attach_peers_local: peers are already attached");
    if (c->capturing) return it_fail(IT_ESTATE, "it_ctx_attach_peers_local: not allowed while recording a graph");
    IT_CUDA(cudaSetDevice(c->device));
    char* bases[IT_MAX_PEERS] = {};
    for (int p = 0; p < world; p++) {
        it_ctx* o = p == rank ? c : all[p];
        IT_CHECK_ARG(o && o->arena_floats == c->arena_floats, "it_ctx_attach_peers_local: rank %d has no context or an arena of another size", p);
        if (o->device != c->device) {
            int can = 0; IT_CUDA(cudaDeviceCanAccessPeer(&can, c->device, o->device));
            if (!can) return it_fail(IT_ECUDA, "it_ctx_attach_peers_local: device %d cannot address the memory of device %d", c->device, o->device);
            const cudaError_t e = cudaDeviceEnablePeerAccess(o->device, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return it_fail(IT_ECUDA, "it_ctx_attach_peers_local: %s", cudaGetErrorString(e));
            cudaGetLastError();
        }
        bases[p] = reinterpret_cast<char*>(o->arena);
    }
    return attach_common(c, rank, world, bases);
}
// How long a kernel of this context waits for a peer's results before it gives up and raises IT_ETIMEOUT (default about
// four seconds).  For tests and for hosts that want to notice a lost peer sooner.
IT_API int it_ctx_set_peer_wait_us(it_ctx* c, double microseconds) {
    IT_CHECK_ARG(c && microseconds > 0.0 && microseconds <= 60e6, "it_ctx_set_peer_wait_us: bad argument");
    if (!c->peers_dev) return it_fail(IT_ESTATE, "it_ctx_set_peer_wait_us: no peers are attached");
    if (c->capturing) return it_fail(IT_ESTATE, "it_ctx_set_peer_wait_us: not allowed while recording a graph");
    IT_CUDA(cudaSetDevice(c->device));
    int khz = 0; IT_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, c->device));
    const long long clocks = (long long)(microseconds * 1e-3 * (double)khz) + 1;
    IT_CUDA(cudaStreamSynchronize(c->stream));
    IT_CUDA(cudaMemcpy(reinterpret_cast<char*>(c->peers_dev) + offsetof(it_peers, wait_clocks), &clocks, sizeof clocks, cudaMemcpyHostToDevice));
    return IT_OK;
}
IT_API int it_ctx_world(const it_ctx* c) { return c ? c->world : 0; }

IT_API int it_sync(it_ctx* c) {
    IT_CHECK_ARG(c, "it_sync: null context");
    if (c->capturing) return it_fail(IT_ESTATE, "it_sync: not allowed while recording a graph");
    IT_CUDA(cudaStreamSynchronize(c->stream));
    return it_check_device_error(c, "it_sync");
}
// After a synchronisation: reports (and clears) the flag a kernel raises when a bounded wait ran out.
int it_check_device_error(it_ctx* c, const char* who) {
    if (c->error_flag_host && *(volatile int*)c->error_flag_host) {
        const int code = *(volatile int*)c->error_flag_host;
        *(volatile int*)c->error_flag_host = 0;
        // a persistent kernel that gave up leaves its barrier words inconsistent and the abort word set
        if (c->grid_sync && !c->capturing) { cudaMemsetAsync(c->grid_sync, 0, 256, c->stream); cudaStreamSynchronize(c->stream); }
        return it_fail(IT_ETIMEOUT, "%s: a kernel gave up on a bounded wait (site %d); its results are not valid", who, code);
    }
    return IT_OK;
}
IT_API int it_capture_begin(it_ctx* c) {
    IT_CHECK_ARG(c, "it_capture_begin: null context");
    if (c->capturing) return it_fail(IT_ESTATE, "it_capture_begin: already recording");
    IT_CUDA(cudaSetDevice(c->device));
    it_note_op(c);
    IT_CUDA(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    c->capturing = true; return IT_OK;
}
IT_API int it_capture_end(it_ctx* c, it_graph** out) {
    IT_CHECK_ARG(c && out, "it_capture_end: null argument");
    *out = nullptr;
    if (!c->capturing) return it_fail(IT_ESTATE, "it_capture_end: not recording");
    c->capturing = false; it_note_op(c);
    cudaGraph_t g = nullptr;
    IT_CUDA(cudaStreamEndCapture(c->stream, &g));
    cudaGraphExec_t ex = nullptr;
    cudaError_t e = cudaGraphInstantiate(&ex, g, 0);
    if (e != cudaSuccess) { cudaGraphDestroy(g); return it_fail(IT_ECUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e)); }
    it_graph* r = new it_graph(); r->ctx = c; r->graph = g; r->exec = ex; *out = r; return IT_OK;
}
IT_API int it_graph_launch(it_ctx* c, it_graph* g) {
    IT_CHECK_ARG(c && g && g->ctx == c, "it_graph_launch: null argument or foreign graph");
    it_note_op(c);
    IT_CUDA(cudaGraphLaunch(g->exec, c->stream)); return IT_OK;
}
IT_API int it_graph_kernel_nodes(const it_graph* g) {
    if (!g) return it_fail(IT_EINVAL, "it_graph_kernel_nodes: null graph");
    size_t n = 0;
    IT_CUDA(cudaGraphGetNodes(g->graph, nullptr, &n));
    std::vector<cudaGraphNode_t> nodes(n);
    if (n) IT_CUDA(cudaGraphGetNodes(g->graph, nodes.data(), &n));
    int kernels = 0;
    for (size_t i = 0; i < n; i++) { cudaGraphNodeType t; IT_CUDA(cudaGraphNodeGetType(nodes[i], &t)); if (t == cudaGraphNodeTypeKernel) kernels++; }
    return kernels;
}
IT_API void it_graph_destroy(it_graph* g) { if (!g) return; cudaSetDevice(g->ctx->device); cudaGraphExecDestroy(g->exec); cudaGraphDestroy(g->graph); delete g; }
IT_API void* it_ctx_stream(it_ctx* c) { return c ? (void*)c->stream : nullptr; }
IT_API float* it_arena_ptr(it_ctx* c) { return c ? c->arena : nullptr; }
IT_API size_t it_arena_floats(it_ctx* c) { return c ? c->arena_floats : 0; }

static int arena_range(it_ctx* c, size_t off, size_t n, const char* who) {
    IT_CHECK_ARG(c, "%s: null context", who);
    IT_CHECK_ARG(off <= c->arena_floats && n <= c->arena_floats - off, "%s: range [%zu, +%zu) outside the arena (%zu floats)", who, off, n, c->arena_floats);
    return IT_OK;
}
IT_API int it_arena_write(it_ctx* c, size_t off, const void* host, size_t n) {
    int r = arena_range(c, off, n, "it_arena_write"); if (r) return r;
    if (c->capturing) return it_fail(IT_ESTATE, "it_arena_write: not allowed while recording a graph");
    IT_CHECK_ARG(host || n == 0, "it_arena_write: null host pointer");
    if (n == 0) return IT_OK;
    it_note_op(c);
    IT_CUDA(cudaMemcpyAsync(c->arena + off, host, n * 4, cudaMemcpyHostToDevice, c->stream));
    IT_CUDA(cudaStreamSynchronize(c->stream)); return IT_OK;
}
IT_API int it_arena_read(it_ctx* c, size_t off, void* host, size_t n) {
    int r = arena_range(c, off, n, "it_arena_read"); if (r) return r;
    if (c->capturing) return it_fail(IT_ESTATE, "it_arena_read: not allowed while recording a graph");
    IT_CHECK_ARG(host || n == 0, "it_arena_read: null host pointer");
    if (n == 0) return IT_OK;
    IT_CUDA(cudaMemcpyAsync(host, c->arena + off, n * 4, cudaMemcpyDeviceToHost, c->stream));
    IT_CUDA(cudaStreamSynchronize(c->stream));
    return it_check_device_error(c, "it_arena_read");
}
IT_API int it_arena_zero(it_ctx* c, size_t off, size_t n) {
    int r = arena_range(c, off, n, "it_arena_zero"); if (r) return r;
    it_note_op(c);
    if (n) IT_CUDA(cudaMemsetAsync(c->arena + off, 0, n * 4, c->stream));
    return IT_OK;
}
IT_API int it_signs_set(it_ctx* c, size_t n, const float* signs) {
    IT_CHECK_ARG(c && signs, "it_signs_set: null argument");
    IT_CHECK_ARG(n > 0 && n % 1024 == 0, "it_signs_set: width %zu is not a multiple of the 1024 Hadamard block", n);
    for (size_t i = 0; i < n; i++) IT_CHECK_ARG(signs[i] == 1.0f || signs[i] == -1.0f, "it_signs_set: sign %zu is %g, not +-1", i, (double)signs[i]);
    IT_CUDA(cudaSetDevice(c->device));
    float*& d = c->signs[n];
    if (!d) IT_CUDA(cudaMalloc(&d, n * 4));
    IT_CUDA(cudaMemcpyAsync(d, signs, n * 4, cudaMemcpyHostToDevice, c->stream));
    IT_CUDA(cudaStreamSynchronize(c->stream)); return IT_OK;
}

// ---------------------------------------------------------------- ternary matrices
static int mat_alloc(it_ctx* c, size_t rows, size_t cols, it_mat** out, const char* who) {
    IT_CHECK_ARG(c && out, "%s: null argument", who);
    *out = nullptr;
    IT_CHECK_ARG(rows > 0 && cols > 0, "%s: empty matrix %zux%zu", who, rows, cols);
    IT_CHECK_ARG(cols % 128 == 0, "%s: cols %zu is not a multiple of the 128-element PQ2_0 block", who, cols);
    IT_CHECK_ARG(rows <= (1u << 30) && cols <= (1u << 24), "%s: matrix %zux%zu too large", who, rows, cols);
    IT_CUDA(cudaSetDevice(c->device));
    it_mat* m = new it_mat(); m->ctx = c; m->rows = rows; m->cols = cols; m->row_groups = (rows + 31) / 32;
    m->bytes = m->row_groups * (cols / 128) * IT_TILE_BYTES; m->tiles = nullptr; m->owns_tiles = true;
    m->sharded = false; m->map.nseg = 0; m->out_rows = rows;
    cudaError_t e = cudaMalloc(&m->tiles, m->bytes);
    if (e != cudaSuccess) { delete m; return it_fail(IT_ENOMEM, "%s: cudaMalloc(%zu): %s", who, m->bytes, cudaGetErrorString(e)); }
    *out = m; return IT_OK;
}
static int mat_from_raw_host(it_ctx* c, const uint8_t* raw, size_t rows, size_t cols, it_mat** out, const char* who) {
    int r = mat_alloc(c, rows, cols, out, who); if (r) return r;
    size_t nbytes = rows * (cols / 128) * 34; uint8_t* tmp = nullptr;
    cudaError_t e = cudaMalloc(&tmp, nbytes);
    if (e == cudaSuccess) e = cudaMemcpyAsync(tmp, raw, nbytes, cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) { r = it_launch_repack_pq2(c, tmp, rows, cols, (*out)->tiles); if (r == IT_OK) e = cudaStreamSynchronize(c->stream); }
    if (tmp) cudaFree(tmp);
    if (e != cudaSuccess || r != IT_OK) { it_matrix_destroy(*out); *out = nullptr; return r ? r : it_fail(IT_ECUDA, "%s: %s", who, cudaGetErrorString(e)); }
    return IT_OK;
}
IT_API int it_matrix_upload_pq2(it_ctx* c, const uint8_t* raw, size_t rows, size_t cols, it_mat** out) {
    IT_CHECK_ARG(raw, "it_matrix_upload_pq2: null data");
    return mat_from_raw_host(c, raw, rows, cols, out, "it_matrix_upload_pq2");
}
IT_API int it_matrix_upload_packed2(it_ctx* c, const uint32_t* words, const float* scales, size_t rows, size_t cols, it_mat** out) {
    IT_CHECK_ARG(words && scales, "it_matrix_upload_packed2: null data");
    IT_CHECK_ARG(rows > 0 && cols > 0 && cols % 128 == 0, "it_matrix_upload_packed2: bad shape %zux%zu", rows, cols);
    size_t nblk = rows * (cols / 128);
    std::vector<uint8_t> raw(nblk * 34);
    for (size_t i = 0; i < nblk; i++) {
        __half h = __float2half_rn(scales[i]);
        IT_CHECK_ARG(__half2float(h) == scales[i], "it_matrix_upload_packed2: scale %zu (%g) is not an f16 value", i, (double)scales[i]);
        unsigned short hb; memcpy(&hb, &h, 2);
        raw[i * 34] = (uint8_t)(hb & 0xff); raw[i * 34 + 1] = (uint8_t)(hb >> 8);
        memcpy(&raw[i * 34 + 2], words + i * 8, 32);   // Packed2 words are the PQ2_0 qs bytes read as little-endian u32
    }
    return mat_from_raw_host(c, raw.data(), rows, cols, out, "it_matrix_upload_packed2");
}
IT_API int it_matrix_synth(it_ctx* c, uint64_t seed, size_t rows, size_t cols, int four_codes, it_mat** out) {
    int r = mat_alloc(c, rows, cols, out, "it_matrix_synth"); if (r) return r;
    size_t nbytes = rows * (cols / 128) * 34; uint8_t* tmp = nullptr;
    cudaError_t e = cudaMalloc(&tmp, nbytes);
    if (e == cudaSuccess) { r = it_launch_synth_pq2(c, seed, rows, cols, four_codes, tmp); if (r == IT_OK) r = it_launch_repack_pq2(c, tmp, rows, cols, (*out)->tiles);
        if (r == IT_OK) e = cudaStreamSynchronize(c->stream); }
    if (tmp) cudaFree(tmp);
    if (e != cudaSuccess || r != IT_OK) { it_matrix_destroy(*out); *out = nullptr; return r ? r : it_fail(e == cudaErrorMemoryAllocation ? IT_ENOMEM : IT_ECUDA, "it_matrix_synth: %s", cudaGetErrorString(e)); }
    return IT_OK;
}
// ---------------------------------------------------------------- row shards
IT_API int it_shard_range(size_t rows, int rank, int world, size_t* row0, size_t* nrows) {
    IT_CHECK_ARG(row0 && nrows, "it_shard_range: null output");
    IT_CHECK_ARG(world >= 1 && world <= IT_MAX_PEERS && rank >= 0 && rank < world, "it_shard_range: bad rank %d of %d", rank, world);
    IT_CHECK_ARG(rows % (size_t)world == 0, "it_shard_range: %zu rows do not split evenly over %d ranks", rows, world);
    *nrows = rows / (size_t)world; *row0 = *nrows * (size_t)rank;
    return IT_OK;
}
IT_API int it_matrix_set_shard(it_mat* m, size_t row0, size_t total_rows) {
    IT_CHECK_ARG(m, "it_matrix_set_shard: null matrix");
    IT_CHECK_ARG(row0 + m->rows <= total_rows && total_rows <= (1u << 30), "it_matrix_set_shard: rows [%zu, %zu) fall outside a matrix of %zu rows", row0, row0 + m->rows, total_rows);
    m->sharded = true; m->map.nseg = 1; m->map.start[0] = 0; m->map.delta[0] = (int)row0; m->map.shift[0] = (int)m->rows; m->out_rows = total_rows;
    return IT_OK;
}
IT_API int it_matrix_synth_rows(it_ctx* c, uint64_t seed, size_t total_rows, size_t cols, int four_codes, size_t row0, size_t nrows, it_mat** out) {
    IT_CHECK_ARG(out, "it_matrix_synth_rows: null output");
    *out = nullptr;
    IT_CHECK_ARG(nrows > 0 && row0 + nrows <= total_rows, "it_matrix_synth_rows: rows [%zu, %zu) fall outside a matrix of %zu rows", row0, row0 + nrows, total_rows);
    int r = mat_alloc(c, nrows, cols, out, "it_matrix_synth_rows"); if (r) return r;
    size_t nbytes = nrows * (cols / 128) * 34; uint8_t* tmp = nullptr;
    cudaError_t e = cudaMalloc(&tmp, nbytes);
    if (e == cudaSuccess) { r = it_launch_synth_pq2(c, seed, nrows, cols, four_codes, tmp, row0); if (r == IT_OK) r = it_launch_repack_pq2(c, tmp, nrows, cols, (*out)->tiles);
        if (r == IT_OK) e = cudaStreamSynchronize(c->stream); }
    if (tmp) cudaFree(tmp);
    if (e != cudaSuccess || r != IT_OK) { it_matrix_destroy(*out); *out = nullptr; return r ? r : it_fail(e == cudaErrorMemoryAllocation ? IT_ENOMEM : IT_ECUDA, "it_matrix_synth_rows: %s", cudaGetErrorString(e)); }
    return it_matrix_set_shard(*out, row0, total_rows);
}

int it_matrix_view(it_ctx* c, size_t rows, size_t cols, uint8_t* tiles, it_mat** out) {
    IT_CHECK_ARG(c && out && tiles && rows > 0 && cols % 128 == 0, "it_matrix_view: bad argument");
    it_mat* m = new it_mat(); m->ctx = c; m->rows = rows; m->cols = cols; m->row_groups = (rows + 31) / 32;
    m->bytes = m->row_groups * (cols / 128) * IT_TILE_BYTES; m->tiles = tiles; m->owns_tiles = false;
    m->sharded = false; m->map.nseg = 0; m->out_rows = rows;
    *out = m; return IT_OK;
}
int it_matrix_synth_view(it_ctx* c, uint64_t seed, size_t rows, size_t cols, uint8_t* tiles, it_mat** out, size_t row0) {
    int r = it_matrix_view(c, rows, cols, tiles, out); if (r) return r;
    size_t nbytes = rows * (cols / 128) * 34; uint8_t* tmp = nullptr;
    cudaError_t e = cudaMalloc(&tmp, nbytes);
    if (e == cudaSuccess) { r = it_launch_synth_pq2(c, seed, rows, cols, 0, tmp, row0); if (r == IT_OK) r = it_launch_repack_pq2(c, tmp, rows, cols, tiles);
        if (r == IT_OK) e = cudaStreamSynchronize(c->stream); }
    if (tmp) cudaFree(tmp);
    if (e != cudaSuccess || r != IT_OK) { it_matrix_destroy(*out); *out = nullptr; return r ? r : it_fail(e == cudaErrorMemoryAllocation ? IT_ENOMEM : IT_ECUDA, "it_matrix_synth_view: %s", cudaGetErrorString(e)); }
    return IT_OK;
}
IT_API int it_matrix_download_pq2(it_ctx* c, const it_mat* m, uint8_t* raw) {
    IT_CHECK_ARG(c && m && raw, "it_matrix_download_pq2: null argument");
    IT_CUDA(cudaSetDevice(c->device));
    size_t nbytes = m->rows * (m->cols / 128) * 34; uint8_t* tmp = nullptr;
    IT_CUDA(cudaMalloc(&tmp, nbytes));
    int r = it_launch_unpack_pq2(c, m->tiles, m->rows, m->cols, tmp);
    cudaError_t e = r == IT_OK ? cudaMemcpyAsync(raw, tmp, nbytes, cudaMemcpyDeviceToHost, c->stream) : cudaSuccess;
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    cudaFree(tmp);
    if (r) return r;
    if (e != cudaSuccess) return it_fail(IT_ECUDA, "it_matrix_download_pq2: %s", cudaGetErrorString(e));
    return IT_OK;
}
IT_API size_t it_matrix_rows(const it_mat* m) { return m ? m->rows : 0; }
IT_API size_t it_matrix_cols(const it_mat* m) { return m ? m->cols : 0; }
IT_API size_t it_matrix_device_bytes(const it_mat* m) { return m ? m->bytes : 0; }
IT_API void it_matrix_destroy(it_mat* m) { if (!m) return; cudaSetDevice(m->ctx->device); if (m->tiles && m->owns_tiles) cudaFree(m->tiles); delete m; }

// ---------------------------------------------------------------- int8-group matrices
static int qmat_alloc(it_ctx* c, size_t rows, size_t cols, it_qmat** out, const char* who) {
    IT_CHECK_ARG(c && out, "%s: null argument", who);
    *out = nullptr;
    IT_CHECK_ARG(rows > 0 && cols > 0 && cols % 32 == 0, "%s: bad shape %zux%zu (cols must be a multiple of 32)", who, rows, cols);
    IT_CUDA(cudaSetDevice(c->device));
    it_qmat* m = new it_qmat(); m->ctx = c; m->rows = rows; m->cols = cols; m->q = nullptr; m->d = nullptr; m->s16 = nullptr; m->sharded = false; m->row0 = 0; m->out_rows = rows;
    m->bytes = rows * cols + rows * (cols / 32) * 2;
    cudaError_t e = cudaMalloc(&m->q, rows * cols);
    if (e == cudaSuccess) e = cudaMalloc(&m->d, rows * (cols / 32) * 2);
    if (e != cudaSuccess) { it_qmatrix_destroy(m); return it_fail(IT_ENOMEM, "%s: cudaMalloc: %s", who, cudaGetErrorString(e)); }
    *out = m; return IT_OK;
}
IT_API int it_qmatrix_upload_q8_0(it_ctx* c, const uint8_t* raw, size_t rows, size_t cols, it_qmat** out) {
    IT_CHECK_ARG(raw, "it_qmatrix_upload_q8_0: null data");
    int r = qmat_alloc(c, rows, cols, out, "it_qmatrix_upload_q8_0"); if (r) return r;
    size_t nblk = rows * cols / 32;
    std::vector<int8_t> q(rows * cols); std::vector<unsigned short> d(nblk);
    for (size_t i = 0; i < nblk; i++) { const uint8_t* b = raw + i * 34; d[i] = (unsigned short)(b[0] | (b[1] << 8)); memcpy(&q[i * 32], b + 2, 32); }
    cudaError_t e = cudaMemcpyAsync((*out)->q, q.data(), q.size(), cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync((*out)->d, d.data(), d.size() * 2, cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) { it_qmatrix_destroy(*out); *out = nullptr; return it_fail(IT_ECUDA, "it_qmatrix_upload_q8_0: %s", cudaGetErrorString(e)); }
    return IT_OK;
}
// Q6_K rows -> int8 values (q - 32) and one f32 scale per 16 weights, scale = d * sub-block scale, exact in f32
// (Q8G16::from_ggml, src/quant.rs:245-257)
IT_API int it_qmatrix_upload_q6_k(it_ctx* c, const uint8_t* raw, size_t rows, size_t cols, it_qmat** out) {
    IT_CHECK_ARG(raw, "it_qmatrix_upload_q6_k: null data");
    IT_CHECK_ARG(cols % 256 == 0, "it_qmatrix_upload_q6_k: cols %zu is not a multiple of the 256-element Q6_K block", cols);
    int r = qmat_alloc(c, rows, cols, out, "it_qmatrix_upload_q6_k"); if (r) return r;
    it_qmat* m = *out;
    cudaFree(m->d); m->d = nullptr;
    const size_t n = rows * cols, nblk = n / 256;
    m->bytes = n + n / 16 * 4;
    std::vector<int8_t> q(n); std::vector<float> sc(n / 16);
    for (size_t i = 0; i < nblk; i++) {
        const uint8_t* b = raw + i * 210;
        unsigned short hb = (unsigned short)(b[208] | (b[209] << 8)); __half h; memcpy(&h, &hb, 2);
        const float d = __half2float(h);
        for (int g = 0; g < 16; g++) sc[i * 16 + g] = d * (float)(int8_t)b[192 + g];
        for (int half = 0; half < 2; half++) {
            const uint8_t* ql = b + half * 64; const uint8_t* qh = b + 128 + half * 32; int8_t* o = &q[i * 256 + half * 128];
            for (int l = 0; l < 32; l++) {
                o[l] = (int8_t)((int)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32);
                o[l + 32] = (int8_t)((int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32);
                o[l + 64] = (int8_t)((int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32);
                o[l + 96] = (int8_t)((int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32);
            }
        }
    }
    cudaError_t e = cudaMalloc(&m->s16, sc.size() * 4);
    if (e == cudaSuccess) e = cudaMemcpyAsync(m->q, q.data(), q.size(), cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(m->s16, sc.data(), sc.size() * 4, cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) { it_qmatrix_destroy(m); *out = nullptr; return it_fail(e == cudaErrorMemoryAllocation ? IT_ENOMEM : IT_ECUDA, "it_qmatrix_upload_q6_k: %s", cudaGetErrorString(e)); }
    return IT_OK;
}
IT_API int it_qmatrix_group16(const it_qmat* m) { return m && m->s16 ? 1 : 0; }
// int8 values [rows*cols], then the f32 scales [rows*cols/16] (for Q8_0 sources each block's scale twice)
IT_API int it_qmatrix_download_g16(it_ctx* c, const it_qmat* m, uint8_t* raw) {
    IT_CHECK_ARG(c && m && raw, "it_qmatrix_download_g16: null argument");
    const size_t n = m->rows * m->cols;
    IT_CUDA(cudaMemcpyAsync(raw, m->q, n, cudaMemcpyDeviceToHost, c->stream));
    if (m->s16) IT_CUDA(cudaMemcpyAsync(raw + n, m->s16, n / 16 * 4, cudaMemcpyDeviceToHost, c->stream));
    else {
        std::vector<unsigned short> d(n / 32);
        IT_CUDA(cudaMemcpyAsync(d.data(), m->d, d.size() * 2, cudaMemcpyDeviceToHost, c->stream));
        IT_CUDA(cudaStreamSynchronize(c->stream));
        for (size_t i = 0; i < n / 32; i++) { __half h; memcpy(&h, &d[i], 2); const float f = __half2float(h); memcpy(raw + n + 8 * i, &f, 4); memcpy(raw + n + 8 * i + 4, &f, 4); }
    }
    IT_CUDA(cudaStreamSynchronize(c->stream));
    return IT_OK;
}
IT_API int it_qmatrix_synth(it_ctx* c, uint64_t seed, size_t rows, size_t cols, it_qmat** out) {
    int r = qmat_alloc(c, rows, cols, out, "it_qmatrix_synth"); if (r) return r;
    r = it_launch_synth_q8_0(c, seed, rows, cols, (*out)->q, (*out)->d);
    cudaError_t e = r == IT_OK ? cudaStreamSynchronize(c->stream) : cudaSuccess;
    if (r || e != cudaSuccess) { it_qmatrix_destroy(*out); *out = nullptr; return r ? r : it_fail(IT_ECUDA, "it_qmatrix_synth: %s", cudaGetErrorString(e)); }
    return IT_OK;
}
IT_API int it_qmatrix_set_shard(it_qmat* m, size_t row0, size_t total_rows) {
    IT_CHECK_ARG(m, "it_qmatrix_set_shard: null matrix");
    IT_CHECK_ARG(row0 + m->rows <= total_rows && total_rows <= (1u << 30), "it_qmatrix_set_shard: rows [%zu, %zu) fall outside a matrix of %zu rows", row0, row0 + m->rows, total_rows);
    m->sharded = true; m->row0 = row0; m->out_rows = total_rows;
    return IT_OK;
}
IT_API int it_qmatrix_synth_rows(it_ctx* c, uint64_t seed, size_t total_rows, size_t cols, size_t row0, size_t nrows, it_qmat** out) {
    IT_CHECK_ARG(out, "it_qmatrix_synth_rows: null output");
    *out = nullptr;
    IT_CHECK_ARG(nrows > 0 && row0 + nrows <= total_rows, "it_qmatrix_synth_rows: rows [%zu, %zu) fall outside a matrix of %zu rows", row0, row0 + nrows, total_rows);
    int r = qmat_alloc(c, nrows, cols, out, "it_qmatrix_synth_rows"); if (r) return r;
    r = it_launch_synth_q8_0(c, seed, nrows, cols, (*out)->q, (*out)->d, row0);
    cudaError_t e = r == IT_OK ? cudaStreamSynchronize(c->stream) : cudaSuccess;
    if (r || e != cudaSuccess) { it_qmatrix_destroy(*out); *out = nullptr; return r ? r : it_fail(IT_ECUDA, "it_qmatrix_synth_rows: %s", cudaGetErrorString(e)); }
    return it_qmatrix_set_shard(*out, row0, total_rows);
}
IT_API int it_qmatrix_download_q8_0(it_ctx* c, const it_qmat* m, uint8_t* raw) {
    IT_CHECK_ARG(c && m && raw, "it_qmatrix_download_q8_0: null argument");
    IT_CHECK_ARG(m->d, "it_qmatrix_download_q8_0: the matrix holds 16-weight groups (use it_qmatrix_download_g16)");
    size_t nblk = m->rows * m->cols / 32;
    std::vector<int8_t> q(m->rows * m->cols); std::vector<unsigned short> d(nblk);
    IT_CUDA(cudaMemcpyAsync(q.data(), m->q, q.size(), cudaMemcpyDeviceToHost, c->stream));
    IT_CUDA(cudaMemcpyAsync(d.data(), m->d, d.size() * 2, cudaMemcpyDeviceToHost, c->stream));
    IT_CUDA(cudaStreamSynchronize(c->stream));
    for (size_t i = 0; i < nblk; i++) { uint8_t* b = raw + i * 34; b[0] = (uint8_t)(d[i] & 0xff); b[1] = (uint8_t)(d[i] >> 8); memcpy(b + 2, &q[i * 32], 32); }
    return IT_OK;
}
IT_API size_t it_qmatrix_rows(const it_qmat* m) { return m ? m->rows : 0; }
IT_API size_t it_qmatrix_cols(const it_qmat* m) { return m ? m->cols : 0; }
IT_API void it_qmatrix_destroy(it_qmat* m) { if (!m) return; cudaSetDevice(m->ctx->device); if (m->q) cudaFree(m->q); if (m->d) cudaFree(m->d); if (m->s16) cudaFree(m->s16); delete m; }

// ---------------------------------------------------------------- q8 activation rows
// Tensor map over the int8 rows for the tile kernel: boxes of 128 bytes (one 128-column block) x 64 rows, written to
// shared memory with the 128-byte swizzle so that fragment loads are free of bank conflicts.
static int make_q8_tensor_map(it_q8* q, size_t rows_alloc) {
    typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static encode_fn encode = nullptr;
    if (!encode) {
        void* fn = nullptr; cudaDriverEntryPointQueryResult qres;
        IT_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) return it_fail(IT_ECUDA, "it_q8_create: the driver does not export cuTensorMapEncodeTiled");
        encode = (encode_fn)fn;
    }
    const cuuint64_t dims[2] = { (cuuint64_t)q->max_n, (cuuint64_t)rows_alloc };
    const cuuint64_t strides[1] = { (cuuint64_t)q->max_n };
    const cuuint32_t box[2] = { 128, 64 };
    const cuuint32_t estr[2] = { 1, 1 };
    const CUresult r = encode(&q->tmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, q->qs, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return it_fail(IT_ECUDA, "it_q8_create: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return IT_OK;
}

IT_API int it_q8_create(it_ctx* c, size_t max_n, size_t max_tok, it_q8** out) {
    IT_CHECK_ARG(c && out, "it_q8_create: null argument");
    *out = nullptr;
    IT_CHECK_ARG(max_n > 0 && max_n % 256 == 0, "it_q8_create: width %zu is not a multiple of the 256-element q8k block", max_n);
    IT_CHECK_ARG(max_tok > 0 && max_tok <= 65535, "it_q8_create: bad row count %zu", max_tok);
    IT_CUDA(cudaSetDevice(c->device));
    it_q8* q = new it_q8(); q->ctx = c; q->max_n = max_n; q->max_tok = max_tok; q->n = 0; q->qs = nullptr; q->d = nullptr; q->sum128 = nullptr;
    const size_t rows_alloc = max_tok < 64 ? 64 : max_tok;      // the tile kernel fetches boxes of 64 rows
    cudaError_t e = cudaMalloc(&q->qs, max_n * rows_alloc);
    if (e == cudaSuccess) e = cudaMemsetAsync(q->qs, 0, max_n * rows_alloc, c->stream);
    if (e == cudaSuccess) e = cudaMalloc(&q->d, max_n / 256 * max_tok * 4);
    if (e == cudaSuccess) e = cudaMalloc(&q->sum128, max_n / 128 * max_tok * 4);
    if (e != cudaSuccess) { it_q8_destroy(q); return it_fail(IT_ENOMEM, "it_q8_create: %s", cudaGetErrorString(e)); }
    const int r = make_q8_tensor_map(q, rows_alloc);
    if (r) { it_q8_destroy(q); return r; }
    *out = q; return IT_OK;
}
IT_API void it_q8_destroy(it_q8* q) { if (!q) return; cudaSetDevice(q->ctx->device); if (q->qs) cudaFree(q->qs); if (q->d) cudaFree(q->d); if (q->sum128) cudaFree(q->sum128); delete q; }
IT_API int it_q8_read(it_ctx* c, const it_q8* q, size_t tok, int8_t* qs, float* d, int32_t* sum128) {
    IT_CHECK_ARG(c && q, "it_q8_read: null argument");
    IT_CHECK_ARG(q->n > 0 && tok < q->max_tok, "it_q8_read: nothing written yet or row %zu out of range", tok);
    if (qs) IT_CUDA(cudaMemcpyAsync(qs, q->qs + tok * q->max_n, q->n, cudaMemcpyDeviceToHost, c->stream));
    if (d) IT_CUDA(cudaMemcpyAsync(d, q->d + tok * (q->max_n / 256), q->n / 256 * 4, cudaMemcpyDeviceToHost, c->stream));
    if (sum128) IT_CUDA(cudaMemcpyAsync(sum128, q->sum128 + tok * (q->max_n / 128), q->n / 128 * 4, cudaMemcpyDeviceToHost, c->stream));
    IT_CUDA(cudaStreamSynchronize(c->stream)); return IT_OK;
}
