// Decoder support ops around the ternary matvecs: rmsnorm, rope, causal conv, delta rule, attention, ...
//
// These follow the reference's CPU forward pass (src/cpu.rs:14-22, :145-164, :194-274) operation for operation
// and in its order of additions, so that results are bit-identical to that code, with three exceptions that are
// stated where they occur: the width-n_embd rmsnorm adds its squares in a fixed lane/tree order (a sequential
// sum of 5120 terms is a 10 us dependency chain), dense f32 rows are summed lane-strided in f64, and exp / log /
// sin / cos come from it_math.h.  None of these kernels is on the HBM roofline; they are sized for latency.
#include "it_internal.h"
#include "it_support.h"
#include "it_math.h"

namespace {

// x[t] = table[tok[t]]  (Model::embed, src/cpu.rs:118-122; the reference computes this on the host, src/vk/mod.rs:766-769)
__global__ void k_embed(const uint32_t* __restrict__ toks, const float* __restrict__ table, int e, float* x) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    const int t = blockIdx.y; const size_t row = toks[t];
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < e / 4; i += gridDim.x * blockDim.x)
        reinterpret_cast<float4*>(x + (size_t)t * e)[i] = reinterpret_cast<const float4*>(table + row * e)[i];
}

// rmsnorm over the embedding width (src/cpu.rs:14-18), one CTA of 256 threads per row.  Sum of squares: thread i
// adds x[i]^2, x[i+256]^2, ... in ascending order; each warp folds with a butterfly (offsets 16..1); the eight warp
// sums are added in ascending order.  out = (x * s) * w with s = 1 / sqrt(ss / n + eps), no fused multiply-add.
__global__ void __launch_bounds__(256) k_rmsnorm_wide(const float* x, size_t x_stride, const float* __restrict__ w, int n, float eps, float* out, size_t out_stride) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    __shared__ float wsum[8];
    const float* xr = x + blockIdx.x * x_stride; float* o = out + blockIdx.x * out_stride;
    float v[32];                                   // n <= 8192: all loads are issued before the first add
#pragma unroll
    for (int k = 0; k < 32; k++) { const int j = threadIdx.x + 256 * k; v[k] = j < n ? xr[j] : 0.f; }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 32; k++) if (threadIdx.x + 256 * k < n) s = it_add(s, it_mul(v[k], v[k]));
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) s = it_add(s, __shfl_xor_sync(0xffffffffu, s, m));
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = s;
    __syncthreads();
    float t = wsum[0];
#pragma unroll
    for (int k = 1; k < 8; k++) t = it_add(t, wsum[k]);
    const float sc = it_div(1.0f, it_sqrt(it_add(it_div(t, (float)n), eps)));
#pragma unroll
    for (int k = 0; k < 32; k++) { const int j = threadIdx.x + 256 * k; if (j < n) o[j] = it_mul(it_mul(v[k], sc), w[j]); }
}

// Per-head norms of width n <= 256, one warp per (head, row), the squares added sequentially as on the CPU.
// mode 0: rmsnorm with weight (q_norm / k_norm, src/cpu.rs:252-256); mode 1: rmsnorm with weight, then * silu(z)
// (gated ssm_norm, src/cpu.rs:233-237); mode 2: l2norm, x / max(sqrt(sum), eps) (src/cpu.rs:164, :214).
__global__ void __launch_bounds__(128) k_norm_head(const float* in, size_t in_hs, size_t in_ts, float* out, size_t out_hs, size_t out_ts,
                                                   int n, int nheads, const float* __restrict__ w, int mode, float eps, const float* z, size_t z_hs, size_t z_ts) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    __shared__ float buf[4][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.x * 4 + warp, t = blockIdx.y;
    if (head >= nheads) return;
    const float* x = in + t * in_ts + head * in_hs;
    for (int i = lane; i < n; i += 32) buf[warp][i] = x[i];
    __syncwarp();
    float s = 0.f;
    if (lane == 0) {
#pragma unroll 8
        for (int i = 0; i < n; i++) s = it_add(s, it_mul(buf[warp][i], buf[warp][i]));
    }
    s = __shfl_sync(0xffffffffu, s, 0);
    const float sc = mode == 2 ? it_div(1.0f, fmaxf(it_sqrt(s), eps)) : it_div(1.0f, it_sqrt(it_add(it_div(s, (float)n), eps)));
    float* o = out + t * out_ts + head * out_hs;
    for (int i = lane; i < n; i += 32) {
        float v = it_mul(buf[warp][i], sc);
        if (mode != 2) v = it_mul(v, w[i]);
        if (mode == 1) v = it_mul(v, it_silu(z[t * z_ts + head * z_hs + i]));
        o[i] = v;
    }
}

// (I)MRoPE for text positions on the first n_rot dims of each head (src/cpu.rs:145-162): the angle of pair i is the
// position multiplied i times by theta_scale, one rounding per step exactly as the CPU's running product.
__global__ void k_rope(float* x, size_t hs, size_t ts, int nheads, int pos0, const int* pos_ptr, int n_rot, float theta_scale, int s0, int s1, int s2, int s3) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    const int half = n_rot / 2, t = blockIdx.y;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= nheads * half) return;
    const int head = idx / half, i = idx % half;
    if (pos_ptr) pos0 += *pos_ptr;
    float theta = (float)(pos0 + t);
    for (int k = 0; k < i; k++) theta = it_mul(theta, theta_scale);
    const int sect = s0 + s1 + s2 + s3, sector = sect > 0 ? i % sect : 0;
    const bool use_e = sect > 0 && !((sector % 3 == 1 && sector < 3 * s1) || (sector % 3 == 2 && sector < 3 * s2) || (sector % 3 == 0 && sector < 3 * s0));
    float s, c; it_sincosf(use_e ? 0.0f : theta, &s, &c);
    float* h = x + t * ts + head * hs;
    const float x0 = h[i], x1 = h[i + half];
    h[i] = it_sub(it_mul(x0, c), it_mul(x1, s));
    h[i + half] = it_add(it_mul(x0, s), it_mul(x1, c));
}

// Causal depthwise conv + SiLU + state shift, token after token (src/cpu.rs:203-212).  One thread per channel; the
// state after token t is copied to checkpoint t when one is given (MTP rollback, src/vk/mod.rs:794).
__global__ void k_conv(const float* mixed, size_t m_ts, const float* __restrict__ w, float* state, float* out, size_t o_ts, int cd, int kk, int nt,
                       float* ck, size_t ck_stride, int nck) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= cd) return;
    float st[8];
    for (int i = 0; i < kk - 1; i++) st[i] = state[(size_t)i * cd + ch];
    for (int t = 0; t < nt; t++) {
        const float m = mixed[t * m_ts + ch];
        float s = 0.f;
        for (int i = 0; i < kk; i++) s = it_add(s, it_mul(i < kk - 1 ? st[i] : m, w[ch * kk + i]));
        out[t * o_ts + ch] = it_silu(s);
        for (int i = 0; i < kk - 2; i++) st[i] = st[i + 1];
        st[kk - 2] = m;
        if (t < nck) for (int i = 0; i < kk - 1; i++) ck[t * ck_stride + (size_t)i * cd + ch] = st[i];
    }
    for (int i = 0; i < kk - 1; i++) state[(size_t)i * cd + ch] = st[i];
}

// The same conv for many rows at once (prompt passes): the output of row t depends only on the inputs of rows t-kk+1 .. t
// (the state is just the last kk-1 inputs), so rows are independent: 128 channels x 8 row lanes per CTA, every sum in the
// tap order of k_conv.  The state is rewritten after all reads of the old one.  No checkpoints (verification passes are short).
__global__ void __launch_bounds__(1024) k_conv_wide(const float* mixed, size_t m_ts, const float* __restrict__ w, float* state, float* out, size_t o_ts, int cd, int kk, int nt) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    const int ch = blockIdx.x * 128 + threadIdx.x;
    const bool live = ch < cd;
    float wt[9];
    if (live) for (int i = 0; i < kk; i++) wt[i] = w[ch * kk + i];
    auto input = [&](int r) { return r >= 0 ? mixed[r * m_ts + ch] : state[(size_t)(kk - 1 + r) * cd + ch]; };   // row r of this pass, or of the state
    if (live) for (int t = threadIdx.y; t < nt; t += 8) {
        float s = 0.f;
        for (int i = 0; i < kk; i++) s = it_add(s, it_mul(input(t - (kk - 1) + i), wt[i]));
        out[t * o_ts + ch] = it_silu(s);
    }
    float keep[8];
    if (live && threadIdx.y == 0) for (int i = 0; i < kk - 1; i++) keep[i] = input(nt - (kk - 1) + i);
    __syncthreads();
    if (live && threadIdx.y == 0) for (int i = 0; i < kk - 1; i++) state[(size_t)i * cd + ch] = keep[i];
}

// Dense f32 rows (ssm_beta / ssm_alpha; cpu::matvec's f32 arm under Numerics::Ggml, src/cpu.rs:36-43: f32 products,
// f64 accumulation).  One CTA of 256 threads per row: thread i adds the products i, i+256, ... in f64, each warp folds
// with a butterfly, the eight warp sums are added in ascending order.  Rows [0, rows) use w0 / y0, rows [rows, 2 rows) w1 / y1.
__global__ void __launch_bounds__(256) k_dense_rows(const float* __restrict__ w0, const float* __restrict__ w1, int rows, int cols, const float* x, size_t x_ts,
                                                    float* y0, float* y1, size_t y_ts) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    __shared__ double wsum[8];
    const int r = blockIdx.x, t = blockIdx.y, row = r < rows ? r : r - rows;
    const float* wr = (r < rows ? w0 : w1) + (size_t)row * cols; const float* xr = x + t * x_ts;
    double s = 0.0;
#pragma unroll 4
    for (int i = threadIdx.x; i < cols; i += 256) s += (double)it_mul(wr[i], xr[i]);
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double tt = wsum[0];
        for (int k = 1; k < 8; k++) tt += wsum[k];
        (r < rows ? y0 : y1)[t * y_ts + row] = (float)tt;
    }
}

// Gated delta rule, token after token (src/cpu.rs:215-232).  One CTA per 32 rows of a head's state matrix; every
// row is updated by one thread with the CPU's two sequential passes, all threads move the tile.  The tile goes through shared memory so that
// global accesses stay coalesced.  State layout [head][j][i] as on the CPU (src/cpu.rs:132).
__global__ void __launch_bounds__(128) k_gdn(const float* co, size_t co_ts, const float* beta, const float* alpha, size_t ba_ts, const float* __restrict__ dt, const float* __restrict__ a,
                                             float* state, float* o, size_t o_ts, int nk, int sd, int qk, int nt, float* ck, size_t ck_stride, int nck) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    extern __shared__ float tile[];            // [32][sd + 1] rows, then q[sd], k[sd]
    const int h = blockIdx.x, j0 = blockIdx.y * 32, tid = threadIdx.x, kh = h % nk, ld = sd + 1, nvec = 32 * sd / 4;
    float* qs = tile + 32 * ld; float* ks = qs + sd;
    float* m = state + ((size_t)h * sd + j0) * sd;
    auto tile_in = [&](const float* src) {     // all 128 threads, 128-bit loads, every load in flight at once
        for (int f = tid; f < nvec; f += 128) { const float4 v = reinterpret_cast<const float4*>(src)[f]; const int r = (4 * f) / sd, i = (4 * f) % sd;
            float* d = tile + r * ld + i; d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w; }
    };
    auto tile_out = [&](float* dst) {
        for (int f = tid; f < nvec; f += 128) { const int r = (4 * f) / sd, i = (4 * f) % sd; const float* d = tile + r * ld + i;
            reinterpret_cast<float4*>(dst)[f] = make_float4(d[0], d[1], d[2], d[3]); }
    };
    tile_in(m);
    float* row = tile + tid * ld;               // threads 0..31 own one row each
    const float scale = it_div(1.0f, it_sqrt((float)sd));
    for (int t = 0; t < nt; t++) {
        const float* c = co + t * co_ts;
        __syncthreads();
        for (int i = tid; i < sd; i += 128) { qs[i] = c[kh * sd + i]; ks[i] = c[qk + kh * sd + i]; }
        __syncthreads();
        if (tid < 32) {
            const float v = c[2 * qk + h * sd + j0 + tid];
            const float bt = it_sigmoid(beta[t * ba_ts + h]);
            const float g = it_mul(it_softplus(it_add(alpha[t * ba_ts + h], dt[h])), a[h]);
            const float eg = it_expf(g);
            float s = 0.f;
#pragma unroll 8
            for (int i = 0; i < sd; i++) { const float r = it_mul(row[i], eg); row[i] = r; s = it_add(s, it_mul(r, ks[i])); }
            const float delta = it_mul(it_sub(v, s), bt);
            float acc = 0.f;
#pragma unroll 8
            for (int i = 0; i < sd; i++) { const float r = it_add(row[i], it_mul(ks[i], delta)); row[i] = r; acc = it_add(acc, it_mul(r, qs[i])); }
            o[t * o_ts + h * sd + j0 + tid] = it_mul(acc, scale);
        }
        if (t < nck) { __syncthreads(); tile_out(ck + t * ck_stride + ((size_t)h * sd + j0) * sd); }
    }
    __syncthreads();
    tile_out(m);
}

// act = silu(g) * u (src/cpu.rs:183)
__global__ void k_silu_mul(const float* g, const float* u, float* out, size_t n) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i < n) out[i] = it_mul(it_silu(g[i]), u[i]);
}

// New K / V rows into the cache: f16 round-to-nearest-even for the trunk (src/cpu.rs:22, :258), f32 for the MTP head.
template <typename T> __device__ __forceinline__ T kv_pack(float v);
template <> __device__ __forceinline__ __half kv_pack<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float kv_pack<float>(float v) { return v; }
__device__ __forceinline__ float2 kv_get2(const __half* p) { return __half22float2(*reinterpret_cast<const __half2*>(p)); }
__device__ __forceinline__ float2 kv_get2(const float* p) { return *reinterpret_cast<const float2*>(p); }

template <typename T>
__global__ void k_kv_store(const float* k, const float* v, size_t ts, T* kc, T* vc, int kvd, int hd, int slot0, const int* pos_ptr) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    if (pos_ptr) slot0 += *pos_ptr;
    const int t = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= kvd) return;
    const size_t ki = sizeof(T) == 2 ? it_kc_index(slot0 + t, i / hd, i % hd, kvd / hd, hd) : (size_t)(slot0 + t) * kvd + i;   // the f16 K cache is tiled
    kc[ki] = kv_pack<T>(k[t * ts + i]);
    const size_t vi = sizeof(T) == 2 ? it_vc_index(slot0 + t, i / hd, i % hd, kvd / hd, hd) : (size_t)(slot0 + t) * kvd + i;       // the f16 V cache is tiled too
    vc[vi] = kv_pack<T>(v[t * ts + i]);
}

// ---------------------------------------------------------------- fused kernels of the decode path (up to 8 rows)
// The three kernels below run the same per-element arithmetic as the separate kernels above, in the same order; they
// only remove kernel boundaries, which dominate a decode step's support work.

// Attention input block in one launch: per-head rmsnorm of q and k (src/cpu.rs:252-256), rope on both (:145-162), and the
// new K / V rows rounded to f16 into the cache (:258).  One warp per job and row: jobs [0, nh) are q heads (q and gate
// interleaved per head, 2*hd apart), [nh, nh + nkv) k heads, [nh + nkv, nh + 2 nkv) v heads (copy only).
__global__ void __launch_bounds__(128) k_attn_prep(float* qkv, size_t ts, int nh, int nkv, int hd, const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                                                   int pos0, const int* pos_ptr, int n_rot, float theta_scale, int s0, int s1, int s2, int s3,
                                                   __half* kc, __half* vc, int slot0) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    __shared__ float buf[4][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int job = blockIdx.x * 4 + warp, t = blockIdx.y, kvd = nkv * hd;
    if (job >= nh + 2 * nkv) return;
    if (pos_ptr) { const int p = *pos_ptr; pos0 += p; slot0 += p; }
    float* row = qkv + t * ts;
    if (job >= nh + nkv) {                                   // v head: into the cache as it is
        const int kh = job - nh - nkv; const float* v = row + (size_t)nh * 2 * hd + kvd + kh * hd;
        for (int i = lane; i < hd; i += 32) vc[it_vc_index(slot0 + t, kh, i, nkv, hd)] = __float2half_rn(v[i]);
        return;
    }
    const bool is_q = job < nh;
    float* x = is_q ? row + (size_t)job * 2 * hd : row + (size_t)nh * 2 * hd + (job - nh) * hd;
    const float* w = is_q ? q_norm : k_norm;
    for (int i = lane; i < hd; i += 32) buf[warp][i] = x[i];
    __syncwarp();
    float s = 0.f;
    if (lane == 0) {
#pragma unroll 8
        for (int i = 0; i < hd; i++) s = it_add(s, it_mul(buf[warp][i], buf[warp][i]));
    }
    s = __shfl_sync(0xffffffffu, s, 0);
    const float sc = it_div(1.0f, it_sqrt(it_add(it_div(s, (float)hd), eps)));
    for (int i = lane; i < hd; i += 32) buf[warp][i] = it_mul(it_mul(buf[warp][i], sc), w[i]);
    __syncwarp();
    const int half = n_rot / 2, sect = s0 + s1 + s2 + s3;
    for (int i = lane; i < half; i += 32) {
        float theta = (float)(pos0 + t);
        for (int k = 0; k < i; k++) theta = it_mul(theta, theta_scale);
        const int sector = sect > 0 ? i % sect : 0;
        const bool use_e = sect > 0 && !((sector % 3 == 1 && sector < 3 * s1) || (sector % 3 == 2 && sector < 3 * s2) || (sector % 3 == 0 && sector < 3 * s0));
        float sn, cs; it_sincosf(use_e ? 0.0f : theta, &sn, &cs);
        const float x0 = buf[warp][i], x1 = buf[warp][i + half];
        buf[warp][i] = it_sub(it_mul(x0, cs), it_mul(x1, sn));
        buf[warp][i + half] = it_add(it_mul(x0, sn), it_mul(x1, cs));
    }
    __syncwarp();
    if (is_q) { for (int i = lane; i < hd; i += 32) x[i] = buf[warp][i]; }
    else { const int kh = job - nh; for (int i = lane; i < hd; i += 32) { x[i] = buf[warp][i]; kc[it_kc_index(slot0 + t, kh, i, nkv, hd)] = __float2half_rn(buf[warp][i]); } }
}

// Delta-net input block in one launch.  CTAs [0, cd/sd): causal conv + SiLU + state shift of one head-wide run of sd
// channels (src/cpu.rs:203-212) and, for the q and k heads (the first 2*nk runs), the l2norm of the run (:214), the
// squares added by one thread in index order.  CTAs after those: one dense f32 row of ssm_beta / ssm_alpha each
// (src/cpu.rs:36-43, :199-200), with the accumulation order of k_dense_rows.  nt <= 8.
__global__ void __launch_bounds__(256) k_conv_l2_dense(const float* mixed, size_t m_ts, const float* __restrict__ cw, float* state, float* out, size_t o_ts, int cd, int kk, int sd, int nk,
                                                       int nt, float* ck, size_t ck_stride, int nck, float eps,
                                                       const float* __restrict__ w0, const float* __restrict__ w1, int rows, int cols, const float* x, size_t x_ts,
                                                       float* y0, float* y1, size_t y_ts) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    __shared__ float vals[8][256];
    __shared__ float scs[8];
    __shared__ double wsum[8];
    const int nruns = cd / sd, tid = threadIdx.x;
    if ((int)blockIdx.x >= nruns) {
        const int job = blockIdx.x - nruns, r = job % (2 * rows), t = job / (2 * rows), rowi = r < rows ? r : r - rows;
        const float* wr = (r < rows ? w0 : w1) + (size_t)rowi * cols; const float* xr = x + t * x_ts;
        double s = 0.0;
#pragma unroll 4
        for (int i = tid; i < cols; i += 256) s += (double)it_mul(wr[i], xr[i]);
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
        if ((tid & 31) == 0) wsum[tid >> 5] = s;
        __syncthreads();
        if (tid == 0) { double tt = wsum[0]; for (int k = 1; k < 8; k++) tt += wsum[k]; (r < rows ? y0 : y1)[t * y_ts + rowi] = (float)tt; }
        return;
    }
    const int run = blockIdx.x, ch = run * sd + tid;
    const bool norm = run < 2 * nk;
    if (tid < sd) {
        float st[8];
        for (int i = 0; i < kk - 1; i++) st[i] = state[(size_t)i * cd + ch];
        for (int t = 0; t < nt; t++) {
            const float m = mixed[t * m_ts + ch];
            float s = 0.f;
            for (int i = 0; i < kk; i++) s = it_add(s, it_mul(i < kk - 1 ? st[i] : m, cw[ch * kk + i]));
            const float v = it_silu(s);
            if (norm) vals[t][tid] = v; else out[t * o_ts + ch] = v;
            for (int i = 0; i < kk - 2; i++) st[i] = st[i + 1];
            st[kk - 2] = m;
            if (t < nck) for (int i = 0; i < kk - 1; i++) ck[t * ck_stride + (size_t)i * cd + ch] = st[i];
        }
        for (int i = 0; i < kk - 1; i++) state[(size_t)i * cd + ch] = st[i];
    }
    if (!norm) return;
    __syncthreads();
    const int warp = tid >> 5, lane = tid & 31;
    if (warp < nt && lane == 0) {                            // warp t: the squares of row t in index order
        float s = 0.f;
#pragma unroll 8
        for (int i = 0; i < sd; i++) s = it_add(s, it_mul(vals[warp][i], vals[warp][i]));
        scs[warp] = it_div(1.0f, fmaxf(it_sqrt(s), eps));
    }
    __syncthreads();
    if (tid < sd) for (int t = 0; t < nt; t++) out[t * o_ts + ch] = it_mul(vals[t][tid], scs[t]);
}

// Gated delta rule (src/cpu.rs:215-232) and the gated per-head norm that follows it (:233-237) in one launch: one CTA
// per head.  Warps 0..SD/32-1 own one state row per thread and walk the tokens; four extra warps take turns to norm the
// outputs of a row (squares added by one lane in index order), weight them and multiply by silu(z) while the row owners
// are already on the next rows (one output buffer per norm warp).  State layout [head][j][i] as on the CPU.
// The head's SD x SD state sits in shared memory for the whole launch, rows unpadded, the 16-byte pieces of row j
// stored at piece index ^ (j & 7): both the coalesced 16-byte moves of the tile and the 16-byte accesses of the row
// owners are then free of bank conflicts.
constexpr int GN_NW = 4;      // norm warps of k_gdn_norm: warp w norms the rows t with t % GN_NW == w out of its own output buffer
template <int SD>
__global__ void __launch_bounds__(SD + 32 * GN_NW, 1) k_gdn_norm(const float* co, size_t co_ts, const float* beta, const float* alpha, size_t ba_ts, const float* __restrict__ dt, const float* __restrict__ a,
                                                      float* state, float* o, size_t o_ts, int nk, int qk, int nt, float* ck, size_t ck_stride, int nck,
                                                      const float* __restrict__ nw, float eps, const float* z, size_t z_ts) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    extern __shared__ __align__(16) float tile[];      // [SD][SD] swizzled rows, then o[GN_NW][SD], the gates of every token, the q / k / v rows of every token
    constexpr int PPR = SD / 4;                         // 16-byte pieces per row
    const int h = blockIdx.x, tid = threadIdx.x, kh = h % nk;
    float* os = tile + SD * SD; float* bts = os + GN_NW * SD; float* egs = bts + IT_GDN_MAXROWS; float* rows = egs + IT_GDN_MAXROWS;      // rows: [nt][3][SD]
    // named barriers: 1 = the row owners among themselves; 2 + w = "the outputs of a row are in buffer w" (the owners arrive,
    // norm warp w waits); 2 + GN_NW + w = "buffer w has been read" (norm warp w arrives, the owners wait before they
    // write the buffer again, GN_NW rows later).  One norm pass (a 128-long ordered sum by one lane, a division, a square
    // root and four silu per lane) takes about three times as long as the owners need for a row: four warps take turns.
    auto owners_sync = [] { asm volatile("bar.sync 1, %0;" :: "n"(SD) : "memory"); };
    auto bar_sync = [](int id) { asm volatile("bar.sync %0, %1;" :: "r"(id), "n"(SD + 32) : "memory"); };
    auto bar_arrive = [](int id) { asm volatile("bar.arrive %0, %1;" :: "r"(id), "n"(SD + 32) : "memory"); };
    if (tid >= SD) {
        // ---- norm warps: row t's outputs -> o, behind the owners
        const int lane = (tid - SD) & 31, w = (tid - SD) >> 5;
        float zr[SD / 32], wr[SD / 32], ov[SD / 32];
#pragma unroll
        for (int i = 0; i < SD / 32; i++) wr[i] = nw[lane + 32 * i];
        const float* ob = os + w * SD;
        for (int t = w; t < nt; t += GN_NW) {
#pragma unroll
            for (int i = 0; i < SD / 32; i++) zr[i] = z[t * z_ts + h * SD + lane + 32 * i];      // in flight while the owners compute
            bar_sync(2 + w);
#pragma unroll
            for (int i = 0; i < SD / 32; i++) ov[i] = ob[lane + 32 * i];
            float sc = 0.f;
            if (lane == 0) {
                float s = 0.f;
#pragma unroll 16
                for (int i = 0; i < SD; i++) s = it_add(s, it_mul(ob[i], ob[i]));
                sc = it_div(1.0f, it_sqrt(it_add(it_div(s, (float)SD), eps)));
            }
            sc = __shfl_sync(0xffffffffu, sc, 0);
            bar_arrive(2 + GN_NW + w);                  // every lane has read what it needs of the buffer
#pragma unroll
            for (int i = 0; i < SD / 32; i++) o[t * o_ts + h * SD + lane + 32 * i] = it_mul(it_mul(it_mul(ov[i], sc), wr[i]), it_silu(zr[i]));
        }
        return;
    }
    float* m = state + (size_t)h * SD * SD;
    auto piece = [&](int j, int c) { return reinterpret_cast<float4*>(tile + j * SD + ((c ^ (j & 7)) << 2)); };
    auto tile_out = [&](float* dst) {
#pragma unroll 8
        for (int f = tid; f < SD * PPR; f += SD) reinterpret_cast<float4*>(dst)[f] = *piece(f / PPR, f % PPR);
    };
    // Everything the pass reads is staged once: the head's state tile and the q, k, v rows of all nt tokens, as
    // asynchronous 16-byte copies that are all in flight together; meanwhile thread t forms token t's gates
    // (sigmoid(beta), exp(softplus(alpha + dt) * a)), which depend on no state.  The token loop then touches neither
    // global memory nor an elementary function.
#pragma unroll 8
    for (int f = tid; f < SD * PPR; f += SD)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((unsigned)__cvta_generic_to_shared(piece(f / PPR, f % PPR))), "l"(reinterpret_cast<const float4*>(m) + f));
    for (int f = tid; f < nt * 3 * PPR; f += SD) {
        const int t = f / (3 * PPR), seg = (f / PPR) % 3, pc = f % PPR;
        const float* src = co + t * co_ts + (seg == 0 ? kh * SD : seg == 1 ? qk + kh * SD : 2 * qk + h * SD) + 4 * pc;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((unsigned)__cvta_generic_to_shared(rows + (t * 3 + seg) * SD + 4 * pc)), "l"(src));
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (int t = tid; t < nt; t += SD) {
        bts[t] = it_sigmoid(beta[t * ba_ts + h]);
        egs[t] = it_expf(it_mul(it_softplus(it_add(alpha[t * ba_ts + h], dt[h])), a[h]));
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    owners_sync();
    // Each owner keeps its state row in registers for the whole launch (the loops below are fully unrolled); the shared
    // tile only stages the coalesced moves from and to global memory.  x[] holds the row already multiplied by the decay
    // of the token that is about to use it.  The two ordered sums of a token, s = sum_i x[i] * k[i] and
    // acc = sum_i st[i] * q[i], are kept in the CPU's index order; what is interleaved is acc of token t with s of token
    // t + 1: both read the state after token t and do not depend on each other, so the two dependent chains of additions
    // run side by side instead of one after the other.
    float x[SD];
    const float scale = it_div(1.0f, it_sqrt((float)SD));
    float s = 0.f;
    {
        const float eg = egs[0]; const float* k0 = rows + SD;
#pragma unroll
        for (int cc = 0; cc < PPR; cc++) {
            const float4 r = *piece(tid, cc); const float4 k4 = *reinterpret_cast<const float4*>(k0 + 4 * cc);
            x[4 * cc] = it_mul(r.x, eg); x[4 * cc + 1] = it_mul(r.y, eg); x[4 * cc + 2] = it_mul(r.z, eg); x[4 * cc + 3] = it_mul(r.w, eg);
            s = it_add(s, it_mul(x[4 * cc], k4.x)); s = it_add(s, it_mul(x[4 * cc + 1], k4.y)); s = it_add(s, it_mul(x[4 * cc + 2], k4.z)); s = it_add(s, it_mul(x[4 * cc + 3], k4.w));
        }
    }
    if (nck > 0) owners_sync();                         // every owner has its row in registers before a checkpoint reuses the tile
    for (int t = 0; t < nt; t++) {
        const float* qt = rows + (t * 3) * SD; const float* kt = qt + SD;
        const float delta = it_mul(it_sub(qt[2 * SD + tid], s), bts[t]);
        const bool last = t + 1 == nt, cks = t < nck;
        const float egn = last ? 1.0f : egs[t + 1];
        const float* kn = last ? kt : kt + 3 * SD;
        float acc = 0.f, s2 = 0.f;
        if (cks && t > 0) owners_sync();                // the copy of the previous checkpoint out of the tile is over
#pragma unroll
        for (int cc = 0; cc < PPR; cc++) {
            const float4 k4 = *reinterpret_cast<const float4*>(kt + 4 * cc), q4 = *reinterpret_cast<const float4*>(qt + 4 * cc), n4 = *reinterpret_cast<const float4*>(kn + 4 * cc);
            const float s0 = it_add(x[4 * cc], it_mul(k4.x, delta)), s1 = it_add(x[4 * cc + 1], it_mul(k4.y, delta));
            const float s2v = it_add(x[4 * cc + 2], it_mul(k4.z, delta)), s3 = it_add(x[4 * cc + 3], it_mul(k4.w, delta));
            acc = it_add(acc, it_mul(s0, q4.x)); acc = it_add(acc, it_mul(s1, q4.y)); acc = it_add(acc, it_mul(s2v, q4.z)); acc = it_add(acc, it_mul(s3, q4.w));
            if (cks) *piece(tid, cc) = make_float4(s0, s1, s2v, s3);       // checkpoint: the state after row t, through the tile
            // after the last token the factor is 1 (the product is then the state itself, bit for bit) and s2 is not used
            x[4 * cc] = it_mul(s0, egn); x[4 * cc + 1] = it_mul(s1, egn); x[4 * cc + 2] = it_mul(s2v, egn); x[4 * cc + 3] = it_mul(s3, egn);
            s2 = it_add(s2, it_mul(x[4 * cc], n4.x)); s2 = it_add(s2, it_mul(x[4 * cc + 1], n4.y)); s2 = it_add(s2, it_mul(x[4 * cc + 2], n4.z)); s2 = it_add(s2, it_mul(x[4 * cc + 3], n4.w));
        }
        const int slot = t % GN_NW;
        if (t >= GN_NW) bar_sync(2 + GN_NW + slot);     // the norm warp has read row t - GN_NW out of this buffer
        os[slot * SD + tid] = it_mul(acc, scale);
        bar_arrive(2 + slot);
        if (cks) { owners_sync(); tile_out(ck + t * ck_stride + (size_t)h * SD * SD); }
        s = s2;
    }
    if (nck > 0) owners_sync();
#pragma unroll
    for (int cc = 0; cc < PPR; cc++) *piece(tid, cc) = make_float4(x[4 * cc], x[4 * cc + 1], x[4 * cc + 2], x[4 * cc + 3]);
    owners_sync();
    tile_out(m);
}

// Causal gated attention for one (head, row) per CTA in the CPU's order (src/cpu.rs:262-272): every score is a
// sequential dot over the head dimension, the exponentials are added in ascending position order by one thread,
// every output element accumulates w[p] * v[p][j] in ascending position order, then * sigmoid(gate).  Loads are
// issued in batches ahead of the dependent additions so that the chains run at arithmetic, not memory, latency.
template <typename T> struct KvVec;
template <> struct KvVec<__half> { static constexpr int N = 8; using V = uint4;
    static __device__ __forceinline__ void unpack(const V& v, float* f) { const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) { const float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; } } };
template <> struct KvVec<float> { static constexpr int N = 4; using V = float4;
    static __device__ __forceinline__ void unpack(const V& v, float* f) { f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; } };

template <typename T>
__global__ void __launch_bounds__(1024) k_attention(const float* q, size_t q_hs, size_t q_ts, const float* gate, const T* __restrict__ kc, const T* __restrict__ vc,
                                                    int kvd, int hd, int nh, int nkv, int slot0, const int* pos_ptr, float* out, size_t o_ts) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    extern __shared__ float sc[];              // [n] scores, then q[hd]
    __shared__ float red[32]; __shared__ float s_sum;
    if (pos_ptr) slot0 += *pos_ptr;
    const int h = blockIdx.x, t = blockIdx.y, n = slot0 + t + 1, kh = h / (nh / nkv), tid = threadIdx.x;
    float* qs = sc + ((n + 3) & ~3);
    const float* qh = q + t * q_ts + h * q_hs;
    for (int j = tid; j < hd; j += 1024) qs[j] = qh[j];
    __syncthreads();
    // the first V chunks are requested now and arrive while the scores are computed
    constexpr int RING = 4, CHUNK_BYTES = 32768;
    T* ring = reinterpret_cast<T*>(reinterpret_cast<unsigned char*>(qs + hd) + ((16u - ((unsigned)__cvta_generic_to_shared(qs + hd) & 15u)) & 15u));
    const int cp = CHUNK_BYTES / (hd * (int)sizeof(T));              // positions per chunk
    const int ppr = hd * (int)sizeof(T) / 16, epp = 16 / (int)sizeof(T);   // 16-byte pieces per row, elements per piece
    const int nchunks = (n + cp - 1) / cp;
    auto issue = [&](int c) {
        if (c < nchunks) {
            const int p0 = c * cp, rows = min(cp, n - p0);
            T* dst = ring + (size_t)(c % RING) * cp * hd;
            for (int i = tid; i < rows * ppr; i += 1024) {
                const int r = i / ppr, k = i % ppr;
                const unsigned d = (unsigned)__cvta_generic_to_shared(dst + r * hd + k * epp);
                const T* vsrc = sizeof(T) == 2 ? vc + it_vc_index(p0 + r, kh, k * epp, nkv, hd) : vc + (size_t)(p0 + r) * kvd + kh * hd + k * epp;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(d), "l"(vsrc));
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (int c = 0; c < RING - 1; c++) issue(c);
    const float scale = it_div(1.0f, it_sqrt((float)hd));
    constexpr int VN = KvVec<T>::N; using Vec = typename KvVec<T>::V;
    const int nvec = hd / VN;                  // vectors per K row
    float mx = -INFINITY;
    for (int p = tid; p < n; p += 1024) {
        // f16 cache: tiled (piece v of 32 consecutive positions is contiguous: the loads of a warp are coalesced); f32 cache: rows
        const Vec* kp = sizeof(T) == 2 ? reinterpret_cast<const Vec*>(kc + it_kc_index(p, kh, 0, nkv, hd)) : reinterpret_cast<const Vec*>(kc + (size_t)p * kvd + kh * hd);
        const int vstep = sizeof(T) == 2 ? 32 : 1;     // distance between consecutive pieces of one position, in vectors
        float s = 0.f;
        for (int v0 = 0; v0 < nvec; v0 += 8) {
            Vec buf[8];
#pragma unroll
            for (int u = 0; u < 8; u++) if (v0 + u < nvec) buf[u] = kp[(v0 + u) * vstep];
            asm volatile("" ::: "memory");       // all eight loads are in flight before the first dependent add
#pragma unroll
            for (int u = 0; u < 8; u++) if (v0 + u < nvec) {
                float f[VN], qv[VN]; KvVec<T>::unpack(buf[u], f);
#pragma unroll
                for (int i = 0; i < VN; i += 4) *reinterpret_cast<float4*>(qv + i) = *reinterpret_cast<const float4*>(qs + (v0 + u) * VN + i);
#pragma unroll
                for (int i = 0; i < VN; i++) s = it_add(s, it_mul(qv[i], f[i]));
            }
        }
        s = it_mul(s, scale); sc[p] = s; mx = fmaxf(mx, s);
    }
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, m));
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int k = 1; k < 32; k++) mx = fmaxf(mx, red[k]);
    for (int p = tid; p < n; p += 1024) sc[p] = it_expf(it_sub(sc[p], mx));
    __syncthreads();
    if (tid == 0) { float s = 0.f;
#pragma unroll 8
        for (int p = 0; p < n; p++) s = it_add(s, sc[p]);
        s_sum = s; }
    __syncthreads();
    const float sum = s_sum;
    for (int p = tid; p < n; p += 1024) sc[p] = it_div(sc[p], sum);
    __syncthreads();
    // Output: thread j adds w[p] * v[p][j] in ascending p.  The V rows of the head stream through a ring of shared-memory
    // chunks filled with 16-byte asynchronous copies by all threads, several chunks ahead, so the chain of additions
    // never waits for global memory.
    float acc0 = 0.f, acc1 = 0.f;
    for (int c = 0; c < nchunks; c++) {
        issue(c + RING - 1);
        asm volatile("cp.async.wait_group %0;" :: "n"(RING - 1) : "memory");
        __syncthreads();
        if (2 * tid < hd) {                                  // two outputs per thread: elements 2*tid, 2*tid + 1
            const int p0 = c * cp, rows = min(cp, n - p0);
            const T* src = ring + (size_t)(c % RING) * cp * hd + 2 * tid;
            int r = 0;
            for (; r + 4 <= rows; r += 4) {
                const float4 w4 = *reinterpret_cast<const float4*>(sc + p0 + r);
                const float w[4] = { w4.x, w4.y, w4.z, w4.w };
                float2 v[4];
#pragma unroll
                for (int u = 0; u < 4; u++) v[u] = kv_get2(src + (r + u) * hd);
#pragma unroll
                for (int u = 0; u < 4; u++) { acc0 = it_add(acc0, it_mul(w[u], v[u].x)); acc1 = it_add(acc1, it_mul(w[u], v[u].y)); }
            }
            for (; r < rows; r++) { const float w = sc[p0 + r]; const float2 v = kv_get2(src + r * hd); acc0 = it_add(acc0, it_mul(w, v.x)); acc1 = it_add(acc1, it_mul(w, v.y)); }
        }
        __syncthreads();
    }
    if (2 * tid < hd) {
        const float* gp = gate + t * q_ts + h * q_hs + 2 * tid;
        float* op = out + t * o_ts + h * hd + 2 * tid;
        op[0] = it_mul(acc0, it_sigmoid(gp[0])); op[1] = it_mul(acc1, it_sigmoid(gp[1]));
    }
}

#define KCHK(name) do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) return it_fail(IT_ECUDA, "launch %s: %s", name, cudaGetErrorString(e__)); } while (0)

}  // namespace

int it_sup_embed(it_ctx* c, const uint32_t* toks_dev, const float* table, int e, int nt, float* x) {
    it_note_op(c); it_pdl(k_embed, dim3(dim3(4, nt)), dim3(256), 0, c->stream, toks_dev, table, e, x); KCHK("embed"); return IT_OK;
}
int it_sup_rmsnorm_wide(it_ctx* c, const float* x, size_t xs, const float* w, int n, float eps, float* out, size_t os, int nt) {
    it_note_op(c); it_pdl(k_rmsnorm_wide, dim3(nt), dim3(256), 0, c->stream, x, xs, w, n, eps, out, os); KCHK("rmsnorm_wide"); return IT_OK;
}
int it_sup_norm_head(it_ctx* c, const float* in, size_t in_hs, size_t in_ts, float* out, size_t out_hs, size_t out_ts, int n, int nheads, const float* w, int mode, float eps,
                     const float* z, size_t z_hs, size_t z_ts, int nt) {
    if (n > 256) return it_fail(IT_EINVAL, "head norm width %d exceeds 256", n);
    it_note_op(c); it_pdl(k_norm_head, dim3(dim3((nheads + 3) / 4, nt)), dim3(128), 0, c->stream, in, in_hs, in_ts, out, out_hs, out_ts, n, nheads, w, mode, eps, z, z_hs, z_ts); KCHK("norm_head"); return IT_OK;
}
int it_sup_rope(it_ctx* c, float* x, size_t hs, size_t ts, int nheads, int nt, int pos0, const int* pos_ptr, int n_rot, float theta_scale, const int* sec) {
    it_note_op(c); const int n = nheads * (n_rot / 2);
    it_pdl(k_rope, dim3(dim3((n + 127) / 128, nt)), dim3(128), 0, c->stream, x, hs, ts, nheads, pos0, pos_ptr, n_rot, theta_scale, sec[0], sec[1], sec[2], sec[3]); KCHK("rope"); return IT_OK;
}
int it_sup_conv(it_ctx* c, const float* mixed, size_t m_ts, const float* w, float* state, float* out, size_t o_ts, int cd, int kk, int nt, float* ck, size_t ck_stride, int nck) {
    if (kk < 2 || kk > 9) return it_fail(IT_EINVAL, "conv kernel size %d not supported", kk);
    it_note_op(c);
    if (nt > 8 && nck == 0) {   // prompt passes: rows in parallel
        it_pdl(k_conv_wide, dim3((cd + 127) / 128), dim3(128, 8), 0, c->stream, mixed, m_ts, w, state, out, o_ts, cd, kk, nt); KCHK("conv_wide"); return IT_OK;
    }
    it_pdl(k_conv, dim3((cd + 127) / 128), dim3(128), 0, c->stream, mixed, m_ts, w, state, out, o_ts, cd, kk, nt, ck, ck_stride, nck); KCHK("conv"); return IT_OK;
}
int it_sup_dense_rows(it_ctx* c, const float* w0, const float* w1, int rows, int cols, const float* x, size_t x_ts, float* y0, float* y1, size_t y_ts, int nt) {
    it_note_op(c); it_pdl(k_dense_rows, dim3(dim3(2 * rows, nt)), dim3(256), 0, c->stream, w0, w1, rows, cols, x, x_ts, y0, y1, y_ts); KCHK("dense_rows"); return IT_OK;
}
int it_sup_gdn(it_ctx* c, const float* co, size_t co_ts, const float* beta, const float* alpha, size_t ba_ts, const float* dt, const float* a, float* state, float* o, size_t o_ts,
               int nv, int nk, int sd, int qk, int nt, float* ck, size_t ck_stride, int nck) {
    if (sd % 32 != 0) return it_fail(IT_EINVAL, "ssm state size %d is not a multiple of 32", sd);
    it_note_op(c); const size_t smem = (32 * (sd + 1) + 2 * sd) * sizeof(float);
    it_pdl(k_gdn, dim3(dim3(nv, sd / 32)), dim3(128), smem, c->stream, co, co_ts, beta, alpha, ba_ts, dt, a, state, o, o_ts, nk, sd, qk, nt, ck, ck_stride, nck); KCHK("gdn"); return IT_OK;
}
int it_sup_silu_mul(it_ctx* c, const float* g, const float* u, float* out, size_t n) {
    it_note_op(c); it_pdl(k_silu_mul, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, c->stream, g, u, out, n); KCHK("silu_mul"); return IT_OK;
}
int it_sup_kv_store(it_ctx* c, const float* k, const float* v, size_t ts, void* kc, void* vc, int kvd, int hd, int slot0, const int* pos_ptr, int nt, int f16) {
    it_note_op(c);
    if (f16) it_pdl(k_kv_store<__half>, dim3(dim3((kvd + 255) / 256, nt)), dim3(256), 0, c->stream, k, v, ts, (__half*)kc, (__half*)vc, kvd, hd, slot0, pos_ptr);
    else it_pdl(k_kv_store<float>, dim3(dim3((kvd + 255) / 256, nt)), dim3(256), 0, c->stream, k, v, ts, (float*)kc, (float*)vc, kvd, hd, slot0, pos_ptr);
    KCHK("kv_store"); return IT_OK;
}
// Positions one attention launch can score: the row of scores, the q row and the ring of V chunks share the CTA's
// dynamic shared memory (IT_ATT_SMEM bytes at most).
#define IT_ATT_SMEM (220 * 1024)
#define IT_ATT_RING (4 * 32768)
int it_sup_attention_max_positions(int hd) {
    const long long room = (long long)IT_ATT_SMEM - IT_ATT_RING - 16 - (long long)hd * 4;
    return room < 4 ? 0 : (int)(room / 4 / 4 * 4);
}
int it_sup_attention(it_ctx* c, const float* q, size_t q_hs, size_t q_ts, const float* gate, const void* kc, const void* vc, int kvd, int hd, int nh, int nkv, int slot0, const int* pos_ptr, int max_pos, float* out, size_t o_ts, int nt, int f16) {
    it_note_op(c);
    // shared memory is sized for the longest row of scores this launch can meet (max_pos when the position is read on the device)
    const int positions = pos_ptr ? max_pos : slot0 + nt;
    const size_t smem = (((size_t)positions + 3) / 4 * 4 + hd) * sizeof(float) + 16 + IT_ATT_RING;   // scores, q, ring of V chunks
    if (hd > 1024 || (hd * (f16 ? 2 : 4)) % 16) return it_fail(IT_EINVAL, "attention: head dimension %d is not supported", hd);
    if (smem > IT_ATT_SMEM) return it_fail(IT_EINVAL, "attention over %d positions exceeds the shared-memory budget (%d positions at head dimension %d)", positions, it_sup_attention_max_positions(hd), hd);
    static bool set[2][16] = {};    // the attribute is per device
    if (!set[f16 ? 1 : 0][c->device & 15]) {
        if (f16) IT_CUDA(cudaFuncSetAttribute(k_attention<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, IT_ATT_SMEM));
        else IT_CUDA(cudaFuncSetAttribute(k_attention<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, IT_ATT_SMEM));
        set[f16 ? 1 : 0][c->device & 15] = true;
    }
    if (f16) it_pdl(k_attention<__half>, dim3(dim3(nh, nt)), dim3(1024), smem, c->stream, q, q_hs, q_ts, gate, (const __half*)kc, (const __half*)vc, kvd, hd, nh, nkv, slot0, pos_ptr, out, o_ts);
    else it_pdl(k_attention<float>, dim3(dim3(nh, nt)), dim3(1024), smem, c->stream, q, q_hs, q_ts, gate, (const float*)kc, (const float*)vc, kvd, hd, nh, nkv, slot0, pos_ptr, out, o_ts);
    KCHK("attention"); return IT_OK;
}

int it_sup_attn_prep(it_ctx* c, float* qkv, size_t ts, int nh, int nkv, int hd, const float* q_norm, const float* k_norm, float eps, int pos0, const int* pos_ptr,
                     int n_rot, float theta_scale, const int* sections, void* kc, void* vc, int nt) {
    it_note_op(c);
    it_pdl(k_attn_prep, dim3(dim3((nh + 2 * nkv + 3) / 4, nt)), dim3(128), 0, c->stream, qkv, ts, nh, nkv, hd, q_norm, k_norm, eps, pos0, pos_ptr, n_rot, theta_scale,
           sections[0], sections[1], sections[2], sections[3], (__half*)kc, (__half*)vc, pos0);
    KCHK("attn_prep"); return IT_OK;
}
int it_sup_conv_l2_dense(it_ctx* c, const float* mixed, size_t m_ts, const float* cw, float* state, float* out, size_t o_ts, int cd, int kk, int sd, int nk, int nt,
                         float* ck, size_t ck_stride, int nck, float eps, const float* w0, const float* w1, int rows, int cols, const float* x, size_t x_ts,
                         float* y0, float* y1, size_t y_ts) {
    it_note_op(c);
    it_pdl(k_conv_l2_dense, dim3(dim3(cd / sd + 2 * rows * nt)), dim3(256), 0, c->stream, mixed, m_ts, cw, state, out, o_ts, cd, kk, sd, nk, nt, ck, ck_stride, nck, eps,
           w0, w1, rows, cols, x, x_ts, y0, y1, y_ts);
    KCHK("conv_l2_dense"); return IT_OK;
}
int it_sup_gdn_norm(it_ctx* c, const float* co, size_t co_ts, const float* beta, const float* alpha, size_t ba_ts, const float* dt, const float* a, float* state, float* o, size_t o_ts,
                    int nv, int nk, int sd, int qk, int nt, float* ck, size_t ck_stride, int nck, const float* nw, float eps, const float* z, size_t z_ts) {
    if (sd != 128) return it_fail(IT_EINVAL, "gdn_norm: the fused kernel is built for a state size of 128");
    it_note_op(c);
    if (nt > IT_GDN_MAXROWS || (reinterpret_cast<uintptr_t>(co) & 15) || co_ts % 4 || qk % 4) return it_fail(IT_EINVAL, "gdn_norm: %d rows or an unaligned conv output", nt);
    const size_t smem = ((size_t)sd * sd + GN_NW * sd + 2 * IT_GDN_MAXROWS + (size_t)nt * 3 * sd) * sizeof(float);
    static bool set[16] = {};       // the attribute is per device
    if (!set[c->device & 15]) { IT_CUDA(cudaFuncSetAttribute(k_gdn_norm<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); set[c->device & 15] = true; }
    it_pdl(k_gdn_norm<128>, dim3(dim3(nv)), dim3(128 + 32 * GN_NW), smem, c->stream, co, co_ts, beta, alpha, ba_ts, dt, a, state, o, o_ts, nk, qk, nt, ck, ck_stride, nck, nw, eps, z, z_ts);
    KCHK("gdn_norm"); return IT_OK;
}
