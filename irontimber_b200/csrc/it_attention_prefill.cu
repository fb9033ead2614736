// Causal gated attention of a prompt pass (many rows at known positions) over the trunk's tiled f16 caches.
//
// k_attention (it_support.cu) gives one CTA to every (head, row) pair, so the K and V rows of a KV head are read once per
// query head that shares it and once per row of the pass: at a 2048-token context a 64-row pass of the 27B shape moves
// 3 GB through L2 per layer.  Here one CTA takes G query heads of one KV group and RW consecutive rows of the pass: every
// K piece it loads feeds G * RW score chains and every V row G * RW output chains, which divides that traffic by G * RW
// and leaves the kernel bound by its additions.
//
// Arithmetic per (head, row) is that of k_attention, operation for operation (src/cpu.rs:262-272): every score a
// sequential dot over the head dimension in index order, scaled; the exponentials of (score - max) added in ascending
// position order by one thread; every weight divided by that sum; every output element accumulating w[p] * v[p][j] in
// ascending position order, then * sigmoid(gate).  Results are bit-identical to k_attention's.
#include "it_math.h"
#include "it_support.h"

namespace {

constexpr int AP_THREADS = 1024;
constexpr int AP_CHUNK_POS = 64;                    // positions per V chunk (two cache tiles)
constexpr int AP_RING = 2;                          // V chunks in flight
constexpr int AP_SMEM = 220 * 1024;

// HD: the head dimension as a compile-time constant (0: taken from the argument): with it every shared-memory address of the
// score loop is an immediate offset, which removes a third of the kernel's instructions (it is bound by instruction issue).
template <int G, int RW, int HD>
__global__ void __launch_bounds__(AP_THREADS, 1) k_attention_group(const float* q, size_t q_hs, size_t q_ts, const float* gate, const __half* __restrict__ kc, const __half* __restrict__ vc,
                                                                   int hd_arg, int nh, int nkv, int slot0, int nt, int npad, float* out, size_t o_ts) {
    IT_PDL_TRIGGER(); IT_PDL_WAIT();
    const int hd = HD ? HD : hd_arg;
    constexpr int Q = G * RW;                       // (head, row) pairs of this CTA; pair g * RW + rw
    extern __shared__ __align__(16) float sm[];
    __shared__ float red[Q][32];
    __shared__ float s_mx[Q], s_sum[Q];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h0 = blockIdx.x * G, t0 = blockIdx.y * RW, kh = h0 / (nh / nkv);
    const int rows_here = min(RW, nt - t0);
    const int nmax = slot0 + t0 + rows_here;        // positions the last row of this CTA sees
    float* sc = sm;                                 // [Q][npad] scores, then weights
    float* qs = sc + (size_t)Q * npad;              // [Q][hd]
    __half* ring = reinterpret_cast<__half*>(qs + Q * hd);            // [AP_RING][AP_CHUNK_POS][hd]
    auto n_of = [&](int rw) { return slot0 + t0 + rw + 1; };          // positions row t0 + rw sees (itself included)
    for (int i = tid; i < Q * hd; i += AP_THREADS) {
        const int qi = i / hd, j = i % hd, g = qi / RW, rw = qi % RW;
        qs[i] = rw < rows_here ? q[(size_t)(t0 + rw) * q_ts + (size_t)(h0 + g) * q_hs + j] : 0.f;
    }
    __syncthreads();
    // the first V chunks are requested now and arrive while the scores are computed
    const int ppr = hd / 8;                         // 16-byte pieces per V row
    const int nchunks = (nmax + AP_CHUNK_POS - 1) / AP_CHUNK_POS;
    auto issue = [&](int c) {
        if (c < nchunks) {
            const int p0 = c * AP_CHUNK_POS, rows = min(AP_CHUNK_POS, nmax - p0);
            __half* dst = ring + (size_t)(c % AP_RING) * AP_CHUNK_POS * hd;
            for (int i = tid; i < rows * ppr; i += AP_THREADS) {
                const int r = i / ppr, k = i % ppr;
                const unsigned d = (unsigned)__cvta_generic_to_shared(dst + r * hd + k * 8);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(d), "l"(vc + it_vc_index((size_t)(p0 + r), kh, k * 8, nkv, hd)));
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (int c = 0; c < AP_RING - 1; c++) issue(c);
    // ---- scores: a position per thread, Q chains side by side on every K piece
    const float scale = it_div(1.0f, it_sqrt((float)hd));
    float mx[Q];
#pragma unroll
    for (int qi = 0; qi < Q; qi++) mx[qi] = -INFINITY;
    for (int p = tid; p < nmax; p += AP_THREADS) {
        const uint4* kp = reinterpret_cast<const uint4*>(kc + it_kc_index((size_t)p, kh, 0, nkv, hd));    // piece v of this position: kp[32 v]
        float s[Q];
#pragma unroll
        for (int qi = 0; qi < Q; qi++) s[qi] = 0.f;
        for (int v0 = 0; v0 < ppr; v0 += 4) {
            uint4 buf[4];
#pragma unroll
            for (int u = 0; u < 4; u++) if (v0 + u < ppr) buf[u] = kp[(v0 + u) * 32];
#pragma unroll
            for (int u = 0; u < 4; u++) if (v0 + u < ppr) {
                const __half2* hh = reinterpret_cast<const __half2*>(&buf[u]);
                const float2 f0 = __half22float2(hh[0]), f1 = __half22float2(hh[1]), f2 = __half22float2(hh[2]), f3 = __half22float2(hh[3]);
#pragma unroll
                for (int qi = 0; qi < Q; qi++) {
                    const float4 qa = *reinterpret_cast<const float4*>(qs + qi * hd + (v0 + u) * 8), qb = *reinterpret_cast<const float4*>(qs + qi * hd + (v0 + u) * 8 + 4);
                    float a = s[qi];
                    a = it_add(a, it_mul(qa.x, f0.x)); a = it_add(a, it_mul(qa.y, f0.y)); a = it_add(a, it_mul(qa.z, f1.x)); a = it_add(a, it_mul(qa.w, f1.y));
                    a = it_add(a, it_mul(qb.x, f2.x)); a = it_add(a, it_mul(qb.y, f2.y)); a = it_add(a, it_mul(qb.z, f3.x)); a = it_add(a, it_mul(qb.w, f3.y));
                    s[qi] = a;
                }
            }
        }
#pragma unroll
        for (int qi = 0; qi < Q; qi++) {
            const int rw = qi % RW;
            if (rw < rows_here && p < n_of(rw)) { const float v = it_mul(s[qi], scale); sc[(size_t)qi * npad + p] = v; mx[qi] = fmaxf(mx[qi], v); }
        }
    }
#pragma unroll
    for (int qi = 0; qi < Q; qi++) {
        float m = mx[qi];
#pragma unroll
        for (int k = 16; k >= 1; k >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, k));
        if (lane == 0) red[qi][warp] = m;
    }
    __syncthreads();
    if (tid < Q) { float m = red[tid][0]; for (int k = 1; k < 32; k++) m = fmaxf(m, red[tid][k]); s_mx[tid] = m; }
    __syncthreads();
#pragma unroll
    for (int qi = 0; qi < Q; qi++) {
        const int rw = qi % RW;
        if (rw < rows_here) { const int n = n_of(rw); const float m = s_mx[qi]; float* row = sc + (size_t)qi * npad; for (int p = tid; p < n; p += AP_THREADS) row[p] = it_expf(it_sub(row[p], m)); }
    }
    __syncthreads();
    if (lane == 0 && warp < Q && warp % RW < rows_here) {              // one thread per pair adds its row in ascending position order
        const int n = n_of(warp % RW); const float* row = sc + (size_t)warp * npad;
        float s = 0.f;
#pragma unroll 8
        for (int p = 0; p < n; p++) s = it_add(s, row[p]);
        s_sum[warp] = s;
    }
    __syncthreads();
#pragma unroll
    for (int qi = 0; qi < Q; qi++) {
        const int rw = qi % RW;
        if (rw < rows_here) { const int n = n_of(rw); const float sum = s_sum[qi]; float* row = sc + (size_t)qi * npad; for (int p = tid; p < n; p += AP_THREADS) row[p] = it_div(row[p], sum); }
    }
    __syncthreads();
    // ---- output: thread (g, j) adds w[p] * v[p][j] in ascending p for each of its rows; the V rows stream through the ring
    const bool live = tid < G * hd;
    const int g = live ? tid / hd : 0, j = live ? tid % hd : 0;
    float acc[RW];
#pragma unroll
    for (int rw = 0; rw < RW; rw++) acc[rw] = 0.f;
    for (int c = 0; c < nchunks; c++) {
        issue(c + AP_RING - 1);
        asm volatile("cp.async.wait_group %0;" :: "n"(AP_RING - 1) : "memory");
        __syncthreads();
        if (live) {
            const int p0 = c * AP_CHUNK_POS;
            const __half* src = ring + (size_t)(c % AP_RING) * AP_CHUNK_POS * hd + j;
#pragma unroll
            for (int rw = 0; rw < RW; rw++) if (rw < rows_here) {
                const int rows = min(AP_CHUNK_POS, n_of(rw) - p0);      // may be <= 0 for the earlier row in the last chunk
                const float* w = sc + (size_t)(g * RW + rw) * npad + p0;
                float a = acc[rw];
                int r = 0;
                for (; r + 4 <= rows; r += 4) {
                    const float4 w4 = *reinterpret_cast<const float4*>(w + r);
                    const float v0 = __half2float(src[(r + 0) * hd]), v1 = __half2float(src[(r + 1) * hd]), v2 = __half2float(src[(r + 2) * hd]), v3 = __half2float(src[(r + 3) * hd]);
                    a = it_add(a, it_mul(w4.x, v0)); a = it_add(a, it_mul(w4.y, v1)); a = it_add(a, it_mul(w4.z, v2)); a = it_add(a, it_mul(w4.w, v3));
                }
                for (; r < rows; r++) a = it_add(a, it_mul(w[r], __half2float(src[r * hd])));
                acc[rw] = a;
            }
        }
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int rw = 0; rw < RW; rw++) if (rw < rows_here) {
            const float gv = gate[(size_t)(t0 + rw) * q_ts + (size_t)(h0 + g) * q_hs + j];
            out[(size_t)(t0 + rw) * o_ts + (size_t)(h0 + g) * hd + j] = it_mul(acc[rw], it_sigmoid(gv));
        }
    }
}

template <int G, int RW, int HD>
int launch_group_hd(it_ctx* c, const float* q, size_t q_hs, size_t q_ts, const float* gate, const __half* kc, const __half* vc, int hd, int nh, int nkv, int slot0, int nt, float* out, size_t o_ts) {
    const int npad = (slot0 + nt + 3) / 4 * 4;
    const size_t smem = ((size_t)G * RW * npad + (size_t)G * RW * hd) * sizeof(float) + (size_t)AP_RING * AP_CHUNK_POS * hd * sizeof(__half);
    if (smem > AP_SMEM) return 1;
    static bool set[16] = {};       // the attribute is per device
    if (!set[c->device & 15]) { IT_CUDA(cudaFuncSetAttribute(k_attention_group<G, RW, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, AP_SMEM)); set[c->device & 15] = true; }
    it_pdl(k_attention_group<G, RW, HD>, dim3(nh / G, (nt + RW - 1) / RW), dim3(AP_THREADS), smem, c->stream, q, q_hs, q_ts, gate, kc, vc, hd, nh, nkv, slot0, nt, npad, out, o_ts);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return it_fail(IT_ECUDA, "launch attention_group: %s", cudaGetErrorString(e));
    return IT_OK;
}

template <int G, int RW>
int launch_group(it_ctx* c, const float* q, size_t q_hs, size_t q_ts, const float* gate, const __half* kc, const __half* vc, int hd, int nh, int nkv, int slot0, int nt, float* out, size_t o_ts) {
    if (hd == 256) return launch_group_hd<G, RW, 256>(c, q, q_hs, q_ts, gate, kc, vc, hd, nh, nkv, slot0, nt, out, o_ts);
    return launch_group_hd<G, RW, 0>(c, q, q_hs, q_ts, gate, kc, vc, hd, nh, nkv, slot0, nt, out, o_ts);
}

}  // namespace

// Prompt-pass attention over the trunk's f16 caches.  Returns 1 (nothing launched) when no grouping of this shape fits
// the shared memory; the caller then uses it_sup_attention.
int it_sup_attention_prefill(it_ctx* c, const float* q, size_t q_hs, size_t q_ts, const float* gate, const void* kc, const void* vc, int hd, int nh, int nkv, int slot0,
                             float* out, size_t o_ts, int nt) {
    if (hd % 8 || nh % nkv) return 1;
    const int rep = nh / nkv;
    const __half* k = (const __half*)kc; const __half* v = (const __half*)vc;
    it_note_op(c);
    int r = 1;
    if (rep % 3 == 0 && 3 * hd <= AP_THREADS) {
        r = launch_group<3, 2>(c, q, q_hs, q_ts, gate, k, v, hd, nh, nkv, slot0, nt, out, o_ts);
        if (r == 1) r = launch_group<3, 1>(c, q, q_hs, q_ts, gate, k, v, hd, nh, nkv, slot0, nt, out, o_ts);
    } else if (rep % 2 == 0 && 2 * hd <= AP_THREADS) {
        r = launch_group<2, 2>(c, q, q_hs, q_ts, gate, k, v, hd, nh, nkv, slot0, nt, out, o_ts);
        if (r == 1) r = launch_group<2, 1>(c, q, q_hs, q_ts, gate, k, v, hd, nh, nkv, slot0, nt, out, o_ts);
    } else if (hd <= AP_THREADS) {
        r = launch_group<1, 2>(c, q, q_hs, q_ts, gate, k, v, hd, nh, nkv, slot0, nt, out, o_ts);
    }
    return r;
}
