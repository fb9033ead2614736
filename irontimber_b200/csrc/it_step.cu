// One greedy decode step of the decoder as ONE persistent kernel.
//
// The per-op schedule of a pass (it_engine_run.cu; the reference's run_chunk_v, src/vk/mod.rs:763-892) is a chain of about
// ten dependent kernels per layer.  At one activation row every kernel is a few microseconds long, so most of a step is
// spent draining and refilling the GPU at kernel boundaries, not streaming weights.  This kernel runs the whole step with
// one CTA per SM that stays resident: the ops of the schedule become phases separated by a barrier over the grid, and a
// producer warp per CTA streams the CTA's share of every ternary matrix of the step, in schedule order, into a ring in
// shared memory.  Weights never depend on activations, so the producer is only ever held back by the ring being full:
// while the CTAs sit in a short phase (Hadamard, delta rule, attention) or in a barrier, the ring already holds the first
// 150 KB per SM of the next matrix, and the HBM stream does not drain at op boundaries.
//
// Arithmetic: every phase performs, per output element, the operations of the kernel it replaces in the same order (the
// kernels of it_support.cu, it_hadamard.cuh, it_matvec_t2.cu), so logits, state and picks are bit-identical to the per-op
// schedule; tests run both and compare.  What changes is only which thread does the work and where intermediate values live.
//
// Phases of a delta-net layer (attention layer in brackets), one grid barrier after each:
//   A  rmsnorm -> Hadamard -> q8k of the residual row                         5 CTAs (one per 1024-block)
//   B  [qkv | gate] ([q | k | v]) ternary matvec                              all CTAs
//   C  conv + l2norm + dense beta/alpha rows + delta rule + gated norm        one CTA per value head
//      (q/k norms + rope + KV store + attention                               one CTA per head)
//   D  permuted Hadamard -> q8k of the block output                           6 CTAs
//   E  output projection, accumulating into the residual                      all CTAs
//   F  rmsnorm -> Hadamard -> q8k                                             5 CTAs
//   G  [gate | up] matvec                                                     all CTAs
//   H  silu(gate) * up -> Hadamard -> q8k                                     17 CTAs
//   I  down projection, accumulating into the residual                        all CTAs
// then output norm + Hadamard + q8k, the LM head with the greedy pick folded into its epilogue, and the pick's hand-over
// to the next step (token slot, position + 1).
//
// Every wait (mbarrier, grid barrier) is bounded; when one runs out the CTA raises the context's error flag and an abort
// word that makes every other CTA leave at its next barrier, drains its copies and returns (IT_ETIMEOUT on the host).
#include "it_engine.h"
#include "it_support.h"
#include "it_math.h"
#include "it_pipe.cuh"
#include "it_hadamard.cuh"
#include <algorithm>
#include <vector>

namespace {

constexpr int ST_CW = 8;                               // tiles per ring slot = warps per consumer group
constexpr int ST_NG = 2;                               // consumer groups; group j takes the chunks k of the CTA's stream with k % ST_NG == j
constexpr int ST_NCONS = ST_CW * ST_NG;                // consumer warps
constexpr int ST_CT = ST_NCONS * 32;                   // consumer threads
constexpr int ST_THREADS = ST_CT + 32;                 // + the producer warp
constexpr int ST_CHUNK = ST_CW * IT_TILE_BYTES;        // bytes of one ring slot
constexpr int ST_SMEM = 227 * 1024;                    // dynamic shared memory of the CTA
constexpr int ST_BARS = 1024;                          // bytes reserved for mbarriers and flags
constexpr int ST_SD = 128;                             // delta-rule state size this kernel is built for
constexpr int ST_VCHUNK = 16384;                       // bytes of one chunk of V rows in the attention phase (two chunks in flight)

struct StepLayer {
    const uint8_t *in_proj, *out_proj, *gate_up, *down;
    const float *attn_norm, *post_norm;
    const float *conv_w, *dt, *a, *beta, *alpha, *ssm_norm;
    float *conv_st, *ssm_st;
    const float *q_norm, *k_norm;
    __half *kc, *vc;
    int recurrent, in_rows;
};

struct StepParams {
    const StepLayer* layers; int n_layer;
    int e, ff, hd, nh, nkv, cd, inner, nv, nk, qk, conv_k, n_rot, n_vocab;
    float eps, theta_scale; int sec[4]; int v_grouped;
    float* arena; size_t x, xn, big1, o, hrow, logits, amx;
    int8_t* qs; float* qd; int32_t* qsum; size_t q_stride;
    const float *sg_e, *sg_inner, *sg_att, *sg_ff;
    const float *tok_embd, *output_norm; const uint8_t* output;
    uint32_t* toks; int* pos;
    unsigned* sync;                    // [0] arrivals, [1] arrivals at the end of the last launch, [2] abort word
    unsigned long long* partials;      // one greedy-pick partial per CTA
    int* error_flag;
    int slots, scratch;                // ring slots; bytes of the phase scratch that follows the ring
    int flags;                         // bit 0: the token is the previous pick (amx) instead of toks[0]; bit 1: hand the pick over (toks[0], pos + 1); bit 2: logits wanted
};

struct Pick { float v; unsigned i; };
__device__ __forceinline__ Pick pick_better(Pick a, Pick b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }

// Per-thread view of the CTA's state that every phase needs.
struct Cta {
    unsigned char* smem; unsigned char* scratch; unsigned bars; volatile int* abort_flag;
    int tid, warp, lane;
    int slot; unsigned ph; int kg;     // ring position of the consumers: next slot, its phase, (chunk index) % ST_NG
    unsigned target;                   // arrivals the next grid barrier waits for
};

__device__ __forceinline__ void cons_sync() { consumer_barrier<ST_CT>(); }

// Barrier over the grid (consumer threads only; the producer warp never takes part).  Writes made by any CTA before the
// barrier are visible to every CTA after it: thread 0 fences, announces the CTA with a release add, waits with acquire
// loads until every CTA of this round has arrived, and fences again before the CTA goes on.  Returns false when the step
// has been given up (by this CTA's own timeout or by another CTA's).
__device__ __forceinline__ bool grid_sync(const StepParams& P, Cta& c, int site) {
    cons_sync();
    if (c.tid == 0 && *c.abort_flag) atomicExch(P.sync + 2, 1u);      // a wait of this CTA ran out: tell the others
    if (c.tid == 0 && !*c.abort_flag) {
        c.target += gridDim.x;
        __threadfence();
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" :: "l"(P.sync) : "memory");
        const long long t0 = clock64();
        for (unsigned it = 0;; it++) {
            unsigned v; asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(P.sync) : "memory");
            if ((int)(v - c.target) >= 0) break;
            if ((it & 63u) == 63u) {
                if (*reinterpret_cast<volatile unsigned*>(P.sync + 2)) { *c.abort_flag = 1; break; }
                if (clock64() - t0 > WAIT_CLOCKS) { atomicExch(P.error_flag, 100 + site); atomicExch(P.sync + 2, 1u); *c.abort_flag = 1; break; }
            }
        }
        __threadfence();
    }
    cons_sync();
    return !*c.abort_flag;
}

// ---------------------------------------------------------------- producer
struct Ring { int s; unsigned ph; int issued; };
__device__ __forceinline__ bool produce_matrix(const StepParams& P, const Cta& c, Ring& r, const uint8_t* tiles, int nb, int rows, int* error_flag) {
    const int rgs = (rows + 31) / 32, cpr = (nb + ST_CW - 1) / ST_CW;
    for (int rg = blockIdx.x; rg < rgs; rg += gridDim.x) {
        const uint8_t* src = tiles + (size_t)rg * nb * IT_TILE_BYTES;
        for (int cq = 0; cq < cpr; cq++) {
            if (!mbar_wait(c.bars + 8 * (P.slots + r.s), r.ph ^ 1u, c.abort_flag, error_flag, 2)) return false;
            const int ntile = min(ST_CW, nb - cq * ST_CW);
            const unsigned bytes = (unsigned)ntile * IT_TILE_BYTES;
            mbar_expect_tx(c.bars + 8 * r.s, bytes);
            bulk_load(smem_u32(c.smem + r.s * ST_CHUNK), src + (size_t)cq * ST_CHUNK, bytes, c.bars + 8 * r.s);
            r.issued++;
            if (++r.s == P.slots) { r.s = 0; r.ph ^= 1u; }
        }
    }
    return true;
}
__device__ void producer(const StepParams& P, const Cta& c) {
    Ring r{0, 0u, 0};
    const int nb_e = P.e / 128;
    bool ok = true;
    for (int il = 0; il < P.n_layer && ok; il++) {
        const StepLayer& L = P.layers[il];
        ok = produce_matrix(P, c, r, L.in_proj, nb_e, L.in_rows, P.error_flag)
          && produce_matrix(P, c, r, L.out_proj, (L.recurrent ? P.inner : P.nh * P.hd) / 128, P.e, P.error_flag)
          && produce_matrix(P, c, r, L.gate_up, nb_e, 2 * P.ff, P.error_flag)
          && produce_matrix(P, c, r, L.down, P.ff / 128, P.e, P.error_flag);
    }
    if (ok && (P.flags & 4)) ok = produce_matrix(P, c, r, P.output, nb_e, P.n_vocab, P.error_flag);
    if (!ok || *c.abort_flag) {
        // leave only after every copy this thread started has landed (each wait bounded by the clock limit)
        const int first = r.issued > P.slots ? r.issued - P.slots : 0;
        for (int k = first; k < r.issued; k++) {
            const long long t0 = clock64();
            while (!mbar_test(c.bars + 8 * (k % P.slots), (unsigned)(k / P.slots) & 1u) && clock64() - t0 < WAIT_CLOCKS) { }
        }
    }
}

// ---------------------------------------------------------------- ternary matvec phase (one activation row)
// Same arithmetic as k_matvec_t2<1> (it_matvec_t2.cu): per 32 x 128 tile eight mma.m16n8k32 (u8 x s8) give the exact
// integer block sums; one warp per row group then adds (d_w * d_x) * float(S - sum128) in ascending block order.
struct MvSmem { int x, dx, s128, terms, wsc, plane, total; };
__host__ __device__ inline MvSmem mv_layout(int nb) {
    MvSmem L; int o = 0;
    L.plane = nb * 32 + 4;
    L.x = o; o += nb * 128 + 16;
    L.dx = o; o += (nb / 2) * 4;
    L.s128 = o; o += nb * 4;
    o = (o + 15) & ~15;
    L.terms = o; o += 2 * L.plane * 4;
    o = (o + 15) & ~15;
    L.wsc = o; o += 2 * nb * 64;
    L.total = o;
    return L;
}

template <bool PICK>
__device__ void matvec_phase(const StepParams& P, Cta& c, int nb, int rows, size_t y_off, int accum, Pick& best) {
    const MvSmem L = mv_layout(nb);
    int8_t* xs = reinterpret_cast<int8_t*>(c.scratch + L.x);
    float* dxs = reinterpret_cast<float*>(c.scratch + L.dx);
    int* sss = reinterpret_cast<int*>(c.scratch + L.s128);
    const int tid = c.tid, warp = c.warp, lane = c.lane;
    {   // the q8k row, its scales and block sums, once per CTA (written by other CTAs before the last barrier: read through L2)
        for (int ch = tid; ch < nb * 8; ch += ST_CT) cp_async16(xs + 16 * ch, P.qs + 16 * ch);
        for (int i = tid; i < nb / 2; i += ST_CT) dxs[i] = __ldcg(P.qd + i);
        for (int i = tid; i < nb; i += ST_CT) sss[i] = __ldcg(P.qsum + i);
        cp_async_wait_all();
        cons_sync();
    }
    const int g = lane >> 2, t = lane & 3;
    const int group = warp / ST_CW, wi = warp % ST_CW;
    const int rgs = (rows + 31) / 32, cpr = (nb + ST_CW - 1) / ST_CW;
    float* arena = P.arena;
    int i = 0;
    for (int rg = blockIdx.x; rg < rgs; rg += gridDim.x, i++) {
        int* tbuf = reinterpret_cast<int*>(c.scratch + L.terms) + (i & 1) * L.plane;
        uint2* wsc = reinterpret_cast<uint2*>(c.scratch + L.wsc + (i & 1) * nb * 64);
        for (int cq = 0; cq < cpr; cq++) {
            const bool mine = c.kg == group;
            const int cs = c.slot; const unsigned cph = c.ph;
            if (++c.slot == P.slots) { c.slot = 0; c.ph ^= 1u; }
            if (++c.kg == ST_NG) c.kg = 0;
            if (!mine) continue;
            const int b = cq * ST_CW + wi;
            const bool ready = mbar_wait(c.bars + 8 * cs, cph, c.abort_flag, P.error_flag, 3);
            if (ready && b < nb) {
                const unsigned char* tile = c.smem + cs * ST_CHUNK + wi * IT_TILE_BYTES;
                const uint4 wa = *reinterpret_cast<const uint4*>(tile + 16 * lane);
                const uint4 wb = *reinterpret_cast<const uint4*>(tile + 512 + 16 * lane);
                const uint4* xp = reinterpret_cast<const uint4*>(xs + 128 * b + 32 * t);
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
                if (t == 0) {
                    // rows g, g + 8, g + 16, g + 24 side by side, still carrying the factors 1, 4, 16, 64: row r of the tile sits at 4 * (r & 7) + (r >> 3)
                    *reinterpret_cast<int4*>(tbuf + b * 32 + 4 * g) = make_int4(cx[0], cx[2], cy[0], cy[2]);
                    wsc[b * 8 + g] = *reinterpret_cast<const uint2*>(tile + 1024 + 8 * g);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(c.bars + 8 * (P.slots + cs));     // the slot may be refilled
        }
        cons_sync();                                                     // every block sum of this row group is in shared memory
        if (warp == (i % ST_NCONS)) {
            // ordered f32 accumulation, one matrix row per lane, while the other warps go on with the next row group
            const int row = rg * 32 + lane;
            if (row < rows) {
                const int* icol = tbuf + 4 * (lane & 7) + (lane >> 3);
                const __half* hs = reinterpret_cast<const __half*>(wsc) + 4 * (lane & 7) + (lane >> 3);
                const int sh = 2 * (lane >> 3);
                float sum = 0.f;
#pragma unroll 8
                for (int b = 0; b < nb; b++)
                    sum = __fadd_rn(sum, __fmul_rn(__fmul_rn(__half2float(hs[b * 32]), dxs[b >> 1]), (float)((icol[b * 32] >> sh) - sss[b])));
                if (accum) sum = __fadd_rn(__ldcg(arena + y_off + row), sum);
                __stcg(arena + y_off + row, sum);
                if (PICK) best = pick_better(best, Pick{ sum, (unsigned)row });
            }
        }
    }
    // the warp that added the last row group may still be reading the terms: the barrier that follows (grid_sync) orders that
}

// ---------------------------------------------------------------- Hadamard + q8k phases
__device__ __forceinline__ void had_phase(const StepParams& P, const Cta& c, int nblocks, const float* in, const float* signs,
                                          unsigned perm_hd, unsigned perm_nk, unsigned perm_rep, const it_had_prologue& pro) {
    if ((int)blockIdx.x < nblocks && c.tid < 256) {
        it_had_smem& sm = *reinterpret_cast<it_had_smem*>(c.scratch);
        it_hadamard_block<true>(sm, (unsigned)c.tid, blockIdx.x, 0, in, 0, 0, nullptr, 0, 0, signs, 1, 0, perm_hd, perm_nk, perm_rep,
                                P.qs, P.qd, P.qsum, P.q_stride, pro);
    }
}

// ---------------------------------------------------------------- delta-net block of one value head
// conv + SiLU (+ l2norm of the q and k runs), the dense beta / alpha rows, the delta rule and the gated norm for head
// blockIdx.x, in the operation order of k_conv_l2_dense and k_gdn_norm (it_support.cu; src/cpu.rs:199-237).  The q / k
// runs of a key group are recomputed by each of the value heads that share it.  The new conv state of the runs this CTA
// is responsible for (its own v run; the q and k runs when it is the first head of the group) is returned in `keep`
// and stored after the next grid barrier, when no CTA reads the old state any more.
struct ConvKeep { int ch; float st[8]; };
__device__ void gdn_phase(const StepParams& P, const StepLayer& L, const Cta& c, ConvKeep& keep) {
    constexpr int SD = ST_SD, PPR = SD / 4;
    const int h = blockIdx.x, tid = c.tid, warp = c.warp, lane = c.lane, kh = h % P.nk, kk = P.conv_k, cd = P.cd;
    float* tile = reinterpret_cast<float*>(c.scratch);               // [SD][SD], 16-byte pieces of row j stored at piece index ^ (j & 7)
    float* vals = tile + SD * SD;                                    // [3][SD]: q, k, v runs after conv + SiLU
    float* os = vals + 3 * SD;                                       // [SD] delta-rule outputs
    float* scs = os + SD;                                            // [2] l2norm scales, [2] beta, alpha
    double* wsum = reinterpret_cast<double*>(scs + 8);               // [16] warp sums of the two dense rows
    const float* A = P.arena;
    auto piece = [&](int j, int cc) { return reinterpret_cast<float4*>(tile + j * SD + ((cc ^ (j & 7)) << 2)); };
    float* m = L.ssm_st + (size_t)h * SD * SD;
    for (int f = tid; f < SD * PPR; f += ST_CT) cp_async16(piece(f / PPR, f % PPR), reinterpret_cast<const float4*>(m) + f);
    asm volatile("cp.async.commit_group;" ::: "memory");
    keep.ch = -1;
    if (tid < 3 * SD) {
        const int r = tid / SD, cc = tid % SD;
        const int ch = (r == 0 ? kh * SD : r == 1 ? P.qk + kh * SD : 2 * P.qk + h * SD) + cc;
        float st[8];
        for (int i = 0; i < kk - 1; i++) st[i] = L.conv_st[(size_t)i * cd + ch];
        const float mx = __ldcg(A + P.big1 + ch);
        float s = 0.f;
        for (int i = 0; i < kk; i++) s = it_add(s, it_mul(i < kk - 1 ? st[i] : mx, L.conv_w[ch * kk + i]));
        vals[r * SD + cc] = it_silu(s);
        if (r == 2 || h < P.nk) {
            keep.ch = ch;
            for (int i = 0; i < kk - 2; i++) keep.st[i] = st[i + 1];
            keep.st[kk - 2] = mx;
        }
    }
    {   // dense rows: warps 0-7 beta row h, warps 8-15 alpha row h (order of k_dense_rows)
        const int half = tid >> 8, t8 = tid & 255;
        const float* wr = (half ? L.alpha : L.beta) + (size_t)h * P.e; const float* xr = A + P.xn;
        double s = 0.0;
#pragma unroll 4
        for (int i = t8; i < P.e; i += 256) s += (double)it_mul(wr[i], __ldcg(xr + i));
#pragma unroll
        for (int mm = 16; mm >= 1; mm >>= 1) s += __shfl_xor_sync(0xffffffffu, s, mm);
        if (lane == 0) wsum[warp] = s;
    }
    cons_sync();
    if (lane == 0 && warp < 2) {                                     // l2norm of the q run (warp 0) and the k run (warp 1): squares in index order
        const float* v = vals + warp * SD;
        float s = 0.f;
#pragma unroll 8
        for (int i = 0; i < SD; i++) s = it_add(s, it_mul(v[i], v[i]));
        scs[warp] = it_div(1.0f, fmaxf(it_sqrt(s), P.eps));
    } else if (lane == 0 && warp < 4) {
        const double* ws = wsum + (warp - 2) * 8;
        double tt = ws[0];
        for (int k = 1; k < 8; k++) tt += ws[k];
        scs[warp] = (float)tt;                                       // scs[2] = beta, scs[3] = alpha
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    cons_sync();
    if (tid < SD) {
        const float q = it_mul(vals[tid], scs[0]), k = it_mul(vals[SD + tid], scs[1]);
        asm volatile("bar.sync 3, %0;" :: "n"(SD) : "memory");       // every owner has read the raw q / k values
        vals[tid] = q; vals[SD + tid] = k;
        asm volatile("bar.sync 3, %0;" :: "n"(SD) : "memory");
        const float* qs = vals; const float* ks = vals + SD;
        const float v = vals[2 * SD + tid];
        const float bt = it_sigmoid(scs[2]);
        const float gg = it_mul(it_softplus(it_add(scs[3], L.dt[h])), L.a[h]);
        const float eg = it_expf(gg);
        const float scale = it_div(1.0f, it_sqrt((float)SD));
        float s = 0.f;
#pragma unroll 4
        for (int cc = 0; cc < PPR; cc++) {
            float4 r = *piece(tid, cc); const float4 k4 = *reinterpret_cast<const float4*>(ks + 4 * cc);
            r.x = it_mul(r.x, eg); r.y = it_mul(r.y, eg); r.z = it_mul(r.z, eg); r.w = it_mul(r.w, eg);
            *piece(tid, cc) = r;
            s = it_add(s, it_mul(r.x, k4.x)); s = it_add(s, it_mul(r.y, k4.y)); s = it_add(s, it_mul(r.z, k4.z)); s = it_add(s, it_mul(r.w, k4.w));
        }
        const float delta = it_mul(it_sub(v, s), bt);
        float acc = 0.f;
#pragma unroll 4
        for (int cc = 0; cc < PPR; cc++) {
            float4 r = *piece(tid, cc); const float4 k4 = *reinterpret_cast<const float4*>(ks + 4 * cc), q4 = *reinterpret_cast<const float4*>(qs + 4 * cc);
            r.x = it_add(r.x, it_mul(k4.x, delta)); r.y = it_add(r.y, it_mul(k4.y, delta)); r.z = it_add(r.z, it_mul(k4.z, delta)); r.w = it_add(r.w, it_mul(k4.w, delta));
            *piece(tid, cc) = r;
            acc = it_add(acc, it_mul(r.x, q4.x)); acc = it_add(acc, it_mul(r.y, q4.y)); acc = it_add(acc, it_mul(r.z, q4.z)); acc = it_add(acc, it_mul(r.w, q4.w));
        }
        os[tid] = it_mul(acc, scale);
    }
    cons_sync();
    // the new state back to global memory (coalesced 16-byte stores by every thread) while warp 0 norms the outputs
    for (int f = tid; f < SD * PPR; f += ST_CT) reinterpret_cast<float4*>(m)[f] = *piece(f / PPR, f % PPR);
    if (warp == 0) {
        float sc = 0.f;
        if (lane == 0) {
            float s = 0.f;
#pragma unroll 8
            for (int i = 0; i < SD; i++) s = it_add(s, it_mul(os[i], os[i]));
            sc = it_div(1.0f, it_sqrt(it_add(it_div(s, (float)SD), P.eps)));
        }
        sc = __shfl_sync(0xffffffffu, sc, 0);
        const float* z = A + P.big1 + cd + h * SD;                   // the gate rows follow the qkv rows in the stacked output
        float* o = P.arena + P.o + h * SD;
#pragma unroll
        for (int i = 0; i < SD / 32; i++) {
            const int j = lane + 32 * i;
            __stcg(o + j, it_mul(it_mul(it_mul(os[j], sc), L.ssm_norm[j]), it_silu(__ldcg(z + j))));
        }
    }
}

// ---------------------------------------------------------------- attention block of one head
// q / k head norms, rope, the new K / V entries and the causal gated attention of head blockIdx.x in the operation order of
// k_attn_prep and k_attention (it_support.cu; src/cpu.rs:252-272).  The k and v rows of the new position are recomputed by
// each of the heads that share the KV head and used from shared memory (after the same f16 rounding the cache applies);
// the first head of the group stores them into the cache.
__device__ void attn_phase(const StepParams& P, const StepLayer& L, const Cta& c) {
    const int h = blockIdx.x, tid = c.tid, warp = c.warp, lane = c.lane, hd = P.hd, nkv = P.nkv, kvd = nkv * hd;
    const int rep = P.nh / nkv, kh = h / rep;
    const bool writer = h % rep == 0;
    const int pos = *P.pos, n = pos + 1;
    float* sc = reinterpret_cast<float*>(c.scratch);                 // [n] scores
    float* qs = sc + ((n + 3) & ~3);                                 // [hd] q head after norm + rope
    float* kl = qs + hd;                                             // [hd] k row of the new position as the cache holds it
    float* vl = kl + hd;                                             // [hd] v row of the new position as the cache holds it
    float* red = vl + hd;                                            // [32] + the sum
    __half* ring = reinterpret_cast<__half*>(reinterpret_cast<unsigned char*>(red + 48) + ((16u - (smem_u32(red + 48) & 15u)) & 15u));
    const float* row = P.arena + P.big1;
    const float* qh = row + (size_t)h * 2 * hd; const float* gate = qh + hd;
    const __half* kc = L.kc; const __half* vc = L.vc;
    const int cp = ST_VCHUNK / (hd * 2), ppr = hd * 2 / 16;          // positions per chunk of V rows; 16-byte pieces per row
    const int nold = n - 1, nchunks = (nold + cp - 1) / cp;
    auto issue = [&](int ck) {
        if (ck < nchunks) {
            const int p0 = ck * cp, rows = min(cp, nold - p0);
            __half* dst = ring + (size_t)(ck & 1) * cp * hd;
            for (int i = tid; i < rows * ppr; i += ST_CT) {
                const int r = i / ppr, k = i % ppr;
                cp_async16(dst + r * hd + k * 8, vc + (size_t)(p0 + r) * kvd + kh * hd + k * 8);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    issue(0);
    if (warp < 2) {
        // warp 0: q head; warp 1: k head.  rmsnorm with the squares added by one lane in index order, weight, rope.
        float* buf = warp == 0 ? qs : kl;
        const float* x = warp == 0 ? qh : row + (size_t)P.nh * 2 * hd + kh * hd;
        const float* w = warp == 0 ? L.q_norm : L.k_norm;
        for (int i = lane; i < hd; i += 32) buf[i] = __ldcg(x + i);
        __syncwarp();
        float s = 0.f;
        if (lane == 0) {
#pragma unroll 8
            for (int i = 0; i < hd; i++) s = it_add(s, it_mul(buf[i], buf[i]));
        }
        s = __shfl_sync(0xffffffffu, s, 0);
        const float scl = it_div(1.0f, it_sqrt(it_add(it_div(s, (float)hd), P.eps)));
        for (int i = lane; i < hd; i += 32) buf[i] = it_mul(it_mul(buf[i], scl), w[i]);
        __syncwarp();
        const int half = P.n_rot / 2, sect = P.sec[0] + P.sec[1] + P.sec[2] + P.sec[3];
        for (int i = lane; i < half; i += 32) {
            float theta = (float)pos;
            for (int k = 0; k < i; k++) theta = it_mul(theta, P.theta_scale);
            const int sector = sect > 0 ? i % sect : 0;
            const bool use_e = sect > 0 && !((sector % 3 == 1 && sector < 3 * P.sec[1]) || (sector % 3 == 2 && sector < 3 * P.sec[2]) || (sector % 3 == 0 && sector < 3 * P.sec[0]));
            float sn, cs; it_sincosf(use_e ? 0.0f : theta, &sn, &cs);
            const float x0 = buf[i], x1 = buf[i + half];
            buf[i] = it_sub(it_mul(x0, cs), it_mul(x1, sn));
            buf[i + half] = it_add(it_mul(x0, sn), it_mul(x1, cs));
        }
        __syncwarp();
        if (warp == 1) for (int i = lane; i < hd; i += 32) {
            const __half hv = __float2half_rn(buf[i]);
            if (writer) const_cast<__half*>(kc)[it_kc_index(pos, kh, i, nkv, hd)] = hv;
            buf[i] = __half2float(hv);
        }
    } else if (warp == 2) {
        const float* v = row + (size_t)P.nh * 2 * hd + kvd + kh * hd;
        for (int i = lane; i < hd; i += 32) {
            const __half hv = __float2half_rn(__ldcg(v + i));
            if (writer) const_cast<__half*>(vc)[(size_t)pos * kvd + kh * hd + i] = hv;
            vl[i] = __half2float(hv);
        }
    }
    cons_sync();
    const float scale = it_div(1.0f, it_sqrt((float)hd));
    const int nvec = hd / 8;
    float mx = -INFINITY;
    for (int p = tid; p < n; p += ST_CT) {
        float s = 0.f;
        if (p < nold) {
            const uint4* kp = reinterpret_cast<const uint4*>(kc + it_kc_index(p, kh, 0, nkv, hd));    // piece v of 32 consecutive positions is contiguous
            for (int v0 = 0; v0 < nvec; v0 += 8) {
                uint4 buf[8];
#pragma unroll
                for (int u = 0; u < 8; u++) if (v0 + u < nvec) buf[u] = __ldcg(kp + (v0 + u) * 32);
#pragma unroll
                for (int u = 0; u < 8; u++) if (v0 + u < nvec) {
                    const __half2* hh = reinterpret_cast<const __half2*>(&buf[u]);
                    const float* qv = qs + (v0 + u) * 8;
#pragma unroll
                    for (int i2 = 0; i2 < 4; i2++) { const float2 f = __half22float2(hh[i2]); s = it_add(s, it_mul(qv[2 * i2], f.x)); s = it_add(s, it_mul(qv[2 * i2 + 1], f.y)); }
                }
            }
        } else {
#pragma unroll 8
            for (int j = 0; j < hd; j++) s = it_add(s, it_mul(qs[j], kl[j]));
        }
        s = it_mul(s, scale); sc[p] = s; mx = fmaxf(mx, s);
    }
#pragma unroll
    for (int mm = 16; mm >= 1; mm >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, mm));
    if (lane == 0) red[warp] = mx;
    cons_sync();
    mx = red[0];
#pragma unroll
    for (int k = 1; k < ST_NCONS; k++) mx = fmaxf(mx, red[k]);
    for (int p = tid; p < n; p += ST_CT) sc[p] = it_expf(it_sub(sc[p], mx));
    cons_sync();
    if (tid == 0) {
        float s = 0.f;
#pragma unroll 8
        for (int p = 0; p < n; p++) s = it_add(s, sc[p]);
        red[32] = s;
    }
    cons_sync();
    const float sum = red[32];
    for (int p = tid; p < n; p += ST_CT) sc[p] = it_div(sc[p], sum);
    cons_sync();
    // output element j adds w[p] * v[p][j] in ascending p; the V rows stream through two chunks in shared memory
    float acc0 = 0.f, acc1 = 0.f;
    for (int ck = 0; ck < nchunks; ck++) {
        issue(ck + 1);
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        cons_sync();
        if (2 * tid < hd) {
            const int p0 = ck * cp, rows = min(cp, nold - p0);
            const __half* src = ring + (size_t)(ck & 1) * cp * hd + 2 * tid;
            int r = 0;
            for (; r + 4 <= rows; r += 4) {
                const float w[4] = { sc[p0 + r], sc[p0 + r + 1], sc[p0 + r + 2], sc[p0 + r + 3] };
                float2 v[4];
#pragma unroll
                for (int u = 0; u < 4; u++) v[u] = __half22float2(*reinterpret_cast<const __half2*>(src + (r + u) * hd));
#pragma unroll
                for (int u = 0; u < 4; u++) { acc0 = it_add(acc0, it_mul(w[u], v[u].x)); acc1 = it_add(acc1, it_mul(w[u], v[u].y)); }
            }
            for (; r < rows; r++) { const float w = sc[p0 + r]; const float2 v = __half22float2(*reinterpret_cast<const __half2*>(src + r * hd)); acc0 = it_add(acc0, it_mul(w, v.x)); acc1 = it_add(acc1, it_mul(w, v.y)); }
        }
        cons_sync();
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (2 * tid < hd) {
        const float w = sc[nold];
        acc0 = it_add(acc0, it_mul(w, vl[2 * tid])); acc1 = it_add(acc1, it_mul(w, vl[2 * tid + 1]));
        float* op = P.arena + P.o + (size_t)h * hd + 2 * tid;
        __stcg(op, it_mul(acc0, it_sigmoid(__ldcg(gate + 2 * tid))));
        __stcg(op + 1, it_mul(acc1, it_sigmoid(__ldcg(gate + 2 * tid + 1))));
    }
}

// ---------------------------------------------------------------- the step
__global__ void __launch_bounds__(ST_THREADS, 1) k_decode_step(const __grid_constant__ StepParams P) {
    extern __shared__ __align__(128) unsigned char smem[];
    Cta c;
    c.smem = smem; c.scratch = smem + P.slots * ST_CHUNK;
    unsigned char* tail = c.scratch + P.scratch;
    c.bars = smem_u32(tail);                                         // full[s] at bars + 8 s, empty[s] at bars + 8 (slots + s)
    c.abort_flag = reinterpret_cast<volatile int*>(tail + ST_BARS - 16);
    c.tid = threadIdx.x; c.warp = c.tid >> 5; c.lane = c.tid & 31;
    c.slot = 0; c.ph = 0u; c.kg = 0;
    if (c.tid == 0) {
        *c.abort_flag = *reinterpret_cast<volatile unsigned*>(P.sync + 2) ? 1 : 0;      // a step that was given up earlier: nothing runs until the host has cleared the words
        for (int s = 0; s < P.slots; s++) { mbar_init(c.bars + 8 * s, 1); mbar_init(c.bars + 8 * (P.slots + s), ST_CW); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (*c.abort_flag) return;
    if (c.warp == ST_NCONS) { if (c.lane == 0) producer(P, c); return; }

    c.target = *reinterpret_cast<volatile unsigned*>(P.sync + 1);
    const int e = P.e, nb_e = e / 128;
    float* A = P.arena;
    const uint32_t tok = (P.flags & 1) ? __float_as_uint(*reinterpret_cast<volatile float*>(A + P.amx)) : *reinterpret_cast<volatile uint32_t*>(P.toks);
    const float* xsrc = P.tok_embd + (size_t)tok * e;               // the residual row of layer 0 is the embedding row (Model::embed, src/cpu.rs:118-122)
    ConvKeep keep; keep.ch = -1;
    Pick best{ -INFINITY, 0xffffffffu };
#define STEP_SYNC(site) do { if (!grid_sync(P, c, site)) goto done; } while (0)
    for (int il = 0; il < P.n_layer; il++) {
        const StepLayer& L = P.layers[il];
        {   // A: rmsnorm -> Hadamard -> q8k; the normed row is kept for the dense rows of a delta-net layer
            if (il == 0 && (int)blockIdx.x < nb_e / 8 && c.tid < 256)
                *reinterpret_cast<float4*>(A + P.x + blockIdx.x * 1024 + 4 * c.tid) = *reinterpret_cast<const float4*>(xsrc + blockIdx.x * 1024 + 4 * c.tid);
            it_had_prologue p; p.mode = 2; p.w = L.attn_norm; p.eps = P.eps; p.n = (unsigned)e; p.xn_out = L.recurrent ? A + P.xn : nullptr; p.xn_stride = e;
            had_phase(P, c, nb_e / 8, il == 0 ? xsrc : A + P.x, P.sg_e, 0, 0, 0, p);
        }
        STEP_SYNC(1);
        matvec_phase<false>(P, c, nb_e, L.in_rows, P.big1, 0, best);
        STEP_SYNC(2);
        if (L.recurrent) { if ((int)blockIdx.x < P.nv) gdn_phase(P, L, c, keep); }
        else if ((int)blockIdx.x < P.nh) attn_phase(P, L, c);
        STEP_SYNC(3);
        if (keep.ch >= 0) { for (int i = 0; i < P.conv_k - 1; i++) L.conv_st[(size_t)i * P.cd + keep.ch] = keep.st[i]; keep.ch = -1; }
        {   // D: Hadamard -> q8k of the block output (delta-net: with the value-head permutation)
            const int w = L.recurrent ? P.inner : P.nh * P.hd;
            const bool perm = L.recurrent && P.v_grouped;
            had_phase(P, c, w / 1024, A + P.o, L.recurrent ? P.sg_inner : P.sg_att, perm ? ST_SD : 0, perm ? P.nk : 0, perm ? P.nv / P.nk : 0, it_had_prologue{});
        }
        STEP_SYNC(4);
        matvec_phase<false>(P, c, (L.recurrent ? P.inner : P.nh * P.hd) / 128, e, P.x, 1, best);
        STEP_SYNC(5);
        { it_had_prologue p; p.mode = 2; p.w = L.post_norm; p.eps = P.eps; p.n = (unsigned)e; p.xn_out = nullptr; p.xn_stride = e;
          had_phase(P, c, nb_e / 8, A + P.x, P.sg_e, 0, 0, 0, p); }
        STEP_SYNC(6);
        matvec_phase<false>(P, c, nb_e, 2 * P.ff, P.big1, 0, best);
        STEP_SYNC(7);
        { it_had_prologue p; p.mode = 1; p.b = A + P.big1 + P.ff; p.b_stride = 2 * (size_t)P.ff;
          had_phase(P, c, P.ff / 1024, A + P.big1, P.sg_ff, 0, 0, 0, p); }
        STEP_SYNC(8);
        matvec_phase<false>(P, c, P.ff / 128, e, P.x, 1, best);
        STEP_SYNC(9);
    }
    {   // output norm (kept as the h_nextn row) -> Hadamard -> q8k
        it_had_prologue p; p.mode = 2; p.w = P.output_norm; p.eps = P.eps; p.n = (unsigned)e; p.xn_out = A + P.hrow; p.xn_stride = e;
        had_phase(P, c, (P.flags & 4) ? nb_e / 8 : 0, A + P.x, P.sg_e, 0, 0, 0, p);
        if (!(P.flags & 4) && blockIdx.x == 0 && c.tid < 256) {
            // no logits wanted: only the normed row, in the order of k_rmsnorm_wide
            it_had_smem& sm = *reinterpret_cast<it_had_smem*>(c.scratch);
            const float* x = A + P.x;
            float v[32];
#pragma unroll
            for (int k = 0; k < 32; k++) { const int j = c.tid + 256 * k; v[k] = j < e ? x[j] : 0.f; }
            float s = 0.f;
#pragma unroll
            for (int k = 0; k < 32; k++) if (c.tid + 256 * k < e) s = it_add(s, it_mul(v[k], v[k]));
#pragma unroll
            for (int mm = 16; mm >= 1; mm >>= 1) s = it_add(s, __shfl_xor_sync(0xffffffffu, s, mm));
            if (c.lane == 0) sm.wsum[c.warp] = s;
            it_had_sync();
            float t = sm.wsum[0];
#pragma unroll
            for (int k = 1; k < 8; k++) t = it_add(t, sm.wsum[k]);
            const float scl = it_div(1.0f, it_sqrt(it_add(it_div(t, (float)e), P.eps)));
#pragma unroll
            for (int k = 0; k < 32; k++) { const int j = c.tid + 256 * k; if (j < e) A[P.hrow + j] = it_mul(it_mul(v[k], scl), P.output_norm[j]); }
        }
    }
    if (P.flags & 4) {
        STEP_SYNC(10);
        matvec_phase<true>(P, c, nb_e, P.n_vocab, P.logits, 0, best);
        // greedy pick (first index of the maximum): lanes -> warp -> CTA -> one partial per CTA
#pragma unroll
        for (unsigned mm = 16; mm > 0; mm >>= 1) { Pick o{ __shfl_xor_sync(0xffffffffu, best.v, mm), __shfl_xor_sync(0xffffffffu, best.i, mm) }; best = pick_better(best, o); }
        cons_sync();                                                 // the ordered sums of the last row group are over: the terms can be overwritten
        Pick* sh = reinterpret_cast<Pick*>(c.scratch);
        if (c.lane == 0) sh[c.warp] = best;
        cons_sync();
        if (c.warp == 0) {
            Pick p = c.lane < ST_NCONS ? sh[c.lane] : Pick{ -INFINITY, 0xffffffffu };
#pragma unroll
            for (unsigned mm = 16; mm > 0; mm >>= 1) { Pick o{ __shfl_xor_sync(0xffffffffu, p.v, mm), __shfl_xor_sync(0xffffffffu, p.i, mm) }; p = pick_better(p, o); }
            if (c.lane == 0) P.partials[blockIdx.x] = ((unsigned long long)__float_as_uint(p.v) << 32) | p.i;
        }
        STEP_SYNC(11);
        if (blockIdx.x == 0 && c.warp == 0) {
            Pick q{ -INFINITY, 0xffffffffu };
            for (unsigned b = c.lane; b < gridDim.x; b += 32) { const unsigned long long u = __ldcg(P.partials + b); q = pick_better(q, Pick{ __uint_as_float((unsigned)(u >> 32)), (unsigned)u }); }
#pragma unroll
            for (unsigned mm = 16; mm > 0; mm >>= 1) { Pick o{ __shfl_xor_sync(0xffffffffu, q.v, mm), __shfl_xor_sync(0xffffffffu, q.i, mm) }; q = pick_better(q, o); }
            if (c.lane == 0) {
                const unsigned pick = q.i == 0xffffffffu ? 0u : q.i;
                A[P.amx] = __uint_as_float(pick);
                if (P.flags & 2) { P.toks[0] = pick; *P.pos += 1; }
            }
        }
    } else {
        STEP_SYNC(11);
    }
    if (blockIdx.x == 0 && c.tid == 0) P.sync[1] = c.target;        // every CTA has read the old value before its first arrival
done:
#undef STEP_SYNC
    return;
}

}  // namespace

// ---------------------------------------------------------------- host side
struct it_step_state {
    StepLayer* layers_dev;
    unsigned long long* partials;
    int grid, slots, scratch;
    bool cooperative;
};

static size_t step_scratch_bytes(const it_model_config& c) {
    const int widest = std::max(std::max(c.n_embd, c.n_ff), std::max(c.ssm_inner, c.n_head * c.head_dim));
    size_t s = (size_t)mv_layout(widest / 128).total;
    s = std::max(s, sizeof(it_had_smem));
    s = std::max(s, (size_t)(ST_SD * ST_SD + 4 * ST_SD + 8) * 4 + 16 * 8 + 64);
    s = std::max(s, ((size_t)c.ctx_len + 4 + 3 * c.head_dim + 48) * 4 + 16 + 2 * (size_t)ST_VCHUNK);
    return (s + 127) / 128 * 128;
}

// Whether this engine's decode step can run as the persistent kernel, and with which geometry.
int it_step_prepare(it_engine* e) {
    const it_model_config& c = e->cfg; it_ctx* cx = e->ctx;
    e->step = nullptr;
    { const char* v = getenv("IT_STEP_KERNEL"); if (v && atoi(v) == 0) return IT_OK; }
    if (e->world != 1) return IT_OK;                                  // row shards exchange results inside the per-op kernels
    if (c.ssm_state != ST_SD || c.conv_k > 9 || c.head_dim > 256 || c.head_dim % 8 || c.n_embd > 8192 || c.n_ff % 1024 || c.ssm_inner % 1024 || (c.n_head * c.head_dim) % 1024) return IT_OK;
    if (c.ssm_vheads > cx->sm_count || c.n_head > cx->sm_count || c.n_ff / 1024 > cx->sm_count || c.ssm_vheads % c.ssm_groups) return IT_OK;
    if (ST_VCHUNK / (c.head_dim * 2) < 1) return IT_OK;
    const size_t scratch = step_scratch_bytes(c);
    const long long ring = (long long)ST_SMEM - (long long)scratch - ST_BARS;
    int slots = (int)(ring / ST_CHUNK);
    if (slots > 48) slots = 48;                                       // 2 * slots mbarriers must fit the reserved bytes
    if (slots < 4) return IT_OK;
    IT_CUDA(cudaSetDevice(cx->device));
    static bool attr_set[16] = {};
    if (!attr_set[cx->device & 15]) { IT_CUDA(cudaFuncSetAttribute(k_decode_step, cudaFuncAttributeMaxDynamicSharedMemorySize, ST_SMEM)); attr_set[cx->device & 15] = true; }
    int per_sm = 0;
    IT_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_decode_step, ST_THREADS, (size_t)slots * ST_CHUNK + scratch + ST_BARS));
    if (per_sm < 1) return IT_OK;
    it_step_state* st = new it_step_state();
    st->grid = cx->sm_count; st->slots = slots; st->scratch = (int)scratch; st->layers_dev = nullptr; st->partials = nullptr;
    { const char* v = getenv("IT_STEP_COOP"); st->cooperative = !v || atoi(v) != 0; }
    std::vector<StepLayer> hl(c.n_layer);
    for (int il = 0; il < c.n_layer; il++) {
        const it_layer& l = e->layers[il]; StepLayer& s = hl[il]; memset(&s, 0, sizeof s);
        s.recurrent = l.recurrent ? 1 : 0; s.in_proj = l.in_proj->tiles; s.in_rows = (int)l.in_proj->rows;
        s.out_proj = (l.recurrent ? l.ssm_out : l.o)->tiles; s.gate_up = l.gate_up->tiles; s.down = l.ffn_down->tiles;
        s.attn_norm = l.attn_norm; s.post_norm = l.post_norm;
        s.conv_w = l.conv_w; s.dt = l.dt; s.a = l.a; s.beta = l.beta; s.alpha = l.alpha; s.ssm_norm = l.ssm_norm; s.conv_st = l.conv_st; s.ssm_st = l.ssm_st;
        s.q_norm = l.q_norm; s.k_norm = l.k_norm; s.kc = l.kc; s.vc = l.vc;
    }
    int r = it_engine_dev_alloc(e, (void**)&st->layers_dev, hl.size() * sizeof(StepLayer), false);
    if (r == IT_OK) r = it_engine_dev_alloc(e, (void**)&st->partials, (size_t)st->grid * sizeof(unsigned long long), true);
    if (r) { delete st; return r; }
    IT_CUDA(cudaMemcpyAsync(st->layers_dev, hl.data(), hl.size() * sizeof(StepLayer), cudaMemcpyHostToDevice, cx->stream));
    IT_CUDA(cudaStreamSynchronize(cx->stream));
    e->step = st;
    return IT_OK;
}
void it_step_release(it_engine* e) { delete e->step; e->step = nullptr; }

// Enqueues one step.  flags: 1 the token is the previous pick, 2 hand the pick over to the next step, 4 logits and pick wanted.
int it_step_launch(it_engine* e, int flags) {
    it_step_state* st = e->step; it_ctx* cx = e->ctx; const it_model_config& c = e->cfg; const it_arena_layout& L = e->lay;
    StepParams P; memset(&P, 0, sizeof P);
    P.layers = st->layers_dev; P.n_layer = c.n_layer;
    P.e = c.n_embd; P.ff = c.n_ff; P.hd = c.head_dim; P.nh = c.n_head; P.nkv = c.n_head_kv; P.cd = it_cfg_conv_dim(c); P.inner = c.ssm_inner; P.nv = c.ssm_vheads;
    P.nk = c.ssm_groups; P.qk = it_cfg_qk(c); P.conv_k = c.conv_k; P.n_rot = c.n_rot; P.n_vocab = c.n_vocab;
    P.eps = c.eps; P.theta_scale = e->theta_scale; for (int i = 0; i < 4; i++) P.sec[i] = c.rope_sections[i]; P.v_grouped = c.gdn_v_grouped;
    P.arena = cx->arena; P.x = L.x; P.xn = L.xn; P.big1 = L.big1; P.o = L.o; P.hrow = L.hrow; P.logits = L.logits; P.amx = L.amx;
    P.qs = e->q8->qs; P.qd = e->q8->d; P.qsum = e->q8->sum128; P.q_stride = e->q8->max_n;
    P.sg_e = cx->signs[(size_t)c.n_embd]; P.sg_inner = cx->signs[(size_t)c.ssm_inner]; P.sg_att = cx->signs[(size_t)c.n_head * c.head_dim]; P.sg_ff = cx->signs[(size_t)c.n_ff];
    P.tok_embd = e->tok_embd; P.output_norm = e->output_norm; P.output = e->output->tiles;
    P.toks = e->toks_dev; P.pos = e->pos_dev;
    P.sync = cx->grid_sync; P.partials = st->partials; P.error_flag = cx->error_flag_dev;
    P.slots = st->slots; P.scratch = st->scratch; P.flags = flags;
    it_note_op(cx);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)st->grid); cfg.blockDim = dim3(ST_THREADS); cfg.dynamicSmemBytes = (size_t)st->slots * ST_CHUNK + st->scratch + ST_BARS; cfg.stream = cx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative; attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = st->cooperative ? 1 : 0;
    IT_CUDA(cudaLaunchKernelEx(&cfg, k_decode_step, P));
    e->q8->n = (size_t)c.n_embd;
    return IT_OK;
}
