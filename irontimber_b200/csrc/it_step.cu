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
#define IT_PIPE_OUTLINE_WAIT  // one copy of the retry loop of bounded waits
#define IT_MATH_OUTLINE      // one copy of division, square root and the elementary functions: this kernel's code size is its speed
#include "it_math.h"
#include "it_engine.h"
#include "it_support.h"
#include "it_pipe.cuh"
#include "it_hadamard.cuh"
#include <algorithm>
#include <vector>

namespace {

constexpr int ST_CW = 4;                               // warps per consumer group
constexpr int ST_NG = 3;                               // consumer groups; group j takes the chunks k of the CTA's stream with k % ST_NG == j
constexpr int ST_TPW = 2;                              // tiles a warp takes from a chunk (computed side by side)
constexpr int ST_TPC = ST_CW * ST_TPW;                 // tiles per chunk = per ring slot
constexpr int ST_NCONS = ST_CW * ST_NG;                // consumer warps
constexpr int ST_CT = ST_NCONS * 32;                   // consumer threads
constexpr int ST_NSUM = 2;                             // warps that only add the per-block terms of finished row groups in block order
constexpr int ST_TB = 3;                               // terms buffers (row groups in flight between the consumer warps and the sum warps)
constexpr int ST_THREADS = ST_CT + (ST_NSUM + 1) * 32; // + the sum warps + the producer warp
constexpr int ST_CHUNK = ST_TPC * IT_TILE_BYTES;       // bytes of one ring slot
constexpr int ST_SMEM = 227 * 1024;                    // dynamic shared memory of the CTA
constexpr int ST_BARS = 1024;                          // bytes reserved for mbarriers and flags
constexpr int ST_SD = 128;                             // delta-rule state size this kernel is built for

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
    unsigned long long* trace;         // optional: clock readings of CTA 0 and of the last CTA at every grid barrier (arrive, leave)
    int slots, scratch;                // ring slots; bytes of the phase scratch that follows the ring
    int attn_g;                        // CTAs that share an attention head
    float* att_sc; int att_stride; unsigned* att_cnt;   // per head: the scores its CTAs exchange [nh][att_stride], their arrival counter [nh]
    int had_base, attn_base;           // first CTA of the Hadamard blocks / of the attention heads (value heads start at CTA 0): roles on
                                       // different CTAs keep each CTA's instruction footprint small
    int gdn_off;                       // where the delta-net block keeps its state tile inside the scratch (clear of the input projection's buffers)
    int flags;                         // bit 0: the token is the previous pick (amx) instead of toks[0]; bit 1: hand the pick over (toks[0], pos + 1); bit 2: logits wanted
};

struct Pick { float v; unsigned i; };
__device__ __forceinline__ Pick pick_better(Pick a, Pick b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }

// Per-thread view of the CTA's state that every phase needs.
struct Cta {
    unsigned char* smem; unsigned char* scratch; unsigned bars; volatile int* abort_flag;
    int tid, warp, lane;
    unsigned q;                        // chunks of the CTA's stream the consumers have passed (slot = q % slots, phase = (q / slots) & 1; slots is a power of two)
    unsigned nseq;                     // row groups this CTA has started in all matvec phases so far (terms buffer = nseq % ST_TB)
    unsigned mph;                      // matvec phases finished so far
    unsigned tf, te, pd, ps;           // mbarriers: terms full [ST_TB], terms empty [ST_TB], phase done, phase started
    unsigned at;                       // mbarriers of the attention block: K full / free, V full / free, eight of each
    const StepLayer* lay;              // the two shared-memory copies of layer descriptions (layer il at lay[il & 1])
    unsigned target;                   // arrivals the next grid barrier waits for
    int nsync;                         // grid barriers passed so far (index into the trace)
    unsigned att_seq;                  // attention blocks this CTA has run in this launch
    float inv_sqrt_sd, inv_sqrt_hd;    // 1 / sqrt(state size), 1 / sqrt(head dimension): formed once per launch
    int evt_on, evt_base;              // diagnostics: this thread records fine-grained events into slots evt_base ..
};
constexpr int ST_TRACE_MAX = 1024;     // barriers recorded per traced CTA
constexpr int ST_EVT_MAX = 2048;       // fine-grained events (diagnostics)
// Diagnostics: slot `id` of the event area receives the nanosecond clock when the chosen thread passes (one store, no read).
// fine-grained events are compiled in only with -DIT_STEP_EVENTS: their two dozen sites cost 2.8 KB of code, about 1 % of a step
#ifndef IT_STEP_EVENTS
#define ST_EV(P, c, id) do { } while (0)
#else
#define ST_EV(P, c, id) do { if ((P).trace && (c).evt_on && (c).lane == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); (P).trace[4 * ST_TRACE_MAX + (id)] = t_; } } while (0)
#endif

__device__ __forceinline__ void cons_sync() { consumer_barrier<ST_CT>(); }
// four u8 x s8 products added to c
__device__ __forceinline__ int dp4a_us(unsigned a, int b, int c) { int d; asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d; }

// Barrier over the grid (consumer threads only; the producer warp never takes part).  Writes made by any CTA before the
// barrier are visible to every CTA after it: thread 0 announces the CTA with a release add and waits with acquire loads
// until every CTA of this round has arrived (the adds form one chain on the counter, so the load that sees the last of
// them is ordered after every CTA's writes).  Returns false when the step
// has been given up (by this CTA's own timeout or by another CTA's).
__device__ __forceinline__ bool grid_sync(const StepParams& P, Cta& c, int site) {
    cons_sync();
    if (c.tid == 0 && *c.abort_flag) atomicExch(P.sync + 2, 1u);      // a wait of this CTA ran out: tell the others
    if (c.tid == 0 && !*c.abort_flag) {
        const bool traced = P.trace && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1) && c.nsync < ST_TRACE_MAX;
        unsigned long long* rec = traced ? P.trace + ((size_t)(blockIdx.x ? 1 : 0) * ST_TRACE_MAX + c.nsync) * 2 : nullptr;
        if (rec) { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); rec[0] = t; }
        c.target += gridDim.x;
        // release: the CTA's writes (ordered before this thread by the barrier above) become visible before the arrival
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
        if (rec) { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); rec[1] = t; }
        c.nsync++;
    }
    cons_sync();
    return !*c.abort_flag;
}

// The ternary matvecs of a step in order: four per layer (input projection, output projection, gate/up, down), then the
// LM head.  Every role of the CTA (producer, consumers, sum warps) walks this list with ONE copy of its loop in the code:
// the kernel is executed once per step, front to back, so its size is what the instruction cache sees.
struct MatDesc { const uint8_t* tiles; int nb, rows, accum, pick; size_t y_off; };
__device__ __forceinline__ MatDesc mat_desc(const StepParams& P, int mp) {
    MatDesc d; d.pick = 0;
    const int il = mp >> 2, sub = mp & 3;
    if (il >= P.n_layer) { d.tiles = P.output; d.nb = P.e / 128; d.rows = P.n_vocab; d.accum = 0; d.y_off = P.logits; d.pick = 1; return d; }
    const StepLayer& L = P.layers[il];
    if (sub == 0) { d.tiles = L.in_proj; d.nb = P.e / 128; d.rows = L.in_rows; d.accum = 0; d.y_off = P.big1; }
    else if (sub == 1) { d.tiles = L.out_proj; d.nb = (L.recurrent ? P.inner : P.nh * P.hd) / 128; d.rows = P.e; d.accum = 1; d.y_off = P.x; }
    else if (sub == 2) { d.tiles = L.gate_up; d.nb = P.e / 128; d.rows = 2 * P.ff; d.accum = 0; d.y_off = P.big1; }
    else { d.tiles = L.down; d.nb = P.ff / 128; d.rows = P.e; d.accum = 1; d.y_off = P.x; }
    return d;
}
__device__ __forceinline__ int mat_count(const StepParams& P) { return 4 * P.n_layer + ((P.flags & 4) ? 1 : 0); }

// ---------------------------------------------------------------- producer
struct Ring { int s; unsigned ph; int issued; };
__device__ __forceinline__ bool produce_matrix(const StepParams& P, const Cta& c, Ring& r, const uint8_t* tiles, int nb, int rows, int* error_flag) {
    const int rgs = (rows + 31) / 32, cpr = (nb + ST_TPC - 1) / ST_TPC;
    for (int rg = blockIdx.x; rg < rgs; rg += gridDim.x) {
        const uint8_t* src = tiles + (size_t)rg * nb * IT_TILE_BYTES;
        for (int cq = 0; cq < cpr; cq++) {
            if (!mbar_wait(c.bars + 8 * (P.slots + r.s), r.ph ^ 1u, c.abort_flag, error_flag, 2)) return false;
            const int ntile = min(ST_TPC, nb - cq * ST_TPC);
            const unsigned bytes = (unsigned)ntile * IT_TILE_BYTES;
            mbar_expect_tx(c.bars + 8 * r.s, bytes);
            bulk_load(smem_u32(c.smem + r.s * ST_CHUNK), src + (size_t)cq * ST_CHUNK, bytes, c.bars + 8 * r.s);
            r.issued++;
            if (++r.s == P.slots) { r.s = 0; r.ph ^= 1u; }
        }
    }
    return true;
}
__device__ __forceinline__ void producer(const StepParams& P, const Cta& c) {
    Ring r{0, 0u, 0};
    bool ok = true;
    const int nmat = mat_count(P);
    for (int mp = 0; mp < nmat && ok; mp++) { const MatDesc d = mat_desc(P, mp); ok = produce_matrix(P, c, r, d.tiles, d.nb, d.rows, P.error_flag); }
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
// Same arithmetic as k_matvec_t2<1> (it_matvec_t2.cu): per 32 x 128 tile the exact integer block sums, the per-block terms
// (d_w * d_x) * float(S - sum128), and per row group one warp that adds the terms in ascending block order.  The sixteen
// consumer warps only form terms; two sum warps add them, a row group at a time, out of ST_TB buffers handed over through
// mbarriers, so that the consumers never stop at a row-group boundary.
struct MvSmem { int x, dx, s128, terms, plane, total; };
__host__ __device__ inline MvSmem mv_layout(int nb) {
    MvSmem L; int o = 0;
    L.plane = nb * 32;
    L.x = o; o += nb * 128 + 16;
    L.dx = o; o += (nb / 2) * 4;
    L.s128 = o; o += nb * 4;
    o = (o + 127) & ~127;
    L.terms = o; o += ST_TB * L.plane * 4;
    L.total = o;
    return L;
}

// prefetch_layer: when set, the delta-net block's state tile of that layer is requested right after the activation row has
// been staged (asynchronous copies for the phase after this one)
__device__ __forceinline__ void gdn_prefetch(const StepParams& P, const StepLayer& L, const Cta& c, int h);
__device__ __forceinline__ void attn_prefetch(const StepParams& P, const StepLayer& L, const Cta& c, int h);
__device__ __forceinline__ void matvec_phase(const StepParams& P, Cta& c, int nb, int rows, const StepLayer* prefetch_layer) {
    const MvSmem L = mv_layout(nb);
    int8_t* xs = reinterpret_cast<int8_t*>(c.scratch + L.x);
    float* dxs = reinterpret_cast<float*>(c.scratch + L.dx);
    int* sss = reinterpret_cast<int*>(c.scratch + L.s128);
    const int tid = c.tid, warp = c.warp, lane = c.lane;
    ST_EV(P, c, c.evt_base + 0);
    if (lane == 0) mbar_arrive(c.ps);                                // the sum warps may enter this phase (they never run ahead of the consumers)
    {   // the q8k row, its scales and block sums, once per CTA (written by other CTAs before the last barrier: read through L2)
        for (int ch = tid; ch < nb * 8; ch += ST_CT) cp_async16(xs + 16 * ch, P.qs + 16 * ch);
        for (int i = tid; i < nb / 2; i += ST_CT) dxs[i] = __ldcg(P.qd + i);
        for (int i = tid; i < nb; i += ST_CT) sss[i] = __ldcg(P.qsum + i);
        cp_async_wait_all();
        if (prefetch_layer) { if (prefetch_layer->recurrent) gdn_prefetch(P, *prefetch_layer, c, (int)blockIdx.x); else attn_prefetch(P, *prefetch_layer, c, (int)blockIdx.x - P.attn_base); }
        cons_sync();
    }
    ST_EV(P, c, c.evt_base + 1);
    const int t = lane & 3;
    const int group = warp / ST_CW, wi = warp % ST_CW;
    const int rgs = (rows + 31) / 32, cpr = (nb + ST_TPC - 1) / ST_TPC;
    const int trow = (lane >> 2) + 8 * t;                            // the matrix row of a tile whose term this lane forms: g + 8 t
    const unsigned smask = (unsigned)P.slots - 1u; const int sshift = 31 - __clz(P.slots);
    // One activation row: integer dot products on the SIMT pipe (dp4a, u8 x s8).  Lane 4 g + t owns the 32 columns
    // 32 t .. 32 t + 31 of a tile and, per 32-bit word, the four matrix rows g, g + 8, g + 16, g + 24 (bit pairs 0..3 of
    // every byte): masking a word with 0x03030303 << 2 i leaves row g + 8 i's four codes scaled by 4^i.  The four lanes of a
    // row group g then add their sums (exact integers) in a reduce-scatter that leaves row g + 8 t with lane t, which forms
    // that row's term.  (At eight activation columns the tensor-core path of it_matvec_t2.cu does this work; at one column
    // its dependent mma chain costs more latency than these short instructions, and this kernel has 16 warps per SM.)
    auto dots = [&](const unsigned char* tile, int b, int (&a)[4]) {
        const uint4 wa = *reinterpret_cast<const uint4*>(tile + 16 * lane);
        const uint4 wb = *reinterpret_cast<const uint4*>(tile + 512 + 16 * lane);
        const uint4* xp = reinterpret_cast<const uint4*>(xs + 128 * b + 32 * t);
        const uint4 xa = xp[0], xb4 = xp[1];
        const uint32_t w[8] = { wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w };
        const int xb[8] = { (int)xa.x, (int)xa.y, (int)xa.z, (int)xa.w, (int)xb4.x, (int)xb4.y, (int)xb4.z, (int)xb4.w };
        a[0] = a[1] = a[2] = a[3] = 0;
#pragma unroll
        for (int k = 0; k < 8; k++) {
            a[0] = dp4a_us(w[k] & 0x03030303u, xb[k], a[0]);
            a[1] = dp4a_us(w[k] & 0x0c0c0c0cu, xb[k], a[1]);
            a[2] = dp4a_us(w[k] & 0x30303030u, xb[k], a[2]);
            a[3] = dp4a_us(w[k] & 0xc0c0c0c0u, xb[k], a[3]);
        }
    };
    auto term = [&](const unsigned char* tile, int b, const int (&a)[4], float* tbuf) {
        const bool hi2 = t & 2, hi1 = t & 1;
        int k0 = hi2 ? a[2] : a[0], k1 = hi2 ? a[3] : a[1];
        const int s0 = hi2 ? a[0] : a[2], s1 = hi2 ? a[1] : a[3];
        k0 += __shfl_xor_sync(0xffffffffu, s0, 2); k1 += __shfl_xor_sync(0xffffffffu, s1, 2);
        int S = hi1 ? k1 : k0;
        S += __shfl_xor_sync(0xffffffffu, hi1 ? k0 : k1, 1);
        const __half dwh = *reinterpret_cast<const __half*>(tile + 1024 + 2 * lane);   // scale of row g + 8 t: half 4 g + t
        tbuf[b * 32 + trow] = __fmul_rn(__fmul_rn(__half2float(dwh), dxs[b >> 1]), (float)((S >> (2 * t)) - sss[b]));
    };
    unsigned n = c.nseq;
    for (int rg = blockIdx.x; rg < rgs; rg += gridDim.x, n++) {
        const unsigned k = n % ST_TB, u = n / ST_TB;
        float* tbuf = reinterpret_cast<float*>(c.scratch + L.terms) + k * L.plane;
        // the buffer's previous row group has been added up (the sum warp's arrival number u - 1)
        if (u && !mbar_wait(c.te + 8 * k, (u - 1) & 1u, c.abort_flag, P.error_flag, 4)) break;
        for (int cq = (int)((unsigned)(group + ST_NG) - c.q % ST_NG) % ST_NG; cq < cpr; cq += ST_NG) {      // the chunks of this row group that fall to this group
            const unsigned q = c.q + (unsigned)cq;
            const int cs = (int)(q & smask); const unsigned cph = (q >> sshift) & 1u;
            const int b0 = cq * ST_TPC + wi, b1 = b0 + ST_CW;
            const bool ready = mbar_wait(c.bars + 8 * cs, cph, c.abort_flag, P.error_flag, 3);
            if (ready && b0 < nb) {
                const unsigned char* tile0 = c.smem + cs * ST_CHUNK + wi * IT_TILE_BYTES;
                const unsigned char* tile1 = tile0 + ST_CW * IT_TILE_BYTES;
                int a0[4], a1[4];
                if (b1 < nb) {          // warp-uniform
                    dots(tile0, b0, a0); dots(tile1, b1, a1);
                    term(tile0, b0, a0, tbuf); term(tile1, b1, a1, tbuf);
                } else {
                    dots(tile0, b0, a0); term(tile0, b0, a0, tbuf);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(c.bars + 8 * (P.slots + cs));     // the slot may be refilled
        }
        c.q += (unsigned)cpr;
        __syncwarp();
        if (lane == 0) mbar_arrive(c.tf + 8 * k);                        // this warp's terms of the row group are in place
    }
    c.nseq = n;
    ST_EV(P, c, c.evt_base + 2);
    // the phase is over when the sum warps have stored its last results
    mbar_wait(c.pd, c.mph & 1u, c.abort_flag, P.error_flag, 5);
    c.mph++;
    ST_EV(P, c, c.evt_base + 3);
}

// The sum warps' side of a matvec phase: warp j adds the row groups whose sequence number is j modulo ST_NSUM.
__device__ __forceinline__ void sum_warps(const StepParams& P, Cta& c) {
    const int j = c.warp - ST_NCONS, lane = c.lane;
    float* arena = P.arena;
    Pick best{ -INFINITY, 0xffffffffu };
    const int nmat = mat_count(P);
    unsigned n = 0;
    bool ok = true;
    for (int mp = 0; mp < nmat && ok; mp++) {
        const MatDesc d = mat_desc(P, mp);
        const MvSmem L = mv_layout(d.nb);
        const int rgs = (d.rows + 31) / 32;
        // not before the consumers have entered the phase: a CTA without row groups in a phase would otherwise run through
        // its phase-done arrivals and leave the consumers waiting on a parity that has come round again
        if (!mbar_wait(c.ps, (unsigned)mp & 1u, c.abort_flag, P.error_flag, 7)) break;
        for (int rg = blockIdx.x; rg < rgs; rg += gridDim.x, n++) {
            if ((int)(n % ST_NSUM) != j) continue;
            const unsigned k = n % ST_TB, u = n / ST_TB;
            const int row = rg * 32 + lane;
            const float old = (d.accum && row < d.rows) ? __ldcg(arena + d.y_off + row) : 0.f;   // on its way while the terms are still being formed
            if (!mbar_wait(c.tf + 8 * k, u & 1u, c.abort_flag, P.error_flag, 6)) { ok = false; break; }
            if (row < d.rows) {
                const float* tcol = reinterpret_cast<const float*>(c.scratch + L.terms) + k * L.plane + lane;
                float sum = 0.f;
#pragma unroll 8
                for (int b = 0; b < d.nb; b++) sum = __fadd_rn(sum, tcol[b * 32]);
                if (d.accum) sum = __fadd_rn(old, sum);
                __stcg(arena + d.y_off + row, sum);
                if (d.pick) best = pick_better(best, Pick{ sum, (unsigned)row });
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(c.te + 8 * k);
        }
        if (d.pick) {       // greedy pick (first index of the maximum) over this warp's rows, left behind the layer descriptions
#pragma unroll
            for (unsigned mm = 16; mm > 0; mm >>= 1) { Pick o{ __shfl_xor_sync(0xffffffffu, best.v, mm), __shfl_xor_sync(0xffffffffu, best.i, mm) }; best = pick_better(best, o); }
            if (lane == 0) reinterpret_cast<Pick*>(const_cast<StepLayer*>(c.lay) + 2)[j] = best;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(c.pd);
    }
}

// ---------------------------------------------------------------- delta-net block of one value head
// conv + SiLU (+ l2norm of the q and k runs), the dense beta / alpha rows, the delta rule and the gated norm for head
// blockIdx.x, in the operation order of k_conv_l2_dense and k_gdn_norm (it_support.cu; src/cpu.rs:199-237).  The q / k
// runs of a key group are recomputed by each of the value heads that share it.  The new conv state of the runs this CTA
// is responsible for (its own v run; the q and k runs when it is the first head of the group) is returned in `keep`
// and stored after the next grid barrier, when no CTA reads the old state any more.
struct ConvKeep { int ch; float mx; };    // a conv channel whose state this thread shifts after the next barrier, and this step's input of that channel
// Issued by the CTA of value head blockIdx.x while the input projection runs: the head's state tile (64 KB, it does not
// depend on this step's activations) into its place in shared memory, and the head's beta / alpha rows into L2.
__device__ __forceinline__ void gdn_prefetch(const StepParams& P, const StepLayer& L, const Cta& c, int h) {
    constexpr int SD = ST_SD, PPR = SD / 4;
    const int tid = c.tid;
    float* tile = reinterpret_cast<float*>(c.scratch + P.gdn_off);
    const float4* m = reinterpret_cast<const float4*>(L.ssm_st + (size_t)h * SD * SD);
    for (int f = tid; f < SD * PPR; f += ST_CT) { const int j = f / PPR, cc = f % PPR; cp_async16(tile + j * SD + ((cc ^ (j & 7)) << 2), m + f); }
    asm volatile("cp.async.commit_group;" ::: "memory");
    const int lines = P.e * 4 / 128;
    for (int i = tid; i < 2 * lines; i += ST_CT) {
        const float* row = (i < lines ? L.beta : L.alpha) + (size_t)h * P.e + (size_t)(i % lines) * 32;
        asm volatile("prefetch.global.L2 [%0];" :: "l"(row));
    }
}
__device__ __forceinline__ void gdn_phase(const StepParams& P, const StepLayer& L, const Cta& c, ConvKeep& keep, int h) {
    constexpr int SD = ST_SD, PPR = SD / 4;
    const int tid = c.tid, warp = c.warp, lane = c.lane, kh = h % P.nk, kk = P.conv_k, cd = P.cd;
    float* tile = reinterpret_cast<float*>(c.scratch + P.gdn_off);   // [SD][SD], 16-byte pieces of row j stored at piece index ^ (j & 7); requested by gdn_prefetch
    float* vals = tile + SD * SD;                                    // [3][SD]: q, k, v runs after conv + SiLU
    float* os = vals + 3 * SD;                                       // [SD] delta-rule outputs
    float* scs = os + SD;                                            // [2] l2norm scales, [2] beta, alpha, [2] sigmoid(beta), exp(decay)
    double* wsum = reinterpret_cast<double*>(scs + 8);               // [16] warp sums of the two dense rows
    float* gzs = reinterpret_cast<float*>(wsum + 16);                // [SD] silu of the head's gate row
    const float* A = P.arena;
    auto piece = [&](int j, int cc) { return reinterpret_cast<float4*>(tile + j * SD + ((cc ^ (j & 7)) << 2)); };
    float* m = L.ssm_st + (size_t)h * SD * SD;
    keep.ch = -1;
    // dense rows: warps 0-7 beta row h, warps 8-15 alpha row h, in the order of k_dense_rows (thread i of 256 adds the products
    // i, i + 256, ... in f64).  The first sixteen products' operands are requested before anything else so that their
    // latency overlaps the conv; the gate values the norm needs at the very end are requested here too.
    // sixteen virtual warps (0-7: beta row h, 8-15: alpha row h) on the CTA's consumer warps; virtual thread i of a row's
    // 256 adds the products i, i + 256, ... in f64 (the order of k_dense_rows)
    const float* xr = A + P.xn;
    float wv[16], xv[16];
    {
        const int t8 = (warp & 7) * 32 + lane; const float* wr = (warp >= 8 ? L.alpha : L.beta) + (size_t)h * P.e;
#pragma unroll
        for (int k = 0; k < 16; k++) { const int i = t8 + 256 * k; wv[k] = i < P.e ? wr[i] : 0.f; xv[k] = i < P.e ? __ldcg(xr + i) : 0.f; }
    }
    // the gate values the norm needs at the very end: warp 0 keeps the norm weights, warp 8 (done early with its share of
    // the dense rows) forms silu(z) while the other warps are still busy
    float zr[SD / 32], nwr[SD / 32];
    if (warp == 0) {
#pragma unroll
        for (int i = 0; i < SD / 32; i++) nwr[i] = L.ssm_norm[lane + 32 * i];
    }
    if (warp == 8) {
#pragma unroll
        for (int i = 0; i < SD / 32; i++) zr[i] = __ldcg(A + P.big1 + cd + h * SD + lane + 32 * i);
    }
    if (tid < 3 * SD) {
        const int r = tid / SD, cc = tid % SD;
        const int ch = (r == 0 ? kh * SD : r == 1 ? P.qk + kh * SD : 2 * P.qk + h * SD) + cc;
        float st[8], cw[8];                                          // kk <= 8 taps: fixed-size loops keep these in registers
#pragma unroll
        for (int i = 0; i < 8; i++) { st[i] = i < kk - 1 ? L.conv_st[(size_t)i * cd + ch] : 0.f; cw[i] = i < kk ? L.conv_w[ch * kk + i] : 0.f; }
        const float mx = __ldcg(A + P.big1 + ch);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) if (i < kk) s = it_add(s, it_mul(i < kk - 1 ? st[i] : mx, cw[i]));
        vals[r * SD + cc] = it_silu(s);
        if (r == 2 || h < P.nk) { keep.ch = ch; keep.mx = mx; }
    }
    ST_EV(P, c, c.evt_base + 5);
    for (int vw = warp; vw < 16; vw += ST_NCONS) {
        const int t8 = (vw & 7) * 32 + lane; const float* wr = (vw >= 8 ? L.alpha : L.beta) + (size_t)h * P.e;
        double s = 0.0;
#pragma unroll 1
        for (int base = 0; base < P.e; base += 16 * 256) {            // one copy of the load and of the add block: the first block of the warp's own row is already in registers
            if (vw != warp || base) {
#pragma unroll
                for (int k = 0; k < 16; k++) { const int i = base + t8 + 256 * k; wv[k] = i < P.e ? wr[i] : 0.f; xv[k] = i < P.e ? __ldcg(xr + i) : 0.f; }
            }
#pragma unroll
            for (int k = 0; k < 16; k++) if (base + t8 + 256 * k < P.e) s += (double)it_mul(wv[k], xv[k]);
        }
#pragma unroll
        for (int mm = 16; mm >= 1; mm >>= 1) s += __shfl_xor_sync(0xffffffffu, s, mm);
        if (lane == 0) wsum[vw] = s;
    }
    ST_EV(P, c, c.evt_base + 6);
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
        const float tf = (float)tt;                                  // warp 2: beta, warp 3: alpha; the gates follow at once, off the owners' path
        scs[warp] = tf;
        if (warp == 2) scs[4] = it_sigmoid(tf);
        else scs[5] = it_expf(it_mul(it_softplus(it_add(tf, L.dt[h])), L.a[h]));
    } else if (warp == 8) {
#pragma unroll
        for (int i = 0; i < SD / 32; i++) gzs[lane + 32 * i] = it_silu(zr[i]);
    }
    ST_EV(P, c, c.evt_base + 7);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    cons_sync();
    ST_EV(P, c, c.evt_base + 8);
    if (tid < SD) {
        const float q = it_mul(vals[tid], scs[0]), k = it_mul(vals[SD + tid], scs[1]);
        asm volatile("bar.sync 3, %0;" :: "n"(SD) : "memory");       // every owner has read the raw q / k values
        vals[tid] = q; vals[SD + tid] = k;
        asm volatile("bar.sync 3, %0;" :: "n"(SD) : "memory");
        const float* qs = vals; const float* ks = vals + SD;
        const float v = vals[2 * SD + tid];
        const float bt = scs[4];
        const float eg = scs[5];
        const float scale = c.inv_sqrt_sd;
        // Two passes over the thread's state row, eight 16-byte pieces at a time (requested together, then used in order).
        // The first pass only reads: s = sum_i (row[i] * eg) * k[i] in index order.  The second forms row[i] * eg again (the
        // same rounded product), adds k[i] * delta, stores the new state and accumulates the output in index order.
        float s = 0.f;
#pragma unroll 1
        for (int c0 = 0; c0 < PPR; c0 += 8) {
            float4 rr[8];
#pragma unroll
            for (int u = 0; u < 8; u++) rr[u] = *piece(tid, c0 + u);
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const float4 k4 = *reinterpret_cast<const float4*>(ks + 4 * (c0 + u));
                s = it_add(s, it_mul(it_mul(rr[u].x, eg), k4.x)); s = it_add(s, it_mul(it_mul(rr[u].y, eg), k4.y));
                s = it_add(s, it_mul(it_mul(rr[u].z, eg), k4.z)); s = it_add(s, it_mul(it_mul(rr[u].w, eg), k4.w));
            }
        }
        const float delta = it_mul(it_sub(v, s), bt);
        float acc = 0.f;
#pragma unroll 1
        for (int c0 = 0; c0 < PPR; c0 += 8) {
            float4 rr[8];
#pragma unroll
            for (int u = 0; u < 8; u++) rr[u] = *piece(tid, c0 + u);
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const float4 k4 = *reinterpret_cast<const float4*>(ks + 4 * (c0 + u)), q4 = *reinterpret_cast<const float4*>(qs + 4 * (c0 + u));
                float4 r;
                r.x = it_add(it_mul(rr[u].x, eg), it_mul(k4.x, delta)); r.y = it_add(it_mul(rr[u].y, eg), it_mul(k4.y, delta));
                r.z = it_add(it_mul(rr[u].z, eg), it_mul(k4.z, delta)); r.w = it_add(it_mul(rr[u].w, eg), it_mul(k4.w, delta));
                *piece(tid, c0 + u) = r;
                acc = it_add(acc, it_mul(r.x, q4.x)); acc = it_add(acc, it_mul(r.y, q4.y)); acc = it_add(acc, it_mul(r.z, q4.z)); acc = it_add(acc, it_mul(r.w, q4.w));
            }
        }
        os[tid] = it_mul(acc, scale);
    }
    ST_EV(P, c, c.evt_base + 9);
    cons_sync();
    ST_EV(P, c, c.evt_base + 10);
    // the new state back to global memory (coalesced 16-byte stores by warps 1..15) while warp 0 norms the outputs
    if (warp > 0) for (int f = tid - 32; f < SD * PPR; f += ST_CT - 32) reinterpret_cast<float4*>(m)[f] = *piece(f / PPR, f % PPR);
    if (warp == 0) {
        float sc = 0.f;
        if (lane == 0) {
            float s = 0.f;
#pragma unroll 8
            for (int i = 0; i < SD; i++) s = it_add(s, it_mul(os[i], os[i]));
            sc = it_div(1.0f, it_sqrt(it_add(it_div(s, (float)SD), P.eps)));
        }
        sc = __shfl_sync(0xffffffffu, sc, 0);
        float* o = P.arena + P.o + h * SD;                           // zr: the gate rows, which follow the qkv rows in the stacked output
#pragma unroll
        for (int i = 0; i < SD / 32; i++) {
            const int j = lane + 32 * i;
            __stcg(o + j, it_mul(it_mul(it_mul(os[j], sc), nwr[i]), gzs[j]));
        }
    }
    ST_EV(P, c, c.evt_base + 11);
}

// ---------------------------------------------------------------- attention block of one head
// q / k head norms, rope, the new K / V entries and the causal gated attention of head h in the operation order of
// k_attn_prep and k_attention (it_support.cu; src/cpu.rs:252-272): every score a sequential dot over the head dimension,
// the exponentials added in ascending position order by one thread, every output element accumulating w[p] * v[p][j] in
// ascending position order.  The k and v rows of the new position are recomputed by each of the heads that share the KV
// head and used from shared memory (after the same f16 rounding the cache applies); the first head of the group stores
// them into the cache.
// Data movement: both caches are tiled (32 positions x head_dim halves = one contiguous 16 KB block per KV head), so a
// loader warp brings whole tiles into a ring of 16 KB slots with one bulk copy each.  One warp per slot scores its K
// tiles, a position per lane, from shared memory; the V tiles follow through the same ring and four warps (two output
// elements per thread) walk them in order.  Full / free mbarriers pace both; they are set up afresh by every attention
// block.  The tiles were sent on their way into L2 while the input projection ran (attn_prefetch).
__device__ __forceinline__ void attn_prefetch(const StepParams& P, const StepLayer& L, const Cta& c, int hg) {
    if (c.warp != 0 || hg < 0 || hg >= P.nh * P.attn_g) return;
    const int G = P.attn_g, h = hg / G, g = hg % G;
    const int kh = h / (P.nh / P.nkv), ntiles = (*P.pos + 31) / 32; const unsigned bytes = (unsigned)(P.hd * 64);
    for (int i = g + G * c.lane; i < ntiles; i += G * 32)               // the K tiles this CTA will score
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(L.kc + it_kc_index((size_t)i * 32, kh, 0, P.nkv, P.hd)), "r"(bytes) : "memory");
    for (int i = g + G * c.lane; i < ntiles; i += G * 32)               // a quarter of the V tiles each: every CTA of the head reads a slice of all of them
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(L.vc + it_vc_index((size_t)i * 32, kh, 0, P.nkv, P.hd)), "r"(bytes) : "memory");
}
constexpr int ST_AT_MAXS = 8, ST_AT_LOADER = ST_NCONS - 1, ST_AT_T = (ST_NCONS - 1) * 32;
// the block's own barrier: every consumer warp but the loader, which runs ahead and only joins the grid barrier
__device__ __forceinline__ void at_sync() { asm volatile("bar.sync 4, %0;" :: "n"(ST_AT_T) : "memory"); }
// G = P.attn_g CTAs share a head (hg = G h + g).  Each forms q and the new position's k and v for itself, scores the K
// tiles i with i % G == g, publishes those scores, meets the head's other CTAs at a counter of their own, reads their
// scores, runs the softmax for itself (one thread adds the exponentials in position order) and accumulates the
// head_dim / G output elements [g head_dim / G, ...) over all positions from row slices of the V tiles.  A single SM can
// keep only so many bytes in flight, so a head's cache traffic is spread over G SMs.
__device__ __forceinline__ void attn_phase(const StepParams& P, const StepLayer& L, Cta& c, int hg) {
    const int tid = c.tid, warp = c.warp, lane = c.lane, hd = P.hd, nkv = P.nkv, kvd = nkv * hd;
    const int G = P.attn_g, h = hg / G, g = hg % G, epc = hd / G;   // elements of the output this CTA owns
    const int vs = it_vc_slice(hd);                                  // elements per V slice: epc is a multiple of it
    const int rep = P.nh / nkv, kh = h / rep;
    const bool writer = h % rep == 0 && g == 0;
    const int pos = *P.pos, n = pos + 1, nold = pos;
    const int ntiles = (nold + 31) / 32;                             // K tiles = V tiles of 32 positions
    const int my_tiles = ntiles > g ? (ntiles - g + G - 1) / G : 0;  // tiles g, g + G, ... are scored here
    const int tile_bytes = hd * 64;                                  // 32 positions x hd halves
    const int vslot_bytes = epc * 64;                                // 32 positions x epc halves: this CTA's slice of a V tile
    float* sc = reinterpret_cast<float*>(c.scratch);                 // [n] scores
    float* qs = sc + ((n + 3) & ~3);                                 // [hd] q head after norm + rope
    float* kl = qs + hd;                                             // [hd] k row of the new position as the cache holds it
    float* vl = kl + hd;                                             // [hd] v row of the new position as the cache holds it
    float* red = vl + hd;                                            // [32] + the sum
    unsigned char* ring = reinterpret_cast<unsigned char*>(red + 48) + ((128u - (smem_u32(red + 48) & 127u)) & 127u);
    const int room = (int)((c.scratch + P.scratch) - ring);
    // K: tile j of this CTA goes to slot j % S and is scored by warp j % S, so every slot is filled and emptied by the same two
    // warps in order.  V: slice j goes to slot j % SV; the output warps walk the slices in order.
    const int S = max(1, min(ST_AT_MAXS, room / tile_bytes)), SV = max(1, min(ST_AT_MAXS, room / vslot_bytes));
    const int vwarps = (epc + 31) / 32;                              // output warps: one element per thread
    const unsigned kf = c.at, ke = c.at + 8 * ST_AT_MAXS, vf = c.at + 16 * ST_AT_MAXS, ve = c.at + 24 * ST_AT_MAXS;
    c.att_seq++;
    if (tid == 0) {
#pragma unroll 1
        for (int k = 0; k < 4 * ST_AT_MAXS; k++) asm volatile("mbarrier.inval.shared::cta.b64 [%0];" :: "r"(c.at + 8 * k) : "memory");
#pragma unroll 1
        for (int k = 0; k < ST_AT_MAXS; k++) { mbar_init(kf + 8 * k, 1); mbar_init(ke + 8 * k, 1); mbar_init(vf + 8 * k, 1); mbar_init(ve + 8 * k, vwarps); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    ST_EV(P, c, c.evt_base + 4);
    cons_sync();                                                     // all twelve warps, the loader included
    ST_EV(P, c, c.evt_base + 5);
    const float* row = P.arena + P.big1;
    const float* qh = row + (size_t)h * 2 * hd; const float* gate = qh + hd;
    const __half* kc = L.kc; const __half* vc = L.vc;

    if (warp == ST_AT_LOADER) {
        // ---- loader: this CTA's K tiles, then its slice of every V tile, as far ahead as the rings allow
#pragma unroll 1
        for (int j = 0; j < my_tiles; j++) {
            const unsigned sl = (unsigned)j % (unsigned)S, u = (unsigned)j / (unsigned)S;
            if (!mbar_wait(ke + 8 * sl, (u & 1u) ^ 1u, c.abort_flag, P.error_flag, 8)) break;
            if (lane == 0) {
                mbar_expect_tx(kf + 8 * sl, (unsigned)tile_bytes);
                bulk_load(smem_u32(ring + sl * tile_bytes), kc + it_kc_index((size_t)(g + G * j) * 32, kh, 0, nkv, hd), (unsigned)tile_bytes, kf + 8 * sl);
            }
        }
        // the V slices go through the same bytes: not before the last K tile of every slot has been scored
        for (int j = my_tiles > S ? my_tiles - S : 0; j < my_tiles; j++) {
            if (!mbar_wait(ke + 8 * (j % S), (unsigned)(j / S) & 1u, c.abort_flag, P.error_flag, 8)) break;
        }
#pragma unroll 1
        for (int i = 0; i < ntiles; i++) {
            const unsigned sl = (unsigned)i % (unsigned)SV, u = (unsigned)i / (unsigned)SV;
            if (!mbar_wait(ve + 8 * sl, (u & 1u) ^ 1u, c.abort_flag, P.error_flag, 9)) break;
            if (lane == 0) {
                // the slices of the tile that hold elements g epc .. (g + 1) epc - 1 are consecutive: one copy
                mbar_expect_tx(vf + 8 * sl, (unsigned)vslot_bytes);
                bulk_load(smem_u32(ring + sl * vslot_bytes), vc + it_vc_index((size_t)i * 32, kh, g * epc, nkv, hd), (unsigned)vslot_bytes, vf + 8 * sl);
            }
        }
        return;                                                      // the loader meets the others at the grid barrier
    }
    if (warp < 2) {
        // warp 0: q head; warp 1: k head.  rmsnorm with the squares added by one lane in index order, weight, rope.
        float* buf = warp == 0 ? qs : kl;
        const float* x = warp == 0 ? qh : row + (size_t)P.nh * 2 * hd + kh * hd;
        const float* w = warp == 0 ? L.q_norm : L.k_norm;
        float wr[8];                                                  // hd <= 256: the norm weights are requested before the sum needs time
#pragma unroll
        for (int k = 0; k < 8; k++) wr[k] = lane + 32 * k < hd ? w[lane + 32 * k] : 0.f;
        for (int i = lane; i < hd; i += 32) buf[i] = __ldcg(x + i);
        __syncwarp();
        float s = 0.f;
        if (lane == 0) {
#pragma unroll 16
            for (int i = 0; i < hd; i++) s = it_add(s, it_mul(buf[i], buf[i]));
        }
        s = __shfl_sync(0xffffffffu, s, 0);
        const float scl = it_div(1.0f, it_sqrt(it_add(it_div(s, (float)hd), P.eps)));
#pragma unroll
        for (int k = 0; k < 8; k++) if (lane + 32 * k < hd) buf[lane + 32 * k] = it_mul(it_mul(buf[lane + 32 * k], scl), wr[k]);
        __syncwarp();
        const int half = P.n_rot / 2, sect = P.sec[0] + P.sec[1] + P.sec[2] + P.sec[3];
#pragma unroll 1
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
            if (writer) const_cast<__half*>(vc)[it_vc_index(pos, kh, i, nkv, hd)] = hv;
            vl[i] = __half2float(hv);
        }
    }
    at_sync();                                                       // q, and the new position's k and v, are in shared memory
    ST_EV(P, c, c.evt_base + 6);
    const float scale = c.inv_sqrt_hd;
    const int nvec = hd / 8;
    float* shared_sc = P.att_sc + (size_t)h * P.att_stride;          // the head's scores, where its CTAs leave theirs for one another
    if (warp < S) {
        // ---- scores: this CTA's tile j by warp j % S, position 32 (g + G j) + lane; piece v of the tile's 32 positions is contiguous
        for (int j = warp; j < my_tiles; j += S) {
            const unsigned sl = (unsigned)j % (unsigned)S, u = (unsigned)j / (unsigned)S;
            if (!mbar_wait(kf + 8 * sl, u & 1u, c.abort_flag, P.error_flag, 10)) break;
            const int p = (g + G * j) * 32 + lane;
            if (p < nold) {
                const uint4* kp = reinterpret_cast<const uint4*>(ring + sl * tile_bytes) + lane;
                float s = 0.f;
#pragma unroll 4
                for (int v = 0; v < nvec; v++) {
                    const uint4 kk = kp[v * 32];
                    const __half2* hh = reinterpret_cast<const __half2*>(&kk);
                    const float4 qa = *reinterpret_cast<const float4*>(qs + v * 8), qb = *reinterpret_cast<const float4*>(qs + v * 8 + 4);
                    float2 f = __half22float2(hh[0]); s = it_add(s, it_mul(qa.x, f.x)); s = it_add(s, it_mul(qa.y, f.y));
                    f = __half22float2(hh[1]); s = it_add(s, it_mul(qa.z, f.x)); s = it_add(s, it_mul(qa.w, f.y));
                    f = __half22float2(hh[2]); s = it_add(s, it_mul(qb.x, f.x)); s = it_add(s, it_mul(qb.y, f.y));
                    f = __half22float2(hh[3]); s = it_add(s, it_mul(qb.z, f.x)); s = it_add(s, it_mul(qb.w, f.y));
                }
                s = it_mul(s, scale); sc[p] = s;
                if (G > 1) __stcg(shared_sc + p, s);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(ke + 8 * sl);
        }
    } else if (warp == ST_AT_MAXS && lane == 0) {
        float s = 0.f;                                               // the new position, from its row in shared memory (every CTA of the head for itself)
#pragma unroll 16
        for (int j = 0; j < hd; j++) s = it_add(s, it_mul(qs[j], kl[j]));
        sc[nold] = it_mul(s, scale);
    }
    ST_EV(P, c, c.evt_base + 7);
    if (G > 1) {
        // ---- the head's CTAs meet: arrival counter of the head (zeroed at the start of the launch), then everyone reads the others' scores
        at_sync();
        if (tid == 0) {
            unsigned* cnt = P.att_cnt + h;
            const unsigned target = (unsigned)G * c.att_seq;
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" :: "l"(cnt) : "memory");
            const long long t0 = clock64();
            for (unsigned it = 0;; it++) {
                unsigned v; asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(cnt) : "memory");
                if ((int)(v - target) >= 0) break;
                if ((it & 63u) == 63u) {
                    if (*reinterpret_cast<volatile unsigned*>(P.sync + 2)) { *c.abort_flag = 1; break; }
                    if (clock64() - t0 > WAIT_CLOCKS) { atomicExch(P.error_flag, 112); atomicExch(P.sync + 2, 1u); *c.abort_flag = 1; break; }
                }
            }
        }
        at_sync();
        if (!*c.abort_flag) {
#pragma unroll 1
            for (int i = 0; i < ntiles; i++) {
                if (i % G == g) continue;
                const int p = i * 32 + (tid & 31);
                if ((tid >> 5) == (i % (ST_NCONS - 1)) && p < nold) sc[p] = __ldcg(shared_sc + p);
            }
        }
        at_sync();
    } else at_sync();
    ST_EV(P, c, c.evt_base + 8);
    float mx = -INFINITY;
#pragma unroll 1
    for (int p = tid; p < n; p += ST_AT_T) mx = fmaxf(mx, sc[p]);
#pragma unroll
    for (int mm = 16; mm >= 1; mm >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, mm));
    if (lane == 0) red[warp] = mx;
    at_sync();
    mx = red[0];
#pragma unroll
    for (int k = 1; k < ST_NCONS - 1; k++) mx = fmaxf(mx, red[k]);
#pragma unroll 1
    for (int p = tid; p < n; p += ST_AT_T) sc[p] = it_expf(it_sub(sc[p], mx));
    at_sync();
    if (tid == 0) {
        float s = 0.f;
#pragma unroll 8
        for (int p = 0; p < n; p++) s = it_add(s, sc[p]);
        red[32] = s;
    }
    at_sync();
    const float sum = red[32];
#pragma unroll 1
    for (int p = tid; p < n; p += ST_AT_T) sc[p] = it_div(sc[p], sum);
    at_sync();
    ST_EV(P, c, c.evt_base + 9);
    if (warp < vwarps) {
        // ---- output: element j adds w[p] * v[p][j] in ascending p; thread tid owns element g epc + tid of the head.  A whole
        // tile's 32 values are read before the first addition, so that the chain of additions never waits for shared memory.
        const bool live = tid < epc;
        float acc = 0.f;
        const int eoff = (tid / vs) * 32 * vs + tid % vs;             // [slice][32][vs]
        for (int i = 0; i < ntiles; i++) {
            const unsigned sl = (unsigned)i % (unsigned)SV, u = (unsigned)i / (unsigned)SV;
            if (!mbar_wait(vf + 8 * sl, u & 1u, c.abort_flag, P.error_flag, 11)) break;
            const int rows = min(32, nold - i * 32);
            if (live) {
                const __half* src = reinterpret_cast<const __half*>(ring + sl * vslot_bytes) + eoff;
                const float* wp = sc + i * 32;
                if (rows == 32) {
                    float vv[32];
#pragma unroll
                    for (int r = 0; r < 32; r++) vv[r] = __half2float(src[r * vs]);
#pragma unroll
                    for (int r4 = 0; r4 < 8; r4++) {
                        const float4 w4 = *reinterpret_cast<const float4*>(wp + 4 * r4);
                        acc = it_add(acc, it_mul(w4.x, vv[4 * r4])); acc = it_add(acc, it_mul(w4.y, vv[4 * r4 + 1]));
                        acc = it_add(acc, it_mul(w4.z, vv[4 * r4 + 2])); acc = it_add(acc, it_mul(w4.w, vv[4 * r4 + 3]));
                    }
                } else {
                    for (int r = 0; r < rows; r++) acc = it_add(acc, it_mul(wp[r], __half2float(src[r * vs])));
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(ve + 8 * sl);
        }
        if (live) {
            const int e0 = g * epc + tid;
            acc = it_add(acc, it_mul(sc[nold], vl[e0]));
            __stcg(P.arena + P.o + (size_t)h * hd + e0, it_mul(acc, it_sigmoid(__ldcg(gate + e0))));
        }
    }
    ST_EV(P, c, c.evt_base + 10);
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
    c.q = 0u; c.nseq = 0u; c.mph = 0u; c.nsync = 0; c.evt_on = 0; c.att_seq = 0u;
    c.tf = c.bars + 8 * (2 * P.slots); c.te = c.tf + 8 * ST_TB; c.pd = c.te + 8 * ST_TB; c.ps = c.pd + 8; c.at = c.bars + 704;
    c.lay = reinterpret_cast<const StepLayer*>(tail + 384);         // two layer descriptions, then the sum warps' greedy picks
    if (c.tid == 0) {
        *c.abort_flag = *reinterpret_cast<volatile unsigned*>(P.sync + 2) ? 1 : 0;      // a step that was given up earlier: nothing runs until the host has cleared the words
        for (int s = 0; s < P.slots; s++) { mbar_init(c.bars + 8 * s, 1); mbar_init(c.bars + 8 * (P.slots + s), ST_CW); }
        for (int k = 0; k < ST_TB; k++) { mbar_init(c.tf + 8 * k, ST_NCONS); mbar_init(c.te + 8 * k, 1); }
        mbar_init(c.pd, ST_NSUM); mbar_init(c.ps, ST_NCONS);
        for (int k = 0; k < 4 * ST_AT_MAXS; k++) mbar_init(c.at + 8 * k, 1);     // set up again, with their counts, by every attention block
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    {   // the first layer's description into shared memory (later ones are copied a layer ahead)
        constexpr int words = (int)(sizeof(StepLayer) / 4);
        if (c.tid < words) reinterpret_cast<uint32_t*>(tail + 384)[c.tid] = reinterpret_cast<const uint32_t*>(P.layers)[c.tid];
    }
    __syncthreads();
    if (*c.abort_flag) return;
    if (c.warp == ST_NCONS + ST_NSUM) { if (c.lane == 0) producer(P, c); return; }
    if (c.warp >= ST_NCONS) { sum_warps(P, c); return; }

    c.target = *reinterpret_cast<volatile unsigned*>(P.sync + 1);
    if (c.tid == 0 && (int)blockIdx.x < P.nh) __stcg(P.att_cnt + blockIdx.x, 0u);       // the heads' arrival counters start every launch at zero (grid barriers precede their first use)
    c.inv_sqrt_sd = it_div(1.0f, it_sqrt((float)ST_SD)); c.inv_sqrt_hd = it_div(1.0f, it_sqrt((float)P.hd));
    if (P.trace && blockIdx.x == 0 && c.tid == 32) P.trace[4 * ST_TRACE_MAX] = 0;
    const int e = P.e, nb_e = e / 128;
    float* A = P.arena;
    const uint32_t tok = (P.flags & 1) ? __float_as_uint(*reinterpret_cast<volatile float*>(A + P.amx)) : *reinterpret_cast<volatile uint32_t*>(P.toks);
    const float* xsrc = P.tok_embd + (size_t)tok * e;               // the residual row of layer 0 is the embedding row (Model::embed, src/cpu.rs:118-122)
    ConvKeep keep; keep.ch = -1; keep.mx = 0.f;
    // Phases: nine per layer (0 norm+Hadamard, 1 input projection, 2 delta-net / attention block, 3 Hadamard of its output,
    // 4 output projection, 5 norm+Hadamard, 6 gate/up, 7 silu*mul+Hadamard, 8 down), then the output norm (+ Hadamard), the LM
    // head and the pick.  One loop, one copy of each kind of phase: the kernel runs front to back once per step, so its code
    // size, not its loop structure, is what the instruction cache sees.
    const bool logits = (P.flags & 4) != 0;
    const int nphase = 9 * P.n_layer + (logits ? 3 : 1);
    for (int ph = 0; ph < nphase; ph++) {
        const int il = ph / 9, sub = ph - 9 * il;
        const bool tail = il >= P.n_layer;
        const StepLayer& L = c.lay[il & 1];
        if (!tail && sub == 0 && il + 1 < P.n_layer && c.warp == ST_NCONS - 1) {          // the next layer's description, long before it is needed
            constexpr int words = (int)(sizeof(StepLayer) / 4);
            uint32_t* dst = reinterpret_cast<uint32_t*>(const_cast<StepLayer*>(c.lay + ((il + 1) & 1)));
            for (int i = c.lane; i < words; i += 32) dst[i] = reinterpret_cast<const uint32_t*>(P.layers + il + 1)[i];
        }
        c.evt_on = (il == 1 || il == 3) && c.warp == 0 && ((sub == 2) ? ((int)blockIdx.x == (il == 1 ? 0 : P.attn_base)) : (blockIdx.x == gridDim.x - 1)); c.evt_base = (il == 1 ? 0 : 256) + 16 * sub;
        const int kind = tail ? (sub == 0 ? 0 : sub == 1 ? 1 : 3) : (sub == 2 ? 2 : sub < 2 ? sub : ((sub & 1) ? 0 : 1));   // 0 Hadamard, 1 matvec, 2 block, 3 pick
        if (kind == 0) {
            it_had_prologue p; const float* in = A + P.x; const float* signs = P.sg_e; int nblocks = nb_e / 8; unsigned ph_hd = 0, ph_nk = 0, ph_rep = 0;
            float shift[6]; const bool shifting = !tail && sub == 3 && keep.ch >= 0;
            if (tail || sub == 0 || sub == 5) {
                // rmsnorm -> Hadamard -> q8k of the residual row; the normed row is kept where a later op reads it in f32
                p.mode = 2; p.w = tail ? P.output_norm : sub == 0 ? L.attn_norm : L.post_norm; p.eps = P.eps; p.n = (unsigned)e; p.xn_stride = e;
                p.xn_out = tail ? A + P.hrow : (sub == 0 && L.recurrent) ? A + P.xn : nullptr;
                if (!tail && sub == 0 && il == 0) {
                    in = xsrc;
                    const int vb0 = (int)blockIdx.x - P.had_base;
                    if (vb0 >= 0 && vb0 < nblocks && c.tid < 256)
                        *reinterpret_cast<float4*>(A + P.x + vb0 * 1024 + 4 * c.tid) = *reinterpret_cast<const float4*>(xsrc + vb0 * 1024 + 4 * c.tid);
                }
            } else if (sub == 3) {
                // the block's output row (delta-net: with the value-head permutation).  The conv state of the channels this
                // thread owns moves on by one input now that no CTA reads the old one: loads here, stores after the transform
                if (shifting) {
#pragma unroll
                    for (int i = 0; i < 6; i++) shift[i] = i < P.conv_k - 2 ? L.conv_st[(size_t)(i + 1) * P.cd + keep.ch] : 0.f;
                }
                const bool perm = L.recurrent && P.v_grouped;
                in = A + P.o; signs = L.recurrent ? P.sg_inner : P.sg_att; nblocks = (L.recurrent ? P.inner : P.nh * P.hd) / 1024;
                if (perm) { ph_hd = ST_SD; ph_nk = (unsigned)P.nk; ph_rep = (unsigned)(P.nv / P.nk); }
            } else {
                p.mode = 1; p.b = A + P.big1 + P.ff; p.b_stride = 2 * (size_t)P.ff;        // silu(gate) * up on the way in
                in = A + P.big1; signs = P.sg_ff; nblocks = P.ff / 1024;
            }
            const int vb = (int)blockIdx.x - P.had_base;
            if (vb >= 0 && vb < nblocks && c.tid < 256) {
                it_had_smem& sm = *reinterpret_cast<it_had_smem*>(c.scratch);
                it_hadamard_block<true>(sm, (unsigned)c.tid, (unsigned)vb, 0, in, 0, 0, nullptr, 0, 0, signs, 1, 0, ph_hd, ph_nk, ph_rep, P.qs, P.qd, P.qsum, P.q_stride, p);
            }
            if (shifting) {
#pragma unroll
                for (int i = 0; i < 6; i++) if (i < P.conv_k - 2) L.conv_st[(size_t)i * P.cd + keep.ch] = shift[i];
                L.conv_st[(size_t)(P.conv_k - 2) * P.cd + keep.ch] = keep.mx;
                keep.ch = -1;
            }
        } else if (kind == 1) {
            int nb, rows;
            if (tail) { nb = nb_e; rows = P.n_vocab; }
            else if (sub == 1) { nb = nb_e; rows = L.in_rows; }
            else if (sub == 4) { nb = (L.recurrent ? P.inner : P.nh * P.hd) / 128; rows = e; }
            else if (sub == 6) { nb = nb_e; rows = 2 * P.ff; }
            else { nb = P.ff / 128; rows = e; }
            const bool block_cta = L.recurrent ? (int)blockIdx.x < P.nv : ((int)blockIdx.x >= P.attn_base && (int)blockIdx.x < P.attn_base + P.nh * P.attn_g);
            matvec_phase(P, c, nb, rows, (!tail && sub == 1 && block_cta) ? &L : nullptr);
            if (tail && c.warp == 0 && c.lane == 0) {
                // greedy pick (first index of the maximum): each sum warp has left the best of its rows behind the layer descriptions
                const Pick* pk = reinterpret_cast<const Pick*>(c.lay + 2);
                Pick pbest = pk[0];
                for (int j = 1; j < ST_NSUM; j++) pbest = pick_better(pbest, pk[j]);
                P.partials[blockIdx.x] = ((unsigned long long)__float_as_uint(pbest.v) << 32) | pbest.i;
            }
        } else if (kind == 2) {
            const int ah = (int)blockIdx.x - P.attn_base;
            if (L.recurrent) { if ((int)blockIdx.x < P.nv) gdn_phase(P, L, c, keep, (int)blockIdx.x); }
            else if (ah >= 0 && ah < P.nh * P.attn_g) attn_phase(P, L, c, ah);
        } else {
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
            break;                                                   // nothing follows the pick
        }
        if (!grid_sync(P, c, 1 + sub + (tail ? 9 : 0))) return;
    }
    if (blockIdx.x == 0 && c.tid == 0) P.sync[1] = c.target;        // every CTA has read the old value before its first arrival
}

}  // namespace

// ---------------------------------------------------------------- host side
struct it_step_state {
    StepLayer* layers_dev;
    unsigned long long* trace;
    unsigned long long* partials;
    int grid, slots, scratch, gdn_off, had_base, attn_base, attn_g, att_stride;
    float* att_sc; unsigned* att_cnt;
    bool cooperative;
};

static size_t step_gdn_off(const it_model_config& c) { return ((size_t)mv_layout(c.n_embd / 128).total + 127) / 128 * 128; }
static size_t step_scratch_bytes(const it_model_config& c) {
    const int widest = std::max(std::max(c.n_embd, c.n_ff), std::max(c.ssm_inner, c.n_head * c.head_dim));
    size_t s = (size_t)mv_layout(widest / 128).total;
    s = std::max(s, sizeof(it_had_smem));
    s = std::max(s, step_gdn_off(c) + (size_t)(ST_SD * ST_SD + 5 * ST_SD + 8) * 4 + 16 * 8 + 64);
    s = std::max(s, ((size_t)c.ctx_len + 4 + 3 * c.head_dim + 48) * 4 + 128 + 3 * (size_t)c.head_dim * 64);
    return (s + 127) / 128 * 128;
}

// Whether this engine's decode step can run as the persistent kernel, and with which geometry.
int it_step_prepare(it_engine* e) {
    const it_model_config& c = e->cfg; it_ctx* cx = e->ctx;
    e->step = nullptr;
    { const char* v = getenv("IT_STEP_KERNEL"); if (v && atoi(v) == 0) return IT_OK; }
    if (e->world != 1) return IT_OK;                                  // row shards exchange results inside the per-op kernels
    if (c.ssm_state != ST_SD || c.conv_k > 8 || c.head_dim > 256 || c.head_dim % 8 || c.n_embd > 8192 || c.n_ff % 1024 || c.ssm_inner % 1024 || (c.n_head * c.head_dim) % 1024) return IT_OK;
    if (c.ssm_vheads > cx->sm_count || c.n_head > cx->sm_count || c.n_ff / 1024 > cx->sm_count || c.ssm_vheads % c.ssm_groups) return IT_OK;
    const size_t scratch = step_scratch_bytes(c);
    const long long ring = (long long)ST_SMEM - (long long)scratch - ST_BARS;
    int slots = 1;
    while (2 * slots <= 16 && (long long)(2 * slots) * ST_CHUNK <= ring) slots *= 2;   // a power of two: slot = chunk index & (slots - 1); at most 16 (the mbarriers share 384 reserved bytes)
    if (slots < 4) return IT_OK;
    IT_CUDA(cudaSetDevice(cx->device));
    static bool attr_set[16] = {};
    if (!attr_set[cx->device & 15]) { IT_CUDA(cudaFuncSetAttribute(k_decode_step, cudaFuncAttributeMaxDynamicSharedMemorySize, ST_SMEM)); attr_set[cx->device & 15] = true; }
    int per_sm = 0;
    IT_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_decode_step, ST_THREADS, (size_t)slots * ST_CHUNK + scratch + ST_BARS));
    if (per_sm < 1) return IT_OK;
    it_step_state* st = new it_step_state();
    st->grid = cx->sm_count; st->slots = slots; st->scratch = (int)scratch; st->gdn_off = (int)step_gdn_off(c);
    {   // Hadamard blocks on the last CTAs, attention heads behind the value heads when they all fit side by side
        const int widest = std::max(std::max(c.n_embd, c.n_ff), std::max(c.ssm_inner, c.n_head * c.head_dim)) / 1024;
        st->had_base = st->grid - widest;
        // several CTAs per attention head when the grid has them: each takes a share of the K tiles and of the output elements
        st->attn_g = 1;
        for (int g = 4; g > 1; g /= 2) if (c.head_dim % g == 0 && (c.head_dim / g) % it_vc_slice(c.head_dim) == 0 && g * c.n_head <= st->grid) { st->attn_g = g; break; }
        { const char* v = getenv("IT_STEP_ATTN_G"); if (v && (atoi(v) == 1 || atoi(v) == 2) && atoi(v) < st->attn_g) st->attn_g = atoi(v); }
        st->attn_base = (c.ssm_vheads + st->attn_g * c.n_head <= st->grid) ? c.ssm_vheads : 0;
    }
    st->layers_dev = nullptr; st->partials = nullptr; st->trace = nullptr; st->att_sc = nullptr; st->att_cnt = nullptr;
    st->att_stride = (c.ctx_len + 32 + 3) / 4 * 4;
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
    if (r == IT_OK) r = it_engine_dev_alloc(e, (void**)&st->att_sc, (size_t)c.n_head * st->att_stride * sizeof(float), true);
    if (r == IT_OK) r = it_engine_dev_alloc(e, (void**)&st->att_cnt, (size_t)c.n_head * sizeof(unsigned), true);
    { const char* v = getenv("IT_STEP_TRACE"); if (r == IT_OK && v && atoi(v) != 0) r = it_engine_dev_alloc(e, (void**)&st->trace, (2 * ST_TRACE_MAX * 2 + ST_EVT_MAX) * sizeof(unsigned long long), true); }
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
    P.slots = st->slots; P.scratch = st->scratch; P.flags = flags; P.trace = st->trace; P.gdn_off = st->gdn_off; P.had_base = st->had_base; P.attn_base = st->attn_base; P.attn_g = st->attn_g; P.att_sc = st->att_sc; P.att_stride = st->att_stride; P.att_cnt = st->att_cnt;
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

// Diagnostics (IT_STEP_TRACE=1 when the engine is built): the nanosecond clock of CTA 0 and of the last CTA when they arrive
// at and leave each grid barrier of the most recent step: out[(cta * max + barrier) * 2 + {0, 1}], cta in {0, 1}.
IT_API int it_engine_step_trace(it_engine* e, uint64_t* out, size_t max_barriers) {
    IT_CHECK_ARG(e && out, "it_engine_step_trace: null argument");
    if (!e->step || !e->step->trace) return it_fail(IT_ESTATE, "it_engine_step_trace: the engine was not built with IT_STEP_TRACE=1, or does not run the step kernel");
    IT_CHECK_ARG(max_barriers == ST_TRACE_MAX || max_barriers == ST_TRACE_MAX + ST_EVT_MAX / 4, "it_engine_step_trace: pass room for %d barriers per CTA", ST_TRACE_MAX);
    IT_CUDA(cudaMemcpyAsync(out, e->step->trace, (2 * ST_TRACE_MAX * 2 + (max_barriers > ST_TRACE_MAX ? ST_EVT_MAX : 0)) * sizeof(unsigned long long), cudaMemcpyDeviceToHost, e->ctx->stream));
    IT_CUDA(cudaStreamSynchronize(e->ctx->stream));
    return IT_OK;
}
