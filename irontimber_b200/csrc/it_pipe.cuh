// Device helpers shared by the ternary matvec and matmul kernels: mbarrier waits with a time limit, bulk asynchronous
// copies into shared memory, and the int8 tensor-core instruction both kernels are built on.
#pragma once
#include <cstdint>
#include "it_internal.h"

namespace {

constexpr long long WAIT_CLOCKS = 1ll << 31;      // about one second
constexpr long long PEER_WAIT_CLOCKS = 1ll << 33; // default limit of a wait for a peer, about four seconds: another process may be a little behind

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_arrive(unsigned bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory"); }
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory"); }
__device__ __forceinline__ bool mbar_test(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// The same with a suspend-time hint: the warp may sleep up to `ns` nanoseconds inside the instruction and wakes when the
// phase completes, so a long wait costs a few instructions instead of a spin loop's thousands of issue slots.
__device__ __forceinline__ bool mbar_test_hint(unsigned bar, unsigned parity, unsigned ns) {
    unsigned ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}
// Non-blocking probe of a phase.
__device__ __forceinline__ bool mbar_poll(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
#ifndef IT_MBAR_SLEEP_NS
#define IT_MBAR_SLEEP_NS 20000u
#endif
// Bounded wait: gives up after WAIT_CLOCKS, or as soon as another thread of the CTA has given up.  The retry loop is one
// function when IT_PIPE_OUTLINE_WAIT is defined (a kernel whose speed is its code size calls it from dozens of places);
// it takes values only, so the caller's state stays in registers.
#ifdef IT_PIPE_OUTLINE_WAIT
#define IT_WAIT_SLOW static __device__ __noinline__
#else
#define IT_WAIT_SLOW __device__ __forceinline__
#endif
IT_WAIT_SLOW bool mbar_wait_retry(unsigned bar, unsigned parity, volatile int* abort_flag, int* error_flag, int site) {
    const long long t0 = clock64();
    for (;;) {
        for (int i = 0; i < 8; i++) if (mbar_test_hint(bar, parity, IT_MBAR_SLEEP_NS)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_CLOCKS) { if (!*abort_flag) atomicExch(error_flag, site); *abort_flag = 1; return false; }
    }
}
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag, int* error_flag, int site = 1) {
    if (mbar_test(bar, parity)) return true;
    return mbar_wait_retry(bar, parity, abort_flag, error_flag, site);
}
__device__ __forceinline__ void bulk_load(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// One box of a tiled tensor map (here: 128 bytes x 64 rows of int8 activations) into shared memory; x must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(unsigned dst, const void* tensor_map, int x, int y, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 :: "r"(dst), "l"(tensor_map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(smem_u32(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory"); }
template <int NTHREADS> __device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" :: "n"(NTHREADS) : "memory"); }
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}


// ---- results of a row shard: pushed into every rank's arena -----------------------------------------------------
// Store of one result at float offset `off` of the arena: on a sharded launch (P != null) the value goes to the same
// offset in every rank's arena (own included), plain peer stores over NVLink; accum adds to this rank's old value,
// which is the same on every rank.
__device__ __forceinline__ void it_result_store(const it_peers* P, float* own_arena, size_t off, float v, int accum) {
    if (accum) v = __fadd_rn(__ldcg(own_arena + off), v);
    if (!P) { own_arena[off] = v; return; }
    const int world = P->world;
    for (int p = 0; p < world; p++) P->arena[p][off] = v;
}
// End of a sharded kernel.  Every thread that stored results has issued __threadfence_system() and the CTA has passed
// a barrier before ONE thread of the CTA calls this.  The last CTA to arrive publishes this rank's slice (a release
// store of the new epoch into every peer's flag word for this rank) and then waits until every peer has published the
// same epoch here, so that when the kernel completes the full result is in this rank's arena.  The wait is bounded;
// when it runs out the error flag is raised and the kernel leaves.
__device__ __forceinline__ void it_shard_finish(const it_peers* P, unsigned total_ctas, int* error_flag) {
    const unsigned old = atomicAdd(P->done, 1u);
    if (old != total_ctas - 1) return;
    *P->done = 0;
    __threadfence_system();
    const unsigned e = *P->epoch + 1u;
    const int rank = P->rank, world = P->world;
    for (int p = 0; p < world; p++) if (p != rank) asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(P->flags[p] + rank), "r"(e) : "memory");
    const long long t0 = clock64();
    for (int q = 0; q < world; q++) {
        if (q == rank) continue;
        const unsigned* f = P->flags[rank] + q;
        for (;;) {
            unsigned v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if ((int)(v - e) >= 0) break;
            if (clock64() - t0 > P->wait_clocks) { atomicExch(error_flag, 21); q = world; break; }
        }
    }
    *P->epoch = e;
}

// Low-latency exchange of one result (the decode path, where an exchange is pure latency).  The value travels as an
// 8-byte (value, epoch) slot written with one store, so it is complete the moment its tag matches: no fence, no flag,
// one NVLink crossing.  The calling thread pushes its result into the slot of output row `grow` in every peer's buffer,
// stores it into its own arena, then collects the results of the same local row of every peer (output row
// grow + (p - rank) * shift) from its own buffer as they arrive and stores them too.  Slots of even and odd epochs
// live in different halves, and a rank cannot run two ops ahead of a peer, so a slot is never overwritten before it was read.
__device__ __forceinline__ void it_result_exchange_ll(const it_peers* P, float* arena, size_t row_off, size_t slot0, int grow, int shift,
                                                      float v, int accum, unsigned e, int* error_flag) {
    if (accum) v = __fadd_rn(__ldcg(arena + row_off + grow), v);
    const int rank = P->rank, world = P->world;
    const size_t half = (size_t)(e & 1u) * P->ll_slots + slot0;
    const unsigned long long packed = ((unsigned long long)e << 32) | (unsigned long long)__float_as_uint(v);
    for (int p = 0; p < world; p++) if (p != rank) asm volatile("st.volatile.global.u64 [%0], %1;" :: "l"(P->ll[p] + half + grow), "l"(packed) : "memory");
    arena[row_off + grow] = v;
    const long long t0 = clock64();
    for (int p = 0; p < world; p++) {
        if (p == rank) continue;
        const int gp = grow + (p - rank) * shift;
        const unsigned long long* slot = P->ll[rank] + half + gp;
        unsigned long long x;
        for (;;) {
            asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(x) : "l"(slot) : "memory");
            if ((unsigned)(x >> 32) == e) break;
            if (clock64() - t0 > P->wait_clocks) { atomicExch(error_flag, 22); return; }
        }
        arena[row_off + gp] = __uint_as_float((unsigned)x);
    }
}
// End of a kernel that exchanged its results slot by slot: the last CTA moves the epoch on.  One thread per CTA, after a CTA barrier.
__device__ __forceinline__ void it_shard_finish_ll(const it_peers* P, unsigned total_ctas) {
    const unsigned old = atomicAdd(P->done, 1u);
    if (old != total_ctas - 1) return;
    *P->done = 0;
    *P->epoch = *P->epoch + 1u;
}

}  // namespace
