// Launchers of the decoder support kernels (it_support.cu), used by the engine.
#pragma once
#include "it_internal.h"

// f16 K cache of the trunk (not the V cache, not the head's f32 caches): positions are stored in tiles of 32, and inside a
// tile the same 16-byte piece (8 elements) of the 32 positions is contiguous, so that one thread per position reads its
// row with fully coalesced 16-byte loads.  Element j of kv head kh at position pos:
__host__ __device__ static inline size_t it_kc_index(size_t pos, int kh, int j, int nkv, int hd) {
    return (((pos >> 5) * (size_t)nkv + kh) * (size_t)(hd >> 3) + (size_t)(j >> 3)) * 256 + (pos & 31) * 8 + (j & 7);
}

// f16 V cache of the trunk: tiles of 32 positions per KV head, [position tile][kv head][slice][32 positions][64 elements]
// (slices of 64 elements; one slice of head_dim elements when head_dim is not a multiple of 64).  The V rows of 32
// positions of one head are one contiguous block (one bulk copy), and so is any run of slices of it: a CTA that owns a
// quarter of a head's output elements fetches its quarter of a tile with one copy.
__host__ __device__ static inline int it_vc_slice(int hd) { return (hd & 63) ? hd : 64; }
__host__ __device__ static inline size_t it_vc_index(size_t pos, int kh, int j, int nkv, int hd) {
    const int vs = it_vc_slice(hd), ns = hd / vs;
    return ((((pos >> 5) * (size_t)nkv + kh) * ns + (size_t)(j / vs)) * 32 + (pos & 31)) * (size_t)vs + (size_t)(j % vs);
}

#define IT_GDN_MAXROWS 64    // rows of one pass the fused delta-rule kernel stages in shared memory (it_sup_gdn_norm)

// Work done on the way into the Hadamard + q8k kernel.  mode 0: nothing.  mode 1: input = silu(x) * b (b is a device
// pointer, rows b_stride apart).  mode 2: input = rmsnorm(x) over the whole row of width n with weight w and eps; when
// xn_out is set the normed f32 row is also stored there (rows xn_stride apart).
struct it_had_prologue {
    int mode = 0;
    const float* b = nullptr; size_t b_stride = 0;
    const float* w = nullptr; float eps = 0.f; unsigned n = 0; float* xn_out = nullptr; size_t xn_stride = 0;
};
int it_sup_hadamard_q8_fused(it_ctx* c, size_t n, size_t ntok, size_t x_off, size_t x_stride, it_q8* out, const it_had_prologue& pro);

int it_sup_embed(it_ctx* c, const uint32_t* toks_dev, const float* table, int e, int nt, float* x);
int it_sup_rmsnorm_wide(it_ctx* c, const float* x, size_t xs, const float* w, int n, float eps, float* out, size_t os, int nt);
int it_sup_norm_head(it_ctx* c, const float* in, size_t in_hs, size_t in_ts, float* out, size_t out_hs, size_t out_ts, int n, int nheads, const float* w, int mode, float eps,
                     const float* z, size_t z_hs, size_t z_ts, int nt);
int it_sup_rope(it_ctx* c, float* x, size_t hs, size_t ts, int nheads, int nt, int pos0, const int* pos_ptr, int n_rot, float theta_scale, const int* sections);
int it_sup_conv(it_ctx* c, const float* mixed, size_t m_ts, const float* w, float* state, float* out, size_t o_ts, int cd, int kk, int nt, float* ck, size_t ck_stride, int nck);
int it_sup_dense_rows(it_ctx* c, const float* w0, const float* w1, int rows, int cols, const float* x, size_t x_ts, float* y0, float* y1, size_t y_ts, int nt);
int it_sup_gdn(it_ctx* c, const float* co, size_t co_ts, const float* beta, const float* alpha, size_t ba_ts, const float* dt, const float* a, float* state, float* o, size_t o_ts,
               int nv, int nk, int sd, int qk, int nt, float* ck, size_t ck_stride, int nck);
int it_sup_silu_mul(it_ctx* c, const float* g, const float* u, float* out, size_t n);
int it_sup_kv_store(it_ctx* c, const float* k, const float* v, size_t ts, void* kc, void* vc, int kvd, int hd, int slot0, const int* pos_ptr, int nt, int f16);   // f16: K goes to the tiled layout
int it_sup_attention(it_ctx* c, const float* q, size_t q_hs, size_t q_ts, const float* gate, const void* kc, const void* vc, int kvd, int hd, int nh, int nkv, int slot0,
                     const int* pos_ptr, int max_pos, float* out, size_t o_ts, int nt, int f16);

// Longest context one attention launch can serve at this head dimension (its row of scores lives in shared memory).
int it_sup_attention_max_positions(int hd);
// Prompt-pass attention over the trunk's tiled f16 caches (it_attention_prefill.cu): same results as it_sup_attention.
// Returns 1 when the shape does not fit (nothing launched), a negative code on error.
int it_sup_attention_prefill(it_ctx* c, const float* q, size_t q_hs, size_t q_ts, const float* gate, const void* kc, const void* vc, int hd, int nh, int nkv, int slot0,
                             float* out, size_t o_ts, int nt);

// Fused forms for passes of up to 8 rows (same arithmetic and order as the separate kernels; see it_support.cu).
int it_sup_attn_prep(it_ctx* c, float* qkv, size_t ts, int nh, int nkv, int hd, const float* q_norm, const float* k_norm, float eps, int pos0, const int* pos_ptr,
                     int n_rot, float theta_scale, const int* sections, void* kc, void* vc, int nt);
int it_sup_conv_l2_dense(it_ctx* c, const float* mixed, size_t m_ts, const float* cw, float* state, float* out, size_t o_ts, int cd, int kk, int sd, int nk, int nt,
                         float* ck, size_t ck_stride, int nck, float eps, const float* w0, const float* w1, int rows, int cols, const float* x, size_t x_ts,
                         float* y0, float* y1, size_t y_ts);
int it_sup_gdn_norm(it_ctx* c, const float* co, size_t co_ts, const float* beta, const float* alpha, size_t ba_ts, const float* dt, const float* a, float* state, float* o, size_t o_ts,
                    int nv, int nk, int sd, int qk, int nt, float* ck, size_t ck_stride, int nck, const float* nw, float eps, const float* z, size_t z_ts);
