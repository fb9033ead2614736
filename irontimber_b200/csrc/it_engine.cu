// Engine construction (random-init weights generated on the device), teardown and read-back for parity tests.
#include "it_engine.h"
#include "it_support.h"
#include <algorithm>
#include <cmath>
#include <cstring>

namespace {

// f32 tensors of the synthetic model: value i = lo + (hi - lo) * u, u = top 24 bits of hash(seed, i) / 2^24, the
// product and the sum rounded separately.
__global__ void k_synth_f32(uint64_t seed, size_t n, float lo, float span, float* out) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float u = __fmul_rn((float)(uint32_t)(it_hash(seed, i) >> 40), 1.0f / 16777216.0f);
        out[i] = __fadd_rn(lo, __fmul_rn(span, u));
    }
}
// the tiled f16 K / V caches (it_kc_index, it_vc_index) back to rows [pos][kvd]
__global__ void k_kc_decode(const __half* src, float* dst, size_t n, int nkv, int hd, int is_v) {
    const size_t kvd = (size_t)nkv * hd;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t pos = i / kvd, r = i % kvd;
        dst[i] = __half2float(src[is_v ? it_vc_index(pos, (int)(r / hd), (int)(r % hd), nkv, hd) : it_kc_index(pos, (int)(r / hd), (int)(r % hd), nkv, hd)]);
    }
}

uint64_t tensor_seed(uint64_t seed, int layer, int tensor) { return it_hash(seed, (uint64_t)(layer + 2) * 64 + (uint64_t)tensor); }

struct Range { float lo, hi; };
Range f32_range(int tensor) {
    switch (tensor) {
        case IT_T_CONV: case IT_T_DT: return { -0.5f, 0.5f };
        case IT_T_A: return { -1.1f, -0.1f };                // decay a < 0, like the model (src/vk/kparity.rs:64)
        case IT_T_BETA: case IT_T_ALPHA: return { -0.05f, 0.05f };
        case IT_T_TOK_EMBD: return { -1.0f, 1.0f };
        default: return { 0.9f, 1.1f };                      // every norm weight
    }
}

int dev_alloc(it_engine* e, void** p, size_t bytes, bool zero) {
    cudaError_t ce = cudaMalloc(p, bytes);
    if (ce != cudaSuccess) return it_fail(IT_ENOMEM, "engine: cudaMalloc(%zu): %s", bytes, cudaGetErrorString(ce));
    e->owned.push_back(*p);
    if (zero) IT_CUDA(cudaMemsetAsync(*p, 0, bytes, e->ctx->stream));
    return IT_OK;
}
// ---- weights come from an it_weight_source; the helpers below own allocation, sharding and the tile layout
int load_f32(it_engine* e, it_weight_source* src, int layer, int tensor, size_t n, float** out) {
    IT_TRY(dev_alloc(e, (void**)out, n * sizeof(float), false));
    return src->f32(e, layer, tensor, n, *out);
}
// rows [row0, row0 + nrows) of a ternary tensor into tile storage that is already allocated
int load_tiles(it_engine* e, it_weight_source* src, int layer, int tensor, size_t rows, size_t cols, size_t row0, size_t nrows, uint8_t* tiles) {
    const size_t nbytes = nrows * (cols / 128) * 34; uint8_t* tmp = nullptr;
    cudaError_t ce = cudaMalloc(&tmp, nbytes);
    if (ce != cudaSuccess) return it_fail(IT_ENOMEM, "engine: staging allocation of %zu bytes failed: %s", nbytes, cudaGetErrorString(ce));
    int r = src->ternary(e, layer, tensor, rows, cols, row0, nrows, tmp);
    if (r == IT_OK) r = it_launch_repack_pq2(e->ctx, tmp, nrows, cols, tiles);
    if (r == IT_OK) ce = cudaStreamSynchronize(e->ctx->stream);
    cudaFree(tmp);
    if (r) return r;
    if (ce != cudaSuccess) return it_fail(IT_ECUDA, "engine: weight repack failed: %s", cudaGetErrorString(ce));
    return IT_OK;
}
// Trunk matrices are split by output rows over the ranks (every row is an independent dot with the replicated
// activations, src/cpu.rs:31-34): this engine loads and holds rows [rank*rows/world, (rank+1)*rows/world) only.
int load_mat(it_engine* e, it_weight_source* src, int layer, int tensor, size_t rows, size_t cols, it_mat** out) {
    size_t row0, n; IT_TRY(it_shard_range(rows, e->rank, e->world, &row0, &n));
    uint8_t* buf = nullptr;
    IT_TRY(dev_alloc(e, (void**)&buf, (n + 31) / 32 * (cols / 128) * IT_TILE_BYTES, false));
    IT_TRY(it_matrix_view(e->ctx, n, cols, buf, out));
    IT_TRY(load_tiles(e, src, layer, tensor, rows, cols, row0, n, buf));
    return e->world > 1 ? it_matrix_set_shard(*out, row0, rows) : IT_OK;
}
// Several ternary matrices with the same column count, stacked row-wise in one allocation: `stack` sees all rows,
// parts[i] is a view of tensor i.  Row counts (per rank) must be multiples of 32 so that every part starts on a row
// group.  On a sharded engine the stack holds this rank's rows of every part, and its row map sends each part's rows
// to their place in the full stacked output.
int load_stack(it_engine* e, it_weight_source* src, int layer, int n, const int* tensors, const size_t* rows, size_t cols, it_mat** parts, it_mat** stack) {
    size_t total = 0, full = 0, local[4], row0[4];
    for (int i = 0; i < n; i++) {
        IT_TRY(it_shard_range(rows[i], e->rank, e->world, &row0[i], &local[i]));
        if (local[i] % 32) return it_fail(IT_EINVAL, "engine: stacked matrix with %zu rows per rank is not a multiple of 32", local[i]);
        total += local[i]; full += rows[i];
    }
    uint8_t* buf = nullptr;
    IT_TRY(dev_alloc(e, (void**)&buf, total / 32 * (cols / 128) * IT_TILE_BYTES, false));
    size_t off = 0;
    for (int i = 0; i < n; i++) {
        uint8_t* tiles = buf + off / 32 * (cols / 128) * IT_TILE_BYTES;
        IT_TRY(it_matrix_view(e->ctx, local[i], cols, tiles, &parts[i]));
        IT_TRY(load_tiles(e, src, layer, tensors[i], rows[i], cols, row0[i], local[i], tiles));
        off += local[i];
    }
    IT_TRY(it_matrix_view(e->ctx, total, cols, buf, stack));
    if (e->world > 1) {
        it_mat* m = *stack; m->sharded = true; m->out_rows = full; m->map.nseg = n;
        size_t lo = 0, go = 0;
        for (int i = 0; i < n; i++) { m->map.start[i] = (int)lo; m->map.delta[i] = (int)(go + row0[i]) - (int)lo; m->map.shift[i] = (int)local[i]; lo += local[i]; go += rows[i]; }
    }
    return IT_OK;
}

// Random-init weights generated on the device from a seed: each tensor's values are a pure function of
// (seed, layer, tensor, element index), so a row shard generates exactly its rows of the full tensor.
struct SynthSource : it_weight_source {
    int signs(it_engine* e, size_t width, std::vector<float>* s) override {
        s->resize(width);
        const uint64_t sd = it_hash(e->seed, 7000 + width / 1024);
        for (size_t i = 0; i < width; i++) (*s)[i] = (it_hash(sd, i) & 1) ? 1.0f : -1.0f;
        return IT_OK;
    }
    int f32(it_engine* e, int layer, int tensor, size_t n, float* dev) override {
        const Range r = f32_range(tensor);
        k_synth_f32<<<e->ctx->sm_count * 4, 256, 0, e->ctx->stream>>>(tensor_seed(e->seed, layer, tensor), n, r.lo, r.hi - r.lo, dev);
        IT_LAUNCH_CHECK("synth_f32"); return IT_OK;
    }
    int ternary(it_engine* e, int layer, int tensor, size_t, size_t cols, size_t row0, size_t nrows, uint8_t* raw_dev) override {
        return it_launch_synth_pq2(e->ctx, tensor_seed(e->seed, layer, tensor), nrows, cols, 0, raw_dev, row0);
    }
    int q8(it_engine* e, int tensor, size_t rows, size_t cols, it_qmat** out) override {
        return it_qmatrix_synth(e->ctx, tensor_seed(e->seed, -1, tensor), rows, cols, out);
    }
};

size_t up64(size_t n) { return (n + 63) / 64 * 64; }

// Fail closed before any device work (validate_geometry, src/vk/mod.rs:207; prefill/config checks :180).
int validate(const it_model_config* c) {
    IT_CHECK_ARG(c, "it_engine_create_synth: null config");
    IT_CHECK_ARG(c->n_layer > 0 && c->n_layer <= 1024 && c->n_vocab > 0, "engine: bad layer or vocabulary count");
    IT_CHECK_ARG(c->n_embd > 0 && c->n_embd % 1024 == 0 && c->n_embd <= 8192 && c->n_ff > 0 && c->n_ff % 1024 == 0, "engine: n_embd (<= 8192) and n_ff must be multiples of the 1024 Hadamard block");
    IT_CHECK_ARG((c->n_head_kv * c->head_dim) % 32 == 0 && c->n_ff % 32 == 0, "engine: stacked matrices need row counts that are multiples of 32");
    IT_CHECK_ARG(c->head_dim > 0 && c->head_dim <= 256 && c->head_dim % 8 == 0, "engine: head_dim must be a multiple of 8 up to 256");
    IT_CHECK_ARG(c->n_head > 0 && c->n_head_kv > 0 && c->n_head % c->n_head_kv == 0, "engine: n_head must be a multiple of n_head_kv");
    IT_CHECK_ARG((c->n_head * c->head_dim) % 1024 == 0 && (c->n_head_kv * c->head_dim) % 4 == 0, "engine: attention width must be a multiple of 1024");
    IT_CHECK_ARG(c->n_rot > 0 && c->n_rot % 2 == 0 && c->n_rot <= c->head_dim, "engine: bad rope dimension count");
    IT_CHECK_ARG(c->conv_k >= 2 && c->conv_k <= 9, "engine: conv kernel size must be 2..9");
    IT_CHECK_ARG(c->ssm_state > 0 && c->ssm_state % 32 == 0 && c->ssm_state <= 256, "engine: ssm_state must be a multiple of 32 up to 256");
    IT_CHECK_ARG(c->ssm_groups > 0 && c->ssm_vheads > 0 && c->ssm_vheads % c->ssm_groups == 0, "engine: ssm_vheads must be a multiple of ssm_groups");
    IT_CHECK_ARG(c->ssm_inner == c->ssm_vheads * c->ssm_state && c->ssm_inner % 1024 == 0, "engine: ssm_inner must equal vheads * state and be a multiple of 1024");
    IT_CHECK_ARG(c->full_attn_interval >= 1, "engine: bad full_attention_interval");
    {   // the attention kernel keeps one row of scores in shared memory: the context capacity is bounded by what fits there
        const int cap = std::min(32768, it_sup_attention_max_positions(c->head_dim));
        IT_CHECK_ARG(c->ctx_len >= 16 && c->ctx_len <= cap, "engine: context capacity %d outside 16..%d (limit of the attention kernel at head dimension %d)", c->ctx_len, cap, c->head_dim);
    }
    IT_CHECK_ARG(c->eps > 0.f && c->rope_base > 1.f, "engine: bad eps or rope base");
    return IT_OK;
}

}  // namespace

IT_API int it_engine_create_synth(int device, const it_model_config* cfg, uint64_t seed, int with_mtp, it_engine** out) {
    return it_engine_create_synth_sharded(device, cfg, seed, with_mtp, 0, 1, out);
}
IT_API int it_engine_create_synth_sharded(int device, const it_model_config* cfg, uint64_t seed, int with_mtp, int rank, int world, it_engine** out) {
    SynthSource src;
    return it_engine_build(device, cfg, seed, with_mtp, rank, world, &src, out);
}

int it_engine_validate_config(const it_model_config* cfg) { return validate(cfg); }
int it_engine_dev_alloc(it_engine* e, void** p, size_t bytes, bool zero) { return dev_alloc(e, p, bytes, zero); }

int it_engine_build(int device, const it_model_config* cfg, uint64_t seed, int with_mtp, int rank, int world, it_weight_source* src, it_engine** out) {
    IT_CHECK_ARG(out && src, "engine: null output or weight source");
    *out = nullptr;
    IT_TRY(validate(cfg));
    IT_CHECK_ARG(world >= 1 && world <= IT_MAX_PEERS && rank >= 0 && rank < world, "engine: bad rank %d of %d", rank, world);
    {   // every trunk matrix must split evenly, stacked ones on row-group boundaries
        const int kvd_ = cfg->n_head_kv * cfg->head_dim, qf_ = 2 * cfg->n_head * cfg->head_dim, cd_ = it_cfg_conv_dim(*cfg);
        const int stacked[] = { cfg->n_ff, cd_, cfg->ssm_inner, qf_, kvd_ };
        for (int v : stacked) IT_CHECK_ARG(v % (32 * world) == 0, "engine: a stacked matrix of %d rows does not split over %d ranks on 32-row boundaries", v, world);
        IT_CHECK_ARG(cfg->n_embd % world == 0 && cfg->n_vocab % world == 0, "engine: n_embd and n_vocab must be multiples of the rank count %d", world);
    }
    const it_model_config& c = *cfg;
    const int e_ = c.n_embd, ff = c.n_ff, hd = c.head_dim, nh = c.n_head, nkv = c.n_head_kv, kvd = nkv * hd, qf = 2 * nh * hd;
    const int cd = it_cfg_conv_dim(c), inner = c.ssm_inner, nv = c.ssm_vheads, sd = c.ssm_state;
    it_engine* e = new it_engine();
    e->ctx = nullptr; e->step = nullptr; e->pin_next = 0; e->cfg = c; e->seed = seed; e->has_mtp = with_mtp != 0; e->rank = rank; e->world = world; e->output = nullptr; e->tok_embd = e->m_tok_embd = nullptr; e->q8 = nullptr; e->step_graph = nullptr; e->host_pin = nullptr; e->small_pin = nullptr; e->small_next = 0;
    { const char* v = getenv("IT_PASS_GRAPHS"); e->record_passes = !v || atoi(v) != 0; }
    e->m_eh = e->m_q = e->m_k = e->m_v = e->m_o = e->m_gate = e->m_up = e->m_down = nullptr;
    e->pos = 0; e->mpos = 1; e->hp_off = 0; e->hp_n = 0; e->last_rows = 0;
    // arena layout
    it_arena_layout& L = e->lay; size_t o = 0;
    auto take = [&](size_t& field, size_t n) { field = o; o += up64(n); };
    L.big1_stride = (size_t)std::max(std::max(cd + inner, qf + 2 * kvd), 2 * ff); L.big2_stride = (size_t)std::max(inner, ff);
    L.o_stride = (size_t)std::max(inner, nh * hd); L.logits_stride = up64((size_t)c.n_vocab) + 64;
    take(L.x, (size_t)IT_MAXT * e_); take(L.xn, (size_t)IT_MAXT * e_); take(L.big1, IT_MAXT * L.big1_stride); take(L.big2, IT_MAXT * L.big2_stride);
    take(L.conv, (size_t)IT_MAXT * cd); take(L.kcur, (size_t)IT_MAXT * kvd); take(L.vcur, (size_t)IT_MAXT * kvd); take(L.o, IT_MAXT * L.o_stride);
    take(L.beta, (size_t)IT_MAXT * nv); take(L.alpha, (size_t)IT_MAXT * nv); take(L.hrow, (size_t)IT_MAXT * e_); take(L.hprev, (size_t)e_);
    take(L.mh, (size_t)(IT_MAXT + 1) * e_); take(L.me, (size_t)IT_MAXT * e_); take(L.mcat, (size_t)IT_MAXT * 2 * e_); take(L.mx, (size_t)IT_MAXT * e_);
    take(L.logits, IT_MAXLOGIT * L.logits_stride); take(L.amx, 64); L.total = o;
    int r = it_ctx_create(device, L.total, &e->ctx);
    if (r) { delete e; return r; }
    auto fail = [&](int code) { it_engine_destroy(e); return code; };
#define E_TRY(expr) do { int r__ = (expr); if (r__) return fail(r__); } while (0)
    e->theta_scale = powf(c.rope_base, -2.0f / (float)c.n_rot);      // the same host expression as src/cpu.rs:147
    const size_t widths[4] = { (size_t)e_, (size_t)inner, (size_t)(nh * hd), (size_t)ff };
    for (size_t wdt : widths) {
        if (e->ctx->signs.count(wdt)) continue;
        std::vector<float> sg; E_TRY(src->signs(e, wdt, &sg));
        if (sg.size() != wdt) return fail(it_fail(IT_EINVAL, "engine: sign vector of width %zu has %zu entries", wdt, sg.size()));
        E_TRY(it_signs_set(e->ctx, wdt, sg.data()));
    }
    e->layers.resize(c.n_layer);
    for (int il = 0; il < c.n_layer; il++) {
        it_layer& l = e->layers[il]; memset(&l, 0, sizeof l);
        l.recurrent = it_cfg_recurrent(c, il);
        E_TRY(load_f32(e, src, il, IT_T_ATTN_NORM, e_, &l.attn_norm)); E_TRY(load_f32(e, src, il, IT_T_POST_NORM, e_, &l.post_norm));
        { const int ts[2] = { IT_T_FFN_GATE, IT_T_FFN_UP }; const size_t rs[2] = { (size_t)ff, (size_t)ff }; it_mat* parts[2];
          E_TRY(load_stack(e, src, il, 2, ts, rs, e_, parts, &l.gate_up)); l.ffn_gate = parts[0]; l.ffn_up = parts[1]; }
        E_TRY(load_mat(e, src, il, IT_T_FFN_DOWN, e_, ff, &l.ffn_down));
        if (l.recurrent) {
            { const int ts[2] = { IT_T_QKV, IT_T_GATE }; const size_t rs[2] = { (size_t)cd, (size_t)inner }; it_mat* parts[2];
              E_TRY(load_stack(e, src, il, 2, ts, rs, e_, parts, &l.in_proj)); l.qkv = parts[0]; l.gate = parts[1]; }
            E_TRY(load_mat(e, src, il, IT_T_SSM_OUT, e_, inner, &l.ssm_out));
            E_TRY(load_f32(e, src, il, IT_T_CONV, (size_t)cd * c.conv_k, &l.conv_w)); E_TRY(load_f32(e, src, il, IT_T_DT, nv, &l.dt)); E_TRY(load_f32(e, src, il, IT_T_A, nv, &l.a));
            E_TRY(load_f32(e, src, il, IT_T_BETA, (size_t)nv * e_, &l.beta)); E_TRY(load_f32(e, src, il, IT_T_ALPHA, (size_t)nv * e_, &l.alpha)); E_TRY(load_f32(e, src, il, IT_T_SSM_NORM, sd, &l.ssm_norm));
            const size_t csz = (size_t)(c.conv_k - 1) * cd, ssz = (size_t)nv * sd * sd;
            E_TRY(dev_alloc(e, (void**)&l.conv_st, csz * 4, true)); E_TRY(dev_alloc(e, (void**)&l.ssm_st, ssz * 4, true));
            E_TRY(dev_alloc(e, (void**)&l.ck_conv, IT_MAXCK * csz * 4, true)); E_TRY(dev_alloc(e, (void**)&l.ck_ssm, IT_MAXCK * ssz * 4, true));
        } else {
            { const int ts[3] = { IT_T_Q, IT_T_K, IT_T_V }; const size_t rs[3] = { (size_t)qf, (size_t)kvd, (size_t)kvd }; it_mat* parts[3];
              E_TRY(load_stack(e, src, il, 3, ts, rs, e_, parts, &l.in_proj)); l.q = parts[0]; l.k = parts[1]; l.v = parts[2]; }
            E_TRY(load_mat(e, src, il, IT_T_O, e_, nh * hd, &l.o));
            E_TRY(load_f32(e, src, il, IT_T_Q_NORM, hd, &l.q_norm)); E_TRY(load_f32(e, src, il, IT_T_K_NORM, hd, &l.k_norm));
            E_TRY(dev_alloc(e, (void**)&l.kc, (size_t)((c.ctx_len + 31) / 32 * 32) * kvd * 2, true));   // tiles of 32 positions
            E_TRY(dev_alloc(e, (void**)&l.vc, (size_t)((c.ctx_len + 31) / 32 * 32) * kvd * 2, true));   // tiled like K (it_vc_index)
        }
    }
    E_TRY(load_f32(e, src, -1, IT_T_TOK_EMBD, (size_t)c.n_vocab * e_, &e->tok_embd));
    E_TRY(load_f32(e, src, -1, IT_T_OUTPUT_NORM, e_, &e->output_norm));
    E_TRY(load_mat(e, src, -1, IT_T_OUTPUT, c.n_vocab, e_, &e->output));
    if (e->has_mtp) {
        E_TRY(src->q8(e, IT_T_MTP_EH, e_, 2 * e_, &e->m_eh)); E_TRY(src->q8(e, IT_T_MTP_Q, qf, e_, &e->m_q)); E_TRY(src->q8(e, IT_T_MTP_K, kvd, e_, &e->m_k));
        E_TRY(src->q8(e, IT_T_MTP_V, kvd, e_, &e->m_v)); E_TRY(src->q8(e, IT_T_MTP_O, e_, nh * hd, &e->m_o)); E_TRY(src->q8(e, IT_T_MTP_GATE, ff, e_, &e->m_gate));
        E_TRY(src->q8(e, IT_T_MTP_UP, ff, e_, &e->m_up)); E_TRY(src->q8(e, IT_T_MTP_DOWN, e_, ff, &e->m_down));
        E_TRY(load_f32(e, src, -1, IT_T_MTP_ENORM, e_, &e->m_enorm)); E_TRY(load_f32(e, src, -1, IT_T_MTP_HNORM, e_, &e->m_hnorm)); E_TRY(load_f32(e, src, -1, IT_T_MTP_ATTN_NORM, e_, &e->m_attn_norm));
        E_TRY(load_f32(e, src, -1, IT_T_MTP_POST_NORM, e_, &e->m_post_norm)); E_TRY(load_f32(e, src, -1, IT_T_MTP_Q_NORM, hd, &e->m_q_norm)); E_TRY(load_f32(e, src, -1, IT_T_MTP_K_NORM, hd, &e->m_k_norm));
        E_TRY(load_f32(e, src, -1, IT_T_MTP_HEAD_NORM, e_, &e->m_head_norm));
        e->m_tok_embd = e->tok_embd; E_TRY(src->mtp_embd(e, &e->m_tok_embd));
        E_TRY(dev_alloc(e, (void**)&e->mkc, (size_t)c.ctx_len * kvd * 4, true)); E_TRY(dev_alloc(e, (void**)&e->mvc, (size_t)c.ctx_len * kvd * 4, true));
    }
    E_TRY(it_q8_create(e->ctx, (size_t)std::max(std::max(e_, ff), std::max(inner, nh * hd)), IT_MAXT, &e->q8));
    E_TRY(dev_alloc(e, (void**)&e->toks_dev, (2 * IT_MAXT + 8) * sizeof(uint32_t), true));
    E_TRY(dev_alloc(e, (void**)&e->pos_dev, 64, true));
    if (cudaHostAlloc((void**)&e->host_pin, (size_t)IT_PIN_SLOTS * IT_PIN_WORDS * sizeof(uint32_t), cudaHostAllocDefault) != cudaSuccess) return fail(it_fail(IT_ENOMEM, "engine: pinned staging allocation failed"));
    if (cudaHostAlloc((void**)&e->small_pin, IT_SMALL_SLOTS * 16 * sizeof(uint32_t), cudaHostAllocDefault) != cudaSuccess) return fail(it_fail(IT_ENOMEM, "engine: pinned staging allocation failed"));
    if (cudaStreamSynchronize(e->ctx->stream) != cudaSuccess) return fail(it_fail(IT_ECUDA, "engine: weight generation failed: %s", cudaGetErrorString(cudaGetLastError())));
    E_TRY(it_step_prepare(e));
#undef E_TRY
    *out = e; return IT_OK;
}

IT_API void it_engine_destroy(it_engine* e) {
    if (!e) return;
    if (e->ctx) { cudaSetDevice(e->ctx->device); cudaStreamSynchronize(e->ctx->stream); }
    if (e->step_graph) it_graph_destroy(e->step_graph);
    it_step_release(e);
    for (auto& kv : e->pass_graphs) it_graph_destroy(kv.second);
    if (e->small_pin) cudaFreeHost(e->small_pin);
    for (it_layer& l : e->layers) {
        it_mat* ms[] = { l.ffn_gate, l.ffn_up, l.ffn_down, l.qkv, l.gate, l.ssm_out, l.q, l.k, l.v, l.o, l.in_proj, l.gate_up };
        for (it_mat* m : ms) it_matrix_destroy(m);
    }
    it_matrix_destroy(e->output);
    it_qmat* qs[] = { e->m_eh, e->m_q, e->m_k, e->m_v, e->m_o, e->m_gate, e->m_up, e->m_down };
    for (it_qmat* q : qs) it_qmatrix_destroy(q);
    it_q8_destroy(e->q8);
    for (void* p : e->owned) cudaFree(p);
    if (e->host_pin) cudaFreeHost(e->host_pin);
    it_ctx_destroy(e->ctx);
    delete e;
}
IT_API it_ctx* it_engine_ctx(it_engine* e) { return e ? e->ctx : nullptr; }
IT_API int it_engine_position(it_engine* e) { return e ? e->pos : -1; }

// ---------------------------------------------------------------- read-back
namespace {
struct TensorRef { int kind; const it_mat* m; const it_qmat* q; const float* f; size_t n; };   // kind 0 none, 1 ternary, 2 q8_0, 3 f32
TensorRef find_tensor(it_engine* e, int layer, int t) {
    const it_model_config& c = e->cfg; const int e_ = c.n_embd, hd = c.head_dim, nv = c.ssm_vheads, cd = it_cfg_conv_dim(c);
    TensorRef r{0, nullptr, nullptr, nullptr, 0};
    auto M = [&](const it_mat* m) { r.kind = m ? 1 : 0; r.m = m; }; auto Q = [&](const it_qmat* q) { r.kind = q ? 2 : 0; r.q = q; };
    auto F = [&](const float* f, size_t n) { r.kind = f ? 3 : 0; r.f = f; r.n = n; };
    if (layer >= 0) {
        if (layer >= c.n_layer) return r;
        const it_layer& l = e->layers[layer];
        switch (t) {
            case IT_T_ATTN_NORM: F(l.attn_norm, e_); break; case IT_T_POST_NORM: F(l.post_norm, e_); break;
            case IT_T_FFN_GATE: M(l.ffn_gate); break; case IT_T_FFN_UP: M(l.ffn_up); break; case IT_T_FFN_DOWN: M(l.ffn_down); break;
            case IT_T_QKV: M(l.qkv); break; case IT_T_GATE: M(l.gate); break; case IT_T_SSM_OUT: M(l.ssm_out); break;
            case IT_T_CONV: F(l.conv_w, (size_t)cd * c.conv_k); break; case IT_T_DT: F(l.dt, nv); break; case IT_T_A: F(l.a, nv); break;
            case IT_T_BETA: F(l.beta, (size_t)nv * e_); break; case IT_T_ALPHA: F(l.alpha, (size_t)nv * e_); break; case IT_T_SSM_NORM: F(l.ssm_norm, c.ssm_state); break;
            case IT_T_Q: M(l.q); break; case IT_T_K: M(l.k); break; case IT_T_V: M(l.v); break; case IT_T_O: M(l.o); break;
            case IT_T_Q_NORM: F(l.q_norm, hd); break; case IT_T_K_NORM: F(l.k_norm, hd); break;
        }
        return r;
    }
    switch (t) {
        case IT_T_TOK_EMBD: F(e->tok_embd, (size_t)c.n_vocab * e_); break; case IT_T_OUTPUT_NORM: F(e->output_norm, e_); break; case IT_T_OUTPUT: M(e->output); break;
        case IT_T_MTP_EH: Q(e->m_eh); break; case IT_T_MTP_Q: Q(e->m_q); break; case IT_T_MTP_K: Q(e->m_k); break; case IT_T_MTP_V: Q(e->m_v); break;
        case IT_T_MTP_O: Q(e->m_o); break; case IT_T_MTP_GATE: Q(e->m_gate); break; case IT_T_MTP_UP: Q(e->m_up); break; case IT_T_MTP_DOWN: Q(e->m_down); break;
    }
    if (e->has_mtp) switch (t) {
        case IT_T_MTP_ENORM: F(e->m_enorm, e_); break; case IT_T_MTP_HNORM: F(e->m_hnorm, e_); break; case IT_T_MTP_ATTN_NORM: F(e->m_attn_norm, e_); break;
        case IT_T_MTP_POST_NORM: F(e->m_post_norm, e_); break; case IT_T_MTP_Q_NORM: F(e->m_q_norm, hd); break; case IT_T_MTP_K_NORM: F(e->m_k_norm, hd); break;
        case IT_T_MTP_HEAD_NORM: F(e->m_head_norm, e_); break; case IT_T_MTP_EMBD: F(e->m_tok_embd, (size_t)c.n_vocab * e_); break;
    }
    return r;
}
}  // namespace

IT_API int it_engine_tensor_bytes(it_engine* e, int layer, int tensor, size_t* nbytes) {
    IT_CHECK_ARG(e && nbytes, "it_engine_tensor_bytes: null argument");
    const TensorRef r = find_tensor(e, layer, tensor);
    IT_CHECK_ARG(r.kind != 0, "it_engine_tensor_bytes: layer %d has no tensor %d", layer, tensor);
    *nbytes = r.kind == 1 ? r.m->rows * (r.m->cols / 128) * 34 : r.kind == 2 ? (r.q->s16 ? r.q->rows * r.q->cols / 16 * 20 : r.q->rows * (r.q->cols / 32) * 34) : r.n * 4;
    return IT_OK;
}
IT_API int it_engine_tensor_read(it_engine* e, int layer, int tensor, void* host) {
    IT_CHECK_ARG(e && host, "it_engine_tensor_read: null argument");
    const TensorRef r = find_tensor(e, layer, tensor);
    IT_CHECK_ARG(r.kind != 0, "it_engine_tensor_read: layer %d has no tensor %d", layer, tensor);
    if (r.kind == 1) return it_matrix_download_pq2(e->ctx, r.m, (uint8_t*)host);
    if (r.kind == 2) return r.q->s16 ? it_qmatrix_download_g16(e->ctx, r.q, (uint8_t*)host) : it_qmatrix_download_q8_0(e->ctx, r.q, (uint8_t*)host);
    IT_CUDA(cudaMemcpyAsync(host, r.f, r.n * 4, cudaMemcpyDeviceToHost, e->ctx->stream));
    IT_CUDA(cudaStreamSynchronize(e->ctx->stream)); return IT_OK;
}
IT_API int it_engine_signs_read(it_engine* e, size_t width, float* host) {
    IT_CHECK_ARG(e && host, "it_engine_signs_read: null argument");
    auto it = e->ctx->signs.find(width);
    IT_CHECK_ARG(it != e->ctx->signs.end(), "it_engine_signs_read: no sign vector of width %zu", width);
    IT_CUDA(cudaMemcpyAsync(host, it->second, width * 4, cudaMemcpyDeviceToHost, e->ctx->stream));
    IT_CUDA(cudaStreamSynchronize(e->ctx->stream)); return IT_OK;
}
IT_API int it_engine_state_read(it_engine* e, int layer, int which, float* host, size_t max_floats, size_t* n_floats) {
    IT_CHECK_ARG(e && n_floats, "it_engine_state_read: null argument");
    const it_model_config& c = e->cfg; const size_t kvd = (size_t)c.n_head_kv * c.head_dim;
    const float* src = nullptr; const __half* hsrc = nullptr; size_t n = 0;
    if (which >= 4) { IT_CHECK_ARG(e->has_mtp, "it_engine_state_read: no MTP head"); n = (size_t)(e->mpos - 1) * kvd; src = which == 4 ? e->mkc : e->mvc; }
    else {
        IT_CHECK_ARG(layer >= 0 && layer < c.n_layer, "it_engine_state_read: bad layer %d", layer);
        const it_layer& l = e->layers[layer];
        if (which < 2) { IT_CHECK_ARG(l.recurrent, "it_engine_state_read: layer %d is not recurrent", layer);
            n = which == 0 ? (size_t)(c.conv_k - 1) * it_cfg_conv_dim(c) : (size_t)c.ssm_vheads * c.ssm_state * c.ssm_state; src = which == 0 ? l.conv_st : l.ssm_st; }
        else { IT_CHECK_ARG(!l.recurrent, "it_engine_state_read: layer %d has no KV cache", layer); n = (size_t)e->pos * kvd; hsrc = which == 2 ? l.kc : l.vc; }
    }
    *n_floats = n;
    if (!host || n == 0) return IT_OK;
    IT_CHECK_ARG(n <= max_floats, "it_engine_state_read: buffer too small (%zu > %zu)", n, max_floats);
    if (hsrc) {   // decode f16 -> f32 on the device (decode_kv_readback, src/vk/mod.rs:965)
        float* tmp = nullptr; IT_CUDA(cudaMalloc(&tmp, n * 4));
        k_kc_decode<<<e->ctx->sm_count, 256, 0, e->ctx->stream>>>(hsrc, tmp, n, c.n_head_kv, c.head_dim, which == 3 ? 1 : 0);
        cudaError_t er = cudaMemcpyAsync(host, tmp, n * 4, cudaMemcpyDeviceToHost, e->ctx->stream);
        if (er == cudaSuccess) er = cudaStreamSynchronize(e->ctx->stream);
        cudaFree(tmp);
        if (er != cudaSuccess) return it_fail(IT_ECUDA, "it_engine_state_read: %s", cudaGetErrorString(er));
        return IT_OK;
    }
    IT_CUDA(cudaMemcpyAsync(host, src, n * 4, cudaMemcpyDeviceToHost, e->ctx->stream));
    IT_CUDA(cudaStreamSynchronize(e->ctx->stream)); return IT_OK;
}
IT_API int it_engine_hidden_read(it_engine* e, size_t row, float* host) {
    IT_CHECK_ARG(e && host && row < IT_MAXT, "it_engine_hidden_read: bad argument");
    return it_arena_read(e->ctx, e->lay.hrow + row * e->cfg.n_embd, host, e->cfg.n_embd);
}
