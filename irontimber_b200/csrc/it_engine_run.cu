// Forward passes, the MtpBackend hooks and the generation loops of the engine.
//
// The schedule of one pass is the reference's run_chunk_v (src/vk/mod.rs:763-892): per layer norm -> Hadamard ->
// grouped ternary matvecs -> delta-rule or attention block -> Hadamard -> output matvec (accumulating into the residual)
// -> norm -> Hadamard -> gate / up -> silu*mul -> Hadamard -> down (accumulating).  Differences: the Hadamard is fused
// with q8k quantisation (the CPU numerics), embeddings are gathered on the device, and a pass takes up to IT_MAXT rows (four
// times the reference's prompt chunk; the chunk size changes no result): passes of more than eight rows run their ternary
// products on the tile kernels.
#include "it_engine.h"
#include "it_support.h"
#include <algorithm>
#include <vector>

namespace {

__global__ void k_set_tokens(const float* amx, uint32_t* toks, int* pos, int advance) {
    // the greedy pick of the step just finished becomes the next step's input; the position moves on
    toks[0] = __float_as_uint(amx[0]);
    if (advance) *pos += advance;
}

int had_mv(it_engine* e, const it_mat* w, int nt, size_t x_off, size_t x_stride, size_t y_off, size_t y_stride, int acc, bool rehad, size_t hd = 0, size_t nk = 0, size_t rep = 0) {
    // `had` + `mv` (src/vk/mod.rs:749, :653); rehad = false reuses the q8 rows of the previous call (grouped matvecs on one input)
    if (rehad) IT_TRY(it_hadamard_q8(e->ctx, w->cols, nt, x_off, x_stride, 1, 1, hd, nk, rep, e->q8));
    return it_matvec_t2(e->ctx, w, nt, e->q8, y_off, y_stride, acc);
}

int logits_and_argmax(it_engine* e, size_t h_off, int rows) {
    // LM head on `rows` output-normed rows + one argmax per row (src/vk/mod.rs:862-876)
    const it_arena_layout& L = e->lay; const it_model_config& c = e->cfg;
    IT_TRY(had_mv(e, e->output, rows, h_off, c.n_embd, L.logits, L.logits_stride, 0, true));
    for (int t = 0; t < rows; t++) IT_TRY(it_argmax(e->ctx, L.logits + t * L.logits_stride, c.n_vocab, L.amx + t));
    return IT_OK;
}

}  // namespace

// The next block of the pinned staging ring.  Copies out of a block are asynchronous and the host runs passes ahead of the
// device, so a block is reused only after a synchronisation has shown that every copy out of the ring has run.
static uint32_t* pin_block(it_engine* e) {
    if (e->pin_next == IT_PIN_SLOTS) { cudaStreamSynchronize(e->ctx->stream); e->pin_next = 0; }
    return e->host_pin + (size_t)IT_PIN_WORDS * (size_t)(e->pin_next++);
}

int it_engine_run_chunk(it_engine* e, const uint32_t* toks, int nt, int logit_rows, int nck, bool from_dev) {
    it_ctx* cx = e->ctx; const it_model_config& c = e->cfg; const it_arena_layout& L = e->lay;
    float* A = cx->arena;
    const int e_ = c.n_embd, ff = c.n_ff, hd = c.head_dim, nh = c.n_head, nkv = c.n_head_kv, kvd = nkv * hd, qf = 2 * nh * hd;
    const int cd = it_cfg_conv_dim(c), inner = c.ssm_inner, nv = c.ssm_vheads, sd = c.ssm_state, nk = c.ssm_groups, qk = it_cfg_qk(c);
    IT_CHECK_ARG(nt >= 1 && nt <= IT_MAXT && nck >= 0 && nck <= IT_MAXCK && nck < nt + 1 && (logit_rows != 2 || nt <= IT_MAXLOGIT), "engine: bad pass geometry");
    if (e->pos + nt > c.ctx_len) return it_fail(IT_ESTATE, "engine: context full (%d + %d > %d)", e->pos, nt, c.ctx_len);   // src/vk/mod.rs:765
    // a single row whose token and position are already on the device: the whole pass is one persistent kernel
    if (e->step && nt == 1 && nck == 0 && from_dev) return it_step_launch(e, logit_rows ? 4 : 0);
    const int* pos_ptr = from_dev ? e->pos_dev : nullptr; const int pos0 = from_dev ? 0 : e->pos;
    if (!from_dev) {
        for (int t = 0; t < nt; t++) if (toks[t] >= (uint32_t)c.n_vocab) return it_fail(IT_EINVAL, "engine: token id %u outside the vocabulary", toks[t]);
        uint32_t* pin = pin_block(e);
        for (int t = 0; t < nt; t++) pin[t] = toks[t];
        IT_CUDA(cudaMemcpyAsync(e->toks_dev, pin, nt * sizeof(uint32_t), cudaMemcpyHostToDevice, cx->stream));
    }
    IT_TRY(it_sup_embed(cx, e->toks_dev, e->tok_embd, e_, nt, A + L.x));
    // rmsnorm fused into the Hadamard + q8k kernel; the normed f32 row is kept only where a dense f32 op needs it
    auto norm_had = [&](const float* w, float* xn_out) {
        it_had_prologue p; p.mode = 2; p.w = w; p.eps = c.eps; p.n = (unsigned)e_; p.xn_out = xn_out; p.xn_stride = e_;
        return it_sup_hadamard_q8_fused(cx, e_, nt, L.x, e_, e->q8, p);
    };
    const size_t s_gdn = (size_t)cd + inner, s_att = (size_t)qf + 2 * kvd, s_ffn = 2 * (size_t)ff;   // row strides of the stacked outputs
    const bool fused = nt <= 8 && sd == 128 && cd % sd == 0 && hd <= 256;    // decode and verification passes: fewer, fused support launches
    for (int il = 0; il < c.n_layer; il++) {
        const it_layer& l = e->layers[il];
        if (l.recurrent) {
            IT_TRY(norm_had(l.attn_norm, A + L.xn));
            IT_TRY(it_matvec_t2(cx, l.in_proj, nt, e->q8, L.big1, s_gdn, 0));                // [qkv | gate] rows
            const size_t csz = (size_t)(c.conv_k - 1) * cd, ssz = (size_t)nv * sd * sd;
            if (fused) {
                // [dense beta/alpha rows | conv | l2norm of q, k] in one launch
                IT_TRY(it_sup_conv_l2_dense(cx, A + L.big1, s_gdn, l.conv_w, l.conv_st, A + L.conv, cd, cd, c.conv_k, sd, nk, nt, l.ck_conv, csz, nck, c.eps,
                                            l.beta, l.alpha, nv, e_, A + L.xn, e_, A + L.beta, A + L.alpha, nv));
            } else {
                IT_TRY(it_sup_dense_rows(cx, l.beta, l.alpha, nv, e_, A + L.xn, e_, A + L.beta, A + L.alpha, nv, nt));
                IT_TRY(it_sup_conv(cx, A + L.big1, s_gdn, l.conv_w, l.conv_st, A + L.conv, cd, cd, c.conv_k, nt, l.ck_conv, csz, nck));
                IT_TRY(it_sup_norm_head(cx, A + L.conv, sd, cd, A + L.conv, sd, cd, sd, 2 * nk, nullptr, 2, c.eps, nullptr, 0, 0, nt));
            }
            if (sd == 128) {
                // [delta rule | gated norm] in one launch, for any number of rows (the state stays in shared memory across the rows)
                // (the kernel stages up to IT_GDN_MAXROWS rows at a time; the state carries over from one launch to the next)
                for (int t0 = 0; t0 < nt; t0 += IT_GDN_MAXROWS) {
                    const int n0 = std::min(IT_GDN_MAXROWS, nt - t0);
                    IT_TRY(it_sup_gdn_norm(cx, A + L.conv + (size_t)t0 * cd, cd, A + L.beta + (size_t)t0 * nv, A + L.alpha + (size_t)t0 * nv, nv, l.dt, l.a, l.ssm_st,
                                           A + L.o + (size_t)t0 * inner, inner, nv, nk, sd, qk, n0, l.ck_ssm, ssz, t0 ? 0 : nck,
                                           l.ssm_norm, c.eps, A + L.big1 + cd + (size_t)t0 * s_gdn, s_gdn));
                }
            } else {
                IT_TRY(it_sup_gdn(cx, A + L.conv, cd, A + L.beta, A + L.alpha, nv, l.dt, l.a, l.ssm_st, A + L.o, inner, nv, nk, sd, qk, nt, l.ck_ssm, ssz, nck));
                IT_TRY(it_sup_norm_head(cx, A + L.o, sd, inner, A + L.o, sd, inner, sd, nv, l.ssm_norm, 1, c.eps, A + L.big1 + cd, sd, s_gdn, nt));
            }
            if (c.gdn_v_grouped) IT_TRY(had_mv(e, l.ssm_out, nt, L.o, inner, L.x, e_, 1, true, sd, nk, nv / nk));
            else IT_TRY(had_mv(e, l.ssm_out, nt, L.o, inner, L.x, e_, 1, true));
        } else {
            float* q = A + L.big1; float* k = q + qf; float* v = k + kvd;                     // [q+gate | k | v] rows
            IT_TRY(norm_had(l.attn_norm, nullptr));
            IT_TRY(it_matvec_t2(cx, l.in_proj, nt, e->q8, L.big1, s_att, 0));
            if (fused) {
                IT_TRY(it_sup_attn_prep(cx, q, s_att, nh, nkv, hd, l.q_norm, l.k_norm, c.eps, pos0, pos_ptr, c.n_rot, e->theta_scale, c.rope_sections, l.kc, l.vc, nt));
            } else {
                IT_TRY(it_sup_norm_head(cx, q, 2 * hd, s_att, q, 2 * hd, s_att, hd, nh, l.q_norm, 0, c.eps, nullptr, 0, 0, nt));
                IT_TRY(it_sup_norm_head(cx, k, hd, s_att, k, hd, s_att, hd, nkv, l.k_norm, 0, c.eps, nullptr, 0, 0, nt));
                IT_TRY(it_sup_rope(cx, q, 2 * hd, s_att, nh, nt, pos0, pos_ptr, c.n_rot, e->theta_scale, c.rope_sections));
                IT_TRY(it_sup_rope(cx, k, hd, s_att, nkv, nt, pos0, pos_ptr, c.n_rot, e->theta_scale, c.rope_sections));
                IT_TRY(it_sup_kv_store(cx, k, v, s_att, l.kc, l.vc, kvd, hd, pos0, pos_ptr, nt, 1));
            }
            // prompt passes: one CTA per group of query heads and pair of rows that share their K / V reads; else one per (head, row)
            int ar = 1;
            static const bool grouped = []{ const char* v = getenv("IT_ATTN_GROUPED"); return !v || atoi(v) != 0; }();
            if (grouped && nt > 8 && !pos_ptr) { ar = it_sup_attention_prefill(cx, q, 2 * hd, s_att, q + hd, l.kc, l.vc, hd, nh, nkv, pos0, A + L.o, (size_t)nh * hd, nt); if (ar < 0) return ar; }
            if (ar == 1) IT_TRY(it_sup_attention(cx, q, 2 * hd, s_att, q + hd, l.kc, l.vc, kvd, hd, nh, nkv, pos0, pos_ptr, c.ctx_len, A + L.o, (size_t)nh * hd, nt, 1));
            IT_TRY(had_mv(e, l.o, nt, L.o, (size_t)nh * hd, L.x, e_, 1, true));
        }
        IT_TRY(norm_had(l.post_norm, nullptr));
        IT_TRY(it_matvec_t2(cx, l.gate_up, nt, e->q8, L.big1, s_ffn, 0));                    // [gate | up] rows
        { it_had_prologue p; p.mode = 1; p.b = A + L.big1 + ff; p.b_stride = s_ffn;           // silu(gate) * up on the way into the Hadamard
          IT_TRY(it_sup_hadamard_q8_fused(cx, ff, nt, L.big1, s_ffn, e->q8, p)); }
        IT_TRY(it_matvec_t2(cx, l.ffn_down, nt, e->q8, L.x, e_, 1));
    }
    // h_nextn rows: output-normed hidden state of every token of this pass (src/vk/mod.rs:858-861, src/cpu.rs:188-189)
    IT_TRY(it_sup_rmsnorm_wide(cx, A + L.x, e_, e->output_norm, e_, c.eps, A + L.hrow, e_, nt));
    if (logit_rows == 2) IT_TRY(logits_and_argmax(e, L.hrow, nt));
    else if (logit_rows == 1) IT_TRY(logits_and_argmax(e, L.hrow + (size_t)(nt - 1) * e_, 1));
    if (!from_dev) e->pos += nt;
    return IT_OK;
}

namespace {

int trunk_pass(it_engine* e, const uint32_t* toks, int nt, int logit_rows, int nck);

// prefill_chunks (src/vk/mod.rs:130-134) with a chunk of IT_MAXT rows; the greedy pick of the last token lands in amx[0]
int eval_tokens(it_engine* e, const uint32_t* toks, size_t n, bool want_last) {
    IT_CHECK_ARG(e && (toks || n == 0), "engine: null argument");
    if (e->pos + (long long)n > e->cfg.ctx_len) return it_fail(IT_ESTATE, "engine: context full (%d + %zu > %d)", e->pos, n, e->cfg.ctx_len);
    for (size_t s = 0; s < n; s += IT_MAXT) {
        const int nt = (int)std::min<size_t>(IT_MAXT, n - s); const bool last = s + nt == n;
        IT_TRY(trunk_pass(e, toks + s, nt, (want_last && last) ? 1 : 0, 0));
    }
    return IT_OK;
}
int read_pick(it_engine* e, size_t slot, uint32_t* out) { return it_arena_read(e->ctx, e->lay.amx + slot, out, 1); }

// One MTP head pass over nt rows at positions pos0.. paired with the h rows at arena offset hoff (mtp_pass_mode,
// src/vk/mod.rs:912-959; arithmetic of cpu_step, src/mtp.rs:100-137).  predict = false only extends the head's KV cache.
// from_dev: the token ids are already in toks_dev[IT_MAXT..] and the first position is read from pos_dev[1] (recorded pass).
int mtp_pass(it_engine* e, const uint32_t* toks, int nt, int pos0, size_t hoff, bool predict, bool from_dev = false) {
    it_ctx* cx = e->ctx; const it_model_config& c = e->cfg; const it_arena_layout& L = e->lay; float* A = cx->arena;
    const int e_ = c.n_embd, ff = c.n_ff, hd = c.head_dim, nh = c.n_head, nkv = c.n_head_kv, kvd = nkv * hd, qf = 2 * nh * hd;
    IT_CHECK_ARG(nt >= 1 && nt <= IT_MAXT && pos0 >= 1 && pos0 + nt <= c.ctx_len, "engine: bad MTP pass geometry");
    const int* pos_ptr = from_dev ? e->pos_dev + 1 : nullptr;
    if (from_dev) pos0 = 0;                                   // the kernels add the device-resident position
    else {
        uint32_t* pin = pin_block(e) + IT_MAXT;
        for (int t = 0; t < nt; t++) pin[t] = toks[t];
        IT_CUDA(cudaMemcpyAsync(e->toks_dev + IT_MAXT, pin, nt * sizeof(uint32_t), cudaMemcpyHostToDevice, cx->stream));
    }
    IT_TRY(it_sup_embed(cx, e->toks_dev + IT_MAXT, e->m_tok_embd, e_, nt, A + L.me));
    IT_TRY(it_sup_rmsnorm_wide(cx, A + L.me, e_, e->m_enorm, e_, c.eps, A + L.mcat, 2 * e_, nt));
    IT_TRY(it_sup_rmsnorm_wide(cx, A + hoff, e_, e->m_hnorm, e_, c.eps, A + L.mcat + e_, 2 * e_, nt));
    IT_TRY(it_matvec_q8(cx, e->m_eh, nt, L.mcat, 2 * e_, L.mx, e_, 0));
    IT_TRY(it_sup_rmsnorm_wide(cx, A + L.mx, e_, e->m_attn_norm, e_, c.eps, A + L.xn, e_, nt));
    const int slot0 = pos0 - 1;
    if (predict) IT_TRY(it_matvec_q8(cx, e->m_q, nt, L.xn, e_, L.big1, qf, 0));
    IT_TRY(it_matvec_q8(cx, e->m_k, nt, L.xn, e_, L.kcur, kvd, 0));
    IT_TRY(it_matvec_q8(cx, e->m_v, nt, L.xn, e_, L.vcur, kvd, 0));
    if (predict) IT_TRY(it_sup_norm_head(cx, A + L.big1, 2 * hd, qf, A + L.big1, 2 * hd, qf, hd, nh, e->m_q_norm, 0, c.eps, nullptr, 0, 0, nt));
    IT_TRY(it_sup_norm_head(cx, A + L.kcur, hd, kvd, A + L.kcur, hd, kvd, hd, nkv, e->m_k_norm, 0, c.eps, nullptr, 0, 0, nt));
    if (predict) IT_TRY(it_sup_rope(cx, A + L.big1, 2 * hd, qf, nh, nt, pos0, pos_ptr, c.n_rot, e->theta_scale, c.rope_sections));
    IT_TRY(it_sup_rope(cx, A + L.kcur, hd, kvd, nkv, nt, pos0, pos_ptr, c.n_rot, e->theta_scale, c.rope_sections));
    IT_TRY(it_sup_kv_store(cx, A + L.kcur, A + L.vcur, kvd, e->mkc, e->mvc, kvd, hd, slot0, pos_ptr, nt, 0));
    if (!predict) return IT_OK;
    IT_TRY(it_sup_attention(cx, A + L.big1, 2 * hd, qf, A + L.big1 + hd, e->mkc, e->mvc, kvd, hd, nh, nkv, slot0, pos_ptr, c.ctx_len, A + L.o, (size_t)nh * hd, nt, 0));
    IT_TRY(it_matvec_q8(cx, e->m_o, nt, L.o, (size_t)nh * hd, L.mx, e_, 1));
    IT_TRY(it_sup_rmsnorm_wide(cx, A + L.mx, e_, e->m_post_norm, e_, c.eps, A + L.xn, e_, nt));
    IT_TRY(it_matvec_q8(cx, e->m_gate, nt, L.xn, e_, L.big1, ff, 0));
    IT_TRY(it_matvec_q8(cx, e->m_up, nt, L.xn, e_, L.big2, ff, 0));
    IT_TRY(it_sup_silu_mul(cx, A + L.big1, A + L.big2, A + L.big1, (size_t)nt * ff));
    IT_TRY(it_matvec_q8(cx, e->m_down, nt, L.big1, ff, L.mx, e_, 1));
    IT_TRY(it_sup_rmsnorm_wide(cx, A + L.mx + (size_t)(nt - 1) * e_, e_, e->m_head_norm, e_, c.eps, A + L.xn, e_, 1));
    return logits_and_argmax(e, L.xn, 1);
}

// ---- recorded passes ------------------------------------------------------------------------------------------
// A pass of a few rows is several hundred short launches, more host time than device time when they are issued one by
// one.  Each shape (rows, logit rows, checkpoints; for the head: rows, hidden-row offset, predict) is recorded once with
// the token ids and the position read from device memory, and replayed after one small copy of ids and position.
uint32_t* stage_slot(it_engine* e) {
    if (e->small_next == IT_SMALL_SLOTS) { cudaStreamSynchronize(e->ctx->stream); e->small_next = 0; }   // every copy out of the ring has run
    return e->small_pin + 16 * (size_t)(e->small_next++);
}
template <typename F> int replay_pass(it_engine* e, uint64_t key, F&& record) {
    it_ctx* cx = e->ctx;
    auto it = e->pass_graphs.find(key);
    if (it == e->pass_graphs.end()) {
        IT_TRY(it_capture_begin(cx));
        const int r = record();
        it_graph* g = nullptr; const int r2 = it_capture_end(cx, &g);
        if (r || r2) { if (g) it_graph_destroy(g); return r ? r : r2; }
        it = e->pass_graphs.emplace(key, g).first;
    }
    return it_graph_launch(cx, it->second);
}
bool can_record(const it_engine* e, int nt) { return e->record_passes && nt <= IT_SMALL_ROWS && !e->ctx->capturing; }

int trunk_pass(it_engine* e, const uint32_t* toks, int nt, int logit_rows, int nck) {
    if (!can_record(e, nt)) return it_engine_run_chunk(e, toks, nt, logit_rows, nck, false);
    const it_model_config& c = e->cfg; it_ctx* cx = e->ctx;
    if (e->pos + nt > c.ctx_len) return it_fail(IT_ESTATE, "engine: context full (%d + %d > %d)", e->pos, nt, c.ctx_len);
    for (int t = 0; t < nt; t++) if (toks[t] >= (uint32_t)c.n_vocab) return it_fail(IT_EINVAL, "engine: token id %u outside the vocabulary", toks[t]);
    uint32_t* slot = stage_slot(e);
    for (int t = 0; t < nt; t++) slot[t] = toks[t];
    slot[8] = (uint32_t)e->pos;
    IT_CUDA(cudaMemcpyAsync(e->toks_dev, slot, nt * sizeof(uint32_t), cudaMemcpyHostToDevice, cx->stream));
    IT_CUDA(cudaMemcpyAsync(e->pos_dev, slot + 8, sizeof(uint32_t), cudaMemcpyHostToDevice, cx->stream));
    IT_TRY(replay_pass(e, 1ull << 60 | (uint64_t)nt | (uint64_t)logit_rows << 8 | (uint64_t)nck << 16,
                       [&]() { return it_engine_run_chunk(e, nullptr, nt, logit_rows, nck, true); }));
    e->pos += nt;
    return IT_OK;
}
int head_pass(it_engine* e, const uint32_t* toks, int nt, int pos0, size_t hoff, bool predict) {
    if (!can_record(e, nt)) return mtp_pass(e, toks, nt, pos0, hoff, predict);
    const it_model_config& c = e->cfg; it_ctx* cx = e->ctx;
    IT_CHECK_ARG(pos0 >= 1 && pos0 + nt <= c.ctx_len, "engine: bad MTP pass geometry");
    uint32_t* slot = stage_slot(e);
    for (int t = 0; t < nt; t++) slot[t] = toks[t];
    slot[8] = (uint32_t)pos0;
    IT_CUDA(cudaMemcpyAsync(e->toks_dev + IT_MAXT, slot, nt * sizeof(uint32_t), cudaMemcpyHostToDevice, cx->stream));
    IT_CUDA(cudaMemcpyAsync(e->pos_dev + 1, slot + 8, sizeof(uint32_t), cudaMemcpyHostToDevice, cx->stream));
    return replay_pass(e, 2ull << 60 | (uint64_t)nt | (uint64_t)(predict ? 1 : 0) << 8 | (uint64_t)hoff << 16,
                       [&]() { return mtp_pass(e, nullptr, nt, 1, hoff, predict, true); });
}

// Recurrent state of every delta-net layer back to checkpoint `ck` (the state after row ck of the last pass): two
// device-to-device copies per layer, recorded once per checkpoint index and replayed as one graph.
int restore_checkpoint(it_engine* e, int ck) {
    const it_model_config& c = e->cfg; it_ctx* cx = e->ctx; it_note_op(cx);
    const size_t csz = (size_t)(c.conv_k - 1) * it_cfg_conv_dim(c), ssz = (size_t)c.ssm_vheads * c.ssm_state * c.ssm_state;
    auto copies = [&]() {
        for (it_layer& l : e->layers) if (l.recurrent) {
            IT_CUDA(cudaMemcpyAsync(l.conv_st, l.ck_conv + (size_t)ck * csz, csz * 4, cudaMemcpyDeviceToDevice, cx->stream));
            IT_CUDA(cudaMemcpyAsync(l.ssm_st, l.ck_ssm + (size_t)ck * ssz, ssz * 4, cudaMemcpyDeviceToDevice, cx->stream));
        }
        return (int)IT_OK;
    };
    if (!e->record_passes || cx->capturing) return copies();
    return replay_pass(e, 3ull << 60 | (uint64_t)ck, copies);
}

int copy_rows(it_engine* e, size_t src, size_t dst, size_t n) {
    it_note_op(e->ctx);
    IT_CUDA(cudaMemcpyAsync(e->ctx->arena + dst, e->ctx->arena + src, n * 4, cudaMemcpyDeviceToDevice, e->ctx->stream)); return IT_OK;
}

}  // namespace

// ---------------------------------------------------------------- Engine trait
IT_API int it_engine_reset(it_engine* e) {   // zero_state, src/vk/mod.rs:645-651
    IT_CHECK_ARG(e, "it_engine_reset: null engine");
    const it_model_config& c = e->cfg; cudaStream_t st = e->ctx->stream; it_note_op(e->ctx);
    for (it_layer& l : e->layers) if (l.recurrent) {
        IT_CUDA(cudaMemsetAsync(l.conv_st, 0, (size_t)(c.conv_k - 1) * it_cfg_conv_dim(c) * 4, st));
        IT_CUDA(cudaMemsetAsync(l.ssm_st, 0, (size_t)c.ssm_vheads * c.ssm_state * c.ssm_state * 4, st));
    }
    e->pos = 0; e->mpos = 1; e->hp_off = 0; e->hp_n = 0; e->last_rows = 0;
    return IT_OK;
}
IT_API int it_engine_eval(it_engine* e, const uint32_t* toks, size_t n, float* logits) {
    IT_CHECK_ARG(n > 0, "it_engine_eval: no tokens");
    IT_TRY(eval_tokens(e, toks, n, logits != nullptr));
    if (logits) return it_arena_read(e->ctx, e->lay.logits, logits, e->cfg.n_vocab);
    return IT_OK;
}
IT_API int it_engine_eval_argmax(it_engine* e, const uint32_t* toks, size_t n, uint32_t* next) {
    IT_CHECK_ARG(n > 0 && next, "it_engine_eval_argmax: bad argument");
    IT_TRY(eval_tokens(e, toks, n, true));
    return read_pick(e, 0, next);
}

namespace {
// Publishes the host's position to the device and records the single-token greedy step once: pick -> token slot,
// one pass with the position read on the device, pick -> token slot and position + 1.
int begin_device_decode(it_engine* e) {
    it_ctx* cx = e->ctx;
    uint32_t* pin = pin_block(e) + 2 * IT_MAXT;
    *pin = (uint32_t)e->pos;
    IT_CUDA(cudaMemcpyAsync(e->pos_dev, pin, 4, cudaMemcpyHostToDevice, cx->stream));
    if (e->step_graph) return IT_OK;
    IT_TRY(it_capture_begin(cx));
    int r;
    if (e->step) r = it_step_launch(e, 1 | 2 | 4);       // takes the previous pick as its token and hands its own pick over
    else {
        k_set_tokens<<<1, 1, 0, cx->stream>>>(cx->arena + e->lay.amx, e->toks_dev, e->pos_dev, 0);
        r = it_engine_run_chunk(e, nullptr, 1, 1, 0, true);
        k_set_tokens<<<1, 1, 0, cx->stream>>>(cx->arena + e->lay.amx, e->toks_dev, e->pos_dev, 1);
    }
    it_graph* g = nullptr; int r2 = it_capture_end(cx, &g);
    if (r || r2) { if (g) it_graph_destroy(g); return r ? r : r2; }
    e->step_graph = g;
    return IT_OK;
}
}  // namespace

// generate_inner, greedy (src/engine.rs:151-174).  After the prompt, every step replays one recorded graph: the pick of
// the previous step is moved into the token slot on the device and the position is read from device memory, so the host
// only reads 4 bytes per token.
IT_API int it_engine_generate(it_engine* e, const uint32_t* prompt, size_t n_prompt, size_t n_predict, uint32_t eos, uint32_t* out, size_t* n_out) {
    IT_CHECK_ARG(e && prompt && n_prompt > 0 && out && n_out, "it_engine_generate: bad argument");
    *n_out = 0;
    if (n_predict == 0) return IT_OK;
    if (e->pos + (long long)n_prompt + (long long)n_predict - 1 > e->cfg.ctx_len) return it_fail(IT_ESTATE, "it_engine_generate: prompt + prediction exceed the context capacity");
    IT_TRY(eval_tokens(e, prompt, n_prompt, true));
    uint32_t t = 0; IT_TRY(read_pick(e, 0, &t));
    out[(*n_out)++] = t;
    if (t == eos || *n_out == n_predict) return IT_OK;
    IT_TRY(begin_device_decode(e));
    while (*n_out < n_predict) {
        IT_TRY(it_graph_launch(e->ctx, e->step_graph));
        e->pos += 1;
        IT_TRY(read_pick(e, 0, &t));
        out[(*n_out)++] = t;
        if (t == eos) break;
    }
    return IT_OK;
}

// n greedy steps chained on the device with no read-back in between: the pick of each step feeds the next one.  Continues
// from the pick left in place by the previous eval_argmax / generate / decode_steps call.  last_pick may be null.
IT_API int it_engine_decode_steps(it_engine* e, size_t n, uint32_t* last_pick) {
    IT_CHECK_ARG(e, "it_engine_decode_steps: null engine");
    if (e->pos < 1) return it_fail(IT_ESTATE, "it_engine_decode_steps: nothing has been evaluated yet");
    if (e->pos + (long long)n > e->cfg.ctx_len) return it_fail(IT_ESTATE, "it_engine_decode_steps: context full");
    IT_TRY(begin_device_decode(e));
    for (size_t i = 0; i < n; i++) { IT_TRY(it_graph_launch(e->ctx, e->step_graph)); e->pos += 1; }
    if (last_pick) return read_pick(e, 0, last_pick);
    return IT_OK;
}

// Kernel launches of one recorded greedy decode step (records the step when it has not been recorded yet).
IT_API int it_engine_step_kernels(it_engine* e) {
    IT_CHECK_ARG(e, "it_engine_step_kernels: null engine");
    if (e->pos < 1) return it_fail(IT_ESTATE, "it_engine_step_kernels: nothing has been evaluated yet");
    IT_TRY(begin_device_decode(e));
    return it_graph_kernel_nodes(e->step_graph);
}

// ---------------------------------------------------------------- MtpBackend trait (impl for VkEngine, src/vk/mod.rs:979-1027)
#define IT_NEED_MTP(e, who) do { IT_CHECK_ARG(e, who ": null engine"); if (!(e)->has_mtp) return it_fail(IT_ESTATE, who ": the engine has no MTP head"); } while (0)

IT_API int it_engine_mtp_reset_all(it_engine* e) { IT_NEED_MTP(e, "it_engine_mtp_reset_all"); return it_engine_reset(e); }

IT_API int it_engine_mtp_prefill(it_engine* e, const uint32_t* prompt, size_t n, uint32_t* next) {
    IT_NEED_MTP(e, "it_engine_mtp_prefill");
    IT_CHECK_ARG(prompt && n > 0 && next, "it_engine_mtp_prefill: bad argument");
    IT_TRY(it_engine_reset(e));
    if ((long long)n > e->cfg.ctx_len) return it_fail(IT_ESTATE, "it_engine_mtp_prefill: prompt longer than the context capacity");
    const it_arena_layout& L = e->lay; const size_t e_ = e->cfg.n_embd;
    for (size_t s = 0; s < n; s += IT_MAXT) {
        const int nt = (int)std::min<size_t>(IT_MAXT, n - s); const bool last = s + nt == n;
        IT_TRY(trunk_pass(e, prompt + s, nt, last ? 1 : 0, 0));
        // MTP catch-up over the pairs (h_{q-1}, x_q), q in [s, s+nt), q >= 1 (src/vk/mod.rs:989-1003)
        if (s > 0) IT_TRY(copy_rows(e, L.hprev, L.mh, e_));
        if (nt > 1) IT_TRY(copy_rows(e, L.hrow, L.mh + e_, (size_t)(nt - 1) * e_));
        IT_TRY(copy_rows(e, L.hrow + (size_t)(nt - 1) * e_, L.hprev, e_));
        if (s == 0) { if (nt > 1) IT_TRY(head_pass(e, prompt + 1, nt - 1, 1, L.mh + e_, false)); }
        else IT_TRY(head_pass(e, prompt + s, nt, (int)s, L.mh, false));
    }
    e->mpos = (int)n; e->hp_off = L.hprev; e->hp_n = 1;
    return read_pick(e, 0, next);
}
IT_API int it_engine_mtp_single(it_engine* e, uint32_t x, uint32_t* next) { IT_NEED_MTP(e, "it_engine_mtp_single"); return it_engine_eval_argmax(e, &x, 1, next); }
IT_API int it_engine_mtp_draft(it_engine* e, const uint32_t* toks, size_t n, uint32_t* draft) {
    IT_NEED_MTP(e, "it_engine_mtp_draft");
    IT_CHECK_ARG(toks && draft && (int)n == e->hp_n && n >= 1, "it_engine_mtp_draft: token count must equal the pending hidden rows");   // src/vk/mod.rs:1008
    IT_TRY(head_pass(e, toks, (int)n, e->mpos, e->hp_off, true));
    e->mpos += (int)n;
    return read_pick(e, 0, draft);
}
IT_API int it_engine_mtp_verify(it_engine* e, uint32_t x, uint32_t d, uint32_t* a0, uint32_t* a1) {
    IT_NEED_MTP(e, "it_engine_mtp_verify");
    IT_CHECK_ARG(a0 && a1, "it_engine_mtp_verify: null output");
    const uint32_t toks[2] = { x, d };
    IT_TRY(trunk_pass(e, toks, 2, 2, 1));                       // both rows' picks, state checkpointed after x
    e->hp_off = e->lay.hrow; e->hp_n = 2;
    uint32_t picks[2]; IT_TRY(it_arena_read(e->ctx, e->lay.amx, picks, 2));
    *a0 = picks[0]; *a1 = picks[1]; return IT_OK;
}
IT_API int it_engine_mtp_reject(it_engine* e) {   // src/vk/mod.rs:1018-1025
    IT_NEED_MTP(e, "it_engine_mtp_reject");
    if (e->pos < 1) return it_fail(IT_ESTATE, "it_engine_mtp_reject: nothing to roll back");
    IT_TRY(restore_checkpoint(e, 0));
    e->pos -= 1; e->hp_off = e->lay.hrow; e->hp_n = 1;
    return IT_OK;
}

// ---------------------------------------------------------------- draft length k (extension, see the header)
IT_API int it_engine_mtp_draft_k(it_engine* e, const uint32_t* toks, size_t n, size_t k, uint32_t* drafts) {
    IT_NEED_MTP(e, "it_engine_mtp_draft_k");
    IT_CHECK_ARG(toks && drafts && (int)n == e->hp_n && n >= 1 && k >= 1 && k <= IT_MAXCK, "it_engine_mtp_draft_k: bad token count or draft length");
    if (e->mpos + (int)n + (int)k - 1 > e->cfg.ctx_len) return it_fail(IT_ESTATE, "it_engine_mtp_draft_k: context full");
    const size_t e_ = e->cfg.n_embd;
    IT_TRY(head_pass(e, toks, (int)n, e->mpos, e->hp_off, true));
    e->mpos += (int)n;
    IT_TRY(read_pick(e, 0, &drafts[0]));
    size_t hid = e->lay.mx + (n - 1) * e_;                  // the head's hidden state before head_norm, last row of the pass
    for (size_t i = 1; i < k; i++) {                        // chained steps: provisional KV entries at positions mpos, mpos + 1, ..
        IT_TRY(head_pass(e, &drafts[i - 1], 1, e->mpos + (int)i - 1, hid, true));
        IT_TRY(read_pick(e, 0, &drafts[i]));
        hid = e->lay.mx;
    }
    return IT_OK;
}
IT_API int it_engine_mtp_verify_k(it_engine* e, uint32_t x, const uint32_t* drafts, size_t k, uint32_t* picks) {
    IT_NEED_MTP(e, "it_engine_mtp_verify_k");
    IT_CHECK_ARG(drafts && picks && k >= 1 && k <= IT_MAXCK, "it_engine_mtp_verify_k: bad argument");
    uint32_t toks[IT_MAXCK + 1]; toks[0] = x;
    for (size_t i = 0; i < k; i++) toks[i + 1] = drafts[i];
    IT_TRY(trunk_pass(e, toks, (int)k + 1, 2, (int)k));                      // a pick per row, state checkpointed after rows 0 .. k - 1
    e->hp_off = e->lay.hrow; e->hp_n = (int)k + 1; e->last_rows = (int)k + 1;
    return it_arena_read(e->ctx, e->lay.amx, picks, k + 1);
}
IT_API int it_engine_mtp_rollback(it_engine* e, size_t keep_rows) {
    IT_NEED_MTP(e, "it_engine_mtp_rollback");
    IT_CHECK_ARG(e->last_rows >= 2 && keep_rows >= 1 && (int)keep_rows <= e->last_rows, "it_engine_mtp_rollback: no verification pass to roll back, or bad row count");
    const int drop = e->last_rows - (int)keep_rows;
    if (drop > 0) {
        IT_TRY(restore_checkpoint(e, (int)keep_rows - 1));      // checkpoint t holds the state after row t
        e->pos -= drop;
    }
    e->hp_off = e->lay.hrow; e->hp_n = (int)keep_rows; e->last_rows = 0;
    return IT_OK;
}

IT_API int64_t it_greedy_mtp_k(const it_mtp_backend_k* b, size_t k, const uint32_t* prompt, size_t np, size_t n,
                               int (*is_eog)(void*, uint32_t), int (*on_tok)(void*, uint32_t), void* cbu, uint32_t* out, int64_t* stats) {
    if (!b || !out || !stats || !is_eog || !on_tok || k < 1 || k > IT_MAXCK) return it_fail(IT_EINVAL, "it_greedy_mtp_k: bad argument");
    enum { DRAFTED, ACCEPTED, STEPS, DRAFT_CALLS, VERIFY_CALLS, SINGLE, TIMED, REJECTED, TERMINAL };
    for (int i = 0; i < 9; i++) stats[i] = 0;
    size_t no = 0;
    auto emit = [&](uint32_t t) { out[no++] = t; const bool go = on_tok(cbu, t) != 0; return go && !is_eog(cbu, t) && no < n; };
    if (n == 0) return 0;
    if (np == 0 || !prompt) return it_fail(IT_EINVAL, "it_greedy_mtp_k: empty MTP prompt");
    uint32_t x = b->prefill(b->user, prompt, np);
    if (!emit(x)) return (int64_t)no;
    uint32_t pending[IT_MAXCK + 1] = { x }; size_t npend = 1;
    for (;;) {
        if (n - no == 1) { const uint32_t a = b->single(b->user, x); stats[SINGLE]++; stats[TIMED]++; emit(a); break; }
        const size_t kk = k < n - no - 1 ? k : n - no - 1;
        uint32_t ds[IT_MAXCK] = {}, picks[IT_MAXCK + 1] = {};
        b->draft_k(b->user, pending, npend, kk, ds); stats[DRAFT_CALLS]++;
        b->verify_k(b->user, x, ds, kk, picks);
        stats[DRAFTED] += (int64_t)kk; stats[STEPS]++; stats[VERIFY_CALLS]++; stats[TIMED] += (int64_t)kk + 1;
        size_t nacc = 0;
        while (nacc < kk && picks[nacc] == ds[nacc]) nacc++;
        stats[ACCEPTED] += (int64_t)nacc; stats[REJECTED] += (int64_t)(kk - nacc);
        bool stop = false;
        for (size_t i = 0; i < nacc; i++)
            if (!emit(ds[i])) { b->rollback(b->user, i + 1); stats[TERMINAL]++; stop = true; break; }
        if (stop) break;
        b->rollback(b->user, nacc + 1);
        if (!emit(picks[nacc])) break;
        x = picks[nacc];
        for (size_t i = 0; i < nacc; i++) pending[i] = ds[i];
        pending[nacc] = picks[nacc]; npend = nacc + 1;
    }
    return (int64_t)no;
}

// ---------------------------------------------------------------- greedy_mtp (src/mtp.rs:166-204)
IT_API int64_t it_greedy_mtp(const it_mtp_backend* b, const uint32_t* prompt, size_t np, size_t n,
                             int (*is_eog)(void*, uint32_t), int (*on_tok)(void*, uint32_t), void* cbu, uint32_t* out, int64_t* stats) {
    if (!b || !out || !stats || !is_eog || !on_tok) return it_fail(IT_EINVAL, "it_greedy_mtp: null argument");
    enum { DRAFTED, ACCEPTED, STEPS, DRAFT_CALLS, VERIFY_CALLS, SINGLE, TIMED, REJECTED, TERMINAL };
    for (int i = 0; i < 9; i++) stats[i] = 0;
    size_t no = 0;
    auto emit = [&](uint32_t t) { out[no++] = t; const bool go = on_tok(cbu, t) != 0; return go && !is_eog(cbu, t) && no < n; };
    if (n == 0) return 0;
    if (np == 0 || !prompt) return it_fail(IT_EINVAL, "it_greedy_mtp: empty MTP prompt");
    uint32_t x = b->prefill(b->user, prompt, np);
    if (!emit(x)) return (int64_t)no;
    uint32_t pending[2] = { x, 0 }; size_t npend = 1;
    for (;;) {
        if (n - no == 1) { const uint32_t a = b->single(b->user, x); stats[SINGLE]++; stats[TIMED]++; emit(a); break; }
        const uint32_t d = b->draft(b->user, pending, npend); stats[DRAFT_CALLS]++;
        uint32_t a0 = 0, a1 = 0; b->verify(b->user, x, d, &a0, &a1);
        stats[DRAFTED]++; stats[STEPS]++; stats[VERIFY_CALLS]++; stats[TIMED] += 2;
        if (a0 == d) {
            stats[ACCEPTED]++;
            if (!emit(d)) { b->reject(b->user); stats[TERMINAL]++; break; }
            if (!emit(a1)) break;
            x = a1; pending[0] = a0; pending[1] = a1; npend = 2;
        } else {
            b->reject(b->user); stats[REJECTED]++;
            if (!emit(a0)) break;
            x = a0; pending[0] = a0; npend = 1;
        }
    }
    return (int64_t)no;
}

namespace {
struct EngineCb { it_engine* e; uint32_t eos; int err; };
uint32_t cb_prefill(void* u, const uint32_t* p, size_t n) { EngineCb* c = (EngineCb*)u; uint32_t t = 0; if (!c->err) c->err = it_engine_mtp_prefill(c->e, p, n, &t); return t; }
uint32_t cb_single(void* u, uint32_t x) { EngineCb* c = (EngineCb*)u; uint32_t t = 0; if (!c->err) c->err = it_engine_mtp_single(c->e, x, &t); return t; }
uint32_t cb_draft(void* u, const uint32_t* p, size_t n) { EngineCb* c = (EngineCb*)u; uint32_t t = 0; if (!c->err) c->err = it_engine_mtp_draft(c->e, p, n, &t); return t; }
void cb_verify(void* u, uint32_t x, uint32_t d, uint32_t* a0, uint32_t* a1) { EngineCb* c = (EngineCb*)u; *a0 = *a1 = 0; if (!c->err) c->err = it_engine_mtp_verify(c->e, x, d, a0, a1); }
void cb_reject(void* u) { EngineCb* c = (EngineCb*)u; if (!c->err) c->err = it_engine_mtp_reject(c->e); }
void cb_reset(void* u) { EngineCb* c = (EngineCb*)u; if (!c->err) c->err = it_engine_mtp_reset_all(c->e); }
int cb_eog(void* u, uint32_t t) { EngineCb* c = (EngineCb*)u; return c->err != 0 || t == c->eos; }
int cb_tok(void*, uint32_t) { return 1; }
}  // namespace

namespace {
void cb_draft_k(void* u, const uint32_t* p, size_t n, size_t k, uint32_t* d) { EngineCb* c = (EngineCb*)u; for (size_t i = 0; i < k; i++) d[i] = 0; if (!c->err) c->err = it_engine_mtp_draft_k(c->e, p, n, k, d); }
void cb_verify_k(void* u, uint32_t x, const uint32_t* d, size_t k, uint32_t* a) { EngineCb* c = (EngineCb*)u; for (size_t i = 0; i <= k; i++) a[i] = 0; if (!c->err) c->err = it_engine_mtp_verify_k(c->e, x, d, k, a); }
void cb_rollback(void* u, size_t keep) { EngineCb* c = (EngineCb*)u; if (!c->err) c->err = it_engine_mtp_rollback(c->e, keep); }
}  // namespace

IT_API int64_t it_engine_generate_mtp_k(it_engine* e, size_t k, const uint32_t* prompt, size_t n_prompt, size_t n_predict, uint32_t eos, uint32_t* out, int64_t* stats) {
    if (!e || !e->has_mtp) return it_fail(IT_ESTATE, "it_engine_generate_mtp_k: the engine has no MTP head");
    if ((long long)n_prompt + (long long)n_predict + (long long)k > e->cfg.ctx_len) return it_fail(IT_ESTATE, "it_engine_generate_mtp_k: prompt + prediction exceed the context capacity");
    EngineCb cb{ e, eos, 0 };
    it_mtp_backend_k b{ &cb, cb_prefill, cb_single, cb_draft_k, cb_verify_k, cb_rollback, cb_reset };
    const int64_t n = it_greedy_mtp_k(&b, k, prompt, n_prompt, n_predict, cb_eog, cb_tok, &cb, out, stats);
    return cb.err ? cb.err : n;
}

IT_API int64_t it_engine_generate_mtp(it_engine* e, const uint32_t* prompt, size_t n_prompt, size_t n_predict, uint32_t eos, uint32_t* out, int64_t* stats) {
    if (!e || !e->has_mtp) return it_fail(IT_ESTATE, "it_engine_generate_mtp: the engine has no MTP head");
    if ((long long)n_prompt + (long long)n_predict > e->cfg.ctx_len) return it_fail(IT_ESTATE, "it_engine_generate_mtp: prompt + prediction exceed the context capacity");
    EngineCb cb{ e, eos, 0 };
    it_mtp_backend b{ &cb, cb_prefill, cb_single, cb_draft, cb_verify, cb_reject, cb_reset };
    const int64_t n = it_greedy_mtp(&b, prompt, n_prompt, n_predict, cb_eog, cb_tok, &cb, out, stats);
    return cb.err ? cb.err : n;
}
