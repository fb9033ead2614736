// The decoder engine: weights, state and arena layout shared by it_engine.cu (construction, read-back) and
// it_engine_run.cu (forward passes, MTP hooks, generation loops).
#pragma once
#include "it_internal.h"
#include <map>
#include <vector>

#define IT_MAXT 256   // activation rows per pass: the prompt chunk of prefill_chunks (src/vk/mod.rs:130-134 uses 64; the chunk size changes no result,
                      // and with 256 rows the tile kernels pay their per-block cost once per 128 rows and the row-parallel kernels fill the GPU)
#define IT_MAXLOGIT 8 // rows of a pass that can get logits and a greedy pick (verification passes)
#define IT_MAXCK 3    // recurrent-state checkpoints per pass (rows 0..2 of a verification pass)

struct it_layer {
    bool recurrent;
    float *attn_norm, *post_norm;
    it_mat *ffn_gate, *ffn_up, *ffn_down;
    // Matrices that multiply the same input are stacked row-wise in one allocation and run as one matvec; the
    // individual tensors above and below are views into it.  in_proj = [qkv; gate] or [q; k; v], gate_up = [ffn_gate; ffn_up].
    it_mat *in_proj, *gate_up;
    // Gated DeltaNet layers
    it_mat *qkv, *gate, *ssm_out;
    float *conv_w, *dt, *a, *beta, *alpha, *ssm_norm;
    float *conv_st, *ssm_st, *ck_conv, *ck_ssm;     // state and its checkpoints [IT_MAXCK][...]
    // attention layers
    it_mat *q, *k, *v, *o;
    float *q_norm, *k_norm;
    __half *kc, *vc;                                 // [ctx_len][n_head_kv * head_dim]
};

struct it_arena_layout {   // element offsets into the context's f32 arena; every row buffer holds IT_MAXT rows
    size_t x, xn, big1, big2, conv, kcur, vcur, o, beta, alpha, hrow, hprev, mh, me, mcat, mx, logits, amx, total;
    size_t big1_stride, big2_stride, o_stride, logits_stride;
};

struct it_step_state;   // geometry and device tables of the persistent decode-step kernel (it_step.cu)

struct it_engine {
    it_ctx* ctx;
    it_step_state* step;                             // null when the step runs op by op (row shards, unsupported geometry, IT_STEP_KERNEL=0)
    it_model_config cfg;
    uint64_t seed;
    bool has_mtp;
    int rank, world;                                 // row shard of the trunk matrices held by this engine (0 of 1: everything)
    std::vector<it_layer> layers;
    float *tok_embd, *output_norm;
    float* m_tok_embd;                               // embedding table of the NextN head: its own (src/mtp.rs:101) or tok_embd
    it_mat* output;
    // MTP head (src/mtp.rs:22-27)
    it_qmat *m_eh, *m_q, *m_k, *m_v, *m_o, *m_gate, *m_up, *m_down;
    float *m_enorm, *m_hnorm, *m_attn_norm, *m_post_norm, *m_q_norm, *m_k_norm, *m_head_norm;
    float *mkc, *mvc;                                // f32 [ctx_len][kvd], slot = position - 1 (src/mtp.rs:95)
    it_q8* q8;
    uint32_t* toks_dev;                              // [0, IT_MAXT) token ids of the trunk pass, [IT_MAXT, 2*IT_MAXT) of the head pass
    int* pos_dev;                                    // position read by the recorded decode step
    it_arena_layout lay;
    float theta_scale;
    std::vector<void*> owned;                        // plain device allocations to free
    int pos, mpos;                                   // trunk position; next MTP position (src/vk/mod.rs: pos, mpos)
    size_t hp_off; int hp_n;                         // pending h rows for the next draft (arena offset, count)
    int last_rows;                                   // rows of the last verification pass (it_engine_mtp_rollback)
    it_graph* step_graph;                            // recorded single-token greedy step
    uint32_t* host_pin;                              // pinned staging, laid out like toks_dev, plus the position at [2*IT_MAXT]
    int pin_next;                                    // host_pin is a ring of IT_PIN_SLOTS such blocks: a block is not rewritten before the copies out of it have run
    // Recorded passes of up to IT_SMALL_ROWS rows (single tokens, verification rows, draft steps of the head), one graph
    // per shape; their token ids and positions are staged through a ring of pinned slots so that a slot is never
    // rewritten while an earlier copy out of it may still be pending.
    std::map<uint64_t, it_graph*> pass_graphs;
    uint32_t* small_pin;                             // IT_SMALL_SLOTS slots of 16 words: [0, 8) token ids, [8] position
    int small_next;
    bool record_passes;                              // environment IT_PASS_GRAPHS (default on)
};
#define IT_PIN_SLOTS 8
#define IT_PIN_WORDS (2 * IT_MAXT + 8)
#define IT_SMALL_ROWS 8
#define IT_SMALL_SLOTS 64

// Where an engine under construction gets its weights.  The engine owns allocation, row sharding and the device
// layouts; a source only fills what it is handed.  Every method returns an IT_* code.
struct it_weight_source {
    virtual ~it_weight_source() {}
    // the +-1 vector of the Hadamard transform for activations of `width` elements (all +1 when the model has none)
    virtual int signs(it_engine* e, size_t width, std::vector<float>* s) = 0;
    // n floats of an f32 tensor into device memory
    virtual int f32(it_engine* e, int layer, int tensor, size_t n, float* dev) = 0;
    // rows [row0, row0 + nrows) of a rows x cols ternary tensor as 34-byte PQ2_0 blocks into device memory
    virtual int ternary(it_engine* e, int layer, int tensor, size_t rows, size_t cols, size_t row0, size_t nrows, uint8_t* raw_dev) = 0;
    // an int8-group matrix of the NextN head
    virtual int q8(it_engine* e, int tensor, size_t rows, size_t cols, it_qmat** out) = 0;
    // the NextN head's own embedding table ([n_vocab][n_embd] floats on the device, owned by the engine); leaves
    // *dev alone when the head shares the trunk's table
    virtual int mtp_embd(it_engine*, float**) { return IT_OK; }
};
int it_engine_build(int device, const it_model_config* cfg, uint64_t seed, int with_mtp, int rank, int world, it_weight_source* src, it_engine** out);
int it_engine_validate_config(const it_model_config* cfg);
int it_engine_dev_alloc(it_engine* e, void** p, size_t bytes, bool zero);   // freed with the engine

// derived sizes (src/model.rs:40-43)
static inline int it_cfg_qk(const it_model_config& c) { return c.ssm_state * c.ssm_groups; }
static inline int it_cfg_conv_dim(const it_model_config& c) { return 2 * it_cfg_qk(c) + c.ssm_inner; }
static inline bool it_cfg_recurrent(const it_model_config& c, int il) { return (il + 1) % c.full_attn_interval != 0; }

#define IT_TRY(expr) do { int r__ = (expr); if (r__) return r__; } while (0)

// Runs one pass over nt <= IT_MAXT tokens (run_chunk_v, src/vk/mod.rs:763-892).  logit_rows: 0 none, 1 last row, 2 every
// row; nck: recurrent-state checkpoints to take (after rows 0..nck-1); from_dev: token ids are already in toks_dev and the
// position is read from pos_dev (recorded decode step).
int it_engine_run_chunk(it_engine* e, const uint32_t* toks, int nt, int logit_rows, int nck, bool from_dev);

// The whole single-row pass as one persistent kernel (it_step.cu).  it_step_prepare decides whether the engine can use it
// (e->step stays null otherwise); it_step_launch enqueues one step: flags 1 = the token is the previous pick (amx) instead
// of toks_dev[0], 2 = hand the pick over to the next step (toks_dev[0] = pick, position + 1), 4 = logits and pick wanted.
int it_step_prepare(it_engine* e);
void it_step_release(it_engine* e);
int it_step_launch(it_engine* e, int flags);
