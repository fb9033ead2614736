/* irontimber_cuda.h - C ABI of the B200 (sm_100a) backend for IronTimber's ternary hot path.
 *
 * The reference has no FFI today: its GPU work goes through the private dispatchers of
 * `VkEngine` (src/vk/mod.rs).  Each entry point below names the reference interface it
 * stands in for (file:line inside the reference project), so that a `--backend cuda` arm
 * can bind it one to one.
 *
 * Conventions
 *  - every function returns 0 on success or a negative IT_E* code; `it_last_error()` gives
 *    the message of the last failure on the calling thread.  Arguments are validated before
 *    anything is launched (the reference validates before touching the device,
 *    src/vk/mod.rs:494-503); nothing aborts.
 *  - one context = one device = one host thread = one compute stream (the reference is
 *    strictly single threaded, src/server.rs:4).  Op launches are stream ordered and do not
 *    block; `it_sync` or any read-back waits.
 *  - activations live in one f32 arena addressed by element offsets, exactly like the
 *    reference's arena (shaders/common.glsl:5, push constants [M,K,ntok,xo,xs,yo,ys,accum]).
 *  - handles are opaque; the caller releases them with the matching destroy call, children
 *    (matrices, q8 buffers) before the context.
 */
#ifndef IRONTIMBER_CUDA_H
#define IRONTIMBER_CUDA_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define IT_OK 0
#define IT_EINVAL (-1)   /* bad argument (shape, alignment, null, out of range) */
#define IT_ECUDA (-2)    /* a CUDA runtime call failed */
#define IT_ENOMEM (-3)   /* device allocation failed */
#define IT_ESTATE (-4)   /* call not valid in the current state */
#define IT_ETIMEOUT (-5) /* a bounded device-side wait ran out */
#define IT_EFORMAT (-6)  /* a model file cannot be read or is not well formed */
#define IT_EUNSUPPORTED (-7) /* a well-formed model that this library does not run (tensor type, layout) */

typedef struct it_ctx it_ctx;
typedef struct it_mat it_mat;   /* ternary (2-bit code) matrix, device resident      */
typedef struct it_qmat it_qmat; /* int8-group matrix (ggml Q8_0 source)             */
typedef struct it_q8 it_q8;     /* q8k-quantised activation rows, device resident    */
typedef struct it_graph it_graph; /* a recorded sequence of op launches                */

const char* it_last_error(void);
int it_version(void);

/* ---- context and arena ---------------------------------------------------------------
 * Replaces Ctx::new_with + the arena allocation of VkEngine (src/vk/mod.rs:267, :567-576). */
int it_ctx_create(int device, size_t arena_floats, it_ctx** out);
void it_ctx_destroy(it_ctx* ctx);
int it_sync(it_ctx* ctx);                                   /* Ctx::submit_wait, src/vk/mod.rs:380 */
void* it_ctx_stream(it_ctx* ctx);                           /* the cudaStream_t every op is launched on */
float* it_arena_ptr(it_ctx* ctx);                           /* device pointer of arena element 0 */
size_t it_arena_floats(it_ctx* ctx);
int it_arena_write(it_ctx* ctx, size_t off, const void* host, size_t n_floats); /* Ctx::upload,   src/vk/mod.rs:427 */
int it_arena_read(it_ctx* ctx, size_t off, void* host, size_t n_floats);        /* Ctx::download */
/* Peers: one process per GPU, up to 8.  it_ctx_ipc_handle writes the 64-byte CUDA IPC handle of this context's arena;
 * the host exchanges the handles (any transport) and gives every context all of them, ordered by rank (its own entry
 * is ignored).  Every rank must create its arena with the same size and issue the same sequence of sharded ops; a
 * sharded op completes on a rank only when every rank's slice has arrived in its arena (bounded wait, IT_ETIMEOUT).
 * No counterpart in the reference (single GPU). */
int it_ctx_ipc_handle(it_ctx* ctx, void* handle64);
int it_ctx_attach_peers(it_ctx* ctx, int rank, int world, const void* handles);
int it_ctx_world(const it_ctx* ctx);
/* The same attachment for contexts that live in one process (a single-process host driving several GPUs, as the reference's
 * single-threaded server would, or two contexts on one GPU): all[p] is rank p's context (the own entry is ignored). */
int it_ctx_attach_peers_local(it_ctx* ctx, int rank, int world, it_ctx* const* all);
/* How long a kernel of this context waits for a peer's results before it gives up and the next it_sync / read-back
 * returns IT_ETIMEOUT (default about four seconds).  Peers must be attached. */
int it_ctx_set_peer_wait_us(it_ctx* ctx, double microseconds);
int it_arena_zero(it_ctx* ctx, size_t off, size_t n_floats);                    /* zero_state,    src/vk/mod.rs:645 */

/* Record the ops issued between begin and end into a CUDA graph and replay them with one launch.
 * Stands where the reference records one command buffer per chunk and submits it once
 * (Ctx::begin / submit_wait, src/vk/mod.rs:363-394).  Calls that wait (it_sync, arena read/write,
 * uploads) are not allowed while recording. */
int it_capture_begin(it_ctx* ctx);
int it_capture_end(it_ctx* ctx, it_graph** out);
int it_graph_launch(it_ctx* ctx, it_graph* g);
void it_graph_destroy(it_graph* g);
int it_graph_kernel_nodes(const it_graph* g);              /* kernel launches one replay makes (>= 0), or a negative code */

/* Hadamard sign vector for activations of width n (prism.hadamard.sign_values; src/model.rs:48-60,
 * uploaded into the params buffer by the reference, src/vk/mod.rs:536).  Values must be +1 or -1. */
int it_signs_set(it_ctx* ctx, size_t n, const float* signs);

/* ---- weights -----------------------------------------------------------------------------
 * Replaces the `mat` upload closure and DevMat (src/vk/mod.rs:459, :579-599).  Accepts either raw
 * PQ2_0 rows (34-byte blocks, src/quant.rs:5-6,21-29) or the reference's Packed2 pair
 * (src/quant.rs:92-119).  cols must be a multiple of 128; any row count is accepted. */
int it_matrix_upload_pq2(it_ctx* ctx, const uint8_t* raw, size_t rows, size_t cols, it_mat** out);
int it_matrix_upload_packed2(it_ctx* ctx, const uint32_t* words, const float* scales, size_t rows, size_t cols, it_mat** out);
/* Synthetic matrix generated on the device: codes uniform over {0,1,2} (or {0,1,2,3} when
 * four_codes != 0), f16 scales uniform in [0.01, 0.05], from a counter hash of (seed, index). */
int it_matrix_synth(it_ctx* ctx, uint64_t seed, size_t rows, size_t cols, int four_codes, it_mat** out);
/* Row shards (no counterpart in the reference, which runs on one GPU; every output row of its matvec is an independent
 * dot with the shared activation row, src/cpu.rs:31-34, which is what makes the split exact).  it_shard_range gives the
 * rows of rank `rank` of `world` (rows must divide evenly; pure host arithmetic).  it_matrix_set_shard marks an uploaded
 * matrix as rows [row0, row0 + rows) of a logical matrix of total_rows rows; it_matrix_synth_rows generates exactly those
 * rows of the matrix that it_matrix_synth would generate for (seed, total_rows, cols).  it_matvec_t2 on a shard writes
 * its results at their positions in the full output row and pushes them into the arena of every attached peer. */
int it_shard_range(size_t rows, int rank, int world, size_t* row0, size_t* nrows);
int it_matrix_set_shard(it_mat* m, size_t row0, size_t total_rows);
int it_matrix_synth_rows(it_ctx* ctx, uint64_t seed, size_t total_rows, size_t cols, int four_codes, size_t row0, size_t nrows, it_mat** out);
/* The same for int8-group matrices (it_matvec_q8 on a shard pushes its rows to every peer). */
int it_qmatrix_set_shard(it_qmat* m, size_t row0, size_t total_rows);
int it_qmatrix_synth_rows(it_ctx* ctx, uint64_t seed, size_t total_rows, size_t cols, size_t row0, size_t nrows, it_qmat** out);
/* Decodes the device layout back to raw PQ2_0 rows (rows*cols/128*34 bytes). */
int it_matrix_download_pq2(it_ctx* ctx, const it_mat* m, uint8_t* raw);
size_t it_matrix_rows(const it_mat* m);
size_t it_matrix_cols(const it_mat* m);
size_t it_matrix_device_bytes(const it_mat* m);
void it_matrix_destroy(it_mat* m);

/* Int8-group matrices of the MTP head: ggml Q8_0 rows (34-byte blocks of 32; src/quant.rs:188-191),
 * what Q8G16::from_ggml consumes (src/quant.rs:235-244).  cols % 32 == 0. */
int it_qmatrix_upload_q8_0(it_ctx* ctx, const uint8_t* raw, size_t rows, size_t cols, it_qmat** out);
int it_qmatrix_synth(it_ctx* ctx, uint64_t seed, size_t rows, size_t cols, it_qmat** out);
int it_qmatrix_download_q8_0(it_ctx* ctx, const it_qmat* m, uint8_t* raw);
/* Q6_K rows (210-byte blocks of 256, cols a multiple of 256) as int8 values q - 32 with one f32 scale per 16 weights,
 * scale = d * sub-block scale (exact in f32): Q8G16::from_ggml's Q6_K arm (src/quant.rs:245-257).  it_matvec_q8 runs both
 * kinds with the same per-16 grouping (Q8G16::dot, src/quant.rs:266-270).  it_qmatrix_download_g16 reads any int8-group
 * matrix back as rows*cols int8 values followed by rows*cols/16 f32 scales; it_qmatrix_group16 tells the kinds apart. */
int it_qmatrix_upload_q6_k(it_ctx* ctx, const uint8_t* raw, size_t rows, size_t cols, it_qmat** out);
int it_qmatrix_download_g16(it_ctx* ctx, const it_qmat* m, uint8_t* raw);
int it_qmatrix_group16(const it_qmat* m);
size_t it_qmatrix_rows(const it_qmat* m);
size_t it_qmatrix_cols(const it_qmat* m);
void it_qmatrix_destroy(it_qmat* m);

/* ---- q8k activation rows ------------------------------------------------------------------
 * Device form of Q8K (src/quant.rs:68-71): per row int8 qs[n], f32 d[n/256], i32 sum128[n/128]. */
int it_q8_create(it_ctx* ctx, size_t max_n, size_t max_tok, it_q8** out);
void it_q8_destroy(it_q8* q);
int it_q8_read(it_ctx* ctx, const it_q8* q, size_t tok, int8_t* qs, float* d, int32_t* sum128);

/* ---- ops -------------------------------------------------------------------------------------
 * Fused forward Hadamard (per 1024-block: optional GDN head permutation, sign multiply, 10 butterfly
 * stages, 1/32) + quantize_row_q8_K: replaces VkEngine::had (src/vk/mod.rs:749-753, shaders/hadamard.comp)
 * followed by quantize_q8k (src/quant.rs:75-90), i.e. Model::prep + the first line of cpu::matvec
 * (src/cpu.rs:115-117, :30).  Reads ntok rows of n floats at x_off + t*x_stride, writes rows 0..ntok-1
 * of `out`.  use_signs != 0 multiplies by the sign vector registered for width n.  perm_hd == 0 means
 * no permutation, otherwise source index = i0 + hd*(k + nk*r) as in shaders/hadamard.comp:13.
 * rotate == 0 skips the transform and only quantises (weights that were not folded, src/cpu.rs:116). */
int it_hadamard_q8(it_ctx* ctx, size_t n, size_t ntok, size_t x_off, size_t x_stride, int rotate, int use_signs,
                   size_t perm_hd, size_t perm_nk, size_t perm_rep, it_q8* out);
/* Plain f32 transform into the arena, forward or inverse (VkEngine::had with an f32 destination). */
int it_hadamard_f32(it_ctx* ctx, size_t n, size_t ntok, size_t in_off, size_t in_stride, size_t out_off, size_t out_stride,
                    int use_signs, size_t perm_hd, size_t perm_nk, size_t perm_rep, int inverse);

/* Ternary matvec / matmul on q8k activations: y[t, r] (+)= sum_b (d_w[r,b] * d_x[t,b/2]) * (sum_j code*q - sum128)
 * in ascending block order, f32, no fused multiply-add - the arithmetic of cpu::matvec's ternary arm with
 * Numerics::Ggml (src/cpu.rs:25-35, :48-63; src/quant.rs:132-147).  Replaces VkEngine::mv (src/vk/mod.rs:653-704)
 * and the kernels it selects (matvec_t2_1, matvec_c8/c8x2, matvec_t2, matmul_t2s, matmul_t2).  Rows 0..ntok-1
 * of x are used; y is written at y_off + t*y_stride + r.  accum != 0 adds into y (residual adds). */
int it_matvec_t2(it_ctx* ctx, const it_mat* w, size_t ntok, const it_q8* x, size_t y_off, size_t y_stride, int accum);
/* Same launch, additionally stores the integer accumulators (sum_j code*q - sum128) per (t, r, block)
 * into sumi[ntok][rows][cols/128] (device memory owned by the caller).  Used by parity tests. */
int it_matvec_t2_sumi(it_ctx* ctx, const it_mat* w, size_t ntok, const it_q8* x, int32_t* sumi_dev);

/* Int8-group matvec with f32 activations: y[t, r] (+)= sum_g scale[r,g] * sum_{j<16} q[r,16g+j] * x[t,16g+j].
 * Replaces VkEngine::mvq (src/vk/mod.rs:742-745, shaders/matvec_q8.comp); CPU twin mtp::mv (src/mtp.rs:93). */
int it_matvec_q8(it_ctx* ctx, const it_qmat* w, size_t ntok, size_t x_off, size_t x_stride, size_t y_off, size_t y_stride, int accum);

/* Greedy pick: index of the first maximum of n logits at logits_off; the u32 result is stored bit-cast
 * in arena element dst_off (shaders/argmax.comp, src/sampling.rs:50; dispatch at src/vk/mod.rs:866,875). */
int it_argmax(it_ctx* ctx, size_t logits_off, size_t n, size_t dst_off);

/* ---- engine: the decoder behind the reference's backend traits ---------------------------------------
 * Model description: the fields of Config (src/model.rs:7-15) that the forward pass uses, plus the context
 * capacity (VkEngine's ctx_len, src/vk/mod.rs:208).  Every ternary matrix is taken to be Hadamard-folded with
 * block 1024, which is what the reference's GPU schedule assumes (src/vk/mod.rs:536, :783-871). */
typedef struct it_model_config {
    int32_t n_layer, n_embd, n_ff, n_vocab, n_head, n_head_kv, head_dim, n_rot;
    float rope_base; int32_t rope_sections[4]; float eps;
    int32_t conv_k, ssm_state, ssm_groups, ssm_vheads, ssm_inner, full_attn_interval, gdn_v_grouped, ctx_len;
} it_model_config;

/* Tensor ids (layer_names, src/model.rs:93-102; MTP head tensors, src/mtp.rs:51-52).  Ids below IT_T_TOK_EMBD
 * are per layer; the others are global and are addressed with layer = -1. */
enum {
    IT_T_ATTN_NORM = 0, IT_T_POST_NORM, IT_T_FFN_GATE, IT_T_FFN_UP, IT_T_FFN_DOWN,
    IT_T_QKV, IT_T_GATE, IT_T_CONV, IT_T_DT, IT_T_A, IT_T_BETA, IT_T_ALPHA, IT_T_SSM_NORM, IT_T_SSM_OUT,
    IT_T_Q, IT_T_K, IT_T_V, IT_T_O, IT_T_Q_NORM, IT_T_K_NORM,
    IT_T_TOK_EMBD, IT_T_OUTPUT_NORM, IT_T_OUTPUT,
    IT_T_MTP_EH, IT_T_MTP_Q, IT_T_MTP_K, IT_T_MTP_V, IT_T_MTP_O, IT_T_MTP_GATE, IT_T_MTP_UP, IT_T_MTP_DOWN,
    IT_T_MTP_ENORM, IT_T_MTP_HNORM, IT_T_MTP_ATTN_NORM, IT_T_MTP_POST_NORM, IT_T_MTP_Q_NORM, IT_T_MTP_K_NORM, IT_T_MTP_HEAD_NORM,
    IT_T_MTP_EMBD,   /* the NextN head's embedding table (its own, or the trunk's) */
    IT_T_COUNT
};

typedef struct it_engine it_engine;

/* Builds an engine with random-init weights of the given architecture generated on the device (ternary matrices as
 * it_matrix_synth, Q8_0 head matrices as it_qmatrix_synth, f32 vectors uniform in fixed ranges, all from counter hashes
 * of `seed`).  with_mtp != 0 adds a NextN head.  Stands where VkEngine::new_with_mtp stands (src/vk/mod.rs:494-631);
 * geometry is validated before the device is touched (validate_geometry, src/vk/mod.rs:207). */
int it_engine_create_synth(int device, const it_model_config* cfg, uint64_t seed, int with_mtp, it_engine** out);
/* The same model with the trunk matrices and the LM head split by output rows over `world` ranks (this engine holds the
 * rows of `rank`); activations, recurrent state, KV cache and the NextN head stay replicated and every rank computes
 * the same tokens.  Attach the peers of it_engine_ctx() before the first pass. */
int it_engine_create_synth_sharded(int device, const it_model_config* cfg, uint64_t seed, int with_mtp, int rank, int world, it_engine** out);
/* ---- model files ------------------------------------------------------------------------
 * An engine with the weights of a qwen35 GGUF file (container v2/v3).  Stands where Gguf::open + Config::from_gguf +
 * Model::load + VkEngine::new_with_mtp stand (src/gguf.rs:99-140, src/model.rs:16-62, src/cpu.rs:91-112,
 * src/vk/mod.rs:494-631).  Accepted, as by the reference's device path: ternary trunk matrices and LM head (PQ2_0, or
 * PTQ1_0 re-coded to the same 2-bit codes and scale), all of them Hadamard-folded with block 1024
 * (prism.hadamard.weight_names; sign_mode "none" or "explicit"); F32 / F16 / BF16 vectors and beta / alpha matrices;
 * an embedding table of any type below, brought back from latent space when prism.hadamard.inverse_weight_names lists
 * it; a tied LM head (no output.weight).  head_path: NULL = no NextN head; "" or the same path = the NextN block
 * appended to the trunk file; another path = a head-only sidecar whose architecture / qwen35.* / tokenizer.* /
 * prism.hadamard.* metadata must equal the trunk's (validate_compatibility, src/mtp.rs:31-43).  The head's matrices
 * must be Q8_0 or Q6_K (rows a multiple of 4, columns of 256, as src/mtp.rs:55), its norms F32, and it may carry its own embedding table
 * (nextn.embed_tokens).  rank / world as in it_engine_create_synth_sharded: a rank reads only its rows of every trunk
 * matrix.  Everything is checked before the device is touched: IT_EFORMAT for a file that cannot be read or is
 * malformed (short, bad magic, duplicate names, tensor outside the file, missing key or tensor, wrong shape),
 * IT_EUNSUPPORTED for a well-formed model outside the set above. */
int it_engine_create_gguf(int device, const char* path, const char* head_path, int ctx_len, int rank, int world, it_engine** out);
/* The same checks without a device: fills the configuration, whether a NextN head was found, and the trunk file's
 * tensor count and tensor bytes.  Outputs other than cfg may be NULL. */
int it_gguf_inspect(const char* path, const char* head_path, int ctx_len, it_model_config* cfg, int* has_mtp, uint64_t* n_tensors, uint64_t* tensor_bytes);
/* Host decoders of the ggml element types the loader reads (F32 0, F16 1, Q8_0 8, Q4_K 12, Q6_K 14, BF16 30, PQ2_0 142,
 * PTQ1_0 143): n elements (a multiple of the type's block) to f32, in ggml's element order and float operation order
 * (src/quant.rs:51-62, :189-228); and PTQ1_0 blocks (28 bytes) re-coded as PQ2_0 blocks (34 bytes). */
int it_gguf_dequant(uint32_t ggml_type, const void* src, size_t n, float* out);
int it_gguf_ptq1_to_pq2(const void* src, size_t nblocks, void* dst);

void it_engine_destroy(it_engine* e);
it_ctx* it_engine_ctx(it_engine* e);
/* Read-back of weights and state for parity tests.  Ternary / Q8_0 tensors come back as raw ggml rows, f32 tensors as f32. */
int it_engine_tensor_bytes(it_engine* e, int layer, int tensor, size_t* nbytes);
int it_engine_tensor_read(it_engine* e, int layer, int tensor, void* host);
int it_engine_signs_read(it_engine* e, size_t width, float* host);
/* which: 0 conv state, 1 ssm state, 2 K cache, 3 V cache (active positions, decoded to f32), 4 MTP K, 5 MTP V. */
int it_engine_state_read(it_engine* e, int layer, int which, float* host, size_t max_floats, size_t* n_floats);
int it_engine_hidden_read(it_engine* e, size_t row, float* host);   /* output-normed hidden row of the last pass (h_nextn) */
int it_engine_position(it_engine* e);

/* Engine trait (src/engine.rs:8-15).  eval: feed tokens, optionally return the last token's logits (n_vocab floats).
 * eval_argmax: feed tokens and return the greedy pick of the last one, reading back 4 bytes (src/vk/mod.rs:900). */
int it_engine_eval(it_engine* e, const uint32_t* toks, size_t n, float* logits_or_null);
int it_engine_eval_argmax(it_engine* e, const uint32_t* toks, size_t n, uint32_t* next);
int it_engine_reset(it_engine* e);
/* generate_inner's greedy path (src/engine.rs:151-174): prefill, then n_predict greedy tokens (stops early on `eos`
 * unless eos is UINT32_MAX).  The decode steps run as one recorded graph per token. */
int it_engine_generate(it_engine* e, const uint32_t* prompt, size_t n_prompt, size_t n_predict, uint32_t eos, uint32_t* out, size_t* n_out);

/* n more greedy steps chained on the device (the pick of a step is the next step's token) without reading anything back
 * in between; continues from the last pick.  Used to time decoding with everything resident; last_pick may be NULL. */
int it_engine_decode_steps(it_engine* e, size_t n, uint32_t* last_pick);
/* Kernel launches of one recorded greedy step (>= 0; counted from the recorded graph), or a negative code. */
int it_engine_step_kernels(it_engine* e);
/* Diagnostics of the persistent decode-step kernel (engine built with the environment value IT_STEP_TRACE=1): the
 * nanosecond clock at which CTA 0 and the last CTA arrived at and left each grid barrier of the most recent step,
 * out[(cta * 1024 + barrier) * 2 + {0 arrive, 1 leave}] with cta in {0, 1}; max_barriers must be 1024. */
int it_engine_step_trace(it_engine* e, uint64_t* out, size_t max_barriers);

/* MtpBackend trait (src/mtp.rs:150-163), one to one. */
int it_engine_mtp_prefill(it_engine* e, const uint32_t* prompt, size_t n, uint32_t* next);
int it_engine_mtp_single(it_engine* e, uint32_t x, uint32_t* next);
int it_engine_mtp_draft(it_engine* e, const uint32_t* toks, size_t n, uint32_t* draft);
int it_engine_mtp_verify(it_engine* e, uint32_t x, uint32_t d, uint32_t* a0, uint32_t* a1);
int it_engine_mtp_reject(it_engine* e);
int it_engine_mtp_reset_all(it_engine* e);

/* greedy_mtp (src/mtp.rs:166-204) over any backend given as a table of callbacks; is_eog / on_tok as in the reference
 * (on_tok returning 0 stops).  stats: drafted, accepted, steps, draft_calls, verify_calls, single_forwards,
 * timed_decode_forwards, rejected, terminal_rollbacks.  Returns the number of tokens written to out, or a negative code. */
typedef struct it_mtp_backend {
    void* user;
    uint32_t (*prefill)(void* user, const uint32_t* prompt, size_t n);
    uint32_t (*single)(void* user, uint32_t x);
    uint32_t (*draft)(void* user, const uint32_t* toks, size_t n);
    void (*verify)(void* user, uint32_t x, uint32_t d, uint32_t* a0, uint32_t* a1);
    void (*reject)(void* user);
    void (*reset_all)(void* user);
} it_mtp_backend;
int64_t it_greedy_mtp(const it_mtp_backend* b, const uint32_t* prompt, size_t n_prompt, size_t n_predict,
                      int (*is_eog)(void* user, uint32_t tok), int (*on_tok)(void* user, uint32_t tok), void* cb_user,
                      uint32_t* out, int64_t stats[9]);
/* generate_mtp (src/engine.rs:180-191): greedy_mtp over this engine's own MtpBackend. */
int64_t it_engine_generate_mtp(it_engine* e, const uint32_t* prompt, size_t n_prompt, size_t n_predict, uint32_t eos, uint32_t* out, int64_t stats[9]);

/* Draft length k = 1..3.  The reference defines k = 1 only (src/mtp.rs:3-8: the head needs the trunk's hidden state of the
 * previous position, which does not exist for a drafted position); this extension keeps its invariant (the output is
 * plain greedy decoding).  Draft i >= 2 feeds the head its own hidden state before head_norm with draft i - 1 as the
 * token, one position on; its KV entry is provisional.  it_engine_mtp_verify_k runs the k + 1 rows [x, d_1 .. d_k]
 * through the trunk with a recurrent-state checkpoint after every row and returns the k + 1 picks; the caller keeps the
 * longest prefix with pick_{i-1} == d_i and calls it_engine_mtp_rollback(keep_rows) (1 <= keep_rows <= k + 1) - always,
 * also when every row is kept.  it_greedy_mtp_k is that loop (k = 1 reproduces it_greedy_mtp's tokens and counters;
 * `rejected` counts discarded drafts); it_engine_generate_mtp_k runs it over this engine. */
int it_engine_mtp_draft_k(it_engine* e, const uint32_t* toks, size_t n, size_t k, uint32_t* drafts);
int it_engine_mtp_verify_k(it_engine* e, uint32_t x, const uint32_t* drafts, size_t k, uint32_t* picks);
int it_engine_mtp_rollback(it_engine* e, size_t keep_rows);
typedef struct it_mtp_backend_k {
    void* user;
    uint32_t (*prefill)(void* user, const uint32_t* prompt, size_t n);
    uint32_t (*single)(void* user, uint32_t x);
    void (*draft_k)(void* user, const uint32_t* toks, size_t n, size_t k, uint32_t* drafts);
    void (*verify_k)(void* user, uint32_t x, const uint32_t* drafts, size_t k, uint32_t* picks);
    void (*rollback)(void* user, size_t keep_rows);
    void (*reset_all)(void* user);
} it_mtp_backend_k;
int64_t it_greedy_mtp_k(const it_mtp_backend_k* b, size_t k, const uint32_t* prompt, size_t n_prompt, size_t n_predict,
                        int (*is_eog)(void* user, uint32_t tok), int (*on_tok)(void* user, uint32_t tok), void* cb_user,
                        uint32_t* out, int64_t stats[9]);
int64_t it_engine_generate_mtp_k(it_engine* e, size_t k, const uint32_t* prompt, size_t n_prompt, size_t n_predict, uint32_t eos, uint32_t* out, int64_t stats[9]);

/* Greedy pick for callers that must not allocate device memory.  No counterpart in the reference: it exists
 * for hosts that hand all of HBM to their own pool at start-up (weights, KV cache, activation arena) and for
 * code paths where the implicit device-wide synchronisation of cudaMalloc / cudaFree is not acceptable, e.g. a
 * sampling step called from inside a serving loop.  Such callers cannot create an it_ctx (which owns an arena
 * and scratch), so this entry point takes raw device pointers and a stream instead and keeps its scratch
 * (8.4 KB: per-CTA partial results and an arrival counter) in a fixed array inside the library image.
 *  - logits_dev: n f32 values, 16-byte aligned; index_dev: one u32 (the first index of the maximum, same rule
 *    as it_argmax); stream: a cudaStream_t of the current device (may be NULL for the default stream).
 *  - n may not exceed 16,777,216 (2^24); larger inputs are refused with IT_EINVAL.
 *  - The call runs on the device that is current in the calling thread.  The first call on each device looks
 *    up the scratch array's device address; make that first call outside any stream capture.
 *  - It calls neither cudaMalloc nor cudaFree nor any allocating library routine.
 *  - All calls on one device share the one scratch array: two calls whose kernels overlap on the GPU (different
 *    streams, no dependency) race on it and give wrong results.  Calls on one stream are safe back to back. */
int it_argmax_static(void* stream, const float* logits_dev, size_t n, uint32_t* index_dev);

#ifdef __cplusplus
}
#endif
#endif
