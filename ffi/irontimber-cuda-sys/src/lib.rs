//! Raw bindings to `libirontimber_cuda.so` (`include/irontimber_cuda.h`), one declaration per exported entry point, in
//! the header's order.  Every function returns 0 or a negative `IT_E*` code unless noted; `it_last_error` gives the
//! message of the last failure on the calling thread.  One context = one device = one host thread.
#![allow(non_camel_case_types)]
use std::os::raw::{c_char, c_int, c_void};

pub const IT_OK: c_int = 0;
pub const IT_EINVAL: c_int = -1;
pub const IT_ECUDA: c_int = -2;
pub const IT_ENOMEM: c_int = -3;
pub const IT_ESTATE: c_int = -4;
pub const IT_ETIMEOUT: c_int = -5;
pub const IT_EFORMAT: c_int = -6;
pub const IT_EUNSUPPORTED: c_int = -7;

#[repr(C)] pub struct it_ctx { _p: [u8; 0] }
#[repr(C)] pub struct it_mat { _p: [u8; 0] }
#[repr(C)] pub struct it_qmat { _p: [u8; 0] }
#[repr(C)] pub struct it_q8 { _p: [u8; 0] }
#[repr(C)] pub struct it_graph { _p: [u8; 0] }
#[repr(C)] pub struct it_engine { _p: [u8; 0] }

/// `it_model_config`: the fields of `Config` (src/model.rs:7-15) the forward pass uses, plus the context capacity.
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct it_model_config {
    pub n_layer: i32, pub n_embd: i32, pub n_ff: i32, pub n_vocab: i32, pub n_head: i32, pub n_head_kv: i32, pub head_dim: i32, pub n_rot: i32,
    pub rope_base: f32, pub rope_sections: [i32; 4], pub eps: f32,
    pub conv_k: i32, pub ssm_state: i32, pub ssm_groups: i32, pub ssm_vheads: i32, pub ssm_inner: i32, pub full_attn_interval: i32, pub gdn_v_grouped: i32, pub ctx_len: i32,
}

/// Tensor ids (`IT_T_*`): per-layer ids below `IT_T_TOK_EMBD`, global ones addressed with layer = -1.
pub const IT_T_ATTN_NORM: c_int = 0; pub const IT_T_POST_NORM: c_int = 1; pub const IT_T_FFN_GATE: c_int = 2; pub const IT_T_FFN_UP: c_int = 3; pub const IT_T_FFN_DOWN: c_int = 4;
pub const IT_T_QKV: c_int = 5; pub const IT_T_GATE: c_int = 6; pub const IT_T_CONV: c_int = 7; pub const IT_T_DT: c_int = 8; pub const IT_T_A: c_int = 9;
pub const IT_T_BETA: c_int = 10; pub const IT_T_ALPHA: c_int = 11; pub const IT_T_SSM_NORM: c_int = 12; pub const IT_T_SSM_OUT: c_int = 13;
pub const IT_T_Q: c_int = 14; pub const IT_T_K: c_int = 15; pub const IT_T_V: c_int = 16; pub const IT_T_O: c_int = 17; pub const IT_T_Q_NORM: c_int = 18; pub const IT_T_K_NORM: c_int = 19;
pub const IT_T_TOK_EMBD: c_int = 20; pub const IT_T_OUTPUT_NORM: c_int = 21; pub const IT_T_OUTPUT: c_int = 22;
pub const IT_T_MTP_EH: c_int = 23; pub const IT_T_MTP_Q: c_int = 24; pub const IT_T_MTP_K: c_int = 25; pub const IT_T_MTP_V: c_int = 26; pub const IT_T_MTP_O: c_int = 27;
pub const IT_T_MTP_GATE: c_int = 28; pub const IT_T_MTP_UP: c_int = 29; pub const IT_T_MTP_DOWN: c_int = 30;
pub const IT_T_MTP_ENORM: c_int = 31; pub const IT_T_MTP_HNORM: c_int = 32; pub const IT_T_MTP_ATTN_NORM: c_int = 33; pub const IT_T_MTP_POST_NORM: c_int = 34;
pub const IT_T_MTP_Q_NORM: c_int = 35; pub const IT_T_MTP_K_NORM: c_int = 36; pub const IT_T_MTP_HEAD_NORM: c_int = 37; pub const IT_T_MTP_EMBD: c_int = 38;

/// Callback table of `it_greedy_mtp` (the methods of `MtpBackend`, src/mtp.rs:150-163).
#[repr(C)]
pub struct it_mtp_backend {
    pub user: *mut c_void,
    pub prefill: Option<unsafe extern "C" fn(user: *mut c_void, prompt: *const u32, n: usize) -> u32>,
    pub single: Option<unsafe extern "C" fn(user: *mut c_void, x: u32) -> u32>,
    pub draft: Option<unsafe extern "C" fn(user: *mut c_void, toks: *const u32, n: usize) -> u32>,
    pub verify: Option<unsafe extern "C" fn(user: *mut c_void, x: u32, d: u32, a0: *mut u32, a1: *mut u32)>,
    pub reject: Option<unsafe extern "C" fn(user: *mut c_void)>,
    pub reset_all: Option<unsafe extern "C" fn(user: *mut c_void)>,
}
/// Callback table of `it_greedy_mtp_k` (draft length k).
#[repr(C)]
pub struct it_mtp_backend_k {
    pub user: *mut c_void,
    pub prefill: Option<unsafe extern "C" fn(user: *mut c_void, prompt: *const u32, n: usize) -> u32>,
    pub single: Option<unsafe extern "C" fn(user: *mut c_void, x: u32) -> u32>,
    pub draft_k: Option<unsafe extern "C" fn(user: *mut c_void, toks: *const u32, n: usize, k: usize, drafts: *mut u32)>,
    pub verify_k: Option<unsafe extern "C" fn(user: *mut c_void, x: u32, drafts: *const u32, k: usize, picks: *mut u32)>,
    pub rollback: Option<unsafe extern "C" fn(user: *mut c_void, keep_rows: usize)>,
    pub reset_all: Option<unsafe extern "C" fn(user: *mut c_void)>,
}
pub type it_tok_cb = Option<unsafe extern "C" fn(user: *mut c_void, tok: u32) -> c_int>;

extern "C" {
    pub fn it_last_error() -> *const c_char;
    pub fn it_version() -> c_int;

    // ---- context and arena (Ctx::new_with + the arena of VkEngine, src/vk/mod.rs:267, :567-576)
    pub fn it_ctx_create(device: c_int, arena_floats: usize, out: *mut *mut it_ctx) -> c_int;
    pub fn it_ctx_destroy(ctx: *mut it_ctx);
    pub fn it_sync(ctx: *mut it_ctx) -> c_int;
    pub fn it_ctx_stream(ctx: *mut it_ctx) -> *mut c_void;
    pub fn it_arena_ptr(ctx: *mut it_ctx) -> *mut f32;
    pub fn it_arena_floats(ctx: *mut it_ctx) -> usize;
    pub fn it_arena_write(ctx: *mut it_ctx, off: usize, host: *const c_void, n_floats: usize) -> c_int;
    pub fn it_arena_read(ctx: *mut it_ctx, off: usize, host: *mut c_void, n_floats: usize) -> c_int;
    pub fn it_ctx_ipc_handle(ctx: *mut it_ctx, handle64: *mut c_void) -> c_int;
    pub fn it_ctx_attach_peers(ctx: *mut it_ctx, rank: c_int, world: c_int, handles: *const c_void) -> c_int;
    pub fn it_ctx_world(ctx: *const it_ctx) -> c_int;
    pub fn it_ctx_attach_peers_local(ctx: *mut it_ctx, rank: c_int, world: c_int, all: *const *mut it_ctx) -> c_int;
    pub fn it_ctx_set_peer_wait_us(ctx: *mut it_ctx, microseconds: f64) -> c_int;
    pub fn it_arena_zero(ctx: *mut it_ctx, off: usize, n_floats: usize) -> c_int;
    pub fn it_capture_begin(ctx: *mut it_ctx) -> c_int;
    pub fn it_capture_end(ctx: *mut it_ctx, out: *mut *mut it_graph) -> c_int;
    pub fn it_graph_launch(ctx: *mut it_ctx, g: *mut it_graph) -> c_int;
    pub fn it_graph_destroy(g: *mut it_graph);
    pub fn it_graph_kernel_nodes(g: *const it_graph) -> c_int;
    pub fn it_signs_set(ctx: *mut it_ctx, n: usize, signs: *const f32) -> c_int;

    // ---- weights (the `mat` upload closure and DevMat, src/vk/mod.rs:459, :579-599)
    pub fn it_matrix_upload_pq2(ctx: *mut it_ctx, raw: *const u8, rows: usize, cols: usize, out: *mut *mut it_mat) -> c_int;
    pub fn it_matrix_upload_packed2(ctx: *mut it_ctx, words: *const u32, scales: *const f32, rows: usize, cols: usize, out: *mut *mut it_mat) -> c_int;
    pub fn it_matrix_synth(ctx: *mut it_ctx, seed: u64, rows: usize, cols: usize, four_codes: c_int, out: *mut *mut it_mat) -> c_int;
    pub fn it_shard_range(rows: usize, rank: c_int, world: c_int, row0: *mut usize, nrows: *mut usize) -> c_int;
    pub fn it_matrix_set_shard(m: *mut it_mat, row0: usize, total_rows: usize) -> c_int;
    pub fn it_matrix_synth_rows(ctx: *mut it_ctx, seed: u64, total_rows: usize, cols: usize, four_codes: c_int, row0: usize, nrows: usize, out: *mut *mut it_mat) -> c_int;
    pub fn it_qmatrix_set_shard(m: *mut it_qmat, row0: usize, total_rows: usize) -> c_int;
    pub fn it_qmatrix_synth_rows(ctx: *mut it_ctx, seed: u64, total_rows: usize, cols: usize, row0: usize, nrows: usize, out: *mut *mut it_qmat) -> c_int;
    pub fn it_matrix_download_pq2(ctx: *mut it_ctx, m: *const it_mat, raw: *mut u8) -> c_int;
    pub fn it_matrix_rows(m: *const it_mat) -> usize;
    pub fn it_matrix_cols(m: *const it_mat) -> usize;
    pub fn it_matrix_device_bytes(m: *const it_mat) -> usize;
    pub fn it_matrix_destroy(m: *mut it_mat);
    pub fn it_qmatrix_upload_q8_0(ctx: *mut it_ctx, raw: *const u8, rows: usize, cols: usize, out: *mut *mut it_qmat) -> c_int;
    pub fn it_qmatrix_synth(ctx: *mut it_ctx, seed: u64, rows: usize, cols: usize, out: *mut *mut it_qmat) -> c_int;
    pub fn it_qmatrix_download_q8_0(ctx: *mut it_ctx, m: *const it_qmat, raw: *mut u8) -> c_int;
    pub fn it_qmatrix_upload_q6_k(ctx: *mut it_ctx, raw: *const u8, rows: usize, cols: usize, out: *mut *mut it_qmat) -> c_int;
    pub fn it_qmatrix_download_g16(ctx: *mut it_ctx, m: *const it_qmat, raw: *mut u8) -> c_int;
    pub fn it_qmatrix_group16(m: *const it_qmat) -> c_int;
    pub fn it_qmatrix_rows(m: *const it_qmat) -> usize;
    pub fn it_qmatrix_cols(m: *const it_qmat) -> usize;
    pub fn it_qmatrix_destroy(m: *mut it_qmat);

    // ---- q8k activation rows (Q8K, src/quant.rs:68-71)
    pub fn it_q8_create(ctx: *mut it_ctx, max_n: usize, max_tok: usize, out: *mut *mut it_q8) -> c_int;
    pub fn it_q8_destroy(q: *mut it_q8);
    pub fn it_q8_read(ctx: *mut it_ctx, q: *const it_q8, tok: usize, qs: *mut i8, d: *mut f32, sum128: *mut i32) -> c_int;

    // ---- ops (VkEngine::had / mv / mvq / argmax, src/vk/mod.rs:749, :653, :742, :866)
    pub fn it_hadamard_q8(ctx: *mut it_ctx, n: usize, ntok: usize, x_off: usize, x_stride: usize, rotate: c_int, use_signs: c_int,
                          perm_hd: usize, perm_nk: usize, perm_rep: usize, out: *mut it_q8) -> c_int;
    pub fn it_hadamard_f32(ctx: *mut it_ctx, n: usize, ntok: usize, in_off: usize, in_stride: usize, out_off: usize, out_stride: usize,
                           use_signs: c_int, perm_hd: usize, perm_nk: usize, perm_rep: usize, inverse: c_int) -> c_int;
    pub fn it_matvec_t2(ctx: *mut it_ctx, w: *const it_mat, ntok: usize, x: *const it_q8, y_off: usize, y_stride: usize, accum: c_int) -> c_int;
    pub fn it_matvec_t2_sumi(ctx: *mut it_ctx, w: *const it_mat, ntok: usize, x: *const it_q8, sumi_dev: *mut i32) -> c_int;
    pub fn it_matvec_q8(ctx: *mut it_ctx, w: *const it_qmat, ntok: usize, x_off: usize, x_stride: usize, y_off: usize, y_stride: usize, accum: c_int) -> c_int;
    pub fn it_argmax(ctx: *mut it_ctx, logits_off: usize, n: usize, dst_off: usize) -> c_int;

    // ---- engine: the decoder behind Engine / ServeEngine / MtpBackend
    pub fn it_engine_create_synth(device: c_int, cfg: *const it_model_config, seed: u64, with_mtp: c_int, out: *mut *mut it_engine) -> c_int;
    pub fn it_engine_create_synth_sharded(device: c_int, cfg: *const it_model_config, seed: u64, with_mtp: c_int, rank: c_int, world: c_int, out: *mut *mut it_engine) -> c_int;
    /// head_path: null = no NextN head; "" = the block appended to the trunk file; else a head-only sidecar (--mtp-head).
    pub fn it_engine_create_gguf(device: c_int, path: *const c_char, head_path: *const c_char, ctx_len: c_int, rank: c_int, world: c_int, out: *mut *mut it_engine) -> c_int;
    pub fn it_gguf_inspect(path: *const c_char, head_path: *const c_char, ctx_len: c_int, cfg: *mut it_model_config, has_mtp: *mut c_int, n_tensors: *mut u64, tensor_bytes: *mut u64) -> c_int;
    pub fn it_gguf_dequant(ggml_type: u32, src: *const c_void, n: usize, out: *mut f32) -> c_int;
    pub fn it_gguf_ptq1_to_pq2(src: *const c_void, nblocks: usize, dst: *mut c_void) -> c_int;
    pub fn it_engine_destroy(e: *mut it_engine);
    pub fn it_engine_ctx(e: *mut it_engine) -> *mut it_ctx;
    pub fn it_engine_tensor_bytes(e: *mut it_engine, layer: c_int, tensor: c_int, nbytes: *mut usize) -> c_int;
    pub fn it_engine_tensor_read(e: *mut it_engine, layer: c_int, tensor: c_int, host: *mut c_void) -> c_int;
    pub fn it_engine_signs_read(e: *mut it_engine, width: usize, host: *mut f32) -> c_int;
    pub fn it_engine_state_read(e: *mut it_engine, layer: c_int, which: c_int, host: *mut f32, max_floats: usize, n_floats: *mut usize) -> c_int;
    pub fn it_engine_hidden_read(e: *mut it_engine, row: usize, host: *mut f32) -> c_int;
    pub fn it_engine_position(e: *mut it_engine) -> c_int;
    pub fn it_engine_eval(e: *mut it_engine, toks: *const u32, n: usize, logits_or_null: *mut f32) -> c_int;
    pub fn it_engine_eval_argmax(e: *mut it_engine, toks: *const u32, n: usize, next: *mut u32) -> c_int;
    pub fn it_engine_reset(e: *mut it_engine) -> c_int;
    pub fn it_engine_generate(e: *mut it_engine, prompt: *const u32, n_prompt: usize, n_predict: usize, eos: u32, out: *mut u32, n_out: *mut usize) -> c_int;
    pub fn it_engine_decode_steps(e: *mut it_engine, n: usize, last_pick: *mut u32) -> c_int;
    pub fn it_engine_step_kernels(e: *mut it_engine) -> c_int;
    pub fn it_engine_step_trace(e: *mut it_engine, out: *mut u64, max_barriers: usize) -> c_int;
    pub fn it_engine_mtp_prefill(e: *mut it_engine, prompt: *const u32, n: usize, next: *mut u32) -> c_int;
    pub fn it_engine_mtp_single(e: *mut it_engine, x: u32, next: *mut u32) -> c_int;
    pub fn it_engine_mtp_draft(e: *mut it_engine, toks: *const u32, n: usize, draft: *mut u32) -> c_int;
    pub fn it_engine_mtp_verify(e: *mut it_engine, x: u32, d: u32, a0: *mut u32, a1: *mut u32) -> c_int;
    pub fn it_engine_mtp_reject(e: *mut it_engine) -> c_int;
    pub fn it_engine_mtp_reset_all(e: *mut it_engine) -> c_int;
    /// Returns the number of tokens written to `out`, or a negative code.  `stats` receives nine counters (MtpStats order).
    pub fn it_greedy_mtp(b: *const it_mtp_backend, prompt: *const u32, n_prompt: usize, n_predict: usize, is_eog: it_tok_cb, on_tok: it_tok_cb, cb_user: *mut c_void,
                         out: *mut u32, stats: *mut i64) -> i64;
    pub fn it_engine_generate_mtp(e: *mut it_engine, prompt: *const u32, n_prompt: usize, n_predict: usize, eos: u32, out: *mut u32, stats: *mut i64) -> i64;
    pub fn it_engine_mtp_draft_k(e: *mut it_engine, toks: *const u32, n: usize, k: usize, drafts: *mut u32) -> c_int;
    pub fn it_engine_mtp_verify_k(e: *mut it_engine, x: u32, drafts: *const u32, k: usize, picks: *mut u32) -> c_int;
    pub fn it_engine_mtp_rollback(e: *mut it_engine, keep_rows: usize) -> c_int;
    pub fn it_greedy_mtp_k(b: *const it_mtp_backend_k, k: usize, prompt: *const u32, n_prompt: usize, n_predict: usize, is_eog: it_tok_cb, on_tok: it_tok_cb, cb_user: *mut c_void,
                           out: *mut u32, stats: *mut i64) -> i64;
    pub fn it_engine_generate_mtp_k(e: *mut it_engine, k: usize, prompt: *const u32, n_prompt: usize, n_predict: usize, eos: u32, out: *mut u32, stats: *mut i64) -> i64;

    /// Greedy pick on caller-owned device buffers without any allocation (see the header for its limits).
    pub fn it_argmax_static(stream: *mut c_void, logits_dev: *const f32, n: usize, index_dev: *mut u32) -> c_int;
}

/// The message of the last failure on this thread.
pub fn last_error() -> String {
    unsafe {
        let p = it_last_error();
        if p.is_null() { String::new() } else { std::ffi::CStr::from_ptr(p).to_string_lossy().into_owned() }
    }
}
