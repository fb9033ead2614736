//! `--backend cuda`: the B200 backend behind the reference's backend traits.  Drop this file into the reference as
//! `src/cuda.rs` (module `bonsai::cuda`, feature `cuda`); `backend_cuda.patch` next to it adds the feature, the module
//! and the three `match backend` arms.  NOT COMPILED in the image this repository was built in (no Rust toolchain);
//! the same entry points are exercised through ctypes by the repository's pytest suite.
//!
//! `CudaEngine` owns an `it_engine`: the library maps the GGUF file itself, uploads and repacks the weights and runs
//! the whole schedule of `VkEngine::run_chunk_v` (src/vk/mod.rs:763-892) and `mtp_pass_mode` (:912-959) on the device.
//! Every trait method is one call; a negative status becomes the reference's panic convention with the library's message.
use crate::engine::{Engine, ServeEngine};
use crate::mtp::MtpBackend;
use irontimber_cuda_sys as sys;
use std::ffi::CString;
use std::os::raw::c_int;
use std::ptr;

fn check(code: c_int, what: &str) {
    if code != sys::IT_OK { panic!("{what}: irontimber_cuda error {code}: {}", sys::last_error()); }
}

pub struct CudaEngine {
    e: *mut sys::it_engine,
    cfg: sys::it_model_config,
    has_mtp: bool,
}

impl CudaEngine {
    /// Stands where `VkEngine::new` / `new_with_mtp` stand (src/vk/mod.rs:494).  `head`: `None` = no NextN head,
    /// `Some("")` = the block appended to the trunk file, `Some(path)` = a head-only sidecar (`--mtp-head`).
    /// Everything is validated before the device is touched; a refused model comes back as `Err(String)`.
    pub fn open(model: &str, head: Option<&str>, ctx_len: usize, device: Option<&str>) -> Result<Self, String> {
        let dev: c_int = match device { Some(s) => s.parse().map_err(|_| format!("--device {s}: expected a CUDA device index"))?, None => 0 };
        let path = CString::new(model).map_err(|e| e.to_string())?;
        let head_c = match head { Some(h) => Some(CString::new(h).map_err(|e| e.to_string())?), None => None };
        let head_p = head_c.as_ref().map_or(ptr::null(), |h| h.as_ptr());
        let mut cfg = sys::it_model_config::default();
        let mut has: c_int = 0;
        let r = unsafe { sys::it_gguf_inspect(path.as_ptr(), head_p, ctx_len as c_int, &mut cfg, &mut has, ptr::null_mut(), ptr::null_mut()) };
        if r != sys::IT_OK { return Err(sys::last_error()); }
        let mut e: *mut sys::it_engine = ptr::null_mut();
        let r = unsafe { sys::it_engine_create_gguf(dev, path.as_ptr(), head_p, ctx_len as c_int, 0, 1, &mut e) };
        if r != sys::IT_OK { return Err(sys::last_error()); }
        Ok(CudaEngine { e, cfg, has_mtp: has != 0 })
    }
    pub fn has_mtp(&self) -> bool { self.has_mtp }
    pub fn n_vocab(&self) -> usize { self.cfg.n_vocab as usize }
    pub fn position(&self) -> usize { unsafe { sys::it_engine_position(self.e) as usize } }
    /// `generate_inner`'s greedy path (src/engine.rs:151-174) with the decode step replayed from one recorded graph.
    pub fn generate_greedy(&mut self, prompt: &[u32], n_predict: usize, eos: Option<u32>) -> Vec<u32> {
        let mut out = vec![0u32; n_predict]; let mut n = 0usize;
        check(unsafe { sys::it_engine_generate(self.e, prompt.as_ptr(), prompt.len(), n_predict, eos.unwrap_or(u32::MAX), out.as_mut_ptr(), &mut n) }, "generate");
        out.truncate(n); out
    }
}
impl Drop for CudaEngine { fn drop(&mut self) { unsafe { sys::it_engine_destroy(self.e) } } }

impl Engine for CudaEngine {                        // src/engine.rs:8-15
    fn eval(&mut self, toks: &[u32], want_logits: bool) -> Option<Vec<f32>> {
        let mut lg = if want_logits { vec![0f32; self.n_vocab()] } else { Vec::new() };
        let p = if want_logits { lg.as_mut_ptr() } else { ptr::null_mut() };
        check(unsafe { sys::it_engine_eval(self.e, toks.as_ptr(), toks.len(), p) }, "eval");
        want_logits.then_some(lg)
    }
    fn eval_argmax(&mut self, toks: &[u32]) -> u32 {
        let mut t = 0u32;
        check(unsafe { sys::it_engine_eval_argmax(self.e, toks.as_ptr(), toks.len(), &mut t) }, "eval_argmax");
        t
    }
    fn reset(&mut self) { check(unsafe { sys::it_engine_reset(self.e) }, "reset"); }
    fn review_snapshot(&self) -> serde_json::Value {
        serde_json::json!({"backend": "cuda", "layers": self.cfg.n_layer, "head_loaded": self.has_mtp, "context_capacity": self.cfg.ctx_len, "kv_dtype": "f16", "position": self.position()})
    }
}

impl ServeEngine for CudaEngine {                   // src/engine.rs:69-78
    fn mtp_backend(&mut self) -> Option<&mut dyn MtpBackend> { if self.has_mtp { Some(self) } else { None } }
    fn as_engine(&mut self) -> &mut dyn Engine { self }
}

impl MtpBackend for CudaEngine {                    // src/mtp.rs:150-163
    fn mtp_prefill(&mut self, prompt: &[u32]) -> u32 {
        let mut t = 0u32; check(unsafe { sys::it_engine_mtp_prefill(self.e, prompt.as_ptr(), prompt.len(), &mut t) }, "mtp_prefill"); t
    }
    fn mtp_single(&mut self, x: u32) -> u32 { let mut t = 0u32; check(unsafe { sys::it_engine_mtp_single(self.e, x, &mut t) }, "mtp_single"); t }
    fn mtp_draft(&mut self, toks: &[u32]) -> u32 {
        let mut t = 0u32; check(unsafe { sys::it_engine_mtp_draft(self.e, toks.as_ptr(), toks.len(), &mut t) }, "mtp_draft"); t
    }
    fn mtp_verify(&mut self, x: u32, d: u32) -> (u32, u32) {
        let (mut a0, mut a1) = (0u32, 0u32);
        check(unsafe { sys::it_engine_mtp_verify(self.e, x, d, &mut a0, &mut a1) }, "mtp_verify");
        (a0, a1)
    }
    fn mtp_reject(&mut self) { check(unsafe { sys::it_engine_mtp_reject(self.e) }, "mtp_reject"); }
    fn reset_all(&mut self) { check(unsafe { sys::it_engine_mtp_reset_all(self.e) }, "reset_all"); }
}
