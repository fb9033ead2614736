"""Host-side mirror of the reference's backend traits over the C ABI.

`CudaEngine` offers the methods of `Engine` (src/engine.rs:8-15: eval, eval_argmax, reset), of `ServeEngine`
(src/engine.rs:69-78: as_engine, mtp_backend) and of `MtpBackend`
(src/mtp.rs:150-163: mtp_prefill, mtp_single, mtp_draft, mtp_verify, mtp_reject, reset_all) with the reference's
names and argument meaning, plus the two generation loops (`generate`, `generate_mtp`; src/engine.rs:151-191).
Everything runs in libirontimber_cuda.so; this file only marshals arguments.
"""
import ctypes as C

import numpy as np

from . import _lib

TENSORS = ("attn_norm", "post_norm", "ffn_gate", "ffn_up", "ffn_down",
           "qkv", "gate", "conv", "dt", "a", "beta", "alpha", "ssm_norm", "ssm_out",
           "q", "k", "v", "o", "q_norm", "k_norm",
           "tok_embd", "output_norm", "output",
           "mtp_eh", "mtp_q", "mtp_k", "mtp_v", "mtp_o", "mtp_gate", "mtp_up", "mtp_down",
           "mtp_enorm", "mtp_hnorm", "mtp_attn_norm", "mtp_post_norm", "mtp_q_norm", "mtp_k_norm", "mtp_head_norm", "mtp_embd")
TENSOR_ID = {n: i for i, n in enumerate(TENSORS)}
GDN_TENSORS = ("qkv", "gate", "conv", "dt", "a", "beta", "alpha", "ssm_norm", "ssm_out")
ATTN_TENSORS = ("q", "k", "v", "o", "q_norm", "k_norm")
COMMON_TENSORS = ("attn_norm", "post_norm", "ffn_gate", "ffn_up", "ffn_down")
GLOBAL_TENSORS = ("tok_embd", "output_norm", "output")
MTP_TENSORS = TENSORS[TENSOR_ID["mtp_eh"]:]
STAT_NAMES = ("drafted", "accepted", "steps", "draft_calls", "verify_calls", "single_forwards",
              "timed_decode_forwards", "rejected", "terminal_rollbacks")
NO_EOS = 0xFFFFFFFF


class ModelConfig(C.Structure):
    """it_model_config (include/irontimber_cuda.h); the fields of Config (src/model.rs:7-15) the forward pass uses."""
    _fields_ = [("n_layer", C.c_int32), ("n_embd", C.c_int32), ("n_ff", C.c_int32), ("n_vocab", C.c_int32),
                ("n_head", C.c_int32), ("n_head_kv", C.c_int32), ("head_dim", C.c_int32), ("n_rot", C.c_int32),
                ("rope_base", C.c_float), ("rope_sections", C.c_int32 * 4), ("eps", C.c_float),
                ("conv_k", C.c_int32), ("ssm_state", C.c_int32), ("ssm_groups", C.c_int32), ("ssm_vheads", C.c_int32),
                ("ssm_inner", C.c_int32), ("full_attn_interval", C.c_int32), ("gdn_v_grouped", C.c_int32), ("ctx_len", C.c_int32)]

    def is_recurrent(self, il):
        return (il + 1) % self.full_attn_interval != 0


def config_27b(n_layer=64, ctx_len=8192, n_vocab=248320):
    """The 27B architecture (tests/model_tests.rs:38-44, src/model.rs:40-43; rope constants from src/vk/kparity.rs:33,42)."""
    return ModelConfig(n_layer=n_layer, n_embd=5120, n_ff=17408, n_vocab=n_vocab, n_head=24, n_head_kv=4, head_dim=256, n_rot=64,
                       rope_base=1e7, rope_sections=(C.c_int32 * 4)(11, 11, 10, 0), eps=1e-6, conv_k=4, ssm_state=128, ssm_groups=16,
                       ssm_vheads=48, ssm_inner=6144, full_attn_interval=4, gdn_v_grouped=1, ctx_len=ctx_len)


def _u32(a):
    return np.ascontiguousarray(a, np.uint32)


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def inspect_gguf(path, head_path=None, ctx_len=4096):
    """Reads and checks a qwen35 model file without a device: (ModelConfig, has_mtp, tensor count, tensor bytes).
    head_path as in CudaEngine.from_gguf."""
    L = _lib.load()
    cfg, has, nt, nb = ModelConfig(), C.c_int(), C.c_uint64(), C.c_uint64()
    hp = None if head_path is None else str(head_path).encode()
    _lib.check(L.it_gguf_inspect(str(path).encode(), hp, ctx_len, C.byref(cfg), C.byref(has), C.byref(nt), C.byref(nb)))
    return cfg, bool(has.value), nt.value, nb.value


class CudaEngine:
    def __init__(self, cfg, seed=1, with_mtp=False, device=0, rank=0, world=1, group=None, _gguf=None):
        """rank / world > 1: this engine holds the rows of `rank` of every trunk matrix; the arenas of all ranks (one
        process per GPU, torch.distributed initialised) are attached to each other before the constructor returns."""
        self.L = _lib.load()
        self.cfg = cfg
        h = C.c_void_p()
        if _gguf is None:
            _lib.check(self.L.it_engine_create_synth_sharded(device, C.byref(cfg), seed, int(with_mtp), rank, world, C.byref(h)))
        else:
            path, hp = _gguf
            _lib.check(self.L.it_engine_create_gguf(device, path, hp, cfg.ctx_len, rank, world, C.byref(h)))
        self.h = h
        self.with_mtp = with_mtp
        self.rank, self.world = rank, world
        if world > 1:
            from .sharding import attach_peers
            attach_peers(self.L, self.L.it_engine_ctx(self.h), rank, world, group)

    @classmethod
    def from_gguf(cls, path, head_path=None, ctx_len=4096, device=0, rank=0, world=1, group=None):
        """An engine with the weights of a qwen35 GGUF file (VkEngine::new_with_mtp over Model::load, src/vk/mod.rs:494,
        src/cpu.rs:91).  head_path: None = no NextN head, "" = the block appended to the trunk file, else a sidecar."""
        hp = None if head_path is None else str(head_path).encode()
        cfg, has_mtp, _, _ = inspect_gguf(path, head_path, ctx_len)
        return cls(cfg, 0, has_mtp, device, rank, world, group, _gguf=(str(path).encode(), hp))

    def sync(self):
        _lib.check(self.L.it_sync(self.L.it_engine_ctx(self.h)))

    def close(self):
        if self.h:
            self.L.it_engine_destroy(self.h)
            self.h = None

    # ---- Engine ----------------------------------------------------------------------------------
    def eval(self, toks, want_logits=True):
        t = _u32(toks)
        lg = np.empty(self.cfg.n_vocab, np.float32) if want_logits else None
        _lib.check(self.L.it_engine_eval(self.h, _p(t), t.size, _p(lg) if want_logits else None))
        return lg

    def eval_argmax(self, toks):
        t = _u32(toks)
        out = C.c_uint32()
        _lib.check(self.L.it_engine_eval_argmax(self.h, _p(t), t.size, C.byref(out)))
        return out.value

    def reset(self):
        _lib.check(self.L.it_engine_reset(self.h))

    # ---- ServeEngine (src/engine.rs:69-78): what a long-lived server holds -------------------------
    def as_engine(self):
        return self

    def mtp_backend(self):
        """The speculative path when a NextN head was loaded at start-up, else None (VkEngine's impl, src/engine.rs:75-78)."""
        return self if self.with_mtp else None

    @property
    def pos(self):
        return int(self.L.it_engine_position(self.h))

    def generate(self, prompt, n_predict, eos=NO_EOS):
        p = _u32(prompt)
        out = np.zeros(max(n_predict, 1), np.uint32)
        n = C.c_size_t()
        _lib.check(self.L.it_engine_generate(self.h, _p(p), p.size, n_predict, eos, _p(out), C.byref(n)))
        return [int(t) for t in out[:n.value]]

    def decode_steps(self, n, read_last=True):
        out = C.c_uint32()
        _lib.check(self.L.it_engine_decode_steps(self.h, n, C.byref(out) if read_last else None))
        return out.value if read_last else None

    def step_kernels(self):
        """Kernel launches of one recorded greedy decode step (counted from the recorded graph)."""
        n = self.L.it_engine_step_kernels(self.h)
        if n < 0:
            _lib.check(n)
        return n

    # ---- MtpBackend --------------------------------------------------------------------------------
    def mtp_prefill(self, prompt):
        p = _u32(prompt); out = C.c_uint32()
        _lib.check(self.L.it_engine_mtp_prefill(self.h, _p(p), p.size, C.byref(out)))
        return out.value

    def mtp_single(self, x):
        out = C.c_uint32()
        _lib.check(self.L.it_engine_mtp_single(self.h, x, C.byref(out)))
        return out.value

    def mtp_draft(self, toks):
        p = _u32(toks); out = C.c_uint32()
        _lib.check(self.L.it_engine_mtp_draft(self.h, _p(p), p.size, C.byref(out)))
        return out.value

    def mtp_verify(self, x, d):
        a0, a1 = C.c_uint32(), C.c_uint32()
        _lib.check(self.L.it_engine_mtp_verify(self.h, x, d, C.byref(a0), C.byref(a1)))
        return a0.value, a1.value

    def mtp_reject(self):
        _lib.check(self.L.it_engine_mtp_reject(self.h))

    def reset_all(self):
        _lib.check(self.L.it_engine_mtp_reset_all(self.h))

    def generate_mtp(self, prompt, n_predict, eos=NO_EOS):
        p = _u32(prompt)
        out = np.zeros(n_predict + 2, np.uint32)
        stats = np.zeros(9, np.int64)
        n = self.L.it_engine_generate_mtp(self.h, _p(p), p.size, n_predict, eos, _p(out), _p(stats))
        if n < 0:
            _lib.check(int(n))
        return [int(t) for t in out[:n]], dict(zip(STAT_NAMES, (int(s) for s in stats)))

    # ---- draft length k (extension; see include/irontimber_cuda.h) ---------------------------------------------
    def mtp_draft_k(self, toks, k):
        t = _u32(toks)
        d = np.zeros(k, np.uint32)
        _lib.check(self.L.it_engine_mtp_draft_k(self.h, _p(t), t.size, k, _p(d)))
        return [int(x) for x in d]

    def mtp_verify_k(self, x, drafts):
        d = _u32(drafts)
        a = np.zeros(d.size + 1, np.uint32)
        _lib.check(self.L.it_engine_mtp_verify_k(self.h, x, _p(d), d.size, _p(a)))
        return [int(v) for v in a]

    def mtp_rollback(self, keep_rows):
        _lib.check(self.L.it_engine_mtp_rollback(self.h, keep_rows))

    def generate_mtp_k(self, prompt, n_predict, k, eos=NO_EOS):
        p = _u32(prompt)
        out = np.zeros(n_predict + 2, np.uint32)
        stats = np.zeros(9, np.int64)
        n = self.L.it_engine_generate_mtp_k(self.h, k, _p(p), p.size, n_predict, eos, _p(out), _p(stats))
        if n < 0:
            _lib.check(int(n))
        return [int(t) for t in out[:n]], dict(zip(STAT_NAMES, (int(s) for s in stats)))

    # ---- read-back for parity tests ---------------------------------------------------------------------
    def tensor(self, name, layer=-1):
        nb = C.c_size_t()
        _lib.check(self.L.it_engine_tensor_bytes(self.h, layer, TENSOR_ID[name], C.byref(nb)))
        raw = np.empty(nb.value, np.uint8)
        _lib.check(self.L.it_engine_tensor_read(self.h, layer, TENSOR_ID[name], _p(raw)))
        return raw

    def signs(self, width):
        s = np.empty(width, np.float32)
        _lib.check(self.L.it_engine_signs_read(self.h, width, _p(s)))
        return s

    def state(self, layer, which):
        n = C.c_size_t()
        _lib.check(self.L.it_engine_state_read(self.h, layer, which, None, 0, C.byref(n)))
        out = np.empty(n.value, np.float32)
        if n.value:
            _lib.check(self.L.it_engine_state_read(self.h, layer, which, _p(out), n.value, C.byref(n)))
        return out

    def hidden(self, row=0):
        out = np.empty(self.cfg.n_embd, np.float32)
        _lib.check(self.L.it_engine_hidden_read(self.h, row, _p(out)))
        return out


def greedy_mtp(backend, prompt, n, is_eog=lambda t: False, on_tok=lambda t: True):
    """greedy_mtp (src/mtp.rs:166-204) as implemented in the library, over any Python object with the MtpBackend methods."""
    L = _lib.load()

    class B(C.Structure):
        _fields_ = [("user", C.c_void_p),
                    ("prefill", C.CFUNCTYPE(C.c_uint32, C.c_void_p, C.POINTER(C.c_uint32), C.c_size_t)),
                    ("single", C.CFUNCTYPE(C.c_uint32, C.c_void_p, C.c_uint32)),
                    ("draft", C.CFUNCTYPE(C.c_uint32, C.c_void_p, C.POINTER(C.c_uint32), C.c_size_t)),
                    ("verify", C.CFUNCTYPE(None, C.c_void_p, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32))),
                    ("reject", C.CFUNCTYPE(None, C.c_void_p)),
                    ("reset_all", C.CFUNCTYPE(None, C.c_void_p))]
    F = dict(B._fields_)

    def _verify(_, x, d, a0, a1):
        r = backend.mtp_verify(x, d)
        a0[0], a1[0] = r[0], r[1]
    be = B(None, F["prefill"](lambda _, p, k: backend.mtp_prefill([p[i] for i in range(k)])),
           F["single"](lambda _, x: backend.mtp_single(x)),
           F["draft"](lambda _, p, k: backend.mtp_draft([p[i] for i in range(k)])),
           F["verify"](_verify), F["reject"](lambda _: backend.mtp_reject()), F["reset_all"](lambda _: backend.reset_all()))
    CB = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_uint32)
    eog, tok = CB(lambda _, t: int(bool(is_eog(t)))), CB(lambda _, t: int(bool(on_tok(t))))
    pr = _u32(prompt)
    out = np.zeros(max(n, 1) + 2, np.uint32)
    stats = np.zeros(9, np.int64)
    k = L.it_greedy_mtp(C.byref(be), _p(pr), pr.size, n, eog, tok, None, _p(out), _p(stats))
    if k < 0:
        _lib.check(int(k))
    return [int(t) for t in out[:k]], dict(zip(STAT_NAMES, (int(s) for s in stats)))


def greedy_mtp_k(backend, prompt, n, k, is_eog=lambda t: False, on_tok=lambda t: True):
    """The library's speculative loop with draft length k (it_greedy_mtp_k) over any Python object with mtp_prefill,
    mtp_single, mtp_draft_k, mtp_verify_k, mtp_rollback and reset_all."""
    L = _lib.load()

    class B(C.Structure):
        _fields_ = [("user", C.c_void_p),
                    ("prefill", C.CFUNCTYPE(C.c_uint32, C.c_void_p, C.POINTER(C.c_uint32), C.c_size_t)),
                    ("single", C.CFUNCTYPE(C.c_uint32, C.c_void_p, C.c_uint32)),
                    ("draft_k", C.CFUNCTYPE(None, C.c_void_p, C.POINTER(C.c_uint32), C.c_size_t, C.c_size_t, C.POINTER(C.c_uint32))),
                    ("verify_k", C.CFUNCTYPE(None, C.c_void_p, C.c_uint32, C.POINTER(C.c_uint32), C.c_size_t, C.POINTER(C.c_uint32))),
                    ("rollback", C.CFUNCTYPE(None, C.c_void_p, C.c_size_t)),
                    ("reset_all", C.CFUNCTYPE(None, C.c_void_p))]
    F = dict(B._fields_)

    def _draft(_, p, np_, kk, out):
        for i, d in enumerate(backend.mtp_draft_k([p[i] for i in range(np_)], kk)):
            out[i] = d

    def _verify(_, x, d, kk, out):
        for i, a in enumerate(backend.mtp_verify_k(x, [d[i] for i in range(kk)])):
            out[i] = a
    be = B(None, F["prefill"](lambda _, p, m: backend.mtp_prefill([p[i] for i in range(m)])), F["single"](lambda _, x: backend.mtp_single(x)),
           F["draft_k"](_draft), F["verify_k"](_verify), F["rollback"](lambda _, keep: backend.mtp_rollback(keep)), F["reset_all"](lambda _: backend.reset_all()))
    CB = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_uint32)
    eog, tok = CB(lambda _, t: int(bool(is_eog(t)))), CB(lambda _, t: int(bool(on_tok(t))))
    pr = _u32(prompt)
    out = np.zeros(max(n, 1) + 2, np.uint32)
    stats = np.zeros(9, np.int64)
    m = L.it_greedy_mtp_k(C.byref(be), k, _p(pr), pr.size, n, eog, tok, None, _p(out), _p(stats))
    if m < 0:
        _lib.check(int(m))
    return [int(t) for t in out[:m]], dict(zip(STAT_NAMES, (int(s) for s in stats)))
