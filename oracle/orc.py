"""ctypes/numpy front end of the CPU oracle (``liborc.so``).  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module; the
product package never does.  The functions mirror the reference's CPU path one to one and
cite the reference file:line they restate (see ``oracle_core.cpp`` for the arithmetic).
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

QK = 128
PQ2_BYTES = 34
PTQ1_BYTES = 28
Q8_0_BYTES = 34
PQ2_0, PTQ1_0 = 0, 1
Q8_0, Q6_K = 0, 1
GGML, F32 = 0, 1


def build(force=False):
    so = os.path.join(_HERE, "liborc.so")
    srcs = [os.path.join(_HERE, f) for f in os.listdir(_HERE) if f.endswith((".cpp", ".h", ".inc"))]
    if force or not os.path.exists(so) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in srcs):
        subprocess.run(["make", "-C", _HERE, "liborc.so"], check=True, capture_output=True)
    return so


def lib():
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "liborc.so")
        if not os.path.exists(so):
            build()
        _LIB = C.CDLL(so)
        _LIB.orc_packed2_dot_q8k.restype = C.c_float
        _LIB.orc_packed2_dot_f32.restype = C.c_float
        _LIB.orc_argmax.restype = C.c_uint32
        _LIB.orc_greedy_mtp.restype = C.c_int64
        _LIB.orc_max_threads.restype = C.c_int
    return _LIB


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def max_threads():
    return int(lib().orc_max_threads())


# ---- weight decode -----------------------------------------------------------------------
def _dequant(fn, raw, block_bytes, block_elems):
    raw = _c(raw, np.uint8)
    nb = raw.size // block_bytes
    out = np.empty(nb * block_elems, np.float32)
    fn(_p(raw), C.c_int64(nb), _p(out))
    return out


def dequant_pq2_0(raw):   # src/quant.rs:51
    return _dequant(lib().orc_dequant_pq2_0, raw, 34, 128)


def dequant_ptq1_0(raw):  # src/quant.rs:58
    return _dequant(lib().orc_dequant_ptq1_0, raw, 28, 128)


def dequant_q8_0(raw):    # src/quant.rs:188
    return _dequant(lib().orc_dequant_q8_0, raw, 34, 32)


def dequant_q6_k(raw):    # src/quant.rs:192
    return _dequant(lib().orc_dequant_q6_k, raw, 210, 256)


def dequant_q4_k(raw):    # src/quant.rs:215
    return _dequant(lib().orc_dequant_q4_k, raw, 144, 256)


def packed2_from_ggml(ty, raw, rows, cols):  # src/quant.rs:100
    raw = _c(raw, np.uint8)
    words = np.empty(rows * cols // 16, np.uint32)
    scales = np.empty(rows * cols // 128, np.float32)
    lib().orc_packed2_from_ggml(C.c_int(ty), _p(raw), C.c_int64(rows), C.c_int64(cols), _p(words), _p(scales))
    return words, scales


def packed2_row_f32(words, scales, cols, r):  # src/quant.rs:121
    out = np.empty(cols, np.float32)
    lib().orc_packed2_row_f32(_p(words), _p(scales), C.c_int64(cols), C.c_int64(r), _p(out))
    return out


def quantize_q8k(x):  # src/quant.rs:75
    x = _c(x, np.float32)
    n = x.size
    assert n % 256 == 0
    d = np.empty(n // 256, np.float32)
    qs = np.empty(n, np.int8)
    s = np.empty(n // 128, np.int32)
    lib().orc_quantize_q8k(_p(x), C.c_int64(n), _p(d), _p(qs), _p(s))
    return d, qs, s


def packed2_dot_q8k(words, scales, cols, r, q):  # src/quant.rs:132
    d, qs, s = q
    return np.float32(lib().orc_packed2_dot_q8k(_p(words), _p(scales), C.c_int64(cols), C.c_int64(r), _p(d), _p(qs), _p(s)))


def packed2_dot_f32(words, scales, cols, r, x):  # src/quant.rs:150
    x = _c(x, np.float32)
    return np.float32(lib().orc_packed2_dot_f32(_p(words), _p(scales), C.c_int64(cols), C.c_int64(r), _p(x)))


def matvec_ternary(raw, rows, cols, x, numerics=GGML, ty=PQ2_0, nthreads=0, want_sumi=False):
    """cpu::matvec ternary arm (src/cpu.rs:25-35) on raw PQ2_0 / PTQ1_0 row data."""
    raw = _c(raw, np.uint8)
    x = _c(x, np.float32)
    assert x.size == cols
    y = np.empty(rows, np.float32)
    sumi = np.empty((rows, cols // 128), np.int32) if want_sumi else None
    lib().orc_matvec_ternary(C.c_int(ty), _p(raw), C.c_int64(rows), C.c_int64(cols), _p(x), C.c_int(numerics), _p(y),
                             C.c_int(nthreads), _p(sumi) if want_sumi else None)
    return (y, sumi) if want_sumi else y


def q8g16_from_ggml(ty, raw, rows, cols):  # src/quant.rs:235
    raw = _c(raw, np.uint8)
    words = np.empty(rows * cols // 4, np.uint32)
    scales = np.empty(rows * cols // 16, np.float32)
    lib().orc_q8g16_from_ggml(C.c_int(ty), _p(raw), C.c_int64(rows), C.c_int64(cols), _p(words), _p(scales))
    return words, scales


def q8g16_row_f32(words, scales, cols, r):
    out = np.empty(cols, np.float32)
    lib().orc_q8g16_row_f32(_p(words), _p(scales), C.c_int64(cols), C.c_int64(r), _p(out))
    return out


def mvq(words, scales, rows, cols, x, nthreads=0):  # src/mtp.rs:93 + src/quant.rs:266
    x = _c(x, np.float32)
    y = np.empty(rows, np.float32)
    lib().orc_mvq(_p(words), _p(scales), C.c_int64(rows), C.c_int64(cols), _p(x), _p(y), C.c_int(nthreads))
    return y


# ---- Hadamard ----------------------------------------------------------------------------
def fwht_blocks(x, block):  # src/hadamard.rs:7
    y = _c(x, np.float32).copy()
    lib().orc_fwht_blocks(_p(y), C.c_int64(y.size), C.c_int64(block))
    return y


def gdn_group_perm(x, hd, nk, rep):  # src/hadamard.rs:23
    x = _c(x, np.float32)
    o = np.empty_like(x)
    lib().orc_gdn_group_perm(_p(x), _p(o), C.c_int64(hd), C.c_int64(nk), C.c_int64(rep))
    return o


def hadamard_forward(x, block=1024, signs=None, perm=None):  # src/hadamard.rs:35 (+ src/cpu.rs:239)
    x = _c(x, np.float32)
    y = np.empty_like(x)
    hd, nk, rep = perm if perm else (0, 0, 0)
    sg = _c(signs, np.float32) if signs is not None else None
    lib().orc_hadamard_forward(_p(x), _p(y), C.c_int64(x.size), C.c_int64(block), _p(sg) if sg is not None else None,
                               C.c_int64(hd), C.c_int64(nk), C.c_int64(rep))
    return y


def hadamard_inverse(z, block=1024, signs=None):  # src/hadamard.rs:41
    z = _c(z, np.float32)
    y = np.empty_like(z)
    sg = _c(signs, np.float32) if signs is not None else None
    lib().orc_hadamard_inverse(_p(z), _p(y), C.c_int64(z.size), C.c_int64(block), _p(sg) if sg is not None else None)
    return y


def argmax(v):  # src/sampling.rs:50
    v = _c(v, np.float32)
    return int(lib().orc_argmax(_p(v), C.c_int64(v.size)))


# ---- speculative loop ----------------------------------------------------------------------
class _Backend(C.Structure):
    _fields_ = [("user", C.c_void_p),
                ("prefill", C.CFUNCTYPE(C.c_uint32, C.c_void_p, C.POINTER(C.c_uint32), C.c_int64)),
                ("single", C.CFUNCTYPE(C.c_uint32, C.c_void_p, C.c_uint32)),
                ("draft", C.CFUNCTYPE(C.c_uint32, C.c_void_p, C.POINTER(C.c_uint32), C.c_int64)),
                ("verify", C.CFUNCTYPE(None, C.c_void_p, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32))),
                ("reject", C.CFUNCTYPE(None, C.c_void_p)),
                ("reset_all", C.CFUNCTYPE(None, C.c_void_p))]


STAT_NAMES = ("drafted", "accepted", "steps", "draft_calls", "verify_calls", "single_forwards",
              "timed_decode_forwards", "rejected", "terminal_rollbacks")


def greedy_mtp(backend, prompt, n, is_eog=lambda t: False, on_tok=lambda t: True):
    """greedy_mtp (src/mtp.rs:166-204) over a Python backend object with the MtpBackend methods."""
    F = dict(_Backend._fields_)

    def _verify(_, x, d, a0, a1):
        r = backend.mtp_verify(x, d)
        a0[0], a1[0] = r[0], r[1]
    be = _Backend(None,
                  F["prefill"](lambda _, p, k: backend.mtp_prefill([p[i] for i in range(k)])),
                  F["single"](lambda _, x: backend.mtp_single(x)),
                  F["draft"](lambda _, p, k: backend.mtp_draft([p[i] for i in range(k)])),
                  F["verify"](_verify),
                  F["reject"](lambda _: backend.mtp_reject()),
                  F["reset_all"](lambda _: backend.reset_all()))
    CB = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_uint32)
    eog = CB(lambda _, t: int(bool(is_eog(t))))
    tok = CB(lambda _, t: int(bool(on_tok(t))))
    pr = np.asarray(prompt, np.uint32)
    out = np.zeros(max(n, 1) + 2, np.uint32)
    stats = np.zeros(9, np.int64)
    k = lib().orc_greedy_mtp(C.byref(be), _p(pr), C.c_int64(pr.size), C.c_int64(n), eog, tok, None, _p(out), _p(stats))
    if k < 0:
        raise ValueError("empty MTP prompt")
    return [int(t) for t in out[:k]], dict(zip(STAT_NAMES, (int(s) for s in stats)))


# ---- decoder model (oracle_model.cpp) --------------------------------------------------------
REFERENCE_ORDER, DEVICE_ORDER = 0, 1

TENSORS = ("attn_norm", "post_norm", "ffn_gate", "ffn_up", "ffn_down",
           "qkv", "gate", "conv", "dt", "a", "beta", "alpha", "ssm_norm", "ssm_out",
           "q", "k", "v", "o", "q_norm", "k_norm",
           "tok_embd", "output_norm", "output",
           "mtp_eh", "mtp_q", "mtp_k", "mtp_v", "mtp_o", "mtp_gate", "mtp_up", "mtp_down",
           "mtp_enorm", "mtp_hnorm", "mtp_attn_norm", "mtp_post_norm", "mtp_q_norm", "mtp_k_norm", "mtp_head_norm", "mtp_embd")
TENSOR_ID = {n: i for i, n in enumerate(TENSORS)}


class ModelConfig(C.Structure):
    """Field-for-field mirror of it_model_config (include/irontimber_cuda.h); Config of src/model.rs:7-15."""
    _fields_ = [("n_layer", C.c_int32), ("n_embd", C.c_int32), ("n_ff", C.c_int32), ("n_vocab", C.c_int32),
                ("n_head", C.c_int32), ("n_head_kv", C.c_int32), ("head_dim", C.c_int32), ("n_rot", C.c_int32),
                ("rope_base", C.c_float), ("rope_sections", C.c_int32 * 4), ("eps", C.c_float),
                ("conv_k", C.c_int32), ("ssm_state", C.c_int32), ("ssm_groups", C.c_int32), ("ssm_vheads", C.c_int32),
                ("ssm_inner", C.c_int32), ("full_attn_interval", C.c_int32), ("gdn_v_grouped", C.c_int32), ("ctx_len", C.c_int32)]

    def is_recurrent(self, il):
        return (il + 1) % self.full_attn_interval != 0

    @property
    def qk_dim(self):
        return self.ssm_state * self.ssm_groups

    @property
    def conv_dim(self):
        return 2 * self.qk_dim + self.ssm_inner


class Model:
    """Host-memory decoder for the oracle: set tensors by name, then run forward_token / mtp_step."""

    def __init__(self, cfg, nthreads=0):
        L = lib()
        L.orc_model_new.restype = C.c_void_p
        L.orc_state_new.restype = C.c_void_p
        L.orc_state_clone.restype = C.c_void_p
        L.orc_mtp_state_new.restype = C.c_void_p
        L.orc_state_read.restype = C.c_int64
        assert L.orc_model_config_bytes() == C.sizeof(ModelConfig)
        self.cfg = cfg
        self.h = C.c_void_p(L.orc_model_new(C.byref(cfg), C.c_int(nthreads)))

    def set(self, name, data, layer=-1):
        a = np.ascontiguousarray(data)
        lib().orc_model_set(self.h, C.c_int(layer), C.c_int(TENSOR_ID[name]), _p(a), C.c_int64(a.nbytes))

    def set_signs(self, signs):
        s = _c(signs, np.float32)
        lib().orc_model_set_signs(self.h, C.c_int64(s.size), _p(s))

    def new_state(self):
        return C.c_void_p(lib().orc_state_new(self.h))

    def clone_state(self, st):
        return C.c_void_p(lib().orc_state_clone(st))

    def assign_state(self, dst, src):
        lib().orc_state_assign(dst, src)

    def free_state(self, st):
        lib().orc_state_free(st)

    def state_pos(self, st):
        return int(lib().orc_state_pos(st))

    def state_h(self, st):
        out = np.empty(self.cfg.n_embd, np.float32)
        lib().orc_state_h(st, _p(out))
        return out

    def state_read(self, st, layer, which):
        n = lib().orc_state_read(st, C.c_int(layer), C.c_int(which), None)
        out = np.empty(n, np.float32)
        lib().orc_state_read(st, C.c_int(layer), C.c_int(which), _p(out))
        return out

    def forward_token(self, st, tok, want_logits=True, mode=REFERENCE_ORDER):
        """Model::forward_token (src/cpu.rs:168)."""
        lg = np.empty(self.cfg.n_vocab, np.float32) if want_logits else None
        lib().orc_forward_token(self.h, st, C.c_uint32(tok), _p(lg) if want_logits else None, C.c_int(mode))
        return lg

    def new_mtp_state(self):
        return C.c_void_p(lib().orc_mtp_state_new())

    def mtp_step(self, ms, h, tok, pos, mode=REFERENCE_ORDER):
        """cpu_step (src/mtp.rs:100)."""
        h = _c(h, np.float32)
        lg = np.empty(self.cfg.n_vocab, np.float32)
        lib().orc_mtp_step(self.h, ms, _p(h), C.c_uint32(tok), C.c_int(pos), _p(lg), C.c_int(mode))
        return lg

    def mtp_step_hidden(self, ms, h, tok, pos, mode=REFERENCE_ORDER):
        """cpu_step that also returns the head's hidden state before head_norm (input of a chained draft step)."""
        h = _c(h, np.float32)
        lg = np.empty(self.cfg.n_vocab, np.float32)
        hid = np.empty(self.cfg.n_embd, np.float32)
        lib().orc_mtp_step_hidden(self.h, ms, _p(h), C.c_uint32(tok), C.c_int(pos), _p(lg), C.c_int(mode), _p(hid))
        return lg, hid

    def close(self):
        if self.h:
            lib().orc_model_free(self.h)
            self.h = None


class CpuMtp:
    """CpuMtp (src/mtp.rs:207-236): the reference's CPU speculative backend over the oracle model."""

    def __init__(self, model, mode=REFERENCE_ORDER):
        self.m, self.mode = model, mode
        self.reset_all()

    def reset_all(self):
        self.st = self.m.new_state(); self.ck = None; self.ms = self.m.new_mtp_state(); self.hpend = []; self.mpos = 1

    def mtp_single(self, x):
        return argmax(self.m.forward_token(self.st, x, True, self.mode))

    def mtp_prefill(self, prompt):
        self.reset_all()
        hs, lg = [], None
        for i, t in enumerate(prompt):
            lg = self.m.forward_token(self.st, t, i + 1 == len(prompt), self.mode)
            hs.append(self.m.state_h(self.st))
        for q in range(1, len(prompt)):
            self.m.mtp_step(self.ms, hs[q - 1], prompt[q], q, self.mode)
        self.mpos = len(prompt); self.hpend = [hs[-1]]
        return argmax(lg)

    def mtp_draft(self, toks):
        assert len(toks) == len(self.hpend)
        lg = None
        for i, t in enumerate(toks):
            lg = self.m.mtp_step(self.ms, self.hpend[i], t, self.mpos, self.mode); self.mpos += 1
        return argmax(lg)

    def mtp_verify(self, x, d):
        l0 = self.m.forward_token(self.st, x, True, self.mode); h0 = self.m.state_h(self.st)
        self.ck = self.m.clone_state(self.st)
        l1 = self.m.forward_token(self.st, d, True, self.mode); h1 = self.m.state_h(self.st)
        self.hpend = [h0, h1]
        return argmax(l0), argmax(l1)

    def mtp_reject(self):
        self.m.assign_state(self.st, self.ck); self.ck = None; self.hpend = self.hpend[:1]

    # ---- draft length k > 1.  The reference defines k = 1 only (src/mtp.rs:3-8: the head consumes the trunk's hidden state
    # of the previous position, which does not exist for a drafted position).  Extension used here and in the CUDA engine:
    # draft i >= 2 feeds the head its OWN hidden state before head_norm, with draft i - 1 as the token, one position on; its
    # KV entry is provisional (the next real pair at that position replaces it).  Verification runs the k + 1 rows
    # [x, d_1 .. d_k] through the trunk with a state copy after every row; the longest prefix with pick_{i-1} == d_i is kept.
    def mtp_draft_k(self, toks, k):
        assert len(toks) == len(self.hpend) and k >= 1
        lg = hid = None
        for i, t in enumerate(toks):
            lg, hid = self.m.mtp_step_hidden(self.ms, self.hpend[i], t, self.mpos, self.mode); self.mpos += 1
        drafts = [argmax(lg)]
        for i in range(1, k):
            lg, hid = self.m.mtp_step_hidden(self.ms, hid, drafts[-1], self.mpos + i - 1, self.mode)
            drafts.append(argmax(lg))
        return drafts

    def mtp_verify_k(self, x, drafts):
        picks, self.hs, self.cks = [], [], []
        for i, t in enumerate([x] + list(drafts)):
            lg = self.m.forward_token(self.st, t, True, self.mode)
            picks.append(argmax(lg)); self.hs.append(self.m.state_h(self.st))
            if i < len(drafts):
                self.cks.append(self.m.clone_state(self.st))
        self.hpend = list(self.hs)
        return picks

    def mtp_rollback(self, keep_rows):
        """Keeps the first keep_rows rows of the last verification (1 <= keep_rows <= k + 1)."""
        if keep_rows <= len(self.cks):
            self.m.assign_state(self.st, self.cks[keep_rows - 1])
        self.hpend = self.hs[:keep_rows]
        for ck in self.cks:
            self.m.free_state(ck)
        self.cks = []


def greedy_mtp_k(backend, prompt, n, k, is_eog=lambda t: False):
    """Speculative greedy loop with draft length k (k = 1 gives greedy_mtp's token list and counters, src/mtp.rs:166-204)."""
    st = dict.fromkeys(STAT_NAMES, 0)
    out = []
    if n == 0:
        return out, st
    if not len(prompt):
        raise ValueError("empty MTP prompt")

    def emit(t):
        out.append(t)
        return not is_eog(t) and len(out) < n
    x = backend.mtp_prefill(list(prompt))
    if not emit(x):
        return out, st
    pending = [x]
    while True:
        if n - len(out) == 1:
            a = backend.mtp_single(x); st["single_forwards"] += 1; st["timed_decode_forwards"] += 1; emit(a); break
        kk = min(k, n - len(out) - 1)
        ds = backend.mtp_draft_k(pending, kk); st["draft_calls"] += 1
        picks = backend.mtp_verify_k(x, ds)
        st["drafted"] += kk; st["steps"] += 1; st["verify_calls"] += 1; st["timed_decode_forwards"] += kk + 1
        nacc = 0
        while nacc < kk and picks[nacc] == ds[nacc]:
            nacc += 1
        st["accepted"] += nacc; st["rejected"] += kk - nacc
        stop = False
        for i in range(nacc):
            if not emit(ds[i]):
                backend.mtp_rollback(i + 1); st["terminal_rollbacks"] += 1; stop = True; break
        if stop:
            break
        backend.mtp_rollback(nacc + 1)
        if not emit(picks[nacc]):
            break
        x = picks[nacc]; pending = ds[:nacc] + [picks[nacc]]
    return out, st


def generate_greedy(model, prompt, n, mode=REFERENCE_ORDER):
    """generate_inner's greedy path (src/engine.rs:151-174): prefill token by token, then n greedy tokens."""
    st = model.new_state()
    lg = None
    for i, t in enumerate(prompt):
        lg = model.forward_token(st, t, i + 1 == len(prompt), mode)
    out = []
    for _ in range(n):
        t = argmax(lg)
        out.append(t)
        if len(out) == n:
            break
        lg = model.forward_token(st, t, True, mode)
    model.free_state(st)
    return out
