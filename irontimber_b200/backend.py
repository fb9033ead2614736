"""Host-side mirror of the reference's GPU op dispatchers over the C ABI.

`CudaBackend` stands where `VkEngine`'s private dispatchers stand in the reference
(src/vk/mod.rs): `mv` (:653), `mvq` (:742), `had` (:749) and the argmax dispatch (:866), with the
same argument meaning - element offsets into one f32 arena, per-token strides, an `acc` flag.
The one structural difference follows the reference's CPU numerics (src/cpu.rs:30): the forward
Hadamard is fused with q8k quantisation and `mv` consumes the quantised rows.

Everything here is ctypes plumbing; all arithmetic runs in libirontimber_cuda.so on the GPU.
"""
import ctypes as C

import numpy as np

from . import _lib

NONE = None


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


class TernaryMatrix:
    """Device-resident PQ2_0 matrix (DevMat, src/vk/mod.rs:459)."""

    def __init__(self, backend, handle):
        self.backend, self.handle = backend, handle
        L = _lib.load()
        self.rows, self.cols = int(L.it_matrix_rows(handle)), int(L.it_matrix_cols(handle))
        self.device_bytes = int(L.it_matrix_device_bytes(handle))

    def download_pq2(self):
        raw = np.empty(self.rows * (self.cols // 128) * 34, np.uint8)
        _lib.check(_lib.load().it_matrix_download_pq2(self.backend.ctx, self.handle, _ptr(raw)))
        return raw

    def close(self):
        if self.handle:
            _lib.load().it_matrix_destroy(self.handle)
            self.handle = None


class Q8Matrix:
    """Device-resident int8-group matrix of the MTP head (Q8G16, src/quant.rs:234)."""

    def __init__(self, backend, handle):
        self.backend, self.handle = backend, handle
        L = _lib.load()
        self.rows, self.cols = int(L.it_qmatrix_rows(handle)), int(L.it_qmatrix_cols(handle))

    def download_q8_0(self):
        raw = np.empty(self.rows * (self.cols // 32) * 34, np.uint8)
        _lib.check(_lib.load().it_qmatrix_download_q8_0(self.backend.ctx, self.handle, _ptr(raw)))
        return raw

    def close(self):
        if self.handle:
            _lib.load().it_qmatrix_destroy(self.handle)
            self.handle = None


class Q8Rows:
    """Device-resident q8k-quantised activation rows (Q8K, src/quant.rs:68)."""

    def __init__(self, backend, max_n, max_tok):
        self.backend, self.max_n, self.max_tok = backend, max_n, max_tok
        h = C.c_void_p()
        _lib.check(_lib.load().it_q8_create(backend.ctx, max_n, max_tok, C.byref(h)))
        self.handle = h
        self.n = 0

    def read(self, tok=0):
        n = self.n
        qs, d, s = np.empty(n, np.int8), np.empty(n // 256, np.float32), np.empty(n // 128, np.int32)
        _lib.check(_lib.load().it_q8_read(self.backend.ctx, self.handle, tok, _ptr(qs), _ptr(d), _ptr(s)))
        return d, qs, s

    def close(self):
        if self.handle:
            _lib.load().it_q8_destroy(self.handle)
            self.handle = None


class CudaBackend:
    def __init__(self, device=0, arena_floats=1 << 22):
        self.L = _lib.load()
        h = C.c_void_p()
        _lib.check(self.L.it_ctx_create(device, arena_floats, C.byref(h)))
        self.ctx = h
        self.arena_floats = arena_floats
        self.device = device

    def close(self):
        if self.ctx:
            self.L.it_ctx_destroy(self.ctx)
            self.ctx = None

    # ---- arena -------------------------------------------------------------------------------
    def upload(self, off, data):
        a = np.ascontiguousarray(data)
        assert a.dtype.itemsize == 4
        _lib.check(self.L.it_arena_write(self.ctx, off, _ptr(a), a.size))

    def download(self, off, n, dtype=np.float32):
        out = np.empty(n, dtype)
        _lib.check(self.L.it_arena_read(self.ctx, off, _ptr(out), n))
        return out

    def zero(self, off, n):
        _lib.check(self.L.it_arena_zero(self.ctx, off, n))

    def sync(self):
        _lib.check(self.L.it_sync(self.ctx))

    @property
    def stream(self):
        return self.L.it_ctx_stream(self.ctx)

    @property
    def arena_ptr(self):
        return self.L.it_arena_ptr(self.ctx)

    # ---- graphs (one recorded command sequence, replayed with one launch) -------------------------
    def capture_begin(self):
        _lib.check(self.L.it_capture_begin(self.ctx))

    def capture_end(self):
        h = C.c_void_p()
        _lib.check(self.L.it_capture_end(self.ctx, C.byref(h)))
        return h

    def graph_launch(self, g):
        _lib.check(self.L.it_graph_launch(self.ctx, g))

    def graph_destroy(self, g):
        self.L.it_graph_destroy(g)

    # ---- weights -------------------------------------------------------------------------------
    def mat(self, raw_pq2, rows, cols):
        raw = np.ascontiguousarray(raw_pq2, np.uint8)
        if raw.size != rows * (cols // 128) * 34:
            raise ValueError("raw PQ2_0 size does not match the shape")
        h = C.c_void_p()
        _lib.check(self.L.it_matrix_upload_pq2(self.ctx, _ptr(raw), rows, cols, C.byref(h)))
        return TernaryMatrix(self, h)

    def mat_packed2(self, words, scales, rows, cols):
        w, s = np.ascontiguousarray(words, np.uint32), np.ascontiguousarray(scales, np.float32)
        h = C.c_void_p()
        _lib.check(self.L.it_matrix_upload_packed2(self.ctx, _ptr(w), _ptr(s), rows, cols, C.byref(h)))
        return TernaryMatrix(self, h)

    def mat_synth(self, seed, rows, cols, four_codes=False):
        h = C.c_void_p()
        _lib.check(self.L.it_matrix_synth(self.ctx, seed, rows, cols, int(four_codes), C.byref(h)))
        return TernaryMatrix(self, h)

    def mat_synth_rows(self, seed, total_rows, cols, row0, nrows, four_codes=False):
        """Rows [row0, row0 + nrows) of the synthetic matrix (seed, total_rows, cols), marked as a row shard."""
        h = C.c_void_p()
        _lib.check(self.L.it_matrix_synth_rows(self.ctx, seed, total_rows, cols, int(four_codes), row0, nrows, C.byref(h)))
        return TernaryMatrix(self, h)

    def mat_shard(self, raw_pq2, nrows, cols, row0, total_rows):
        """Uploaded rows [row0, row0 + nrows) of a logical matrix of total_rows rows."""
        m = self.mat(raw_pq2, nrows, cols)
        _lib.check(self.L.it_matrix_set_shard(m.handle, row0, total_rows))
        return m

    # ---- peers (one process per GPU) ----------------------------------------------------------------
    def attach_peers(self, rank=0, world=1, group=None):
        from .sharding import attach_peers
        attach_peers(self.L, self.ctx, rank, world, group)

    def attach_peers_local(self, rank, backends):
        """Peers that live in this process (one CudaBackend per rank, in rank order): it_ctx_attach_peers_local."""
        arr = (C.c_void_p * len(backends))(*[b.ctx for b in backends])
        _lib.check(self.L.it_ctx_attach_peers_local(self.ctx, rank, len(backends), arr))

    def set_peer_wait_us(self, microseconds):
        _lib.check(self.L.it_ctx_set_peer_wait_us(self.ctx, float(microseconds)))

    def qmat(self, raw_q8_0, rows, cols):
        raw = np.ascontiguousarray(raw_q8_0, np.uint8)
        if raw.size != rows * (cols // 32) * 34:
            raise ValueError("raw Q8_0 size does not match the shape")
        h = C.c_void_p()
        _lib.check(self.L.it_qmatrix_upload_q8_0(self.ctx, _ptr(raw), rows, cols, C.byref(h)))
        return Q8Matrix(self, h)

    def qmat_synth_rows(self, seed, total_rows, cols, row0, nrows):
        """Rows [row0, row0 + nrows) of the synthetic int8-group matrix (seed, total_rows, cols), marked as a row shard."""
        h = C.c_void_p()
        _lib.check(self.L.it_qmatrix_synth_rows(self.ctx, seed, total_rows, cols, row0, nrows, C.byref(h)))
        return Q8Matrix(self, h)

    def qmat_synth(self, seed, rows, cols):
        h = C.c_void_p()
        _lib.check(self.L.it_qmatrix_synth(self.ctx, seed, rows, cols, C.byref(h)))
        return Q8Matrix(self, h)

    def set_signs(self, signs):
        s = np.ascontiguousarray(signs, np.float32)
        _lib.check(self.L.it_signs_set(self.ctx, s.size, _ptr(s)))

    def q8_rows(self, max_n, max_tok=1):
        return Q8Rows(self, max_n, max_tok)

    # ---- ops (argument order of the reference's dispatchers) -----------------------------------------
    def had_q8(self, n, ntok, io, its, out, perm=None, signs=True, rotate=True):
        """had (src/vk/mod.rs:749) fused with quantize_q8k (src/quant.rs:75): rows -> `out` (Q8Rows)."""
        hd, nk, rep = perm if perm else (0, 0, 0)
        _lib.check(self.L.it_hadamard_q8(self.ctx, n, ntok, io, its, int(rotate), int(signs), hd, nk, rep, out.handle))
        out.n = n

    def had(self, n, ntok, io, its, oo, ots, perm=None, inverse=False, signs=True):
        """had (src/vk/mod.rs:749) with an f32 destination in the arena."""
        hd, nk, rep = perm if perm else (0, 0, 0)
        _lib.check(self.L.it_hadamard_f32(self.ctx, n, ntok, io, its, oo, ots, int(signs), hd, nk, rep, int(inverse)))

    def mv(self, w, ntok, x, yo, ys, acc=False):
        """mv (src/vk/mod.rs:653): y[t, :] (+)= W x[t] for ntok quantised rows of `x`."""
        _lib.check(self.L.it_matvec_t2(self.ctx, w.handle, ntok, x.handle, yo, ys, int(acc)))

    def mv_sumi(self, w, ntok, x):
        """Integer accumulators of `mv` per (token, row, block); test hook."""
        import torch
        out = torch.empty((ntok, w.rows, w.cols // 128), dtype=torch.int32, device=f"cuda:{self.device}")
        self.sync()
        _lib.check(self.L.it_matvec_t2_sumi(self.ctx, w.handle, ntok, x.handle, C.c_void_p(out.data_ptr())))
        self.sync()
        return out.cpu().numpy()

    def mvq(self, w, ntok, xo, xs, yo, ys, acc=False):
        """mvq (src/vk/mod.rs:742)."""
        _lib.check(self.L.it_matvec_q8(self.ctx, w.handle, ntok, xo, xs, yo, ys, int(acc)))

    def argmax(self, off, n, dst):
        """argmax dispatch (src/vk/mod.rs:866): stores the u32 index bit-cast into arena[dst]."""
        _lib.check(self.L.it_argmax(self.ctx, off, n, dst))

    def read_u32(self, off):
        return int(self.download(off, 1, np.uint32)[0])
