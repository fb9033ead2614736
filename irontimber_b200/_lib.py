"""Loads libirontimber_cuda.so and declares the C ABI of include/irontimber_cuda.h.

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libirontimber_cuda.so")

c_size = C.c_size_t
P = C.c_void_p

# name -> (restype, argtypes); mirrors include/irontimber_cuda.h one to one
SIGNATURES = {
    "it_last_error": (C.c_char_p, []),
    "it_version": (C.c_int, []),
    "it_ctx_create": (C.c_int, [C.c_int, c_size, C.POINTER(P)]),
    "it_ctx_destroy": (None, [P]),
    "it_sync": (C.c_int, [P]),
    "it_ctx_stream": (P, [P]),
    "it_arena_ptr": (P, [P]),
    "it_arena_floats": (c_size, [P]),
    "it_arena_write": (C.c_int, [P, c_size, P, c_size]),
    "it_arena_read": (C.c_int, [P, c_size, P, c_size]),
    "it_arena_zero": (C.c_int, [P, c_size, c_size]),
    "it_capture_begin": (C.c_int, [P]),
    "it_capture_end": (C.c_int, [P, C.POINTER(P)]),
    "it_graph_launch": (C.c_int, [P, P]),
    "it_graph_destroy": (None, [P]),
    "it_graph_kernel_nodes": (C.c_int, [P]),
    "it_signs_set": (C.c_int, [P, c_size, P]),
    "it_matrix_upload_pq2": (C.c_int, [P, P, c_size, c_size, C.POINTER(P)]),
    "it_matrix_upload_packed2": (C.c_int, [P, P, P, c_size, c_size, C.POINTER(P)]),
    "it_matrix_synth": (C.c_int, [P, C.c_uint64, c_size, c_size, C.c_int, C.POINTER(P)]),
    "it_shard_range": (C.c_int, [c_size, C.c_int, C.c_int, C.POINTER(c_size), C.POINTER(c_size)]),
    "it_matrix_set_shard": (C.c_int, [P, c_size, c_size]),
    "it_matrix_synth_rows": (C.c_int, [P, C.c_uint64, c_size, c_size, C.c_int, c_size, c_size, C.POINTER(P)]),
    "it_qmatrix_set_shard": (C.c_int, [P, c_size, c_size]),
    "it_qmatrix_synth_rows": (C.c_int, [P, C.c_uint64, c_size, c_size, c_size, c_size, C.POINTER(P)]),
    "it_ctx_ipc_handle": (C.c_int, [P, P]),
    "it_ctx_attach_peers": (C.c_int, [P, C.c_int, C.c_int, P]),
    "it_ctx_world": (C.c_int, [P]),
    "it_ctx_attach_peers_local": (C.c_int, [P, C.c_int, C.c_int, P]),
    "it_ctx_set_peer_wait_us": (C.c_int, [P, C.c_double]),
    "it_matrix_download_pq2": (C.c_int, [P, P, P]),
    "it_matrix_rows": (c_size, [P]),
    "it_matrix_cols": (c_size, [P]),
    "it_matrix_device_bytes": (c_size, [P]),
    "it_matrix_destroy": (None, [P]),
    "it_qmatrix_upload_q8_0": (C.c_int, [P, P, c_size, c_size, C.POINTER(P)]),
    "it_qmatrix_synth": (C.c_int, [P, C.c_uint64, c_size, c_size, C.POINTER(P)]),
    "it_qmatrix_download_q8_0": (C.c_int, [P, P, P]),
    "it_qmatrix_rows": (c_size, [P]),
    "it_qmatrix_cols": (c_size, [P]),
    "it_qmatrix_destroy": (None, [P]),
    "it_q8_create": (C.c_int, [P, c_size, c_size, C.POINTER(P)]),
    "it_q8_destroy": (None, [P]),
    "it_q8_read": (C.c_int, [P, P, c_size, P, P, P]),
    "it_hadamard_q8": (C.c_int, [P, c_size, c_size, c_size, c_size, C.c_int, C.c_int, c_size, c_size, c_size, P]),
    "it_hadamard_f32": (C.c_int, [P, c_size, c_size, c_size, c_size, c_size, c_size, C.c_int, c_size, c_size, c_size, C.c_int]),
    "it_matvec_t2": (C.c_int, [P, P, c_size, P, c_size, c_size, C.c_int]),
    "it_matvec_t2_sumi": (C.c_int, [P, P, c_size, P, P]),
    "it_matvec_q8": (C.c_int, [P, P, c_size, c_size, c_size, c_size, c_size, C.c_int]),
    "it_argmax": (C.c_int, [P, c_size, c_size, c_size]),
    "it_argmax_static": (C.c_int, [P, P, c_size, P]),
    "it_engine_create_synth": (C.c_int, [C.c_int, P, C.c_uint64, C.c_int, C.POINTER(P)]),
    "it_engine_create_synth_sharded": (C.c_int, [C.c_int, P, C.c_uint64, C.c_int, C.c_int, C.c_int, C.POINTER(P)]),
    "it_qmatrix_upload_q6_k": (C.c_int, [P, P, c_size, c_size, C.POINTER(P)]),
    "it_qmatrix_download_g16": (C.c_int, [P, P, P]),
    "it_qmatrix_group16": (C.c_int, [P]),
    "it_engine_create_gguf": (C.c_int, [C.c_int, C.c_char_p, C.c_char_p, C.c_int, C.c_int, C.c_int, C.POINTER(P)]),
    "it_gguf_inspect": (C.c_int, [C.c_char_p, C.c_char_p, C.c_int, P, C.POINTER(C.c_int), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "it_gguf_dequant": (C.c_int, [C.c_uint32, P, c_size, P]),
    "it_gguf_ptq1_to_pq2": (C.c_int, [P, c_size, P]),
    "it_engine_destroy": (None, [P]),
    "it_engine_ctx": (P, [P]),
    "it_engine_tensor_bytes": (C.c_int, [P, C.c_int, C.c_int, C.POINTER(c_size)]),
    "it_engine_tensor_read": (C.c_int, [P, C.c_int, C.c_int, P]),
    "it_engine_signs_read": (C.c_int, [P, c_size, P]),
    "it_engine_state_read": (C.c_int, [P, C.c_int, C.c_int, P, c_size, C.POINTER(c_size)]),
    "it_engine_hidden_read": (C.c_int, [P, c_size, P]),
    "it_engine_position": (C.c_int, [P]),
    "it_engine_eval": (C.c_int, [P, P, c_size, P]),
    "it_engine_eval_argmax": (C.c_int, [P, P, c_size, C.POINTER(C.c_uint32)]),
    "it_engine_reset": (C.c_int, [P]),
    "it_engine_generate": (C.c_int, [P, P, c_size, c_size, C.c_uint32, P, C.POINTER(c_size)]),
    "it_engine_decode_steps": (C.c_int, [P, c_size, C.POINTER(C.c_uint32)]),
    "it_engine_step_kernels": (C.c_int, [P]),
    "it_engine_step_trace": (C.c_int, [P, P, c_size]),
    "it_engine_mtp_prefill": (C.c_int, [P, P, c_size, C.POINTER(C.c_uint32)]),
    "it_engine_mtp_single": (C.c_int, [P, C.c_uint32, C.POINTER(C.c_uint32)]),
    "it_engine_mtp_draft": (C.c_int, [P, P, c_size, C.POINTER(C.c_uint32)]),
    "it_engine_mtp_verify": (C.c_int, [P, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
    "it_engine_mtp_reject": (C.c_int, [P]),
    "it_engine_mtp_reset_all": (C.c_int, [P]),
    "it_greedy_mtp": (C.c_int64, [P, P, c_size, c_size, P, P, P, P, P]),
    "it_engine_generate_mtp": (C.c_int64, [P, P, c_size, c_size, C.c_uint32, P, P]),
    "it_engine_mtp_draft_k": (C.c_int, [P, P, c_size, c_size, P]),
    "it_engine_mtp_verify_k": (C.c_int, [P, C.c_uint32, P, c_size, P]),
    "it_engine_mtp_rollback": (C.c_int, [P, c_size]),
    "it_greedy_mtp_k": (C.c_int64, [P, c_size, P, c_size, c_size, P, P, P, P, P]),
    "it_engine_generate_mtp_k": (C.c_int64, [P, c_size, P, c_size, c_size, C.c_uint32, P, P]),
}

_lib = None


class IronTimberError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"irontimber_cuda error {code}: {msg}")
        self.code = code


def load():
    """Returns the loaded library; raises if it has not been built (python -m irontimber_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m irontimber_b200.build`")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)   # AttributeError if the header and the library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(code):
    if code != 0:
        raise IronTimberError(code, load().it_last_error().decode("utf-8", "replace"))
