"""CPU-only checks of the drop-in boundary: the library loads, exports every symbol the header
declares, and rejects bad calls before touching a device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from irontimber_b200 import build, _lib
    build.build()
    return _lib.load()


def header_symbols():
    src = open(os.path.join(ROOT, "include", "irontimber_cuda.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(it_[a-z0-9_]+)\s*\(", src)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    from irontimber_b200 import _lib
    names = header_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes table and header disagree"


def test_calls_fail_cleanly_without_a_device_or_with_bad_arguments(lib):
    h = C.c_void_p()
    assert lib.it_ctx_create(0, 1000, C.byref(h)) != 0          # not a multiple of 64, or no device: never a crash
    assert lib.it_last_error()
    assert lib.it_ctx_create(0, 1024, None) == -1
    assert lib.it_sync(None) == -1
    assert lib.it_argmax(None, 0, 1, 2) == -1
    assert lib.it_matvec_t2(None, None, 1, None, 0, 0, 0) == -1
    assert lib.it_arena_write(None, 0, None, 0) == -1
    lib.it_ctx_destroy(None); lib.it_matrix_destroy(None); lib.it_qmatrix_destroy(None); lib.it_q8_destroy(None)


def test_context_capacity_beyond_the_attention_kernel_is_refused_before_device_work(lib):
    """The attention kernel keeps a row of scores in shared memory, so the engine refuses a context capacity it could
    not serve (about 23 k positions at head dimension 256) when it is built, with the limit in the message."""
    from irontimber_b200.engine import config_27b
    h = C.c_void_p()
    cfg = config_27b(n_layer=4, ctx_len=24000, n_vocab=2048)
    assert lib.it_engine_create_synth(0, C.byref(cfg), 1, 0, C.byref(h)) == -1
    msg = lib.it_last_error().decode()
    assert "context capacity 24000" in msg and "23292" in msg


def test_rust_sys_crate_declares_exactly_the_headers_entry_points():
    """ffi/irontimber-cuda-sys/src/lib.rs (not compiled here: no Rust toolchain) must bind every entry point of the
    header and nothing else, so that it cannot drift from the library."""
    src = open(os.path.join(ROOT, "ffi", "irontimber-cuda-sys", "src", "lib.rs")).read()
    block = src[src.index('extern "C" {'):]
    block = block[:block.index("\n}\n")]
    names = sorted(set(re.findall(r"pub fn (it_[a-z0-9_]+)\s*\(", block)))
    assert names == header_symbols()
    # and the engine wrapper only calls what the crate declares
    eng = open(os.path.join(ROOT, "ffi", "cuda_engine.rs")).read()
    assert set(re.findall(r"sys::(it_[a-z0-9_]+)\s*\(", eng)) <= set(names)
