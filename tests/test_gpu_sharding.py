"""Row-sharded ternary products on the GPU.

On one GPU the shard code path (row map, pushes through the peer table, the end-of-kernel handshake) runs with the
context attached to itself; with two or more GPUs one process per GPU runs the real exchange over peer memory and the
results must equal the single-GPU ones bit for bit.
"""
import numpy as np
import pytest

from tests.util import bits, synth_pq2, tiny_config

pytestmark = pytest.mark.gpu


def _gpus():
    import torch
    return torch.cuda.device_count()


@pytest.mark.parametrize("rows,cols,ntok,acc", [(1024, 1024, 1, False), (1000, 2048, 3, True), (4096, 5120, 1, True), (2048, 1024, 40, False), (192, 1024, 70, True)])
def test_shards_on_one_gpu_fill_the_full_output(orc, rows, cols, ntok, acc):
    from irontimber_b200.backend import CudaBackend
    be = CudaBackend(0, arena_floats=1 << 22)
    try:
        be.attach_peers(0, 1)
        rng = np.random.default_rng(rows + ntok)
        raw = synth_pq2(77, rows, cols)
        cut = (rows // 2 + 31) // 32 * 32 if rows % 64 else rows // 2
        rb = raw.reshape(rows, -1)
        parts = [be.mat_shard(np.ascontiguousarray(rb[:cut]).reshape(-1), cut, cols, 0, rows),
                 be.mat_shard(np.ascontiguousarray(rb[cut:]).reshape(-1), rows - cut, cols, cut, rows)]
        synth = [be.mat_synth_rows(77, rows, cols, 0, cut), be.mat_synth_rows(77, rows, cols, cut, rows - cut)]
        for a, b in zip(parts, synth):                       # generated rows == uploaded rows of the full matrix
            assert np.array_equal(a.download_pq2(), b.download_pq2())
        X = rng.standard_normal((ntok, cols)).astype(np.float32)
        y0 = rng.standard_normal(ntok * rows).astype(np.float32)
        yo = ((ntok * cols + 63) // 64) * 64
        q = be.q8_rows(cols, ntok)
        be.upload(0, X); be.upload(yo, y0)
        be.had_q8(cols, ntok, 0, cols, q, signs=False, rotate=False)
        for m in synth:
            be.mv(m, ntok, q, yo, rows, acc=acc)
        got = be.download(yo, ntok * rows).reshape(ntok, rows)
        for t in range(ntok):
            want = orc.matvec_ternary(raw, rows, cols, X[t])
            if acc:
                want = y0.reshape(ntok, rows)[t] + want
            assert np.array_equal(bits(got[t]), bits(want))
        for m in parts + synth:
            m.close()
        q.close()
    finally:
        be.close()


@pytest.mark.parametrize("rows,cols,ntok,acc", [(1000, 1024, 1, False), (4096, 5120, 3, True)])
def test_q8_shards_on_one_gpu_equal_the_full_matrix(rows, cols, ntok, acc):
    """Int8-group matvec (the NextN head / q8 LM head kind) on row shards: same bits as the unsharded launch."""
    from irontimber_b200.backend import CudaBackend
    be = CudaBackend(0, arena_floats=1 << 22)
    try:
        be.attach_peers(0, 1)
        rng = np.random.default_rng(rows)
        full = be.qmat_synth(31, rows, cols)
        cut = rows // 2
        parts = [be.qmat_synth_rows(31, rows, cols, 0, cut), be.qmat_synth_rows(31, rows, cols, cut, rows - cut)]
        raw = full.download_q8_0().reshape(rows, -1)
        assert np.array_equal(parts[0].download_q8_0().reshape(cut, -1), raw[:cut])
        assert np.array_equal(parts[1].download_q8_0().reshape(rows - cut, -1), raw[cut:])
        X = rng.standard_normal((ntok, cols)).astype(np.float32)
        y0 = rng.standard_normal(ntok * rows).astype(np.float32)
        yo = ((ntok * cols + 63) // 64) * 64
        be.upload(0, X); be.upload(yo, y0)
        be.mvq(full, ntok, 0, cols, yo, rows, acc=acc)
        want = be.download(yo, ntok * rows)
        be.upload(yo, y0)
        for m in parts:
            be.mvq(m, ntok, 0, cols, yo, rows, acc=acc)
        got = be.download(yo, ntok * rows)
        assert np.array_equal(bits(got), bits(want))
        for m in parts + [full]:
            m.close()
    finally:
        be.close()


def test_shard_without_peers_is_refused():
    from irontimber_b200 import _lib
    from irontimber_b200.backend import CudaBackend
    be = CudaBackend(0, arena_floats=1 << 20)
    try:
        w = be.mat_synth_rows(5, 512, 1024, 256, 256)
        q = be.q8_rows(1024, 1)
        be.upload(0, np.ones(1024, np.float32))
        be.had_q8(1024, 1, 0, 1024, q, signs=False, rotate=False)
        with pytest.raises(_lib.IronTimberError):
            be.mv(w, 1, q, 2048, 512)
        w.close(); q.close()
    finally:
        be.close()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("rows,cols,ntok,acc", [(4096, 5120, 1, False), (2048, 1024, 3, True), (2048, 2048, 40, False)])
def test_two_gpus_sharded_matvec_bit_exact(orc, rows, cols, ntok, acc):
    if _gpus() < 2:
        pytest.skip("needs two GPUs")
    from tests.mp_workers import gpu_sharded_matvec, run_ranks
    res = run_ranks(gpu_sharded_matvec, 2, 99, rows, cols, ntok, acc)
    raw = synth_pq2(99, rows, cols)
    for X, y0, got in res:                                    # every rank holds the full result
        for t in range(ntok):
            want = orc.matvec_ternary(raw, rows, cols, X[t])
            if acc:
                want = y0.reshape(ntok, rows)[t] + want
            assert np.array_equal(bits(got[t]), bits(want))


@pytest.mark.timeout(900)
def test_two_gpus_sharded_engine_equals_single_gpu():
    if _gpus() < 2:
        pytest.skip("needs two GPUs")
    from irontimber_b200.engine import CudaEngine, ModelConfig
    from tests.mp_workers import gpu_sharded_engine, run_ranks
    prompt = [int(t) for t in np.random.default_rng(4).integers(0, 1000, 70)]      # one pass of 64 rows and one of 6
    eng = CudaEngine(tiny_config(ModelConfig, n_layer=4, ctx_len=128), seed=11, with_mtp=True)
    try:
        lg = eng.eval(prompt); eng.reset()
        hist = eng.generate(prompt, 12)
        spec = eng.generate_mtp(prompt, 12)
    finally:
        eng.close()
    for lg_r, hist_r, spec_r in run_ranks(gpu_sharded_engine, 2, 4, prompt, 12, True):
        assert np.array_equal(bits(lg_r), bits(lg))
        assert hist_r == hist and spec_r == spec


def test_model_file_loaded_as_row_shards_matches_single_gpu(tmp_path, orc):
    """Two ranks load their rows of the same GGUF file (PQ2_0 and PTQ1_0 matrices, Q6_K / Q8_0 head in a sidecar): logits and
    token histories equal the single-GPU engine built from the file."""
    if _gpus() < 2:
        pytest.skip("needs two GPUs")
    from irontimber_b200.engine import CudaEngine, ModelConfig
    from tests import gguf_writer as W
    from tests.mp_workers import gpu_sharded_gguf_engine, run_ranks
    from tests.test_gguf import dequant
    from tests.util import tensor_shapes
    cfg = tiny_config(ModelConfig, n_layer=4, ctx_len=128)
    tk, tt, hk, ht, _ = W.build_model(np.random.default_rng(21), cfg, tensor_shapes(cfg), dequant, lambda z, s: orc.hadamard_inverse(z, 1024, s),
                                      head="sidecar", head_embd=True, head_type="mixed")
    trunk, head = str(tmp_path / "trunk.gguf"), str(tmp_path / "head.gguf")
    W.write_gguf(trunk, tk, tt); W.write_gguf(head, hk, ht)
    prompt = [int(t) for t in np.random.default_rng(4).integers(0, 1000, 70)]
    eng = CudaEngine.from_gguf(trunk, head, ctx_len=128)
    try:
        lg = eng.eval(prompt); eng.reset()
        hist = eng.generate(prompt, 12)
        spec = eng.generate_mtp(prompt, 12)
    finally:
        eng.close()
    for lg_r, hist_r, spec_r in run_ranks(gpu_sharded_gguf_engine, 2, trunk, head, prompt, 12):
        assert np.array_equal(bits(lg_r), bits(lg))
        assert hist_r == hist and spec_r == spec
