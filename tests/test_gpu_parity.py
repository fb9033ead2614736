"""GPU parity: every kernel of the hot path, called through the C ABI, against the CPU oracle.

Bit-exact for weight decode, q8k quantisation, integer accumulators and the ternary matvec's f32
output; 1e-4 scaled (the reference's own kernel-parity tolerance, src/vk/kparity.rs:3) for the
f32-activation int8-group matvec, whose summation order differs from the CPU's.
Fixture recipe follows src/vk/kparity.rs:18-46,71-73: M in {999, 1000, 1001}, K = 1024,
ntok in {1,2,3,5,7,11,13,21}, accumulate on/off, three- and four-code weights.
"""
import os

import numpy as np
import pytest

from tests.util import bits, make_pq2, make_q8_0, synth_pq2, synth_q8_0

pytestmark = pytest.mark.gpu
DATA = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_data")


@pytest.fixture(scope="module")
def be():
    from irontimber_b200.backend import CudaBackend
    b = CudaBackend(0, arena_floats=1 << 24)
    yield b
    b.close()


def oracle_mv(orc, raw, rows, cols, x_rows):
    return np.stack([orc.matvec_ternary(raw, rows, cols, x) for x in x_rows])


def run_mv(be, orc, raw, rows, cols, X, signs=None, perm=None, acc=False, rotate=True):
    """Uploads X rows, runs had_q8 + mv on the GPU and the same on the oracle; returns (gpu, want)."""
    ntok = X.shape[0]
    w = be.mat(raw, rows, cols)
    q = be.q8_rows(cols, ntok)
    xo, yo = 0, ((ntok * cols + 63) // 64) * 64
    ys = ((rows + 3) // 4) * 4
    be.upload(xo, X)
    if signs is not None:
        be.set_signs(signs)
    y0 = np.random.default_rng(1).standard_normal(ntok * ys).astype(np.float32)
    be.upload(yo, y0)
    be.had_q8(cols, ntok, xo, cols, q, perm=perm, signs=signs is not None, rotate=rotate)
    be.mv(w, ntok, q, yo, ys, acc=acc)
    got = be.download(yo, ntok * ys).reshape(ntok, ys)[:, :rows]
    want = np.empty((ntok, rows), np.float32)
    for t in range(ntok):
        hx = orc.hadamard_forward(X[t], 1024, signs, perm) if rotate else X[t]
        want[t] = orc.matvec_ternary(raw, rows, cols, hx)
        if acc:
            want[t] = y0.reshape(ntok, ys)[t, :rows] + want[t]
    # padding columns of y must be untouched
    assert np.array_equal(bits(be.download(yo, ntok * ys).reshape(ntok, ys)[:, rows:]), bits(y0.reshape(ntok, ys)[:, rows:]))
    w.close(); q.close()
    return got, want


def test_repack_roundtrip_and_synth_rule(be):
    rng = np.random.default_rng(11)
    for rows, cols in [(1, 128), (33, 256), (1000, 1024), (64, 5120)]:
        raw, _, _ = make_pq2(rng, rows, cols, ncodes=4)
        w = be.mat(raw, rows, cols)
        assert np.array_equal(w.download_pq2(), raw)
        assert w.device_bytes == ((rows + 31) // 32) * (cols // 128) * 1088
        w.close()
    for four in (False, True):
        w = be.mat_synth(1234, 70, 1024, four_codes=four)
        assert np.array_equal(w.download_pq2(), synth_pq2(1234, 70, 1024, four))
        w.close()
    qm = be.qmat_synth(99, 12, 512)
    assert np.array_equal(qm.download_q8_0(), synth_q8_0(99, 12, 512))
    qm.close()


def test_packed2_upload_equals_pq2_upload(be, orc):
    rng = np.random.default_rng(12)
    raw, _, _ = make_pq2(rng, 40, 1024, ncodes=4)
    words, scales = orc.packed2_from_ggml(orc.PQ2_0, raw, 40, 1024)
    w = be.mat_packed2(words, scales, 40, 1024)
    assert np.array_equal(w.download_pq2(), raw)
    w.close()


@pytest.mark.parametrize("n,ntok", [(1024, 1), (2048, 3), (5120, 2), (6144, 1), (17408, 2)])
@pytest.mark.parametrize("mode", ["signs", "nosign", "perm", "norotate"])
def test_hadamard_q8_bit_exact(be, orc, n, ntok, mode):
    rng = np.random.default_rng(n + ntok)
    X = rng.standard_normal((ntok, n)).astype(np.float32)
    X[0, :256] = 0.0                       # an all-zero q8k block
    X[0, 300] = 2.5; X[0, 301] = -2.5      # equal magnitudes: the first one decides the sign of iscale
    signs = np.where(rng.integers(0, 2, n) == 1, 1.0, -1.0).astype(np.float32) if mode in ("signs", "perm") else None
    perm = None
    if mode == "perm":
        perm = (128, 4, n // 512) if n % 512 == 0 else None
        if perm is None:
            pytest.skip("width not divisible")
    if signs is not None:
        be.set_signs(signs)
    q = be.q8_rows(n, ntok)
    be.upload(0, X)
    be.had_q8(n, ntok, 0, n, q, perm=perm, signs=signs is not None, rotate=mode != "norotate")
    for t in range(ntok):
        hx = orc.hadamard_forward(X[t], 1024, signs, perm) if mode != "norotate" else X[t]
        d, qs, s = orc.quantize_q8k(hx)
        gd, gqs, gs = q.read(t)
        assert np.array_equal(gqs, qs)
        assert np.array_equal(bits(gd), bits(d))
        assert np.array_equal(gs, s)
    q.close()


@pytest.mark.parametrize("inverse", [False, True])
def test_hadamard_f32_bit_exact(be, orc, inverse):
    rng = np.random.default_rng(5)
    n, ntok = 2048, 3
    X = rng.standard_normal((ntok, n)).astype(np.float32)
    signs = np.where(rng.integers(0, 2, n) == 1, 1.0, -1.0).astype(np.float32)
    be.set_signs(signs)
    be.upload(0, X)
    out = 1 << 20
    be.had(n, ntok, 0, n, out, n, inverse=inverse)
    got = be.download(out, ntok * n).reshape(ntok, n)
    for t in range(ntok):
        want = orc.hadamard_inverse(X[t], 1024, signs) if inverse else orc.hadamard_forward(X[t], 1024, signs)
        assert np.array_equal(bits(got[t]), bits(want))
    if not inverse:   # permuted forward, as used before ssm_out (src/vk/mod.rs:809)
        be.had(n, ntok, 0, n, out, n, perm=(128, 4, 4))
        got = be.download(out, ntok * n).reshape(ntok, n)
        for t in range(ntok):
            assert np.array_equal(bits(got[t]), bits(orc.hadamard_forward(X[t], 1024, signs, (128, 4, 4))))


@pytest.mark.parametrize("rows", [999, 1000, 1001])
@pytest.mark.parametrize("ntok,acc", [(1, True), (1, False), (2, False), (3, True), (5, False), (7, False), (11, True), (13, False), (21, False)])
def test_matvec_t2_kparity_grid_bit_exact(be, orc, rows, ntok, acc):
    rng = np.random.default_rng(rows * 100 + ntok)
    cols = 1024
    raw, _, _ = make_pq2(rng, rows, cols, ncodes=4 if ntok % 2 else 3)
    X = rng.standard_normal((ntok, cols)).astype(np.float32)
    signs = np.where(rng.integers(0, 2, cols) == 1, 1.0, -1.0).astype(np.float32)
    got, want = run_mv(be, orc, raw, rows, cols, X, signs=signs, acc=acc)
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("rows,cols", [(17408, 5120), (5120, 6144), (5120, 17408), (1024, 5120)])
def test_matvec_t2_model_shapes_bit_exact(be, orc, rows, cols):
    rng = np.random.default_rng(rows + cols)
    raw = synth_pq2(rows * 7 + cols, rows, cols)
    X = rng.standard_normal((2, cols)).astype(np.float32)
    signs = np.where(rng.integers(0, 2, cols) == 1, 1.0, -1.0).astype(np.float32)
    got, want = run_mv(be, orc, raw, rows, cols, X[:1], signs=signs)
    assert np.array_equal(bits(got), bits(want))
    got, want = run_mv(be, orc, raw, rows, cols, X, signs=signs, acc=True)
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("rows,cols,ntok,acc", [(1001, 1024, 22, False), (999, 1024, 64, True), (1000, 2048, 65, False), (96, 1024, 130, True),
                                               (17408, 5120, 64, False), (5120, 17408, 64, True), (10240, 5120, 40, False), (1024, 5120, 64, False),
                                               (17408, 5120, 128, False), (2048, 5120, 200, True), (1024, 2048, 512, False), (640, 6144, 129, True)])
@pytest.mark.parametrize("kernel", ["tc", "legacy"])
def test_matmul_t2_tile_kernel_bit_exact(be, orc, rows, cols, ntok, acc, kernel, monkeypatch):
    """More than eight activation rows go through the tile kernel (the role of matmul_t2, src/vk/mod.rs:655-677): every
    row tile width of its policy, ragged row groups and ragged activation tiles, same bits as the CPU's row-by-row matvec.
    Both implementations are forced in turn: "tc" = tcgen05.mma with accumulators in tensor memory (64 activation rows per
    CTA, 128 when there are more than 64), "legacy" = mma.sync."""
    monkeypatch.setenv("IT_MATMUL", kernel)
    rng = np.random.default_rng(rows + cols + ntok)
    raw = synth_pq2(rows * 3 + cols, rows, cols) if rows >= 1024 else make_pq2(rng, rows, cols, ncodes=4)[0]
    X = rng.standard_normal((ntok, cols)).astype(np.float32)
    signs = np.where(rng.integers(0, 2, cols) == 1, 1.0, -1.0).astype(np.float32)
    got, want = run_mv(be, orc, raw, rows, cols, X, signs=signs, acc=acc)
    assert np.array_equal(bits(got), bits(want))


def test_matvec_t2_integer_accumulators_bit_exact(be, orc):
    rng = np.random.default_rng(77)
    rows, cols, ntok = 333, 2048, 4
    raw, _, _ = make_pq2(rng, rows, cols, ncodes=4)
    X = (rng.standard_normal((ntok, cols)) * 3).astype(np.float32)
    w = be.mat(raw, rows, cols); q = be.q8_rows(cols, ntok)
    be.upload(0, X)
    be.had_q8(cols, ntok, 0, cols, q, signs=False, rotate=False)
    got = be.mv_sumi(w, ntok, q)
    for t in range(ntok):
        _, sumi = orc.matvec_ternary(raw, rows, cols, X[t], want_sumi=True)
        assert np.array_equal(got[t], sumi)
    w.close(); q.close()


def test_matvec_t2_extreme_codes_and_activations(be, orc):
    """All-code-3 weights against saturated activations: the largest accumulators the format allows."""
    rows, cols = 64, 1024
    raw = np.zeros((rows, cols // 128, 34), np.uint8)
    raw[:, :, 0:2] = np.frombuffer(np.float16(0.05).tobytes(), np.uint8)
    raw[:, :, 2:] = 0xFF
    raw[1::2, :, 2:] = 0x00          # odd rows: all code 0 (-1)
    X = np.full((2, cols), 7.0, np.float32); X[1] = -7.0
    got, want = run_mv(be, orc, raw.reshape(-1), rows, cols, X, rotate=False)
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("prefix,rows,cols", [("attn_k3", 3, 5120), ("ssm_out4", 4, 6144)])
def test_matvec_t2_on_reference_fixture_weights(be, orc, prefix, rows, cols):
    """The reference's own PQ2_0 rows (tests/data, decoded bit-exactly by the oracle) through the GPU path."""
    raw = np.fromfile(os.path.join(DATA, prefix + ".raw"), np.uint8)
    rng = np.random.default_rng(3)
    X = rng.standard_normal((2, cols)).astype(np.float32)
    got, want = run_mv(be, orc, raw, rows, cols, X, rotate=True)
    assert np.array_equal(bits(got), bits(want))
    w = be.mat(raw, rows, cols)
    assert np.array_equal(w.download_pq2(), raw)
    w.close()


@pytest.mark.parametrize("rows,cols,ntok,acc", [(1000, 256, 1, False), (1000, 256, 3, True), (5120, 10240, 1, False), (1024, 5120, 2, False), (5120, 17408, 1, True), (37, 512, 5, False)])
def test_matvec_q8_within_kernel_parity_tolerance(be, orc, rows, cols, ntok, acc):
    rng = np.random.default_rng(rows + cols + ntok)
    raw = make_q8_0(rng, rows, cols)
    X = rng.standard_normal((ntok, cols)).astype(np.float32)
    w = be.qmat(raw, rows, cols)
    words, scales = orc.q8g16_from_ggml(orc.Q8_0, raw, rows, cols)
    yo = ((ntok * cols + 63) // 64) * 64
    y0 = rng.standard_normal(ntok * rows).astype(np.float32)
    be.upload(0, X); be.upload(yo, y0)
    be.mvq(w, ntok, 0, cols, yo, rows, acc=acc)
    got = be.download(yo, ntok * rows).reshape(ntok, rows)
    for t in range(ntok):
        want = orc.mvq(words, scales, rows, cols, X[t]) + (y0.reshape(ntok, rows)[t] if acc else 0)
        assert np.max(np.abs(got[t] - want) / np.maximum(1.0, np.abs(want))) <= 1e-4
    assert np.array_equal(w.download_q8_0(), raw)
    w.close()


def test_matvec_q8_on_reference_fixture_weights(be, orc):
    raw = np.fromfile(os.path.join(DATA, "mtp_q80_3.raw"), np.uint8)
    rows, cols = 3, 5120
    X = np.random.default_rng(4).standard_normal(cols).astype(np.float32)
    w = be.qmat(raw, rows, cols)
    words, scales = orc.q8g16_from_ggml(orc.Q8_0, raw, rows, cols)
    be.upload(0, X)
    be.mvq(w, 1, 0, cols, 8192, rows)
    got = be.download(8192, rows)
    want = orc.mvq(words, scales, rows, cols, X)
    assert np.max(np.abs(got - want) / np.maximum(1.0, np.abs(want))) <= 1e-4
    w.close()


@pytest.mark.parametrize("n", [1, 5, 5000, 248320, 4096 * 296 + 3])
def test_argmax_first_maximum(be, orc, n):
    rng = np.random.default_rng(n)
    v = rng.standard_normal(n).astype(np.float32)
    dst = ((n + 67) // 4) * 4
    for trial in range(3):
        if trial == 1 and n > 4:      # ties: the lowest index wins
            m = v.max() + 1.0
            v[[n // 3, n // 2, n - 1]] = m
        if trial == 2:
            v[:] = -np.inf
        be.upload(0, v)
        be.argmax(0, n, dst)
        assert be.read_u32(dst) == orc.argmax(v)
    be.argmax(0, n, dst)              # scratch is reusable back to back
    assert be.read_u32(dst) == 0
