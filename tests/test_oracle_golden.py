"""Pins the CPU oracle against the reference's golden vectors and known-answer unit tests.

Sources restated here: tests/dequant_vs_ggml.rs (bit-exact decode and repack), src/quant.rs:164-185
(code map, q8k bound), src/hadamard.rs:49-71 (FWHT vs the explicit matrix, round trip),
src/sampling.rs:100-105 (argmax), tests/mtp_loop_regressions.rs (ten loop scenarios).
"""
import os

import numpy as np
import pytest

DATA = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_data")


def _raw(name):
    return np.fromfile(os.path.join(DATA, name + ".raw"), np.uint8)


def _f32(name):
    return np.fromfile(os.path.join(DATA, name + ".f32"), np.float32)


def _bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.mark.parametrize("prefix,rows,cols", [("ssm_out4", 4, 6144), ("attn_k3", 3, 5120)])
@pytest.mark.parametrize("ext,ty", [("", 0), (".ptq1", 1)])
def test_ternary_dequant_and_repack_bit_exact(orc, prefix, rows, cols, ext, ty):
    raw, want = _raw(prefix + ext), _f32(prefix + ext)
    got = orc.dequant_pq2_0(raw) if ty == 0 else orc.dequant_ptq1_0(raw)
    assert np.array_equal(_bits(got), _bits(want))
    words, scales = orc.packed2_from_ggml(ty, raw, rows, cols)
    for r in range(rows):
        assert np.array_equal(_bits(orc.packed2_row_f32(words, scales, cols, r)), _bits(want[r * cols:(r + 1) * cols]))


@pytest.mark.parametrize("prefix,kind", [("mtp_q80_3", "q8_0"), ("mtp_q6k3", "q6_k"), ("mtp_q4k3", "q4_k")])
def test_kquant_dequant_and_q8g16_repack_bit_exact(orc, prefix, kind):
    rows, cols = 3, 5120
    raw, want = _raw(prefix), _f32(prefix)
    got = {"q8_0": orc.dequant_q8_0, "q6_k": orc.dequant_q6_k, "q4_k": orc.dequant_q4_k}[kind](raw)
    assert np.array_equal(_bits(got), _bits(want))
    if kind != "q4_k":
        words, scales = orc.q8g16_from_ggml(0 if kind == "q8_0" else 1, raw, rows, cols)
        for r in range(rows):
            assert np.array_equal(_bits(orc.q8g16_row_f32(words, scales, cols, r)), _bits(want[r * cols:(r + 1) * cols]))


def test_pq2_codes_map(orc):
    b = np.zeros(34, np.uint8)
    b[0:2] = np.frombuffer(np.float16(0.5).tobytes(), np.uint8)
    b[2] = 0b11_10_01_00
    o = orc.dequant_pq2_0(b)
    assert list(o[:4]) == [-0.5, 0.0, 0.5, 1.0]
    assert np.all(o[4:] == -0.5)


def test_q8k_roundtrip_bounds(orc):
    x = np.array([((i * 37 % 101) - 50.0) / 7.0 for i in range(512)], np.float32)
    d, qs, s = orc.quantize_q8k(x)
    for i in range(512):
        assert abs(np.float32(qs[i]) * d[i // 256] - x[i]) <= abs(d[i // 256]) * 0.5 + 1e-6
    assert np.array_equal(s, qs.astype(np.int32).reshape(-1, 128).sum(1))


def test_q8k_zero_block_and_max_code(orc):
    x = np.zeros(512, np.float32)
    x[300] = 3.0  # block 1: max positive -> iscale negative -> code -127
    d, qs, s = orc.quantize_q8k(x)
    assert d[0] == 0.0 and np.all(qs[:256] == 0)
    assert qs[300] == -127 and d[1] == np.float32(1.0) / (np.float32(-127.0) / np.float32(3.0))
    x[300] = -3.0  # max negative -> iscale positive -> -127 as well (iscale * x = -127)
    d, qs, s = orc.quantize_q8k(x)
    assert qs[300] == -127


def test_fwht_matches_explicit_matrix(orc):
    n = 64
    x = np.array([np.sin(np.float32(i) * np.float32(0.37)) for i in range(n)], np.float32)
    y = orc.fwht_blocks(x, n)
    for r in range(n):
        s = sum((-1.0 if bin(r & c).count("1") % 2 else 1.0) * float(x[c]) for c in range(n))
        assert abs(s / np.sqrt(n) - float(y[r])) < 1e-5


def test_hadamard_inverse_roundtrip(orc):
    signs = np.array([-1.0 if i % 3 == 0 else 1.0 for i in range(256)], np.float32)
    x = np.arange(256, dtype=np.float32) - 100.0
    r = orc.hadamard_inverse(orc.hadamard_forward(x, 128, signs), 128, signs)
    assert np.max(np.abs(r - x)) < 1e-3


def test_gdn_group_perm_matches_index_formula(orc):
    hd, nk, rep = 128, 4, 4
    x = np.arange(hd * nk * rep, dtype=np.float32)
    o = orc.gdn_group_perm(x, hd, nk, rep)
    # gather form used by the reference's GPU transform: src = i0 + hd*(k + nk*r) (shaders/hadamard.comp:13)
    g = np.arange(x.size)
    i0, q = g % hd, g // hd
    r, k = q % rep, q // rep
    assert np.array_equal(o, x[i0 + hd * (k + nk * r)])


def test_argmax_first_maximum(orc):
    assert orc.argmax([0.1, 2.0, -1.0, 2.0]) == 1
    assert orc.argmax([5.0]) == 0
    assert orc.argmax([-3.0, -3.0]) == 0


def test_ternary_matvec_matches_independent_numpy(orc):
    """The q8k integer dot has no fixture in the reference: cross-check against numpy (int64 sums, f32 epilogue)."""
    rng = np.random.default_rng(7)
    rows, cols = 37, 1024
    codes = rng.integers(0, 4, (rows, cols), dtype=np.uint8)
    d16 = rng.uniform(0.01, 0.05, (rows, cols // 128)).astype(np.float16)
    raw = np.zeros((rows, cols // 128, 34), np.uint8)
    raw[:, :, 0:2] = d16.view(np.uint8).reshape(rows, cols // 128, 2)
    c4 = codes.reshape(rows, cols // 128, 32, 4)
    raw[:, :, 2:] = c4[..., 0] | (c4[..., 1] << 2) | (c4[..., 2] << 4) | (c4[..., 3] << 6)
    x = rng.standard_normal(cols).astype(np.float32)
    y, sumi = orc.matvec_ternary(raw, rows, cols, x, want_sumi=True)
    d, qs, s128 = orc.quantize_q8k(x)
    ref_sumi = (codes.astype(np.int64).reshape(rows, -1, 128) * qs.astype(np.int64).reshape(-1, 128)).sum(2) - s128
    assert np.array_equal(sumi, ref_sumi)
    want = np.zeros(rows, np.float32)
    for b in range(cols // 128):
        want = want + (d16[:, b].astype(np.float32) * d[b // 2]) * ref_sumi[:, b].astype(np.float32)
    assert np.array_equal(_bits(y), _bits(want))
    # Packed2::dot_q8k is the same arithmetic on the repacked layout
    words, scales = orc.packed2_from_ggml(0, raw, rows, cols)
    for r in range(rows):
        assert _bits(orc.packed2_dot_q8k(words, scales, cols, r, (d, qs, s128))) == _bits(y[r])
    # and the f32-activation mode stays within quantisation error of it
    yf = orc.matvec_ternary(raw, rows, cols, x, numerics=orc.F32)
    assert np.max(np.abs(yf - y)) < 0.05 * np.max(np.abs(yf)) + 1e-3
    for r in (0, rows - 1):
        assert abs(orc.packed2_dot_f32(words, scales, cols, r, x) - yf[r]) <= 1e-4 * max(1.0, abs(yf[r]))


def test_thread_count_never_changes_a_result(orc):
    rng = np.random.default_rng(3)
    rows, cols = 300, 512
    raw = rng.integers(0, 256, (rows, cols // 128, 34), dtype=np.uint8)
    raw[:, :, 0:2] = np.frombuffer(np.float16(0.02).tobytes(), np.uint8)
    x = rng.standard_normal(cols).astype(np.float32)
    a = orc.matvec_ternary(raw, rows, cols, x, nthreads=1)
    b = orc.matvec_ternary(raw, rows, cols, x, nthreads=4)
    assert np.array_equal(_bits(a), _bits(b))


def test_mvq_matches_numpy(orc):
    rng = np.random.default_rng(5)
    rows, cols = 12, 256
    raw = np.zeros((rows * cols // 32, 34), np.uint8)
    raw[:, 0:2] = rng.uniform(0.001, 0.01, (rows * cols // 32, 1)).astype(np.float16).view(np.uint8)
    raw[:, 2:] = rng.integers(-127, 128, (rows * cols // 32, 32)).astype(np.int8).view(np.uint8)
    words, scales = orc.q8g16_from_ggml(0, raw, rows, cols)
    x = rng.standard_normal(cols).astype(np.float32)
    y = orc.mvq(words, scales, rows, cols, x)
    w = np.stack([orc.q8g16_row_f32(words, scales, cols, r) for r in range(rows)])
    assert np.allclose(y, w.astype(np.float64) @ x.astype(np.float64), rtol=1e-4, atol=1e-4)


# ---- tests/mtp_loop_regressions.rs restated with the same scripted backend ----------------
class Script:
    def __init__(self, bad=False):
        self.pos = 0; self.calls = 0; self.rejected = 0; self.drafts = 0; self.bad = bad

    def mtp_single(self, x):
        a = 10 + self.pos; self.pos += 1; self.calls += 1; return a

    def mtp_prefill(self, p):
        self.pos = len(p); return 10

    def mtp_draft(self, toks):
        self.drafts += 1; return 99 if self.bad else 10 + self.pos

    def mtp_verify(self, x, d):
        a = 10 + self.pos; self.pos += 2; self.calls += 2; return (a, a + 1)

    def mtp_reject(self):
        self.pos -= 1; self.rejected += 1

    def reset_all(self):
        self.pos = 0


def loop_scenarios(run):
    """Shared by the oracle loop and the product loop: `run(backend, prompt, n, is_eog, on_tok) -> (tokens, stats)`."""
    b = Script(); o, s = run(b, [1], 2, lambda t: False, lambda t: True)
    assert o == [10, 11] and b.calls == 1 and s["drafted"] == 0
    b = Script(); o, _ = run(b, [1], 9, lambda t: t == 11, lambda t: True)
    assert o == [10, 11] and b.pos == 2
    for n in (2, 4, 6, 8):
        b = Script(); o, s = run(b, [1], n, lambda t: False, lambda t: True)
        assert len(o) == n and b.calls == n - 1 and s["timed_decode_forwards"] == n - 1
    b = Script(); assert run(b, [1], 0, lambda t: False, lambda t: True)[0] == [] and b.pos == 0
    b = Script(); assert run(b, [1], 9, lambda t: t == 10, lambda t: True)[0] == [10] and b.calls == 0
    b = Script(); assert run(b, [1], 9, lambda t: t == 11, lambda t: True)[0] == [10, 11]
    b = Script(bad=True); assert run(b, [1], 9, lambda t: t == 11, lambda t: True)[0] == [10, 11] and b.rejected == 1
    for n in (1, 3, 5, 7, 9):
        b = Script(); assert run(b, [1], n, lambda t: False, lambda t: True)[0] == list(range(10, 10 + n))
    b = Script(); assert run(b, [1], 9, lambda t: False, lambda t: t < 11)[0] == [10, 11]
    b = Script(bad=True); o, s = run(b, [1], 9, lambda t: False, lambda t: True)
    assert o == list(range(10, 19)) and s["accepted"] == 0


def test_greedy_mtp_loop_scenarios(orc):
    loop_scenarios(orc.greedy_mtp)
