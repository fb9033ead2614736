"""Shared helpers for the tests: seeded synthetic inputs in the reference's formats."""
import numpy as np

M64 = (1 << 64) - 1


def make_pq2(rng, rows, cols, ncodes=3, dlo=0.01, dhi=0.05):
    """Random PQ2_0 rows (src/quant.rs:21-29): returns (raw uint8 [rows*cols/128*34], codes, f16 scales)."""
    nb = cols // 128
    codes = rng.integers(0, ncodes, (rows, cols), dtype=np.uint8)
    d16 = rng.uniform(dlo, dhi, (rows, nb)).astype(np.float16)
    raw = np.zeros((rows, nb, 34), np.uint8)
    raw[:, :, 0:2] = d16.view(np.uint8).reshape(rows, nb, 2)
    c4 = codes.reshape(rows, nb, 32, 4)
    raw[:, :, 2:] = c4[..., 0] | (c4[..., 1] << 2) | (c4[..., 2] << 4) | (c4[..., 3] << 6)
    return raw.reshape(-1), codes, d16


def make_q8_0(rng, rows, cols, dlo=0.002, dhi=0.006):
    """Random ggml Q8_0 rows (src/quant.rs:188-191)."""
    nblk = rows * cols // 32
    raw = np.zeros((nblk, 34), np.uint8)
    raw[:, 0:2] = rng.uniform(dlo, dhi, (nblk, 1)).astype(np.float16).view(np.uint8)
    raw[:, 2:] = rng.integers(-127, 128, (nblk, 32)).astype(np.int8).view(np.uint8)
    return raw.reshape(-1)


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


# ---- numpy mirror of the library's synthetic-data rule (it_matrix_synth / it_qmatrix_synth) -------
def _mix64(z):
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xbf58476d1ce4e5b9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94d049bb133111eb)
    return z ^ (z >> np.uint64(31))


def synth_hash(seed, idx):
    """idx-th output of splitmix64 seeded with `seed` (the reference's RNG, src/sampling.rs:43)."""
    with np.errstate(over="ignore"):
        idx = np.asarray(idx, np.uint64)
        return _mix64(np.uint64(seed & M64) + np.uint64(0x9e3779b97f4a7c15) * (idx + np.uint64(1)))


def synth_pq2(seed, rows, cols, four_codes=False):
    nb = cols // 128
    n = rows * cols
    h = synth_hash(seed, np.arange(n // 2, dtype=np.uint64))
    v = np.empty(n, np.uint32)
    v[0::2] = (h & np.uint64(0xffffffff)).astype(np.uint32)
    v[1::2] = (h >> np.uint64(32)).astype(np.uint32)
    codes = ((v & 3) if four_codes else (v % 3)).astype(np.uint8).reshape(rows, cols)
    hb = synth_hash(seed ^ 0x5ca1e5, np.arange(rows * nb, dtype=np.uint64))
    u = (hb >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)
    d16 = (np.float32(0.01) + np.float32(0.04) * u).astype(np.float16).reshape(rows, nb)
    raw = np.zeros((rows, nb, 34), np.uint8)
    raw[:, :, 0:2] = d16.view(np.uint8).reshape(rows, nb, 2)
    c4 = codes.reshape(rows, nb, 32, 4)
    raw[:, :, 2:] = c4[..., 0] | (c4[..., 1] << 2) | (c4[..., 2] << 4) | (c4[..., 3] << 6)
    return raw.reshape(-1)


def synth_q8_0(seed, rows, cols):
    n = rows * cols
    h = synth_hash(seed, np.arange(n // 2, dtype=np.uint64))
    q = np.empty(n, np.int8)
    q[0::2] = ((h & np.uint64(0xffffffff)) % np.uint64(255)).astype(np.int64) - 127
    q[1::2] = ((h >> np.uint64(32)) % np.uint64(255)).astype(np.int64) - 127
    hb = synth_hash(seed ^ 0x5ca1e5, np.arange(n // 32, dtype=np.uint64))
    u = (hb >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)
    d16 = (np.float32(0.002) + np.float32(0.004) * u).astype(np.float16)
    raw = np.zeros((n // 32, 34), np.uint8)
    raw[:, 0:2] = d16.view(np.uint8).reshape(-1, 2)
    raw[:, 2:] = q.view(np.uint8).reshape(-1, 32)
    return raw.reshape(-1)
