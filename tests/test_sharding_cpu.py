"""Row sharding, host side, on CPU: the library's split rule through the C ABI, and two gloo ranks that compute the
oracle matvec of their own rows and all-gather the slices (what the GPU path does with peer stores)."""
import ctypes as C

import numpy as np
import pytest

from irontimber_b200 import _lib
from irontimber_b200.sharding import gather_rows, shard_range
from tests.mp_workers import oracle_sharded_matvec, run_ranks


def test_shard_range_rule():
    assert shard_range(17408, 3, 8) == (3 * 2176, 2176)          # 17408 / 8 = 2176 rows per rank
    assert shard_range(248320, 7, 8) == (7 * 31040, 31040)       # LM head: 31040 rows per rank
    assert shard_range(5120, 0, 1) == (0, 5120)
    covered = [shard_range(1024, r, 4) for r in range(4)]
    assert [c[0] for c in covered] == [0, 256, 512, 768] and all(c[1] == 256 for c in covered)
    L = _lib.load()
    r0, n = C.c_size_t(), C.c_size_t()
    assert L.it_shard_range(1000, 0, 3, C.byref(r0), C.byref(n)) == -1      # uneven split is refused, not rounded
    assert L.it_shard_range(1024, 4, 4, C.byref(r0), C.byref(n)) == -1      # rank outside the world
    assert L.it_shard_range(1024, 0, 9, C.byref(r0), C.byref(n)) == -1      # more ranks than a node has GPUs


def test_gather_rows_restores_order():
    parts = [np.arange(r * 4, r * 4 + 4, dtype=np.float32) for r in range(3)]
    assert np.array_equal(gather_rows(parts), np.arange(12, dtype=np.float32))


@pytest.mark.timeout(300)
def test_two_gloo_ranks_reproduce_the_full_matvec():
    res = run_ranks(oracle_sharded_matvec, 2, 41, 1024, 1024)
    for same_bits, pick, want_pick in res:
        assert same_bits and pick == want_pick
