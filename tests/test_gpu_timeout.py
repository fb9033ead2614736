"""A bounded device-side wait that runs out, on ONE GPU and without faulting anything.

Two contexts on the same GPU are attached to each other as ranks 0 and 1 of a row-sharded pair.  Only rank 0 launches its
half of a sharded matvec: its kernel stores its rows into both arenas (all addresses valid) and then waits for rank 1's
rows, which never come.  With the wait limit lowered to two milliseconds the kernel gives up by itself, raises the
context's status word and returns; the host sees IT_ETIMEOUT at the next synchronisation, the flag clears, and the
context goes on working (an unsharded matvec afterwards is bit-exact).
"""
import time

import numpy as np
import pytest

from tests.util import bits, synth_pq2

pytestmark = pytest.mark.gpu


def test_peer_wait_runs_out_and_the_context_stays_usable(orc):
    from irontimber_b200 import _lib
    from irontimber_b200.backend import CudaBackend
    rows, cols = 2048, 1024
    b0, b1 = CudaBackend(0, arena_floats=1 << 18), CudaBackend(0, arena_floats=1 << 18)
    try:
        b0.attach_peers_local(0, [b0, b1])
        b1.attach_peers_local(1, [b0, b1])
        b0.set_peer_wait_us(2000.0)
        rng = np.random.default_rng(3)
        signs = np.where(rng.integers(0, 2, cols) == 1, 1.0, -1.0).astype(np.float32)
        x = rng.standard_normal(cols).astype(np.float32)
        b0.set_signs(signs)
        q = b0.q8_rows(cols, 1)
        b0.upload(0, x)
        b0.had_q8(cols, 1, 0, cols, q)
        half = b0.mat_synth_rows(77, rows, cols, 0, rows // 2)        # rank 0's rows of the logical matrix
        b0.sync()
        t0 = time.perf_counter()
        b0.mv(half, 1, q, 4096, rows)                                 # rank 1 never launches its half
        with pytest.raises(_lib.IronTimberError) as err:
            b0.sync()
        waited = time.perf_counter() - t0
        assert err.value.code == -5 and "bounded wait" in str(err.value) and "site 22" in str(err.value)
        assert waited < 1.0                                           # the lowered limit, not the four-second default
        b0.sync()                                                     # the flag was cleared by the failed call
        # rank 0's own rows did land in its arena (its peer would have collected them from its slot buffer in its own launch)
        want = orc.matvec_ternary(synth_pq2(77, rows, cols), rows, cols, orc.hadamard_forward(x, 1024, signs))
        assert np.array_equal(bits(b0.download(4096, rows // 2)), bits(want[: rows // 2]))
        # the context is usable: an unsharded product afterwards is bit-exact
        full = b0.mat_synth(77, rows, cols)
        b0.mv(full, 1, q, 8192, rows)
        assert np.array_equal(bits(b0.download(8192, rows)), bits(want))
        full.close(); half.close(); q.close()
    finally:
        b1.close(); b0.close()
