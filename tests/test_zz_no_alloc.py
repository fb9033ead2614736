"""The allocation-free argmax entry point against the regular one, through the C ABI.

`it_argmax_static` serves callers that own all device memory themselves and may not call cudaMalloc
(see include/irontimber_cuda.h): it gets raw device pointers and keeps its scratch inside the library.
Here the device buffers come from torch, standing in for such a caller's own pool.  Two calls in a row
check that the shared scratch is left ready for the next call.  This file sorts last on purpose so that
a run which stops at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_static_argmax_matches_regular_argmax_twice_in_a_row():
    import torch
    from irontimber_b200 import _lib
    from irontimber_b200.backend import CudaBackend
    L = _lib.load()
    torch.cuda.set_device(0)
    be = CudaBackend(0, arena_floats=1 << 20)
    try:
        rng = np.random.default_rng(2024)
        stream = torch.cuda.Stream()
        out = torch.zeros(1, dtype=torch.int32, device="cuda:0")
        for call, n in enumerate((248320, 5000)):
            v = rng.standard_normal(n).astype(np.float32)
            v[[n // 5, n // 2]] = v.max() + 1.0          # a tie: the lower index must win in both paths
            be.upload(0, v)
            dst = ((n + 67) // 4) * 4
            be.argmax(0, n, dst)
            want = be.read_u32(dst)
            dev = torch.from_numpy(v).to("cuda:0")
            torch.cuda.synchronize()
            _lib.check(L.it_argmax_static(C.c_void_p(stream.cuda_stream), C.c_void_p(dev.data_ptr()), n, C.c_void_p(out.data_ptr())))
            stream.synchronize()
            got = int(out.cpu().numpy().view(np.uint32)[0])
            assert got == want == n // 5, f"call {call}"
        # beyond the stated maximum the call is refused before anything is launched
        assert L.it_argmax_static(None, C.c_void_p(dev.data_ptr()), (1 << 24) + 1, C.c_void_p(out.data_ptr())) == -1
        assert b"scratch limit" in L.it_last_error()
    finally:
        be.close()
