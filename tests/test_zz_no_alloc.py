"""gn_op_gemm_nt_static -- the product C = A B^T + bias for hosts that cannot allocate device memory (their
own pool owns all of HBM, or a per-step latency budget rules out the allocator lock).  Its operand planes
live in a fixed array inside the library instead of cudaMalloc'ed buffers.  Checked here, through the C ABI,
against the regular entry point (gn_op_gemm_nt, tensor-core engine) on two calls in a row: the second call
finds the first call's planes in the shared array and must not be disturbed by them.  The file name makes
pytest collect it last."""
import ctypes as C

import numpy as np
import pytest

from tests.parity import norm_err

pytestmark = pytest.mark.gpu


def _f(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def test_static_scratch_gemm_matches_regular_entry_point_twice():
    from goneuron_b200 import _lib
    from goneuron_b200.sequential import Device
    L = _lib.load()
    dev = Device(0)
    try:
        for call, (M, N, K) in enumerate([(300, 520, 100), (512, 256, 70)]):      # second call: smaller planes over the first call's
            rng = np.random.default_rng(100 + call)
            A = rng.standard_normal((M, K)).astype(np.float32)
            B = rng.standard_normal((N, K)).astype(np.float32)
            bias = rng.standard_normal(N).astype(np.float32)
            ref = np.empty((M, N), np.float32)
            _lib.check(L.gn_op_gemm_nt(dev.handle, 1, M, N, K, _f(A), _f(B), _f(bias), _f(ref)))
            dA, dB, db = dev.alloc(A), dev.alloc(B), dev.alloc(bias)
            dC = dev.alloc(np.zeros((M, N), np.float32))
            _lib.check(L.gn_op_gemm_nt_static(dev.handle, M, N, K, dA, dB, db, dC))
            out = np.empty((M, N), np.float32)
            _lib.check(L.gn_device_download(dev.handle, _f(out), dC, out.size))
            for p in (dA, dB, db, dC):
                dev.free(p)
            assert norm_err(out, ref) <= 1e-6, (call, norm_err(out, ref))
            f64 = A.astype(np.float64) @ B.astype(np.float64).T + bias
            assert norm_err(out, f64) <= 1e-5
        # beyond the fixed array: a clear error, no allocation attempted
        rc = L.gn_op_gemm_nt_static(dev.handle, 4096, 4096, 1024, dA, dB, None, dC)
        assert rc == -1 and b"scratch" in L.gn_last_error()
    finally:
        dev.close()
