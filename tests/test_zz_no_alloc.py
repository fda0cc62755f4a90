"""gn_op_gemm_nt_static -- the product C = A B^T + bias for hosts that cannot allocate device memory (their
own pool owns all of HBM, or a per-step latency budget rules out the allocator lock).  Its operand planes
live in a fixed array inside the library instead of cudaMalloc'ed buffers.  Checked here, through the C ABI,
against the regular entry point (gn_op_gemm_nt, tensor-core engine) on calls in a row: each later call finds the
earlier call's planes in the shared array and must not be disturbed by them.  The property the entry point exists
for is asserted too: the device's free memory is the same before and after the calls.  The file name makes pytest
collect it last."""
import ctypes as C

import numpy as np
import pytest

from tests.parity import norm_err

pytestmark = pytest.mark.gpu


def _f(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _free_bytes():
    import torch
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info(0)[0]


def test_static_scratch_gemm_matches_regular_entry_point_twice():
    from goneuron_b200 import _lib
    from goneuron_b200.sequential import Device
    L = _lib.load()
    dev = Device(0)
    try:
        # second call: smaller planes over the first call's; third: a contraction longer than one accumulator run (cut into slices)
        for call, (M, N, K) in enumerate([(300, 520, 100), (512, 256, 70), (128, 192, 9000)]):
            rng = np.random.default_rng(100 + call)
            A = rng.standard_normal((M, K)).astype(np.float32)
            B = rng.standard_normal((N, K)).astype(np.float32)
            bias = rng.standard_normal(N).astype(np.float32)
            ref = np.empty((M, N), np.float32)
            _lib.check(L.gn_op_gemm_nt(dev.handle, 1, M, N, K, _f(A), _f(B), _f(bias), _f(ref)))
            dA, dB, db = dev.alloc(A), dev.alloc(B), dev.alloc(bias)
            dC = dev.alloc(np.zeros((M, N), np.float32))
            if call == 0:
                _lib.check(L.gn_op_gemm_nt_static(dev.handle, M, N, K, dA, dB, db, dC))     # the first call on a device resolves the array's address
            free_before = _free_bytes()
            _lib.check(L.gn_op_gemm_nt_static(dev.handle, M, N, K, dA, dB, db, dC))
            assert _free_bytes() == free_before, "the entry point allocated or freed device memory"
            out = np.empty((M, N), np.float32)
            _lib.check(L.gn_device_download(dev.handle, _f(out), dC, out.size))
            assert norm_err(out, ref) <= 1e-6, (call, norm_err(out, ref))
            f64 = A.astype(np.float64) @ B.astype(np.float64).T + bias
            assert norm_err(out, f64) <= 1e-5
            if call == 2:
                # beyond the fixed array: a clear error before anything is touched (live pointers all the same)
                rc = L.gn_op_gemm_nt_static(dev.handle, 4096, 4096, 1024, dA, dB, None, dC)
                assert rc == -1 and b"scratch" in L.gn_last_error()
            for p in (dA, dB, db, dC):
                dev.free(p)
    finally:
        dev.close()
