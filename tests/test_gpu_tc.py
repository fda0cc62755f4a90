"""The tcgen05 split-operand (TF32 + 2 x BF16) contraction engine against float64 numpy and against the exact-fp32 SIMT engine,
through the C ABI: C = A B^T + bias, ragged and tile-aligned shapes."""
import ctypes as C

import numpy as np
import pytest

from tests.parity import norm_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    from goneuron_b200.sequential import Device
    d = Device(0)
    yield d
    d.close()


def _gemm(device, engine, A, B, bias):
    from goneuron_b200 import _lib
    out = np.empty((A.shape[0], B.shape[0]), np.float32)
    f = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))
    _lib.check(_lib.load().gn_op_gemm_nt(device.handle, engine, A.shape[0], B.shape[0], A.shape[1], f(A), f(B), f(bias) if bias is not None else None, f(out)))
    return out


@pytest.mark.parametrize("M,N,K", [(128, 256, 32), (128, 256, 64), (256, 512, 256), (300, 520, 100), (129, 70, 70), (1, 8, 5),
                                   (2048, 1024, 1024), (4096, 256, 4096),
                                   (256, 384, 70000)])          # a weight-gradient shape: contraction over all tokens, cut into slices
def test_tc_gemm_matches_fp64(device, M, N, K):
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((N, K)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    ref = A.astype(np.float64) @ B.astype(np.float64).T + bias
    tc = _gemm(device, 1, A, B, bias)
    simt = _gemm(device, 0, A, B, bias)
    e_tc, e_simt = norm_err(tc, ref), norm_err(simt, ref)
    # fp32-level accuracy: within a small factor of the exact-fp32 engine's own rounding error, far below 1e-4
    print(f"M{M} N{N} K{K}: tc {e_tc:.2e} simt {e_simt:.2e}")
    assert e_tc <= 2e-6 + 4 * e_simt + 5e-9 * K, (e_tc, e_simt)
    # a single-pass TF32 product would sit near 5e-4 * sqrt(K)/K-ish; make sure we are not that
    assert e_tc < 3e-5


def test_tc_gemm_exact_small_integers(device):
    # integer-valued operands below 2^10 are exact in TF32: the result must be exact
    rng = np.random.default_rng(3)
    A = rng.integers(-8, 9, size=(256, 96)).astype(np.float32)
    B = rng.integers(-8, 9, size=(256, 96)).astype(np.float32)
    out = _gemm(device, 1, A, B, None)
    assert np.array_equal(out, (A.astype(np.int64) @ B.astype(np.int64).T).astype(np.float32))
