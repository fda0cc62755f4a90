"""The tcgen05 split-operand (three BF16 products per fp32 product) contraction engine against float64 numpy and against the exact-fp32 SIMT engine,
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
                                   (256, 384, 70000),           # a weight-gradient shape: contraction over all tokens, cut into slices
                                   # more tiles than SMs with a short last round: its tiles run as half tiles (256- and 128-wide tilings)
                                   (25600, 256, 96), (12800, 500, 64), (25600, 128, 96), (5760, 1024, 128)])
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
    # a single-pass BF16 or TF32 product would sit near 1e-3; make sure we are not that
    assert e_tc < 3e-5


def test_tc_gemm_exact_small_integers(device):
    # small integer-valued operands are exact in BF16: the result must be exact
    rng = np.random.default_rng(3)
    A = rng.integers(-8, 9, size=(256, 96)).astype(np.float32)
    B = rng.integers(-8, 9, size=(256, 96)).astype(np.float32)
    out = _gemm(device, 1, A, B, None)
    assert np.array_equal(out, (A.astype(np.int64) @ B.astype(np.int64).T).astype(np.float32))


def test_bounded_wait_gives_up_and_the_context_stays_usable(device):
    """Failure detection without a GPU fault: with a poll limit of 1 the kernel's first wait for a tile that TMA has only
    just been asked for runs out.  The kernel must stop its pipeline and return, the call must report GN_ERR_TIMEOUT
    quickly, the status word must be cleared, and the next ordinary call on the same context must be correct."""
    import time
    from goneuron_b200 import _lib
    L = _lib.load()
    rng = np.random.default_rng(11)
    A, B = rng.standard_normal((1024, 512)).astype(np.float32), rng.standard_normal((768, 512)).astype(np.float32)
    bias = rng.standard_normal(768).astype(np.float32)
    good = _gemm(device, 1, A, B, bias)
    out = np.empty((1024, 768), np.float32)
    f = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))
    _lib.check(L.gn_ctx_set_spin_limit(device.handle, 1))
    try:
        t0 = time.perf_counter()
        rc = L.gn_op_gemm_nt(device.handle, 1, 1024, 768, 512, f(A), f(B), f(bias), f(out))
        dt = time.perf_counter() - t0
    finally:
        _lib.check(L.gn_ctx_set_spin_limit(device.handle, 0))
    assert rc == -6 and b"bounded wait" in L.gn_last_error(), (rc, L.gn_last_error())
    assert dt < 5.0, dt
    again = _gemm(device, 1, A, B, bias)          # status word cleared, pipeline state fresh
    assert np.array_equal(again, good)


def test_timed_out_step_leaves_parameters_alone(device):
    """A training step in which a device-side wait gave up returns GN_ERR_TIMEOUT and has changed neither the
    parameters nor the optimiser state; the same step repeated with the default limit then equals a fresh run."""
    from goneuron_b200 import _lib, configs
    from goneuron_b200.sequential import Adam, Sequential
    kw = dict(vocab=1000, dim=256, seq_len=128, heads=4, ff_dim=1024, n_blocks=1)
    layers, loss_kind, params, x, y, lr = configs.make_case("transformer_large", batch=8, **kw)
    fresh = Sequential(layers, device).Compile(Adam(lr), loss_kind)
    fresh.SetParams(params)
    l_ref = fresh.TrainBatch(x, y)
    p_ref = fresh.Params()
    fresh.Close()
    model = Sequential(layers, device).Compile(Adam(lr), loss_kind)
    model.SetParams(params)
    _lib.check(_lib.load().gn_ctx_set_spin_limit(device.handle, 1))
    try:
        with pytest.raises(_lib.GoNeuronCudaError) as ei:
            model.TrainBatch(x, y)
    finally:
        _lib.check(_lib.load().gn_ctx_set_spin_limit(device.handle, 0))
    assert ei.value.code == -6
    m, v, t = model.AdamState()
    assert t == 0 and not m.any() and not v.any() and np.array_equal(model.Params(), params)
    assert model.TrainBatch(x, y) == l_ref and np.array_equal(model.Params(), p_ref)
    model.Close()
