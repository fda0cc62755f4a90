"""Multi-head attention kernels through the C ABI (gn_op_attention) against float64 numpy: the warp-level
tensor-core kernels (engine 0) and the tcgen05 / tensor-memory kernels (engine 1), forward and backward.
Arithmetic restated from internal/layer/transformer.go:470-503 and :589-657."""
import ctypes as C

import numpy as np
import pytest

from tests.parity import norm_err

pytestmark = pytest.mark.gpu

TOL = 1e-4   # normalised max error; both engines run split-operand products and land near 1e-6


@pytest.fixture(scope="module")
def device():
    from goneuron_b200.sequential import Device
    d = Device(0)
    yield d
    d.close()


def reference(Q, K, V, dO, B, T, D, H, causal):
    hd = D // H
    q, k, v, g = (x.astype(np.float64).reshape(B, T, H, hd).transpose(0, 2, 1, 3) for x in (Q, K, V, dO))
    s = q @ k.transpose(0, 1, 3, 2) / np.sqrt(hd)
    if causal:
        s = np.where(np.tril(np.ones((T, T), bool)), s, -np.inf)
    m = s.max(-1, keepdims=True)
    e = np.exp(s - m)
    l = e.sum(-1, keepdims=True)
    p = e / l
    o = p @ v
    dv = p.transpose(0, 1, 3, 2) @ g
    dp = g @ v.transpose(0, 1, 3, 2)
    ds = p * (dp - (dp * p).sum(-1, keepdims=True)) / np.sqrt(hd)
    dq, dk = ds @ k, ds.transpose(0, 1, 3, 2) @ q
    back = lambda x: x.transpose(0, 2, 1, 3).reshape(B * T, D)
    return back(o), m.reshape(-1), l.reshape(-1), back(dq), back(dk), back(dv)


def run(device, engine, Q, K, V, dO, B, T, D, H, causal):
    from goneuron_b200 import _lib
    f = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))
    O, dQ, dK, dV = (np.empty_like(Q) for _ in range(4))
    M, L = np.empty(B * H * T, np.float32), np.empty(B * H * T, np.float32)
    _lib.check(_lib.load().gn_op_attention(device.handle, engine, B, T, D, H, causal, f(Q), f(K), f(V), f(dO), f(O), f(M), f(L), f(dQ), f(dK), f(dV)))
    return O, M, L, dQ, dK, dV


CASES = [  # engine, B, T, D, H, causal
    (0, 2, 80, 128, 2, 1), (0, 3, 150, 96, 3, 1), (0, 2, 64, 64, 4, 0),
    (1, 1, 128, 64, 1, 1), (1, 2, 128, 128, 2, 1), (1, 3, 256, 128, 2, 1), (1, 2, 512, 192, 3, 1), (1, 2, 256, 128, 2, 0),
]


@pytest.mark.parametrize("engine,B,T,D,H,causal", CASES)
def test_attention_matches_fp64(device, engine, B, T, D, H, causal):
    rng = np.random.default_rng(100 * T + D + engine)
    Q, K, V, dO = (rng.standard_normal((B * T, D)).astype(np.float32) * sc for sc in (1.5, 1.5, 1.0, 1.0))
    got = run(device, engine, Q, K, V, dO, B, T, D, H, causal)
    ref = reference(Q, K, V, dO, B, T, D, H, causal)
    # the row statistics are only defined up to the shift of the maximum: compare m + log(l)
    lse_got = got[1].astype(np.float64) + np.log(got[2].astype(np.float64))
    lse_ref = ref[1] + np.log(ref[2])
    assert np.max(np.abs(lse_got - lse_ref)) < 1e-4
    for name, a, b in zip(("O", "dQ", "dK", "dV"), (got[0], got[3], got[4], got[5]), (ref[0], ref[3], ref[4], ref[5])):
        e = norm_err(a, b)
        assert e < TOL, f"{name}: normalised error {e:.3e}"


def test_attention_bounded_waits_fail_fast_and_the_context_stays_usable(device):
    """Failure detection without a GPU fault: with a poll limit of 1 the first wait of the tcgen05 attention kernels runs
    out; the status word is set at once, every other wait of the launch then gives up within a few polls, the kernels run
    their loops to the end and release tensor memory, the call reports GN_ERR_TIMEOUT quickly, and the next call is correct."""
    import time
    from goneuron_b200 import _lib
    L = _lib.load()
    B, T, D, H = 2, 512, 128, 2
    rng = np.random.default_rng(77)
    Q, K, V, dO = (rng.standard_normal((B * T, D)).astype(np.float32) for _ in range(4))
    good = run(device, 1, Q, K, V, dO, B, T, D, H, 1)
    f = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))
    O, dQ, dK, dV = (np.empty_like(Q) for _ in range(4))
    _lib.check(L.gn_ctx_set_spin_limit(device.handle, 1))
    try:
        t0 = time.perf_counter()
        rc = L.gn_op_attention(device.handle, 1, B, T, D, H, 1, f(Q), f(K), f(V), f(dO), f(O), None, None, f(dQ), f(dK), f(dV))
        dt = time.perf_counter() - t0
    finally:
        _lib.check(L.gn_ctx_set_spin_limit(device.handle, 0))
    assert rc == -6 and b"bounded wait" in L.gn_last_error(), (rc, L.gn_last_error())
    assert dt < 5.0, dt
    again = run(device, 1, Q, K, V, dO, B, T, D, H, 1)
    for a, b in zip(good, again):
        assert np.array_equal(a, b)
