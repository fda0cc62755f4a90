"""The per-layer entry points (gn_op_layernorm, gn_op_conv2d, gn_op_softmax_ce, gn_op_lstm): one layer's kernels on host
arrays through the C ABI, each against the CPU checker where a one-layer model expresses it (Conv2D) and against a
float64 numpy restatement of the reference's formulas otherwise.  Tolerance 1e-4 normalised, as for whole steps."""
import ctypes as C

import numpy as np
import pytest

from goneuron_b200 import descriptors as D
from tests.parity import TOL, norm_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    from goneuron_b200.sequential import Device
    d = Device(0)
    yield d
    d.close()


def _f(a):
    return a.ctypes.data_as(C.POINTER(C.c_float)) if a is not None else None


@pytest.mark.parametrize("rows,n", [(37, 48), (64, 1024), (9, 1100), (300, 512)])
def test_layernorm_op(device, rows, n):
    """layernorm.go:193-304 forward; :385-441 backward, whose second term is divided by N * std^2."""
    from goneuron_b200 import _lib
    rng = np.random.default_rng(rows + n)
    x = rng.standard_normal((rows, n)).astype(np.float32) * 2 + 0.3
    gamma, beta = rng.uniform(0.5, 1.5, n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    dy = rng.standard_normal((rows, n)).astype(np.float32)
    y, dx, dg, db = np.empty_like(x), np.empty_like(x), np.empty(n, np.float32), np.empty(n, np.float32)
    _lib.check(_lib.load().gn_op_layernorm(device.handle, rows, n, _f(x), _f(gamma), _f(beta), _f(dy), _f(y), _f(dx), _f(dg), _f(db)))
    X, G, U = x.astype(np.float64), gamma.astype(np.float64), dy.astype(np.float64)
    mu = X.mean(1, keepdims=True); xc = X - mu; sd = np.sqrt((xc ** 2).mean(1, keepdims=True) + 1e-5)
    assert norm_err(y, G * xc / sd + beta) <= TOL
    q = U * G
    dx_ref = (q - q.sum(1, keepdims=True) / n) / sd - xc * (q * xc).sum(1, keepdims=True) / (n * sd ** 2)
    assert norm_err(dx, dx_ref) <= TOL
    assert norm_err(dg, (U * xc / sd).sum(0)) <= TOL and norm_err(db, U.sum(0)) <= TOL


@pytest.mark.parametrize("engine", [0, 1])
@pytest.mark.parametrize("shape", [dict(B=6, inC=3, outC=16, k=3, s=1, p=1, H=32, W=32, act=D.RELU),
                                   dict(B=5, inC=16, outC=32, k=3, s=1, p=1, H=16, W=16, act=D.RELU),
                                   dict(B=3, inC=2, outC=5, k=5, s=1, p=2, H=11, W=9, act=D.TANH),
                                   dict(B=4, inC=3, outC=4, k=3, s=2, p=1, H=13, W=13, act=D.LINEAR)])
def test_conv2d_op(device, oracle, engine, shape):
    """One Conv2D layer, both engines, against the CPU checker's one-layer model (conv2d.go:716-959, :997-1174): output, weight
    and bias gradients; the input gradient against the transposed convolution in float64."""
    from goneuron_b200 import _lib
    B, inC, outC, k, s, p, H, W, act = (shape[q] for q in ("B", "inC", "outC", "k", "s", "p", "H", "W", "act"))
    oH, oW = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
    rng = np.random.default_rng(B * 100 + inC * 10 + outC)
    x = rng.standard_normal((B, inC * H * W)).astype(np.float32)
    w = (rng.standard_normal(outC * inC * k * k) * 0.3).astype(np.float32)
    bias = (rng.standard_normal(outC) * 0.1).astype(np.float32)
    t = rng.standard_normal((B, outC * oH * oW)).astype(np.float32)
    layers = [D.Conv2D(inC, outC, k, s, p, act, H, W)]
    params = np.concatenate([w, bias])
    ref = oracle.OracleState(layers, D.MSE, params)
    y_ref = ref.forward_batch(x, threads=2, precision=64)
    ref.train_batch(x, t, threads=2, precision=64, step=False)
    n_out = outC * oH * oW
    dy = (2.0 / n_out * (y_ref.astype(np.float64) - t)).astype(np.float32)          # MSE gradient (loss.go:86-105)
    y, dx = np.empty_like(y_ref), np.empty_like(x)
    dw, db = np.empty_like(w), np.empty_like(bias)
    _lib.check(_lib.load().gn_op_conv2d(device.handle, engine, B, inC, outC, k, s, p, H, W, act, _f(x), _f(w), _f(bias), _f(dy), _f(y), _f(dx), _f(dw), _f(db)))
    assert norm_err(y, y_ref) <= TOL
    nW = w.size
    assert norm_err(dw / B, ref.grads[:nW]) <= TOL and norm_err(db / B, ref.grads[nW:]) <= TOL       # the checker's gradients are batch means
    # input gradient: dz = dy * act'(z), dx = transposed convolution of dz with w
    X = x.reshape(B, inC, H, W).astype(np.float64); Wt = w.reshape(outC, inC, k, k).astype(np.float64)
    Xp = np.pad(X, ((0, 0), (0, 0), (p, p), (p, p)))
    z = np.zeros((B, outC, oH, oW))
    for kh in range(k):
        for kw in range(k):
            z += np.einsum("bchw,oc->bohw", Xp[:, :, kh:kh + s * oH:s, kw:kw + s * oW:s], Wt[:, :, kh, kw])
    z += bias.astype(np.float64)[None, :, None, None]
    der = {D.RELU: (z > 0).astype(np.float64), D.LINEAR: np.ones_like(z), D.TANH: 1 - np.tanh(z) ** 2}[act]
    dz = dy.reshape(B, outC, oH, oW).astype(np.float64) * der
    dxp = np.zeros_like(Xp)
    for kh in range(k):
        for kw in range(k):
            dxp[:, :, kh:kh + s * oH:s, kw:kw + s * oW:s] += np.einsum("bohw,oc->bchw", dz, Wt[:, :, kh, kw])
    dx_ref = dxp[:, :, p:p + H, p:p + W].reshape(B, -1)
    assert norm_err(dx, dx_ref) <= TOL


@pytest.mark.parametrize("B,V,logsm", [(7, 10, 0), (5, 8192, 1), (3, 32000, 1), (4, 33, 0)])
def test_softmax_ce_op(device, B, V, logsm):
    """Head + CrossEntropy: probabilities / log-probabilities, the clipped loss (loss.go:129-138) and the gradient after the
    second application of the head's Jacobian (loss.go:165-178 with layer.go:504-560)."""
    from goneuron_b200 import _lib
    rng = np.random.default_rng(V + B)
    z = (rng.standard_normal((B, V)) * 2).astype(np.float32)
    y = np.zeros((B, V), np.float32); y[np.arange(B), rng.integers(0, V, B)] = 1
    out, loss, dz = np.empty_like(z), np.empty(B, np.float32), np.empty_like(z)
    _lib.check(_lib.load().gn_op_softmax_ce(device.handle, B, V, logsm, _f(z), _f(y), _f(out), _f(loss), _f(dz)))
    Z = z.astype(np.float64); Z = Z - Z.max(1, keepdims=True)
    ls = Z - np.log(np.exp(Z).sum(1, keepdims=True)); pr = np.exp(ls)
    a = ls if logsm else pr
    assert norm_err(out, a) <= TOL
    assert norm_err(loss, -(y * np.log(np.maximum(a, 1e-10))).sum(1)) <= TOL
    u = a - y
    dz_ref = u - pr * u.sum(1, keepdims=True) if logsm else pr * (u - (u * pr).sum(1, keepdims=True))
    assert norm_err(dz, dz_ref) <= TOL


@pytest.mark.parametrize("engine", [0, 1])
@pytest.mark.parametrize("B,T,I,H", [(5, 7, 5, 24), (9, 64, 16, 128)])
def test_lstm_op(device, engine, B, T, I, H):
    """The literal recurrence (lstm.go:276-407: only the input gate receives wx x + wh h) and the gate deltas of
    back-propagation through time with the carried hidden gradient (lstm.go:476-691, unroller.go:190-209)."""
    from goneuron_b200 import _lib
    rng = np.random.default_rng(B + T + H)
    x = rng.standard_normal((B, T * I)).astype(np.float32)
    wx, wh = (rng.standard_normal((4 * H, I)) * 0.4).astype(np.float32), (rng.standard_normal((4 * H, H)) * 0.2).astype(np.float32)
    b = (rng.standard_normal(4 * H) * 0.3).astype(np.float32); b[H:2 * H] += 1
    g_last = rng.standard_normal((B, H)).astype(np.float32)
    h_all, c_all, dgate = np.empty((B, T, H), np.float32), np.empty((B, T, H), np.float32), np.empty((B, T, 4 * H), np.float32)
    _lib.check(_lib.load().gn_op_lstm(device.handle, engine, B, T, I, H, _f(x), _f(wx), _f(wh), _f(b), _f(g_last), _f(h_all), _f(c_all), _f(dgate)))
    sig = lambda v: 1 / (1 + np.exp(-v))
    X, Wx, Wh, bb = x.reshape(B, T, I).astype(np.float64), wx.astype(np.float64), wh.astype(np.float64), b.astype(np.float64)
    f, gc, o = sig(bb[H:2 * H]), np.tanh(bb[2 * H:3 * H]), sig(bb[3 * H:])
    h, c = np.zeros((B, H)), np.zeros((B, H)); Hs, Cs, Is = [], [], []
    for t in range(T):
        i = sig(bb[:H] + X[:, t] @ Wx[:H].T + h @ Wh[:H].T)
        c = f * c + i * gc; h = o * np.tanh(c)
        Hs.append(h); Cs.append(c); Is.append(i)
    assert norm_err(h_all, np.stack(Hs, 1)) <= TOL and norm_err(c_all, np.stack(Cs, 1)) <= TOL
    G, dc_next, Dref = g_last.astype(np.float64), np.zeros((B, H)), np.zeros((B, T, 4 * H))
    for t in range(T - 1, -1, -1):
        tc = np.tanh(Cs[t]); cprev = Cs[t - 1] if t > 0 else np.zeros((B, H))
        dc = G * o * (1 - tc ** 2) + dc_next
        d = np.concatenate([dc * gc * Is[t] * (1 - Is[t]), dc * cprev * f * (1 - f), dc * Is[t] * (1 - gc ** 2), G * tc * o * (1 - o)], 1)
        dc_next = dc * f
        Dref[:, t] = d
        G = G + d @ Wh                                                       # carried, not replaced
    assert norm_err(dgate, Dref) <= TOL
