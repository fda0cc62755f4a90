"""ctypes binding of the CPU checker (oracle/goneuron_oracle.cpp).

TEST INFRASTRUCTURE: imported only by tests/, by the smoke check and by the
benchmark's CPU-baseline legs.  The shipped package never imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

from goneuron_b200.descriptors import LayerDesc, layers_to_array

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libgoneuron_oracle.so")
_lib = None


def build(force=False):
    """Compile the checker with the Makefile next to this file."""
    src = os.path.join(_HERE, "goneuron_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _SO


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        f32p, i64p = C.POINTER(C.c_float), C.POINTER(C.c_int64)
        L.gno_last_error.restype = C.c_char_p
        L.gno_param_count.argtypes = [C.c_void_p, C.c_int, i64p, i64p, i64p]
        L.gno_train_batch.argtypes = [C.c_void_p, C.c_int, C.c_int, f32p, f32p, f32p, f32p, C.POINTER(C.c_int),
                                      C.c_float, C.c_float, C.c_float, C.c_float, f32p, f32p, C.c_int, C.c_int,
                                      C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, f32p, C.POINTER(C.c_double), f32p]
        L.gno_forward_batch.argtypes = [C.c_void_p, C.c_int, f32p, f32p, C.c_int, f32p, C.c_int, C.c_int, f32p, C.c_int]
        L.gno_state_count.argtypes = [C.c_void_p, C.c_int, i64p]
        L.gno_activation.argtypes = [C.c_int, f32p, C.c_int]
        L.gno_activation_deriv.argtypes = [C.c_int, f32p, C.c_int]
        L.gno_loss.argtypes = [C.c_int, f32p, f32p, C.c_int]
        L.gno_loss.restype = C.c_float
        L.gno_loss_grad.argtypes = [C.c_int, f32p, f32p, f32p, C.c_int]
        L.gno_adam.argtypes = [f32p, f32p, f32p, f32p, C.c_int64, C.c_float, C.c_float, C.c_float, C.c_float, C.c_int, C.c_int]
        L.gno_rope.argtypes = [f32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
        L.gno_gemm_nt.argtypes = [C.c_int, C.c_int, C.c_int, f32p, f32p, f32p, f32p, C.c_int]
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.POINTER(C.c_float)) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def param_count(layers):
    arr = layers_to_array(layers)
    n, i, o = C.c_int64(), C.c_int64(), C.c_int64()
    rc = lib().gno_param_count(arr, len(layers), C.byref(n), C.byref(i), C.byref(o))
    if rc:
        raise ValueError(lib().gno_last_error().decode())
    return n.value, i.value, o.value


class OracleState:
    """Parameters + Adam state of one model, stepped by the CPU checker."""

    def __init__(self, layers, loss_kind, params, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8):
        self.layers = list(layers)
        self.loss_kind = int(loss_kind)
        self.params = _f32(params).copy()
        self.m = np.zeros_like(self.params)
        self.v = np.zeros_like(self.params)
        self.grads = np.zeros_like(self.params)
        n = C.c_int64()
        lib().gno_state_count(layers_to_array(self.layers), len(self.layers), C.byref(n))
        # BatchNorm2D running statistics: mean 0 | variance 1 per layer (batchnorm2d.go:124-128)
        self.state = np.zeros(n.value, np.float32)
        off = 0
        for l in self.layers:
            if l.kind == 11:
                self.state[off + l.in_size:off + 2 * l.in_size] = 1.0
                off += 2 * l.in_size
        self.timestep = 0
        self.lr, self.beta1, self.beta2, self.eps = lr, beta1, beta2, eps
        self.seconds = 0.0

    def train_batch(self, x, y, W=1, threads=1, precision=64, step=True, global_batch=0, first_sample=0):
        x, y = _f32(x), _f32(y)
        batch = x.shape[0]
        arr = layers_to_array(self.layers)
        ts = C.c_int(self.timestep)
        loss = C.c_float()
        sec = C.c_double()
        rc = lib().gno_train_batch(arr, len(self.layers), self.loss_kind, _p(self.params), _p(self.grads), _p(self.m),
                                   _p(self.v), C.byref(ts), self.lr, self.beta1, self.beta2, self.eps, _p(x), _p(y), batch,
                                   W, threads, precision, 1 if step else 0, global_batch, first_sample, C.byref(loss), C.byref(sec), _p(self.state) if self.state.size else None)
        if rc:
            raise ValueError(lib().gno_last_error().decode())
        self.timestep = ts.value
        self.seconds = sec.value
        return loss.value

    def forward_batch(self, x, threads=1, precision=64, training=False):
        x = _f32(x)
        _, _, out = param_count(self.layers)
        res = np.empty((x.shape[0], out), dtype=np.float32)
        arr = layers_to_array(self.layers)
        rc = lib().gno_forward_batch(arr, len(self.layers), _p(self.params), _p(x), x.shape[0], _p(res), threads, precision, _p(self.state) if self.state.size else None, 1 if training else 0)
        if rc:
            raise ValueError(lib().gno_last_error().decode())
        return res


def activation(act, x):
    x = _f32(x).copy()
    lib().gno_activation(int(act), _p(x), x.size)
    return x


def activation_deriv(act, x):
    x = _f32(x).copy()
    lib().gno_activation_deriv(int(act), _p(x), x.size)
    return x


def loss(kind, p, y):
    p, y = _f32(p), _f32(y)
    return lib().gno_loss(int(kind), _p(p), _p(y), p.size)


def loss_grad(kind, p, y):
    p, y = _f32(p), _f32(y)
    g = np.empty_like(p)
    lib().gno_loss_grad(int(kind), _p(p), _p(y), _p(g), p.size)
    return g


def adam(p, g, m, v, lr, b1, b2, eps, t, precision=32):
    p, g, m, v = _f32(p).copy(), _f32(g), _f32(m).copy(), _f32(v).copy()
    lib().gno_adam(_p(p), _p(g), _p(m), _p(v), p.size, lr, b1, b2, eps, t, precision)
    return p, m, v


def rope(x, T, heads, hd, conjugate=False, precision=32):
    """Rotary embeddings on x [T, heads * hd] (transformer.go:212-236)."""
    x = _f32(x).copy()
    if lib().gno_rope(_p(x), T, heads, hd, 1 if conjugate else 0, precision):
        raise ValueError(lib().gno_last_error().decode())
    return x


def gemm_nt(A, B, bias=None, precision=32):
    A, B = _f32(A), _f32(B)
    M, K = A.shape
    N = B.shape[0]
    bias = _f32(bias) if bias is not None else None
    out = np.empty((M, N), dtype=np.float32)
    lib().gno_gemm_nt(M, N, K, _p(A), _p(B), _p(bias), _p(out), precision)
    return out
