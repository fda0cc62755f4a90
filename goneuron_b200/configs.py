"""The five benchmark models as layer lists, and their seeded synthetic inputs.

Weights are Glorot-uniform from a seed and uploaded through the flat parameter buffer on
both sides of every comparison: the reference's own constructors leave the parameters of
MultiHeadAttention / TransformerBlock at zero (their Build re-binds sub-layers to fresh
buffers, internal/layer/transformer.go:367-379, :1035-1056), so initial weights are always
supplied by the caller.  Flat layout = Network.initBuffers (internal/net/net.go:91-127)."""
import math

import numpy as np

from . import descriptors as D


def mlp(in_size=784, hidden=128, classes=10):
    return [D.Dense(in_size, hidden, D.RELU), D.Dense(hidden, classes, D.SOFTMAX)], D.CROSS_ENTROPY


def cnn(hw=32, c0=3, c1=16, c2=32, classes=10):
    h2, h4 = hw // 2, hw // 4
    return [D.Conv2D(c0, c1, 3, 1, 1, D.RELU, hw, hw), D.MaxPool2D(c1, 2, 2, 0, hw, hw),
            D.Conv2D(c1, c2, 3, 1, 1, D.RELU, h2, h2), D.MaxPool2D(c2, 2, 2, 0, h2, h2),
            D.Flatten(), D.Dense(c2 * h4 * h4, classes, D.SOFTMAX)], D.CROSS_ENTROPY


def mlp_ln(in_size=24, hidden=48, norm=16, classes=4):
    """Dense -> LayerNorm over consecutive rows of `norm` -> Dense: exercises the stand-alone LayerNorm layer."""
    return [D.Dense(in_size, hidden, D.TANH), D.LayerNorm(norm), D.Dense(hidden, classes, D.SOFTMAX)], D.CROSS_ENTROPY


def cnn1d(length=40, c0=3, c1=8, c2=6, classes=4, act=D.RELU):
    """Conv1D -> Conv1D (stride 2) -> Flatten -> Dense: exercises Conv1D (conv1d.go), whose backward pass ignores the
    activation's derivative."""
    l2 = (length + 2 - 3) // 2 + 1
    return [D.Conv1D(c0, c1, 5, 1, 2, act, length), D.Conv1D(c1, c2, 3, 2, 1, D.TANH, length), D.Flatten(),
            D.Dense(c2 * l2, classes, D.SOFTMAX)], D.CROSS_ENTROPY


def mlp_rms(in_size=24, hidden=48, norm=16, classes=4):
    """Dense -> RMSNorm over consecutive rows of `norm` -> Dense: exercises RMSNorm (rmsnorm.go)."""
    return [D.Dense(in_size, hidden, D.TANH), D.RMSNorm(norm), D.Dense(hidden, classes, D.SOFTMAX)], D.CROSS_ENTROPY


def mlp_act(act=D.GELU, alpha=None, in_size=20, hidden=32, classes=4):
    """Dense(act) -> Dense(act) -> Dense(softmax): exercises the element-wise activations (activations.go)."""
    return [D.Dense(in_size, hidden, act, alpha), D.Dense(hidden, hidden, act, alpha), D.Dense(hidden, classes, D.SOFTMAX)], D.CROSS_ENTROPY


def mlp_drop(in_size=40, hidden=64, classes=5, p=0.3):
    """Dense -> Dropout -> Dense: exercises Dropout's mask stream (dropout.go)."""
    return [D.Dense(in_size, hidden, D.RELU), D.Dropout(p, hidden), D.Dense(hidden, classes, D.SOFTMAX)], D.CROSS_ENTROPY


def cnn_avg(hw=12, c0=2, c1=6, classes=4):
    """Conv -> AvgPool2D with overlapping, padded windows -> Flatten -> Dense: exercises AvgPool2D (avgpool2d.go)."""
    oh = (hw + 2 - 3) // 2 + 1
    return [D.Conv2D(c0, c1, 3, 1, 1, D.RELU, hw, hw), D.AvgPool2D(c1, 3, 2, 1, hw, hw), D.Flatten(),
            D.Dense(c1 * oh * oh, classes, D.SOFTMAX)], D.CROSS_ENTROPY


def cnn_bn(hw=16, c0=3, c1=8, classes=5):
    """Conv -> BatchNorm2D -> MaxPool -> Flatten -> Dense: exercises BatchNorm2D (used by the reference's CIFAR example)."""
    h2 = hw // 2
    return [D.Conv2D(c0, c1, 3, 1, 1, D.RELU, hw, hw), D.BatchNorm2D(c1, hw, hw), D.MaxPool2D(c1, 2, 2, 0, hw, hw),
            D.Flatten(), D.Dense(c1 * h2 * h2, classes, D.SOFTMAX)], D.CROSS_ENTROPY


def recurrent(in_size=16, hidden=128, seq_len=64):
    return [D.SequenceUnrollerLSTM(in_size, hidden, seq_len, False), D.Dense(hidden, 1, D.LINEAR)], D.MSE


def recurrent_gru(in_size=16, hidden=64, seq_len=24, return_seq=False):
    """SequenceUnroller(GRU) -> Dense: exercises the GRU layer (gru.go) with its literal backward pass."""
    out = hidden * seq_len if return_seq else hidden
    return [D.SequenceUnrollerGRU(in_size, hidden, seq_len, return_seq), D.Dense(out, 2, D.LINEAR)], D.MSE


def transformer(vocab, dim, seq_len, heads, ff_dim, n_blocks, ff_act=D.RELU, rms_norm=False, rope=False, causal=True):
    """The benchmark Transformers are causal with CLS pooling of token 0, so only token 0 of a sequence ever receives a
    gradient; causal=False lets every token contribute (used by the tests of the block variants)."""
    layers = [D.Embedding(vocab, dim, seq_len), D.PositionalEncoding(seq_len, dim)]
    layers += [D.TransformerBlock(dim, heads, seq_len, ff_dim, causal, ff_act, rms_norm, rope) for _ in range(n_blocks)]
    layers += [D.CLSPooling(seq_len, dim), D.Dense(dim, vocab, D.LOGSOFTMAX)]
    return layers, D.CROSS_ENTROPY


CONFIGS = {
    # name: (builder, kwargs, batch, lr)
    "mlp": (mlp, {}, 64, 1e-3),
    "cnn": (cnn, {}, 128, 1e-3),
    "cnn_bn": (cnn_bn, {}, 32, 1e-3),
    "cnn_avg": (cnn_avg, {}, 16, 1e-3),
    "mlp_drop": (mlp_drop, {}, 24, 1e-3),
    "mlp_act": (mlp_act, {}, 12, 1e-3),
    "mlp_rms": (mlp_rms, {}, 16, 1e-3),
    "cnn1d": (cnn1d, {}, 12, 1e-3),
    "mlp_ln": (mlp_ln, {}, 16, 1e-3),
    "lstm": (recurrent, {}, 256, 1e-3),
    "gru": (recurrent_gru, {}, 32, 1e-3),
    "transformer_small": (transformer, dict(vocab=8192, dim=256, seq_len=128, heads=8, ff_dim=1024, n_blocks=4), 64, 3e-4),
    "transformer_large": (transformer, dict(vocab=32000, dim=1024, seq_len=512, heads=16, ff_dim=4096, n_blocks=8), 256, 1e-4),
}
SEEDS = {"gru": 1247, "cnn1d": 1246, "mlp_rms": 1245, "mlp_act": 1244, "mlp_drop": 1243, "cnn_avg": 1242, "mlp_ln": 1241, "cnn_bn": 1240, "mlp": 1235, "cnn": 1236, "lstm": 1237, "transformer_small": 1238, "transformer_large": 1239}


def build(name, **override):
    fn, kw, batch, lr = CONFIGS[name]
    kw = dict(kw)
    kw.update(override)
    layers, loss = fn(**kw)
    return layers, loss, batch, lr


def _glorot(rng, shape, fan_in, fan_out):
    a = math.sqrt(6.0 / (fan_in + fan_out))
    return rng.uniform(-a, a, size=shape).astype(np.float32)


def _dense_params(rng, i, o):
    return [_glorot(rng, (o, i), i, o).ravel(), np.zeros(o, np.float32)]


def init_params(layers, rng):
    """Flat parameter vector in the reference's layout, Glorot-uniform weights, zero biases,
    LSTM forget-gate bias 1 (lstm.go:191-193), LayerNorm gamma 1 / beta 0, Embedding
    U(+-sqrt(3/d)) (embedding.go:50), positional table U(+-sqrt(1/d)) (transformer.go:60)."""
    parts = []
    for l in layers:
        k = l.kind
        if k == D.DENSE:
            parts += _dense_params(rng, l.in_size, l.out_size)
        elif k == D.CONV2D:
            kk = l.kernel * l.kernel
            parts += [_glorot(rng, (l.out_size, l.in_size, l.kernel, l.kernel), l.in_size * kk, l.out_size * kk).ravel(),
                      np.zeros(l.out_size, np.float32)]
        elif k == D.CONV1D:
            parts += [_glorot(rng, (l.out_size, l.in_size, l.kernel), l.in_size * l.kernel, l.out_size * l.kernel).ravel(),
                      rng.uniform(-0.1, 0.1, size=l.out_size).astype(np.float32)]
        elif k == D.LSTM_UNROLLED:
            H, i = l.out_size, l.in_size
            b = np.zeros(4 * H, np.float32)
            b[H:2 * H] = 1.0
            parts += [_glorot(rng, (4 * H, i), i, H).ravel(), _glorot(rng, (4 * H, H), H, H).ravel(), b]
        elif k == D.GRU_UNROLLED:
            H, i = l.out_size, l.in_size
            parts += [_glorot(rng, (3 * H, i), i, H).ravel(), _glorot(rng, (2 * H, H), H, H).ravel(), rng.uniform(-0.1, 0.1, size=3 * H).astype(np.float32)]
        elif k == D.EMBEDDING:
            a = math.sqrt(3.0 / l.out_size)
            parts.append(rng.uniform(-a, a, size=l.in_size * l.out_size).astype(np.float32))
        elif k == D.POSENC:
            a = math.sqrt(1.0 / l.dim)
            parts.append(rng.uniform(-a, a, size=l.seq_len * l.dim).astype(np.float32))
        elif k == D.TRANSFORMER_BLOCK:
            d, f = l.dim, l.ff_dim
            for _ in range(4):
                parts += _dense_params(rng, d, d)
            if l.kernel:                                   # RMSNorm: gain only
                parts += [rng.uniform(0.8, 1.2, size=d).astype(np.float32) for _ in range(2)]
            else:
                parts += [np.ones(d, np.float32), np.zeros(d, np.float32)] * 2
            if l.activation == D.SILU:                     # SwiGLU: gate and up projections, no biases
                parts += [_glorot(rng, (f, d), d, f).ravel(), _glorot(rng, (f, d), d, f).ravel()]
            else:
                parts += _dense_params(rng, d, f)
            parts += _dense_params(rng, f, d)
        elif k == D.LAYERNORM:
            parts += [np.ones(l.dim, np.float32), np.zeros(l.dim, np.float32)]
        elif k == D.RMSNORM:
            parts.append(rng.uniform(0.5, 1.5, size=l.dim).astype(np.float32))
        elif k == D.BATCHNORM2D:
            parts += [rng.uniform(0.5, 1.5, size=l.in_size).astype(np.float32), rng.uniform(-0.5, 0.5, size=l.in_size).astype(np.float32)]
    return np.concatenate(parts) if parts else np.zeros(0, np.float32)


class ReferenceRNG:
    """The reference's own generator (internal/layer/layer.go:61-75): the 64-bit LCG s <- s * 6364136223846793005 + 1,
    RandFloat() = float32(s >> 33) / float32(1 << 31).  Vectorised: n consecutive outputs by doubling (the m-step map of an
    affine recurrence is again affine), in wrapping uint64 arithmetic."""
    A = np.uint64(6364136223846793005)

    def __init__(self, seed):
        self.state = np.uint64(seed & 0xFFFFFFFFFFFFFFFF)

    def rand_float(self, n):
        """The next n values of RandFloat() as float32."""
        if n <= 0:
            return np.zeros(0, np.float32)
        with np.errstate(over="ignore"):
            st = np.empty(n, np.uint64)
            st[0] = self.state * self.A + np.uint64(1)
            am, cm, m = self.A, np.uint64(1), 1            # the m-step map s -> am * s + cm
            while m < n:
                k = min(m, n - m)
                st[m:m + k] = st[:k] * am + cm
                cm = am * cm + cm
                am = am * am
                m *= 2
        self.state = st[-1]
        return (st >> np.uint64(33)).astype(np.float32) / np.float32(1 << 31)


def reference_init_params(layers):
    """Flat parameter vector exactly as the reference's constructors initialise it, generator seeds included
    (Dense: layer.go:312-319, seed in*1000 + out*100 + 42; Conv2D: conv2d.go:126-134, seed 42; LSTM: lstm.go:181-200, seed
    in*1000 + out*100 + 142, forget-gate bias 1; Embedding: embedding.go:50-56, seed 42; positional table:
    transformer.go:58-63, seed T + d + 42; LayerNorm gamma 1 / beta 0: layernorm.go:92-95).  Every expression is evaluated in
    float32, operation by operation, as the Go code does.  Equal-shaped layers start identical, as in the reference.
    TransformerBlock parameters are all zero after the reference's Build (transformer.go:367-379, :1035-1056): they are
    returned as zeros here too, which is why the Transformer configs are always run with uploaded weights instead."""
    f32 = np.float32
    parts = []
    for l in layers:
        k = l.kind
        if k == D.DENSE:
            i, o = l.in_size, l.out_size
            scale = f32(math.sqrt(2.0 / (float(i) + float(o))))
            rng = ReferenceRNG(i * 1000 + o * 100 + 42)
            w = rng.rand_float(o * i) * f32(2) * scale - scale
            b = rng.rand_float(o) * f32(0.2) - f32(0.1)
            parts += [w.astype(f32), b.astype(f32)]
        elif k == D.CONV2D:
            n = l.out_size * l.in_size * l.kernel * l.kernel
            scale = f32(math.sqrt(2.0 / float(l.in_size * l.kernel * l.kernel)))
            rng = ReferenceRNG(42)
            w = rng.rand_float(n) * f32(2) * scale - scale
            b = rng.rand_float(l.out_size) * f32(0.2) - f32(0.1)
            parts += [w.astype(f32), b.astype(f32)]
        elif k == D.LSTM_UNROLLED:
            H, i = l.out_size, l.in_size
            si = f32(math.sqrt(2.0 / float(i + 4 * H))); sr = f32(math.sqrt(2.0 / float(H + 4 * H)))
            rng = ReferenceRNG(i * 1000 + H * 100 + 142)
            r = rng.rand_float(4 * H * (i + H)).reshape(4 * H, i + H)        # per gate row: in input weights, then H recurrent weights
            wx = r[:, :i] * f32(2) * si - si
            wh = r[:, i:] * f32(2) * sr - sr
            b = np.zeros(4 * H, f32); b[H:2 * H] = 1.0
            parts += [np.ascontiguousarray(wx, f32).ravel(), np.ascontiguousarray(wh, f32).ravel(), b]
        elif k == D.GRU_UNROLLED:
            H, i = l.out_size, l.in_size                                      # gru.go:126-147, seed in*1000 + out*100 + 242, biases zero
            scale = f32(math.sqrt(2.0 / (float(i) + float(H))))
            rng = ReferenceRNG(i * 1000 + H * 100 + 242)
            wx = rng.rand_float(3 * H * i) * f32(2) * scale - scale
            wh = rng.rand_float(2 * H * H) * f32(2) * scale - scale
            parts += [wx.astype(f32), wh.astype(f32), np.zeros(3 * H, f32)]
        elif k == D.EMBEDDING:
            scale = f32(math.sqrt(3.0 / float(l.out_size)))
            parts.append((scale * (f32(2) * ReferenceRNG(42).rand_float(l.in_size * l.out_size) - f32(1))).astype(f32))
        elif k == D.POSENC:
            scale = f32(math.sqrt(1.0 / float(l.dim)))
            parts.append((ReferenceRNG(l.seq_len + l.dim + 42).rand_float(l.seq_len * l.dim) * f32(2) * scale - scale).astype(f32))
        elif k == D.TRANSFORMER_BLOCK:
            d, f = l.dim, l.ff_dim
            n_norm = 2 * d if l.kernel else 4 * d
            n_ff1 = 2 * d * f if l.activation == D.SILU else d * f + f
            parts.append(np.zeros(4 * (d * d + d) + n_norm + n_ff1 + (f * d + d), f32))
        elif k == D.LAYERNORM:
            parts += [np.ones(l.dim, f32), np.zeros(l.dim, f32)]
        elif k in (D.RMSNORM,):
            parts.append(np.ones(l.dim, f32))
        elif k == D.BATCHNORM2D:
            parts += [np.ones(l.in_size, f32), np.zeros(l.in_size, f32)]
        elif k == D.CONV1D:
            raise ValueError("reference_init_params: Conv1D is not one of the layers whose reference initialiser is restated")
    return np.concatenate(parts) if parts else np.zeros(0, f32)


def make_inputs(name, layers, batch, rng):
    """Seeded synthetic batch with the shapes and value distributions the benchmark names."""
    first, last = layers[0], layers[-1]
    if first.kind == D.EMBEDDING:
        T = first.seq_len
        x = rng.integers(0, first.in_size, size=(batch, T)).astype(np.float32)
        tgt = rng.integers(0, last.out_size, size=batch)
        y = np.zeros((batch, last.out_size), np.float32)
        y[np.arange(batch), tgt] = 1.0
    elif first.kind in (D.LSTM_UNROLLED, D.GRU_UNROLLED):
        x = rng.standard_normal((batch, first.seq_len * first.in_size)).astype(np.float32)
        y = rng.standard_normal((batch, last.out_size)).astype(np.float32)
    elif first.kind == D.CONV1D:
        x = rng.standard_normal((batch, first.in_size * first.in_w)).astype(np.float32)
        tgt = rng.integers(0, last.out_size, size=batch)
        y = np.zeros((batch, last.out_size), np.float32)
        y[np.arange(batch), tgt] = 1.0
    elif first.kind == D.CONV2D:
        x = rng.standard_normal((batch, first.in_size * first.in_h * first.in_w)).astype(np.float32)
        tgt = rng.integers(0, last.out_size, size=batch)
        y = np.zeros((batch, last.out_size), np.float32)
        y[np.arange(batch), tgt] = 1.0
    else:
        x = rng.random((batch, first.in_size), dtype=np.float32)
        tgt = rng.integers(0, last.out_size, size=batch)
        y = np.zeros((batch, last.out_size), np.float32)
        y[np.arange(batch), tgt] = 1.0
    return x, y


def make_case(name, batch=None, seed=None, init="glorot", **override):
    """(layers, loss, params, x, y, lr) for a named config; draw order weights -> inputs -> labels.
    init = "reference" replaces the seeded Glorot weights by the reference's own deterministic initialisation."""
    layers, loss, b, lr = build(name, **override)
    batch = batch or b
    rng = np.random.Generator(np.random.PCG64(seed if seed is not None else SEEDS[name]))
    params = init_params(layers, rng)
    if init == "reference":
        params = reference_init_params(layers)
    x, y = make_inputs(name, layers, batch, rng)
    return layers, loss, params, x, y, lr
