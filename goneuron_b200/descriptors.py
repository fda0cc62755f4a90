"""Layer descriptors: the Python mirror of `gn_layer_desc` (include/goneuron_cuda.h) and
constructors named after the reference's (goneuron/goneuron.go:59-340, internal/layer)."""
import ctypes as C

# gn_layer_kind
DENSE, CONV2D, MAXPOOL2D, FLATTEN, LSTM_UNROLLED, EMBEDDING, POSENC, TRANSFORMER_BLOCK, CLS_POOLING, LAYERNORM, BATCHNORM2D, AVGPOOL2D, DROPOUT, RMSNORM, CONV1D, GRU_UNROLLED = range(1, 17)
# gn_activation
LINEAR, RELU, SIGMOID, TANH, SOFTMAX, LOGSOFTMAX, GELU, SILU, LEAKY_RELU, ELU = range(10)
# gn_loss_kind
MSE, CROSS_ENTROPY = 0, 1


class LayerDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "kind", "activation", "in_size", "out_size", "kernel", "stride", "padding", "in_h", "in_w",
        "seq_len", "dim", "heads", "ff_dim", "causal", "return_seq", "reserved")]

    def __repr__(self):
        return "LayerDesc(" + ", ".join(f"{n}={getattr(self, n)}" for n, _ in self._fields_ if getattr(self, n)) + ")"


def layers_to_array(layers):
    arr = (LayerDesc * len(layers))()
    for i, l in enumerate(layers):
        arr[i] = l
    return arr


def Dense(in_size, out_size, activation=LINEAR, alpha=None):
    """layer.NewDense(in, out, act) -- internal/layer/layer.go:224-340.  `alpha`: slope / scale of LEAKY_RELU / ELU
    (activations.NewLeakyReLU, NewELU); None selects 0.01 / 1."""
    return LayerDesc(kind=DENSE, in_size=in_size, out_size=out_size, activation=activation, reserved=0 if alpha is None else _float_bits(alpha))


def Conv2D(in_channels, out_channels, kernel, stride, padding, activation, in_h, in_w, alpha=None):
    """layer.NewConv2D(inC, outC, k, stride, pad, act) + SetInputDimensions(h, w) -- conv2d.go:60-140, :686-691."""
    return LayerDesc(kind=CONV2D, in_size=in_channels, out_size=out_channels, kernel=kernel, stride=stride,
                     padding=padding, activation=activation, in_h=in_h, in_w=in_w, reserved=0 if alpha is None else _float_bits(alpha))


def Conv1D(in_channels, out_channels, kernel, stride, padding, activation, length, alpha=None):
    """layer.NewConv1D(inC, outC, k, stride, pad, act) on inputs of `length` positions -- conv1d.go:65."""
    return LayerDesc(kind=CONV1D, in_size=in_channels, out_size=out_channels, kernel=kernel, stride=stride, padding=padding,
                     activation=activation, in_w=length, reserved=0 if alpha is None else _float_bits(alpha))


def RMSNorm(dim, eps=1e-5):
    """layer.NewRMSNorm(dim, eps), applied to consecutive rows of `dim` -- rmsnorm.go:49."""
    return LayerDesc(kind=RMSNORM, dim=dim, reserved=_float_bits(eps))


def Dropout(p, in_size):
    """layer.NewDropout(p, inSize) -- dropout.go:36."""
    return LayerDesc(kind=DROPOUT, in_size=in_size, dim=_float_bits(p))


def AvgPool2D(in_channels, kernel, stride, padding, in_h, in_w):
    """layer.NewAvgPool2D(inC, k, stride, pad) -- avgpool2d.go:43."""
    return LayerDesc(kind=AVGPOOL2D, in_size=in_channels, kernel=kernel, stride=stride, padding=padding, in_h=in_h, in_w=in_w)


def MaxPool2D(in_channels, kernel, stride, padding, in_h, in_w):
    """layer.NewMaxPool2D(inC, k, stride, pad) -- maxpool2d.go:46."""
    return LayerDesc(kind=MAXPOOL2D, in_size=in_channels, kernel=kernel, stride=stride, padding=padding, in_h=in_h, in_w=in_w)


def Flatten():
    """layer.NewFlatten() -- reshape.go:64-96."""
    return LayerDesc(kind=FLATTEN)


def SequenceUnrollerLSTM(in_size, hidden, seq_len, return_seq=False):
    """layer.NewSequenceUnroller(layer.NewLSTM(in, hidden), T, returnSeq) -- unroller.go:57, lstm.go:276."""
    return LayerDesc(kind=LSTM_UNROLLED, in_size=in_size, out_size=hidden, seq_len=seq_len, return_seq=int(return_seq))


def SequenceUnrollerGRU(in_size, hidden, seq_len, return_seq=False):
    """layer.NewSequenceUnroller(layer.NewGRU(in, hidden), T, returnSeq) -- unroller.go:57, gru.go:81."""
    return LayerDesc(kind=GRU_UNROLLED, in_size=in_size, out_size=hidden, seq_len=seq_len, return_seq=int(return_seq))


def Embedding(vocab, dim, seq_len=0):
    """layer.NewEmbedding(vocab, dim) -- embedding.go:30-60."""
    return LayerDesc(kind=EMBEDDING, in_size=vocab, out_size=dim, seq_len=seq_len)


def PositionalEncoding(seq_len, dim):
    """layer.NewPositionalEncoding(T, dim) -- transformer.go:12-84."""
    return LayerDesc(kind=POSENC, seq_len=seq_len, dim=dim)


def TransformerBlock(dim, heads, seq_len, ff_dim, causal=True, ff_act=RELU, rms_norm=False, rope=False):
    """layer.NewTransformerBlock(dim, heads, T, ffDim, causal) -- transformer.go:859-1279; with the keyword arguments
    layer.NewTransformerBlockExt(..., actType, normType, useRoPE) -- transformer.go:899-957: ff_act RELU (ActReLU), GELU
    (ActGELU) or SILU (ActSwiGLU: the first feed-forward layer is a SwiGLU, swiglu.go); rms_norm selects RMSNorm (NormRMS);
    rope applies rotary embeddings to q and k (transformer.go:212-236).  Descriptor fields: activation, kernel, stride."""
    return LayerDesc(kind=TRANSFORMER_BLOCK, dim=dim, heads=heads, seq_len=seq_len, ff_dim=ff_dim, causal=int(causal),
                     activation=0 if ff_act == RELU else ff_act, kernel=int(bool(rms_norm)), stride=int(bool(rope)))


def CLSPooling(seq_len, dim):
    """layer.NewCLSPooling(T, dim) -- transformer.go:1647-1777."""
    return LayerDesc(kind=CLS_POOLING, seq_len=seq_len, dim=dim)


def LayerNorm(dim):
    """layer.NewLayerNorm(dim, 1e-5, true) applied to consecutive rows of `dim` -- layernorm.go:193-441."""
    return LayerDesc(kind=LAYERNORM, dim=dim)


def _float_bits(v):
    import struct
    return struct.unpack("<i", struct.pack("<f", v))[0]


def BatchNorm2D(num_features, in_h, in_w, eps=1e-5, momentum=0.1):
    """layer.NewBatchNorm2D(C, eps, momentum, affine=true) + SetInputDimensions(h, w) -- batchnorm2d.go:67-160."""
    return LayerDesc(kind=BATCHNORM2D, in_size=num_features, in_h=in_h, in_w=in_w, dim=_float_bits(momentum), reserved=_float_bits(eps))
