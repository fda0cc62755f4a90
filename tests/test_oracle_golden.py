"""Pins the CPU checker (float instantiation) to the reference's own golden vectors and
known-answer tables (tests/golden/reference_fixtures.json, made by make_reference_fixtures.py).
Tolerances are the reference's: internal/validation/pytorch_validation_test.go:164-344."""
import json
import os

import numpy as np
import pytest

from goneuron_b200 import descriptors as D

FX = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_fixtures.json")))


@pytest.mark.parametrize("case", ["dense_simple", "dense_batch"])
def test_dense_forward(oracle, case):
    f = FX[case]
    out = oracle.gemm_nt(np.array(f["input"]), np.array(f["weights"]), np.array(f["biases"]))
    np.testing.assert_allclose(out, np.array(f["output"], np.float32), atol=1e-4, rtol=0)
    # the same numbers through a one-layer Network forward
    layers = [D.Dense(4, 3, D.LINEAR)]
    st = oracle.OracleState(layers, D.MSE, np.concatenate([np.array(f["weights"], np.float32).ravel(), np.array(f["biases"], np.float32)]))
    np.testing.assert_allclose(st.forward_batch(np.array(f["input"]), precision=32), np.array(f["output"], np.float32), atol=1e-4, rtol=0)


def test_dense_simple_literal():
    # the value the reference documents for dense_simple
    np.testing.assert_allclose(np.array(FX["dense_simple"]["output"]).ravel(), [3.0674953, 0.60423696, 1.6263502], rtol=1e-6)


@pytest.mark.parametrize("name,act,tol", [("relu", D.RELU, 1e-5), ("sigmoid", D.SIGMOID, 1e-5), ("tanh", D.TANH, 1e-5),
                                          ("leaky_relu", D.LEAKY_RELU, 1e-6), ("elu", D.ELU, 1e-6)])
def test_scalar_activations(oracle, name, act, tol):
    f = FX["activation_" + name]
    np.testing.assert_allclose(oracle.activation(act, np.array(f["input"]).ravel()), np.array(f["output"], np.float32).ravel(), atol=tol, rtol=0)


@pytest.mark.parametrize("name,act", [("softmax", D.SOFTMAX), ("log_softmax", D.LOGSOFTMAX)])
def test_row_activations_fixture(oracle, name, act):
    f = FX["activation_" + name]
    for row, exp in zip(f["input"], f["output"]):
        np.testing.assert_allclose(oracle.activation(act, np.array(row)), np.array(exp, np.float32), atol=1e-4, rtol=0)


@pytest.mark.parametrize("table,act", [("softmax_table", D.SOFTMAX), ("log_softmax_table", D.LOGSOFTMAX)])
def test_row_activations_tables(oracle, table, act):
    for x, exp in FX[table]:
        np.testing.assert_allclose(oracle.activation(act, np.array(x, np.float32)), np.array(exp, np.float32), atol=1e-6, rtol=0)


def test_mse(oracle):
    f = FX["loss_mse"]
    assert abs(oracle.loss(D.MSE, f["y_pred"], f["y_true"]) - f["loss"][0]) < 1e-5
    for p, y, exp in FX["mse_table"]:
        assert abs(oracle.loss(D.MSE, p, y) - exp) < 1e-6
    for p, y, exp in FX["mse_grad_table"]:
        np.testing.assert_allclose(oracle.loss_grad(D.MSE, p, y), np.array(exp, np.float32), atol=1e-6, rtol=0)


def test_cross_entropy_tables(oracle):
    for p, y, lo, hi in FX["ce_range_table"]:
        v = oracle.loss(D.CROSS_ENTROPY, p, y)
        assert lo <= v <= hi
    for p, y, exp in FX["ce_grad_table"]:
        np.testing.assert_allclose(oracle.loss_grad(D.CROSS_ENTROPY, p, y), np.array(exp, np.float32), atol=1e-6, rtol=0)


def test_logsoftmax_against_torch_logits_ce(oracle):
    # torch.nn.CrossEntropyLoss over logits = mean of -log_softmax(logits)[target]
    f = FX["loss_cross_entropy_logits"]
    vals = [-oracle.activation(D.LOGSOFTMAX, np.array(row))[int(t)] for row, t in zip(f["logits"], f["targets"])]
    assert abs(np.mean(vals) - f["loss"][0]) < 1e-5


def test_cross_entropy_of_logsoftmax_is_constant(oracle):
    # every log-probability is <= 0 < 1e-10, so the clipped loss is -log(1e-10) per one-hot sample
    lp = oracle.activation(D.LOGSOFTMAX, np.array([0.3, -1.0, 2.0], np.float32))
    assert abs(oracle.loss(D.CROSS_ENTROPY, lp, [0, 1, 0]) - 23.02585) < 1e-4


def test_adam_single_step(oracle):
    f = FX["optimizer_adam_step"]
    z = np.zeros(3, np.float32)
    # a fresh optimiser called directly (no NewStep) uses exponent t = 1: opt.go:237
    p, m, v = oracle.adam(f["param"], f["grad"], z, z, f["lr"][0], f["beta1"][0], f["beta2"][0], f["eps"][0], 1)
    np.testing.assert_allclose(p, np.array(f["param_updated"], np.float32), atol=1e-3, rtol=0)   # reference tolerance
    np.testing.assert_allclose(p, np.array(f["param_updated"], np.float32), atol=2e-6, rtol=0)   # and much tighter
    np.testing.assert_allclose(m, 0.1 * np.array(f["grad"], np.float32), rtol=1e-6)


def test_adam_first_network_step_uses_t2(oracle):
    # Network.Step calls NewStep() (counter -> 1) and StepInPlace uses counter + 1
    layers = [D.Dense(2, 1, D.LINEAR)]
    w = np.array([0.5, -0.25, 0.1], np.float32)
    st = oracle.OracleState(layers, D.MSE, w, lr=1e-2)
    x, y = np.array([[1.0, 2.0]], np.float32), np.array([[0.7]], np.float32)
    st.train_batch(x, y, precision=32)
    g = st.grads.copy()
    p2, _, _ = oracle.adam(w, g, np.zeros(3), np.zeros(3), 1e-2, 0.9, 0.999, 1e-8, 2)
    np.testing.assert_array_equal(st.params, p2)
    assert st.timestep == 1
    pred = w[0] * 1 + w[1] * 2 + w[2]
    np.testing.assert_allclose(g, 2 * (pred - 0.7) * np.array([1, 2, 1]), rtol=1e-6)


def test_conv2d_simple(oracle):
    f = FX["conv2d_simple"]
    layers = [D.Conv2D(1, 1, f["kernel"], f["stride"], f["padding"], D.LINEAR, 3, 3)]
    params = np.array([f["weight_fill"]] * 4 + [f["bias_fill"]], np.float32)
    st = oracle.OracleState(layers, D.MSE, params)
    out = st.forward_batch(np.array(f["input"], np.float32).reshape(1, 9), precision=32)
    np.testing.assert_allclose(out.ravel(), np.array(f["output"], np.float32).ravel(), atol=1e-4, rtol=0)


def test_avgpool2d_known_answers(oracle):
    """internal/layer/avgpool2d_test.go:8-35 (2x2 stride 2 on 4x4), :37-65 (2x2 stride 1 on 3x3), :84-114 (backward:
    a unit output gradient spreads 0.25 to every input of its window)."""
    st = oracle.OracleState([D.AvgPool2D(1, 2, 2, 0, 4, 4)], D.MSE, np.zeros(0, np.float32))
    out = st.forward_batch(np.arange(1, 17, dtype=np.float32).reshape(1, 16), precision=32)
    assert np.array_equal(out.ravel(), np.array([3.5, 5.5, 11.5, 13.5], np.float32))
    st = oracle.OracleState([D.AvgPool2D(1, 2, 1, 0, 3, 3)], D.MSE, np.zeros(0, np.float32))
    out = st.forward_batch(np.arange(1, 10, dtype=np.float32).reshape(1, 9), precision=32)
    assert np.array_equal(out.ravel(), np.array([3, 4, 6, 7], np.float32))
    # backward: an identity Dense in front makes the pooled layer's input gradient visible as the Dense bias gradient
    layers = [D.Dense(16, 16, D.LINEAR), D.AvgPool2D(1, 2, 2, 0, 4, 4)]
    params = np.concatenate([np.eye(16, dtype=np.float32).ravel(), np.zeros(16, np.float32)])
    st = oracle.OracleState(layers, D.MSE, params)
    x = np.arange(1, 17, dtype=np.float32).reshape(1, 16)
    y = np.array([[3.5, 5.5, 11.5, 13.5]], np.float32) - 2.0          # MSE gradient 2/n (p - y) = 1 for n = 4
    st.train_batch(x, y, precision=32, step=False)
    assert np.allclose(st.grads[256:], 0.25, atol=1e-7)


def test_gelu_silu_follow_their_formulas(oracle):
    """The reference holds no stored vector for GELU (tanh form, activations.go:241-275) or SiLU (:277-309): the checker is
    compared with the formulas evaluated in float64, value and derivative (by central differences)."""
    x = np.linspace(-4, 4, 41).astype(np.float32)
    xd = x.astype(np.float64)
    gelu = lambda v: 0.5 * v * (1 + np.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3)))
    silu = lambda v: v / (1 + np.exp(-v))
    for act, f in ((D.GELU, gelu), (D.SILU, silu)):
        np.testing.assert_allclose(oracle.activation(act, x), f(xd), atol=2e-6, rtol=0)
        h = 1e-5
        np.testing.assert_allclose(oracle.activation_deriv(act, x), (f(xd + h) - f(xd - h)) / (2 * h), atol=2e-5, rtol=0)


def test_rmsnorm_known_answer(oracle):
    """internal/layer/rmsnorm_test.go:8-28: x = [1, 2, 3, 4], eps = 1e-5, gamma = 1 -> x / sqrt(30 / 4 + 1e-5)."""
    # (a normalisation layer takes its row count from the layer in front of it: an identity Dense supplies it)
    params = np.concatenate([np.eye(4, dtype=np.float32).ravel(), np.zeros(4, np.float32), np.ones(4, np.float32)])
    st = oracle.OracleState([D.Dense(4, 4, D.LINEAR), D.RMSNorm(4, 1e-5)], D.MSE, params)
    x = np.array([[1, 2, 3, 4]], np.float32)
    rms = np.float32(np.sqrt(np.float64(np.float32(30.0) / np.float32(4.0) + np.float32(1e-5))))
    np.testing.assert_allclose(st.forward_batch(x, precision=32).ravel(), x.ravel() / rms, atol=1e-6, rtol=0)


def test_conv1d_known_answer(oracle):
    """internal/layer/conv1d_test.go:69-84: one channel, kernel [1, 0, 1], bias 0, padding 1 on [0, 1, 2, 3, 4]:
    the worked example in the test gives 1 and 2 for the first two positions; the definition gives [1, 2, 4, 6, 3]."""
    st = oracle.OracleState([D.Conv1D(1, 1, 3, 1, 1, D.LINEAR, 5)], D.MSE, np.array([1, 0, 1, 0], np.float32))
    out = st.forward_batch(np.array([[0, 1, 2, 3, 4]], np.float32), precision=32)
    assert np.array_equal(out.ravel(), np.array([1, 2, 4, 6, 3], np.float32))


def test_layernorm_known_answers(oracle):
    """internal/layer/layernorm_test.go:8-35 (x = [1, 2, 3, 4], gamma 1, beta 0 -> (x - 2.5) / sqrt(1.25 + 1e-5)) and :98-123
    (two rows [1..4], [5..8], each normalised on its own)."""
    # (a normalisation layer takes its row count from the layer in front of it: an identity Dense supplies it)
    params = np.concatenate([np.eye(8, dtype=np.float32).ravel(), np.zeros(8, np.float32), np.ones(4, np.float32), np.zeros(4, np.float32)])
    st = oracle.OracleState([D.Dense(8, 8, D.LINEAR), D.LayerNorm(4)], D.MSE, params)
    x = np.arange(1, 9, dtype=np.float32).reshape(1, 8)
    std = np.float32(np.sqrt(1.25 + 1e-5))
    want = np.concatenate([(x[0, :4] - np.float32(2.5)) / std, (x[0, 4:] - np.float32(6.5)) / std])
    np.testing.assert_allclose(st.forward_batch(x, precision=32).ravel(), want, atol=1e-5, rtol=0)


def test_maxpool2d_known_answers(oracle):
    """internal/layer/maxpool2d_test.go:8-35 (2x2 stride 2 on 4x4 -> [6, 8, 14, 16]), :37-65 (2x2 stride 1 on 3x3 ->
    [5, 6, 8, 9]), :84-108 (a gradient of ones reaches exactly the arg-max positions 5, 7, 13, 15)."""
    st = oracle.OracleState([D.MaxPool2D(1, 2, 2, 0, 4, 4)], D.MSE, np.zeros(0, np.float32))
    x = np.arange(1, 17, dtype=np.float32).reshape(1, 16)
    assert np.array_equal(st.forward_batch(x, precision=32).ravel(), np.array([6, 8, 14, 16], np.float32))
    st = oracle.OracleState([D.MaxPool2D(1, 2, 1, 0, 3, 3)], D.MSE, np.zeros(0, np.float32))
    assert np.array_equal(st.forward_batch(np.arange(1, 10, dtype=np.float32).reshape(1, 9), precision=32).ravel(), np.array([5, 6, 8, 9], np.float32))
    layers = [D.Dense(16, 16, D.LINEAR), D.MaxPool2D(1, 2, 2, 0, 4, 4)]
    params = np.concatenate([np.eye(16, dtype=np.float32).ravel(), np.zeros(16, np.float32)])
    st = oracle.OracleState(layers, D.MSE, params)
    y = np.array([[6, 8, 14, 16]], np.float32) - 2.0                  # MSE gradient 2/n (p - y) = 1 for n = 4
    st.train_batch(x, y, precision=32, step=False)
    want = np.zeros(16, np.float32); want[[5, 7, 13, 15]] = 1
    assert np.array_equal(st.grads[256:], want)                      # the identity Dense's bias gradient = the pool's input gradient


def test_batchnorm2d_known_answer(oracle):
    """internal/layer/batchnorm2d_test.go:8-30: two channels with two positions each, [1, 5 | 2, 6] -> [-1, 1, -1, 1]."""
    params = np.array([1, 1, 0, 0], np.float32)                      # gamma 1, beta 0
    st = oracle.OracleState([D.BatchNorm2D(2, 1, 2)], D.MSE, params)
    out = st.forward_batch(np.array([[1, 5, 2, 6]], np.float32), precision=32, training=True)
    np.testing.assert_allclose(out.ravel(), [-1, 1, -1, 1], atol=1e-5, rtol=0)


def test_swiglu_known_answer(oracle):
    """internal/layer/swiglu_test.go:30-53: w = 2, v = 3, x = 1 -> swish(2) * 3 = 5.284782.  The layer lives inside a
    TransformerBlock here, so it is pinned through a block whose other parts are switched off by zero weights."""
    # SwiGLU: block of width 1, one head, one token; attention output 0 (zero projections), RMSNorm with gain g:
    # r1 = x, n1 = g * x / sqrt(x^2 + eps); choose x, g so that n1 = 1; ff2 = identity -> block output before norm 2 = n1 + swiglu(n1)
    x0 = np.float32(1.0)
    g = np.float32(np.sqrt(np.float64(x0 * x0) + 1e-5))
    blk = D.TransformerBlock(1, 1, 1, 1, True, ff_act=D.SILU, rms_norm=True)
    #        wq wk wv wo (W, b each)        rms1 rms2  swiglu W, V   ff2 W, b
    params = np.array([0, 0, 0, 0, 0, 0, 0, 0, g, 1, 2, 3, 1, 0], np.float32)
    st = oracle.OracleState([D.Dense(1, 1, D.LINEAR), blk], D.MSE, np.concatenate([np.array([1, 0], np.float32), params]))
    out = st.forward_batch(np.array([[x0]], np.float32), precision=64)
    # the block's output is RMSNorm(r2) with gain 1: r2 / sqrt(r2^2 + eps), r2 = 1 + 5.284782
    r2 = 1.0 + 5.284782
    np.testing.assert_allclose(out.ravel(), [r2 / np.sqrt(r2 * r2 + 1e-5)], atol=2e-6, rtol=0)


def test_rope_known_answers(oracle):
    """internal/layer/rope_test.go:8-49: head size 4, two positions of [1, 2, 3, 4]: position 0 is unchanged, at position 1
    the pair (x0, x2) = (1, 3) turns by theta_0 = 1 radian; :51-79: the conjugate rotation undoes the rotation."""
    x = np.array([1, 2, 3, 4, 1, 2, 3, 4], np.float32)
    y = oracle.rope(x, 2, 1, 4)
    assert np.array_equal(y[:4], x[:4])
    c0, s0 = np.float32(np.cos(np.float64(np.float32(1.0)))), np.float32(np.sin(np.float64(np.float32(1.0))))
    assert abs(y[4] - (1 * c0 - 3 * s0)) <= 1e-5 and abs(y[6] - (1 * s0 + 3 * c0)) <= 1e-5
    rng = np.random.default_rng(3)
    z = rng.standard_normal(10 * 4 * 32).astype(np.float32)
    back = oracle.rope(oracle.rope(z, 10, 4, 32), 10, 4, 32, conjugate=True)
    np.testing.assert_allclose(back, z, atol=1e-5, rtol=0)


def test_embedding_known_answers(oracle):
    """internal/layer/embedding_test.go:8-34: the output is the table's rows of the given ids; :36-82: a gradient of ones
    reaches exactly the rows that were looked up, one per dimension, and every other row stays zero."""
    V, d, T = 5, 3, 3
    table = np.arange(V * d, dtype=np.float32) * np.float32(0.25) - np.float32(1.0)
    ids = np.array([[0, 2, 4]], np.float32)
    st = oracle.OracleState([D.Embedding(V, d, T)], D.MSE, table)
    out = st.forward_batch(ids, precision=32).ravel()
    assert np.array_equal(out, table.reshape(V, d)[[0, 2, 4]].ravel())
    # MSE gradient 2 (p - y) / n with n = 9: targets 4.5 below the outputs make it exactly 1 everywhere
    st.train_batch(ids, (out - np.float32(4.5)).reshape(1, -1), precision=32, step=False)
    g = st.grads.reshape(V, d)
    np.testing.assert_allclose(g[[0, 2, 4]], 1.0, atol=1e-6, rtol=0)
    assert not g[[1, 3]].any()


def test_gru_parameter_layout_size(oracle):
    """internal/layer/gru_test.go:62-75: NewGRU(4, 8) holds 3*8*4 input weights, 2*8*8 recurrent weights and 3*8 biases."""
    assert oracle.param_count([D.SequenceUnrollerGRU(4, 8, 5)])[0] == 3 * 8 * 4 + 2 * 8 * 8 + 3 * 8


def test_dropout_known_answers(oracle):
    """internal/layer/dropout_test.go:8-34: with rate 0.5 and an input of 100 ones, between 30 and 70 outputs survive in
    training mode (and a survivor is scaled by 1 / keep); :36-54: in inference mode the input passes through unchanged;
    :101-108: the layer has no parameters."""
    layers = [D.Dropout(0.5, 100)]
    assert oracle.param_count(layers)[0] == 0
    st = oracle.OracleState(layers, D.MSE, np.zeros(0, np.float32))
    ones = np.ones((1, 100), np.float32)
    out = st.forward_batch(ones, precision=32, training=True).ravel()
    kept = out != 0
    assert 30 <= int(kept.sum()) <= 70
    assert np.array_equal(out[kept], np.full(int(kept.sum()), 2.0, np.float32))
    ramp = np.arange(100, dtype=np.float32).reshape(1, -1)
    assert np.array_equal(st.forward_batch(ramp, precision=32, training=False).ravel(), ramp.ravel())
