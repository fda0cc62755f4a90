"""Collects the reference's own golden vectors for the training hot path into one small JSON
fixture, so that the tests can run where the reference checkout is absent.

Source of every number: the PyTorch-generated little-endian float32 files the reference
commits under scripts/pytorch_validation/test_data/pytorch_refs/<case>/ (read by
internal/validation/pytorch_validation_test.go:164-344), and the known-answer tables written
as literals in internal/loss/loss_pytorch_test.go:22-160 and
internal/activations/activations_pytorch_test.go:92-150 (transcribed below as data).

Run:  python tests/golden/make_reference_fixtures.py /path/to/GoNeuron
"""
import json
import os
import sys

import numpy as np


def read(case_dir, name, shape=None):
    a = np.fromfile(os.path.join(case_dir, name + ".bin"), dtype="<f4")
    return a.reshape(shape).tolist() if shape else a.tolist()


def main(ref):
    root = os.path.join(ref, "scripts", "pytorch_validation", "test_data", "pytorch_refs")
    out = {"source": "GoNeuron scripts/pytorch_validation/test_data/pytorch_refs + *_pytorch_test.go literals"}
    for case in ("dense_simple", "dense_batch"):
        d = os.path.join(root, case)
        meta = json.load(open(os.path.join(d, "metadata.json")))
        out[case] = {k: read(d, k, meta["inputs"][k]["shape"]) for k in ("input", "weights", "biases")}
        out[case]["output"] = read(d, "output", meta["outputs"]["output"]["shape"])
    for act in ("relu", "sigmoid", "tanh", "softmax", "log_softmax", "leaky_relu", "elu"):   # leaky_relu: slope 0.01; elu: alpha 1
        d = os.path.join(root, "activation_" + act)
        meta = json.load(open(os.path.join(d, "metadata.json")))
        out["activation_" + act] = {"input": read(d, "input", meta["inputs"]["input"]["shape"]),
                                    "output": read(d, "output", meta["outputs"]["output"]["shape"])}
    d = os.path.join(root, "loss_mse")
    out["loss_mse"] = {"y_pred": read(d, "y_pred"), "y_true": read(d, "y_true"), "loss": read(d, "loss")}
    d = os.path.join(root, "loss_cross_entropy")   # torch CE over logits: pins log-softmax, not loss.CrossEntropy
    out["loss_cross_entropy_logits"] = {"logits": read(d, "logits", (2, 3)), "targets": read(d, "targets"), "loss": read(d, "loss")}
    d = os.path.join(root, "optimizer_adam_step")
    out["optimizer_adam_step"] = {k: read(d, k) for k in ("param", "grad", "lr", "beta1", "beta2", "eps", "param_updated")}
    d = os.path.join(root, "conv2d_simple")         # generator sets weight = 1, bias = 0, k=2, s=1, p=0
    out["conv2d_simple"] = {"input": read(d, "input", (1, 3, 3)), "output": read(d, "output", (1, 2, 2)),
                            "kernel": 2, "stride": 1, "padding": 0, "weight_fill": 1.0, "bias_fill": 0.0}
    # literals of the reference's Go tests
    out["mse_table"] = [[[1, 2, 3], [1, 2, 3], 0.0], [[1, 2], [1.5, 2], 0.125], [[1, 2, 3], [0, 1, 2], 1.0],
                        [[1, 1], [0, 2], 1.0], [[0.5], [0.0], 0.25], [[2.0], [-1.0], 9.0], [[-1.5], [0.5], 4.0]]
    out["mse_grad_table"] = [[[1, 2], [1, 2], [0, 0]], [[1.5, 2], [1, 2], [0.5, 0]], [[0, 0], [1, 1], [-1, -1]],
                             [[0.5, 0.5], [0, 1], [0.5, -0.5]]]
    out["ce_range_table"] = [[[1.0], [1.0], 0.0, 1e-6], [[0.0], [0.0], 0.0, 1e-6], [[0.9], [1.0], 0.1, 0.11], [[0.1], [1.0], 2.2, 2.4]]
    out["ce_grad_table"] = [[[1, 0], [1, 0], [0, 0]], [[0.7, 0.3], [1, 0], [-0.3, 0.3]], [[0.5], [1.0], [-0.5]], [[0.5], [0.0], [0.5]]]
    out["softmax_table"] = [[[1, 2, 3], [0.09003057317, 0.2447284710, 0.6652409558]], [[0, 0, 0], [1 / 3, 1 / 3, 1 / 3]],
                            [[-1, 0, 1], [0.09003057317, 0.2447284710, 0.6652409558]], [[2.0], [1.0]]]
    out["log_softmax_table"] = [[[1, 2, 3], [-2.407605964, -1.407605964, -0.4076059643]], [[0, 0, 0], [-1.098612289] * 3],
                                [[-1, 0, 1], [-2.407605964, -1.407605964, -0.4076059643]], [[2.0], [0.0]]]
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_fixtures.json")
    json.dump(out, open(dst, "w"), indent=1)
    print("wrote", dst)


if __name__ == "__main__":
    main(sys.argv[1])
