"""CPU-only checks: the C-ABI library loads and exports every declared symbol, the descriptor layout
matches the header, the flat parameter counts match the reference's layout, and failures are status codes."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from goneuron_b200 import _lib, configs, descriptors as D

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from goneuron_b200 import build
    build.build()
    return _lib.load()


def test_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "goneuron_cuda.h")).read()
    declared = set(re.findall(r"^(?:int|const char\*)\s+(gn_[a-z0-9_]+)\s*\(", header, flags=re.M))
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_descriptor_layout():
    assert C.sizeof(D.LayerDesc) == 16 * 4
    header = open(os.path.join(ROOT, "include", "goneuron_cuda.h")).read()
    body = header[header.index("typedef struct gn_layer_desc {"):header.index("} gn_layer_desc;")]
    fields = re.findall(r"int32_t\s+(\w+);", body)
    assert fields == [n for n, _ in D.LayerDesc._fields_]


def test_no_device_is_a_status_code(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    rc = lib.gn_init(0, C.byref(h))
    assert rc == -3 and b"CUDA" in lib.gn_last_error()
    with pytest.raises(_lib.GoNeuronCudaError):
        _lib.check(rc)


def test_null_handles_are_rejected(lib):
    assert lib.gn_model_param_count(None, None) == -1
    assert lib.gn_model_destroy(None) == 0 and lib.gn_shutdown(None) == 0     # idempotent no-ops
    assert lib.gn_train_batch(None, None, None, 1, 0, 0, None) == -1


@pytest.mark.parametrize("name,count", [("mlp", 101770), ("cnn", 25578), ("lstm", 74369), ("transformer_small", 7394304)])
def test_flat_param_counts(oracle, name, count):
    layers, _, _, _ = configs.build(name)
    n, _, _ = oracle.param_count(layers)
    assert n == count
    assert configs.init_params(layers, np.random.default_rng(0)).size == count


def test_large_transformer_param_count():
    layers, _, _, _ = configs.build("transformer_large")
    d, f, v, t = 1024, 4096, 32000, 512
    per_block = 4 * (d * d + d) + 4 * d + d * f + f + f * d + d
    assert v * d + t * d + 8 * per_block + d * v + v == 166862080


def test_reference_generator_and_initialisers():
    """The reference's LCG (layer.go:61-75) restated with wrapping uint64 arithmetic, against plain Python integers; and the
    shapes, seeds and fixed entries of the initialisers built on it."""
    import numpy as np
    from goneuron_b200 import configs

    def lcg(seed, n):
        s, out = seed, []
        for _ in range(n):
            s = (s * 6364136223846793005 + 1) % (1 << 64)
            out.append(np.float32(s >> 33) / np.float32(1 << 31))
        return np.array(out, np.float32)

    rng = configs.ReferenceRNG(784 * 1000 + 128 * 100 + 42)
    got = np.concatenate([rng.rand_float(1000), rng.rand_float(1), rng.rand_float(77)])      # state carries over between calls
    assert np.array_equal(got, lcg(784 * 1000 + 128 * 100 + 42, 1078))
    layers, _, _, _ = configs.build("mlp")
    p = configs.reference_init_params(layers)
    assert p.size == 101770
    scale = np.float32(np.sqrt(2.0 / (784.0 + 128.0)))
    r = lcg(784 * 1000 + 128 * 100 + 42, 784 * 128 + 128)
    assert np.array_equal(p[:784 * 128], r[:784 * 128] * np.float32(2) * scale - scale)
    assert np.array_equal(p[784 * 128:784 * 128 + 128], r[784 * 128:] * np.float32(0.2) - np.float32(0.1))
    layers, _, _, _ = configs.build("lstm")
    p = configs.reference_init_params(layers)
    H, i = 128, 16
    b = p[4 * H * i + 4 * H * H:4 * H * i + 4 * H * H + 4 * H]
    assert p.size == 74369 and np.array_equal(b[H:2 * H], np.ones(H, np.float32)) and not b[:H].any() and not b[2 * H:].any()
    # equal-shaped layers start identical (the seed depends only on the shape)
    from goneuron_b200 import descriptors as D
    q = configs.reference_init_params([D.Dense(8, 8, D.RELU), D.Dense(8, 8, D.RELU)])
    assert np.array_equal(q[:72], q[72:])


def test_every_environment_switch_is_documented():
    """Each GONEURON_CUDA_* variable the library reads has a row in the integration notes' table of switches."""
    import glob
    import os
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    read = set()
    for path in glob.glob(os.path.join(root, "goneuron_b200", "csrc", "*.cu*")):
        read |= set(re.findall(r'getenv\("(GONEURON_CUDA_[A-Z0-9_]+)"\)', open(path).read()))
    assert len(read) >= 10
    doc = open(os.path.join(root, "INTEGRATION.md")).read()
    missing = sorted(v for v in read if v not in doc)
    assert not missing, missing
