"""goneuron_b200 -- B200 (sm_100a) training backend for GoNeuron models.

The compute lives in csrc/ (CUDA kernels + the C ABI declared in include/goneuron_cuda.h);
this package is the thin host-side mirror of the reference's Sequential API used by the
tests and the benchmark; a Go host binds the same C ABI through cgo."""
from . import descriptors  # noqa: F401
