"""ctypes loader of libgoneuron_cuda.so.  There is no CPU fallback: if the library is missing
the import of anything that computes fails with a clear error."""
import ctypes as C
import os

from .descriptors import LayerDesc

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "libgoneuron_cuda.so")
UNIQUE_ID_BYTES = 128

# every symbol include/goneuron_cuda.h declares
EXPORTS = [
    "gn_init", "gn_get_unique_id", "gn_init_rank", "gn_shutdown", "gn_ctx_world_size", "gn_ctx_set_spin_limit", "gn_synchronize", "gn_timer_start", "gn_timer_stop", "gn_last_error",
    "gn_model_create", "gn_model_destroy", "gn_model_param_count", "gn_model_in_size", "gn_model_out_size",
    "gn_model_set_params", "gn_model_get_params", "gn_model_get_grads", "gn_adam_set", "gn_adam_get_state",
    "gn_adam_set_state", "gn_train_batch", "gn_train_batch_device", "gn_forward_batch", "gn_device_alloc",
    "gn_device_free", "gn_device_upload", "gn_device_download", "gn_model_last_stats", "gn_model_set_profiling",
    "gn_op_gemm_nt", "gn_op_adam", "gn_op_layernorm", "gn_op_conv2d", "gn_op_softmax_ce", "gn_op_lstm", "gn_op_gemm_nt_static", "gn_op_attention", "gn_model_state_count", "gn_model_get_state", "gn_model_set_state",
]


class StepStats(C.Structure):
    _fields_ = [("kernel_launches", C.c_int64), ("step_ms", C.c_float), ("allreduce_ms", C.c_float),
                ("gemm_ms", C.c_float), ("gemm_launches", C.c_int64), ("gemm_flops", C.c_double),
                ("gemm_bytes", C.c_double), ("split_bytes", C.c_double)]


class GoNeuronCudaError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"libgoneuron_cuda error {code}: {msg}")
        self.code = code


_lib = None


def load():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(SO_PATH):
        raise ImportError(f"{SO_PATH} is missing: build it with `python -m goneuron_b200.build` "
                          "(there is no CPU fallback)")
    L = C.CDLL(SO_PATH)
    f32p, vp, i64p = C.POINTER(C.c_float), C.c_void_p, C.POINTER(C.c_int64)
    L.gn_last_error.restype = C.c_char_p
    L.gn_init.argtypes = [C.c_int, C.POINTER(vp)]
    L.gn_get_unique_id.argtypes = [C.c_char_p]
    L.gn_init_rank.argtypes = [C.c_int, C.c_int, C.c_int, C.c_char_p, C.POINTER(vp)]
    L.gn_shutdown.argtypes = [vp]
    L.gn_ctx_world_size.argtypes = [vp, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    L.gn_synchronize.argtypes = [vp]
    L.gn_ctx_set_spin_limit.argtypes = [vp, C.c_uint]
    L.gn_timer_start.argtypes = [vp]
    L.gn_timer_stop.argtypes = [vp, f32p]
    L.gn_model_create.argtypes = [vp, C.POINTER(LayerDesc), C.c_int, C.c_int, C.c_int, C.POINTER(vp)]
    L.gn_model_destroy.argtypes = [vp]
    for n in ("gn_model_param_count", "gn_model_in_size", "gn_model_out_size"):
        getattr(L, n).argtypes = [vp, i64p]
    L.gn_model_set_params.argtypes = [vp, f32p, C.c_int64]
    L.gn_model_get_params.argtypes = [vp, f32p, C.c_int64]
    L.gn_model_get_grads.argtypes = [vp, f32p, C.c_int64]
    L.gn_adam_set.argtypes = [vp, C.c_float, C.c_float, C.c_float, C.c_float, C.c_int]
    L.gn_adam_get_state.argtypes = [vp, f32p, f32p, C.c_int64, C.POINTER(C.c_int)]
    L.gn_adam_set_state.argtypes = [vp, f32p, f32p, C.c_int64, C.c_int]
    L.gn_train_batch.argtypes = [vp, f32p, f32p, C.c_int, C.c_int, C.c_int, f32p]
    L.gn_train_batch_device.argtypes = [vp, vp, vp, C.c_int, C.c_int, C.c_int, f32p]
    L.gn_forward_batch.argtypes = [vp, f32p, C.c_int, f32p]
    L.gn_device_alloc.argtypes = [vp, C.c_int64, C.POINTER(vp)]
    L.gn_device_free.argtypes = [vp, vp]
    L.gn_device_upload.argtypes = [vp, vp, f32p, C.c_int64]
    L.gn_device_download.argtypes = [vp, f32p, vp, C.c_int64]
    L.gn_model_last_stats.argtypes = [vp, C.POINTER(StepStats)]
    L.gn_model_set_profiling.argtypes = [vp, C.c_int]
    L.gn_op_gemm_nt.argtypes = [vp, C.c_int, C.c_int, C.c_int, C.c_int, f32p, f32p, f32p, f32p]
    L.gn_op_adam.argtypes = [vp, f32p, f32p, f32p, f32p, C.c_int64, C.c_float, C.c_float, C.c_float, C.c_float, C.c_int, C.c_float]
    L.gn_model_state_count.argtypes = [vp, i64p]
    L.gn_model_get_state.argtypes = [vp, f32p, C.c_int64]
    L.gn_model_set_state.argtypes = [vp, f32p, C.c_int64]
    L.gn_op_gemm_nt_static.argtypes = [vp, C.c_int, C.c_int, C.c_int, vp, vp, vp, vp]
    L.gn_op_layernorm.argtypes = [vp, C.c_int64, C.c_int] + [f32p] * 8
    L.gn_op_conv2d.argtypes = [vp] + [C.c_int] * 10 + [f32p] * 8
    L.gn_op_softmax_ce.argtypes = [vp, C.c_int, C.c_int, C.c_int] + [f32p] * 5
    L.gn_op_lstm.argtypes = [vp] + [C.c_int] * 5 + [f32p] * 8
    L.gn_op_attention.argtypes = [vp] + [C.c_int] * 6 + [f32p] * 10
    _lib = L
    return L


def check(rc):
    if rc != 0:
        raise GoNeuronCudaError(rc, load().gn_last_error().decode(errors="replace"))
