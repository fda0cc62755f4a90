"""Host-side mirror of the reference's Sequential API over the C ABI.

Names and argument meaning follow internal/net/sequential.go (Compile :26-37, Fit :110-115,
TrainBatch :102-107, Predict :118-122, PredictBatch :133-164, Evaluate :172-183) and
internal/net/net.go (Params/Gradients/SetParams :549-571, :787-810).  Errors surface as
GoNeuronCudaError where the reference returns `error`."""
import ctypes as C

import numpy as np

from . import _lib
from .descriptors import layers_to_array


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


class Device:
    """One B200 (layer.Device, internal/layer/device.go:27-30).  With world_size > 1 each rank owns one."""

    def __init__(self, device=0, rank=0, world_size=1, unique_id=None):
        L = _lib.load()
        h = C.c_void_p()
        if world_size > 1:
            _lib.check(L.gn_init_rank(device, rank, world_size, unique_id, C.byref(h)))
        else:
            _lib.check(L.gn_init(device, C.byref(h)))
        self.handle, self.rank, self.world_size, self.device = h, rank, world_size, device

    @staticmethod
    def unique_id():
        buf = C.create_string_buffer(_lib.UNIQUE_ID_BYTES)
        _lib.check(_lib.load().gn_get_unique_id(buf))
        return buf.raw

    def synchronize(self):
        _lib.check(_lib.load().gn_synchronize(self.handle))

    def timer_start(self):
        _lib.check(_lib.load().gn_timer_start(self.handle))

    def timer_stop(self):
        ms = C.c_float()
        _lib.check(_lib.load().gn_timer_stop(self.handle, C.byref(ms)))
        return ms.value

    def alloc(self, host_array):
        """Copies a host array into device memory; returns an opaque device pointer (freed by free())."""
        a = _f32(host_array)
        d = C.c_void_p()
        L = _lib.load()
        _lib.check(L.gn_device_alloc(self.handle, a.size, C.byref(d)))
        _lib.check(L.gn_device_upload(self.handle, d, _p(a), a.size))
        return d

    def free(self, dptr):
        _lib.load().gn_device_free(self.handle, dptr)

    def close(self):
        if self.handle:
            _lib.load().gn_shutdown(self.handle)
            self.handle = None


class Adam:
    """opt.NewAdam(lr) -- internal/opt/opt.go:93-121."""

    def __init__(self, learning_rate, beta1=0.9, beta2=0.999, epsilon=1e-8):
        self.LearningRate, self.Beta1, self.Beta2, self.Epsilon = learning_rate, beta1, beta2, epsilon


class Sequential:
    """goneuron.NewSequential(layers...) bound to a Device."""

    def __init__(self, layers, device=None, virtual_workers=1):
        self.layers = list(layers)
        self.device = device or Device(0)
        self.virtual_workers = virtual_workers
        self.handle = None
        self.opt = None

    def Compile(self, optimizer, loss):
        L = _lib.load()
        h = C.c_void_p()
        arr = layers_to_array(self.layers)
        _lib.check(L.gn_model_create(self.device.handle, arr, len(self.layers), int(loss), self.virtual_workers, C.byref(h)))
        self.handle, self.opt, self.loss = h, optimizer, loss
        n = C.c_int64()
        _lib.check(L.gn_model_param_count(h, C.byref(n)))
        self.n_params = n.value
        _lib.check(L.gn_model_in_size(h, C.byref(n)))
        self.in_size = n.value
        _lib.check(L.gn_model_out_size(h, C.byref(n)))
        self.out_size = n.value
        return self

    # -- parameters -------------------------------------------------------------
    def SetParams(self, params):
        a = _f32(params)
        _lib.check(_lib.load().gn_model_set_params(self.handle, _p(a), a.size))

    def Params(self):
        a = np.empty(self.n_params, np.float32)
        _lib.check(_lib.load().gn_model_get_params(self.handle, _p(a), a.size))
        return a

    def Gradients(self):
        a = np.empty(self.n_params, np.float32)
        _lib.check(_lib.load().gn_model_get_grads(self.handle, _p(a), a.size))
        return a

    def AdamState(self):
        m, v, t = np.empty(self.n_params, np.float32), np.empty(self.n_params, np.float32), C.c_int()
        _lib.check(_lib.load().gn_adam_get_state(self.handle, _p(m), _p(v), m.size, C.byref(t)))
        return m, v, t.value

    def SetAdamState(self, m, v, timestep):
        m, v = _f32(m), _f32(v)
        _lib.check(_lib.load().gn_adam_set_state(self.handle, _p(m), _p(v), m.size, timestep))

    def State(self):
        """Non-parameter layer state (BatchNorm2D running mean | running variance per layer, in layer order)."""
        n = C.c_int64()
        _lib.check(_lib.load().gn_model_state_count(self.handle, C.byref(n)))
        a = np.empty(n.value, np.float32)
        if n.value:
            _lib.check(_lib.load().gn_model_get_state(self.handle, _p(a), a.size))
        return a

    def SetState(self, state):
        a = _f32(state)
        _lib.check(_lib.load().gn_model_set_state(self.handle, _p(a), a.size))

    # -- checkpoints ------------------------------------------------------------
    def Checkpoint(self):
        """Everything a resumed run needs: parameters (Network.Save, net.go:863-1075), the optimiser's moments and
        step counter (which the reference does not checkpoint, opt.go:312-322) and the non-parameter layer state."""
        m, v, t = self.AdamState()
        return {"params": self.Params(), "adam_m": m, "adam_v": v, "adam_timestep": np.int64(t), "state": self.State()}

    def Restore(self, ckpt):
        self.SetParams(ckpt["params"])
        self.SetAdamState(ckpt["adam_m"], ckpt["adam_v"], int(ckpt["adam_timestep"]))
        if np.asarray(ckpt["state"]).size:
            self.SetState(ckpt["state"])

    @staticmethod
    def _ckpt_path(path):
        """np.savez appends ".npz" to a name without it; Save and Load agree on the file name by doing the same."""
        path = str(path)
        return path if path.endswith(".npz") else path + ".npz"

    def Save(self, path):
        with open(self._ckpt_path(path), "wb") as f:
            np.savez(f, **self.Checkpoint())

    def Load(self, path):
        with np.load(self._ckpt_path(path)) as f:
            self.Restore({k: f[k] for k in f.files})

    # -- training ---------------------------------------------------------------
    def _push_opt(self):
        o = self.opt   # re-read every step: schedulers mutate LearningRate on the host (opt/scheduler.go)
        _lib.check(_lib.load().gn_adam_set(self.handle, o.LearningRate, o.Beta1, o.Beta2, o.Epsilon, -1))

    def TrainBatch(self, batch_x, batch_y, global_batch=0, first_sample=0):
        x, y = _f32(batch_x), _f32(batch_y)
        if x.shape[0] != y.shape[0]:
            raise ValueError("batchX and batchY differ in length")
        self._push_opt()
        loss = C.c_float()
        _lib.check(_lib.load().gn_train_batch(self.handle, _p(x), _p(y), x.shape[0], global_batch, first_sample, C.byref(loss)))
        return loss.value

    def TrainBatchDevice(self, x_dev, y_dev, batch, global_batch=0, first_sample=0):
        self._push_opt()
        loss = C.c_float()
        _lib.check(_lib.load().gn_train_batch_device(self.handle, x_dev, y_dev, batch, global_batch, first_sample, C.byref(loss)))
        return loss.value

    def Fit(self, x, y, epochs, batch_size, callbacks=()):
        """Network.Fit (net.go:351-407): consecutive slices, no shuffling, last batch may be short;
        returns the mean of the batch losses of the last epoch."""
        x, y = _f32(x), _f32(y)
        n = x.shape[0]
        epoch_loss = 0.0
        for epoch in range(epochs):
            losses = []
            for s in range(0, n, batch_size):
                losses.append(self.TrainBatch(x[s:s + batch_size], y[s:s + batch_size]))
            epoch_loss = float(np.mean(losses)) if losses else 0.0
            stop = False
            for cb in callbacks:
                if cb(epoch, epoch_loss, self) is False:
                    stop = True
            if stop:
                break
        return epoch_loss

    def PredictBatch(self, x):
        x = _f32(x)
        out = np.empty((x.shape[0], self.out_size), np.float32)
        _lib.check(_lib.load().gn_forward_batch(self.handle, _p(x), x.shape[0], _p(out)))
        return out

    def Predict(self, x):
        return self.PredictBatch(_f32(x).reshape(1, -1))[0]

    def Evaluate(self, x, y):
        """Sequential.Evaluate (sequential.go:172-183): mean per-sample loss without a weight update.  The forward pass
        runs on the device; the per-sample loss of the few outputs is formed on the host in float32, term by term as
        loss.go:53-69 (MSE) and :120-138 (CrossEntropy, probabilities clipped at 1e-10) do."""
        p = self.PredictBatch(x)
        y = _f32(y)
        if self.loss == 0:
            d = p - y
            per = np.sum(d * d, axis=1, dtype=np.float32) / np.float32(p.shape[1])
        else:
            per = -np.sum(y * np.log(np.maximum(p, np.float32(1e-10)).astype(np.float64)).astype(np.float32), axis=1, dtype=np.float32)
        return float(np.sum(per, dtype=np.float32) / np.float32(p.shape[0]))

    def stats(self):
        s = _lib.StepStats()
        _lib.check(_lib.load().gn_model_last_stats(self.handle, C.byref(s)))
        return s

    def set_profiling(self, level):
        _lib.check(_lib.load().gn_model_set_profiling(self.handle, level))

    def Close(self):
        if self.handle:
            _lib.load().gn_model_destroy(self.handle)
            self.handle = None
