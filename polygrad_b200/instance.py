"""polygrad model instances (``PolyInstance``) driven through the C API.

Mirrors ``py/polygrad/instance.py`` for the forward path and adds what that
wrapper leaves out: ``set_device`` (polygrad ``src/instance.c:582``) and the
device readback / upload calls (``src/instance.c:479-501``).  Model graphs come
from polygrad's own builders: ``poly_gpt2_build``
(``src/modelzoo/models/gpt2.c:173``) and ``poly_mlp_instance``
(``src/model_mlp.c:77``).
"""
import ctypes
import json
import zlib

import numpy as np

from . import ffi


def seeded_normal(name, shape, seed, std=0.02):
    """Parameter values ~ N(0, std), a pure function of (seed, name)."""
    rng = np.random.default_rng([int(seed), zlib.crc32(name.encode())])
    return (rng.standard_normal(shape) * std).astype(np.float32)


def gpt2_init(seed):
    """Random-init rule for GPT-2 instances: every tensor ~ N(0, 0.02) except
    LayerNorm gains, which are 1 + N(0, 0.02) so that activations keep unit scale."""
    def init(name, shape):
        w = seeded_normal(name, shape, seed)
        if 'ln_' in name and name.endswith('weight'):
            w = w + np.float32(1.0)
        return w
    return init


class Instance:
    def __init__(self, lib, handle):
        if not handle:
            raise RuntimeError('instance builder returned NULL')
        self.lib, self.h = lib, handle
        self.device = ffi.DEVICE_CPU
        self.bufs = {}
        for i in range(lib.poly_instance_buf_count(handle)):
            name = lib.poly_instance_buf_name(handle, i).decode()
            shape = (ctypes.c_int64 * 8)()
            nd = lib.poly_instance_buf_shape(handle, i, shape, 8)
            self.bufs[name] = (i, tuple(shape[j] for j in range(nd)), lib.poly_instance_buf_role(handle, i))
        self.params = [lib.poly_instance_param_name(handle, i).decode()
                       for i in range(lib.poly_instance_param_count(handle))]
        self._keep = []

    # ---- builders ----
    @classmethod
    def gpt2(cls, lib, vocab_size, n_embd, n_head, n_layer, max_seq_len, max_batch, norm_eps=1e-5):
        cfg = ffi.GPT2Config(vocab_size, n_embd, n_head, n_layer, max_seq_len, norm_eps)
        inst = cls(lib, lib.poly_gpt2_build(ctypes.byref(cfg), max_batch))
        inst.config = dict(vocab_size=vocab_size, n_embd=n_embd, n_head=n_head, n_layer=n_layer,
                           max_seq_len=max_seq_len, max_batch=max_batch)
        return inst

    @classmethod
    def mlp(cls, lib, layers, activation='relu', bias=True, batch_size=1, seed=42, loss='none'):
        spec = json.dumps({'layers': list(layers), 'activation': activation, 'bias': bool(bias),
                           'loss': loss, 'batch_size': int(batch_size), 'seed': int(seed)}).encode()
        return cls(lib, lib.poly_mlp_instance(spec, len(spec)))

    # ---- data ----
    def shape(self, name):
        return self.bufs[name][1]

    def write(self, name, array):
        """Set a named buffer (parameter or input) in whichever memory it lives."""
        idx, shape, _ = self.bufs[name]
        a = np.ascontiguousarray(array, dtype=np.float32).reshape(-1)
        n = int(np.prod(shape)) if shape else 1
        if a.size != n:
            raise ValueError(f'{name}: expected {n} elements, got {a.size}')
        if self.device == ffi.DEVICE_CUDA:
            if self.lib.poly_instance_upload_buf(self.h, idx, a.ctypes.data, a.nbytes) != 0:
                raise RuntimeError(f'upload of {name} failed')
        else:
            numel = ctypes.c_int64(0)
            p = self.lib.poly_instance_buf_data(self.h, idx, ctypes.byref(numel))
            ctypes.memmove(p, a.ctypes.data, a.nbytes)

    def read(self, name):
        idx, shape, _ = self.bufs[name]
        n = int(np.prod(shape)) if shape else 1
        out = np.empty(n, dtype=np.float32)
        if self.device == ffi.DEVICE_CUDA:
            if self.lib.poly_instance_readback_buf(self.h, idx, out.ctypes.data, out.nbytes) != 0:
                raise RuntimeError(f'readback of {name} failed')
        else:
            numel = ctypes.c_int64(0)
            p = self.lib.poly_instance_buf_data(self.h, idx, ctypes.byref(numel))
            ctypes.memmove(out.ctypes.data, p, out.nbytes)
        return out.reshape(shape)

    def export_weights(self):
        """All parameters as safetensors bytes (poly_instance_export_weights, src/instance.h:86)."""
        n = ctypes.c_int(0)
        p = self.lib.poly_instance_export_weights(self.h, ctypes.byref(n))
        if not p:
            raise RuntimeError('poly_instance_export_weights failed')
        return ctypes.string_at(p, n.value)      # the C buffer is left to the process (no matching free is exported)

    def import_weights(self, blob):
        """Safetensors bytes into the instance's buffers wherever they live; returns the
        bytes that went to device buffers."""
        moved = ctypes.c_longlong(0)
        if self.lib.poly_b200_instance_import_weights(self.h, blob, len(blob), ctypes.byref(moved)) != 0:
            raise RuntimeError('poly_b200_instance_import_weights failed: ' + self.lib.last_error())
        return moved.value

    def init_params(self, fn):
        for name in self.params:
            self.write(name, fn(name, self.shape(name)))

    def set_device(self, device_id):
        rc = self.lib.poly_instance_set_device(self.h, device_id)
        if rc != 0:
            msg = self.lib.last_error() if self.lib.has_cuda else ''
            raise RuntimeError(f'poly_instance_set_device({device_id}) failed: {msg}')
        self.device = device_id

    # ---- execution ----
    def forward(self, **inputs):
        """Run the forward entrypoint; keyword arguments are host arrays bound by
        buffer name (copied to the device inside the call when device-resident)."""
        n = len(inputs)
        io = (ffi.PolyIOBinding * max(n, 1))()
        keep = []
        for i, (name, arr) in enumerate(inputs.items()):
            a = np.ascontiguousarray(arr, dtype=np.float32)
            keep.append(a)
            io[i].name = name.encode()
            io[i].data = a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))
        rc = self.lib.poly_instance_forward(self.h, io, n)
        if rc != 0:
            msg = self.lib.last_error() if self.lib.has_cuda else ''
            raise RuntimeError(f'poly_instance_forward failed ({rc}) {msg}')

    def _bind(self, inputs):
        n = len(inputs)
        io = (ffi.PolyIOBinding * max(n, 1))()
        keep = []
        for i, (name, arr) in enumerate(inputs.items()):
            a = np.ascontiguousarray(arr, dtype=np.float32)
            keep.append(a)
            io[i].name = name.encode()
            io[i].data = a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))
        return io, n, keep

    def set_optimizer(self, kind, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0):
        """poly_instance_set_optimizer (src/instance.h:147); call before the first train_step."""
        if self.lib.poly_instance_set_optimizer(self.h, kind, lr, beta1, beta2, eps, weight_decay) != 0:
            raise RuntimeError('poly_instance_set_optimizer failed')

    def train_step(self, **io_arrays):
        """One forward + backward + optimizer update of the 'loss' entrypoint
        (poly_instance_train_step, src/instance.c:1242); returns the loss."""
        io, n, keep = self._bind(io_arrays)
        loss = ctypes.c_float(0)
        rc = self.lib.poly_instance_train_step(self.h, io, n, ctypes.byref(loss))
        if rc != 0:
            msg = self.lib.last_error() if self.lib.has_cuda else ''
            raise RuntimeError(f'poly_instance_train_step failed ({rc}) {msg}')
        return loss.value

    def value_and_grad(self, entrypoint='loss', **io_arrays):
        """Loss of a differentiable entrypoint; gradients stay inside the instance
        (poly_instance_value_and_grad, src/instance.c:1003)."""
        io, n, keep = self._bind(io_arrays)
        loss = ctypes.c_float(0)
        rc = self.lib.poly_instance_value_and_grad(self.h, entrypoint.encode(), io, n, ctypes.byref(loss))
        if rc != 0:
            msg = self.lib.last_error() if self.lib.has_cuda else ''
            raise RuntimeError(f'poly_instance_value_and_grad failed ({rc}) {msg}')
        return loss.value

    def gpt2_inputs(self, tokens):
        """Input buffers for a GPT-2 instance: token ids (as float32, which is how
        polygrad's builder takes them), positions and the arange helper."""
        t = self.config['max_seq_len']
        return dict(x=np.asarray(tokens, dtype=np.float32),
                    positions=np.arange(t, dtype=np.float32),
                    arange=np.arange(t, dtype=np.float32))

    def free(self):
        if self.h:
            self.lib.poly_instance_free(self.h)
            self.h = None
