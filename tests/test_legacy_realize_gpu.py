"""polygrad's older eager path, poly_realize_cuda (src/frontend.c:2450): it schedules on every call,
keeps its own host-pointer-keyed device buffers and a program cache, and drives the device only
through the 13 backend symbols (linearize, render, compile, launch with its own grid numbers, alloc,
copies).  polygrad's Python Tensor uses it.  It must keep working on top of this backend unchanged."""
import ctypes

import numpy as np
import pytest

from conftest import assert_close
from polygrad_b200 import ffi
from polygrad_b200.tensor import Device

pytestmark = pytest.mark.gpu


def realize_legacy(lib, dev, tensor):
    n = tensor.numel()
    out_buf = lib.poly_buffer_by_id(dev.ctx, n, ffi.DTYPE_IDS['float32'])
    out = np.zeros(n, np.float32)
    sink = lib.poly_sink1(dev.ctx, lib.poly_store_val(dev.ctx, out_buf, tensor.uop))
    pairs = list(tensor.leaves) + [(out_buf, out)]
    binds = (ffi.PolyBufferBinding * len(pairs))()
    for i, (buf, host) in enumerate(pairs):
        binds[i].buffer = buf
        binds[i].handle.ptr = host.ctypes.data          # host pointers: the path uploads them itself
        binds[i].handle.nbytes = host.nbytes
        binds[i].handle.domain = ffi.DEVICE_CPU
    lib.poly_realize_cuda.restype = ctypes.c_int
    lib.poly_realize_cuda.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ffi.PolyBufferBinding), ctypes.c_int]
    lib.poly_cuda_copyback.restype = ctypes.c_int
    lib.poly_cuda_copyback.argtypes = [ctypes.POINTER(ffi.PolyBufferBinding), ctypes.c_int]
    assert lib.poly_realize_cuda(dev.ctx, sink, binds, len(pairs)) == 0, lib.last_error()
    assert lib.poly_cuda_copyback(binds, len(pairs)) == 0
    return out.reshape(tensor.shape)


def test_legacy_path_runs_on_the_backend(ref_lib, gpu):
    cpu, cuda = Device(ref_lib, ffi.DEVICE_CPU), Device(gpu, ffi.DEVICE_CUDA)
    rng = np.random.default_rng(12)
    x = rng.standard_normal((96, 320)).astype(np.float32)
    w = rng.standard_normal((320, 64)).astype(np.float32)
    for build in (lambda t, v: (t * 2 + 1).exp(), lambda t, v: t.softmax(-1), lambda t, v: t.dot(v).relu(),
                  lambda t, v: t.permute(1, 0)):
        want = build(cpu.tensor(x), cpu.tensor(w)).numpy()
        got = realize_legacy(gpu, cuda, build(cuda.tensor(x), cuda.tensor(w)))
        assert_close(got, want, 1e-5, 'legacy realize')
    # a second call with the same graph shape goes through the path's program cache
    got = realize_legacy(gpu, cuda, (cuda.tensor(x) * 2 + 1).exp())
    assert_close(got, np.exp(x * 2 + 1), 1e-5, 'legacy realize, cached programs')
    gpu.poly_cuda_flush_buffers()
    gpu.poly_cuda_prog_cache_flush()
