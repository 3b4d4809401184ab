"""polygrad's older eager entry point, poly_realize_cuda (src/frontend.c:2450), which polygrad's
Python Tensor uses: host pointers in the bindings, results fetched with poly_cuda_copyback.

The reference code schedules on every call, keeps its own host-pointer-keyed device buffers and a
program cache, and drives the device only through the 13 backend symbols (linearize, render,
compile, launch with its own grid numbers, alloc, copies); it still runs unchanged on this backend
(POLY_B200_LEGACY=ref).  By default the entry point compiles the schedule into a plan instead, so
the eager API gets the fused kernels, and runs it on the host pointers directly."""
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


@pytest.mark.parametrize('route', ['plan', 'ref'])
def test_legacy_path_runs_on_the_backend(ref_lib, gpu, monkeypatch, route):
    if route == 'ref':
        monkeypatch.setenv('POLY_B200_LEGACY', 'ref')
    else:
        monkeypatch.delenv('POLY_B200_LEGACY', raising=False)
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


def test_eager_entry_runs_fused_kernels(gpu, monkeypatch):
    """softmax is three scheduled kernels; through the plan route it is one launch, through the
    reference route three.  Repeated calls (a new SINK each, as polygrad's Tensor makes them) reuse the
    compiled programs and leave no plan behind."""
    cuda = Device(gpu, ffi.DEVICE_CUDA)
    x = np.random.default_rng(4).standard_normal((512, 1024)).astype(np.float32)
    e = np.exp(x - x.max(-1, keepdims=True))
    want = e / e.sum(-1, keepdims=True)
    monkeypatch.delenv('POLY_B200_LEGACY', raising=False)
    realize_legacy(gpu, cuda, cuda.tensor(x).softmax(-1))          # compiles
    held = gpu.stats()['bytes_allocated']
    gpu.poly_b200_stats_reset()
    for _ in range(20):
        got = realize_legacy(gpu, cuda, cuda.tensor(x).softmax(-1))
    st = gpu.stats()
    assert_close(got, want, 1e-5, 'softmax through the eager entry')
    assert st['launches'] == 20 and st['programs_compiled'] == 0
    assert st['bytes_allocated'] <= held + (1 << 20)
    monkeypatch.setenv('POLY_B200_LEGACY', 'ref')
    gpu.poly_b200_stats_reset()
    got = realize_legacy(gpu, cuda, cuda.tensor(x).softmax(-1))
    assert_close(got, want, 1e-5, 'softmax through the reference route')
    assert gpu.stats()['launches'] == 3
    gpu.poly_cuda_flush_buffers()
    gpu.poly_cuda_prog_cache_flush()
