"""polygrad's older eager entry point, poly_realize_cuda (src/frontend.c:2450), which polygrad's
Python Tensor uses: host pointers in the bindings, results fetched with poly_cuda_copyback.

The reference code schedules on every call, keeps its own host-pointer-keyed device buffers and a
program cache, and drives the device only through the 13 backend symbols (linearize, render,
compile, launch with its own grid numbers, alloc, copies); it still runs unchanged on this backend
(POLY_B200_LEGACY=ref).  By default the entry point compiles the schedule into a plan instead, so
the eager API gets the fused kernels; the plan is kept and found again by the graph's structure, and
what a call writes stays on the device until poly_cuda_copyback asks for it."""
import ctypes

import numpy as np
import pytest

from conftest import assert_close
from polygrad_b200 import ffi
from polygrad_b200.tensor import Device

pytestmark = pytest.mark.gpu


def bindings(pairs):
    binds = (ffi.PolyBufferBinding * len(pairs))()
    for i, (buf, host) in enumerate(pairs):
        binds[i].buffer = buf
        binds[i].handle.ptr = host.ctypes.data          # host pointers: the path uploads them itself
        binds[i].handle.nbytes = host.nbytes
        binds[i].handle.domain = ffi.DEVICE_CPU
    return binds


def realize_only(lib, dev, tensor, out=None):
    """poly_realize_cuda without the copy back: returns (output BUFFER, host array, pairs)."""
    n = tensor.numel()
    out_buf = lib.poly_buffer_by_id(dev.ctx, n, ffi.DTYPE_IDS['float32'])
    out = np.zeros(n, np.float32) if out is None else out
    sink = lib.poly_sink1(dev.ctx, lib.poly_store_val(dev.ctx, out_buf, tensor.uop))
    pairs = list(tensor.leaves) + [(out_buf, out)]
    assert lib.poly_realize_cuda(dev.ctx, sink, bindings(pairs), len(pairs)) == 0, lib.last_error()
    return out_buf, out, pairs


def realize_legacy(lib, dev, tensor):
    """What polygrad's Tensor does (py/polygrad/tensor.py:322-364): realize, then copy every binding back."""
    _, out, pairs = realize_only(lib, dev, tensor)
    assert lib.poly_cuda_copyback(bindings(pairs), len(pairs)) == 0
    return out.reshape(tensor.shape)


def leaf_of(dev, buf, host, shape):
    """A tensor over an existing BUFFER node and its host array (what polygrad's Tensor is after a realize)."""
    from polygrad_b200.tensor import Tensor, _i64
    uop = buf if len(shape) == 1 else dev.lib.poly_reshape(dev.ctx, buf, _i64(shape), len(shape))
    return Tensor(dev, uop, shape, 'float32', [(buf, host)])


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
    plan of the first and allocate nothing more."""
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


def test_eager_plans_are_found_again_by_structure(gpu, monkeypatch):
    """Every call below brings new leaves, a new output BUFFER and a new SINK, with new values in new
    host arrays; the plan compiled for the first serves the rest, bound to the new buffers by position.
    A graph of another shape, or the same one under another contraction policy, gets its own plan."""
    monkeypatch.delenv('POLY_B200_LEGACY', raising=False)
    gpu.poly_cuda_prog_cache_flush()
    cuda = Device(gpu, ffi.DEVICE_CUDA)
    rng = np.random.default_rng(21)
    before = gpu.eager_stats()
    for i in range(12):
        x = rng.standard_normal((192, 160)).astype(np.float32) * (1 + i)
        w = rng.standard_normal((160, 96)).astype(np.float32)
        got = realize_legacy(gpu, cuda, (cuda.tensor(x).dot(cuda.tensor(w)) * 0.5).relu())
        assert_close(got, np.maximum(x.astype(np.float64) @ w * 0.5, 0), 1e-5, f'call {i}')
    st = gpu.eager_stats()
    assert st['misses'] - before['misses'] == 1 and st['hits'] - before['hits'] == 11
    assert st['plans_kept'] == before['plans_kept'] + 1 and st['buffers_resident'] == 0
    x = rng.standard_normal((96, 160)).astype(np.float32)                  # other extents: another plan
    got = realize_legacy(gpu, cuda, (cuda.tensor(x).dot(cuda.tensor(w)) * 0.5).relu())
    assert_close(got, np.maximum(x.astype(np.float64) @ w * 0.5, 0), 1e-5, 'other extents')
    assert gpu.eager_stats()['misses'] - before['misses'] == 2
    gpu.poly_b200_set_gemm_policy(1)
    try:
        got = realize_legacy(gpu, cuda, (cuda.tensor(x).dot(cuda.tensor(w)) * 0.5).relu())
    finally:
        gpu.poly_b200_set_gemm_policy(0)
    assert gpu.eager_stats()['misses'] - before['misses'] == 3
    assert_close(got, np.maximum(x.astype(np.float64) @ w * 0.5, 0), 2e-2, 'bf16 policy')
    kept = gpu.eager_stats()['plans_kept']
    cuda.close()                                   # a context takes its plans with it
    assert gpu.eager_stats()['plans_kept'] == kept - 3


def test_results_stay_on_the_device_until_copied_back(gpu, monkeypatch):
    """poly_realize_cuda leaves what it wrote on the device (reference: src/frontend.c:2650-2660); a
    second realize that binds the first one's output reads it there -- nothing is uploaded for it and
    the host array is still untouched -- and poly_cuda_copyback fetches either result."""
    monkeypatch.delenv('POLY_B200_LEGACY', raising=False)
    cuda = Device(gpu, ffi.DEVICE_CUDA)
    x = np.random.default_rng(5).standard_normal((256, 512)).astype(np.float32)
    y_host = np.full(x.size, -7.0, np.float32)
    y_buf, _, y_pairs = realize_only(gpu, cuda, (cuda.tensor(x) * 0.25).exp(), out=y_host)
    assert (y_host == -7.0).all() and gpu.eager_stats()['buffers_resident'] == 1
    gpu.poly_b200_stats_reset()
    z_buf, z_host, z_pairs = realize_only(gpu, cuda, leaf_of(cuda, y_buf, y_host, x.shape).sum(-1))
    st = gpu.stats()
    assert st['bytes_htod'] == 0 and st['bytes_dtoh'] == 0
    assert (y_host == -7.0).all() and gpu.eager_stats()['buffers_resident'] == 2
    assert gpu.poly_cuda_copyback(bindings(z_pairs[-1:]), 1) == 0
    assert_close(z_host, np.exp(x.astype(np.float64) * 0.25).sum(-1), 1e-5, 'sum of the resident result')
    assert (y_host == -7.0).all()
    assert gpu.poly_cuda_copyback(bindings(y_pairs), len(y_pairs)) == 0
    assert_close(y_host.reshape(x.shape), np.exp(x.astype(np.float64) * 0.25), 1e-5, 'first result')
    assert gpu.eager_stats()['buffers_resident'] == 0
    assert gpu.stats()['bytes_dtoh'] == y_host.nbytes + z_host.nbytes
    cuda.close()


def test_host_memory_handed_out_again_is_uploaded(gpu, monkeypatch):
    """A result that was never copied back, whose host array then serves another tensor: the other
    tensor has its own BUFFER node, so its values are uploaded and the stale device copy is dropped,
    not written over the new owner's data."""
    monkeypatch.delenv('POLY_B200_LEGACY', raising=False)
    cuda = Device(gpu, ffi.DEVICE_CUDA)
    x = np.linspace(-1, 1, 4096, dtype=np.float32)
    host = np.zeros(4096, np.float32)
    realize_only(gpu, cuda, cuda.tensor(x) * 3, out=host)              # 3x stays on the device
    assert gpu.eager_stats()['buffers_resident'] == 1
    host[:] = np.arange(4096, dtype=np.float32)                        # the array now belongs to someone else
    other = cuda.lib.poly_buffer_by_id(cuda.ctx, 4096, ffi.DTYPE_IDS['float32'])
    got = realize_legacy(gpu, cuda, leaf_of(cuda, other, host, (4096,)) + 1)
    assert_close(got, np.arange(4096) + 1.0, 1e-6, 'values of the new owner')
    assert np.array_equal(host, np.arange(4096, dtype=np.float32))
    assert gpu.eager_stats()['buffers_resident'] == 0
    cuda.close()


def test_write_back_at_once_when_asked(gpu, monkeypatch):
    monkeypatch.delenv('POLY_B200_LEGACY', raising=False)
    monkeypatch.setenv('POLY_B200_EAGER_RESIDENT', '0')
    monkeypatch.setenv('POLY_B200_EAGER_CACHE', '0')
    cuda = Device(gpu, ffi.DEVICE_CUDA)
    x = np.random.default_rng(6).standard_normal((64, 96)).astype(np.float32)
    kept = gpu.eager_stats()['plans_kept']
    _, out, _ = realize_only(gpu, cuda, cuda.tensor(x).softmax(-1))
    e = np.exp(x - x.max(-1, keepdims=True))
    assert_close(out.reshape(x.shape), e / e.sum(-1, keepdims=True), 1e-5, 'written back by the call itself')
    assert gpu.eager_stats()['plans_kept'] == kept and gpu.eager_stats()['buffers_resident'] == 0
    cuda.close()
