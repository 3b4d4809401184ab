"""Kernels outside the recognised classes -- integer and 64-bit arithmetic, casts, predicates,
transcendental chains, reductions along non-contiguous axes, multi-axis reductions -- go through
the general renderer (every scheduled UOp tree rendered to CUDA C and compiled for sm_100a).  Same
graph on stock polygrad's CPU backend and on the B200; float32 within 1e-5, integers exact."""
import numpy as np
import pytest

from conftest import assert_close
from polygrad_b200 import ffi
from polygrad_b200.tensor import Device

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def devices(ref_lib, gpu):
    return Device(ref_lib, ffi.DEVICE_CPU), Device(gpu, ffi.DEVICE_CUDA)


X = np.random.default_rng(31).standard_normal((37, 130)).astype(np.float32)
POS = np.abs(X) + 0.5

FLOAT_CASES = {
    'log_sqrt': (POS, lambda t: t.log() + t.sqrt()),
    'sin': (X, lambda t: (t * 3).sin()),
    'sigmoid_chain': (X, lambda t: (t.sigmoid() * t).tanh() - t.relu()),
    'div': (POS, lambda t: (t + 1) / (t * t + 2)),
    'where_eq': (np.round(X), lambda t: t.eq(t * 0).where(t + 5, -1.0)),
    'f64_roundtrip': (X, lambda t: (t.cast('float64') * 1.5 + 0.25).cast('float32')),
    'sum_axis0_noncontiguous': (X, lambda t: t.sum(0)),
    'max_axis0': (X, lambda t: t.max(0)),
    'sum_all': (X, lambda t: t.sum(1).sum(0)),
    'mean_of_exp': (X, lambda t: t.exp().mean(-1)),
    'broadcast_row_col': (X, lambda t: t - t.mean(-1, keepdim=True) + t.max(0, keepdim=True)),
    'pad_then_reduce': (X, lambda t: t.pad(((2, 1), (3, 0))).sum(-1)),
    'permute_then_softmax': (X, lambda t: t.permute(1, 0).softmax(-1)),
}


@pytest.mark.parametrize('name', sorted(FLOAT_CASES))
def test_float_graphs(devices, name):
    cpu, cuda = devices
    x, build = FLOAT_CASES[name]
    want = build(cpu.tensor(x)).numpy()
    got = build(cuda.tensor(x)).numpy()
    assert got.shape == want.shape
    assert_close(got, want, 1e-5, name)


def test_int32_arithmetic_is_exact(devices):
    cpu, cuda = devices
    x = np.round(X * 50).astype(np.float32)
    build = lambda t: ((t.cast('int32') * 7 + 3).cast('float32') - t * 2)
    want = build(cpu.tensor(x)).numpy()
    got = build(cuda.tensor(x)).numpy()
    assert np.array_equal(got, want)
    build_i = lambda t: (t.cast('int32') * 3 + 1)
    want_i = build_i(cpu.tensor(x)).numpy()
    got_i = build_i(cuda.tensor(x)).numpy()
    assert want_i.dtype == np.int32 and np.array_equal(got_i, want_i)
