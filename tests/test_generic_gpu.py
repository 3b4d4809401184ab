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


BIG = np.random.default_rng(32).standard_normal((1536, 2048)).astype(np.float32)

B64 = BIG.astype(np.float64)
LONG_REDUCTIONS = {
    # one output over 3.1 M elements: cut into parts, one block each, combined in index order
    'sum_of_squares_to_a_scalar': (lambda t: (t * t).reshape(1536 * 2048).sum(-1), np.array([(B64 * B64).sum()]), (B64 * B64).sum()),
    # a reduction of a reduction with the same operation: one reduction over both axes
    'sum_of_row_sums': (lambda t: t.sum(-1).sum(-1), np.array([B64.sum()]), np.abs(B64).sum()),
    'max_of_row_maxima': (lambda t: t.max(-1).max(-1), np.array([B64.max()]), 0.0),
    # a handful of outputs, each over 0.5 M elements
    'six_partial_sums': (lambda t: (t * 0.5).reshape(6, 256 * 2048).sum(-1), (B64 * 0.5).reshape(6, -1).sum(-1),
                         np.abs(B64 * 0.5).reshape(6, -1).sum(-1).max()),
}


@pytest.mark.parametrize('name', sorted(LONG_REDUCTIONS))
def test_long_reductions_to_few_outputs(devices, gpu, name):
    """A few outputs that each reduce a very long range (a loss scalar over every logit) are cut into
    parts over many blocks; the block that finishes last combines the partial results in a fixed
    order, so two runs give the same bits.  The yardstick is the sum in float64: a float32 sum of
    3 M terms taken serially (what the CPU backend does) is itself 0.3 % off, so the CPU result is
    only required to be no closer to the truth than the B200's by more than its own error allows."""
    cpu, cuda = devices
    build, truth, magnitude = LONG_REDUCTIONS[name]
    want = build(cpu.tensor(BIG)).numpy()
    gpu.poly_b200_stats_reset()
    got = build(cuda.tensor(BIG)).numpy()
    assert gpu.stats()['launches'] == 1
    again = build(cuda.tensor(BIG)).numpy()
    assert got.shape == want.shape == truth.shape
    # partial sums of at most a few thousand terms each, then a few hundred partials: 1e-6 of the magnitudes
    assert np.abs(got.astype(np.float64) - truth).max() <= 2e-6 * magnitude
    assert np.abs(want.astype(np.float64) - truth).max() <= 1e-2 * magnitude
    assert np.array_equal(got.view(np.uint32), again.view(np.uint32))
