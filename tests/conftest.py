import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# The stock polygrad CPU runtime execs "clang" per kernel (src/runtime_cpu.c:128);
# the image only has gcc, so tests put a forwarding script first on PATH.
os.environ['PATH'] = os.path.join(ROOT, 'oracle', 'shim') + os.pathsep + os.environ.get('PATH', '')

REF_LIB = os.path.join(ROOT, 'oracle', '_ref', 'libpolygrad_ref.so')


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a B200 (run with -m gpu)')


@pytest.fixture(scope='session')
def ref_lib():
    """Stock polygrad built from its own sources (CPU backend): the checker."""
    from polygrad_b200 import ffi
    if not os.path.isfile(REF_LIB):
        pytest.skip('oracle/_ref/libpolygrad_ref.so not built (make -C oracle ref)')
    return ffi.load_reference(REF_LIB)


@pytest.fixture(scope='session')
def product_lib():
    from polygrad_b200 import ffi
    return ffi.product()


@pytest.fixture(scope='session')
def gpu(product_lib):
    """The product library initialised on a real device; fails (not skips) without one."""
    assert product_lib.poly_cuda_init() == 0, 'no usable B200: ' + product_lib.last_error()
    return product_lib


def assert_close(got, want, rtol, what=''):
    """|got-want| <= atol + rtol*|want| with atol = rtol * rms(want)."""
    import numpy as np
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f'{what}: shape {got.shape} vs {want.shape}'
    finite = np.isfinite(want)
    assert np.array_equal(np.isfinite(got), finite), f'{what}: non-finite pattern differs'
    assert np.array_equal(got[~finite], want[~finite], equal_nan=True), f'{what}: inf/nan values differ'
    rms = float(np.sqrt(np.mean(want[finite] ** 2))) if finite.any() else 0.0
    atol = rtol * rms
    err = np.abs(got[finite] - want[finite])
    bound = atol + rtol * np.abs(want[finite])
    bad = err > bound
    assert not bad.any(), (f'{what}: {int(bad.sum())}/{err.size} outside tolerance rtol={rtol}; '
                           f'max err {err.max():.3e}, rms(want) {rms:.3e}')
