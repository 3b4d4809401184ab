"""Embedding lookup on the B200 against stock polygrad on the CPU, bit for bit.
polygrad writes table[ids] as a one-hot contraction over float32 ids and a
float32 arange buffer (src/modelzoo/models/gpt2.c:93-153); the result is defined
for any contents of both, and the kernel must reproduce it for all of them."""
import numpy as np
import pytest

from polygrad_b200 import ffi
from polygrad_b200.tensor import Device, embedding

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def devices(ref_lib, gpu):
    return Device(ref_lib, ffi.DEVICE_CPU), Device(gpu, ffi.DEVICE_CUDA)


def both(devices, ids, arange, table):
    out = []
    for dev in devices:
        out.append(embedding(dev.tensor(ids), dev.tensor(arange), dev.tensor(table)).numpy())
    want, got = out
    assert got.shape == want.shape == ids.shape + (table.shape[1],)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    return got


def table_of(V, D, seed=0):
    t = np.random.default_rng(seed).standard_normal((V, D)).astype(np.float32)
    t[0, 0] = -0.0                       # comes out as +0.0: the sum starts from +0
    return t


@pytest.mark.parametrize('V,D,shape', [(50, 24, (7,)), (211, 96, (2, 48)), (1000, 64, (3, 5)), (37, 130, (4, 4))])
def test_identity_arange(devices, V, D, shape):
    rng = np.random.default_rng(V)
    ids = rng.integers(0, V, shape).astype(np.float32)
    got = both(devices, ids, np.arange(V, dtype=np.float32), table_of(V, D))
    tab = table_of(V, D)
    assert np.array_equal(got, tab[ids.astype(np.int64)] + 0.0)


def test_ids_without_a_match_give_zero_rows(devices):
    V, D = 40, 16
    ids = np.array([3.0, -1.0, 40.0, 1e9, 2.5, np.nan, np.inf, -np.inf, 0.0, 39.0, -0.0], np.float32)
    got = both(devices, ids, np.arange(V, dtype=np.float32), table_of(V, D))
    for i in (1, 2, 3, 4, 5, 6, 7):
        assert not got[i].any()
    assert np.signbit(got[8, 0]) == False and np.array_equal(got[10], got[8])  # noqa: E712


def test_increasing_arange_that_is_not_the_identity(devices):
    """Sorted but shifted and scaled: the id is not the row number."""
    V, D = 64, 8
    arange = (np.arange(V, dtype=np.float32) * 3.0 - 20.0)
    ids = np.array([-20.0, -17.0, 169.0, 0.0, 1.0, 100.0, 10.0], np.float32)
    got = both(devices, ids, arange, table_of(V, D))
    tab = table_of(V, D)
    assert np.array_equal(got[1], tab[1] + 0.0) and np.array_equal(got[2], tab[63] + 0.0) and not got[3].any()


def test_unsorted_arange(devices):
    V, D = 97, 12
    arange = np.random.default_rng(5).permutation(V).astype(np.float32)
    ids = np.random.default_rng(6).integers(0, V, (3, 9)).astype(np.float32)
    both(devices, ids, arange, table_of(V, D))


def test_arange_with_duplicates_sums_rows_in_order(devices):
    V, D = 30, 10
    arange = np.arange(V, dtype=np.float32)
    arange[[4, 11, 29]] = 7.0            # id 7 now selects rows 4, 7, 11 and 29
    arange[2] = np.nan
    ids = np.array([7.0, 4.0, 2.0, 5.0], np.float32)
    got = both(devices, ids, arange, table_of(V, D))
    assert not got[1].any() and not got[2].any()


def test_arange_all_equal(devices):
    """More matches than the kernel keeps in its list: the ordered scan path."""
    V, D = 20, 6
    ids = np.array([1.0, 2.0], np.float32)
    both(devices, ids, np.ones(V, np.float32), table_of(V, D))
