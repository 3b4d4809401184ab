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


# ── the lookup's gradient ───────────────────────────────────────────────
def lookup_gradient(dev, ids, arange, g):
    """out[v, d] = sum over the token axes of where(ids == arange[v], g[..., d], 0), as the backward of the
    lookup writes it (one axis: a single sum; two axes: a sum of a sum)."""
    V, D = arange.shape[0], g.shape[-1]
    full = ids.shape + (V, D)
    i = dev.tensor(ids).reshape(*ids.shape, 1, 1).expand(*full)
    a = dev.tensor(arange).reshape(*([1] * ids.ndim), V, 1).expand(*full)
    gg = dev.tensor(g).reshape(*ids.shape, 1, D).expand(*full)
    out = i.eq(a).where(gg, 0.0)
    for _ in ids.shape:
        out = out.sum(0)
    return out.numpy()


def both_gradients(devices, gpu, ids, arange, g):
    want = lookup_gradient(devices[0], ids, arange, g)
    gpu.poly_b200_stats_reset()
    got = lookup_gradient(devices[1], ids, arange, g)
    st = gpu.stats()
    assert st['launches_generated'] == 0 and st['launches_precompiled'] >= 1, st      # a precompiled kernel took it
    assert got.shape == want.shape == (arange.shape[0], g.shape[-1])
    return got, want


@pytest.mark.parametrize('shape', [(96,), (3, 32), (2, 700)], ids=str)
def test_lookup_gradient_sums_rows_by_token(devices, gpu, shape):
    """For every table row the gradient rows of the tokens that name it, added in token order from +0.  One
    token axis goes through the lookup kernel with the roles of ids and arange exchanged (several matches per
    row): bit for bit the CPU's sum.  Two token axes (batch, position) go through the kernel that scans the
    tokens per group of table rows; written as a sum of a sum the CPU adds per-position partial sums, the
    kernel one running sum, so those agree to float32 rounding (1e-5 of the summed magnitudes)."""
    V, D = 40, 24
    rng = np.random.default_rng(len(shape))
    ids = rng.integers(0, V, shape).astype(np.float32)
    g = rng.standard_normal(shape + (D,)).astype(np.float32)
    got, want = both_gradients(devices, gpu, ids, np.arange(V, dtype=np.float32), g)
    flat_ids, flat_g = ids.reshape(-1).astype(np.int64), g.reshape(-1, D).astype(np.float64)
    exact = np.zeros((V, D))
    np.add.at(exact, flat_ids, flat_g)
    tol = 1e-5 * np.abs(flat_g).sum(0).max()
    if len(shape) == 1:
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.abs(got - want).max() <= tol and np.abs(got - exact).max() <= tol


def test_lookup_gradient_odd_ids_and_tables(devices, gpu):
    """Ids that name no row (NaN, out of range, fractional) contribute nothing; a table numbering with
    duplicates sends a token's gradient to every row carrying its number; rows nobody names are +0."""
    V, D = 24, 8
    arange = np.arange(V, dtype=np.float32)
    arange[5] = 3.0                                   # rows 3 and 5 carry the same number
    arange[7] = np.nan                                # a row no id can name
    ids = np.array([[3.0, 3.0, np.nan, -1.0, 24.0, 2.5, 7.0, 0.0], [23.0, 3.0, 5.0, 0.0, 1e9, -0.0, 11.0, 11.0]], np.float32)
    g = np.random.default_rng(9).standard_normal(ids.shape + (D,)).astype(np.float32)
    got, want = both_gradients(devices, gpu, ids, arange, g)
    assert np.array_equal(np.isnan(got), np.isnan(want)) and np.abs(got - want).max() <= 1e-5 * np.abs(g).sum()
    assert np.array_equal(got[3], got[5]) and got[3].any()
    assert not got[7].any() and not got[5 + 1].any() and not np.signbit(got[7]).any()


def test_lookup_gradient_of_one_repeated_token(devices, gpu):
    """More matches for one row than the kernel lists (a batch that repeats one token 1500 times): the
    ordered scan takes over."""
    V, D = 32, 16
    ids = np.full((3, 500), 9.0, np.float32)
    ids[1, 17] = 4.0
    g = np.random.default_rng(10).standard_normal(ids.shape + (D,)).astype(np.float32)
    got, want = both_gradients(devices, gpu, ids, np.arange(V, dtype=np.float32), g)
    assert np.abs(got - want).max() <= 1e-5 * np.abs(g).sum(axis=(0, 1)).max()
    exact = g.astype(np.float64).sum(axis=(0, 1)) - g[1, 17]
    assert np.abs(got[9] - exact).max() <= 1e-5 * np.abs(g).sum(axis=(0, 1)).max()
    assert np.array_equal(got[4], g[1, 17] + 0.0) and not got[0].any()
