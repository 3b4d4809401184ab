"""Row-op kernels on the B200 against stock polygrad on the CPU: the same graph,
built by polygrad's frontend, realized once per backend (the pattern of
polygrad test/test_cuda.c:438-516).  Tolerance for fp32 elementwise and
reduction kernels: 1e-5 relative; movement ops bit-exact."""
import numpy as np
import pytest

from conftest import assert_close
from polygrad_b200 import ffi
from polygrad_b200.tensor import Device

pytestmark = pytest.mark.gpu

RTOL = 1e-5

OPS = {
    'affine': lambda t: t * 2 + 1,
    'exp': lambda t: t.exp(),
    'tanh': lambda t: t.tanh(),
    'gelu': lambda t: t.gelu(),
    'sum': lambda t: t.sum(-1),
    'max': lambda t: t.max(-1),
    'mean': lambda t: t.mean(-1),
    'var': lambda t: t.var(-1),
    'sum0': lambda t: t.sum(0),
    'softmax': lambda t: t.softmax(-1),
    'layernorm': lambda t: t.layernorm(-1, 1e-5),
    # polygrad has no RMSNorm builder; this is the composition a caller writes
    'rmsnorm': lambda t: t / ((t * t).mean(-1, keepdim=True) + 1e-6).sqrt(),
}
EXACT = {
    'permute': lambda t: t.permute(1, 0),
    'flip0': lambda t: t[::-1],
    'flip1': lambda t: t[:, ::-1],
    'step3': lambda t: t[:, ::3],
    'shrink': lambda t: t.shrink(((1, t.shape[0] - 1), (3, t.shape[1] - 2))),
    'pad': lambda t: t.pad(((1, 2), (0, 3))),
}
SHAPES = [(64, 128), (33, 257), (5, 4096), (256, 1000), (1, 7), (256, 10)]   # (256, 10): the MLP's class scores


@pytest.fixture(scope='module')
def devices(ref_lib, gpu):
    return Device(ref_lib, ffi.DEVICE_CPU), Device(gpu, ffi.DEVICE_CUDA)


@pytest.mark.parametrize('shape', SHAPES, ids=str)
@pytest.mark.parametrize('name', sorted(OPS))
def test_rowop_matches_cpu(devices, name, shape):
    cpu, cuda = devices
    x = np.random.default_rng(hash((name, shape)) % 2**32).standard_normal(shape).astype(np.float32)
    want = OPS[name](cpu.tensor(x)).numpy()
    got = OPS[name](cuda.tensor(x)).numpy()
    assert_close(got, want, RTOL, f'{name}{shape}')


@pytest.mark.parametrize('shape', SHAPES[:4], ids=str)
@pytest.mark.parametrize('name', sorted(EXACT))
def test_movement_bit_exact(devices, name, shape):
    cpu, cuda = devices
    x = np.random.default_rng(7).standard_normal(shape).astype(np.float32)
    want = EXACT[name](cpu.tensor(x)).numpy()
    got = EXACT[name](cuda.tensor(x)).numpy()
    assert got.shape == want.shape
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name


@pytest.mark.parametrize('shape', [(3, 64, 128), (2, 100, 36), (4, 31, 50)], ids=str)
def test_batched_transpose_bit_exact(devices, shape):
    cpu, cuda = devices
    x = np.random.default_rng(11).standard_normal(shape).astype(np.float32)
    want = cpu.tensor(x).permute(0, 2, 1).numpy()
    got = cuda.tensor(x).permute(0, 2, 1).numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.array_equal(got, x.transpose(0, 2, 1))


def test_matmul_small(devices):
    cpu, cuda = devices
    rng = np.random.default_rng(3)
    a = rng.uniform(-1, 1, (96, 200)).astype(np.float32)
    b = rng.uniform(-1, 1, (200, 72)).astype(np.float32)
    want = cpu.tensor(a).dot(cpu.tensor(b)).numpy()
    got = cuda.tensor(a).dot(cuda.tensor(b)).numpy()
    assert_close(got, want, RTOL, 'matmul')
