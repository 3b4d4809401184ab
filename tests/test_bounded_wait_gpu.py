"""Every barrier wait in the tensor-core kernels is bounded: a wait that cannot complete gives up,
records a code in a device word that the host reports at its next synchronisation, and the kernel
returns.  The library's self-test provokes exactly that with a barrier nothing arrives at (and a
short limit), then clears the word; afterwards the context must still compute."""
import numpy as np
import pytest

from conftest import assert_close
from polygrad_b200 import ffi
from polygrad_b200.tensor import Device

pytestmark = pytest.mark.gpu


def test_wait_that_cannot_complete_gives_up_and_context_survives(gpu):
    assert gpu.poly_b200_selftest_bounded_wait() == 0, gpu.last_error()
    assert gpu.poly_b200_synchronize() == 0, gpu.last_error()       # the error word was cleared
    cuda = Device(gpu, ffi.DEVICE_CUDA)
    rng = np.random.default_rng(8)
    a = rng.uniform(-1, 1, (256, 128)).astype(np.float32)
    b = rng.uniform(-1, 1, (128, 192)).astype(np.float32)
    gpu.poly_b200_set_gemm_policy(1)
    try:
        got = cuda.tensor(a).dot(cuda.tensor(b)).numpy()
    finally:
        gpu.poly_b200_set_gemm_policy(0)
    assert_close(got, a @ b, 2e-2, 'contraction after the self-test')
