"""poly_b200_gemm_noalloc: the bf16 tensor-core contraction for callers that
cannot allocate device memory (inside a stream capture, with device memory
fully committed elsewhere, or where a driver allocation's implicit
synchronisation is unacceptable).  Its scratch is a fixed array inside the
library instead of pool memory.

Checked against numpy on the same bfloat16-rounded operands accumulated in
float64 (1e-4) and against the allocating entry point poly_b200_gemm, on calls
in a row with different operands (the shared scratch keeps the previous call's
contents: the third problem is smaller and has a K that is not a multiple of 8,
so its padded rows lie over what the larger call left); that the call leaves
the runtime's pool untouched; and for the size limit.  Runs last so that a
failure here cannot hide the other tests' results."""
import ctypes

import numpy as np
import pytest

from conftest import assert_close

pytestmark = pytest.mark.gpu


def _dev(lib, a):
    d = lib.poly_cuda_alloc(a.nbytes)
    assert d
    assert lib.poly_cuda_copy_htod(d, a.ctypes.data, a.nbytes) == 0
    return d


def _bf16_round(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def _pool_state(lib):
    n = lib.poly_b200_pool_free_sizes(None, 0)
    return lib.stats()['bytes_allocated'], n


def _run(lib, fn_name, a, b, bias, relu):
    m, k = a.shape
    n = b.shape[1]
    da, db, dx = _dev(lib, a), _dev(lib, b), _dev(lib, bias)
    dc = lib.poly_cuda_alloc(m * n * 4)
    if fn_name == 'poly_b200_gemm':
        rc = lib.poly_b200_gemm(m, n, k, da, k, 1, db, n, 1, dc, n, dx, relu, 0)
    else:
        before = _pool_state(lib)
        rc = lib.poly_b200_gemm_noalloc(m, n, k, da, k, 1, db, n, 1, dc, n, dx, relu)
        # the defining property: nothing taken from the driver, nothing taken from or given to the pool
        assert _pool_state(lib) == before
    assert rc == 0, lib.last_error()
    out = np.empty((m, n), np.float32)
    assert lib.poly_cuda_copy_dtoh(out.ctypes.data, dc, out.nbytes) == 0
    for d in (da, db, dx, dc):
        lib.poly_cuda_free(d)
    return out


def test_noalloc_matches_float64_and_the_allocating_entry(gpu):
    gpu.poly_b200_set_gemm_policy(1)
    try:
        for call, (m, n, k) in enumerate([(300, 200, 136), (512, 768, 256), (130, 70, 100)]):
            rng = np.random.default_rng(100 + call)
            a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
            b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
            bias = rng.uniform(-1, 1, n).astype(np.float32)
            relu = call & 1
            want = _bf16_round(a).astype(np.float64) @ _bf16_round(b).astype(np.float64) + bias
            if relu:
                want = np.maximum(want, 0)
            got = _run(gpu, 'poly_b200_gemm_noalloc', a, b, bias, relu)
            sibling = _run(gpu, 'poly_b200_gemm', a, b, bias, relu)
            assert np.abs(want).max() > 0
            assert_close(got, want.astype(np.float32), 1e-4, f'call {call} vs float64')
            assert_close(got, sibling, 1e-4, f'call {call} vs poly_b200_gemm')
    finally:
        gpu.poly_b200_set_gemm_policy(0)


def test_noalloc_rejects_sizes_beyond_the_array(gpu):
    # (M + N) * K * 2 bytes = 3 * 8192 * 2048 * 2 > 32 MiB; the pointers are never touched
    d = gpu.poly_cuda_alloc(64)
    rc = gpu.poly_b200_gemm_noalloc(16384, 8192, 2048, d, 2048, 1, d, 8192, 1, d, 8192, None, 0)
    gpu.poly_cuda_free(d)
    assert rc == -1
    assert 'scratch' in gpu.last_error()
