"""Contractions on the B200 against stock polygrad on the CPU.

fp32 kernel: 1e-5 relative (atol = rtol * rms).  Tensor-core kernel (bf16
operands, fp32 accumulation): the CPU path computes the same bf16 products and
sums them in fp32 in k order, so the two differ only in summation order; the
test allows 1e-4 (the stated bound for bf16 GEMM is 2e-2).  Under the bf16
compute policy the comparison is against the CPU result on fp32 operands with
the stated 2e-2 bound, and against the bf16-operand CPU result with 1e-4."""
import numpy as np
import pytest

from conftest import assert_close
from polygrad_b200 import ffi
from polygrad_b200.tensor import Device

pytestmark = pytest.mark.gpu

SHAPES = [(128, 256, 64), (300, 200, 100), (129, 65, 17), (64, 10, 512), (1, 384, 96), (512, 512, 512),
          (257, 1000, 72)]


@pytest.fixture(scope='module')
def devices(ref_lib, gpu):
    return Device(ref_lib, ffi.DEVICE_CPU), Device(gpu, ffi.DEVICE_CUDA)


@pytest.fixture
def policy(gpu):
    def set_policy(bf16):
        gpu.poly_b200_set_gemm_policy(int(bf16))
    yield set_policy
    gpu.poly_b200_set_gemm_policy(0)


def _ab(shape, seed=0):
    m, n, k = shape
    rng = np.random.default_rng([seed, m, n, k])
    return rng.uniform(-1, 1, (m, k)).astype(np.float32), rng.uniform(-1, 1, (k, n)).astype(np.float32)


@pytest.mark.parametrize('shape', SHAPES, ids=str)
def test_fp32(devices, policy, shape):
    cpu, cuda = devices
    policy(False)
    a, b = _ab(shape)
    want = cpu.tensor(a).dot(cpu.tensor(b)).numpy()
    got = cuda.tensor(a).dot(cuda.tensor(b)).numpy()
    assert_close(got, want, 1e-5, f'fp32 {shape}')


@pytest.mark.parametrize('shape', SHAPES, ids=str)
def test_fp32_transposed_operands(devices, policy, shape):
    """A read through permute (m contiguous) and B through permute (k contiguous, the lm-head form)."""
    cpu, cuda = devices
    policy(False)
    a, b = _ab(shape, 1)
    at, bt = np.ascontiguousarray(a.T), np.ascontiguousarray(b.T)
    want = cpu.tensor(at).permute(1, 0).dot(cpu.tensor(bt).permute(1, 0)).numpy()
    got = cuda.tensor(at).permute(1, 0).dot(cuda.tensor(bt).permute(1, 0)).numpy()
    assert_close(got, want, 1e-5, f'fp32 T {shape}')


@pytest.mark.parametrize('shape', SHAPES, ids=str)
def test_bf16_buffers(devices, shape):
    cpu, cuda = devices
    a, b = _ab(shape, 2)
    f = lambda d: d.tensor(a, 'bfloat16').cast('float32').dot(d.tensor(b, 'bfloat16').cast('float32')).numpy()
    assert_close(f(cuda), f(cpu), 1e-4, f'bf16 {shape}')


@pytest.mark.parametrize('shape', SHAPES, ids=str)
def test_fp16_buffers(devices, gpu, shape):
    """float16 operands, fp32 accumulation.  Stock polygrad cannot run this graph on the CPU here
    (its C renderer's __fp16 does not compile with gcc on x86), so the reference is numpy on the
    same float16-rounded operands, accumulated in float64."""
    _, cuda = devices
    a, b = _ab(shape, 6)
    a16, b16 = a.astype(np.float16), b.astype(np.float16)
    want = (a16.astype(np.float64) @ b16.astype(np.float64)).astype(np.float32)
    gpu.poly_b200_stats_reset()
    got = cuda.tensor(a16).cast('float32').dot(cuda.tensor(b16).cast('float32')).numpy()
    assert_close(got, want, 1e-4, f'fp16 {shape}')
    if shape[2] >= 16 and shape[0] * shape[1] >= 64:
        assert gpu.stats()['launches_precompiled'] >= 1      # the tensor-core kernel, not the general renderer


@pytest.mark.parametrize('shape', SHAPES, ids=str)
def test_bf16_policy(devices, policy, shape):
    cpu, cuda = devices
    a, b = _ab(shape, 3)
    want32 = cpu.tensor(a).dot(cpu.tensor(b)).numpy()
    want16 = cpu.tensor(a, 'bfloat16').cast('float32').dot(cpu.tensor(b, 'bfloat16').cast('float32')).numpy()
    policy(True)
    got = cuda.tensor(a).dot(cuda.tensor(b)).numpy()
    assert_close(got, want16, 1e-4, f'policy vs bf16 operands {shape}')
    assert_close(got, want32, 2e-2, f'policy vs fp32 {shape}')


@pytest.mark.parametrize('width', [64, 128, 192, 256])
@pytest.mark.parametrize('shape', [(300, 500, 100), (257, 1000, 72), (512, 768, 256)], ids=str)
def test_every_tile_width(devices, policy, monkeypatch, width, shape):
    """The tensor-core kernel picks its tile width per problem; here each width is forced in turn
    (ragged last tiles in m, n and k included)."""
    cpu, cuda = devices
    a, b = _ab(shape, 4)
    want16 = cpu.tensor(a, 'bfloat16').cast('float32').dot(cpu.tensor(b, 'bfloat16').cast('float32')).numpy()
    monkeypatch.setenv('POLY_B200_TC_BN', str(width))
    policy(True)
    got = cuda.tensor(a).dot(cuda.tensor(b)).numpy()
    assert_close(got, want16, 1e-4, f'width {width} {shape}')


@pytest.mark.parametrize('epilogue', ['plain', 'bias', 'bias_relu'])
@pytest.mark.parametrize('shape', [(300, 333, 64), (130, 1001, 96), (257, 50257 // 64 + 2, 48), (64, 67, 32)], ids=str)
def test_float32_rows_that_are_not_16_byte_aligned(devices, policy, monkeypatch, shape, epilogue):
    """A float32 result whose row pitch is not a multiple of four floats (the 50257-wide logits): the staged
    tile goes out an element per lane, rows of any alignment, with and without a bias and ReLU, ragged last
    chunk included.  Within the bf16 tolerance of the CPU, and the same bits on a second run."""
    cpu, cuda = devices
    a, b = _ab(shape, 8)
    bias = np.random.default_rng(shape[1]).uniform(-1, 1, (shape[1],)).astype(np.float32)

    def build(d, bf16):
        ta, tb = (d.tensor(a, 'bfloat16').cast('float32'), d.tensor(b, 'bfloat16').cast('float32')) if bf16 else (d.tensor(a), d.tensor(b))
        out = ta.dot(tb)
        if epilogue != 'plain':
            out = out + d.tensor(bias)
        return out.relu() if epilogue == 'bias_relu' else out
    want16 = build(cpu, True).numpy()
    policy(True)
    got = build(cuda, False).numpy()
    again = build(cuda, False).numpy()
    assert_close(got, want16, 1e-4, f'unaligned rows {shape} {epilogue}')
    assert np.array_equal(got.view(np.uint32), again.view(np.uint32))


@pytest.mark.parametrize('shape', [(300, 500, 100), (257, 1000, 72), (512, 768, 256), (129, 65, 17), (1024, 256, 2048)], ids=str)
def test_cta_pairs(devices, policy, monkeypatch, shape):
    """The cta_group::2 form of the kernel (two CTAs per 256 x 256 tile), forced for shapes that would
    not choose it: ragged tiles, a second CTA with a single row or none at all."""
    cpu, cuda = devices
    a, b = _ab(shape, 5)
    want16 = cpu.tensor(a, 'bfloat16').cast('float32').dot(cpu.tensor(b, 'bfloat16').cast('float32')).numpy()
    monkeypatch.setenv('POLY_B200_TC_BN', '256')
    monkeypatch.setenv('POLY_B200_TC_CTAS', '2')
    policy(True)
    got = cuda.tensor(a).dot(cuda.tensor(b)).numpy()
    assert_close(got, want16, 1e-4, f'pairs {shape}')


@pytest.mark.parametrize('bf16', [False, True], ids=['fp32', 'bf16'])
def test_batched_attention_shapes(devices, policy, bf16):
    """q . k^T and p . v with (batch, head) batch axes read through permuted views."""
    cpu, cuda = devices
    policy(bf16)
    rng = np.random.default_rng(5)
    B, T, H, hd = 2, 48, 3, 16
    q = rng.standard_normal((B, T, H, hd)).astype(np.float32)
    k = rng.standard_normal((B, T, H, hd)).astype(np.float32)

    def scores(d):
        qq = d.tensor(q).permute(0, 2, 1, 3)
        kk = d.tensor(k).permute(0, 2, 1, 3).permute(0, 1, 3, 2)
        s = qq.dot(kk)
        return s.dot(d.tensor(k).permute(0, 2, 1, 3))
    policy(False)
    want = scores(cpu).numpy()
    policy(bf16)
    got = scores(cuda).numpy()
    assert_close(got, want, 2e-2 if bf16 else 1e-5, 'attention contractions')


def test_weights_cache_follows_updates(gpu, policy):
    """A bf16 copy of an operand is reused while its buffer is unchanged and
    rebuilt after the buffer is rewritten (an instance's weights)."""
    from polygrad_b200.instance import Instance
    policy(True)
    x = np.random.default_rng(0).standard_normal((8, 32)).astype(np.float32)
    inst = Instance.mlp(gpu, [32, 64, 16], 'relu', True, 8, seed=1)
    inst.set_device(ffi.DEVICE_CUDA)
    inst.forward(x=x)
    y0 = inst.read('output').copy()
    inst.forward(x=x)
    assert np.array_equal(inst.read('output'), y0)
    name = inst.params[0]
    inst.write(name, np.zeros(inst.shape(name), np.float32))
    inst.forward(x=x)
    y1 = inst.read('output')
    assert not np.array_equal(y1, y0)
    inst.free()


@pytest.mark.parametrize('bf16_policy', [False, True], ids=['fp32_policy', 'bf16_policy'])
@pytest.mark.parametrize('shape', [(128, 256, 64), (300, 200, 100), (257, 1000, 72)], ids=str)
def test_scaled_sum_behind_an_addend(devices, policy, gpu, shape, bf16_policy):
    """p - lr * (a @ b): the update of a parameter by a gradient that is itself a
    contraction (reference src/instance.c:1158-1162) schedules as one kernel and
    runs on the fp32 contraction kernel with the scale in its epilogue, under
    either policy (a scaled sum is never rounded to bf16)."""
    cpu, cuda = devices
    policy(bf16_policy)
    a, b = _ab(shape, 9)
    p = np.random.default_rng(5).standard_normal((shape[0], shape[1])).astype(np.float32)
    want = (cpu.tensor(p) - cpu.tensor(a).dot(cpu.tensor(b)) * 0.01).numpy()
    gpu.poly_b200_stats_reset()
    got = (cuda.tensor(p) - cuda.tensor(a).dot(cuda.tensor(b)) * 0.01).numpy()
    assert_close(got, want, 1e-5, f'scaled sum {shape}')
    st = gpu.stats()
    assert st['launches'] == 1 and st['launches_precompiled'] == 1


@pytest.mark.parametrize('shape', SHAPES + [(1024, 1024, 512), (1000, 900, 333), (512, 256, 3072)], ids=str)
def test_fp32_as_three_tf32_products(devices, policy, gpu, monkeypatch, shape):
    """POLY_B200_FP32=tc: float32 contractions on the tensor cores, a = hi + lo in tf32 and
    a.b = hi.hi + hi.lo + lo.hi with fp32 accumulation in TMEM.  That accumulation truncates: against a
    float64 product the error grows linearly with K (about 1e-8 * K of the result's rms; a CPU float32
    sum stays at 2e-7 to 4e-7), which is why this variant is opt-in (the default promotes partial sums,
    next test) and its bound against the CPU is 1e-4 here."""
    cpu, cuda = devices
    policy(False)
    monkeypatch.setenv('POLY_B200_FP32', 'tc')
    a, b = _ab(shape, 4)
    want = cpu.tensor(a).dot(cpu.tensor(b)).numpy()
    gpu.poly_b200_stats_reset()
    got = cuda.tensor(a).dot(cuda.tensor(b)).numpy()
    assert_close(got, want, 1e-4, f'fp32 via tf32x3 {shape}')
    exact = a.astype(np.float64) @ b.astype(np.float64)
    rms = np.sqrt(np.mean(exact ** 2))
    err_tc = np.sqrt(np.mean((got - exact) ** 2)) / rms
    assert err_tc <= 1e-6 + 2e-8 * shape[2], err_tc
    if shape[2] >= 16:
        assert gpu.stats()['launches_precompiled'] >= 3          # two splits and the contraction, not the CUDA-core kernel


@pytest.mark.parametrize('shape', SHAPES + [(1024, 1024, 512), (1000, 900, 333), (512, 256, 3072), (256, 512, 8192)], ids=str)
def test_fp32_tf32_products_with_promoted_partial_sums(devices, policy, gpu, monkeypatch, shape):
    """POLY_B200_FP32=tcp (the default for large problems): the three-product scheme with the partial sum of
    every eight k-blocks (32 instructions) moved from tensor memory to registers and added there with rounded float32 adds.
    The error against a float64 product no longer grows with K: the float32 bound of 1e-5 against the
    CPU holds at every K, and the error stays within a small multiple of the CPU's own rounding."""
    cpu, cuda = devices
    policy(False)
    monkeypatch.setenv('POLY_B200_FP32', 'tcp')
    a, b = _ab(shape, 4)
    want = cpu.tensor(a).dot(cpu.tensor(b)).numpy()
    gpu.poly_b200_stats_reset()
    got = cuda.tensor(a).dot(cuda.tensor(b)).numpy()
    assert_close(got, want, 1e-5, f'fp32 via promoted tf32x3 {shape}')
    exact = a.astype(np.float64) @ b.astype(np.float64)
    rms = np.sqrt(np.mean(exact ** 2))
    err_tc = np.sqrt(np.mean((got - exact) ** 2)) / rms
    err_cpu = np.sqrt(np.mean((want - exact) ** 2)) / rms
    assert err_tc <= max(4 * err_cpu, 1.5e-6), (err_tc, err_cpu)
    if shape[2] >= 16:
        assert gpu.stats()['launches_precompiled'] >= 3


@pytest.mark.parametrize('route', ['tcp', 'tc'])
def test_fp32_tensor_core_route_batched_views(devices, policy, monkeypatch, route):
    """The attention contractions with (batch, head) batch axes on the float32 tensor-core routes: q and k
    are permuted views of [B, T, H, hd] storage (split where they lie, two batch strides each), the
    scores feed the second contraction as a dense batched operand."""
    cpu, cuda = devices
    policy(False)
    rng = np.random.default_rng(9)
    B, T, H, hd = 2, 160, 3, 32
    q = rng.standard_normal((B, T, H, hd)).astype(np.float32)
    k = rng.standard_normal((B, T, H, hd)).astype(np.float32)

    def chain(d):
        qq = d.tensor(q).permute(0, 2, 1, 3)
        kk = d.tensor(k).permute(0, 2, 1, 3).permute(0, 1, 3, 2)
        return qq.dot(kk).dot(d.tensor(k).permute(0, 2, 1, 3))
    monkeypatch.setenv('POLY_B200_FP32', 'simt')
    want = chain(cpu).numpy()
    monkeypatch.setenv('POLY_B200_FP32', route)
    got = chain(cuda).numpy()
    assert_close(got, want, 1e-5 if route == 'tcp' else 1e-4, f'batched attention contractions, {route}')


@pytest.mark.parametrize('tokens,d_in,d_out', [(512, 192, 320), (1000, 77, 130)], ids=str)
def test_fp32_tensor_core_route_transposed_operands(devices, policy, gpu, monkeypatch, tokens, d_in, d_out):
    """The weight-gradient form x^T . dy on the promoted tensor-core route: both operands are stored with
    their row axis contiguous and the contraction axis (the tokens) strided, so both are transposed and
    split into their tf32 parts in one pass (POLY_B200_SPLIT_TR=0: gathered into a dense copy first, then
    split; same bits)."""
    cpu, cuda = devices
    policy(False)
    rng = np.random.default_rng([tokens, d_in])
    x = rng.standard_normal((tokens, d_in)).astype(np.float32)
    dy = rng.standard_normal((tokens, d_out)).astype(np.float32)
    monkeypatch.setenv('POLY_B200_FP32', 'simt')
    want = cpu.tensor(x).permute(1, 0).dot(cpu.tensor(dy)).numpy()
    monkeypatch.setenv('POLY_B200_FP32', 'tcp')
    gpu.poly_b200_stats_reset()
    got = cuda.tensor(x).permute(1, 0).dot(cuda.tensor(dy)).numpy()
    assert gpu.stats()['launches_precompiled'] == 3             # two transposing splits and the contraction
    assert_close(got, want, 1e-5, 'x^T . dy, promoted tf32x3')
    monkeypatch.setenv('POLY_B200_SPLIT_TR', '0')
    two_pass = cuda.tensor(x).permute(1, 0).dot(cuda.tensor(dy)).numpy()
    assert np.array_equal(got.view(np.uint32), two_pass.view(np.uint32))


FUSED_FORMS = {
    # an operand that is computed on the fly: the scheduler folds the sum into the reduction
    'sum_of_two_as_operand': lambda t: (t['a'] + t['a2']).dot(t['b']),
    # an activation in front of the contraction
    'relu_operand_and_bias': lambda t: t['a'].relu().dot(t['b']) + t['bias'],
    # two contractions added in one kernel
    'sum_of_two_contractions': lambda t: t['a'].dot(t['b']) + t['a2'].dot(t['b2']),
    # a scaled contraction behind an elementwise expression of two buffers
    'update_by_two_products': lambda t: t['x'] - (t['a'].dot(t['b']) + t['a2'].dot(t['b2'])) * 0.05,
}


@pytest.mark.parametrize('form', sorted(FUSED_FORMS))
def test_kernels_with_fused_operands_or_several_contractions(devices, policy, gpu, form):
    """Graphs whose contraction the scheduler fuses with a computed operand, or several contractions it
    puts into one kernel: by default (the contractions hold 2^24 multiply-adds here) such a kernel is cut
    into operand temporaries, one contraction each and an elementwise remainder, all on precompiled or
    vectorised kernels; with POLY_B200_OUTLINE=0 it runs whole as generated code.  Both within 1e-5 of
    the CPU."""
    cpu, cuda = devices
    policy(False)
    m, n, k = 256, 384, 192
    rng = np.random.default_rng([m, n, k, 11])
    arrays = dict(a=rng.uniform(-1, 1, (m, k)), a2=rng.uniform(-1, 1, (m, k)), b=rng.uniform(-1, 1, (k, n)),
                  b2=rng.uniform(-1, 1, (k, n)), bias=rng.uniform(-1, 1, (n,)), x=rng.uniform(-1, 1, (m, n)))
    arrays = {name: v.astype(np.float32) for name, v in arrays.items()}
    build = FUSED_FORMS[form]
    want = build({name: cpu.tensor(v) for name, v in arrays.items()}).numpy()
    gpu.poly_b200_stats_reset()
    got = build({name: cuda.tensor(v) for name, v in arrays.items()}).numpy()
    st = gpu.stats()
    assert_close(got, want, 1e-5, form)
    assert st['launches_precompiled'] >= 1, 'no contraction kernel ran'


def test_fp32_default_routes(devices, policy, gpu, monkeypatch):
    """Large float32 contractions take the tensor-core route with promoted partial sums by default,
    small ones the CUDA-core kernel; both within 1e-5 of the CPU."""
    cpu, cuda = devices
    policy(False)
    a, b = _ab((1024, 1024, 1024), 8)
    want = cpu.tensor(a).dot(cpu.tensor(b)).numpy()
    monkeypatch.delenv('POLY_B200_FP32', raising=False)
    got = cuda.tensor(a).dot(cuda.tensor(b)).numpy()
    monkeypatch.setenv('POLY_B200_FP32', 'tcp')
    tcp = cuda.tensor(a).dot(cuda.tensor(b)).numpy()
    monkeypatch.setenv('POLY_B200_FP32', 'simt')
    simt = cuda.tensor(a).dot(cuda.tensor(b)).numpy()
    assert_close(got, want, 1e-5, 'fp32 default route')
    assert_close(simt, want, 1e-5, 'fp32 CUDA-core route')
    assert np.array_equal(got, tcp) and not np.array_equal(got, simt)
    a, b = _ab((128, 256, 64), 8)                      # below the size threshold
    monkeypatch.delenv('POLY_B200_FP32', raising=False)
    small = cuda.tensor(a).dot(cuda.tensor(b)).numpy()
    monkeypatch.setenv('POLY_B200_FP32', 'simt')
    assert np.array_equal(small, cuda.tensor(a).dot(cuda.tensor(b)).numpy())


def test_fp32_tensor_core_route_keeps_infinities(devices, policy, monkeypatch):
    """hi carries an infinity, lo is forced to zero: the result is +-inf or NaN exactly where the CPU's is."""
    cpu, cuda = devices
    policy(False)
    monkeypatch.setenv('POLY_B200_FP32', 'tc')
    a, b = _ab((128, 64, 32), 2)
    a[3, 5] = np.inf
    a[7, 1] = -np.inf
    want = cpu.tensor(a).dot(cpu.tensor(b)).numpy()
    got = cuda.tensor(a).dot(cuda.tensor(b)).numpy()
    assert np.array_equal(np.isinf(got), np.isinf(want)) and np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(np.sign(got[np.isinf(want)]), np.sign(want[np.isinf(want)]))
    fin = np.isfinite(want)
    assert_close(got[fin], want[fin], 1e-4, 'finite rows')


def _bf16_round(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


@pytest.mark.parametrize('m,n,k', [(256, 512, 128), (300, 3072, 768), (129, 68, 40)])
@pytest.mark.parametrize('flags', [1, 3], ids=['bf16_result', 'gelu_bf16_result'])
def test_gemm_ex_result_formats(gpu, m, n, k, flags):
    """poly_b200_gemm_ex: the contraction's result (+ bias) stored as bfloat16, optionally through
    tanh-GELU first, against numpy in float64 on the same bfloat16-rounded operands.  Bound: the
    bfloat16 rounding of the result (2^-9 relative) plus the tanh approximation (2^-11): 4e-3."""
    from polygrad_b200.tensor import f32_to_bf16_bits
    rng = np.random.default_rng([m, n, k, flags])
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = (rng.uniform(-1, 1, (k, n)) * (2.0 / np.sqrt(k))).astype(np.float32)
    bias = rng.uniform(-0.5, 0.5, n).astype(np.float32)
    a16, b16 = f32_to_bf16_bits(a), f32_to_bf16_bits(b)
    want = _bf16_round(a).astype(np.float64) @ _bf16_round(b).astype(np.float64) + bias
    if flags & 2:
        want = 0.5 * want * (1 + np.tanh(0.7978845608028654 * (want + 0.044715 * want ** 3)))
    bufs = []
    for arr in (a16, b16, bias):
        d = gpu.poly_cuda_alloc(arr.nbytes)
        assert d and gpu.poly_cuda_copy_htod(d, arr.ctypes.data, arr.nbytes) == 0
        bufs.append(d)
    dc = gpu.poly_cuda_alloc(m * n * 2)
    rc = gpu.poly_b200_gemm_ex(m, n, k, bufs[0], k, 1, bufs[1], n, 1, dc, n, bufs[2], 1, flags)
    assert rc == 0, gpu.last_error()
    got16 = np.empty((m, n), np.uint16)
    assert gpu.poly_cuda_copy_dtoh(got16.ctypes.data, dc, got16.nbytes) == 0
    for d in bufs + [dc]:
        gpu.poly_cuda_free(d)
    got = (got16.astype(np.uint32) << 16).view(np.float32)
    assert np.abs(got).max() > 0
    assert_close(got, want.astype(np.float32), 4e-3, f'gemm_ex flags={flags} {m}x{n}x{k}')
