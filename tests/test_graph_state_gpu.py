"""What a CUDA-graph replay must keep true about device buffers, and the direct
entry points' bookkeeping.

* A replayed training plan updates weights in place; a forward plan of the same
  instance holds bfloat16 copies of those weights and must notice (polygrad's
  PolyInstance shares its buffers between entrypoints, src/instance.c:783-830,
  1242-1330).
* Scratch a captured plan addresses belongs to that plan until its graph is
  destroyed (polygrad keeps a plan's intermediates for the life of the plan,
  src/exec_plan.c:860-881): no later allocation may receive it.
* poly_b200_gemm on a buffer that poly_cuda_memset zeroed lazily.

Tolerances: bf16 policy vs the fp32 CPU run 2e-2; fp32 1e-5; bit equality where
stated."""
import ctypes

import numpy as np
import pytest

from conftest import assert_close
from polygrad_b200 import ffi
from polygrad_b200.instance import Instance, gpt2_init

pytestmark = pytest.mark.gpu


def _fwd_train_fwd(lib, device, cfg, tokens, lr, n_train):
    inst = Instance.gpt2(lib, **cfg)
    inst.init_params(gpt2_init(7))
    if device != ffi.DEVICE_CPU:
        inst.set_device(device)
    inst.set_optimizer(ffi.OPTIM_SGD, lr)
    io = inst.gpt2_inputs(tokens)
    for _ in range(3):                       # the forward plan reaches its graph
        inst.forward(**io)
    before = inst.read('output').copy()
    losses = [inst.train_step(**io) for _ in range(n_train)]   # replays as a graph from the third step
    inst.forward(**io)
    after = inst.read('output').copy()
    inst.free()
    return before, after, losses


def test_forward_sees_weights_updated_by_a_replayed_training_graph(ref_lib, gpu):
    cfg = dict(vocab_size=64, n_embd=48, n_head=4, n_layer=2, max_seq_len=16, max_batch=2)
    tokens = np.random.default_rng(17).integers(0, cfg['vocab_size'], (cfg['max_batch'], cfg['max_seq_len']))
    want_before, want_after, want_l = _fwd_train_fwd(ref_lib, ffi.DEVICE_CPU, cfg, tokens, 1e-5, 6)
    gpu.poly_b200_set_gemm_policy(1)
    try:
        got_before, got_after, got_l = _fwd_train_fwd(gpu, ffi.DEVICE_CUDA, cfg, tokens, 1e-5, 6)
    finally:
        gpu.poly_b200_set_gemm_policy(0)
    # the training must move the logits by far more than the tolerance, or the test shows nothing
    moved = np.sqrt(np.mean((want_after - want_before) ** 2)) / np.sqrt(np.mean(want_before ** 2))
    assert moved > 0.1, moved
    np.testing.assert_allclose(got_l, want_l, rtol=2e-2)
    assert_close(got_before, want_before, 2e-2, 'logits before training')
    assert_close(got_after, want_after, 2e-2, 'logits after six training steps')


def _free_sizes(lib):
    n = lib.poly_b200_pool_free_sizes(None, 0)
    buf = (ctypes.c_ulonglong * max(n, 1))()
    lib.poly_b200_pool_free_sizes(buf, n)
    return [int(buf[i]) for i in range(n)]


def _forward_n(lib, cfg, tokens, n, seed, between=None):
    inst = Instance.gpt2(lib, **cfg)
    inst.init_params(gpt2_init(seed))
    inst.set_device(ffi.DEVICE_CUDA)
    io = inst.gpt2_inputs(tokens)
    outs = []
    for i in range(n):
        inst.forward(**io)
        outs.append(inst.read('output').copy())
        if between is not None:
            between(i)
    return inst, outs


def test_scratch_of_a_captured_plan_is_not_handed_out_again(gpu, monkeypatch):
    """fp32 contractions forced onto the three-tf32 route: every call splits its A operand into pool
    scratch, so the captured forward addresses scratch blocks.  Between replays every block the pool
    could hand out is taken and filled with a pattern, for two instances of different models in
    turn; the patterns must survive the replays and the logits must be those of the run without
    graphs, bit for bit."""
    monkeypatch.setenv('POLY_B200_FP32', 'tcp')
    cfgs = [dict(vocab_size=160, n_embd=64, n_head=2, n_layer=2, max_seq_len=32, max_batch=2),
            dict(vocab_size=96, n_embd=128, n_head=4, n_layer=1, max_seq_len=64, max_batch=1)]
    toks = [np.random.default_rng(5 + i).integers(0, c['vocab_size'], (c['max_batch'], c['max_seq_len']))
            for i, c in enumerate(cfgs)]
    monkeypatch.setenv('POLY_B200_GRAPH', '0')
    plain = []
    for c, t in zip(cfgs, toks):
        inst, outs = _forward_n(gpu, c, t, 1, 9)
        plain.append(outs[0])
        inst.free()
    monkeypatch.delenv('POLY_B200_GRAPH')

    taken = []          # (device pointer, pattern)

    def grab_all_free_blocks(i):
        if i < 2:            # the third forward captures the graph; leave the pool alone until then
            return
        for k, size in enumerate(_free_sizes(gpu)):
            d = gpu.poly_cuda_alloc(size)
            assert d
            pat = np.full(size // 4, np.float32(1000 + len(taken) + k), np.float32)
            assert gpu.poly_cuda_copy_htod(d, pat.ctypes.data, pat.nbytes) == 0
            taken.append((d, pat))

    insts = []
    for c, t, want in zip(cfgs, toks, plain):
        inst, outs = _forward_n(gpu, c, t, 6, 9, between=grab_all_free_blocks)   # graph from the third forward
        insts.append(inst)
        for i, got in enumerate(outs):
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f'forward {i} differs from the run without graphs'
    # replay the first instance again now that the second one has allocated and captured
    io = insts[0].gpt2_inputs(toks[0])
    for _ in range(2):
        insts[0].forward(**io)
        assert np.array_equal(insts[0].read('output').view(np.uint32), plain[0].view(np.uint32))
    assert len(taken) > 0
    for d, pat in taken:
        back = np.empty_like(pat)
        assert gpu.poly_cuda_copy_dtoh(back.ctypes.data, d, back.nbytes) == 0
        assert np.array_equal(back, pat), 'a replay wrote into a buffer allocated after the capture'
        gpu.poly_cuda_free(d)
    for inst in insts:
        inst.free()


def _dev(lib, a):
    d = lib.poly_cuda_alloc(a.nbytes)
    assert d and lib.poly_cuda_copy_htod(d, a.ctypes.data, a.nbytes) == 0
    return d


def _bf16_round(a):
    """float32 -> nearest-even bfloat16 -> float32 (finite inputs)."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


@pytest.mark.parametrize('m,n,k,relu', [(300, 200, 136, 0), (512, 768, 256, 1), (130, 50257 // 64, 100, 0)])
def test_direct_gemm_bf16_policy_against_float64(gpu, m, n, k, relu):
    """poly_b200_gemm under the bf16 policy against numpy on the same bfloat16-rounded operands
    accumulated in float64 (1e-4: only the summation order and fp32 rounding differ)."""
    rng = np.random.default_rng([m, n, k])
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    bias = rng.uniform(-1, 1, n).astype(np.float32)
    want = _bf16_round(a).astype(np.float64) @ _bf16_round(b).astype(np.float64) + bias
    if relu:
        want = np.maximum(want, 0)
    da, db, dx = _dev(gpu, a), _dev(gpu, b), _dev(gpu, bias)
    dc = gpu.poly_cuda_alloc(m * n * 4)
    gpu.poly_b200_set_gemm_policy(1)
    try:
        # C zeroed lazily first: the fill must not fire after the contraction has written C
        assert gpu.poly_cuda_memset(dc, 0, m * n * 4) == 0
        assert gpu.poly_b200_gemm(m, n, k, da, k, 1, db, n, 1, dc, n, dx, relu, 0) == 0, gpu.last_error()
    finally:
        gpu.poly_b200_set_gemm_policy(0)
    got = np.empty((m, n), np.float32)
    assert gpu.poly_cuda_copy_dtoh(got.ctypes.data, dc, got.nbytes) == 0
    for d in (da, db, dx, dc):
        gpu.poly_cuda_free(d)
    assert np.abs(got).max() > 0
    assert_close(got, want.astype(np.float32), 1e-4, f'gemm {m}x{n}x{k}')


def test_direct_gemm_strided_views_and_unaligned_rows(gpu):
    """A read through a transposed view (a_sm = 1), B k-contiguous (the lm-head form), and a C whose
    row pitch is not a multiple of 16 bytes (a 50257-wide vocabulary has such rows): float32 policy
    against the float64 product (1e-5), bf16 policy against the rounded operands (1e-4)."""
    m, n, k, c_sm = 200, 333, 96, 335
    rng = np.random.default_rng(3)
    at = rng.uniform(-1, 1, (k, m)).astype(np.float32)        # A[m, k] = at[k, m]
    bt = rng.uniform(-1, 1, (n, k)).astype(np.float32)        # B[k, n] = bt[n, k]
    da, db = _dev(gpu, at), _dev(gpu, bt)
    for policy, rtol in ((0, 1e-5), (1, 1e-4)):
        dc = _dev(gpu, np.full((m, c_sm), -7.0, np.float32))
        gpu.poly_b200_set_gemm_policy(policy)
        try:
            assert gpu.poly_b200_gemm(m, n, k, da, 1, m, db, 1, k, dc, c_sm, None, 0, 0) == 0, gpu.last_error()
        finally:
            gpu.poly_b200_set_gemm_policy(0)
        got = np.empty((m, c_sm), np.float32)
        assert gpu.poly_cuda_copy_dtoh(got.ctypes.data, dc, got.nbytes) == 0
        gpu.poly_cuda_free(dc)
        a, b = (at.T, bt.T) if policy == 0 else (_bf16_round(at).T, _bf16_round(bt).T)
        want = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
        assert_close(got[:, :n], want, rtol, f'policy {policy}')
        assert np.all(got[:, n:] == -7.0), 'columns beyond N were written'
    gpu.poly_cuda_free(da)
    gpu.poly_cuda_free(db)
