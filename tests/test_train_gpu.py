"""Training steps on the B200 against stock polygrad on the CPU.

poly_instance_train_step (src/instance.c:1242) runs forward, backward and the
optimizer update as one plan whose parameters are updated in place; the loss
scalar, the optimizer moments and the bias corrections are bound as host
pointers even when the instance lives on the device (src/instance.c:1298-1311),
and poly_instance_value_and_grad binds the loss and every gradient that way
(src/instance.c:1028-1043).  The plan executor runs such buffers from device
copies, so the same calls work after poly_instance_set_device(CUDA).

polygrad's MLP builder supports a loss only at batch size 1 (the target buffer
is not reshaped, src/model_mlp.c:258-274), which is also how its own training
tests run (test/test_mlp.c:248-370): the cases here use batch size 1 at the
widths of the benchmark MLP.

Tolerance: 1e-5 relative per step for the loss and 1e-5 (SGD) / 1e-4 (Adam,
AdamW: a division by sqrt(v)+eps follows the gradients) for the parameters
after five steps, atol = rtol * rms.
"""
import os

import numpy as np
import pytest

from conftest import assert_close
from polygrad_b200 import ffi
from polygrad_b200.instance import Instance, gpt2_init

pytestmark = pytest.mark.gpu

LAYERS = [784, 512, 10]
STEPS = 5


def _data(loss):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((1, LAYERS[0])).astype(np.float32)
    if loss == 'cross_entropy':
        y = np.zeros((1, LAYERS[-1]), dtype=np.float32)
        y[0, 3] = 1.0
    else:
        y = rng.standard_normal((1, LAYERS[-1])).astype(np.float32)
    return x, y


def _train(lib, device, loss, optim, lr):
    inst = Instance.mlp(lib, LAYERS, 'relu', True, 1, seed=42, loss=loss)
    x, y = _data(loss)
    if device != ffi.DEVICE_CPU:
        inst.set_device(device)          # before the first step: the moments are created afterwards
    inst.set_optimizer(optim, lr, weight_decay=0.01 if optim == ffi.OPTIM_ADAMW else 0.0)
    losses = [inst.train_step(x=x, y=y) for _ in range(STEPS)]
    params = {n: inst.read(n).copy() for n in inst.params}
    inst.free()
    return np.array(losses), params


@pytest.mark.parametrize('loss', ['mse', 'cross_entropy'])
@pytest.mark.parametrize('optim,lr,ptol', [(ffi.OPTIM_SGD, 0.001, 1e-5), (ffi.OPTIM_ADAM, 0.0001, 1e-4),
                                           (ffi.OPTIM_ADAMW, 0.0001, 1e-4)])
def test_mlp_train_steps_match_cpu(ref_lib, gpu, loss, optim, lr, ptol):
    want_l, want_p = _train(ref_lib, ffi.DEVICE_CPU, loss, optim, lr)
    got_l, got_p = _train(gpu, ffi.DEVICE_CUDA, loss, optim, lr)
    assert want_l[-1] < want_l[0], 'the reference run itself must learn'
    np.testing.assert_allclose(got_l, want_l, rtol=1e-5 * STEPS, atol=1e-7)
    for name in want_p:
        assert_close(got_p[name], want_p[name], ptol, f'{name} after {STEPS} steps')


def test_parameters_change_on_the_device(gpu):
    """The update happens in the device-resident parameters (nothing is trained
    on the host and copied over): read back before and after one step."""
    inst = Instance.mlp(gpu, LAYERS, 'relu', True, 1, seed=42, loss='mse')
    x, y = _data('mse')
    inst.set_device(ffi.DEVICE_CUDA)
    inst.set_optimizer(ffi.OPTIM_SGD, 0.05)
    before = {n: inst.read(n).copy() for n in inst.params}
    gpu.poly_b200_stats_reset()
    inst.train_step(x=x, y=y)
    assert gpu.stats()['launches'] > 0
    after = {n: inst.read(n) for n in inst.params}
    assert any(np.abs(after[n] - before[n]).max() > 0 for n in inst.params)
    inst.free()


@pytest.mark.parametrize('loss', ['mse', 'cross_entropy'])
def test_value_and_grad_loss_matches_cpu(ref_lib, gpu, loss):
    x, y = _data(loss)
    vals = []
    for lib, dev in ((ref_lib, ffi.DEVICE_CPU), (gpu, ffi.DEVICE_CUDA)):
        inst = Instance.mlp(lib, LAYERS, 'relu', True, 1, seed=42, loss=loss)
        if dev != ffi.DEVICE_CPU:
            inst.set_device(dev)
        vals.append([inst.value_and_grad('loss', x=x, y=y) for _ in range(2)])
        inst.free()
    np.testing.assert_allclose(vals[1], vals[0], rtol=1e-5, atol=1e-7)
    assert vals[1][0] == vals[1][1], 'value_and_grad does not update anything'


def _train_gpt2(lib, device, cfg, tokens, optim, lr, steps):
    inst = Instance.gpt2(lib, **cfg)
    inst.init_params(gpt2_init(7))
    if device != ffi.DEVICE_CPU:
        inst.set_device(device)
    inst.set_optimizer(optim, lr)
    losses = [inst.train_step(**inst.gpt2_inputs(tokens)) for _ in range(steps)]
    params = {n: inst.read(n).copy() for n in inst.params}
    inst.free()
    return np.array(losses), params


@pytest.mark.parametrize('optim,lr', [(ffi.OPTIM_SGD, 1e-5), (ffi.OPTIM_ADAMW, 1e-4)], ids=['sgd', 'adamw'])
def test_gpt2_train_steps_match_cpu(ref_lib, gpu, optim, lr):
    """A full GPT-2 training step (polygrad's 'loss' entrypoint: the sum of the
    squared logits, src/modelzoo/models/gpt2.c:527-546) through every layer's
    backward: embedding, LayerNorm, attention, GELU and the tied head.  fp32
    contractions; loss within 1e-4 relative per step, parameters within 1e-4
    (SGD) / 1e-3 (AdamW) after three steps.

    The key third of each c_attn bias is left out under AdamW: softmax does not
    depend on a bias added to every key, so its gradient is rounding noise
    around zero, which Adam's division by sqrt(v) turns into steps of +-lr in
    either implementation; those entries are only checked to stay within
    steps * lr of each other."""
    cfg = dict(vocab_size=64, n_embd=48, n_head=4, n_layer=2, max_seq_len=16, max_batch=2)
    tokens = np.random.default_rng(17).integers(0, cfg['vocab_size'], (cfg['max_batch'], cfg['max_seq_len']))
    want_l, want_p = _train_gpt2(ref_lib, ffi.DEVICE_CPU, cfg, tokens, optim, lr, 3)
    got_l, got_p = _train_gpt2(gpu, ffi.DEVICE_CUDA, cfg, tokens, optim, lr, 3)
    assert want_l[-1] < want_l[0], 'the reference run itself must learn'
    np.testing.assert_allclose(got_l, want_l, rtol=1e-4)
    ptol = 1e-4 if optim == ffi.OPTIM_SGD else 1e-3
    d = cfg['n_embd']
    for name in want_p:
        got, want = got_p[name], want_p[name]
        if optim != ffi.OPTIM_SGD and name.endswith('attn.c_attn.bias'):
            assert np.abs(got[d:2 * d] - want[d:2 * d]).max() <= 2 * 3 * lr * 1.01
            got, want = np.delete(got, np.s_[d:2 * d]), np.delete(want, np.s_[d:2 * d])
        assert_close(got, want, ptol, f'{name} after 3 steps')


@pytest.mark.parametrize('optim,lr,route', [(ffi.OPTIM_SGD, 1e-5, None), (ffi.OPTIM_SGD, 1e-5, 'tcp'), (ffi.OPTIM_ADAMW, 1e-4, None)],
                         ids=['sgd', 'sgd_tensor_cores', 'adamw'])
def test_gpt2_train_steps_with_backward_kernels_cut(ref_lib, gpu, monkeypatch, optim, lr, route):
    """The same three steps with every backward kernel that holds a contraction cut into operand
    temporaries, contraction steps and an elementwise remainder (at this width the cut would not pay
    and is forced): weight gradients whose operand is a sum of gradient contributions, the tied
    embedding's gradient (head contraction + lookup selection + update in one scheduled kernel), the
    q/k/v gradients written side by side, and under AdamW the moment updates that each hold the
    gradient's contraction.  Same tolerances as the uncut run.  `sgd_tensor_cores` also sends every
    float32 contraction the tensor-core kernel accepts through it (three tf32 products, operands split --
    and, where their rows are the contiguous axis, transposed -- on the way; scaled sums included), as
    happens by default from 2^30 multiply-adds."""
    monkeypatch.setenv('POLY_B200_OUTLINE_MIN_WORK', '0')
    if route:
        monkeypatch.setenv('POLY_B200_FP32', route)
    else:
        monkeypatch.delenv('POLY_B200_FP32', raising=False)
    cfg = dict(vocab_size=64, n_embd=48, n_head=4, n_layer=2, max_seq_len=16, max_batch=2)
    tokens = np.random.default_rng(17).integers(0, cfg['vocab_size'], (cfg['max_batch'], cfg['max_seq_len']))
    want_l, want_p = _train_gpt2(ref_lib, ffi.DEVICE_CPU, cfg, tokens, optim, lr, 3)
    cut_before = gpu.poly_b200_kernels_cut()
    got_l, got_p = _train_gpt2(gpu, ffi.DEVICE_CUDA, cfg, tokens, optim, lr, 3)
    assert gpu.poly_b200_kernels_cut() - cut_before >= 2 * cfg['n_layer'] + 1
    np.testing.assert_allclose(got_l, want_l, rtol=1e-4)
    ptol = 1e-4 if optim == ffi.OPTIM_SGD else 1e-3
    d = cfg['n_embd']
    for name in want_p:
        got, want, first = got_p[name], want_p[name], _initial(cfg, name)
        if optim != ffi.OPTIM_SGD and name.endswith('attn.c_attn.bias'):
            # gradients that are rounding noise around zero (see test_gpt2_train_steps_match_cpu)
            assert np.abs(got[d:2 * d] - want[d:2 * d]).max() <= 2 * 3 * lr * 1.01
            got, want, first = (np.delete(a, np.s_[d:2 * d]) for a in (got, want, first))
        assert_close(got, want, ptol, f'{name} after 3 steps, kernels cut')
        moved = want.astype(np.float64) - first
        if optim == ffi.OPTIM_SGD and np.sqrt(np.mean(moved ** 2)) > 1e-6:
            assert_close(got.astype(np.float64) - first, moved, 2e-2, f'update of {name}')


_INITIAL = {}


def _initial(cfg, name):
    key = tuple(sorted(cfg.items()))
    if key not in _INITIAL:
        from polygrad_b200 import ffi as _f
        inst = Instance.gpt2(_f.load_reference(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                                            'oracle', '_ref', 'libpolygrad_ref.so')), **cfg)
        inst.init_params(gpt2_init(7))
        _INITIAL[key] = {n: inst.read(n).astype(np.float64) for n in inst.params}
        inst.free()
    return _INITIAL[key][name]


GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'train.npz')


@pytest.mark.parametrize('loss', ['mse', 'cross_entropy'])
def test_mlp_training_against_committed_fixture(gpu, loss):
    """Five SGD steps from the fixture's initial parameters against what stock polygrad produced
    (tests/golden/train.npz): needs neither polygrad's CPU library nor its sources."""
    g = np.load(GOLDEN)
    names = sorted(k.split(':', 2)[2] for k in g.files if k.startswith(f'mlp_{loss}:init:'))
    inst = Instance.mlp(gpu, [96, 64, 10], 'relu', True, 1, seed=42, loss=loss)
    inst.set_device(ffi.DEVICE_CUDA)
    for n in names:
        inst.write(n, g[f'mlp_{loss}:init:{n}'])
    inst.set_optimizer(ffi.OPTIM_SGD, 0.01)
    losses = [inst.train_step(x=g[f'mlp_{loss}:x'], y=g[f'mlp_{loss}:y']) for _ in range(5)]
    np.testing.assert_allclose(losses, g[f'mlp_{loss}:losses'], rtol=5e-5)
    for n in names:
        assert_close(inst.read(n), g[f'mlp_{loss}:final:{n}'], 1e-5, n)
    inst.free()


def test_gpt2_training_against_committed_fixture(gpu):
    g = np.load(GOLDEN)
    keys = ('vocab_size', 'n_embd', 'n_head', 'n_layer', 'max_seq_len', 'max_batch')
    cfg = {k: int(v) for k, v in zip(keys, g['gpt2:cfg'])}
    losses, params = _train_gpt2(gpu, ffi.DEVICE_CUDA, cfg, g['gpt2:tokens'], ffi.OPTIM_SGD, 1e-5, 3)
    np.testing.assert_allclose(losses, g['gpt2:losses'], rtol=1e-4)
    for n, got in params.items():
        assert_close(got, g[f'gpt2:final:{n}'], 1e-4, n)


def test_gpt2_training_under_bf16_policy(ref_lib, gpu):
    """Five SGD steps with the contractions of the forward and backward pass on the tensor cores
    (operands rounded to bfloat16, fp32 accumulation): every step's loss within 2e-2 of the fp32 CPU
    run.  From the third step on the plan replays as a CUDA graph, and the bfloat16 copies of the
    weights must follow the in-place updates -- a stale copy would leave the loss where it was."""
    cfg = dict(vocab_size=64, n_embd=48, n_head=4, n_layer=2, max_seq_len=16, max_batch=2)
    tokens = np.random.default_rng(17).integers(0, cfg['vocab_size'], (cfg['max_batch'], cfg['max_seq_len']))
    want_l, want_p = _train_gpt2(ref_lib, ffi.DEVICE_CPU, cfg, tokens, ffi.OPTIM_SGD, 1e-5, 5)
    gpu.poly_b200_set_gemm_policy(1)
    try:
        gpu.poly_b200_stats_reset()
        got_l, got_p = _train_gpt2(gpu, ffi.DEVICE_CUDA, cfg, tokens, ffi.OPTIM_SGD, 1e-5, 5)
        assert gpu.stats()['launches_precompiled'] > 0
    finally:
        gpu.poly_b200_set_gemm_policy(0)
    assert want_l[-1] < 0.9 * want_l[0]
    np.testing.assert_allclose(got_l, want_l, rtol=2e-2)
    for name in want_p:
        assert_close(got_p[name], want_p[name], 2e-2, f'{name} after 5 steps, bf16 policy')
