"""The CPU restatement (oracle/polyref.py + polyref_port.c) pinned against
(a) fixtures produced by stock polygrad (tests/golden/*.npz),
(b) polygrad's own known-answer fixture test/fixtures/mlp_cross.json
    (MLP [2,4,1], every parameter (j % 7 - 3) * 0.1, input [1, 2] -> -0.34),
(c) stock polygrad itself where oracle/_ref is built."""
import os

import numpy as np
import pytest

from conftest import ROOT, assert_close
from oracle import polyref
from polygrad_b200.instance import gpt2_init

G = os.path.join(ROOT, 'tests', 'golden')


@pytest.fixture(scope='module')
def rowops():
    return np.load(os.path.join(G, 'rowops.npz'))


@pytest.mark.parametrize('name,fn', [
    ('affine', lambda x: x * np.float32(2) + np.float32(1)),
    ('exp', polyref.exp), ('tanh', polyref.tanh), ('gelu', polyref.gelu),
    ('sum', polyref.row_sum), ('max', polyref.row_max), ('mean', polyref.row_mean),
    ('var', polyref.row_var), ('softmax', polyref.softmax), ('layernorm', polyref.layernorm),
])
def test_rowops_against_polygrad_fixture(rowops, name, fn):
    # exp2/sigmoid go through libm here and through polynomials in polygrad: a few ulp
    assert_close(fn(rowops['x']), rowops[name], 2e-6, name)


@pytest.mark.parametrize('name,fn', [
    ('permute', lambda x: x.T), ('flip0', lambda x: x[::-1]), ('flip1', lambda x: x[:, ::-1]),
    ('step3', lambda x: x[:, ::3]),
])
def test_movement_against_polygrad_fixture(rowops, name, fn):
    assert np.array_equal(fn(rowops['x']), rowops[name])


def test_reductions_bit_exact(rowops):
    """Same accumulation order as polygrad's CPU kernels, so sums agree bitwise."""
    for name, fn in (('sum', polyref.row_sum), ('max', polyref.row_max), ('mean', polyref.row_mean)):
        assert np.array_equal(fn(rowops['x']).view(np.uint32), rowops[name].view(np.uint32)), name


def test_matmul_bit_exact():
    m = np.load(os.path.join(G, 'matmul.npz'))
    assert np.array_equal(polyref.matmul(m['a'], m['b']).view(np.uint32), m['f32'].view(np.uint32))
    assert np.array_equal(polyref.matmul(m['a'], m['b'], bf16=True).view(np.uint32), m['bf16'].view(np.uint32))


def test_mlp_fixture():
    m = np.load(os.path.join(G, 'mlp.npz'))
    ws = [m['param:layers.0.weight'], m['param:layers.1.weight']] if 'param:layers.0.weight' in m.files else None
    if ws is None:
        names = sorted(k for k in m.files if k.startswith('param:'))
        ws = [m[k] for k in names if k.endswith('weight')]
        bs = [m[k] for k in names if k.endswith('bias')]
    else:
        bs = [m['param:layers.0.bias'], m['param:layers.1.bias']]
    out = polyref.mlp_forward(m['x'], ws, bs)
    assert_close(out, m['output'].reshape(out.shape), 1e-6, 'mlp')


def test_mlp_known_answer():
    """polygrad test/fixtures/mlp_cross.json: output -0.3400000035762787."""
    w1 = np.array([(j % 7 - 3) * 0.1 for j in range(8)], np.float32).reshape(4, 2)
    b1 = np.array([(j % 7 - 3) * 0.1 for j in range(4)], np.float32)
    w2 = np.array([(j % 7 - 3) * 0.1 for j in range(4)], np.float32).reshape(1, 4)
    b2 = np.array([(0 % 7 - 3) * 0.1], np.float32)
    out = polyref.mlp_forward(np.array([[1.0, 2.0]], np.float32), [w1, w2], [b1, b2])
    assert abs(float(out[0, 0]) - (-0.3400000035762787)) < 1e-7


def test_gpt2_fixture():
    g = np.load(os.path.join(G, 'gpt2_toy.npz'))
    keys = ('vocab_size', 'n_embd', 'n_head', 'n_layer', 'max_seq_len', 'max_batch')
    cfg = dict(zip(keys, (int(v) for v in g['cfg'])))
    out = polyref.gpt2_forward(cfg, gpt2_init(int(g['seed'])), g['tokens'])
    assert_close(out, g['logits'], 2e-5, 'gpt2 logits')


def test_embedding_semantics():
    """Ids that match no arange entry give a +0 row; -0.0 table entries come out as +0.0."""
    table = np.array([[1.0, -0.0], [2.0, 3.0], [4.0, 5.0]], np.float32)
    ids = np.array([1.0, 7.0, 0.5, np.nan, 0.0], np.float32)
    out = polyref.embedding(ids, np.arange(3, dtype=np.float32), table)
    assert np.array_equal(out[0], table[1]) and not out[1].any() and not out[2].any() and not out[3].any()
    assert out[4, 0] == 1.0 and np.signbit(out[4, 1]) == False  # noqa: E712


def test_against_stock_polygrad(ref_lib):
    """Where stock polygrad is built here, run it live on a fresh seed."""
    from polygrad_b200 import ffi
    from polygrad_b200.tensor import Device
    cpu = Device(ref_lib, ffi.DEVICE_CPU)
    x = np.random.default_rng(99).standard_normal((9, 70)).astype(np.float32)
    t = cpu.tensor(x)
    assert_close(polyref.softmax(x), t.softmax(-1).numpy(), 2e-6, 'softmax')
    assert_close(polyref.layernorm(x), t.layernorm(-1, 1e-5).numpy(), 2e-6, 'layernorm')
    w = np.random.default_rng(98).uniform(-1, 1, (70, 13)).astype(np.float32)
    assert np.array_equal(polyref.matmul(x, w), t.dot(cpu.tensor(w)).numpy())


# ── training steps ──────────────────────────────────────────────────────────
def _mlp_case(g, loss):
    names = sorted(k.split(':', 2)[2] for k in g.files if k.startswith(f'mlp_{loss}:init:'))
    init = {n: g[f'mlp_{loss}:init:{n}'] for n in names}
    final = {n: g[f'mlp_{loss}:final:{n}'] for n in names}
    return names, init, final


@pytest.mark.parametrize('loss', ['mse', 'cross_entropy'])
def test_mlp_training_restatement_against_polygrad_fixture(loss):
    """polyref.mlp_train_sgd against five poly_instance_train_step calls of stock polygrad
    (tests/golden/train.npz): loss of every step and every parameter afterwards within 1e-5."""
    g = np.load(os.path.join(G, 'train.npz'))
    names, init, final = _mlp_case(g, loss)
    ws = [init[n] for n in names if n.endswith('weight')]
    bs = [init[n] for n in names if n.endswith('bias')]
    losses, ws2, bs2 = polyref.mlp_train_sgd(ws, bs, g[f'mlp_{loss}:x'], g[f'mlp_{loss}:y'], 0.01, 5, loss)
    np.testing.assert_allclose(losses, g[f'mlp_{loss}:losses'], rtol=2e-5)
    for got, n in zip(ws2, [n for n in names if n.endswith('weight')]):
        assert_close(got, final[n], 1e-5, n)
    for got, n in zip(bs2, [n for n in names if n.endswith('bias')]):
        assert_close(got, final[n], 1e-5, n)
    assert losses[-1] < losses[0]


def test_training_fixture_reproduced_by_polygrad(ref_lib):
    """Where stock polygrad is built, it reproduces its own training fixture."""
    from polygrad_b200 import ffi
    from polygrad_b200.instance import Instance
    g = np.load(os.path.join(G, 'train.npz'))
    names, init, final = _mlp_case(g, 'mse')
    inst = Instance.mlp(ref_lib, [96, 64, 10], 'relu', True, 1, seed=42, loss='mse')
    for n in names:
        inst.write(n, init[n])
    inst.set_optimizer(ffi.OPTIM_SGD, 0.01)
    losses = [inst.train_step(x=g['mlp_mse:x'], y=g['mlp_mse:y']) for _ in range(5)]
    np.testing.assert_allclose(losses, g['mlp_mse:losses'], rtol=1e-6)
    for n in names:
        assert_close(inst.read(n), final[n], 1e-6, n)
    inst.free()
