"""Regenerates tests/golden/*.npz by running STOCK polygrad (CPU backend, built
by `make -C oracle ref` from its own sources) on seeded inputs.

    python tests/golden/make_golden.py            # everything
    python tests/golden/make_golden.py train      # train.npz only

Needs the polygrad checkout; the committed .npz files are what travels.  Every
case stores its inputs and polygrad's output, so tests need neither the
checkout nor the library to use them.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
os.environ['PATH'] = os.path.join(ROOT, 'oracle', 'shim') + os.pathsep + os.environ.get('PATH', '')

from polygrad_b200 import ffi                      # noqa: E402
from polygrad_b200.instance import Instance, gpt2_init  # noqa: E402
from polygrad_b200.tensor import Device            # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def main():
    ref = ffi.load_reference(os.path.join(ROOT, 'oracle', '_ref', 'libpolygrad_ref.so'))
    if sys.argv[1:] == ['train']:          # only the training fixture
        make_training(ref)
        return
    cpu = Device(ref, ffi.DEVICE_CPU)
    rng = np.random.default_rng(20240607)

    # row ops on a ragged shape
    x = rng.standard_normal((37, 203)).astype(np.float32)
    t = cpu.tensor(x)
    rowops = dict(
        x=x,
        affine=(t * 2 + 1).numpy(), exp=t.exp().numpy(), tanh=t.tanh().numpy(), gelu=t.gelu().numpy(),
        sum=t.sum(-1).numpy(), max=t.max(-1).numpy(), mean=t.mean(-1).numpy(), var=t.var(-1).numpy(),
        softmax=t.softmax(-1).numpy(), layernorm=t.layernorm(-1, 1e-5).numpy(),
        permute=t.permute(1, 0).numpy(), flip0=t[::-1].numpy(), flip1=t[:, ::-1].numpy(), step3=t[:, ::3].numpy(),
    )
    np.savez_compressed(os.path.join(OUT, 'rowops.npz'), **rowops)

    # matmul fp32 and bf16-operand
    a = rng.uniform(-1, 1, (45, 130)).astype(np.float32)
    b = rng.uniform(-1, 1, (130, 61)).astype(np.float32)
    f32 = cpu.tensor(a).dot(cpu.tensor(b)).numpy()
    bf = cpu.tensor(a, 'bfloat16').cast('float32').dot(cpu.tensor(b, 'bfloat16').cast('float32')).numpy()
    np.savez_compressed(os.path.join(OUT, 'matmul.npz'), a=a, b=b, f32=f32, bf16=bf)

    # MLP config (reduced batch) with polygrad's own seeded Kaiming init
    xm = rng.standard_normal((16, 784)).astype(np.float32)
    inst = Instance.mlp(ref, [784, 512, 10], 'relu', True, 16, seed=42)
    params = {n: inst.read(n).copy() for n in inst.params}
    inst.forward(x=xm)
    np.savez_compressed(os.path.join(OUT, 'mlp.npz'), x=xm, output=inst.read('output'),
                        **{'param:' + k: v for k, v in params.items()})
    inst.free()

    # GPT-2, toy dimensions, logits
    cfg = dict(vocab_size=97, n_embd=48, n_head=4, n_layer=2, max_seq_len=24, max_batch=2)
    tokens = rng.integers(0, cfg['vocab_size'], (2, 24))
    inst = Instance.gpt2(ref, **cfg)
    inst.init_params(gpt2_init(7))
    inst.forward(**inst.gpt2_inputs(tokens))
    np.savez_compressed(os.path.join(OUT, 'gpt2_toy.npz'), tokens=tokens, logits=inst.read('output'),
                        cfg=np.array([cfg[k] for k in ('vocab_size', 'n_embd', 'n_head', 'n_layer', 'max_seq_len', 'max_batch')]),
                        seed=np.array(7))
    inst.free()
    make_training(ref)
    print('golden fixtures written to', OUT)


def make_training(ref):
    """train.npz: poly_instance_train_step on the CPU backend.  A small MLP (batch 1: polygrad's MLP
    builder supports a loss at that batch size only) under SGD with both losses, and a two-layer GPT-2 under SGD: inputs, initial parameters, the loss of every step and
    every parameter after the last one."""
    rng = np.random.default_rng(20240608)
    out = {}
    x = rng.standard_normal((1, 96)).astype(np.float32)
    for loss in ('mse', 'cross_entropy'):
        y = rng.standard_normal((1, 10)).astype(np.float32)
        if loss == 'cross_entropy':
            y = np.zeros((1, 10), np.float32)
            y[0, 7] = 1.0
        inst = Instance.mlp(ref, [96, 64, 10], 'relu', True, 1, seed=42, loss=loss)
        for n in inst.params:
            out[f'mlp_{loss}:init:{n}'] = inst.read(n).copy()
        inst.set_optimizer(ffi.OPTIM_SGD, 0.01)
        out[f'mlp_{loss}:x'], out[f'mlp_{loss}:y'] = x, y
        out[f'mlp_{loss}:losses'] = np.array([inst.train_step(x=x, y=y) for _ in range(5)], np.float32)
        for n in inst.params:
            out[f'mlp_{loss}:final:{n}'] = inst.read(n).copy()
        inst.free()
    cfg = dict(vocab_size=64, n_embd=48, n_head=4, n_layer=2, max_seq_len=16, max_batch=2)
    tokens = rng.integers(0, cfg['vocab_size'], (2, 16))
    inst = Instance.gpt2(ref, **cfg)
    inst.init_params(gpt2_init(7))
    inst.set_optimizer(ffi.OPTIM_SGD, 1e-5)
    out['gpt2:tokens'] = tokens
    out['gpt2:cfg'] = np.array([cfg[k] for k in ('vocab_size', 'n_embd', 'n_head', 'n_layer', 'max_seq_len', 'max_batch')])
    out['gpt2:losses'] = np.array([inst.train_step(**inst.gpt2_inputs(tokens)) for _ in range(3)], np.float32)
    for n in inst.params:
        out[f'gpt2:final:{n}'] = inst.read(n).copy()
    inst.free()
    np.savez_compressed(os.path.join(OUT, 'train.npz'), **out)


if __name__ == '__main__':
    main()
