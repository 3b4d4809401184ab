"""Regenerates tests/golden/gpt2_1.5b_t32.npz: STOCK polygrad (CPU backend, built by
`make -C oracle ref` from its own sources) running GPT-2 1.5B -- 48 layers, d = 1600,
25 heads, vocabulary 50257 -- on one seeded sequence of 32 tokens with seeded weights.

    python tests/golden/make_golden_gpt2_large.py        # about 10 minutes on one core

Scheduling and compiling the 1258 kernels of the 48-layer graph takes the CPU backend
five minutes and a forward another two to three, too long for a test run, so the result
is committed instead: the logits of every position at 2048 seeded vocabulary columns,
each position's largest logit, its index and the margin to the runner-up, and the
root-mean-square of all logits.  Weights and token ids are functions of the seed
(polygrad_b200.instance.gpt2_init, numpy's default_rng), so a test rebuilds the same
model on the device from the seed alone.
"""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
os.environ['PATH'] = os.path.join(ROOT, 'oracle', 'shim') + os.pathsep + os.environ.get('PATH', '')

from polygrad_b200 import ffi                              # noqa: E402
from polygrad_b200.instance import Instance, gpt2_init     # noqa: E402

ARCH = dict(vocab_size=50257, n_embd=1600, n_head=25, n_layer=48)
T, SEED, N_COLS = 32, 3, 2048


def main():
    ref = ffi.load_reference(os.path.join(ROOT, 'oracle', '_ref', 'libpolygrad_ref.so'))
    tokens = np.random.default_rng([77, T]).integers(0, ARCH['vocab_size'], (8, T))
    t0 = time.time()
    inst = Instance.gpt2(ref, **dict(ARCH, max_seq_len=T, max_batch=1))
    inst.init_params(gpt2_init(SEED))
    inst.forward(**inst.gpt2_inputs(tokens[:1]))
    logits = inst.read('output')[0].copy()            # [T, V]
    inst.free()
    cols = np.sort(np.random.default_rng(5).choice(ARCH['vocab_size'], N_COLS, replace=False))
    top2 = np.partition(logits, -2, axis=-1)[:, -2:]
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), 'gpt2_1.5b_t32.npz'),
                        arch=np.array([ARCH['vocab_size'], ARCH['n_embd'], ARCH['n_head'], ARCH['n_layer'], T, SEED]),
                        tokens=tokens, cols=cols, logits_cols=logits[:, cols],
                        argmax=logits.argmax(-1), top=top2[:, 1], margin=top2[:, 1] - top2[:, 0],
                        rms=np.float64(np.sqrt(np.mean(logits.astype(np.float64) ** 2))),
                        row_sum=logits.astype(np.float64).sum(-1), cpu_seconds=np.float64(time.time() - t0))
    print(f'done in {time.time() - t0:.0f} s, rms {np.sqrt(np.mean(logits.astype(np.float64) ** 2)):.4f}')


if __name__ == '__main__':
    main()
