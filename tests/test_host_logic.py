"""Host-side logic, no GPU: the C-ABI library loads and exports what
include/poly_b200.h declares; the kernel classifier and renderer process
polygrad's scheduled kernels (dry run: programs are rendered and compiled by
NVRTC, which needs no device, and launches are ignored)."""
import ctypes
import json
import os
import re
import subprocess
import sys

import pytest

from conftest import ROOT

HEADER = os.path.join(ROOT, 'include', 'poly_b200.h')


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(poly_(?:cuda|b200|linearize|render|compile)_?\w*)\s*\(', text)))


def test_library_exports_every_declared_symbol(product_lib):
    names = declared_symbols()
    assert 'poly_cuda_launch' in names and 'poly_linearize_cuda' in names and len(names) >= 25
    missing = [n for n in names if not hasattr(product_lib.c, n)]
    assert not missing, missing


def test_kernel_library_is_standalone():
    """The runtime + kernels library has no polygrad dependency."""
    from polygrad_b200 import ffi
    lib = ctypes.CDLL(ffi.KERNEL_LIB)
    for n in ('poly_cuda_init', 'poly_cuda_alloc', 'poly_compile_cuda', 'poly_cuda_launch', 'poly_b200_stats'):
        assert hasattr(lib, n)


def test_no_device_fails_loudly():
    """Without a GPU (and without the dry-run switch) the backend reports an
    error; it never computes on the CPU."""
    code = ("import sys; sys.path.insert(0, %r)\n"
            "from polygrad_b200 import ffi\n"
            "lib = ffi.product()\n"
            "import torch\n"
            "if torch.cuda.is_available(): print('HAS_GPU'); sys.exit(0)\n"
            "assert lib.poly_cuda_init() != 0\n"
            "assert not lib.poly_cuda_available()\n"
            "assert lib.poly_cuda_alloc(16) == 0\n"
            "print('OK', lib.last_error())\n") % ROOT
    env = dict(os.environ)
    env.pop('POLY_B200_DRYRUN', None)
    r = subprocess.run([sys.executable, '-c', code], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert 'OK' in r.stdout or 'HAS_GPU' in r.stdout


DRY = r'''
import json, os, sys
sys.path.insert(0, %(root)r)
import numpy as np
from polygrad_b200 import ffi
from polygrad_b200.instance import Instance, gpt2_init
lib = ffi.product()
assert lib.poly_cuda_init() == 0
kinds = {}
import ctypes
cfg = dict(vocab_size=211, n_embd=96, n_head=4, n_layer=2, max_seq_len=48, max_batch=2)
inst = Instance.gpt2(lib, **cfg)
inst.init_params(gpt2_init(1))
inst.set_device(ffi.DEVICE_CUDA)
inst.forward(**inst.gpt2_inputs(np.zeros((2, 48))))
print(json.dumps(lib.stats()))
'''


def test_gpt2_plan_lowers_in_dry_run():
    env = dict(os.environ, POLY_B200_DRYRUN='1', POLY_DUMP_KERNELS='1', POLY_B200_CACHE='0')
    r = subprocess.run([sys.executable, '-c', DRY % dict(root=ROOT)], env=env, capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stderr[-4000:]
    # one program per scheduled kernel (polygrad's count for GPT-2 is 10 + 26 per layer) ...
    n_layer = 2
    per_kernel = re.findall(r'^=== CUDA KERNEL plan\d+_k\d+ ===\n//PB200 1\n//kind (\w+)', r.stderr, flags=re.M)
    assert len(per_kernel) == 10 + 26 * n_layer
    assert per_kernel.count('gather') == 2               # token and position embeddings
    assert per_kernel.count('gemm') == 6 * n_layer + 1   # qkv, scores, attn.v, c_proj, fc, proj per layer + logits
    # ... plus the programs the plan passes build from them
    fused = re.findall(r'^=== CUDA KERNEL rowfused_k\d+ ===', r.stderr, flags=re.M)
    assert len(fused) >= 3 * n_layer + 1                  # LN1, softmax, LN2 per layer + final LN
    stats = json.loads(r.stdout.strip().splitlines()[-1])
    assert stats['memsets_executed'] <= 4           # zero fills are elided when kernels overwrite whole buffers


DRY_BF16 = r'''
import os, sys
sys.path.insert(0, %(root)r)
import numpy as np
from polygrad_b200 import ffi
from polygrad_b200.instance import Instance, gpt2_init
lib = ffi.product()
assert lib.poly_cuda_init() == 0
cfg = dict(vocab_size=320, n_embd=128, n_head=2, n_layer=2, max_seq_len=128, max_batch=2)
inst = Instance.gpt2(lib, **cfg)
inst.init_params(gpt2_init(1))
inst.set_device(ffi.DEVICE_CUDA)
inst.forward(**inst.gpt2_inputs(np.zeros((2, 128))))
'''


def test_bf16_policy_plan_passes_in_dry_run():
    """Under the bf16 contraction policy, per layer: the attention chain becomes one step, the q/k/v
    slice copies are folded into its operand strides, and the operands of the four projections (and of
    the attention) are produced as bfloat16 by the step before them."""
    env = dict(os.environ, POLY_B200_DRYRUN='1', POLY_B200_DEBUG='1', POLY_B200_CACHE='0', POLY_B200_GEMM='bf16')
    r = subprocess.run([sys.executable, '-c', DRY_BF16 % dict(root=ROOT)], env=env, capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stderr[-4000:]
    n_layer = 2
    m = re.search(r'pb_fuse: (\d+) copy kernels elided, (\d+) kernels folded into row kernels, (\d+) attention chains fused', r.stderr)
    assert m and int(m.group(3)) == n_layer
    m = re.search(r'pb_operands: (\d+) copies folded into operand strides, (\d+) operands stored as bfloat16, '
                  r'(\d+) attention outputs written as bfloat16 matrices, (\d+) attention steps reuse a mask classification', r.stderr)
    assert m, r.stderr[-2000:]
    assert int(m.group(1)) == 3 * n_layer                 # q, k, v
    assert int(m.group(2)) == 4 * n_layer + 1             # LN1->qkv, qkv->attention, LN2->fc, GELU->proj; final LN->logits
    assert int(m.group(3)) == n_layer
    assert int(m.group(4)) == n_layer - 1                 # the mask is classified once
    m = re.search(r'(\d+) GELU kernels moved into contraction epilogues', r.stderr)
    assert m and int(m.group(1)) == n_layer               # recognised by evaluating the kernel's scalar function
    m = re.search(r'pb_plan: (\d+) steps', r.stderr)
    # per layer: LN1 (with the residual add before it), qkv, attention, c_proj, LN2 (with its add), fc (with GELU), proj;
    # around them: two gathers, the mask generator, final LN (with the last add), logits
    assert m and int(m.group(1)) == 5 + 7 * n_layer


def test_gelu_epilogue_can_be_switched_off():
    env = dict(os.environ, POLY_B200_DRYRUN='1', POLY_B200_DEBUG='1', POLY_B200_CACHE='0', POLY_B200_GEMM='bf16',
               POLY_B200_EPILOGUE='0')
    r = subprocess.run([sys.executable, '-c', DRY_BF16 % dict(root=ROOT)], env=env, capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stderr[-4000:]
    assert re.search(r' 0 GELU kernels moved into contraction epilogues', r.stderr)
    m = re.search(r'pb_plan: (\d+) steps', r.stderr)
    assert m and int(m.group(1)) == 5 + 8 * 2


DRY_TRAIN = '''
import sys
sys.path.insert(0, %(root)r)
import numpy as np
from polygrad_b200 import ffi
from polygrad_b200.instance import Instance, gpt2_init
lib = ffi.product()
inst = Instance.gpt2(lib, 64, 48, 4, 1, 16, 2)
inst.init_params(gpt2_init(3))
inst.set_device(ffi.DEVICE_CUDA)
inst.set_optimizer(ffi.OPTIM_SGD, 1e-3)
inst.train_step(**inst.gpt2_inputs(np.zeros((2, 16))))
inst.train_step(**inst.gpt2_inputs(np.zeros((2, 16))))
'''


def test_training_plan_in_dry_run():
    """A training step's plan updates the bound parameters in place: it is run as scheduled (no pass
    moves work across the update), its weight-gradient contractions with plain operands carry the
    learning-rate scale, and the loss scalar -- a host pointer in a device plan -- is accepted."""
    env = dict(os.environ, POLY_B200_DRYRUN='1', POLY_B200_DEBUG='2', POLY_B200_CACHE='0')
    r = subprocess.run([sys.executable, '-c', DRY_TRAIN % dict(root=ROOT)], env=env, capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stderr[-4000:]
    assert 'plan updates bound buffers in place' in r.stderr
    assert 'kernels folded into row kernels' not in r.stderr
    steps = re.findall(r'pb_plan: step +\d+ item +\d+ (\S+) +(.*)', r.stderr)
    kinds = [k for k, _ in steps]
    assert kinds.count('gather') == 2 and kinds.count('gemm') >= 13
    # every bound buffer that is written (parameters, logits are not part of this plan, loss) has one writer
    written = [a for _, args in steps for a in args.split() if a[0] in 'Wwb' and a.endswith('x')]
    assert len(written) == len(set(written)) and len(written) >= 17


DRY_EAGER = '''
import json, sys
sys.path.insert(0, %(root)r)
import numpy as np
from polygrad_b200 import ffi
from polygrad_b200.tensor import Device
lib = ffi.product()
assert lib.poly_cuda_init() == 0

def bindings(pairs):
    b = (ffi.PolyBufferBinding * len(pairs))()
    for i, (buf, host) in enumerate(pairs):
        b[i].buffer = buf; b[i].handle.ptr = host.ctypes.data
        b[i].handle.nbytes = host.nbytes; b[i].handle.domain = ffi.DEVICE_CPU
    return b

dev = Device(lib, ffi.DEVICE_CUDA)
x = np.arange(64 * 32, dtype=np.float32).reshape(64, 32)
log = []
for i in range(4):
    t = dev.tensor(x + i).softmax(-1)
    out_buf = lib.poly_buffer_by_id(dev.ctx, t.numel(), ffi.DTYPE_IDS['float32'])
    out = np.full(t.numel(), 7.0, np.float32)
    sink = lib.poly_sink1(dev.ctx, lib.poly_store_val(dev.ctx, out_buf, t.uop))
    pairs = list(t.leaves) + [(out_buf, out)]
    assert lib.poly_realize_cuda(dev.ctx, sink, bindings(pairs), len(pairs)) == 0
    after_run = dict(lib.eager_stats(), untouched=bool((out == 7).all()), **lib.stats())
    assert lib.poly_cuda_copyback(bindings(pairs), len(pairs)) == 0
    log.append([after_run, dict(lib.eager_stats(), **lib.stats())])
dev.close()
log.append(lib.eager_stats())
print(json.dumps(log))
'''


def test_eager_entry_keeps_plans_and_results_in_dry_run():
    """The eager entry point's bookkeeping, with no device: the second and later calls (new leaves,
    new output buffer, new SINK) find the first call's plan; only the buffer the graph reads is
    uploaded; the result is left where the plan wrote it until poly_cuda_copyback, which copies that
    buffer alone; destroying the context releases the plan."""
    import json
    env = dict(os.environ, POLY_B200_DRYRUN='1', POLY_B200_DRYRUN_NOCOMPILE='1')
    env.pop('POLY_B200_LEGACY', None)
    r = subprocess.run([sys.executable, '-c', DRY_EAGER % dict(root=ROOT)], env=env, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-4000:]
    log = json.loads(r.stdout.strip().splitlines()[-1])
    nbytes = 64 * 32 * 4
    for i, (ran, copied) in enumerate(log[:4]):
        assert ran['misses'] == 1 and ran['hits'] == i and ran['plans_kept'] == 1
        assert ran['buffers_resident'] == 1 and ran['untouched']
        assert ran['bytes_htod'] == (i + 1) * nbytes and ran['bytes_dtoh'] == i * nbytes
        assert copied['buffers_resident'] == 0 and copied['bytes_dtoh'] == (i + 1) * nbytes
    assert log[4]['plans_kept'] == 0 and log[4]['buffers_resident'] == 0


def test_backward_kernels_are_cut_in_dry_run():
    """With the cut forced at a width where it would not pay, the training plan's kernels that hold
    contractions next to other work are lowered as several steps: operand temporaries and remainders as
    generated code, every contraction as a contraction program, the lookup's gradient as a scatter program
    (kept in place, not turned into a one-hot temporary), the q/k/v gradients over their windows."""
    env = dict(os.environ, POLY_B200_DRYRUN='1', POLY_B200_DEBUG='1', POLY_B200_CACHE='0', POLY_DUMP_KERNELS='1',
               POLY_B200_OUTLINE_MIN_WORK='0')
    r = subprocess.run([sys.executable, '-c', DRY_TRAIN % dict(root=ROOT)], env=env, capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stderr[-4000:]
    m = re.search(r'pb_plan: (\d+) kernels cut into contractions and elementwise pieces', r.stderr)
    assert m and int(m.group(1)) >= 4
    pieces = re.findall(r'^=== CUDA KERNEL (plan\d+_k\d+)_p(\d+) ===\n//PB200 1\n//kind (\w+)', r.stderr, flags=re.M)
    by_kernel = {}
    for name, _, kind in pieces:
        by_kernel.setdefault(name, []).append(kind)
    assert len(by_kernel) >= 4
    for name, kinds in by_kernel.items():
        assert kinds[-1] in ('jit', 'gemm'), (name, kinds)                 # the remainder, or a single contraction
        assert any(k in ('gemm', 'scatter') for k in kinds), (name, kinds)
    all_kinds = [k for kinds in by_kernel.values() for k in kinds]
    assert all_kinds.count('scatter') >= 1                                 # the lookups' gradients (token and position tables)
    assert any(kinds.count('gemm') == 3 for kinds in by_kernel.values())   # q, k and v gradients of the one layer
    assert 'stays whole' not in r.stderr
