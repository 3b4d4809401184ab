"""Two ranks on two GPUs through the library's NCCL communicator (skipped where fewer than two
GPUs are visible; the same host logic runs on CPU ranks in test_shard_gloo.py).  Ranks leave only
after their last collective has finished; NVLS is off for the run."""
import json
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _gpu_count():
    try:
        out = subprocess.run(['nvidia-smi', '-L'], capture_output=True, text=True, timeout=30).stdout
        return sum(1 for line in out.splitlines() if line.startswith('GPU '))
    except (OSError, subprocess.SubprocessError):
        return 0


def test_two_ranks_gather_micro_batches_bit_exact(tmp_path):
    if _gpu_count() < 2:
        pytest.skip('needs two GPUs')
    s = socket.socket(); s.bind(('127.0.0.1', 0)); port = s.getsockname()[1]; s.close()
    out = tmp_path / 'rank0.json'
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', '2',
           '--master-addr', '127.0.0.1', '--master-port', str(port), os.path.join(HERE, 'nccl_worker.py'), str(out)]
    env = dict(os.environ, NCCL_NVLS_ENABLE='0', OMP_NUM_THREADS='1')
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, (p.stdout[-2000:], p.stderr[-4000:])
    r = json.load(open(out))
    assert r['world'] == 2 and r['finite'] and r['nonzero'] and r['distinct']
    assert all(r['equal']) and len(r['equal']) == 6
    assert r['max'] == 2.0


@pytest.mark.parametrize('inline', ['0', '1'], ids=['after_the_replay', 'between_the_launches'])
def test_two_ranks_train_on_the_mean_gradient(tmp_path, ref_lib, inline):
    """Data-parallel SGD: two ranks, the same parameters, different tokens, three steps with the
    backend averaging every updated parameter over the ranks.  Stock polygrad on the CPU takes, for
    each step, one step per rank's tokens from the common parameters and averages the results --
    for SGD the same as one step on the mean gradient.  Both replicas must end bit-identical to each
    other, and within the single-GPU training tolerance (1e-4) of the CPU.  Both places the averaging
    can happen are run: after the plan's graph replay (what a plan this small gets) and between the
    launches, behind the rest of the backward pass (what a plan with 1 GB or more to average gets)."""
    if _gpu_count() < 2:
        pytest.skip('needs two GPUs')
    import numpy as np
    from conftest import assert_close
    from polygrad_b200 import ffi
    from polygrad_b200.instance import Instance, gpt2_init
    sys.path.insert(0, HERE)
    import nccl_train_worker as w
    s = socket.socket(); s.bind(('127.0.0.1', 0)); port = s.getsockname()[1]; s.close()
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', '2',
           '--master-addr', '127.0.0.1', '--master-port', str(port), os.path.join(HERE, 'nccl_train_worker.py'), str(tmp_path)]
    env = dict(os.environ, NCCL_NVLS_ENABLE='0', OMP_NUM_THREADS='1', POLY_B200_AVERAGE_INLINE=inline)
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, (p.stdout[-2000:], p.stderr[-4000:])
    got = [np.load(tmp_path / f'rank{r}.npz') for r in range(2)]
    names = [k for k in got[0].files if k.startswith('p:')]
    assert int(got[0]['calls']) == w.STEPS * (int(got[0]['n_params']) + 1)
    for k in names:
        assert np.array_equal(got[0][k].view(np.uint32), got[1][k].view(np.uint32)), f'replicas differ in {k}'
    assert np.array_equal(got[0]['losses'], got[1]['losses'])          # the loss is averaged too

    # the checker: stock polygrad, CPU (plain SGD keeps no state, so one instance serves every step)
    cpu = Instance.gpt2(ref_lib, **w.CFG)
    cpu.init_params(gpt2_init(w.INIT_SEED))
    cpu.set_optimizer(ffi.OPTIM_SGD, w.LR)
    first = {n: cpu.read(n).copy() for n in cpu.params}
    params, want_losses = first, []
    for step in range(w.STEPS):
        outs, losses = [], []
        for r in range(2):
            for n, v in params.items():
                cpu.write(n, v)
            losses.append(cpu.train_step(**cpu.gpt2_inputs(w.tokens_of(r, 2, step))))
            outs.append({n: cpu.read(n).copy() for n in cpu.params})
        params = {n: ((outs[0][n].astype(np.float64) + outs[1][n]) / 2).astype(np.float32) for n in outs[0]}
        want_losses.append((losses[0] + losses[1]) / 2)
    cpu.free()
    np.testing.assert_allclose(got[0]['losses'], want_losses, rtol=1e-4)
    for n in params:
        assert_close(got[0]['p:' + n], params[n], 1e-4, f'{n} after {w.STEPS} averaged steps')
        # and the distance travelled, which is what the mean gradient decides (fp32 cancellation: 2e-2)
        moved_want = params[n].astype(np.float64) - first[n]
        if np.sqrt(np.mean(moved_want ** 2)) > 1e-5:
            assert_close(got[0]['p:' + n].astype(np.float64) - first[n], moved_want, 2e-2, f'update of {n}')
    assert sum(int(not np.array_equal(first[n], params[n])) for n in params) >= len(params) // 2
