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
