"""The N>1 path on CPU: two gloo ranks, launched the way the bench is launched
(torch.distributed.run on 127.0.0.1)."""
import json
import os
import socket
import subprocess
import sys

import numpy as np

from polygrad_b200 import shard

HERE = os.path.dirname(os.path.abspath(__file__))


def free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def test_shards_tile_the_global_batch():
    g = shard.global_tokens(9, 4, 2, 16, 100)
    assert g.shape == (8, 16) and g.dtype == np.float32 and g.min() >= 0 and g.max() < 100
    for r in range(4):
        assert np.array_equal(g[2 * r:2 * r + 2], shard.shard_tokens(9, r, 2, 16, 100))
    assert not np.array_equal(g[0:2], g[2:4])


def test_shard_rows_partition():
    for n in (0, 1, 7, 8, 1000):
        for world in (1, 2, 3, 8):
            spans = [shard.shard_rows(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def test_two_gloo_ranks_equal_one_global_forward(tmp_path):
    out = tmp_path / 'rank0.json'
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', '2',
           '--master-addr', '127.0.0.1', '--master-port', str(free_port()),
           os.path.join(HERE, 'gloo_worker.py'), str(out)]
    env = dict(os.environ, OMP_NUM_THREADS='1')
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    r = json.load(open(out))
    assert r['world'] == 2 and r['rows'] == 6
    assert r['max_abs_diff'] == 0.0            # rows are independent: sharding changes nothing
    assert r['slowest'] == 11.0
    assert r['spans'] == [[0, 4], [4, 7]]


def test_two_ranks_drive_the_micro_batch_loop(tmp_path):
    """poly_b200_forward_microbatches on two ranks in dry-run mode: micro-batch i of rank r is number
    i * world + r of the global batch and lands in that slot of the root's buffer; each micro-batch's
    token ids are uploaded before its forward."""
    out = tmp_path / 'micro.json'
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', '2',
           '--master-addr', '127.0.0.1', '--master-port', str(free_port()),
           os.path.join(HERE, 'gloo_micro_worker.py'), str(out)]
    env = dict(os.environ, OMP_NUM_THREADS='1')
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    r = json.load(open(out))
    assert r['world'] == 2 and r['uniform']
    assert r['order'] == [0, 1, 0, 1, 0, 1]          # slot i * world + r holds rank r's micro-batch i
    assert r['x_last'] == r['x_want']
    # data-parallel training steps: with update averaging on, each step of each rank issues one
    # all-reduce per parameter plus one for the loss, the same sizes in the same order on both ranks
    # (NCCL matches collectives by order); with it off, none
    a0, a1 = r['averaging']
    n = a0['n_params']
    assert n > 0 and a0['per_step'] == a1['per_step']
    assert [c for c, _ in a0['per_step']] == [n + 1, 2 * (n + 1), 3 * (n + 1)]
    assert len({h for _, h in a0['per_step']}) == 3
    assert a0['after_off'] == 3 * (n + 1) and a1['after_off'] == 3 * (n + 1)
