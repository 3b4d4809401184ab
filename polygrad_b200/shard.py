"""Data-parallel sharding of the forward path: one process per GPU, weights
replicated, batch rows split across ranks.  The forward has no cross-row
dependency (polygrad's GPT-2 graph, src/modelzoo/models/gpt2.c:320-526, treats
every sequence independently), so the data path needs no collective; the only
exchange is the optional gather of results to rank 0 and the max-over-ranks of
the step time.  Everything here works on the `gloo` backend on CPU as well as
on `nccl`."""
import os

import numpy as np


def rank_env():
    """(rank, world, local_rank) from the launcher's environment; (0, 1, 0) when
    started as a plain process."""
    return (int(os.environ.get('RANK', '0')), int(os.environ.get('WORLD_SIZE', '1')),
            int(os.environ.get('LOCAL_RANK', '0')))


def shard_tokens(seed, rank, batch, seq_len, vocab):
    """Rank `rank`'s rows of the global synthetic batch: `batch` sequences of
    `seq_len` token ids in [0, vocab), as float32 (polygrad's token input dtype).
    Depends on (seed, rank) only, so any process can rebuild any rank's shard."""
    rng = np.random.default_rng([seed, rank])
    return rng.integers(0, vocab, (batch, seq_len)).astype(np.float32)


def global_tokens(seed, world, batch, seq_len, vocab):
    """The whole job's batch: rank shards stacked in rank order."""
    return np.concatenate([shard_tokens(seed, r, batch, seq_len, vocab) for r in range(world)], axis=0)


def shard_rows(n_rows, rank, world):
    """[lo, hi) of `n_rows` rows owned by `rank` when a fixed-size set is split
    (strong scaling); the first n_rows % world ranks take one extra row."""
    base, extra = divmod(n_rows, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def gather_to_root(dist, src, dst_list, rank):
    """Gather equally shaped tensors to rank 0 (dst_list is None elsewhere)."""
    dist.gather(src, dst_list if rank == 0 else None, dst=0)


def max_over_ranks(dist, value, device='cpu'):
    """The slowest rank's value; every rank gets it."""
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
