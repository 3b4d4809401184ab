"""Worker for test_shard_gloo.py: one rank of a world-size-N CPU job.  Each rank
computes the forward of its own batch shard with the numpy oracle, the last
position's logits are gathered to rank 0, and the step time goes through the
max-over-ranks reduction, i.e. the multi-rank host logic of bench.py on gloo."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import polyref                                       # noqa: E402
from polygrad_b200 import shard                                  # noqa: E402
from polygrad_b200.instance import gpt2_init                     # noqa: E402

CFG = dict(vocab_size=64, n_embd=32, n_head=2, n_layer=2, max_seq_len=8, norm_eps=1e-5)
SEED, B = 5, 3


def main():
    out_path = sys.argv[1]
    rank, world, _ = shard.rank_env()
    dist.init_process_group('gloo')
    init = gpt2_init(SEED)
    tokens = shard.shard_tokens(SEED, rank, B, CFG['max_seq_len'], CFG['vocab_size'])
    logits = polyref.gpt2_forward(CFG, init, tokens)             # [B, T, V]
    src = torch.from_numpy(np.ascontiguousarray(logits[:, -1, :]))
    dst = [torch.empty_like(src) for _ in range(world)] if rank == 0 else None
    shard.gather_to_root(dist, src, dst, rank)
    slowest = shard.max_over_ranks(dist, 10.0 + rank)
    lo, hi = shard.shard_rows(7, rank, world)
    spans = [None] * world
    dist.all_gather_object(spans, (lo, hi))
    if rank == 0:
        whole = polyref.gpt2_forward(CFG, init, shard.global_tokens(SEED, world, B, CFG['max_seq_len'], CFG['vocab_size']))
        got = torch.cat(dst, 0).numpy()
        json.dump(dict(world=world, max_abs_diff=float(np.abs(got - whole[:, -1, :]).max()),
                       rows=int(got.shape[0]), slowest=slowest, spans=spans), open(out_path, 'w'))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
