"""Worker for test_multi_gpu.py: one rank (one GPU) of a data-parallel training job.  Every rank
holds the same parameters, runs polygrad's training step on its own tokens, and the backend averages
each updated parameter (and the loss) over the ranks right after the step that writes it.  Each rank
saves its losses and final parameters; the parent compares them with stock polygrad on the CPU."""
import ctypes
import os
import sys

import numpy as np
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from polygrad_b200 import ffi, shard                             # noqa: E402
from polygrad_b200.instance import Instance, gpt2_init           # noqa: E402

CFG = dict(vocab_size=64, n_embd=48, n_head=4, n_layer=2, max_seq_len=16, max_batch=2)
STEPS, SEED, INIT_SEED, LR = 4, 23, 7, 1e-5


def tokens_of(rank, world, step):
    return shard.shard_tokens(SEED, step * world + rank, CFG['max_batch'], CFG['max_seq_len'], CFG['vocab_size'])


def main():
    out_dir = sys.argv[1]
    rank, world, local_rank = shard.rank_env()
    os.environ['NCCL_NVLS_ENABLE'] = '0'
    lib = ffi.product()
    lib.poly_b200_set_device(local_rank)
    assert lib.poly_cuda_init() == 0, lib.last_error()
    dist.init_process_group('gloo')
    ident = (ctypes.c_ubyte * 128)()
    box = [None]
    if rank == 0:
        assert lib.poly_b200_comm_unique_id(ident, 128) > 0, lib.last_error()
        box[0] = bytes(ident)
    dist.broadcast_object_list(box, src=0)
    ident = (ctypes.c_ubyte * 128).from_buffer_copy(box[0])
    assert lib.poly_b200_comm_init(rank, world, ident, 128) == 0, lib.last_error()

    inst = Instance.gpt2(lib, **CFG)
    inst.init_params(gpt2_init(INIT_SEED))
    inst.set_device(ffi.DEVICE_CUDA)
    inst.set_optimizer(ffi.OPTIM_SGD, LR)
    lib.poly_b200_set_update_averaging(1)
    losses = [inst.train_step(**inst.gpt2_inputs(tokens_of(rank, world, s))) for s in range(STEPS)]
    assert lib.poly_b200_synchronize() == 0, lib.last_error()
    calls, trace = ctypes.c_ulonglong(), ctypes.c_ulonglong()
    lib.poly_b200_average_trace(ctypes.byref(calls), ctypes.byref(trace))
    params = {n: inst.read(n).copy() for n in inst.params}
    np.savez(os.path.join(out_dir, f'rank{rank}.npz'), losses=np.array(losses), calls=calls.value,
             n_params=len(inst.params), **{'p:' + n: v for n, v in params.items()})
    inst.free()
    dist.barrier()                      # nobody leaves while a peer may still be in a collective
    lib.poly_b200_comm_destroy()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
