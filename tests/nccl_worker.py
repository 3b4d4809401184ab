"""Worker for test_multi_gpu.py: one rank (one GPU) of a data-parallel job through the
library's own communicator.  Every rank runs its micro-batches of the global batch with
poly_b200_forward_microbatches, each result gathered to rank 0 by NCCL behind the next
micro-batch; rank 0 then recomputes every micro-batch of every rank itself and compares
bit for bit (replicas hold the same weights and run the same kernels)."""
import ctypes
import json
import os
import sys

import numpy as np
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from polygrad_b200 import ffi, shard                             # noqa: E402
from polygrad_b200.instance import Instance, gpt2_init           # noqa: E402

CFG = dict(vocab_size=512, n_embd=128, n_head=2, n_layer=2, max_seq_len=128, max_batch=2)
N_MICRO, SEED = 3, 11


def main():
    out_path = sys.argv[1]
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

    lib.poly_b200_set_gemm_policy(1)
    inst = Instance.gpt2(lib, **CFG)
    inst.init_params(gpt2_init(SEED))
    inst.set_device(ffi.DEVICE_CUDA)
    out_idx, out_shape, _ = inst.bufs['output']
    n_out = int(np.prod(out_shape))

    def tokens_of(r, i):
        return shard.shard_tokens(SEED, lib.poly_b200_shard_micro_index(r, world, i), CFG['max_batch'],
                                  CFG['max_seq_len'], CFG['vocab_size'])
    micro = [tokens_of(rank, i) for i in range(N_MICRO)]
    ptrs = (ctypes.POINTER(ctypes.c_float) * N_MICRO)(*[m.ctypes.data_as(ctypes.POINTER(ctypes.c_float)) for m in micro])
    # first forward: positions / arange inputs and the plan
    inst.forward(**inst.gpt2_inputs(micro[0]))
    root_dst = lib.poly_cuda_alloc(n_out * 4 * N_MICRO * world) if rank == 0 else 0
    for _ in range(2):                                   # twice: the second round replays captured graphs
        rc = lib.poly_b200_forward_microbatches(inst.h, b'x', ptrs, N_MICRO, out_idx, n_out * 4, root_dst or None, 0, 1)
        assert rc == 0, lib.last_error()
        assert lib.poly_b200_comm_wait() == 0 and lib.poly_b200_synchronize() == 0, lib.last_error()
    result = dict(world=world)
    if rank == 0:
        got = np.empty((N_MICRO * world, n_out), np.float32)
        assert lib.poly_cuda_copy_dtoh(got.ctypes.data, root_dst, got.nbytes) == 0
        equal = []
        for i in range(N_MICRO):
            for r in range(world):
                inst.forward(**inst.gpt2_inputs(tokens_of(r, i)))
                want = inst.read('output').reshape(-1)
                equal.append(bool(np.array_equal(got[i * world + r].view(np.uint32), want.view(np.uint32))))
        result.update(equal=equal, finite=bool(np.isfinite(got).all()), nonzero=bool(np.abs(got).max() > 0))
        # slots of different ranks must differ (different tokens)
        result['distinct'] = bool(not np.array_equal(got[0], got[1]))
        lib.poly_cuda_free(root_dst)
    t = ctypes.c_double(1.0 + rank)
    assert lib.poly_b200_comm_max(ctypes.byref(t)) == 0
    result['max'] = t.value
    if rank == 0:
        json.dump(result, open(out_path, 'w'))
    inst.free()
    dist.barrier()
    lib.poly_b200_comm_destroy()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
