"""Worker for test_shard_gloo.py: one rank of a CPU job that drives the library's
batch-sharded forward (poly_b200_forward_microbatches) in dry-run mode, where host
memory stands in for device buffers, launches are ignored and the root's part of a
gather is a host copy.  The other ranks' parts travel over gloo to the offsets the
library names, i.e. everything but the NCCL transfer itself runs."""
import ctypes
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

os.environ['POLY_B200_DRYRUN'] = '1'
os.environ['POLY_B200_DRYRUN_NOCOMPILE'] = '1'
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from polygrad_b200 import ffi, shard                             # noqa: E402
from polygrad_b200.instance import Instance, gpt2_init           # noqa: E402

CFG = dict(vocab_size=32, n_embd=16, n_head=2, n_layer=1, max_seq_len=8, max_batch=2)
N_MICRO = 3


def main():
    out_path = sys.argv[1]
    rank, world, _ = shard.rank_env()
    dist.init_process_group('gloo')
    lib = ffi.product()
    assert lib.poly_cuda_init() == 0
    ident = (ctypes.c_ubyte * 128)()
    assert lib.poly_b200_comm_init(rank, world, ident, 128) == 0
    inst = Instance.gpt2(lib, **CFG)
    inst.init_params(gpt2_init(1))
    inst.set_device(ffi.DEVICE_CUDA)
    out_idx, out_shape, _ = inst.bufs['output']
    n_out = int(np.prod(out_shape))
    # launches are ignored in dry-run mode: put a recognisable "result" into the output buffer
    inst.write('output', np.full(n_out, 100.0 + rank, np.float32))
    micro = [shard.shard_tokens(7, lib.poly_b200_shard_micro_index(rank, world, i), CFG['max_batch'],
                                CFG['max_seq_len'], CFG['vocab_size']) for i in range(N_MICRO)]
    ptrs = (ctypes.POINTER(ctypes.c_float) * N_MICRO)(*[m.ctypes.data_as(ctypes.POINTER(ctypes.c_float)) for m in micro])
    root_dst = np.zeros((N_MICRO * world, n_out), np.float32)
    rc = lib.poly_b200_forward_microbatches(inst.h, b'x', ptrs, N_MICRO, out_idx, n_out * 4,
                                            root_dst.ctypes.data if rank == 0 else None, 0, 1)
    assert rc == 0, lib.last_error()
    # the transfer NCCL would do, to the same places
    mine = torch.from_numpy(inst.read('output').reshape(-1).copy())
    for i in range(N_MICRO):
        parts = [torch.empty_like(mine) for _ in range(world)] if rank == 0 else None
        dist.gather(mine, parts, dst=0)
        if rank == 0:
            for r in range(1, world):
                slot = lib.poly_b200_shard_micro_index(0, world, i) + lib.poly_b200_gather_offset(r, 1)
                root_dst[slot] = parts[r].numpy()
    if rank == 0:
        order = [int(round(float(row[0]) - 100.0)) for row in root_dst]
        json.dump(dict(world=world, order=order, uniform=bool(all(np.all(row == row[0]) for row in root_dst)),
                       x_last=np.asarray(inst.read('x')).reshape(-1)[:4].tolist(),
                       x_want=micro[-1].reshape(-1)[:4].tolist()), open(out_path, 'w'))
    inst.free()

    # a data-parallel training step: every rank must issue the same all-reduces in the same order
    trainer = Instance.gpt2(lib, **CFG)
    trainer.init_params(gpt2_init(2))
    trainer.set_device(ffi.DEVICE_CUDA)
    trainer.set_optimizer(ffi.OPTIM_SGD, 1e-2)
    lib.poly_b200_set_update_averaging(1)
    calls, trace = ctypes.c_ulonglong(), ctypes.c_ulonglong()
    per_step = []
    for step in range(3):
        trainer.train_step(**trainer.gpt2_inputs(micro[step]))
        lib.poly_b200_average_trace(ctypes.byref(calls), ctypes.byref(trace))
        per_step.append([calls.value, trace.value])
    lib.poly_b200_set_update_averaging(0)
    trainer.train_step(**trainer.gpt2_inputs(micro[0]))
    lib.poly_b200_average_trace(ctypes.byref(calls), ctypes.byref(trace))
    mine = dict(per_step=per_step, after_off=calls.value, n_params=lib.poly_instance_param_count(trainer.h))
    traces = [None] * world if rank == 0 else None
    dist.gather_object(mine, traces, dst=0)
    if rank == 0:
        result = json.load(open(out_path))
        result['averaging'] = traces
        json.dump(result, open(out_path, 'w'))
    trainer.free()
    lib.poly_b200_comm_destroy()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
