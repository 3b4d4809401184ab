/*
 * pb_shard.c -- batch-sharded forward: this rank's share of a global batch run as
 * micro-batches through one instance, each micro-batch's result gathered to a root
 * rank behind the next micro-batch's compute.
 *
 * polygrad's graphs have static shapes: a GPT-2 instance built with max_batch = 8
 * runs 8 sequences per forward (reference src/modelzoo/models/gpt2.c:173-318) and
 * poly_instance_forward (src/instance.c:830) runs exactly one such batch on one
 * device.  A global batch of 64 sequences over N ranks is therefore 64 / (8 N)
 * forwards of the same plan per rank.  Batch rows never interact in the forward
 * graph, so ranks exchange nothing while computing; the only collective is the
 * gather of the results (pb_comm.cu), which this loop overlaps with compute:
 * forward i+1 is enqueued right after the snapshot of forward i's output.
 *
 * Global order of micro-batches: round-robin over ranks, micro-batch i of rank r is
 * number i * world + r; on the root its result lies at
 * root_dst + (i * world + r) * out_bytes.
 */
#include "instance.h"
#include "../../../include/poly_b200.h"
#include <stdio.h>
#include <string.h>

int poly_b200_shard_micro_index(int rank, int world, int i) { return i * world + rank; }

int poly_b200_forward_microbatches(PolyInstance *inst, const char *input_name, const float *const *inputs, int n_micro,
                                   int out_buf, size_t out_bytes, void *root_dst, int root, int gather) {
  if (!inst || !input_name || !inputs || n_micro < 0 || out_buf < 0) return -1;
  const int rank = poly_b200_comm_rank() < 0 ? 0 : poly_b200_comm_rank();
  const int world = poly_b200_comm_world() < 1 ? 1 : poly_b200_comm_world();
  unsigned long long out_dev = 0;
  for (int i = 0; i < n_micro; i++) {
    PolyIOBinding io;
    io.name = input_name;
    io.data = (float *)inputs[i];
    if (poly_instance_forward(inst, &io, 1) != 0) return -1;
    if (!gather) continue;
    if (!out_dev) {
      /* where the instance keeps its output on the device: a one-element readback tells */
      float probe;
      if (poly_instance_readback_buf(inst, out_buf, &probe, sizeof probe) != 0) return -1;
      out_dev = poly_b200_last_dtoh_src();
      if (!out_dev) return -1;
    }
    char *dst = root_dst ? (char *)root_dst + (size_t)poly_b200_shard_micro_index(0, world, i) * out_bytes : NULL;
    if (poly_b200_gather_async((const void *)(uintptr_t)out_dev, out_bytes, rank == root ? dst : NULL, root) != 0) return -1;
  }
  return 0;
}
