/*
 * pb_outline.h -- one scheduled kernel cut into several that run one after the
 * other through temporaries (pb_outline.c).
 */
#ifndef PB_OUTLINE_H
#define PB_OUTLINE_H

#include "pb_kern.h"

#define PB_MAX_TEMPS  12
#define PB_MAX_PIECES 16

typedef struct {
  PolyUOp *sink;                      /* a kernel tree like a scheduled one */
  int n_params;
  int param_src[PB_MAX_PARAMS];       /* parameter i is the parent's parameter param_src[i] (>= 0) or temporary -(param_src[i] + 1) */
  bool must_be_contraction;           /* the cut only pays if this piece is recognised as one */
} PbPiece;

/* Cuts the kernel under `sink` (already simplified).  Returns the number of
 * pieces written (in execution order, the last one writes the parent's
 * output), or 0 when the kernel is left as it is.  temp_numel[t] receives the
 * float32 element count of temporary t. */
int pb_outline(PolyCtx *ctx, PolyUOp *sink, PbPiece *pieces, int cap, int64_t *temp_numel, int *n_temps);

#endif
