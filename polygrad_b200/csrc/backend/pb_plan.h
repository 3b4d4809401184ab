/*
 * pb_plan.h -- the CUDA plan: a list of steps over plan slots (pb_exec_plan.c)
 * and the passes that rewrite that list (pb_fuse.c).
 */
#ifndef PB_PLAN_H
#define PB_PLAN_H

#include "pb_kern.h"
#include "exec_plan.h"
#include "frontend.h"
#include "codegen.h"
#include "../../../include/poly_b200.h"

/* One launchable step.  Steps start as one per scheduled kernel, in execution
 * order; passes may mark steps dead or replace their program. */
typedef struct {
  int item;                      /* schedule item this step came from (-1: synthesised) */
  PolyUOp *sink;                 /* the kernel, simplified (what poly_linearize_cuda returned) */
  PolyCudaProgram *prog;
  char *text;                    /* program text the program was compiled from */
  int n_params, n_vars;
  int slot[PB_MAX_PARAMS];       /* plan slot of each parameter */
  char rw[PB_MAX_PARAMS + 1];    /* 'r' read, 'w' partly written, 'W' wholly overwritten, 'b' both, '-' unused */
  int precompiled;
  bool dead;
  bool fused_rows;               /* program is a row-fused chain; chain[] lists the member steps, this one last */
  int chain[8], n_chain;
  bool chain_keep[8];            /* member whose own result is still stored by the fused kernel (read outside the chain) */
  unsigned long long dptr[PB_MAX_PARAMS];
  void *argv[PB_MAX_PARAMS];
} PbStep;

typedef struct {
  PolyCompiledPlan base;         /* polygrad code reads base.schedule (src/instance.c:158) */
  PolyCtx *ctx;
  PbStep *steps; int n_steps;
  int n_slots, n_sched_slots;    /* schedule slots first, then slots added by passes */
  int64_t *slot_bytes, *slot_off;
  int *slot_alias;               /* >= 0: this slot is another slot's storage */
  char *slot_inter;              /* intermediate (plan-owned) or external */
  void **slot_ptr;
  /* bound buffers that live in pageable host memory are run from a device copy */
  char *slot_acc;                /* per schedule slot: PB_ACC_READ | PB_ACC_WRITE over all live steps */
  void **ext_seen; char *ext_host;   /* last pointer bound to an external slot and whether it was host memory */
  unsigned long long *stage;     /* the device copy, allocated on first use */
  unsigned long long arena; int64_t arena_bytes;
  int *zero_step, *zero_slot, n_zero;
  void *graph; unsigned long long graph_epoch; void **graph_ext;
  long long graph_kernels, graph_precompiled;
  void **graph_acc_ptr; char *graph_acc_mode; int n_graph_acc;   /* accesses to bound buffers a replay reports */
  int runs, graph_failures;
  /* a plan that updates bound buffers in place (a training step): after step avg_at[i] nothing in the
   * plan writes bound float32 slot avg_slot[i] any more; sorted by step */
  int *avg_at, *avg_slot, n_avg;
} PbPlan;

enum { PB_ACC_READ = 1, PB_ACC_WRITE = 2 };

/* The plan behind a handle, NULL when the handle is one of polygrad's own plans (pb_exec_plan.c). */
PbPlan *pb_plan_of(PolyCompiledPlan *plan);

int  pb_plan_resolve(const PbPlan *p, int slot);
int  pb_plan_add_slot(PbPlan *p, int64_t bytes);
void pb_step_release(PbStep *st);

/* Rewrites the step list in place (pb_fuse.c). */
void pb_plan_fuse(PbPlan *p);
/* Does some step read a bound buffer that another step writes (an optimizer step does)? */
bool pb_plan_updates_in_place(const PbPlan *p);

/* Helpers shared by the passes. */
typedef struct { int writers, readers, first_write, last_write, last_read; } PbSlotUse;
void pb_slot_usage(const PbPlan *p, PbSlotUse *u);
bool pb_step_reads(const PbPlan *p, const PbStep *st, int slot);
bool pb_step_writes(const PbPlan *p, const PbStep *st, int slot);
const char *pb_hdr_line(const char *text, const char *key, char *buf, size_t cap);
char *pb_render_chain(const PbPlan *p, const int *order, const bool *keep, int no, bool out_bf16, PbFuseOut *fo);

/* Passes over the operands of precompiled steps (pb_operands.c): strided copies
 * folded into the consumer's strides, bfloat16 storage of contraction operands. */
void pb_plan_operands(PbPlan *p);

#endif
