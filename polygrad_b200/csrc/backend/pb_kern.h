/*
 * pb_kern.h -- analysis view of one scheduled polygrad kernel.
 *
 * The scheduler hands each kernel to the CUDA backend as a SINK over
 * END(..., RANGE) wrappers around STORE(INDEX(PARAM, idx), value)
 * (reference: src/exec_plan.c:529-533 passes the scheduled root to
 * poly_linearize_cuda; src/rangeify.c:1527-1639 builds that root).  After one
 * poly_symbolic_simple() rewrite the index expressions are canonical and every
 * reduction is still a single REDUCE node, which is the form analysed here.
 *
 * Only pb_outline.c creates UOps (kernels cut out of a scheduled kernel); everything
 * else reads the kernel and never rewrites it.
 */
#ifndef PB_KERN_H
#define PB_KERN_H

#include "polygrad.h"
#include <stdint.h>
#include <stdbool.h>
#include <stddef.h>

#define PB_MAX_RANGES 48
#define PB_MAX_PARAMS 64
#define PB_MAX_VARS   16
#define PB_MAX_STORES 8
#define PB_MAX_AXES   12

/* ── growable string ─────────────────────────────────────────────────── */
typedef struct { char *s; size_t n, cap; } PbStr;
void pb_str_init(PbStr *b);
void pb_str_free(PbStr *b);
void pb_str_printf(PbStr *b, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
void pb_str_puts(PbStr *b, const char *s);
char *pb_str_take(PbStr *b); /* returns malloc'd buffer, resets b */

/* ── node table ──────────────────────────────────────────────────────── */
typedef struct {
  PolyUOp *u;
  uint64_t deps;     /* bit r set: value depends on range r (REDUCE removes its own ranges) */
  int n_uses;        /* number of distinct parents */
  int only_parent;   /* node index of the parent when n_uses == 1 */
  bool has_reduce;   /* subtree contains a REDUCE */
} PbNode;

typedef struct {
  PolyUOp *u;        /* STORE */
  PolyUOp *index;    /* INDEX(PARAM, idx[, gate]) */
  PolyUOp *value;
  int param;         /* PARAM.arg.i of the destination */
  int loop[PB_MAX_AXES]; /* range ids closed by the END chain, outermost END last */
  int n_loop;
} PbStore;

typedef struct {
  PolyUOp *sink;
  PbNode *nodes; int n_nodes, cap_nodes;     /* topological order (sources first) */
  PolyUOp **map_keys; int *map_vals; int map_cap;

  PolyUOp *ranges[PB_MAX_RANGES]; int n_ranges;
  int64_t  extent[PB_MAX_RANGES];             /* -1 when the bound is a DEFINE_VAR */
  int      extent_var[PB_MAX_RANGES];         /* var index when extent == -1 */
  bool     is_reduce[PB_MAX_RANGES];

  PolyUOp *params[PB_MAX_PARAMS]; int n_params; /* indexed by PARAM.arg.i */
  PolyUOp *vars[PB_MAX_VARS]; int n_vars;

  PbStore stores[PB_MAX_STORES]; int n_stores;
  int n_reduce_nodes;
  bool uses_half, uses_bf16, uses_f64;
  char err[256];
} PbKern;

/* Build the table.  Returns 0, or -1 with k->err set. */
int  pb_kern_build(PbKern *k, PolyUOp *sink);
void pb_kern_free(PbKern *k);
int  pb_kern_node(const PbKern *k, PolyUOp *u);   /* node index or -1 */
int  pb_kern_range_id(const PbKern *k, PolyUOp *r);

/* Evaluate an integer index expression at a point (vals[r] = value of range r,
 * var_vals[v] = value of DEFINE_VAR v).  Returns false when the tree holds an
 * op the evaluator does not model. */
bool pb_eval_int(const PbKern *k, PolyUOp *e, const int64_t *vals,
                 const int64_t *var_vals, int64_t *out);

/* An index expression fitted as offset + sum(stride[r] * range r). */
typedef struct {
  bool ok;                 /* fitted and verified */
  int64_t offset;
  int64_t stride[PB_MAX_RANGES];
} PbAffine;

/* Fit e over the ranges in `mask`; verification samples corners, full axis
 * lines and random interior points.  Ranges with var extents use the var's
 * max value. */
void pb_fit_affine(const PbKern *k, PolyUOp *e, uint64_t mask, PbAffine *out);

/* ── virtual axes: a kernel range, or one factor of a split range ────── */
typedef struct {
  int range;        /* kernel range id */
  int64_t extent;   /* extent of this factor */
  int64_t mult;     /* contribution to the range value: value += x * mult */
  bool reduce;
} VAxis;

typedef struct {
  bool ok;
  int64_t offset;
  int64_t stride[2 * PB_MAX_AXES];
} VFit;

/* Build virtual axes for the ranges in `mask` such that every expression in
 * exprs[] is affine in them (pb_classify.c); va needs 2 * PB_MAX_AXES entries. */
bool pb_find_axes(const PbKern *k, uint64_t mask, PolyUOp **exprs, int n_exprs,
                  VAxis *va, int *nva, VFit *fits);

/* c as an equality test of two values, in any of the forms the frontend produces (pb_classify.c). */
bool pb_match_equal(PolyUOp *c, PolyUOp **a, PolyUOp **b);

/* C type used in generated code for a scalar dtype (NULL if unsupported). */
const char *pb_ctype(PolyDType dt);

/* ── renderers (pb_codegen.c) ────────────────────────────────────────── */
/* Render the kernel as CUDA C for run-time compilation, preceded by the
 * "//PB200" header lines the runtime parses.  Returns malloc'd text or NULL. */
char *pb_render_jit(PbKern *k, const char *fn_name);
char *pb_render_elementwise_bf16(PbKern *k);

/* Several kernels of one plan rendered as one row-wise kernel: reductions over
 * the same contiguous axis feed later kernels of the chain through registers
 * instead of memory (softmax: max, sum of exp, normalise; layernorm: mean,
 * variance, normalise), and elementwise producers are evaluated in place. */
enum { PB_FUSE_PRODUCER = 0, PB_FUSE_PHASE = 1, PB_FUSE_FINAL = 2 };
typedef struct {
  PbKern *k;
  const int *slot;     /* plan slot of each kernel parameter */
  int role;
  bool keep_out;       /* a producer whose result is also read outside the chain: it is stored as well */
} PbFuseIn;
typedef struct {
  int n_params;
  int slot[PB_MAX_PARAMS];
  char rw[PB_MAX_PARAMS + 1];
} PbFuseOut;
/* in[] in execution order, the final kernel last.  out_bf16: store the result as
 * bfloat16 (for a buffer only tensor-core contractions read).  NULL if the chain
 * does not have the required shape. */
char *pb_render_rowfused(PbFuseIn *in, int n, bool out_bf16, PbFuseOut *out);

/* ── pattern lowerings (pb_classify.c) ───────────────────────────────── */
/* Try to express the kernel as one of the precompiled kernels (GEMM, row
 * gather, strided copy).  Returns malloc'd header-only text, or NULL when the
 * kernel is not of that class. */
char *pb_classify_aot(PbKern *k, const char *fn_name);

#endif
