/*
 * pb_fuse.c -- passes over a CUDA plan's step list.
 *
 * polygrad's model builders put a CONTIGUOUS realize barrier after almost every
 * op (reference: src/modelzoo/models/gpt2.c:38, 362-498), so a GPT-2 layer is 26
 * kernels, 4 of which only copy a buffer to a new one.  The scheduler's kernel
 * split is kept -- results must stay those of the reference kernels -- but a
 * plan may skip work whose result is already in memory:
 *
 *   copy elision   a kernel that stores in[i] to out[i] for every i of two
 *                  same-sized buffers is dropped and `out` becomes a second
 *                  name for `in` (or the producer of `in` writes `out`
 *                  directly when `out` is a bound buffer).
 */
#include "pb_plan.h"
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct { int writers, readers, first_write, last_write, last_read; } SlotUse;

static void slot_usage(const PbPlan *p, SlotUse *u) {
  for (int i = 0; i < p->n_slots; i++) { u[i].writers = u[i].readers = 0; u[i].first_write = u[i].last_write = u[i].last_read = -1; }
  for (int s = 0; s < p->n_steps; s++) {
    const PbStep *st = &p->steps[s];
    if (st->dead) continue;
    for (int a = 0; a < st->n_params; a++) {
      int sl = pb_plan_resolve(p, st->slot[a]);
      char m = st->rw[a];
      if (m == 'r' || m == 'b') { u[sl].readers++; u[sl].last_read = s; }
      if (m == 'w' || m == 'W' || m == 'b') { u[sl].writers++; if (u[sl].first_write < 0) u[sl].first_write = s; u[sl].last_write = s; }
    }
  }
}

/* Is this step `out[i] = in[i]` over all of two equally sized buffers?  Returns
 * the parameter positions of out and in. */
static bool is_identity_copy(const PbStep *st, int *p_out, int *p_in) {
  if (st->precompiled || st->n_params != 2 || st->n_vars) return false;
  PbKern k;
  if (pb_kern_build(&k, st->sink) != 0) { pb_kern_free(&k); return false; }
  bool ok = false;
  if (k.n_stores == 1 && k.n_reduce_nodes == 0) {
    PbStore *s = &k.stores[0];
    PolyUOp *v = s->value;
    if (s->index->n_src == 2 && v->op == POLY_OP_LOAD && v->src[0]->op == POLY_OP_INDEX && v->src[0]->n_src == 2 &&
        v->src[0]->src[0]->op == POLY_OP_PARAM && v->src[0]->src[1] == s->index->src[1]) {
      int po = s->param, pi = (int)v->src[0]->src[0]->arg.i;
      PolyDType a = k.params[po]->dtype, b = k.params[pi]->dtype;
      if (po != pi && po < 2 && pi < 2 && a.priority == b.priority && a.bitsize == b.bitsize && a.ptr_size == b.ptr_size &&
          st->rw[po] == 'W') { *p_out = po; *p_in = pi; ok = true; }
    }
  }
  pb_kern_free(&k);
  return ok;
}

static int elide_copies(PbPlan *p) {
  int removed = 0;
  SlotUse *u = malloc(sizeof(SlotUse) * (size_t)p->n_slots);
  for (int s = 0; s < p->n_steps; s++) {
    PbStep *st = &p->steps[s];
    if (st->dead) continue;
    int po, pi;
    if (!is_identity_copy(st, &po, &pi)) continue;
    slot_usage(p, u);
    int out = pb_plan_resolve(p, st->slot[po]), in = pb_plan_resolve(p, st->slot[pi]);
    if (out == in || p->slot_bytes[out] != p->slot_bytes[in]) continue;
    if (p->slot_inter[out] && u[out].writers == 1 && u[in].last_write < s) {
      /* readers of `out` read `in`; nothing writes `in` afterwards */
      p->slot_alias[out] = in;
      st->dead = true; removed++;
    } else if (!p->slot_inter[out] && p->slot_inter[in] && u[in].writers == 1 && u[in].readers == 1 &&
               u[out].writers == 1 && u[out].readers == 0) {
      /* the only producer of `in` can write the bound buffer directly */
      const PbStep *w = &p->steps[u[in].first_write];
      bool whole = false;
      for (int a = 0; a < w->n_params; a++) if (pb_plan_resolve(p, w->slot[a]) == in && w->rw[a] == 'W') whole = true;
      if (!whole) continue;
      p->slot_alias[in] = out;
      st->dead = true; removed++;
    }
  }
  free(u);
  return removed;
}

void pb_plan_fuse(PbPlan *p) {
  int copies = elide_copies(p);
  if (getenv("POLY_B200_DEBUG")) fprintf(stderr, "pb_fuse: %d copy kernels elided\n", copies);
}
