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

/* ── row fusion ──────────────────────────────────────────────────────── */
/* A chain ends in a kernel F and contains the kernels whose only purpose is to
 * feed it: row reductions (their one-value-per-row results stay in registers)
 * and elementwise producers (evaluated in place).  poly_softmax and
 * poly_layernorm (reference: src/frontend.c:1131-1159, 3585-3625) each schedule
 * as two reductions plus an elementwise kernel; with the caller's scale/mask or
 * affine kernel around them that is 3-4 passes over the tensor, here one. */
#define CHAIN_MAX 8

static bool step_fusable(const PbStep *st) { return !st->dead && !st->precompiled && st->n_vars == 0 && st->sink; }

static bool step_reads(const PbPlan *p, const PbStep *st, int slot) {
  for (int a = 0; a < st->n_params; a++)
    if ((st->rw[a] == 'r' || st->rw[a] == 'b') && pb_plan_resolve(p, st->slot[a]) == slot) return true;
  return false;
}
static bool step_writes(const PbPlan *p, const PbStep *st, int slot) {
  for (int a = 0; a < st->n_params; a++)
    if ((st->rw[a] == 'w' || st->rw[a] == 'W' || st->rw[a] == 'b') && pb_plan_resolve(p, st->slot[a]) == slot) return true;
  return false;
}
static int step_out_slot(const PbPlan *p, const PbStep *st) {
  for (int a = 0; a < st->n_params; a++)
    if (st->rw[a] == 'W' || st->rw[a] == 'w' || st->rw[a] == 'b') return pb_plan_resolve(p, st->slot[a]);
  return -1;
}

static int fuse_rows(PbPlan *p) {
  int fused = 0;
  SlotUse *u = malloc(sizeof(SlotUse) * (size_t)p->n_slots);
  for (int f = 0; f < p->n_steps; f++) {
    if (!step_fusable(&p->steps[f])) continue;
    slot_usage(p, u);
    int mem[CHAIN_MAX]; int nm = 0;
    mem[nm++] = f;
    /* closure over single-writer intermediates read by members */
    for (int i = 0; i < nm; i++) {
      const PbStep *m = &p->steps[mem[i]];
      for (int a = 0; a < m->n_params; a++) {
        if (m->rw[a] != 'r') continue;
        int sl = pb_plan_resolve(p, m->slot[a]);
        if (!p->slot_inter[sl] || u[sl].writers != 1) continue;
        int w = u[sl].first_write;
        if (w >= f || !step_fusable(&p->steps[w])) continue;
        bool have = false;
        for (int j = 0; j < nm; j++) if (mem[j] == w) have = true;
        if (!have && nm < CHAIN_MAX) mem[nm++] = w;
      }
    }
    /* drop members whose result is also needed outside the chain */
    for (bool changed = true; changed;) {
      changed = false;
      for (int i = 1; i < nm; i++) {
        int sl = step_out_slot(p, &p->steps[mem[i]]);
        bool outside = sl < 0 || !p->slot_inter[sl];
        for (int s = 0; s < p->n_steps && !outside; s++) {
          if (p->steps[s].dead || !step_reads(p, &p->steps[s], sl)) continue;
          bool in_chain = false;
          for (int j = 0; j < nm; j++) if (mem[j] == s) in_chain = true;
          if (!in_chain) outside = true;
        }
        if (outside) { mem[i] = mem[nm - 1]; nm--; changed = true; break; }
      }
    }
    if (nm < 2) continue;
    /* order by step, final last */
    for (int i = 1; i < nm; i++) for (int j = i; j > 1 && mem[j] < mem[j - 1]; j--) { int t = mem[j]; mem[j] = mem[j - 1]; mem[j - 1] = t; }
    int order[CHAIN_MAX]; int no = 0;
    for (int i = 1; i < nm; i++) order[no++] = mem[i];
    order[no++] = f;
    /* nothing outside the chain may overwrite what the chain reads, between its first member and F */
    bool hazard = false;
    for (int s = order[0]; s < f && !hazard; s++) {
      bool in_chain = false;
      for (int j = 0; j < no; j++) if (order[j] == s) in_chain = true;
      if (in_chain || p->steps[s].dead) continue;
      for (int j = 0; j < no && !hazard; j++) {
        const PbStep *m = &p->steps[order[j]];
        for (int a = 0; a < m->n_params; a++)
          if (m->rw[a] == 'r' && step_writes(p, &p->steps[s], pb_plan_resolve(p, m->slot[a]))) hazard = true;
      }
    }
    if (hazard) continue;

    PbKern kerns[CHAIN_MAX]; PbFuseIn in[CHAIN_MAX]; int slots[CHAIN_MAX][PB_MAX_PARAMS];
    bool built = true; int n_phase = 0;
    int nb = 0;
    for (int j = 0; j < no && built; j++) {
      PbStep *m = &p->steps[order[j]];
      if (pb_kern_build(&kerns[j], m->sink) != 0) { pb_kern_free(&kerns[j]); built = false; break; }
      nb = j + 1;
      for (int a = 0; a < PB_MAX_PARAMS; a++) slots[j][a] = -1;
      for (int a = 0; a < m->n_params; a++) slots[j][a] = pb_plan_resolve(p, m->slot[a]);
      in[j].k = &kerns[j]; in[j].slot = slots[j];
      in[j].role = (j == no - 1) ? PB_FUSE_FINAL : (kerns[j].n_reduce_nodes ? PB_FUSE_PHASE : PB_FUSE_PRODUCER);
      if (in[j].role == PB_FUSE_PHASE) n_phase++;
    }
    char *text = NULL; PbFuseOut fo;
    if (built && n_phase > 0) text = pb_render_rowfused(in, no, false, &fo);
    for (int j = 0; j < nb; j++) pb_kern_free(&kerns[j]);
    if (!text) continue;
    char name[64]; snprintf(name, sizeof name, "rowfused_k%d", p->steps[f].item);
    if (getenv("POLY_DUMP_KERNELS")) fprintf(stderr, "=== CUDA KERNEL %s ===\n%s\n=== END ===\n", name, text);
    PolyCudaProgram *prog = poly_compile_cuda(text, name);
    if (!prog) { free(text); continue; }
    PbStep *fs = &p->steps[f];
    poly_cuda_program_destroy(fs->prog); free(fs->text);
    fs->prog = prog; fs->text = text; fs->sink = NULL;
    fs->n_params = fo.n_params;
    for (int a = 0; a < fo.n_params; a++) { fs->slot[a] = fo.slot[a]; fs->rw[a] = fo.rw[a]; }
    fs->rw[fo.n_params] = 0;
    for (int j = 0; j < no - 1; j++) p->steps[order[j]].dead = true;
    fused += no - 1;
  }
  free(u);
  return fused;
}

void pb_plan_fuse(PbPlan *p) {
  int copies = elide_copies(p);
  int rows = 0;
  const char *e = getenv("POLY_B200_FUSE");
  if (!e || strcmp(e, "copies") != 0) rows = fuse_rows(p);
  if (getenv("POLY_B200_DEBUG")) fprintf(stderr, "pb_fuse: %d copy kernels elided, %d kernels folded into row kernels\n", copies, rows);
}
