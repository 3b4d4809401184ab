/*
 * pb_outline.c -- cutting one scheduled kernel into several.
 *
 * polygrad's scheduler fuses as much as it can into a kernel.  In backward
 * graphs that produces kernels a contraction unit cannot take as they are:
 *
 *   - a contraction whose operand is computed on the fly: a weight gradient
 *     dW = sum_t (g1[t,i] + g2[t,i]) * x[t,j] where the scheduler folded the sum
 *     of two gradient contributions into the reduction, or the embedding
 *     gradient sum_t onehot(tok[t] == v) * g[t,d]
 *     (reference: the backward rules of src/autograd.c applied to
 *     src/modelzoo/models/gpt2.c, fused by src/sched/rangeify.c);
 *   - several reductions in one kernel: the tied embedding's gradient is the sum
 *     of the head's and the lookup's, followed by the parameter update
 *     (src/instance.c:1157-1162), all in one kernel.
 *
 * The reference renders such a kernel as one thread per output with serial
 * loops over the reduction (src/render_cuda.c); so does the general renderer
 * here.  This pass instead cuts the kernel into pieces that run one after the
 * other through temporaries:
 *
 *   1. a computed operand of a contraction becomes its own elementwise kernel,
 *      written over exactly the (virtual) axes it depends on, and the
 *      contraction reads the temporary with a plain load;
 *   2. if the kernel then still is not a single contraction with a known
 *      epilogue, each contraction is cut out into a kernel that writes a
 *      temporary laid out like the kernel's output, and the remainder reads
 *      those temporaries elementwise.  A contraction that only counts inside a
 *      window of an output axis -- the gradients of q, k and v written side by
 *      side into one buffer: where(0 <= c - 96 < 48, sum(...), 0) + ... -- is
 *      computed over that window alone (the axis is replaced by a shorter one,
 *      shifted), and the remainder reads the temporary at the shifted position
 *      under the same condition.
 *
 * The pieces are ordinary kernel trees (SINK over END over STORE), so the
 * classifier and the renderers treat them like scheduled kernels.  The caller
 * keeps the cut only if every contraction in it is then recognised.
 */
#include "pb_outline.h"
#include "pat.h"
#include "codegen.h"
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define DBG(...) do { if (getenv("POLY_B200_DEBUG")) { fprintf(stderr, "pb_outline: " __VA_ARGS__); fputc('\n', stderr); } } while (0)

/* ── substitution map ────────────────────────────────────────────────── */
typedef struct { PolyUOp **key, **val; int cap, n; } Sub;

static size_t sub_slot(const void *p, int cap) {
  uintptr_t x = (uintptr_t)p; x ^= x >> 15; x *= (uintptr_t)0x9E3779B97F4A7C15ull; x ^= x >> 31;
  return (size_t)x & (size_t)(cap - 1);
}
static PolyUOp *sub_get(const Sub *m, PolyUOp *u) {
  if (!m->cap) return NULL;
  for (size_t i = sub_slot(u, m->cap);; i = (i + 1) & (size_t)(m->cap - 1)) {
    if (!m->key[i]) return NULL;
    if (m->key[i] == u) return m->val[i];
  }
}
static void sub_put(Sub *m, PolyUOp *u, PolyUOp *v) {
  if ((m->n + 1) * 2 > m->cap) {
    int ncap = m->cap ? m->cap * 2 : 256;
    PolyUOp **nk = calloc((size_t)ncap, sizeof *nk), **nv = calloc((size_t)ncap, sizeof *nv);
    for (int i = 0; i < m->cap; i++) if (m->key[i]) {
      size_t j = sub_slot(m->key[i], ncap);
      while (nk[j]) j = (j + 1) & (size_t)(ncap - 1);
      nk[j] = m->key[i]; nv[j] = m->val[i];
    }
    free(m->key); free(m->val); m->key = nk; m->val = nv; m->cap = ncap;
  }
  size_t j = sub_slot(u, m->cap);
  while (m->key[j] && m->key[j] != u) j = (j + 1) & (size_t)(m->cap - 1);
  if (!m->key[j]) m->n++;
  m->key[j] = u; m->val[j] = v;
}
static void sub_free(Sub *m) { free(m->key); free(m->val); memset(m, 0, sizeof *m); }

/* u with every node that has an entry in m replaced by it (sources first) */
static PolyUOp *rebuild(PolyCtx *ctx, Sub *m, PolyUOp *u) {
  PolyUOp *got = sub_get(m, u);
  if (got) return got;
  PolyUOp *src[64];
  bool changed = false;
  if (u->n_src > 64) return NULL;
  for (int i = 0; i < u->n_src; i++) {
    src[i] = rebuild(ctx, m, u->src[i]);
    if (!src[i]) return NULL;
    if (src[i] != u->src[i]) changed = true;
  }
  PolyUOp *r = changed ? poly_uop(ctx, u->op, u->dtype, src, u->n_src, u->arg) : u;
  if (r) sub_put(m, u, r);
  return r;
}

/* ── small builders ──────────────────────────────────────────────────── */
typedef struct {
  PolyCtx *ctx;
  PbKern *k;
  PolyDType t_int;        /* dtype of the kernel's index arithmetic */
  PolyUOp *end_like;      /* an END of the kernel: dtype and arg for new ones */
} Cut;

static PolyUOp *ci(Cut *c, int64_t v) { return poly_uop0(c->ctx, POLY_OP_CONST, c->t_int, poly_arg_int(v)); }
static PolyUOp *ibin(Cut *c, PolyOps op, PolyUOp *a, PolyUOp *b) { return poly_uop2(c->ctx, op, c->t_int, a, b, poly_arg_none()); }
static PolyUOp *iadd(Cut *c, PolyUOp *a, PolyUOp *b) { return !a ? b : !b ? a : ibin(c, POLY_OP_ADD, a, b); }
static PolyUOp *iscale(Cut *c, PolyUOp *a, int64_t f) { return f == 1 ? a : ibin(c, POLY_OP_MUL, a, ci(c, f)); }

static bool is_f32(PolyDType d) { return !d.is_ptr && d.count == 1 && d.priority == 13; }
static bool is_plain_load(PolyUOp *u) {
  return u->op == POLY_OP_LOAD && u->n_src == 1 && u->src[0]->op == POLY_OP_INDEX && u->src[0]->n_src == 2 &&
         u->src[0]->src[0]->op == POLY_OP_PARAM;
}
static bool const_f32(PolyUOp *u) { return u->op == POLY_OP_CONST && is_f32(u->dtype); }
/* u without a float constant factor and without a widening cast */
static PolyUOp *operand_core(PolyUOp *u) {
  for (int guard = 0; guard < 4; guard++) {
    if (u->op == POLY_OP_MUL && const_f32(u->src[1])) u = u->src[0];
    else if (u->op == POLY_OP_MUL && const_f32(u->src[0])) u = u->src[1];
    else if (u->op == POLY_OP_CAST && is_f32(u->dtype) && u->src[0]->op == POLY_OP_LOAD) u = u->src[0];
    else break;
  }
  return u;
}

static PolyUOp *param_like(Cut *c, PolyUOp *like, int index, int64_t numel) {
  PolyDType dt = like->dtype;
  if (numel >= 0) dt.ptr_size = numel;
  return poly_uop0(c->ctx, POLY_OP_PARAM, dt, poly_arg_int(index));
}

/* SINK(END(...END(STORE(INDEX(dst, idx), value), r0)..., rn)) */
static PolyUOp *wrap_store(Cut *c, PolyUOp *dst_param, PolyUOp *idx, PolyUOp *value, PolyUOp **ranges, int n_ranges) {
  PbStore *st = &c->k->stores[0];
  PolyUOp *index = poly_uop2(c->ctx, POLY_OP_INDEX, st->index->dtype, dst_param, idx, st->index->arg);
  PolyUOp *cur = poly_uop2(c->ctx, POLY_OP_STORE, st->u->dtype, index, value, st->u->arg);
  for (int i = 0; i < n_ranges && cur; i++)
    cur = poly_uop2(c->ctx, POLY_OP_END, c->end_like->dtype, cur, ranges[i], c->end_like->arg);
  return cur ? poly_uop1(c->ctx, POLY_OP_SINK, c->k->sink->dtype, cur, c->k->sink->arg) : NULL;
}

/* ── what an expression is made of ───────────────────────────────────── */
typedef struct { PolyUOp *ld[16]; int n; bool bad; } Loads;

static void gather_loads(PbKern *k, PolyUOp *u, Loads *out, Sub *seen) {
  if (out->bad || sub_get(seen, u)) return;
  sub_put(seen, u, u);
  switch (u->op) {
  case POLY_OP_LOAD:
    if (!is_plain_load(u) || out->n >= 16) { out->bad = true; return; }
    out->ld[out->n++] = u;
    return;
  case POLY_OP_CONST: return;
  case POLY_OP_RANGE: case POLY_OP_DEFINE_VAR: case POLY_OP_REDUCE: case POLY_OP_PARAM: case POLY_OP_INDEX:
    out->bad = true; return;       /* a range used as a value (a mask from indices), a nested reduction */
  default: break;
  }
  for (int i = 0; i < u->n_src; i++) gather_loads(k, u->src[i], out, seen);
}

/* ── step 1: a computed operand becomes a temporary ──────────────────── */
typedef struct {
  PolyUOp *sink;          /* the kernel that fills the temporary */
  int64_t numel;
  int parent_param[PB_MAX_PARAMS]; int n_params;   /* its parameters 1.. in terms of the parent's */
  PolyUOp *read_index;    /* where the parent reads it, over the parent's ranges */
} Operand;

/* e may be an expression built here (not a node of the kernel); deps_of is a node of the kernel
 * that depends on the same ranges. */
static bool materialize(Cut *c, PolyUOp *e, PolyUOp *deps_of, Operand *out) {
  PbKern *k = c->k;
  memset(out, 0, sizeof *out);
  if (!is_f32(e->dtype)) return false;
  Loads ls = { .n = 0 };
  Sub seen = {0};
  gather_loads(k, e, &ls, &seen);
  sub_free(&seen);
  if (ls.bad || ls.n == 0) { DBG("operand: not loads and arithmetic only"); return false; }
  const uint64_t mask = k->nodes[pb_kern_node(k, deps_of)].deps;
  for (int r = 0; r < k->n_ranges; r++) if ((mask >> r & 1) && k->extent[r] < 0) return false;
  PolyUOp *exprs[16];
  for (int i = 0; i < ls.n; i++) exprs[i] = ls.ld[i]->src[0]->src[1];
  VAxis va[2 * PB_MAX_AXES]; int nva = 0; VFit fit[16];
  if (!pb_find_axes(k, mask, exprs, ls.n, va, &nva, fit)) { DBG("operand: indices not affine"); return false; }
  /* every load must stay inside its buffer over the whole index space: the temporary is
   * filled for every point of it, also those the parent would have masked away */
  for (int i = 0; i < ls.n; i++) {
    int64_t lo = fit[i].offset, hi = fit[i].offset;
    for (int a = 0; a < nva; a++) { int64_t s = fit[i].stride[a] * (va[a].extent - 1); if (s > 0) hi += s; else lo += s; }
    const int64_t numel = k->params[ls.ld[i]->src[0]->src[0]->arg.i]->dtype.ptr_size;
    if (lo < 0 || (numel >= 0 && hi >= numel)) { DBG("operand: a load leaves its buffer"); return false; }
  }
  /* the axes the operand really depends on, laid out like the largest buffer it reads (so that the
   * kernel filling it reads that buffer in order); axes that buffer does not have go outermost */
  int big = 0;
  for (int i = 1; i < ls.n; i++)
    if (k->params[ls.ld[i]->src[0]->src[0]->arg.i]->dtype.ptr_size > k->params[ls.ld[big]->src[0]->src[0]->arg.i]->dtype.ptr_size) big = i;
  int ax[2 * PB_MAX_AXES]; int64_t key[2 * PB_MAX_AXES]; int na = 0;
  int64_t numel = 1;
  for (int a = 0; a < nva; a++) {
    if (va[a].extent <= 1) continue;
    int64_t best = INT64_MAX;
    for (int i = 0; i < ls.n; i++) { int64_t s = llabs(fit[i].stride[a]); if (s && s < best) best = s; }
    if (best == INT64_MAX) continue;
    ax[na] = a;
    key[na] = fit[big].stride[a] ? llabs(fit[big].stride[a]) : (INT64_MAX / 2 + best);
    na++;
    numel *= va[a].extent;
    if (numel >= ((int64_t)1 << 30)) { DBG("operand: temporary too large"); return false; }
  }
  if (na == 0 || na > PB_MAX_AXES) return false;
  for (int i = 1; i < na; i++)
    for (int j = i; j > 0 && key[j - 1] < key[j]; j--) {
      int t = ax[j]; ax[j] = ax[j - 1]; ax[j - 1] = t;
      int64_t tk = key[j]; key[j] = key[j - 1]; key[j - 1] = tk;
    }
  int64_t rm[2 * PB_MAX_AXES];
  { int64_t s = 1; for (int i = na - 1; i >= 0; i--) { rm[i] = s; s *= va[ax[i]].extent; } }

  /* the kernel that fills it */
  PolyUOp *ranges[PB_MAX_AXES];
  PolyUOp *idx_t = NULL;
  for (int i = 0; i < na; i++) {
    ranges[i] = poly_uop1(c->ctx, POLY_OP_RANGE, c->t_int, ci(c, va[ax[i]].extent), poly_arg_range(i, POLY_AXIS_LOOP));
    idx_t = iadd(c, idx_t, iscale(c, ranges[i], rm[i]));
  }
  if (!idx_t) idx_t = ci(c, 0);
  Sub m = {0};
  int new_of_parent[PB_MAX_PARAMS];
  for (int p = 0; p < PB_MAX_PARAMS; p++) new_of_parent[p] = -1;
  out->n_params = 0;
  for (int i = 0; i < ls.n; i++) {
    PolyUOp *ld = ls.ld[i], *index = ld->src[0];
    const int pp = (int)index->src[0]->arg.i;
    if (new_of_parent[pp] < 0) { new_of_parent[pp] = 1 + out->n_params; out->parent_param[out->n_params++] = pp; }
    PolyUOp *np = param_like(c, index->src[0], new_of_parent[pp], -1);
    PolyUOp *ni = fit[i].offset ? ci(c, fit[i].offset) : NULL;
    for (int j = 0; j < na; j++) if (fit[i].stride[ax[j]]) ni = iadd(c, ni, iscale(c, ranges[j], fit[i].stride[ax[j]]));
    if (!ni) ni = ci(c, 0);
    PolyUOp *nindex = poly_uop2(c->ctx, POLY_OP_INDEX, index->dtype, np, ni, index->arg);
    sub_put(&m, ld, poly_uop1(c->ctx, POLY_OP_LOAD, ld->dtype, nindex, ld->arg));
  }
  PolyUOp *value = rebuild(c->ctx, &m, e);
  sub_free(&m);
  if (!value) return false;
  PolyUOp *dst = param_like(c, k->params[k->stores[0].param], 0, numel);
  out->sink = wrap_store(c, dst, idx_t, value, ranges, na);
  out->numel = numel;
  if (!out->sink) return false;

  /* where the parent finds an element: the same row-major position, from its own ranges */
  PolyUOp *ridx = NULL;
  for (int i = 0; i < na; i++) {
    const VAxis *v = &va[ax[i]];
    PolyUOp *t = k->ranges[v->range];
    if (v->mult > 1) t = ibin(c, POLY_OP_IDIV, t, ci(c, v->mult));
    if (v->mult * v->extent < k->extent[v->range]) t = ibin(c, POLY_OP_MOD, t, ci(c, v->extent));
    ridx = iadd(c, ridx, iscale(c, t, rm[i]));
  }
  out->read_index = ridx ? ridx : ci(c, 0);
  return true;
}

/* ── the pass ────────────────────────────────────────────────────────── */
static void collect_params(PolyUOp *u, Sub *seen, bool *used) {
  if (sub_get(seen, u)) return;
  sub_put(seen, u, u);
  if (u->op == POLY_OP_PARAM) { if (u->arg.i >= 0 && u->arg.i < PB_MAX_PARAMS) used[u->arg.i] = true; return; }
  for (int i = 0; i < u->n_src; i++) collect_params(u->src[i], seen, used);
}

/* `root` with its parameters renumbered first, first + 1, ... in order of their old numbers;
 * old_of_new[] receives the old number of each new one (entries below `first` are not touched). */
static PolyUOp *renumber_params(Cut *c, PolyUOp *root, int first, int *old_of_new, int *n_new) {
  bool used[PB_MAX_PARAMS] = {false};
  Sub seen = {0};
  collect_params(root, &seen, used);
  sub_free(&seen);
  Sub pm = {0};
  int n = first;
  for (int p = 0; p < PB_MAX_PARAMS; p++) {
    if (!used[p]) continue;
    if (n >= PB_MAX_PARAMS) { sub_free(&pm); return NULL; }
    PolyUOp *old = NULL;
    for (int j = 0; j < c->k->n_nodes && !old; j++)
      if (c->k->nodes[j].u->op == POLY_OP_PARAM && c->k->nodes[j].u->arg.i == p) old = c->k->nodes[j].u;
    if (!old) { sub_free(&pm); return NULL; }
    sub_put(&pm, old, param_like(c, old, n, -1));
    old_of_new[n++] = p;
  }
  PolyUOp *r = rebuild(c->ctx, &pm, root);
  sub_free(&pm);
  *n_new = n;
  return r;
}

/* Is this reduction a contraction: a sum of products in which one factor walks output axes the
 * other does not, and the other way round, and both walk the reduction?  (A row statistic,
 * sum_k a[row,k] * b[row,k], is not: the row-wise renderer is the right tool for it.) */
/* The two factors of a summed product.  The scheduler also writes a product with a 0/1 factor as a
 * selection, sum where(c, y, 0) (the lookup's gradient: c is "token t is entry v"); then *a is the
 * condition and *selects is set. */
static bool reduce_factors(PolyUOp *red, PolyUOp **a, PolyUOp **b, bool *selects) {
  if (red->op != POLY_OP_REDUCE || !is_f32(red->dtype)) return false;
  PolyOps rop = red->arg.kind == POLY_ARG_OPS ? red->arg.ops : (PolyOps)red->arg.i;
  if (rop != POLY_OP_ADD) return false;
  PolyUOp *v = red->src[0];
  if (v->op == POLY_OP_MUL) { *a = v->src[0]; *b = v->src[1]; *selects = false; return true; }
  if (v->op == POLY_OP_WHERE && v->src[2]->op == POLY_OP_CONST && is_f32(v->src[1]->dtype) &&
      ((v->src[2]->arg.kind == POLY_ARG_FLOAT && v->src[2]->arg.f == 0.0) || (v->src[2]->arg.kind == POLY_ARG_INT && v->src[2]->arg.i == 0))) {
    *a = v->src[0]; *b = v->src[1]; *selects = true; return true;
  }
  return false;
}

static bool contraction_like(PbKern *k, PolyUOp *red) {
  PolyUOp *fa, *fb; bool selects;
  if (!reduce_factors(red, &fa, &fb, &selects)) return false;
  PbStore *st = &k->stores[0];
  uint64_t mask = 0;
  for (int i = 0; i < st->n_loop; i++) mask |= (uint64_t)1 << st->loop[i];
  for (int i = 1; i < red->n_src; i++) { int r = pb_kern_range_id(k, red->src[i]); if (r < 0) return false; mask |= (uint64_t)1 << r; }
  Loads la = { .n = 0 }, lb = { .n = 0 };
  Sub seen = {0};
  gather_loads(k, fa, &la, &seen); sub_free(&seen);
  gather_loads(k, fb, &lb, &seen); sub_free(&seen);
  if (la.bad || lb.bad || la.n == 0 || lb.n == 0 || la.n + lb.n > 15) { DBG("reduction: factors are not loads and arithmetic only (%d %d %d %d)", la.bad, lb.bad, la.n, lb.n); return false; }
  PolyUOp *exprs[16]; int ne = 0;
  for (int i = 0; i < la.n; i++) exprs[ne++] = la.ld[i]->src[0]->src[1];
  for (int i = 0; i < lb.n; i++) exprs[ne++] = lb.ld[i]->src[0]->src[1];
  VAxis va[2 * PB_MAX_AXES]; int nva = 0; VFit fit[16];
  if (!pb_find_axes(k, mask, exprs, ne, va, &nva, fit)) { DBG("reduction: indices not affine"); return false; }
  int64_t M = 1, N = 1, K = 1;
  for (int a = 0; a < nva; a++) {
    if (va[a].extent <= 1) continue;
    bool in_a = false, in_b = false;
    for (int i = 0; i < la.n; i++) if (fit[i].stride[a]) in_a = true;
    for (int i = 0; i < lb.n; i++) if (fit[la.n + i].stride[a]) in_b = true;
    if (va[a].reduce) { if (in_a && in_b) K *= va[a].extent; }
    else if (in_a && !in_b) M *= va[a].extent;
    else if (in_b && !in_a) N *= va[a].extent;
  }
  DBG("reduction: M %lld N %lld K %lld", (long long)M, (long long)N, (long long)K);
  return M >= 8 && N >= 8 && K >= 8;
}

/* where(ids[t] == arange[v], y, 0) summed over the tokens: the lookup's gradient, which has a kernel of
 * its own (classify_scatter) -- one side of the equality walks only the reduction, the other only output
 * axes, both plain loads. */
static bool lookup_selection(PbKern *k, PolyUOp *red, PolyUOp *cond) {
  PolyUOp *a, *b;
  if (!pb_match_equal(cond, &a, &b) || !is_plain_load(a) || !is_plain_load(b)) return false;
  PbStore *st = &k->stores[0];
  uint64_t mask = 0;
  for (int i = 0; i < st->n_loop; i++) mask |= (uint64_t)1 << st->loop[i];
  for (int i = 1; i < red->n_src; i++) { int r = pb_kern_range_id(k, red->src[i]); if (r >= 0) mask |= (uint64_t)1 << r; }
  /* by what the indices really walk (they may mention ranges they do not depend on) */
  PolyUOp *exprs[2] = { a->src[0]->src[1], b->src[0]->src[1] };
  VAxis va[2 * PB_MAX_AXES]; int nva = 0; VFit fit[2];
  if (!pb_find_axes(k, mask, exprs, 2, va, &nva, fit)) return false;
  bool a_red = false, a_out = false, b_red = false, b_out = false;
  for (int i = 0; i < nva; i++) {
    if (va[i].extent <= 1) continue;
    if (fit[0].stride[i]) { if (va[i].reduce) a_red = true; else a_out = true; }
    if (fit[1].stride[i]) { if (va[i].reduce) b_red = true; else b_out = true; }
  }
  return (a_red && !a_out && b_out && !b_red) || (b_red && !b_out && a_out && !a_red);
}

static int64_t reduce_work(PbKern *k, PolyUOp *red) {
  int64_t w = 1;
  for (int r = 0; r < k->n_ranges; r++) {
    bool mine = false;
    for (int i = 1; i < red->n_src; i++) if (pb_kern_range_id(k, red->src[i]) == r) mine = true;
    if ((mine || !k->is_reduce[r]) && k->extent[r] > 0) w *= k->extent[r];
  }
  return w;
}

static bool setup_cut(Cut *c, PolyCtx *ctx, PbKern *k) {
  memset(c, 0, sizeof *c);
  c->ctx = ctx; c->k = k;
  if (k->n_ranges == 0) return false;
  c->t_int = k->ranges[0]->dtype;
  for (int i = 0; i < k->n_nodes; i++) if (k->nodes[i].u->op == POLY_OP_END) c->end_like = k->nodes[i].u;
  return c->end_like != NULL;
}

static PolyUOp *some_f32_load(PbKern *k) {
  for (int j = 0; j < k->n_nodes; j++) if (is_plain_load(k->nodes[j].u) && is_f32(k->nodes[j].u->dtype)) return k->nodes[j].u;
  return NULL;
}

/* ── a reduction that counts only inside a window of the output axes ─── */
typedef struct { int range; int64_t shift, extent; bool lo, hi; } Window;   /* 0 <= range + shift < extent */

static bool range_plus_const(PbKern *k, PolyUOp *e, int *range, int64_t *shift) {
  if (e->op == POLY_OP_RANGE) { *range = pb_kern_range_id(k, e); *shift = 0; return *range >= 0; }
  if (e->op == POLY_OP_ADD && e->src[0]->op == POLY_OP_RANGE && e->src[1]->op == POLY_OP_CONST && e->src[1]->arg.kind == POLY_ARG_INT) {
    *range = pb_kern_range_id(k, e->src[0]); *shift = e->src[1]->arg.i; return *range >= 0;
  }
  if (e->op == POLY_OP_ADD && e->src[1]->op == POLY_OP_RANGE && e->src[0]->op == POLY_OP_CONST && e->src[0]->arg.kind == POLY_ARG_INT) {
    *range = pb_kern_range_id(k, e->src[1]); *shift = e->src[0]->arg.i; return *range >= 0;
  }
  return false;
}

static bool int_const(PolyUOp *u, int64_t *v) {
  if (u->op != POLY_OP_CONST || u->arg.kind != POLY_ARG_INT) return false;
  *v = u->arg.i; return true;
}

/* mask as a conjunction of  !(e < 0)  and  e < E  with e = range (+ const) */
static bool parse_windows(PbKern *k, PolyUOp *mask, Window *w, int *n, int cap) {
  if (mask->op == POLY_OP_AND) return parse_windows(k, mask->src[0], w, n, cap) && parse_windows(k, mask->src[1], w, n, cap);
  int r; int64_t shift, bound;
  bool is_lo;
  if (mask->op == POLY_OP_NEG && mask->src[0]->op == POLY_OP_CMPLT && int_const(mask->src[0]->src[1], &bound) && bound == 0 &&
      range_plus_const(k, mask->src[0]->src[0], &r, &shift)) is_lo = true;
  else if (mask->op == POLY_OP_CMPLT && int_const(mask->src[1], &bound) && range_plus_const(k, mask->src[0], &r, &shift)) is_lo = false;
  else return false;
  int at = -1;
  for (int i = 0; i < *n; i++) if (w[i].range == r && w[i].shift == shift) at = i;
  if (at < 0) {
    /* a second, different shift of the same range would be another window: not handled */
    for (int i = 0; i < *n; i++) if (w[i].range == r) {
      const bool triv_old = w[i].shift == 0, triv_new = shift == 0;
      if (!triv_old && !triv_new) return false;
    }
    if (*n >= cap) return false;
    at = (*n)++;
    w[at] = (Window){ r, shift, -1, false, false };
  }
  if (is_lo) w[at].lo = true; else { w[at].hi = true; w[at].extent = bound; }
  return true;
}

/* The piece that computes `red` over its window: the windowed output axes replaced by shorter ones.
 * On success *sink_out is the kernel (simplified), *numel its temporary's size and *read_index where the
 * parent finds an element, over the parent's own ranges. */
static bool windowed_piece(Cut *c, PolyUOp *red, PolyUOp *mask, PolyUOp **sink_out, int64_t *numel, PolyUOp **read_index,
                           int *old_of_new, int *n_params) {
  PbKern *k = c->k;
  PbStore *st = &k->stores[0];
  Window w[PB_MAX_AXES]; int nw = 0;
  if (!parse_windows(k, mask, w, &nw, PB_MAX_AXES)) { DBG("window: condition is not a conjunction of range tests"); return false; }
  /* per loop range: the window, or the whole range */
  int64_t shift[PB_MAX_RANGES], ext[PB_MAX_RANGES];
  for (int r = 0; r < k->n_ranges; r++) { shift[r] = 0; ext[r] = k->extent[r]; }
  bool any = false;
  for (int i = 0; i < nw; i++) {
    const Window *x = &w[i];
    if (k->is_reduce[x->range]) return false;
    if (x->shift == 0 && (!x->hi || x->extent >= k->extent[x->range])) continue;         /* always true */
    if (!x->hi || (!x->lo && x->shift != 0)) return false;       /* a range is never negative: 0 <= r needs no test */
    if (-x->shift < 0 || x->extent - x->shift > k->extent[x->range] || x->extent < 1) return false;
    if (shift[x->range] != 0 || ext[x->range] != k->extent[x->range]) return false;       /* two windows on one range */
    shift[x->range] = x->shift; ext[x->range] = x->extent; any = true;
  }
  if (!any) return false;
  Sub m = {0};
  PolyUOp *ranges[PB_MAX_AXES];
  PolyUOp *idx_t = NULL, *ridx = NULL;
  int64_t rm = 1, total = 1;
  for (int i = 0; i < st->n_loop; i++) total *= ext[st->loop[i]];
  if (total >= ((int64_t)1 << 30)) { sub_free(&m); return false; }
  /* laid out like the output: the axis with the largest output stride outermost */
  int order[PB_MAX_AXES];
  {
    uint64_t lm = 0;
    for (int i = 0; i < st->n_loop; i++) { lm |= (uint64_t)1 << st->loop[i]; order[i] = i; }
    PbAffine oa;
    pb_fit_affine(k, st->index->src[1], lm, &oa);
    if (oa.ok)
      for (int i = 1; i < st->n_loop; i++)
        for (int j = i; j > 0 && llabs(oa.stride[st->loop[order[j - 1]]]) < llabs(oa.stride[st->loop[order[j]]]); j--) {
          int t = order[j]; order[j] = order[j - 1]; order[j - 1] = t;
        }
  }
  rm = total;
  for (int o = 0; o < st->n_loop; o++) {
    const int i = order[o], r = st->loop[i];
    rm /= ext[r];
    PolyUOp *nr = k->ranges[r];
    if (shift[r] != 0 || ext[r] != k->extent[r]) {
      nr = poly_uop1(c->ctx, POLY_OP_RANGE, c->t_int, ci(c, ext[r]), poly_arg_range(64 + r, POLY_AXIS_LOOP));
      sub_put(&m, k->ranges[r], shift[r] ? ibin(c, POLY_OP_ADD, nr, ci(c, -shift[r])) : nr);
    }
    ranges[i] = nr;
    idx_t = iadd(c, idx_t, iscale(c, nr, rm));
    PolyUOp *pos = shift[r] ? ibin(c, POLY_OP_ADD, k->ranges[r], ci(c, shift[r])) : k->ranges[r];
    ridx = iadd(c, ridx, iscale(c, pos, rm));
  }
  PolyUOp *value = rebuild(c->ctx, &m, red);
  sub_free(&m);
  if (!value || !idx_t) return false;
  value = renumber_params(c, value, 1, old_of_new, n_params);
  if (!value) return false;
  PolyUOp *sink = wrap_store(c, param_like(c, k->params[st->param], 0, total), idx_t, value, ranges, st->n_loop);
  if (!sink) return false;
  sink = poly_graph_rewrite(c->ctx, sink, poly_symbolic_simple());
  if (!sink) return false;
  /* is it a contraction now? */
  PbKern kp;
  bool good = false;
  if (pb_kern_build(&kp, sink) == 0 && kp.n_reduce_nodes == 1 && kp.n_stores == 1) {
    for (int i = 0; i < kp.n_nodes && !good; i++)
      if (kp.nodes[i].u->op == POLY_OP_REDUCE) good = contraction_like(&kp, kp.nodes[i].u);
  }
  pb_kern_free(&kp);
  if (!good) { DBG("window: the reduction over its window is not a contraction"); return false; }
  *sink_out = sink; *numel = total; *read_index = ridx;
  return true;
}

int pb_outline(PolyCtx *ctx, PolyUOp *sink, PbPiece *pieces, int cap, int64_t *temp_numel, int *n_temps) {
  *n_temps = 0;
  int n_pieces = 0, result = 0;
  int source_of[PB_MAX_PARAMS];           /* of the kernel being cut as it grows parameters: parent's parameter or -(temp + 1) */
  PbKern k;
  if (pb_kern_build(&k, sink) != 0) { pb_kern_free(&k); return 0; }
  PolyUOp *current = sink;
  Cut c;
  if (k.n_stores != 1 || k.n_vars != 0 || k.n_reduce_nodes < 1 || k.stores[0].index->n_src != 2 || !setup_cut(&c, ctx, &k)) goto done;
  if (!is_f32(k.stores[0].value->dtype) || k.params[k.stores[0].param]->dtype.ptr_size < 0) goto done;
  for (int r = 0; r < k.n_ranges; r++) if (k.extent[r] < 0) goto done;
  int next_param = k.n_params;
  for (int p = 0; p < next_param; p++) source_of[p] = p;

  /* which reductions are contractions, and is there enough work in them to pay for the cut */
  int64_t min_work = (int64_t)1 << 22;
  { const char *e = getenv("POLY_B200_OUTLINE_MIN_WORK"); if (e && e[0]) min_work = atoll(e); }
  PolyUOp *reds[PB_MAX_TEMPS]; int n_red = 0; int64_t work = 0;
  for (int i = 0; i < k.n_nodes; i++) {
    PolyUOp *u = k.nodes[i].u, *fa, *fb; bool selects;
    if (u->op != POLY_OP_REDUCE) continue;
    if (k.nodes[pb_kern_node(&k, u->src[0])].has_reduce) goto done;       /* nested */
    if (!reduce_factors(u, &fa, &fb, &selects)) continue;
    work += reduce_work(&k, u);
    if (contraction_like(&k, u)) {
      if (n_red >= PB_MAX_TEMPS) goto done;
      reds[n_red++] = u;
    }
  }
  if (work < min_work) goto done;
  PolyUOp *load_like = some_f32_load(&k);
  if (!load_like) goto done;

  /* step 1: computed operands */
  {
    Sub subst = {0};
    bool ok = true;
    for (int i = 0; i < n_red && ok; i++) {
      PolyUOp *f[2]; bool selects;
      reduce_factors(reds[i], &f[0], &f[1], &selects);
      PolyUOp *put_back[2] = { NULL, NULL };
      for (int s = 1; s >= 0 && ok; s--) {
        /* what is stored: the factor without constant scale, or the 0/1 value of a condition */
        PolyUOp *e = operand_core(f[s]), *deps_of = e, *stored = e;
        if (selects && s == 0 && lookup_selection(&k, reds[i], f[0])) continue;   /* stays: the scatter kernel takes it */
        if (selects && s == 0) {
          e = f[0]; deps_of = f[0];
          stored = poly_uop3(ctx, POLY_OP_WHERE, reds[i]->dtype, f[0],
                             poly_uop0(ctx, POLY_OP_CONST, reds[i]->dtype, poly_arg_float(1.0)),
                             poly_uop0(ctx, POLY_OP_CONST, reds[i]->dtype, poly_arg_float(0.0)), poly_arg_none());
          if (!stored) { ok = false; break; }
        } else if (is_plain_load(e)) continue;
        PolyUOp *have = sub_get(&subst, e);
        if (!have) {
          Operand op;
          if (!materialize(&c, stored, deps_of, &op) || n_pieces >= cap - 1 || *n_temps >= PB_MAX_TEMPS || next_param >= PB_MAX_PARAMS) { ok = false; break; }
          const int t = (*n_temps)++;
          temp_numel[t] = op.numel;
          PbPiece *pc = &pieces[n_pieces++];
          memset(pc, 0, sizeof *pc);
          pc->sink = op.sink;
          pc->n_params = 1 + op.n_params;
          pc->param_src[0] = -(t + 1);
          for (int q = 0; q < op.n_params; q++) pc->param_src[1 + q] = op.parent_param[q];
          /* the kernel reads the temporary through a new parameter */
          PolyUOp *np = param_like(&c, k.params[k.stores[0].param], next_param, op.numel);
          PolyUOp *nindex = poly_uop2(ctx, POLY_OP_INDEX, k.stores[0].index->dtype, np, op.read_index, k.stores[0].index->arg);
          have = poly_uop1(ctx, POLY_OP_LOAD, load_like->dtype, nindex, load_like->arg);
          source_of[next_param++] = -(t + 1);
          if (!(selects && s == 0)) sub_put(&subst, e, have);
        }
        put_back[s] = have;
      }
      if (ok && selects && put_back[0]) {
        /* where(c, y, 0) becomes onehot * y, y with whatever was substituted in it */
        PolyUOp *y = rebuild(ctx, &subst, f[1]);
        PolyUOp *prod = y && put_back[0] ? poly_uop2(ctx, POLY_OP_MUL, reds[i]->dtype, put_back[0], y, poly_arg_none()) : NULL;
        if (!prod) { ok = false; break; }
        sub_put(&subst, reds[i]->src[0], prod);
      }
    }
    if (ok && subst.n > 0) current = rebuild(ctx, &subst, sink);
    sub_free(&subst);
    if (!ok || !current) goto done;
  }

  /* is the kernel a single recognisable contraction now? */
  bool single = false;
  {
    PbKern k2;
    if (pb_kern_build(&k2, current) == 0 && k2.n_reduce_nodes == 1) {
      char *hdr = pb_classify_aot(&k2, "outline");
      if (hdr) { single = strstr(hdr, "//kind gemm") != NULL || strstr(hdr, "//kind scatter") != NULL; free(hdr); }
    }
    pb_kern_free(&k2);
  }
  if (single && n_pieces == 0) goto done;                /* nothing was cut: the kernel is what it was */

  /* step 2: each contraction into a temporary laid out like the output */
  if (!single) {
    PbKern k2;
    if (pb_kern_build(&k2, current) != 0) { pb_kern_free(&k2); goto done; }
    Cut c2;
    bool ok = k2.n_stores == 1 && setup_cut(&c2, ctx, &k2);
    PbStore *st = &k2.stores[0];
    const int64_t out_numel = ok ? k2.params[st->param]->dtype.ptr_size : 0;
    PolyUOp *ranges[PB_MAX_AXES];
    for (int i = 0; ok && i < st->n_loop; i++) ranges[i] = k2.ranges[st->loop[i]];
    Sub subst2 = {0};
    for (int i = 0; i < k2.n_nodes && ok; i++) {
      PolyUOp *u = k2.nodes[i].u;
      if (u->op != POLY_OP_REDUCE) continue;
      if (n_pieces >= cap - 1 || *n_temps >= PB_MAX_TEMPS || next_param >= PB_MAX_PARAMS) { ok = false; break; }
      PbPiece *pc = &pieces[n_pieces];
      memset(pc, 0, sizeof *pc);
      int old_of_new[PB_MAX_PARAMS], np = 0;
      int64_t numel = out_numel;
      PolyUOp *read_index = st->index->src[1];
      if (contraction_like(&k2, u)) {
        PolyUOp *value = renumber_params(&c2, u, 1, old_of_new, &np);
        if (!value) { ok = false; break; }
        pc->sink = wrap_store(&c2, param_like(&c2, k2.params[st->param], 0, out_numel), st->index->src[1], value, ranges, st->n_loop);
        if (!pc->sink) { ok = false; break; }
      } else {
        /* where(window, sum, 0): the sum over its window alone */
        const PbNode *nd = &k2.nodes[i];
        PolyUOp *par = nd->n_uses == 1 && nd->only_parent >= 0 ? k2.nodes[nd->only_parent].u : NULL;
        PolyUOp *fa, *fb; bool selects;
        if (!par || par->op != POLY_OP_WHERE || par->src[1] != u || par->src[2]->op != POLY_OP_CONST ||
            !reduce_factors(u, &fa, &fb, &selects) || selects) continue;
        if (!windowed_piece(&c2, u, par->src[0], &pc->sink, &numel, &read_index, old_of_new, &np)) continue;
      }
      const int t = (*n_temps)++;
      temp_numel[t] = numel;
      pc->n_params = np;
      pc->param_src[0] = -(t + 1);
      for (int q = 1; q < np; q++) pc->param_src[q] = source_of[old_of_new[q]];
      pc->must_be_contraction = true;
      n_pieces++;
      PolyUOp *npar = param_like(&c2, k2.params[st->param], next_param, numel);
      PolyUOp *nindex = poly_uop2(ctx, POLY_OP_INDEX, st->index->dtype, npar, read_index, st->index->arg);
      sub_put(&subst2, u, poly_uop1(ctx, POLY_OP_LOAD, load_like->dtype, nindex, load_like->arg));
      source_of[next_param++] = -(t + 1);
    }
    if (ok && subst2.n > 0) current = rebuild(ctx, &subst2, current); else ok = false;
    sub_free(&subst2);
    pb_kern_free(&k2);
    if (!ok || !current) goto done;
  }

  /* the remainder, with the parameters it still uses numbered from 0 */
  {
    PbKern k3;
    if (pb_kern_build(&k3, current) != 0) { pb_kern_free(&k3); goto done; }
    Cut c3;
    PbPiece *pc = &pieces[n_pieces];
    memset(pc, 0, sizeof *pc);
    int old_of_new[PB_MAX_PARAMS], np = 0;
    PolyUOp *root = setup_cut(&c3, ctx, &k3) ? renumber_params(&c3, current, 0, old_of_new, &np) : NULL;
    pb_kern_free(&k3);
    if (!root || np == 0 || old_of_new[0] != k.stores[0].param) goto done;   /* the output stays parameter 0 of what it was */
    pc->sink = root;
    pc->n_params = np;
    for (int q = 0; q < np; q++) pc->param_src[q] = source_of[old_of_new[q]];
    pc->must_be_contraction = single;
    n_pieces++;
    result = n_pieces;
  }
done:
  pb_kern_free(&k);
  return result;
}
