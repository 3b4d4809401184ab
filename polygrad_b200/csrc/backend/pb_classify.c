/*
 * pb_classify.c -- recognises scheduled kernels that map onto precompiled
 * sm_100a kernels and describes them in a "//PB200" header.
 *
 *   gather  polygrad lowers embedding lookups to a one-hot contraction over the
 *           whole table: sum_v where(idx[t] == arange[v], table[v, d], 0)
 *           (reference: src/modelzoo/models/gpt2.c:93-153,
 *           src/frontend.c:3494-3583).  Recognised by shape, executed as a
 *           search of `arange` followed by a row copy.
 *   gemm    polygrad's matmul is reshape/expand -> MUL -> REDUCE(ADD)
 *           (reference: src/frontend.c:1029-1129), optionally followed by
 *           "+ bias" and ReLU fused by the scheduler.  Recognised as a single
 *           ADD-reduction of a product of two loads whose index expressions
 *           are affine in the kernel's ranges (after splitting a range where
 *           a view introduced div/mod, e.g. the head-merge read in
 *           src/modelzoo/models/gpt2.c:436-452).
 *   scatter the gradient of that lookup: for every table row, the sum of the
 *           gradient rows whose token is that row; executed as a scan of the
 *           tokens per group of table rows followed by ordered row sums.
 *   copy    a pure data movement whose source and destination differ in their
 *           contiguous axis (permute): executed as a tiled transpose.
 *
 * Everything is derived from the index expressions themselves, evaluated
 * numerically (pb_eval_int), never from loop nesting or names.
 */
#include "pb_kern.h"
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

/* POLY_B200_DEBUG=1 prints why a kernel was not given to a precompiled kernel */
#define REJECT(why) do { if (getenv("POLY_B200_DEBUG")) fprintf(stderr, "pb_classify: %s:%d: %s\n", __func__, __LINE__, why); return NULL; } while (0)

/* virtual axes (VAxis, VFit): pb_kern.h */
static uint64_t rng_next(uint64_t *s) {
  uint64_t x = *s; x ^= x << 13; x ^= x >> 7; x ^= x << 17; *s = x; return x;
}

static bool veval(const PbKern *k, PolyUOp *e, const VAxis *va, int nva, const int64_t *x, int64_t *out) {
  int64_t vals[PB_MAX_RANGES] = {0};
  for (int i = 0; i < nva; i++) vals[va[i].range] += x[i] * va[i].mult;
  return pb_eval_int(k, e, vals, NULL, out);
}

static void vfit(const PbKern *k, PolyUOp *e, const VAxis *va, int nva, VFit *f) {
  memset(f, 0, sizeof *f);
  int64_t x[2 * PB_MAX_AXES] = {0};
  int64_t base;
  if (!veval(k, e, va, nva, x, &base)) return;
  f->offset = base;
  for (int i = 0; i < nva; i++) {
    if (va[i].extent <= 1) continue;
    x[i] = 1;
    int64_t v;
    if (!veval(k, e, va, nva, x, &v)) return;
    f->stride[i] = v - base;
    x[i] = 0;
  }
  /* axis lines */
  for (int i = 0; i < nva; i++) {
    int64_t ext = va[i].extent;
    int64_t step = ext > 2048 ? ext / 2048 : 1;
    for (int64_t t = 0; t < ext; t += step) {
      x[i] = t;
      int64_t v;
      if (!veval(k, e, va, nva, x, &v) || v != base + f->stride[i] * t) return;
    }
    x[i] = ext - 1;
    int64_t v;
    if (!veval(k, e, va, nva, x, &v) || v != base + f->stride[i] * (ext - 1)) return;
    x[i] = 0;
  }
  /* corners and random interior points */
  uint64_t seed = 0x2545f4914f6cdd1dULL;
  for (int t = 0; t < 8192; t++) {
    int64_t expect = base;
    for (int i = 0; i < nva; i++) {
      int64_t ext = va[i].extent;
      int64_t xi;
      if (t < 64) xi = ((t >> (i % 6)) & 1) ? ext - 1 : 0;
      else xi = (int64_t)(rng_next(&seed) % (uint64_t)ext);
      x[i] = xi;
      expect += f->stride[i] * xi;
    }
    int64_t v;
    if (!veval(k, e, va, nva, x, &v) || v != expect) return;
  }
  f->ok = true;
}

/* Constants used as divisors/moduli inside e (split candidates). */
static void collect_divisors(PolyUOp *e, int64_t *out, int *n, int cap, int depth) {
  if (depth > 64) return;
  if ((e->op == POLY_OP_IDIV || e->op == POLY_OP_MOD) && e->n_src == 2 && e->src[1]->op == POLY_OP_CONST) {
    int64_t c = e->src[1]->arg.i;
    bool have = false;
    for (int i = 0; i < *n; i++) if (out[i] == c) have = true;
    if (!have && *n < cap && c > 1) out[(*n)++] = c;
  }
  if (e->op == POLY_OP_LOAD) return;
  for (int i = 0; i < e->n_src; i++) collect_divisors(e->src[i], out, n, cap, depth + 1);
}

/* Build virtual axes for the ranges in `mask` such that every expression in
 * exprs[] is affine; tries no split, one split, two splits of different
 * ranges, then one range split in three. */
bool pb_find_axes(const PbKern *k, uint64_t mask, PolyUOp **exprs, int n_exprs,
                  VAxis *va, int *nva, VFit *fits) {
  int ids[PB_MAX_RANGES]; int n = 0;
  for (int r = 0; r < k->n_ranges; r++) if (mask >> r & 1) ids[n++] = r;
  if (n > PB_MAX_AXES) return false;
  int64_t cands[16]; int nc = 0;
  for (int i = 0; i < n_exprs; i++) collect_divisors(exprs[i], cands, &nc, 16, 0);

  /* split plans: (range index a, factor fa), (range index b, factor fb); -1 = none */
  for (int plan = 0; plan < 3; plan++) {
    int amax = plan >= 1 ? n : 1, bmax = plan >= 2 ? n : 1;
    int camax = plan >= 1 ? nc : 1, cbmax = plan >= 2 ? nc : 1;
    for (int a = 0; a < amax; a++) for (int ca = 0; ca < camax; ca++)
    for (int b = (plan >= 2 ? a + 1 : 0); b < bmax; b++) for (int cb = 0; cb < cbmax; cb++) {
      int sa = plan >= 1 ? a : -1, sb = plan >= 2 ? b : -1;
      int64_t fa = plan >= 1 ? cands[ca] : 0, fb = plan >= 2 ? cands[cb] : 0;
      if (sa >= 0 && (k->extent[ids[sa]] % fa || fa >= k->extent[ids[sa]])) continue;
      if (sb >= 0 && (k->extent[ids[sb]] % fb || fb >= k->extent[ids[sb]])) continue;
      int m = 0;
      for (int i = 0; i < n; i++) {
        int r = ids[i];
        int64_t f = (i == sa) ? fa : (i == sb) ? fb : 0;
        if (f) {
          va[m++] = (VAxis){r, k->extent[r] / f, f, k->is_reduce[r]};
          va[m++] = (VAxis){r, f, 1, k->is_reduce[r]};
        } else {
          va[m++] = (VAxis){r, k->extent[r], 1, k->is_reduce[r]};
        }
      }
      bool all = true;
      for (int i = 0; i < n_exprs && all; i++) { vfit(k, exprs[i], va, m, &fits[i]); all = fits[i].ok; }
      if (all) { *nva = m; return true; }
    }
  }
  /* one range in three parts (a flat [out][head][dim] index read through a head permutation) */
  int64_t outer[16 + 16 * 16]; int no = 0;          /* the outer factor may be a product of two divisors */
  for (int i = 0; i < nc; i++) outer[no++] = cands[i];
  for (int i = 0; i < nc; i++) for (int j = i; j < nc; j++) {
    const int64_t pr = cands[i] * cands[j];
    bool have = false;
    for (int q = 0; q < no; q++) if (outer[q] == pr) have = true;
    if (!have && pr < ((int64_t)1 << 40)) outer[no++] = pr;
  }
  for (int a = 0; a < n; a++) for (int ca = 0; ca < no; ca++) for (int cb = 0; cb < nc; cb++) {
    const int64_t fa = outer[ca], fb = cands[cb], ext = k->extent[ids[a]];
    if (fb >= fa || fa % fb || fa >= ext || ext % fa) continue;
    int m = 0;
    for (int i = 0; i < n; i++) {
      int r = ids[i];
      if (i == a) {
        va[m++] = (VAxis){r, ext / fa, fa, k->is_reduce[r]};
        va[m++] = (VAxis){r, fa / fb, fb, k->is_reduce[r]};
        va[m++] = (VAxis){r, fb, 1, k->is_reduce[r]};
      } else va[m++] = (VAxis){r, k->extent[r], 1, k->is_reduce[r]};
    }
    bool all = true;
    for (int i = 0; i < n_exprs && all; i++) { vfit(k, exprs[i], va, m, &fits[i]); all = fits[i].ok; }
    if (all) { *nva = m; return true; }
  }
  return false;
}

/* scalar dtype tests by priority: loads carry leftover pointer fields that make
 * poly_dtype_eq against the predefined constants fail */
static bool is_f32(PolyDType d) { return !d.is_ptr && d.count == 1 && d.priority == 13; }
static bool is_bf16(PolyDType d) { return !d.is_ptr && d.count == 1 && d.priority == 12; }
static bool is_f16(PolyDType d) { return !d.is_ptr && d.count == 1 && d.priority == 11; }

static bool const_is(PolyUOp *u, double v) {
  if (u->op != POLY_OP_CONST) return false;
  if (u->arg.kind == POLY_ARG_FLOAT) return u->arg.f == v;
  if (u->arg.kind == POLY_ARG_INT) return (double)u->arg.i == v;
  if (u->arg.kind == POLY_ARG_BOOL) return (double)u->arg.b == v;
  return false;
}

static bool const_f32(PolyUOp *u, float *out) {
  if (u->op != POLY_OP_CONST || !is_f32(u->dtype)) return false;
  if (u->arg.kind == POLY_ARG_FLOAT) { *out = (float)u->arg.f; return true; }
  if (u->arg.kind == POLY_ARG_INT) { *out = (float)u->arg.i; return true; }
  return false;
}

/* u as scale * red: red itself, -red, c * red or red * c. */
static bool scaled_by_const(PolyUOp *u, PolyUOp *red, float *scale) {
  float c;
  if (u == red) { *scale = 1.0f; return true; }
  if (u->op == POLY_OP_NEG && u->src[0] == red) { *scale = -1.0f; return true; }
  if (u->op == POLY_OP_MUL && u->src[1] == red && const_f32(u->src[0], &c)) { *scale = c; return true; }
  if (u->op == POLY_OP_MUL && u->src[0] == red && const_f32(u->src[1], &c)) { *scale = c; return true; }
  return false;
}

/* u without a float32 constant factor; the factor is multiplied into *scale. */
static PolyUOp *strip_const_scale(PolyUOp *u, float *scale) {
  float c;
  if (u->op != POLY_OP_MUL) return u;
  if (const_f32(u->src[1], &c)) { *scale *= c; return u->src[0]; }
  if (const_f32(u->src[0], &c)) { *scale *= c; return u->src[1]; }
  return u;
}

static bool is_plain_load(PolyUOp *u) {
  return u->op == POLY_OP_LOAD && u->src[0]->op == POLY_OP_INDEX && u->src[0]->n_src == 2 &&
         u->src[0]->src[0]->op == POLY_OP_PARAM;
}
static int load_param(PolyUOp *ld) { return (int)ld->src[0]->src[0]->arg.i; }
static PolyUOp *load_index(PolyUOp *ld) { return ld->src[0]->src[1]; }
static int64_t param_numel(const PbKern *k, int p) { return k->params[p]->dtype.ptr_size; }

static bool all_const_extents(const PbKern *k) {
  for (int r = 0; r < k->n_ranges; r++) if (k->extent[r] < 0) return false;
  return k->n_vars == 0;
}

/* Range of an affine expression over the axes; false if it leaves [0, numel). */
static bool in_bounds(const VFit *f, const VAxis *va, int nva, int64_t numel) {
  int64_t lo = f->offset, hi = f->offset;
  for (int i = 0; i < nva; i++) {
    int64_t s = f->stride[i] * (va[i].extent - 1);
    if (s > 0) hi += s; else lo += s;
  }
  return lo >= 0 && hi < numel;
}

/* ── gather ──────────────────────────────────────────────────────────── */
/* equality test of two loads, in any of the forms the frontend produces */
bool pb_match_equal(PolyUOp *c, PolyUOp **a, PolyUOp **b) {
  if (c->op == POLY_OP_CAST) return pb_match_equal(c->src[0], a, b);
  if (c->op == POLY_OP_CMPEQ) { *a = c->src[0]; *b = c->src[1]; return true; }
  if (c->op == POLY_OP_NEG && c->src[0]->op == POLY_OP_CMPNE) { *a = c->src[0]->src[0]; *b = c->src[0]->src[1]; return true; }
  if (c->op == POLY_OP_WHERE && c->src[0]->op == POLY_OP_CMPNE && const_is(c->src[1], 0.0) &&
      c->src[2]->op == POLY_OP_CONST && !const_is(c->src[2], 0.0)) {
    *a = c->src[0]->src[0]; *b = c->src[0]->src[1]; return true;
  }
  return false;
}

static char *classify_gather(PbKern *k) {
  if (k->n_stores != 1 || k->n_reduce_nodes != 1 || !all_const_extents(k)) REJECT("pattern");
  PbStore *st = &k->stores[0];
  if (st->index->n_src != 2 || st->value->op != POLY_OP_REDUCE) REJECT("pattern");
  PolyUOp *red = st->value;
  if (red->n_src != 2) REJECT("pattern");
  PolyOps rop = red->arg.kind == POLY_ARG_OPS ? red->arg.ops : (PolyOps)red->arg.i;
  if (rop != POLY_OP_ADD) REJECT("pattern");
  int rv = pb_kern_range_id(k, red->src[1]);
  PolyUOp *w = red->src[0];
  if (w->op != POLY_OP_WHERE || !const_is(w->src[2], 0.0)) REJECT("pattern");
  PolyUOp *ea, *eb;
  if (!pb_match_equal(w->src[0], &ea, &eb)) REJECT("pattern");
  PolyUOp *tab = w->src[1];
  if (!is_plain_load(ea) || !is_plain_load(eb) || !is_plain_load(tab)) REJECT("pattern");
  uint64_t rbit = (uint64_t)1 << rv;
  uint64_t da = k->nodes[pb_kern_node(k, ea)].deps, db = k->nodes[pb_kern_node(k, eb)].deps;
  PolyUOp *idx, *ar;
  if (!(da & rbit) && db == rbit) { idx = ea; ar = eb; }
  else if (!(db & rbit) && da == rbit) { idx = eb; ar = ea; }
  else REJECT("pattern");
  if (!is_f32(idx->dtype) || !is_f32(ar->dtype) || !is_f32(tab->dtype) || !is_f32(red->dtype)) REJECT("dtype");

  uint64_t mask = rbit;
  for (int i = 0; i < st->n_loop; i++) mask |= (uint64_t)1 << st->loop[i];
  PolyUOp *exprs[4] = { st->index->src[1], load_index(idx), load_index(ar), load_index(tab) };
  VAxis va[2 * PB_MAX_AXES]; int nva; VFit fit[4];
  if (!pb_find_axes(k, mask, exprs, 4, va, &nva, fit)) REJECT("pattern");
  int params[4] = { st->param, load_param(idx), load_param(ar), load_param(tab) };
  for (int i = 0; i < 4; i++) if (!in_bounds(&fit[i], va, nva, param_numel(k, params[i]))) REJECT("pattern");
  /* arange must be read as arange[v] */
  int vax = -1;
  for (int i = 0; i < nva; i++) if (va[i].range == rv) { if (vax >= 0) REJECT("pattern"); vax = i; }
  if (vax < 0 || fit[2].offset != 0 || fit[2].stride[vax] != 1) REJECT("pattern");
  if (fit[0].stride[vax] != 0 || fit[1].stride[vax] != 0 || fit[3].stride[vax] == 0) REJECT("pattern");
  /* the destination must not alias an input */
  for (int i = 1; i < 4; i++) if (params[i] == params[0]) REJECT("pattern");

  /* token axes carry the index; feature axes walk a table row */
  PbStr h; pb_str_init(&h);
  pb_str_puts(&h, "//PB200 1\n//kind gather\n");
  pb_str_printf(&h, "//nparams %d\n", k->n_params);
  pb_str_printf(&h, "//params %d %d %d %d\n", params[0], params[1], params[2], params[3]);
  pb_str_printf(&h, "//vocab %lld %lld\n", (long long)va[vax].extent, (long long)fit[3].stride[vax]);
  pb_str_printf(&h, "//offsets %lld %lld %lld\n", (long long)fit[0].offset, (long long)fit[1].offset, (long long)fit[3].offset);
  int ntok = 0, nfeat = 0;
  PbStr tok, feat; pb_str_init(&tok); pb_str_init(&feat);
  for (int i = 0; i < nva; i++) {
    if (i == vax || va[i].extent == 1) continue;
    if (fit[3].stride[i] != 0 && fit[1].stride[i] == 0) {
      pb_str_printf(&feat, " %lld %lld %lld", (long long)va[i].extent, (long long)fit[0].stride[i], (long long)fit[3].stride[i]);
      nfeat++;
    } else if (fit[3].stride[i] == 0) {
      pb_str_printf(&tok, " %lld %lld %lld", (long long)va[i].extent, (long long)fit[0].stride[i], (long long)fit[1].stride[i]);
      ntok++;
    } else { pb_str_free(&tok); pb_str_free(&feat); pb_str_free(&h); REJECT("pattern"); }
  }
  if (ntok > 4 || nfeat > 3) { pb_str_free(&tok); pb_str_free(&feat); pb_str_free(&h); REJECT("pattern"); }
  pb_str_printf(&h, "//tok%s\n//feat%s\n", tok.s ? tok.s : "", feat.s ? feat.s : "");
  pb_str_free(&tok); pb_str_free(&feat);
  return pb_str_take(&h);
}

/* ── scatter: the lookup's gradient ──────────────────────────────────── */
/* The backward of the one-hot lookup sums, for every table row v, the rows of the incoming gradient
 * whose token is v:  out[v, d] = sum_t where(ids[t] == arange[v], g[t, d], 0)  (reference: the gradient of
 * the WHERE/REDUCE pair of src/modelzoo/models/gpt2.c:93-153 under src/autograd.c).  Same tree as the
 * lookup with the roles of the axes exchanged: the reduction runs over the token axes, `arange` is
 * indexed by an output axis. */
static char *classify_scatter(PbKern *k) {
  if (k->n_stores != 1 || k->n_reduce_nodes < 1 || k->n_reduce_nodes > 2 || !all_const_extents(k)) REJECT("pattern");
  PbStore *st = &k->stores[0];
  if (st->index->n_src != 2 || st->value->op != POLY_OP_REDUCE) REJECT("pattern");
  PolyUOp *red = st->value;
  PolyOps rop = red->arg.kind == POLY_ARG_OPS ? red->arg.ops : (PolyOps)red->arg.i;
  if (rop != POLY_OP_ADD || red->n_src < 2) REJECT("pattern");
  /* a sum of a sum (x.sum(0).sum(0) over batch and position) is one sum over both */
  PolyUOp *inner = NULL;
  if (k->n_reduce_nodes == 2) {
    inner = red->src[0];
    if (inner->op != POLY_OP_REDUCE || inner->n_src < 2 || k->nodes[pb_kern_node(k, inner)].n_uses != 1) REJECT("pattern");
    PolyOps iop = inner->arg.kind == POLY_ARG_OPS ? inner->arg.ops : (PolyOps)inner->arg.i;
    if (iop != POLY_OP_ADD || !is_f32(inner->dtype)) REJECT("pattern");
  }
  uint64_t rmask = 0;
  for (int i = 1; i < red->n_src; i++) { int r = pb_kern_range_id(k, red->src[i]); if (r < 0) REJECT("pattern"); rmask |= (uint64_t)1 << r; }
  for (int i = 1; inner && i < inner->n_src; i++) { int r = pb_kern_range_id(k, inner->src[i]); if (r < 0) REJECT("pattern"); rmask |= (uint64_t)1 << r; }
  PolyUOp *w = inner ? inner->src[0] : red->src[0];
  if (w->op != POLY_OP_WHERE || !const_is(w->src[2], 0.0)) REJECT("pattern");
  PolyUOp *ea, *eb;
  if (!pb_match_equal(w->src[0], &ea, &eb)) REJECT("pattern");
  PolyUOp *src = w->src[1];
  if (!is_plain_load(ea) || !is_plain_load(eb) || !is_plain_load(src)) REJECT("pattern");
  if (!is_f32(ea->dtype) || !is_f32(eb->dtype) || !is_f32(src->dtype) || !is_f32(red->dtype)) REJECT("dtype");
  if (k->params[st->param]->dtype.priority != 13) REJECT("dtype");

  uint64_t mask = rmask;
  for (int i = 0; i < st->n_loop; i++) mask |= (uint64_t)1 << st->loop[i];
  /* which side of the equality is the token's id and which the table row's number is read off the
   * strides (the index expressions may mention ranges they do not depend on) */
  PolyUOp *exprs[4] = { st->index->src[1], load_index(ea), load_index(eb), load_index(src) };
  VAxis va[2 * PB_MAX_AXES]; int nva; VFit fit[4];
  if (!pb_find_axes(k, mask, exprs, 4, va, &nva, fit)) REJECT("pattern");
  bool a_red = false, a_out = false, b_red = false, b_out = false;
  for (int i = 0; i < nva; i++) {
    if (va[i].extent <= 1) continue;
    if (fit[1].stride[i]) { if (va[i].reduce) a_red = true; else a_out = true; }
    if (fit[2].stride[i]) { if (va[i].reduce) b_red = true; else b_out = true; }
  }
  PolyUOp *idx, *ar;
  if (a_red && !a_out && b_out && !b_red) { idx = ea; ar = eb; }
  else if (b_red && !b_out && a_out && !a_red) { idx = eb; ar = ea; VFit t = fit[1]; fit[1] = fit[2]; fit[2] = t; }
  else REJECT("pattern");
  int params[4] = { st->param, load_param(idx), load_param(ar), load_param(src) };
  for (int i = 0; i < 4; i++) if (!in_bounds(&fit[i], va, nva, param_numel(k, params[i]))) REJECT("pattern");
  for (int i = 1; i < 4; i++) if (params[i] == params[0]) REJECT("pattern");
  /* one output axis is the table row: arange is read as arange[v] there and nowhere else */
  int vax = -1;
  for (int i = 0; i < nva; i++) if (va[i].extent > 1 && fit[2].stride[i] != 0) { if (vax >= 0) REJECT("pattern"); vax = i; }
  if (vax < 0 || va[vax].reduce || fit[2].offset != 0 || fit[2].stride[vax] != 1) REJECT("pattern");
  if (fit[0].stride[vax] == 0 || fit[1].stride[vax] != 0 || fit[3].stride[vax] != 0) REJECT("pattern");

  PbStr h; pb_str_init(&h);
  pb_str_puts(&h, "//PB200 1\n//kind scatter\n");
  pb_str_printf(&h, "//nparams %d\n", k->n_params);
  pb_str_printf(&h, "//params %d %d %d %d\n", params[0], params[1], params[2], params[3]);
  pb_str_printf(&h, "//vocab %lld %lld\n", (long long)va[vax].extent, (long long)fit[0].stride[vax]);
  pb_str_printf(&h, "//offsets %lld %lld %lld\n", (long long)fit[0].offset, (long long)fit[1].offset, (long long)fit[3].offset);
  int ntok = 0, nfeat = 0;
  PbStr tok, feat; pb_str_init(&tok); pb_str_init(&feat);
  /* token axes (reduced): innermost first, i.e. the later virtual axis of a later range first */
  for (int i = nva - 1; i >= 0; i--) {
    if (i == vax || va[i].extent == 1) continue;
    if (va[i].reduce) {
      if (fit[0].stride[i] != 0) { pb_str_free(&tok); pb_str_free(&feat); pb_str_free(&h); REJECT("pattern"); }
      pb_str_printf(&tok, " %lld %lld %lld", (long long)va[i].extent, (long long)fit[1].stride[i], (long long)fit[3].stride[i]);
      ntok++;
    } else {
      /* a feature axis: walks the output and the source, not the ids */
      if (fit[1].stride[i] != 0 || fit[0].stride[i] == 0) { pb_str_free(&tok); pb_str_free(&feat); pb_str_free(&h); REJECT("pattern"); }
      pb_str_printf(&feat, " %lld %lld %lld", (long long)va[i].extent, (long long)fit[0].stride[i], (long long)fit[3].stride[i]);
      nfeat++;
    }
  }
  if (ntok < 1 || ntok > 4 || nfeat > 3) { pb_str_free(&tok); pb_str_free(&feat); pb_str_free(&h); REJECT("pattern"); }
  pb_str_printf(&h, "//tok%s\n//feat%s\n", tok.s ? tok.s : "", feat.s ? feat.s : "");
  pb_str_free(&tok); pb_str_free(&feat);
  return pb_str_take(&h);
}

/* ── gemm ────────────────────────────────────────────────────────────── */
static PolyUOp *strip_cast_to_f32(PolyUOp *u) {
  if (u->op == POLY_OP_CAST && is_f32(u->dtype)) return u->src[0];
  return u;
}

static const char *operand_dtype(PolyUOp *ld) {
  if (is_f32(ld->dtype)) return "f32";
  if (is_bf16(ld->dtype)) return "bf16";
  if (is_f16(ld->dtype)) return "f16";
  return NULL;
}

static char *classify_gemm(PbKern *k) {
  if (k->n_stores != 1 || k->n_reduce_nodes != 1 || !all_const_extents(k)) REJECT("pattern");
  PbStore *st = &k->stores[0];
  if (st->index->n_src != 2) REJECT("pattern");
  PolyUOp *red = NULL;
  for (int i = 0; i < k->n_nodes; i++) if (k->nodes[i].u->op == POLY_OP_REDUCE) red = k->nodes[i].u;
  PolyOps rop = red->arg.kind == POLY_ARG_OPS ? red->arg.ops : (PolyOps)red->arg.i;
  if (rop != POLY_OP_ADD || !is_f32(red->dtype)) REJECT("not an fp32 sum");
  if (red->src[0]->op != POLY_OP_MUL) REJECT("pattern");
  /* an operand multiplied by a constant (the 2 of d(x^2)/dx in front of a backward
   * contraction) scales the whole sum: sum((c*a)*b) = c * sum(a*b) up to rounding */
  float operand_scale = 1.0f;
  PolyUOp *la = strip_cast_to_f32(strip_const_scale(red->src[0]->src[0], &operand_scale));
  PolyUOp *lb = strip_cast_to_f32(strip_const_scale(red->src[0]->src[1], &operand_scale));
  if (!is_plain_load(la) || !is_plain_load(lb)) REJECT("pattern");
  const char *dta = operand_dtype(la), *dtb = operand_dtype(lb);
  if (!dta || !dtb || strcmp(dta, dtb) != 0) REJECT("pattern");
  if (k->params[st->param]->dtype.priority != 13) REJECT("output is not fp32");

  /* epilogue: REDUCE | REDUCE + load | max(REDUCE + load, 0) | max(REDUCE, 0), and with
   * the sum scaled by a constant: load + c * REDUCE | load - c * REDUCE (the update of
   * a parameter by its gradient, reference src/instance.c:1158-1162) */
  PolyUOp *v = st->value, *addend = NULL;
  bool relu = false;
  float alpha = 1.0f;
  if (v->op == POLY_OP_MAX && const_is(v->src[1], 0.0)) {
    /* (x>0)?x:0 */
    relu = true; v = v->src[0];
  } else if (v->op == POLY_OP_WHERE && v->src[0]->op == POLY_OP_CMPLT && const_is(v->src[0]->src[0], 0.0) &&
             v->src[0]->src[1] == v->src[1] && const_is(v->src[2], 0.0)) {
    /* poly_relu: where(0 < x, x, 0) (reference src/frontend.c:582-587); same values as the MAX form */
    relu = true; v = v->src[1];
  }
  if (v->op == POLY_OP_ADD) {
    if (is_plain_load(v->src[1]) && scaled_by_const(v->src[0], red, &alpha)) addend = v->src[1];
    else if (is_plain_load(v->src[0]) && scaled_by_const(v->src[1], red, &alpha)) addend = v->src[0];
    else REJECT("pattern");
    v = red;
  } else if (v->op == POLY_OP_SUB) {
    if (!is_plain_load(v->src[0]) || !scaled_by_const(v->src[1], red, &alpha)) REJECT("pattern");
    addend = v->src[0]; alpha = -alpha;
    v = red;
  }
  if (v != red) REJECT("pattern");
  alpha *= operand_scale;
  if (alpha != 1.0f && strcmp(dta, "f32") != 0) REJECT("scaled sum of 16-bit operands");
  if (addend && !is_f32(addend->dtype)) REJECT("addend dtype");
  if (addend && (k->nodes[pb_kern_node(k, addend)].deps & ~k->nodes[pb_kern_node(k, st->u)].deps)) REJECT("pattern");

  uint64_t mask = 0, rmask = 0;
  for (int i = 0; i < st->n_loop; i++) mask |= (uint64_t)1 << st->loop[i];
  for (int i = 1; i < red->n_src; i++) { int r = pb_kern_range_id(k, red->src[i]); rmask |= (uint64_t)1 << r; }
  mask |= rmask;
  PolyUOp *exprs[4] = { st->index->src[1], load_index(la), load_index(lb), addend ? load_index(addend) : NULL };
  int ne = addend ? 4 : 3;
  VAxis va[2 * PB_MAX_AXES]; int nva; VFit fit[4];
  if (!pb_find_axes(k, mask, exprs, ne, va, &nva, fit)) REJECT("pattern");
  int params[4] = { st->param, load_param(la), load_param(lb), addend ? load_param(addend) : -1 };
  for (int i = 0; i < ne; i++) if (!in_bounds(&fit[i], va, nva, param_numel(k, params[i]))) REJECT("pattern");
  if (params[1] == params[0] || params[2] == params[0]) REJECT("pattern");
  /* an addend aliasing the output is fine only element for element */
  if (addend && params[3] == params[0]) {
    if (fit[3].offset != fit[0].offset) REJECT("pattern");
    for (int i = 0; i < nva; i++) if (fit[3].stride[i] != fit[0].stride[i]) REJECT("pattern");
  }

  PbStr ax; pb_str_init(&ax);
  int nm = 0, nn = 0, nk = 0, nb = 0;
  int64_t M = 1, N = 1, K = 1;
  for (int i = 0; i < nva; i++) {
    if (va[i].extent == 1) continue;
    int64_t sc = fit[0].stride[i], sa = fit[1].stride[i], sb = fit[2].stride[i], sx = addend ? fit[3].stride[i] : 0;
    char kind;
    if (va[i].reduce) {
      if (sc != 0 || sx != 0) { pb_str_free(&ax); REJECT("axes"); }
      if (sa == 0 || sb == 0) { pb_str_free(&ax); REJECT("axes"); }  /* not a contraction axis */
      kind = 'k'; nk++; K *= va[i].extent;
    } else {
      if (sc == 0) { pb_str_free(&ax); REJECT("axes"); }               /* several iterations write one element */
      if (sa != 0 && sb == 0) { kind = 'm'; nm++; M *= va[i].extent; }
      else if (sa == 0 && sb != 0) { kind = 'n'; nn++; N *= va[i].extent; }
      else { kind = 'b'; nb++; }
    }
    pb_str_printf(&ax, "//axis %c %lld %lld %lld %lld %lld\n", kind, (long long)va[i].extent,
                  (long long)sc, (long long)sa, (long long)sb, (long long)sx);
  }
  if (nk == 0 || nm > 4 || nn > 4 || nk > 4 || nb > 4) { pb_str_free(&ax); REJECT("axes"); }
  /* the output (and the addend) must be a strided matrix per batch entry: its
   * m axes, taken from the largest output stride down, must nest exactly, and
   * so must its n axes; operands that do not nest are packed by the runtime */
  for (int pass = 0; pass < 2; pass++) {
    int ids[2 * PB_MAX_AXES]; int n = 0;
    for (int i = 0; i < nva; i++) {
      if (va[i].extent == 1 || va[i].reduce) continue;
      int64_t sa = fit[1].stride[i], sb = fit[2].stride[i];
      bool is_m = sa != 0 && sb == 0, is_n = sa == 0 && sb != 0;
      if ((pass == 0 && is_m) || (pass == 1 && is_n)) ids[n++] = i;
    }
    for (int i = 1; i < n; i++) {
      int a = ids[i], j = i - 1;
      while (j >= 0 && fit[0].stride[ids[j]] < fit[0].stride[a]) { ids[j + 1] = ids[j]; j--; }
      ids[j + 1] = a;
    }
    for (int i = 0; i + 1 < n; i++) {
      if (fit[0].stride[ids[i]] != fit[0].stride[ids[i + 1]] * va[ids[i + 1]].extent) { pb_str_free(&ax); REJECT("axes"); }
      if (addend) {
        int64_t s0 = fit[3].stride[ids[i]], s1 = fit[3].stride[ids[i + 1]];
        if (s0 != s1 * va[ids[i + 1]].extent) { pb_str_free(&ax); REJECT("axes"); }
      }
    }
    if (n > 0 && fit[0].stride[ids[n - 1]] < 0) { pb_str_free(&ax); REJECT("axes"); }
  }
  /* tiny contractions are not worth a tiled kernel */
  if (K < 8 || M * N < 64) { pb_str_free(&ax); REJECT("axes"); }

  PbStr h; pb_str_init(&h);
  pb_str_puts(&h, "//PB200 1\n//kind gemm\n");
  pb_str_printf(&h, "//nparams %d\n", k->n_params);
  pb_str_printf(&h, "//params %d %d %d %d\n", params[0], params[1], params[2], params[3]);
  pb_str_printf(&h, "//dtype %s\n", dta);
  pb_str_printf(&h, "//offsets %lld %lld %lld %lld\n", (long long)fit[0].offset, (long long)fit[1].offset,
                (long long)fit[2].offset, (long long)(addend ? fit[3].offset : 0));
  pb_str_printf(&h, "//relu %d\n", relu ? 1 : 0);
  if (alpha != 1.0f) { uint32_t bits; memcpy(&bits, &alpha, 4); pb_str_printf(&h, "//alpha %lld\n", (long long)bits); }
  pb_str_printf(&h, "//numel %lld %lld %lld %lld\n", (long long)param_numel(k, params[0]), (long long)param_numel(k, params[1]),
                (long long)param_numel(k, params[2]), (long long)(addend ? param_numel(k, params[3]) : 0));
  /* several "//axis" lines share a key; number them */
  {
    char *p = ax.s; int idx = 0;
    while (p && *p) {
      char *eol = strchr(p, '\n');
      if (eol) *eol = 0;
      pb_str_printf(&h, "//axis%d %s\n", idx++, p + 7);
      p = eol ? eol + 1 : NULL;
    }
    pb_str_printf(&h, "//naxes %d\n", idx);
  }
  pb_str_free(&ax);
  return pb_str_take(&h);
}

/* ── transposing copy ────────────────────────────────────────────────── */
static char *classify_transpose(PbKern *k) {
  if (k->n_stores != 1 || k->n_reduce_nodes != 0 || !all_const_extents(k)) REJECT("shape");
  PbStore *st = &k->stores[0];
  if (st->index->n_src != 2 || !is_plain_load(st->value)) REJECT("not a plain copy");
  PolyUOp *ld = st->value;
  int po = st->param, pi = load_param(ld);
  if (po == pi) REJECT("in place");
  PolyDType a = k->params[po]->dtype, b = k->params[pi]->dtype;
  if (a.bitsize != 32 || b.bitsize != 32 || a.priority != b.priority) REJECT("element type");
  uint64_t mask = 0;
  for (int i = 0; i < st->n_loop; i++) mask |= (uint64_t)1 << st->loop[i];
  PolyUOp *exprs[2] = { st->index->src[1], load_index(ld) };
  VAxis va[2 * PB_MAX_AXES]; int nva; VFit fit[2];
  if (!pb_find_axes(k, mask, exprs, 2, va, &nva, fit)) REJECT("not affine");
  if (!in_bounds(&fit[0], va, nva, param_numel(k, po)) || !in_bounds(&fit[1], va, nva, param_numel(k, pi))) REJECT("bounds");
  int x = -1, y = -1;
  for (int i = 0; i < nva; i++) {
    if (va[i].extent <= 1) continue;
    if (fit[0].stride[i] == 1) x = i;
    if (fit[1].stride[i] == 1) y = i;
  }
  if (x < 0 || y < 0 || x == y) REJECT("same contiguous axis");
  if (va[x].extent < 32 || va[y].extent < 32) REJECT("small");
  if (fit[1].stride[x] <= 0 || fit[0].stride[y] <= 0) REJECT("negative stride");
  /* the store must cover distinct elements: every other axis has a non-zero output stride */
  int64_t total = 1;
  for (int i = 0; i < nva; i++) { if (va[i].extent > 1 && fit[0].stride[i] == 0) REJECT("broadcast store"); total *= va[i].extent; }
  PbStr h; pb_str_init(&h);
  pb_str_puts(&h, "//PB200 1\n//kind copy\n");
  pb_str_printf(&h, "//nparams %d\n//params %d %d\n", k->n_params, po, pi);
  pb_str_printf(&h, "//xy %lld %lld %lld %lld\n", (long long)va[x].extent, (long long)va[y].extent,
                (long long)fit[1].stride[x], (long long)fit[0].stride[y]);
  pb_str_printf(&h, "//offsets %lld %lld\n", (long long)fit[0].offset, (long long)fit[1].offset);
  PbStr bt; pb_str_init(&bt); int nb = 0;
  for (int i = 0; i < nva; i++) {
    if (i == x || i == y || va[i].extent <= 1) continue;
    pb_str_printf(&bt, " %lld %lld %lld", (long long)va[i].extent, (long long)fit[0].stride[i], (long long)fit[1].stride[i]);
    nb++;
  }
  if (nb > 6) { pb_str_free(&bt); pb_str_free(&h); REJECT("too many axes"); }
  pb_str_printf(&h, "//batch%s\n", bt.s ? bt.s : "");
  pb_str_free(&bt);
  /* whole-buffer overwrite when the strides tile [0, numel) */
  bool full = fit[0].offset == 0 && total == param_numel(k, po);
  if (full) {
    int ord[2 * PB_MAX_AXES]; int n = 0;
    for (int i = 0; i < nva; i++) if (va[i].extent > 1) ord[n++] = i;
    for (int i = 1; i < n; i++) { int v = ord[i], j = i - 1; while (j >= 0 && fit[0].stride[ord[j]] > fit[0].stride[v]) { ord[j + 1] = ord[j]; j--; } ord[j + 1] = v; }
    int64_t expect = 1;
    for (int i = 0; i < n; i++) { if (fit[0].stride[ord[i]] != expect) { full = false; break; } expect *= va[ord[i]].extent; }
  }
  pb_str_printf(&h, "//full %d\n", full ? 1 : 0);
  return pb_str_take(&h);
}

char *pb_classify_aot(PbKern *k, const char *fn_name) {
  (void)fn_name;
  char *r = classify_gather(k);
  if (r) return r;
  r = classify_scatter(k);
  if (r) return r;
  r = classify_gemm(k);
  if (r) return r;
  r = classify_transpose(k);
  if (r) return r;
  return NULL;
}
