/*
 * pb_codegen.c -- renders one scheduled polygrad kernel as CUDA C for sm_100a.
 *
 * This is the backend's general path: every kernel that is not lowered to a
 * precompiled kernel (GEMM, gather, strided copy) is rendered here and compiled
 * at plan-compile time.  It replaces the reference renderer
 * (src/render_cuda.c:196-570) and its thread mapping (src/codegen.c:4149-4218,
 * which parallelises only the outermost loop): here
 *   - every LOOP range of a store is folded into one flat 64-bit-safe thread
 *     index, ordered so that the axis with the smallest store stride varies
 *     fastest across a warp (coalesced stores and, for same-layout inputs,
 *     coalesced loads);
 *   - pure elementwise kernels whose operands are contiguous or broadcast along
 *     that axis move 128 bits per thread per access;
 *   - a kernel that is one reduction over a memory-contiguous axis gives each
 *     output to a warp or a block: lanes stride over the reduce range, partials
 *     are combined with warp shuffles and one shared-memory exchange, lane 0
 *     applies the epilogue and stores;
 *   - integer index arithmetic is integer arithmetic (the reference routes int
 *     MULACC through __fmaf_rn, src/render_cuda.c:155-158) and widens to 64 bit
 *     when a buffer or the thread count needs it;
 *   - every access of the scalar paths is bounds-checked against the PARAM's
 *     element count, so a mis-scheduled kernel cannot fault the device.
 *
 * Op semantics follow the reference CPU renderer (src/render_c.c:932-1033):
 * MAX is (a>b)?a:b, WHERE is ?:, IDIV and MOD are C division and remainder,
 * RECIPROCAL is 1/x, MULACC is a*b+c.  EXP2, LOG2, SIN and SQRT map to the CUDA
 * math library instead of the reference's polynomial decompositions
 * (src/codegen.c:2156-2679).
 */
#include "pb_kern.h"
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

typedef struct Gen Gen;
struct Gen {
  PbKern *k;
  PbStr out;
  PbStr *o;            /* where text goes: &out, or another generator's buffer */
  const char *pfx;     /* prefix of temp names (several kernels in one function) */
  char (*range_expr)[40];        /* when set: text that stands for range r */
  char (*param_expr)[24];        /* when set: name of parameter i */
  int64_t *param_numel;          /* when set: element count of parameter i as bound in this function */
  bool (*load_hook)(Gen *g, int id);  /* may emit a LOAD node itself (returns true) */
  void *ud;
  int *emitted;        /* per node: scope depth of its declaration, -1 = none */
  int *scope_log; int n_log, cap_log;
  int *scope_mark; int depth;   /* scope_mark[d] = n_log when depth d opened */
  uint64_t bound;
  bool wide;
  const char *idx_t;
  int indent;
  bool failed;
  int vec;             /* >1 while emitting the lane-replicated body of a vector kernel */
  int lane;            /* current lane when vec > 1 */
  uint64_t lane_dep;   /* mask with the bit of the vectorised range */
};

static void ind(Gen *g) { for (int i = 0; i < g->indent; i++) pb_str_puts(g->o, "  "); }

static bool is_idx_dtype(PolyDType dt) {
  return !dt.is_ptr && (dt.priority == 5 || (dt.priority == -1 && dt.bitsize == 800));
}

static const char *ctype_of(Gen *g, PolyDType dt) {
  if (is_idx_dtype(dt)) return g->idx_t;
  return pb_ctype(dt);
}

static bool is_float_dt(PolyDType dt) { return dt.priority >= 11 && dt.priority <= 14; }
static bool is_small_float(PolyDType dt) { return dt.priority == 11 || dt.priority == 12; }

/* Lane suffix: nodes that depend on the vectorised range get one temp per lane. */
static void temp_name(Gen *g, int id, char *buf, size_t cap) {
  if (g->vec > 1 && (g->k->nodes[id].deps & g->lane_dep))
    snprintf(buf, cap, "t%s%d_%d", g->pfx, id, g->lane);
  else
    snprintf(buf, cap, "t%s%d", g->pfx, id);
}

static void const_literal(Gen *g, PolyUOp *u, char *buf, size_t cap) {
  PolyDType dt = u->dtype;
  double f = 0; int64_t i = 0;
  switch (u->arg.kind) {
  case POLY_ARG_FLOAT: f = u->arg.f; i = (int64_t)u->arg.f; break;
  case POLY_ARG_INT:   i = u->arg.i; f = (double)u->arg.i; break;
  case POLY_ARG_BOOL:  i = u->arg.b; f = u->arg.b; break;
  default: break;
  }
  if (dt.priority == 0) { snprintf(buf, cap, "%s", i ? "true" : "false"); return; }
  if (dt.priority == 13) {
    float ff = (float)f; uint32_t bits; memcpy(&bits, &ff, 4);
    snprintf(buf, cap, "__int_as_float(0x%08x) /*%.9g*/", bits, (double)ff); return;
  }
  if (dt.priority == 14) {
    uint64_t bits; memcpy(&bits, &f, 8);
    snprintf(buf, cap, "__longlong_as_double(0x%016llxLL) /*%.17g*/", (unsigned long long)bits, f); return;
  }
  if (is_small_float(dt)) {
    float ff = (float)f; uint32_t bits; memcpy(&bits, &ff, 4);
    snprintf(buf, cap, "(%s)__int_as_float(0x%08x)", pb_ctype(dt), bits); return;
  }
  if (is_idx_dtype(dt)) {
    if (g->wide) snprintf(buf, cap, "%lldLL", (long long)i);
    else snprintf(buf, cap, "%lld", (long long)i);
    return;
  }
  const char *ct = pb_ctype(dt);
  if (!ct) { g->failed = true; snprintf(buf, cap, "0"); return; }
  if (poly_dtype_is_unsigned(dt)) snprintf(buf, cap, "(%s)%lluULL", ct, (unsigned long long)i);
  else snprintf(buf, cap, "(%s)%lldLL", ct, (long long)i);
}

static void ref(Gen *g, PolyUOp *u, char *buf, size_t cap) {
  switch (u->op) {
  case POLY_OP_CONST: const_literal(g, u, buf, cap); return;
  case POLY_OP_RANGE: {
    int r = pb_kern_range_id(g->k, u);
    if (g->range_expr) {
      if (g->vec > 1 && ((uint64_t)1 << r) == g->lane_dep) snprintf(buf, cap, "(%s+%d)", g->range_expr[r], g->lane);
      else snprintf(buf, cap, "%s", g->range_expr[r]);
    }
    else if (g->vec > 1 && ((uint64_t)1 << r) == g->lane_dep) snprintf(buf, cap, "(r%d+%d)", r, g->lane);
    else snprintf(buf, cap, "r%d", r);
    return;
  }
  case POLY_OP_DEFINE_VAR:
    for (int v = 0; v < g->k->n_vars; v++)
      if (g->k->vars[v] == u) { snprintf(buf, cap, "((%s)v%d)", g->idx_t, v); return; }
    g->failed = true; snprintf(buf, cap, "0"); return;
  case POLY_OP_PARAM:
    if (g->param_expr) snprintf(buf, cap, "%s", g->param_expr[u->arg.i]);
    else snprintf(buf, cap, "p%d", (int)u->arg.i);
    return;
  default: temp_name(g, pb_kern_node(g->k, u), buf, cap); return;
  }
}

static void log_emit(Gen *g, int id) {
  g->emitted[id] = g->depth;
  if (g->n_log == g->cap_log) {
    g->cap_log = g->cap_log ? g->cap_log * 2 : 256;
    g->scope_log = realloc(g->scope_log, sizeof(int) * (size_t)g->cap_log);
  }
  g->scope_log[g->n_log++] = id;
}
static void open_scope(Gen *g) { g->depth++; g->scope_mark[g->depth] = g->n_log; }
static void close_scope(Gen *g) {
  while (g->n_log > g->scope_mark[g->depth]) g->emitted[g->scope_log[--g->n_log]] = -1;
  g->depth--;
}

static void emit(Gen *g, int id);

static void emit_src(Gen *g, PolyUOp *u) {
  switch (u->op) {
  case POLY_OP_CONST: case POLY_OP_RANGE: case POLY_OP_DEFINE_VAR: case POLY_OP_PARAM: return;
  default: emit(g, pb_kern_node(g->k, u));
  }
}

static const char *reduce_identity(PolyOps op, PolyDType dt, char *buf, size_t cap, Gen *g) {
  const char *ct = ctype_of(g, dt);
  if (op == POLY_OP_ADD) snprintf(buf, cap, "(%s)0", ct);
  else if (op == POLY_OP_MUL) snprintf(buf, cap, "(%s)1", ct);
  else if (op == POLY_OP_MAX) {
    if (dt.priority == 13) snprintf(buf, cap, "__int_as_float(0xff800000)");
    else if (dt.priority == 14) snprintf(buf, cap, "(-__longlong_as_double(0x7ff0000000000000LL))");
    else if (is_small_float(dt)) snprintf(buf, cap, "(%s)__int_as_float(0xff800000)", ct);
    else if (dt.priority == 0) snprintf(buf, cap, "false");
    else if (poly_dtype_is_unsigned(dt)) snprintf(buf, cap, "(%s)0", ct);
    else if (is_idx_dtype(dt)) snprintf(buf, cap, g->wide ? "(-9223372036854775807LL-1)" : "(-2147483647-1)");
    else if (dt.priority == 7) snprintf(buf, cap, "(-9223372036854775807LL-1)");
    else if (dt.priority == 3) snprintf(buf, cap, "(short)-32768");
    else if (dt.priority == 1) snprintf(buf, cap, "(signed char)-128");
    else { g->failed = true; snprintf(buf, cap, "0"); }
  } else { g->failed = true; snprintf(buf, cap, "0"); }
  return buf;
}

static void combine_expr(PolyOps op, const char *a, const char *b, char *buf, size_t cap) {
  if (op == POLY_OP_ADD) snprintf(buf, cap, "(%s+%s)", a, b);
  else if (op == POLY_OP_MUL) snprintf(buf, cap, "(%s*%s)", a, b);
  else snprintf(buf, cap, "((%s>%s)?%s:%s)", a, b, a, b);
}

static PolyOps reduce_op(PolyUOp *u) {
  if (u->arg.kind == POLY_ARG_OPS) return u->arg.ops;
  if (u->arg.kind == POLY_ARG_INT) return (PolyOps)u->arg.i;
  if (u->arg.kind == POLY_ARG_REDUCE_AXIS) return u->arg.reduce_axis.op;
  return POLY_OP_ADD;
}

/* Emit, at the current scope, every node under `id` that can already be
 * computed (all its ranges bound): loop-invariant code motion before a loop. */
static void hoist(Gen *g, int id) {
  PbNode *n = &g->k->nodes[id];
  if (g->emitted[id] >= 0) return;
  switch (n->u->op) {
  case POLY_OP_CONST: case POLY_OP_RANGE: case POLY_OP_DEFINE_VAR: case POLY_OP_PARAM: return;
  default: break;
  }
  if ((n->deps & ~g->bound) == 0 && n->u->op != POLY_OP_INDEX) { emit(g, id); return; }
  int first = (n->u->op == POLY_OP_REDUCE) ? 1 : n->u->n_src; /* only the value of a REDUCE */
  for (int i = 0; i < (n->u->op == POLY_OP_REDUCE ? first : n->u->n_src); i++)
    hoist(g, pb_kern_node(g->k, n->u->src[i]));
}

static void range_bound_str(Gen *g, int r, char *buf, size_t cap) {
  if (g->k->extent[r] >= 0) snprintf(buf, cap, g->wide ? "%lldLL" : "%lld", (long long)g->k->extent[r]);
  else snprintf(buf, cap, "((%s)v%d)", g->idx_t, g->k->extent_var[r]);
}

static void emit_reduce_serial(Gen *g, int id) {
  PolyUOp *u = g->k->nodes[id].u;
  PolyOps op = reduce_op(u);
  int vid = pb_kern_node(g->k, u->src[0]);
  hoist(g, vid);
  char idn[96], name[32];
  temp_name(g, id, name, sizeof name);
  reduce_identity(op, u->dtype, idn, sizeof idn, g);
  ind(g); pb_str_printf(g->o, "%s acc_%s = %s;\n", ctype_of(g, u->dtype), name, idn);
  uint64_t saved = g->bound;
  for (int i = 1; i < u->n_src; i++) {
    int r = pb_kern_range_id(g->k, u->src[i]);
    char bs[64]; range_bound_str(g, r, bs, sizeof bs);
    ind(g); pb_str_printf(g->o, "for (%s r%d = 0; r%d < %s; ++r%d) {\n", g->idx_t, r, r, bs, r);
    g->indent++;
    g->bound |= (uint64_t)1 << r;
  }
  open_scope(g);
  emit_src(g, u->src[0]);
  char v[64], cmb[256], acc[48];
  ref(g, u->src[0], v, sizeof v);
  snprintf(acc, sizeof acc, "acc_%s", name);
  combine_expr(op, acc, v, cmb, sizeof cmb);
  ind(g); pb_str_printf(g->o, "%s = %s;\n", acc, cmb);
  close_scope(g);
  for (int i = 1; i < u->n_src; i++) { g->indent--; ind(g); pb_str_puts(g->o, "}\n"); }
  g->bound = saved;
  ind(g); pb_str_printf(g->o, "const %s %s = %s;\n", ctype_of(g, u->dtype), name, acc);
  log_emit(g, id);
}

static void emit_load(Gen *g, int id) {
  PolyUOp *u = g->k->nodes[id].u;
  PolyUOp *ix = u->src[0];
  if (ix->op != POLY_OP_INDEX || ix->src[0]->op != POLY_OP_PARAM) { g->failed = true; return; }
  PolyUOp *p = ix->src[0];
  emit_src(g, ix->src[1]);
  if (ix->n_src > 2) emit_src(g, ix->src[2]);
  char name[40], is[96], gs[96], pn[32];
  temp_name(g, id, name, sizeof name);
  ref(g, ix->src[1], is, sizeof is);
  ref(g, p, pn, sizeof pn);
  const char *ct = ctype_of(g, u->dtype);
  if (!ct) { g->failed = true; return; }
  long long numel = g->param_numel ? (long long)g->param_numel[p->arg.i] : (long long)p->dtype.ptr_size;
  ind(g);
  if (ix->n_src > 2) {
    ref(g, ix->src[2], gs, sizeof gs);
    pb_str_printf(g->o, "const %s %s = (%s) ? (%s)pb_ld(%s, %s, %lldLL) : (%s)0;\n",
                  ct, name, gs, ct, pn, is, numel, ct);
  } else {
    pb_str_printf(g->o, "const %s %s = (%s)pb_ld(%s, %s, %lldLL);\n",
                  ct, name, ct, pn, is, numel);
  }
  log_emit(g, id);
}

static void unary_math(Gen *g, PolyUOp *u, const char *f32, const char *f64, const char *a, char *buf, size_t cap) {
  if (u->dtype.priority == 14) snprintf(buf, cap, "%s(%s)", f64, a);
  else if (is_small_float(u->dtype)) snprintf(buf, cap, "(%s)%s((float)%s)", pb_ctype(u->dtype), f32, a);
  else snprintf(buf, cap, "%s(%s)", f32, a);
  (void)g;
}

static void emit(Gen *g, int id) {
  if (id < 0) { g->failed = true; return; }
  if (g->emitted[id] >= 0) return;
  PolyUOp *u = g->k->nodes[id].u;
  switch (u->op) {
  case POLY_OP_CONST: case POLY_OP_RANGE: case POLY_OP_DEFINE_VAR: case POLY_OP_PARAM: case POLY_OP_INDEX:
    return;
  case POLY_OP_REDUCE: emit_reduce_serial(g, id); return;
  case POLY_OP_LOAD:
    if (g->load_hook && g->load_hook(g, id)) return;
    emit_load(g, id); return;
  default: break;
  }
  for (int i = 0; i < u->n_src; i++) emit_src(g, u->src[i]);
  char a[128] = "", b[128] = "", c[128] = "", e[640], name[40];
  if (u->n_src > 0) ref(g, u->src[0], a, sizeof a);
  if (u->n_src > 1) ref(g, u->src[1], b, sizeof b);
  if (u->n_src > 2) ref(g, u->src[2], c, sizeof c);
  const char *ct = ctype_of(g, u->dtype);
  if (!ct) { g->failed = true; return; }
  PolyDType dt = u->dtype;
  switch (u->op) {
  case POLY_OP_CAST: {
    PolyDType sd = u->src[0]->dtype;
    if (is_small_float(sd) && !is_float_dt(dt)) snprintf(e, sizeof e, "(%s)(float)(%s)", ct, a);
    else if (is_small_float(dt) && !is_float_dt(sd)) snprintf(e, sizeof e, "(%s)(float)(%s)", ct, a);
    else if (is_small_float(dt) && is_small_float(sd) && dt.priority != sd.priority) snprintf(e, sizeof e, "(%s)(float)(%s)", ct, a);
    else if (dt.priority == 0 && is_float_dt(sd)) snprintf(e, sizeof e, "((float)(%s) != 0.0f)", a);
    else snprintf(e, sizeof e, "(%s)(%s)", ct, a);
    break;
  }
  case POLY_OP_BITCAST: snprintf(e, sizeof e, "pb_bitcast<%s>(%s)", ct, a); break;
  case POLY_OP_EXP2: unary_math(g, u, "exp2f", "exp2", a, e, sizeof e); break;
  case POLY_OP_LOG2: unary_math(g, u, "log2f", "log2", a, e, sizeof e); break;
  case POLY_OP_SIN:  unary_math(g, u, "sinf", "sin", a, e, sizeof e); break;
  case POLY_OP_SQRT: unary_math(g, u, "sqrtf", "sqrt", a, e, sizeof e); break;
  case POLY_OP_TRUNC: unary_math(g, u, "truncf", "trunc", a, e, sizeof e); break;
  case POLY_OP_RECIPROCAL:
    if (dt.priority == 14) snprintf(e, sizeof e, "(1.0/%s)", a);
    else if (is_small_float(dt)) snprintf(e, sizeof e, "(%s)(1.0f/(float)%s)", ct, a);
    else snprintf(e, sizeof e, "(1.0f/%s)", a);
    break;
  case POLY_OP_NEG:
    if (dt.priority == 0) snprintf(e, sizeof e, "(!%s)", a); else snprintf(e, sizeof e, "(-%s)", a);
    break;
  case POLY_OP_ADD: snprintf(e, sizeof e, "(%s+%s)", a, b); break;
  case POLY_OP_SUB: snprintf(e, sizeof e, "(%s-%s)", a, b); break;
  case POLY_OP_MUL:
    if (dt.priority == 0) snprintf(e, sizeof e, "(%s&&%s)", a, b); else snprintf(e, sizeof e, "(%s*%s)", a, b);
    break;
  case POLY_OP_FDIV: snprintf(e, sizeof e, "(%s/%s)", a, b); break;
  case POLY_OP_IDIV: snprintf(e, sizeof e, "(%s/%s)", a, b); break;
  case POLY_OP_MOD:  snprintf(e, sizeof e, "(%s%%%s)", a, b); break;
  case POLY_OP_SHL:  snprintf(e, sizeof e, "(%s<<%s)", a, b); break;
  case POLY_OP_SHR:  snprintf(e, sizeof e, "(%s>>%s)", a, b); break;
  case POLY_OP_AND:  snprintf(e, sizeof e, dt.priority == 0 ? "(%s&&%s)" : "(%s&%s)", a, b); break;
  case POLY_OP_OR:   snprintf(e, sizeof e, dt.priority == 0 ? "(%s||%s)" : "(%s|%s)", a, b); break;
  case POLY_OP_XOR:  snprintf(e, sizeof e, dt.priority == 0 ? "(%s!=%s)" : "(%s^%s)", a, b); break;
  case POLY_OP_CMPLT: snprintf(e, sizeof e, "(%s<%s)", a, b); break;
  case POLY_OP_CMPNE: snprintf(e, sizeof e, "(%s!=%s)", a, b); break;
  case POLY_OP_CMPEQ: snprintf(e, sizeof e, "(%s==%s)", a, b); break;
  case POLY_OP_MAX:  snprintf(e, sizeof e, "((%s>%s)?%s:%s)", a, b, a, b); break;
  case POLY_OP_POW:
    if (dt.priority == 14) snprintf(e, sizeof e, "pow(%s,%s)", a, b);
    else snprintf(e, sizeof e, "(%s)powf((float)%s,(float)%s)", ct, a, b);
    break;
  case POLY_OP_WHERE: {
    PolyDType cd = u->src[0]->dtype;
    if (is_small_float(cd)) snprintf(e, sizeof e, "(((float)%s != 0.0f)?%s:%s)", a, b, c);
    else snprintf(e, sizeof e, "(%s?%s:%s)", a, b, c);
    break;
  }
  case POLY_OP_MULACC:
    if (dt.priority == 13) snprintf(e, sizeof e, "fmaf(%s,%s,%s)", a, b, c);
    else if (dt.priority == 14) snprintf(e, sizeof e, "fma(%s,%s,%s)", a, b, c);
    else snprintf(e, sizeof e, "((%s*%s)+%s)", a, b, c);
    break;
  default:
    snprintf(g->k->err, sizeof g->k->err, "no rendering for %s", poly_op_name(u->op));
    g->failed = true; return;
  }
  temp_name(g, id, name, sizeof name);
  ind(g); pb_str_printf(g->o, "const %s %s = %s;\n", ct, name, e);
  log_emit(g, id);
}

/* ── launch-size expression: product of constants and var arguments ──── */
static void size_expr(PbKern *k, const int *ranges, int n, PbStr *s) {
  int64_t c = 1; bool any_var = false;
  for (int i = 0; i < n; i++) {
    int r = ranges[i];
    if (k->extent[r] >= 0) c *= k->extent[r];
  }
  pb_str_printf(s, "c%lld", (long long)c);
  for (int i = 0; i < n; i++) {
    int r = ranges[i];
    if (k->extent[r] < 0) { pb_str_printf(s, "*v%d", k->extent_var[r]); any_var = true; }
  }
  (void)any_var;
}

static int64_t range_max(const PbKern *k, int r) {
  return k->extent[r] >= 0 ? k->extent[r] : k->vars[k->extent_var[r]]->arg.define_var.max_val;
}

/* Order a store's loop axes: smallest |store stride| first (fastest thread axis). */
static void order_loop_axes(PbKern *k, PbStore *st, int *order, PbAffine *aff_out) {
  uint64_t m = 0;
  for (int i = 0; i < st->n_loop; i++) m |= (uint64_t)1 << st->loop[i];
  PbAffine aff;
  pb_fit_affine(k, st->index->src[1], m, &aff);
  for (int i = 0; i < st->n_loop; i++) order[i] = st->loop[i];
  if (aff.ok) {
    for (int i = 1; i < st->n_loop; i++) {
      int r = order[i]; int j = i - 1;
      int64_t sr = llabs(aff.stride[r]); if (sr == 0) sr = INT64_MAX;
      while (j >= 0) {
        int64_t sj = llabs(aff.stride[order[j]]); if (sj == 0) sj = INT64_MAX;
        if (sj <= sr) break;
        order[j + 1] = order[j]; j--;
      }
      order[j + 1] = r;
    }
  }
  if (aff_out) *aff_out = aff;
}

static void emit_decompose(Gen *g, const char *lin, const int *order, int n) {
  ind(g); pb_str_printf(g->o, "%s rem_ = %s;\n", g->idx_t, lin);
  for (int i = 0; i < n; i++) {
    int r = order[i];
    char bs[64]; range_bound_str(g, r, bs, sizeof bs);
    ind(g);
    if (i == n - 1) pb_str_printf(g->o, "const %s r%d = rem_;\n", g->idx_t, r);
    else pb_str_printf(g->o, "const %s r%d = rem_ %% %s; rem_ /= %s;\n", g->idx_t, r, bs, bs);
    g->bound |= (uint64_t)1 << r;
  }
}

static void emit_store(Gen *g, PbStore *st) {
  PolyUOp *ix = st->index;
  emit_src(g, ix->src[1]);
  if (ix->n_src > 2) emit_src(g, ix->src[2]);
  emit_src(g, st->value);
  char is[64], vs[96], gs[64];
  ref(g, ix->src[1], is, sizeof is);
  ref(g, st->value, vs, sizeof vs);
  PolyUOp *p = ix->src[0];
  PolyDType base = p->dtype; base.is_ptr = false; base.count = 1;
  const char *pt = pb_ctype(base);
  ind(g);
  if (ix->n_src > 2) {
    ref(g, ix->src[2], gs, sizeof gs);
    pb_str_printf(g->o, "if (%s) pb_st(p%d, %s, %lldLL, (%s)(%s));\n", gs, st->param, is,
                  (long long)p->dtype.ptr_size, pt, vs);
  } else {
    pb_str_printf(g->o, "pb_st(p%d, %s, %lldLL, (%s)(%s));\n", st->param, is,
                  (long long)p->dtype.ptr_size, pt, vs);
  }
}

static const char *PRELUDE =
  "template <class T> __device__ __forceinline__ T pb_ld(const T* __restrict__ p, long long i, long long n) {\n"
  "  return ((unsigned long long)i < (unsigned long long)n) ? p[i] : T(0);\n"
  "}\n"
  "template <class T> __device__ __forceinline__ void pb_st(T* __restrict__ p, long long i, long long n, T v) {\n"
  "  if ((unsigned long long)i < (unsigned long long)n) p[i] = v;\n"
  "}\n"
  "template <class T, class S> __device__ __forceinline__ T pb_bitcast(S s) {\n"
  "  static_assert(sizeof(T) == sizeof(S), \"bitcast size\");\n"
  "  T t; memcpy(&t, &s, sizeof(T)); return t;\n"
  "}\n";

/* Parameter (index + 1) whose buffer holds bfloat16 although the kernel computes
 * its value as float; 0 = none.  Set around one render call only. */
static int s_bf16_out_param1 = 0;

static void emit_signature(Gen *g, const bool *written, int block) {
  PbKern *k = g->k;
  pb_str_printf(g->o, "extern \"C\" __global__ void __launch_bounds__(%d) pb200_kernel(", block);
  bool first = true;
  for (int i = 0; i < k->n_params; i++) {
    if (!first) pb_str_puts(g->o, ", ");
    first = false;
    if (!k->params[i]) { pb_str_printf(g->o, "const void* __restrict__ p%d", i); continue; }
    PolyDType base = k->params[i]->dtype; base.is_ptr = false; base.count = 1;
    const char *ct = pb_ctype(base);
    if (!ct) { g->failed = true; ct = "float"; }
    if (s_bf16_out_param1 == i + 1) ct = "__nv_bfloat16";
    pb_str_printf(g->o, "%s%s* __restrict__ p%d", written[i] ? "" : "const ", ct, i);
  }
  for (int v = 0; v < k->n_vars; v++) {
    if (!first) pb_str_puts(g->o, ", ");
    first = false;
    pb_str_printf(g->o, "const int v%d", v);
  }
  if (!first) pb_str_puts(g->o, ", ");
  pb_str_puts(g->o, "const long long n_work)");
}

/* Which params are read (bit 0) / written (bit 1), and whether the write covers
 * the whole buffer exactly once (bit 2). */
static void param_usage(PbKern *k, int *usage) {
  for (int i = 0; i < k->n_params; i++) usage[i] = 0;
  for (int i = 0; i < k->n_nodes; i++) {
    PolyUOp *u = k->nodes[i].u;
    if (u->op == POLY_OP_LOAD && u->src[0]->op == POLY_OP_INDEX && u->src[0]->src[0]->op == POLY_OP_PARAM)
      usage[u->src[0]->src[0]->arg.i] |= 1;
  }
  for (int s = 0; s < k->n_stores; s++) {
    PbStore *st = &k->stores[s];
    usage[st->param] |= 2;
    if (st->index->n_src > 2) continue;           /* gated store: partial */
    uint64_t m = 0; int64_t total = 1; bool var = false;
    for (int i = 0; i < st->n_loop; i++) {
      m |= (uint64_t)1 << st->loop[i];
      if (k->extent[st->loop[i]] < 0) var = true; else total *= k->extent[st->loop[i]];
    }
    if (var) continue;
    PbAffine aff; pb_fit_affine(k, st->index->src[1], m, &aff);
    if (!aff.ok || aff.offset != 0) continue;
    if (total != k->params[st->param]->dtype.ptr_size) continue;
    /* strides must be a permutation of a dense layout: sort by stride, check products */
    int ord[PB_MAX_AXES]; int n = 0;
    for (int i = 0; i < st->n_loop; i++) if (k->extent[st->loop[i]] > 1) ord[n++] = st->loop[i];
    for (int i = 1; i < n; i++) {
      int r = ord[i], j = i - 1;
      while (j >= 0 && aff.stride[ord[j]] > aff.stride[r]) { ord[j + 1] = ord[j]; j--; }
      ord[j + 1] = r;
    }
    int64_t expect = 1; bool dense = true;
    for (int i = 0; i < n; i++) {
      if (aff.stride[ord[i]] != expect) { dense = false; break; }
      expect *= k->extent[ord[i]];
    }
    if (dense) usage[st->param] |= 4;
  }
}

static void emit_header(PbKern *k, PbStr *h, const char *launch_line, const int *usage) {
  pb_str_puts(h, "//PB200 1\n//kind jit\n//entry pb200_kernel\n");
  pb_str_printf(h, "//nparams %d\n//nvars %d\n", k->n_params, k->n_vars);
  pb_str_printf(h, "%s\n", launch_line);
  pb_str_puts(h, "//rw");
  for (int i = 0; i < k->n_params; i++) {
    const char *c = "-";
    if ((usage[i] & 3) == 1) c = "r";
    else if ((usage[i] & 3) == 3) c = "rw";
    else if (usage[i] & 4) c = "W";
    else if (usage[i] & 2) c = "w";
    pb_str_printf(h, " %s", c);
  }
  pb_str_puts(h, "\n");
}

/* ── collect the loads feeding a value (for layout decisions) ────────── */
typedef struct { int node; PbAffine aff; } LoadInfo;

static int collect_loads(PbKern *k, int id, LoadInfo *out, int cap, int n, bool *seen) {
  if (seen[id]) return n;
  seen[id] = true;
  PolyUOp *u = k->nodes[id].u;
  if (u->op == POLY_OP_LOAD) {
    if (n < cap) { out[n].node = id; n++; }
  }
  for (int i = 0; i < u->n_src; i++) {
    int s = pb_kern_node(k, u->src[i]);
    if (s >= 0) n = collect_loads(k, s, out, cap, n, seen);
  }
  return n;
}

/* ── reduction kernel: one warp or one block per output element ──────── */
static bool reduce_dtype_ok(PolyDType dt) {
  return dt.priority == 13 || dt.priority == 14 || dt.priority == 5 || dt.priority == 7 ||
         dt.priority == 6 || dt.priority == 8 || (dt.priority == -1 && dt.bitsize == 800);
}

static char *render_group_reduce(PbKern *k, const int *usage) {
  if (k->n_stores != 1 || k->n_reduce_nodes < 1 || k->n_reduce_nodes > 2) return NULL;
  PbStore *st = &k->stores[0];
  int rid = -1;
  for (int i = 0; i < k->n_nodes; i++) if (k->nodes[i].u->op == POLY_OP_REDUCE) rid = i;   /* sources come first: the outer one */
  PolyUOp *red = k->nodes[rid].u;
  if (!reduce_dtype_ok(red->dtype)) return NULL;
  PolyOps op = reduce_op(red);
  if (op != POLY_OP_ADD && op != POLY_OP_MAX && op != POLY_OP_MUL) return NULL;
  /* the REDUCE must feed the store value, not the store index or gate */
  if (k->nodes[pb_kern_node(k, st->index)].has_reduce) return NULL;
  /* a reduction of a reduction with the same operation (x.sum(-1).sum(-1)) is one reduction over
   * the axes of both */
  PolyUOp *inner = NULL;
  if (k->n_reduce_nodes == 2) {
    inner = red->src[0];
    if (inner->op != POLY_OP_REDUCE || reduce_op(inner) != op || !poly_dtype_eq(inner->dtype, red->dtype) ||
        k->nodes[pb_kern_node(k, inner)].n_uses != 1) return NULL;
  }
  PolyUOp *val = inner ? inner->src[0] : red->src[0];

  int raxes[PB_MAX_AXES]; int nr = 0; int64_t ktot = 1;
  uint64_t rmask = 0;
  for (int pass = 0; pass < (inner ? 2 : 1); pass++) {
    PolyUOp *from = pass == 0 ? red : inner;
    for (int i = 1; i < from->n_src; i++) {
      int r = pb_kern_range_id(k, from->src[i]);
      if (r < 0 || nr >= PB_MAX_AXES) return NULL;
      if (k->extent[r] < 0) return NULL;
      raxes[nr++] = r; ktot *= k->extent[r]; rmask |= (uint64_t)1 << r;
    }
  }
  if (ktot < 64) return NULL;

  /* loads under the reduction: is there one that is contiguous along a reduce axis? */
  bool *seen = calloc((size_t)k->n_nodes, 1);
  LoadInfo loads[32];
  int nl = collect_loads(k, pb_kern_node(k, val), loads, 32, 0, seen);
  free(seen);
  uint64_t all = 0;
  for (int r = 0; r < k->n_ranges; r++) all |= (uint64_t)1 << r;
  int fastest = -1; int64_t best = INT64_MAX;
  int64_t loop_best = INT64_MAX;      /* smallest stride any loop axis has in a reduce-dependent load */
  int64_t mat_best = INT64_MAX;       /* smallest reduce-axis stride among loads that also walk an output axis */
  for (int i = 0; i < nl; i++) {
    PolyUOp *ld = k->nodes[loads[i].node].u;
    if (!(k->nodes[loads[i].node].deps & rmask)) continue;
    pb_fit_affine(k, ld->src[0]->src[1], all, &loads[i].aff);
    if (!loads[i].aff.ok) {
      /* an index with div/mod of a flattened output range is not affine; what decides
       * coalescing is how far the address moves for one step of each axis, so take the
       * unit-step differences at the origin in place of strides (static extents only) */
      int64_t v0[PB_MAX_RANGES] = {0}, base;
      if (k->n_vars != 0 || !pb_eval_int(k, ld->src[0]->src[1], v0, NULL, &base)) continue;
      bool probed = true;
      for (int r = 0; r < k->n_ranges && probed; r++) {
        loads[i].aff.stride[r] = 0;
        if (!(all >> r & 1) || k->extent[r] < 2) continue;
        int64_t v1[PB_MAX_RANGES] = {0}, at;
        v1[r] = 1;
        if (!pb_eval_int(k, ld->src[0]->src[1], v1, NULL, &at)) probed = false;
        else loads[i].aff.stride[r] = at - base;
      }
      if (!probed) continue;
    }
    bool matrix = false;          /* walks an output axis as well: a matrix operand, not a per-row vector */
    for (int j = 0; j < st->n_loop; j++)
      if (loads[i].aff.stride[st->loop[j]] != 0 && range_max(k, st->loop[j]) > 1) matrix = true;
    for (int j = 0; j < nr; j++) {
      int64_t s = llabs(loads[i].aff.stride[raxes[j]]);
      if (s != 0 && k->extent[raxes[j]] > 1 && s < best) { best = s; fastest = raxes[j]; }
      if (matrix && s != 0 && k->extent[raxes[j]] > 1 && s < mat_best) mat_best = s;
    }
    for (int j = 0; j < st->n_loop; j++) {
      int64_t s = llabs(loads[i].aff.stride[st->loop[j]]);
      if (s != 0 && range_max(k, st->loop[j]) > 1 && s < loop_best) loop_best = s;
    }
  }
  if (fastest < 0) return NULL;
  /* vectors indexed by the reduce axes alone (per-row statistics) are contiguous along them but
   * small; when every matrix operand is strided along the reduce axes and contiguous along an
   * output axis, a thread per output is the coalesced mapping */
  int64_t n_out_max = 1;
  for (int i = 0; i < st->n_loop; i++) n_out_max *= range_max(k, st->loop[i]);
  /* A thread per output is the coalesced mapping when an output axis is the memory-contiguous
   * one and no reduce axis is -- but only with enough outputs to fill the machine: a bias
   * gradient (a few hundred outputs, each a sum over every token) is a handful of blocks walking
   * long serial loops there, and far faster with a warp per output even though its loads stride. */
  const bool enough_outputs = n_out_max >= 32768;
  if (enough_outputs && best != 1 && loop_best == 1) return NULL;
  if (enough_outputs && mat_best != INT64_MAX && mat_best != 1 && loop_best == 1) return NULL;

  int group, block;
  if (ktot >= 2048 || n_out_max < 2048) { group = ktot >= 8192 ? 512 : 256; if (ktot < 512) group = 128; block = group; }
  else { group = 32; block = 256; }

  /* A few outputs, each a very long reduction (a loss: one scalar over every logit), would occupy
   * a few SMs.  The reduction is then cut into `split` interleaved parts, one block each; a block
   * leaves its partial result in module-scope memory and takes a ticket, and the block that draws
   * the last ticket combines the partials in index order (so the result does not depend on which
   * block finishes when), applies the rest of the kernel and resets the ticket counter. */
  int split = 1;
  {
    const char *e = getenv("POLY_B200_SPLIT_REDUCE");
    if (!(e && e[0] == '0') && group == block && k->n_vars == 0 && n_out_max <= 256 && ktot >= ((int64_t)1 << 17)) {
      int64_t want = (148 * 4 + n_out_max - 1) / n_out_max, by_len = ktot / ((int64_t)group * 16);
      if (want > by_len) want = by_len;
      if (want > 1024) want = 1024;
      if (want >= 2) split = (int)want;
    }
  }

  Gen g; memset(&g, 0, sizeof g);
  g.k = k;
  g.emitted = malloc(sizeof(int) * (size_t)k->n_nodes);
  for (int i = 0; i < k->n_nodes; i++) g.emitted[i] = -1;
  g.scope_mark = calloc(64, sizeof(int));
  bool wide = n_out_max * (int64_t)group >= ((int64_t)1 << 31);
  for (int i = 0; i < k->n_params; i++)
    if (k->params[i] && k->params[i]->dtype.ptr_size >= ((int64_t)1 << 31)) wide = true;
  g.wide = wide; g.idx_t = wide ? "long long" : "int";
  pb_str_init(&g.out); g.o = &g.out; g.pfx = "";

  bool written[PB_MAX_PARAMS];
  for (int i = 0; i < k->n_params; i++) written[i] = (usage[i] & 2) != 0;

  const char *rt = ctype_of(&g, red->dtype);
  pb_str_puts(g.o, PRELUDE);
  if (split > 1) {
    pb_str_printf(g.o, "__device__ %s part_[%lld];\n__device__ unsigned int ticket_[%lld];\n", rt,
                  (long long)(n_out_max * split), (long long)n_out_max);
  }
  emit_signature(&g, written, block);
  pb_str_puts(g.o, " {\n");
  g.indent = 1;
  int per_block = block / group;
  ind(&g); pb_str_printf(g.o, "const int lane_ = threadIdx.x %% %d;\n", group);
  if (split > 1) {
    ind(&g); pb_str_printf(g.o, "const int split_ = blockIdx.x %% %d;\n", split);
    ind(&g); pb_str_printf(g.o, "const long long out_ = blockIdx.x / %d;\n", split);
  } else {
    ind(&g); pb_str_printf(g.o, "const long long out_ = (long long)blockIdx.x * %d + threadIdx.x / %d;\n", per_block, group);
  }
  if (group == block) { ind(&g); pb_str_printf(g.o, "__shared__ %s red_[32];\n", rt); }
  /* whole groups leave together, so the shuffles below always see full warps */
  if (split > 1) { ind(&g); pb_str_puts(g.o, "if (blockIdx.x >= n_work) return;\n"); }
  else { ind(&g); pb_str_puts(g.o, "if (out_ >= n_work) return;\n"); }
  int order[PB_MAX_AXES];
  order_loop_axes(k, st, order, NULL);
  if (st->n_loop > 0) emit_decompose(&g, wide ? "out_" : "(int)out_", order, st->n_loop);

  /* loop-invariant part of the reduced value */
  int vid = pb_kern_node(k, val);
  hoist(&g, vid);

  char idn[96];
  reduce_identity(op, red->dtype, idn, sizeof idn, &g);
  ind(&g); pb_str_printf(g.o, "%s acc_ = %s;\n", rt, idn);
  /* reduce axes: the contiguous one fastest */
  int rorder[PB_MAX_AXES]; int n = 0;
  rorder[n++] = fastest;
  for (int j = nr - 1; j >= 0; j--) if (raxes[j] != fastest) rorder[n++] = raxes[j];
  if (split > 1) {
    ind(&g); pb_str_printf(g.o, "for (long long kk_ = (long long)split_ * %d + lane_; kk_ < %lldLL; kk_ += %lldLL) {\n",
                           group, (long long)ktot, (long long)group * split);
    ind(&g); pb_str_printf(g.o, "  const %s k_ = (%s)kk_;\n", g.idx_t, g.idx_t);
  } else {
    ind(&g); pb_str_printf(g.o, "for (%s k_ = lane_; k_ < %lld; k_ += %d) {\n", g.idx_t, (long long)ktot, group);
  }
  g.indent++;
  uint64_t saved = g.bound;
  open_scope(&g);
  if (nr == 1) {
    ind(&g); pb_str_printf(g.o, "const %s r%d = k_;\n", g.idx_t, fastest);
    g.bound |= (uint64_t)1 << fastest;
  } else {
    emit_decompose(&g, "k_", rorder, nr);
  }
  emit_src(&g, val);
  char v[64], cmb[256];
  ref(&g, val, v, sizeof v);
  combine_expr(op, "acc_", v, cmb, sizeof cmb);
  ind(&g); pb_str_printf(g.o, "acc_ = %s;\n", cmb);
  close_scope(&g);
  g.bound = saved;
  g.indent--;
  ind(&g); pb_str_puts(g.o, "}\n");

  /* combine across the group */
  char sh[256];
  ind(&g); pb_str_puts(g.o, "#pragma unroll\n");
  ind(&g); pb_str_puts(g.o, "for (int o_ = 16; o_ > 0; o_ >>= 1) {\n");
  ind(&g); pb_str_printf(g.o, "  const %s x_ = __shfl_xor_sync(0xffffffffu, acc_, o_);\n", rt);
  combine_expr(op, "acc_", "x_", sh, sizeof sh);
  ind(&g); pb_str_printf(g.o, "  acc_ = %s;\n", sh);
  ind(&g); pb_str_puts(g.o, "}\n");
  if (group == block) {
    int nw = block / 32;
    ind(&g); pb_str_puts(g.o, "if ((threadIdx.x & 31) == 0) red_[threadIdx.x >> 5] = acc_;\n");
    ind(&g); pb_str_puts(g.o, "__syncthreads();\n");
    ind(&g); pb_str_puts(g.o, "if (threadIdx.x != 0) return;\n");
    ind(&g); pb_str_puts(g.o, "acc_ = red_[0];\n");
    ind(&g); pb_str_printf(g.o, "for (int w_ = 1; w_ < %d; ++w_) { const %s x_ = red_[w_]; acc_ = %s; }\n", nw, rt, sh);
    if (split > 1) {
      ind(&g); pb_str_printf(g.o, "part_[out_ * %d + split_] = acc_;\n", split);
      ind(&g); pb_str_puts(g.o, "__threadfence();\n");
      ind(&g); pb_str_printf(g.o, "if (atomicAdd(&ticket_[out_], 1u) != %du) return;\n", split - 1);
      ind(&g); pb_str_puts(g.o, "__threadfence();\n");
      ind(&g); pb_str_printf(g.o, "const volatile %s* vp_ = part_ + out_ * %d;\n", rt, split);
      ind(&g); pb_str_puts(g.o, "acc_ = vp_[0];\n");
      ind(&g); pb_str_printf(g.o, "for (int w_ = 1; w_ < %d; ++w_) { const %s x_ = vp_[w_]; acc_ = %s; }\n", split, rt, sh);
      ind(&g); pb_str_puts(g.o, "ticket_[out_] = 0u;\n");
    }
  } else {
    ind(&g); pb_str_puts(g.o, "if (lane_ != 0) return;\n");
  }
  char name[32]; temp_name(&g, rid, name, sizeof name);
  ind(&g); pb_str_printf(g.o, "const %s %s = acc_;\n", rt, name);
  log_emit(&g, rid);
  emit_store(&g, st);
  pb_str_puts(g.o, "}\n");

  char *res = NULL;
  if (!g.failed) {
    PbStr h; pb_str_init(&h);
    PbStr sz; pb_str_init(&sz);
    size_expr(k, st->loop, st->n_loop, &sz);
    char line[512];
    if (split > 1) snprintf(line, sizeof line, "//launch group block=%d group=%d work=c%lld", block, group, (long long)(n_out_max * split));
    else snprintf(line, sizeof line, "//launch group block=%d group=%d work=%s", block, group, sz.s);
    pb_str_free(&sz);
    emit_header(k, &h, line, usage);
    if (k->uses_half) pb_str_puts(&h, "#include <cuda_fp16.h>\n");
    if (k->uses_bf16) pb_str_puts(&h, "#include <cuda_bf16.h>\n");
    pb_str_puts(&h, g.out.s);
    res = pb_str_take(&h);
  }
  pb_str_free(&g.out);
  free(g.emitted); free(g.scope_log); free(g.scope_mark);
  return res;
}

/* ── vectorised elementwise kernel ───────────────────────────────────── */
/* Conditions: one store, no REDUCE, all extents constant, the fastest store
 * axis x has store stride 1 and extent % 4 == 0, every load is affine with
 * stride 1 or 0 along x, and every other stride and offset of a stride-1
 * operand keeps 16-byte alignment.  All element types 4 bytes wide.
 * Each thread handles 4 consecutive x; grid-stride is not needed because the
 * grid covers the element count exactly. */
static char *render_vec_elementwise(PbKern *k, const int *usage) {
  if (k->n_stores != 1 || k->n_reduce_nodes != 0 || k->n_vars != 0) return NULL;
  PbStore *st = &k->stores[0];
  if (st->index->n_src > 2 || st->n_loop == 0) return NULL;
  for (int i = 0; i < st->n_loop; i++) if (k->extent[st->loop[i]] < 0) return NULL;
  int order[PB_MAX_AXES]; PbAffine saff;
  order_loop_axes(k, st, order, &saff);
  if (!saff.ok) return NULL;
  int x = -1;
  for (int i = 0; i < st->n_loop; i++) if (k->extent[order[i]] > 1) { x = order[i]; break; }
  if (x < 0 || saff.stride[x] != 1 || k->extent[x] % 4 != 0) return NULL;
  uint64_t m = 0;
  for (int i = 0; i < st->n_loop; i++) m |= (uint64_t)1 << st->loop[i];
  PolyDType ob = k->params[st->param]->dtype;
  if (ob.bitsize != 32 || (ob.priority != 13 && ob.priority != 5 && ob.priority != 6)) return NULL;
  const bool out_bf16 = s_bf16_out_param1 == st->param + 1;
  if (s_bf16_out_param1 && (!out_bf16 || ob.priority != 13)) return NULL;
  if (saff.offset % 4) return NULL;
  for (int i = 0; i < st->n_loop; i++) if (st->loop[i] != x && saff.stride[st->loop[i]] % 4) return NULL;

  bool *seen = calloc((size_t)k->n_nodes, 1);
  LoadInfo loads[24];
  int nl = collect_loads(k, pb_kern_node(k, st->value), loads, 24, 0, seen);
  free(seen);
  if (nl >= 24) return NULL;
  bool vec_load[24], rev_load[24];
  for (int i = 0; i < nl; i++) {
    PolyUOp *ld = k->nodes[loads[i].node].u;
    PolyUOp *ix = ld->src[0];
    if (ix->op != POLY_OP_INDEX || ix->src[0]->op != POLY_OP_PARAM || ix->n_src > 2) return NULL;
    if (ix->src[0]->dtype.bitsize != 32) return NULL;
    if ((int)ix->src[0]->arg.i == st->param) {
      if (out_bf16) return NULL;
      /* reading the buffer being written is only safe element-for-element */
      pb_fit_affine(k, ix->src[1], m, &loads[i].aff);
      if (!loads[i].aff.ok) return NULL;
      if (loads[i].aff.offset != saff.offset) return NULL;
      for (int j = 0; j < st->n_loop; j++)
        if (loads[i].aff.stride[st->loop[j]] != saff.stride[st->loop[j]]) return NULL;
    }
    pb_fit_affine(k, ix->src[1], m, &loads[i].aff);
    if (!loads[i].aff.ok) return NULL;
    int64_t sx = loads[i].aff.stride[x];
    rev_load[i] = false;
    if (sx == 1) {
      if (loads[i].aff.offset % 4) return NULL;
      for (int j = 0; j < st->n_loop; j++)
        if (st->loop[j] != x && loads[i].aff.stride[st->loop[j]] % 4) return NULL;
      vec_load[i] = true;
    } else if (sx == -1) {
      /* a flipped axis: elements x..x+3 are the 4 words ending at offset - x, reversed */
      if ((loads[i].aff.offset - 3) % 4) return NULL;
      for (int j = 0; j < st->n_loop; j++)
        if (st->loop[j] != x && loads[i].aff.stride[st->loop[j]] % 4) return NULL;
      vec_load[i] = true; rev_load[i] = true;
    } else if (sx == 0) vec_load[i] = false;
    else return NULL;
    /* bounds: the largest index must stay inside the buffer */
    int64_t lo = loads[i].aff.offset, hi = loads[i].aff.offset;
    for (int j = 0; j < st->n_loop; j++) {
      int64_t s = loads[i].aff.stride[st->loop[j]] * (k->extent[st->loop[j]] - 1);
      if (s > 0) hi += s; else lo += s;
    }
    if (lo < 0 || hi >= ix->src[0]->dtype.ptr_size) return NULL;
  }
  {
    int64_t lo = saff.offset, hi = saff.offset;
    for (int j = 0; j < st->n_loop; j++) {
      int64_t s = saff.stride[st->loop[j]] * (k->extent[st->loop[j]] - 1);
      if (s > 0) hi += s; else lo += s;
    }
    if (lo < 0 || hi >= ob.ptr_size) return NULL;
  }

  int64_t total = 1;
  for (int i = 0; i < st->n_loop; i++) total *= k->extent[st->loop[i]];
  int64_t n_threads = total / 4;

  Gen g; memset(&g, 0, sizeof g);
  g.k = k;
  g.emitted = malloc(sizeof(int) * (size_t)k->n_nodes);
  for (int i = 0; i < k->n_nodes; i++) g.emitted[i] = -1;
  g.scope_mark = calloc(64, sizeof(int));
  bool wide = total >= ((int64_t)1 << 31);
  for (int i = 0; i < k->n_params; i++)
    if (k->params[i] && k->params[i]->dtype.ptr_size >= ((int64_t)1 << 31)) wide = true;
  g.wide = wide; g.idx_t = wide ? "long long" : "int";
  pb_str_init(&g.out); g.o = &g.out; g.pfx = "";
  bool written[PB_MAX_PARAMS];
  for (int i = 0; i < k->n_params; i++) written[i] = (usage[i] & 2) != 0;

  pb_str_puts(g.o, PRELUDE);
  pb_str_puts(g.o,
    "template <class T> struct pb_v4 { T x, y, z, w; };\n"
    "template <class T> __device__ __forceinline__ void pb_ld4(const T* p, T* o) {\n"
    "  const uint4 v = *reinterpret_cast<const uint4*>(p);\n"
    "  memcpy(o, &v, 16);\n"
    "}\n"
    "template <class T> __device__ __forceinline__ void pb_ld4r(const T* p, T* o) {\n"
    "  const uint4 v = *reinterpret_cast<const uint4*>(p);\n"
    "  T t[4]; memcpy(t, &v, 16); o[0] = t[3]; o[1] = t[2]; o[2] = t[1]; o[3] = t[0];\n"
    "}\n"
    "template <class T> __device__ __forceinline__ void pb_st4(T* p, const T* o) {\n"
    "  uint4 v; memcpy(&v, o, 16);\n"
    "  *reinterpret_cast<uint4*>(p) = v;\n"
    "}\n");
  emit_signature(&g, written, 256);
  pb_str_puts(g.o, " {\n");
  g.indent = 1;
  ind(&g); pb_str_puts(g.o, "const long long gid_ = (long long)blockIdx.x * blockDim.x + threadIdx.x;\n");
  ind(&g); pb_str_puts(g.o, "if (gid_ >= n_work) return;\n");
  /* decompose: x in units of 4 */
  ind(&g); pb_str_printf(g.o, "%s rem_ = %s;\n", g.idx_t, wide ? "gid_" : "(int)gid_");
  for (int i = 0; i < st->n_loop; i++) {
    int r = order[i];
    int64_t ext = (r == x) ? k->extent[r] / 4 : k->extent[r];
    ind(&g);
    if (i == st->n_loop - 1) pb_str_printf(g.o, "const %s q%d = rem_;\n", g.idx_t, r);
    else pb_str_printf(g.o, "const %s q%d = rem_ %% %lld; rem_ /= %lld;\n", g.idx_t, r, (long long)ext, (long long)ext);
    ind(&g);
    if (r == x) pb_str_printf(g.o, "const %s r%d = q%d * 4;\n", g.idx_t, r, r);
    else pb_str_printf(g.o, "const %s r%d = q%d;\n", g.idx_t, r, r);
    g.bound |= (uint64_t)1 << r;
  }
  /* vector loads first (independent, so they are all in flight together) */
  for (int i = 0; i < nl; i++) {
    if (!vec_load[i]) continue;
    PolyUOp *ld = k->nodes[loads[i].node].u;
    PolyUOp *ix = ld->src[0];
    PolyDType base = ix->src[0]->dtype; base.is_ptr = false; base.count = 1;
    const char *pt = pb_ctype(base);
    ind(&g); pb_str_printf(g.o, "%s l%d_[4]; { %s o_ = %lld", pt, loads[i].node, g.idx_t,
                           (long long)(loads[i].aff.offset - (rev_load[i] ? 3 : 0)));
    for (int j = 0; j < st->n_loop; j++) {
      int64_t s = loads[i].aff.stride[st->loop[j]];
      if (s) pb_str_printf(g.o, " + r%d*%lld", st->loop[j], (long long)s);
    }
    if (rev_load[i]) pb_str_printf(g.o, "; pb_ld4r(p%d + o_, l%d_); }\n", (int)ix->src[0]->arg.i, loads[i].node);
    else pb_str_printf(g.o, "; pb_ld4(p%d + o_, l%d_); }\n", (int)ix->src[0]->arg.i, loads[i].node);
  }
  ind(&g); {
    PolyDType base = ob; base.is_ptr = false; base.count = 1;
    pb_str_printf(g.o, "%s o4_[4];\n", pb_ctype(base));
  }
  /* lane-independent part once */
  g.vec = 1;
  g.lane_dep = (uint64_t)1 << x;
  /* emit nodes not depending on x */
  {
    uint64_t saved = g.bound;
    g.bound &= ~((uint64_t)1 << x);
    hoist(&g, pb_kern_node(k, st->value));
    g.bound = saved;
  }
  g.vec = 4;
  for (int lane = 0; lane < 4; lane++) {
    g.lane = lane;
    /* bind vector loads for this lane */
    for (int i = 0; i < nl; i++) {
      if (!vec_load[i]) continue;
      char nm[32]; temp_name(&g, loads[i].node, nm, sizeof nm);
      PolyUOp *ld = k->nodes[loads[i].node].u;
      ind(&g); pb_str_printf(g.o, "const %s %s = (%s)l%d_[%d];\n", ctype_of(&g, ld->dtype), nm,
                             ctype_of(&g, ld->dtype), loads[i].node, lane);
      log_emit(&g, loads[i].node);
    }
    emit_src(&g, st->value);
    char vs[96]; ref(&g, st->value, vs, sizeof vs);
    PolyDType base = ob; base.is_ptr = false; base.count = 1;
    ind(&g); pb_str_printf(g.o, "o4_[%d] = (%s)(%s);\n", lane, pb_ctype(base), vs);
    /* forget lane-dependent temps so the next lane re-emits them under its own names */
    for (int i = 0; i < k->n_nodes; i++)
      if (g.emitted[i] >= 0 && (k->nodes[i].deps & g.lane_dep)) g.emitted[i] = -1;
  }
  ind(&g); pb_str_printf(g.o, "{ %s o_ = %lld", g.idx_t, (long long)saff.offset);
  for (int j = 0; j < st->n_loop; j++) {
    int64_t s = saff.stride[st->loop[j]];
    if (s) pb_str_printf(g.o, " + r%d*%lld", st->loop[j], (long long)s);
  }
  if (out_bf16)
    pb_str_printf(g.o, "; __nv_bfloat162 q0_ = __floats2bfloat162_rn(o4_[0], o4_[1]), q1_ = __floats2bfloat162_rn(o4_[2], o4_[3]); "
                       "uint2 w_; w_.x = *reinterpret_cast<unsigned*>(&q0_); w_.y = *reinterpret_cast<unsigned*>(&q1_); "
                       "*reinterpret_cast<uint2*>(p%d + o_) = w_; }\n", st->param);
  else pb_str_printf(g.o, "; pb_st4(p%d + o_, o4_); }\n", st->param);
  pb_str_puts(g.o, "}\n");

  char *res = NULL;
  if (!g.failed) {
    PbStr h; pb_str_init(&h);
    char line[256];
    snprintf(line, sizeof line, "//launch flat block=256 work=c%lld", (long long)n_threads);
    emit_header(k, &h, line, usage);
    if (out_bf16) pb_str_puts(&h, "#include <cuda_bf16.h>\n");
    pb_str_puts(&h, g.out.s);
    res = pb_str_take(&h);
  }
  pb_str_free(&g.out);
  free(g.emitted); free(g.scope_log); free(g.scope_mark);
  return res;
}

/* ── general kernel: one thread per output element ───────────────────── */
static char *render_flat(PbKern *k, const int *usage) {
  Gen g; memset(&g, 0, sizeof g);
  g.k = k;
  g.emitted = malloc(sizeof(int) * (size_t)k->n_nodes);
  for (int i = 0; i < k->n_nodes; i++) g.emitted[i] = -1;
  g.scope_mark = calloc(64, sizeof(int));
  bool wide = false;
  for (int i = 0; i < k->n_params; i++)
    if (k->params[i] && k->params[i]->dtype.ptr_size >= ((int64_t)1 << 31)) wide = true;
  for (int s = 0; s < k->n_stores; s++) {
    int64_t t = 1;
    for (int i = 0; i < k->stores[s].n_loop; i++) t *= range_max(k, k->stores[s].loop[i]);
    if (t >= ((int64_t)1 << 31)) wide = true;
  }
  g.wide = wide; g.idx_t = wide ? "long long" : "int";
  pb_str_init(&g.out); g.o = &g.out; g.pfx = "";
  bool written[PB_MAX_PARAMS];
  for (int i = 0; i < k->n_params; i++) written[i] = (usage[i] & 2) != 0;

  pb_str_puts(g.o, PRELUDE);
  emit_signature(&g, written, 256);
  pb_str_puts(g.o, " {\n");
  g.indent = 1;
  ind(&g); pb_str_puts(g.o, "const long long gid_ = (long long)blockIdx.x * blockDim.x + threadIdx.x;\n");

  PbStr work; pb_str_init(&work);
  /* stores with the same loop set share one section (and their common subexpressions) */
  bool done[PB_MAX_STORES] = {0};
  for (int s = 0; s < k->n_stores; s++) {
    if (done[s]) continue;
    PbStore *st = &k->stores[s];
    uint64_t m = 0;
    for (int i = 0; i < st->n_loop; i++) m |= (uint64_t)1 << st->loop[i];
    if (work.n) pb_str_puts(&work, "|");
    size_expr(k, st->loop, st->n_loop, &work);
    ind(&g); pb_str_puts(g.o, "{\n"); g.indent++;
    /* section size */
    ind(&g); pb_str_puts(g.o, "long long tot_ = 1;");
    for (int i = 0; i < st->n_loop; i++) {
      char bs[64]; range_bound_str(&g, st->loop[i], bs, sizeof bs);
      pb_str_printf(g.o, " tot_ *= %s;", bs);
    }
    pb_str_puts(g.o, "\n");
    ind(&g); pb_str_puts(g.o, "if (gid_ < tot_) {\n"); g.indent++;
    open_scope(&g);
    uint64_t saved = g.bound;
    int order[PB_MAX_AXES];
    order_loop_axes(k, st, order, NULL);
    if (st->n_loop > 0) emit_decompose(&g, wide ? "gid_" : "(int)gid_", order, st->n_loop);
    for (int s2 = s; s2 < k->n_stores; s2++) {
      PbStore *st2 = &k->stores[s2];
      uint64_t m2 = 0;
      for (int i = 0; i < st2->n_loop; i++) m2 |= (uint64_t)1 << st2->loop[i];
      if (done[s2] || m2 != m) continue;
      done[s2] = true;
      emit_store(&g, st2);
    }
    close_scope(&g);
    g.bound = saved;
    g.indent--; ind(&g); pb_str_puts(g.o, "}\n");
    g.indent--; ind(&g); pb_str_puts(g.o, "}\n");
  }
  pb_str_puts(g.o, "}\n");

  char *res = NULL;
  if (!g.failed) {
    PbStr h; pb_str_init(&h);
    PbStr line; pb_str_init(&line);
    pb_str_printf(&line, "//launch flat block=256 work=%s", work.s);
    emit_header(k, &h, line.s, usage);
    pb_str_free(&line);
    if (k->uses_half) pb_str_puts(&h, "#include <cuda_fp16.h>\n");
    if (k->uses_bf16) pb_str_puts(&h, "#include <cuda_bf16.h>\n");
    pb_str_puts(&h, g.out.s);
    res = pb_str_take(&h);
  } else if (!k->err[0]) {
    snprintf(k->err, sizeof k->err, "rendering failed");
  }
  pb_str_free(&work);
  pb_str_free(&g.out);
  free(g.emitted); free(g.scope_log); free(g.scope_mark);
  return res;
}

char *pb_render_jit(PbKern *k, const char *fn_name) {
  (void)fn_name; /* the entry point has a fixed name so identical kernels share one binary */
  int usage[PB_MAX_PARAMS];
  param_usage(k, usage);
  const char *force = getenv("POLY_B200_JIT");  /* "flat" forces the general mapping (debugging) */
  if (!force || strcmp(force, "flat") != 0) {
    char *r = NULL;
    if (k->n_reduce_nodes == 1 && k->n_stores == 1) {
      /* a lone row reduction: the row-wise renderer gives it 128-bit loads */
      int ident[PB_MAX_PARAMS]; bool all_used = true;
      for (int a = 0; a < k->n_params; a++) { ident[a] = a; if (!k->params[a] || !(usage[a] & 3)) all_used = false; }
      if (all_used) {
        PbFuseIn in = { k, ident, PB_FUSE_FINAL, false };
        PbFuseOut fo;
        r = pb_render_rowfused(&in, 1, false, &fo);
        if (r) {
          bool same = fo.n_params == k->n_params;
          for (int a = 0; same && a < fo.n_params; a++) if (fo.slot[a] != a) same = false;
          if (!same) { free(r); r = NULL; }
        }
      }
      if (r) return r;
    }
    r = render_group_reduce(k, usage);
    if (r) return r;
    r = render_vec_elementwise(k, usage);
    if (r) return r;
  }
  return render_flat(k, usage);
}

/* The kernel's one elementwise store rendered so that its float values land in a
 * bfloat16 buffer of the same element layout (round to nearest even).  NULL when
 * the kernel is not a vectorisable elementwise kernel with a float output. */
char *pb_render_elementwise_bf16(PbKern *k) {
  if (k->n_stores != 1 || k->n_reduce_nodes != 0) return NULL;
  int usage[PB_MAX_PARAMS];
  param_usage(k, usage);
  s_bf16_out_param1 = k->stores[0].param + 1;
  char *r = render_vec_elementwise(k, usage);
  s_bf16_out_param1 = 0;
  return r;
}

/* ════════════════════════════════════════════════════════════════════════
 *  Row-fused kernels
 * ════════════════════════════════════════════════════════════════════════ */
#define RF_MAX 8

typedef struct {
  int n;
  PbFuseIn *in;
  Gen g[RF_MAX];
  int wslot[RF_MAX];                 /* slot each kernel writes */
  int map[RF_MAX][PB_MAX_RANGES];    /* kernel range -> canonical range (a range id of the final kernel), -1 unmapped */
  int c_range[RF_MAX];               /* the kernel's own range that runs along the row */
  int usage[RF_MAX][PB_MAX_PARAMS];
  int fparam[RF_MAX][PB_MAX_PARAMS]; /* fused parameter index of each kernel parameter, -1 internal/unused */
  char range_expr[RF_MAX][PB_MAX_RANGES][40];
  char param_expr[RF_MAX][PB_MAX_PARAMS][24];
  int canon_c;                       /* canonical range along the row */
  int V, G, NI, RPB; int64_t C;
  bool final_reduce, out_bf16;
  int red_node[RF_MAX];              /* REDUCE node of each phase */
  bool *vec_load[RF_MAX];            /* per node: LOAD served by a 128-bit access */
} RowFuse;

static RowFuse *rf_of(Gen *g) { return (RowFuse *)g->ud; }
static int rf_index(RowFuse *rf, Gen *g) { return (int)(g - rf->g); }

static int rf_writer_of(RowFuse *rf, int slot) {
  for (int i = 0; i < rf->n - 1; i++) if (rf->wslot[i] == slot) return i;
  return -1;
}

static void rf_all_open(RowFuse *rf) { for (int i = 0; i < rf->n; i++) open_scope(&rf->g[i]); }
static void rf_all_close(RowFuse *rf) { for (int i = 0; i < rf->n; i++) close_scope(&rf->g[i]); }
static void rf_set_indent(RowFuse *rf, int ind_) { for (int i = 0; i < rf->n; i++) rf->g[i].indent = ind_; }
static void rf_set_lane(RowFuse *rf, int lane) { for (int i = 0; i < rf->n; i++) rf->g[i].lane = lane; }
static void rf_forget_lane_temps(RowFuse *rf) {
  for (int i = 0; i < rf->n; i++) {
    Gen *g = &rf->g[i];
    if (!g->lane_dep) continue;
    for (int id = 0; id < g->k->n_nodes; id++)
      if (g->emitted[id] >= 0 && (g->k->nodes[id].deps & g->lane_dep)) g->emitted[id] = -1;
  }
}

/* LOAD nodes of a fused kernel: values that never reach memory come from the
 * chain itself; contiguous external loads are 128-bit. */
static bool rf_load_hook(Gen *g, int id) {
  RowFuse *rf = rf_of(g);
  int ki = rf_index(rf, g);
  PolyUOp *u = g->k->nodes[id].u;
  PolyUOp *ix = u->src[0];
  if (ix->op != POLY_OP_INDEX || ix->src[0]->op != POLY_OP_PARAM) return false;
  int pi = (int)ix->src[0]->arg.i;
  int w = rf_writer_of(rf, rf->in[ki].slot[pi]);
  char name[40];
  temp_name(g, id, name, sizeof name);
  const char *ct = ctype_of(g, u->dtype);
  if (w >= 0) {
    if (rf->in[w].role == PB_FUSE_PHASE) {
      ind(g); pb_str_printf(g->o, "const %s %s = stat%d_;\n", ct, name, w);
    } else {
      Gen *pg = &rf->g[w];
      PbStore *st = &pg->k->stores[0];
      emit_src(pg, st->value);
      char v[96]; ref(pg, st->value, v, sizeof v);
      ind(g); pb_str_printf(g->o, "const %s %s = (%s)(%s);\n", ct, name, ct, v);
    }
    log_emit(g, id);
    return true;
  }
  if (rf->V == 4 && rf->vec_load[ki][id]) {
    if (g->lane == 0) {
      emit_src(g, ix->src[1]);
      char is[96], pn[32]; ref(g, ix->src[1], is, sizeof is); ref(g, ix->src[0], pn, sizeof pn);
      PolyDType base = ix->src[0]->dtype; base.is_ptr = false; base.count = 1;
      ind(g); pb_str_printf(g->o, "%s lv%s%d_[4]; pb_ld4(%s + %s, lv%s%d_);\n", pb_ctype(base), g->pfx, id, pn, is, g->pfx, id);
    }
    ind(g); pb_str_printf(g->o, "const %s %s = (%s)lv%s%d_[%d];\n", ct, name, ct, g->pfx, id, g->lane);
    log_emit(g, id);
    return true;
  }
  return false;
}

/* Fit the index of node `ld` (a LOAD) or of a store over all ranges of kernel k. */
static bool rf_fit(PbKern *k, PolyUOp *index_expr, PbAffine *a) {
  uint64_t all = 0;
  for (int r = 0; r < k->n_ranges; r++) all |= (uint64_t)1 << r;
  pb_fit_affine(k, index_expr, all, a);
  return a->ok;
}

/* All loads of parameter `pi` in kernel k share one index?  Returns it fitted. */
static bool rf_param_load_index(PbKern *k, int pi, PbAffine *a, int *n_loads) {
  PolyUOp *first = NULL; *n_loads = 0;
  for (int i = 0; i < k->n_nodes; i++) {
    PolyUOp *u = k->nodes[i].u;
    if (u->op != POLY_OP_LOAD || u->src[0]->op != POLY_OP_INDEX || u->src[0]->src[0]->op != POLY_OP_PARAM) continue;
    if ((int)u->src[0]->src[0]->arg.i != pi) continue;
    if (u->src[0]->n_src > 2) return false;
    (*n_loads)++;
    if (!first) first = u->src[0]->src[1];
    else if (first != u->src[0]->src[1]) return false;
  }
  if (!first) return true;
  return rf_fit(k, first, a);
}

static int rf_find_reduce(PbKern *k) {
  for (int i = 0; i < k->n_nodes; i++) if (k->nodes[i].u->op == POLY_OP_REDUCE) return i;
  return -1;
}

/* Map kernel ki's ranges through the buffer it writes, using an already mapped
 * consumer kj.  Both indices are compared in canonical ranges. */
static bool rf_map_through(RowFuse *rf, int ki, int kj) {
  PbKern *kp = rf->in[ki].k, *kc = rf->in[kj].k;
  PbStore *st = &kp->stores[0];
  if (st->index->n_src > 2) return false;
  PbAffine ws, ls;
  if (!rf_fit(kp, st->index->src[1], &ws)) return false;
  int pj = -1;
  for (int a = 0; a < kc->n_params; a++) if (kc->params[a] && rf->in[kj].slot[a] == rf->wslot[ki]) pj = a;
  if (pj < 0) return true;                      /* kj does not read it */
  int nl = 0;
  if (!rf_param_load_index(kc, pj, &ls, &nl)) return false;
  if (nl == 0) return true;
  if (ls.offset != ws.offset) return false;
  /* consumer strides in canonical ranges */
  int64_t cs[PB_MAX_RANGES] = {0};
  for (int r = 0; r < kc->n_ranges; r++) {
    if (ls.stride[r] == 0 || kc->extent[r] <= 1) continue;
    int cr = rf->map[kj][r];
    if (cr < 0) return false;
    if (cs[cr] != 0) return false;
    cs[cr] = ls.stride[r];
  }
  PbKern *kf = rf->in[rf->n - 1].k;
  bool used[PB_MAX_RANGES] = {0};
  for (int i = 0; i < st->n_loop; i++) {
    int q = st->loop[i];
    if (kp->extent[q] <= 1) { if (rf->map[ki][q] < 0) rf->map[ki][q] = -2; continue; }
    if (ws.stride[q] == 0) return false;
    int found = -1;
    for (int cr = 0; cr < kf->n_ranges; cr++)
      if (!used[cr] && cs[cr] == ws.stride[q] && kf->extent[cr] == kp->extent[q]) { found = cr; break; }
    if (found < 0) return false;
    used[found] = true;
    if (rf->map[ki][q] >= 0 && rf->map[ki][q] != found) return false;
    rf->map[ki][q] = found;
  }
  for (int cr = 0; cr < kf->n_ranges; cr++) if (cs[cr] != 0 && !used[cr]) return false;
  return true;
}

static void rf_free(RowFuse *rf) {
  for (int i = 0; i < rf->n; i++) {
    free(rf->g[i].emitted); free(rf->g[i].scope_log); free(rf->g[i].scope_mark); free(rf->vec_load[i]);
  }
}

char *pb_render_rowfused(PbFuseIn *in, int n, bool out_bf16, PbFuseOut *out) {
  if (n < 1 || n > RF_MAX) return NULL;
  RowFuse *rf = calloc(1, sizeof *rf);
  rf->n = n; rf->in = in; rf->out_bf16 = out_bf16;
  char *result = NULL;
  PbKern *kf = in[n - 1].k;
  PbStr text; pb_str_init(&text);

  /* shape checks */
  int n_phase = 0;
  for (int i = 0; i < n; i++) {
    PbKern *k = in[i].k;
    if (k->n_stores != 1 || k->n_vars) goto done;
    for (int r = 0; r < k->n_ranges; r++) if (k->extent[r] < 0) goto done;
    rf->wslot[i] = in[i].slot[k->stores[0].param];
    param_usage(k, rf->usage[i]);
    rf->red_node[i] = -1;
    for (int r = 0; r < k->n_ranges; r++) rf->map[i][r] = -1;
    if (in[i].role == PB_FUSE_PRODUCER) { if (k->n_reduce_nodes != 0) goto done; }
    else if (in[i].keep_out) goto done;
    else if (in[i].role == PB_FUSE_PHASE) {
      if (k->n_reduce_nodes != 1) goto done;
      rf->red_node[i] = rf_find_reduce(k);
      PolyUOp *red = k->nodes[rf->red_node[i]].u;
      if (red->n_src != 2 || red->dtype.priority != 13) goto done;
      PolyOps op = reduce_op(red);
      if (op != POLY_OP_ADD && op != POLY_OP_MAX) goto done;
      if (k->nodes[pb_kern_node(k, k->stores[0].index)].has_reduce) goto done;
      n_phase++;
    }
    if (i < n - 1 && !(rf->usage[i][k->stores[0].param] & 4)) goto done;   /* internal buffers are written whole */
  }
  if (kf->n_reduce_nodes > 1) goto done;
  rf->final_reduce = kf->n_reduce_nodes == 1;
  if (rf->final_reduce) {
    rf->red_node[n - 1] = rf_find_reduce(kf);
    PolyUOp *red = kf->nodes[rf->red_node[n - 1]].u;
    PolyOps op = reduce_op(red);
    if (red->n_src != 2 || red->dtype.priority != 13 || (op != POLY_OP_ADD && op != POLY_OP_MAX)) goto done;
    if (out_bf16) goto done;
  }
  if (n_phase == 0 && !rf->final_reduce) goto done;
  if (kf->stores[0].index->n_src > 2) goto done;
  for (int i = 0; i < n - 1; i++) for (int j = 0; j < n - 1; j++) if (i != j && rf->wslot[i] == rf->wslot[j]) goto done;
  for (int i = 0; i < n - 1; i++) if (rf->wslot[i] == rf->wslot[n - 1]) goto done;

  /* candidates for the row axis in the final kernel */
  int64_t C = -1;
  for (int i = 0; i < n; i++) if (rf->red_node[i] >= 0) {
    PbKern *k = in[i].k;
    int r = pb_kern_range_id(k, k->nodes[rf->red_node[i]].u->src[1]);
    if (C < 0) C = k->extent[r]; else if (C != k->extent[r]) goto done;
    rf->c_range[i] = r;
  }
  if (C < 32) goto done;
  PbStore *fst = &kf->stores[0];
  PbAffine fs;
  if (!rf_fit(kf, fst->index->src[1], &fs)) goto done;
  bool mapped = false;
  for (int cand = 0; cand < kf->n_ranges && !mapped; cand++) {
    if (rf->final_reduce) { if (cand != rf->c_range[n - 1]) continue; }
    else {
      bool is_loop = false;
      for (int i = 0; i < fst->n_loop; i++) if (fst->loop[i] == cand) is_loop = true;
      if (!is_loop || kf->extent[cand] != C || fs.stride[cand] == 0) continue;
    }
    rf->canon_c = cand;
    for (int i = 0; i < n; i++) for (int r = 0; r < in[i].k->n_ranges; r++) rf->map[i][r] = -1;
    for (int r = 0; r < kf->n_ranges; r++) rf->map[n - 1][r] = r;
    bool ok = true;
    for (int i = n - 2; i >= 0 && ok; i--) {
      if (in[i].role == PB_FUSE_PHASE) rf->map[i][rf->c_range[i]] = cand;
      bool any = false;
      for (int j = i + 1; j < n && ok; j++) {
        /* does kj read what ki writes? */
        PbKern *kc = in[j].k; bool reads = false;
        for (int a = 0; a < kc->n_params; a++) if (kc->params[a] && in[j].slot[a] == rf->wslot[i] && (rf->usage[j][a] & 1)) reads = true;
        if (!reads) continue;
        any = true;
        ok = rf_map_through(rf, i, j);
      }
      if (!any) ok = false;
      /* every range of the kernel must be placed; a statistic must not vary along the row */
      PbKern *k = in[i].k;
      for (int r = 0; r < k->n_ranges && ok; r++) {
        if (k->extent[r] <= 1) continue;
        if (rf->map[i][r] < 0) ok = false;
      }
      if (ok && in[i].role == PB_FUSE_PHASE)
        for (int q = 0; q < k->stores[0].n_loop; q++) if (rf->map[i][k->stores[0].loop[q]] == cand) ok = false;
      if (ok && in[i].role == PB_FUSE_PRODUCER) {
        /* exactly one of its ranges runs along the row */
        int cnt = 0;
        for (int r = 0; r < k->n_ranges; r++) if (rf->map[i][r] == cand) { rf->c_range[i] = r; cnt++; }
        if (cnt != 1) ok = false;
      }
    }
    /* statistics read by the final kernel must be row-invariant there */
    if (ok && !rf->final_reduce) rf->c_range[n - 1] = cand;
    mapped = ok;
  }
  if (!mapped) goto done;
  rf->C = C;

  /* fused parameter list */
  out->n_params = 0;
  for (int i = 0; i < n; i++) {
    PbKern *k = in[i].k;
    for (int a = 0; a < k->n_params; a++) {
      rf->fparam[i][a] = -1;
      if (!k->params[a] || !(rf->usage[i][a] & 3)) continue;
      int sl = in[i].slot[a];
      int w = rf_writer_of(rf, sl);
      if (w >= 0 && w == i && in[i].keep_out && a == k->stores[0].param && !(rf->usage[i][a] & 1)) {
        /* a producer whose result lives on: written by the final pass next to the final result */
        if (out->n_params >= PB_MAX_PARAMS || k->params[a]->dtype.bitsize != 32 || k->params[a]->dtype.priority != 13) goto done;
        int f = out->n_params++; out->slot[f] = sl; out->rw[f] = (rf->usage[i][a] & 4) ? 'W' : 'w';
        rf->fparam[i][a] = f;
        continue;
      }
      if (w >= 0) {
        /* internal: reads are replaced; the write itself disappears */
        if ((rf->usage[i][a] & 1) && w >= i) goto done;     /* read before it is produced */
        continue;
      }
      int f = -1;
      for (int x = 0; x < out->n_params; x++) if (out->slot[x] == sl) f = x;
      if (f < 0) {
        if (out->n_params >= PB_MAX_PARAMS) goto done;
        f = out->n_params++; out->slot[f] = sl; out->rw[f] = 'r';
      }
      if (i == n - 1 && a == fst->param) out->rw[f] = (rf->usage[i][a] & 1) ? 'b' : ((rf->usage[i][a] & 4) ? 'W' : 'w');
      else if (out->slot[f] == rf->wslot[n - 1] && out->rw[f] != 'r') out->rw[f] = 'b';
      rf->fparam[i][a] = f;
      /* element type must be 4 bytes wide for every external operand */
      if (k->params[a]->dtype.bitsize != 32) goto done;
    }
  }
  out->rw[out->n_params] = 0;
  /* the output buffer may only be read element-for-element, which a row kernel does not guarantee */
  for (int x = 0; x < out->n_params; x++) if (out->rw[x] == 'b') goto done;

  /* vector width: every row-dependent external access contiguous and aligned */
  rf->V = (C % 4 == 0) ? 4 : 1;
  for (int i = 0; i < n; i++) {
    PbKern *k = in[i].k;
    rf->vec_load[i] = calloc((size_t)k->n_nodes, 1);
    uint64_t cbit = (uint64_t)1 << rf->c_range[i];
    for (int id = 0; id < k->n_nodes; id++) {
      PolyUOp *u = k->nodes[id].u;
      if (u->op != POLY_OP_LOAD) continue;
      PolyUOp *ix = u->src[0];
      if (ix->op != POLY_OP_INDEX || ix->src[0]->op != POLY_OP_PARAM) goto done;
      int pi = (int)ix->src[0]->arg.i;
      if (rf_writer_of(rf, in[i].slot[pi]) >= 0) continue;
      if (!(k->nodes[id].deps & cbit)) continue;
      PbAffine a;
      bool fit = ix->n_src == 2 && rf_fit(k, ix->src[1], &a);
      bool vec = fit && a.stride[rf->c_range[i]] == 1 && a.offset % 4 == 0;
      if (vec) {
        int64_t lo = a.offset, hi = a.offset;
        for (int r = 0; r < k->n_ranges; r++) {
          if (r != rf->c_range[i] && a.stride[r] % 4) vec = false;
          int64_t sp = a.stride[r] * (k->extent[r] - 1);
          if (sp > 0) hi += sp; else lo += sp;
        }
        if (lo < 0 || hi >= ix->src[0]->dtype.ptr_size) vec = false;
      }
      rf->vec_load[i][id] = vec;
      if (!vec && fit && a.stride[rf->c_range[i]] == 0) continue;   /* row-invariant after all */
      if (!vec) rf->V = 1;
    }
  }
  for (int i = 0; i < n - 1; i++) {
    if (!in[i].keep_out) continue;
    if (rf->final_reduce) goto done;                 /* there is no elementwise final pass to store from */
    PbKern *k = in[i].k;
    PbAffine ps;
    if (k->stores[0].index->n_src > 2 || !rf_fit(k, k->stores[0].index->src[1], &ps)) goto done;
    if (ps.stride[rf->c_range[i]] != 1 || ps.offset % 4) rf->V = 1;
    int64_t lo = ps.offset, hi = ps.offset;
    for (int r = 0; r < k->n_ranges; r++) {
      if (r != rf->c_range[i] && ps.stride[r] % 4) rf->V = 1;
      int64_t sp = ps.stride[r] * (k->extent[r] - 1);
      if (sp > 0) hi += sp; else lo += sp;
    }
    if (lo < 0 || hi >= k->params[k->stores[0].param]->dtype.ptr_size) rf->V = 1;
  }
  if (!rf->final_reduce) {
    if (fs.stride[rf->canon_c] != 1 || fs.offset % 4) rf->V = 1;
    int64_t lo = fs.offset, hi = fs.offset;
    for (int r = 0; r < kf->n_ranges; r++) {
      if (r != rf->canon_c && fs.stride[r] % 4) rf->V = 1;
      int64_t sp = fs.stride[r] * (kf->extent[r] - 1);
      if (sp > 0) hi += sp; else lo += sp;
    }
    if (lo < 0 || hi >= kf->params[fst->param]->dtype.ptr_size) rf->V = 1;
    if (out_bf16 && rf->V != 4) goto done;
  }
  {
    int64_t per = (C + rf->V * 8 - 1) / (rf->V * 8);
    int G = 32; while (G < per && G < 1024) G *= 2;
    rf->G = G;
    rf->NI = (int)((C + (int64_t)G * rf->V - 1) / ((int64_t)G * rf->V));
    if (rf->NI > 32) goto done;
    rf->RPB = G >= 256 ? 1 : 256 / G;
  }

  /* rows */
  int row_axes[PB_MAX_AXES]; int n_row = 0; int64_t n_rows = 1;
  {
    int order[PB_MAX_AXES];
    order_loop_axes(kf, fst, order, NULL);
    for (int i = 0; i < fst->n_loop; i++) if (order[i] != rf->canon_c) { row_axes[n_row++] = order[i]; n_rows *= kf->extent[order[i]]; }
  }
  bool wide = n_rows * rf->G >= ((int64_t)1 << 31);
  for (int i = 0; i < n; i++) for (int a = 0; a < in[i].k->n_params; a++)
    if (in[i].k->params[a] && in[i].k->params[a]->dtype.ptr_size >= ((int64_t)1 << 31)) wide = true;

  /* generators */
  static const char *PFX[RF_MAX] = {"a", "b", "c", "d", "e", "f", "g", "h"};
  for (int i = 0; i < n; i++) {
    Gen *g = &rf->g[i];
    PbKern *k = in[i].k;
    g->k = k; g->o = &text; g->pfx = PFX[i]; g->ud = rf; g->load_hook = rf_load_hook;
    g->emitted = malloc(sizeof(int) * (size_t)k->n_nodes);
    for (int x = 0; x < k->n_nodes; x++) g->emitted[x] = -1;
    g->scope_mark = calloc(64, sizeof(int));
    g->wide = wide; g->idx_t = wide ? "long long" : "int";
    g->range_expr = rf->range_expr[i]; g->param_expr = rf->param_expr[i];
    for (int r = 0; r < k->n_ranges; r++) {
      int cr = rf->map[i][r];
      if (cr == rf->canon_c && r == rf->c_range[i]) snprintf(rf->range_expr[i][r], 40, "c_");
      else if (cr >= 0) snprintf(rf->range_expr[i][r], 40, "r%d", cr);
      else snprintf(rf->range_expr[i][r], 40, "0");
    }
    for (int a = 0; a < k->n_params; a++) snprintf(rf->param_expr[i][a], 24, "p%d", rf->fparam[i][a]);
    g->vec = rf->V; g->lane = 0; g->lane_dep = (uint64_t)1 << rf->c_range[i];
    g->bound = 0;
    for (int r = 0; r < k->n_ranges; r++) if (r != rf->c_range[i]) g->bound |= (uint64_t)1 << r;
  }

  /* ── text ── */
  const int G = rf->G, V = rf->V, NI = rf->NI, RPB = rf->RPB, block = G * RPB;
  pb_str_puts(&text, PRELUDE);
  pb_str_puts(&text,
    "template <class T> __device__ __forceinline__ void pb_ld4(const T* p, T* o) {\n"
    "  const uint4 v = *reinterpret_cast<const uint4*>(p); memcpy(o, &v, 16);\n}\n"
    "template <class T> __device__ __forceinline__ void pb_st4(T* p, const T* o) {\n"
    "  uint4 v; memcpy(&v, o, 16); *reinterpret_cast<uint4*>(p) = v;\n}\n");
  pb_str_printf(&text, "extern \"C\" __global__ void __launch_bounds__(%d) pb200_kernel(", block);
  for (int x = 0; x < out->n_params; x++) {
    /* element type from any kernel parameter bound to this slot */
    const char *ct = "float";
    for (int i = 0; i < n; i++) for (int a = 0; a < in[i].k->n_params; a++)
      if (rf->fparam[i][a] == x) { PolyDType b = in[i].k->params[a]->dtype; b.is_ptr = false; b.count = 1; ct = pb_ctype(b); }
    bool is_out = out->slot[x] == rf->wslot[n - 1];
    if (is_out && out_bf16) ct = "__nv_bfloat16";
    pb_str_printf(&text, "%s%s* __restrict__ p%d, ", (is_out || out->rw[x] != 'r') ? "" : "const ", ct, x);
  }
  pb_str_puts(&text, "const long long n_work) {\n");
  rf_set_indent(rf, 1);
  Gen *gf = &rf->g[n - 1];
  ind(gf); pb_str_printf(&text, "const int lane_ = threadIdx.x %% %d, rib_ = threadIdx.x / %d;\n", G, G);
  ind(gf); pb_str_printf(&text, "long long row_ = (long long)blockIdx.x * %d + rib_;\n", RPB);
  ind(gf); pb_str_puts(&text, "const bool live_ = row_ < n_work;\n");
  ind(gf); pb_str_puts(&text, "if (!live_) row_ = n_work - 1;\n");
  if (n_row > 0) {
    ind(gf); pb_str_printf(&text, "%s rem_ = (%s)row_;\n", gf->idx_t, gf->idx_t);
    for (int i = 0; i < n_row; i++) {
      int r = row_axes[i];
      ind(gf);
      if (i == n_row - 1) pb_str_printf(&text, "const %s r%d = rem_;\n", gf->idx_t, r);
      else pb_str_printf(&text, "const %s r%d = rem_ %% %lld; rem_ /= %lld;\n", gf->idx_t, r, (long long)kf->extent[r], (long long)kf->extent[r]);
    }
  }
  /* extent-1 ranges of the final kernel */
  for (int r = 0; r < kf->n_ranges; r++) {
    bool isrow = false;
    for (int i = 0; i < n_row; i++) if (row_axes[i] == r) isrow = true;
    if (!isrow && r != rf->canon_c && !(rf->final_reduce && r == rf->c_range[n - 1])) {
      ind(gf); pb_str_printf(&text, "const %s r%d = 0;\n", gf->idx_t, r);
    }
  }

  for (int i = 0; i < n; i++) {
    const bool is_final = i == n - 1;
    if (in[i].role == PB_FUSE_PRODUCER) continue;
    Gen *g = &rf->g[i];
    PbKern *k = in[i].k;
    PbStore *st = &k->stores[0];
    if (!is_final || rf->final_reduce) {
      /* ── a reduction phase ── */
      PolyUOp *red = k->nodes[rf->red_node[i]].u;
      PolyOps op = reduce_op(red);
      int vid = pb_kern_node(k, red->src[0]);
      hoist(g, vid);
      char idn[96]; reduce_identity(op, red->dtype, idn, sizeof idn, g);
      ind(g); pb_str_printf(&text, "float acc%d_ = %s;\n", i, idn);
      ind(g); pb_str_puts(&text, "#pragma unroll\n");
      ind(g); pb_str_printf(&text, "for (int i_ = 0; i_ < %d; ++i_) {\n", NI);
      rf_set_indent(rf, 2);
      ind(g); pb_str_printf(&text, "const %s c_ = (lane_ + i_ * %d) * %d;\n", g->idx_t, G, V);
      ind(g); pb_str_printf(&text, "if (c_ < %lld) {\n", (long long)C);
      rf_set_indent(rf, 3);
      rf_all_open(rf);
      for (int r = 0; r < rf->n; r++) rf->g[r].bound |= rf->g[r].lane_dep;
      for (int lane = 0; lane < V; lane++) {
        rf_set_lane(rf, lane);
        emit_src(g, red->src[0]);
        char v[96], acc[24], cmb[256];
        ref(g, red->src[0], v, sizeof v);
        snprintf(acc, sizeof acc, "acc%d_", i);
        combine_expr(op, acc, v, cmb, sizeof cmb);
        ind(g); pb_str_printf(&text, "%s = %s;\n", acc, cmb);
        if (V > 1) rf_forget_lane_temps(rf);
      }
      rf_set_lane(rf, 0);
      for (int r = 0; r < rf->n; r++) rf->g[r].bound &= ~rf->g[r].lane_dep;
      rf_all_close(rf);
      rf_set_indent(rf, 2); ind(g); pb_str_puts(&text, "}\n");
      rf_set_indent(rf, 1); ind(g); pb_str_puts(&text, "}\n");
      /* combine across the group */
      char sh[256], accn[24]; snprintf(accn, sizeof accn, "acc%d_", i);
      combine_expr(op, accn, "x_", sh, sizeof sh);
      ind(g); pb_str_puts(&text, "#pragma unroll\n");
      ind(g); pb_str_printf(&text, "for (int o_ = 16; o_ > 0; o_ >>= 1) { const float x_ = __shfl_xor_sync(0xffffffffu, %s, o_); %s = %s; }\n", accn, accn, sh);
      if (G > 32) {
        int nw = G / 32;
        ind(g); pb_str_printf(&text, "__shared__ float red%d_[%d][%d];\n", i, RPB, nw);
        ind(g); pb_str_printf(&text, "if ((lane_ & 31) == 0) red%d_[rib_][lane_ >> 5] = %s;\n", i, accn);
        ind(g); pb_str_puts(&text, "__syncthreads();\n");
        ind(g); pb_str_printf(&text, "%s = red%d_[rib_][0];\n", accn, i);
        ind(g); pb_str_printf(&text, "#pragma unroll\n");
        ind(g); pb_str_printf(&text, "for (int w_ = 1; w_ < %d; ++w_) { const float x_ = red%d_[rib_][w_]; %s = %s; }\n", nw, i, accn, sh);
      }
      /* the kernel's own expression after the reduction */
      char name[40]; temp_name(g, rf->red_node[i], name, sizeof name);
      ind(g); pb_str_printf(&text, "const float %s = %s;\n", name, accn);
      log_emit(g, rf->red_node[i]);
      emit_src(g, st->value);
      char sv[96]; ref(g, st->value, sv, sizeof sv);
      if (!is_final) { ind(g); pb_str_printf(&text, "const float stat%d_ = (float)(%s);\n", i, sv); }
      else {
        emit_src(g, st->index->src[1]);
        char is[96], pn[32]; ref(g, st->index->src[1], is, sizeof is); ref(g, st->index->src[0], pn, sizeof pn);
        ind(g); pb_str_printf(&text, "if (live_ && lane_ == 0) pb_st(%s, %s, %lldLL, (float)(%s));\n", pn, is,
                              (long long)k->params[st->param]->dtype.ptr_size, sv);
      }
    } else {
      /* ── the final elementwise pass ── */
      hoist(g, pb_kern_node(k, st->value));
      ind(g); pb_str_puts(&text, "#pragma unroll\n");
      ind(g); pb_str_printf(&text, "for (int i_ = 0; i_ < %d; ++i_) {\n", NI);
      rf_set_indent(rf, 2);
      ind(g); pb_str_printf(&text, "const %s c_ = (lane_ + i_ * %d) * %d;\n", g->idx_t, G, V);
      ind(g); pb_str_printf(&text, "if (c_ < %lld) {\n", (long long)C);
      rf_set_indent(rf, 3);
      rf_all_open(rf);
      for (int r = 0; r < rf->n; r++) rf->g[r].bound |= rf->g[r].lane_dep;
      char pn[32]; ref(g, st->index->src[0], pn, sizeof pn);
      char is0[96] = "";
      if (V == 4) {
        /* address of the 4-wide store: the index at lane 0, emitted first so that
         * lane 0's own use of the same expression finds it declared */
        ind(g); pb_str_puts(&text, "float o4_[4];\n");
        rf_set_lane(rf, 0);
        emit_src(g, st->index->src[1]);
        ref(g, st->index->src[1], is0, sizeof is0);
      }
      /* producers whose result is kept: their store index (lane 0) and a 4-wide buffer */
      char kis[RF_MAX][96];
      for (int w = 0; w < n - 1; w++) {
        kis[w][0] = 0;
        if (!in[w].keep_out) continue;
        Gen *pg = &rf->g[w];
        PbStore *pst = &pg->k->stores[0];
        if (V == 4) {
          ind(g); pb_str_printf(&text, "float k4_%d_[4];\n", w);
          rf_set_lane(rf, 0);
          emit_src(pg, pst->index->src[1]);
          ref(pg, pst->index->src[1], kis[w], sizeof kis[w]);
        }
      }
      for (int lane = 0; lane < V; lane++) {
        rf_set_lane(rf, lane);
        for (int w = 0; w < n - 1; w++) {
          if (!in[w].keep_out) continue;
          Gen *pg = &rf->g[w];
          PbStore *pst = &pg->k->stores[0];
          emit_src(pg, pst->value);
          char kv[96]; ref(pg, pst->value, kv, sizeof kv);
          if (V == 4) { ind(g); pb_str_printf(&text, "k4_%d_[%d] = (float)(%s);\n", w, lane, kv); }
          else {
            emit_src(pg, pst->index->src[1]);
            char kidx[96], kpn[32]; ref(pg, pst->index->src[1], kidx, sizeof kidx); ref(pg, pst->index->src[0], kpn, sizeof kpn);
            ind(g); pb_str_printf(&text, "if (live_) pb_st(%s, %s, %lldLL, (float)(%s));\n", kpn, kidx,
                                  (long long)pg->k->params[pst->param]->dtype.ptr_size, kv);
          }
        }
        emit_src(g, st->value);
        char v[96]; ref(g, st->value, v, sizeof v);
        if (V == 4) { ind(g); pb_str_printf(&text, "o4_[%d] = (float)(%s);\n", lane, v); }
        else {
          emit_src(g, st->index->src[1]);
          char is[96]; ref(g, st->index->src[1], is, sizeof is);
          ind(g); pb_str_printf(&text, "if (live_) pb_st(%s, %s, %lldLL, (float)(%s));\n", pn, is,
                                (long long)k->params[st->param]->dtype.ptr_size, v);
        }
        if (V > 1 && lane < V - 1) rf_forget_lane_temps(rf);
      }
      if (V == 4) {
        const char *is = is0;
        ind(g);
        if (out_bf16)
          pb_str_printf(&text, "if (live_) { __nv_bfloat162 q0_ = __floats2bfloat162_rn(o4_[0], o4_[1]), q1_ = __floats2bfloat162_rn(o4_[2], o4_[3]); "
                               "uint2 w_; w_.x = *reinterpret_cast<unsigned*>(&q0_); w_.y = *reinterpret_cast<unsigned*>(&q1_); "
                               "*reinterpret_cast<uint2*>(%s + %s) = w_; }\n", pn, is);
        else pb_str_printf(&text, "if (live_) pb_st4(%s + %s, o4_);\n", pn, is);
        for (int w = 0; w < n - 1; w++) {
          if (!in[w].keep_out) continue;
          Gen *pg = &rf->g[w];
          char kpn[32]; ref(pg, pg->k->stores[0].index->src[0], kpn, sizeof kpn);
          ind(g); pb_str_printf(&text, "if (live_) pb_st4(%s + %s, k4_%d_);\n", kpn, kis[w], w);
        }
      }
      rf_set_lane(rf, 0);
      for (int r = 0; r < rf->n; r++) rf->g[r].bound &= ~rf->g[r].lane_dep;
      rf_all_close(rf);
      rf_set_indent(rf, 2); ind(g); pb_str_puts(&text, "}\n");
      rf_set_indent(rf, 1); ind(g); pb_str_puts(&text, "}\n");
    }
  }
  pb_str_puts(&text, "}\n");
  bool failed = false;
  for (int i = 0; i < n; i++) if (rf->g[i].failed) failed = true;
  if (!failed) {
    PbStr h; pb_str_init(&h);
    pb_str_puts(&h, "//PB200 1\n//kind jit\n//entry pb200_kernel\n");
    pb_str_printf(&h, "//nparams %d\n//nvars 0\n", out->n_params);
    pb_str_printf(&h, "//launch group block=%d group=%d work=c%lld\n", block, G, (long long)n_rows);
    pb_str_puts(&h, "//rw");
    for (int x = 0; x < out->n_params; x++) pb_str_printf(&h, " %s", out->rw[x] == 'W' ? "W" : (out->rw[x] == 'w' ? "w" : "r"));
    pb_str_printf(&h, "\n//fused %d kernels, row length %lld, %d lanes per row, %d-wide\n", n, (long long)C, G, V);
    if (out_bf16) pb_str_puts(&h, "#include <cuda_bf16.h>\n");
    pb_str_puts(&h, text.s);
    result = pb_str_take(&h);
  }
done:
  pb_str_free(&text);
  rf_free(rf);
  free(rf);
  return result;
}
