/*
 * pb_kern.c -- node table, host-side index evaluation and affine fitting for
 * one scheduled kernel (see pb_kern.h).
 */
#include "pb_kern.h"
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

/* ── growable string ─────────────────────────────────────────────────── */
void pb_str_init(PbStr *b) { b->s = NULL; b->n = 0; b->cap = 0; }
void pb_str_free(PbStr *b) { free(b->s); pb_str_init(b); }
static void pb_str_reserve(PbStr *b, size_t extra) {
  if (b->n + extra + 1 <= b->cap) return;
  size_t nc = b->cap ? b->cap * 2 : 1024;
  while (nc < b->n + extra + 1) nc *= 2;
  b->s = realloc(b->s, nc);
  b->cap = nc;
}
void pb_str_puts(PbStr *b, const char *s) {
  size_t l = strlen(s);
  pb_str_reserve(b, l);
  memcpy(b->s + b->n, s, l + 1);
  b->n += l;
}
void pb_str_printf(PbStr *b, const char *fmt, ...) {
  va_list ap, ap2;
  va_start(ap, fmt);
  va_copy(ap2, ap);
  int l = vsnprintf(NULL, 0, fmt, ap);
  va_end(ap);
  if (l > 0) {
    pb_str_reserve(b, (size_t)l);
    vsnprintf(b->s + b->n, (size_t)l + 1, fmt, ap2);
    b->n += (size_t)l;
  }
  va_end(ap2);
}
char *pb_str_take(PbStr *b) {
  if (!b->s) { pb_str_reserve(b, 0); b->s[0] = 0; }
  char *r = b->s;
  pb_str_init(b);
  return r;
}

/* ── pointer map ─────────────────────────────────────────────────────── */
static uint64_t ptr_hash(const void *p) {
  uint64_t x = (uint64_t)(uintptr_t)p;
  x ^= x >> 33; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33;
  return x;
}
static void map_grow(PbKern *k) {
  int oc = k->map_cap;
  PolyUOp **ok = k->map_keys; int *ov = k->map_vals;
  k->map_cap = oc ? oc * 2 : 1024;
  k->map_keys = calloc((size_t)k->map_cap, sizeof(PolyUOp *));
  k->map_vals = calloc((size_t)k->map_cap, sizeof(int));
  for (int i = 0; i < oc; i++) {
    if (!ok[i]) continue;
    uint64_t h = ptr_hash(ok[i]) & (uint64_t)(k->map_cap - 1);
    while (k->map_keys[h]) h = (h + 1) & (uint64_t)(k->map_cap - 1);
    k->map_keys[h] = ok[i]; k->map_vals[h] = ov[i];
  }
  free(ok); free(ov);
}
int pb_kern_node(const PbKern *k, PolyUOp *u) {
  if (!k->map_cap) return -1;
  uint64_t h = ptr_hash(u) & (uint64_t)(k->map_cap - 1);
  while (k->map_keys[h]) {
    if (k->map_keys[h] == u) return k->map_vals[h];
    h = (h + 1) & (uint64_t)(k->map_cap - 1);
  }
  return -1;
}
static void map_put(PbKern *k, PolyUOp *u, int v) {
  if ((k->n_nodes + 1) * 2 > k->map_cap) map_grow(k);
  uint64_t h = ptr_hash(u) & (uint64_t)(k->map_cap - 1);
  while (k->map_keys[h]) h = (h + 1) & (uint64_t)(k->map_cap - 1);
  k->map_keys[h] = u; k->map_vals[h] = v;
}

int pb_kern_range_id(const PbKern *k, PolyUOp *r) {
  for (int i = 0; i < k->n_ranges; i++) if (k->ranges[i] == r) return i;
  return -1;
}

/* ── build ───────────────────────────────────────────────────────────── */
static int visit(PbKern *k, PolyUOp *u) {
  int id = pb_kern_node(k, u);
  if (id >= 0) return id;
  /* iterative post-order would be safer for very deep graphs; kernels here
   * are a few hundred nodes deep at most */
  int src_ids[64];
  if (u->n_src > 64) { snprintf(k->err, sizeof k->err, "node with %d sources", u->n_src); return -2; }
  for (int i = 0; i < u->n_src; i++) {
    src_ids[i] = visit(k, u->src[i]);
    if (src_ids[i] == -2) return -2;
  }
  if (k->n_nodes == k->cap_nodes) {
    k->cap_nodes = k->cap_nodes ? k->cap_nodes * 2 : 256;
    k->nodes = realloc(k->nodes, (size_t)k->cap_nodes * sizeof(PbNode));
  }
  id = k->n_nodes;
  PbNode *n = &k->nodes[id];
  memset(n, 0, sizeof *n);
  n->u = u; n->only_parent = -1;
  map_put(k, u, id);
  k->n_nodes++;

  for (int i = 0; i < u->n_src; i++) {
    PbNode *s = &k->nodes[src_ids[i]];
    bool dup = false;
    for (int j = 0; j < i; j++) if (src_ids[j] == src_ids[i]) dup = true;
    if (!dup) { s->n_uses++; s->only_parent = id; }
    n = &k->nodes[id];
    n->deps |= s->deps;
    n->has_reduce |= s->has_reduce;
  }
  n = &k->nodes[id];

  switch (u->op) {
  case POLY_OP_RANGE: {
    if (k->n_ranges >= PB_MAX_RANGES) { snprintf(k->err, sizeof k->err, "too many ranges"); return -2; }
    int r = k->n_ranges++;
    k->ranges[r] = u;
    PolyAxisType at = poly_range_axis_type(u->arg);
    k->is_reduce[r] = (at == POLY_AXIS_REDUCE || at == POLY_AXIS_GROUP_REDUCE || at == POLY_AXIS_UNROLL);
    k->extent[r] = -1; k->extent_var[r] = -1;
    if (u->n_src < 1) { snprintf(k->err, sizeof k->err, "RANGE without bound"); return -2; }
    PolyUOp *b = u->src[0];
    if (b->op == POLY_OP_CONST) k->extent[r] = b->arg.i;
    else if (b->op == POLY_OP_DEFINE_VAR) {
      for (int v = 0; v < k->n_vars; v++) if (k->vars[v] == b) k->extent_var[r] = v;
    } else { snprintf(k->err, sizeof k->err, "RANGE bound is %s", poly_op_name(b->op)); return -2; }
    n->deps = (uint64_t)1 << r;
    break;
  }
  case POLY_OP_DEFINE_VAR:
    if (k->n_vars >= PB_MAX_VARS) { snprintf(k->err, sizeof k->err, "too many vars"); return -2; }
    k->vars[k->n_vars++] = u;
    break;
  case POLY_OP_PARAM: {
    int64_t pi = u->arg.i;
    if (pi < 0 || pi >= PB_MAX_PARAMS) { snprintf(k->err, sizeof k->err, "param index %lld", (long long)pi); return -2; }
    k->params[pi] = u;
    if (pi + 1 > k->n_params) k->n_params = (int)pi + 1;
    break;
  }
  case POLY_OP_REDUCE:
    for (int i = 1; i < u->n_src; i++) {
      int r = pb_kern_range_id(k, u->src[i]);
      if (r >= 0) n->deps &= ~((uint64_t)1 << r);
    }
    n->has_reduce = true;
    k->n_reduce_nodes++;
    break;
  default: break;
  }
  if (!u->dtype.is_ptr) {
    if (u->dtype.priority == 11) k->uses_half = true;
    if (u->dtype.priority == 12) k->uses_bf16 = true;
    if (u->dtype.priority == 14) k->uses_f64 = true;
  } else {
    if (u->dtype.priority == 11) k->uses_half = true;
    if (u->dtype.priority == 12) k->uses_bf16 = true;
  }
  return id;
}

static int collect_stores(PbKern *k, PolyUOp *u, int *loop, int n_loop) {
  switch (u->op) {
  case POLY_OP_SINK: case POLY_OP_GROUP: case POLY_OP_NOOP:
    for (int i = 0; i < u->n_src; i++)
      if (collect_stores(k, u->src[i], loop, n_loop) < 0) return -1;
    return 0;
  case POLY_OP_END: {
    int l2[PB_MAX_AXES]; int n2 = n_loop;
    memcpy(l2, loop, sizeof(int) * (size_t)n_loop);
    for (int i = 1; i < u->n_src; i++) {
      int r = pb_kern_range_id(k, u->src[i]);
      if (r < 0) { snprintf(k->err, sizeof k->err, "END closes a non-range"); return -1; }
      if (n2 >= PB_MAX_AXES) { snprintf(k->err, sizeof k->err, "too many loop axes"); return -1; }
      l2[n2++] = r;
    }
    return collect_stores(k, u->src[0], l2, n2);
  }
  case POLY_OP_STORE: {
    if (k->n_stores >= PB_MAX_STORES) { snprintf(k->err, sizeof k->err, "too many stores"); return -1; }
    if (u->n_src < 2 || u->src[0]->op != POLY_OP_INDEX || u->src[0]->src[0]->op != POLY_OP_PARAM) {
      snprintf(k->err, sizeof k->err, "STORE target is not INDEX(PARAM)"); return -1;
    }
    PbStore *s = &k->stores[k->n_stores++];
    s->u = u; s->index = u->src[0]; s->value = u->src[1];
    s->param = (int)u->src[0]->src[0]->arg.i;
    /* STORE may list its ranges as extra sources in some scheduler forms */
    s->n_loop = 0;
    for (int i = n_loop - 1; i >= 0; i--) s->loop[s->n_loop++] = loop[i];
    for (int i = 2; i < u->n_src; i++) {
      int r = pb_kern_range_id(k, u->src[i]);
      if (r >= 0) {
        bool have = false;
        for (int j = 0; j < s->n_loop; j++) if (s->loop[j] == r) have = true;
        if (!have && s->n_loop < PB_MAX_AXES) s->loop[s->n_loop++] = r;
      }
    }
    return 0;
  }
  default:
    snprintf(k->err, sizeof k->err, "unexpected %s under SINK", poly_op_name(u->op));
    return -1;
  }
}

int pb_kern_build(PbKern *k, PolyUOp *sink) {
  memset(k, 0, sizeof *k);
  k->sink = sink;
  if (!sink || sink->op != POLY_OP_SINK) { snprintf(k->err, sizeof k->err, "root is not a SINK"); return -1; }
  if (visit(k, sink) < 0) return -1;
  /* range bounds that are vars were visited before the var list was complete
   * only if the var came later; resolve again */
  for (int r = 0; r < k->n_ranges; r++) {
    if (k->extent[r] >= 0) continue;
    PolyUOp *b = k->ranges[r]->src[0];
    for (int v = 0; v < k->n_vars; v++) if (k->vars[v] == b) k->extent_var[r] = v;
    if (k->extent_var[r] < 0) { snprintf(k->err, sizeof k->err, "unresolved range bound"); return -1; }
  }
  int loop[PB_MAX_AXES];
  if (collect_stores(k, sink, loop, 0) < 0) return -1;
  if (k->n_stores == 0) { snprintf(k->err, sizeof k->err, "kernel has no STORE"); return -1; }
  for (int s = 0; s < k->n_stores; s++) {
    PbStore *st = &k->stores[s];
    /* every range the store depends on must be one of its loop axes */
    uint64_t m = 0;
    for (int i = 0; i < st->n_loop; i++) m |= (uint64_t)1 << st->loop[i];
    int ni = pb_kern_node(k, st->u);
    if (k->nodes[ni].deps & ~m) { snprintf(k->err, sizeof k->err, "STORE depends on a range no END closes"); return -1; }
    for (int i = 0; i < st->n_loop; i++)
      if (k->is_reduce[st->loop[i]]) { snprintf(k->err, sizeof k->err, "STORE inside a reduce range"); return -1; }
  }
  return 0;
}

void pb_kern_free(PbKern *k) {
  free(k->nodes); free(k->map_keys); free(k->map_vals);
  k->nodes = NULL; k->map_keys = NULL; k->map_vals = NULL;
}

/* ── integer evaluation ──────────────────────────────────────────────── */
bool pb_eval_int(const PbKern *k, PolyUOp *e, const int64_t *vals,
                 const int64_t *var_vals, int64_t *out) {
  int64_t a, b, c;
  switch (e->op) {
  case POLY_OP_CONST:
    if (e->arg.kind == POLY_ARG_INT) { *out = e->arg.i; return true; }
    if (e->arg.kind == POLY_ARG_BOOL) { *out = e->arg.b ? 1 : 0; return true; }
    return false;
  case POLY_OP_RANGE: {
    int r = pb_kern_range_id(k, e);
    if (r < 0) return false;
    *out = vals[r]; return true;
  }
  case POLY_OP_DEFINE_VAR:
    for (int v = 0; v < k->n_vars; v++)
      if (k->vars[v] == e) { *out = var_vals ? var_vals[v] : e->arg.define_var.max_val; return true; }
    return false;
  case POLY_OP_CAST:
    if (!poly_dtype_is_int(e->dtype) && !poly_dtype_is_bool(e->dtype)) return false;
    if (!poly_dtype_is_int(e->src[0]->dtype) && !poly_dtype_is_bool(e->src[0]->dtype)) return false;
    return pb_eval_int(k, e->src[0], vals, var_vals, out);
  case POLY_OP_NEG:
    if (!pb_eval_int(k, e->src[0], vals, var_vals, &a)) return false;
    *out = poly_dtype_is_bool(e->dtype) ? !a : -a; return true;
  case POLY_OP_WHERE:
    if (!pb_eval_int(k, e->src[0], vals, var_vals, &a)) return false;
    if (!pb_eval_int(k, e->src[1], vals, var_vals, &b)) return false;
    if (!pb_eval_int(k, e->src[2], vals, var_vals, &c)) return false;
    *out = a ? b : c; return true;
  case POLY_OP_MULACC:
    if (!pb_eval_int(k, e->src[0], vals, var_vals, &a)) return false;
    if (!pb_eval_int(k, e->src[1], vals, var_vals, &b)) return false;
    if (!pb_eval_int(k, e->src[2], vals, var_vals, &c)) return false;
    *out = a * b + c; return true;
  default: break;
  }
  if (e->n_src != 2) return false;
  if (!poly_dtype_is_int(e->src[0]->dtype) && !poly_dtype_is_bool(e->src[0]->dtype)) return false;
  if (!pb_eval_int(k, e->src[0], vals, var_vals, &a)) return false;
  if (!pb_eval_int(k, e->src[1], vals, var_vals, &b)) return false;
  switch (e->op) {
  case POLY_OP_ADD: *out = a + b; return true;
  case POLY_OP_SUB: *out = a - b; return true;
  case POLY_OP_MUL: *out = a * b; return true;
  case POLY_OP_IDIV: if (b == 0) return false; *out = a / b; return true;
  case POLY_OP_MOD:  if (b == 0) return false; *out = a % b; return true;
  case POLY_OP_SHL: *out = a << b; return true;
  case POLY_OP_SHR: *out = a >> b; return true;
  case POLY_OP_AND: *out = a & b; return true;
  case POLY_OP_OR:  *out = a | b; return true;
  case POLY_OP_XOR: *out = a ^ b; return true;
  case POLY_OP_MAX: *out = a > b ? a : b; return true;
  case POLY_OP_CMPLT: *out = a < b; return true;
  case POLY_OP_CMPNE: *out = a != b; return true;
  case POLY_OP_CMPEQ: *out = a == b; return true;
  default: return false;
  }
}

/* ── affine fit ──────────────────────────────────────────────────────── */
static int64_t range_extent_max(const PbKern *k, int r) {
  if (k->extent[r] >= 0) return k->extent[r];
  return k->vars[k->extent_var[r]]->arg.define_var.max_val;
}

static uint64_t rng_next(uint64_t *s) {
  uint64_t x = *s; x ^= x << 13; x ^= x >> 7; x ^= x << 17; *s = x; return x;
}

void pb_fit_affine(const PbKern *k, PolyUOp *e, uint64_t mask, PbAffine *out) {
  memset(out, 0, sizeof *out);
  int64_t vals[PB_MAX_RANGES] = {0};
  int64_t base;
  if (!pb_eval_int(k, e, vals, NULL, &base)) return;
  out->offset = base;
  int ids[PB_MAX_RANGES]; int n = 0;
  for (int r = 0; r < k->n_ranges; r++) {
    if (!(mask >> r & 1)) continue;
    ids[n++] = r;
    int64_t ext = range_extent_max(k, r);
    if (ext <= 1) { out->stride[r] = 0; continue; }
    vals[r] = 1;
    int64_t v;
    if (!pb_eval_int(k, e, vals, NULL, &v)) return;
    out->stride[r] = v - base;
    vals[r] = 0;
  }
  /* verify: full line along every axis (bounded), all-max corner, random points */
  for (int i = 0; i < n; i++) {
    int r = ids[i];
    int64_t ext = range_extent_max(k, r);
    int64_t step = ext > 4096 ? ext / 4096 : 1;
    for (int64_t x = 0; x < ext; x += step) {
      vals[r] = x;
      int64_t v;
      if (!pb_eval_int(k, e, vals, NULL, &v)) return;
      if (v != base + out->stride[r] * x) return;
    }
    vals[r] = ext - 1;
    int64_t v;
    if (!pb_eval_int(k, e, vals, NULL, &v)) return;
    if (v != base + out->stride[r] * (ext - 1)) return;
    vals[r] = 0;
  }
  uint64_t seed = 0x9e3779b97f4a7c15ULL;
  for (int t = 0; t < 4096 + 1; t++) {
    int64_t expect = base;
    for (int i = 0; i < n; i++) {
      int r = ids[i];
      int64_t ext = range_extent_max(k, r);
      int64_t x = (t == 0) ? ext - 1 : (int64_t)(rng_next(&seed) % (uint64_t)(ext > 0 ? ext : 1));
      if (ext <= 0) x = 0;
      vals[r] = x;
      expect += out->stride[r] * x;
    }
    int64_t v;
    if (!pb_eval_int(k, e, vals, NULL, &v)) return;
    if (v != expect) return;
  }
  out->ok = true;
}

/* ── dtype names in generated CUDA ───────────────────────────────────── */
const char *pb_ctype(PolyDType dt) {
  switch (dt.priority) {
  case 0:  return "bool";
  case 1:  return "signed char";
  case 2:  return "unsigned char";
  case 3:  return "short";
  case 4:  return "unsigned short";
  case 5:  return "int";
  case 6:  return "unsigned int";
  case 7:  return "long long";
  case 8:  return "unsigned long long";
  case 11: return "__half";
  case 12: return "__nv_bfloat16";
  case 13: return "float";
  case 14: return "double";
  case -1: return dt.bitsize == 800 ? "int" : NULL; /* index dtype */
  default: return NULL;
  }
}
