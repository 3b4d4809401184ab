/*
 * pb_eager.c -- the eager entry point: poly_realize_cuda, poly_cuda_copyback,
 * poly_cuda_flush_buffers, poly_cuda_prog_cache_flush.
 *
 * Reference: src/frontend.c:2450-2687.  polygrad's Python Tensor(device='cuda')
 * is the caller (py/polygrad/tensor.py:322-364): it builds a new output BUFFER
 * and a new SINK for every realize, binds HOST pointers, calls
 * poly_realize_cuda and then poly_cuda_copyback on the same bindings.  The
 * reference schedules the graph on every call, uploads every binding into a
 * device buffer it keeps per host pointer, runs the kernels one by one (an
 * allocation and a synchronisation each) and leaves results on the device
 * until poly_cuda_copyback copies every binding back.
 *
 * Here
 *  - the graph is compiled into a plan like any other (arena, elided copies,
 *    fused row chains, fused attention, tensor-core contractions) and the plan
 *    is KEPT: plans are found again by the graph's structure with BUFFER nodes
 *    compared by position, so the new SINK a caller makes for the same
 *    computation reuses the plan of the first one and only its buffers are
 *    rebound.  polygrad's own plan cache cannot serve these callers: it is
 *    keyed by the SINK's address (src/frontend.c:2118-2140);
 *  - only buffers a step reads are uploaded;
 *  - buffers a step writes stay on the device, as in the reference, until
 *    poly_cuda_copyback asks for them; a later realize that binds the same
 *    BUFFER node and host pointer reads the device copy in place, with no
 *    round trip through host memory.  The identity is the BUFFER node together
 *    with the host pointer: nodes are never reused within a context, so host
 *    memory that was freed and handed out again cannot be mistaken for a
 *    tensor that is still on the device.
 *
 * Graphs with DEFINE_VAR parameters keep the reference route, as does
 * everything under POLY_B200_LEGACY=ref.  POLY_B200_EAGER_CACHE=0 builds and
 * frees a plan per call; POLY_B200_EAGER_RESIDENT=0 copies written buffers
 * back before poly_realize_cuda returns.
 */
#include "pb_plan.h"
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

int poly_b200_ptr_on_host(const void *p);

/* polygrad's own definitions, compiled under other names */
int  poly_ref_realize_cuda(PolyCtx *ctx, PolyUOp *tensor_sink, PolyBufferBinding *bindings, int n_bindings);
int  poly_ref_cuda_copyback(PolyBufferBinding *bindings, int n_bindings);
void poly_ref_cuda_flush_buffers(void);
void poly_ref_cuda_prog_cache_flush(void);
void poly_ref_frontend_ctx_cleanup(PolyCtx *ctx);

static bool env_off(const char *name) { const char *v = getenv(name); return v && v[0] == '0' && !v[1]; }
static bool env_ref(const char *name) { const char *v = getenv(name); return v && strcmp(v, "ref") == 0; }

/* ── a graph in visiting order ───────────────────────────────────────── */
/* Depth first, sources left to right, every node numbered at its first visit
 * after its sources; BUFFER nodes are leaves here (their sources name the
 * buffer, which is what must not matter).  Two graphs compute the same thing
 * on positionally matching buffers exactly when their lists agree entry by
 * entry in op, dtype, arg and the numbers of their sources. */
typedef struct {
  PolyUOp **node; int *src_at, *src; int n, cap, n_src, src_cap;
  int *bufs; int n_bufs, bufs_cap;            /* indices of the BUFFER nodes, in visiting order */
  PolyUOp **keys; int *vals; int tcap;        /* node -> index */
  uint32_t hash;
  bool failed;
} Lin;

static void lin_free(Lin *l) {
  free(l->node); free(l->src_at); free(l->src); free(l->bufs); free(l->keys); free(l->vals);
  memset(l, 0, sizeof *l);
}

static size_t ptr_slot(const void *p, int cap) {
  uintptr_t x = (uintptr_t)p; x ^= x >> 17; x *= (uintptr_t)0x9E3779B97F4A7C15ull; x ^= x >> 29;
  return (size_t)x & (size_t)(cap - 1);
}

static int lin_find(const Lin *l, const PolyUOp *u) {
  if (!l->tcap) return -1;
  for (size_t i = ptr_slot(u, l->tcap);; i = (i + 1) & (size_t)(l->tcap - 1)) {
    if (!l->keys[i]) return -1;
    if (l->keys[i] == u) return l->vals[i];
  }
}

static bool lin_put(Lin *l, PolyUOp *u, int idx) {
  if ((l->n + 1) * 2 > l->tcap) {
    int ncap = l->tcap ? l->tcap * 2 : 256;
    PolyUOp **nk = calloc((size_t)ncap, sizeof *nk); int *nv = malloc(sizeof(int) * (size_t)ncap);
    if (!nk || !nv) { free(nk); free(nv); return false; }
    for (int i = 0; i < l->tcap; i++) if (l->keys[i]) {
      size_t j = ptr_slot(l->keys[i], ncap);
      while (nk[j]) j = (j + 1) & (size_t)(ncap - 1);
      nk[j] = l->keys[i]; nv[j] = l->vals[i];
    }
    free(l->keys); free(l->vals); l->keys = nk; l->vals = nv; l->tcap = ncap;
  }
  size_t j = ptr_slot(u, l->tcap);
  while (l->keys[j]) j = (j + 1) & (size_t)(l->tcap - 1);
  l->keys[j] = u; l->vals[j] = idx;
  return true;
}

static int lin_visit(Lin *l, PolyUOp *u) {
  if (l->failed || !u) { l->failed = true; return -1; }
  int at = lin_find(l, u);
  if (at >= 0) return at;
  const bool leaf = u->op == POLY_OP_BUFFER;
  int kids[64], *k = kids, nk = leaf ? 0 : (int)u->n_src;
  if (nk > 64 && !(k = malloc(sizeof(int) * (size_t)nk))) { l->failed = true; return -1; }
  for (int i = 0; i < nk; i++) k[i] = lin_visit(l, u->src[i]);
  if (!l->failed && l->n == l->cap) {
    int ncap = l->cap ? l->cap * 2 : 128;
    PolyUOp **nn = realloc(l->node, sizeof *nn * (size_t)ncap);
    if (nn) l->node = nn;
    int *na = realloc(l->src_at, sizeof(int) * (size_t)(ncap + 1));
    if (na) l->src_at = na;
    if (!nn || !na) l->failed = true; else l->cap = ncap;
  }
  if (!l->failed && l->n_src + nk > l->src_cap) {
    int ncap = (l->src_cap ? l->src_cap * 2 : 256) + nk;
    int *ns = realloc(l->src, sizeof(int) * (size_t)ncap);
    if (!ns) l->failed = true; else { l->src = ns; l->src_cap = ncap; }
  }
  if (!l->failed && leaf && l->n_bufs == l->bufs_cap) {
    int ncap = l->bufs_cap ? l->bufs_cap * 2 : 16;
    int *nb = realloc(l->bufs, sizeof(int) * (size_t)ncap);
    if (!nb) l->failed = true; else { l->bufs = nb; l->bufs_cap = ncap; }
  }
  int idx = -1;
  if (!l->failed && lin_put(l, u, l->n)) {
    idx = l->n++;
    l->node[idx] = u;
    l->src_at[idx] = l->n_src;
    for (int i = 0; i < nk; i++) l->src[l->n_src++] = k[i];
    l->src_at[idx + 1] = l->n_src;
    if (leaf) l->bufs[l->n_bufs++] = idx;
    uint32_t h = l->hash;
    h ^= (uint32_t)u->op;              h *= 0x01000193u;
    h ^= (uint32_t)u->dtype.priority;  h *= 0x01000193u;
    h ^= (uint32_t)u->dtype.bitsize;   h *= 0x01000193u;
    h ^= poly_arg_hash(u->arg);        h *= 0x01000193u;
    for (int i = 0; i < nk; i++) { h ^= (uint32_t)k[i]; h *= 0x01000193u; }
    l->hash = h;
  } else l->failed = true;
  if (k != kids) free(k);
  return idx;
}

static bool lin_build(Lin *l, PolyUOp *sink) {
  memset(l, 0, sizeof *l);
  l->hash = 0x811c9dc5u;
  lin_visit(l, sink);
  if (l->failed) { lin_free(l); return false; }
  return true;
}

static bool lin_same(const Lin *a, const Lin *b) {
  if (a->n != b->n || a->n_src != b->n_src || a->n_bufs != b->n_bufs || a->hash != b->hash) return false;
  for (int i = 0; i < a->n; i++) {
    const PolyUOp *x = a->node[i], *y = b->node[i];
    if (x->op != y->op || !poly_dtype_eq(x->dtype, y->dtype) || !poly_arg_eq(x->arg, y->arg)) return false;
    if (a->src_at[i + 1] - a->src_at[i] != b->src_at[i + 1] - b->src_at[i]) return false;
  }
  return memcmp(a->src, b->src, sizeof(int) * (size_t)a->n_src) == 0;
}

/* ── kept plans ──────────────────────────────────────────────────────── */
#define PB_EAGER_PLANS 128
typedef struct {
  PolyCtx *ctx; int policy;
  Lin lin;                        /* the graph the plan was compiled from */
  PolySchedule *sched; PolyCompiledPlan *plan;
  int *slot_buf;                  /* per schedule slot: which BUFFER of lin.bufs it is, -1 for intermediates */
  unsigned long long used;
} Kept;
static Kept g_kept[PB_EAGER_PLANS];
static int g_n_kept = 0;
static unsigned long long g_tick = 0, g_hits = 0, g_misses = 0;

static void kept_release(Kept *k) {
  if (k->plan) poly_compiled_plan_free(k->plan);
  if (k->sched) poly_schedule_free(k->sched);
  free(k->slot_buf);
  lin_free(&k->lin);
  memset(k, 0, sizeof *k);
}

static void kept_drop_at(int i) {
  kept_release(&g_kept[i]);
  g_kept[i] = g_kept[--g_n_kept];
  memset(&g_kept[g_n_kept], 0, sizeof g_kept[0]);
}

/* ── results that are still on the device ────────────────────────────── */
typedef struct { PolyCtx *ctx; PolyUOp *buf; void *host; size_t bytes; unsigned long long dptr; } Resident;
static Resident *g_res = NULL;
static int g_n_res = 0, g_res_cap = 0;

static int res_find(const PolyUOp *buf, const void *host) {
  for (int i = 0; i < g_n_res; i++) if (g_res[i].buf == buf && g_res[i].host == host) return i;
  return -1;
}

static void res_drop_at(int i) {
  poly_cuda_free(g_res[i].dptr);
  g_res[i] = g_res[--g_n_res];
}

/* Host memory bound under another BUFFER node now belongs to another tensor:
 * whatever was left on the device for the old one can never be asked for
 * again, and writing it back would overwrite the new owner's data. */
static void res_drop_overlapping(const PolyUOp *buf, const void *host, size_t bytes) {
  const char *lo = host, *hi = lo + bytes;
  for (int i = g_n_res - 1; i >= 0; i--) {
    const char *rl = g_res[i].host, *rh = rl + g_res[i].bytes;
    if (g_res[i].buf != buf && rl < hi && lo < rh) res_drop_at(i);
  }
}

static bool res_add(PolyCtx *ctx, PolyUOp *buf, void *host, size_t bytes, unsigned long long dptr) {
  if (g_n_res == g_res_cap) {
    int ncap = g_res_cap ? g_res_cap * 2 : 64;
    Resident *nr = realloc(g_res, sizeof *nr * (size_t)ncap);
    if (!nr) return false;
    g_res = nr; g_res_cap = ncap;
  }
  g_res[g_n_res++] = (Resident){ ctx, buf, host, bytes, dptr };
  return true;
}

/* ── one call ────────────────────────────────────────────────────────── */
typedef struct { unsigned long long dptr; int res; bool ours; } Bound;

static int run_bound(PolyCtx *ctx, PbPlan *p, const PolySchedule *sched, const int *slot_buf, const Lin *now,
                     PolyBufferBinding *bindings, int n_bindings) {
  const int ns = sched->n_buf_slots;
  const bool resident = !env_off("POLY_B200_EAGER_RESIDENT");
  void **slot_data = calloc((size_t)(ns > 0 ? ns : 1), sizeof(void *));
  Bound *bd = calloc((size_t)(ns > 0 ? ns : 1), sizeof *bd);
  PolyUOp **slot_uop = calloc((size_t)(ns > 0 ? ns : 1), sizeof *slot_uop);
  void **slot_host = calloc((size_t)(ns > 0 ? ns : 1), sizeof(void *));
  int rc = (slot_data && bd && slot_uop && slot_host) ? 0 : -1;
  for (int s = 0; s < ns && rc == 0; s++) {
    bd[s].res = -1;
    if (sched->buf_slots[s].is_intermediate) continue;
    PolyUOp *uop = slot_buf ? (slot_buf[s] >= 0 ? now->node[now->bufs[slot_buf[s]]] : NULL) : sched->buf_slots[s].buf_uop;
    void *h = NULL;
    for (int b = 0; b < n_bindings; b++) if (bindings[b].buffer == uop) { h = bindings[b].handle.ptr; break; }
    slot_uop[s] = uop; slot_host[s] = h; slot_data[s] = h;
    if (!h || !p->slot_acc[s] || !resident || !poly_b200_ptr_on_host(h)) continue;   /* the plan stages host memory itself */
    const size_t bytes = (size_t)p->slot_bytes[s];
    res_drop_overlapping(uop, h, bytes);
    int r = res_find(uop, h);
    if (r >= 0 && g_res[r].bytes != bytes) { res_drop_at(r); r = -1; }
    if (r >= 0) { bd[s].dptr = g_res[r].dptr; slot_data[s] = (void *)(uintptr_t)bd[s].dptr; continue; }
    bd[s].dptr = poly_cuda_alloc(bytes);
    bd[s].ours = true;
    if (!bd[s].dptr) { rc = -1; break; }
    if ((p->slot_acc[s] & PB_ACC_READ) && poly_cuda_copy_htod(bd[s].dptr, h, bytes) != 0) { rc = -1; break; }
    slot_data[s] = (void *)(uintptr_t)bd[s].dptr;
  }
  if (rc == 0) rc = poly_compiled_plan_run(&p->base, slot_data, ns, NULL, 0);
  /* what was written stays; what was only read goes back to the pool (the pool orders the reuse
   * of a block after the work that was issued before it was freed) */
  for (int s = 0; s < ns; s++) {
    if (!bd || !bd[s].ours || !bd[s].dptr) continue;
    if (rc == 0 && (p->slot_acc[s] & PB_ACC_WRITE) &&
        res_add(ctx, slot_uop[s], slot_host[s], (size_t)p->slot_bytes[s], bd[s].dptr)) continue;
    if (rc == 0 && (p->slot_acc[s] & PB_ACC_WRITE) &&
        poly_cuda_copy_dtoh(slot_host[s], bd[s].dptr, (size_t)p->slot_bytes[s]) != 0) rc = -1;
    poly_cuda_free(bd[s].dptr);
  }
  free(slot_data); free(bd); free(slot_uop); free(slot_host);
  return rc;
}

static int *map_slots(const PolySchedule *sched, const Lin *l) {
  int *m = malloc(sizeof(int) * (size_t)(sched->n_buf_slots > 0 ? sched->n_buf_slots : 1));
  if (!m) return NULL;
  for (int s = 0; s < sched->n_buf_slots; s++) {
    m[s] = -1;
    if (sched->buf_slots[s].is_intermediate) continue;
    int at = lin_find(l, sched->buf_slots[s].buf_uop);
    for (int b = 0; at >= 0 && b < l->n_bufs; b++) if (l->bufs[b] == at) { m[s] = b; break; }
  }
  return m;
}

int poly_realize_cuda(PolyCtx *ctx, PolyUOp *tensor_sink, PolyBufferBinding *bindings, int n_bindings) {
  if (env_ref("POLY_B200_LEGACY") || env_ref("POLY_B200_PLAN"))
    return poly_ref_realize_cuda(ctx, tensor_sink, bindings, n_bindings);
  if (!tensor_sink || tensor_sink->op != POLY_OP_SINK) {
    fprintf(stderr, "polygrad: realize_cuda: expected SINK\n");
    return -1;
  }
  if (!poly_cuda_available()) {
    fprintf(stderr, "polygrad: realize_cuda: CUDA not available\n");
    return -1;
  }
  const bool keep = !env_off("POLY_B200_EAGER_CACHE");
  const int policy = poly_b200_gemm_policy();
  Lin now;
  bool have_lin = keep && lin_build(&now, tensor_sink);
  if (have_lin) {
    for (int i = 0; i < g_n_kept; i++) {
      Kept *k = &g_kept[i];
      if (k->ctx != ctx || k->policy != policy || !lin_same(&k->lin, &now)) continue;
      k->used = ++g_tick; g_hits++;
      int rc = run_bound(ctx, pb_plan_of(k->plan), k->sched, k->slot_buf, &now, bindings, n_bindings);
      lin_free(&now);
      return rc;
    }
  }
  g_misses++;
  PolySchedule *sched = poly_schedule_for(ctx, tensor_sink, POLY_MODE_CALL);
  if (!sched) { if (have_lin) lin_free(&now); return -1; }
  PolyCompiledPlan *plan = poly_compile_schedule(ctx, sched, POLY_DEVICE_CUDA);
  if (!plan || !pb_plan_of(plan)) {
    if (plan) poly_compiled_plan_free(plan);
    poly_schedule_free(sched);
    if (have_lin) lin_free(&now);
    return poly_ref_realize_cuda(ctx, tensor_sink, bindings, n_bindings);
  }
  int *slot_buf = have_lin ? map_slots(sched, &now) : NULL;
  int rc = run_bound(ctx, pb_plan_of(plan), sched, NULL, NULL, bindings, n_bindings);
  if (rc == 0 && slot_buf) {
    if (g_n_kept == PB_EAGER_PLANS) {            /* the least recently used one makes room */
      int lru = 0;
      for (int i = 1; i < g_n_kept; i++) if (g_kept[i].used < g_kept[lru].used) lru = i;
      if (poly_b200_synchronize() != 0) rc = -1;
      kept_drop_at(lru);
    }
    g_kept[g_n_kept++] = (Kept){ ctx, policy, now, sched, plan, slot_buf, ++g_tick };
    return rc;
  }
  /* not kept: results must not depend on anything the plan owns once it is gone */
  if (rc == 0 && poly_b200_synchronize() != 0) rc = -1;
  free(slot_buf);
  poly_compiled_plan_free(plan);
  poly_schedule_free(sched);
  if (have_lin) lin_free(&now);
  return rc;
}

/* Reference: src/frontend.c:2676 copies every binding it holds a device buffer
 * for.  Here only results that are still on the device have one. */
int poly_cuda_copyback(PolyBufferBinding *bindings, int n_bindings) {
  int rc = 0;
  for (int b = 0; b < n_bindings; b++) {
    int r = bindings[b].buffer ? res_find(bindings[b].buffer, bindings[b].handle.ptr) : -1;
    if (r < 0) continue;
    if (poly_cuda_copy_dtoh(g_res[r].host, g_res[r].dptr, g_res[r].bytes) != 0) rc = -1;
    res_drop_at(r);
  }
  int ref = poly_ref_cuda_copyback(bindings, n_bindings);
  return rc != 0 ? rc : ref;
}

/* Reference: src/frontend.c:2670 frees its device buffers without copying. */
void poly_cuda_flush_buffers(void) {
  while (g_n_res > 0) res_drop_at(g_n_res - 1);
  free(g_res); g_res = NULL; g_res_cap = 0;
  poly_ref_cuda_flush_buffers();
}

/* Reference: src/frontend.c:2444 destroys the programs of its eager path. */
void poly_cuda_prog_cache_flush(void) {
  if (g_n_kept > 0) poly_b200_synchronize();
  while (g_n_kept > 0) kept_drop_at(g_n_kept - 1);
  poly_ref_cuda_prog_cache_flush();
}

/* poly_ctx_destroy calls this (src/uop.c:206-209): nothing kept here may
 * outlive the context whose nodes it points to. */
void poly_frontend_ctx_cleanup(PolyCtx *ctx) {
  if (!ctx) return;
  bool synced = false;
  for (int i = g_n_kept - 1; i >= 0; i--) {
    if (g_kept[i].ctx != ctx) continue;
    if (!synced) { poly_b200_synchronize(); synced = true; }
    kept_drop_at(i);
  }
  for (int i = g_n_res - 1; i >= 0; i--) if (g_res[i].ctx == ctx) res_drop_at(i);
  poly_ref_frontend_ctx_cleanup(ctx);
}

void poly_b200_eager_stats(unsigned long long *hits, unsigned long long *misses, int *plans_kept, int *buffers_resident) {
  if (hits) *hits = g_hits;
  if (misses) *misses = g_misses;
  if (plans_kept) *plans_kept = g_n_kept;
  if (buffers_resident) *buffers_resident = g_n_res;
}
