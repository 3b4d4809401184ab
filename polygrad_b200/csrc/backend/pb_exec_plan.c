/*
 * pb_exec_plan.c -- plan compiler and executor for the CUDA device.
 *
 * Takes over three entry points of polygrad's src/exec_plan.c for
 * POLY_DEVICE_CUDA and forwards every other device to the original code, which
 * is compiled under the names poly_ref_* (see the Makefile):
 *
 *   poly_compile_schedule   (reference: src/exec_plan.c:801)
 *   poly_compiled_plan_run  (reference: src/exec_plan.c:934)
 *   poly_compiled_plan_free (reference: src/exec_plan.c:1062)
 *
 * What changes relative to the reference plan for CUDA:
 *   - the reference allocates one buffer per intermediate for the life of the
 *     plan (src/exec_plan.c:860-881) and zeroes all of them before every run
 *     (:946-963).  Here intermediates live in one arena, placed by live range,
 *     and only a buffer whose first access is not a whole-buffer overwrite is
 *     zeroed, right before that access;
 *   - the reference launches one kernel at a time with two mallocs and a device
 *     synchronisation each (:584-608).  Here argument blocks are persistent,
 *     launches are asynchronous, and from the third run on the whole step is
 *     replayed as one CUDA graph for as long as the bound buffers and the
 *     converted weight copies stay valid;
 *   - passes over the step list remove kernels that only re-materialise a
 *     buffer (the scheduler's CONTIGUOUS barriers, src/modelzoo/models/gpt2.c:38)
 *     and fuse the softmax chain (pb_fuse.c).
 *
 * Kernels with DEFINE_VAR parameters (dynamic shapes) keep the reference plan
 * path, which drives the same backend symbols one kernel at a time.
 * POLY_B200_PLAN=ref forces that path for everything (debugging).
 */
#include "pb_plan.h"
#include "pb_outline.h"
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

/* runtime (libpolyb200.so) */
int poly_b200_program_info(PolyCudaProgram *prog, char *rw, int cap, int *n_params, int *n_vars, int *precompiled);
int poly_b200_program_stale(PolyCudaProgram *prog, void **args);
unsigned long long poly_b200_pool_epoch(void);
int poly_b200_capture_begin(void);
void *poly_b200_capture_end(int discard);
int poly_b200_graph_launch(void *exec, unsigned long long n_kernels, unsigned long long n_precompiled);
void poly_b200_graph_destroy(void *exec);
int poly_b200_memset_now(unsigned long long ptr, unsigned char val, size_t bytes);
int poly_b200_timing_active(void);
int poly_b200_ptr_on_host(const void *p);
int poly_b200_note_access(const void *p, char mode);
int poly_b200_average_enqueue(void *ptr, size_t count);
int poly_b200_average_join(void);
void poly_b200_average_group_bytes(size_t bytes);

/* the original plan code, compiled under other names */
PolyCompiledPlan *poly_ref_compile_schedule(PolyCtx *ctx, PolySchedule *schedule, PolyDeviceId device);
int poly_ref_compiled_plan_run(PolyCompiledPlan *plan, void **slot_data, int n_slots,
                               struct PolyVarBinding *var_bindings, int n_var_bindings);
void poly_ref_compiled_plan_free(PolyCompiledPlan *plan);

#define PB_MAX_PLANS 1024
static PbPlan *g_plans[PB_MAX_PLANS];

static PbPlan *as_pb_plan(PolyCompiledPlan *p) {
  for (int i = 0; i < PB_MAX_PLANS; i++) if ((PolyCompiledPlan *)g_plans[i] == p) return g_plans[i];
  return NULL;
}

static bool env_is(const char *name, const char *val) {
  const char *e = getenv(name);
  return e && strcmp(e, val) == 0;
}

/* ── lowering one item ───────────────────────────────────────────────── */
static int lower_step(PolyCtx *ctx, PolySchedule *sched, int item_idx, const char *fn_name, PbStep *st) {
  PolyExecItem *item = &sched->items[item_idx];
  memset(st, 0, sizeof *st);
  st->item = item_idx;
  int n_lin = 0;
  PolyUOp **lin = poly_linearize_cuda(ctx, item->root, &n_lin);
  if (!lin) return -1;
  st->sink = lin[0];
  char *src = poly_render_cuda(lin, n_lin, fn_name, 256);
  free(lin);
  if (!src) return -1;
  if (getenv("POLY_DUMP_KERNELS")) fprintf(stderr, "=== CUDA KERNEL %s ===\n%s\n=== END ===\n", fn_name, src);
  st->prog = poly_compile_cuda(src, fn_name);
  if (!st->prog) { fprintf(stderr, "=== FAILED CUDA KERNEL %s ===\n%s\n=== END ===\n", fn_name, src); free(src); return -1; }
  st->text = src;
  int np = 0, nv = 0, pre = 0;
  poly_b200_program_info(st->prog, st->rw, (int)sizeof st->rw, &np, &nv, &pre);
  st->precompiled = pre;
  st->n_vars = nv;
  if (np > item->n_buf_slots || np > PB_MAX_PARAMS) {
    fprintf(stderr, "polygrad: cuda: kernel %s has %d parameters, schedule lists %d\n", fn_name, np, item->n_buf_slots);
    return -1;
  }
  st->n_params = np;
  for (int i = 0; i < np; i++) st->slot[i] = item->buf_slot_indices[i];
  return 0;
}

static long long g_kernels_cut = 0;
/* Scheduled kernels that plans compiled so far run as several steps (pb_outline.c). */
long long poly_b200_kernels_cut(void) { return g_kernels_cut; }

/* A kernel the renderer had to take as generated code although it holds contractions: cut it
 * (pb_outline.c), lower the pieces, and keep them if every contraction among them is now run by
 * the contraction kernels.  Temporaries become plan slots and are placed in the arena like any
 * other intermediate.  Returns the number of steps written to out (0: the kernel stays whole). */
static int lower_cut(PbPlan *p, PolyCtx *ctx, PolySchedule *sched, int item_idx, const char *fn_name, const PbStep *whole, PbStep *out) {
  PbPiece pieces[PB_MAX_PIECES];
  int64_t temp_numel[PB_MAX_TEMPS];
  int n_temps = 0;
  const int n = pb_outline(ctx, whole->sink, pieces, PB_MAX_PIECES, temp_numel, &n_temps);
  if (n < 2) return 0;
  PolyExecItem *item = &sched->items[item_idx];
  int temp_slot[PB_MAX_TEMPS];
  for (int t = 0; t < n_temps; t++) temp_slot[t] = -1;
  int done = 0;
  bool ok = true;
  for (int i = 0; i < n && ok; i++) {
    PbStep *st = &out[i];
    memset(st, 0, sizeof *st);
    st->item = item_idx;
    char name[96];
    snprintf(name, sizeof name, "%s_p%d", fn_name, i);
    int n_lin = 0;
    PolyUOp **lin = poly_linearize_cuda(ctx, pieces[i].sink, &n_lin);
    if (!lin) { ok = false; break; }
    st->sink = lin[0];
    char *src = poly_render_cuda(lin, n_lin, name, 256);
    free(lin);
    if (!src) { ok = false; break; }
    if (pieces[i].must_be_contraction && !strstr(src, "//kind gemm") && !strstr(src, "//kind scatter")) {
      if (getenv("POLY_B200_DEBUG")) fprintf(stderr, "pb_plan: %s: piece %d is not recognised as a contraction; the kernel stays whole\n", fn_name, i);
      free(src); ok = false; break;
    }
    if (getenv("POLY_DUMP_KERNELS")) fprintf(stderr, "=== CUDA KERNEL %s ===\n%s\n=== END ===\n", name, src);
    st->prog = poly_compile_cuda(src, name);
    st->text = src;
    done = i + 1;
    if (!st->prog) { ok = false; break; }
    int np = 0, nv = 0, pre = 0;
    poly_b200_program_info(st->prog, st->rw, (int)sizeof st->rw, &np, &nv, &pre);
    st->precompiled = pre; st->n_vars = nv; st->n_params = np;
    if (np != pieces[i].n_params || nv != 0) { ok = false; break; }
    for (int a = 0; a < np && ok; a++) {
      const int src_of = pieces[i].param_src[a];
      if (src_of >= 0) {
        if (src_of >= item->n_buf_slots) ok = false;
        else st->slot[a] = item->buf_slot_indices[src_of];
      } else {
        const int t = -src_of - 1;
        if (t >= n_temps) { ok = false; break; }
        if (temp_slot[t] < 0) temp_slot[t] = pb_plan_add_slot(p, temp_numel[t] * (int64_t)sizeof(float));
        st->slot[a] = temp_slot[t];
      }
    }
  }
  if (!ok) {
    for (int i = 0; i < done; i++) pb_step_release(&out[i]);
    return 0;
  }
  return n;
}

void pb_step_release(PbStep *st) {
  if (st->prog) poly_cuda_program_destroy(st->prog);
  free(st->text);
  st->prog = NULL; st->text = NULL;
}

/* ── arena placement by live range ───────────────────────────────────── */
typedef struct { int64_t off, size; } Hole;

static int place_intermediates(PbPlan *p) {
  int ns = p->n_slots;
  int *first = malloc(sizeof(int) * (size_t)ns), *last = malloc(sizeof(int) * (size_t)ns);
  char *first_mode = calloc((size_t)ns, 1);
  for (int i = 0; i < ns; i++) { first[i] = -1; last[i] = -1; }
  for (int s = 0; s < p->n_steps; s++) {
    PbStep *st = &p->steps[s];
    if (st->dead) continue;
    for (int a = 0; a < st->n_params; a++) {
      char m = st->rw[a];
      if (m == '-' || m == 0) continue;
      int sl = pb_plan_resolve(p, st->slot[a]);
      if (first[sl] < 0) { first[sl] = s; first_mode[sl] = m; }
      else if (first[sl] == s && m != 'W') first_mode[sl] = m;   /* also read in its first step */
      last[sl] = s;
    }
  }
  /* zero fills: an intermediate whose first access does not overwrite all of it */
  p->n_zero = 0;
  for (int i = 0; i < ns; i++) if (p->slot_inter[i] && first[i] >= 0 && first_mode[i] != 'W') p->n_zero++;
  p->zero_step = malloc(sizeof(int) * (size_t)(p->n_zero + 1));
  p->zero_slot = malloc(sizeof(int) * (size_t)(p->n_zero + 1));
  int nz = 0;
  for (int i = 0; i < ns; i++) if (p->slot_inter[i] && first[i] >= 0 && first_mode[i] != 'W') { p->zero_step[nz] = first[i]; p->zero_slot[nz] = i; nz++; }

  Hole *holes = malloc(sizeof(Hole) * (size_t)(ns + 2));
  int nh = 0;
  int64_t top = 0;
  for (int s = 0; s < p->n_steps; s++) {
    /* allocate what is first touched here (largest first keeps fragmentation low) */
    for (;;) {
      int pick = -1;
      for (int i = 0; i < ns; i++)
        if (p->slot_inter[i] && first[i] == s && p->slot_off[i] < 0 && (pick < 0 || p->slot_bytes[i] > p->slot_bytes[pick])) pick = i;
      if (pick < 0) break;
      int64_t need = (p->slot_bytes[pick] + 255) & ~(int64_t)255;
      if (need == 0) need = 256;
      int best = -1;
      for (int h = 0; h < nh; h++) if (holes[h].size >= need && (best < 0 || holes[h].size < holes[best].size)) best = h;
      if (best >= 0) {
        p->slot_off[pick] = holes[best].off;
        holes[best].off += need; holes[best].size -= need;
        if (holes[best].size == 0) { holes[best] = holes[nh - 1]; nh--; }
      } else {
        /* grow: extend a hole that ends at the top, else append */
        int tail = -1;
        for (int h = 0; h < nh; h++) if (holes[h].off + holes[h].size == top) tail = h;
        if (tail >= 0) { p->slot_off[pick] = holes[tail].off; top = holes[tail].off + need; holes[tail] = holes[nh - 1]; nh--; }
        else { p->slot_off[pick] = top; top += need; }
      }
    }
    /* release what is last touched here */
    for (int i = 0; i < ns; i++) {
      if (!p->slot_inter[i] || last[i] != s || p->slot_off[i] < 0) continue;
      int64_t off = p->slot_off[i], size = (p->slot_bytes[i] + 255) & ~(int64_t)255;
      if (size == 0) size = 256;
      /* merge with neighbours */
      for (int h = 0; h < nh;) {
        if (holes[h].off + holes[h].size == off) { off = holes[h].off; size += holes[h].size; holes[h] = holes[nh - 1]; nh--; h = 0; continue; }
        if (off + size == holes[h].off) { size += holes[h].size; holes[h] = holes[nh - 1]; nh--; h = 0; continue; }
        h++;
      }
      holes[nh].off = off; holes[nh].size = size; nh++;
    }
  }
  p->arena_bytes = top;
  free(holes); free(first); free(last); free(first_mode);
  return 0;
}

int pb_plan_resolve(const PbPlan *p, int slot) {
  int guard = 0;
  while (p->slot_alias[slot] >= 0 && guard++ < 64) slot = p->slot_alias[slot];
  return slot;
}

int pb_plan_add_slot(PbPlan *p, int64_t bytes) {
  int n = p->n_slots + 1;
  p->slot_bytes = realloc(p->slot_bytes, sizeof(int64_t) * (size_t)n);
  p->slot_off = realloc(p->slot_off, sizeof(int64_t) * (size_t)n);
  p->slot_alias = realloc(p->slot_alias, sizeof(int) * (size_t)n);
  p->slot_inter = realloc(p->slot_inter, (size_t)n);
  p->slot_ptr = realloc(p->slot_ptr, sizeof(void *) * (size_t)n);
  p->slot_bytes[n - 1] = bytes; p->slot_off[n - 1] = -1; p->slot_alias[n - 1] = -1; p->slot_inter[n - 1] = 1; p->slot_ptr[n - 1] = NULL;
  p->n_slots = n;
  return n - 1;
}

/* ── compile ─────────────────────────────────────────────────────────── */
static void plan_destroy(PbPlan *p) {
  if (!p) return;
  for (int i = 0; i < PB_MAX_PLANS; i++) if (g_plans[i] == p) g_plans[i] = NULL;
  if (p->graph) poly_b200_graph_destroy(p->graph);
  for (int s = 0; s < p->n_steps; s++) pb_step_release(&p->steps[s]);
  if (p->arena) poly_cuda_free(p->arena);
  free(p->steps); free(p->slot_bytes); free(p->slot_off); free(p->slot_alias); free(p->slot_inter); free(p->slot_ptr);
  free(p->zero_step); free(p->zero_slot); free(p->graph_ext); free(p->graph_acc_ptr); free(p->graph_acc_mode);
  if (p->stage) for (int i = 0; i < p->n_sched_slots; i++) if (p->stage[i]) poly_cuda_free(p->stage[i]);
  free(p->stage); free(p->slot_acc); free(p->ext_seen); free(p->ext_host);
  free(p->avg_at); free(p->avg_slot);
  free(p->base.slot_to_data);
  free(p);
}

PolyCompiledPlan *poly_compile_schedule(PolyCtx *ctx, PolySchedule *sched, PolyDeviceId device) {
  if (device != POLY_DEVICE_CUDA || env_is("POLY_B200_PLAN", "ref"))
    return poly_ref_compile_schedule(ctx, sched, device);
  if (!ctx || !sched) return NULL;
  if (poly_cuda_init() != 0) return NULL;

  PbPlan *p = calloc(1, sizeof *p);
  if (!p) return NULL;
  p->base.schedule = sched;
  p->base.device = device;
  p->base.allocator = &POLY_CUDA_ALLOCATOR;
  p->ctx = ctx;
  int steps_cap = sched->n_items + PB_MAX_PIECES;
  p->n_steps = 0;
  p->steps = calloc((size_t)steps_cap, sizeof(PbStep));

  static int plan_counter = 0;
  bool has_vars = false;
  for (int s = 0; s < sched->n_items && !has_vars; s++)
    if (sched->items[sched->exec_order[s]].n_var_uops > 0) has_vars = true;
  if (has_vars) { plan_destroy(p); return poly_ref_compile_schedule(ctx, sched, device); }

  p->n_slots = 0;
  for (int i = 0; i < sched->n_buf_slots; i++) {
    int idx = pb_plan_add_slot(p, sched->buf_slots[i].nbytes > 0 ? sched->buf_slots[i].nbytes : (int64_t)sizeof(float));
    p->slot_inter[idx] = sched->buf_slots[i].is_intermediate ? 1 : 0;
  }
  p->n_sched_slots = sched->n_buf_slots;

  int n_cut = 0;
  for (int s = 0; s < sched->n_items; s++) {
    int k = sched->exec_order[s];
    if (sched->items[k].kind != POLY_EXEC_COMPUTE) {
      fprintf(stderr, "polygrad: compile_schedule: non-COMPUTE item %d not supported\n", k);
      plan_destroy(p); return NULL;
    }
    if (p->n_steps + PB_MAX_PIECES > steps_cap) {
      steps_cap = steps_cap * 2 + PB_MAX_PIECES;
      PbStep *ns = realloc(p->steps, sizeof(PbStep) * (size_t)steps_cap);
      if (!ns) { plan_destroy(p); return NULL; }
      memset(ns + p->n_steps, 0, sizeof(PbStep) * (size_t)(steps_cap - p->n_steps));
      p->steps = ns;
    }
    char fn_name[64];
    snprintf(fn_name, sizeof fn_name, "plan%d_k%d", plan_counter, k);
    PbStep *st = &p->steps[p->n_steps];
    if (lower_step(ctx, sched, k, fn_name, st) != 0) {
      fprintf(stderr, "polygrad: compile_schedule: backend 'cuda' failed for kernel %d\n", k);
      p->n_steps++;                       /* so that what the step already holds is released */
      plan_destroy(p); return NULL;
    }
    int n_here = 1;
    if (!st->precompiled && !env_is("POLY_B200_OUTLINE", "0")) {
      PbStep cut[PB_MAX_PIECES];
      int n = lower_cut(p, ctx, sched, k, fn_name, st, cut);
      if (n > 0) {
        pb_step_release(st);
        memcpy(st, cut, sizeof(PbStep) * (size_t)n);
        n_here = n; n_cut++;
      }
    }
    p->n_steps += n_here;
  }
  plan_counter++;
  g_kernels_cut += n_cut;
  if (n_cut > 0 && getenv("POLY_B200_DEBUG")) fprintf(stderr, "pb_plan: %d kernels cut into contractions and elementwise pieces\n", n_cut);

  if (!env_is("POLY_B200_FUSE", "0")) pb_plan_fuse(p);

  if (place_intermediates(p) != 0) { plan_destroy(p); return NULL; }
  if (p->arena_bytes > 0) {
    p->arena = poly_cuda_alloc((size_t)p->arena_bytes);
    if (!p->arena) { plan_destroy(p); return NULL; }
  }
  for (int i = 0; i < p->n_slots; i++)
    if (p->slot_inter[i] && p->slot_off[i] >= 0) p->slot_ptr[i] = (void *)(uintptr_t)(p->arena + (unsigned long long)p->slot_off[i]);

  /* how the live steps use each bound buffer (decides the copies around a run
   * when the buffer turns out to be host memory) */
  {
    size_t n = (size_t)(sched->n_buf_slots > 0 ? sched->n_buf_slots : 1);
    p->slot_acc = calloc(n, 1); p->ext_host = calloc(n, 1);
    p->ext_seen = calloc(n, sizeof(void *)); p->stage = calloc(n, sizeof(unsigned long long));
    for (int s = 0; s < p->n_steps; s++) {
      const PbStep *st = &p->steps[s];
      if (st->dead) continue;
      for (int a = 0; a < st->n_params; a++) {
        int sl = pb_plan_resolve(p, st->slot[a]);
        if (sl < 0 || sl >= sched->n_buf_slots) continue;
        char m = st->rw[a];
        if (m == 'r' || m == 'b' || m == 'w') p->slot_acc[sl] |= PB_ACC_READ;      /* a partial write keeps the rest */
        if (m == 'w' || m == 'W' || m == 'b') p->slot_acc[sl] |= PB_ACC_WRITE;
      }
    }
  }

  /* where a data-parallel training step averages what it wrote: after the last write of each bound
   * float32 buffer of a plan that updates in place (parameters, the loss) */
  if (pb_plan_updates_in_place(p)) {
    const int n = sched->n_buf_slots;
    int *last = malloc(sizeof(int) * (size_t)(n > 0 ? n : 1));
    p->avg_at = malloc(sizeof(int) * (size_t)(n > 0 ? n : 1));
    p->avg_slot = malloc(sizeof(int) * (size_t)(n > 0 ? n : 1));
    for (int i = 0; i < n; i++) last[i] = -1;
    for (int s = 0; s < p->n_steps; s++) {
      const PbStep *st = &p->steps[s];
      if (st->dead) continue;
      for (int a = 0; a < st->n_params; a++) {
        int sl = pb_plan_resolve(p, st->slot[a]);
        char m = st->rw[a];
        if (sl >= 0 && sl < n && !p->slot_inter[sl] && (m == 'w' || m == 'W' || m == 'b')) last[sl] = s;
      }
    }
    for (int s = 0; s < p->n_steps; s++)
      for (int i = 0; i < n; i++)
        if (last[i] == s && poly_dtype_eq(poly_dtype_scalar(sched->buf_slots[i].dtype), POLY_FLOAT32)) {
          p->avg_at[p->n_avg] = s; p->avg_slot[p->n_avg] = i; p->n_avg++;
        }
    free(last);
  }

  /* fields other polygrad code may look at */
  p->base.n_slot_to_data = sched->n_buf_slots;
  p->base.slot_to_data = calloc((size_t)(sched->n_buf_slots > 0 ? sched->n_buf_slots : 1), sizeof(void *));

  if (env_is("POLY_B200_DEBUG", "2")) {
    /* the step list: kind, item, and each parameter's slot with its access */
    for (int i = 0; i < p->n_steps; i++) {
      const PbStep *st = &p->steps[i];
      if (st->dead) continue;
      char kind[24] = "jit";
      if (st->precompiled && st->text) pb_hdr_line(st->text, "kind", kind, sizeof kind);
      else if (st->fused_rows) snprintf(kind, sizeof kind, "rows(%d)", st->n_chain);
      fprintf(stderr, "pb_plan: step %3d item %3d %-8s", i, st->item, kind);
      for (int a = 0; a < st->n_params; a++) fprintf(stderr, " %c%d%s", st->rw[a], pb_plan_resolve(p, st->slot[a]), p->slot_inter[pb_plan_resolve(p, st->slot[a])] ? "" : "x");
      fprintf(stderr, "\n");
    }
  }
  if (getenv("POLY_B200_DEBUG")) {
    int live = 0, dead = 0; int64_t sum = 0;
    for (int s = 0; s < p->n_steps; s++) { if (p->steps[s].dead) dead++; else live++; }
    for (int i = 0; i < p->n_slots; i++) if (p->slot_inter[i] && p->slot_off[i] >= 0) sum += p->slot_bytes[i];
    fprintf(stderr, "pb_plan: %d steps (%d removed), arena %.1f MB for %.1f MB of intermediates, %d zero fills\n",
            live, dead, p->arena_bytes / 1e6, sum / 1e6, p->n_zero);
  }

  for (int i = 0; i < PB_MAX_PLANS; i++) if (!g_plans[i]) { g_plans[i] = p; return &p->base; }
  fprintf(stderr, "polygrad: cuda: too many live plans\n");
  plan_destroy(p);
  return NULL;
}

/* ── run ─────────────────────────────────────────────────────────────── */
static int g_average_updates = -1;
static bool average_updates(void) {
  if (g_average_updates < 0) { const char *e = getenv("POLY_B200_AVERAGE_UPDATES"); g_average_updates = (e && e[0] == '1') ? 1 : 0; }
  return g_average_updates == 1;
}
/* Data-parallel training (there is nothing like it in the reference: one device, src/runtime_cuda.c:192):
 * while on, every plan that updates bound buffers in place averages each of them over the ranks of the
 * communicator (poly_b200_comm_init) right after the step that writes it last, behind the rest of
 * the plan.  Exact for plain SGD, whose update is linear in the gradient. */
void poly_b200_set_update_averaging(int on) { g_average_updates = on ? 1 : 0; }
int  poly_b200_update_averaging(void) { return average_updates() ? 1 : 0; }

/* Where the averaging happens.  Launch by launch, each all-reduce can be issued right after the step
 * that writes the buffer last, so that the transfers hide behind the rest of the backward pass; but
 * then the plan cannot be replayed as a CUDA graph, and launching a few hundred steps one by one costs
 * more than the overlap wins until the transfers are long: with 268 MB to average on two GPUs
 * (V = 50257, D = 768, 4 layers; 17.8 ms per step alone) the step took 19.2 ms that way and 18.6 ms with
 * the graph replayed and everything averaged after it in a few NCCL groups.  So a plan keeps its
 * graph and averages afterwards unless it has 1 GB or more to average.
 * POLY_B200_AVERAGE_INLINE=0/1 forces one or the other. */
static bool average_inline(const PbPlan *p) {
  if (p->n_avg == 0 || !average_updates()) return false;
  const char *e = getenv("POLY_B200_AVERAGE_INLINE");
  if (e && (e[0] == '0' || e[0] == '1') && !e[1]) return e[0] == '1';
  int64_t bytes = 0;
  for (int i = 0; i < p->n_avg; i++) bytes += p->slot_bytes[p->avg_slot[i]];
  return bytes >= ((int64_t)1 << 30);
}

static int average_after(PbPlan *p) {
  int rc = 0;
  poly_b200_average_group_bytes((size_t)1 << 30);      /* nothing left to hide behind: as few groups as possible */
  for (int i = 0; i < p->n_avg && rc == 0; i++) {
    const int sl = p->avg_slot[i];
    if (p->slot_ptr[sl]) rc = poly_b200_average_enqueue(p->slot_ptr[sl], (size_t)p->slot_bytes[sl] / sizeof(float));
  }
  poly_b200_average_group_bytes(0);
  return rc != 0 ? rc : poly_b200_average_join();
}

static int run_eager(PbPlan *p) {
  int zi = 0, ai = 0;
  const bool avg = average_inline(p);
  for (int s = 0; s < p->n_steps; s++) {
    for (zi = 0; zi < p->n_zero; zi++)
      if (p->zero_step[zi] == s) {
        int sl = p->zero_slot[zi];
        if (poly_b200_memset_now((unsigned long long)(uintptr_t)p->slot_ptr[sl], 0, (size_t)p->slot_bytes[sl]) != 0) return -1;
      }
    PbStep *st = &p->steps[s];
    if (st->dead) continue;
    for (int a = 0; a < st->n_params; a++) {
      int sl = pb_plan_resolve(p, st->slot[a]);
      st->dptr[a] = (unsigned long long)(uintptr_t)p->slot_ptr[sl];
      st->argv[a] = &st->dptr[a];
      if (!st->dptr[a] && st->rw[a] != '-') {
        fprintf(stderr, "polygrad: plan_run: missing data for param %d (slot %d) in kernel %d\n", a, sl, st->item);
        return -1;
      }
    }
    if (poly_cuda_launch(st->prog, st->argv, st->n_params, 1, 1, 1, 256, 1, 1) != 0) return -1;
    for (; avg && ai < p->n_avg && p->avg_at[ai] <= s; ai++) {
      const int sl = p->avg_slot[ai];
      if (p->avg_at[ai] == s && p->slot_ptr[sl] &&
          poly_b200_average_enqueue(p->slot_ptr[sl], (size_t)p->slot_bytes[sl] / sizeof(float)) != 0) return -1;
    }
  }
  if (avg && poly_b200_average_join() != 0) return -1;
  return 0;
}

/* The accesses of the live steps to bound (external) buffers, in step order, as the
 * eager run reports them launch by launch; a graph replay reports the same list. */
static void record_graph_accesses(PbPlan *p) {
  int cap = 0;
  for (int s = 0; s < p->n_steps; s++) if (!p->steps[s].dead) cap += p->steps[s].n_params;
  free(p->graph_acc_ptr); free(p->graph_acc_mode);
  p->graph_acc_ptr = malloc(sizeof(void *) * (size_t)(cap + 1));
  p->graph_acc_mode = malloc((size_t)(cap + 1));
  p->n_graph_acc = 0;
  for (int s = 0; s < p->n_steps; s++) {
    const PbStep *st = &p->steps[s];
    if (st->dead) continue;
    for (int a = 0; a < st->n_params; a++) {
      const char m = st->rw[a];
      if (m == '-' || m == 0) continue;
      const int sl = pb_plan_resolve(p, st->slot[a]);
      if (sl < 0 || sl >= p->n_sched_slots || p->slot_inter[sl] || !p->slot_ptr[sl]) continue;
      /* repeated reads of one buffer tell the runtime nothing new */
      if (m == 'r') {
        bool seen = false;
        for (int i = p->n_graph_acc - 1; i >= 0 && !seen; i--)
          if (p->graph_acc_ptr[i] == p->slot_ptr[sl]) seen = true;
        if (seen) continue;
      }
      p->graph_acc_ptr[p->n_graph_acc] = p->slot_ptr[sl];
      p->graph_acc_mode[p->n_graph_acc] = m;
      p->n_graph_acc++;
    }
  }
}

static bool graph_valid(PbPlan *p) {
  if (!p->graph) return false;
  if (p->graph_epoch != poly_b200_pool_epoch()) return false;
  for (int i = 0; i < p->n_sched_slots; i++)
    if (!p->slot_inter[i] && p->graph_ext[i] != p->slot_ptr[i]) return false;
  for (int s = 0; s < p->n_steps; s++) {
    PbStep *st = &p->steps[s];
    if (st->dead || !st->precompiled) continue;
    if (poly_b200_program_stale(st->prog, st->argv)) return false;
  }
  return true;
}

/* Bound buffers in pageable host memory.  polygrad binds a few that way even
 * when everything else is on the device: the loss scalar, the gradient outputs
 * of value_and_grad and the optimizer's moments and bias corrections
 * (reference: src/instance.c:1028-1043, 1298-1311, all CPU-domain pointers in a
 * CUDA plan's slot table).  A kernel cannot address them, so each runs from a
 * device copy of its own: filled before the steps when a step reads it, copied
 * back after them when a step wrote it.  Pinned and managed memory is device
 * addressable and is used in place. */
static int bind_slots(PbPlan *p, void **slot_data, int n_slots, int *n_staged) {
  *n_staged = 0;
  for (int i = 0; i < p->n_sched_slots; i++) {
    if (p->slot_inter[i]) continue;
    void *h = (i < n_slots) ? slot_data[i] : NULL;
    p->base.slot_to_data[i] = h;
    p->slot_ptr[i] = h;
    if (!h || !p->slot_acc[i]) continue;
    if (h != p->ext_seen[i]) { p->ext_seen[i] = h; p->ext_host[i] = (char)(poly_b200_ptr_on_host(h) ? 1 : 0); }
    if (!p->ext_host[i]) continue;
    if (!p->stage[i]) {
      p->stage[i] = poly_cuda_alloc((size_t)p->slot_bytes[i]);
      if (!p->stage[i]) return -1;
    }
    if ((p->slot_acc[i] & PB_ACC_READ) && poly_cuda_copy_htod(p->stage[i], h, (size_t)p->slot_bytes[i]) != 0) return -1;
    p->slot_ptr[i] = (void *)(uintptr_t)p->stage[i];
    (*n_staged)++;
  }
  return 0;
}

static int return_slots(PbPlan *p) {
  for (int i = 0; i < p->n_sched_slots; i++) {
    if (p->slot_inter[i] || !p->ext_host[i] || !p->stage[i] || !p->base.slot_to_data[i]) continue;
    if (p->slot_ptr[i] != (void *)(uintptr_t)p->stage[i] || !(p->slot_acc[i] & PB_ACC_WRITE)) continue;
    if (poly_cuda_copy_dtoh(p->base.slot_to_data[i], p->stage[i], (size_t)p->slot_bytes[i]) != 0) return -1;
  }
  return 0;
}

static int run_steps(PbPlan *p);

int poly_compiled_plan_run(PolyCompiledPlan *plan, void **slot_data, int n_slots,
                           struct PolyVarBinding *var_bindings, int n_var_bindings) {
  PbPlan *p = plan ? as_pb_plan(plan) : NULL;
  if (!p) return poly_ref_compiled_plan_run(plan, slot_data, n_slots, var_bindings, n_var_bindings);
  int n_staged = 0;
  if (bind_slots(p, slot_data, n_slots, &n_staged) != 0) return -1;
  int rc = run_steps(p);
  if (rc == 0 && p->n_avg > 0 && average_updates() && !average_inline(p)) rc = average_after(p);
  if (rc == 0 && n_staged > 0) rc = return_slots(p);
  return rc;
}

static int run_steps(PbPlan *p) {
  p->runs++;
  const bool graphs = !env_is("POLY_B200_GRAPH", "0") && p->graph_failures < 4 && !getenv("POLY_B200_DRYRUN") &&
                      !poly_b200_timing_active() &&    /* per-launch timing needs individual launches */
                      !average_inline(p);              /* collectives are issued between the launches */
  if (graphs && graph_valid(p)) {
    /* what the launches of an eager run tell the runtime about bound buffers: pending zero fills
     * are materialised or dropped, and written buffers get a new version, so that converted
     * copies of them held by other plans (a forward plan's bf16 weights after a training step)
     * are seen to be stale */
    for (int i = 0; i < p->n_graph_acc; i++)
      if (poly_b200_note_access(p->graph_acc_ptr[i], p->graph_acc_mode[i]) != 0) return -1;
    return poly_b200_graph_launch(p->graph, (unsigned long long)p->graph_kernels, (unsigned long long)p->graph_precompiled);
  }
  if (p->graph) { poly_b200_graph_destroy(p->graph); p->graph = NULL; p->runs = 1; }
  if (graphs && p->runs >= 3) {
    if (poly_b200_capture_begin() == 0) {
      PolyB200Stats before, after;
      poly_b200_stats(&before);
      int rc = run_eager(p);
      poly_b200_stats(&after);
      void *g = poly_b200_capture_end(rc != 0);
      if (g) {
        p->graph = g;
        p->graph_epoch = poly_b200_pool_epoch();
        p->graph_kernels = (long long)(after.launches - before.launches);
        p->graph_precompiled = (long long)(after.launches_precompiled - before.launches_precompiled);
        free(p->graph_ext);
        p->graph_ext = malloc(sizeof(void *) * (size_t)(p->n_sched_slots + 1));
        for (int i = 0; i < p->n_sched_slots; i++) p->graph_ext[i] = p->slot_ptr[i];
        record_graph_accesses(p);
        /* the captured work has not run yet; the capture run itself has noted its accesses */
        return poly_b200_graph_launch(p->graph, 0, 0);
      }
      p->graph_failures++;
      /* fall through: issue the step directly */
    }
  }
  return run_eager(p);
}

void poly_compiled_plan_free(PolyCompiledPlan *plan) {
  PbPlan *p = plan ? as_pb_plan(plan) : NULL;
  if (!p) { poly_ref_compiled_plan_free(plan); return; }
  plan_destroy(p);
}

PbPlan *pb_plan_of(PolyCompiledPlan *plan) { return plan ? as_pb_plan(plan) : NULL; }
