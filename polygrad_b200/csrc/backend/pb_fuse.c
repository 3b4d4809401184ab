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


void pb_slot_usage(const PbPlan *p, PbSlotUse *u) {
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
  if (st->precompiled || st->fused_rows || st->n_params != 2 || st->n_vars) return false;
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
  PbSlotUse *u = malloc(sizeof(PbSlotUse) * (size_t)p->n_slots);
  for (int s = 0; s < p->n_steps; s++) {
    PbStep *st = &p->steps[s];
    if (st->dead) continue;
    int po, pi;
    if (!is_identity_copy(st, &po, &pi)) continue;
    pb_slot_usage(p, u);
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

static bool step_fusable(const PbStep *st) { return !st->dead && !st->precompiled && !st->fused_rows && st->n_vars == 0 && st->sink; }

bool pb_step_reads(const PbPlan *p, const PbStep *st, int slot) {
  for (int a = 0; a < st->n_params; a++)
    if ((st->rw[a] == 'r' || st->rw[a] == 'b') && pb_plan_resolve(p, st->slot[a]) == slot) return true;
  return false;
}
bool pb_step_writes(const PbPlan *p, const PbStep *st, int slot) {
  for (int a = 0; a < st->n_params; a++)
    if ((st->rw[a] == 'w' || st->rw[a] == 'W' || st->rw[a] == 'b') && pb_plan_resolve(p, st->slot[a]) == slot) return true;
  return false;
}
static int step_out_slot(const PbPlan *p, const PbStep *st) {
  for (int a = 0; a < st->n_params; a++)
    if (st->rw[a] == 'W' || st->rw[a] == 'w' || st->rw[a] == 'b') return pb_plan_resolve(p, st->slot[a]);
  return -1;
}

/* Renders the member steps order[0..no) (the last one is the final kernel) as one
 * row kernel; NULL when the chain does not have a supported form. */
char *pb_render_chain(const PbPlan *p, const int *order, const bool *keep, int no, bool out_bf16, PbFuseOut *fo) {
  PbKern kerns[CHAIN_MAX]; PbFuseIn in[CHAIN_MAX]; int slots[CHAIN_MAX][PB_MAX_PARAMS];
  bool built = true; int n_phase = 0;
  int nb = 0;
  for (int j = 0; j < no && built; j++) {
    const PbStep *m = &p->steps[order[j]];
    const int *own = m->slot; int n_own = m->n_params;
    /* a step that already is a fused chain carries the fused parameter list; its
     * own kernel's parameters are those of the schedule item */
    if (m->fused_rows) { own = p->base.schedule->items[m->item].buf_slot_indices; n_own = p->base.schedule->items[m->item].n_buf_slots; }
    if (pb_kern_build(&kerns[j], m->sink) != 0) { pb_kern_free(&kerns[j]); built = false; break; }
    nb = j + 1;
    for (int a = 0; a < PB_MAX_PARAMS; a++) slots[j][a] = -1;
    for (int a = 0; a < n_own && a < PB_MAX_PARAMS; a++) slots[j][a] = pb_plan_resolve(p, own[a]);
    in[j].k = &kerns[j]; in[j].slot = slots[j];
    in[j].role = (j == no - 1) ? PB_FUSE_FINAL : (kerns[j].n_reduce_nodes ? PB_FUSE_PHASE : PB_FUSE_PRODUCER);
    in[j].keep_out = keep && keep[j];
    if (in[j].role == PB_FUSE_PHASE) n_phase++;
  }
  char *text = NULL;
  if (built && n_phase > 0) text = pb_render_rowfused(in, no, out_bf16, fo);
  for (int j = 0; j < nb; j++) pb_kern_free(&kerns[j]);
  return text;
}

static bool env_no_keep(void) { const char *e = getenv("POLY_B200_FUSE_KEEP"); return e && e[0] == '0'; }

static int fuse_rows(PbPlan *p) {
  int fused = 0;
  PbSlotUse *u = malloc(sizeof(PbSlotUse) * (size_t)p->n_slots);
  for (int f = 0; f < p->n_steps; f++) {
    if (!step_fusable(&p->steps[f])) continue;
    pb_slot_usage(p, u);
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
    /* a member whose result is also needed outside the chain is dropped -- unless it is an elementwise
     * producer (the fused kernel can store its value as well) whose outside readers all run after F */
    bool keep_m[CHAIN_MAX] = {false};
    for (bool changed = true; changed;) {
      changed = false;
      for (int i = 1; i < nm; i++) {
        int sl = step_out_slot(p, &p->steps[mem[i]]);
        bool outside = sl < 0 || !p->slot_inter[sl], early = false;
        for (int s = 0; s < p->n_steps; s++) {
          if (p->steps[s].dead || !pb_step_reads(p, &p->steps[s], sl)) continue;
          bool in_chain = false;
          for (int j = 0; j < nm; j++) if (mem[j] == s) in_chain = true;
          if (!in_chain) { outside = true; if (s < f) early = true; }
        }
        keep_m[i] = false;
        /* (its result must be as large as the final one: a broadcast operand such as a mask would be
         * stored once per row block) */
        const int fsl = step_out_slot(p, &p->steps[f]);
        if (outside && sl >= 0 && p->slot_inter[sl] && !early && !env_no_keep() && fsl >= 0 &&
            p->slot_bytes[sl] == p->slot_bytes[fsl]) {
          PbKern kk;
          bool elementwise = pb_kern_build(&kk, p->steps[mem[i]].sink) == 0 && kk.n_reduce_nodes == 0 && kk.n_stores == 1;
          pb_kern_free(&kk);
          if (elementwise) { keep_m[i] = true; outside = false; }
        }
        if (outside) { mem[i] = mem[nm - 1]; keep_m[i] = keep_m[nm - 1]; nm--; changed = true; break; }
      }
    }
    if (nm < 2) continue;
    /* order by step, final last */
    for (int i = 1; i < nm; i++) for (int j = i; j > 1 && mem[j] < mem[j - 1]; j--) {
      int t = mem[j]; mem[j] = mem[j - 1]; mem[j - 1] = t;
      bool tk = keep_m[j]; keep_m[j] = keep_m[j - 1]; keep_m[j - 1] = tk;
    }
    int order[CHAIN_MAX]; bool keep[CHAIN_MAX]; int no = 0;
    for (int i = 1; i < nm; i++) { keep[no] = keep_m[i]; order[no++] = mem[i]; }
    keep[no] = false; order[no++] = f;
    /* nothing outside the chain may overwrite what the chain reads, between its first member and F */
    bool hazard = false;
    for (int s = order[0]; s < f && !hazard; s++) {
      bool in_chain = false;
      for (int j = 0; j < no; j++) if (order[j] == s) in_chain = true;
      if (in_chain || p->steps[s].dead) continue;
      for (int j = 0; j < no && !hazard; j++) {
        const PbStep *m = &p->steps[order[j]];
        for (int a = 0; a < m->n_params; a++)
          if (m->rw[a] == 'r' && pb_step_writes(p, &p->steps[s], pb_plan_resolve(p, m->slot[a]))) hazard = true;
      }
    }
    if (hazard) continue;

    PbFuseOut fo;
    char *text = pb_render_chain(p, order, keep, no, false, &fo);
    if (!text) continue;
    char name[64]; snprintf(name, sizeof name, "rowfused_k%d", p->steps[f].item);
    if (getenv("POLY_DUMP_KERNELS")) fprintf(stderr, "=== CUDA KERNEL %s ===\n%s\n=== END ===\n", name, text);
    PolyCudaProgram *prog = poly_compile_cuda(text, name);
    if (!prog) { free(text); continue; }
    PbStep *fs = &p->steps[f];
    poly_cuda_program_destroy(fs->prog); free(fs->text);
    fs->prog = prog; fs->text = text;
    fs->fused_rows = true; fs->n_chain = no;
    for (int j = 0; j < no; j++) { fs->chain[j] = order[j]; fs->chain_keep[j] = keep[j]; }
    fs->n_params = fo.n_params;
    for (int a = 0; a < fo.n_params; a++) { fs->slot[a] = fo.slot[a]; fs->rw[a] = fo.rw[a]; }
    fs->rw[fo.n_params] = 0;
    for (int j = 0; j < no - 1; j++) p->steps[order[j]].dead = true;
    fused += no - 1;
  }
  free(u);
  return fused;
}

/* ── attention ───────────────────────────────────────────────────────── */
/* scores = q.kT  ->  softmax(scores*scale + mask)  ->  out = p.v, where the
 * middle is a row-fused chain of exactly the four kernels polygrad's GPT-2
 * builder and poly_softmax produce (reference: src/modelzoo/models/gpt2.c:
 * 402-434, src/frontend.c:1131-1159), nothing else reads scores or p, and the
 * bf16 contraction policy is on.  The three steps become one (pb_attention.cu). */
const char *pb_hdr_line(const char *text, const char *key, char *buf, size_t cap) {
  size_t kl = strlen(key);
  for (const char *p = text; p && p[0] == '/' && p[1] == '/'; ) {
    const char *eol = strchr(p, '\n');
    size_t len = eol ? (size_t)(eol - p) : strlen(p);
    if (len >= 2 + kl && strncmp(p + 2, key, kl) == 0 && (len == 2 + kl || p[2 + kl] == ' ')) {
      size_t vl = len > 3 + kl ? len - 3 - kl : 0;
      if (vl >= cap) vl = cap - 1;
      memcpy(buf, p + 3 + kl, vl); buf[vl] = 0;
      return buf;
    }
    if (!eol) break;
    p = eol + 1;
  }
  return NULL;
}

typedef struct { char kind; long long ext, sc, sa, sb, sx; } GAxis;
typedef struct { int params[4]; int relu; char dtype[8]; GAxis ax[16]; int nax; } GHdr;

static bool parse_gemm_hdr(const char *text, GHdr *g) {
  char buf[256];
  if (!pb_hdr_line(text, "kind", buf, sizeof buf) || strcmp(buf, "gemm") != 0) return false;
  if (!pb_hdr_line(text, "params", buf, sizeof buf) || sscanf(buf, "%d %d %d %d", &g->params[0], &g->params[1], &g->params[2], &g->params[3]) != 4) return false;
  if (!pb_hdr_line(text, "relu", buf, sizeof buf)) return false;
  g->relu = atoi(buf);
  if (!pb_hdr_line(text, "dtype", buf, sizeof buf)) return false;
  snprintf(g->dtype, sizeof g->dtype, "%.7s", buf);
  if (!pb_hdr_line(text, "naxes", buf, sizeof buf)) return false;
  g->nax = atoi(buf);
  if (g->nax > 16) return false;
  for (int i = 0; i < g->nax; i++) {
    char key[16]; snprintf(key, sizeof key, "axis%d", i);
    if (!pb_hdr_line(text, key, buf, sizeof buf)) return false;
    if (sscanf(buf, "%c %lld %lld %lld %lld %lld", &g->ax[i].kind, &g->ax[i].ext, &g->ax[i].sc, &g->ax[i].sa, &g->ax[i].sb, &g->ax[i].sx) != 6) return false;
  }
  return true;
}

static bool u_const_near(PolyUOp *u, double v, double rel) {
  if (u->op != POLY_OP_CONST || u->arg.kind != POLY_ARG_FLOAT) return false;
  double d = u->arg.f - v; if (d < 0) d = -d;
  return d <= rel * (v < 0 ? -v : v);
}
static bool u_load_of(PolyUOp *u, int param) {
  return u->op == POLY_OP_LOAD && u->src[0]->op == POLY_OP_INDEX && u->src[0]->n_src == 2 &&
         u->src[0]->src[0]->op == POLY_OP_PARAM && (int)u->src[0]->src[0]->arg.i == param;
}
static int kern_param_of_slot(const PbPlan *p, const PbStep *st, int slot) {
  for (int a = 0; a < st->n_params; a++) if (pb_plan_resolve(p, st->slot[a]) == slot) return a;
  return -1;
}
/* exp2((x - m) * log2e) with x, m loads of the given parameters */
static bool u_is_shifted_exp(PolyUOp *u, int px, int pm) {
  if (u->op != POLY_OP_EXP2) return false;
  PolyUOp *m = u->src[0];
  if (m->op != POLY_OP_MUL) return false;
  PolyUOp *d = NULL;
  if (u_const_near(m->src[1], 1.4426950408889634, 1e-6)) d = m->src[0];
  else if (u_const_near(m->src[0], 1.4426950408889634, 1e-6)) d = m->src[1];
  if (!d || d->op != POLY_OP_SUB) return false;
  return u_load_of(d->src[0], px) && u_load_of(d->src[1], pm);
}

#define ABRK { if (getenv("POLY_B200_DEBUG")) fprintf(stderr, "pb_fuse: attention candidate rejected at line %d\n", __LINE__); break; }
static int fuse_attention(PbPlan *p) {
  if (!poly_b200_gemm_policy()) return 0;
  int fused = 0;
  PbSlotUse *u = malloc(sizeof(PbSlotUse) * (size_t)p->n_slots);
  for (int r = 0; r < p->n_steps; r++) {
    PbStep *R = &p->steps[r];
    if (R->dead || !R->fused_rows || R->n_chain != 4) continue;
    pb_slot_usage(p, u);
    PbStep *E = &p->steps[R->chain[0]], *MX = &p->steps[R->chain[1]], *SM = &p->steps[R->chain[2]], *NM = R;
    if (!E->sink || !MX->sink || !SM->sink || !NM->sink) continue;
    PbKern ke, kmx, ksm, knm;
    bool b1 = pb_kern_build(&ke, E->sink) == 0, b2 = pb_kern_build(&kmx, MX->sink) == 0;
    bool b3 = pb_kern_build(&ksm, SM->sink) == 0, b4 = pb_kern_build(&knm, NM->sink) == 0;
    char *text = NULL; int g1i = -1, g2i = -1;
    int slots5[5] = {-1, -1, -1, -1, -1}; char outmode = 'w';
    do {
      if (!(b1 && b2 && b3 && b4)) ABRK;
      if (ke.n_stores != 1 || kmx.n_stores != 1 || ksm.n_stores != 1 || knm.n_stores != 1) ABRK;
      if (ke.n_reduce_nodes != 0 || kmx.n_reduce_nodes != 1 || ksm.n_reduce_nodes != 1 || knm.n_reduce_nodes != 0) ABRK;
      /* items of the original schedule give the slots of each kernel's own parameters */
      const PolySchedule *sched = p->base.schedule;
      const int *se = sched->items[E->item].buf_slot_indices, *smx = sched->items[MX->item].buf_slot_indices;
      const int *ssm = sched->items[SM->item].buf_slot_indices, *snm = sched->items[NM->item].buf_slot_indices;
      #define SLOT(arr, i) pb_plan_resolve(p, (arr)[i])
      int x_slot = SLOT(se, ke.stores[0].param), mx_slot = SLOT(smx, kmx.stores[0].param);
      int sm_slot = SLOT(ssm, ksm.stores[0].param), p_slot = SLOT(snm, knm.stores[0].param);
      /* E: x = s * scale + mask */
      PolyUOp *ev = ke.stores[0].value;
      if (ev->op != POLY_OP_ADD) ABRK;
      PolyUOp *mul = NULL, *mload = NULL;
      if (ev->src[0]->op == POLY_OP_MUL && ev->src[1]->op == POLY_OP_LOAD) { mul = ev->src[0]; mload = ev->src[1]; }
      else if (ev->src[1]->op == POLY_OP_MUL && ev->src[0]->op == POLY_OP_LOAD) { mul = ev->src[1]; mload = ev->src[0]; }
      else ABRK;
      PolyUOp *sload = NULL, *cst = NULL;
      if (mul->src[0]->op == POLY_OP_LOAD && mul->src[1]->op == POLY_OP_CONST) { sload = mul->src[0]; cst = mul->src[1]; }
      else if (mul->src[1]->op == POLY_OP_LOAD && mul->src[0]->op == POLY_OP_CONST) { sload = mul->src[1]; cst = mul->src[0]; }
      else ABRK;
      if (cst->arg.kind != POLY_ARG_FLOAT || sload->src[0]->n_src != 2 || mload->src[0]->n_src != 2) ABRK;
      if (sload->src[0]->src[1] != ke.stores[0].index->src[1]) ABRK;          /* s read where x is written */
      int ps = (int)sload->src[0]->src[0]->arg.i, pmask = (int)mload->src[0]->src[0]->arg.i;
      int s_slot = SLOT(se, ps), mask_slot = SLOT(se, pmask);
      if (s_slot == mask_slot || !p->slot_inter[s_slot] || !p->slot_inter[p_slot]) ABRK;
      /* MAX, SUM, NORM: the softmax of x */
      PolyUOp *rmx = kmx.stores[0].value, *rsm = ksm.stores[0].value, *nv = knm.stores[0].value;
      if (rmx->op != POLY_OP_REDUCE || rmx->n_src != 2 || !u_load_of(rmx->src[0], kern_param_of_slot(p, MX, x_slot))) ABRK;
      if ((rmx->arg.kind == POLY_ARG_OPS ? rmx->arg.ops : (PolyOps)rmx->arg.i) != POLY_OP_MAX) ABRK;
      if (rsm->op != POLY_OP_REDUCE || rsm->n_src != 2 || (rsm->arg.kind == POLY_ARG_OPS ? rsm->arg.ops : (PolyOps)rsm->arg.i) != POLY_OP_ADD) ABRK;
      {
        int px = -1, pm = -1;
        for (int a = 0; a < ksm.n_params; a++) { if (SLOT(ssm, a) == x_slot) px = a; if (SLOT(ssm, a) == mx_slot) pm = a; }
        if (px < 0 || pm < 0 || !u_is_shifted_exp(rsm->src[0], px, pm)) ABRK;
        px = pm = -1; int pz = -1;
        for (int a = 0; a < knm.n_params; a++) { if (SLOT(snm, a) == x_slot) px = a; if (SLOT(snm, a) == mx_slot) pm = a; if (SLOT(snm, a) == sm_slot) pz = a; }
        if (px < 0 || pm < 0 || pz < 0 || nv->op != POLY_OP_FDIV || !u_is_shifted_exp(nv->src[0], px, pm) || !u_load_of(nv->src[1], pz)) ABRK;
      }
      /* producers and consumers */
      if (u[s_slot].writers != 1 || u[p_slot].writers != 1) ABRK;
      g1i = u[s_slot].first_write;
      int readers_p = 0;
      for (int s2 = 0; s2 < p->n_steps; s2++) if (!p->steps[s2].dead && pb_step_reads(p, &p->steps[s2], p_slot)) { readers_p++; g2i = s2; }
      if (readers_p != 1 || g2i <= r || g1i >= R->chain[0]) ABRK;
      PbStep *G1 = &p->steps[g1i], *G2 = &p->steps[g2i];
      if (G1->dead || G2->dead || !G1->precompiled || !G2->precompiled) ABRK;
      GHdr h1, h2;
      if (!parse_gemm_hdr(G1->text, &h1) || !parse_gemm_hdr(G2->text, &h2)) ABRK;
      if (strcmp(h1.dtype, "f32") || strcmp(h2.dtype, "f32") || h1.relu || h2.relu || h1.params[3] >= 0 || h2.params[3] >= 0) ABRK;
      if (pb_plan_resolve(p, G1->slot[h1.params[0]]) != s_slot || pb_plan_resolve(p, G2->slot[h2.params[1]]) != p_slot) ABRK;
      /* mask strides: E's ranges named by their stride in the scores */
      uint64_t all = 0;
      for (int q = 0; q < ke.n_ranges; q++) all |= (uint64_t)1 << q;
      PbAffine xs, ms;
      pb_fit_affine(&ke, ke.stores[0].index->src[1], all, &xs);
      pb_fit_affine(&ke, mload->src[0]->src[1], all, &ms);
      if (!xs.ok || !ms.ok) ABRK;
      long long c_sm = -1;
      for (int i = 0; i < h1.nax; i++) if (h1.ax[i].kind == 'm') c_sm = h1.ax[i].sc;
      long long msq = 0, msk = 0; bool okm = c_sm > 1;
      for (int q = 0; q < ke.n_ranges && okm; q++) {
        if (ke.extent[q] <= 1) continue;
        if (xs.stride[q] == c_sm) msq = ms.stride[q];
        else if (xs.stride[q] == 1) msk = ms.stride[q];
        else if (ms.stride[q] != 0) okm = false;           /* mask varies over batch or head */
      }
      if (!okm) ABRK;
      /* nothing between the first contraction and the second may overwrite q, k or the mask */
      int q_slot = pb_plan_resolve(p, G1->slot[h1.params[1]]), k_slot = pb_plan_resolve(p, G1->slot[h1.params[2]]);
      int v_slot = pb_plan_resolve(p, G2->slot[h2.params[2]]), o_slot = pb_plan_resolve(p, G2->slot[h2.params[0]]);
      bool hazard = false;
      for (int s2 = g1i + 1; s2 < g2i && !hazard; s2++) {
        if (p->steps[s2].dead) continue;
        /* q and k were read at the first contraction, the mask at the scale+mask kernel; all are now read later */
        if (pb_step_writes(p, &p->steps[s2], q_slot) || pb_step_writes(p, &p->steps[s2], k_slot) ||
            (s2 > R->chain[0] && pb_step_writes(p, &p->steps[s2], mask_slot)) ||
            pb_step_reads(p, &p->steps[s2], o_slot) || pb_step_writes(p, &p->steps[s2], o_slot)) hazard = true;
        if (s2 != R->chain[0] && s2 != r && pb_step_reads(p, &p->steps[s2], s_slot)) hazard = true;
      }
      if (hazard || u[s_slot].readers != 1) ABRK;
      if (o_slot == q_slot || o_slot == k_slot || o_slot == v_slot || o_slot == mask_slot) ABRK;
      /* program text: both contraction headers under prefixes */
      PbStr t; pb_str_init(&t);
      float scale = (float)cst->arg.f; unsigned bits; memcpy(&bits, &scale, 4);
      outmode = G2->rw[h2.params[0]] == 'W' ? 'W' : 'w';
      pb_str_printf(&t, "//PB200 1\n//kind attn\n//scale %08x\n//mask %lld %lld %lld\n//outmode %c\n", bits, (long long)ms.offset, msq, msk, outmode);
      for (int which = 0; which < 2; which++) {
        const char *src = which ? G2->text : G1->text;
        for (const char *q = src; q && q[0] == '/' && q[1] == '/'; ) {
          const char *eol = strchr(q, '\n');
          size_t len = eol ? (size_t)(eol - q) : strlen(q);
          if (strncmp(q, "//PB200", 7) != 0 && strncmp(q, "//kind", 6) != 0)
            pb_str_printf(&t, "//g%d.%.*s\n", which + 1, (int)(len - 2), q + 2);
          if (!eol) ABRK;
          q = eol + 1;
        }
      }
      text = pb_str_take(&t);
      slots5[0] = q_slot; slots5[1] = k_slot; slots5[2] = v_slot; slots5[3] = mask_slot; slots5[4] = o_slot;
      #undef SLOT
    } while (0);
    if (b1) pb_kern_free(&ke); else pb_kern_free(&ke);
    pb_kern_free(&kmx); pb_kern_free(&ksm); pb_kern_free(&knm);
    if (!text) continue;
    char name[64]; snprintf(name, sizeof name, "attention_k%d", p->steps[g2i].item);
    if (getenv("POLY_DUMP_KERNELS")) fprintf(stderr, "=== CUDA KERNEL %s ===\n%s\n=== END ===\n", name, text);
    PolyCudaProgram *prog = poly_compile_cuda(text, name);
    if (!prog) { free(text); continue; }
    PbStep *G2 = &p->steps[g2i];
    poly_cuda_program_destroy(G2->prog); free(G2->text);
    G2->prog = prog; G2->text = text; G2->n_params = 5; G2->precompiled = 1;
    for (int a = 0; a < 5; a++) G2->slot[a] = slots5[a];
    memcpy(G2->rw, "rrrr", 4); G2->rw[4] = outmode; G2->rw[5] = 0;
    p->steps[g1i].dead = true; R->dead = true;
    fused++;
  }
  free(u);
  return fused;
}



/* Does the plan update a bound buffer in place -- read it in one step and
 * write it in another?  An optimizer step does (reference: the ASSIGN nodes of
 * src/instance.c:1155-1212; the scheduler orders every reader of the old value
 * before the writer, src/sched/rangeify.c:3099-3152).  The passes below move
 * work later in the list (a producer into the chain that consumes it, a copy
 * into the strides of its readers) on the assumption that a buffer written once
 * keeps its value; such a plan therefore runs its steps as scheduled. */
bool pb_plan_updates_in_place(const PbPlan *p) {
  PbSlotUse *u = malloc(sizeof(PbSlotUse) * (size_t)p->n_slots);
  pb_slot_usage(p, u);
  bool found = false;
  for (int i = 0; i < p->n_sched_slots && !found; i++)
    if (!p->slot_inter[i] && u[i].writers > 0 && u[i].readers > 0) found = true;
  free(u);
  return found;
}

void pb_plan_fuse(PbPlan *p) {
  if (pb_plan_updates_in_place(p)) {
    if (getenv("POLY_B200_DEBUG")) fprintf(stderr, "pb_fuse: plan updates bound buffers in place; steps run as scheduled\n");
    return;
  }
  int copies = elide_copies(p);
  int rows = 0;
  const char *e = getenv("POLY_B200_FUSE");
  if (!e || strcmp(e, "copies") != 0) rows = fuse_rows(p);
  int attn = 0;
  if (!e || (strcmp(e, "copies") != 0 && strcmp(e, "rows") != 0)) attn = fuse_attention(p);
  if (getenv("POLY_B200_DEBUG"))
    fprintf(stderr, "pb_fuse: %d copy kernels elided, %d kernels folded into row kernels, %d attention chains fused\n", copies, rows, attn);
  if (!e || (strcmp(e, "copies") != 0 && strcmp(e, "rows") != 0 && strcmp(e, "attn") != 0)) pb_plan_operands(p);
}
