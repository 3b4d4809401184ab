/*
 * pb_operands.c -- plan passes over the operands of precompiled steps
 * (contractions and fused attention), whose programs address their operands
 * through an offset and one stride per axis.
 *
 *   view folding     polygrad realises every slice and permutation that feeds a
 *                    contraction as a copy kernel (reference: the CONTIGUOUS
 *                    barriers in src/modelzoo/models/gpt2.c:362-498; q, k and v
 *                    are three such copies of the qkv projection).  When a
 *                    copy's destination is read only through stride-described
 *                    operands, the copy's index map is composed into those
 *                    strides and the copy is dropped.
 *   bf16 storage     under the bf16 contraction policy an fp32 operand is
 *                    rounded to bfloat16 on its way into the tensor cores.  An
 *                    intermediate that nothing but such operands reads is stored
 *                    as bfloat16 by its producer (same element layout, 2-byte
 *                    elements) and read in place: the values reaching the
 *                    tensor cores are bit for bit the same, the conversion pass
 *                    and half of the producer's write traffic disappear.
 *   attention output written as bfloat16 in the row-major [rows][k] layout the
 *                    following projection reads.
 *
 * Index maps are composed numerically: a candidate set of strides is derived
 * from single steps along each axis and then verified on every axis end and on
 * random interior points; a map that does not verify leaves the plan unchanged.
 */
#include "pb_plan.h"
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

/* ── headers of precompiled programs ─────────────────────────────────── */
enum { OP_C = 0, OP_A = 1, OP_B = 2, OP_X = 3 };
typedef struct { char kind; long long ext, s[4]; } HAxis;          /* strides in C, A, B, X */
typedef struct {
  int nparams, params[4], relu, nax, abf16, cbf16, gelu;
  long long alpha; int has_alpha;      /* bits of the float32 scale of the sum, when it is not 1 */
  long long off[4], numel[4];
  char dtype[8];
  HAxis ax[16];
} HGemm;
typedef struct { char scale[16]; long long mask[3]; char outmode; int qkv16, obf16, tiles; HGemm g1, g2; } HAttn;

static const char *hget(const char *text, const char *pre, const char *key, char *buf, size_t cap) {
  char full[48]; snprintf(full, sizeof full, "%s%s", pre, key);
  return pb_hdr_line(text, full, buf, cap);
}

static bool hgemm_parse(const char *text, const char *pre, HGemm *g) {
  char buf[256];
  memset(g, 0, sizeof *g);
  if (!hget(text, pre, "nparams", buf, sizeof buf)) return false;
  g->nparams = atoi(buf);
  if (!hget(text, pre, "params", buf, sizeof buf) || sscanf(buf, "%d %d %d %d", &g->params[0], &g->params[1], &g->params[2], &g->params[3]) != 4) return false;
  if (!hget(text, pre, "offsets", buf, sizeof buf) || sscanf(buf, "%lld %lld %lld %lld", &g->off[0], &g->off[1], &g->off[2], &g->off[3]) != 4) return false;
  if (!hget(text, pre, "numel", buf, sizeof buf) || sscanf(buf, "%lld %lld %lld %lld", &g->numel[0], &g->numel[1], &g->numel[2], &g->numel[3]) != 4) return false;
  if (!hget(text, pre, "relu", buf, sizeof buf)) return false;
  g->relu = atoi(buf);
  if (!hget(text, pre, "dtype", buf, sizeof buf)) return false;
  snprintf(g->dtype, sizeof g->dtype, "%.7s", buf);
  if (!hget(text, pre, "naxes", buf, sizeof buf)) return false;
  g->nax = atoi(buf);
  if (g->nax < 0 || g->nax > 16) return false;
  for (int i = 0; i < g->nax; i++) {
    char key[16]; snprintf(key, sizeof key, "axis%d", i);
    HAxis *a = &g->ax[i];
    if (!hget(text, pre, key, buf, sizeof buf) ||
        sscanf(buf, "%c %lld %lld %lld %lld %lld", &a->kind, &a->ext, &a->s[0], &a->s[1], &a->s[2], &a->s[3]) != 6) return false;
  }
  g->abf16 = hget(text, pre, "abf16", buf, sizeof buf) ? atoi(buf) : 0;
  g->cbf16 = hget(text, pre, "cbf16", buf, sizeof buf) ? atoi(buf) : 0;
  g->gelu = hget(text, pre, "gelu", buf, sizeof buf) ? atoi(buf) : 0;
  g->has_alpha = hget(text, pre, "alpha", buf, sizeof buf) ? 1 : 0;
  if (g->has_alpha) g->alpha = atoll(buf);
  return true;
}

static void hgemm_emit(PbStr *t, const char *pre, const HGemm *g) {
  pb_str_printf(t, "//%snparams %d\n//%sparams %d %d %d %d\n//%sdtype %s\n", pre, g->nparams, pre, g->params[0], g->params[1],
                g->params[2], g->params[3], pre, g->dtype);
  pb_str_printf(t, "//%soffsets %lld %lld %lld %lld\n//%srelu %d\n", pre, g->off[0], g->off[1], g->off[2], g->off[3], pre, g->relu);
  pb_str_printf(t, "//%snumel %lld %lld %lld %lld\n", pre, g->numel[0], g->numel[1], g->numel[2], g->numel[3]);
  for (int i = 0; i < g->nax; i++)
    pb_str_printf(t, "//%saxis%d %c %lld %lld %lld %lld %lld\n", pre, i, g->ax[i].kind, g->ax[i].ext, g->ax[i].s[0], g->ax[i].s[1],
                  g->ax[i].s[2], g->ax[i].s[3]);
  pb_str_printf(t, "//%snaxes %d\n", pre, g->nax);
  if (g->abf16) pb_str_printf(t, "//%sabf16 1\n", pre);
  if (g->cbf16) pb_str_printf(t, "//%scbf16 1\n", pre);
  if (g->gelu) pb_str_printf(t, "//%sgelu 1\n", pre);
  if (g->has_alpha) pb_str_printf(t, "//%salpha %lld\n", pre, g->alpha);
}

static char *gemm_text(const HGemm *g) {
  PbStr t; pb_str_init(&t);
  pb_str_puts(&t, "//PB200 1\n//kind gemm\n");
  hgemm_emit(&t, "", g);
  return pb_str_take(&t);
}

static bool hattn_parse(const char *text, HAttn *a) {
  char buf[128];
  memset(a, 0, sizeof *a);
  if (!pb_hdr_line(text, "kind", buf, sizeof buf) || strcmp(buf, "attn") != 0) return false;
  if (!pb_hdr_line(text, "scale", buf, sizeof buf)) return false;
  snprintf(a->scale, sizeof a->scale, "%.15s", buf);
  if (!pb_hdr_line(text, "mask", buf, sizeof buf) || sscanf(buf, "%lld %lld %lld", &a->mask[0], &a->mask[1], &a->mask[2]) != 3) return false;
  if (!pb_hdr_line(text, "outmode", buf, sizeof buf)) return false;
  a->outmode = buf[0];
  a->qkv16 = pb_hdr_line(text, "qkv16", buf, sizeof buf) ? atoi(buf) : 0;
  a->obf16 = pb_hdr_line(text, "obf16", buf, sizeof buf) ? atoi(buf) : 0;
  a->tiles = pb_hdr_line(text, "tiles", buf, sizeof buf) ? atoi(buf) : 0;
  return hgemm_parse(text, "g1.", &a->g1) && hgemm_parse(text, "g2.", &a->g2);
}

static char *attn_text(const HAttn *a) {
  PbStr t; pb_str_init(&t);
  pb_str_printf(&t, "//PB200 1\n//kind attn\n//scale %s\n//mask %lld %lld %lld\n//outmode %c\n", a->scale, a->mask[0], a->mask[1], a->mask[2], a->outmode);
  if (a->qkv16) pb_str_puts(&t, "//qkv16 1\n");
  if (a->obf16) pb_str_puts(&t, "//obf16 1\n");
  if (a->tiles) pb_str_printf(&t, "//tiles %d\n", a->tiles);
  hgemm_emit(&t, "g1.", &a->g1);
  hgemm_emit(&t, "g2.", &a->g2);
  return pb_str_take(&t);
}

typedef enum { K_OTHER, K_GEMM, K_ATTN } StepKind;
static StepKind step_kind(const PbStep *st) {
  char buf[32];
  if (st->dead || !st->precompiled || !st->text || !pb_hdr_line(st->text, "kind", buf, sizeof buf)) return K_OTHER;
  if (strcmp(buf, "gemm") == 0) return K_GEMM;
  if (strcmp(buf, "attn") == 0) return K_ATTN;
  return K_OTHER;
}

static void step_set_program(PbStep *st, PolyCudaProgram *prog, char *text) {
  poly_cuda_program_destroy(st->prog); free(st->text);
  st->prog = prog; st->text = text;
}

static PolyCudaProgram *compile_step_text(const PbStep *st, const char *text, const char *what) {
  char name[64]; snprintf(name, sizeof name, "%s_k%d", what, st->item);
  if (getenv("POLY_DUMP_KERNELS")) fprintf(stderr, "=== CUDA KERNEL %s ===\n%s\n=== END ===\n", name, text);
  return poly_compile_cuda(text, name);
}

/* The operands a precompiled step reads, by the step's parameter position:
 * which header (0: the gemm's / attention's g1, 1: g2) and which operand. */
typedef struct { int param, which, op; } OperandUse;
static int step_operand_uses(StepKind kind, const HGemm *g, OperandUse *out) {
  int n = 0;
  if (kind == K_GEMM) {
    out[n++] = (OperandUse){g->params[OP_A], 0, OP_A};
    out[n++] = (OperandUse){g->params[OP_B], 0, OP_B};
    if (g->params[OP_X] >= 0) out[n++] = (OperandUse){g->params[OP_X], 0, OP_X};
  } else if (kind == K_ATTN) {
    out[n++] = (OperandUse){0, 0, OP_A};     /* q */
    out[n++] = (OperandUse){1, 0, OP_B};     /* k */
    out[n++] = (OperandUse){2, 1, OP_B};     /* v */
  }
  return n;
}

/* ── composing an index map into an operand's strides ────────────────── */
/* A bijection-free description of "element e of buffer Y is element g(e) of
 * buffer X": Y's elements enumerated in mixed radix (ext[0] fastest), each digit
 * with a stride in X. */
typedef struct { int n; long long ext[PB_MAX_RANGES], sx[PB_MAX_RANGES], off, numel; } IndexMap;

static long long map_apply(const IndexMap *m, long long e) {
  long long r = m->off;
  for (int i = 0; i < m->n; i++) { r += (e % m->ext[i]) * m->sx[i]; e /= m->ext[i]; }
  return r;
}

static unsigned long long rng_next(unsigned long long *s) { *s = *s * 6364136223846793005ULL + 1442695040888963407ULL; return *s >> 17; }

/* Rewrites operand `op` of g (offset and strides) so that it addresses X instead
 * of Y.  False when the operand's accesses do not map affinely. */
static bool compose_operand(HGemm *g, int op, const IndexMap *m) {
  long long hi = g->off[op];
  for (int i = 0; i < g->nax; i++) {
    if (g->ax[i].ext < 1 || g->ax[i].s[op] < 0) return false;
    hi += (g->ax[i].ext - 1) * g->ax[i].s[op];
  }
  if (g->off[op] < 0 || hi >= m->numel) return false;
  const long long base = map_apply(m, g->off[op]);
  long long ns[16];
  for (int i = 0; i < g->nax; i++)
    ns[i] = (g->ax[i].ext > 1 && g->ax[i].s[op] != 0) ? map_apply(m, g->off[op] + g->ax[i].s[op]) - base : 0;
  unsigned long long seed = 0x9E3779B97F4A7C15ULL;
  for (int trial = 0; trial < 4096 + 2 * g->nax + 1; trial++) {
    long long e = g->off[op], want = base;
    for (int i = 0; i < g->nax; i++) {
      long long x;
      if (trial < g->nax) x = (i == trial) ? g->ax[i].ext - 1 : 0;                 /* each axis end */
      else if (trial < 2 * g->nax) x = (i == trial - g->nax) ? 0 : g->ax[i].ext - 1; /* all ends but one */
      else if (trial == 2 * g->nax) x = g->ax[i].ext - 1;                           /* far corner */
      else x = (long long)(rng_next(&seed) % (unsigned long long)g->ax[i].ext);
      e += x * g->ax[i].s[op]; want += x * ns[i];
    }
    if (map_apply(m, e) != want) return false;
  }
  g->off[op] = base;
  for (int i = 0; i < g->nax; i++) g->ax[i].s[op] = ns[i];
  return true;
}

/* Is this step a pure copy out[o(r)] = in[i(r)] that overwrites all of `out`?
 * Fills the map from out's element index to in's. */
static bool copy_index_map(const PbPlan *p, const PbStep *st, int *p_out, int *p_in, IndexMap *m) {
  if (st->dead || st->precompiled || st->fused_rows || !st->sink || st->n_vars || st->n_params != 2) return false;
  PbKern k;
  if (pb_kern_build(&k, st->sink) != 0) { pb_kern_free(&k); return false; }
  bool ok = false;
  do {
    if (k.n_stores != 1 || k.n_reduce_nodes != 0 || k.n_ranges > PB_MAX_RANGES) break;
    PbStore *s = &k.stores[0];
    PolyUOp *v = s->value;
    if (s->index->n_src != 2 || v->op != POLY_OP_LOAD || v->src[0]->op != POLY_OP_INDEX || v->src[0]->n_src != 2 ||
        v->src[0]->src[0]->op != POLY_OP_PARAM) break;
    const int po = s->param, pi = (int)v->src[0]->src[0]->arg.i;
    if (po == pi || po > 1 || pi > 1 || st->rw[po] != 'W') break;
    PolyDType a = k.params[po]->dtype, b = k.params[pi]->dtype;
    if (a.priority != 13 || b.priority != 13 || a.bitsize != 32 || b.bitsize != 32) break;
    uint64_t all = 0;
    for (int q = 0; q < k.n_ranges; q++) { if (k.extent[q] < 1) all = ~(uint64_t)0; all |= (uint64_t)1 << q; }
    if (all == ~(uint64_t)0) break;
    PbAffine so, si;
    pb_fit_affine(&k, s->index->src[1], all, &so);
    pb_fit_affine(&k, v->src[0]->src[1], all, &si);
    if (!so.ok || !si.ok || so.offset != 0) break;
    /* out must be dense: ranges sorted by their out stride tile [0, numel) */
    int idx[PB_MAX_RANGES]; int n = 0;
    for (int q = 0; q < k.n_ranges; q++) if (k.extent[q] > 1) idx[n++] = q;
    for (int i = 1; i < n; i++) for (int j = i; j > 0 && so.stride[idx[j]] < so.stride[idx[j - 1]]; j--) { int t = idx[j]; idx[j] = idx[j - 1]; idx[j - 1] = t; }
    long long expect = 1; bool dense = true;
    for (int i = 0; i < n; i++) { if (so.stride[idx[i]] != expect) { dense = false; break; } expect *= k.extent[idx[i]]; }
    if (!dense || expect != a.ptr_size) break;
    m->n = n; m->off = si.offset; m->numel = expect;
    for (int i = 0; i < n; i++) { m->ext[i] = k.extent[idx[i]]; m->sx[i] = si.stride[idx[i]]; }
    /* the source range must lie inside the source buffer */
    long long lo = si.offset, hi = si.offset;
    for (int i = 0; i < n; i++) { long long d = (m->ext[i] - 1) * m->sx[i]; if (d > 0) hi += d; else lo += d; }
    if (lo < 0 || hi >= b.ptr_size) break;
    *p_out = po; *p_in = pi;
    ok = true;
  } while (0);
  pb_kern_free(&k);
  (void)p;
  return ok;
}

static int fold_views(PbPlan *p) {
  int folded = 0;
  PbSlotUse *u = malloc(sizeof(PbSlotUse) * (size_t)p->n_slots);
  for (int c = 0; c < p->n_steps; c++) {
    PbStep *C = &p->steps[c];
    int po, pi; IndexMap m;
    if (!copy_index_map(p, C, &po, &pi, &m)) continue;
    pb_slot_usage(p, u);
    const int y = pb_plan_resolve(p, C->slot[po]), x = pb_plan_resolve(p, C->slot[pi]);
    if (x == y || !p->slot_inter[y] || u[y].writers != 1 || u[y].readers < 1) continue;
    /* every reader: a precompiled step after the copy that reads y only through stride-described operands,
     * with x unchanged in between */
    enum { MAXR = 8 };
    int readers[MAXR]; char *rtext[MAXR] = {0}; int nr = 0; bool ok = true;
    for (int s = 0; s < p->n_steps && ok; s++) {
      PbStep *R = &p->steps[s];
      if (R->dead || s == c || !pb_step_reads(p, R, y)) continue;
      StepKind kind = step_kind(R);
      if (s < c || kind == K_OTHER || nr >= MAXR) { ok = false; break; }
      for (int w = c + 1; w <= s && ok; w++) if (!p->steps[w].dead && pb_step_writes(p, &p->steps[w], x)) ok = false;
      if (!ok) break;
      HGemm g; HAttn a; HGemm *hdr[2];
      if (kind == K_GEMM) { if (!hgemm_parse(R->text, "", &g)) { ok = false; break; } hdr[0] = &g; hdr[1] = NULL; }
      else { if (!hattn_parse(R->text, &a)) { ok = false; break; } hdr[0] = &a.g1; hdr[1] = &a.g2; }
      if ((kind == K_GEMM && (g.abf16 || strcmp(g.dtype, "f32") != 0)) || (kind == K_ATTN && a.qkv16)) { ok = false; break; }
      OperandUse uses[4]; int nu = step_operand_uses(kind, hdr[0], uses);
      bool covered[PB_MAX_PARAMS] = {0};
      for (int i = 0; i < nu && ok; i++) {
        if (pb_plan_resolve(p, R->slot[uses[i].param]) != y) continue;
        HGemm *h = hdr[uses[i].which];
        if (!compose_operand(h, uses[i].op, &m)) { ok = false; break; }
        h->numel[uses[i].op] = p->slot_bytes[x] / 4;
        covered[uses[i].param] = true;
      }
      for (int q = 0; q < R->n_params && ok; q++)
        if (pb_plan_resolve(p, R->slot[q]) == y && !covered[q]) ok = false;       /* read some other way (mask, addend of attention ...) */
      if (!ok) break;
      readers[nr] = s;
      rtext[nr++] = kind == K_GEMM ? gemm_text(&g) : attn_text(&a);
    }
    PolyCudaProgram *rprog[MAXR] = {0};
    for (int i = 0; i < nr && ok; i++) {
      rprog[i] = compile_step_text(&p->steps[readers[i]], rtext[i], "folded");
      if (!rprog[i]) ok = false;
    }
    if (!ok || nr == 0) {
      for (int i = 0; i < nr; i++) { if (rprog[i]) poly_cuda_program_destroy(rprog[i]); free(rtext[i]); }
      continue;
    }
    for (int i = 0; i < nr; i++) {
      PbStep *R = &p->steps[readers[i]];
      step_set_program(R, rprog[i], rtext[i]);
      for (int q = 0; q < R->n_params; q++) if (pb_plan_resolve(p, R->slot[q]) == y) R->slot[q] = x;
    }
    C->dead = true;
    folded++;
  }
  free(u);
  return folded;
}

/* ── bfloat16 storage ────────────────────────────────────────────────── */
#define RETYPE_MAX_READERS 4
static int retype_bf16(PbPlan *p) {
  int done = 0;
  PbSlotUse *u = malloc(sizeof(PbSlotUse) * (size_t)p->n_slots);
  for (int x = 0; x < p->n_slots; x++) {
    if (pb_plan_resolve(p, x) != x || !p->slot_inter[x]) continue;
    pb_slot_usage(p, u);
    if (u[x].writers != 1 || u[x].readers < 1) continue;
    const int w = u[x].first_write;
    PbStep *W = &p->steps[w];
    if (W->dead || W->n_vars) continue;
    const StepKind wkind = step_kind(W);
    if (W->precompiled ? wkind != K_GEMM : !W->sink) continue;
    bool whole = false;
    for (int a = 0; a < W->n_params; a++) if (pb_plan_resolve(p, W->slot[a]) == x) whole = W->rw[a] == 'W';
    if (!whole) continue;

    /* readers: contractions taking the slot as A only, attention taking it as q, k and v */
    int readers[RETYPE_MAX_READERS]; char *rtext[RETYPE_MAX_READERS] = {0}; int nr = 0; bool ok = true;
    for (int s = 0; s < p->n_steps && ok; s++) {
      PbStep *R = &p->steps[s];
      if (R->dead || !pb_step_reads(p, R, x)) continue;
      const StepKind kind = step_kind(R);
      if (s <= w || kind == K_OTHER || nr >= RETYPE_MAX_READERS) { ok = false; break; }
      if (kind == K_GEMM) {
        HGemm g;
        if (!hgemm_parse(R->text, "", &g) || strcmp(g.dtype, "f32") != 0 || g.abf16 || g.has_alpha) { ok = false; break; }
        for (int a = 0; a < R->n_params; a++) if (pb_plan_resolve(p, R->slot[a]) == x && a != g.params[OP_A]) ok = false;
        g.abf16 = 1;
        if (ok) rtext[nr] = gemm_text(&g);
      } else {
        HAttn a;
        if (!hattn_parse(R->text, &a) || a.qkv16) { ok = false; break; }
        for (int q = 0; q < R->n_params; q++) if ((pb_plan_resolve(p, R->slot[q]) == x) != (q < 3)) ok = false;
        a.qkv16 = 1;
        if (ok) rtext[nr] = attn_text(&a);
      }
      if (ok) readers[nr++] = s;
    }
    if (!ok || nr == 0) { for (int i = 0; i < nr; i++) free(rtext[i]); continue; }

    /* the producer with a bfloat16 store */
    char *wtext = NULL;
    if (wkind == K_GEMM) {
      HGemm g;
      if (hgemm_parse(W->text, "", &g) && strcmp(g.dtype, "f32") == 0 && !g.cbf16 && !g.has_alpha &&
          pb_plan_resolve(p, W->slot[g.params[OP_C]]) == x && g.params[OP_X] != g.params[OP_C]) { g.cbf16 = 1; wtext = gemm_text(&g); }
    } else if (W->fused_rows) {
      PbFuseOut fo;
      wtext = pb_render_chain(p, W->chain, W->chain_keep, W->n_chain, true, &fo);
      if (wtext) {
        bool same = fo.n_params == W->n_params;
        for (int a = 0; same && a < fo.n_params; a++) if (fo.slot[a] != pb_plan_resolve(p, W->slot[a]) || fo.rw[a] != W->rw[a]) same = false;
        if (!same) { free(wtext); wtext = NULL; }
      }
    } else {
      PbKern k;
      if (pb_kern_build(&k, W->sink) == 0 && k.n_stores == 1 && pb_plan_resolve(p, W->slot[k.stores[0].param]) == x)
        wtext = pb_render_elementwise_bf16(&k);
      pb_kern_free(&k);
    }
    PolyCudaProgram *wprog = wtext ? compile_step_text(W, wtext, "bf16out") : NULL;
    PolyCudaProgram *rprog[RETYPE_MAX_READERS] = {0};
    bool all = wprog != NULL;
    for (int i = 0; i < nr && all; i++) {
      rprog[i] = compile_step_text(&p->steps[readers[i]], rtext[i], "bf16in");
      if (!rprog[i]) all = false;
    }
    if (!all) {
      if (wprog) poly_cuda_program_destroy(wprog);
      free(wtext);
      for (int i = 0; i < nr; i++) { if (rprog[i]) poly_cuda_program_destroy(rprog[i]); free(rtext[i]); }
      continue;
    }
    step_set_program(W, wprog, wtext);
    for (int i = 0; i < nr; i++) step_set_program(&p->steps[readers[i]], rprog[i], rtext[i]);
    done++;
  }
  free(u);
  return done;
}

/* ── GELU into the producing contraction's epilogue ──────────────────── */
/* polygrad's GPT-2 MLP is fc contraction (+bias) -> GELU -> projection (reference
 * src/modelzoo/models/gpt2.c:478-490); the GELU is a kernel of its own that reads the
 * 8192 x 3072 float32 result and, under the bf16 policy, stores bfloat16 for the
 * projection.  When that kernel is the only reader of the contraction's result it moves
 * into the contraction's epilogue: bias, GELU, round to bfloat16, store.
 *
 * The elementwise kernel is recognised by what it computes, not by the shape of its op
 * tree: its scalar function is evaluated on the host in double precision at sample
 * points and compared with 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
 * (poly_gelu, reference src/frontend.c:603-614).  The epilogue evaluates the same formula
 * with the hardware tanh approximation (relative error about 2^-11, below the bfloat16
 * rounding that follows), so the result is not bit-identical to the separate kernel's:
 * the pass runs only under the bf16 policy, whose bound is 2e-2, and POLY_B200_EPILOGUE=0
 * switches it off. */
#include <math.h>

static bool eval_scalar(const PbKern *k, PolyUOp *u, PolyUOp *x_load, double x, double *out, int depth) {
  if (depth > 64) return false;
  if (u == x_load) { *out = x; return true; }
  double a = 0, b = 0, c = 0;
  switch (u->op) {
  case POLY_OP_CONST:
    if (u->arg.kind == POLY_ARG_FLOAT) *out = (double)(float)u->arg.f;
    else if (u->arg.kind == POLY_ARG_INT) *out = (double)u->arg.i;
    else if (u->arg.kind == POLY_ARG_BOOL) *out = u->arg.b ? 1.0 : 0.0;
    else return false;
    return true;
  case POLY_OP_CAST:
    if (u->n_src != 1 || u->dtype.priority != 13) return false;
    return eval_scalar(k, u->src[0], x_load, x, out, depth + 1);
  case POLY_OP_NEG: case POLY_OP_EXP2: case POLY_OP_LOG2: case POLY_OP_SQRT: case POLY_OP_RECIPROCAL:
    if (u->n_src != 1 || !eval_scalar(k, u->src[0], x_load, x, &a, depth + 1)) return false;
    *out = u->op == POLY_OP_NEG ? -a : u->op == POLY_OP_EXP2 ? exp2(a) : u->op == POLY_OP_LOG2 ? log2(a) :
           u->op == POLY_OP_SQRT ? sqrt(a) : 1.0 / a;
    return true;
  case POLY_OP_ADD: case POLY_OP_SUB: case POLY_OP_MUL: case POLY_OP_FDIV: case POLY_OP_MAX:
  case POLY_OP_CMPLT: case POLY_OP_CMPNE: case POLY_OP_CMPEQ:
    if (u->n_src != 2 || !eval_scalar(k, u->src[0], x_load, x, &a, depth + 1) ||
        !eval_scalar(k, u->src[1], x_load, x, &b, depth + 1)) return false;
    switch (u->op) {
    case POLY_OP_ADD: *out = a + b; break;
    case POLY_OP_SUB: *out = a - b; break;
    case POLY_OP_MUL: *out = a * b; break;
    case POLY_OP_FDIV: *out = a / b; break;
    case POLY_OP_MAX: *out = a > b ? a : b; break;
    case POLY_OP_CMPLT: *out = a < b; break;
    case POLY_OP_CMPNE: *out = a != b; break;
    default: *out = a == b; break;
    }
    return true;
  case POLY_OP_WHERE:
    if (u->n_src != 3 || !eval_scalar(k, u->src[0], x_load, x, &a, depth + 1) ||
        !eval_scalar(k, u->src[1], x_load, x, &b, depth + 1) || !eval_scalar(k, u->src[2], x_load, x, &c, depth + 1)) return false;
    *out = a != 0.0 ? b : c;
    return true;
  case POLY_OP_MULACC:
    if (u->n_src != 3 || !eval_scalar(k, u->src[0], x_load, x, &a, depth + 1) ||
        !eval_scalar(k, u->src[1], x_load, x, &b, depth + 1) || !eval_scalar(k, u->src[2], x_load, x, &c, depth + 1)) return false;
    *out = a * b + c;
    return true;
  default:
    return false;      /* loads of other buffers, ranges, integer arithmetic: not a function of x alone */
  }
}

/* Is the step out[i] = gelu(in[i]) over two buffers of the same element layout? */
static bool step_is_gelu(const PbStep *st, int *p_out, int *p_in) {
  if (st->dead || st->precompiled || st->fused_rows || !st->sink || st->n_vars || st->n_params != 2) return false;
  PbKern k;
  if (pb_kern_build(&k, st->sink) != 0) { pb_kern_free(&k); return false; }
  bool ok = false;
  do {
    if (k.n_stores != 1 || k.n_reduce_nodes != 0 || k.n_ranges > PB_MAX_RANGES) break;
    PbStore *s = &k.stores[0];
    if (s->index->n_src != 2) break;
    const int po = s->param, pi = 1 - po;
    if (po < 0 || po > 1 || st->rw[po] != 'W' || st->rw[pi] != 'r') break;
    PolyDType a = k.params[po]->dtype, b = k.params[pi]->dtype;
    if (a.priority != 13 || b.priority != 13 || a.bitsize != 32 || b.bitsize != 32 || a.ptr_size != b.ptr_size) break;
    /* the one load: every LOAD node in the tree must be the same INDEX(PARAM pi, idx) as the store's index expression */
    PolyUOp *x_load = NULL; bool one = true;
    for (int n = 0; n < k.n_nodes && one; n++) {
      PolyUOp *u = k.nodes[n].u;
      if (u->op != POLY_OP_LOAD) continue;
      if (u->src[0]->op != POLY_OP_INDEX || u->src[0]->n_src != 2 || u->src[0]->src[0]->op != POLY_OP_PARAM ||
          (int)u->src[0]->src[0]->arg.i != pi || (x_load && x_load != u)) one = false;
      else x_load = u;
    }
    if (!one || !x_load) break;
    uint64_t all = 0;
    for (int q = 0; q < k.n_ranges; q++) { if (k.extent[q] < 1) all = ~(uint64_t)0; all |= (uint64_t)1 << q; }
    if (all == ~(uint64_t)0) break;
    PbAffine so, si;
    pb_fit_affine(&k, s->index->src[1], all, &so);
    pb_fit_affine(&k, x_load->src[0]->src[1], all, &si);
    if (!so.ok || !si.ok || so.offset != 0 || si.offset != 0) break;
    bool same = true; long long covered = 1;
    for (int q = 0; q < k.n_ranges; q++) { if (so.stride[q] != si.stride[q]) same = false; covered *= k.extent[q]; }
    if (!same || covered != a.ptr_size) break;
    /* the function itself */
    static const double xs[] = {-9.0, -6.5, -4.0, -3.0, -2.25, -1.5, -1.0, -0.75, -0.5, -0.25, -0.1, -1e-3, 0.0, 1e-3, 0.1,
                                0.25, 0.5, 0.75, 1.0, 1.5, 2.25, 3.0, 4.0, 6.5, 9.0, 0.3333, -0.6667, 1.2345, -2.718, 5.5};
    bool match = true;
    for (size_t i = 0; i < sizeof xs / sizeof xs[0] && match; i++) {
      double y = 0;
      if (!eval_scalar(&k, s->value, x_load, xs[i], &y, 0)) { match = false; break; }
      const double x = xs[i], want = 0.5 * x * (1.0 + tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)));
      if (!(fabs(y - want) <= 2e-6 * (1.0 + fabs(want)))) match = false;
    }
    if (!match) break;
    *p_out = po; *p_in = pi;
    ok = true;
  } while (0);
  pb_kern_free(&k);
  return ok;
}

static int fuse_gelu_epilogue(PbPlan *p) {
  int done = 0;
  PbSlotUse *u = malloc(sizeof(PbSlotUse) * (size_t)p->n_slots);
  for (int e = 0; e < p->n_steps; e++) {
    PbStep *E = &p->steps[e];
    int po, pi;
    if (!step_is_gelu(E, &po, &pi)) continue;
    pb_slot_usage(p, u);
    const int y = pb_plan_resolve(p, E->slot[po]), x = pb_plan_resolve(p, E->slot[pi]);
    if (x == y || !p->slot_inter[x] || !p->slot_inter[y] || u[x].writers != 1 || u[x].readers != 1 || u[y].writers != 1) continue;
    /* y is stored as bfloat16: every reader is a contraction that takes it as a bfloat16 A operand */
    bool y16 = u[y].readers >= 1;
    for (int s = 0; s < p->n_steps && y16; s++) {
      PbStep *R = &p->steps[s];
      if (R->dead || s == e || !pb_step_reads(p, R, y)) continue;
      HGemm g;
      if (s < e || step_kind(R) != K_GEMM || !hgemm_parse(R->text, "", &g) || !g.abf16 ||
          pb_plan_resolve(p, R->slot[g.params[OP_A]]) != y) y16 = false;
    }
    if (!y16) continue;
    /* the producer: a plain contraction writing all of x */
    const int w = u[x].first_write;
    PbStep *W = &p->steps[w];
    HGemm g;
    if (w >= e || step_kind(W) != K_GEMM || !hgemm_parse(W->text, "", &g) || strcmp(g.dtype, "f32") != 0 || g.cbf16 || g.gelu ||
        g.relu || g.has_alpha || pb_plan_resolve(p, W->slot[g.params[OP_C]]) != x || g.params[OP_X] == g.params[OP_C] ||
        W->rw[g.params[OP_C]] != 'W') continue;
    /* nothing between the two steps may touch y (it becomes the contraction's output) */
    bool clear = true;
    for (int s = w; s < e && clear; s++)
      if (!p->steps[s].dead && (pb_step_reads(p, &p->steps[s], y) || pb_step_writes(p, &p->steps[s], y))) clear = false;
    if (!clear) continue;
    g.cbf16 = 1; g.gelu = 1;
    char *text = gemm_text(&g);
    PolyCudaProgram *prog = compile_step_text(W, text, "gelu_epilogue");
    if (!prog) { free(text); continue; }
    step_set_program(W, prog, text);
    W->slot[g.params[OP_C]] = y;
    E->dead = true;
    done++;
  }
  free(u);
  return done;
}

/* ── attention output in the layout the next projection reads ────────── */
/* out is [batch.., row, d] through strides; its only reader is a contraction
 * whose A operand walks it as rows x k with k split over (head, d), which is not
 * a matrix with one row pitch.  Both sides are rewritten to a dense row-major
 * bfloat16 [rows][k] matrix in the same buffer. */
static int relayout_attention_out(PbPlan *p) {
  int done = 0;
  PbSlotUse *u = malloc(sizeof(PbSlotUse) * (size_t)p->n_slots);
  for (int w = 0; w < p->n_steps; w++) {
    PbStep *W = &p->steps[w];
    if (step_kind(W) != K_ATTN) continue;
    HAttn a;
    if (!hattn_parse(W->text, &a) || a.obf16 || a.outmode != 'W') continue;
    pb_slot_usage(p, u);
    const int o = pb_plan_resolve(p, W->slot[4]);
    if (!p->slot_inter[o] || u[o].writers != 1 || u[o].readers != 1) continue;
    const int r = u[o].last_read;
    PbStep *R = &p->steps[r];
    HGemm g;
    if (r <= w || step_kind(R) != K_GEMM || !hgemm_parse(R->text, "", &g) || strcmp(g.dtype, "f32") != 0 || g.abf16) continue;
    bool only_a = true;
    for (int q = 0; q < R->n_params; q++) if (pb_plan_resolve(p, R->slot[q]) == o && q != g.params[OP_A]) only_a = false;
    if (!only_a || g.off[OP_A] != 0) continue;
    /* the consumer's A axes, k innermost (by old stride), then m; batch axes of the consumer are not handled */
    int order[16]; int n = 0; long long K = 1, M = 1; bool okx = true;
    for (int pass = 0; pass < 2; pass++) {
      const char want = pass == 0 ? 'k' : 'm';
      int first = n;
      for (int i = 0; i < g.nax; i++) if (g.ax[i].kind == want && g.ax[i].ext > 1) order[n++] = i;
      for (int i = first + 1; i < n; i++) for (int j = i; j > first && g.ax[order[j]].s[OP_A] < g.ax[order[j - 1]].s[OP_A]; j--) { int t = order[j]; order[j] = order[j - 1]; order[j - 1] = t; }
      for (int i = first; i < n; i++) { if (pass == 0) K *= g.ax[order[i]].ext; else M *= g.ax[order[i]].ext; }
    }
    for (int i = 0; i < g.nax; i++) if (g.ax[i].kind == 'b' && g.ax[i].ext > 1) okx = false;
    if (!okx || M * K != a.g2.numel[OP_C] || K % 8) continue;
    /* phi: old element offset -> new element offset.  The consumer's A walk is a bijection onto
     * [0, M*K) iff its strides, sorted, tile the buffer. */
    IndexMap phi; phi.n = 0; phi.off = 0; phi.numel = M * K;
    {
      int byold[16]; int nb = 0;
      for (int i = 0; i < n; i++) byold[nb++] = order[i];
      for (int i = 1; i < nb; i++) for (int j = i; j > 0 && g.ax[byold[j]].s[OP_A] < g.ax[byold[j - 1]].s[OP_A]; j--) { int t = byold[j]; byold[j] = byold[j - 1]; byold[j - 1] = t; }
      long long expect = 1;
      for (int i = 0; i < nb; i++) { if (g.ax[byold[i]].s[OP_A] != expect) okx = false; expect *= g.ax[byold[i]].ext; }
      if (!okx || expect != M * K) continue;
      /* new stride of each consumer axis: position in (k axes, then m axes) */
      long long ns[16] = {0}, wgt = 1;
      for (int i = 0; i < n; i++) { ns[order[i]] = wgt; wgt *= g.ax[order[i]].ext; }
      for (int i = 0; i < nb; i++) { phi.ext[phi.n] = g.ax[byold[i]].ext; phi.sx[phi.n++] = ns[byold[i]]; }
      for (int i = 0; i < g.nax; i++) g.ax[i].s[OP_A] = (g.ax[i].ext > 1 && (g.ax[i].kind == 'k' || g.ax[i].kind == 'm')) ? ns[i] : 0;
    }
    /* the attention's output strides through phi */
    if (!compose_operand(&a.g2, OP_C, &phi)) continue;
    a.obf16 = 1; g.abf16 = 1;
    char *wt = attn_text(&a), *rt = gemm_text(&g);
    PolyCudaProgram *wp = compile_step_text(W, wt, "attn_bf16out");
    PolyCudaProgram *rp = wp ? compile_step_text(R, rt, "bf16in") : NULL;
    if (!wp || !rp) { if (wp) poly_cuda_program_destroy(wp); free(wt); free(rt); continue; }
    step_set_program(W, wp, wt);
    step_set_program(R, rp, rt);
    done++;
  }
  free(u);
  return done;
}


/* ── one mask classification per mask ────────────────────────────────── */
/* Every attention step classifies its mask by tile before it runs.  Steps that
 * read the same mask buffer in the same way, with no write to it in between,
 * share one classification: the first computes it into a small plan buffer, the
 * others read that. */
static int share_mask_tiles(PbPlan *p) {
  int shared = 0;
  for (int f = 0; f < p->n_steps; f++) {
    PbStep *F = &p->steps[f];
    HAttn fa;
    if (step_kind(F) != K_ATTN || F->n_params != 5 || !hattn_parse(F->text, &fa) || fa.tiles) continue;
    const int mslot = pb_plan_resolve(p, F->slot[3]);
    long long T = 0;
    for (int i = 0; i < fa.g1.nax; i++) if (fa.g1.ax[i].kind == 'm') T = fa.g1.ax[i].ext;
    if (T < 128) continue;
    int members[64]; int nm = 0;
    for (int s = f + 1; s < p->n_steps && nm < 64; s++) {
      PbStep *S = &p->steps[s];
      if (S->dead) continue;
      if (pb_step_writes(p, S, mslot)) break;
      HAttn a;
      if (step_kind(S) != K_ATTN || S->n_params != 5 || !hattn_parse(S->text, &a) || a.tiles) continue;
      long long Ts = 0;
      for (int i = 0; i < a.g1.nax; i++) if (a.g1.ax[i].kind == 'm') Ts = a.g1.ax[i].ext;
      if (pb_plan_resolve(p, S->slot[3]) == mslot && Ts == T && memcmp(a.mask, fa.mask, sizeof a.mask) == 0) members[nm++] = s;
    }
    if (nm == 0) continue;
    /* one record of eight floats per 128 x 128 tile of the mask */
    const int tslot = pb_plan_add_slot(p, 8 * (T / 128) * (T / 128) * (int64_t)sizeof(float));
    int ok_members = 0;
    for (int i = -1; i < nm; i++) {
      PbStep *S = i < 0 ? F : &p->steps[members[i]];
      HAttn a;
      hattn_parse(S->text, &a);
      a.tiles = i < 0 ? 1 : 2;
      char *text = attn_text(&a);
      PolyCudaProgram *prog = compile_step_text(S, text, "attn_tiles");
      if (!prog) { free(text); if (i < 0) break; continue; }
      step_set_program(S, prog, text);
      S->slot[5] = tslot; S->rw[5] = i < 0 ? 'W' : 'r'; S->rw[6] = 0; S->n_params = 6;
      if (i >= 0) ok_members++;
    }
    shared += ok_members;
  }
  return shared;
}

void pb_plan_operands(PbPlan *p) {
  const char *e = getenv("POLY_B200_OPERANDS");     /* "0": none, "fold": view folding only */
  if (e && strcmp(e, "0") == 0) return;
  int folded = fold_views(p), kept = 0, outs = 0, gelus = 0;
  if (poly_b200_gemm_policy() && !(e && strcmp(e, "fold") == 0)) {
    kept = retype_bf16(p);
    outs = relayout_attention_out(p);
    const char *ep = getenv("POLY_B200_EPILOGUE");
    if (!(ep && strcmp(ep, "0") == 0)) gelus = fuse_gelu_epilogue(p);
  }
  int tiles = (e && strcmp(e, "notiles") == 0) ? 0 : share_mask_tiles(p);
  if (getenv("POLY_B200_DEBUG"))
    fprintf(stderr, "pb_operands: %d copies folded into operand strides, %d operands stored as bfloat16, "
                    "%d attention outputs written as bfloat16 matrices, "
                    "%d attention steps reuse a mask classification, %d GELU kernels moved into contraction epilogues\n",
            folded, kept, outs, tiles, gelus);
}
