/*
 * pb_gather.cu -- embedding lookup.
 *
 * polygrad expresses  out[t, d] = table[ids[t], d]  as a one-hot contraction
 *   out[t, d] = sum_v  (ids[t] == arange[v]) ? table[v, d] : 0
 * over the whole table (reference: src/modelzoo/models/gpt2.c:93-153), where ids
 * and arange are float32 buffers.  The kernel keeps those semantics for any
 * buffer contents: one block per token searches `arange` for every v that
 * equals the token's id (none for NaN, out-of-range or fractional ids, which
 * therefore give a row of +0), then adds the matching rows in ascending v
 * starting from +0, exactly like the reference accumulation, so a -0.0f table
 * entry comes out as +0.0f there and here.
 *
 * A first small kernel checks whether `arange` is strictly increasing (true for
 * the 0..V-1 buffer the builders make; false for anything with NaNs or
 * duplicates).  If it is, an id matches at most one v, found by trying v = id
 * and otherwise by bisection, and the full search is skipped; if not, every
 * block searches all of `arange` as described above.  Either way the result is
 * the reference's.
 *
 * HBM traffic is the table rows read plus the output rows written.
 */
#include "../runtime/pb_runtime.h"
#include <cstdio>

struct GatherArgs {
  float *out; const float *ids; const float *arange; const float *table;
  long long vocab, table_vstride;
  long long out_off, ids_off, table_off;
  int ntok; long long tok_ext[4], tok_out[4], tok_ids[4];
  int nfeat; long long feat_ext[3], feat_out[3], feat_tab[3];
  long long n_tokens, n_feat;
  const int *sorted;              /* 1: arange is strictly increasing */
};

#define GATHER_THREADS 256
#define GATHER_MAX_MATCH 8

__global__ void __launch_bounds__(1024) pb200_gather_check_sorted(const float *arange, long long vocab, int *flag) {
  bool ok = true;
  for (long long v = threadIdx.x; v + 1 < vocab; v += 1024) ok = ok & (arange[v] < arange[v + 1]);
  if (vocab == 1) ok = arange[0] == arange[0];
  const int all = __syncthreads_and(ok ? 1 : 0);
  if (threadIdx.x == 0) *flag = all;
}

__global__ void __launch_bounds__(GATHER_THREADS) pb200_gather_rows(const GatherArgs a) {
  __shared__ int s_count;
  __shared__ long long s_match[GATHER_MAX_MATCH];
  for (long long tok = blockIdx.x; tok < a.n_tokens; tok += gridDim.x) {
    long long rem = tok, o_out = a.out_off, o_ids = a.ids_off;
    for (int i = 0; i < a.ntok; i++) {
      const long long x = rem % a.tok_ext[i]; rem /= a.tok_ext[i];
      o_out += x * a.tok_out[i]; o_ids += x * a.tok_ids[i];
    }
    if (threadIdx.x == 0) s_count = 0;
    __syncthreads();
    const float id = a.ids[o_ids];
    if (*a.sorted) {
      /* strictly increasing: at most one match */
      if (threadIdx.x == 0 && id == id) {
        long long v = -1;
        const long long guess = (id >= 0.0f && id < (float)a.vocab) ? (long long)id : -1;
        if (guess >= 0 && a.arange[guess] == id) v = guess;
        else {
          long long lo = 0, hi = a.vocab - 1;
          while (lo <= hi) {
            const long long mid = (lo + hi) >> 1;
            const float x = a.arange[mid];
            if (x == id) { v = mid; break; }
            if (x < id) lo = mid + 1; else hi = mid - 1;
          }
        }
        if (v >= 0) { s_match[0] = v; s_count = 1; }
      }
    } else {
      for (long long v = threadIdx.x; v < a.vocab; v += GATHER_THREADS) {
        if (a.arange[v] == id) {
          const int slot = atomicAdd(&s_count, 1);
          if (slot < GATHER_MAX_MATCH) s_match[slot] = v;
        }
      }
    }
    __syncthreads();
    const int count = s_count;
    if (count > 1 && count <= GATHER_MAX_MATCH && threadIdx.x == 0) {
      /* ascending v: the order the reference adds in */
      for (int i = 1; i < count; i++) {
        long long x = s_match[i]; int j = i - 1;
        while (j >= 0 && s_match[j] > x) { s_match[j + 1] = s_match[j]; j--; }
        s_match[j + 1] = x;
      }
    }
    __syncthreads();
    for (long long f = threadIdx.x; f < a.n_feat; f += GATHER_THREADS) {
      long long fr = f, o = o_out, t = a.table_off;
      for (int i = 0; i < a.nfeat; i++) {
        const long long x = fr % a.feat_ext[i]; fr /= a.feat_ext[i];
        o += x * a.feat_out[i]; t += x * a.feat_tab[i];
      }
      float acc = 0.0f;
      if (count <= GATHER_MAX_MATCH) {
        for (int i = 0; i < count; i++) acc = acc + a.table[t + s_match[i] * a.table_vstride];
      } else {
        /* pathological arange with many duplicates: plain ordered scan */
        for (long long v = 0; v < a.vocab; v++)
          if (a.arange[v] == id) acc = acc + a.table[t + v * a.table_vstride];
      }
      a.out[o] = acc;
    }
    __syncthreads();
  }
}

struct GatherProgram : PbAotProgram {
  GatherArgs a{};
  int n_launches() const override { return 2; }
  int p_out, p_ids, p_arange, p_table;
  int launch(void *const *bufs, cudaStream_t stream) override {
    GatherArgs g = a;
    g.out = (float *)bufs[p_out]; g.ids = (const float *)bufs[p_ids];
    g.arange = (const float *)bufs[p_arange]; g.table = (const float *)bufs[p_table];
    if (g.n_tokens <= 0 || g.n_feat <= 0) return 0;
    /* a block per token (the blocks are short: one search or bisection, one row copy) */
    long long grid = g.n_tokens < (1LL << 20) ? g.n_tokens : (1LL << 20);
    int *flag = (int *)pb_scratch_alloc(sizeof(int));
    if (!flag) { pb_set_error("gather: out of scratch memory"); return -1; }
    pb200_gather_check_sorted<<<1, 1024, 0, stream>>>(g.arange, g.vocab, flag);
    g.sorted = flag;
    pb200_gather_rows<<<(unsigned)grid, GATHER_THREADS, 0, stream>>>(g);
    pb_scratch_free(flag);            /* stream-ordered pool: safe once the work is enqueued */
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { pb_set_error("gather launch: %s", cudaGetErrorString(e)); return -1; }
    return 0;
  }
};

PbAotProgram *pb_make_gather(const PbHeader &h, std::string &err) {
  auto params = h.getv("params"), vocab = h.getv("vocab"), off = h.getv("offsets");
  auto tok = h.getv("tok"), feat = h.getv("feat");
  if (params.size() != 4 || vocab.size() != 2 || off.size() != 3 || tok.size() % 3 || feat.size() % 3 ||
      tok.size() > 12 || feat.size() > 9) { err = "malformed gather header"; return nullptr; }
  GatherProgram *p = new GatherProgram();
  p->n_params = (int)h.geti("nparams");
  p->p_out = (int)params[0]; p->p_ids = (int)params[1]; p->p_arange = (int)params[2]; p->p_table = (int)params[3];
  p->rw.assign((size_t)p->n_params, '-');
  for (int i = 1; i < 4; i++) p->rw[(size_t)params[i]] = 'r';
  p->rw[(size_t)params[0]] = 'w';
  GatherArgs &a = p->a;
  a.vocab = vocab[0]; a.table_vstride = vocab[1];
  a.out_off = off[0]; a.ids_off = off[1]; a.table_off = off[2];
  a.ntok = (int)tok.size() / 3; a.nfeat = (int)feat.size() / 3;
  a.n_tokens = 1; a.n_feat = 1;
  for (int i = 0; i < a.ntok; i++) { a.tok_ext[i] = tok[3 * i]; a.tok_out[i] = tok[3 * i + 1]; a.tok_ids[i] = tok[3 * i + 2]; a.n_tokens *= a.tok_ext[i]; }
  for (int i = 0; i < a.nfeat; i++) { a.feat_ext[i] = feat[3 * i]; a.feat_out[i] = feat[3 * i + 1]; a.feat_tab[i] = feat[3 * i + 2]; a.n_feat *= a.feat_ext[i]; }
  /* feature axes: smallest output stride first so that consecutive threads write consecutive floats */
  for (int i = 1; i < a.nfeat; i++)
    for (int j = i; j > 0 && llabs(a.feat_out[j]) < llabs(a.feat_out[j - 1]); j--) {
      std::swap(a.feat_ext[j], a.feat_ext[j - 1]); std::swap(a.feat_out[j], a.feat_out[j - 1]); std::swap(a.feat_tab[j], a.feat_tab[j - 1]);
    }
  return p;
}

/* ── the lookup's gradient ───────────────────────────────────────────── */
/* out[v, d] = sum_t (ids[t] == arange[v]) ? src[t, d] : 0 for every table row v (reference: the backward
 * of the one-hot lookup, which polygrad runs as a contraction over all tokens for every row).  A block
 * owns SCATTER_ROWS consecutive rows: its threads scan the tokens once, noting which token matches
 * which of the block's rows (any `arange` contents: NaNs match nothing, duplicates match several rows),
 * the few matches are put in token order, and every (row, d) element is the sum of its matching source
 * rows in that order, starting from +0 -- the order and the value of the reference's accumulation, in
 * which the non-matching tokens add +0.  Rows nobody refers to are written as +0.
 * HBM traffic: the output written once, the ids read once per block (from L2), the matching source rows. */
struct ScatterArgs {
  float *out; const float *ids; const float *arange; const float *src;
  long long vocab, out_vstride;
  long long out_off, ids_off, src_off;
  int ntok; long long tok_ext[4], tok_ids[4], tok_src[4];
  int nfeat; long long feat_ext[3], feat_out[3], feat_src[3];
  long long n_tokens, n_feat;
};

#define SCATTER_THREADS 256
#define SCATTER_ROWS 16
#define SCATTER_MAX_MATCH 1024

__global__ void __launch_bounds__(SCATTER_THREADS) pb200_scatter_rows(const ScatterArgs a) {
  __shared__ float s_ar[SCATTER_ROWS];
  __shared__ int s_count;
  __shared__ unsigned long long s_match[SCATTER_MAX_MATCH];      /* (row << 40) | token, sorted ascending */
  __shared__ int s_first[SCATTER_ROWS + 1];
  const long long v0 = (long long)blockIdx.x * SCATTER_ROWS;
  const int rows = (int)min((long long)SCATTER_ROWS, a.vocab - v0);
  if (threadIdx.x < SCATTER_ROWS) s_ar[threadIdx.x] = threadIdx.x < rows ? a.arange[v0 + threadIdx.x] : __int_as_float(0x7fc00000);
  if (threadIdx.x == 0) s_count = 0;
  __syncthreads();
  for (long long t = threadIdx.x; t < a.n_tokens; t += SCATTER_THREADS) {
    long long rem = t, o = a.ids_off;
    for (int i = 0; i < a.ntok; i++) { const long long x = rem % a.tok_ext[i]; rem /= a.tok_ext[i]; o += x * a.tok_ids[i]; }
    const float id = a.ids[o];
#pragma unroll
    for (int r = 0; r < SCATTER_ROWS; r++) {
      if (id == s_ar[r]) {
        const int slot = atomicAdd(&s_count, 1);
        if (slot < SCATTER_MAX_MATCH) s_match[slot] = ((unsigned long long)r << 40) | (unsigned long long)t;
      }
    }
  }
  __syncthreads();
  const int count = s_count;
  const bool listed = count <= SCATTER_MAX_MATCH;
  if (listed && threadIdx.x == 0) {
    /* by row, then by token: the order the reference adds in */
    for (int i = 1; i < count; i++) {
      const unsigned long long x = s_match[i]; int j = i - 1;
      while (j >= 0 && s_match[j] > x) { s_match[j + 1] = s_match[j]; j--; }
      s_match[j + 1] = x;
    }
    int at = 0;
    for (int r = 0; r <= SCATTER_ROWS; r++) {
      while (at < count && (int)(s_match[at] >> 40) < r) at++;
      s_first[r] = at;
    }
  }
  __syncthreads();
  const long long elems = (long long)rows * a.n_feat;
  for (long long e = threadIdx.x; e < elems; e += SCATTER_THREADS) {
    const int r = (int)(e / a.n_feat);
    long long fr = e % a.n_feat, o = a.out_off + (v0 + r) * a.out_vstride, s = a.src_off;
    for (int i = 0; i < a.nfeat; i++) { const long long x = fr % a.feat_ext[i]; fr /= a.feat_ext[i]; o += x * a.feat_out[i]; s += x * a.feat_src[i]; }
    float acc = 0.0f;
    if (listed) {
      for (int m = s_first[r]; m < s_first[r + 1]; m++) {
        long long rem = (long long)(s_match[m] & 0xffffffffffull), so = s;
        for (int i = 0; i < a.ntok; i++) { const long long x = rem % a.tok_ext[i]; rem /= a.tok_ext[i]; so += x * a.tok_src[i]; }
        acc = acc + a.src[so];
      }
    } else {
      /* more matches than the list holds (a batch of one repeated token): plain ordered scan */
      const float want = s_ar[r];
      for (long long t = 0; t < a.n_tokens; t++) {
        long long rem = t, oi = a.ids_off, so = s;
        for (int i = 0; i < a.ntok; i++) { const long long x = rem % a.tok_ext[i]; rem /= a.tok_ext[i]; oi += x * a.tok_ids[i]; so += x * a.tok_src[i]; }
        if (a.ids[oi] == want) acc = acc + a.src[so];
      }
    }
    a.out[o] = acc;
  }
}

struct ScatterProgram : PbAotProgram {
  ScatterArgs a{};
  int n_launches() const override { return 1; }
  int p_out, p_ids, p_arange, p_src;
  int launch(void *const *bufs, cudaStream_t stream) override {
    ScatterArgs g = a;
    g.out = (float *)bufs[p_out]; g.ids = (const float *)bufs[p_ids];
    g.arange = (const float *)bufs[p_arange]; g.src = (const float *)bufs[p_src];
    if (g.vocab <= 0 || g.n_feat <= 0) return 0;
    const long long grid = (g.vocab + SCATTER_ROWS - 1) / SCATTER_ROWS;
    if (grid > 2147483647LL) { pb_set_error("scatter: too many table rows"); return -1; }
    pb200_scatter_rows<<<(unsigned)grid, SCATTER_THREADS, 0, stream>>>(g);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { pb_set_error("scatter launch: %s", cudaGetErrorString(e)); return -1; }
    return 0;
  }
};

PbAotProgram *pb_make_scatter(const PbHeader &h, std::string &err) {
  auto params = h.getv("params"), vocab = h.getv("vocab"), off = h.getv("offsets");
  auto tok = h.getv("tok"), feat = h.getv("feat");
  if (params.size() != 4 || vocab.size() != 2 || off.size() != 3 || tok.size() % 3 || feat.size() % 3 ||
      tok.empty() || tok.size() > 12 || feat.size() > 9) { err = "malformed scatter header"; return nullptr; }
  ScatterProgram *p = new ScatterProgram();
  p->n_params = (int)h.geti("nparams");
  p->p_out = (int)params[0]; p->p_ids = (int)params[1]; p->p_arange = (int)params[2]; p->p_src = (int)params[3];
  p->rw.assign((size_t)p->n_params, '-');
  for (int i = 1; i < 4; i++) p->rw[(size_t)params[i]] = 'r';
  p->rw[(size_t)params[0]] = 'w';
  ScatterArgs &a = p->a;
  a.vocab = vocab[0]; a.out_vstride = vocab[1];
  a.out_off = off[0]; a.ids_off = off[1]; a.src_off = off[2];
  a.ntok = (int)tok.size() / 3; a.nfeat = (int)feat.size() / 3;
  a.n_tokens = 1; a.n_feat = 1;
  for (int i = 0; i < a.ntok; i++) { a.tok_ext[i] = tok[3 * i]; a.tok_ids[i] = tok[3 * i + 1]; a.tok_src[i] = tok[3 * i + 2]; a.n_tokens *= a.tok_ext[i]; }
  for (int i = 0; i < a.nfeat; i++) { a.feat_ext[i] = feat[3 * i]; a.feat_out[i] = feat[3 * i + 1]; a.feat_src[i] = feat[3 * i + 2]; a.n_feat *= a.feat_ext[i]; }
  if (a.n_tokens >= (1LL << 40)) { err = "scatter: too many tokens"; delete p; return nullptr; }
  /* feature axes: smallest output stride first so that consecutive threads write consecutive floats */
  for (int i = 1; i < a.nfeat; i++)
    for (int j = i; j > 0 && llabs(a.feat_out[j]) < llabs(a.feat_out[j - 1]); j--) {
      std::swap(a.feat_ext[j], a.feat_ext[j - 1]); std::swap(a.feat_out[j], a.feat_out[j - 1]); std::swap(a.feat_src[j], a.feat_src[j - 1]);
    }
  return p;
}
