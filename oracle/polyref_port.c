/*
 * polyref_port.c -- plain-C restatement of the arithmetic of polygrad's CPU
 * backend for the kernels on the execution path.  TEST INFRASTRUCTURE ONLY:
 * nothing in the product path links, loads or calls this file.
 *
 * polygrad's CPU backend renders every scheduled kernel as scalar C loops
 * (src/render_c.c:1046-1608) compiled with -O2 and no FMA contraction; a
 * reduction is `acc = acc + value` in increasing range order, starting from 0
 * (src/codegen.c:1424-1583).  The functions below restate those loops for
 * fixed kernel shapes.  Compile with -ffp-contract=off.
 */
#include <stddef.h>
#include <stdint.h>
#include <math.h>

/* C[m,n] = sum_k A[m*a_sm + k*a_sk] * B[k*b_sk + n*b_sn], k ascending, unfused;
 * optional + bias[n] then relu as where(0 < x, x, 0).
 * polygrad: poly_dot src/frontend.c:1029-1129; bias/relu fused by the scheduler
 * (src/model_mlp.c:227-235, src/modelzoo/models/gpt2.c:59-83). */
void polyref_matmul_f32(const float *A, const float *B, float *C, int64_t M, int64_t N, int64_t K,
                        int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn,
                        const float *bias, int relu) {
  for (int64_t m = 0; m < M; m++)
    for (int64_t n = 0; n < N; n++) {
      float acc = 0.0f;
      for (int64_t k = 0; k < K; k++) {
        float p = A[m * a_sm + k * a_sk] * B[k * b_sk + n * b_sn];
        acc = acc + p;
      }
      if (bias) acc = acc + bias[n];
      if (relu) acc = (0.0f < acc) ? acc : 0.0f;
      C[m * N + n] = acc;
    }
}

/* Same contraction with operands rounded to bfloat16 first (round to nearest
 * even), products and sums in fp32: what a bf16 buffer cast to fp32 before the
 * MUL computes (src/frontend.c:710 poly_cast_by_id + poly_dot). */
static float bf16_round(float x) {
  uint32_t u; __builtin_memcpy(&u, &x, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return x;
  u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;
  float r; __builtin_memcpy(&r, &u, 4);
  return r;
}
void polyref_matmul_bf16(const float *A, const float *B, float *C, int64_t M, int64_t N, int64_t K,
                         int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn,
                         const float *bias, int relu) {
  for (int64_t m = 0; m < M; m++)
    for (int64_t n = 0; n < N; n++) {
      float acc = 0.0f;
      for (int64_t k = 0; k < K; k++) {
        float p = bf16_round(A[m * a_sm + k * a_sk]) * bf16_round(B[k * b_sk + n * b_sn]);
        acc = acc + p;
      }
      if (bias) acc = acc + bias[n];
      if (relu) acc = (0.0f < acc) ? acc : 0.0f;
      C[m * N + n] = acc;
    }
}

/* out[t,d] = sum_v (ids[t] == arange[v]) ? table[v,d] : 0, v ascending from +0.
 * polygrad: embedding() src/modelzoo/models/gpt2.c:93-153.  Written as the
 * search it is equivalent to, adding the matching rows in the same order. */
void polyref_embedding(const float *ids, const float *arange, const float *table, float *out,
                       int64_t n_tok, int64_t V, int64_t D) {
  for (int64_t t = 0; t < n_tok; t++) {
    for (int64_t d = 0; d < D; d++) out[t * D + d] = 0.0f;
    for (int64_t v = 0; v < V; v++) {
      if (ids[t] != arange[v]) continue;
      for (int64_t d = 0; d < D; d++) out[t * D + d] = out[t * D + d] + table[v * D + d];
    }
  }
}

/* Row reductions over the last axis of [R, C], c ascending.
 * polygrad: do_reduce src/frontend.c:921-966 (mean = sum / C in the same kernel). */
void polyref_row_sum(const float *x, float *out, int64_t R, int64_t C) {
  for (int64_t r = 0; r < R; r++) { float a = 0.0f; for (int64_t c = 0; c < C; c++) a = a + x[r * C + c]; out[r] = a; }
}
void polyref_row_max(const float *x, float *out, int64_t R, int64_t C) {
  for (int64_t r = 0; r < R; r++) {
    float a = -INFINITY;
    for (int64_t c = 0; c < C; c++) { float v = x[r * C + c]; a = (a > v) ? a : v; }
    out[r] = a;
  }
}
/* sum_c (x - mean[r])^2, c ascending (src/frontend.c:968-992; layernorm :3585-3625) */
void polyref_row_sqdev(const float *x, const float *mean, float *out, int64_t R, int64_t C) {
  for (int64_t r = 0; r < R; r++) {
    float a = 0.0f;
    for (int64_t c = 0; c < C; c++) { float d = x[r * C + c] + (-mean[r]); a = a + d * d; }
    out[r] = a;
  }
}
