/*
 * pb_attention.cu -- softmax(Q Kᵀ · scale + mask) · V without materialising the
 * T x T score matrix.
 *
 * polygrad's GPT-2 builder computes attention as six realised kernels per layer
 * (reference: src/modelzoo/models/gpt2.c:402-434): scores = q.kᵀ, scores*scale +
 * mask, row max, row sum of exp, normalise, attn.v -- each a full pass over the
 * [B, H, T, T] tensor (403 MB at 8 x 12 x 1024 x 1024).  When a plan contains
 * exactly that chain, with nothing else reading the intermediates, and the bf16
 * contraction policy is on, the chain is replaced by this kernel
 * (pb_fuse.c); its arithmetic is the chain's: x = s*scale + mask in fp32,
 * p = exp2((x - rowmax) * log2e), out = (sum p v) / (sum p), with q, k, v and p
 * rounded to bf16 for the two contractions and fp32 accumulation, the row max
 * and row sum carried across blocks of 128 keys (the usual online form: a new
 * running max rescales what has been accumulated).  No causal structure is
 * assumed: the mask is an arbitrary additive [T, T] buffer.  A block of keys is
 * left out only where that provably changes nothing: its mask tile holds one
 * value c, and c + S < L - 100, where S bounds |q.k * scale| for the block
 * (largest row norms of q and k, Cauchy-Schwarz) and L is a lower bound of every
 * row's running maximum taken from the blocks already processed.  Then each
 * probability of the block is exp2 of less than -126 -- exactly 0 in this
 * kernel's arithmetic -- and the running maximum cannot move, so sums and
 * accumulators are bit for bit what processing the block would leave (for
 * finite v).  The -1e9 upper triangle of a causal mask goes this way.
 *
 * Q, K and V are bfloat16 matrices of 64-element rows addressed through strides
 * (row pitch and up to three batch strides), so the three slices of a fused
 * qkv projection are read where they lie; V is used as stored ([key][d], the
 * "MN-major" B operand of the second contraction), nothing is transposed.
 *
 * One CTA per (batch*head, block of 128 query rows), 9 warps, two CTAs per SM:
 *   warp 8   lane 0 issues the TMA loads (Q once; K and V blocks, each
 *            prefetched as soon as the MMA that read the previous one has
 *            finished) and the tcgen05.mma instructions:
 *            S = Q Kᵀ (128x128x64) into tensor memory, then PV = P V
 *            (128x64x128) into another 64 columns;
 *   warps 0-7  two threads per query row (64 keys and 32 output columns each):
 *            read S from tensor memory in 32-column chunks (pass 1: the row max of
 *            x = s*scale + mask, exchanged through shared memory; pass 2: the
 *            scores again, x and the exponentials), write P as bf16 into shared
 *            memory in the swizzled K-major tile layout the MMA reads, then add
 *            PV to the row's fp32 accumulators in registers.
 * Head size 64, T a multiple of 128.  All barrier waits are bounded.
 */
#include "pb_gemm.h"
#include "../../../include/poly_b200.h"
#include <dlfcn.h>

__device__ int pb200_attn_error_flag = 0;
#define PB_TC_ERROR_FLAG pb200_attn_error_flag
#include "pb_tc_ptx.cuh"

#define AT_BQ 128      /* query rows per CTA */
#define AT_BK 128      /* keys per block */
#define AT_HD 64
#define AT_REC 8       /* floats per mask-tile record, see pb200_mask_tiles */
#define AT_THREADS 288
#define AT_SMEM (16384 /*Q*/ + 16384 /*K*/ + 16384 /*V: 128 keys x 128 B*/ + 32768 /*P: 2 x 16 KB*/ + 256 + 1024)

/* 2^x by the special-function unit (ex2.approx: relative error about 2^-22; the
 * results are rounded to bfloat16 right after). */
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct AttnArgs {
  float *O; const float *mask;
  long long mask_sq, mask_sk;     /* mask[q*mask_sq + k*mask_sk] */
  float scale;
  int mask_vec;                   /* mask rows contiguous and 16-byte aligned */
  const float *tile_const;        /* per (query block, key block) one record of AT_REC floats, see pb200_mask_tiles */
  const float *qn, *kn;           /* per (batch*head, block of 128 rows): upper bound of the largest row 2-norm; null: no skipping */
  int T, n_qblocks;
  int nb; int bext[3]; long long o_sb[3]; long long o_sm;   /* O[batch..][row*o_sm + d] */
  int out_bf16;                   /* O holds bfloat16 (same element offsets) */
};

__global__ void __launch_bounds__(AT_THREADS, 2)
pb200_flash_attn(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const AttnArgs g) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *sm = smem_raw + (base - raw);
  const uint32_t s_q = base, s_k = base + 16384, s_v = base + 32768, s_p = base + 49152;
  uint64_t *bars = reinterpret_cast<uint64_t *>(sm + 81920);
  const uint32_t bar_q = smem_u32(bars), bar_k = bar_q + 8, bar_v = bar_q + 16, bar_s = bar_q + 24, bar_p = bar_q + 32, bar_o = bar_q + 40, bar_x = bar_q + 48;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ float xchg[2][AT_BQ];     /* per-row exchange between the two threads of a row */
  __shared__ unsigned long long s_live;    /* bit j: key block j is processed */

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  /* late query blocks first: under a causal mask they process the most key blocks, and the
   * hardware hands out CTAs in index order, so the short ones fill the tail */
  const int n_bh = gridDim.x / g.n_qblocks;
  const int qb = g.n_qblocks - 1 - (int)(blockIdx.x / n_bh), bh = blockIdx.x % n_bh;
  const int nkb = g.T / AT_BK;

  if (threadIdx.x == 0) {
    /* which key blocks to process (see the head of this file) */
    unsigned long long live = 0;
    float lrun = __int_as_float(0xff800000);
    for (int j = 0; j < nkb; j++) {
      const float c = g.tile_const[AT_REC * (qb * nkb + j)], lmin = g.tile_const[AT_REC * (qb * nkb + j) + 1];
      float S = 0.0f;
      bool skip = false;
      if (g.qn) {
        S = fabsf(g.scale) * g.qn[bh * g.n_qblocks + qb] * g.kn[bh * nkb + j];
        skip = (c == c) && (c + S < lrun - 100.0f);
      }
      if (!skip) { live |= 1ull << j; lrun = fmaxf(lrun, lmin - S); }
    }
    s_live = live;
    abort_flag = 0;
    mbar_init(bar_q, 1); mbar_init(bar_k, 1); mbar_init(bar_v, 1);
    mbar_init(bar_s, 1); mbar_init(bar_p, 8); mbar_init(bar_o, 1); mbar_init(bar_x, 8);   /* one arrival per softmax warp */
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tmem_s = tmem, tmem_pv = tmem + 128;

  if (warp == 8) {
    if (lane == 0) {
      /* instruction descriptors: bf16 x bf16 -> fp32, M = 128.  S: both operands K-major.
       * PV: A (P) K-major, B (V) MN-major (bit 16): V's rows are keys (K), each 64 contiguous d (N). */
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(AT_BK >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(AT_HD >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      int c0 = 0, c1 = 0, c2 = 0;
      {
        int rem = bh;
        if (g.nb > 0) { c0 = rem % g.bext[0]; rem /= g.bext[0]; }
        if (g.nb > 1) { c1 = rem % g.bext[1]; rem /= g.bext[1]; }
        if (g.nb > 2) { c2 = rem % g.bext[2]; }
      }
      mbar_expect_tx(bar_q, 16384);
      tma_load_5d(s_q, &map_q, bar_q, 0, qb * AT_BQ, c0, c1, c2);
      unsigned long long rem = s_live;
      const int j0 = __ffsll((long long)rem) - 1;          /* the first block is always processed */
      mbar_expect_tx(bar_k, 16384);
      tma_load_5d(s_k, &map_k, bar_k, 0, j0 * AT_BK, c0, c1, c2);
      mbar_expect_tx(bar_v, 16384);
      tma_load_5d(s_v, &map_v, bar_v, 0, j0 * AT_BK, c0, c1, c2);
      bool ok = mbar_wait(bar_q, 0, &abort_flag, 11) && mbar_wait(bar_k, 0, &abort_flag, 12);
      const uint64_t dq = make_smem_desc(s_q), dk = make_smem_desc(s_k);
      if (ok) {
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < AT_HD / 16; k++) tc_mma_bf16(tmem_s, dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_s, k ? 1u : 0u);
        tc_commit(bar_s);
      }
      for (uint32_t it = 0; rem && ok; it++) {
        rem &= rem - 1;                                    /* this block; what is left are the later ones */
        const bool more = rem != 0;
        const int jn = more ? __ffsll((long long)rem) - 1 : 0;
        const uint32_t ph = it & 1u;
        /* K is free once S is complete: prefetch the next block of keys */
        if (!mbar_wait(bar_s, ph, &abort_flag, 13)) break;
        if (more) { mbar_expect_tx(bar_k, 16384); tma_load_5d(s_k, &map_k, bar_k, 0, jn * AT_BK, c0, c1, c2); }
        if (!mbar_wait(bar_p, ph, &abort_flag, 14)) break;     /* P written, S and the previous PV consumed */
        if (!mbar_wait(bar_v, ph, &abort_flag, 15)) break;
        tc_fence_after_sync();
        /* 16 keys per instruction: 32 bytes along a row of P (K-major), two 8-key groups
         * of 1024 bytes of V (MN-major: the stride between 8-key groups is the descriptor's
         * stride byte offset, 1024) */
#pragma unroll
        for (int h = 0; h < 2; h++) {
          const uint64_t da = make_smem_desc(s_p + h * 16384), db = make_smem_desc(s_v + h * 8192);
#pragma unroll
          for (int k = 0; k < 4; k++) tc_mma_bf16(tmem_pv, da + (uint64_t)(k * 2), db + (uint64_t)(k * 128), idesc_o, (h | k) ? 1u : 0u);
        }
        tc_commit(bar_o);
        /* the next block's scores follow at once: S is free, and the softmax threads find
         * them ready when they come back from adding this block's PV */
        if (more) {
          if (!mbar_wait(bar_k, ph ^ 1u, &abort_flag, 12)) break;
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < AT_HD / 16; k++) tc_mma_bf16(tmem_s, dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_s, k ? 1u : 0u);
          tc_commit(bar_s);
        }
        if (!mbar_wait(bar_o, ph, &abort_flag, 16)) break;
        if (more) {
          mbar_expect_tx(bar_v, 16384);
          tma_load_5d(s_v, &map_v, bar_v, 0, jn * AT_BK, c0, c1, c2);
        }
      }
    }
  } else {
    /* ── softmax: two threads per query row (warps w and w+4 share the row's
     * tensor-memory lanes); each owns 64 of the block's 128 keys and 32 of the
     * 64 output columns ── */
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;                 /* row within the block = tensor-memory lane */
    const long long q = (long long)qb * AT_BQ + row;
    const float *mrow = g.mask + q * g.mask_sq;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_cols = tmem_s + lane_addr + half * 64, pv_cols = tmem_pv + lane_addr + half * 32;
    const float LOG2E = 1.44269504088896340736f;
    float m_run = __int_as_float(0xff800000), l_run = 0.0f;   /* l_run: this thread's keys only */
    float acc[32];
#pragma unroll
    for (int d = 0; d < 32; d++) acc[d] = 0.0f;
    uint8_t *p_row = sm + 49152 + half * 16384 + (row >> 3) * 1024 + (row & 7) * 128;
    bool ok = true;
    uint32_t xph = 0;
    uint32_t it = 0;
    for (unsigned long long rem = s_live; rem && ok; rem &= rem - 1, it++) {
      const int j = __ffsll((long long)rem) - 1;
      const uint32_t ph = it & 1u;
      const float *mj = mrow + ((long long)j * AT_BK + half * 64) * g.mask_sk;
      const float tile_c = g.tile_const[AT_REC * (qb * nkb + j)];
      const bool tile_is_const = (tile_c == tile_c);
      if (!__all_sync(0xffffffffu, mbar_wait(bar_s, ph, &abort_flag, 17))) { ok = false; break; }
      tc_fence_after_sync();
      /* pass 1: the largest x = s*scale + mask over this thread's keys.  Nothing is written back: pass 2
       * loads the scores again and forms the same x (one fused multiply-add per element, against a
       * tensor-memory store and the wait for it).  Where the mask tile is one value c and the scale is
       * not negative, x is a non-decreasing function of s, so the largest x is that of the largest s. */
      float m_part = __int_as_float(0xff800000);
      const bool plain_max = tile_is_const && g.scale >= 0.0f;
#pragma unroll 1
      for (int c = 0; c < 2; c++) {
        uint32_t r[32];
        tc_ld32(s_cols + c * 32, r);
        tc_wait_ld();
        if (plain_max) {
#pragma unroll
          for (int i = 0; i < 32; i++) m_part = fmaxf(m_part, __uint_as_float(r[i]));
        } else if (tile_is_const) {
#pragma unroll
          for (int i = 0; i < 32; i++) m_part = fmaxf(m_part, fmaf(__uint_as_float(r[i]), g.scale, tile_c));
        } else if (g.mask_vec) {
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const float4 mv = reinterpret_cast<const float4 *>(mj + c * 32)[i];
            const float x0 = fmaf(__uint_as_float(r[4 * i]), g.scale, mv.x), x1 = fmaf(__uint_as_float(r[4 * i + 1]), g.scale, mv.y);
            const float x2 = fmaf(__uint_as_float(r[4 * i + 2]), g.scale, mv.z), x3 = fmaf(__uint_as_float(r[4 * i + 3]), g.scale, mv.w);
            m_part = fmaxf(m_part, fmaxf(fmaxf(x0, x1), fmaxf(x2, x3)));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i++)
            m_part = fmaxf(m_part, fmaf(__uint_as_float(r[i]), g.scale, mj[(long long)(c * 32 + i) * g.mask_sk]));
        }
      }
      if (plain_max) m_part = fmaf(m_part, g.scale, tile_c);
      xchg[half][row] = m_part;
      /* exchange through an mbarrier rather than bar.sync: its wait is bounded like all others.
       * One arrival per warp (256 arrivals on one shared-memory word serialise). */
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_x);
      if (!__all_sync(0xffffffffu, mbar_wait(bar_x, xph & 1u, &abort_flag, 19))) { ok = false; break; }
      xph++;
      const float m_other = xchg[half ^ 1][row];
      const float m_new = fmaxf(m_run, fmaxf(m_part, m_other));
      const float m_scaled = m_new * LOG2E;
      const float alpha = fast_exp2((m_run - m_new) * LOG2E);   /* 0 on the first block (m_run = -inf) */
      float l_blk = 0.0f;
      /* pass 2: p = exp2((x - m_new) * log2e), written as bf16 into the K-major swizzled tile */
#pragma unroll 1
      for (int c = 0; c < 2; c++) {
        uint32_t r[32];
        tc_ld32(s_cols + c * 32, r);
        tc_wait_ld();
        if (!tile_is_const) {
          /* x in place of s (the mask values come from L1 this time) */
          if (g.mask_vec) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
              const float4 mv = reinterpret_cast<const float4 *>(mj + c * 32)[i];
              r[4 * i] = __float_as_uint(fmaf(__uint_as_float(r[4 * i]), g.scale, mv.x));
              r[4 * i + 1] = __float_as_uint(fmaf(__uint_as_float(r[4 * i + 1]), g.scale, mv.y));
              r[4 * i + 2] = __float_as_uint(fmaf(__uint_as_float(r[4 * i + 2]), g.scale, mv.z));
              r[4 * i + 3] = __float_as_uint(fmaf(__uint_as_float(r[4 * i + 3]), g.scale, mv.w));
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; i++)
              r[i] = __float_as_uint(fmaf(__uint_as_float(r[i]), g.scale, mj[(long long)(c * 32 + i) * g.mask_sk]));
          }
        }
#pragma unroll
        for (int i8 = 0; i8 < 4; i8++) {
          uint32_t w[4];
#pragma unroll
          for (int i2 = 0; i2 < 4; i2++) {
            const int i = i8 * 8 + i2 * 2;
            float x0 = __uint_as_float(r[i]), x1 = __uint_as_float(r[i + 1]);
            if (tile_is_const) { x0 = fmaf(x0, g.scale, tile_c); x1 = fmaf(x1, g.scale, tile_c); }
            const float p0 = fast_exp2(fmaf(x0, LOG2E, -m_scaled)), p1 = fast_exp2(fmaf(x1, LOG2E, -m_scaled));
            __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
            l_blk += p0 + p1;
            w[i2] = *reinterpret_cast<uint32_t *>(&pb);
          }
          const int chunk = c * 4 + i8;                         /* 16-byte chunk within the 128-byte row */
          *reinterpret_cast<uint4 *>(p_row + ((chunk ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      l_run = l_run * alpha + l_blk;
      m_run = m_new;
      /* the running maximum moves in the first blocks of a row and seldom afterwards: where no row of
       * the warp moved, alpha is exactly 1 and the rescale is skipped (same bits either way) */
      if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
        for (int d = 0; d < 32; d++) acc[d] *= alpha;
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);
      if (!__all_sync(0xffffffffu, mbar_wait(bar_o, ph, &abort_flag, 18))) { ok = false; break; }
      tc_fence_after_sync();
      {
        uint32_t r[32];
        tc_ld32(pv_cols, r);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i++) acc[i] += __uint_as_float(r[i]);
      }
    }
    /* total row sum = the two threads' partial sums */
    if (ok) {
      xchg[half][row] = l_run;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_x);
      ok = __all_sync(0xffffffffu, mbar_wait(bar_x, xph & 1u, &abort_flag, 20));
    }
    if (ok) {
      const float l_tot = l_run + xchg[half ^ 1][row];
      int rem = bh; long long ob = 0;
      for (int i = 0; i < g.nb; i++) { const int x = rem % g.bext[i]; rem /= g.bext[i]; ob += x * g.o_sb[i]; }
      const long long oe = ob + q * g.o_sm + half * 32;
      const float inv = 1.0f / l_tot;
      if (g.out_bf16) {
        __nv_bfloat16 *o = reinterpret_cast<__nv_bfloat16 *>(g.O) + oe;
#pragma unroll
        for (int d = 0; d < 32; d += 8) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const __nv_bfloat162 v2 = __floats2bfloat162_rn(acc[d + 2 * i] * inv, acc[d + 2 * i + 1] * inv);
            w[i] = *reinterpret_cast<const uint32_t *>(&v2);
          }
          *reinterpret_cast<uint4 *>(o + d) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      } else {
        float *o = g.O + oe;
#pragma unroll
        for (int d = 0; d < 32; d += 4)
          *reinterpret_cast<float4 *>(o + d) = make_float4(acc[d] * inv, acc[d + 1] * inv, acc[d + 2] * inv, acc[d + 3] * inv);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (abort_flag) { for (int i = 0; i < 2000; i++) __nanosleep(1000); }
  if (warp == 8) {
    tc_fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
  }
}

/* ── second arrangement of the same computation ──────────────────────────
 * The output accumulator stays in tensor memory: PV = P V is added there by the tensor
 * cores block after block (accumulate flag), so the softmax threads neither read PV back
 * nor carry 32 accumulators each; that leaves registers for a whole block of scores (64
 * per thread), which are loaded ONCE, reduced to the row maximum, and turned into
 * probabilities from registers.  As soon as every thread holds its scores the S region is
 * free, so the next block's S = Q K' runs under this block's exponentials.  When a row's
 * running maximum moves (the first blocks of a row; seldom afterwards) its part of the
 * accumulator is rescaled in tensor memory (load, multiply, store) between two PV products.
 * V is double-buffered so that the next block's V is requested one product ahead.
 * Arithmetic per element is that of pb200_flash_attn (x = fma(s, scale, mask), p =
 * exp2(fma(x, log2e, -m log2e)), bf16 P, fp32 sums); the block sums of P V are added by the
 * tensor cores instead of with rounded fp32 adds. */
#define AT2_SMEM (16384 /*Q*/ + 16384 /*K*/ + 32768 /*V: 2 x 16 KB*/ + 32768 /*P: 2 x 16 KB*/ + 256 + 1024)

__global__ void __launch_bounds__(AT_THREADS, 2)
pb200_flash_attn2(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, const AttnArgs g) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *sm = smem_raw + (base - raw);
  const uint32_t s_q = base, s_k = base + 16384, s_v = base + 32768, s_p = base + 65536;
  uint64_t *bars = reinterpret_cast<uint64_t *>(sm + 98304);
  const uint32_t bar_q = smem_u32(bars), bar_k = bar_q + 8, bar_v = bar_q + 16 /* two */, bar_s = bar_q + 32, bar_p = bar_q + 40,
                 bar_o = bar_q + 48, bar_f = bar_q + 56, bar_x = bar_q + 64 /* four: one per pair of warps sharing rows */;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ float xchg[2][AT_BQ];
  __shared__ unsigned long long s_live;
  /* per key block, from the mask-tile records and the row-norm bounds: fetched by 64 threads at once, because the
   * choice of blocks below is a serial scan that would otherwise wait for global memory once per block */
  __shared__ float s_tc[64], s_lm[64], s_kn[64], s_kind[64], s_d[64], s_lo[64], s_hi[64];
  __shared__ float s_qn;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_bh = gridDim.x / g.n_qblocks;
  const int qb = g.n_qblocks - 1 - (int)(blockIdx.x / n_bh), bh = blockIdx.x % n_bh;
  const int nkb = g.T / AT_BK;

  if ((int)threadIdx.x < nkb) {
    const int j = threadIdx.x;
    const float *rec = g.tile_const + (long long)AT_REC * (qb * nkb + j);
    const float4 r0 = *reinterpret_cast<const float4 *>(rec), r1 = *reinterpret_cast<const float4 *>(rec + 4);
    s_tc[j] = r0.x; s_lm[j] = r0.y; s_kind[j] = r0.z; s_d[j] = r0.w; s_lo[j] = r1.x; s_hi[j] = r1.y;
    s_kn[j] = g.qn ? g.kn[bh * nkb + j] : 0.0f;
  }
  if (threadIdx.x == 64) s_qn = g.qn ? g.qn[bh * g.n_qblocks + qb] : 0.0f;
  /* batch coordinates of this (batch, head) for the tensor maps */
  int c0 = 0, c1 = 0, c2 = 0;
  if (warp == 8) {
    int rem = bh;
    if (g.nb > 0) { c0 = rem % g.bext[0]; rem /= g.bext[0]; }
    if (g.nb > 1) { c1 = rem % g.bext[1]; rem /= g.bext[1]; }
    if (g.nb > 2) { c2 = rem % g.bext[2]; }
    if (lane == 0) {
      abort_flag = 0;
      mbar_init(bar_q, 1); mbar_init(bar_k, 1); mbar_init(bar_v, 1); mbar_init(bar_v + 8, 1);
      mbar_init(bar_s, 1); mbar_init(bar_p, 8); mbar_init(bar_o, 1); mbar_init(bar_f, 8);
      for (int i = 0; i < 4; i++) mbar_init(bar_x + 8 * i, 2);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      /* Q and the first block of keys and values are requested at once: block 0 is always processed (nothing can be
       * left out before a running maximum exists), so these loads run under the rest of the set-up */
      mbar_expect_tx(bar_q, 16384);
      tma_load_5d(s_q, &map_q, bar_q, 0, qb * AT_BQ, c0, c1, c2);
      mbar_expect_tx(bar_k, 16384);
      tma_load_5d(s_k, &map_k, bar_k, 0, 0, c0, c1, c2);
      mbar_expect_tx(bar_v, 16384);
      tma_load_5d(s_v, &map_v, bar_v, 0, 0, c0, c1, c2);
    }
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    /* which key blocks to process (see the head of this file) */
    unsigned long long live = 0;
    float lrun = __int_as_float(0xff800000);
    const float qn = s_qn;
    for (int j = 0; j < nkb; j++) {
      const float c = s_tc[j], lmin = s_lm[j];
      float S = 0.0f;
      bool skip = false;
      if (g.qn) {
        S = fabsf(g.scale) * qn * s_kn[j];
        skip = (c == c) && (c + S < lrun - 100.0f);
      }
      if (!skip || j == 0) { live |= 1ull << j; lrun = fmaxf(lrun, lmin - S); }
    }
    s_live = live;
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tmem_s = tmem, tmem_pv = tmem + 128;

  if (warp == 8) {
    if (lane == 0) {
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(AT_BK >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(AT_HD >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      unsigned long long rem = s_live;                     /* bit 0 is always set; its loads are under way */
      bool ok = mbar_wait(bar_q, 0, &abort_flag, 11) && mbar_wait(bar_k, 0, &abort_flag, 12);
      const uint64_t dq = make_smem_desc(s_q), dk = make_smem_desc(s_k);
      if (ok) {
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < AT_HD / 16; k++) tc_mma_bf16(tmem_s, dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_s, k ? 1u : 0u);
        tc_commit(bar_s);
      }
      for (uint32_t it = 0; rem && ok; it++) {
        rem &= rem - 1;
        const bool more = rem != 0;
        const int jn = more ? __ffsll((long long)rem) - 1 : 0;
        const uint32_t ph = it & 1u;
        /* S(it) complete (it was issued one iteration ago).  The key block after this one is normally on its
         * way already (requested below, one iteration ahead); only the very first request happens here */
        if (!mbar_wait(bar_s, ph, &abort_flag, 13)) break;
        if (more && it == 0) { mbar_expect_tx(bar_k, 16384); tma_load_5d(s_k, &map_k, bar_k, 0, jn * AT_BK, c0, c1, c2); }
        /* V buffer (it+1)&1 was last read by PV(it-1): request the next block of values once that product is done */
        if (more) {
          if (it > 0 && !mbar_wait(bar_o, (it - 1) & 1u, &abort_flag, 16)) break;
          const uint32_t vb = (it + 1) & 1u;
          mbar_expect_tx(bar_v + 8 * vb, 16384);
          tma_load_5d(s_v + vb * 16384, &map_v, bar_v + 8 * vb, 0, jn * AT_BK, c0, c1, c2);
        }
        /* every softmax thread holds its scores of block it: S may be overwritten */
        if (!mbar_wait(bar_f, ph, &abort_flag, 21)) break;
        if (more) {
          if (!mbar_wait(bar_k, ph ^ 1u, &abort_flag, 12)) break;
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < AT_HD / 16; k++) tc_mma_bf16(tmem_s, dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_s, k ? 1u : 0u);
          tc_commit(bar_s);
          /* that product is short; once it has read K, the keys of the block after next are requested -- a whole
           * iteration before they are needed, instead of at the moment they are */
          const unsigned long long rem2 = rem & (rem - 1);
          if (rem2) {
            if (!mbar_wait(bar_s, ph ^ 1u, &abort_flag, 23)) break;
            mbar_expect_tx(bar_k, 16384);
            tma_load_5d(s_k, &map_k, bar_k, 0, (__ffsll((long long)rem2) - 1) * AT_BK, c0, c1, c2);
          }
        }
        /* P(it) written (and the accumulator rescaled where a maximum moved): add P V */
        if (!mbar_wait(bar_p, ph, &abort_flag, 14)) break;
        if (!mbar_wait(bar_v + 8 * ph, (it >> 1) & 1u, &abort_flag, 15)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int h = 0; h < 2; h++) {
          const uint64_t da = make_smem_desc(s_p + h * 16384), db = make_smem_desc(s_v + ph * 16384 + h * 8192);
#pragma unroll
          for (int k = 0; k < 4; k++) tc_mma_bf16(tmem_pv, da + (uint64_t)(k * 2), db + (uint64_t)(k * 128), idesc_o, (it | (uint32_t)h | (uint32_t)k) ? 1u : 0u);
        }
        tc_commit(bar_o);
      }
    }
  } else {
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;
    const long long q = (long long)qb * AT_BQ + row;
    const float *mrow = g.mask + q * g.mask_sq;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_cols = tmem_s + lane_addr + half * 64, pv_cols = tmem_pv + lane_addr + half * 32;
    const uint32_t bar_xq = bar_x + 8 * quarter;
    const float LOG2E = 1.44269504088896340736f;
    float m_run = __int_as_float(0xff800000), l_run = 0.0f;
    uint8_t *p_row = sm + 65536 + half * 16384 + (row >> 3) * 1024 + (row & 7) * 128;
    /* where this thread's 32 output values go (the divisions are kept off the end of the kernel) */
    long long oe;
    {
      int rem = bh; long long ob = 0;
      for (int i = 0; i < g.nb; i++) { const int x = rem % g.bext[i]; rem /= g.bext[i]; ob += x * g.o_sb[i]; }
      oe = ob + q * g.o_sm + half * 32;
    }
    bool ok = true;
    uint32_t xph = 0, it = 0;
    for (unsigned long long rem = s_live; rem && ok; rem &= rem - 1, it++) {
      const int j = __ffsll((long long)rem) - 1;
      const uint32_t ph = it & 1u;
      const float tile_c = s_tc[j];
      const bool tile_is_const = (tile_c == tile_c), tile_is_step = s_kind[j] == 2.0f;
      if (!__all_sync(0xffffffffu, mbar_wait(bar_s, ph, &abort_flag, 17))) { ok = false; break; }
      tc_fence_after_sync();
      /* this thread's 64 scores, once */
      uint32_t r0[32], r1[32];
      tc_ld32(s_cols, r0);
      tc_ld32(s_cols + 32, r1);
      tc_wait_ld();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_f);
      /* The largest x = fma(s, scale, mask) of this thread's keys.  Where the tile is one value c and the scale is
       * not negative, x is a non-decreasing function of s: the largest x is that of the largest s, and the scores
       * stay as they are (the exponent below is formed from them directly).  Otherwise x replaces s in place. */
      float m_part = __int_as_float(0xff800000);
      const bool plain = tile_is_const && g.scale >= 0.0f, step = tile_is_step && g.scale >= 0.0f;
      const float lo = s_lo[j], hi = s_hi[j];
      const int thr = (int)s_d[j] + row - half * 64;        /* key k of the thread's 64 has the value lo where k > thr, else hi */
      if (plain) {
#pragma unroll
        for (int i = 0; i < 32; i++) m_part = fmaxf(m_part, fmaxf(__uint_as_float(r0[i]), __uint_as_float(r1[i])));
        m_part = fmaf(m_part, g.scale, tile_c);
      } else if (step) {
        /* two values: the largest score of either side of the step, then x of each (the scores stay as they are) */
        float m_lo = __int_as_float(0xff800000), m_hi = m_lo;
        const float ninf = m_lo;
#pragma unroll
        for (int i = 0; i < 32; i++) {
          const float a = __uint_as_float(r0[i]), b = __uint_as_float(r1[i]);
          m_lo = fmaxf(m_lo, fmaxf(i > thr ? a : ninf, 32 + i > thr ? b : ninf));
          m_hi = fmaxf(m_hi, fmaxf(i > thr ? ninf : a, 32 + i > thr ? ninf : b));
        }
        m_part = fmaxf(m_lo == ninf ? ninf : fmaf(m_lo, g.scale, lo), m_hi == ninf ? ninf : fmaf(m_hi, g.scale, hi));
      } else {
        const float *mj = mrow + ((long long)j * AT_BK + half * 64) * g.mask_sk;
#pragma unroll
        for (int c = 0; c < 2; c++) {
          uint32_t (&r)[32] = c ? r1 : r0;
          if (tile_is_const) {
#pragma unroll
            for (int i = 0; i < 32; i++) r[i] = __float_as_uint(fmaf(__uint_as_float(r[i]), g.scale, tile_c));
          } else if (tile_is_step) {
            /* (negative scale) the entries of a step tile from the indices: no loads */
#pragma unroll
            for (int i = 0; i < 32; i++) r[i] = __float_as_uint(fmaf(__uint_as_float(r[i]), g.scale, (c * 32 + i > thr) ? lo : hi));
          } else if (g.mask_vec) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
              const float4 mv = reinterpret_cast<const float4 *>(mj + c * 32)[i];
              r[4 * i] = __float_as_uint(fmaf(__uint_as_float(r[4 * i]), g.scale, mv.x));
              r[4 * i + 1] = __float_as_uint(fmaf(__uint_as_float(r[4 * i + 1]), g.scale, mv.y));
              r[4 * i + 2] = __float_as_uint(fmaf(__uint_as_float(r[4 * i + 2]), g.scale, mv.z));
              r[4 * i + 3] = __float_as_uint(fmaf(__uint_as_float(r[4 * i + 3]), g.scale, mv.w));
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; i++)
              r[i] = __float_as_uint(fmaf(__uint_as_float(r[i]), g.scale, mj[(long long)(c * 32 + i) * g.mask_sk]));
          }
#pragma unroll
          for (int i = 0; i < 32; i++) m_part = fmaxf(m_part, __uint_as_float(r[i]));
        }
      }
      /* the row's other half is with the thread of the same lane four warps away: one barrier per such pair */
      xchg[half][row] = m_part;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_xq);
      if (!__all_sync(0xffffffffu, mbar_wait(bar_xq, xph & 1u, &abort_flag, 19))) { ok = false; break; }
      xph++;
      const float m_other = xchg[half ^ 1][row];
      const float m_new = fmaxf(m_run, fmaxf(m_part, m_other));
      const float m_scaled = m_new * LOG2E;
      const float alpha = fast_exp2((m_run - m_new) * LOG2E);
      /* probabilities p = exp2((x - m) log2e), two at a time (packed fp32 multiply-adds), packed as bf16 pairs over
       * the scores.  plain: x log2e - m log2e = s (scale log2e) + (c log2e - m log2e), one multiply-add per pair. */
      const bool raw = plain || step;                  /* r0, r1 still hold the scores */
      const float2 mul2 = raw ? make_float2(g.scale * LOG2E, g.scale * LOG2E) : make_float2(LOG2E, LOG2E);
      const float add_hi = plain ? fmaf(tile_c, LOG2E, -m_scaled) : step ? fmaf(hi, LOG2E, -m_scaled) : -m_scaled;
      const float add_lo = step ? fmaf(lo, LOG2E, -m_scaled) : add_hi;
      float2 l2 = make_float2(0.0f, 0.0f);
      if (step) {
#pragma unroll
        for (int c = 0; c < 2; c++) {
          uint32_t (&r)[32] = c ? r1 : r0;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float2 add2 = make_float2(c * 32 + i > thr ? add_lo : add_hi, c * 32 + i + 1 > thr ? add_lo : add_hi);
            const float2 e = __ffma2_rn(make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), mul2, add2);
            const float2 pp = make_float2(fast_exp2(e.x), fast_exp2(e.y));
            __nv_bfloat162 pb = __floats2bfloat162_rn(pp.x, pp.y);
            l2 = __fadd2_rn(l2, pp);
            r[i >> 1] = *reinterpret_cast<uint32_t *>(&pb);
          }
        }
      } else {
        const float2 add2 = make_float2(add_hi, add_hi);
#pragma unroll
        for (int c = 0; c < 2; c++) {
          uint32_t (&r)[32] = c ? r1 : r0;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float2 e = __ffma2_rn(make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), mul2, add2);
            const float2 pp = make_float2(fast_exp2(e.x), fast_exp2(e.y));
            __nv_bfloat162 pb = __floats2bfloat162_rn(pp.x, pp.y);
            l2 = __fadd2_rn(l2, pp);
            r[i >> 1] = *reinterpret_cast<uint32_t *>(&pb);
          }
        }
      }
      l_run = l_run * alpha + (l2.x + l2.y);
      m_run = m_new;
      /* the P tile and the accumulator are still in use by the previous block's product until it is done */
      if (it > 0) {
        if (!__all_sync(0xffffffffu, mbar_wait(bar_o, (it - 1) & 1u, &abort_flag, 18))) { ok = false; break; }
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, alpha != 1.0f)) {
          uint32_t o[32];
          tc_ld32(pv_cols, o);
          tc_wait_ld();
#pragma unroll
          for (int d = 0; d < 32; d++) o[d] = __float_as_uint(__uint_as_float(o[d]) * alpha);
          tc_st32(pv_cols, o);
          tc_wait_st();
        }
      }
#pragma unroll
      for (int c = 0; c < 2; c++) {
        const uint32_t (&r)[32] = c ? r1 : r0;
#pragma unroll
        for (int i8 = 0; i8 < 4; i8++) {
          const int chunk = c * 4 + i8;
          *reinterpret_cast<uint4 *>(p_row + ((chunk ^ (row & 7)) << 4)) = make_uint4(r[4 * i8], r[4 * i8 + 1], r[4 * i8 + 2], r[4 * i8 + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);
    }
    /* the last product, then the row sums of both halves */
    if (ok && it > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar_o, (it - 1) & 1u, &abort_flag, 22));
    if (ok) {
      tc_fence_after_sync();
      xchg[half][row] = l_run;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_xq);
      ok = __all_sync(0xffffffffu, mbar_wait(bar_xq, xph & 1u, &abort_flag, 20));
    }
    if (ok) {
      uint32_t o[32];
      tc_ld32(pv_cols, o);
      tc_wait_ld();
      const float l_tot = l_run + xchg[half ^ 1][row];
      const float inv = 1.0f / l_tot;
      if (g.out_bf16) {
        __nv_bfloat16 *op = reinterpret_cast<__nv_bfloat16 *>(g.O) + oe;
#pragma unroll
        for (int d = 0; d < 32; d += 8) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const __nv_bfloat162 v2 = __floats2bfloat162_rn(__uint_as_float(o[d + 2 * i]) * inv, __uint_as_float(o[d + 2 * i + 1]) * inv);
            w[i] = *reinterpret_cast<const uint32_t *>(&v2);
          }
          *reinterpret_cast<uint4 *>(op + d) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      } else {
        float *op = g.O + oe;
#pragma unroll
        for (int d = 0; d < 32; d += 4)
          *reinterpret_cast<float4 *>(op + d) = make_float4(__uint_as_float(o[d]) * inv, __uint_as_float(o[d + 1]) * inv,
                                                            __uint_as_float(o[d + 2]) * inv, __uint_as_float(o[d + 3]) * inv);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (abort_flag) { for (int i = 0; i < 2000; i++) __nanosleep(1000); }
  if (warp == 8) {
    tc_fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
  }
}

/* Classifies the mask by 128 x 128 tile into one record of AT_REC floats per tile:
 *   [0] the tile's value if all its entries are equal (the zeros below and the -1e9 above
 *       the diagonal of a causal mask, for instance), so that the attention kernel adds it
 *       without reading the tile; NaN otherwise;
 *   [1] the smallest, over the tile's rows, of the row's largest entry (-inf if a row holds a
 *       NaN) -- after the tile is processed every row's running maximum is at least that much
 *       minus the bound on |score|;
 *   [2] 2.0 for a "step" tile, whose entry (r, c) is [4] where c - r > [3] and [5] elsewhere
 *       (the diagonal tiles of a causal mask: -1e9 above the diagonal, 0 on and below it), so
 *       that the kernel forms the entries from the indices instead of loading 64 KB; else 0.
 * Every claim is checked bit for bit against all 16384 entries: exact for every mask. */
__global__ void __launch_bounds__(256) pb200_mask_tiles(const float *mask, long long sq, long long sk, int nk, float *out) {
  const int qi = blockIdx.y, ki = blockIdx.x;
  const float *t = mask + (long long)qi * AT_BQ * sq + (long long)ki * AT_BK * sk;
  const float first = t[0];
  /* step hypothesis from the corners and from row 0: lo = top right, hi = bottom left, and row 0 holds hi in
   * columns 0 .. d and lo beyond (d = -1: lo from column 0 on) */
  const unsigned lo_b = __float_as_uint(t[(long long)(AT_BK - 1) * sk]), hi_b = __float_as_uint(t[(long long)(AT_BQ - 1) * sq]);
  __shared__ int s_d;
  if (threadIdx.x == 0) s_d = -1;
  __syncthreads();
  if (threadIdx.x < AT_BK && __float_as_uint(t[(long long)threadIdx.x * sk]) == hi_b) atomicMax(&s_d, (int)threadIdx.x);
  __syncthreads();
  const int d = s_d;
  /* differences are OR-ed, not tested one by one, so that the loads are independent */
  unsigned diff = 0, sdiff = 0;
  if (sk == 1 && (sq & 3) == 0 && (reinterpret_cast<uintptr_t>(t) & 15) == 0) {
#pragma unroll 8
    for (int e = threadIdx.x; e < AT_BQ * AT_BK / 4; e += 256) {
      const int r = e / (AT_BK / 4), c = (e % (AT_BK / 4)) * 4;
      const uint4 v = *reinterpret_cast<const uint4 *>(t + (long long)r * sq + c);
      const unsigned f = __float_as_uint(first);
      diff |= (v.x ^ f) | (v.y ^ f) | (v.z ^ f) | (v.w ^ f);
      sdiff |= (v.x ^ (c - r > d ? lo_b : hi_b)) | (v.y ^ (c + 1 - r > d ? lo_b : hi_b)) |
               (v.z ^ (c + 2 - r > d ? lo_b : hi_b)) | (v.w ^ (c + 3 - r > d ? lo_b : hi_b));
    }
  } else {
#pragma unroll 8
    for (int e = threadIdx.x; e < AT_BQ * AT_BK; e += 256) {
      const int r = e / AT_BK, c = e % AT_BK;
      const unsigned v = __float_as_uint(t[(long long)r * sq + (long long)c * sk]);
      diff |= v ^ __float_as_uint(first);
      sdiff |= v ^ (c - r > d ? lo_b : hi_b);
    }
  }
  const bool same = diff == 0;
  const int all = __syncthreads_and(same ? 1 : 0);
  const int step = __syncthreads_and(sdiff == 0 ? 1 : 0);
  /* row maxima: a warp per row, 16 rows per warp */
  const int wid = threadIdx.x >> 5, ln = threadIdx.x & 31;
  float mx = __int_as_float(0x7f800000);               /* running min over this warp's rows */
  for (int r = wid; r < AT_BQ; r += 8) {
    const float *tr = t + (long long)r * sq;
    float m = __int_as_float(0xff800000); bool nan = false;
#pragma unroll
    for (int k = ln; k < AT_BK; k += 32) { const float v = tr[(long long)k * sk]; nan |= !(v == v); m = fmaxf(m, v); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o)); nan |= __shfl_xor_sync(0xffffffffu, nan ? 1 : 0, o) != 0; }
    if (nan) m = __int_as_float(0xff800000);
    mx = fminf(mx, m);
  }
  /* min over the 128 rows */
  __shared__ float s_min[8];
  if (ln == 0) s_min[wid] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = s_min[0];
    for (int i = 1; i < 8; i++) m = fminf(m, s_min[i]);
    float *rec = out + (long long)AT_REC * (qi * nk + ki);
    const float lo = __uint_as_float(lo_b), hi = __uint_as_float(hi_b);
    const bool is_const = all && first == first;
    rec[0] = is_const ? first : __int_as_float(0x7fc00000);
    rec[1] = m;
    /* a step tile has two different finite-or-infinite values (NaNs are left to the general path) */
    rec[2] = (!is_const && step && lo == lo && hi == hi && lo_b != hi_b) ? 2.0f : 0.0f;
    rec[3] = (float)d; rec[4] = lo; rec[5] = hi; rec[6] = 0.0f; rec[7] = 0.0f;
  }
}

/* Per (batch*head, block of 128 rows): an upper bound of the largest 2-norm of a row
 * of q and of k (bfloat16 rows of 64 through strides). */
struct BoundsArgs {
  const __nv_bfloat16 *q, *k; long long q_rs, k_rs, q_bs[3], k_bs[3];
  int nb, bext[3], nblk;
  float *qn, *kn;
};
__global__ void __launch_bounds__(128) pb200_attn_bounds(const BoundsArgs a) {
  const int blk = blockIdx.x % a.nblk, bh = blockIdx.x / a.nblk;
  long long oq = 0, ok = 0; int rem = bh;
  for (int i = 0; i < a.nb; i++) { const int x = rem % a.bext[i]; rem /= a.bext[i]; oq += x * a.q_bs[i]; ok += x * a.k_bs[i]; }
  /* 8 threads per row (16 bytes each: a row is one 128-byte line), 16 rows per pass */
  const int sub = threadIdx.x & 7, grp = threadIdx.x >> 3;
  float nq = 0.f, nk = 0.f;            /* largest squared norm seen by this thread's row group */
  /* all 16 loads of the thread in flight before the arithmetic */
  uint4 vqs[8], vks[8];
#pragma unroll
  for (int r = 0; r < 8; r++) {
    const long long row = (long long)blk * 128 + r * 16 + grp;
    vqs[r] = *reinterpret_cast<const uint4 *>(a.q + oq + row * a.q_rs + sub * 8);
    vks[r] = *reinterpret_cast<const uint4 *>(a.k + ok + row * a.k_rs + sub * 8);
  }
#pragma unroll
  for (int r = 0; r < 8; r++) {
    const uint4 vq = vqs[r], vk = vks[r];
    const uint32_t wq[4] = {vq.x, vq.y, vq.z, vq.w}, wk[4] = {vk.x, vk.y, vk.z, vk.w};
    float sq_ = 0.f, sk_ = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float q0 = __uint_as_float(wq[j] << 16), q1 = __uint_as_float(wq[j] & 0xffff0000u);
      const float k0 = __uint_as_float(wk[j] << 16), k1 = __uint_as_float(wk[j] & 0xffff0000u);
      sq_ = fmaf(q0, q0, fmaf(q1, q1, sq_)); sk_ = fmaf(k0, k0, fmaf(k1, k1, sk_));
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) { sq_ += __shfl_xor_sync(0xffffffffu, sq_, o); sk_ += __shfl_xor_sync(0xffffffffu, sk_, o); }
    nq = (nq != nq || sq_ != sq_) ? __int_as_float(0x7fc00000) : fmaxf(nq, sq_);
    nk = (nk != nk || sk_ != sk_) ? __int_as_float(0x7fc00000) : fmaxf(nk, sk_);
  }
  /* NaN rows give NaN norms, and a NaN bound never permits a skip */
  __shared__ float s_q[4], s_k[4];
  float mq = nq, mk = nk;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float oq2 = __shfl_xor_sync(0xffffffffu, mq, o), ok2 = __shfl_xor_sync(0xffffffffu, mk, o);
    mq = (mq != mq || oq2 != oq2) ? __int_as_float(0x7fc00000) : fmaxf(mq, oq2);
    mk = (mk != mk || ok2 != ok2) ? __int_as_float(0x7fc00000) : fmaxf(mk, ok2);
  }
  if ((threadIdx.x & 31) == 0) { s_q[threadIdx.x >> 5] = mq; s_k[threadIdx.x >> 5] = mk; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float x = s_q[0], y = s_k[0];
    for (int i = 1; i < 4; i++) {
      x = (x != x || s_q[i] != s_q[i]) ? __int_as_float(0x7fc00000) : fmaxf(x, s_q[i]);
      y = (y != y || s_k[i] != s_k[i]) ? __int_as_float(0x7fc00000) : fmaxf(y, s_k[i]);
    }
    /* rounded up: the sums above and the tensor cores' own accumulation round */
    a.qn[blockIdx.x] = sqrtf(x) * 1.001f;
    a.kn[blockIdx.x] = sqrtf(y) * 1.001f;
  }
}

/* ── host ────────────────────────────────────────────────────────────── */
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn attn_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) { void *lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL); if (lib) fn = (EncodeTiledFn)dlsym(lib, "cuTensorMapEncodeTiled"); }
  return fn;
}

/* bf16 rows of 64, `T` rows `row_stride` elements apart, batch axes bext[i] with strides bs[i] */
static int attn_map(CUtensorMap *map, const PbAttnOperand &op, long long T, int nb, const int *bext, int box_rows) {
  EncodeTiledFn enc = attn_encode();
  if (!enc) { pb_set_error("attention: cuTensorMapEncodeTiled not available"); return -1; }
  if ((reinterpret_cast<uintptr_t>(op.ptr) & 15) || op.row_stride % 8 || op.row_stride < AT_HD) {
    pb_set_error("attention: operand rows must be 16-byte aligned"); return -1;
  }
  cuuint64_t dims[5] = {AT_HD, (cuuint64_t)T, 1, 1, 1};
  cuuint64_t strides[4] = {(cuuint64_t)op.row_stride * 2, 0, 0, 0};
  cuuint64_t span = (cuuint64_t)T * (cuuint64_t)op.row_stride * 2;
  for (int i = 0; i < 3; i++) {
    if (i < nb) {
      if (op.bstride[i] <= 0 || op.bstride[i] % 8) { pb_set_error("attention: operand batch strides must be positive multiples of 8 elements"); return -1; }
      dims[2 + i] = (cuuint64_t)bext[i]; strides[1 + i] = (cuuint64_t)op.bstride[i] * 2;
      if (strides[1 + i] * dims[2 + i] > span) span = strides[1 + i] * dims[2 + i];
    } else strides[1 + i] = span;          /* an axis of extent 1: any 16-byte multiple */
  }
  cuuint32_t box[5] = {AT_HD, (cuuint32_t)box_rows, 1, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult rc = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void *>(op.ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) { pb_set_error("attention: cuTensorMapEncodeTiled failed (%d)", (int)rc); return -1; }
  return 0;
}

int pb_attention_error(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, pb200_attn_error_flag, sizeof v) != cudaSuccess) return -1;
  return v;
}

/* at most 64 key blocks: the set of processed blocks is a 64-bit mask */
bool pb_attention_supported(long long T, long long hd) { return hd == AT_HD && T >= AT_BK && T % AT_BK == 0 && T / AT_BK <= 64; }

/* q, k, v: bf16 through strides; mask fp32 [T x T] through strides; out fp32 or bf16 (out_bf16)
 * at element offsets Σ batch_i*o_sb[i] + row*o_sm + d. */
int pb_attention_launch(const PbAttnOperand &q, const PbAttnOperand &k, const PbAttnOperand &v,
                        const float *mask, long long mask_sq, long long mask_sk,
                        float scale, void *out, bool out_bf16, int nb, const int *bext, const long long *o_sb, long long o_sm,
                        long long BH, long long T, cudaStream_t stream, float *tiles_buf, int tiles_mode) {
  if (!pb_attention_supported(T, AT_HD)) { pb_set_error("attention: unsupported sequence length %lld", T); return -1; }
  if (nb > 3) { pb_set_error("attention: more than three batch axes"); return -1; }
  const int oal = out_bf16 ? 8 : 4;
  bool o_ok = (reinterpret_cast<uintptr_t>(out) & 15) == 0 && o_sm % oal == 0;
  for (int i = 0; i < nb; i++) if (o_sb[i] % oal) o_ok = false;
  if (!o_ok) { pb_set_error("attention: output rows must be 16-byte aligned"); return -1; }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(pb200_flash_attn, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(pb200_flash_attn2, cudaFuncAttributeMaxDynamicSharedMemorySize, AT2_SMEM);
    if (e != cudaSuccess) { pb_set_error("attention: cannot reserve shared memory: %s", cudaGetErrorString(e)); return -1; }
    configured = true;
  }
  /* POLY_B200_ATTN=1: the first arrangement (accumulators in registers) */
  const char *variant = getenv("POLY_B200_ATTN");
  const bool v1 = variant && variant[0] == '1';
  CUtensorMap mq, mk, mv;
  if (attn_map(&mq, q, T, nb, bext, AT_BQ) != 0) return -1;
  if (attn_map(&mk, k, T, nb, bext, AT_BK) != 0) return -1;
  if (attn_map(&mv, v, T, nb, bext, AT_BK) != 0) return -1;
  AttnArgs g{};
  g.O = (float *)out; g.out_bf16 = out_bf16 ? 1 : 0; g.mask = mask; g.mask_sq = mask_sq; g.mask_sk = mask_sk; g.scale = scale;
  g.T = (int)T; g.n_qblocks = (int)(T / AT_BQ);
  g.mask_vec = (mask_sk == 1 && mask_sq % 4 == 0 && (reinterpret_cast<uintptr_t>(mask) & 15) == 0) ? 1 : 0;
  g.nb = nb; g.o_sm = o_sm;
  for (int i = 0; i < nb; i++) { g.bext[i] = bext[i]; g.o_sb[i] = o_sb[i]; }
  long long grid = BH * g.n_qblocks;
  if (grid > 2147483647LL) { pb_set_error("attention: grid too large"); return -1; }
  const int nq = g.n_qblocks, nk = (int)(T / AT_BK);
  float *tiles = tiles_mode ? tiles_buf : (float *)pb_scratch_alloc((size_t)AT_REC * nq * nk * sizeof(float));
  if (!tiles) { pb_set_error("attention: out of scratch memory"); return -1; }
  /* bounds on |q.k| per block, for leaving out key blocks that cannot contribute (POLY_B200_ATTN_SKIP=0: never) */
  float *norms = nullptr;
  {
    const char *e = getenv("POLY_B200_ATTN_SKIP");
    if (!(e && e[0] == '0')) {
      norms = (float *)pb_scratch_alloc((size_t)2 * BH * nq * sizeof(float));
      if (!norms) { if (!tiles_mode) pb_scratch_free(tiles); pb_set_error("attention: out of scratch memory"); return -1; }
      BoundsArgs ba{};
      ba.q = (const __nv_bfloat16 *)q.ptr; ba.k = (const __nv_bfloat16 *)k.ptr; ba.q_rs = q.row_stride; ba.k_rs = k.row_stride;
      ba.nb = nb; ba.nblk = nq;
      for (int i = 0; i < nb; i++) { ba.bext[i] = bext[i]; ba.q_bs[i] = q.bstride[i]; ba.k_bs[i] = k.bstride[i]; }
      ba.qn = norms; ba.kn = norms + BH * nq;
      pb200_attn_bounds<<<(unsigned)(BH * nq), 128, 0, stream>>>(ba);
      g.qn = ba.qn; g.kn = ba.kn;
    }
  }
  if (tiles_mode != 2) pb200_mask_tiles<<<dim3((unsigned)nk, (unsigned)nq), 256, 0, stream>>>(mask, mask_sq, mask_sk, nk, tiles);
  g.tile_const = tiles;
  if (!tiles_mode) pb_scratch_free(tiles);   /* stream-ordered pool: safe to hand back once the work is enqueued */
  pb_scratch_free(norms);
  pb_tc_mark_used();
  pb_tc_configure_backoff();
  if (v1) pb200_flash_attn<<<(unsigned)grid, AT_THREADS, AT_SMEM, stream>>>(mq, mk, mv, g);
  else pb200_flash_attn2<<<(unsigned)grid, AT_THREADS, AT2_SMEM, stream>>>(mq, mk, mv, g);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { pb_set_error("attention launch: %s", cudaGetErrorString(e)); return -1; }
  return 0;
}

/* Direct entry: q, k, v float32 [B][T][H][64] (the layout GPT-2's projections
 * produce), mask float32 [T][T], out float32 [B][H][T][64]. */
extern "C" int poly_b200_attention(const float *q, const float *k, const float *v, const float *mask, float scale,
                                   float *out, int B, int H, int T) {
  if (poly_cuda_init() != 0) return -1;
  if (!q || !k || !v || !mask || !out || B <= 0 || H <= 0) { pb_set_error("poly_b200_attention: bad arguments"); return -1; }
  if (!pb_attention_supported(T, AT_HD)) { pb_set_error("poly_b200_attention: T must be a positive multiple of %d (head size %d)", AT_BK, AT_HD); return -1; }
  cudaStream_t stream = (cudaStream_t)poly_b200_stream();
  const long long BH = (long long)B * H, D = (long long)H * AT_HD;
  const size_t bytes = (size_t)BH * T * AT_HD * 2;
  if (pb_note_read(q) != 0 || pb_note_read(k) != 0 || pb_note_read(v) != 0 || pb_note_read(mask) != 0 ||
      pb_note_write(out, (size_t)BH * T * AT_HD * 4) != 0) return -1;
  void *qb = pb_scratch_alloc(bytes), *kb = pb_scratch_alloc(bytes), *vb = pb_scratch_alloc(bytes);
  int rc = -1;
  if (qb && kb && vb) {
    /* fp32 [b][t][h][d] -> bf16 in the same layout */
    const long long ext[2] = {D, (long long)B * T}, str[2] = {1, D};
    rc = pb_pack_launch(q, qb, 2, ext, str, PB_F32, PB_BF16, D, D, stream);
    if (rc == 0) rc = pb_pack_launch(k, kb, 2, ext, str, PB_F32, PB_BF16, D, D, stream);
    if (rc == 0) rc = pb_pack_launch(v, vb, 2, ext, str, PB_F32, PB_BF16, D, D, stream);
    const int bext[2] = {H, B};
    const long long o_sb[2] = {(long long)T * AT_HD, (long long)H * T * AT_HD};
    PbAttnOperand oq{qb, D, {AT_HD, (long long)T * D, 0}}, ok{kb, D, {AT_HD, (long long)T * D, 0}}, ov{vb, D, {AT_HD, (long long)T * D, 0}};
    if (rc == 0) rc = pb_attention_launch(oq, ok, ov, mask, T, 1, scale, out, false, 2, bext, o_sb, AT_HD, BH, T, stream);
    if (rc == 0) pb_count_launch(true, 4);
  } else pb_set_error("poly_b200_attention: out of scratch memory");
  pb_scratch_free(qb); pb_scratch_free(kb); pb_scratch_free(vb);
  return rc;
}


/* ── plan program: a recognised attention chain ──────────────────────── */
/* Header: "//kind attn", the two contractions of the chain under the key
 * prefixes "g1." (scores = q.kᵀ) and "g2." (out = p.v), the scale constant and
 * the mask's offset and strides.  Parameters: q, k, v, mask, out. */
struct AttnProgram : PbAotProgram {
  PbGemmProgram *g1 = nullptr, *g2 = nullptr;
  float scale = 1.0f;
  long long mask_off = 0, mask_sq = 0, mask_sk = 0;
  long long T = 0, BH = 0;
  bool qkv_bf16 = false;     /* q, k, v buffers hold bfloat16 and are read in place */
  bool out_bf16 = false;     /* out is written as bfloat16 */
  int tiles_mode = 0;        /* 1: the mask classification is computed into parameter 5, 2: read from it (same mask) */
  ~AttnProgram() override { delete g1; delete g2; }
  int n_launches() const override { return (qkv_bf16 ? 3 : 6) - (tiles_mode == 2 ? 1 : 0); }

  /* q/k/v as the contractions address them: rows of 64 contiguous values */
  void views(PbAttnOperand *q, PbAttnOperand *k, PbAttnOperand *v, void *const *bufs) const {
    const int nb = (int)g2->b_ax.size();
    *q = PbAttnOperand{(const __nv_bfloat16 *)bufs[0] + g1->off_a, g1->m_ax[0].sa, {0, 0, 0}};
    *k = PbAttnOperand{(const __nv_bfloat16 *)bufs[1] + g1->off_b, g1->n_ax[0].sb, {0, 0, 0}};
    *v = PbAttnOperand{(const __nv_bfloat16 *)bufs[2] + g2->off_b, g2->k_ax[0].sb, {0, 0, 0}};
    for (int i = 0; i < nb; i++) { q->bstride[i] = g1->b_ax[i].sa; k->bstride[i] = g1->b_ax[i].sb; v->bstride[i] = g2->b_ax[i].sb; }
  }
  bool views_ok() const {
    if (g1->k_ax.size() != 1 || g1->k_ax[0].sa != 1 || g1->k_ax[0].sb != 1 || g2->n_ax.size() != 1 || g2->n_ax[0].sb != 1) return false;
    if (g1->off_a % 8 || g1->off_b % 8 || g2->off_b % 8) return false;
    if (g1->m_ax[0].sa % 8 || g1->n_ax[0].sb % 8 || g2->k_ax[0].sb % 8) return false;
    if (g1->m_ax[0].sa < AT_HD || g1->n_ax[0].sb < AT_HD || g2->k_ax[0].sb < AT_HD) return false;
    for (size_t i = 0; i < g2->b_ax.size(); i++) {
      const long long s[3] = {g1->b_ax[i].sa, g1->b_ax[i].sb, g2->b_ax[i].sb};
      for (long long x : s) if (x <= 0 || x % 8) return false;
    }
    return true;
  }

  int launch(void *const *bufs, cudaStream_t stream) override {
    int bext[3]; long long o_sb[3];
    const int nb = (int)g2->b_ax.size();
    for (int i = 0; i < nb; i++) { bext[i] = (int)g2->b_ax[i].ext; o_sb[i] = g2->b_ax[i].sc; }
    const float *mask = (const float *)bufs[3] + mask_off;
    void *out = out_bf16 ? (void *)((__nv_bfloat16 *)bufs[4] + g2->off_c) : (void *)((float *)bufs[4] + g2->off_c);
    if (qkv_bf16) {
      PbAttnOperand q, k, v;
      views(&q, &k, &v, bufs);
      return pb_attention_launch(q, k, v, mask, mask_sq, mask_sk, scale, out, out_bf16, nb, bext, o_sb, g2->c_sm, BH, T, stream,
                                 tiles_mode ? (float *)bufs[5] : nullptr, tiles_mode);
    }
    /* fp32 operands: dense bf16 copies [batch][row][64] */
    const size_t bytes = (size_t)BH * T * AT_HD * 2;
    void *qb = pb_scratch_alloc(bytes), *kb = pb_scratch_alloc(bytes), *vb = pb_scratch_alloc(bytes);
    int rc = -1;
    if (qb && kb && vb) {
      rc = g1->pack_into(qb, bufs[0], g1->off_a, true, PB_F32, PB_BF16, AT_HD, stream);
      if (rc == 0) rc = g1->pack_into(kb, bufs[1], g1->off_b, false, PB_F32, PB_BF16, AT_HD, stream);
      if (rc == 0) {
        /* v as [batch][key][d]: axes d, key, batch (fastest first) */
        long long ext[PB_PACK_MAX_AXES], str[PB_PACK_MAX_AXES]; int na = 0;
        ext[na] = AT_HD; str[na++] = g2->n_ax[0].sb;
        ext[na] = T; str[na++] = g2->k_ax[0].sb;
        for (int i = 0; i < nb; i++) { ext[na] = g2->b_ax[i].ext; str[na++] = g2->b_ax[i].sb; }
        rc = pb_pack_launch((const float *)bufs[2] + g2->off_b, vb, na, ext, str, PB_F32, PB_BF16, AT_HD, AT_HD, stream);
      }
      /* dense copies: batch index = the same mixed radix as the output's */
      PbAttnOperand q{qb, AT_HD, {0, 0, 0}}, k{kb, AT_HD, {0, 0, 0}}, v{vb, AT_HD, {0, 0, 0}};
      long long bs = T * AT_HD;
      for (int i = 0; i < nb; i++) { q.bstride[i] = k.bstride[i] = v.bstride[i] = bs; bs *= bext[i]; }
      if (rc == 0)
        rc = pb_attention_launch(q, k, v, mask, mask_sq, mask_sk, scale, out, out_bf16, nb, bext, o_sb, g2->c_sm, BH, T, stream,
                                 tiles_mode ? (float *)bufs[5] : nullptr, tiles_mode);
    } else pb_set_error("attention: out of scratch memory");
    pb_scratch_free(qb); pb_scratch_free(kb); pb_scratch_free(vb);
    return rc;
  }
};

PbAotProgram *pb_make_attn(const PbHeader &h, std::string &err) {
  AttnProgram *p = new AttnProgram();
  p->g1 = pb_parse_gemm(h, "g1.", err);
  p->g2 = p->g1 ? pb_parse_gemm(h, "g2.", err) : nullptr;
  if (!p->g1 || !p->g2) { delete p; return nullptr; }
  PbGemmProgram &a = *p->g1, &b = *p->g2;
  bool ok = a.dtype == PB_F32 && b.dtype == PB_F32 && !a.has_x && !b.has_x && !a.relu && !b.relu;
  ok = ok && a.K == AT_HD && a.M == a.N && b.K == a.N && b.M == a.M && b.N == AT_HD && a.nbatch == b.nbatch;
  ok = ok && pb_attention_supported(a.M, a.K) && b.c_sn == 1 && b.c_sm % 4 == 0 && a.b_ax.size() == b.b_ax.size() && a.b_ax.size() <= 3;
  ok = ok && a.k_ax.size() == 1 && b.n_ax.size() == 1;
  /* the probabilities are read in the layout the scores were written in */
  ok = ok && a.c_sn == 1 && a.m_ax.size() == 1 && a.n_ax.size() == 1 && b.m_ax.size() == 1 && b.k_ax.size() == 1;
  if (ok) ok = b.m_ax[0].sa == a.c_sm && b.k_ax[0].sa == 1;
  for (size_t i = 0; ok && i < a.b_ax.size(); i++)
    ok = a.b_ax[i].ext == b.b_ax[i].ext && a.b_ax[i].sc == b.b_ax[i].sa && b.b_ax[i].sc % 4 == 0;
  if (!ok) { err = "attention chain does not have the supported shape"; delete p; return nullptr; }
  p->T = a.M; p->BH = a.nbatch;
  const std::string &sc = h.get("scale");
  unsigned bits = (unsigned)strtoul(sc.c_str(), nullptr, 16);
  memcpy(&p->scale, &bits, 4);
  auto m = h.getv("mask");
  if (m.size() != 3) { err = "malformed attention header"; delete p; return nullptr; }
  p->mask_off = m[0]; p->mask_sq = m[1]; p->mask_sk = m[2];
  p->qkv_bf16 = h.geti("qkv16") != 0;
  p->out_bf16 = h.geti("obf16") != 0;
  if (p->qkv_bf16 && !p->views_ok()) { err = "attention: operands cannot be read in place"; delete p; return nullptr; }
  if (p->out_bf16) {
    bool o8 = b.c_sm % 8 == 0 && b.off_c % 8 == 0;
    for (auto &ax : b.b_ax) if (ax.sc % 8) o8 = false;
    if (!o8) { err = "attention: bfloat16 output rows would not be 16-byte aligned"; delete p; return nullptr; }
  }
  p->n_params = 5;
  p->rw = "rrrr";
  p->rw.push_back(h.get("outmode") == "W" ? 'W' : 'w');
  p->tiles_mode = (int)h.geti("tiles");
  if (p->tiles_mode < 0 || p->tiles_mode > 2) { err = "malformed attention header"; delete p; return nullptr; }
  if (p->tiles_mode) { p->n_params = 6; p->rw.push_back(p->tiles_mode == 1 ? 'W' : 'r'); }
  return p;
}
