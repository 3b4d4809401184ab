/*
 * pb_gemm_tc.cu -- bf16 x bf16 -> fp32 contraction on the 5th-generation tensor
 * cores (tcgen05), operands staged by TMA, accumulators in tensor memory.
 *
 * Problem: C[b, m, n] = sum_k A[b, m, k] * B[b, n, k] (+ X) (relu), A and B
 * bfloat16 with k contiguous ("K-major"), C float32 row-major.
 * polygrad produces this either from bf16 buffers cast to float before the MUL,
 * or -- under POLY_B200_GEMM=bf16 -- from fp32 buffers whose values are rounded
 * to bf16 (nearest even) on the way in; products and sums stay fp32.
 *
 * One persistent CTA per SM, 10 warps, no clusters and no multicast:
 *   warp 0     allocates tensor memory; one lane issues the TMA loads
 *              (cp.async.bulk.tensor, 128-byte swizzle) into a ring of stages;
 *   warp 1     one lane issues tcgen05.mma (128 x BN x 16 per instruction, 4 per
 *              64-wide k block) and commits completion to the stage's "empty"
 *              barrier and, after the last k block, to the tile's "full" barrier;
 *   warps 2-9  epilogue: tcgen05.ld 32 lanes x 32 columns at a time (a thread gets
 *              32 consecutive values of one row), transposed through swizzled
 *              shared memory so that a warp writes 128 contiguous bytes of one
 *              row per store whatever the row pitch (a 50257-wide vocabulary has
 *              no 16-byte aligned rows); the addend and relu are applied on the
 *              way out.  Writing each thread's row as 128-bit stores straight
 *              from registers was measured and is slower (32 rows per store).
 * Two accumulator buffers in tensor memory let the MMA warp start the next tile
 * while the epilogue drains the previous one.
 *
 * For long K the same kernel runs as CTA pairs (template parameter CTAS = 2, a
 * cluster of two CTAs on neighbouring SMs): tcgen05.mma.cta_group::2 with M =
 * 256 computes a 256 x 256 tile, 128 rows in each CTA's tensor memory; each CTA
 * stages its own 128 rows of A and one half of the tile's B rows (the tensor
 * cores read both halves), so a stage is 32 KB instead of 48 and six fit.  The
 * first CTA of the pair issues the MMAs; both CTAs' TMA loads count their bytes
 * on its "full" barrier (cp.async.bulk.tensor.cta_group::2, no multicast), its
 * commits arrive on the "empty" and "accumulator full" barriers of both CTAs
 * (tcgen05.commit ... multicast::cluster), and the epilogue warps of both CTAs
 * arrive on its "accumulator empty" barrier through mapa / shared::cluster.
 *
 * Every wait on an mbarrier is bounded: after a few seconds without progress the
 * CTA records an error code, stops issuing work, frees its tensor memory and
 * returns; the host reports the code at the next synchronisation point.
 */
#include "pb_gemm.h"
#include "../../../include/poly_b200.h"
#include <cuda.h>
#include <dlfcn.h>
#include <cstdio>
#include <cstring>

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 320

__device__ int pb200_tc_error_flag = 0;

struct TcArgs {
  float *C; const float *X;
  int M, N, K;
  long long c_sm, x_sm, x_sn;
  int nb; int bext[4]; long long c_sb[4], x_sb[4];
  int has_x, relu;
  int ab_fmt;                      /* operand format: 0 float16, 1 bfloat16 (64 per 128-byte tile row), 2 tf32 (32 per row) */
  int vec_io;                      /* C rows (and addend rows) 16-byte aligned, N % 4 == 0 */
  int c_bf16;                      /* C holds bfloat16 (needs vec_io) */
  int gelu;                        /* tanh-GELU after the addend (bfloat16 results only) */
  int pack16;                      /* bfloat16 result, N and the row pitch multiples of 8, addend absent or one value per column:
                                      bias, activation and rounding happen in registers and the staged tile holds bfloat16 */
  int tiles_m, tiles_n, n_tiles;   /* n_tiles = nbatch * tiles_m * tiles_n */
  int m_fast;                      /* consecutive tiles differ in the row tile (else in the column tile) */
  int kchunk;                      /* PROMOTE kernels: k-blocks summed in tensor memory before the partial sum moves to registers */
  float alpha;                     /* PROMOTE kernels: the sum is scaled by this before the addend (a parameter update behind a gradient) */
  int stream_out;                  /* the result is far larger than L2: its stores are marked evict-first (unaligned float32 rows) */
};

#define PB_TC_ERROR_FLAG pb200_tc_error_flag
#include "pb_tc_ptx.cuh"

/* 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) with the hardware tanh approximation (relative
 * error about 2^-11); only used where the value is rounded to bfloat16 (2^-9) right afterwards. */
__device__ __forceinline__ float gelu_tanh_approx(float x) {
  const float u = x * fmaf(0.0356774081f, x * x, 0.7978845608f);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  const float h = 0.5f * x;
  return fmaf(h, t, h);
}

/* Shared-memory and global accesses of the epilogue by explicit state space (a pointer derived from the
 * dynamic shared-memory base is otherwise treated as generic, which costs address checks and keeps the
 * compiler from reordering loads of the staged tile around the global stores). */
__device__ __forceinline__ void sts_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t lds_b32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void stg_b32(void *p, uint32_t a) {
  asm volatile("st.global.b32 [%0], %1;" ::"l"(p), "r"(a) : "memory");
}
/* streaming store: the line is the first to leave L2 (a result far larger than L2 must not push the operands out) */
__device__ __forceinline__ void stg_b32_cs(void *p, uint32_t a) {
  asm volatile("st.global.cs.b32 [%0], %1;" ::"l"(p), "r"(a) : "memory");
}
__device__ __forceinline__ void stg_v4(void *p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

/* Tile t of a batch entry -> (row tile, column tile).  Consecutive tiles run at the
 * same time on different SMs; they walk along the axis of the SMALLER operand, so
 * that the larger one is streamed from memory once while the smaller one stays in
 * L2 (a 50257 x 768 vocabulary matrix against 8192 x 768 activations: the other
 * order re-reads the vocabulary once per row tile, 64 times). */
__device__ __forceinline__ void tile_coords(const TcArgs &g, int t, int *mt, int *nt) {
  const int in_batch = t % (g.tiles_n * g.tiles_m);
  if (g.m_fast) { *mt = in_batch % g.tiles_m; *nt = in_batch / g.tiles_m; }
  else { *nt = in_batch % g.tiles_n; *mt = in_batch / g.tiles_n; }
}

/* CTAS = 2: two CTAs on neighbouring SMs (a cluster of 2) work on one 256 x BN tile with
 * cta_group::2 MMAs; each holds its 128 rows of A and half of the tile's B rows. */
template <int BN, int CTAS>
struct TcSmem {
  static constexpr int STAGE_A = TC_BM * TC_BK * 2;
  static constexpr int STAGE_B = (BN / CTAS) * TC_BK * 2;
  static constexpr int STAGE = STAGE_A + STAGE_B;
  static constexpr int STAGES = CTAS == 2 ? (BN >= 192 ? 6 : 8) : ((BN == 256) ? 4 : (BN == 192 ? 4 : (BN == 128 ? 6 : 8)));
  static constexpr int EPI = 8 * 32 * 32 * 4;
  static constexpr int BYTES = STAGES * STAGE + EPI + 256 + 1024; /* + barriers + alignment slack */
};

template <int BN, int CTAS, bool PROMOTE = false, bool TF32 = false>
__global__ void __launch_bounds__(TC_THREADS, 1)
pb200_gemm_tc(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const TcArgs g) {
  using S = TcSmem<BN, CTAS>;
  static_assert(!PROMOTE || (CTAS == 1 && BN <= 128), "partial sums in registers: single CTAs, tiles up to 128 wide");
  /* CTA pair: rank within the pair, the pair's index and count (tiles are handed out per pair) */
  const uint32_t rank = CTAS == 2 ? cluster_ctarank() : 0u;
  const int unit = blockIdx.x / CTAS, n_units = gridDim.x / CTAS;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;              /* swizzled tiles need 1024-byte alignment */
  uint8_t *sm = smem_raw + (base - raw);
  float *epi = reinterpret_cast<float *>(sm + S::STAGES * S::STAGE);
  uint64_t *bars = reinterpret_cast<uint64_t *>(sm + S::STAGES * S::STAGE + S::EPI);
  /* bars: full[STAGES], empty[STAGES], tfull[2], tempty[2] */
  const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * S::STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * S::STAGES, bar_tempty = bar_tfull + 16;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int bk = TF32 ? TC_BK / 2 : TC_BK;           /* elements along k in one 128-byte tile row */
  const int kblocks = (g.K + bk - 1) / bk;
  /* two accumulator buffers; the allocation is a power of two */
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < S::STAGES; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
    /* the accumulator-empty barrier of the pair's first CTA collects the epilogue warps of both CTAs */
    for (int b = 0; b < 2; b++) { mbar_init(bar_tfull + 8 * b, 1); mbar_init(bar_tempty + 8 * b, 8 * CTAS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    if constexpr (CTAS == 2) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  /* the other CTA's barriers must exist before anything of this CTA signals them */
  if constexpr (CTAS == 2) cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    /* ── TMA producer ── */
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int t = unit; t < g.n_tiles && ok; t += n_units) {
        int nt, mt; const int bz = t / (g.tiles_n * g.tiles_m);
        tile_coords(g, t, &mt, &nt);
        for (int kb = 0; kb < kblocks; kb++) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, &abort_flag, 1)) { ok = false; break; }
          const uint32_t sa = base + stage * S::STAGE, sb = sa + S::STAGE_A;
          if constexpr (CTAS == 2) {
            /* both CTAs' bytes are counted on the first CTA's barrier, whose MMA thread waits for them */
            const uint32_t full0 = mapa_shared(bar_full + 8 * stage, 0);
            if (rank == 0) mbar_expect_tx(bar_full + 8 * stage, 2 * S::STAGE);
            tma_load_3d_pair(sa, &map_a, full0, kb * bk, (mt * 2 + (int)rank) * TC_BM, bz);
            tma_load_3d_pair(sb, &map_b, full0, kb * bk, nt * BN + (int)rank * (BN / 2), bz);
          } else {
            mbar_expect_tx(bar_full + 8 * stage, S::STAGE);
            tma_load_3d(sa, &map_a, bar_full + 8 * stage, kb * bk, mt * TC_BM, bz);
            tma_load_3d(sb, &map_b, bar_full + 8 * stage, kb * bk, nt * BN, bz);
          }
          if (++stage == S::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    /* ── MMA issuer ── */
    if (lane == 0 && rank == 0) {
      /* D float32; A and B float16 (format 0), bfloat16 (1) or tf32 (2, a compile-time variant), both
       * K-major.  A tile row is 128 bytes in every format and one instruction consumes 32 of them
       * (16 or 8 elements). */
      const uint32_t fmt = TF32 ? 2u : (uint32_t)g.ab_fmt;
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((TC_BM * CTAS) >> 4) << 24);
      uint32_t stage = 0, phase = 0, it = 0;
      bool ok = true;
      /* the four instructions of one k-block; `first` clears the accumulator */
      auto issue_block = [&](uint32_t tmem_d, bool first) {
        const uint32_t sa = base + stage * S::STAGE, sb = sa + S::STAGE_A;
        const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sb);
#pragma unroll
        for (int k = 0; k < TC_BK / 16; k++) {
          const uint32_t accum = (!first || k) ? 1u : 0u;
          if constexpr (CTAS == 2) {
            if constexpr (TF32) tc_mma_tf32_pair(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
            else tc_mma_bf16_pair(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
          } else {
            if constexpr (TF32) tc_mma_tf32(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
            else tc_mma_bf16(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
          }
        }
        /* frees the stage (in both CTAs of a pair) when these MMAs have read it */
        if constexpr (CTAS == 2) tc_commit_pair(bar_empty + 8 * stage, 3); else tc_commit(bar_empty + 8 * stage);
        if (++stage == S::STAGES) { stage = 0; phase ^= 1u; }
      };
      if constexpr (!PROMOTE) {
        /* one accumulator buffer per tile */
        for (int t = unit; t < g.n_tiles && ok; t += n_units, it++) {
          const uint32_t buf = it & 1u, use = it >> 1;
          if (!mbar_wait(bar_tempty + 8 * buf, (use & 1u) ^ 1u, &abort_flag, 2)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t tmem_d = tmem_base + buf * BN;
          for (int kb = 0; kb < kblocks; kb++) {
            if (!mbar_wait(bar_full + 8 * stage, phase, &abort_flag, 3)) { ok = false; break; }
            tc_fence_after_sync();
            issue_block(tmem_d, kb == 0);
          }
          if (ok) { if constexpr (CTAS == 2) tc_commit_pair(bar_tfull + 8 * buf, 3); else tc_commit(bar_tfull + 8 * buf); }   /* accumulator complete */
        }
      } else {
        /* one accumulator buffer per chunk of g.kchunk k-blocks: the epilogue warps add each chunk's
         * sum to registers (rounded float32 adds), because the tensor cores' own accumulation
         * truncates and would drift over a long k axis */
        for (int t = unit; t < g.n_tiles && ok; t += n_units) {
          for (int kb0 = 0; kb0 < kblocks && ok; kb0 += g.kchunk, it++) {
            const uint32_t buf = it & 1u, use = it >> 1;
            if (!mbar_wait(bar_tempty + 8 * buf, (use & 1u) ^ 1u, &abort_flag, 2)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t tmem_d = tmem_base + buf * BN;
            const int kend = min(kb0 + g.kchunk, kblocks);
            for (int kb = kb0; kb < kend; kb++) {
              if (!mbar_wait(bar_full + 8 * stage, phase, &abort_flag, 3)) { ok = false; break; }
              tc_fence_after_sync();
              issue_block(tmem_d, kb == kb0);
            }
            if (ok) tc_commit(bar_tfull + 8 * buf);
          }
        }
      }
    }
  } else {
    /* ── epilogue: 8 warps; warp w reads tensor-memory lanes 32*(w%4) .. +31 (the
     * hardware ties a warp to that quarter) and one half of the tile's columns ── */
    const int q = warp & 3, half = (warp - 2) >> 2;
    float *stg = epi + (warp - 2) * 32 * 32;
    /* addresses into this warp's 4 KB staging tile, fixed for the whole kernel.  float32 tile: 32 rows x 128 B,
     * thread `lane` writes row `lane` (16-byte chunk c at c ^ (lane & 7)) and reads, in pass i8, row i8*4 + lane/8,
     * chunk lane%8.  bfloat16 tile: 32 rows x 64 B, chunk c of row r at c ^ ((r >> 1) & 3); pass i4 reads row
     * i4*8 + lane/4, chunk lane%4.  Bytes 2048.. of the tile hold the bias of the warp's 128 columns then. */
    const uint32_t stg_s = smem_u32(stg);
    const uint32_t wr32 = stg_s + lane * 128, wr16 = stg_s + lane * 64;
    const uint32_t rd32_a = stg_s + (lane >> 3) * 128 + (((lane & 7) ^ (lane >> 3)) << 4);          /* passes with even i8 */
    const uint32_t rd32_b = stg_s + (4 + (lane >> 3)) * 128 + (((lane & 7) ^ (4 + (lane >> 3))) << 4); /* odd i8 */
    const uint32_t rd16 = stg_s + (lane >> 2) * 64 + (((lane & 3) ^ ((lane >> 3) & 3)) << 4);       /* (row >> 1) & 3 does not depend on the pass */
    uint32_t it = 0;
    bool ok = true;
    for (int t = unit; t < g.n_tiles && ok; t += n_units) {
      int nt, mt;
      tile_coords(g, t, &mt, &nt);
      int bz = t / (g.tiles_n * g.tiles_m);
      long long oc = 0, ox = 0;
      for (int i = 0; i < g.nb; i++) { const int x = bz % g.bext[i]; bz /= g.bext[i]; oc += x * g.c_sb[i]; ox += x * g.x_sb[i]; }
      constexpr int NCH = (BN / 2) / 32;
      const int colh = nt * BN + half * (BN / 2);
      const int row0 = (mt * CTAS + (int)rank) * TC_BM + q * 32;
      const int rows = min(32, g.M - row0);
      float *__restrict__ C = g.C + oc;
      const float *__restrict__ X = g.has_x ? g.X + ox : nullptr;
      const bool x_bcast = X && g.x_sm == 0;       /* bias: one value per column */
      /* float32 result with a bias: this lane's four bias values of every 32-column chunk, fetched before the
       * accumulator is waited for */
      [[maybe_unused]] float4 xb4[NCH];
      if (x_bcast && g.vec_io && !g.c_bf16) {
#pragma unroll
        for (int ci = 0; ci < NCH; ci++) {
          const int n = colh + ci * 32 + (lane & 7) * 4;
          xb4[ci] = n < g.N ? __ldg(reinterpret_cast<const float4 *>(X + n)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      if (g.pack16 && X) {
        /* the bias of this warp's columns, once per tile, beside the staged tile (all lanes read the same
         * 16 bytes at a time later: a broadcast) */
        float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
        if (lane * 4 < BN / 2 && colh + lane * 4 < g.N) b = __ldg(reinterpret_cast<const float4 *>(X + colh + lane * 4));
        sts_v4(stg_s + 2048 + lane * 16, __float_as_uint(b.x), __float_as_uint(b.y), __float_as_uint(b.z), __float_as_uint(b.w));
        __syncwarp();
      }
      uint32_t buf = 0;
      [[maybe_unused]] float acc[PROMOTE ? NCH : 1][32];
      if constexpr (PROMOTE) {
        /* the tile arrives as partial sums over g.kchunk k-blocks each; add them up here */
#pragma unroll
        for (int ci = 0; ci < NCH; ci++)
#pragma unroll
          for (int j = 0; j < 32; j++) acc[ci][j] = 0.0f;
        for (int kb0 = 0; kb0 < kblocks && ok; kb0 += g.kchunk, it++) {
          buf = it & 1u;
          if (!mbar_wait(bar_tfull + 8 * buf, (it >> 1) & 1u, &abort_flag, 4)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t tb = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + half * (BN / 2);
#pragma unroll
          for (int ci = 0; ci < NCH; ci++) {
            if (colh + ci * 32 < g.N) {
              uint32_t part[32];
              tc_ld32(tb + ci * 32, part);
              tc_wait_ld();
#pragma unroll
              for (int j = 0; j < 32; j++) acc[ci][j] += __uint_as_float(part[j]);
            }
          }
          tc_fence_before_sync();
          if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
        }
        if (!ok) break;
      } else {
        buf = it & 1u;
        const uint32_t use = it >> 1;
        it++;
        if (!mbar_wait(bar_tfull + 8 * buf, use & 1u, &abort_flag, 4)) { ok = false; break; }
        tc_fence_after_sync();
      }
      /* chunks of 32 columns; the tensor-memory load of the next chunk is in
       * flight while this one is transposed and stored */
      const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + half * (BN / 2);
      [[maybe_unused]] uint32_t r[PROMOTE ? 1 : 2][32];
      /* the value of column j of chunk ci: from registers (PROMOTE) or from the load in flight */
      auto val = [&](int ci, int j) -> float {
        if constexpr (PROMOTE) return acc[ci][j] * g.alpha; else return __uint_as_float(r[ci & 1][j]);
      };
      if constexpr (!PROMOTE) { if (colh < g.N) tc_ld32(tbase, r[0]); }
#pragma unroll
      for (int ci = 0; ci < NCH; ci++) {
        const int col0 = colh + ci * 32;
        if (col0 < g.N) {
          if constexpr (!PROMOTE) {
            tc_wait_ld();
            if (ci + 1 < NCH && col0 + 32 < g.N) tc_ld32(tbase + (ci + 1) * 32, r[(ci + 1) & 1]);
          }
          if (g.pack16) {
            /* bfloat16 result: the thread's 32 values of its row get bias, activation and rounding here, in
             * registers, and the staged tile is 32 rows x 64 bytes -- half the shared-memory traffic of staging
             * float32 and converting on the way out. */
            uint32_t w[16];
#pragma unroll
            for (int j4 = 0; j4 < 8; j4++) {
              float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
              if (X) { const uint4 u = lds_v4(stg_s + 2048 + (ci * 8 + j4) * 16); b4 = make_float4(__uint_as_float(u.x), __uint_as_float(u.y), __uint_as_float(u.z), __uint_as_float(u.w)); }
              float v0 = val(ci, j4 * 4) + b4.x, v1 = val(ci, j4 * 4 + 1) + b4.y, v2 = val(ci, j4 * 4 + 2) + b4.z, v3 = val(ci, j4 * 4 + 3) + b4.w;
              if (g.relu) { v0 = (0.f < v0) ? v0 : 0.f; v1 = (0.f < v1) ? v1 : 0.f; v2 = (0.f < v2) ? v2 : 0.f; v3 = (0.f < v3) ? v3 : 0.f; }
              if (g.gelu) { v0 = gelu_tanh_approx(v0); v1 = gelu_tanh_approx(v1); v2 = gelu_tanh_approx(v2); v3 = gelu_tanh_approx(v3); }
              const __nv_bfloat162 lo = __floats2bfloat162_rn(v0, v1), hi = __floats2bfloat162_rn(v2, v3);
              w[j4 * 2] = *reinterpret_cast<const uint32_t *>(&lo); w[j4 * 2 + 1] = *reinterpret_cast<const uint32_t *>(&hi);
            }
            const uint32_t sw = (lane >> 1) & 3;
#pragma unroll
            for (int c = 0; c < 4; c++) sts_v4(wr16 + ((c ^ sw) << 4), w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
            __syncwarp();
            const int n = col0 + (lane & 3) * 8;
            if (n < g.N) {
              uint4 v[4];
#pragma unroll
              for (int i4 = 0; i4 < 4; i4++) v[i4] = lds_v4(rd16 + i4 * 512);
              __nv_bfloat16 *cb = reinterpret_cast<__nv_bfloat16 *>(g.C) + (C - g.C) + (long long)(row0 + (lane >> 2)) * g.c_sm + n;
              const long long cstep = 8 * g.c_sm;
#pragma unroll
              for (int i4 = 0; i4 < 4; i4++) {
                if (i4 * 8 + (lane >> 2) < rows) stg_v4(cb, v[i4].x, v[i4].y, v[i4].z, v[i4].w);
                cb += cstep;
              }
            }
          } else if (g.vec_io && !g.c_bf16 && (!X || x_bcast)) {
            /* float32 result, no addend or one value per column: the staged 32 x 32 tile is read back with all
             * eight loads in flight, then bias / relu and eight 128-bit stores of 4 rows x 128 B each */
#pragma unroll
            for (int c = 0; c < 8; c++)
              sts_v4(wr32 + ((c ^ (lane & 7)) << 4), __float_as_uint(val(ci, c * 4)), __float_as_uint(val(ci, c * 4 + 1)),
                     __float_as_uint(val(ci, c * 4 + 2)), __float_as_uint(val(ci, c * 4 + 3)));
            __syncwarp();
            const int n = col0 + (lane & 7) * 4;
            if (n < g.N) {
              uint4 v[8];
#pragma unroll
              for (int i8 = 0; i8 < 8; i8++) v[i8] = lds_v4(((i8 & 1) ? rd32_b : rd32_a) + (i8 >> 1) * 1024);
              const float4 xb = X ? xb4[ci] : make_float4(0.f, 0.f, 0.f, 0.f);
              float *cp = C + (long long)(row0 + (lane >> 3)) * g.c_sm + n;
              const long long cstep = 4 * g.c_sm;
#pragma unroll
              for (int i8 = 0; i8 < 8; i8++) {
                float a0 = __uint_as_float(v[i8].x) + xb.x, a1 = __uint_as_float(v[i8].y) + xb.y, a2 = __uint_as_float(v[i8].z) + xb.z, a3 = __uint_as_float(v[i8].w) + xb.w;
                if (g.relu) { a0 = (0.f < a0) ? a0 : 0.f; a1 = (0.f < a1) ? a1 : 0.f; a2 = (0.f < a2) ? a2 : 0.f; a3 = (0.f < a3) ? a3 : 0.f; }
                if (i8 * 4 + (lane >> 3) < rows) stg_v4(cp, __float_as_uint(a0), __float_as_uint(a1), __float_as_uint(a2), __float_as_uint(a3));
                cp += cstep;
              }
            }
          } else if (g.vec_io) {
            /* rows of C (and of the addend) are 16-byte aligned: 128-bit shared and
             * global accesses, 16-byte chunks XOR-swizzled by row so that both the
             * row-per-thread writes and the 4-rows-per-warp reads are conflict-free */
            float4 *stg4 = reinterpret_cast<float4 *>(stg);
#pragma unroll
            for (int c4 = 0; c4 < 8; c4++)
              stg4[lane * 8 + (c4 ^ (lane & 7))] = make_float4(val(ci, c4 * 4), val(ci, c4 * 4 + 1), val(ci, c4 * 4 + 2), val(ci, c4 * 4 + 3));
            __syncwarp();
            const int c4 = lane & 7, rsub = lane >> 3;
            const int n = col0 + c4 * 4;
            if (n < g.N) {
              float4 xb = make_float4(0.f, 0.f, 0.f, 0.f);
              if (x_bcast) xb = *reinterpret_cast<const float4 *>(X + n);
              float *cp = C + (long long)(row0 + rsub) * g.c_sm + n;
              const float *xp = (X && !x_bcast) ? X + (long long)(row0 + rsub) * g.x_sm + n : nullptr;
              const long long cstep = 4 * g.c_sm, xstep = 4 * g.x_sm;
#pragma unroll
              for (int i8 = 0; i8 < 8; i8++) {
                const int rr = i8 * 4 + rsub;
                if (rr < rows) {
                  float4 v = stg4[rr * 8 + (c4 ^ (rr & 7))];
                  if (xp) { const float4 x4 = *reinterpret_cast<const float4 *>(xp); v.x += x4.x; v.y += x4.y; v.z += x4.z; v.w += x4.w; }
                  else { v.x += xb.x; v.y += xb.y; v.z += xb.z; v.w += xb.w; }
                  if (g.relu) { v.x = (0.f < v.x) ? v.x : 0.f; v.y = (0.f < v.y) ? v.y : 0.f; v.z = (0.f < v.z) ? v.z : 0.f; v.w = (0.f < v.w) ? v.w : 0.f; }
                  if (g.c_bf16) {
                    if (g.gelu) { v.x = gelu_tanh_approx(v.x); v.y = gelu_tanh_approx(v.y); v.z = gelu_tanh_approx(v.z); v.w = gelu_tanh_approx(v.w); }
                    /* same element offset, 2-byte elements */
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                    uint2 w; w.x = *reinterpret_cast<const uint32_t *>(&lo); w.y = *reinterpret_cast<const uint32_t *>(&hi);
                    *reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(g.C) + (cp - g.C)) = w;
                  } else
                  *reinterpret_cast<float4 *>(cp) = v;
                }
                cp += cstep;
                if (xp) xp += xstep;
              }
            }
          } else if (!g.c_bf16 && (!X || x_bcast)) {
            /* float32 result whose rows are not 16-byte aligned (a 50257-wide vocabulary): staged like the aligned
             * tile, read back a row per pass with lane = column, eight rows' loads in flight at a time; a warp's
             * store is 128 contiguous bytes of one row */
#pragma unroll
            for (int c = 0; c < 8; c++)
              sts_v4(wr32 + ((c ^ (lane & 7)) << 4), __float_as_uint(val(ci, c * 4)), __float_as_uint(val(ci, c * 4 + 1)),
                     __float_as_uint(val(ci, c * 4 + 2)), __float_as_uint(val(ci, c * 4 + 3)));
            __syncwarp();
            const int n = col0 + lane;
            if (n < g.N) {
              const float xb = X ? X[(long long)n * g.x_sn] : 0.0f;
              float *cp = C + (long long)row0 * g.c_sm + n;
              const uint32_t rd = stg_s + (lane & 3) * 4, hi = (uint32_t)lane >> 2;
#pragma unroll
              for (int r8 = 0; r8 < 4; r8++) {
                uint32_t v[8];
#pragma unroll
                for (int i = 0; i < 8; i++) v[i] = lds_b32(rd + (r8 * 8 + i) * 128 + ((hi ^ (uint32_t)i) << 4));   /* word `lane` of row r8*8+i */
#pragma unroll
                for (int i = 0; i < 8; i++) {
                  float a = __uint_as_float(v[i]) + xb;
                  if (g.relu) a = (0.f < a) ? a : 0.f;
                  if (r8 * 8 + i < rows) { if (g.stream_out) stg_b32_cs(cp, __float_as_uint(a)); else stg_b32(cp, __float_as_uint(a)); }
                  cp += g.c_sm;
                }
              }
            }
          } else {
#pragma unroll
          for (int j = 0; j < 32; j++) stg[lane * 32 + (j ^ lane)] = val(ci, j);
          __syncwarp();
          const int n = col0 + lane;
          if (n < g.N) {
            const float xb = x_bcast ? X[(long long)n * g.x_sn] : 0.0f;
            float *cp = C + (long long)row0 * g.c_sm + n;
            const float *xp = (X && !x_bcast) ? X + (long long)row0 * g.x_sm + (long long)n * g.x_sn : nullptr;
            for (int rr = 0; rr < rows; rr++) {
              float v = stg[rr * 32 + (lane ^ rr)];
              if (xp) v = v + xp[(long long)rr * g.x_sm]; else v = v + xb;
              if (g.relu) v = (0.0f < v) ? v : 0.0f;
              cp[(long long)rr * g.c_sm] = v;
            }
          }
          }
          __syncwarp();
        }
      }
      if constexpr (!PROMOTE) {
        tc_fence_before_sync();
        if (lane == 0) {
          if constexpr (CTAS == 2) mbar_arrive_cluster(mapa_shared(bar_tempty + 8 * buf, 0));
          else mbar_arrive(bar_tempty + 8 * buf);
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (abort_flag) {
    /* let copies that were already issued land before the shared memory goes away */
    for (int i = 0; i < 2000; i++) __nanosleep(1000);
  }
  /* neither CTA of a pair leaves while the other may still signal its barriers or read its tiles */
  if constexpr (CTAS == 2) cluster_sync_all();
  if (warp == 0) {
    tc_fence_after_sync();
    if constexpr (CTAS == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

/* Self-test of the bounded wait: one thread waits on a barrier that nothing ever arrives at,
 * with a short limit; it must give up, record its code in the error word and return. */
#define TC_PROBE_CODE 90
__global__ void pb200_wait_probe(int *gave_up) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_flag, TC_PROBE_CODE, 1u << 14);
    *gave_up = ok ? 0 : 1;
  }
}

extern "C" int poly_b200_selftest_bounded_wait(void) {
  if (poly_cuda_init() != 0) return -1;
  cudaStream_t stream = (cudaStream_t)poly_b200_stream();
  int *flag = (int *)pb_scratch_alloc(sizeof(int));
  if (!flag) { pb_set_error("selftest: out of scratch memory"); return -1; }
  int zero = 0, gave_up = -1, code = -1;
  cudaError_t e = cudaMemcpyAsync(flag, &zero, sizeof zero, cudaMemcpyHostToDevice, stream);
  if (e == cudaSuccess) { pb200_wait_probe<<<1, 32, 0, stream>>>(flag); e = cudaGetLastError(); }
  if (e == cudaSuccess) e = cudaMemcpyAsync(&gave_up, flag, sizeof gave_up, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  pb_scratch_free(flag);
  if (e != cudaSuccess) { pb_set_error("selftest: %s", cudaGetErrorString(e)); return -1; }
  /* the wait's code must be in the error word; clear it again so that later work is not reported as failed */
  if (cudaMemcpyFromSymbol(&code, pb200_tc_error_flag, sizeof code) != cudaSuccess) { pb_set_error("selftest: cannot read the error word"); return -1; }
  if (cudaMemcpyToSymbol(pb200_tc_error_flag, &zero, sizeof zero) != cudaSuccess) { pb_set_error("selftest: cannot clear the error word"); return -1; }
  if (gave_up != 1 || code != TC_PROBE_CODE) { pb_set_error("selftest: bounded wait did not report (gave_up %d, code %d)", gave_up, code); return -1; }
  return 0;
}

/* ── host side ───────────────────────────────────────────────────────── */
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (lib) fn = (EncodeTiledFn)dlsym(lib, "cuTensorMapEncodeTiled");
  }
  return fn;
}

/* rows x K bf16, K contiguous, row pitch `pitch` elements, `nbatch` matrices `bpitch` elements apart */
static int make_map(CUtensorMap *map, const void *ptr, long long K, long long rows, long long nbatch,
                    long long pitch, long long bpitch, int box_rows, int fmt = 1) {
  EncodeTiledFn enc = encode_tiled();
  if (!enc) { pb_set_error("gemm: cuTensorMapEncodeTiled not available"); return -1; }
  cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)nbatch};
  const cuuint64_t esz = fmt == 2 ? 4 : 2;
  cuuint64_t strides[2] = {(cuuint64_t)pitch * esz, (cuuint64_t)(nbatch > 1 ? bpitch : rows * pitch) * esz};
  cuuint32_t box[3] = {(cuuint32_t)(fmt == 2 ? TC_BK / 2 : TC_BK), (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = fmt == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : fmt == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUresult rc = enc(map, dt, 3, const_cast<void *>(ptr),
                    dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) { pb_set_error("gemm: cuTensorMapEncodeTiled failed (%d)", (int)rc); return -1; }
  return 0;
}

/* One-time set-up of a kernel variant (the runtime drives one device per process). */
template <int BN, int CTAS, bool PROMOTE = false, bool TF32 = false>
static int tc_configure() {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(pb200_gemm_tc<BN, CTAS, PROMOTE, TF32>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmem<BN, CTAS>::BYTES);
    if (e != cudaSuccess) { pb_set_error("gemm: cannot reserve %d bytes of shared memory: %s", TcSmem<BN, CTAS>::BYTES, cudaGetErrorString(e)); return -1; }
    configured = true;
  }
  return 0;
}

static int sm_count() {
  static int sms = 0;
  if (!sms) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); if (sms <= 0) sms = 148; }
  return sms;
}

template <int BN, int CTAS, bool PROMOTE = false, bool TF32 = false>
static int tc_launch(const CUtensorMap &ma, const CUtensorMap &mb, TcArgs &g, long long nbatch, cudaStream_t stream) {
  if (tc_configure<BN, CTAS, PROMOTE, TF32>() != 0) return -1;
  g.tiles_m = (g.M + TC_BM * CTAS - 1) / (TC_BM * CTAS);
  g.tiles_n = (g.N + BN - 1) / BN;
  long long tiles = (long long)g.tiles_m * g.tiles_n * nbatch;
  if (tiles > 2147483647LL) { pb_set_error("gemm: too many tiles"); return -1; }
  g.n_tiles = (int)tiles;
  g.m_fast = g.N > g.M ? 1 : 0;
  {
    const char *e = getenv("POLY_B200_TC_STREAM");           /* "0": ordinary stores (measurements) */
    g.stream_out = !(e && e[0] == '0') && (double)g.M * (double)g.N * (double)nbatch * 4.0 >= 512.0 * 1024 * 1024;
  }
  const int units = sm_count() / CTAS;
  const int grid = (int)(tiles < units ? tiles : units) * CTAS;
  cudaError_t e;
  if (CTAS == 1) {
    pb200_gemm_tc<BN, CTAS, PROMOTE, TF32><<<grid, TC_THREADS, TcSmem<BN, CTAS>::BYTES, stream>>>(ma, mb, g);
    e = cudaGetLastError();
  } else {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(TC_THREADS); cfg.dynamicSmemBytes = TcSmem<BN, CTAS>::BYTES; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTAS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, pb200_gemm_tc<BN, CTAS, PROMOTE, TF32>, ma, mb, g);
  }
  if (e != cudaSuccess) { pb_set_error("tensor-core gemm launch: %s", cudaGetErrorString(e)); return -1; }
  return 0;
}

int pb_gemm_tc_error(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, pb200_tc_error_flag, sizeof v) != cudaSuccess) return -1;
  return v;
}

/* K-major bf16 copy of operand A or B: [nbatch][rows][Kp], Kp = K rounded up to 8
 * (TMA wants 16-byte row pitches; the box never reads past K, so the tail is
 * never used).  An operand whose buffer version did not change since the last
 * call (weights) is served from the program's cache; one that changes on every
 * call (activations) is converted into pool scratch that the caller frees. */
static const void *tc_operand(PbGemmProgram &p, PbTcOperand &cache, const void *src_buf, long long off, bool is_a,
                              long long rows, long long Kp, cudaStream_t stream, void **scratch) {
  *scratch = nullptr;
  const size_t bytes = (size_t)(p.nbatch * rows * Kp) * 2;
  const uint64_t ver = pb_buffer_version(src_buf);
  if (cache.data && cache.src == src_buf && cache.version == ver && cache.bytes == bytes && ver != 0) return cache.data;
  const bool transient = cache.misses >= 2 || ver == 0;
  void *dst;
  if (transient) {
    if (cache.data) { pb_scratch_free(cache.data); cache.data = nullptr; cache.bytes = 0; }
    dst = pb_scratch_alloc(bytes);
    if (!dst) return nullptr;
    *scratch = dst;
  } else {
    if (cache.data && cache.bytes != bytes) { pb_scratch_free(cache.data); cache.data = nullptr; }
    if (!cache.data) { cache.data = pb_scratch_alloc(bytes); cache.bytes = bytes; }
    if (!cache.data) return nullptr;
    dst = cache.data;
    cache.src = src_buf; cache.version = ver; cache.misses++;
  }
  if (p.pack_into(dst, src_buf, off, is_a, p.dtype, p.dtype == PB_F16 ? PB_F16 : PB_BF16, Kp, stream) != 0) {
    if (*scratch) { pb_scratch_free(*scratch); *scratch = nullptr; }
    return nullptr;
  }
  return dst;
}

/* ── fp32 contractions on the tensor cores: three tf32 products ─────────
 * a = hi + lo with hi = tf32(a), lo = tf32(a - hi) carries 22 bits of a's
 * mantissa; a.b ~ hi.hi + hi.lo + lo.hi leaves out terms of relative size
 * 2^-22.  The three products are one contraction over a k axis three times as
 * long: A' = [hi | hi | lo], B' = [hi | lo | hi], each segment Kp = K rounded up
 * to 4 elements (16-byte rows) and zero-filled past K.  Accumulation is fp32 in
 * TMEM, which truncates: summed over the whole k axis there, the error against
 * a float64 product is about 1e-8 * K of the result's rms (a CPU float32 sum:
 * 2e-7 to 4e-7).  The PROMOTE kernels therefore hand the partial sum of every
 * few k-blocks to the epilogue warps, which add them up in registers; that
 * keeps the error at the CPU's level for every K and is the float32 default. */
__device__ __forceinline__ float tf32_rna(float a) {
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(a));
  return __uint_as_float(u);
}

struct SplitSrc {                      /* the source as [batch axes][rows][k], k contiguous */
  const float *src; long long pitch; long long rows;
  int nb; int bext[4]; long long bstr[4];
};

/* one value into its three segments: x0 goes to [0, Kp), x1 to [Kp, 2Kp), x2 to [2Kp, 3Kp) */
__device__ __forceinline__ void split_one(float a, int is_b, float &x0, float &x1, float &x2) {
  if (!(fabsf(a) <= 3.4028235e38f)) {
    /* an infinity or a NaN meets only the other operand's hi part, once: inf * b keeps b's sign
     * (and inf * 0 is NaN) as in the plain product, instead of meeting lo parts of either sign */
    x0 = a; x1 = 0.0f; x2 = 0.0f;
    return;
  }
  float hi = tf32_rna(a);
  if (!(fabsf(hi) <= 3.4028235e38f)) hi = __uint_as_float(__float_as_uint(a) & 0xffffe000u);   /* rounding overflowed: truncate */
  const float lo = tf32_rna(a - hi);
  x0 = hi; x1 = is_b ? lo : hi; x2 = is_b ? hi : lo;
}

__global__ void __launch_bounds__(256) pb200_split_tf32x3(const SplitSrc in, float *__restrict__ dst,
                                                          long long total, int K, int Kp, int is_b) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / Kp; const int k = (int)(i % Kp);
    long long bz = row / in.rows, so = (row % in.rows) * in.pitch;
    for (int d = 0; d < in.nb; d++) { so += (bz % in.bext[d]) * in.bstr[d]; bz /= in.bext[d]; }
    const float a = k < K ? in.src[so + k] : 0.0f;
    float *o = dst + row * 3 * Kp;
    split_one(a, is_b, o[k], o[Kp + k], o[2 * Kp + k]);
  }
}

/* The same with four consecutive k per thread: one 128-bit load, three 128-bit stores.  Needs rows of the
 * source that start on 16-byte boundaries (Kp is a multiple of 4, so the destination's always do). */
__global__ void __launch_bounds__(256) pb200_split_tf32x3_v4(const SplitSrc in, float *__restrict__ dst,
                                                             long long total4, int K, int Kp, int is_b) {
  const int kq = Kp >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / kq; const int k = (int)(i % kq) << 2;
    long long bz = row / in.rows, so = (row % in.rows) * in.pitch;
    for (int d = 0; d < in.nb; d++) { so += (bz % in.bext[d]) * in.bstr[d]; bz /= in.bext[d]; }
    float4 a;
    if (k + 3 < K) a = *reinterpret_cast<const float4 *>(in.src + so + k);
    else {
      a.x = k < K ? in.src[so + k] : 0.0f; a.y = k + 1 < K ? in.src[so + k + 1] : 0.0f;
      a.z = k + 2 < K ? in.src[so + k + 2] : 0.0f; a.w = 0.0f;
    }
    float4 x0, x1, x2;
    split_one(a.x, is_b, x0.x, x1.x, x2.x); split_one(a.y, is_b, x0.y, x1.y, x2.y);
    split_one(a.z, is_b, x0.z, x1.z, x2.z); split_one(a.w, is_b, x0.w, x1.w, x2.w);
    float *o = dst + row * 3 * Kp + k;
    *reinterpret_cast<float4 *>(o) = x0;
    *reinterpret_cast<float4 *>(o + Kp) = x1;
    *reinterpret_cast<float4 *>(o + 2 * Kp) = x2;
  }
}

/* An operand stored with its row axis contiguous and k strided (a weight gradient reads the
 * activations transposed): 32 x 32 tiles through shared memory, read along the rows, written along k
 * in the split form.  dst row of (batch z, r) is z * R + r; k in [K, Kp) is zero-filled. */
struct SplitTrArgs {
  const float *src; float *dst;
  int R, K, Kp; long long s_k;
  int naxes; int ext[6]; long long sstride[6];     /* the other axes of the source, fastest first */
  int is_b;
};

__global__ void __launch_bounds__(256) pb200_split_tf32x3_tr(const SplitTrArgs a) {
  __shared__ float tile[32][33];
  long long rem = blockIdx.z, o = 0;
  for (int d = 0; d < a.naxes; d++) { const long long x = rem % a.ext[d]; rem /= a.ext[d]; o += x * a.sstride[d]; }
  const int r0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int j = ty; j < 32; j += 8) {
    const int k = k0 + j, r = r0 + tx;
    tile[j][tx] = (k < a.K && r < a.R) ? a.src[o + (long long)k * a.s_k + r] : 0.0f;
  }
  __syncthreads();
  for (int j = ty; j < 32; j += 8) {
    const int r = r0 + j, k = k0 + tx;
    if (r < a.R && k < a.Kp) {
      float *d = a.dst + ((long long)blockIdx.z * a.R + r) * 3 * a.Kp;
      split_one(tile[tx][j], a.is_b, d[k], d[a.Kp + k], d[2 * a.Kp + k]);
    }
  }
}

/* [nbatch][rows][3 * Kp] float32 copy of A or B in the split form; cached like the bf16 copies. */
static const void *tc_operand_x3(PbGemmProgram &p, PbTcOperand &cache, const void *src_buf, long long off, bool is_a,
                                 long long rows, long long Kp, cudaStream_t stream, void **scratch) {
  *scratch = nullptr;
  const size_t bytes = (size_t)(p.nbatch * rows * 3 * Kp) * 4;
  const uint64_t ver = pb_buffer_version(src_buf);
  if (cache.data && cache.src == src_buf && cache.version == ver && cache.bytes == bytes && ver != 0) return cache.data;
  const bool transient = cache.misses >= 2 || ver == 0;
  void *dst;
  if (transient) {
    if (cache.data) { pb_scratch_free(cache.data); cache.data = nullptr; cache.bytes = 0; }
    dst = pb_scratch_alloc(bytes);
    if (!dst) return nullptr;
    *scratch = dst;
  } else {
    if (cache.data && cache.bytes != bytes) { pb_scratch_free(cache.data); cache.data = nullptr; }
    if (!cache.data) { cache.data = pb_scratch_alloc(bytes); cache.bytes = bytes; }
    if (!cache.data) return nullptr;
    dst = cache.data;
    cache.src = src_buf; cache.version = ver; cache.misses++;
  }
  /* an operand that already is a K-major matrix (an activation as the model stores it) is split
   * where it lies; anything else is gathered into a dense [rows][Kp] copy first */
  const bool direct = is_a ? p.a_direct : p.b_direct;
  const long long sk = is_a ? p.a_sk : p.b_sk, srow = is_a ? p.a_sm : p.b_sn;
  bool in_place = direct && (sk == 1 || p.K == 1) && srow >= 0 && p.b_ax.size() <= 4;
  for (auto &b : p.b_ax) if ((is_a ? b.sa : b.sb) < 0) in_place = false;
  void *dense = nullptr;
  bool ok = true;
  SplitSrc in{};
  in.rows = rows;
  if (in_place) {
    in.src = (const float *)src_buf + off; in.pitch = rows > 1 ? srow : 0;
    in.nb = (int)p.b_ax.size();
    for (int i = 0; i < in.nb; i++) { in.bext[i] = (int)p.b_ax[i].ext; in.bstr[i] = is_a ? p.b_ax[i].sa : p.b_ax[i].sb; }
  } else {
    /* a strided matrix per batch entry with its rows contiguous and k strided (a weight gradient reads the
     * activations transposed; the token axes (batch, position) nest into one k axis): transposed and split
     * in one pass */
    auto sel = [&](const PbGemmAxis &x) { return is_a ? x.sa : x.sb; };
    const char *e = getenv("POLY_B200_SPLIT_TR");
    if (!(e && e[0] == '0') && direct && srow == 1 && sk > 1 && rows > 1 && p.b_ax.size() <= 6 && rows <= 2147483647LL) {
      SplitTrArgs t{};
      t.src = (const float *)src_buf + off; t.dst = (float *)dst;
      t.R = (int)rows; t.K = (int)p.K; t.Kp = (int)Kp; t.s_k = sk; t.is_b = is_a ? 0 : 1;
      long long nz = 1;
      bool fits = true;
      for (size_t i = 0; i < p.b_ax.size(); i++) {
        if (sel(p.b_ax[i]) < 0) fits = false;
        t.ext[t.naxes] = (int)p.b_ax[i].ext; t.sstride[t.naxes++] = sel(p.b_ax[i]); nz *= p.b_ax[i].ext;
      }
      if (nz > 65535 || (Kp + 31) / 32 > 65535) fits = false;
      if (fits) {
        dim3 grid((unsigned)((t.R + 31) / 32), (unsigned)((Kp + 31) / 32), (unsigned)nz);
        pb200_split_tf32x3_tr<<<grid, 256, 0, stream>>>(t);
        ok = cudaGetLastError() == cudaSuccess;
        p.launches++;
        if (!ok) {
          if (*scratch) { pb_scratch_free(*scratch); *scratch = nullptr; }
          else cache.version = 0;
          return nullptr;
        }
        return dst;
      }
    }
    dense = pb_scratch_alloc((size_t)(p.nbatch * rows * Kp) * 4);
    ok = dense != nullptr && p.pack_into(dense, src_buf, off, is_a, PB_F32, PB_F32, Kp, stream) == 0;
    in.src = (const float *)dense; in.pitch = Kp; in.rows = p.nbatch * rows; in.nb = 0;
  }
  if (ok) {
    const long long total = p.nbatch * rows * Kp;
    bool v4 = (reinterpret_cast<uintptr_t>(in.src) & 15) == 0 && in.pitch % 4 == 0;
    for (int i = 0; i < in.nb; i++) if (in.bstr[i] % 4) v4 = false;
    long long blocks = ((v4 ? total / 4 : total) + 255) / 256;
    if (blocks > 148LL * 32) blocks = 148LL * 32;
    if (v4) pb200_split_tf32x3_v4<<<(unsigned)blocks, 256, 0, stream>>>(in, (float *)dst, total / 4, (int)p.K, (int)Kp, is_a ? 0 : 1);
    else pb200_split_tf32x3<<<(unsigned)blocks, 256, 0, stream>>>(in, (float *)dst, total, (int)p.K, (int)Kp, is_a ? 0 : 1);
    ok = cudaGetLastError() == cudaSuccess;
    p.launches++;
  }
  pb_scratch_free(dense);           /* stream-ordered pool: reusable by later work on this stream */
  if (!ok) {
    if (*scratch) { pb_scratch_free(*scratch); *scratch = nullptr; }
    else cache.version = 0;
    return nullptr;
  }
  return dst;
}

/* A bf16 operand that is already K-major with 16-byte aligned rows is read in
 * place by TMA; anything else goes through tc_operand. */
struct TcView { const void *ptr; long long pitch, bpitch; };

static bool tc_in_place(const PbGemmProgram &p, const void *buf, long long off, bool is_a, TcView *v) {
  if (p.dtype == PB_F32 && !(is_a && p.a_bf16)) return false;
  const bool direct = is_a ? p.a_direct : p.b_direct;
  const long long sk = is_a ? p.a_sk : p.b_sk, srow = is_a ? p.a_sm : p.b_sn;
  const long long rows = is_a ? p.M : p.N;
  if (!direct || (sk != 1 && p.K > 1) || p.b_ax.size() > 1) return false;
  long long pitch = rows > 1 ? srow : p.K;
  long long bp = p.b_ax.empty() ? rows * pitch : (is_a ? p.b_ax[0].sa : p.b_ax[0].sb);
  const char *ptr = (const char *)buf + off * 2;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || pitch % 8 || pitch < p.K || (p.nbatch > 1 && (bp % 8 || bp <= 0))) return false;
  v->ptr = ptr; v->pitch = pitch; v->bpitch = bp;
  return true;
}

bool pb_gemm_tc_static_ok(const PbGemmProgram &p) {
  if (p.c_sn != 1 && !(p.c_sm == 1 && p.M > 1)) return false;
  if (p.K < 16) return false;
  TcView v;
  if (p.a_bf16 && !tc_in_place(p, nullptr, p.off_a, true, &v)) return false;
  if (p.c_bf16) {
    const bool swap = p.c_sn != 1 || p.N == 1;
    const long long c_sm = swap ? p.c_sn : p.c_sm, N = swap ? p.M : p.N;
    if (c_sm % 4 || N % 4 || p.off_c % 4) return false;
    for (auto &a : p.b_ax) if (a.sc % 4) return false;
    if (p.has_x) {
      const long long x_sn = swap ? p.x_sm : p.x_sn, x_sm = swap ? p.x_sn : p.x_sm;
      if (x_sn != 1 || x_sm % 4 || p.off_x % 4) return false;
      for (auto &a : p.b_ax) if (a.sx % 4) return false;
    }
  }
  return true;
}

int pb_gemm_tc_run(PbGemmProgram &p, void *const *bufs, cudaStream_t stream, int fp32_mode) {
  const bool fp32x3 = fp32_mode != 0, promote = fp32_mode == 2;
  /* output must be a row-major (or column-major: swap roles) matrix per batch entry */
  bool swap = false;
  if (p.c_sn != 1 || p.N == 1) { if (p.c_sm == 1 && p.M > 1) swap = true; else if (p.c_sn != 1) return PB_TC_UNSUPPORTED; }
  if (p.K < 16) return PB_TC_UNSUPPORTED;
  if (p.alpha != 1.0f && !promote) return PB_TC_UNSUPPORTED;      /* only the promoted kernels scale the sum */
  const long long Kp = fp32x3 ? ((p.K + 3) & ~3LL) : ((p.K + 7) & ~7LL);
  void *scr_a = nullptr, *scr_b = nullptr;
  TcView va, vb;
  if (fp32x3) {
    if (p.dtype != PB_F32 || p.a_bf16 || p.c_bf16 || 3 * Kp > 2147483647LL) return PB_TC_UNSUPPORTED;
    va.ptr = tc_operand_x3(p, p.tc_a, bufs[p.p_a], p.off_a, true, p.M, Kp, stream, &scr_a);
    va.pitch = 3 * Kp; va.bpitch = p.M * 3 * Kp;
    vb.ptr = va.ptr ? tc_operand_x3(p, p.tc_b, bufs[p.p_b], p.off_b, false, p.N, Kp, stream, &scr_b) : nullptr;
    vb.pitch = 3 * Kp; vb.bpitch = p.N * 3 * Kp;
  } else if (!tc_in_place(p, bufs[p.p_a], p.off_a, true, &va)) {
    if (p.a_bf16) { pb_set_error("gemm: bfloat16 A operand is not addressable in place (alignment)"); return -1; }
    va.ptr = tc_operand(p, p.tc_a, bufs[p.p_a], p.off_a, true, p.M, Kp, stream, &scr_a);
    va.pitch = Kp; va.bpitch = p.M * Kp;
  }
  if (!fp32x3 && va.ptr && !tc_in_place(p, bufs[p.p_b], p.off_b, false, &vb)) {
    vb.ptr = tc_operand(p, p.tc_b, bufs[p.p_b], p.off_b, false, p.N, Kp, stream, &scr_b);
    vb.pitch = Kp; vb.bpitch = p.N * Kp;
  }
  if (!va.ptr || !vb.ptr) { pb_scratch_free(scr_a); pb_scratch_free(scr_b); return -1; }

  TcArgs g{};
  long long rowsA = p.M, rowsB = p.N;
  if (swap) { std::swap(va, vb); std::swap(rowsA, rowsB); }
  g.M = (int)rowsA; g.N = (int)rowsB; g.K = fp32x3 ? (int)(3 * Kp) : (int)p.K;
  g.C = (float *)bufs[p.p_c] + p.off_c;
  g.c_sm = swap ? p.c_sn : p.c_sm;
  g.has_x = p.has_x ? 1 : 0; g.relu = p.relu ? 1 : 0;
  g.alpha = p.alpha;
  g.ab_fmt = fp32x3 ? 2 : (p.dtype == PB_F16 ? 0 : 1);
  if (p.has_x) { g.X = (const float *)bufs[p.p_x] + p.off_x; g.x_sm = swap ? p.x_sn : p.x_sm; g.x_sn = swap ? p.x_sm : p.x_sn; }
  g.nb = (int)p.b_ax.size();
  for (int i = 0; i < g.nb; i++) { g.bext[i] = (int)p.b_ax[i].ext; g.c_sb[i] = p.b_ax[i].sc; g.x_sb[i] = p.b_ax[i].sx; }

  {
    auto al = [](const void *ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
    bool v = al(g.C) && (g.c_sm % 4 == 0) && (g.N % 4 == 0);
    for (int i = 0; i < g.nb; i++) if (g.c_sb[i] % 4) v = false;
    if (g.has_x) {
      if (g.x_sn != 1 || g.x_sm % 4 || !al(g.X)) v = false;
      for (int i = 0; i < g.nb; i++) if (g.x_sb[i] % 4) v = false;
    }
    g.vec_io = v ? 1 : 0;
    g.c_bf16 = p.c_bf16 ? 1 : 0;
    g.gelu = p.gelu ? 1 : 0;
    {
      bool pk = p.c_bf16 && v && g.N % 8 == 0 && g.c_sm % 8 == 0 && (!g.has_x || g.x_sm == 0) &&
                (reinterpret_cast<uintptr_t>(bufs[p.p_c]) & 15) == 0 && p.off_c % 8 == 0;
      for (int i = 0; i < g.nb; i++) if (g.c_sb[i] % 8 || (g.has_x && g.x_sb[i] != 0)) pk = false;
      const char *e = getenv("POLY_B200_TC_PACK16");        /* "0": stage float32 and convert on the way out (measurements) */
      g.pack16 = pk && !(e && e[0] == '0') ? 1 : 0;
    }
    if (p.c_bf16) {
      /* the kernel only forms element offsets from this base; elements are 2 bytes */
      g.C = reinterpret_cast<float *>(reinterpret_cast<__nv_bfloat16 *>(bufs[p.p_c]) + p.off_c);
      if (!v || (reinterpret_cast<uintptr_t>(bufs[p.p_c]) & 15)) {
        pb_set_error("gemm: bfloat16 result needs 16-byte aligned rows");
        pb_scratch_free(scr_a); pb_scratch_free(scr_b); return -1;
      }
    }
  }
  /* tile width: least estimated time = waves over the 148 SMs x time of one tile, the latter
   * modelled as K*width (mainloop) plus a fixed 94000 (epilogue and pipeline fill, fitted to
   * measurements at K = 768 and K = 8192); a wider tile wins ties within 5 % (it moves fewer
   * operand bytes per flop) */
  int BN = 256;
  double best_cost = 0;
  const double k_model = fp32x3 ? 2.0 * g.K : (double)g.K;      /* in 2-byte elements: a tf32 tile row holds half as many */
  {
    static const int widths[4] = {64, 128, 192, 256};
    double best = -1;
    const long long tm = (g.M + TC_BM - 1) / TC_BM;
    for (int wi = 0; wi < (promote ? 2 : 4); wi++) {      /* partial sums in registers: tiles up to 128 wide */
      const int bn = widths[wi];
      if (bn > 64 && g.N <= widths[wi - 1]) continue;
      const long long tiles = tm * ((g.N + bn - 1) / bn) * p.nbatch;
      const double cost = (double)((tiles + 147) / 148) * (k_model * bn + 94000.0);
      if (best < 0 || cost <= best * 1.05) { if (best < 0 || cost < best) best = cost; BN = bn; }
    }
    best_cost = best;
    const char *f = getenv("POLY_B200_TC_BN");           /* forces a width (measurements) */
    if (f) { const int v = atoi(f); if (v == 64 || v == 128 || ((v == 192 || v == 256) && !promote)) BN = v; }
  }
  /* CTA pairs (cta_group::2, one 256 x 256 tile per pair): each CTA stages half as much of B, which
   * pays where the mainloop is the bound -- K of 1024 or more, and enough tiles to fill the 74 pairs.
   * With short K the epilogue is the bound and pairs gain nothing (measured: 8192^3 1235 -> 1384 TFLOP/s,
   * 8192 x 3072 x 1024 915 -> 999, 8192 x 2304 x 768 802 -> 765).  In the time model a pair's mainloop costs 0.85 of two single
   * tiles'.  POLY_B200_TC_CTAS=1|2 forces the choice (2 implies the 256-wide tile). */
  int ctas = 1;
  if (!promote && g.M > TC_BM && g.N > 128) {
    const long long pair_tiles = ((g.M + 2 * TC_BM - 1) / (2 * TC_BM)) * ((g.N + 255) / 256) * p.nbatch;
    const double pair_cost = (double)((pair_tiles + 73) / 74) * (0.85 * k_model * 256 + 94000.0);
    if (k_model >= 1024 && pair_tiles >= 74 && pair_cost <= best_cost && !getenv("POLY_B200_TC_BN")) { ctas = 2; BN = 256; }
    const char *c = getenv("POLY_B200_TC_CTAS");
    if (c && atoi(c) == 1) ctas = 1;
    if (c && atoi(c) == 2) { ctas = 2; BN = 256; }
  }
  CUtensorMap ma, mb;
  int rc = make_map(&ma, va.ptr, g.K, rowsA, p.nbatch, va.pitch, va.bpitch, TC_BM, g.ab_fmt);
  if (rc == 0) rc = make_map(&mb, vb.ptr, g.K, rowsB, p.nbatch, vb.pitch, vb.bpitch, BN / ctas, g.ab_fmt);
  if (rc != 0) { pb_scratch_free(scr_a); pb_scratch_free(scr_b); return -1; }
  pb_tc_mark_used();
  pb_tc_configure_backoff();
  if (promote) {
    /* eight 128-byte k-blocks (32 instructions, 256 elements of the tripled k axis) per partial sum:
     * measured on GPT-2 124M fp32, 2 blocks cost 58.9 ms per step, 4: 45.2, 8: 43.7, 16: 43.1 (no
     * promotion: 42.5), and at 16 the error against a float64 product starts to show;
     * POLY_B200_TC_KCHUNK overrides (measurements) */
    const char *kc = getenv("POLY_B200_TC_KCHUNK");
    g.kchunk = kc && atoi(kc) > 0 ? atoi(kc) : 8;
    rc = BN == 128 ? tc_launch<128, 1, true, true>(ma, mb, g, p.nbatch, stream) : tc_launch<64, 1, true, true>(ma, mb, g, p.nbatch, stream);
  } else if (fp32x3) {
    if (ctas == 2) rc = tc_launch<256, 2, false, true>(ma, mb, g, p.nbatch, stream);
    else if (BN == 256) rc = tc_launch<256, 1, false, true>(ma, mb, g, p.nbatch, stream);
    else if (BN == 192) rc = tc_launch<192, 1, false, true>(ma, mb, g, p.nbatch, stream);
    else if (BN == 128) rc = tc_launch<128, 1, false, true>(ma, mb, g, p.nbatch, stream);
    else rc = tc_launch<64, 1, false, true>(ma, mb, g, p.nbatch, stream);
  }
  else if (ctas == 2) rc = tc_launch<256, 2>(ma, mb, g, p.nbatch, stream);
  else if (BN == 256) rc = tc_launch<256, 1>(ma, mb, g, p.nbatch, stream);
  else if (BN == 192) rc = tc_launch<192, 1>(ma, mb, g, p.nbatch, stream);
  else if (BN == 128) rc = tc_launch<128, 1>(ma, mb, g, p.nbatch, stream);
  else rc = tc_launch<64, 1>(ma, mb, g, p.nbatch, stream);
  p.launches++;
  /* stream-ordered pool: later work on this stream may reuse the blocks */
  pb_scratch_free(scr_a); pb_scratch_free(scr_b);
  return rc;
}


int pb_gemm_tc_prepare_raw(void) {
  if (!encode_tiled()) { pb_set_error("gemm: cuTensorMapEncodeTiled not available"); return -1; }
  sm_count();
  if (tc_configure<256, 1>() != 0 || tc_configure<128, 1>() != 0 || tc_configure<64, 1>() != 0) return -1;
  return 0;
}

/* Runs the tensor-core kernel on operands that are already bfloat16, K-major
 * ([rows][pitch], pitch a multiple of 8 elements, 16-byte aligned base).  Uses no
 * memory beyond its arguments. */
int pb_gemm_tc_launch_raw(const void *a_bf16, long long a_pitch, const void *b_bf16, long long b_pitch,
                          float *C, long long c_sm, long long M, long long N, long long K,
                          const float *bias, int relu, cudaStream_t stream) {
  TcArgs g{};
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.C = C; g.c_sm = c_sm;
  g.has_x = bias ? 1 : 0; g.relu = relu ? 1 : 0;
  g.alpha = 1.0f;
  g.ab_fmt = 1;
  g.X = bias; g.x_sm = 0; g.x_sn = 1;
  g.nb = 0;
  g.vec_io = ((reinterpret_cast<uintptr_t>(C) & 15) == 0 && c_sm % 4 == 0 && N % 4 == 0 &&
              (!bias || (reinterpret_cast<uintptr_t>(bias) & 15) == 0)) ? 1 : 0;
  const int BN = N > 128 ? 256 : (N > 64 ? 128 : 64);
  CUtensorMap ma, mb;
  if (make_map(&ma, a_bf16, K, M, 1, a_pitch, M * a_pitch, TC_BM) != 0) return -1;
  if (make_map(&mb, b_bf16, K, N, 1, b_pitch, N * b_pitch, BN) != 0) return -1;
  pb_tc_mark_used();
  pb_tc_configure_backoff();
  if (BN == 256) return tc_launch<256, 1>(ma, mb, g, 1, stream);
  if (BN == 128) return tc_launch<128, 1>(ma, mb, g, 1, stream);
  return tc_launch<64, 1>(ma, mb, g, 1, stream);
}
