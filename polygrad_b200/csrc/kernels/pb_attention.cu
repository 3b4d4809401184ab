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
 * assumed: the mask is an arbitrary additive [T, T] buffer and every block of
 * keys is processed, as in the reference.
 *
 * One CTA per (batch*head, block of 128 query rows), 5 warps, up to two CTAs
 * per SM:
 *   warp 4   lane 0 issues the TMA loads (Q once; K and Vᵀ blocks, each
 *            prefetched as soon as the MMA that read the previous one has
 *            finished) and the tcgen05.mma instructions:
 *            S = Q Kᵀ (128x128x64) into tensor memory, then PV = P Vᵀᵀ
 *            (128x64x128) into another 64 columns;
 *   warps 0-3  one query row per thread: read S from tensor memory in 32-column
 *            chunks (two passes: row max, then exponentials), write P as bf16
 *            into shared memory in the swizzled K-major tile layout the MMA
 *            reads, then add PV to the row's 64 fp32 accumulators in registers.
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
#define AT_THREADS 160
#define AT_SMEM (16384 /*Q*/ + 16384 /*K*/ + 16384 /*Vt: 2 x 8 KB*/ + 32768 /*P: 2 x 16 KB*/ + 256 + 1024)

struct AttnArgs {
  float *O; const float *mask;
  long long mask_sq, mask_sk;     /* mask[q*mask_sq + k*mask_sk] */
  float scale;
  int mask_vec;                   /* mask rows contiguous and 16-byte aligned */
  int T, n_qblocks;
  int nb; int bext[4]; long long o_sb[4]; long long o_sm;   /* O[batch..][row*o_sm + d] */
};

__global__ void __launch_bounds__(AT_THREADS, 2)
pb200_flash_attn(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_vt, const AttnArgs g) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *sm = smem_raw + (base - raw);
  const uint32_t s_q = base, s_k = base + 16384, s_v = base + 32768, s_p = base + 49152;
  uint64_t *bars = reinterpret_cast<uint64_t *>(sm + 81920);
  const uint32_t bar_q = smem_u32(bars), bar_k = bar_q + 8, bar_v = bar_q + 16, bar_s = bar_q + 24, bar_p = bar_q + 32, bar_o = bar_q + 40;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = blockIdx.x % g.n_qblocks, bh = blockIdx.x / g.n_qblocks;
  const int nkb = g.T / AT_BK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(bar_q, 1); mbar_init(bar_k, 1); mbar_init(bar_v, 1);
    mbar_init(bar_s, 1); mbar_init(bar_p, 128); mbar_init(bar_o, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tmem_s = tmem, tmem_pv = tmem + 128;

  if (warp == 4) {
    if (lane == 0) {
      /* instruction descriptors: bf16 x bf16 -> fp32, both operands K-major, M = 128 */
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(AT_BK >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(AT_HD >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      mbar_expect_tx(bar_q, 16384);
      tma_load_3d(s_q, &map_q, bar_q, 0, qb * AT_BQ, bh);
      mbar_expect_tx(bar_k, 16384);
      tma_load_3d(s_k, &map_k, bar_k, 0, 0, bh);
      mbar_expect_tx(bar_v, 16384);
      tma_load_3d(s_v, &map_vt, bar_v, 0, 0, bh);
      tma_load_3d(s_v + 8192, &map_vt, bar_v, 64, 0, bh);
      bool ok = mbar_wait(bar_q, 0, &abort_flag, 11);
      for (int j = 0; j < nkb && ok; j++) {
        const uint32_t ph = (uint32_t)j & 1u;
        if (!mbar_wait(bar_k, ph, &abort_flag, 12)) break;
        tc_fence_after_sync();
        {
          const uint64_t da = make_smem_desc(s_q), db = make_smem_desc(s_k);
#pragma unroll
          for (int k = 0; k < AT_HD / 16; k++) tc_mma_bf16(tmem_s, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_s, k ? 1u : 0u);
          tc_commit(bar_s);
        }
        /* K is free once S is complete: prefetch the next block of keys */
        if (!mbar_wait(bar_s, ph, &abort_flag, 13)) break;
        if (j + 1 < nkb) { mbar_expect_tx(bar_k, 16384); tma_load_3d(s_k, &map_k, bar_k, 0, (j + 1) * AT_BK, bh); }
        if (!mbar_wait(bar_p, ph, &abort_flag, 14)) break;     /* P written, previous PV consumed */
        if (!mbar_wait(bar_v, ph, &abort_flag, 15)) break;
        tc_fence_after_sync();
        {
#pragma unroll
          for (int h = 0; h < 2; h++) {
            const uint64_t da = make_smem_desc(s_p + h * 16384), db = make_smem_desc(s_v + h * 8192);
#pragma unroll
            for (int k = 0; k < 4; k++) tc_mma_bf16(tmem_pv, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_o, (h | k) ? 1u : 0u);
          }
          tc_commit(bar_o);
        }
        if (!mbar_wait(bar_o, ph, &abort_flag, 16)) break;
        if (j + 1 < nkb) {
          mbar_expect_tx(bar_v, 16384);
          tma_load_3d(s_v, &map_vt, bar_v, (j + 1) * AT_BK, 0, bh);
          tma_load_3d(s_v + 8192, &map_vt, bar_v, (j + 1) * AT_BK + 64, 0, bh);
        }
      }
    }
  } else {
    /* ── softmax: thread = one query row ── */
    const int row = warp * 32 + lane;                    /* row within the block = tensor-memory lane */
    const long long q = (long long)qb * AT_BQ + row;
    const float *mrow = g.mask + q * g.mask_sq;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    const float LOG2E = 1.44269504088896340736f;
    float m_run = __int_as_float(0xff800000), l_run = 0.0f;
    float acc[AT_HD];
#pragma unroll
    for (int d = 0; d < AT_HD; d++) acc[d] = 0.0f;
    uint8_t *p_row = sm + 49152 + (row >> 3) * 1024 + (row & 7) * 128;
    bool ok = true;
    for (int j = 0; j < nkb && ok; j++) {
      const uint32_t ph = (uint32_t)j & 1u;
      if (!mbar_wait(bar_s, ph, &abort_flag, 17)) { ok = false; break; }
      tc_fence_after_sync();
      const float *mj = mrow + (long long)j * AT_BK * g.mask_sk;
      /* pass 1: x = s*scale + mask, written back over S in tensor memory; row max of the block */
      float m_blk = __int_as_float(0xff800000);
#pragma unroll 1
      for (int c = 0; c < AT_BK / 32; c++) {
        uint32_t r[32];
        tc_ld32(tmem_s + lane_addr + c * 32, r);
        tc_wait_ld();
        if (g.mask_vec) {
          const float4 *m4 = reinterpret_cast<const float4 *>(mj + c * 32);
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const float4 mv = m4[i];
            const float x0 = __uint_as_float(r[4 * i]) * g.scale + mv.x, x1 = __uint_as_float(r[4 * i + 1]) * g.scale + mv.y;
            const float x2 = __uint_as_float(r[4 * i + 2]) * g.scale + mv.z, x3 = __uint_as_float(r[4 * i + 3]) * g.scale + mv.w;
            r[4 * i] = __float_as_uint(x0); r[4 * i + 1] = __float_as_uint(x1); r[4 * i + 2] = __float_as_uint(x2); r[4 * i + 3] = __float_as_uint(x3);
            const float a01 = (x0 > x1) ? x0 : x1, a23 = (x2 > x3) ? x2 : x3;
            const float a = (a01 > a23) ? a01 : a23;
            m_blk = (m_blk > a) ? m_blk : a;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i++) {
            const float x = __uint_as_float(r[i]) * g.scale + mj[(long long)(c * 32 + i) * g.mask_sk];
            r[i] = __float_as_uint(x);
            m_blk = (m_blk > x) ? m_blk : x;
          }
        }
        tc_st32(tmem_s + lane_addr + c * 32, r);
      }
      tc_wait_st();
      const float m_new = (m_run > m_blk) ? m_run : m_blk;
      const float alpha = exp2f((m_run - m_new) * LOG2E);       /* 0 on the first block (m_run = -inf) */
      float l_blk = 0.0f;
      /* pass 2: p = exp2((x - m_new) * log2e), written as bf16 into the K-major swizzled tile */
#pragma unroll 1
      for (int c = 0; c < AT_BK / 32; c++) {
        uint32_t r[32];
        tc_ld32(tmem_s + lane_addr + c * 32, r);
        tc_wait_ld();
        uint8_t *dst = p_row + (c >> 1) * 16384;               /* 64-key half */
#pragma unroll
        for (int i8 = 0; i8 < 4; i8++) {
          uint32_t w[4];
#pragma unroll
          for (int i2 = 0; i2 < 4; i2++) {
            const int i = i8 * 8 + i2 * 2;
            const float p0 = exp2f((__uint_as_float(r[i]) - m_new) * LOG2E), p1 = exp2f((__uint_as_float(r[i + 1]) - m_new) * LOG2E);
            __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
            /* the sum uses the rounded values, i.e. exactly what the second contraction multiplies */
            l_blk += __low2float(pb) + __high2float(pb);
            w[i2] = *reinterpret_cast<uint32_t *>(&pb);
          }
          const int chunk = (c & 1) * 4 + i8;                   /* 16-byte chunk within the 128-byte row */
          *reinterpret_cast<uint4 *>(dst + ((chunk ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      l_run = l_run * alpha + l_blk;
      m_run = m_new;
#pragma unroll
      for (int d = 0; d < AT_HD; d++) acc[d] *= alpha;
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(bar_p);
      if (!mbar_wait(bar_o, ph, &abort_flag, 18)) { ok = false; break; }
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < AT_HD / 32; c++) {
        uint32_t r[32];
        tc_ld32(tmem_pv + lane_addr + c * 32, r);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i++) acc[c * 32 + i] += __uint_as_float(r[i]);
      }
    }
    if (ok) {
      int rem = bh; long long ob = 0;
      for (int i = 0; i < g.nb; i++) { const int x = rem % g.bext[i]; rem /= g.bext[i]; ob += x * g.o_sb[i]; }
      float *o = g.O + ob + q * g.o_sm;
      const float inv = 1.0f / l_run;
#pragma unroll
      for (int d = 0; d < AT_HD; d += 4)
        *reinterpret_cast<float4 *>(o + d) = make_float4(acc[d] * inv, acc[d + 1] * inv, acc[d + 2] * inv, acc[d + 3] * inv);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (abort_flag) { for (int i = 0; i < 2000; i++) __nanosleep(1000); }
  if (warp == 4) {
    tc_fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
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

static int attn_map(CUtensorMap *map, const void *ptr, long long inner, long long rows, long long nbatch, int box_inner, int box_rows) {
  EncodeTiledFn enc = attn_encode();
  if (!enc) { pb_set_error("attention: cuTensorMapEncodeTiled not available"); return -1; }
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)nbatch};
  cuuint64_t strides[2] = {(cuuint64_t)inner * 2, (cuuint64_t)rows * inner * 2};
  cuuint32_t box[3] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult rc = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(ptr), dims, strides, box, estr,
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

bool pb_attention_supported(long long T, long long hd) { return hd == AT_HD && T >= AT_BK && T % AT_BK == 0; }

/* qb, kb: bf16 [BH][T][64]; vtb: bf16 [BH][64][T]; mask fp32 [T x T] via strides; out fp32. */
int pb_attention_launch(const void *qb, const void *kb, const void *vtb, const float *mask, long long mask_sq, long long mask_sk,
                        float scale, float *out, int nb, const int *bext, const long long *o_sb, long long o_sm,
                        long long BH, long long T, cudaStream_t stream) {
  if (!pb_attention_supported(T, AT_HD)) { pb_set_error("attention: unsupported sequence length %lld", T); return -1; }
  if ((reinterpret_cast<uintptr_t>(out) & 15) || o_sm % 4) { pb_set_error("attention: output rows must be 16-byte aligned"); return -1; }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(pb200_flash_attn, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM);
    if (e != cudaSuccess) { pb_set_error("attention: cannot reserve shared memory: %s", cudaGetErrorString(e)); return -1; }
    configured = true;
  }
  CUtensorMap mq, mk, mv;
  if (attn_map(&mq, qb, AT_HD, T, BH, 64, AT_BQ) != 0) return -1;
  if (attn_map(&mk, kb, AT_HD, T, BH, 64, AT_BK) != 0) return -1;
  if (attn_map(&mv, vtb, T, AT_HD, BH, 64, AT_HD) != 0) return -1;
  AttnArgs g{};
  g.O = out; g.mask = mask; g.mask_sq = mask_sq; g.mask_sk = mask_sk; g.scale = scale;
  g.T = (int)T; g.n_qblocks = (int)(T / AT_BQ);
  g.mask_vec = (mask_sk == 1 && mask_sq % 4 == 0 && (reinterpret_cast<uintptr_t>(mask) & 15) == 0) ? 1 : 0;
  g.nb = nb; g.o_sm = o_sm;
  for (int i = 0; i < nb && i < 4; i++) { g.bext[i] = bext[i]; g.o_sb[i] = o_sb[i]; }
  for (int i = 0; i < nb; i++) if (o_sb[i] % 4) { pb_set_error("attention: output batch strides must be 16-byte aligned"); return -1; }
  long long grid = BH * g.n_qblocks;
  if (grid > 2147483647LL) { pb_set_error("attention: grid too large"); return -1; }
  pb_tc_mark_used();
  pb200_flash_attn<<<(unsigned)grid, AT_THREADS, AT_SMEM, stream>>>(mq, mk, mv, g);
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
  void *qb = pb_scratch_alloc(bytes), *kb = pb_scratch_alloc(bytes), *vb = pb_scratch_alloc(bytes);
  int rc = -1;
  if (qb && kb && vb) {
    /* [b][t][h][d] -> [b*H + h][t][d]: axes d, t, h, b */
    const long long ext[4] = {AT_HD, T, H, B}, str[4] = {1, D, AT_HD, (long long)T * D};
    /* Vᵀ: [b*H + h][d][t]: axes t, d, h, b */
    const long long extv[4] = {T, AT_HD, H, B}, strv[4] = {D, 1, AT_HD, (long long)T * D};
    rc = pb_pack_launch(q, qb, 4, ext, str, PB_F32, PB_BF16, AT_HD, AT_HD, stream);
    if (rc == 0) rc = pb_pack_launch(k, kb, 4, ext, str, PB_F32, PB_BF16, AT_HD, AT_HD, stream);
    if (rc == 0) rc = pb_pack_launch(v, vb, 4, extv, strv, PB_F32, PB_BF16, T, T, stream);
    const int bext[2] = {H, B};
    const long long o_sb[2] = {(long long)T * AT_HD, (long long)H * T * AT_HD};
    if (rc == 0) rc = pb_attention_launch(qb, kb, vb, mask, T, 1, scale, out, 2, bext, o_sb, AT_HD, BH, T, stream);
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
  ~AttnProgram() override { delete g1; delete g2; }
  int n_launches() const override { return 4; }
  int launch(void *const *bufs, cudaStream_t stream) override {
    const size_t bytes = (size_t)BH * T * AT_HD * 2;
    void *qb = pb_scratch_alloc(bytes), *kb = pb_scratch_alloc(bytes), *vb = pb_scratch_alloc(bytes);
    int rc = -1;
    if (qb && kb && vb) {
      rc = g1->pack_into(qb, bufs[0], g1->off_a, true, PB_F32, PB_BF16, AT_HD, stream);
      if (rc == 0) rc = g1->pack_into(kb, bufs[1], g1->off_b, false, PB_F32, PB_BF16, AT_HD, stream);
      if (rc == 0) rc = g2->pack_into(vb, bufs[2], g2->off_b, false, PB_F32, PB_BF16, T, stream);
      int bext[4]; long long o_sb[4];
      const int nb = (int)g2->b_ax.size();
      for (int i = 0; i < nb; i++) { bext[i] = (int)g2->b_ax[i].ext; o_sb[i] = g2->b_ax[i].sc; }
      if (rc == 0)
        rc = pb_attention_launch(qb, kb, vb, (const float *)bufs[3] + mask_off, mask_sq, mask_sk, scale,
                                 (float *)bufs[4] + g2->off_c, nb, bext, o_sb, g2->c_sm, BH, T, stream);
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
  ok = ok && pb_attention_supported(a.M, a.K) && b.c_sn == 1 && b.c_sm % 4 == 0 && a.b_ax.size() == b.b_ax.size() && a.b_ax.size() <= 4;
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
  p->n_params = 5;
  p->rw = "rrrr";
  p->rw.push_back(h.get("outmode") == "W" ? 'W' : 'w');
  return p;
}
