/*
 * pb_gemm.cu -- plans a recognised contraction and runs it.
 *
 * polygrad's matmul (reference: src/frontend.c:1029-1129) reaches the backend as
 * C[b.., m.., n..] = sum_k A[...] * B[...] (+ X[...]) (relu) with every operand
 * described by an offset and one stride per axis.  The plan
 *   1. orders the m axes (and the n axes) by output stride, which fixes the
 *      canonical row and column index of C;
 *   2. for A and B checks whether their strides nest in that same order; an
 *      operand that does not (e.g. the head-merged attention output read as
 *      [B, T, H*hd] from [B, H, T, hd] storage) is packed into a dense scratch
 *      matrix by a strided copy first;
 *   3. launches the fp32 CUDA-core kernel, or -- for bf16 operands or under the
 *      bf16 compute policy (POLY_B200_GEMM=bf16) -- converts both operands to
 *      K-major bf16 (weights once, cached per buffer version) and runs the
 *      tcgen05 tensor-core kernel (pb_gemm_tc.cu).
 *
 * fp32 kernel: 128x128 block tile, 16-deep k slices, 256 threads, 8x8 register
 * tile per thread as four 4x4 quadrants so that shared-memory reads are 128-bit
 * and conflict-free; global loads are 128-bit when the operand's contiguous
 * axis allows, register-staged double buffering.  FMA accumulation in k order
 * within a thread (the reference CPU kernel adds products one by one in the
 * same k order, unfused: results agree to fp32 rounding, not bitwise).
 */
#include "../runtime/pb_runtime.h"
#include "pb_gemm.h"
#include "../../../include/poly_b200.h"
#include <algorithm>
#include <cstdio>
#include <cstring>

/* ── strided pack: dst dense [outer..., inner] <- src with per-axis strides ── */
struct PackArgs {
  const void *src; void *dst;
  int naxes; long long ext[PB_PACK_MAX_AXES], sstride[PB_PACK_MAX_AXES]; /* axis 0 is the fastest of dst */
  long long total;
  long long inner, dpitch;   /* dst element i lives at (i / inner) * dpitch + i % inner */
};

template <typename TS, typename TD>
__global__ void __launch_bounds__(256) pb200_pack(const PackArgs a) {
  const TS *__restrict__ src = (const TS *)a.src;
  TD *__restrict__ dst = (TD *)a.dst;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.total; i += (long long)gridDim.x * blockDim.x) {
    long long rem = i, o = 0;
#pragma unroll 4
    for (int d = 0; d < a.naxes; d++) { const long long x = rem % a.ext[d]; rem /= a.ext[d]; o += x * a.sstride[d]; }
    dst[(i / a.inner) * a.dpitch + (i % a.inner)] = (TD)src[o];
  }
}

/* Fast path: the innermost source axis is contiguous and a multiple of 8 long,
 * so every thread converts 8 consecutive elements: two 128-bit loads, one
 * 128-bit store.  The remaining (outer) axes are decomposed once per 8 elements. */
struct PackVecArgs {
  const float *src; __nv_bfloat16 *dst;
  int naxes; int ext[PB_PACK_MAX_AXES]; long long sstride[PB_PACK_MAX_AXES]; /* outer axes (axis 0 fastest) */
  int run8;              /* chunks of 8 in one contiguous source run */
  long long inner, dpitch; /* destination: element e lives at (e / inner) * dpitch + e % inner */
  long long total8;
};

__global__ void __launch_bounds__(256) pb200_pack_f32_bf16_vec8(const PackVecArgs a) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.total8; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % a.run8);
    const long long rest = i / a.run8;
    long long rem = rest, o = 0;
#pragma unroll 4
    for (int d = 0; d < a.naxes; d++) { const long long x = rem % a.ext[d]; rem /= a.ext[d]; o += x * a.sstride[d]; }
    const long long e = (rest * a.run8 + c) * 8;
    const float4 v0 = *reinterpret_cast<const float4 *>(a.src + o + c * 8);
    const float4 v1 = *reinterpret_cast<const float4 *>(a.src + o + c * 8 + 4);
    __nv_bfloat162 p0 = __floats2bfloat162_rn(v0.x, v0.y), p1 = __floats2bfloat162_rn(v0.z, v0.w);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(v1.x, v1.y), p3 = __floats2bfloat162_rn(v1.z, v1.w);
    uint4 out;
    out.x = *reinterpret_cast<unsigned *>(&p0); out.y = *reinterpret_cast<unsigned *>(&p1);
    out.z = *reinterpret_cast<unsigned *>(&p2); out.w = *reinterpret_cast<unsigned *>(&p3);
    *reinterpret_cast<uint4 *>(a.dst + (e / a.inner) * a.dpitch + (e % a.inner)) = out;
  }
}

/* Transposing path: the source is contiguous along a row axis `r` (extent R,
 * stride 1) while the destination wants k fastest.  32x32 tiles through shared
 * memory; the other axes are batch.  dst[(b * R + r) * dpitch + k]. */
struct PackTrArgs {
  const float *src; __nv_bfloat16 *dst;
  int R, K; long long s_k;                 /* source: r stride 1, k stride s_k */
  int naxes; int ext[PB_PACK_MAX_AXES]; long long sstride[PB_PACK_MAX_AXES]; /* batch axes of the source */
  long long dpitch;
};

__global__ void __launch_bounds__(256) pb200_pack_f32_bf16_tr(const PackTrArgs a) {
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
    if (r < a.R && k < a.K) a.dst[((long long)blockIdx.z * a.R + r) * a.dpitch + k] = __float2bfloat16_rn(tile[tx][j]);
  }
}

int pb_pack_launch(const void *src, void *dst, int naxes, const long long *ext, const long long *sstride,
                   int src_dtype, int dst_dtype, long long inner, long long dpitch, cudaStream_t stream) {
  if (naxes > PB_PACK_MAX_AXES) { pb_set_error("pack: too many axes"); return -1; }
  long long total = 1;
  for (int i = 0; i < naxes; i++) total *= ext[i];
  if (total == 0) return 0;
  cudaError_t e;
  const bool f2b = src_dtype == PB_F32 && dst_dtype == PB_BF16;
  /* merge leading axes that are contiguous in the source into one inner run */
  int lead = 0; long long run = 1;
  while (lead < naxes && sstride[lead] == run && run < inner) { run *= ext[lead]; lead++; }
  if (f2b && inner > 0 && run % 8 == 0 && inner % run == 0 && inner % 8 == 0 && dpitch % 8 == 0 &&
      (reinterpret_cast<uintptr_t>(src) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    bool ok = true;
    for (int i = lead; i < naxes; i++) if (sstride[i] % 4 != 0 || ext[i] > 2147483647LL) ok = false;
    if (ok) {
      PackVecArgs a; a.src = (const float *)src; a.dst = (__nv_bfloat16 *)dst;
      a.naxes = naxes - lead;
      for (int i = lead; i < naxes; i++) { a.ext[i - lead] = (int)ext[i]; a.sstride[i - lead] = sstride[i]; }
      a.run8 = (int)(run / 8); a.inner = inner; a.dpitch = dpitch; a.total8 = total / 8;
      long long blocks = (a.total8 + 255) / 256;
      if (blocks > 148LL * 64) blocks = 148LL * 64;
      pb200_pack_f32_bf16_vec8<<<(unsigned)blocks, 256, 0, stream>>>(a);
      e = cudaGetLastError();
      if (e != cudaSuccess) { pb_set_error("pack launch: %s", cudaGetErrorString(e)); return -1; }
      return 0;
    }
  }
  /* transposing case: exactly one k axis (axis 0, strided) and a row axis with stride 1 right after it */
  if (f2b && inner > 0 && naxes >= 2 && ext[0] == inner && sstride[1] == 1 && sstride[0] != 1 &&
      ext[0] <= 2147483647LL && ext[1] <= 2147483647LL) {
    long long nb = 1;
    for (int i = 2; i < naxes; i++) nb *= ext[i];
    if (nb <= 65535 && (ext[0] + 31) / 32 <= 65535) {
      PackTrArgs a; a.src = (const float *)src; a.dst = (__nv_bfloat16 *)dst;
      a.K = (int)ext[0]; a.R = (int)ext[1]; a.s_k = sstride[0];
      a.naxes = naxes - 2;
      for (int i = 2; i < naxes; i++) { a.ext[i - 2] = (int)ext[i]; a.sstride[i - 2] = sstride[i]; }
      a.dpitch = dpitch;
      dim3 grid((unsigned)((a.R + 31) / 32), (unsigned)((a.K + 31) / 32), (unsigned)nb);
      pb200_pack_f32_bf16_tr<<<grid, 256, 0, stream>>>(a);
      e = cudaGetLastError();
      if (e != cudaSuccess) { pb_set_error("pack launch: %s", cudaGetErrorString(e)); return -1; }
      return 0;
    }
  }
  PackArgs a; a.src = src; a.dst = dst; a.naxes = naxes; a.total = total;
  a.inner = inner > 0 ? inner : 1; a.dpitch = inner > 0 ? dpitch : 1;
  for (int i = 0; i < naxes; i++) { a.ext[i] = ext[i]; a.sstride[i] = sstride[i]; }
  long long blocks = (a.total + 255) / 256;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  if (src_dtype == PB_F32 && dst_dtype == PB_F32) pb200_pack<float, float><<<(unsigned)blocks, 256, 0, stream>>>(a);
  else if (src_dtype == PB_F32 && dst_dtype == PB_BF16) pb200_pack<float, __nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>(a);
  else if ((src_dtype == PB_BF16 && dst_dtype == PB_BF16) || (src_dtype == PB_F16 && dst_dtype == PB_F16))
    pb200_pack<__nv_bfloat16, __nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>(a);     /* a copy of 16-bit elements */
  else { pb_set_error("pack: unsupported dtypes"); return -1; }
  e = cudaGetLastError();
  if (e != cudaSuccess) { pb_set_error("pack launch: %s", cudaGetErrorString(e)); return -1; }
  return 0;
}

/* ── fp32 kernel ─────────────────────────────────────────────────────── */
#define BM 128
#define BN 128
#define BK 16

struct SgemmArgs {
  const float *A, *B; float *C; const float *X;
  int M, N, K;
  long long a_sm, a_sk, b_sk, b_sn, c_sm, c_sn, x_sm, x_sn;
  int nb; int bext[4]; long long a_sb[4], b_sb[4], c_sb[4], x_sb[4];
  int relu; int has_x;
  float alpha;          /* the sum is scaled by alpha before the addend: X + alpha * (A.B) */
};

/* Load a BMxBK tile of an operand whose "row" axis has stride s_row and whose k
 * axis has stride s_k into smem laid out [BK][ROWS+PAD].  KMAJOR: k contiguous. */
template <bool KMAJOR, bool VEC>
__device__ __forceinline__ void load_tile(const float *__restrict__ base, long long s_row, long long s_k,
                                          int row0, int k0, int rows, int K, float (&reg)[8]) {
  const int tid = threadIdx.x;
  if (KMAJOR) {
    /* 128 rows x 16 k: thread t handles rows (t/4) and (t/4)+64, k quad (t%4)*4 */
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int r = row0 + (tid >> 2) + h * 64;
      const int k = k0 + (tid & 3) * 4;
      if (VEC && r < rows && k + 3 < K) {
        const float4 v = *reinterpret_cast<const float4 *>(base + (long long)r * s_row + k);
        reg[h * 4 + 0] = v.x; reg[h * 4 + 1] = v.y; reg[h * 4 + 2] = v.z; reg[h * 4 + 3] = v.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; j++)
          reg[h * 4 + j] = (r < rows && k + j < K) ? base[(long long)r * s_row + (long long)(k + j) * s_k] : 0.0f;
      }
    }
  } else {
    /* row axis contiguous: thread t handles k = t/32 and t/32+8, row quad (t%32)*4 */
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int k = k0 + (tid >> 5) + h * 8;
      const int r = row0 + (tid & 31) * 4;
      if (VEC && k < K && r + 3 < rows) {
        const float4 v = *reinterpret_cast<const float4 *>(base + (long long)k * s_k + r);
        reg[h * 4 + 0] = v.x; reg[h * 4 + 1] = v.y; reg[h * 4 + 2] = v.z; reg[h * 4 + 3] = v.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; j++)
          reg[h * 4 + j] = (k < K && r + j < rows) ? base[(long long)k * s_k + (long long)(r + j) * s_row] : 0.0f;
      }
    }
  }
}

template <bool KMAJOR>
__device__ __forceinline__ void store_tile(float (*sm)[BM + 4], const float (&reg)[8]) {
  const int tid = threadIdx.x;
  if (KMAJOR) {
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int r = (tid >> 2) + h * 64;
      const int k = (tid & 3) * 4;
#pragma unroll
      for (int j = 0; j < 4; j++) sm[k + j][r] = reg[h * 4 + j];
    }
  } else {
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int k = (tid >> 5) + h * 8;
      const int r = (tid & 31) * 4;
      *reinterpret_cast<float4 *>(&sm[k][r]) = make_float4(reg[h * 4 + 0], reg[h * 4 + 1], reg[h * 4 + 2], reg[h * 4 + 3]);
    }
  }
}

template <bool A_KMAJOR, bool B_KMAJOR, bool VEC_A, bool VEC_B>
__global__ void __launch_bounds__(256, 2) pb200_sgemm(const SgemmArgs g) {
  __shared__ __align__(16) float As[2][BK][BM + 4];
  __shared__ __align__(16) float Bs[2][BK][BN + 4];

  /* batch offsets */
  long long oa = 0, ob = 0, oc = 0, ox = 0;
  {
    int rem = blockIdx.z;
    for (int i = 0; i < g.nb; i++) {
      const int x = rem % g.bext[i]; rem /= g.bext[i];
      oa += x * g.a_sb[i]; ob += x * g.b_sb[i]; oc += x * g.c_sb[i]; ox += x * g.x_sb[i];
    }
  }
  const float *__restrict__ A = g.A + oa;
  const float *__restrict__ B = g.B + ob;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 8; j++) acc[i][j] = 0.0f;

  float ra[8], rb[8];
  load_tile<A_KMAJOR, VEC_A>(A, g.a_sm, g.a_sk, m0, 0, g.M, g.K, ra);
  load_tile<B_KMAJOR, VEC_B>(B, g.b_sn, g.b_sk, n0, 0, g.N, g.K, rb);
  store_tile<A_KMAJOR>(As[0], ra);
  store_tile<B_KMAJOR>(Bs[0], rb);
  __syncthreads();

  const int nk = (g.K + BK - 1) / BK;
  for (int kt = 0; kt < nk; kt++) {
    const int cur = kt & 1;
    if (kt + 1 < nk) {
      load_tile<A_KMAJOR, VEC_A>(A, g.a_sm, g.a_sk, m0, (kt + 1) * BK, g.M, g.K, ra);
      load_tile<B_KMAJOR, VEC_B>(B, g.b_sn, g.b_sk, n0, (kt + 1) * BK, g.N, g.K, rb);
    }
#pragma unroll
    for (int k = 0; k < BK; k++) {
      const float4 a0 = *reinterpret_cast<const float4 *>(&As[cur][k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4 *>(&As[cur][k][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4 *>(&Bs[cur][k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4 *>(&Bs[cur][k][64 + tx * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (kt + 1 < nk) {
      store_tile<A_KMAJOR>(As[cur ^ 1], ra);
      store_tile<B_KMAJOR>(Bs[cur ^ 1], rb);
    }
    __syncthreads();
  }

  /* epilogue */
  float *__restrict__ C = g.C + oc;
  const float *__restrict__ X = g.has_x ? g.X + ox : nullptr;
  const bool vec_c = (g.c_sn == 1) && ((g.c_sm & 3) == 0) && ((oc & 3) == 0) && ((reinterpret_cast<uintptr_t>(g.C) & 15) == 0);
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
    if (m >= g.M) continue;
#pragma unroll
    for (int jh = 0; jh < 2; jh++) {
      const int n = n0 + jh * 64 + tx * 4;
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float t = __fmul_rn(acc[i][jh * 4 + j], g.alpha);
        if (X && n + j < g.N) t = t + X[(long long)m * g.x_sm + (long long)(n + j) * g.x_sn];
        if (g.relu) t = (0.0f < t) ? t : 0.0f;
        v[j] = t;
      }
      if (vec_c && n + 3 < g.N) {
        *reinterpret_cast<float4 *>(C + (long long)m * g.c_sm + n) = make_float4(v[0], v[1], v[2], v[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; j++)
          if (n + j < g.N) C[(long long)m * g.c_sm + (long long)(n + j) * g.c_sn] = v[j];
      }
    }
  }
}

typedef void (*SgemmFn)(const SgemmArgs);
template <bool AK, bool BKm>
static SgemmFn pick_vec(bool va, bool vb) {
  if (va && vb) return pb200_sgemm<AK, BKm, true, true>;
  if (va) return pb200_sgemm<AK, BKm, true, false>;
  if (vb) return pb200_sgemm<AK, BKm, false, true>;
  return pb200_sgemm<AK, BKm, false, false>;
}

/* Small problems: a 128 x 128 tiling would leave most SMs idle (the 256 x 784 x 512 and
 * 256 x 512 x 10 layers of an MLP are 8 and 2 such tiles).  32 x 32 tiles, 256 threads,
 * 2 x 2 results per thread, any strides; same accumulation as the large kernel
 * (k ascending, one fused multiply-add per product). */
#define SB 32
__global__ void __launch_bounds__(256) pb200_sgemm_small(const SgemmArgs g) {
  __shared__ float As[2][SB][SB + 1];      /* [k][m] */
  __shared__ float Bs[2][SB][SB + 1];      /* [k][n] */
  long long oa = 0, ob = 0, oc = 0, ox = 0;
  {
    int rem = blockIdx.z;
    for (int i = 0; i < g.nb; i++) {
      const int x = rem % g.bext[i]; rem /= g.bext[i];
      oa += x * g.a_sb[i]; ob += x * g.b_sb[i]; oc += x * g.c_sb[i]; ox += x * g.x_sb[i];
    }
  }
  const float *__restrict__ A = g.A + oa;
  const float *__restrict__ B = g.B + ob;
  const int m0 = blockIdx.y * SB, n0 = blockIdx.x * SB;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  /* element e of a 32 x 32 tile: consecutive threads along the operand's contiguous axis */
  const bool a_kfast = g.a_sk == 1, b_kfast = g.b_sk == 1 && g.b_sn != 1;
  float ra[4], rb[4];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int e = tid + i * 256;
      const int ka = a_kfast ? (e & 31) : (e >> 5), ma = a_kfast ? (e >> 5) : (e & 31);
      const int kb = b_kfast ? (e & 31) : (e >> 5), nb = b_kfast ? (e >> 5) : (e & 31);
      ra[i] = (m0 + ma < g.M && k0 + ka < g.K) ? A[(long long)(m0 + ma) * g.a_sm + (long long)(k0 + ka) * g.a_sk] : 0.0f;
      rb[i] = (n0 + nb < g.N && k0 + kb < g.K) ? B[(long long)(k0 + kb) * g.b_sk + (long long)(n0 + nb) * g.b_sn] : 0.0f;
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int e = tid + i * 256;
      const int ka = a_kfast ? (e & 31) : (e >> 5), ma = a_kfast ? (e >> 5) : (e & 31);
      const int kb = b_kfast ? (e & 31) : (e >> 5), nb = b_kfast ? (e >> 5) : (e & 31);
      As[buf][ka][ma] = ra[i];
      Bs[buf][kb][nb] = rb[i];
    }
  };
  float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  fetch(0);
  stash(0);
  __syncthreads();
  const int nk = (g.K + SB - 1) / SB;
  for (int kt = 0; kt < nk; kt++) {
    const int cur = kt & 1;
    if (kt + 1 < nk) fetch((kt + 1) * SB);
#pragma unroll
    for (int k = 0; k < SB; k++) {
      const float a0 = As[cur][k][ty * 2], a1 = As[cur][k][ty * 2 + 1];
      const float b0 = Bs[cur][k][tx * 2], b1 = Bs[cur][k][tx * 2 + 1];
      acc[0][0] = fmaf(a0, b0, acc[0][0]); acc[0][1] = fmaf(a0, b1, acc[0][1]);
      acc[1][0] = fmaf(a1, b0, acc[1][0]); acc[1][1] = fmaf(a1, b1, acc[1][1]);
    }
    if (kt + 1 < nk) stash(cur ^ 1);
    __syncthreads();
  }
  float *__restrict__ C = g.C + oc;
  const float *__restrict__ X = g.has_x ? g.X + ox : nullptr;
#pragma unroll
  for (int i = 0; i < 2; i++) {
    const int m = m0 + ty * 2 + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 2; j++) {
      const int n = n0 + tx * 2 + j;
      if (n >= g.N) continue;
      float t = __fmul_rn(acc[i][j], g.alpha);
      if (X) t = t + X[(long long)m * g.x_sm + (long long)n * g.x_sn];
      if (g.relu) t = (0.0f < t) ? t : 0.0f;
      C[(long long)m * g.c_sm + (long long)n * g.c_sn] = t;
    }
  }
}

static int sgemm_launch(const SgemmArgs &g, long long nbatch, cudaStream_t stream) {
  /* fewer large tiles than SMs: the small-tile kernel spreads the work */
  {
    const long long big = (long long)((g.M + BM - 1) / BM) * ((g.N + BN - 1) / BN) * nbatch;
    const long long small = (long long)((g.M + SB - 1) / SB) * ((g.N + SB - 1) / SB) * nbatch;
    if (big < 74 && small <= 65535LL * 16 && nbatch <= 65535) {
      dim3 grid((unsigned)((g.N + SB - 1) / SB), (unsigned)((g.M + SB - 1) / SB), (unsigned)nbatch);
      if (grid.y <= 65535) {
        pb200_sgemm_small<<<grid, 256, 0, stream>>>(g);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) { pb_set_error("sgemm launch: %s", cudaGetErrorString(e)); return -1; }
        return 0;
      }
    }
  }
  /* operand layout: contiguous along k, or along the row/column axis */
  const bool a_k = (g.a_sk == 1) || g.K == 1, b_k = (g.b_sk == 1 && g.b_sn != 1);
  const bool a_ok = a_k ? true : (g.a_sm == 1), b_ok = b_k ? true : (g.b_sn == 1);
  auto aligned = [](const void *p, long long ld, const long long *sb, int nb) {
    if (reinterpret_cast<uintptr_t>(p) & 15) return false;
    if (ld & 3) return false;
    for (int i = 0; i < nb; i++) if (sb[i] & 3) return false;
    return true;
  };
  const bool va = a_ok && aligned(g.A, a_k ? g.a_sm : g.a_sk, g.a_sb, g.nb);
  const bool vb = b_ok && aligned(g.B, b_k ? g.b_sn : g.b_sk, g.b_sb, g.nb);
  SgemmFn fn;
  if (a_k && b_k) fn = pick_vec<true, true>(va, vb);
  else if (a_k) fn = pick_vec<true, false>(va, vb);
  else if (b_k) fn = pick_vec<false, true>(va, vb);
  else fn = pick_vec<false, false>(va, vb);
  dim3 grid((unsigned)((g.N + BN - 1) / BN), (unsigned)((g.M + BM - 1) / BM), (unsigned)nbatch);
  if (grid.y > 65535 || grid.z > 65535) { pb_set_error("gemm: grid too large (%u, %u)", grid.y, grid.z); return -1; }
  fn<<<grid, 256, 0, stream>>>(g);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { pb_set_error("sgemm launch: %s", cudaGetErrorString(e)); return -1; }
  return 0;
}

/* ── plan ────────────────────────────────────────────────────────────── */
typedef PbGemmAxis Axis;

/* Do the strides sel(axes[i]) nest in this order?  Returns the innermost stride. */
template <class F>
static bool nests(const std::vector<Axis> &ax, F sel, long long *inner) {
  if (ax.empty()) { *inner = 0; return true; }
  for (size_t i = 0; i + 1 < ax.size(); i++)
    if (sel(ax[i]) != sel(ax[i + 1]) * ax[i + 1].ext) return false;
  *inner = sel(ax.back());
  return true;
}

static int g_policy = -1;
bool pb_gemm_policy_bf16(void) {
  if (g_policy < 0) { const char *e = getenv("POLY_B200_GEMM"); g_policy = (e && strcmp(e, "bf16") == 0) ? 1 : 0; }
  return g_policy == 1;
}
extern "C" void poly_b200_set_gemm_policy(int bf16) { g_policy = bf16 ? 1 : 0; }
extern "C" int poly_b200_gemm_policy(void) { return pb_gemm_policy_bf16() ? 1 : 0; }

bool PbGemmProgram::stale(void *const *bufs) {
  if (tc_a.data && tc_a.src == bufs[p_a] && tc_a.version != pb_buffer_version(bufs[p_a])) return true;
  if (tc_b.data && tc_b.src == bufs[p_b] && tc_b.version != pb_buffer_version(bufs[p_b])) return true;
  if (tc_a.data && tc_a.src != bufs[p_a]) return true;
  if (tc_b.data && tc_b.src != bufs[p_b]) return true;
  return false;
}

PbGemmProgram::~PbGemmProgram() { pb_scratch_free(tc_a.data); pb_scratch_free(tc_b.data); }

int PbGemmProgram::pack_into(void *dst, const void *src, long long off, bool is_a, int src_dtype, int dst_dtype,
                             long long kpitch, cudaStream_t stream) {
  std::vector<long long> ext, str;
  auto sel = [&](const Axis &x) { return is_a ? x.sa : x.sb; };
  for (int i = (int)k_ax.size() - 1; i >= 0; i--) { ext.push_back(k_ax[i].ext); str.push_back(sel(k_ax[i])); }
  const std::vector<Axis> &rows = is_a ? m_ax : n_ax;
  for (int i = (int)rows.size() - 1; i >= 0; i--) { ext.push_back(rows[i].ext); str.push_back(sel(rows[i])); }
  for (size_t i = 0; i < b_ax.size(); i++) { ext.push_back(b_ax[i].ext); str.push_back(sel(b_ax[i])); }
  const char *s = (const char *)src + off * (src_dtype == PB_F32 ? 4 : 2);
  if (pb_pack_launch(s, dst, (int)ext.size(), ext.data(), str.data(), src_dtype, dst_dtype, K, kpitch, stream) != 0) return -1;
  launches++;
  return 0;
}

void *PbGemmProgram::pack_operand(const void *src, long long off, bool is_a, int src_dtype, int dst_dtype, cudaStream_t stream) {
  const size_t esz = dst_dtype == PB_F32 ? 4 : 2;
  const long long rowsz = is_a ? M : N;
  void *dst = pb_scratch_alloc((size_t)(nbatch * rowsz * K) * esz);
  if (!dst) return nullptr;
  if (pack_into(dst, src, off, is_a, src_dtype, dst_dtype, K, stream) != 0) { pb_scratch_free(dst); return nullptr; }
  return dst;
}

int PbGemmProgram::launch(void *const *bufs, cudaStream_t stream) {
  launches = 0;
  /* a scaled sum (an optimizer update fused behind a weight gradient) is a float32 contraction */
  if (dtype != PB_F32 || a_bf16 || c_bf16 || (pb_gemm_policy_bf16() && alpha == 1.0f)) {
    int rc = pb_gemm_tc_run(*this, bufs, stream);
    if (rc != PB_TC_UNSUPPORTED) return rc;
    if (dtype != PB_F32 || a_bf16 || c_bf16) { pb_set_error("gemm: 16-bit operands need the tensor-core kernel, which rejected this shape"); return -1; }
  }
  /* float32 contractions of at least 2^30 multiply-adds run on the tensor cores as three tf32
   * products, the partial sums of every eight k-blocks added up in registers (float32-accurate:
   * the 1e-5 bound of this path holds at every K; a scale factor is applied to the sum before the
   * addend).  Small ones stay on the CUDA-core kernels.  POLY_B200_FP32=simt keeps everything there; =tcp sends every shape the tensor-core
   * kernel accepts; =tc sums the whole k axis in tensor memory instead, whose accumulation
   * truncates (error about 1e-8 * K of the result's rms; a few percent faster). */
  {
    const char *m = getenv("POLY_B200_FP32");
    int mode = 0;
    /* back-to-back calls favour this route from far smaller sizes (256 x 784 x 512: 26.6 us on the CUDA
     * cores, 20.6 us here), but inside a short dependent chain its extra launch and longer start-up
     * cost more than they save: with the threshold at 2^26 the MLP forward went from 44.6 to 52.8 us
     * and a small training step from 3.85 to 4.27 ms (and a single 2^28 contraction in that step cost
     * 0.3 ms), so the threshold is 2^30 multiply-adds, 1024^3 */
    if (!m) mode = (double)M * (double)N * (double)K * (double)nbatch >= 1073741824.0 ? 2 : 0;
    else if (strcmp(m, "tc") == 0) mode = 1;
    else if (strcmp(m, "tcp") == 0) mode = 2;
    if (alpha != 1.0f && mode == 1) mode = 0;          /* a scaled sum: the promoted kernels or the CUDA cores */
    if (mode) {
      int rc = pb_gemm_tc_run(*this, bufs, stream, mode);
      if (rc != PB_TC_UNSUPPORTED) return rc;
    }
  }
  SgemmArgs g{};
  void *pa = nullptr, *pb = nullptr;
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.nb = (int)b_ax.size();
  for (int i = 0; i < g.nb; i++) {
    g.bext[i] = (int)b_ax[i].ext; g.c_sb[i] = b_ax[i].sc; g.x_sb[i] = b_ax[i].sx;
    g.a_sb[i] = b_ax[i].sa; g.b_sb[i] = b_ax[i].sb;
  }
  if (a_direct) { g.A = (const float *)bufs[p_a] + off_a; g.a_sm = a_sm; g.a_sk = a_sk; }
  else {
    pa = pack_operand(bufs[p_a], off_a, true, PB_F32, PB_F32, stream);
    if (!pa) return -1;
    g.A = (const float *)pa; g.a_sm = K; g.a_sk = 1;
    long long s = M * K;
    for (int i = 0; i < g.nb; i++) { g.a_sb[i] = s; s *= b_ax[i].ext; }
  }
  if (b_direct) { g.B = (const float *)bufs[p_b] + off_b; g.b_sk = b_sk; g.b_sn = b_sn; }
  else {
    pb = pack_operand(bufs[p_b], off_b, false, PB_F32, PB_F32, stream);
    if (!pb) { pb_scratch_free(pa); return -1; }
    g.B = (const float *)pb; g.b_sn = K; g.b_sk = 1;
    long long s = N * K;
    for (int i = 0; i < g.nb; i++) { g.b_sb[i] = s; s *= b_ax[i].ext; }
  }
  g.C = (float *)bufs[p_c] + off_c; g.c_sm = c_sm; g.c_sn = c_sn;
  g.has_x = has_x ? 1 : 0; g.relu = relu ? 1 : 0; g.alpha = alpha;
  if (has_x) { g.X = (const float *)bufs[p_x] + off_x; g.x_sm = x_sm; g.x_sn = x_sn; }
  int rc;
  if (g.c_sn != 1 && g.c_sm == 1) {
    /* column-major output: compute the transposed problem so that stores stay contiguous */
    SgemmArgs t = g;
    t.A = g.B; t.B = g.A; t.M = g.N; t.N = g.M;
    t.a_sm = g.b_sn; t.a_sk = g.b_sk; t.b_sk = g.a_sk; t.b_sn = g.a_sm;
    t.c_sm = g.c_sn; t.c_sn = g.c_sm; t.x_sm = g.x_sn; t.x_sn = g.x_sm;
    for (int i = 0; i < g.nb; i++) { t.a_sb[i] = g.b_sb[i]; t.b_sb[i] = g.a_sb[i]; }
    rc = sgemm_launch(t, nbatch, stream);
  } else rc = sgemm_launch(g, nbatch, stream);
  launches++;
  /* stream-ordered pool: the blocks may be reused by later launches on the same stream */
  pb_scratch_free(pa); pb_scratch_free(pb);
  return rc;
}

PbAotProgram *pb_make_gemm(const PbHeader &h, std::string &err) { return pb_parse_gemm(h, "", err); }

/* Keys are looked up as prefix + name, so a header may carry several contractions. */
PbGemmProgram *pb_parse_gemm(const PbHeader &h0, const char *prefix, std::string &err) {
  struct Prefixed {
    const PbHeader &h; std::string pre;
    const std::string &get(const char *k) const { return h.get((pre + k).c_str()); }
    long long geti(const char *k, long long d = 0) const { return h.geti((pre + k).c_str(), d); }
    std::vector<long long> getv(const char *k) const { return h.getv((pre + k).c_str()); }
  } h{h0, prefix};
  auto params = h.getv("params"), off = h.getv("offsets");
  if (params.size() != 4 || off.size() != 4) { err = "malformed gemm header"; return nullptr; }
  PbGemmProgram *p = new PbGemmProgram();
  p->n_params = (int)h.geti("nparams");
  p->p_c = (int)params[0]; p->p_a = (int)params[1]; p->p_b = (int)params[2]; p->p_x = (int)params[3];
  p->has_x = p->p_x >= 0;
  p->relu = h.geti("relu") != 0;
  if (!h.get("alpha").empty()) { uint32_t bits = (uint32_t)h.geti("alpha"); memcpy(&p->alpha, &bits, 4); }
  const std::string &dt = h.get("dtype");
  if (dt == "f32") p->dtype = PB_F32; else if (dt == "bf16") p->dtype = PB_BF16; else if (dt == "f16") p->dtype = PB_F16;
  else { err = "gemm operand dtype '" + dt + "' has no kernel"; delete p; return nullptr; }
  p->off_c = off[0]; p->off_a = off[1]; p->off_b = off[2]; p->off_x = off[3];
  p->rw.assign((size_t)p->n_params, '-');
  p->rw[(size_t)p->p_a] = 'r'; p->rw[(size_t)p->p_b] = 'r';
  if (p->has_x) p->rw[(size_t)p->p_x] = 'r';
  int naxes = (int)h.geti("naxes");
  p->M = p->N = p->K = p->nbatch = 1;
  for (int i = 0; i < naxes; i++) {
    char key[32]; snprintf(key, sizeof key, "axis%d", i);
    const std::string &line = h.get(key);
    Axis a{}; char kind = 0;
    if (sscanf(line.c_str(), "%c %lld %lld %lld %lld %lld", &kind, &a.ext, &a.sc, &a.sa, &a.sb, &a.sx) != 6) {
      err = "malformed gemm axis line"; delete p; return nullptr;
    }
    a.kind = kind;
    if (kind == 'm') { p->m_ax.push_back(a); p->M *= a.ext; }
    else if (kind == 'n') { p->n_ax.push_back(a); p->N *= a.ext; }
    else if (kind == 'k') { p->k_ax.push_back(a); p->K *= a.ext; }
    else if (kind == 'b') { p->b_ax.push_back(a); p->nbatch *= a.ext; }
    else { err = "unknown gemm axis kind"; delete p; return nullptr; }
  }
  auto by_sc = [](const Axis &x, const Axis &y) { return x.sc > y.sc; };
  std::sort(p->m_ax.begin(), p->m_ax.end(), by_sc);
  std::sort(p->n_ax.begin(), p->n_ax.end(), by_sc);
  std::sort(p->k_ax.begin(), p->k_ax.end(), [](const Axis &x, const Axis &y) { return x.sa > y.sa; });
  if (!nests(p->m_ax, [](const Axis &x) { return x.sc; }, &p->c_sm) ||
      !nests(p->n_ax, [](const Axis &x) { return x.sc; }, &p->c_sn)) { err = "gemm output axes do not nest"; delete p; return nullptr; }
  if (p->has_x && (!nests(p->m_ax, [](const Axis &x) { return x.sx; }, &p->x_sm) ||
                   !nests(p->n_ax, [](const Axis &x) { return x.sx; }, &p->x_sn))) { err = "gemm addend axes do not nest"; delete p; return nullptr; }
  long long t;
  p->a_direct = nests(p->m_ax, [](const Axis &x) { return x.sa; }, &p->a_sm) &&
                nests(p->k_ax, [](const Axis &x) { return x.sa; }, &p->a_sk);
  p->b_direct = nests(p->n_ax, [](const Axis &x) { return x.sb; }, &p->b_sn) &&
                nests(p->k_ax, [](const Axis &x) { return x.sb; }, &p->b_sk);
  (void)t;
  if (p->m_ax.empty()) p->a_sm = 0;
  if (p->n_ax.empty()) p->b_sn = 0;
  /* the fp32 kernel wants one operand axis with unit stride, and positive strides */
  if (p->a_direct && !((p->a_sk == 1 || p->a_sm == 1) && p->a_sk > 0 && p->a_sm >= 0)) p->a_direct = false;
  if (p->b_direct && !((p->b_sk == 1 || p->b_sn == 1) && p->b_sk > 0 && p->b_sn >= 0)) p->b_direct = false;
  if (p->M > 2147483647LL || p->N > 2147483647LL || p->K > 2147483647LL || p->nbatch > 65535) {
    err = "gemm extents out of range"; delete p; return nullptr;
  }
  /* full overwrite of the output? dense if the output strides tile [0, numel) */
  auto numel = h.getv("numel");
  long long covered = p->M * p->N * p->nbatch;
  bool dense = !numel.empty() && covered == numel[0] && p->off_c == 0;
  if (dense) {
    std::vector<std::pair<long long, long long>> se;
    for (auto &a : p->m_ax) se.push_back({a.sc, a.ext});
    for (auto &a : p->n_ax) se.push_back({a.sc, a.ext});
    for (auto &a : p->b_ax) se.push_back({a.sc, a.ext});
    std::sort(se.begin(), se.end());
    long long expect = 1;
    for (auto &x : se) { if (x.first != expect) { dense = false; break; } expect *= x.second; }
  }
  bool x_is_c = p->has_x && p->p_x == p->p_c;
  p->rw[(size_t)p->p_c] = x_is_c ? 'b' : (dense ? 'W' : 'w');
  p->a_bf16 = h.geti("abf16") != 0;
  p->c_bf16 = h.geti("cbf16") != 0;
  p->gelu = h.geti("gelu") != 0;
  if (p->gelu && (!p->c_bf16 || p->relu)) { err = "gemm: the GELU epilogue needs a bfloat16 result and no relu"; delete p; return nullptr; }
  if (p->alpha != 1.0f && p->dtype != PB_F32) { err = "gemm: a scaled sum needs fp32 operands"; delete p; return nullptr; }
  if ((p->a_bf16 || p->c_bf16) && (p->dtype != PB_F32 || x_is_c || p->alpha != 1.0f || !pb_gemm_tc_static_ok(*p))) {
    err = "gemm: bfloat16 operand/result storage is not possible for this shape"; delete p; return nullptr;
  }
  return p;
}

/* ── direct entry point ──────────────────────────────────────────────── */
/* C[m, n] = sum_k A[m*a_sm + k*a_sk] * B[k*b_sk + n*b_sn] (+ bias[n]) (relu), with
 * plain device pointers.  Programs are kept per argument shape so that bf16
 * copies of constant operands are reused between calls. */
#include <tuple>
static std::map<std::tuple<long long, long long, long long, long long, long long, long long, long long, long long, int, int, int>,
                PbGemmProgram *> g_direct;

static int gemm_direct(long long M, long long N, long long K, const void *A, long long a_sm, long long a_sk,
                       const void *B, long long b_sk, long long b_sn, void *C, long long c_sm, const float *bias,
                       int relu, int operands_bf16, int flags);

extern "C" int poly_b200_gemm(long long M, long long N, long long K,
                              const void *A, long long a_sm, long long a_sk,
                              const void *B, long long b_sk, long long b_sn,
                              float *C, long long c_sm, const float *bias, int relu, int operands_bf16) {
  return gemm_direct(M, N, K, A, a_sm, a_sk, B, b_sk, b_sn, C, c_sm, bias, relu, operands_bf16, 0);
}

/* flags: POLY_B200_GEMM_C_BF16 stores C as bfloat16, POLY_B200_GEMM_GELU applies tanh-GELU before that store. */
extern "C" int poly_b200_gemm_ex(long long M, long long N, long long K,
                                 const void *A, long long a_sm, long long a_sk,
                                 const void *B, long long b_sk, long long b_sn,
                                 void *C, long long c_sm, const float *bias, int operands_bf16, int flags) {
  if ((flags & POLY_B200_GEMM_GELU) && !(flags & POLY_B200_GEMM_C_BF16)) { pb_set_error("poly_b200_gemm_ex: the GELU epilogue stores bfloat16"); return -1; }
  return gemm_direct(M, N, K, A, a_sm, a_sk, B, b_sk, b_sn, C, c_sm, bias, 0, operands_bf16, flags);
}

static int gemm_direct(long long M, long long N, long long K, const void *A, long long a_sm, long long a_sk,
                       const void *B, long long b_sk, long long b_sn, void *C, long long c_sm, const float *bias,
                       int relu, int operands_bf16, int flags) {
  if (poly_cuda_init() != 0) return -1;
  if (M <= 0 || N <= 0 || K <= 0 || !A || !B || !C) { pb_set_error("poly_b200_gemm: bad arguments"); return -1; }
  auto key = std::make_tuple(M, N, K, a_sm, a_sk, b_sk, b_sn, c_sm, relu + 16 * flags, operands_bf16, bias ? 1 : 0);
  PbGemmProgram *p = nullptr;
  auto it = g_direct.find(key);
  if (it != g_direct.end()) p = it->second;
  else {
    p = new PbGemmProgram();
    p->n_params = 4; p->p_c = 0; p->p_a = 1; p->p_b = 2; p->p_x = bias ? 3 : -1;
    p->has_x = bias != nullptr; p->relu = relu != 0;
    p->dtype = operands_bf16 ? PB_BF16 : PB_F32;
    p->M = M; p->N = N; p->K = K; p->nbatch = 1;
    p->m_ax.push_back(PbGemmAxis{'m', M, c_sm, a_sm, 0, 0});
    p->n_ax.push_back(PbGemmAxis{'n', N, 1, 0, b_sn, bias ? 1 : 0});
    p->k_ax.push_back(PbGemmAxis{'k', K, 0, a_sk, b_sk, 0});
    p->c_sm = c_sm; p->c_sn = 1; p->x_sm = 0; p->x_sn = 1;
    p->a_sm = a_sm; p->a_sk = a_sk; p->b_sk = b_sk; p->b_sn = b_sn;
    p->a_direct = (a_sk == 1 || a_sm == 1) && a_sk > 0 && a_sm >= 0;
    p->b_direct = (b_sk == 1 || b_sn == 1) && b_sk > 0 && b_sn >= 0;
    p->rw = "Wrrr";
    p->c_bf16 = (flags & POLY_B200_GEMM_C_BF16) != 0;
    p->gelu = (flags & POLY_B200_GEMM_GELU) != 0;
    if (p->c_bf16 && !pb_gemm_tc_static_ok(*p)) { delete p; pb_set_error("poly_b200_gemm_ex: a bfloat16 result needs N, c_sm multiples of 4 and K >= 16"); return -1; }
    g_direct[key] = p;
  }
  void *bufs[4] = {C, const_cast<void *>(A), const_cast<void *>(B), const_cast<float *>(bias)};
  if (pb_note_read(A) != 0 || pb_note_read(B) != 0 || pb_note_read(bias) != 0 ||
      pb_note_write(C, c_sm == N ? (size_t)(M * N) * (p->c_bf16 ? 2 : 4) : 0) != 0) return -1;
  int rc = p->launch(bufs, (cudaStream_t)poly_b200_stream());
  if (rc == 0) pb_count_launch(true, p->n_launches());
  return rc;
}
