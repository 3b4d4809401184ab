/*
 * pb_gemm_noalloc.cu -- the bf16 tensor-core contraction for callers that must
 * not allocate device memory.
 *
 * poly_b200_gemm converts its float32 operands to bfloat16 in scratch buffers
 * taken from the runtime's pool, which calls cudaMalloc whenever the pool has no
 * block of the right size.  Some callers cannot tolerate that: code running
 * inside a CUDA stream capture (an allocation is illegal there), a serving
 * process that has handed all free device memory to its own arena, or a
 * latency-critical loop where a driver allocation (which synchronises the
 * device) is not acceptable.  For them the scratch lives in a fixed array that
 * is part of the library image: every GPU that loads the library holds
 * POLY_B200_NOALLOC_SCRATCH_BYTES of it until the process exits.
 */
#include "pb_gemm.h"
#include "../../../include/poly_b200.h"

#define NOALLOC_BYTES POLY_B200_NOALLOC_SCRATCH_BYTES

/* In host code this name is only a handle for cudaGetSymbolAddress; the device
 * address is looked up once per device below. */
static __device__ __align__(256) unsigned char pb200_noalloc_scratch[NOALLOC_BYTES];

static unsigned char *g_scratch_ptr[64];   /* device address of the array, per device ordinal */

extern "C" int poly_b200_gemm_noalloc(long long M, long long N, long long K,
                                      const float *A, long long a_sm, long long a_sk,
                                      const float *B, long long b_sk, long long b_sn,
                                      float *C, long long c_sm, const float *bias, int relu) {
  if (poly_cuda_init() != 0) return -1;
  if (M <= 0 || N <= 0 || K < 16 || !A || !B || !C) { pb_set_error("poly_b200_gemm_noalloc: bad arguments"); return -1; }
  const long long Kp = (K + 7) & ~7LL;
  const unsigned long long need_a = (unsigned long long)M * Kp * 2, need_b = (unsigned long long)N * Kp * 2;
  const unsigned long long off_b = (need_a + 255) & ~255ULL;
  if (off_b + need_b > NOALLOC_BYTES) {
    pb_set_error("poly_b200_gemm_noalloc: (M + N) * K = (%lld + %lld) * %lld needs %llu bytes of scratch, the fixed array holds %llu",
                 M, N, K, off_b + need_b, (unsigned long long)NOALLOC_BYTES);
    return -1;
  }
  const int dev = poly_b200_device();
  if (dev < 0 || dev >= 64) { pb_set_error("poly_b200_gemm_noalloc: device ordinal %d out of range", dev); return -1; }
  if (!g_scratch_ptr[dev]) {
    /* set-up, first call on this device (the runtime made it current) */
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, pb200_noalloc_scratch);
    if (e != cudaSuccess || !p) { pb_set_error("poly_b200_gemm_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e)); return -1; }
    g_scratch_ptr[dev] = (unsigned char *)p;
    /* the rest of the one-time set-up, so that no later call does any: the kernel variants'
     * shared-memory attribute and the driver entry point that encodes tensor maps */
    if (pb_gemm_tc_prepare_raw() != 0) { g_scratch_ptr[dev] = nullptr; return -1; }
  }
  unsigned char *sa = g_scratch_ptr[dev], *sb = sa + off_b;
  cudaStream_t stream = (cudaStream_t)poly_b200_stream();
  /* bookkeeping for operands that are pool buffers (a host-side table lookup; allocates nothing) */
  if (pb_note_read(A) != 0 || pb_note_read(B) != 0 || pb_note_read(bias) != 0 ||
      pb_note_write(C, c_sm == N ? (size_t)(M * N) * 4 : 0) != 0) return -1;
  /* Both operands are rewritten in full on every call (the array keeps whatever
   * the previous call left; nothing in it has to start at zero: the kernel never
   * reads the pitch padding beyond K). */
  const long long ext_a[2] = {K, M}, str_a[2] = {a_sk, a_sm};
  const long long ext_b[2] = {K, N}, str_b[2] = {b_sk, b_sn};
  if (pb_pack_launch(A, sa, 2, ext_a, str_a, PB_F32, PB_BF16, K, Kp, stream) != 0) return -1;
  if (pb_pack_launch(B, sb, 2, ext_b, str_b, PB_F32, PB_BF16, K, Kp, stream) != 0) return -1;
  if (pb_gemm_tc_launch_raw(sa, Kp, sb, Kp, C, c_sm, M, N, K, bias, relu, stream) != 0) return -1;
  pb_count_launch(true, 3);
  return 0;
}
