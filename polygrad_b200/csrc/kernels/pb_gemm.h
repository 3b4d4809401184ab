/*
 * pb_gemm.h -- the planned contraction shared by the fp32 kernel (pb_gemm.cu)
 * and the tensor-core kernel (pb_gemm_tc.cu).
 */
#ifndef PB_GEMM_H
#define PB_GEMM_H

#include "../runtime/pb_runtime.h"
#include <cuda_bf16.h>
#include <vector>

enum { PB_F32 = 0, PB_BF16 = 1, PB_F16 = 2 };      /* storage type of a contraction's operands */
#define PB_PACK_MAX_AXES 12
#define PB_TC_UNSUPPORTED 77

/* dst[i] (dense, axis 0 fastest) = (dst type) src[sum_d x_d * sstride[d]] */
int pb_pack_launch(const void *src, void *dst, int naxes, const long long *ext, const long long *sstride,
                   int src_dtype, int dst_dtype, long long inner, long long dpitch, cudaStream_t stream);

/* One axis of the contraction: kind m/n/k/b, extent, and the stride it has in
 * the output C, in A, in B and in the addend X (0 where it does not appear). */
struct PbGemmAxis { char kind; long long ext, sc, sa, sb, sx; };

/* A bf16, K-major copy of one operand, kept while the source is unchanged. */
struct PbTcOperand {
  void *data = nullptr; size_t bytes = 0;
  const void *src = nullptr; uint64_t version = 0;
  int misses = 0;      /* conversions done; an operand that changes every call stops being cached */
};

struct PbGemmProgram : PbAotProgram {
  int p_c = -1, p_a = -1, p_b = -1, p_x = -1;
  int dtype = PB_F32;                 /* storage type of A and B */
  long long off_c = 0, off_a = 0, off_b = 0, off_x = 0;
  bool relu = false, has_x = false;
  float alpha = 1.0f;                 /* C = X + alpha * sum (relu); 1 except for fused optimizer updates */
  bool a_bf16 = false;                /* A's buffer holds bfloat16 (same element layout) although dtype is f32 */
  bool c_bf16 = false;                /* C is written as bfloat16 (round to nearest even) into the same element layout */
  bool gelu = false;                  /* tanh-GELU applied after the addend, before the bfloat16 store (needs c_bf16) */
  std::vector<PbGemmAxis> m_ax, n_ax, k_ax, b_ax;   /* m, n by output stride (largest first); k by A stride */
  long long M = 1, N = 1, K = 1, nbatch = 1;
  bool a_direct = false, b_direct = false;          /* strides nest: usable without packing */
  long long a_sm = 0, a_sk = 0, b_sk = 0, b_sn = 0, c_sm = 0, c_sn = 0, x_sm = 0, x_sn = 0;
  int launches = 1;
  PbTcOperand tc_a, tc_b;

  ~PbGemmProgram() override;
  int n_launches() const override { return launches; }
  int launch(void *const *bufs, cudaStream_t stream) override;
  bool stale(void *const *bufs) override;

  /* Dense [batch.., rows.., k..] copy (k fastest) of A or B in dst_dtype into dst. */
  int pack_into(void *dst, const void *src, long long off, bool is_a, int src_dtype, int dst_dtype,
                long long kpitch, cudaStream_t stream);
  void *pack_operand(const void *src, long long off, bool is_a, int src_dtype, int dst_dtype, cudaStream_t stream);
};

/* Builds the planned contraction from header lines whose keys start with `prefix`. */
PbGemmProgram *pb_parse_gemm(const PbHeader &h, const char *prefix, std::string &err);

/* Fused attention (pb_attention.cu). */
bool pb_attention_supported(long long T, long long hd);
/* A bfloat16 matrix of 64-element rows: element (batch.., row, d) at
 * ptr[sum_i batch_i * bstride[i] + row * row_stride + d]. */
struct PbAttnOperand { const void *ptr; long long row_stride; long long bstride[3]; };
int pb_attention_launch(const PbAttnOperand &q, const PbAttnOperand &k, const PbAttnOperand &v,
                        const float *mask, long long mask_sq, long long mask_sk,
                        float scale, void *out, bool out_bf16, int nb, const int *bext, const long long *o_sb, long long o_sm,
                        long long BH, long long T, cudaStream_t stream, float *tiles = nullptr, int tiles_mode = 0);
/* tiles_mode 1: the mask classification (a record of eight floats per 128 x 128 tile of the mask) is computed into `tiles`,
 * 2: it is read from there; 0: the launch uses scratch of its own. */

/* Can the tensor-core kernel run this problem whatever the buffer addresses are
 * (16-byte aligned bases assumed), reading A in place when a_bf16 and writing
 * bfloat16 when c_bf16? */
bool pb_gemm_tc_static_ok(const PbGemmProgram &p);

/* Tensor-core path: returns 0 / -1, or PB_TC_UNSUPPORTED when the shape is not handled. */
/* fp32_mode 0: 16-bit operands.  1: float32 operands as three tf32 products, summed in tensor memory.
 * 2: the same with the partial sums moved to registers every few k-blocks (float32-accurate). */
int pb_gemm_tc_run(PbGemmProgram &p, void *const *bufs, cudaStream_t stream, int fp32_mode = 0);

/* The tensor-core kernel on ready-made bfloat16 K-major operands; touches no
 * memory beyond its arguments. */
int pb_gemm_tc_launch_raw(const void *a_bf16, long long a_pitch, const void *b_bf16, long long b_pitch,
                          float *C, long long c_sm, long long M, long long N, long long K,
                          const float *bias, int relu, cudaStream_t stream);

/* One-time set-up of everything pb_gemm_tc_launch_raw may need (shared-memory attribute of
 * each tile-width variant, the tensor-map encoder, the SM count).  0 / -1. */
int pb_gemm_tc_prepare_raw(void);

/* POLY_B200_GEMM=bf16: run fp32 contractions with operands rounded to bf16
 * (round-to-nearest-even), products and sums in fp32, on the tensor cores. */
bool pb_gemm_policy_bf16(void);

#endif
