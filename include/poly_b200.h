/*
 * poly_b200.h -- C ABI of the B200 (sm_100a) execution backend for polygrad.
 *
 * Part 1 is the drop-in boundary: the CUDA backend symbols that polygrad's
 * exec_plan.c / frontend.c / instance.c call.  Linking this library in place of
 * polygrad's src/render_cuda.c + src/runtime_cuda.c (and compiling the rest of
 * polygrad with -DPOLY_HAS_CUDA=1) replaces the CUDA row of the backend table
 * (polygrad src/exec_plan.c:753-787) without editing any polygrad file.
 * Signatures are those of polygrad src/codegen.h:114-139.
 *
 * Part 2 are additions: device selection, stream-level synchronisation and
 * timing, statistics, and direct entry points to the precompiled kernels.
 *
 * Conventions (same as polygrad's): int results are 0 on success and -1 on
 * error with a line on stderr prefixed "polygrad: cuda:"; device pointers
 * travel as unsigned long long; the library is driven from one host thread.
 * All work is enqueued on one internal CUDA stream; only poly_cuda_copy_dtoh,
 * poly_b200_synchronize and poly_b200_event_elapsed_ms wait for the device.
 * There is no CPU fallback: without a usable GPU every compute entry fails.
 */
#ifndef POLY_B200_H
#define POLY_B200_H

#include <stddef.h>
#include <stdint.h>
#include <stdbool.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ── Part 1: polygrad CUDA backend symbols ───────────────────────────── */

struct PolyUOp; struct PolyCtx;
typedef struct PolyCudaProgram PolyCudaProgram;

/* Replaces polygrad src/render_cuda.c:176.  Returns a malloc'd one-element
 * array holding the simplified kernel SINK; the caller frees it. */
struct PolyUOp **poly_linearize_cuda(struct PolyCtx *ctx, struct PolyUOp *sink, int *n_out);

/* Replaces polygrad src/render_cuda.c:196.  Returns malloc'd program text: a
 * "//PB200" header naming a precompiled kernel and its arguments, or the header
 * followed by CUDA C for run-time compilation.  The caller frees it. */
char *poly_render_cuda(struct PolyUOp **uops, int n, const char *fn_name, int launch_bounds);

/* Replaces polygrad src/runtime_cuda.c:192 and :240. */
int  poly_cuda_init(void);
bool poly_cuda_available(void);

/* Replace polygrad src/runtime_cuda.c:245, :259.  Pooled: freed blocks are
 * kept for reuse until poly_b200_trim(). */
unsigned long long poly_cuda_alloc(size_t bytes);
void poly_cuda_free(unsigned long long ptr);

/* Replace polygrad src/runtime_cuda.c:268, :278.  copy_dtoh returns after the
 * data is in dst (it orders after all earlier work). */
int poly_cuda_copy_htod(unsigned long long dst, const void *src, size_t bytes);
int poly_cuda_copy_dtoh(void *dst, unsigned long long src, size_t bytes);

/* Replaces polygrad src/runtime_cuda.c:288.  Accepts only text produced by
 * poly_render_cuda. */
PolyCudaProgram *poly_compile_cuda(const char *source, const char *fn_name);

/* Replaces polygrad src/runtime_cuda.c:386.  args[i] points to the i-th
 * argument: a device pointer for buffer parameters, and for each DEFINE_VAR
 * parameter a pointer to the host int holding its value (what
 * polygrad src/exec_plan.c:1039-1040 supplies).  The grid and block arguments
 * are ignored. */
int poly_cuda_launch(PolyCudaProgram *prog, void **args, int n_args,
                     int gx, int gy, int gz, int bx, int by, int bz);

/* Replaces polygrad src/runtime_cuda.c:408.  Reports errors seen so far; does
 * not wait unless POLY_B200_SYNC=1 (later work is stream-ordered anyway). */
int poly_cuda_sync(void);

/* Replace polygrad src/runtime_cuda.c:418, :426.  A whole-buffer zero fill is
 * recorded and only executed if something reads the buffer before a kernel
 * overwrites all of it. */
void poly_cuda_program_destroy(PolyCudaProgram *prog);
int  poly_cuda_memset(unsigned long long ptr, unsigned char val, size_t bytes);

/* ── Part 2: additions (no counterpart in polygrad) ──────────────────── */

/* Select the CUDA device for this process.  Must be called before the first
 * poly_cuda_init(); otherwise POLY_B200_DEVICE, then LOCAL_RANK, then 0. */
int  poly_b200_set_device(int device);
int  poly_b200_device(void);

/* Arithmetic of fp32 contractions (polygrad matmuls on float32 buffers):
 *   0  float32 arithmetic (default): contractions of at least 2^30 multiply-adds
 *      run on the tensor cores as three tf32 products per multiply (a = hi + lo,
 *      hi.hi + hi.lo + lo.hi) with the partial sums added up in float32
 *      registers, within 1e-5 of the CPU at every K; smaller ones are fp32 FMAs
 *      on the CUDA cores.  POLY_B200_FP32=simt|tcp|tc forces a route (tc: the
 *      sums stay in tensor memory, error about 1e-8 * K of the result's rms);
 *   1  operands rounded to bfloat16 (nearest even), products and sums in fp32,
 *      on the tensor cores.  Also selected by POLY_B200_GEMM=bf16.
 * Contractions whose buffers are bfloat16 always take the tensor-core kernel. */
void poly_b200_set_gemm_policy(int bf16);
int  poly_b200_gemm_policy(void);

/* The contraction kernels with plain device pointers (what the backend runs for
 * polygrad's poly_dot, src/frontend.c:1029):
 *   C[m*c_sm + n] = sum_k A[m*a_sm + k*a_sk] * B[k*b_sk + n*b_sn] (+ bias[n]) (relu)
 * A and B are float32, or bfloat16 when operands_bf16 != 0; C and bias float32.
 * float32 operands follow the current policy (poly_b200_set_gemm_policy).
 * Stream-ordered; 0 / -1. */
int poly_b200_gemm(long long M, long long N, long long K,
                   const void *A, long long a_sm, long long a_sk,
                   const void *B, long long b_sk, long long b_sn,
                   float *C, long long c_sm, const float *bias, int relu, int operands_bf16);

/* The same with a choice of result format (no counterpart in polygrad; what the plan executor
 * runs when a contraction's only reader takes bfloat16): POLY_B200_GEMM_C_BF16 stores C as
 * bfloat16 (C then points to 2-byte elements, c_sm counts elements; N and c_sm multiples of 4),
 * POLY_B200_GEMM_GELU applies GELU in its tanh form (polygrad's poly_gelu, src/frontend.c:603)
 * after the bias and before that rounding, evaluated with the hardware tanh approximation
 * (relative error about 2^-11, below bfloat16's 2^-9).  Tensor-core kernel only. */
#define POLY_B200_GEMM_C_BF16 1
#define POLY_B200_GEMM_GELU   2
int poly_b200_gemm_ex(long long M, long long N, long long K,
                      const void *A, long long a_sm, long long a_sk,
                      const void *B, long long b_sk, long long b_sn,
                      void *C, long long c_sm, const float *bias, int operands_bf16, int flags);

/* Diagnostics: runs a one-thread kernel that waits, with a short limit, on a barrier nothing
 * arrives at -- the situation every barrier wait of the tensor-core kernels is bounded
 * against -- and checks that the wait gives up, records its code in the device error word
 * and returns, leaving the context usable.  Clears the error word again.  0 = as designed.
 * (No counterpart in polygrad.) */
int poly_b200_selftest_bounded_wait(void);

/* out[b,h,t,:] = softmax_k(q[b,t,h,:] . k[b,k,h,:] * scale + mask[t,k]) . v[b,k,h,:]
 * as one kernel (the T x T scores never reach memory): the arithmetic of the
 * six-kernel chain polygrad's GPT-2 builder schedules
 * (src/modelzoo/models/gpt2.c:402-434) under the bf16 contraction policy.
 * q, k, v float32 [B][T][H][64]; mask float32 [T][T]; out float32 [B][H][T][64].
 * Head size 64, T a multiple of 128 up to 8192.  Blocks of 128 keys whose mask
 * tile is one value far enough below every row's running maximum to contribute
 * exactly nothing (the -1e9 triangle of a causal mask) are left out; the result
 * is bit for bit that of processing them (POLY_B200_ATTN_SKIP=0 processes all).
 * Stream-ordered; 0 / -1. */
int poly_b200_attention(const float *q, const float *k, const float *v, const float *mask, float scale,
                        float *out, int B, int H, int T);

/* No counterpart in polygrad.  The same bf16 tensor-core contraction as
 * poly_b200_gemm under the bf16 policy (float32 operands rounded to bfloat16,
 * fp32 products and sums), for callers that cannot let the library allocate:
 * inside a stream capture, in a process whose device memory is fully committed,
 * or where a driver allocation's implicit synchronisation is not acceptable.
 * It calls no cudaMalloc / cudaFree and does not touch the runtime's pool; the
 * converted operands go into a fixed array of POLY_B200_NOALLOC_SCRATCH_BYTES
 * that belongs to the library image (each GPU that loads the library holds it
 * until the process exits).  Sizes with (M + N) * roundup8(K) * 2 bytes beyond
 * that are rejected with -1 and a message.  The first call on a device looks up
 * the array's device address; make that call before any stream capture.  All
 * calls share the array: calls that overlap on the GPU (different streams or
 * processes sharing a context) race; on the library's single stream they do not.
 * K >= 16. */
#define POLY_B200_NOALLOC_SCRATCH_BYTES (32u << 20)
int poly_b200_gemm_noalloc(long long M, long long N, long long K,
                           const float *A, long long a_sm, long long a_sk,
                           const float *B, long long b_sk, long long b_sn,
                           float *C, long long c_sm, const float *bias, int relu);

/* Wait for all enqueued work.  0 / -1. */
int  poly_b200_synchronize(void);

/* The internal stream as a cudaStream_t. */
void *poly_b200_stream(void);

/* Page-locked host memory for fast copies (cudaHostAlloc). */
void *poly_b200_host_alloc(size_t bytes);
void  poly_b200_host_free(void *p);

/* Deferred readbacks.  polygrad reads an instance buffer back synchronously
 * (poly_instance_readback_buf -> poly_cuda_copy_dtoh, src/instance.c:479-501).  After
 * poly_b200_readback_defer(1) a copy_dtoh of at least 1 MiB into page-locked host memory
 * (poly_b200_host_alloc) returns at once: the source is snapshotted on the device and crosses
 * PCIe on a second stream while later launches run; the bytes are in place after
 * poly_b200_readback_wait().  At most two such copies are in flight; the caller alternates
 * between two host buffers.  0 / -1. */
int poly_b200_readback_defer(int on);
int poly_b200_readback_wait(void);

/* ── data-parallel ranks (no counterpart in polygrad, whose CUDA runtime drives device 0 of
 * one process only, src/runtime_cuda.c:192-243) ─────────────────────────────────────────
 * One process per GPU; ranks hold replicas of the weights and disjoint batch rows and exchange
 * nothing while a forward runs.  The one collective is the gather of results to a root rank,
 * over NCCL point-to-point calls on a second stream (NCCL is loaded with dlopen on first use).
 *
 * poly_b200_comm_unique_id   rank 0 makes an id (returns its size, <= 128 bytes) and hands it to
 *                            the other ranks by whatever means the launcher offers;
 * poly_b200_comm_init        every rank joins; the runtime's device is the rank's device;
 * poly_b200_gather_async     snapshots `bytes` at src on the main stream and sends them to the
 *                            root behind whatever is launched next; on the root, rank r's bytes
 *                            land at root_dst + poly_b200_gather_offset(r, bytes).  The root's
 *                            buffer must stay untouched until the transfers have finished;
 * poly_b200_comm_join        makes the main stream wait for the transfers enqueued so far;
 * poly_b200_comm_wait        blocks the host until they are done;
 * poly_b200_comm_max         replaces *value by its maximum over the ranks (step times).
 * All return 0 / -1 unless stated. */
int    poly_b200_comm_unique_id(void *id, size_t cap);
int    poly_b200_comm_init(int rank, int world, const void *id, size_t id_bytes);
int    poly_b200_comm_rank(void);
int    poly_b200_comm_world(void);
size_t poly_b200_gather_offset(int rank, size_t bytes);
int    poly_b200_gather_async(const void *src, size_t bytes, void *root_dst, int root);
int    poly_b200_comm_join(void);
int    poly_b200_comm_wait(void);
int    poly_b200_comm_max(double *value);
void   poly_b200_comm_destroy(void);

/* Data-parallel training steps.  polygrad builds one plan per training step in which every gradient is
 * fused into the update of its parameter (src/instance.c:1150-1215), so there is no gradient buffer to
 * reduce; for plain SGD, p - lr * g is linear in g and averaging the UPDATED parameters over the ranks
 * equals one step on the mean gradient.  While update averaging is on (also POLY_B200_AVERAGE_UPDATES=1),
 * every plan that updates bound buffers in place (poly_instance_train_step's) all-reduces each bound float32
 * buffer it writes -- parameters and the loss -- with ncclAvg.  A plan with less than 1 GB to average keeps its
 * CUDA graph and averages after the replay in a few NCCL groups; a larger one runs launch by launch and issues
 * each all-reduce right after the step that writes the buffer last, on the communicator's stream behind the rest
 * of the backward pass.  Either way the plan returns with the main stream ordered after the all-reduces.  With Adam the
 * moments are averaged as well, which is local-step averaging, not a step on the mean gradient.
 * Every rank must run the same plan: poly_b200_average_trace returns the number of all-reduces issued so far
 * and a running hash of their element counts, equal on all ranks when they did. */
void poly_b200_set_update_averaging(int on);
int  poly_b200_update_averaging(void);
int  poly_b200_average_enqueue(void *ptr, size_t count);   /* float32, in place, behind the main stream's work so far */
int  poly_b200_average_join(void);                          /* main stream waits for the all-reduces enqueued so far */
void poly_b200_average_group_bytes(size_t bytes);           /* enqueued buffers go out in NCCL groups of this size (0: 1 MB) or 64 buffers */
void poly_b200_average_trace(unsigned long long *calls, unsigned long long *hash);

/* This rank's share of a global batch as n_micro forwards of one instance (exported by
 * libpolygrad_b200.so; poly_instance_forward, polygrad src/instance.c:830, runs one batch of
 * the instance's static shape).  inputs[i] is micro-batch i's host array for the input buffer
 * `input_name`.  With gather != 0 each micro-batch's output buffer (index out_buf, out_bytes
 * bytes) is gathered to `root` behind the next micro-batch's compute; micro-batch i of rank r
 * is number poly_b200_shard_micro_index(r, world, i) = i * world + r of the global batch and
 * lands at root_dst + that number * out_bytes.  0 / -1. */
struct PolyInstance;
int poly_b200_shard_micro_index(int rank, int world, int i);
int poly_b200_forward_microbatches(struct PolyInstance *inst, const char *input_name, const float *const *inputs,
                                   int n_micro, int out_buf, size_t out_bytes, void *root_dst, int root, int gather);

/* `rows` rows of row_bytes, src_pitch bytes apart in one device buffer, into a dense device
 * buffer (polygrad's allocator has no device-to-device copy: copy_between is unimplemented,
 * src/exec_plan.c:290-294).  Stream-ordered; 0 / -1. */
int poly_b200_copy_rows(unsigned long long dst, unsigned long long src, size_t row_bytes, size_t src_pitch, size_t rows);

/* Device address that the most recent poly_cuda_copy_dtoh read from.  polygrad's
 * instance API hides device handles; a one-element readback followed by this
 * call tells a caller where an instance buffer lives (for NCCL, for example). */
unsigned long long poly_b200_last_dtoh_src(void);

/* Release cached free blocks of the pool back to the driver. */
void poly_b200_trim(void);

/* Sizes of the pool's free blocks, i.e. what the next poly_cuda_alloc calls can be served
 * from without a driver allocation: returns their count and writes the first `cap` sizes.
 * Scratch that a captured CUDA graph addresses is never among them (it stays with the graph
 * until the plan is freed or recaptured; polygrad keeps a plan's intermediates for the life
 * of the plan in the same way, src/exec_plan.c:860-881, 1062). */
int poly_b200_pool_free_sizes(unsigned long long *sizes, int cap);

/* Tells the runtime about an access to a device buffer made outside poly_cuda_launch
 * (mode 'r' read, 'w' partial write, 'W' whole-buffer overwrite, 'b' read and write): a zero
 * fill recorded by poly_cuda_memset is carried out (or dropped before 'W') and a written
 * buffer's converted operand copies are invalidated.  Host-side bookkeeping; 0 / -1. */
int poly_b200_note_access(const void *ptr, char mode);

/* CUDA events on the internal stream, for timing. */
void *poly_b200_event_create(void);
int   poly_b200_event_record(void *event);
float poly_b200_event_elapsed_ms(void *start, void *stop); /* waits for stop; <0 on error */
void  poly_b200_event_destroy(void *event);

/* Per-launch device timing: between begin and end every kernel launch of the
 * library is bracketed by CUDA events on its stream (plans run launch by launch
 * instead of as a graph); end waits and returns the summed kernel time in ms. */
void   poly_b200_timing_begin(void);
double poly_b200_timing_end(int *n_launches);
int    poly_b200_timing_active(void);

/* Counters since process start (or since the last reset). */
typedef struct {
  uint64_t launches;            /* kernels launched by this library */
  uint64_t launches_precompiled;/* ... of which precompiled (GEMM, gather, copy, convert) */
  uint64_t launches_generated;  /* ... of which compiled at run time from rendered CUDA C */
  uint64_t memsets_elided;      /* zero fills dropped because the buffer was fully overwritten first */
  uint64_t memsets_executed;
  uint64_t bytes_allocated;     /* bytes currently held from the driver (live + cached) */
  uint64_t programs_compiled;   /* NVRTC compilations (cache misses) */
  uint64_t programs_cached;     /* programs served from the in-process or disk cache */
  uint64_t bytes_htod;          /* bytes copied host -> device by poly_cuda_copy_htod */
  uint64_t bytes_dtoh;          /* bytes copied device -> host by poly_cuda_copy_dtoh */
} PolyB200Stats;
void poly_b200_stats(PolyB200Stats *out);
void poly_b200_stats_reset(void);

/* Safetensors weights into an instance wherever its buffers live (exported by
 * libpolygrad_b200.so, which contains polygrad's instance code).  Replaces
 * poly_instance_import_weights (polygrad src/instance.c:522-550), which fills
 * the host arrays only -- stale once poly_instance_set_device(CUDA) has moved
 * the buffers -- and takes float32 files only.  Here F32, BF16 and F16 tensors
 * are accepted (16-bit ones are widened to the instance's float32 buffers),
 * float32 tensors of a device-resident instance go from the file bytes to the
 * device in one copy each, and len may exceed 2 GB.  Tensors are matched by
 * buffer name; unknown names are reported and skipped; a size mismatch or an
 * integer dtype is an error (-1).  *bytes_to_device (may be NULL) receives the
 * bytes copied to device buffers. */
struct PolyInstance;
int poly_b200_instance_import_weights(struct PolyInstance *inst, const unsigned char *data, long long len,
                                      long long *bytes_to_device);

/* Scheduled kernels that were cut into contraction and elementwise steps by the plans compiled so far
 * (exported by libpolygrad_b200.so).  A backward kernel in which the scheduler fused a computed operand
 * or several reductions into one kernel is run as: operand temporaries, one contraction per reduction,
 * an elementwise remainder.  POLY_B200_OUTLINE=0 switches the cut off; POLY_B200_OUTLINE_MIN_WORK sets
 * the multiply-adds a kernel's contractions must hold for it (default 4194304). */
long long poly_b200_kernels_cut(void);

/* The eager entry points (exported by libpolygrad_b200.so; declared in polygrad's src/frontend.h:424-430,
 * defined by the reference at src/frontend.c:2444, 2450, 2670, 2676 and here in backend/pb_eager.c):
 *   int  poly_realize_cuda(PolyCtx *, PolyUOp *sink, PolyBufferBinding *, int n)   host pointers in the bindings
 *   int  poly_cuda_copyback(PolyBufferBinding *, int n)    results left on the device -> host
 *   void poly_cuda_flush_buffers(void)                     drop what is left on the device, uncopied
 *   void poly_cuda_prog_cache_flush(void)                  drop the kept plans
 * poly_b200_eager_stats reports how many calls found a kept plan for their graph (compared by structure,
 * buffers by position) and how many compiled one, the plans kept now and the results now on the device.
 * Any pointer may be NULL. */
void poly_b200_eager_stats(unsigned long long *hits, unsigned long long *misses, int *plans_kept, int *buffers_resident);

/* Text of the last error reported by this library ("" if none). */
const char *poly_b200_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* POLY_B200_H */
