/*
 * pb_comm.cu -- the collectives of the data-parallel paths: gathering every
 * rank's logits to a root rank (forward), and averaging what a training step
 * wrote over the ranks (see the end of the file), over NVLink with NCCL.
 *
 * polygrad has no multi-device execution at all (its CUDA runtime is a singleton
 * on device 0, reference src/runtime_cuda.c:192-243).  Here one process drives one
 * GPU, ranks hold replicas of the weights and disjoint batch rows, and nothing is
 * exchanged while a forward runs.  What a rank produces is gathered afterwards:
 *
 *   main stream   forward i | snapshot i | forward i+1 | snapshot i+1 | ...
 *   comm stream               wait(i)  ncclSend/Recv i   wait(i+1) ...
 *
 * The result buffer of a plan is overwritten by the next forward, so the bytes to
 * send are first copied into one of two staging buffers on the main stream (a
 * device-to-device copy at HBM speed); the NCCL transfer then runs on a second
 * stream behind the next forward.  Only plain NCCL point-to-point calls are used:
 * no kernel of this library reads a peer's memory.
 *
 * NCCL is loaded with dlopen on first use, so the library has no link-time
 * dependency on it; a process that already loaded an NCCL (torch's) shares it.
 */
#include "pb_runtime.h"
#include "../../../include/poly_b200.h"

#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

static struct {
  void *lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*GroupStart)(void) = nullptr;
  ncclResult_t (*GroupEnd)(void) = nullptr;
  ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
} NC;

static struct {
  ncclComm_t comm = nullptr;
  int rank = -1, world = 0;
  cudaStream_t stream = nullptr;
  void *stage[2] = {nullptr, nullptr}; size_t stage_bytes[2] = {0, 0};
  cudaEvent_t ready[2] = {nullptr, nullptr}, done[2] = {nullptr, nullptr};
  bool used[2] = {false, false};
  int next = 0;
  /* averaging of updated buffers */
  cudaEvent_t avg_ready = nullptr, avg_done = nullptr;
  bool avg_pending = false;
  unsigned long long avg_calls = 0, avg_groups = 0, avg_trace = 1469598103934665603ull;
} CM;

static struct { void *ptr; size_t count; } g_avg_wait[64];
static int g_n_avg_wait = 0;
static size_t g_avg_wait_bytes = 0, g_avg_group_bytes = (size_t)1 << 20;

static bool load_nccl() {
  if (NC.lib) return true;
  const char *names[] = {"libnccl.so.2", "libnccl.so", nullptr};
  for (int i = 0; names[i] && !NC.lib; i++) NC.lib = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
  if (!NC.lib) { pb_set_error("cannot load libnccl.so.2: %s", dlerror()); return false; }
#define L(field, name) *(void **)(&NC.field) = dlsym(NC.lib, name); if (!NC.field) { pb_set_error("libnccl lacks %s", name); NC.lib = nullptr; return false; }
  L(GetUniqueId, "ncclGetUniqueId");
  L(CommInitRank, "ncclCommInitRank");
  L(CommDestroy, "ncclCommDestroy");
  L(GroupStart, "ncclGroupStart");
  L(GroupEnd, "ncclGroupEnd");
  L(Send, "ncclSend");
  L(Recv, "ncclRecv");
  L(AllReduce, "ncclAllReduce");
  L(GetErrorString, "ncclGetErrorString");
#undef L
  return true;
}

#define PB_NCCL(call)                                                          \
  do {                                                                         \
    ncclResult_t r_ = (call);                                                  \
    if (r_ != ncclSuccess) { pb_set_error("%s failed: %s", #call, NC.GetErrorString(r_)); return -1; } \
  } while (0)
#define PB_CU(call)                                                            \
  do {                                                                         \
    cudaError_t e_ = (call);                                                   \
    if (e_ != cudaSuccess) { pb_set_error("%s failed: %s", #call, cudaGetErrorString(e_)); return -1; } \
  } while (0)

extern "C" int poly_b200_comm_unique_id(void *id, size_t cap) {
  if (!id || cap < sizeof(ncclUniqueId)) { pb_set_error("poly_b200_comm_unique_id: needs %zu bytes", sizeof(ncclUniqueId)); return -1; }
  if (poly_cuda_init() == 0 && pb_dry_run()) { memset(id, 0, sizeof(ncclUniqueId)); return (int)sizeof(ncclUniqueId); }
  if (!load_nccl()) return -1;
  ncclUniqueId u;
  PB_NCCL(NC.GetUniqueId(&u));
  memcpy(id, &u, sizeof u);
  return (int)sizeof u;
}

extern "C" int poly_b200_comm_init(int rank, int world, const void *id, size_t id_bytes) {
  if (CM.comm) { pb_set_error("poly_b200_comm_init: already initialised"); return -1; }
  if (world < 1 || rank < 0 || rank >= world || !id || id_bytes < sizeof(ncclUniqueId)) { pb_set_error("poly_b200_comm_init: bad arguments"); return -1; }
  if (poly_cuda_init() != 0) return -1;
  if (pb_dry_run()) { CM.rank = rank; CM.world = world; return 0; }
  if (!load_nccl()) return -1;
  ncclUniqueId u;
  memcpy(&u, id, sizeof u);
  PB_NCCL(NC.CommInitRank(&CM.comm, world, u, rank));
  PB_CU(cudaStreamCreateWithFlags(&CM.stream, cudaStreamNonBlocking));
  for (int i = 0; i < 2; i++) {
    PB_CU(cudaEventCreateWithFlags(&CM.ready[i], cudaEventDisableTiming));
    PB_CU(cudaEventCreateWithFlags(&CM.done[i], cudaEventDisableTiming));
  }
  CM.rank = rank; CM.world = world;
  return 0;
}

extern "C" int poly_b200_comm_rank(void) { return CM.rank; }
extern "C" int poly_b200_comm_world(void) { return CM.world; }

/* Where rank r's `bytes` land in the root's buffer. */
extern "C" size_t poly_b200_gather_offset(int r, size_t bytes) { return (size_t)r * bytes; }

extern "C" int poly_b200_gather_async(const void *src, size_t bytes, void *root_dst, int root) {
  if (CM.world < 1) { pb_set_error("poly_b200_gather_async: call poly_b200_comm_init first"); return -1; }
  if (!src || bytes == 0 || root < 0 || root >= CM.world || (CM.rank == root && !root_dst)) { pb_set_error("poly_b200_gather_async: bad arguments"); return -1; }
  if (pb_dry_run()) { if (CM.rank == root) memcpy((char *)root_dst + poly_b200_gather_offset(root, bytes), src, bytes); return 0; }
  cudaStream_t main_stream = (cudaStream_t)poly_b200_stream();
  if (pb_note_read(src) != 0) return -1;
  if (CM.rank == root) {
    /* the root's own part needs no staging: it is copied into place on the main stream; the
     * receives below write disjoint parts of root_dst */
    if (poly_b200_note_access(root_dst, 'w') != 0) return -1;
    PB_CU(cudaMemcpyAsync((char *)root_dst + poly_b200_gather_offset(root, bytes), src, bytes, cudaMemcpyDeviceToDevice, main_stream));
    if (CM.world == 1) return 0;
    const int k = CM.next; CM.next ^= 1;
    PB_CU(cudaEventRecord(CM.ready[k], main_stream));
    PB_CU(cudaStreamWaitEvent(CM.stream, CM.ready[k], 0));
    PB_NCCL(NC.GroupStart());
    for (int r = 0; r < CM.world; r++)
      if (r != root) PB_NCCL(NC.Recv((char *)root_dst + poly_b200_gather_offset(r, bytes), bytes, ncclUint8, r, CM.comm, CM.stream));
    PB_NCCL(NC.GroupEnd());
    PB_CU(cudaEventRecord(CM.done[k], CM.stream));
    CM.used[k] = true;
    return 0;
  }
  const int k = CM.next; CM.next ^= 1;
  if (CM.stage_bytes[k] < bytes) {
    if (CM.stage[k]) { if (CM.used[k]) PB_CU(cudaEventSynchronize(CM.done[k])); pb_scratch_free(CM.stage[k]); }
    CM.stage[k] = pb_scratch_alloc(bytes);
    CM.stage_bytes[k] = CM.stage[k] ? bytes : 0;
    if (!CM.stage[k]) return -1;
  }
  if (CM.used[k]) PB_CU(cudaStreamWaitEvent(main_stream, CM.done[k], 0));      /* the send that last read this staging buffer */
  PB_CU(cudaMemcpyAsync(CM.stage[k], src, bytes, cudaMemcpyDeviceToDevice, main_stream));
  PB_CU(cudaEventRecord(CM.ready[k], main_stream));
  PB_CU(cudaStreamWaitEvent(CM.stream, CM.ready[k], 0));
  PB_NCCL(NC.Send(CM.stage[k], bytes, ncclUint8, root, CM.comm, CM.stream));
  PB_CU(cudaEventRecord(CM.done[k], CM.stream));
  CM.used[k] = true;
  return 0;
}

/* Makes the main stream wait for every transfer enqueued so far (so that an event recorded on
 * it afterwards covers them), without blocking the host. */
extern "C" int poly_b200_comm_join(void) {
  if (pb_dry_run() || !CM.stream) return 0;
  cudaStream_t main_stream = (cudaStream_t)poly_b200_stream();
  for (int k = 0; k < 2; k++)
    if (CM.used[k]) PB_CU(cudaStreamWaitEvent(main_stream, CM.done[k], 0));
  return 0;
}

extern "C" int poly_b200_comm_wait(void) {
  if (pb_dry_run() || !CM.stream) return 0;
  PB_CU(cudaStreamSynchronize(CM.stream));
  return 0;
}

/* max over ranks of one double (the step time), through NCCL on the comm stream */
extern "C" int poly_b200_comm_max(double *value) {
  if (!value) return -1;
  if (CM.world <= 1 || pb_dry_run()) return 0;
  double *d = (double *)pb_scratch_alloc(sizeof(double));
  if (!d) return -1;
  PB_CU(cudaMemcpyAsync(d, value, sizeof(double), cudaMemcpyHostToDevice, CM.stream));
  PB_NCCL(NC.AllReduce(d, d, 1, ncclFloat64, ncclMax, CM.comm, CM.stream));
  PB_CU(cudaMemcpyAsync(value, d, sizeof(double), cudaMemcpyDeviceToHost, CM.stream));
  PB_CU(cudaStreamSynchronize(CM.stream));
  pb_scratch_free(d);
  return 0;
}

extern "C" void poly_b200_comm_destroy(void) {
  if (CM.stream) cudaStreamSynchronize(CM.stream);
  for (int k = 0; k < 2; k++) {
    if (CM.stage[k]) pb_scratch_free(CM.stage[k]);
    CM.stage[k] = nullptr; CM.stage_bytes[k] = 0; CM.used[k] = false;
    if (CM.ready[k]) cudaEventDestroy(CM.ready[k]);
    if (CM.done[k]) cudaEventDestroy(CM.done[k]);
    CM.ready[k] = CM.done[k] = nullptr;
  }
  if (CM.comm && NC.CommDestroy) NC.CommDestroy(CM.comm);
  if (CM.stream) cudaStreamDestroy(CM.stream);
  if (CM.avg_ready) cudaEventDestroy(CM.avg_ready);
  if (CM.avg_done) cudaEventDestroy(CM.avg_done);
  CM.avg_ready = CM.avg_done = nullptr; CM.avg_pending = false;
  g_n_avg_wait = 0; g_avg_wait_bytes = 0;
  CM.comm = nullptr; CM.stream = nullptr; CM.rank = -1; CM.world = 0; CM.next = 0;
}

/* ── averaging what a training step wrote ────────────────────────────── */
/* polygrad fuses every gradient into the update of its parameter inside one
 * plan (reference src/instance.c:1150-1215: ASSIGN(p, p - lr * grad) per
 * parameter, all in one SINK), so a data-parallel step has no gradient buffer
 * to reduce.  For plain SGD the update is linear in the gradient:
 *     mean_r(p - lr * g_r) = p - lr * mean_r(g_r),
 * so averaging each parameter over the ranks right after its update gives
 * exactly the parameters of one step on the mean gradient.  The plan executor
 * calls poly_b200_average_enqueue after the last step that writes a bound
 * buffer: the all-reduces run on the second stream behind the rest of the
 * backward pass, and poly_b200_average_join makes the main stream wait for
 * all of them before the plan returns.  Every rank issues the same calls in
 * the same order (same plan), which is what NCCL requires;
 * poly_b200_average_trace exposes a running hash of the sizes to check that. */
/* Small buffers (biases, LayerNorm gains) wait for company: the all-reduces of up to 64 buffers or
 * 1 MB (poly_b200_average_group_bytes: when nothing is left to overlap with, larger groups mean
 * fewer launches) go out as one NCCL group behind one event.  The rule depends only on the sizes,
 * so every rank forms the same groups. */
extern "C" void poly_b200_average_group_bytes(size_t bytes) { g_avg_group_bytes = bytes ? bytes : ((size_t)1 << 20); }

static int average_flush(void) {
  if (g_n_avg_wait == 0) return 0;
  cudaStream_t main_stream = (cudaStream_t)poly_b200_stream();
  if (!CM.avg_ready) {
    PB_CU(cudaEventCreateWithFlags(&CM.avg_ready, cudaEventDisableTiming));
    PB_CU(cudaEventCreateWithFlags(&CM.avg_done, cudaEventDisableTiming));
  }
  PB_CU(cudaEventRecord(CM.avg_ready, main_stream));
  PB_CU(cudaStreamWaitEvent(CM.stream, CM.avg_ready, 0));
  const int n = g_n_avg_wait;
  g_n_avg_wait = 0; g_avg_wait_bytes = 0;
  PB_NCCL(NC.GroupStart());
  for (int i = 0; i < n; i++)
    PB_NCCL(NC.AllReduce(g_avg_wait[i].ptr, g_avg_wait[i].ptr, g_avg_wait[i].count, ncclFloat32, ncclAvg, CM.comm, CM.stream));
  PB_NCCL(NC.GroupEnd());
  CM.avg_pending = true;
  CM.avg_groups++;
  return 0;
}

extern "C" int poly_b200_average_enqueue(void *ptr, size_t count) {
  if (!ptr || count == 0) { pb_set_error("poly_b200_average_enqueue: bad arguments"); return -1; }
  CM.avg_calls++;
  CM.avg_trace = (CM.avg_trace ^ (unsigned long long)count) * 1099511628211ull;
  if (pb_dry_run() || CM.world <= 1) return 0;
  if (poly_b200_note_access(ptr, 'b') != 0) return -1;
  g_avg_wait[g_n_avg_wait].ptr = ptr; g_avg_wait[g_n_avg_wait].count = count;
  g_n_avg_wait++; g_avg_wait_bytes += count * sizeof(float);
  if (g_n_avg_wait == 64 || g_avg_wait_bytes >= g_avg_group_bytes) return average_flush();
  return 0;
}

extern "C" int poly_b200_average_join(void) {
  if (average_flush() != 0) return -1;
  if (!CM.avg_pending) return 0;
  cudaStream_t main_stream = (cudaStream_t)poly_b200_stream();
  PB_CU(cudaEventRecord(CM.avg_done, CM.stream));
  PB_CU(cudaStreamWaitEvent(main_stream, CM.avg_done, 0));
  CM.avg_pending = false;
  return 0;
}

extern "C" void poly_b200_average_trace(unsigned long long *calls, unsigned long long *hash) {
  if (calls) *calls = CM.avg_calls;
  if (hash) *hash = CM.avg_trace;
}
