/*
 * pb_runtime.cu -- device runtime behind polygrad's CUDA backend symbols.
 *
 * Replaces polygrad src/runtime_cuda.c (driver-API singleton, cuMemAlloc per
 * buffer, synchronous copies, NVRTC to PTX, launch on the NULL stream followed
 * by cuCtxSynchronize for every kernel).  Design here:
 *   - one non-blocking stream; launches, copies and fills are stream-ordered
 *     and the host only waits in copy_dtoh / poly_b200_synchronize;
 *   - a size-class pool over cudaMalloc, so plan intermediates and scratch
 *     operands are recycled without driver calls;
 *   - whole-buffer zero fills (polygrad zeroes every plan intermediate before
 *     every run, src/exec_plan.c:946-963) are recorded and dropped when the next
 *     access to the buffer is a kernel that overwrites all of it;
 *   - programs are either precompiled sm_100a kernels selected by a text header,
 *     or CUDA C compiled by NVRTC straight to sm_100a machine code, cached in
 *     the process and on disk;
 *   - no CPU fallback: without a device every entry point reports an error.
 *     POLY_B200_DRYRUN=1 (host-logic tests only) accepts programs and ignores
 *     launches, with host memory standing in for device buffers.
 */
#include "pb_runtime.h"
#include "../../../include/poly_b200.h"

#include <dlfcn.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>
#include <unordered_map>
#include <memory>
#include <sstream>
#include <vector>

/* ── errors ──────────────────────────────────────────────────────────── */
static char g_last_error[1024];

void pb_set_error(const char *fmt, ...) {
  va_list ap; va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof g_last_error, fmt, ap);
  va_end(ap);
  fprintf(stderr, "polygrad: cuda: %s\n", g_last_error);
}

extern "C" const char *poly_b200_last_error(void) { return g_last_error; }

#define PB_CUDA(call)                                                          \
  do {                                                                         \
    cudaError_t e_ = (call);                                                   \
    if (e_ != cudaSuccess) {                                                   \
      pb_set_error("%s failed: %s", #call, cudaGetErrorString(e_));            \
      return -1;                                                               \
    }                                                                          \
  } while (0)

/* ── state ───────────────────────────────────────────────────────────── */
struct Buf {
  size_t size;        /* rounded size of the block */
  size_t requested;
  bool pending_zero;
  uint64_t version;
};

struct Runtime {
  bool inited = false, ok = false, dry = false;
  int device = -1;
  cudaStream_t stream = nullptr;
  std::map<uintptr_t, Buf> live;
  std::multimap<size_t, void *> free_blocks;
  size_t held = 0;
  uint64_t version_counter = 1;
  int n_pending = 0;
  bool force_sync = false;
  bool capturing = false, capture_failed = false;
  /* blocks given back while a stream capture is open: their addresses are baked into the
   * captured work, so they stay out of the free list until the graph is destroyed */
  std::vector<std::pair<size_t, void *>> capture_hold;
  uint64_t pool_epoch = 1;       /* bumps when cached blocks go back to the driver */
  /* deferred readbacks: device-to-host copies that run on a second stream behind later work */
  bool defer = false;
  cudaStream_t copy_stream = nullptr;
  void *defer_stage[2] = {nullptr, nullptr}; size_t defer_bytes[2] = {0, 0};
  cudaEvent_t defer_ready[2] = {nullptr, nullptr}, defer_done[2] = {nullptr, nullptr};
  bool defer_used[2] = {false, false};
  int defer_next = 0;
  PolyB200Stats st{};
};
static Runtime R;

bool pb_dry_run(void) { return R.dry; }

void pb_count_launch(bool precompiled, int n) {
  R.st.launches += (uint64_t)n;
  if (precompiled) R.st.launches_precompiled += (uint64_t)n; else R.st.launches_generated += (uint64_t)n;
}

/* ── driver + NVRTC entry points, loaded on demand ───────────────────── */
typedef int CUresult_;
typedef struct CUmod_st *CUmodule_;
typedef struct CUfunc_st *CUfunction_;
typedef struct CUstream_st *CUstream_;
static struct {
  void *lib = nullptr;
  CUresult_ (*ModuleLoadData)(CUmodule_ *, const void *) = nullptr;
  CUresult_ (*ModuleGetFunction)(CUfunction_ *, CUmodule_, const char *) = nullptr;
  CUresult_ (*ModuleUnload)(CUmodule_) = nullptr;
  CUresult_ (*LaunchKernel)(CUfunction_, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                            unsigned, CUstream_, void **, void **) = nullptr;
  CUresult_ (*GetErrorString)(CUresult_, const char **) = nullptr;
} DRV;

typedef struct _nvrtcProgram *nvrtcProgram_;
static struct {
  void *lib = nullptr;
  int (*CreateProgram)(nvrtcProgram_ *, const char *, const char *, int, const char *const *, const char *const *) = nullptr;
  int (*CompileProgram)(nvrtcProgram_, int, const char *const *) = nullptr;
  int (*GetCUBINSize)(nvrtcProgram_, size_t *) = nullptr;
  int (*GetCUBIN)(nvrtcProgram_, char *) = nullptr;
  int (*GetProgramLogSize)(nvrtcProgram_, size_t *) = nullptr;
  int (*GetProgramLog)(nvrtcProgram_, char *) = nullptr;
  int (*DestroyProgram)(nvrtcProgram_ *) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  int (*Version)(int *, int *) = nullptr;
} RTC;

static bool load_driver() {
  if (DRV.lib) return true;
  DRV.lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
  if (!DRV.lib) { pb_set_error("cannot load libcuda.so.1: %s", dlerror()); return false; }
#define L(field, name) *(void **)(&DRV.field) = dlsym(DRV.lib, name); if (!DRV.field) { pb_set_error("libcuda lacks %s", name); return false; }
  L(ModuleLoadData, "cuModuleLoadData");
  L(ModuleGetFunction, "cuModuleGetFunction");
  L(ModuleUnload, "cuModuleUnload");
  L(LaunchKernel, "cuLaunchKernel");
  L(GetErrorString, "cuGetErrorString");
#undef L
  return true;
}

static bool load_nvrtc() {
  if (RTC.lib) return true;
  const char *names[] = {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12", nullptr};
  for (int i = 0; names[i] && !RTC.lib; i++) RTC.lib = dlopen(names[i], RTLD_NOW);
  if (!RTC.lib) { pb_set_error("cannot load libnvrtc.so.12: %s", dlerror()); return false; }
#define L(field, name) *(void **)(&RTC.field) = dlsym(RTC.lib, name); if (!RTC.field) { pb_set_error("libnvrtc lacks %s", name); return false; }
  L(CreateProgram, "nvrtcCreateProgram");
  L(CompileProgram, "nvrtcCompileProgram");
  L(GetCUBINSize, "nvrtcGetCUBINSize");
  L(GetCUBIN, "nvrtcGetCUBIN");
  L(GetProgramLogSize, "nvrtcGetProgramLogSize");
  L(GetProgramLog, "nvrtcGetProgramLog");
  L(DestroyProgram, "nvrtcDestroyProgram");
  L(GetErrorString, "nvrtcGetErrorString");
  L(Version, "nvrtcVersion");
#undef L
  return true;
}

/* ── init ────────────────────────────────────────────────────────────── */
static int requested_device = -1;

extern "C" int poly_b200_set_device(int device) {
  if (R.inited && R.device != device) {
    pb_set_error("poly_b200_set_device(%d) after the runtime was initialised on device %d", device, R.device);
    return -1;
  }
  requested_device = device;
  return 0;
}

extern "C" int poly_b200_device(void) { return R.device; }

extern "C" int poly_cuda_init(void) {
  if (R.inited) return R.ok ? 0 : -1;
  R.inited = true;
  const char *dry = getenv("POLY_B200_DRYRUN");
  R.dry = dry && dry[0] && dry[0] != '0';
  const char *fs = getenv("POLY_B200_SYNC");
  R.force_sync = fs && fs[0] && fs[0] != '0';
  if (R.dry) { R.ok = true; R.device = 0; return 0; }
  int dev = requested_device;
  if (dev < 0) { const char *e = getenv("POLY_B200_DEVICE"); if (e && e[0]) dev = atoi(e); }
  if (dev < 0) { const char *e = getenv("LOCAL_RANK"); if (e && e[0]) dev = atoi(e); }
  if (dev < 0) dev = 0;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    pb_set_error("no CUDA device (%s)", e != cudaSuccess ? cudaGetErrorString(e) : "count is 0");
    cudaGetLastError();
    return -1;
  }
  if (dev >= count) { pb_set_error("device %d requested, %d present", dev, count); return -1; }
  PB_CUDA(cudaSetDevice(dev));
  PB_CUDA(cudaFree(0));
  cudaDeviceProp prop;
  PB_CUDA(cudaGetDeviceProperties(&prop, dev));
  if (prop.major != 10) {
    pb_set_error("device %d is sm_%d%d; this library holds sm_100a code only", dev, prop.major, prop.minor);
    return -1;
  }
  PB_CUDA(cudaStreamCreateWithFlags(&R.stream, cudaStreamNonBlocking));
  if (!load_driver()) return -1;
  R.device = dev;
  R.ok = true;
  return 0;
}

extern "C" bool poly_cuda_available(void) { return poly_cuda_init() == 0; }

static inline bool ready() { return (R.inited || poly_cuda_init() == 0) && R.ok; }

extern "C" void *poly_b200_stream(void) { return ready() ? (void *)R.stream : nullptr; }

static bool g_tc_used = false;
void pb_tc_mark_used(void) { g_tc_used = true; }

static int check_device_flags(void) {
  if (!g_tc_used) return 0;
  int code = pb_gemm_tc_error();
  if (code == 0) code = pb_attention_error();
  if (code != 0) { pb_set_error("tensor-core kernel: a barrier wait ran out (code %d); results are invalid", code); return -1; }
  return 0;
}

extern "C" int poly_b200_synchronize(void) {
  if (!ready()) return -1;
  if (R.dry) return 0;
  PB_CUDA(cudaStreamSynchronize(R.stream));
  return check_device_flags();
}

extern "C" int poly_cuda_sync(void) {
  if (!ready()) return -1;
  if (R.dry) return 0;
  if (R.force_sync) return poly_b200_synchronize();
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) { pb_set_error("asynchronous error: %s", cudaGetErrorString(e)); return -1; }
  return 0;
}

/* ── pool ────────────────────────────────────────────────────────────── */
static size_t round_size(size_t b) {
  if (b == 0) b = 1;
  if (b < ((size_t)1 << 20)) return (b + 511) & ~(size_t)511;
  return (b + ((size_t)2 << 20) - 1) & ~(((size_t)2 << 20) - 1);
}

static void *pool_alloc(size_t bytes) {
  size_t rs = round_size(bytes);
  void *p = nullptr;
  auto it = R.free_blocks.find(rs);
  if (R.capturing) {
    /* a block this capture already used and released: the captured work is one ordered chain,
     * so a later node may use it again */
    for (size_t i = 0; i < R.capture_hold.size() && !p; i++)
      if (R.capture_hold[i].first == rs) { p = R.capture_hold[i].second; R.capture_hold.erase(R.capture_hold.begin() + (long)i); }
  }
  if (p) {}
  else if (it != R.free_blocks.end()) { p = it->second; R.free_blocks.erase(it); }
  else if (R.dry) { p = calloc(1, rs); }
  else if (R.capturing) {
    /* no driver allocation inside a stream capture: the caller abandons the capture */
    R.capture_failed = true;
    return nullptr;
  }
  else {
    cudaError_t e = cudaMalloc(&p, rs);
    if (e != cudaSuccess) {
      /* give cached blocks back and retry once */
      cudaGetLastError();
      poly_b200_trim();
      e = cudaMalloc(&p, rs);
      if (e != cudaSuccess) { cudaGetLastError(); pb_set_error("cudaMalloc(%zu) failed: %s", rs, cudaGetErrorString(e)); return nullptr; }
    }
    R.held += rs;
  }
  if (!p) return nullptr;
  Buf b{rs, bytes, false, R.version_counter++};
  R.live[(uintptr_t)p] = b;
  R.st.bytes_allocated = R.held;
  return p;
}

static void pool_free(void *p) {
  auto it = R.live.find((uintptr_t)p);
  if (it == R.live.end()) return;
  if (it->second.pending_zero) R.n_pending--;
  if (R.capturing) R.capture_hold.push_back({it->second.size, p});
  else R.free_blocks.insert({it->second.size, p});
  R.live.erase(it);
}

extern "C" void poly_b200_trim(void) {
  if (!R.ok) return;
  R.pool_epoch++;
  if (!R.dry && !R.free_blocks.empty()) cudaStreamSynchronize(R.stream);
  for (auto &kv : R.free_blocks) {
    if (R.dry) free(kv.second); else { cudaFree(kv.second); R.held -= kv.first; }
  }
  R.free_blocks.clear();
  R.st.bytes_allocated = R.held;
}

/* Sizes of the blocks the pool could hand out without asking the driver (diagnostics, tests).
 * Returns how many there are; writes the first `cap` sizes. */
extern "C" int poly_b200_pool_free_sizes(unsigned long long *sizes, int cap) {
  int n = 0;
  for (auto &kv : R.free_blocks) { if (sizes && n < cap) sizes[n] = kv.first; n++; }
  return n;
}

extern "C" unsigned long long poly_cuda_alloc(size_t bytes) {
  if (!ready()) return 0;
  return (unsigned long long)(uintptr_t)pool_alloc(bytes);
}

extern "C" void poly_cuda_free(unsigned long long ptr) {
  if (!R.ok || !ptr) return;
  pool_free((void *)(uintptr_t)ptr);
}

void *pb_scratch_alloc(size_t bytes) { return ready() ? pool_alloc(bytes) : nullptr; }
void pb_scratch_free(void *p) { if (p) pool_free(p); }

/* The tracked allocation containing p, or end(). */
static std::map<uintptr_t, Buf>::iterator find_buf(const void *p) {
  uintptr_t a = (uintptr_t)p;
  auto it = R.live.upper_bound(a);
  if (it == R.live.begin()) return R.live.end();
  --it;
  if (a >= it->first && a < it->first + it->second.size) return it;
  return R.live.end();
}

uint64_t pb_buffer_version(const void *p) {
  auto it = find_buf(p);
  return it == R.live.end() ? 0 : it->second.version;
}

static int materialize_zero(std::map<uintptr_t, Buf>::iterator it) {
  if (!it->second.pending_zero) return 0;
  it->second.pending_zero = false;
  R.n_pending--;
  R.st.memsets_executed++;
  if (R.dry) { memset((void *)it->first, 0, it->second.requested); return 0; }
  PB_CUDA(cudaMemsetAsync((void *)it->first, 0, it->second.requested, R.stream));
  return 0;
}

/* Note an access before enqueueing it.  mode: 'r' read, 'w' partial write,
 * 'b' read+write, 'W' whole-buffer overwrite. */
static int note_access(const void *p, char mode) {
  auto it = find_buf(p);
  if (it == R.live.end()) return 0;
  if (it->second.pending_zero) {
    if (mode == 'W' && (uintptr_t)p == it->first) {
      it->second.pending_zero = false; R.n_pending--; R.st.memsets_elided++;
    } else if (materialize_zero(it) != 0) return -1;
  }
  if (mode != 'r') it->second.version = R.version_counter++;
  return 0;
}

/* The same for code outside this file.  Reads are free while no zero fill is pending. */
extern "C" int poly_b200_note_access(const void *p, char mode) {
  if (!R.ok) return 0;
  if (mode == 'r' && R.n_pending == 0) return 0;
  return note_access(p, mode);
}

/* A write of `bytes` starting at p: a whole-buffer overwrite when it covers the allocation. */
int pb_note_write(const void *p, size_t bytes) {
  auto it = find_buf(p);
  if (it == R.live.end()) return 0;
  const bool whole = (uintptr_t)p == it->first && bytes >= it->second.requested;
  return note_access(p, whole ? 'W' : 'w');
}
int pb_note_read(const void *p) { return p ? poly_b200_note_access(p, 'r') : 0; }

extern "C" int poly_cuda_memset(unsigned long long ptr, unsigned char val, size_t bytes) {
  if (!ready()) return -1;
  void *p = (void *)(uintptr_t)ptr;
  auto it = find_buf(p);
  if (it != R.live.end()) {
    it->second.version = R.version_counter++;
    if (val == 0 && (uintptr_t)p == it->first && bytes >= it->second.requested) {
      if (!it->second.pending_zero) { it->second.pending_zero = true; R.n_pending++; }
      return 0;
    }
    if (materialize_zero(it) != 0) return -1;
  }
  R.st.memsets_executed++;
  if (R.dry) { memset(p, val, bytes); return 0; }
  PB_CUDA(cudaMemsetAsync(p, val, bytes, R.stream));
  return 0;
}

extern "C" int poly_cuda_copy_htod(unsigned long long dst, const void *src, size_t bytes) {
  if (!ready()) return -1;
  void *p = (void *)(uintptr_t)dst;
  auto it = find_buf(p);
  char mode = (it != R.live.end() && (uintptr_t)p == it->first && bytes >= it->second.requested) ? 'W' : 'w';
  if (note_access(p, mode) != 0) return -1;
  R.st.bytes_htod += bytes;
  if (R.dry) { memcpy(p, src, bytes); return 0; }
  /* pageable sources are staged before the call returns, pinned ones are not:
   * wait so that the caller may reuse src in both cases */
  PB_CUDA(cudaMemcpyAsync(p, src, bytes, cudaMemcpyHostToDevice, R.stream));
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, src) == cudaSuccess && attr.type == cudaMemoryTypeHost)
    PB_CUDA(cudaStreamSynchronize(R.stream));
  else cudaGetLastError();
  return 0;
}

/* Is p ordinary (pageable) host memory, which a kernel cannot address?  Memory
 * of this library's pool, other device allocations, pinned and managed memory
 * all answer no. */
extern "C" int poly_b200_ptr_on_host(const void *p) {
  if (!p || !ready()) return 0;
  if (find_buf(p) != R.live.end()) return 0;
  if (R.dry) return 1;
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) { cudaGetLastError(); return 1; }
  return attr.type == cudaMemoryTypeUnregistered ? 1 : 0;
}

static unsigned long long g_last_dtoh_src = 0;
extern "C" unsigned long long poly_b200_last_dtoh_src(void) { return g_last_dtoh_src; }

extern "C" void *poly_b200_host_alloc(size_t bytes) {
  if (!ready()) return nullptr;
  if (R.dry) return malloc(bytes ? bytes : 1);
  void *p = nullptr;
  if (cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocDefault) != cudaSuccess) {
    pb_set_error("cudaHostAlloc(%zu) failed: %s", bytes, cudaGetErrorString(cudaGetLastError()));
    return nullptr;
  }
  return p;
}
extern "C" void poly_b200_host_free(void *p) {
  if (!p) return;
  if (R.dry) free(p); else cudaFreeHost(p);
}

/* ── deferred readbacks ──────────────────────────────────────────────────
 * polygrad reads results back synchronously (poly_instance_readback_buf ->
 * poly_cuda_copy_dtoh, reference src/instance.c:479-501), so a caller that wants the
 * full logits on the host pays compute + PCIe per step.  While deferral is on, a
 * copy_dtoh whose destination is page-locked host memory returns at once: the source
 * is snapshotted into one of two device staging buffers on the main stream (a
 * device-to-device copy, about 0.5 ms for 1.65 GB) and copied to the host from there
 * on a second stream, so the next steps run while the bytes cross PCIe.  The data is
 * in place after poly_b200_readback_wait(). */
static int defer_dtoh(void *dst, const void *src, size_t bytes) {
  if (!R.copy_stream) {
    PB_CUDA(cudaStreamCreateWithFlags(&R.copy_stream, cudaStreamNonBlocking));
    for (int i = 0; i < 2; i++) {
      PB_CUDA(cudaEventCreateWithFlags(&R.defer_ready[i], cudaEventDisableTiming));
      PB_CUDA(cudaEventCreateWithFlags(&R.defer_done[i], cudaEventDisableTiming));
    }
  }
  const int k = R.defer_next;
  R.defer_next ^= 1;
  if (R.defer_bytes[k] < bytes) {
    if (R.defer_stage[k]) {
      if (R.defer_used[k]) PB_CUDA(cudaEventSynchronize(R.defer_done[k]));
      pool_free(R.defer_stage[k]);
    }
    R.defer_stage[k] = pool_alloc(bytes);
    R.defer_bytes[k] = R.defer_stage[k] ? bytes : 0;
    if (!R.defer_stage[k]) return -1;
  }
  /* the staging buffer is free again when the copy that last read it has finished */
  if (R.defer_used[k]) PB_CUDA(cudaStreamWaitEvent(R.stream, R.defer_done[k], 0));
  PB_CUDA(cudaMemcpyAsync(R.defer_stage[k], src, bytes, cudaMemcpyDeviceToDevice, R.stream));
  PB_CUDA(cudaEventRecord(R.defer_ready[k], R.stream));
  PB_CUDA(cudaStreamWaitEvent(R.copy_stream, R.defer_ready[k], 0));
  PB_CUDA(cudaMemcpyAsync(dst, R.defer_stage[k], bytes, cudaMemcpyDeviceToHost, R.copy_stream));
  PB_CUDA(cudaEventRecord(R.defer_done[k], R.copy_stream));
  R.defer_used[k] = true;
  return 0;
}

extern "C" int poly_b200_readback_defer(int on) {
  if (!ready()) return -1;
  R.defer = on != 0 && !R.dry;
  return 0;
}

extern "C" int poly_b200_readback_wait(void) {
  if (!ready()) return -1;
  if (R.dry || !R.copy_stream) return 0;
  PB_CUDA(cudaStreamSynchronize(R.copy_stream));
  return check_device_flags();
}

extern "C" int poly_cuda_copy_dtoh(void *dst, unsigned long long src, size_t bytes) {
  if (!ready()) return -1;
  void *p = (void *)(uintptr_t)src;
  g_last_dtoh_src = src;
  if (note_access(p, 'r') != 0) return -1;
  R.st.bytes_dtoh += bytes;
  if (R.dry) { memcpy(dst, p, bytes); return 0; }
  if (R.defer && !R.capturing && bytes >= ((size_t)1 << 20)) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, dst) == cudaSuccess && attr.type == cudaMemoryTypeHost) return defer_dtoh(dst, p, bytes);
    cudaGetLastError();
  }
  PB_CUDA(cudaMemcpyAsync(dst, p, bytes, cudaMemcpyDeviceToHost, R.stream));
  PB_CUDA(cudaStreamSynchronize(R.stream));
  return check_device_flags();
}

/* `rows` rows of row_bytes each, src_pitch apart in a device buffer, into a dense device buffer
 * (the last position's logits of every sequence, for example).  Stream-ordered. */
extern "C" int poly_b200_copy_rows(unsigned long long dst, unsigned long long src, size_t row_bytes, size_t src_pitch, size_t rows) {
  if (!ready()) return -1;
  void *d = (void *)(uintptr_t)dst; const void *s = (const void *)(uintptr_t)src;
  if (note_access(s, 'r') != 0 || note_access(d, 'w') != 0) return -1;
  if (R.dry) { for (size_t r = 0; r < rows; r++) memcpy((char *)d + r * row_bytes, (const char *)s + r * src_pitch, row_bytes); return 0; }
  PB_CUDA(cudaMemcpy2DAsync(d, row_bytes, s, src_pitch, row_bytes, rows, cudaMemcpyDeviceToDevice, R.stream));
  return 0;
}

/* ── events ──────────────────────────────────────────────────────────── */
extern "C" void *poly_b200_event_create(void) {
  if (!ready() || R.dry) return nullptr;
  cudaEvent_t ev;
  if (cudaEventCreate(&ev) != cudaSuccess) return nullptr;
  return (void *)ev;
}
extern "C" int poly_b200_event_record(void *event) {
  if (!ready() || !event) return -1;
  PB_CUDA(cudaEventRecord((cudaEvent_t)event, R.stream));
  return 0;
}
extern "C" float poly_b200_event_elapsed_ms(void *start, void *stop) {
  if (!start || !stop) return -1.0f;
  if (cudaEventSynchronize((cudaEvent_t)stop) != cudaSuccess) return -1.0f;
  float ms = -1.0f;
  if (cudaEventElapsedTime(&ms, (cudaEvent_t)start, (cudaEvent_t)stop) != cudaSuccess) return -1.0f;
  return ms;
}
extern "C" void poly_b200_event_destroy(void *event) { if (event) cudaEventDestroy((cudaEvent_t)event); }

extern "C" void poly_b200_stats(PolyB200Stats *out) { if (out) { R.st.bytes_allocated = R.held; *out = R.st; } }
extern "C" void poly_b200_stats_reset(void) { uint64_t held = R.held; R.st = PolyB200Stats{}; R.st.bytes_allocated = held; }

/* ── header parsing ──────────────────────────────────────────────────── */
static const std::string EMPTY;
const std::string &PbHeader::get(const char *k) const {
  auto it = kv.find(k); return it == kv.end() ? EMPTY : it->second;
}
long long PbHeader::geti(const char *k, long long dflt) const {
  auto it = kv.find(k); if (it == kv.end() || it->second.empty()) return dflt;
  return atoll(it->second.c_str());
}
std::vector<long long> PbHeader::getv(const char *k) const {
  std::vector<long long> v; std::istringstream ss(get(k)); long long x;
  while (ss >> x) v.push_back(x);
  return v;
}

static bool parse_header(const char *src, PbHeader &h) {
  if (strncmp(src, "//PB200 ", 8) != 0) return false;
  const char *p = src;
  while (p[0] == '/' && p[1] == '/') {
    const char *eol = strchr(p, '\n');
    size_t len = eol ? (size_t)(eol - p) : strlen(p);
    std::string line(p + 2, len - 2);
    size_t sp = line.find(' ');
    if (sp == std::string::npos) h.kv[line] = "";
    else h.kv[line.substr(0, sp)] = line.substr(sp + 1);
    if (!eol) break;
    p = eol + 1;
  }
  return true;
}

/* ── run-time compiled programs ──────────────────────────────────────── */
struct Module { CUmodule_ mod = nullptr; CUfunction_ fn = nullptr; };
static std::unordered_map<uint64_t, std::shared_ptr<Module>> g_modules;
static std::unordered_map<uint64_t, bool> g_dry_compiled;

struct WorkTerm { long long c; std::vector<int> vars; };

struct PolyCudaProgram {
  enum Kind { JIT, AOT } kind = JIT;
  std::string name;
  /* JIT */
  std::shared_ptr<Module> module;
  int n_params = 0, n_vars = 0;
  bool group_launch = false;
  int block = 256, group = 1;
  std::vector<WorkTerm> work;   /* max over terms */
  std::string rw;               /* per param */
  /* AOT */
  PbAotProgram *aot = nullptr;
  ~PolyCudaProgram() { delete aot; }
};

static uint64_t fnv1a(const void *data, size_t n, uint64_t h = 1469598103934665603ULL) {
  const unsigned char *p = (const unsigned char *)data;
  for (size_t i = 0; i < n; i++) { h ^= p[i]; h *= 1099511628211ULL; }
  return h;
}

static std::string cache_dir() {
  const char *off = getenv("POLY_B200_CACHE");
  if (off && off[0] == '0') return "";
  const char *d = getenv("POLY_B200_CACHE_DIR");
  std::string dir;
  if (d && d[0]) dir = d;
  else { const char *home = getenv("HOME"); if (!home || !home[0]) return ""; dir = std::string(home) + "/.cache/polygrad_b200"; }
  std::string parent = dir.substr(0, dir.find_last_of('/'));
  mkdir(parent.c_str(), 0755);
  mkdir(dir.c_str(), 0755);
  return dir;
}

static bool read_file(const std::string &path, std::vector<char> &out) {
  FILE *f = fopen(path.c_str(), "rb");
  if (!f) return false;
  fseek(f, 0, SEEK_END); long n = ftell(f); fseek(f, 0, SEEK_SET);
  if (n <= 0) { fclose(f); return false; }
  out.resize((size_t)n);
  bool ok = fread(out.data(), 1, (size_t)n, f) == (size_t)n;
  fclose(f);
  return ok;
}

static void write_file_atomic(const std::string &path, const std::vector<char> &data) {
  std::string tmp = path + "." + std::to_string((long)getpid()) + ".tmp";
  FILE *f = fopen(tmp.c_str(), "wb");
  if (!f) return;
  bool ok = fwrite(data.data(), 1, data.size(), f) == data.size();
  fclose(f);
  if (ok) rename(tmp.c_str(), path.c_str()); else unlink(tmp.c_str());
}

static bool nvrtc_compile(const char *source, std::vector<char> &cubin) {
  if (!load_nvrtc()) return false;
  nvrtcProgram_ prog = nullptr;
  int rc = RTC.CreateProgram(&prog, source, "pb200_kernel.cu", 0, nullptr, nullptr);
  if (rc != 0) { pb_set_error("nvrtcCreateProgram: %s", RTC.GetErrorString(rc)); return false; }
  std::string inc = "--include-path=";
  const char *home = getenv("CUDA_HOME");
  inc += (home && home[0]) ? std::string(home) + "/include" : "/usr/local/cuda/include";
  const char *opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-default-device", inc.c_str()};
  rc = RTC.CompileProgram(prog, 4, opts);
  if (rc != 0) {
    size_t ls = 0; RTC.GetProgramLogSize(prog, &ls);
    std::string log(ls + 1, '\0');
    if (ls) RTC.GetProgramLog(prog, &log[0]);
    pb_set_error("NVRTC compilation failed: %s\n%s\n--- source ---\n%s", RTC.GetErrorString(rc), log.c_str(), source);
    RTC.DestroyProgram(&prog);
    return false;
  }
  size_t n = 0;
  RTC.GetCUBINSize(prog, &n);
  cubin.resize(n);
  RTC.GetCUBIN(prog, cubin.data());
  RTC.DestroyProgram(&prog);
  R.st.programs_compiled++;
  return n > 0;
}

static std::shared_ptr<Module> get_module(const char *source) {
  uint64_t key = fnv1a(source, strlen(source));
  key = fnv1a("sm_100a;v1", 10, key);
  auto it = g_modules.find(key);
  if (it != g_modules.end()) { R.st.programs_cached++; return it->second; }
  if (R.dry) {
    /* compile (NVRTC needs no device) so that host-only tests check the text */
    auto m = std::make_shared<Module>();
    const char *skip = getenv("POLY_B200_DRYRUN_NOCOMPILE");
    if (!(skip && skip[0] == '1') && !g_dry_compiled.count(key)) {
      std::vector<char> cubin;
      if (!nvrtc_compile(source, cubin)) return nullptr;
      g_dry_compiled[key] = true;
    }
    g_modules[key] = m;
    return m;
  }
  std::vector<char> cubin;
  std::string dir = cache_dir();
  char name[64]; snprintf(name, sizeof name, "/%016llx.cubin", (unsigned long long)key);
  bool from_disk = !dir.empty() && read_file(dir + name, cubin);
  if (from_disk) R.st.programs_cached++;
  else {
    if (!nvrtc_compile(source, cubin)) return nullptr;
    if (!dir.empty()) write_file_atomic(dir + name, cubin);
  }
  auto m = std::make_shared<Module>();
  CUresult_ rc = DRV.ModuleLoadData(&m->mod, cubin.data());
  if (rc != 0 && from_disk) {
    /* a stale or damaged cache entry: rebuild */
    if (!nvrtc_compile(source, cubin)) return nullptr;
    write_file_atomic(dir + name, cubin);
    rc = DRV.ModuleLoadData(&m->mod, cubin.data());
  }
  if (rc != 0) { const char *s = "?"; DRV.GetErrorString(rc, &s); pb_set_error("cuModuleLoadData: %s", s); return nullptr; }
  rc = DRV.ModuleGetFunction(&m->fn, m->mod, "pb200_kernel");
  if (rc != 0) { const char *s = "?"; DRV.GetErrorString(rc, &s); pb_set_error("cuModuleGetFunction: %s", s); return nullptr; }
  g_modules[key] = m;
  return m;
}

static bool parse_work(const std::string &s, std::vector<WorkTerm> &out) {
  std::istringstream alts(s);
  std::string alt;
  while (std::getline(alts, alt, '|')) {
    WorkTerm t{1, {}};
    std::istringstream fs(alt);
    std::string f;
    while (std::getline(fs, f, '*')) {
      if (f.empty()) return false;
      if (f[0] == 'c') t.c *= atoll(f.c_str() + 1);
      else if (f[0] == 'v') t.vars.push_back(atoi(f.c_str() + 1));
      else return false;
    }
    out.push_back(t);
  }
  return !out.empty();
}

/* ── per-launch device timing (measurement aid) ──────────────────────── */
static bool g_timing = false;
static std::vector<std::pair<cudaEvent_t, cudaEvent_t>> g_timing_events;
static std::vector<std::string> g_timing_names;

extern "C" int poly_b200_timing_active(void) { return g_timing ? 1 : 0; }
extern "C" void poly_b200_timing_begin(void) {
  for (auto &e : g_timing_events) { cudaEventDestroy(e.first); cudaEventDestroy(e.second); }
  g_timing_events.clear();
  g_timing_names.clear();
  g_timing = true;
}
/* Stops timing and returns the summed device time of the launches since
 * poly_b200_timing_begin, in milliseconds; *n_launches receives their count.
 * POLY_B200_TIMING_DUMP=1 also lists every launch (index, program, ms) on stderr. */
extern "C" double poly_b200_timing_end(int *n_launches) {
  g_timing = false;
  double total = 0.0;
  if (R.ok && !R.dry) cudaStreamSynchronize(R.stream);
  const char *dump = getenv("POLY_B200_TIMING_DUMP");
  size_t i = 0;
  for (auto &e : g_timing_events) {
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, e.first, e.second) == cudaSuccess) total += ms;
    if (dump && dump[0] == '1')
      fprintf(stderr, "pb_timing: %4zu %-28s %9.4f ms\n", i, i < g_timing_names.size() ? g_timing_names[i].c_str() : "?", ms);
    cudaEventDestroy(e.first); cudaEventDestroy(e.second);
    i++;
  }
  if (n_launches) *n_launches = (int)g_timing_events.size();
  g_timing_events.clear();
  g_timing_names.clear();
  return total;
}
static void timing_mark(bool before, const char *name = nullptr) {
  if (!g_timing || R.dry) return;
  if (before) {
    cudaEvent_t a, b;
    if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return;
    g_timing_events.push_back({a, b});
    g_timing_names.push_back(name ? name : "");
    cudaEventRecord(a, R.stream);
  } else if (!g_timing_events.empty()) cudaEventRecord(g_timing_events.back().second, R.stream);
}

extern "C" PolyCudaProgram *poly_compile_cuda(const char *source, const char *fn_name) {
  if (!ready()) return nullptr;
  if (!source) { pb_set_error("poly_compile_cuda: null source"); return nullptr; }
  PbHeader h;
  if (!parse_header(source, h)) {
    pb_set_error("poly_compile_cuda: text for %s was not produced by poly_render_cuda", fn_name ? fn_name : "?");
    return nullptr;
  }
  std::unique_ptr<PolyCudaProgram> p(new PolyCudaProgram());
  p->name = fn_name ? fn_name : "";
  const std::string &kind = h.get("kind");
  if (kind == "jit") {
    p->kind = PolyCudaProgram::JIT;
    p->n_params = (int)h.geti("nparams");
    p->n_vars = (int)h.geti("nvars");
    std::istringstream ls(h.get("launch"));
    std::string mode, tok;
    ls >> mode;
    p->group_launch = (mode == "group");
    std::string work;
    while (ls >> tok) {
      if (tok.rfind("block=", 0) == 0) p->block = atoi(tok.c_str() + 6);
      else if (tok.rfind("group=", 0) == 0) p->group = atoi(tok.c_str() + 6);
      else if (tok.rfind("work=", 0) == 0) work = tok.substr(5);
    }
    if (!parse_work(work, p->work) || p->block <= 0 || p->block > 1024 || p->group <= 0 || p->block % p->group) {
      pb_set_error("poly_compile_cuda: bad launch line '%s'", h.get("launch").c_str());
      return nullptr;
    }
    std::istringstream rs(h.get("rw"));
    while (rs >> tok) {
      char c = '-';
      if (tok == "r") c = 'r'; else if (tok == "rw") c = 'b'; else if (tok == "W") c = 'W'; else if (tok == "w") c = 'w';
      p->rw.push_back(c);
    }
    if ((int)p->rw.size() != p->n_params) { pb_set_error("poly_compile_cuda: rw line does not match nparams"); return nullptr; }
    p->module = get_module(source);
    if (!p->module) return nullptr;
  } else {
    p->kind = PolyCudaProgram::AOT;
    std::string err;
    if (kind == "gather") p->aot = pb_make_gather(h, err);
    else if (kind == "scatter") p->aot = pb_make_scatter(h, err);
    else if (kind == "gemm") p->aot = pb_make_gemm(h, err);
    else if (kind == "copy") p->aot = pb_make_copy(h, err);
    else if (kind == "attn") p->aot = pb_make_attn(h, err);
    else err = "unknown program kind '" + kind + "'";
    if (!p->aot) { pb_set_error("poly_compile_cuda: %s", err.c_str()); return nullptr; }
    p->n_params = p->aot->n_params;
    p->rw = p->aot->rw;
  }
  return p.release();
}

extern "C" void poly_cuda_program_destroy(PolyCudaProgram *prog) { delete prog; }

extern "C" int poly_cuda_launch(PolyCudaProgram *prog, void **args, int n_args,
                                int gx, int gy, int gz, int bx, int by, int bz) {
  (void)gx; (void)gy; (void)gz; (void)bx; (void)by; (void)bz;
  if (!ready()) return -1;
  if (!prog || !args) { pb_set_error("poly_cuda_launch: null program or args"); return -1; }
  if (n_args < prog->n_params + prog->n_vars) {
    pb_set_error("poly_cuda_launch: %s expects %d arguments, got %d", prog->name.c_str(), prog->n_params + prog->n_vars, n_args);
    return -1;
  }
  void *bufs[64];
  if (prog->n_params > 64) { pb_set_error("poly_cuda_launch: too many parameters"); return -1; }
  for (int i = 0; i < prog->n_params; i++) {
    bufs[i] = (void *)(uintptr_t)(*(unsigned long long *)args[i]);
    char m = prog->rw[(size_t)i];
    if (m == '-') continue;
    if (!bufs[i]) { pb_set_error("poly_cuda_launch: %s: parameter %d is null", prog->name.c_str(), i); return -1; }
    if (note_access(bufs[i], m) != 0) return -1;
  }
  if (prog->kind == PolyCudaProgram::AOT) {
    if (R.dry) return 0;
    timing_mark(true, prog->name.c_str());
    int rc = prog->aot->launch(bufs, R.stream);
    timing_mark(false);
    if (rc == 0) pb_count_launch(true, prog->aot->n_launches());
    return rc;
  }
  int vars[16];
  for (int v = 0; v < prog->n_vars && v < 16; v++) {
    const int *hp = (const int *)(uintptr_t)(*(unsigned long long *)args[prog->n_params + v]);
    if (!hp) { pb_set_error("poly_cuda_launch: null var pointer"); return -1; }
    vars[v] = *hp;
  }
  long long work = 0;
  for (const WorkTerm &t : prog->work) {
    long long w = t.c;
    for (int v : t.vars) w *= (v < prog->n_vars ? vars[v] : 0);
    if (w > work) work = w;
  }
  if (work <= 0) return 0;
  long long per_block = prog->group_launch ? prog->block / prog->group : prog->block;
  long long grid = (work + per_block - 1) / per_block;
  if (grid > 2147483647LL) { pb_set_error("poly_cuda_launch: %s needs %lld blocks", prog->name.c_str(), grid); return -1; }
  if (R.dry) return 0;
  void *kargs[64 + 16 + 1];
  int n = 0;
  for (int i = 0; i < prog->n_params; i++) kargs[n++] = &bufs[i];
  for (int v = 0; v < prog->n_vars; v++) kargs[n++] = &vars[v];
  kargs[n++] = &work;
  timing_mark(true, prog->name.c_str());
  CUresult_ rc = DRV.LaunchKernel(prog->module->fn, (unsigned)grid, 1, 1, (unsigned)prog->block, 1, 1, 0,
                                  (CUstream_)R.stream, kargs, nullptr);
  timing_mark(false);
  if (rc != 0) { const char *s = "?"; DRV.GetErrorString(rc, &s); pb_set_error("cuLaunchKernel(%s): %s", prog->name.c_str(), s); return -1; }
  pb_count_launch(false, 1);
  return 0;
}


/* ── plan support: program facts, stream capture ─────────────────────── */
extern "C" int poly_b200_program_info(PolyCudaProgram *prog, char *rw, int cap, int *n_params, int *n_vars, int *precompiled) {
  if (!prog) return -1;
  if (n_params) *n_params = prog->n_params;
  if (n_vars) *n_vars = prog->n_vars;
  if (precompiled) *precompiled = prog->kind == PolyCudaProgram::AOT;
  if (rw && cap > 0) {
    int n = (int)prog->rw.size() < cap - 1 ? (int)prog->rw.size() : cap - 1;
    memcpy(rw, prog->rw.data(), (size_t)n); rw[n] = 0;
  }
  return 0;
}

extern "C" int poly_b200_program_stale(PolyCudaProgram *prog, void **args) {
  if (!prog || prog->kind != PolyCudaProgram::AOT) return 0;
  void *bufs[64];
  for (int i = 0; i < prog->n_params && i < 64; i++) bufs[i] = args[i] ? (void *)(uintptr_t)(*(unsigned long long *)args[i]) : nullptr;
  return prog->aot->stale(bufs) ? 1 : 0;
}

extern "C" unsigned long long poly_b200_pool_epoch(void) { return R.pool_epoch; }

extern "C" int poly_b200_capture_begin(void) {
  if (!ready() || R.dry || R.capturing) return -1;
  R.capture_failed = false;
  if (cudaStreamBeginCapture(R.stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { cudaGetLastError(); return -1; }
  R.capturing = true;
  return 0;
}

/* An executable graph together with the pool blocks its nodes address: scratch that the
 * captured steps took and gave back.  The blocks return to the free list when the graph
 * is destroyed, not before (every replay writes them). */
struct GraphBox {
  cudaGraphExec_t exec = nullptr;
  std::vector<std::pair<size_t, void *>> held;
};

static void release_held(std::vector<std::pair<size_t, void *>> &held) {
  for (auto &b : held) R.free_blocks.insert({b.first, b.second});
  held.clear();
}

/* Ends the capture.  Returns an executable graph, or NULL when the capture was
 * abandoned (the enqueued work is then discarded and must be re-issued). */
extern "C" void *poly_b200_capture_end(int discard) {
  if (!R.capturing) return nullptr;
  R.capturing = false;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(R.stream, &graph);
  cudaGraphExec_t exec = nullptr;
  if (e != cudaSuccess || !graph) { cudaGetLastError(); graph = nullptr; }
  else if (discard || R.capture_failed) { cudaGraphDestroy(graph); graph = nullptr; }
  else {
    e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) { cudaGetLastError(); exec = nullptr; }
  }
  if (!exec) { release_held(R.capture_hold); return nullptr; }     /* the captured work never runs */
  GraphBox *box = new GraphBox();
  box->exec = exec;
  box->held.swap(R.capture_hold);
  return (void *)box;
}

extern "C" int poly_b200_graph_launch(void *graph, unsigned long long n_kernels, unsigned long long n_precompiled) {
  if (!graph) return -1;
  PB_CUDA(cudaGraphLaunch(((GraphBox *)graph)->exec, R.stream));
  R.st.launches += n_kernels; R.st.launches_precompiled += n_precompiled; R.st.launches_generated += n_kernels - n_precompiled;
  return 0;
}

/* Bytes of pool scratch a graph keeps out of circulation (diagnostics, tests). */
extern "C" unsigned long long poly_b200_graph_held_bytes(void *graph) {
  unsigned long long n = 0;
  if (graph) for (auto &b : ((GraphBox *)graph)->held) n += b.first;
  return n;
}

extern "C" void poly_b200_graph_destroy(void *graph) {
  if (!graph) return;
  GraphBox *box = (GraphBox *)graph;
  cudaGraphExecDestroy(box->exec);
  release_held(box->held);       /* stream-ordered pool: later work on the stream may take them */
  delete box;
}

/* Stream-ordered fill used by plans for buffers a kernel only partly writes. */
extern "C" int poly_b200_memset_now(unsigned long long ptr, unsigned char val, size_t bytes) {
  if (!ready()) return -1;
  void *p = (void *)(uintptr_t)ptr;
  auto it = find_buf(p);
  if (it != R.live.end()) { if (it->second.pending_zero) { it->second.pending_zero = false; R.n_pending--; } it->second.version = R.version_counter++; }
  R.st.memsets_executed++;
  if (R.dry) { memset(p, val, bytes); return 0; }
  PB_CUDA(cudaMemsetAsync(p, val, bytes, R.stream));
  return 0;
}
