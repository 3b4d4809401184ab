/*
 * pb_runtime.h -- internal interface between the runtime core and the
 * precompiled kernels.
 */
#ifndef PB_RUNTIME_H
#define PB_RUNTIME_H

#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>
#include <string>
#include <map>
#include <vector>

/* Key/value view of the "//PB200" header lines of a program text. */
struct PbHeader {
  std::map<std::string, std::string> kv;   /* "//key rest of line" */
  bool has(const char *k) const { return kv.count(k) != 0; }
  const std::string &get(const char *k) const;
  long long geti(const char *k, long long dflt = 0) const;
  std::vector<long long> getv(const char *k) const; /* whitespace-separated integers */
};

/* A precompiled-kernel program: created from a header, launched with the
 * kernel's buffer arguments (device pointers in PARAM order). */
struct PbAotProgram {
  virtual ~PbAotProgram() {}
  /* rw[i]: 'r' read, 'w' partially written, 'W' fully overwritten, 'b' read and written, '-' unused */
  std::string rw;
  int n_params = 0;
  virtual int launch(void *const *bufs, cudaStream_t stream) = 0;
  virtual int n_launches() const { return 1; }
  /* true when a cached, converted copy of an operand no longer matches its source buffer */
  virtual bool stale(void *const *bufs) { (void)bufs; return false; }
};

/* Factories, one per kernel family; return nullptr and set err on bad headers. */
PbAotProgram *pb_make_gather(const PbHeader &h, std::string &err);
PbAotProgram *pb_make_scatter(const PbHeader &h, std::string &err);
PbAotProgram *pb_make_gemm(const PbHeader &h, std::string &err);
PbAotProgram *pb_make_copy(const PbHeader &h, std::string &err);
PbAotProgram *pb_make_attn(const PbHeader &h, std::string &err);

/* Runtime services for kernels that need scratch memory or mode flags. */
void *pb_scratch_alloc(size_t bytes);          /* pooled; nullptr on failure */
void  pb_scratch_free(void *p);
bool  pb_dry_run(void);
void  pb_set_error(const char *fmt, ...);
void  pb_count_launch(bool precompiled, int n = 1);

/* Device buffers are tracked so that cached, converted copies of constant
 * operands (bf16 weights) can be invalidated when the source is written. */
uint64_t pb_buffer_version(const void *p);      /* changes whenever p's allocation is written */

/* Entry points that launch on caller-supplied device pointers report their accesses like
 * poly_cuda_launch does: a pending (lazy) zero fill of a pool buffer is materialised before a
 * read or partial write and dropped before a whole-buffer overwrite, and a written buffer
 * gets a new version.  Host-side bookkeeping only; allocates nothing. */
int pb_note_read(const void *p);
int pb_note_write(const void *p, size_t bytes);

/* The tensor-core kernel bounds its barrier waits and records a code when one
 * runs out; the runtime reads it back at synchronisation points. */
int  pb_gemm_tc_error(void);                    /* 0 = none, >0 = which wait gave up, <0 = cannot read */
int  pb_attention_error(void);
void pb_tc_mark_used(void);

#endif
