/*
 * pb_copy.cu -- data movement whose source and destination are contiguous along
 * different axes (polygrad's permute followed by CONTIGUOUS, reference:
 * src/sched.c:886): a tiled transpose.
 *
 *   out[o_off + x + y*o_sy + sum_b i_b*o_sb] = in[i_off + x*i_sx + y + sum_b i_b*i_sb]
 *
 * 32 x 32 tiles of 4-byte elements through padded shared memory: reads are
 * coalesced along y (the source's contiguous axis), writes along x (the
 * destination's).  Bit-exact.  HBM traffic: every element read once, written once.
 */
#include "../runtime/pb_runtime.h"
#include <cstdio>

struct TransposeArgs {
  const unsigned *in; unsigned *out;
  long long X, Y, i_sx, o_sy, i_off, o_off;
  int nb; long long bext[6], i_sb[6], o_sb[6];
};

__global__ void __launch_bounds__(256) pb200_transpose_tiles(const TransposeArgs a) {
  __shared__ unsigned tile[32][33];
  long long rem = blockIdx.z, io = a.i_off, oo = a.o_off;
  for (int i = 0; i < a.nb; i++) { const long long x = rem % a.bext[i]; rem /= a.bext[i]; io += x * a.i_sb[i]; oo += x * a.o_sb[i]; }
  const long long x0 = (long long)blockIdx.x * 32, y0 = (long long)blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const long long x = x0 + ty + j, y = y0 + tx;
    if (x < a.X && y < a.Y) tile[ty + j][tx] = a.in[io + x * a.i_sx + y];
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const long long y = y0 + ty + j, x = x0 + tx;
    if (x < a.X && y < a.Y) a.out[oo + x + y * a.o_sy] = tile[tx][ty + j];
  }
}

/* 64 x 64 tiles, 128-bit global accesses on both sides (X, Y multiples of 4 and
 * 16-byte aligned rows). */
__global__ void __launch_bounds__(256) pb200_transpose_tiles_v4(const TransposeArgs a) {
  __shared__ unsigned tile[64][65];
  long long rem = blockIdx.z, io = a.i_off, oo = a.o_off;
  for (int i = 0; i < a.nb; i++) { const long long x = rem % a.bext[i]; rem /= a.bext[i]; io += x * a.i_sb[i]; oo += x * a.o_sb[i]; }
  const long long x0 = (long long)blockIdx.x * 64, y0 = (long long)blockIdx.y * 64;
  const int q = threadIdx.x & 15, r = threadIdx.x >> 4;      /* 16 quads per row, 16 rows per pass */
#pragma unroll
  for (int j = 0; j < 64; j += 16) {
    const long long x = x0 + r + j, y = y0 + q * 4;
    if (x < a.X && y < a.Y) {
      const uint4 v = *reinterpret_cast<const uint4 *>(a.in + io + x * a.i_sx + y);
      tile[r + j][q * 4 + 0] = v.x; tile[r + j][q * 4 + 1] = v.y; tile[r + j][q * 4 + 2] = v.z; tile[r + j][q * 4 + 3] = v.w;
    }
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 64; j += 16) {
    const long long y = y0 + r + j, x = x0 + q * 4;
    if (x < a.X && y < a.Y) {
      uint4 v;
      v.x = tile[q * 4 + 0][r + j]; v.y = tile[q * 4 + 1][r + j]; v.z = tile[q * 4 + 2][r + j]; v.w = tile[q * 4 + 3][r + j];
      *reinterpret_cast<uint4 *>(a.out + oo + x + y * a.o_sy) = v;
    }
  }
}

struct TransposeProgram : PbAotProgram {
  TransposeArgs a{};
  int p_out = 0, p_in = 1;
  long long nbatch = 1;
  int launch(void *const *bufs, cudaStream_t stream) override {
    TransposeArgs g = a;
    g.out = (unsigned *)bufs[p_out]; g.in = (const unsigned *)bufs[p_in];
    bool v4 = g.X % 4 == 0 && g.Y % 4 == 0 && g.i_sx % 4 == 0 && g.o_sy % 4 == 0 && g.i_off % 4 == 0 && g.o_off % 4 == 0 &&
              (reinterpret_cast<uintptr_t>(g.in) & 15) == 0 && (reinterpret_cast<uintptr_t>(g.out) & 15) == 0;
    for (int i = 0; i < g.nb; i++) if (g.i_sb[i] % 4 || g.o_sb[i] % 4) v4 = false;
    if (v4) {
      dim3 grid((unsigned)((g.X + 63) / 64), (unsigned)((g.Y + 63) / 64), (unsigned)nbatch);
      pb200_transpose_tiles_v4<<<grid, 256, 0, stream>>>(g);
    } else {
      dim3 grid((unsigned)((g.X + 31) / 32), (unsigned)((g.Y + 31) / 32), (unsigned)nbatch);
      pb200_transpose_tiles<<<grid, 256, 0, stream>>>(g);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { pb_set_error("transpose launch: %s", cudaGetErrorString(e)); return -1; }
    return 0;
  }
};

PbAotProgram *pb_make_copy(const PbHeader &h, std::string &err) {
  auto params = h.getv("params"), xy = h.getv("xy"), off = h.getv("offsets"), bt = h.getv("batch");
  if (params.size() != 2 || xy.size() != 4 || off.size() != 2 || bt.size() % 3 || bt.size() > 18) { err = "malformed copy header"; return nullptr; }
  TransposeProgram *p = new TransposeProgram();
  p->n_params = (int)h.geti("nparams");
  p->p_out = (int)params[0]; p->p_in = (int)params[1];
  p->rw.assign((size_t)p->n_params, '-');
  p->rw[(size_t)p->p_in] = 'r';
  p->rw[(size_t)p->p_out] = h.get("full") == "1" ? 'W' : 'w';
  p->a.X = xy[0]; p->a.Y = xy[1]; p->a.i_sx = xy[2]; p->a.o_sy = xy[3];
  p->a.o_off = off[0]; p->a.i_off = off[1];
  p->a.nb = (int)bt.size() / 3;
  for (int i = 0; i < p->a.nb; i++) { p->a.bext[i] = bt[3 * i]; p->a.o_sb[i] = bt[3 * i + 1]; p->a.i_sb[i] = bt[3 * i + 2]; p->nbatch *= bt[3 * i]; }
  if (p->nbatch > 65535 || (p->a.Y + 31) / 32 > 65535) { err = "transpose grid out of range"; delete p; return nullptr; }
  return p;
}
