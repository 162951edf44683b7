// fp32 tile engine shared by the factor, inverse and precondition kernels.
//
// One CTA of 256 threads computes a 128x128 tile of C[m][n] = sum_k A(k,m) *
// B(k,n) with an 8x8 register micro-tile per thread.  Operands are described
// by `Operand`: a virtual (k, column) matrix that is either a strided view of
// device memory (optionally with one appended column of ones / of a vector) or
// the im2col patch matrix of an NCHW tensor, gathered on the fly.  The k-loop
// is double buffered through shared memory (16 k per stage).
#pragma once

#include "common.cuh"

namespace kfac {

constexpr int TM = 128;      // tile rows (M)
constexpr int TN = 128;      // tile cols (N)
constexpr int TK = 16;       // k per stage
constexpr int NT = 256;      // threads per CTA
constexpr int SLD = TM + 4;  // shared-memory row pitch (floats)

struct Operand {
  const float* base;
  const float* extra;  // values of the appended column (NULL: ones)
  long long s_outer;   // row offset = (k / period) * s_outer
  long long s_inner;   //            + (k % period) * s_inner
  long long s_col;     // column stride
  int period;
  int ncols;      // columns stored in memory
  int extra_idx;  // index of the appended column, -1 if none
  int kfast;      // 1: consecutive threads walk k, 0: walk columns
  int mode;       // 0 strided, 1 im2col
  int C, H, W, ks, st, pd, Ho, Wo;  // im2col geometry
};

inline Operand strided_operand(const float* base, long long s_row,
                               long long s_col, int ncols) {
  Operand o = {};
  o.base = base;
  o.extra = nullptr;
  o.s_outer = s_row;
  o.s_inner = 0;
  o.s_col = s_col;
  o.period = 1;
  o.ncols = ncols;
  o.extra_idx = -1;
  o.kfast = (s_row == 1) ? 1 : 0;
  o.mode = 0;
  return o;
}

__device__ __forceinline__ long long operand_rowoff(const Operand& op,
                                                    long long k) {
  if (op.period == 1) return k * op.s_outer;
  long long q = k / op.period;
  return q * op.s_outer + (k - q * op.period) * op.s_inner;
}

// Column tables of an im2col operand for the 128 columns of a tile.
__device__ __forceinline__ void im2col_tables(const Operand& op, int c0,
                                              int* s_coff, int* s_kykx,
                                              int tid) {
  if (tid < TM) {
    int c = c0 + tid;
    int coff = 0, info = -1;
    if (c < op.ncols) {
      int kk = op.ks * op.ks;
      int ch = c / kk;
      int r = c - ch * kk;
      int ky = r / op.ks;
      int kx = r - ky * op.ks;
      coff = ch * op.H * op.W + ky * op.W + kx;
      info = (ky << 16) | kx;
    } else if (c == op.extra_idx) {
      info = -2;
    }
    s_coff[tid] = coff;
    s_kykx[tid] = info;
  }
}

// Fetch this thread's 8 elements of the (TK x 128) operand tile at (k0, c0).
__device__ __forceinline__ void operand_load(const Operand& op, int c0,
                                             long long k0, long long kend,
                                             const int* s_coff,
                                             const int* s_kykx, int tid,
                                             float r[8]) {
  if (op.kfast) {
    long long k = k0 + (tid & 15);
    bool kval = k < kend;
    if (op.mode == 0) {
      long long roff = kval ? operand_rowoff(op, k) : 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        int c = c0 + (tid >> 4) + 16 * j;
        float v = 0.f;
        if (kval) {
          if (c < op.ncols)
            v = op.base[roff + (long long)c * op.s_col];
          else if (c == op.extra_idx)
            v = op.extra ? op.extra[k] : 1.f;
        }
        r[j] = v;
      }
    } else {
      int how = op.Ho * op.Wo;
      long long n = k / how;
      int rem = (int)(k - n * how);
      int oy = rem / op.Wo;
      int ox = rem - oy * op.Wo;
      int iy0 = oy * op.st - op.pd;
      int ix0 = ox * op.st - op.pd;
      long long roff = n * op.C * op.H * op.W + (long long)iy0 * op.W + ix0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        int cl = (tid >> 4) + 16 * j;
        int info = s_kykx[cl];
        float v = 0.f;
        if (kval) {
          if (info >= 0) {
            int iy = iy0 + (info >> 16);
            int ix = ix0 + (info & 0xffff);
            if ((unsigned)iy < (unsigned)op.H && (unsigned)ix < (unsigned)op.W)
              v = op.base[roff + s_coff[cl]];
          } else if (info == -2) {
            v = 1.f;
          }
        }
        r[j] = v;
      }
    }
  } else {
    int c = c0 + (tid & 127);
    bool real = c < op.ncols;
    bool extra = c == op.extra_idx;
    const float* pc = op.base + (long long)c * op.s_col;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      long long k = k0 + (tid >> 7) + 2 * j;
      float v = 0.f;
      if (k < kend) {
        if (real)
          v = pc[operand_rowoff(op, k)];
        else if (extra)
          v = op.extra ? op.extra[k] : 1.f;
      }
      r[j] = v;
    }
  }
}

__device__ __forceinline__ void operand_store(int kfast, float (*S)[SLD],
                                              int tid, const float r[8]) {
  if (kfast) {
#pragma unroll
    for (int j = 0; j < 8; ++j) S[tid & 15][(tid >> 4) + 16 * j] = r[j];
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) S[(tid >> 7) + 2 * j][tid & 127] = r[j];
  }
}

struct TileSmem {
  float a[2][TK][SLD];
  float b[2][TK][SLD];
  int coff[2][TM];
  int kykx[2][TM];
};

// acc[i][j] += sum_{k in [kbeg,kend)} A(k, m0 + row(i)) * B(k, n0 + col(j)),
// row(i) = ty*4 + i (i<4) or 64 + ty*4 + i-4, col likewise with tx.
__device__ __forceinline__ void tile_mainloop(const Operand& A,
                                              const Operand& B, int m0, int n0,
                                              long long kbeg, long long kend,
                                              TileSmem& sm, float acc[8][8]) {
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  if (A.mode == 1) im2col_tables(A, m0, sm.coff[0], sm.kykx[0], tid);
  if (B.mode == 1) im2col_tables(B, n0, sm.coff[1], sm.kykx[1], tid);
  if (A.mode == 1 || B.mode == 1) __syncthreads();

  long long nk = (kend > kbeg) ? (kend - kbeg + TK - 1) / TK : 0;
  float ra[8], rb[8];
  if (nk > 0) {
    operand_load(A, m0, kbeg, kend, sm.coff[0], sm.kykx[0], tid, ra);
    operand_load(B, n0, kbeg, kend, sm.coff[1], sm.kykx[1], tid, rb);
    operand_store(A.kfast, sm.a[0], tid, ra);
    operand_store(B.kfast, sm.b[0], tid, rb);
  }
  __syncthreads();
  for (long long it = 0; it < nk; ++it) {
    const int buf = (int)(it & 1);
    const bool more = it + 1 < nk;
    if (more) {
      long long k0 = kbeg + (it + 1) * TK;
      operand_load(A, m0, k0, kend, sm.coff[0], sm.kykx[0], tid, ra);
      operand_load(B, n0, k0, kend, sm.coff[1], sm.kykx[1], tid, rb);
    }
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float4 a0 = *reinterpret_cast<const float4*>(&sm.a[buf][kk][ty * 4]);
      float4 a1 = *reinterpret_cast<const float4*>(&sm.a[buf][kk][64 + ty * 4]);
      float4 b0 = *reinterpret_cast<const float4*>(&sm.b[buf][kk][tx * 4]);
      float4 b1 = *reinterpret_cast<const float4*>(&sm.b[buf][kk][64 + tx * 4]);
      float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (more) {
      operand_store(A.kfast, sm.a[buf ^ 1], tid, ra);
      operand_store(B.kfast, sm.b[buf ^ 1], tid, rb);
    }
    __syncthreads();
  }
}

__device__ __forceinline__ int tile_row(int ty, int i) {
  return (i < 4) ? ty * 4 + i : 64 + ty * 4 + (i - 4);
}

// Lower-triangular tile enumeration: index t -> (bi, bj), bj <= bi.
__device__ __forceinline__ void tri_tile(int t, int& bi, int& bj) {
  int i = (int)((sqrtf(8.f * (float)t + 1.f) - 1.f) * 0.5f);
  while ((i + 1) * (i + 2) / 2 <= t) ++i;
  while (i * (i + 1) / 2 > t) --i;
  bi = i;
  bj = t - i * (i + 1) / 2;
}

// ---------------------------------------------------------------- grouped GEMM
enum GemmFlags {
  G_LOWER = 1,     // square problem, only tiles with bj <= bi
  G_MIRROR = 2,    // also write C[n][m] for off-diagonal tiles
  G_KBEG_N0 = 4,   // B(k, n) is zero for k < n: start at the tile's n0
  G_KEND_M0 = 8,   // A(k, m) is zero for k > m: stop after the tile's rows
  G_KBEG_M0 = 16,  // A(k, m) is zero for k < m: start at the tile's m0
  G_PRECOND = 32,  // epilogue splits into kf_W / kf_b and applies momentum
  G_SAME_AB = 64   // A and B are the same operand (X^T X): a tile on the
                   // diagonal may take its A rows from the staged B rows
};

struct GemmDesc {
  Operand A, B;
  float* C;
  long long ldc;
  long long K;
  int M, N;
  float alpha, beta;
  int flags;
  int tile_begin;
  int tiles_m, tiles_n;
  float *kfW, *kfb, *pW, *pb, *vW, *vb;
  int dW;
  int splits;              // tensor-core engine: CTAs along the contraction
  int ntiles;              // tiles of one split (virtual tile = split * ntiles + tile)
  long long k_per_split;
  float* partial;          // partial tiles when splits > 1
  const int* gate;         // if set and *gate == 0 the problem is skipped
  float* C2;               // if set, C's new values are stored here as well
                           // (same row pitch; plain epilogue only)
  // factor builds from staged operands: tensor maps (device memory) of the
  // hi and lo bf16 planes of X^T, see stage.cu
  const void* tmap_hi;
  const void* tmap_lo;
};

int launch_grouped_gemm(const GemmDesc* descs_dev, int ndesc, int total_tiles,
                        float lr, float momentum, cudaStream_t stream);

// Tensor-core engine (tc_gemm.cu): 128 x 256 tiles, tcgen05 split-TF32.
int engine();   // 1: tensor cores (default), 0: fp32 FFMA tiles
int tc_tiles(GemmDesc& g);
// Opt the tile kernels into their shared-memory sizes on the current device
// (once per device; the launch helpers call it, plans call it before capture).
int tc_prepare();
int launch_tc_grouped(const GemmDesc* descs_dev, int ndesc, int total_tiles,
                      float lr, float momentum, bool tails,
                      cudaStream_t stream);
bool tc_desc_has_tails(const GemmDesc& g);
size_t tc_factor_workspace_bytes(long long rows, int d, bool staged = true);
size_t tc_pad_bytes(const Operand& X, int n, int nhwc = 0);
int run_factor_tc(const Operand& X, long long rows, int d, float alpha,
                  float beta, float* out, void* workspace,
                  size_t workspace_bytes, cudaStream_t stream,
                  bool staged = true);
struct FactorJob {      // one factor of a grouped build
  Operand X;
  long long rows;
  int d;
  int n;                // batch size (im2col operands)
  int nhwc;             // im2col operand: the tensor is stored channels-last
  float alpha, beta;
  float* out;
};
size_t tc_factor_group_workspace_bytes(int count, const FactorJob* jobs,
                                       bool staged = true);
// Staging pass (stage.cu): bytes of both bf16 planes of one operand; staging
// of a group into `ws` with two tensor maps per job written to `tmaps`.
size_t tc_stage_bytes(long long rows, int d);
int tc_stage_group(int count, const FactorJob* jobs, char* ws, void* tmaps,
                   cudaStream_t stream);
int run_factor_group_tc(int count, const FactorJob* jobs, void* workspace,
                        size_t workspace_bytes, cudaStream_t stream,
                        bool staged = true);

// Host helper: fill tile counts of a descriptor and return its tile count.
inline int gemm_desc_tiles(GemmDesc& g) {
  g.tiles_m = (g.M + TM - 1) / TM;
  g.tiles_n = (g.N + TN - 1) / TN;
  if (g.flags & G_LOWER) return g.tiles_m * (g.tiles_m + 1) / 2;
  return g.tiles_m * g.tiles_n;
}

}  // namespace kfac
