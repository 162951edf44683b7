// Kronecker-factor construction: out = alpha * X^T X + beta * out where X is a
// dense matrix, the im2col patch matrix of an NCHW input or an NCHW output
// gradient viewed as (n*ho*wo, c).  X is gathered tile by tile and never
// written to memory.  Only tiles on or below the diagonal are computed; the
// epilogue mirrors them.  Long contractions are split across CTAs; partial
// tiles go through a workspace and are summed in a fixed order.
#include <algorithm>
#include <mutex>
#include <vector>

#include "gemm_simt.cuh"

namespace kfac {

struct FactorSplit {
  int nt;          // tiles per side
  int tiles;       // nt (nt + 1) / 2
  int splits;      // CTAs along the contraction
  long long rows_per_split;
};

static FactorSplit factor_split(long long rows, int d) {
  FactorSplit s;
  s.nt = (d + TM - 1) / TM;
  s.tiles = s.nt * (s.nt + 1) / 2;
  long long target = 4LL * sm_count();             // ~2 waves of 2 CTAs / SM
  long long by_tiles = (target + s.tiles - 1) / s.tiles;
  long long by_rows = (rows + 1023) / 1024;        // >= 64 k-stages per CTA
  long long sp = by_tiles < by_rows ? by_tiles : by_rows;
  if (sp < 1) sp = 1;
  long long rps = (rows + sp - 1) / sp;
  rps = (rps + TK - 1) / TK * TK;
  if (rps < TK) rps = TK;
  s.splits = (int)((rows + rps - 1) / rps);
  if (s.splits < 1) s.splits = 1;
  s.rows_per_split = rps;
  return s;
}

__global__ void __launch_bounds__(NT, 2)
factor_kernel(Operand X, long long rows, int d, int tiles,
              long long rows_per_split, int splits, float alpha, float beta,
              float* __restrict__ out, float* __restrict__ partial) {
  __shared__ TileSmem sm;
  int bi, bj;
  tri_tile(blockIdx.x, bi, bj);
  const int m0 = bi * TM, n0 = bj * TN;
  const long long kbeg = (long long)blockIdx.y * rows_per_split;
  const long long kend = min(rows, kbeg + rows_per_split);

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  tile_mainloop(X, X, m0, n0, kbeg, kend, sm, acc);

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  if (splits > 1) {
    float* p = partial + ((long long)blockIdx.y * tiles + blockIdx.x) * (TM * TN);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int lr = tile_row(ty, i);
      *reinterpret_cast<float4*>(p + lr * TN + tx * 4) =
          make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
      *reinterpret_cast<float4*>(p + lr * TN + 64 + tx * 4) =
          make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
    }
    return;
  }
  const bool mirror = bi != bj;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int r = m0 + tile_row(ty, i);
    if (r >= d) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      int c = n0 + tile_row(tx, j);
      if (c >= d) continue;
      float* q = out + (long long)r * d + c;
      float v = alpha * acc[i][j];
      if (beta != 0.f) v += beta * (*q);
      *q = v;
      if (mirror) out[(long long)c * d + r] = v;
    }
  }
}

// Sum the partial tiles of every split (ascending split order), scale, blend
// with the previous contents and write both triangles.
__global__ void __launch_bounds__(NT)
factor_reduce_kernel(const float* __restrict__ partial, int tiles, int splits,
                     int d, float alpha, float beta, float* __restrict__ out) {
  int bi, bj;
  tri_tile(blockIdx.x, bi, bj);
  const int m0 = bi * TM, n0 = bj * TN;
  const int tid = threadIdx.x;
  const int lr = blockIdx.y * 8 + (tid >> 5);
  const int lc = (tid & 31) * 4;
  const int r = m0 + lr;
  if (r >= d) return;
  const float* p = partial + (long long)blockIdx.x * (TM * TN) + lr * TN + lc;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int sp = 0; sp < splits; ++sp) {
    float4 v = *reinterpret_cast<const float4*>(p + (long long)sp * tiles * (TM * TN));
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  const float vals[4] = {s.x, s.y, s.z, s.w};
  const bool mirror = bi != bj;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    int c = n0 + lc + e;
    if (c >= d) continue;
    float* q = out + (long long)r * d + c;
    float v = alpha * vals[e];
    if (beta != 0.f) v += beta * (*q);
    *q = v;
    if (mirror) out[(long long)c * d + r] = v;
  }
}

// Built-in scratch for kfac_factor_dense_noalloc: room for
// kNoAllocTiles partial 128x128 tiles.  Lives in every context that loads the
// library, from load until exit.
constexpr int kNoAllocTiles = 512;
constexpr size_t kNoAllocBytes =
    (size_t)kNoAllocTiles * TM * TN * sizeof(float);  // 32 MiB
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocTiles * TM * TN];

// Device address of g_noalloc_scratch on the current device.  In host code the
// array's name is only a handle, so the address is looked up once per device
// (with that device current) and cached.
static int noalloc_scratch_address(float** out) {
  static std::mutex mu;
  static float* cached[64] = {nullptr};
  int dev = 0;
  KFAC_CUDA(cudaGetDevice(&dev));
  KFAC_REQUIRE(dev >= 0 && dev < 64, "device index %d unsupported", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    float* ptr = nullptr;
    KFAC_CUDA(cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch));
    KFAC_REQUIRE(ptr != nullptr, "built-in scratch has no device address");
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return KFAC_OK;
}

static int run_factor(const Operand& X, long long rows, int d, float alpha,
                      float beta, float* out, void* workspace,
                      size_t workspace_bytes, cudaStream_t stream,
                      bool staged = true) {
  KFAC_REQUIRE(out != nullptr && X.base != nullptr, "factor: null pointer");
  KFAC_REQUIRE(rows > 0 && d > 0, "factor: rows=%lld d=%d must be positive",
               rows, d);
  if (engine() == 1)
    return run_factor_tc(X, rows, d, alpha, beta, out, workspace,
                         workspace_bytes, stream, staged);
  FactorSplit s = factor_split(rows, d);
  float* partial = nullptr;
  if (s.splits > 1) {
    size_t need = (size_t)s.splits * s.tiles * TM * TN * sizeof(float);
    if (workspace == nullptr || workspace_bytes < need)
      return fail(KFAC_ERR_WORKSPACE,
                  "factor: workspace of %zu bytes needed, %zu given", need,
                  workspace_bytes);
    partial = static_cast<float*>(workspace);
  }
  dim3 grid(s.tiles, s.splits);
  factor_kernel<<<grid, NT, 0, stream>>>(X, rows, d, s.tiles,
                                         s.rows_per_split, s.splits, alpha,
                                         beta, out, partial);
  KFAC_LAUNCH_CHECK("factor_kernel");
  if (s.splits > 1) {
    dim3 rgrid(s.tiles, TM / 8);
    factor_reduce_kernel<<<rgrid, NT, 0, stream>>>(partial, s.tiles, s.splits,
                                                   d, alpha, beta, out);
    KFAC_LAUNCH_CHECK("factor_reduce_kernel");
  }
  return KFAC_OK;
}

// ------------------------------------------------------------ BN sample grads
// ---- grouped BatchNormalization work: all layers of a step in two launches
struct BnItem {
  const float* x;
  const float* gy;
  float* out;        // (n, 2c) per-sample gradients
  float* stats;      // 2c floats: mean, 1 / sqrt(var + eps)
  int n, c, hw;
  int nhwc;          // 0: (n, c, hw) planes, 1: (n, hw, c) channels-last
  float eps, scale;
  int stat_begin;    // first block of this layer in the statistics launch
  int grad_begin;    // first block of this layer in the gradient launch
  int chan_begin;    // first channel of this layer in the finishing launch
};

constexpr int kBnItemsMax = 256;

__device__ __forceinline__ int bn_find_item(const int* begins, int n, int b) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (begins[mid] <= b) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// Sums of x and x^2 per (sample, channel), in double precision, into the
// scratch behind the statistics; the gradient kernel turns them into the
// batch mean and 1/sqrt(var + eps).  Planes: a warp per (sample, channel).
// Channels-last: a block per (sample, 8 channels).
__global__ void __launch_bounds__(256)
bn_stats_group_kernel(const BnItem* __restrict__ items, int nitems) {
  __shared__ int s_begin[kBnItemsMax];
  __shared__ double sh[2][32][9];
  for (int i = threadIdx.x; i < nitems; i += blockDim.x)
    s_begin[i] = items[i].stat_begin;
  __syncthreads();
  const BnItem it = items[bn_find_item(s_begin, nitems, blockIdx.x)];
  const int b = blockIdx.x - it.stat_begin;
  const long long per = (long long)it.n * it.hw;
  if (!it.nhwc) {
    // planes: a warp per (sample, channel) plane; its sums go to the
    // per-sample scratch like the channels-last ones
    const long long warp = (long long)b * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (warp >= (long long)it.n * it.c) return;
    const int smp = (int)(warp / it.c), ch = (int)(warp - (long long)smp * it.c);
    const float* px = it.x + warp * it.hw;
    double s = 0.0, ss = 0.0;
    for (int i = lane; i < it.hw; i += 32) {
      const double v = px[i];
      s += v;
      ss += v * v;
    }
    for (int o = 16; o > 0; o >>= 1) {
      s += __shfl_down_sync(0xffffffffu, s, o);
      ss += __shfl_down_sync(0xffffffffu, ss, o);
    }
    if (lane == 0) {
      double* part = reinterpret_cast<double*>(it.stats + 2 * it.c);
      part[(long long)smp * 2 * it.c + ch] = s;
      part[(long long)smp * 2 * it.c + it.c + ch] = ss;
    }
    return;
  }
  // channels-last: a block per (sample, 8 channels); 8 channels along the
  // fastest thread index (one 32-byte sector per pixel), 32 pixels in
  // flight per block.  The block leaves its sample's sums in the scratch
  // behind the statistics (doubles, [sample][2c]); the gradient kernel adds
  // the samples up in a fixed order.
  const int groups = (it.c + 7) >> 3;
  const int smp = b / groups, cg = b - smp * groups;
  const int cx = threadIdx.x & 7, px = threadIdx.x >> 3;
  const int ch = 8 * cg + cx;
  double s = 0.0, ss = 0.0;
  if (ch < it.c) {
    const float* p = it.x + (long long)smp * it.hw * it.c + ch;
    for (int q = px; q < it.hw; q += 32) {
      const double v = p[(long long)q * it.c];
      s += v;
      ss += v * v;
    }
  }
  double (*acc)[32][9] = reinterpret_cast<double (*)[32][9]>(&sh[0][0][0]);
  acc[0][px][cx] = s;
  acc[1][px][cx] = ss;
  __syncthreads();
  if (px == 0 && ch < it.c) {
    s = ss = 0.0;
    for (int k = 0; k < 32; ++k) { s += acc[0][k][cx]; ss += acc[1][k][cx]; }
    double* part = reinterpret_cast<double*>(it.stats + 2 * it.c);
    part[(long long)smp * 2 * it.c + ch] = s;
    part[(long long)smp * 2 * it.c + it.c + ch] = ss;
  }
}

// Batch mean and 1/sqrt(var + eps) of every channel from the per-sample sums,
// added up in a fixed order: a thread per channel over all layers.
__global__ void __launch_bounds__(256)
bn_finish_stats_kernel(const BnItem* __restrict__ items, int nitems,
                       int channels) {
  __shared__ int s_begin[kBnItemsMax];
  for (int i = threadIdx.x; i < nitems; i += blockDim.x)
    s_begin[i] = items[i].chan_begin;
  __syncthreads();
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= channels) return;
  const BnItem& it = items[bn_find_item(s_begin, nitems, g)];
  const int ch = g - it.chan_begin;
  const double* part = reinterpret_cast<const double*>(it.stats + 2 * it.c);
  double ds = 0.0, dss = 0.0;
  for (int k = 0; k < it.n; ++k) {
    ds += part[(long long)k * 2 * it.c + ch];
    dss += part[(long long)k * 2 * it.c + it.c + ch];
  }
  const double per = (double)it.n * it.hw;
  const double mean = ds / per;
  double var = dss / per - mean * mean;
  if (var < 0.0) var = 0.0;
  it.stats[ch] = (float)mean;
  it.stats[it.c + ch] = (float)(1.0 / sqrt(var + (double)it.eps));
}

// out[s, j] = scale * sum_p gy xhat, out[s, c + j] = scale * sum_p gy.
// Planes: a warp per (sample, channel).  Channels-last: a block per (sample,
// 32 channels), lanes along channels.
__global__ void __launch_bounds__(256)
bn_grads_group_kernel(const BnItem* __restrict__ items, int nitems) {
  __shared__ int s_begin[kBnItemsMax];
  __shared__ float sh[2][32][9];
  for (int i = threadIdx.x; i < nitems; i += blockDim.x)
    s_begin[i] = items[i].grad_begin;
  __syncthreads();
  const BnItem it = items[bn_find_item(s_begin, nitems, blockIdx.x)];
  const int b = blockIdx.x - it.grad_begin;
  if (!it.nhwc) {
    const long long warp = (long long)b * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (warp >= (long long)it.n * it.c) return;
    const int smp = (int)(warp / it.c), ch = (int)(warp - (long long)smp * it.c);
    const float mean = it.stats[ch], istd = it.stats[it.c + ch];
    const float* px = it.x + warp * it.hw;
    const float* pg = it.gy + warp * it.hw;
    float a = 0.f, g0 = 0.f;
    for (int i = lane; i < it.hw; i += 32) {
      const float g = pg[i] * it.scale;
      a += g * ((px[i] - mean) * istd);
      g0 += g;
    }
    for (int o = 16; o > 0; o >>= 1) {
      a += __shfl_down_sync(0xffffffffu, a, o);
      g0 += __shfl_down_sync(0xffffffffu, g0, o);
    }
    if (lane == 0) {
      it.out[(long long)smp * 2 * it.c + ch] = a;
      it.out[(long long)smp * 2 * it.c + it.c + ch] = g0;
    }
    return;
  }
  // channels-last: a block per (sample, 8 channels), as in the statistics
  // kernel
  const int groups = (it.c + 7) >> 3;
  const int smp = b / groups, cg = b - smp * groups;
  const int cx = threadIdx.x & 7, px = threadIdx.x >> 3;
  const int ch = 8 * cg + cx;
  float a = 0.f, g0 = 0.f;
  if (ch < it.c) {
    const float mean = it.stats[ch], istd = it.stats[it.c + ch];
    const float* pxp = it.x + (long long)smp * it.hw * it.c + ch;
    const float* pg = it.gy + (long long)smp * it.hw * it.c + ch;
    for (int q = px; q < it.hw; q += 32) {
      const float g = pg[(long long)q * it.c] * it.scale;
      a += g * ((pxp[(long long)q * it.c] - mean) * istd);
      g0 += g;
    }
  }
  float (*acc)[32][9] = reinterpret_cast<float (*)[32][9]>(&sh[0][0][0]);
  acc[0][px][cx] = a;
  acc[1][px][cx] = g0;
  __syncthreads();
  if (px == 0 && ch < it.c) {
    a = g0 = 0.f;
    for (int k = 0; k < 32; ++k) { a += acc[0][k][cx]; g0 += acc[1][k][cx]; }
    it.out[(long long)smp * 2 * it.c + ch] = a;
    it.out[(long long)smp * 2 * it.c + it.c + ch] = g0;
  }
}

// Preconditioning of all BatchNormalization blocks: y = F_inv [g_gamma;
// g_beta], a warp per row.
struct BnPrecondItem {
  const float* Finv;
  const float* g0;     // gradient of gamma (c floats)
  const float* g1;     // gradient of beta
  float* y0;           // preconditioned gradients
  float* y1;
  float* p0;           // parameters and velocities for the fused update
  float* p1;
  float* v0;
  float* v1;
  int* flag;           // [0] NaN marker of this call, [1] fallback counter
  int c;
  int row_begin;       // first block (8 rows) of this layer in launch 1
};

__global__ void __launch_bounds__(256)
bn_precond_group_kernel(const BnPrecondItem* __restrict__ items, int nitems) {
  __shared__ int s_begin[kBnItemsMax];
  for (int i = threadIdx.x; i < nitems; i += blockDim.x)
    s_begin[i] = items[i].row_begin;
  __syncthreads();
  const BnPrecondItem it = items[bn_find_item(s_begin, nitems, blockIdx.x)];
  const int d = 2 * it.c;
  const int row = (blockIdx.x - it.row_begin) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= d) return;
  const float* mr = it.Finv + (long long)row * d;
  float s = 0.f;
  for (int k = lane; k < d; k += 32)
    s += mr[k] * (k < it.c ? it.g0[k] : it.g1[k - it.c]);
  for (int o = 16; o > 0; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
  if (lane == 0) {
    if (row < it.c) it.y0[row] = s; else it.y1[row - it.c] = s;
    if (isnan(s)) atomicExch(&it.flag[0], 1);
  }
}

// Second launch, a block per layer: where the product contained a NaN the raw
// gradients take its place (the reference's _check_nan fallback); then,
// if parameters are given, v = momentum v - lr kf; p += v.
__global__ void __launch_bounds__(256)
bn_finish_group_kernel(const BnPrecondItem* __restrict__ items, float lr,
                       float momentum) {
  const BnPrecondItem it = items[blockIdx.x];
  __shared__ int f;
  if (threadIdx.x == 0) f = it.flag[0];
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * it.c; i += blockDim.x) {
    const bool first = i < it.c;
    const int k = first ? i : i - it.c;
    float* y = first ? it.y0 : it.y1;
    float kf = y[k];
    if (f != 0) {
      kf = (first ? it.g0 : it.g1)[k];
      y[k] = kf;
    }
    float* p = first ? it.p0 : it.p1;
    if (p != nullptr) {
      float* v = first ? it.v0 : it.v1;
      const float nv = momentum * v[k] - lr * kf;
      v[k] = nv;
      p[k] += nv;
    }
  }
  if (threadIdx.x == 0 && f != 0) {
    it.flag[0] = 0;
    it.flag[1] += 1;
  }
}

// ---- low-rank form of the BatchNormalization blocks ------------------------
// The factor of a BatchNormalization block is F = sum_s w_s U_s^T U_s over the
// per-sample gradient matrices U_s (n x 2c) of the last few steps (running
// average weights w_s), so its rank is at most m = steps * n, far below 2c
// for the wide layers.  With D = diag(d_gamma ... d_beta ...) the damped
// inverse applied to a gradient g is
//   (D + H^T H)^-1 g = D^-1/2 ( g' - Hs^T (I + Hs Hs^T)^-1 Hs g' ),
//   H = rows sqrt(w_s) u,  Hs = H D^-1/2,  g' = D^-1/2 g,
// which needs the m x m matrix I + Hs Hs^T instead of the 2c x 2c factor.
// Kernel 1 scales the stored rows into Hs; the factor engine forms Hs Hs^T;
// the inverse plan inverts I + Hs Hs^T; kernel 2 applies the formula.
constexpr int kLowRankSlots = 32;

struct BnLowRankItem {
  const float* hist;   // (m x 2c) stored per-sample gradients, slot after slot
  float* Hs;           // (m x 2c) scaled copy
  const float* Minv;   // (m x m) inverse of I + Hs Hs^T (kernel 2)
  const float* g0;     // gradient of gamma, of beta
  const float* g1;
  float* y0;           // preconditioned gradients
  float* y1;
  float* p0;           // parameters / velocities of the fused update (or null)
  float* p1;
  float* v0;
  float* v1;
  int* flag;           // [0] scratch, [1] fallback counter
  int c, m, rows_per_slot;
  float dinv0, dinv1;  // d_gamma^-1/2, d_beta^-1/2
  int blk_begin;       // first block of this layer in the per-row launches
  int col_begin;       // first block of this layer in the per-column launch
  float* vy;           // scratch: v (m floats), then y (m floats)
  float slot_scale[kLowRankSlots];   // sqrt(weight) of every slot (0: unused)
};

__global__ void __launch_bounds__(256)
bn_lowrank_scale_kernel(const BnLowRankItem* __restrict__ items, int nitems) {
  __shared__ int s_begin[kBnItemsMax];
  for (int i = threadIdx.x; i < nitems; i += blockDim.x)
    s_begin[i] = items[i].blk_begin;
  __syncthreads();
  const int idx = bn_find_item(s_begin, nitems, blockIdx.x);
  const BnLowRankItem* it = items + idx;
  const int row = blockIdx.x - it->blk_begin;       // one block per stored row
  const int c = it->c, d = 2 * c;
  const float s = it->slot_scale[row / it->rows_per_slot];
  const float a0 = s * it->dinv0, a1 = s * it->dinv1;
  const float* src = it->hist + (long long)row * d;
  float* dst = it->Hs + (long long)row * d;
  for (int k = threadIdx.x; k < d; k += blockDim.x)
    dst[k] = s == 0.f ? 0.f : src[k] * (k < c ? a0 : a1);
}

// Applying the low-rank form, four grouped launches over all blocks:
//   v = Hs g'          (a CTA per row of Hs; g' = D^-1/2 g on the fly)
//   y = Minv v         (a CTA per row of Minv)
//   kf = D^-1/2 (g' - Hs^T y)   (a thread per column; NaN raises flag[0])
//   finish             (a CTA per block: NaN fallback, fused update)
// v and y live in a scratch the launcher takes from the descriptor ring.
__device__ __forceinline__ int lowrank_find(const int* begins, int n, int b) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (begins[mid] <= b) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ float block_sum_256(float s, float* red) {
  for (int o = 16; o > 0; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  float t = 0.f;
  if (threadIdx.x == 0)
    for (int k = 0; k < 8; ++k) t += red[k];
  return t;                      // valid in thread 0
}

__global__ void __launch_bounds__(256)
bn_lowrank_v_kernel(const BnLowRankItem* __restrict__ items, int nitems) {
  __shared__ int s_begin[kBnItemsMax];
  __shared__ float red[8];
  for (int i = threadIdx.x; i < nitems; i += blockDim.x)
    s_begin[i] = items[i].blk_begin;
  __syncthreads();
  const BnLowRankItem* it = items + lowrank_find(s_begin, nitems, blockIdx.x);
  const int a = blockIdx.x - it->blk_begin;
  const int c = it->c, d = 2 * c;
  const float* hr = it->Hs + (long long)a * d;
  float s = 0.f;
  for (int k = threadIdx.x; k < d; k += 256) {
    const float g = k < c ? it->g0[k] * it->dinv0 : it->g1[k - c] * it->dinv1;
    s += hr[k] * g;
  }
  s = block_sum_256(s, red);
  if (threadIdx.x == 0) it->vy[a] = s;
}

__global__ void __launch_bounds__(256)
bn_lowrank_y_kernel(const BnLowRankItem* __restrict__ items, int nitems) {
  __shared__ int s_begin[kBnItemsMax];
  __shared__ float red[8];
  for (int i = threadIdx.x; i < nitems; i += blockDim.x)
    s_begin[i] = items[i].blk_begin;
  __syncthreads();
  const BnLowRankItem* it = items + lowrank_find(s_begin, nitems, blockIdx.x);
  const int a = blockIdx.x - it->blk_begin;
  const int m = it->m;
  const float* mr = it->Minv + (long long)a * m;
  float s = 0.f;
  for (int b = threadIdx.x; b < m; b += 256) s += mr[b] * it->vy[b];
  s = block_sum_256(s, red);
  if (threadIdx.x == 0) it->vy[m + a] = s;
}

__global__ void __launch_bounds__(256)
bn_lowrank_out_kernel(const BnLowRankItem* __restrict__ items, int nitems) {
  __shared__ int s_begin[kBnItemsMax];
  __shared__ float y[kLowRankSlots * 64];      // a run of 2048 rows at a time
  for (int i = threadIdx.x; i < nitems; i += blockDim.x)
    s_begin[i] = items[i].col_begin;
  __syncthreads();
  const BnLowRankItem* it = items + lowrank_find(s_begin, nitems, blockIdx.x);
  const int c = it->c, d = 2 * c, m = it->m;
  const int k = (blockIdx.x - it->col_begin) * 256 + threadIdx.x;
  float s = 0.f;
  for (int a0 = 0; a0 < m; a0 += kLowRankSlots * 64) {
    const int na = min(kLowRankSlots * 64, m - a0);
    __syncthreads();
    for (int a = threadIdx.x; a < na; a += 256) y[a] = it->vy[m + a0 + a];
    __syncthreads();
    if (k < d) {
      const float* hc = it->Hs + (long long)a0 * d + k;
      for (int a = 0; a < na; ++a) s += hc[(long long)a * d] * y[a];
    }
  }
  if (k < d) {
    const bool first = k < c;
    const float dinv = first ? it->dinv0 : it->dinv1;
    const float g = first ? it->g0[k] : it->g1[k - c];
    const float r = (g * dinv - s) * dinv;
    (first ? it->y0 : it->y1)[first ? k : k - c] = r;
    if (isnan(r)) atomicOr(&it->flag[0], 1);
  }
}

__global__ void __launch_bounds__(256)
bn_lowrank_finish_kernel(const BnLowRankItem* __restrict__ items, float lr,
                         float momentum) {
  const BnLowRankItem* it = items + blockIdx.x;
  const int c = it->c, d = 2 * c;
  const int bad = it->flag[0];
  __syncthreads();
  for (int k = threadIdx.x; k < d; k += 256) {
    const bool first = k < c;
    const int j = first ? k : k - c;
    float* out = first ? it->y0 : it->y1;
    // NaN anywhere: the raw gradients take the result's place
    const float r = bad ? (first ? it->g0 : it->g1)[j] : out[j];
    if (bad) out[j] = r;
    float* p = first ? it->p0 : it->p1;
    if (p != nullptr) {
      float* vel = first ? it->v0 : it->v1;
      const float nv = momentum * vel[j] - lr * r;
      vel[j] = nv;
      p[j] += nv;
    }
  }
  if (threadIdx.x == 0 && bad) {
    it->flag[1] += 1;
    it->flag[0] = 0;
  }
}

__global__ void axpby_kernel(long long count, float a,
                             const float* __restrict__ x, float b,
                             const float* y, float* out) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < count; i += stride) {
    float v = a * x[i];
    if (b != 0.f) v += b * y[i];
    out[i] = v;
  }
}

// out_i = a * x_i + b * y_i for many arrays in one launch: a work item is a
// run of 8192 elements of one array; a block finds its array by bisection in a
// shared-memory copy of the arrays' first items.
struct AxpbyArr {
  const float* x;
  const float* y;
  float* out;
  long long n;
  int item_begin;
};

constexpr int kAxpbyArrMax = 1024;
constexpr int kAxpbyChunk = 8192;

__global__ void __launch_bounds__(256)
axpby_group_kernel(const AxpbyArr* __restrict__ arrs, int narr, int total_items,
                   float a, float b) {
  __shared__ int s_begin[kAxpbyArrMax];
  for (int i = threadIdx.x; i < narr; i += blockDim.x)
    s_begin[i] = arrs[i].item_begin;
  __syncthreads();
  for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
    int lo = 0, hi = narr - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s_begin[mid] <= item) lo = mid; else hi = mid - 1;
    }
    const AxpbyArr r = arrs[lo];
    const long long base = (long long)(item - r.item_begin) * kAxpbyChunk;
#pragma unroll 4
    for (int k = threadIdx.x; k < kAxpbyChunk; k += 256) {
      const long long i = base + k;
      if (i < r.n) {
        float v = a * r.x[i];
        if (b != 0.f) v += b * r.y[i];
        r.out[i] = v;
      }
    }
  }
}

// Weight rescaling of the ImageNet recipe: w *= target / (|w| + eps) when that
// factor is below 1.  Pass 1 adds block sums of squares into *sumsq (cleared
// by the caller), pass 2 scales.
__global__ void __launch_bounds__(256)
sumsq_kernel(long long count, const float* __restrict__ w,
             float* __restrict__ sumsq) {
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
       i < count; i += (long long)gridDim.x * blockDim.x)
    s += w[i] * w[i];
  __shared__ float sh[8];
  for (int o = 16; o > 0; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    s = 0.f;
    for (int k = 0; k < 8; ++k) s += sh[k];
    atomicAdd(sumsq, s);
  }
}

__global__ void __launch_bounds__(256)
norm_clip_kernel(long long count, float* __restrict__ w,
                 const float* __restrict__ sumsq, float target, float eps,
                 float* __restrict__ scale_out) {
  const float scale = target / (sqrtf(*sumsq) + eps);
  if (scale_out != nullptr && blockIdx.x == 0 && threadIdx.x == 0)
    *scale_out = scale;
  if (!(scale < 1.f)) return;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
       i < count; i += (long long)gridDim.x * blockDim.x)
    w[i] *= scale;
}

__global__ void momentum_kernel(long long count, const float* __restrict__ grad,
                                float* param, float* v, float lr,
                                float momentum) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < count; i += stride) {
    float nv = momentum * v[i] - lr * grad[i];
    v[i] = nv;
    param[i] += nv;
  }
}

}  // namespace kfac

using namespace kfac;

extern "C" size_t kfac_factor_workspace_bytes(int64_t rows, int d) {
  if (rows <= 0 || d <= 0) return 0;
  if (engine() == 1) return tc_factor_workspace_bytes(rows, d);
  FactorSplit s = factor_split(rows, d);
  if (s.splits <= 1) return 0;
  return (size_t)s.splits * s.tiles * TM * TN * sizeof(float);
}

extern "C" int kfac_factor_dense(const float* x, int64_t rows, int d_in,
                                 int64_t ld, int add_ones_col, float alpha,
                                 float beta, float* out, void* workspace,
                                 size_t workspace_bytes, void* stream) {
  KFAC_REQUIRE(ld >= d_in, "factor_dense: ld=%lld < d_in=%d", (long long)ld,
               d_in);
  Operand X = strided_operand(x, ld, 1, d_in);
  if (add_ones_col) X.extra_idx = d_in;
  return run_factor(X, rows, d_in + (add_ones_col ? 1 : 0), alpha, beta, out,
                    workspace, workspace_bytes, (cudaStream_t)stream);
}

static Operand conv_input_operand(const float* x, int c, int h, int w,
                                  int ksize, int stride, int pad,
                                  int add_ones_col) {
  const int ho = (h + 2 * pad - ksize) / stride + 1;
  const int wo = (w + 2 * pad - ksize) / stride + 1;
  Operand X = {};
  X.base = x;
  X.ncols = c * ksize * ksize;
  X.extra_idx = add_ones_col ? X.ncols : -1;
  X.kfast = 1;
  X.mode = 1;
  X.period = 1;
  X.C = c; X.H = h; X.W = w; X.ks = ksize; X.st = stride; X.pd = pad;
  X.Ho = ho; X.Wo = wo;
  if (ksize == 1 && pad == 0 && stride == 1) {
    // 1x1 convolution: the patch matrix is the NCHW tensor viewed as
    // (n*h*w, c); no gather needed.
    X = strided_operand(x, 0, (long long)h * w, c);
    X.period = h * w;
    X.s_outer = (long long)c * h * w;
    X.s_inner = 1;
    X.kfast = 1;
    X.extra_idx = add_ones_col ? c : -1;
  }
  return X;
}

extern "C" size_t kfac_factor_conv_workspace_bytes(int n, int c, int h, int w,
                                                   int ksize, int stride,
                                                   int pad, int add_ones_col) {
  if (n <= 0 || c <= 0 || h <= 0 || w <= 0 || ksize <= 0 || stride <= 0 ||
      pad < 0)
    return 0;
  const int ho = (h + 2 * pad - ksize) / stride + 1;
  const int wo = (w + 2 * pad - ksize) / stride + 1;
  if (ho <= 0 || wo <= 0) return 0;
  const int d = c * ksize * ksize + (add_ones_col ? 1 : 0);
  size_t bytes = kfac_factor_workspace_bytes((int64_t)n * ho * wo, d);
  if (engine() == 1) {
    Operand X = conv_input_operand(nullptr, c, h, w, ksize, stride, pad,
                                   add_ones_col);
    bytes += tc_pad_bytes(X, n);
  }
  return bytes;
}

extern "C" int kfac_factor_conv_input(const float* x, int n, int c, int h,
                                      int w, int ksize, int stride, int pad,
                                      int add_ones_col, float alpha, float beta,
                                      float* out, void* workspace,
                                      size_t workspace_bytes, void* stream) {
  KFAC_REQUIRE(n > 0 && c > 0 && h > 0 && w > 0 && ksize > 0 && stride > 0 &&
                   pad >= 0,
               "factor_conv_input: bad geometry n=%d c=%d h=%d w=%d k=%d s=%d "
               "p=%d", n, c, h, w, ksize, stride, pad);
  KFAC_REQUIRE((long long)n * c * h * w < (1LL << 31),
               "factor_conv_input: input has more than 2^31 elements");
  int ho = (h + 2 * pad - ksize) / stride + 1;
  int wo = (w + 2 * pad - ksize) / stride + 1;
  KFAC_REQUIRE(ho > 0 && wo > 0, "factor_conv_input: empty output");
  Operand X = conv_input_operand(x, c, h, w, ksize, stride, pad,
                                 add_ones_col);
  int d = c * ksize * ksize + (add_ones_col ? 1 : 0);
  return run_factor(X, (long long)n * ho * wo, d, alpha, beta, out, workspace,
                    workspace_bytes, (cudaStream_t)stream);
}

extern "C" int kfac_factor_conv_grad(const float* gy, int n, int c, int ho,
                                     int wo, float alpha, float beta,
                                     float* out, void* workspace,
                                     size_t workspace_bytes, void* stream) {
  KFAC_REQUIRE(n > 0 && c > 0 && ho > 0 && wo > 0,
               "factor_conv_grad: bad geometry n=%d c=%d ho=%d wo=%d", n, c, ho,
               wo);
  Operand X = strided_operand(gy, 0, (long long)ho * wo, c);
  X.period = ho * wo;
  X.s_outer = (long long)c * ho * wo;
  X.s_inner = 1;
  X.kfast = 1;
  return run_factor(X, (long long)n * ho * wo, c, alpha, beta, out, workspace,
                    workspace_bytes, (cudaStream_t)stream);
}

extern "C" int kfac_bn_sample_grads_group(int count,
                                          const kfac_bn_item* items,
                                          void* stream) {
  KFAC_REQUIRE(count > 0 && items != nullptr, "bn_sample_grads_group: no items");
  KFAC_REQUIRE(count <= kBnItemsMax,
               "bn_sample_grads_group: %d layers in one call, at most %d",
               count, kBnItemsMax);
  std::vector<BnItem> tab(count);
  long long sb = 0, gb = 0, cbeg = 0;
  for (int i = 0; i < count; ++i) {
    const kfac_bn_item& k = items[i];
    KFAC_REQUIRE(k.x && k.gy && k.out && k.stats,
                 "bn_sample_grads_group: null pointer at %d", i);
    KFAC_REQUIRE(k.n > 0 && k.c > 0 && k.hw > 0 &&
                     (k.layout == 0 || k.layout == 1),
                 "bn_sample_grads_group: bad shape or layout at %d", i);
    BnItem& t = tab[i];
    t.x = k.x; t.gy = k.gy; t.out = k.out; t.stats = k.stats;
    t.n = k.n; t.c = k.c; t.hw = k.hw;
    t.nhwc = (k.layout == 1 && k.hw > 1) ? 1 : 0;
    t.eps = k.eps; t.scale = k.scale;
    t.stat_begin = (int)sb;
    t.grad_begin = (int)gb;
    t.chan_begin = (int)cbeg;
    cbeg += k.c;
    const long long cg = (k.c + 7) / 8;
    sb += t.nhwc ? (long long)k.n * cg : ((long long)k.n * k.c + 7) / 8;
    gb += t.nhwc ? (long long)k.n * cg : ((long long)k.n * k.c + 7) / 8;
    KFAC_REQUIRE(sb < (1ll << 31) && gb < (1ll << 31),
                 "bn_sample_grads_group: too many blocks");
  }
  void* dev = nullptr;
  int rc = ring_alloc(tab.size() * sizeof(BnItem), &dev);
  if (rc != KFAC_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  KFAC_CUDA(cudaMemcpyAsync(dev, tab.data(), tab.size() * sizeof(BnItem),
                            cudaMemcpyHostToDevice, st));
  bn_stats_group_kernel<<<(int)sb, 256, 0, st>>>(static_cast<BnItem*>(dev),
                                                 count);
  KFAC_LAUNCH_CHECK("bn_stats_group_kernel");
  KFAC_REQUIRE(cbeg < (1ll << 31), "bn_sample_grads_group: too many channels");
  bn_finish_stats_kernel<<<(int)((cbeg + 255) / 256), 256, 0, st>>>(
      static_cast<BnItem*>(dev), count, (int)cbeg);
  KFAC_LAUNCH_CHECK("bn_finish_stats_kernel");
  bn_grads_group_kernel<<<(int)gb, 256, 0, st>>>(static_cast<BnItem*>(dev),
                                                 count);
  KFAC_LAUNCH_CHECK("bn_grads_group_kernel");
  return KFAC_OK;
}

extern "C" int kfac_bn_sample_grads(const float* x, const float* gy, int n,
                                    int c, int hw, float eps, float scale,
                                    float* out, float* stats, void* stream) {
  kfac_bn_item it;
  it.x = x; it.gy = gy; it.out = out; it.stats = stats;
  it.n = n; it.c = c; it.hw = hw; it.layout = 0; it.eps = eps;
  it.scale = scale;
  return kfac_bn_sample_grads_group(1, &it, stream);
}

extern "C" int kfac_bn_precondition_group(
    int count, const int* channels, const float* const* F_inv,
    const float* const* grad_gamma, const float* const* grad_beta,
    float* const* kf_gamma, float* const* kf_beta, float* const* param_gamma,
    float* const* param_beta, float* const* mom_gamma, float* const* mom_beta,
    int* const* nan_flags, float lr, float momentum, void* stream) {
  KFAC_REQUIRE(count > 0 && channels && F_inv && grad_gamma && grad_beta &&
                   kf_gamma && kf_beta && nan_flags,
               "bn_precondition_group: null argument or count=%d", count);
  KFAC_REQUIRE(count <= kBnItemsMax,
               "bn_precondition_group: %d layers in one call, at most %d",
               count, kBnItemsMax);
  std::vector<BnPrecondItem> tab(count);
  long long rb = 0;
  for (int i = 0; i < count; ++i) {
    KFAC_REQUIRE(channels[i] > 0 && F_inv[i] && grad_gamma[i] && grad_beta[i] &&
                     kf_gamma[i] && kf_beta[i] && nan_flags[i],
                 "bn_precondition_group: bad layer %d", i);
    BnPrecondItem& t = tab[i];
    t.Finv = F_inv[i];
    t.g0 = grad_gamma[i]; t.g1 = grad_beta[i];
    t.y0 = kf_gamma[i]; t.y1 = kf_beta[i];
    const bool fused = param_gamma && param_gamma[i];
    if (fused)
      KFAC_REQUIRE(param_beta && param_beta[i] && mom_gamma && mom_gamma[i] &&
                       mom_beta && mom_beta[i],
                   "bn_precondition_group: fused update of layer %d lacks a "
                   "parameter or velocity pointer", i);
    t.p0 = fused ? param_gamma[i] : nullptr;
    t.p1 = fused ? param_beta[i] : nullptr;
    t.v0 = fused ? mom_gamma[i] : nullptr;
    t.v1 = fused ? mom_beta[i] : nullptr;
    t.flag = nan_flags[i];
    t.c = channels[i];
    t.row_begin = (int)rb;
    rb += (2LL * channels[i] + 7) / 8;
    KFAC_REQUIRE(rb < (1ll << 31), "bn_precondition_group: too many rows");
  }
  void* dev = nullptr;
  int rc = ring_alloc(tab.size() * sizeof(BnPrecondItem), &dev);
  if (rc != KFAC_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  KFAC_CUDA(cudaMemcpyAsync(dev, tab.data(), tab.size() * sizeof(BnPrecondItem),
                            cudaMemcpyHostToDevice, st));
  bn_precond_group_kernel<<<(int)rb, 256, 0, st>>>(
      static_cast<BnPrecondItem*>(dev), count);
  KFAC_LAUNCH_CHECK("bn_precond_group_kernel");
  bn_finish_group_kernel<<<count, 256, 0, st>>>(
      static_cast<BnPrecondItem*>(dev), lr, momentum);
  KFAC_LAUNCH_CHECK("bn_finish_group_kernel");
  return KFAC_OK;
}

static int lowrank_table(int count, const kfac_bn_lowrank_item* items,
                         std::vector<BnLowRankItem>& tab, long long& blocks) {
  KFAC_REQUIRE(count > 0 && items != nullptr, "bn_lowrank: no items");
  KFAC_REQUIRE(count <= kBnItemsMax, "bn_lowrank: %d layers, at most %d",
               count, kBnItemsMax);
  tab.resize(count);
  blocks = 0;
  for (int i = 0; i < count; ++i) {
    const kfac_bn_lowrank_item& k = items[i];
    KFAC_REQUIRE(k.hist && k.scaled && k.c > 0 && k.rows_per_slot > 0 &&
                     k.slots > 0 && k.slots <= kLowRankSlots,
                 "bn_lowrank: bad item %d", i);
    BnLowRankItem& t = tab[i];
    t.hist = k.hist; t.Hs = k.scaled; t.Minv = k.m_inv;
    t.g0 = k.grad_gamma; t.g1 = k.grad_beta;
    t.y0 = k.kf_gamma; t.y1 = k.kf_beta;
    t.p0 = k.param_gamma; t.p1 = k.param_beta;
    t.v0 = k.mom_gamma; t.v1 = k.mom_beta;
    t.flag = k.nan_flag;
    t.c = k.c; t.rows_per_slot = k.rows_per_slot;
    t.m = k.slots * k.rows_per_slot;
    KFAC_REQUIRE(k.damp_gamma > 0.f && k.damp_beta > 0.f,
                 "bn_lowrank: damping must be positive (item %d)", i);
    t.dinv0 = 1.f / sqrtf(k.damp_gamma);
    t.dinv1 = 1.f / sqrtf(k.damp_beta);
    for (int s = 0; s < kLowRankSlots; ++s)
      t.slot_scale[s] = s < k.slots && k.slot_weight[s] > 0.f
                            ? sqrtf(k.slot_weight[s]) : 0.f;
    t.blk_begin = (int)blocks;
    blocks += t.m;
  }
  KFAC_REQUIRE(blocks < (1ll << 31), "bn_lowrank: too many rows");
  return KFAC_OK;
}

extern "C" int kfac_bn_lowrank_scale(int count,
                                     const kfac_bn_lowrank_item* items,
                                     void* stream) {
  std::vector<BnLowRankItem> tab;
  long long blocks = 0;
  int rc = lowrank_table(count, items, tab, blocks);
  if (rc != KFAC_OK) return rc;
  void* dev = nullptr;
  rc = ring_alloc(tab.size() * sizeof(BnLowRankItem), &dev);
  if (rc != KFAC_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  KFAC_CUDA(cudaMemcpyAsync(dev, tab.data(), tab.size() * sizeof(BnLowRankItem),
                            cudaMemcpyHostToDevice, st));
  bn_lowrank_scale_kernel<<<(int)blocks, 256, 0, st>>>(
      static_cast<const BnLowRankItem*>(dev), count);
  KFAC_LAUNCH_CHECK("bn_lowrank_scale_kernel");
  return KFAC_OK;
}

extern "C" int kfac_bn_lowrank_apply(int count,
                                     const kfac_bn_lowrank_item* items,
                                     float lr, float momentum, void* stream) {
  std::vector<BnLowRankItem> tab;
  long long blocks = 0;
  int rc = lowrank_table(count, items, tab, blocks);
  if (rc != KFAC_OK) return rc;
  for (int i = 0; i < count; ++i) {
    const kfac_bn_lowrank_item& k = items[i];
    KFAC_REQUIRE(k.m_inv && k.grad_gamma && k.grad_beta && k.kf_gamma &&
                     k.kf_beta && k.nan_flag,
                 "bn_lowrank_apply: null pointer in item %d", i);
    KFAC_REQUIRE(!k.param_gamma ||
                     (k.param_beta && k.mom_gamma && k.mom_beta),
                 "bn_lowrank_apply: fused update of item %d lacks a pointer",
                 i);
  }
  // v and y of every block from the descriptor ring
  long long vy_floats = 0, cols = 0;
  for (BnLowRankItem& t : tab) {
    t.col_begin = (int)cols;
    cols += (2 * t.c + 255) / 256;
    vy_floats += 2 * t.m;
  }
  KFAC_REQUIRE(cols < (1ll << 31), "bn_lowrank_apply: too many columns");
  void* vy = nullptr;
  rc = ring_alloc((size_t)vy_floats * sizeof(float), &vy);
  if (rc != KFAC_OK) return rc;
  {
    float* p = static_cast<float*>(vy);
    for (BnLowRankItem& t : tab) {
      t.vy = p;
      p += 2 * t.m;
    }
  }
  void* dev = nullptr;
  rc = ring_alloc(tab.size() * sizeof(BnLowRankItem), &dev);
  if (rc != KFAC_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  KFAC_CUDA(cudaMemcpyAsync(dev, tab.data(), tab.size() * sizeof(BnLowRankItem),
                            cudaMemcpyHostToDevice, st));
  const BnLowRankItem* d_items = static_cast<const BnLowRankItem*>(dev);
  bn_lowrank_v_kernel<<<(int)blocks, 256, 0, st>>>(d_items, count);
  KFAC_LAUNCH_CHECK("bn_lowrank_v_kernel");
  bn_lowrank_y_kernel<<<(int)blocks, 256, 0, st>>>(d_items, count);
  KFAC_LAUNCH_CHECK("bn_lowrank_y_kernel");
  bn_lowrank_out_kernel<<<(int)cols, 256, 0, st>>>(d_items, count);
  KFAC_LAUNCH_CHECK("bn_lowrank_out_kernel");
  bn_lowrank_finish_kernel<<<count, 256, 0, st>>>(d_items, lr, momentum);
  KFAC_LAUNCH_CHECK("bn_lowrank_finish_kernel");
  return KFAC_OK;
}

extern "C" int kfac_axpby(int64_t count, float a, const float* x, float b,
                          const float* y, float* out, void* stream) {
  if (count <= 0) return KFAC_OK;
  KFAC_REQUIRE(x && out && (b == 0.f || y), "axpby: null pointer");
  int blocks = ceil_div(count, 256 * 4);
  int cap = sm_count() * 16;
  if (blocks > cap) blocks = cap;
  axpby_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(count, a, x, b, y,
                                                         out);
  KFAC_LAUNCH_CHECK("axpby_kernel");
  return KFAC_OK;
}

extern "C" int kfac_axpby_group(int n_arrays, const int64_t* counts, float a,
                                const float* const* x, float b,
                                const float* const* y, float* const* out,
                                void* stream) {
  if (n_arrays <= 0) return KFAC_OK;
  KFAC_REQUIRE(counts && x && out && (b == 0.f || y),
               "axpby_group: null argument");
  KFAC_REQUIRE(n_arrays <= kAxpbyArrMax,
               "axpby_group: %d arrays in one call, at most %d", n_arrays,
               kAxpbyArrMax);
  std::vector<AxpbyArr> tab(n_arrays);
  long long items = 0;
  for (int i = 0; i < n_arrays; ++i) {
    KFAC_REQUIRE(counts[i] >= 0, "axpby_group: negative count at %d", i);
    KFAC_REQUIRE(counts[i] == 0 || (x[i] && out[i] && (b == 0.f || y[i])),
                 "axpby_group: null pointer at %d", i);
    tab[i].x = x[i];
    tab[i].y = b == 0.f ? nullptr : y[i];
    tab[i].out = out[i];
    tab[i].n = counts[i];
    tab[i].item_begin = (int)items;
    items += (counts[i] + kAxpbyChunk - 1) / kAxpbyChunk;
    KFAC_REQUIRE(items < (1ll << 31), "axpby_group: too many elements");
  }
  if (items == 0) return KFAC_OK;
  void* dev = nullptr;
  int rc = ring_alloc(tab.size() * sizeof(AxpbyArr), &dev);
  if (rc != KFAC_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  KFAC_CUDA(cudaMemcpyAsync(dev, tab.data(), tab.size() * sizeof(AxpbyArr),
                            cudaMemcpyHostToDevice, st));
  const long long cap = (long long)sm_count() * 8;
  const int grid = (int)(items < cap ? items : cap);
  axpby_group_kernel<<<grid, 256, 0, st>>>(static_cast<const AxpbyArr*>(dev),
                                           n_arrays, (int)items, a, b);
  KFAC_LAUNCH_CHECK("axpby_group_kernel");
  return KFAC_OK;
}

extern "C" int kfac_momentum_update(int64_t count, const float* grad,
                                    float* param, float* v, float lr,
                                    float momentum, void* stream) {
  if (count <= 0) return KFAC_OK;
  KFAC_REQUIRE(grad && param && v, "momentum_update: null pointer");
  int blocks = ceil_div(count, 256 * 4);
  int cap = sm_count() * 16;
  if (blocks > cap) blocks = cap;
  momentum_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(count, grad, param,
                                                            v, lr, momentum);
  KFAC_LAUNCH_CHECK("momentum_kernel");
  return KFAC_OK;
}

extern "C" int kfac_normalize_weight(int64_t count, float* w,
                                     float target_norm, float eps,
                                     float* scratch, void* stream) {
  if (count <= 0) return KFAC_OK;
  KFAC_REQUIRE(w && scratch, "normalize_weight: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  KFAC_CUDA(cudaMemsetAsync(scratch, 0, sizeof(float), st));
  int blocks = ceil_div(count, 256 * 8);
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  sumsq_kernel<<<blocks, 256, 0, st>>>(count, w, scratch);
  KFAC_LAUNCH_CHECK("sumsq_kernel");
  norm_clip_kernel<<<blocks, 256, 0, st>>>(count, w, scratch, target_norm, eps,
                                           scratch + 1);
  KFAC_LAUNCH_CHECK("norm_clip_kernel");
  return KFAC_OK;
}

extern "C" size_t kfac_factor_noalloc_max_bytes(void) { return kNoAllocBytes; }

extern "C" int kfac_factor_dense_noalloc(const float* x, int64_t rows,
                                         int d_in, int64_t ld,
                                         int add_ones_col, float alpha,
                                         float beta, float* out,
                                         void* stream) {
  KFAC_REQUIRE(ld >= d_in, "factor_dense_noalloc: ld=%lld < d_in=%d",
               (long long)ld, d_in);
  const int d = d_in + (add_ones_col ? 1 : 0);
  // (no staging pass here: its planes would not fit the built-in scratch and
  // its tensor maps travel through an allocated table)
  size_t need = engine() == 1 ? tc_factor_workspace_bytes(rows, d, false)
                              : kfac_factor_workspace_bytes(rows, d);
  if (need > kNoAllocBytes)
    return fail(KFAC_ERR_WORKSPACE,
                "factor_dense_noalloc: rows=%lld d=%d needs %zu bytes of "
                "scratch, the built-in scratch holds %zu; use "
                "kfac_factor_dense with a caller workspace",
                (long long)rows, d, need, kNoAllocBytes);
  float* scratch = nullptr;
  int rc = noalloc_scratch_address(&scratch);
  if (rc != KFAC_OK) return rc;
  Operand X = strided_operand(x, ld, 1, d_in);
  if (add_ones_col) X.extra_idx = d_in;
  // Every partial tile is written in full before it is read, so nothing in
  // the shared scratch has to be cleared between calls.
  return run_factor(X, rows, d, alpha, beta, out, scratch, kNoAllocBytes,
                    (cudaStream_t)stream, false);
}

// ------------------------------------------------------------ grouped build
static int job_from_item(const kfac_factor_item& it, FactorJob& job) {
  job.alpha = it.alpha;
  job.beta = it.beta;
  job.out = it.out;
  job.n = it.n;
  job.nhwc = 0;
  KFAC_REQUIRE(it.layout == 0 ||
                   (it.layout == 1 && it.kind == KFAC_FACTOR_CONV_INPUT),
               "factor_group: layout %d of item kind %d unsupported", it.layout,
               it.kind);
  if (it.kind == KFAC_FACTOR_DENSE) {
    KFAC_REQUIRE(it.ld >= it.d_in && it.rows > 0 && it.d_in > 0,
                 "factor_group: bad dense item");
    job.X = strided_operand(it.x, it.ld, 1, it.d_in);
    if (it.add_ones_col) job.X.extra_idx = it.d_in;
    job.rows = it.rows;
    job.d = it.d_in + (it.add_ones_col ? 1 : 0);
    job.n = 0;
  } else if (it.kind == KFAC_FACTOR_DENSE_T) {
    // X given transposed: x is (d_in x rows) row-major with pitch ld, i.e.
    // out = alpha * x x^T + beta * out, contraction along x's rows
    KFAC_REQUIRE(it.ld >= it.rows && it.rows > 0 && it.d_in > 0 &&
                     !it.add_ones_col,
                 "factor_group: bad transposed dense item");
    job.X = strided_operand(it.x, 1, it.ld, it.d_in);
    job.rows = it.rows;
    job.d = it.d_in;
    job.n = 0;
  } else if (it.kind == KFAC_FACTOR_CONV_INPUT) {
    KFAC_REQUIRE(it.n > 0 && it.c > 0 && it.h > 0 && it.w > 0 && it.ksize > 0 &&
                     it.stride > 0 && it.pad >= 0,
                 "factor_group: bad conv input item");
    KFAC_REQUIRE((long long)it.n * it.c * it.h * it.w < (1LL << 31),
                 "factor_group: input has more than 2^31 elements");
    const int ho = (it.h + 2 * it.pad - it.ksize) / it.stride + 1;
    const int wo = (it.w + 2 * it.pad - it.ksize) / it.stride + 1;
    KFAC_REQUIRE(ho > 0 && wo > 0, "factor_group: empty output");
    job.X = conv_input_operand(it.x, it.c, it.h, it.w, it.ksize, it.stride,
                               it.pad, it.add_ones_col);
    job.rows = (long long)it.n * ho * wo;
    job.d = it.c * it.ksize * it.ksize + (it.add_ones_col ? 1 : 0);
    job.nhwc = it.layout;
    KFAC_REQUIRE(!job.nhwc || engine() == 1,
                 "factor_group: channels-last inputs need the tensor-core "
                 "engine");
  } else if (it.kind == KFAC_FACTOR_CONV_GRAD) {
    KFAC_REQUIRE(it.n > 0 && it.c > 0 && it.h > 0 && it.w > 0,
                 "factor_group: bad conv grad item");
    job.X = strided_operand(it.x, 0, (long long)it.h * it.w, it.c);
    job.X.period = it.h * it.w;
    job.X.s_outer = (long long)it.c * it.h * it.w;
    job.X.s_inner = 1;
    job.X.kfast = 1;
    job.rows = (long long)it.n * it.h * it.w;
    job.d = it.c;
    job.n = 0;
  } else {
    return fail(KFAC_ERR_INVALID, "factor_group: unknown kind %d", it.kind);
  }
  KFAC_REQUIRE(it.x != nullptr && it.out != nullptr,
               "factor_group: null pointer");
  return KFAC_OK;
}

static size_t simt_item_bytes(const FactorJob& job) {
  FactorSplit s = factor_split(job.rows, job.d);
  return s.splits > 1 ? (size_t)s.splits * s.tiles * TM * TN * sizeof(float)
                      : 0;
}

extern "C" size_t kfac_factor_group_workspace_bytes(
    int count, const kfac_factor_item* items) {
  if (count <= 0 || items == nullptr) return 0;
  std::vector<FactorJob> jobs(count);
  for (int i = 0; i < count; ++i)
    if (job_from_item(items[i], jobs[i]) != KFAC_OK) return 0;
  if (engine() == 1) return tc_factor_group_workspace_bytes(count, jobs.data());
  size_t m = 0;
  for (int i = 0; i < count; ++i) m = std::max(m, simt_item_bytes(jobs[i]));
  return m;
}

extern "C" int kfac_factor_group(int count, const kfac_factor_item* items,
                                 void* workspace, size_t workspace_bytes,
                                 void* stream) {
  KFAC_REQUIRE(count > 0 && items != nullptr, "factor_group: no items");
  std::vector<FactorJob> jobs(count);
  for (int i = 0; i < count; ++i) {
    int rc = job_from_item(items[i], jobs[i]);
    if (rc != KFAC_OK) return rc;
  }
  if (engine() == 1)
    return run_factor_group_tc(count, jobs.data(), workspace, workspace_bytes,
                               (cudaStream_t)stream);
  for (int i = 0; i < count; ++i) {   // fp32 engine: one factor after another
    int rc = run_factor(jobs[i].X, jobs[i].rows, jobs[i].d, jobs[i].alpha,
                        jobs[i].beta, jobs[i].out, workspace, workspace_bytes,
                        (cudaStream_t)stream);
    if (rc != KFAC_OK) return rc;
  }
  return KFAC_OK;
}
