// Grouped fp32 tile GEMM: one launch covers the tiles of many independent
// problems (all layers of a stage).  Used by the inverse and the
// precondition stages.
#include <atomic>

#include "gemm_simt.cuh"

namespace kfac {

static __thread char g_err[512];
char* error_buffer() { return g_err; }

static std::atomic<long long> g_launches(0);
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
void count_launches(long long n) {
  g_launches.fetch_add(n, std::memory_order_relaxed);
}
long long launch_count_now() {
  return g_launches.load(std::memory_order_relaxed);
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) !=
            cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

__global__ void __launch_bounds__(NT, 2)
gemm_grouped_kernel(const GemmDesc* __restrict__ descs, int ndesc, float lr,
                    float momentum) {
  __shared__ TileSmem sm;
  __shared__ GemmDesc sd;
  const int tid = threadIdx.x;
  const int tile = blockIdx.x;

  // locate the problem that owns this tile (tile_begin is ascending)
  int lo = 0, hi = ndesc - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (descs[mid].tile_begin <= tile) lo = mid; else hi = mid - 1;
  }
  {
    const int* src = reinterpret_cast<const int*>(descs + lo);
    int* dst = reinterpret_cast<int*>(&sd);
    for (int i = tid; i < (int)(sizeof(GemmDesc) / sizeof(int)); i += NT)
      dst[i] = src[i];
  }
  __syncthreads();
  if (sd.gate != nullptr && *sd.gate == 0) return;   // uniform per CTA

  const int lt = tile - sd.tile_begin;
  int bi, bj;
  if (sd.flags & G_LOWER) {
    tri_tile(lt, bi, bj);
  } else {
    bi = lt / sd.tiles_n;
    bj = lt - bi * sd.tiles_n;
  }
  const int m0 = bi * TM, n0 = bj * TN;
  long long kbeg = 0, kend = sd.K;
  if (sd.flags & G_KBEG_N0) kbeg = n0;
  if (sd.flags & G_KBEG_M0) kbeg = m0;
  if (sd.flags & G_KEND_M0) kend = min((long long)(m0 + TM), sd.K);

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  tile_mainloop(sd.A, sd.B, m0, n0, kbeg, kend, sm, acc);

  const int tx = tid & 15, ty = tid >> 4;
  if (sd.flags & G_PRECOND) {
    const int dW = sd.dW;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int r = m0 + tile_row(ty, i);
      if (r >= sd.M) continue;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        int c = n0 + tile_row(tx, j);
        if (c >= sd.N) continue;
        float kf = acc[i][j];
        float *okf, *op, *ov;
        long long idx;
        if (c < dW) {
          idx = (long long)r * dW + c;
          okf = sd.kfW; op = sd.pW; ov = sd.vW;
        } else {
          idx = r;
          okf = sd.kfb; op = sd.pb; ov = sd.vb;
        }
        if (okf) okf[idx] = kf;
        if (op) {
          float v = momentum * ov[idx] - lr * kf;
          ov[idx] = v;
          op[idx] += v;
        }
      }
    }
    return;
  }

  const bool mirror = (sd.flags & G_MIRROR) && (bi != bj);
  const float alpha = sd.alpha, beta = sd.beta;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int r = m0 + tile_row(ty, i);
    if (r >= sd.M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      int c = n0 + tile_row(tx, j);
      if (c >= sd.N) continue;
      float* p = sd.C + (long long)r * sd.ldc + c;
      float v = alpha * acc[i][j];
      if (beta != 0.f) v += beta * (*p);
      *p = v;
      if (mirror) sd.C[(long long)c * sd.ldc + r] = v;
      if (sd.C2 != nullptr) sd.C2[(long long)r * sd.ldc + c] = v;
    }
  }
}

int launch_grouped_gemm(const GemmDesc* descs_dev, int ndesc, int total_tiles,
                        float lr, float momentum, cudaStream_t stream) {
  if (ndesc <= 0 || total_tiles <= 0) return KFAC_OK;
  gemm_grouped_kernel<<<total_tiles, NT, 0, stream>>>(descs_dev, ndesc, lr,
                                                      momentum);
  KFAC_LAUNCH_CHECK("gemm_grouped_kernel");
  return KFAC_OK;
}

}  // namespace kfac

extern "C" int kfac_abi_version(void) { return 2; }
extern "C" const char* kfac_last_error(void) { return kfac::error_buffer(); }
extern "C" int64_t kfac_launch_count(void) {
  return kfac::g_launches.load(std::memory_order_relaxed);
}
