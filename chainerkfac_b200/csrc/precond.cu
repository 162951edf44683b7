// Preconditioning kf = G_inv * [grad_W, grad_b] * A_inv for all layers in two
// grouped launches; the second launch's epilogue splits the result into the
// weight and bias parts and can apply the momentum update in place.
#include <vector>

#include "gemm_simt.cuh"

using namespace kfac;

static size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

extern "C" size_t kfac_precond_workspace_bytes(int count, const int* dG,
                                               const int* dW,
                                               const int* has_bias) {
  if (count <= 0 || !dG || !dW) return 0;
  size_t total = align256(2 * (size_t)count * sizeof(GemmDesc));
  for (int i = 0; i < count; ++i) {
    size_t dA = (size_t)dW[i] + ((has_bias && has_bias[i]) ? 1 : 0);
    total += align256((size_t)dG[i] * dA * sizeof(float));
  }
  return total;
}

extern "C" int kfac_precondition(
    int count, const int* dG, const int* dW, const float* const* G_inv,
    const float* const* A_inv, const float* const* grad_W,
    const float* const* grad_b, float* const* kf_W, float* const* kf_b,
    float* const* param_W, float* const* param_b, float* const* mom_W,
    float* const* mom_b, float lr, float momentum, void* workspace,
    size_t workspace_bytes, void* stream) {
  KFAC_REQUIRE(count > 0 && dG && dW && G_inv && A_inv && grad_W,
               "precondition: null argument or count=%d", count);
  std::vector<int> hb(count);
  for (int i = 0; i < count; ++i) {
    KFAC_REQUIRE(dG[i] > 0 && dW[i] > 0, "precondition: bad dims at %d", i);
    KFAC_REQUIRE(G_inv[i] && A_inv[i] && grad_W[i],
                 "precondition: null matrix pointer at %d", i);
    hb[i] = (grad_b && grad_b[i]) ? 1 : 0;
    bool fused = param_W && param_W[i];
    KFAC_REQUIRE(fused || (kf_W && kf_W[i]),
                 "precondition: layer %d has neither kf_W nor param_W", i);
    if (fused)
      KFAC_REQUIRE(mom_W && mom_W[i], "precondition: mom_W missing at %d", i);
    if (hb[i]) {
      KFAC_REQUIRE(fused || (kf_b && kf_b[i]),
                   "precondition: layer %d has a bias gradient but no kf_b", i);
      if (fused)
        KFAC_REQUIRE(param_b && param_b[i] && mom_b && mom_b[i],
                     "precondition: param_b/mom_b missing at %d", i);
    }
  }
  size_t need = kfac_precond_workspace_bytes(count, dG, dW, hb.data());
  if (workspace == nullptr || workspace_bytes < need)
    return fail(KFAC_ERR_WORKSPACE,
                "precondition: workspace of %zu bytes needed, %zu given", need,
                workspace_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = static_cast<char*>(workspace);
  GemmDesc* descs_dev = reinterpret_cast<GemmDesc*>(ws);
  ws += align256(2 * (size_t)count * sizeof(GemmDesc));

  std::vector<GemmDesc> descs(2 * count);
  int tiles1 = 0, tiles2 = 0;
  const bool use_tc = engine() == 1;
  for (int i = 0; i < count; ++i) {
    const int dg = dG[i], dw = dW[i], da = dw + hb[i];
    float* T = reinterpret_cast<float*>(ws);
    ws += align256((size_t)dg * da * sizeof(float));
    // T = G_inv * [grad_W, grad_b]
    GemmDesc& g = descs[i];
    g = GemmDesc();
    g.A = strided_operand(G_inv[i], 1, dg, dg);    // A(k, m) = G_inv[m][k]
    g.B = strided_operand(grad_W[i], dw, 1, dw);   // B(k, n) = grad[k][n]
    if (hb[i]) { g.B.extra_idx = dw; g.B.extra = grad_b[i]; }
    g.C = T; g.ldc = da; g.M = dg; g.N = da; g.K = dg;
    g.alpha = 1.f; g.beta = 0.f; g.flags = 0;
    g.tile_begin = tiles1;
    g.splits = 1;
    tiles1 += use_tc ? tc_tiles(g) : gemm_desc_tiles(g);
    // kf = T * A_inv, split and (optionally) applied
    GemmDesc& h = descs[count + i];
    h = GemmDesc();
    h.A = strided_operand(T, 1, da, dg);           // A(k, m) = T[m][k]
    h.B = strided_operand(A_inv[i], 1, da, da);    // B(k, n) = A_inv[n][k]
    h.C = nullptr; h.ldc = 0; h.M = dg; h.N = da; h.K = da;
    h.alpha = 1.f; h.beta = 0.f; h.flags = G_PRECOND;
    h.kfW = kf_W ? kf_W[i] : nullptr;
    h.kfb = (hb[i] && kf_b) ? kf_b[i] : nullptr;
    const bool fused = param_W && param_W[i];
    h.pW = fused ? param_W[i] : nullptr;
    h.vW = fused ? mom_W[i] : nullptr;
    h.pb = (fused && hb[i]) ? param_b[i] : nullptr;
    h.vb = (fused && hb[i]) ? mom_b[i] : nullptr;
    h.dW = dw;
    h.tile_begin = tiles2;
    h.splits = 1;
    tiles2 += use_tc ? tc_tiles(h) : gemm_desc_tiles(h);
  }
  KFAC_CUDA(cudaMemcpyAsync(descs_dev, descs.data(),
                            descs.size() * sizeof(GemmDesc),
                            cudaMemcpyHostToDevice, st));
  if (use_tc) {
    bool t1 = false, t2 = false;
    for (int i = 0; i < count; ++i) {
      t1 = t1 || tc_desc_has_tails(descs[i]);
      t2 = t2 || tc_desc_has_tails(descs[count + i]);
    }
    int rc = launch_tc_grouped(descs_dev, count, tiles1, 0.f, 0.f, t1, st);
    if (rc != KFAC_OK) return rc;
    return launch_tc_grouped(descs_dev + count, count, tiles2, lr, momentum,
                             t2, st);
  }
  int rc = launch_grouped_gemm(descs_dev, count, tiles1, 0.f, 0.f, st);
  if (rc != KFAC_OK) return rc;
  return launch_grouped_gemm(descs_dev + count, count, tiles2, lr, momentum, st);
}

// y = M x, one warp per row.
__global__ void symv_split_kernel(const float* __restrict__ m, int d, int d0,
                                  const float* __restrict__ x0,
                                  const float* __restrict__ x1, float* y0,
                                  float* y1, int* nan_flag) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= d) return;
  const float* mr = m + (long long)row * d;
  float s = 0.f;
  for (int c = lane; c < d; c += 32) {
    float xv = c < d0 ? x0[c] : x1[c - d0];
    s += mr[c] * xv;
  }
  for (int o = 16; o > 0; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
  if (lane == 0) {
    if (row < d0) y0[row] = s; else y1[row - d0] = s;
    if (nan_flag && isnan(s)) atomicExch(nan_flag, 1);
  }
}

// The reference's fallback for a block whose preconditioned gradient contains
// NaN (batch_normalization.py:159-173 with _check_nan): use the raw gradient.
// flag[0] is this call's NaN marker (cleared here), flag[1] counts fallbacks.
__global__ void __launch_bounds__(256)
symv_nan_fallback_kernel(int* __restrict__ flag, int d, int d0,
                         const float* __restrict__ x0,
                         const float* __restrict__ x1, float* y0, float* y1) {
  __shared__ int f;
  if (threadIdx.x == 0) f = flag[0];
  __syncthreads();
  if (f == 0) return;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    if (i < d0) y0[i] = x0[i]; else y1[i - d0] = x1[i - d0];
  }
  if (threadIdx.x == 0) {
    flag[0] = 0;
    flag[1] += 1;
  }
}

extern "C" int kfac_symv_split(const float* m, int d, int d0, const float* x0,
                               const float* x1, float* y0, float* y1,
                               int* nan_flag_dev, void* stream) {
  KFAC_REQUIRE(m && x0 && y0 && d > 0 && d0 > 0 && d0 <= d,
               "symv_split: bad argument");
  KFAC_REQUIRE(d0 == d || (x1 && y1), "symv_split: second piece missing");
  int blocks = ceil_div((long long)d * 32, 256);
  symv_split_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(
      m, d, d0, x0, x1, y0, y1, nan_flag_dev);
  KFAC_LAUNCH_CHECK("symv_split_kernel");
  if (nan_flag_dev != nullptr) {
    symv_nan_fallback_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(
        nan_flag_dev, d, d0, x0, x1, y0, y1);
    KFAC_LAUNCH_CHECK("symv_nan_fallback_kernel");
  }
  return KFAC_OK;
}
