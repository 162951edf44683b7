// Staging pass of the factor builds: every operand X (rows K x columns d, in
// whatever layout the caller holds it: strided rows, the implicit patch
// matrix of an NCHW or channels-last convolution input, a transposed view)
// is written once as X^T split into two bf16 planes, hi[d][kp] and lo[d][kp]
// with x = hi + lo (kp = K rounded up to 8: rows are 16-byte multiples).
// The planes are what the tensor-core kernel then reads with TMA
// (cp.async.bulk.tensor, 64-byte swizzle): 32 k of 256 columns per box land
// in shared memory in exactly the K-major layout the MMA descriptors expect,
// zero-filled past K and past d, so the X^T X kernel needs no producer warps,
// no address arithmetic, no bounds handling and no zero-bordered copy of
// padded inputs.  The pass reads each input element once per filter tap it
// feeds (from L1/L2 after the first) and writes 4 bytes per patch-matrix
// element; it is HBM-bound.
#include <cuda.h>

#include <algorithm>
#include <vector>

#include "gemm_simt.cuh"

namespace kfac {

namespace {

constexpr int kStageJobsMax = 512;
constexpr int kChunkK = 2048;     // k per work item of the k-fast kernel
constexpr int kTileK = 64;        // k per tile of the transposing kernel
constexpr int kTileC = 32;        // columns (channels) per tile

struct StageJob {
  Operand X;
  unsigned short* hi;   // bf16 bit patterns
  unsigned short* lo;
  long long K, kp;
  int nhwc;             // im2col operand stored channels-last
  int c_begin, c_count; // k-fast kernel: the columns this job stages
  int kparts;           // work items along k
  int cblocks, taps;    // transposing kernel: channel blocks, filter taps
  long long item_begin;
};

__device__ __forceinline__ void split2(float x0, float x1, unsigned& hi,
                                       unsigned& lo) {
  // same rounding as the in-kernel split of the gather path: bf16 by adding
  // half an ulp (ties away from zero), the remainder rounded the same way
  const unsigned r0 = __float_as_uint(x0) + 0x8000u;
  const unsigned r1 = __float_as_uint(x1) + 0x8000u;
  hi = __byte_perm(r0, r1, 0x7632);
  const float l0 = x0 - __uint_as_float(r0 & 0xffff0000u);
  const float l1 = x1 - __uint_as_float(r1 & 0xffff0000u);
  lo = __byte_perm(__float_as_uint(l0) + 0x8000u,
                   __float_as_uint(l1) + 0x8000u, 0x7632);
}

__device__ __forceinline__ void store8(const StageJob& j, long long row,
                                       long long k0, const float v[8]) {
  unsigned h[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) split2(v[2 * i], v[2 * i + 1], h[i], l[i]);
  const long long off = row * j.kp + k0;
  *reinterpret_cast<uint4*>(j.hi + off) = make_uint4(h[0], h[1], h[2], h[3]);
  *reinterpret_cast<uint4*>(j.lo + off) = make_uint4(l[0], l[1], l[2], l[3]);
}

// Job of a flat work-item index, by bisection over the first items.
__device__ __forceinline__ int find_job(const long long* begin, int njobs,
                                        long long item) {
  int lo = 0, hi = njobs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (begin[mid] <= item) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// ---- k-fast: a thread stages 8 consecutive k of one column.  Coalesced when
// the source is contiguous along k (NCHW patches, transposed views, NCHW
// gradients); also stages the appended ones column of every operand.
__global__ void __launch_bounds__(256)
stage_kfast_kernel(const StageJob* __restrict__ jobs, int njobs,
                   long long items) {
  __shared__ long long s_begin[kStageJobsMax];
  for (int i = threadIdx.x; i < njobs; i += 256) s_begin[i] = jobs[i].item_begin;
  __syncthreads();
  for (long long item = blockIdx.x; item < items; item += gridDim.x) {
    const int ji = find_job(s_begin, njobs, item);
    const StageJob& j = jobs[ji];
    const long long local = item - j.item_begin;
    const int c = j.c_begin + (int)(local / j.kparts);
    const long long k0 =
        (local % j.kparts) * kChunkK + (long long)threadIdx.x * 8;
    if (k0 >= j.kp) continue;
    const Operand& X = j.X;
    float v[8];
    if (c == X.extra_idx) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const long long k = k0 + i;
        v[i] = k < j.K ? (X.extra ? X.extra[k] : 1.f) : 0.f;
      }
    } else if (X.mode == 0) {
      const float* p = X.base + (long long)c * X.s_col;
      long long q = k0 / X.period;
      long long r = k0 - q * X.period;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[i] = (k0 + i < j.K) ? p[q * X.s_outer + r * X.s_inner] : 0.f;
        if (++r == X.period) { r = 0; ++q; }
      }
    } else {
      const int kk = X.ks * X.ks;
      const int ch = c / kk;
      const int tap = c - ch * kk;
      const int ky = tap / X.ks, kx = tap - ky * X.ks;
      const int hw = X.Ho * X.Wo;
      long long n = k0 / hw;
      int rem = (int)(k0 - n * hw);
      int oy = rem / X.Wo, ox = rem - oy * X.Wo;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int iy = oy * X.st + ky - X.pd, ix = ox * X.st + kx - X.pd;
        float x = 0.f;
        if (k0 + i < j.K && iy >= 0 && iy < X.H && ix >= 0 && ix < X.W) {
          const long long a =
              j.nhwc ? ((n * X.H + iy) * X.W + ix) * X.C + ch
                     : ((n * X.C + ch) * X.H + iy) * X.W + ix;
          x = X.base[a];
        }
        v[i] = x;
        if (++ox == X.Wo) {
          ox = 0;
          if (++oy == X.Ho) { oy = 0; ++n; }
        }
      }
    }
    store8(j, c, k0, v);
  }
}

// ---- transposing: sources that are contiguous along the columns (rows x d
// matrices, channels-last tensors).  A block reads 64 k of 32 consecutive
// channels of one filter tap with the channels along the lanes, turns the
// tile in shared memory and writes 8 k per thread.
__global__ void __launch_bounds__(256)
stage_cfast_kernel(const StageJob* __restrict__ jobs, int njobs,
                   long long items) {
  __shared__ long long s_begin[kStageJobsMax];
  __shared__ float tile[kTileK][kTileC + 1];
  for (int i = threadIdx.x; i < njobs; i += 256) s_begin[i] = jobs[i].item_begin;
  __syncthreads();
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  for (long long item = blockIdx.x; item < items; item += gridDim.x) {
    const int ji = find_job(s_begin, njobs, item);
    const StageJob& j = jobs[ji];
    const Operand& X = j.X;
    long long local = item - j.item_begin;
    const long long kt = local % j.kparts;
    local /= j.kparts;
    const int cb = (int)(local % j.cblocks);
    const int tap = (int)(local / j.cblocks);
    const long long k0 = kt * kTileK;
    const int ch0 = cb * kTileC;
    const int nch = X.mode == 0 ? X.ncols : X.C;
    const int ch = ch0 + lane;
    // load: warp w takes k0 + w + 8 r, lanes walk the channels
    if (X.mode == 0) {
#pragma unroll
      for (int r = 0; r < kTileK / 8; ++r) {
        const long long k = k0 + wrp + 8 * r;
        float x = 0.f;
        if (k < j.K && ch < nch) x = X.base[operand_rowoff(X, k) + ch];
        tile[wrp + 8 * r][lane] = x;
      }
    } else {
      const int ky = tap / X.ks, kx = tap - ky * X.ks;
      const int hw = X.Ho * X.Wo;
#pragma unroll
      for (int r = 0; r < kTileK / 8; ++r) {
        const long long k = k0 + wrp + 8 * r;
        float x = 0.f;
        if (k < j.K && ch < nch) {
          const long long n = k / hw;
          const int rem = (int)(k - n * hw);
          const int oy = rem / X.Wo, ox = rem - oy * X.Wo;
          const int iy = oy * X.st + ky - X.pd, ix = ox * X.st + kx - X.pd;
          if (iy >= 0 && iy < X.H && ix >= 0 && ix < X.W)
            x = X.base[((n * X.H + iy) * X.W + ix) * X.C + ch];
        }
        tile[wrp + 8 * r][lane] = x;
      }
    }
    __syncthreads();
    // store: thread t writes 8 k of column t / 8
    const int col = threadIdx.x >> 3, kg = threadIdx.x & 7;
    if (ch0 + col < nch && k0 + 8 * kg < j.kp) {
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = tile[8 * kg + i][col];
      const long long row =
          X.mode == 0 ? (long long)(ch0 + col)
                      : (long long)(ch0 + col) * (X.ks * X.ks) + tap;
      store8(j, row, k0 + 8 * kg, v);
    }
    __syncthreads();
  }
}

// cuTensorMapEncodeTiled through the runtime's driver entry point: the
// library must load on machines without a driver (build checks, CPU tests).
typedef CUresult (*EncodeTiledFn)(
    CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
    CUtensorMapFloatOOBfill);

int encode_tiled_fn(EncodeTiledFn* out) {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    KFAC_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p,
                                      cudaEnableDefault, &q));
    KFAC_REQUIRE(q == cudaDriverEntryPointSuccess && p != nullptr,
                 "factor: the driver has no cuTensorMapEncodeTiled");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  *out = fn;
  return KFAC_OK;
}

size_t plane_bytes(long long rows, int d) {
  const long long kp = (rows + 7) & ~7LL;
  return ((size_t)d * kp * 2 + 255) & ~(size_t)255;
}

}  // namespace

size_t tc_stage_bytes(long long rows, int d) { return 2 * plane_bytes(rows, d); }

// Stages the operands of `count` factor jobs into `ws` (tc_stage_bytes each,
// in job order) and encodes two tensor maps per job (hi plane, lo plane) into
// `tmaps` (host memory, 2 * count entries of 128 bytes, 64-byte aligned).
int tc_stage_group(int count, const FactorJob* jobs, char* ws, void* tmaps,
                   cudaStream_t stream) {
  std::vector<StageJob> kfast, cfast;
  long long kitems = 0, citems = 0;
  EncodeTiledFn encode = nullptr;
  {
    const int rc = encode_tiled_fn(&encode);
    if (rc != KFAC_OK) return rc;
  }
  CUtensorMap* maps = static_cast<CUtensorMap*>(tmaps);
  for (int i = 0; i < count; ++i) {
    const FactorJob& job = jobs[i];
    StageJob s = {};
    s.X = job.X;
    s.nhwc = job.nhwc;
    s.K = job.rows;
    s.kp = (job.rows + 7) & ~7LL;
    s.hi = reinterpret_cast<unsigned short*>(ws);
    s.lo = reinterpret_cast<unsigned short*>(ws + plane_bytes(job.rows, job.d));
    ws += tc_stage_bytes(job.rows, job.d);
    const Operand& X = job.X;
    const bool columns_contiguous =
        (X.mode == 0 && X.s_col == 1 && X.ncols >= 8) ||
        (X.mode == 1 && job.nhwc && X.C >= 8);
    if (columns_contiguous) {
      StageJob t = s;
      const int nch = X.mode == 0 ? X.ncols : X.C;
      t.cblocks = (nch + kTileC - 1) / kTileC;
      t.taps = X.mode == 0 ? 1 : X.ks * X.ks;
      t.kparts = (int)((s.kp + kTileK - 1) / kTileK);
      t.item_begin = citems;
      citems += (long long)t.taps * t.cblocks * t.kparts;
      cfast.push_back(t);
      if (X.extra_idx >= 0) {
        s.c_begin = X.extra_idx;
        s.c_count = 1;
      }
    } else {
      s.c_begin = 0;
      s.c_count = job.d;
    }
    if (s.c_count > 0) {
      s.kparts = (int)((s.kp + kChunkK - 1) / kChunkK);
      s.item_begin = kitems;
      kitems += (long long)s.c_count * s.kparts;
      kfast.push_back(s);
    }
    for (int h = 0; h < 2; ++h) {
      const cuuint64_t dims[2] = {(cuuint64_t)job.rows, (cuuint64_t)job.d};
      const cuuint64_t strides[1] = {(cuuint64_t)s.kp * 2};
      const cuuint32_t box[2] = {32, 256};
      const cuuint32_t es[2] = {1, 1};
      const CUresult r = encode(
          &maps[2 * i + h], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
          h == 0 ? (void*)s.hi : (void*)s.lo, dims, strides, box, es,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
          CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS)
        return fail(KFAC_ERR_CUDA,
                    "factor: cuTensorMapEncodeTiled failed (%d) for a %lld x "
                    "%d operand", (int)r, job.rows, job.d);
    }
  }
  for (int pass = 0; pass < 2; ++pass) {
    std::vector<StageJob>& v = pass == 0 ? kfast : cfast;
    const long long items_all = pass == 0 ? kitems : citems;
    for (size_t b = 0; b < v.size(); b += kStageJobsMax) {
      const size_t nj = std::min<size_t>(kStageJobsMax, v.size() - b);
      std::vector<StageJob> part(v.begin() + b, v.begin() + b + nj);
      const long long first = part[0].item_begin;
      for (StageJob& s : part) s.item_begin -= first;
      const long long items =
          (b + nj < v.size() ? v[b + nj].item_begin : items_all) - first;
      void* dev = nullptr;
      int rc = ring_alloc(part.size() * sizeof(StageJob), &dev);
      if (rc != KFAC_OK) return rc;
      KFAC_CUDA(cudaMemcpyAsync(dev, part.data(),
                                part.size() * sizeof(StageJob),
                                cudaMemcpyHostToDevice, stream));
      const int grid = (int)std::min<long long>(items, (long long)sm_count() * 16);
      if (pass == 0)
        stage_kfast_kernel<<<grid, 256, 0, stream>>>(
            static_cast<const StageJob*>(dev), (int)nj, items);
      else
        stage_cfast_kernel<<<grid, 256, 0, stream>>>(
            static_cast<const StageJob*>(dev), (int)nj, items);
      KFAC_LAUNCH_CHECK(pass == 0 ? "stage_kfast_kernel" : "stage_cfast_kernel");
    }
  }
  return KFAC_OK;
}

}  // namespace kfac
