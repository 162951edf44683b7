// Wire format of the factor / gradient collectives: many arrays concatenated
// into one flat fp32 buffer, symmetric factors as packed row-major lower
// triangles.  Pack visits only the d(d+1)/2 stored elements; unpack mirrors
// the triangle, scales (mean over ranks) and can blend into a running average.
#include <mutex>
#include <vector>

#include "common.cuh"

namespace kfac {

struct WireArray {
  float* ptr;
  long long nelems;    // elements of the array in memory
  long long wire_off;  // offset of its slot in the wire buffer
  long long wire_n;    // elements of its slot
  int tri;             // matrix side if packed as a triangle, else 0
  int select;
};

// Small per-device ring of device memory for descriptor tables that are built
// per call.  Successive calls use successive slices, so a table is not
// overwritten while the kernel that reads it may still be queued, as long as
// fewer than a ring's worth of calls are in flight.
static const size_t kRingBytes = 8u << 20;
static std::mutex g_ring_mu;
static char* g_ring[64] = {nullptr};
static size_t g_ring_pos[64] = {0};

int ring_alloc(size_t bytes, void** out) {
  int dev = 0;
  KFAC_CUDA(cudaGetDevice(&dev));
  KFAC_REQUIRE(dev >= 0 && dev < 64, "device index %d unsupported", dev);
  bytes = (bytes + 255) & ~(size_t)255;
  KFAC_REQUIRE(bytes <= kRingBytes / 4,
               "descriptor table of %zu bytes is too large", bytes);
  std::lock_guard<std::mutex> lock(g_ring_mu);
  if (g_ring[dev] == nullptr) {
    void* p = nullptr;
    KFAC_CUDA(cudaMalloc(&p, kRingBytes));
    g_ring[dev] = static_cast<char*>(p);
    g_ring_pos[dev] = 0;
  }
  if (g_ring_pos[dev] + bytes > kRingBytes) g_ring_pos[dev] = 0;
  *out = g_ring[dev] + g_ring_pos[dev];
  g_ring_pos[dev] += bytes;
  return KFAC_OK;
}

__device__ __forceinline__ void tri_index(long long w, int& r, int& c) {
  long long i = (long long)((sqrt(8.0 * (double)w + 1.0) - 1.0) * 0.5);
  while ((i + 1) * (i + 2) / 2 <= w) ++i;
  while (i * (i + 1) / 2 > w) --i;
  r = (int)i;
  c = (int)(w - i * (i + 1) / 2);
}

__global__ void wire_pack_kernel(const WireArray* __restrict__ arrs,
                                 int zero_skipped, float* __restrict__ wire) {
  const WireArray a = arrs[blockIdx.y];
  float* dst = wire + a.wire_off;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (!a.select) {
    if (zero_skipped)
      for (; w < a.wire_n; w += stride) dst[w] = 0.f;
    return;
  }
  if (a.tri > 0) {
    for (; w < a.wire_n; w += stride) {
      int r, c;
      tri_index(w, r, c);
      dst[w] = a.ptr[(long long)r * a.tri + c];
    }
  } else {
    for (; w < a.wire_n; w += stride) dst[w] = a.ptr[w];
  }
}

__global__ void wire_unpack_kernel(const WireArray* __restrict__ arrs,
                                   float scale, float ema_r,
                                   const float* __restrict__ wire) {
  const WireArray a = arrs[blockIdx.y];
  if (!a.select) return;
  const float* src = wire + a.wire_off;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
       i < a.nelems; i += stride) {
    long long w = i;
    if (a.tri > 0) {
      int r = (int)(i / a.tri);
      int c = (int)(i - (long long)r * a.tri);
      int hi = r > c ? r : c, lo = r > c ? c : r;
      w = (long long)hi * (hi + 1) / 2 + lo;
    }
    float v = src[w] * scale;
    if (ema_r >= 0.f) v = ema_r * v + (1.f - ema_r) * a.ptr[i];
    a.ptr[i] = v;
  }
}

static int build_table(int n_arrays, float* const* arrays,
                       const int64_t* nelems, const int* tri_dim,
                       const int* select, std::vector<WireArray>& tab,
                       long long& total) {
  KFAC_REQUIRE(n_arrays > 0 && arrays && nelems && tri_dim,
               "wire: null argument or n_arrays=%d", n_arrays);
  tab.resize(n_arrays);
  total = 0;
  for (int i = 0; i < n_arrays; ++i) {
    WireArray& a = tab[i];
    a.ptr = arrays[i];
    a.nelems = nelems[i];
    a.tri = tri_dim[i];
    a.select = select ? (select[i] != 0) : 1;
    KFAC_REQUIRE(a.nelems >= 0 && a.tri >= 0, "wire: bad size at %d", i);
    if (a.tri > 0) {
      KFAC_REQUIRE(a.nelems == (long long)a.tri * a.tri,
                   "wire: array %d is not a square matrix of side %d", i,
                   a.tri);
      a.wire_n = (long long)a.tri * (a.tri + 1) / 2;
    } else {
      a.wire_n = a.nelems;
    }
    KFAC_REQUIRE(!a.select || a.ptr || a.nelems == 0,
                 "wire: null array pointer at %d", i);
    a.wire_off = total;
    total += a.wire_n;
  }
  return KFAC_OK;
}

}  // namespace kfac

using namespace kfac;

extern "C" int64_t kfac_wire_nelems(int n_arrays, const int64_t* nelems,
                                    const int* tri_dim) {
  int64_t total = 0;
  for (int i = 0; i < n_arrays; ++i)
    total += tri_dim[i] > 0 ? (int64_t)tri_dim[i] * (tri_dim[i] + 1) / 2
                            : nelems[i];
  return total;
}

extern "C" int kfac_wire_pack(int n_arrays, const float* const* arrays,
                              const int64_t* nelems, const int* tri_dim,
                              const int* select, int zero_skipped, float* wire,
                              void* stream) {
  std::vector<WireArray> tab;
  long long total = 0;
  int rc = build_table(n_arrays, const_cast<float* const*>(arrays), nelems,
                       tri_dim, select, tab, total);
  if (rc != KFAC_OK) return rc;
  KFAC_REQUIRE(wire != nullptr || total == 0, "wire_pack: null wire buffer");
  void* tab_dev = nullptr;
  rc = ring_alloc(tab.size() * sizeof(WireArray), &tab_dev);
  if (rc != KFAC_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  KFAC_CUDA(cudaMemcpyAsync(tab_dev, tab.data(), tab.size() * sizeof(WireArray),
                            cudaMemcpyHostToDevice, st));
  dim3 grid(32, n_arrays);
  wire_pack_kernel<<<grid, 256, 0, st>>>(
      static_cast<const WireArray*>(tab_dev), zero_skipped, wire);
  KFAC_LAUNCH_CHECK("wire_pack_kernel");
  return KFAC_OK;
}

extern "C" int kfac_wire_unpack(int n_arrays, float* const* arrays,
                                const int64_t* nelems, const int* tri_dim,
                                const int* select, float scale, float ema_r,
                                const float* wire, void* stream) {
  std::vector<WireArray> tab;
  long long total = 0;
  int rc = build_table(n_arrays, arrays, nelems, tri_dim, select, tab, total);
  if (rc != KFAC_OK) return rc;
  KFAC_REQUIRE(wire != nullptr || total == 0, "wire_unpack: null wire buffer");
  void* tab_dev = nullptr;
  rc = ring_alloc(tab.size() * sizeof(WireArray), &tab_dev);
  if (rc != KFAC_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  KFAC_CUDA(cudaMemcpyAsync(tab_dev, tab.data(), tab.size() * sizeof(WireArray),
                            cudaMemcpyHostToDevice, st));
  dim3 grid(32, n_arrays);
  wire_unpack_kernel<<<grid, 256, 0, st>>>(
      static_cast<const WireArray*>(tab_dev), scale, ema_r, wire);
  KFAC_LAUNCH_CHECK("wire_unpack_kernel");
  return KFAC_OK;
}
