// Wire format of the factor / gradient collectives: many arrays concatenated
// into one flat fp32 buffer, symmetric factors as packed row-major lower
// triangles.  Pack visits only the d(d+1)/2 stored elements; unpack mirrors
// the triangle, scales (mean over ranks) and can blend into a running average.
#include <algorithm>
#include <mutex>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace kfac {

// Element types of the wire buffer (KFAC_WIRE_*): values are rounded to the
// wire type when packed and widened to fp32 when unpacked; sums over wire
// buffers are formed in fp32.
template <typename W> __device__ __forceinline__ W to_wire(float v);
template <> __device__ __forceinline__ float to_wire<float>(float v) { return v; }
template <> __device__ __forceinline__ __half to_wire<__half>(float v) {
  return __float2half_rn(v);
}
template <> __device__ __forceinline__ __nv_bfloat16 to_wire<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
__device__ __forceinline__ float from_wire(float v) { return v; }
__device__ __forceinline__ float from_wire(__half v) { return __half2float(v); }
__device__ __forceinline__ float from_wire(__nv_bfloat16 v) {
  return __bfloat162float(v);
}


struct WireArray {
  float* ptr;
  long long nelems;    // elements of the array in memory
  long long wire_off;  // offset of its slot in the wire buffer
  long long wire_n;    // elements of its slot
  long long item_begin;  // first work item of this array in the launch
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

// Work is cut into items that one 256-thread block handles: a 64x64 tile of a
// packed triangle (tile column <= tile row), or a run of kChunk elements of a
// plain array.  item_begin is the running count of items over the arrays of
// the call, so a block finds its array by bisection and its tile by inverting
// t = tr(tr+1)/2 + tc.
static const int kTile = 64;
static const int kChunk = 8192;
static const int kMaxWires = 16;

struct WireSources {
  const void* p[kMaxWires];
  int n;
};

__device__ __forceinline__ void tri_index(long long w, int& r, int& c) {
  long long i = (long long)((sqrt(8.0 * (double)w + 1.0) - 1.0) * 0.5);
  while ((i + 1) * (i + 2) / 2 <= w) ++i;
  while (i * (i + 1) / 2 > w) --i;
  r = (int)i;
  c = (int)(w - i * (i + 1) / 2);
}

// Both kernels are persistent: a block walks work items blockIdx.x,
// blockIdx.x + gridDim.x, ... so that the start-up of a block (table load) is
// paid once and the memory pipeline stays full across items.  The first work
// item of every array is cached in shared memory; an item's array is found by
// bisection there (arrays without items share their successor's first item
// and are skipped by taking the last array whose first item is <= item).
static const int kTabCap = 1024;
static const int kBlocksPerSm = 8;

__device__ __forceinline__ void load_item_table(
    const WireArray* __restrict__ arrs, int n_arrays, int* s_begin) {
  for (int i = threadIdx.x; i < n_arrays; i += blockDim.x)
    s_begin[i] = (int)arrs[i].item_begin;
  __syncthreads();
}

__device__ __forceinline__ int find_array(const int* s_begin, int n_arrays,
                                          int item) {
  int lo = 0, hi = n_arrays - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (s_begin[mid] <= item) lo = mid; else hi = mid - 1;
  }
  return lo;
}

template <typename W>
__global__ void __launch_bounds__(256, kBlocksPerSm)
wire_pack_kernel(const WireArray* __restrict__ arrs, int n_arrays,
                 int total_items, W* __restrict__ wire) {
  __shared__ int s_begin[kTabCap];
  load_item_table(arrs, n_arrays, s_begin);
  const int tx = threadIdx.x & (kTile - 1), ty = threadIdx.x >> 6;
  for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
    const WireArray a = arrs[find_array(s_begin, n_arrays, item)];
    const int t = item - (int)a.item_begin;
    W* __restrict__ dst = wire + a.wire_off;
    if (a.tri > 0 && a.select) {
      int tr, tc;
      tri_index(t, tr, tc);
      const int d = a.tri;
      const int c = tc * kTile + tx;
      const float* __restrict__ src = a.ptr;
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        const int rb = tr * kTile + half * 32 + ty;
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = rb + 4 * i;
          if (r < d && c <= r) v[i] = src[(long long)r * d + c];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = rb + 4 * i;
          if (r < d && c <= r)
            dst[(long long)r * (r + 1) / 2 + c] = to_wire<W>(v[i]);
        }
      }
    } else {
      // plain array, or the slot of a skipped array that is to be cleared
      const long long base = (long long)t * kChunk;
      const float* __restrict__ src = a.ptr;
#pragma unroll 8
      for (int k = threadIdx.x; k < kChunk; k += 256) {
        const long long w = base + k;
        if (w < a.wire_n) dst[w] = to_wire<W>(a.select ? src[w] : 0.f);
      }
    }
  }
}

// Unpack sums the same slot of `srcs.n` wire buffers in the order given (this
// GPU's own buffer and its peers' over NVLink when the pointers are peer
// mappings), scales, optionally blends into the destination, and writes the
// tile and its mirror image, both as coalesced rows.  A tile is handled in
// four passes of 16 rows (4 elements per thread and source in flight, few
// registers, 8 blocks per SM).
template <typename W>
__global__ void __launch_bounds__(256, kBlocksPerSm)
wire_unpack_kernel(const WireArray* __restrict__ arrs, int n_arrays,
                   int total_items, float scale, float ema_r,
                   WireSources srcs) {
  __shared__ float tile[kTile][kTile + 1];
  __shared__ int s_begin[kTabCap];
  load_item_table(arrs, n_arrays, s_begin);
  const int tx = threadIdx.x & (kTile - 1), ty = threadIdx.x >> 6;
  for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
    const WireArray a = arrs[find_array(s_begin, n_arrays, item)];
    const int t = item - (int)a.item_begin;
    float* __restrict__ dst = a.ptr;
    if (a.tri > 0) {
      int tr, tc;
      tri_index(t, tr, tc);
      const int d = a.tri;
      const int c = tc * kTile + tx;
      const long long off = a.wire_off + c;
#pragma unroll 1
      for (int pass = 0; pass < 4; ++pass) {
        const int rb = tr * kTile + pass * 16 + ty;   // rows rb, rb+4, ...
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < srcs.n; ++s) {
          const W* __restrict__ src = static_cast<const W*>(srcs.p[s]) + off;
          float x[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int r = rb + 4 * i;
            x[i] = (r < d && c <= r)
                       ? from_wire(src[(long long)r * (r + 1) / 2]) : 0.f;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[i] += x[i];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = rb + 4 * i;
          float v = acc[i] * scale;
          if (r < d && c <= r) {
            float* q = dst + (long long)r * d + c;
            if (ema_r >= 0.f) v = ema_r * v + (1.f - ema_r) * *q;
            *q = v;
          }
          tile[pass * 16 + ty + 4 * i][tx] = v;
        }
      }
      __syncthreads();
      // mirror: element (row cc, column rw) takes the value of (rw, cc), cc < rw
      const int rw = tr * kTile + tx;
#pragma unroll
      for (int i = 0; i < kTile / 4; ++i) {
        const int cc = tc * kTile + ty + 4 * i;
        if (rw < d && cc < rw)
          dst[(long long)cc * d + rw] = tile[tx][ty + 4 * i];
      }
      __syncthreads();
    } else {
      const long long base = (long long)t * kChunk;
      for (int k0 = 0; k0 < kChunk; k0 += 256 * 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < srcs.n; ++s) {
          const W* __restrict__ src =
              static_cast<const W*>(srcs.p[s]) + a.wire_off;
          float x[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const long long w = base + k0 + i * 256 + threadIdx.x;
            x[i] = w < a.wire_n ? from_wire(src[w]) : 0.f;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[i] += x[i];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const long long w = base + k0 + i * 256 + threadIdx.x;
          if (w < a.wire_n) {
            float v = acc[i] * scale;
            if (ema_r >= 0.f) v = ema_r * v + (1.f - ema_r) * dst[w];
            dst[w] = v;
          }
        }
      }
    }
  }
}

static int build_table(int n_arrays, float* const* arrays,
                       const int64_t* nelems, const int* tri_dim,
                       const int* select, bool skipped_get_items,
                       std::vector<WireArray>& tab, long long& total,
                       long long& items) {
  KFAC_REQUIRE(n_arrays > 0 && arrays && nelems && tri_dim,
               "wire: null argument or n_arrays=%d", n_arrays);
  tab.resize(n_arrays);
  total = 0;
  items = 0;
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
    a.item_begin = items;
    if (a.select && a.tri > 0) {
      long long t = (a.tri + kTile - 1) / kTile;
      items += t * (t + 1) / 2;
    } else if (a.select || skipped_get_items) {
      items += (a.wire_n + kChunk - 1) / kChunk;
    }
  }
  KFAC_REQUIRE(items < (1ll << 31), "wire: too many work items (%lld)", items);
  KFAC_REQUIRE(n_arrays <= kTabCap, "wire: %d arrays in one call, at most %d",
               n_arrays, kTabCap);
  return KFAC_OK;
}

static int upload_table(const std::vector<WireArray>& tab, cudaStream_t st,
                        const WireArray** out) {
  void* tab_dev = nullptr;
  int rc = ring_alloc(tab.size() * sizeof(WireArray), &tab_dev);
  if (rc != KFAC_OK) return rc;
  KFAC_CUDA(cudaMemcpyAsync(tab_dev, tab.data(), tab.size() * sizeof(WireArray),
                            cudaMemcpyHostToDevice, st));
  *out = static_cast<const WireArray*>(tab_dev);
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

extern "C" int kfac_wire_pack_as(int wire_dtype, int n_arrays,
                                 const float* const* arrays,
                                 const int64_t* nelems, const int* tri_dim,
                                 const int* select, int zero_skipped,
                                 void* wire, void* stream) {
  KFAC_REQUIRE(wire_dtype >= 0 && wire_dtype <= 2,
               "wire_pack: unknown wire dtype %d", wire_dtype);
  std::vector<WireArray> tab;
  long long total = 0, items = 0;
  int rc = build_table(n_arrays, const_cast<float* const*>(arrays), nelems,
                       tri_dim, select, zero_skipped != 0, tab, total, items);
  if (rc != KFAC_OK) return rc;
  KFAC_REQUIRE(wire != nullptr || total == 0, "wire_pack: null wire buffer");
  if (items == 0) return KFAC_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const WireArray* tab_dev = nullptr;
  rc = upload_table(tab, st, &tab_dev);
  if (rc != KFAC_OK) return rc;
  const unsigned grid = (unsigned)std::min<long long>(
      items, (long long)sm_count() * kBlocksPerSm);
  if (wire_dtype == KFAC_WIRE_F16)
    wire_pack_kernel<__half><<<grid, 256, 0, st>>>(
        tab_dev, n_arrays, (int)items, static_cast<__half*>(wire));
  else if (wire_dtype == KFAC_WIRE_BF16)
    wire_pack_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        tab_dev, n_arrays, (int)items, static_cast<__nv_bfloat16*>(wire));
  else
    wire_pack_kernel<float><<<grid, 256, 0, st>>>(
        tab_dev, n_arrays, (int)items, static_cast<float*>(wire));
  KFAC_LAUNCH_CHECK("wire_pack_kernel");
  return KFAC_OK;
}

extern "C" int kfac_wire_pack(int n_arrays, const float* const* arrays,
                              const int64_t* nelems, const int* tri_dim,
                              const int* select, int zero_skipped, float* wire,
                              void* stream) {
  return kfac_wire_pack_as(KFAC_WIRE_F32, n_arrays, arrays, nelems, tri_dim,
                           select, zero_skipped, wire, stream);
}

extern "C" int kfac_wire_unpack_sum_as(int wire_dtype, int n_arrays,
                                       float* const* arrays,
                                       const int64_t* nelems,
                                       const int* tri_dim, const int* select,
                                       float scale, float ema_r,
                                       const void* const* wires, int n_wires,
                                       void* stream) {
  KFAC_REQUIRE(wire_dtype >= 0 && wire_dtype <= 2,
               "wire_unpack: unknown wire dtype %d", wire_dtype);
  KFAC_REQUIRE(wires != nullptr && n_wires >= 1 && n_wires <= kMaxWires,
               "wire_unpack: %d wire buffers given, 1..%d supported", n_wires,
               kMaxWires);
  std::vector<WireArray> tab;
  long long total = 0, items = 0;
  int rc = build_table(n_arrays, arrays, nelems, tri_dim, select, false, tab,
                       total, items);
  if (rc != KFAC_OK) return rc;
  WireSources srcs;
  srcs.n = n_wires;
  for (int s = 0; s < kMaxWires; ++s) srcs.p[s] = s < n_wires ? wires[s] : nullptr;
  for (int s = 0; s < n_wires; ++s)
    KFAC_REQUIRE(wires[s] != nullptr || total == 0,
                 "wire_unpack: null wire buffer %d", s);
  if (items == 0) return KFAC_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const WireArray* tab_dev = nullptr;
  rc = upload_table(tab, st, &tab_dev);
  if (rc != KFAC_OK) return rc;
  const unsigned grid = (unsigned)std::min<long long>(
      items, (long long)sm_count() * kBlocksPerSm);
  if (wire_dtype == KFAC_WIRE_F16)
    wire_unpack_kernel<__half><<<grid, 256, 0, st>>>(
        tab_dev, n_arrays, (int)items, scale, ema_r, srcs);
  else if (wire_dtype == KFAC_WIRE_BF16)
    wire_unpack_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        tab_dev, n_arrays, (int)items, scale, ema_r, srcs);
  else
    wire_unpack_kernel<float><<<grid, 256, 0, st>>>(
        tab_dev, n_arrays, (int)items, scale, ema_r, srcs);
  KFAC_LAUNCH_CHECK("wire_unpack_kernel");
  return KFAC_OK;
}

extern "C" int kfac_wire_unpack_sum(int n_arrays, float* const* arrays,
                                    const int64_t* nelems, const int* tri_dim,
                                    const int* select, float scale,
                                    float ema_r, const float* const* wires,
                                    int n_wires, void* stream) {
  return kfac_wire_unpack_sum_as(
      KFAC_WIRE_F32, n_arrays, arrays, nelems, tri_dim, select, scale, ema_r,
      reinterpret_cast<const void* const*>(wires), n_wires, stream);
}

extern "C" int kfac_wire_unpack(int n_arrays, float* const* arrays,
                                const int64_t* nelems, const int* tri_dim,
                                const int* select, float scale, float ema_r,
                                const float* wire, void* stream) {
  return kfac_wire_unpack_sum(n_arrays, arrays, nelems, tri_dim, select, scale,
                              ema_r, &wire, 1, stream);
}
