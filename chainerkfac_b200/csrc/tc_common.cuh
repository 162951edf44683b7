// tcgen05 / mbarrier building blocks shared by the tile engine (tc_gemm.cu)
// and the diagonal kernel of the inverse (inverse.cu): shared-memory and
// instruction descriptors for K-major, 128-byte-swizzled fp32 (TF32) operand
// tiles, MMA issue / commit, accumulator loads from tensor memory, bounded
// barrier waits, and the split of fp32 values into two TF32 terms.
#pragma once

#include "common.cuh"

namespace kfac {

constexpr int TC_BM = 128;
constexpr unsigned TC_SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ unsigned smem_u32(const void* p) {
  return (unsigned)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(count));
}

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// Bounded wait on a phase parity; false if the limit ran out or the CTA is
// already aborting.
__device__ __forceinline__ bool mbar_wait_status(unsigned long long* bar,
                                                 unsigned parity,
                                                 volatile int* abort_flag,
                                                 int* status_word,
                                                 unsigned limit = TC_SPIN_LIMIT) {
  const unsigned addr = smem_u32(bar);
  {
    // fast path: the phase is usually complete already; test_wait answers
    // without the suspend machinery of try_wait
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  for (unsigned i = 0; i < limit; ++i) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  atomicExch(status_word, 1);
  return false;
}

__device__ __forceinline__ unsigned long long tc_smem_desc(unsigned addr) {
  // K-major, 128-byte swizzle: 8-row groups 1024 bytes apart.
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFF) >> 4);         // start address
  d |= (unsigned long long)1 << 16;                         // LBO (unused)
  d |= (unsigned long long)(1024 >> 4) << 32;               // SBO
  d |= (unsigned long long)1 << 46;                         // descriptor version
  d |= (unsigned long long)2 << 61;                         // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ unsigned tc_instr_desc(int n) {
  // D = f32, A = B = tf32, both K-major, M = 128, N = n
  return (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(n >> 3) << 17) |
         ((unsigned)(TC_BM >> 4) << 24);
}

__device__ __forceinline__ void tc_mma(unsigned tmem_d, unsigned long long da,
                                       unsigned long long db, unsigned idesc,
                                       unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tc_commit(unsigned long long* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
      ::"r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void tc_ld16(unsigned taddr, float v[16]) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
        "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Byte offset of element (row, k) inside a K-major SW128 tile (k < 32).
__device__ __forceinline__ int sw128_chunk_off(int row, int chunk) {
  return row * 128 + ((chunk ^ (row & 7)) << 4);
}

__device__ __forceinline__ void sts128(unsigned addr, float4 v) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
               "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

// hi = x rounded to TF32 (nearest, ties away from zero), lo = x - hi (exact in
// fp32; the tensor core reads its top 11 bits).  The rounding is two integer
// instructions (add half an ulp of TF32, clear the low 13 bits): cvt.rna
// would be one, but conversions issue on the quarter-rate XU pipe, which the
// producers saturate.
__device__ __forceinline__ float tf32_round(float x) {
  return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
}

__device__ __forceinline__ void store_split(unsigned hi_addr, unsigned lo_addr,
                                            float4 x) {
  float4 h, l;
  h.x = tf32_round(x.x); h.y = tf32_round(x.y);
  h.z = tf32_round(x.z); h.w = tf32_round(x.w);
  l.x = x.x - h.x; l.y = x.y - h.y; l.z = x.z - h.z; l.w = x.w - h.w;
  sts128(hi_addr, h);
  sts128(lo_addr, l);
}

}  // namespace kfac
