// Tensor-core tile engine for sm_100a: tcgen05.mma (kind::tf32) with fp32
// accumulators in tensor memory, fp32 operands split into two TF32 terms
// (x = hi + lo with hi rounded to nearest, C += hi*hi + hi*lo + lo*hi) so that
// results keep near-fp32 accuracy (a single TF32 pass misses the 1e-4 bound on
// large factors).
//
// One CTA (16 producer/epilogue warps + 1 MMA warp) owns a 128 x N tile,
// N <= 256.  Producer warps gather the operands from global memory (strided
// views, transposing views or im2col patches of an NCHW tensor), split them
// and write the K-major, 128-byte-swizzled shared-memory layout that the MMA
// descriptors expect; two stages of 32 k each are kept in flight through
// mbarriers.  The epilogue moves the accumulator tile TMEM -> registers ->
// shared memory and writes rows (and, for symmetric outputs, mirrored columns)
// with coalesced stores.  Every barrier wait is bounded; a wait that runs out
// raises a status word instead of hanging.
//
// Factor builds (X^T X) have their own kernel further down, tc_pair_kernel:
// 256 x 256 tiles, operands split into two bf16 terms (kind::f16 MMAs), the
// im2col gather laid out with lanes along k.
#include <algorithm>
#include <mutex>
#include <vector>

#include "gemm_simt.cuh"
#include "tc_common.cuh"

namespace kfac {

constexpr int TC_BN = 256;
constexpr int TC_BK = 32;
// Producer warps per CTA (template parameter PW of the kernel, a multiple of
// 8 that divides 96).  24 warps (72 registers per thread) gain 20 % on an
// im2col gather with long image rows (128 pixels) but nothing at the 7..56
// pixel rows of ResNet-50, where the per-thread offset bookkeeping that more
// threads replicate costs as much as the extra warps hide; strided operands
// need the 96 registers that only the 16-warp CTA leaves per thread.
constexpr int TC_PW_STRIDED = 16;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 4;   // 16 KB
constexpr int TC_B_BYTES = TC_BN * TC_BK * 4;   // 32 KB
// one stage: [A hi][B hi][A lo][B lo]; a lo tile lies TC_LO_OFF after its hi
constexpr int TC_LO_OFF = TC_A_BYTES + TC_B_BYTES;
constexpr int TC_STAGE_BYTES = 2 * TC_LO_OFF;   // 96 KB
// The A rows and then the B rows of a tile form one space of 384 rows; a
// task index covers a band of 4 * PW of them (each warp 4 rows, or one
// 16-byte column of 32 rows) and a thread has one task per band.
template <int PW>
struct TcMap {
  static constexpr int kProducers = PW * 32;
  static constexpr int kThreads = PW * 32 + 32;
  static constexpr int kBand = PW * 4;
  static constexpr int kTasks = (TC_BM + TC_BN) / kBand;
  static_assert((TC_BM + TC_BN) % kBand == 0 && PW % 8 == 0 && TC_BM % 32 == 0,
                "producer mapping");
};
constexpr int TC_STAGES = 2;
constexpr int TC_EPI_PITCH = TC_BN + 1;         // floats
constexpr int TC_SMEM_BYTES = TC_STAGES * TC_STAGE_BYTES + 8192 + 1024;
// Two accumulators per tile: columns [0, 256) collect hi*hi, columns
// [256, 512) the two cross terms, which are 2^-12 smaller; they are added in
// the epilogue.  Keeping them apart means only one MMA in three adds into the
// large sum.
constexpr int TC_TMEM_COLS = 2 * TC_BN;

static __device__ int g_tc_status = 0;

#ifdef KFAC_TC_TRACE
// Debug build only: CTA (0,0) records clock64() at fixed points of the
// producer / MMA loops, 8 slots per k-block.
__device__ long long* g_tc_trace = nullptr;
__device__ int g_tc_trace_cap = 0;
#define TC_TRACE(kb, slot)                                                   \
  do {                                                                       \
    if (g_tc_trace && blockIdx.x == 0 &&                  \
        ((kb) * 8 + (slot)) < g_tc_trace_cap)                                \
      g_tc_trace[(kb) * 8 + (slot)] = clock64();                             \
  } while (0)
#else
#define TC_TRACE(kb, slot) do {} while (0)
#endif

struct TcControl {
  unsigned long long full[TC_STAGES];
  unsigned long long empty[TC_STAGES];
  unsigned long long accum;
  unsigned tmem_base;
  volatile int abort_flag;
  int found;
  int coff_a[TC_BM];
  int kykx_a[TC_BM];
  int coff_b[TC_BN];
  int kykx_b[TC_BN];
  GemmDesc desc;
};

// Bounded wait on a phase parity; false if the limit ran out or the CTA is
// already aborting (the status word behind kfac_tc_status is then set).
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar,
                                          unsigned parity,
                                          volatile int* abort_flag) {
  return mbar_wait_status(bar, parity, abort_flag, &g_tc_status);
}

// im2col column tables for `rows` columns of a tile starting at column c0.
__device__ __forceinline__ void tc_im2col_tables(const Operand& op, int c0,
                                                 int rows, int* coff, int* kykx,
                                                 int tid, int nthreads) {
  for (int i = tid; i < rows; i += nthreads) {
    int c = c0 + i;
    int off = 0, info = -1;
    if (c < op.ncols) {
      int kk = op.ks * op.ks;
      int ch = c / kk;
      int r = c - ch * kk;
      int ky = r / op.ks;
      int kx = r - ky * op.ks;
      off = ch * op.H * op.W + ky * op.W + kx;
      info = (ky << 16) | kx;
    } else if (c == op.extra_idx) {
      info = -2;
    }
    coff[i] = off;
    kykx[i] = info;
  }
}

// Sources of constant columns: rows of the tile that lie beyond the operand
// read zeros, the appended bias column reads ones; both without branches in
// the hot loop (their address multiplier is 0).
static __device__ __align__(256) float g_zero_page[64];
static __device__ __align__(256) float g_ones_page[64] = {
    1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1,
    1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1,
    1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1};

// A producer thread moves TcMap<PW>::kTasks 16-byte chunks (4 consecutive k of one
// tile row) per k-block, task t in band t of the 384 tile rows.  Within a
// band the 8-warp group g = warp / 8 owns rows [32g, 32g + 32): operands
// contiguous along k (and im2col operands) give a warp 4 rows x 8 chunks
// (row = 4 * warp + lane / 8, chunk = lane % 8); operands contiguous along the
// column index give it one chunk of 32 rows (row = 32g + lane, chunk =
// warp % 8), so that a warp's loads of one k are 32 consecutive addresses.
// Whether a task is an A row or a B row depends only on (t, g): uniform per
// warp.  Per task everything that does not change with k is computed once:
// the element address is
//     p + (long long)o_j * m        (one multiply-add per element)
// where o_j is the k-dependent offset shared by all tasks of the thread that
// belong to the same operand.
struct PTask {
  const char* p;    // column base (or the zero / ones page), as bytes
  int m;            // byte multiplier of the k-dependent offset (0 for pages)
  unsigned soff;    // swizzled byte offset inside the stage, ~0u: idle task
};

// 1: band t holds only A rows, 0: only B rows, -1: depends on the warp group
template <int PW>
__host__ __device__ constexpr int tc_band_side(int t) {
  return 4 * PW * (t + 1) <= TC_BM ? 1 : (4 * PW * t >= TC_BM ? 0 : -1);
}

template <int PW>
__device__ __forceinline__ bool tc_task_is_a(int t, int warp) {
  return tc_band_side<PW>(t) >= 0 ? tc_band_side<PW>(t) == 1
                                  : 4 * PW * t + 32 * (warp >> 3) < TC_BM;
}

template <bool IM2COL, int PW>
__device__ __forceinline__ void tc_task_setup(const Operand& A,
                                              const Operand& B, int m0, int n0,
                                              int rows_b, bool skip_a,
                                              const TcControl* ctl,
                                              int warp, int lane,
                                              PTask task[TcMap<PW>::kTasks]) {
#pragma unroll
  for (int t = 0; t < TcMap<PW>::kTasks; ++t) {
    const bool is_a = tc_task_is_a<PW>(t, warp);
    const Operand& op = is_a ? A : B;
    const bool kf = IM2COL || op.kfast;
    const int band_row = kf ? warp * 4 + (lane >> 3) : 32 * (warp >> 3) + lane;
    const int row = TcMap<PW>::kBand * t + band_row - (is_a ? 0 : TC_BM);
    const int rows = is_a ? (skip_a ? 0 : TC_BM) : rows_b;
    const int chunk = kf ? (lane & 7) : (warp & 7);
    PTask v;
    v.soff = row < rows ? (unsigned)((is_a ? 0 : TC_A_BYTES) + row * 128 +
                                     ((chunk ^ (row & 7)) << 4))
                        : ~0u;
    const float* p = g_zero_page;
    int m = 0;
    if (row < rows) {
      const int c = (is_a ? m0 : n0) + row;
      if (IM2COL) {
        const int info = (is_a ? ctl->kykx_a : ctl->kykx_b)[row];
        if (info >= 0) {
          p = op.base + (is_a ? ctl->coff_a : ctl->coff_b)[row];
          m = 1;
        } else if (info == -2) {
          p = g_ones_page;
        }
      } else if (c < op.ncols) {
        p = op.base + (long long)c * op.s_col;
        m = op.period == 1 ? (int)op.s_outer : 1;
      } else if (c == op.extra_idx) {
        if (op.extra) { p = op.extra; m = 1; }
        else p = g_ones_page;
      }
    }
    v.p = reinterpret_cast<const char*>(p);
    v.m = m * 4;
    task[t] = v;
  }
}

// Position of a thread's chunk (4 consecutive k) in an operand's row space,
// kept incrementally from k-block to k-block so that the hot loop has no
// integer division.
struct KState {
  int k;           // first k of the chunk (contractions are < 2^31 long)
  int a, b, c;     // strided with a period: k = a * period + b
                   // im2col: k = (a * Ho + b) * Wo + c
};

template <bool IM2COL>
__device__ __forceinline__ void kstate_init(const Operand& op, long long k,
                                            KState& s) {
  s.k = (int)k;
  s.a = s.b = s.c = 0;
  if (IM2COL) {
    const int how = op.Ho * op.Wo;
    s.a = (int)(k / how);
    const int rem = (int)(k - (long long)s.a * how);
    s.b = rem / op.Wo;
    s.c = rem - s.b * op.Wo;
  } else if (op.period != 1) {
    s.a = (int)(k / op.period);
    s.b = (int)(k - (long long)s.a * op.period);
  }
}

template <bool IM2COL, int BK = TC_BK>
__device__ __forceinline__ void kstate_advance(const Operand& op, KState& s) {
  s.k += BK;
  if (IM2COL) {
    s.c += BK;
    while (s.c >= op.Wo) {
      s.c -= op.Wo;
      if (++s.b >= op.Ho) { s.b = 0; ++s.a; }
    }
  } else if (op.period != 1) {
    s.b += BK;
    while (s.b >= op.period) { s.b -= op.period; ++s.a; }
  }
}

// Element offsets of a chunk's 4 k (strided: row offsets; im2col: pixel
// offsets of an unpadded convolution -- a padded input is copied into a
// zero-bordered buffer first, so every tap of every pixel is in range).
// With TAILS, offsets of k at or beyond kend are 0 (a legal address; the
// value is zeroed after the load).
template <bool IM2COL, bool TAILS, int J = 4>
__device__ __forceinline__ void tc_koffsets(const Operand& op,
                                            const KState& ks, int kend,
                                            int o[J]) {
  const int k = ks.k;
  if (IM2COL) {
    int n = ks.a, oy = ks.b, ox = ks.c;
    const int chw = op.C * op.H * op.W;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      o[j] = n * chw + oy * op.st * op.W + ox * op.st;
      if (TAILS && k + j >= kend) o[j] = 0;
      if (++ox >= op.Wo) {
        ox = 0;
        if (++oy >= op.Ho) { oy = 0; ++n; }
      }
    }
    return;
  }
  if (op.period == 1) {
#pragma unroll
    for (int j = 0; j < J; ++j) o[j] = k + j;
  } else {
#pragma unroll
    for (int j = 0; j < J; ++j) {
      int q = ks.a, r = ks.b + j;
      while (r >= op.period) { r -= op.period; ++q; }
      o[j] = (int)((long long)q * op.s_outer + (long long)r * op.s_inner);
    }
  }
  if (TAILS) {
#pragma unroll
    for (int j = 0; j < J; ++j) if (k + j >= kend) o[j] = 0;
  }
}

// Gather the chunks of one operand (SIDE_A: the A rows, else the B rows) for
// one k-block into registers.  The loads are issued back to back, each from
// an address that is always legal; nothing between two loads depends on a
// loaded value.  `vec` (uniform per tile): every chunk of this operand is
// 16-byte aligned and contiguous.
template <bool TAILS, int PW, bool SIDE_A>
__device__ __forceinline__ void tc_load_side(
    const PTask task[TcMap<PW>::kTasks], const int o[4], int k, int kend,
    bool vec, int warp, float4 v[TcMap<PW>::kTasks]) {
  constexpr int NT = TcMap<PW>::kTasks;
  const bool tail = TAILS && (k + 3 >= kend);
  if (vec && !tail) {
#pragma unroll
    for (int t = 0; t < NT; ++t)
      if (tc_task_is_a<PW>(t, warp) == SIDE_A && task[t].soff != ~0u)
        v[t] = *reinterpret_cast<const float4*>(
            task[t].p + (long long)o[0] * task[t].m);
  } else {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      if (tc_task_is_a<PW>(t, warp) != SIDE_A || task[t].soff == ~0u) continue;
      v[t].x = *reinterpret_cast<const float*>(task[t].p + (long long)o[0] * task[t].m);
      v[t].y = *reinterpret_cast<const float*>(task[t].p + (long long)o[1] * task[t].m);
      v[t].z = *reinterpret_cast<const float*>(task[t].p + (long long)o[2] * task[t].m);
      v[t].w = *reinterpret_cast<const float*>(task[t].p + (long long)o[3] * task[t].m);
    }
  }
  if (tail) {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      if (tc_task_is_a<PW>(t, warp) != SIDE_A) continue;
      if (k + 0 >= kend) v[t].x = 0.f;
      if (k + 1 >= kend) v[t].y = 0.f;
      if (k + 2 >= kend) v[t].z = 0.f;
      if (k + 3 >= kend) v[t].w = 0.f;
    }
  }
}

// True when every 16-byte chunk of a k-contiguous strided operand is aligned
// and contiguous for k-blocks that start at kbeg (uniform for the tile).
__device__ __forceinline__ bool tc_operand_vec(const Operand& op,
                                               long long kbeg) {
  if (op.mode != 0 || !op.kfast) return false;
  if ((reinterpret_cast<uintptr_t>(op.base) & 15) != 0) return false;
  if ((op.s_col & 3) != 0 || (kbeg & 3) != 0) return false;
  if (op.extra_idx >= 0 && op.extra != nullptr) return false;
  if (op.period == 1) return op.s_outer == 1;
  return (op.period & 3) == 0 && (op.s_outer & 3) == 0 && op.s_inner == 1;
}

template <int NT>
__device__ __forceinline__ void tc_store_tile(const PTask task[NT],
                                              unsigned stage,
                                              const float4 v[NT]) {
#pragma unroll
  for (int t = 0; t < NT; ++t)
    if (task[t].soff != ~0u)
      store_split(stage + task[t].soff, stage + TC_LO_OFF + task[t].soff, v[t]);
}

// Lower-triangular enumeration with 128-row x 256-column tiles: tile (bi, bj)
// exists iff 2 * bj <= bi.  Tiles before row bi: a(a+1) for bi = 2a, (a+1)^2
// for bi = 2a + 1.
__device__ __forceinline__ void tc_tri_tile(int t, int& bi, int& bj) {
  int a = (int)sqrtf((float)t);
  while ((a + 1) * (a + 1) <= t) ++a;
  while (a * a > t) --a;
  if (t < a * (a + 1)) {
    bi = 2 * a - 1;
    bj = t - a * a;
  } else {
    bi = 2 * a;
    bj = t - a * (a + 1);
  }
}

template <bool IM2COL, bool TAILS, int PW>
__global__ void __launch_bounds__(TcMap<PW>::kThreads, 1)
tc_gemm_kernel(const GemmDesc* __restrict__ descs, int ndesc,
               const __grid_constant__ GemmDesc inline_desc, float lr,
               float momentum) {
  extern __shared__ unsigned char tc_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
  TcControl* ctl =
      reinterpret_cast<TcControl*>(smem + TC_STAGES * TC_STAGE_BYTES);
  constexpr int TC_PRODUCERS = TcMap<PW>::kProducers;
  constexpr int TC_PWARPS = PW;
  constexpr int TC_THREADS = TcMap<PW>::kThreads;
  constexpr int TC_NTASK = TcMap<PW>::kTasks;
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x;

  // ---- locate the problem and copy its descriptor to shared memory.  The
  // search is one parallel round: thread t tests descriptor t (tile_begin is
  // ascending), instead of a chain of dependent global loads.
  {
    const GemmDesc* src = &inline_desc;
    if (descs != nullptr) {
      for (int i = tid; i < ndesc; i += TC_THREADS) {
        const int lo = descs[i].tile_begin;
        const int hi = (i + 1 < ndesc) ? descs[i + 1].tile_begin : 0x7fffffff;
        if (lo <= tile && tile < hi) ctl->found = i;
      }
      __syncthreads();
      src = descs + ctl->found;
    }
    const int* s = reinterpret_cast<const int*>(src);
    int* d = reinterpret_cast<int*>(&ctl->desc);
    for (int i = tid; i < (int)(sizeof(GemmDesc) / sizeof(int)); i += TC_THREADS)
      d[i] = s[i];
  }
  if (tid == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(&ctl->full[s], TC_PRODUCERS / 32);
      mbar_init(&ctl->empty[s], 1);
    }
    mbar_init(&ctl->accum, 1);
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == TC_PRODUCERS / 32) {
    asm volatile(
        "tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
        ::"r"(smem_u32(&ctl->tmem_base)), "r"(TC_TMEM_COLS)
        : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;"
                 ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

  const GemmDesc& g = ctl->desc;
  const unsigned tmem = ctl->tmem_base;
  int lt = tile - g.tile_begin, split = 0;
  if (g.splits > 1) {
    split = lt / g.ntiles;
    lt -= split * g.ntiles;
  }
  int bi, bj;
  if (g.flags & G_LOWER) {
    tc_tri_tile(lt, bi, bj);
  } else {
    bi = lt / g.tiles_n;
    bj = lt - bi * g.tiles_n;
  }
  const int m0 = bi * TC_BM, n0 = bj * TC_BN;
  int n_valid = min(TC_BN, g.N - n0);
  if (g.flags & G_LOWER) n_valid = min(n_valid, m0 + TC_BM - n0);
  const int n_inst = (n_valid + 15) & ~15;
  const int m_valid = min(TC_BM, g.M - m0);

  long long kbeg = 0, kend = g.K;
  if (g.splits > 1) {
    kbeg = (long long)split * g.k_per_split;
    kend = min(g.K, kbeg + g.k_per_split);
  }
  if (g.flags & G_KBEG_N0) kbeg = max(kbeg, (long long)n0);
  if (g.flags & G_KBEG_M0) kbeg = max(kbeg, (long long)m0);
  if (g.flags & G_KEND_M0) kend = min(kend, (long long)(m0 + TC_BM));
  // a gated-off problem runs no k-blocks and stores nothing
  const bool gated_off = g.gate != nullptr && *g.gate == 0;
  const int nkb = (kend > kbeg && !gated_off)
                      ? (int)((kend - kbeg + TC_BK - 1) / TC_BK) : 0;
  // X^T X on a diagonal tile: the tile's A rows are rows [m0 - n0, m0 - n0 +
  // 128) of its B rows (m0 - n0 is 0 or 128), so only B is staged and the A
  // descriptors point into the B tiles.
  const bool share_ab = (g.flags & G_SAME_AB) && (g.flags & G_LOWER) &&
                        bj == (bi >> 1);

  if (warp < TC_PRODUCERS / 32) {
    // ===================== producers =====================
    if (IM2COL) {
      tc_im2col_tables(g.A, m0, TC_BM, ctl->coff_a, ctl->kykx_a, tid,
                       TC_PRODUCERS);
      tc_im2col_tables(g.B, n0, n_inst, ctl->coff_b, ctl->kykx_b, tid,
                       TC_PRODUCERS);
      asm volatile("bar.sync 1, %0;" ::"r"(TC_PRODUCERS) : "memory");
    }
    const Operand A = g.A, B = g.B;   // register copies: loop invariant
    float4 v[TC_NTASK];
    PTask task[TC_NTASK];
    tc_task_setup<IM2COL, PW>(A, B, m0, n0, n_inst, share_ab, ctl, warp, lane,
                              task);
    const int kend_i = (int)kend;
    KState ka, kb_state;
    {
      const bool a_kf = IM2COL || A.kfast;
      const bool b_kf = IM2COL || B.kfast;
      kstate_init<IM2COL>(A, kbeg + 4 * (a_kf ? (lane & 7) : (warp & 7)), ka);
      kstate_init<IM2COL>(B, kbeg + 4 * (b_kf ? (lane & 7) : (warp & 7)),
                          kb_state);
    }
    const unsigned smem_base = smem_u32(smem);
    const bool vec_a = !IM2COL && tc_operand_vec(A, kbeg);
    const bool vec_b = !IM2COL && tc_operand_vec(B, kbeg);
    // iteration kb stores k-block kb-1 (loaded one iteration earlier) and
    // issues the loads of k-block kb, which then fly while the tensor core
    // works and while this warp waits for the stage to drain
    for (int kb = 0; kb <= nkb; ++kb) {
      if (kb > 0) {
        const int pb = kb - 1;
        const int s = pb % TC_STAGES;
        if (tid == 0) TC_TRACE(pb, 0);
        if (pb >= TC_STAGES) {
          if (!mbar_wait(&ctl->empty[s], ((pb / TC_STAGES) - 1) & 1,
                         &ctl->abort_flag))
            break;
        }
        if (tid == 0) TC_TRACE(pb, 1);
        tc_store_tile<TC_NTASK>(task, smem_base + s * TC_STAGE_BYTES, v);
        if (tid == 0) TC_TRACE(pb, 2);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->full[s]);
        if (tid == 0) TC_TRACE(pb, 3);
      }
      if (kb < nkb) {
        int oa[4], ob[4];
        tc_koffsets<IM2COL, TAILS>(A, ka, kend_i, oa);
        if (IM2COL) {
          // both operands are the same patch matrix and use the same chunk
          // mapping: one set of pixel offsets serves both
#pragma unroll
          for (int j = 0; j < 4; ++j) ob[j] = oa[j];
        } else {
          tc_koffsets<IM2COL, TAILS>(B, kb_state, kend_i, ob);
        }
        tc_load_side<TAILS, PW, true>(task, oa, ka.k, kend_i, vec_a, warp, v);
        tc_load_side<TAILS, PW, false>(task, ob, IM2COL ? ka.k : kb_state.k,
                                       kend_i, vec_b, warp, v);
        kstate_advance<IM2COL>(A, ka);
        if (!IM2COL) kstate_advance<IM2COL>(B, kb_state);
        if (tid == 0) TC_TRACE(kb, 4);
      }
    }
  } else {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      const unsigned idesc = tc_instr_desc(n_inst);
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % TC_STAGES;
        TC_TRACE(kb, 5);
        if (!mbar_wait(&ctl->full[s], (kb / TC_STAGES) & 1, &ctl->abort_flag))
          break;
        TC_TRACE(kb, 6);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned sa = smem_u32(smem + s * TC_STAGE_BYTES);
        const unsigned a_off =
            share_ab ? (unsigned)(TC_A_BYTES + (m0 - n0) * 128) : 0u;
        const unsigned long long a_hi = tc_smem_desc(sa + a_off);
        const unsigned long long b_hi = tc_smem_desc(sa + TC_A_BYTES);
        const unsigned long long a_lo = tc_smem_desc(sa + TC_LO_OFF + a_off);
        const unsigned long long b_lo =
            tc_smem_desc(sa + TC_LO_OFF + TC_A_BYTES);
#pragma unroll
        for (int kk = 0; kk < TC_BK / 8; ++kk) {
          const unsigned long long adv = (unsigned long long)(kk * 32 >> 4);
          tc_mma(tmem + TC_BN, a_lo + adv, b_hi + adv, idesc, (kb | kk) != 0);
          tc_mma(tmem + TC_BN, a_hi + adv, b_lo + adv, idesc, 1);
          tc_mma(tmem, a_hi + adv, b_hi + adv, idesc, (kb | kk) != 0);
        }
        tc_commit(&ctl->empty[s]);
        TC_TRACE(kb, 7);
      }
      tc_commit(&ctl->accum);
    }
    __syncwarp();
  }

  // ===================== epilogue =====================
  float* stage = reinterpret_cast<float*>(smem);
  bool ok = true;
  if (warp < TC_PRODUCERS / 32) {
    if (nkb > 0) {
      ok = mbar_wait(&ctl->accum, 0, &ctl->abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    // warp w reads the 32 accumulator rows of its TMEM quarter q = w % 4;
    // the TC_PWARPS / 4 warps of a quarter take 16-column slices in turn
    const int q = warp & 3, h = warp >> 2;
    const int row = q * 32 + lane;
    for (int c0 = h * 16; c0 < n_inst; c0 += 16 * (TC_PWARPS / 4)) {
      float v[16];
      if (nkb > 0 && ok) {
        float w[16];
        tc_ld16(tmem + ((unsigned)(q * 32) << 16) + (unsigned)c0, v);
        tc_ld16(tmem + ((unsigned)(q * 32) << 16) + (unsigned)(TC_BN + c0), w);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] += w[i];
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) stage[row * TC_EPI_PITCH + c0 + i] = v[i];
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == TC_PRODUCERS / 32) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                 ::"r"(tmem), "r"(TC_TMEM_COLS)
                 : "memory");
  }
  if (warp >= TC_PRODUCERS / 32 || ctl->abort_flag || gated_off) return;

  if (g.splits > 1) {
    float* p = g.partial + ((long long)split * g.ntiles + lt) * (TC_BM * TC_BN);
    for (int r = warp; r < TC_BM; r += TC_PWARPS)
      for (int c = lane; c < n_inst; c += 32)
        p[r * TC_BN + c] = stage[r * TC_EPI_PITCH + c];
    return;
  }
  if (g.flags & G_PRECOND) {
    const int dW = g.dW;
    for (int r = warp; r < m_valid; r += TC_PWARPS) {
      const int gr = m0 + r;
      float ov[TC_BN / 32], op[TC_BN / 32];
      if (g.pW != nullptr) {
#pragma unroll
        for (int i = 0; i < TC_BN / 32; ++i) {
          const int c = lane + 32 * i, gc = n0 + c;
          ov[i] = op[i] = 0.f;
          if (c < n_valid) {
            if (gc < dW) {
              ov[i] = g.vW[(long long)gr * dW + gc];
              op[i] = g.pW[(long long)gr * dW + gc];
            } else if (g.pb != nullptr) {
              ov[i] = g.vb[gr];
              op[i] = g.pb[gr];
            }
          }
        }
      }
#pragma unroll
      for (int i = 0; i < TC_BN / 32; ++i) {
        const int c = lane + 32 * i, gc = n0 + c;
        if (c >= n_valid) continue;
        const float kf = stage[r * TC_EPI_PITCH + c];
        if (gc < dW) {
          const long long idx = (long long)gr * dW + gc;
          if (g.kfW) g.kfW[idx] = kf;
          if (g.pW) {
            const float nv = momentum * ov[i] - lr * kf;
            g.vW[idx] = nv;
            g.pW[idx] = op[i] + nv;
          }
        } else {
          if (g.kfb) g.kfb[gr] = kf;
          if (g.pb) {
            const float nv = momentum * ov[i] - lr * kf;
            g.vb[gr] = nv;
            g.pb[gr] = op[i] + nv;
          }
        }
      }
    }
    return;
  }
  const float alpha = g.alpha, beta = g.beta;
  const bool lower = (g.flags & G_LOWER) != 0;
  const bool mirror = (g.flags & G_MIRROR) != 0;
  // rows: C[gr][gc] = alpha * acc + beta * C[gr][gc]; the final value is kept
  // in the staging tile for the mirrored pass.  A lane owns columns lane,
  // lane + 32, ...; all of a row's reads of C are issued before any is used.
  for (int r = warp; r < m_valid; r += TC_PWARPS) {
    const int gr = m0 + r;
    float* crow = g.C + (long long)gr * g.ldc + n0;
    const int cend = lower ? min(n_valid, gr - n0 + 1) : n_valid;
    float old[TC_BN / 32];
    if (beta != 0.f) {
#pragma unroll
      for (int i = 0; i < TC_BN / 32; ++i) {
        const int c = lane + 32 * i;
        old[i] = c < cend ? crow[c] : 0.f;
      }
    }
#pragma unroll
    for (int i = 0; i < TC_BN / 32; ++i) {
      const int c = lane + 32 * i;
      if (c < cend) {
        float v = alpha * stage[r * TC_EPI_PITCH + c];
        if (beta != 0.f) v += beta * old[i];
        crow[c] = v;
        if (g.C2 != nullptr) g.C2[(long long)gr * g.ldc + n0 + c] = v;
        if (mirror) stage[r * TC_EPI_PITCH + c] = v;
      }
    }
  }
  if (mirror) {
    asm volatile("bar.sync 1, %0;" ::"r"(TC_PRODUCERS) : "memory");
    for (int c = warp; c < n_valid; c += TC_PWARPS) {
      const int gc = n0 + c;
      for (int r = lane; r < m_valid; r += 32) {
        const int gr = m0 + r;
        if (gc < gr) g.C[(long long)gc * g.ldc + gr] = stage[r * TC_EPI_PITCH + c];
      }
    }
  }
}

// ---- split-bf16 operands (factor builds) ----
// x = hi + lo with hi = bf16(x), lo = bf16(x - hi): 16 significant bits,
// products hi*hi + hi*lo + lo*hi are exact in the fp32 accumulator.  Halves
// the shared-memory bytes per k of the split-TF32 scheme (stores and tensor
// core operand reads), which is what bounds the tile kernels.
__device__ __forceinline__ unsigned tc_instr_desc_bf16(int n) {
  // D = f32, A = B = bf16, both K-major, M = 128, N = n
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) |
         ((unsigned)(TC_BM >> 4) << 24);
}

__device__ __forceinline__ void tc_mma_bf16(unsigned tmem_d,
                                            unsigned long long da,
                                            unsigned long long db,
                                            unsigned idesc,
                                            unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Two consecutive k -> one word of the hi tile and one of the lo tile (the
// first k in the low half).  Rounding to bf16 is an integer add of half an ulp
// (ties away from zero); the byte permute then takes the upper halves.  No
// cvt: conversions issue on the quarter-rate XU pipe (measured at 130 % of its
// sustained peak with cvt.rn.bf16x2 here).
__device__ __forceinline__ void split_bf16x2(float x0, float x1, unsigned& hi,
                                             unsigned& lo) {
  const unsigned r0 = __float_as_uint(x0) + 0x8000u;
  const unsigned r1 = __float_as_uint(x1) + 0x8000u;
  hi = __byte_perm(r0, r1, 0x7632);
  const float l0 = x0 - __uint_as_float(r0 & 0xffff0000u);
  const float l1 = x1 - __uint_as_float(r1 & 0xffff0000u);
  lo = __byte_perm(__float_as_uint(l0) + 0x8000u,
                   __float_as_uint(l1) + 0x8000u, 0x7632);
}

__device__ __forceinline__ void store_split_bf16(unsigned hi_addr,
                                                 unsigned lo_addr, float4 a,
                                                 float4 b) {
  unsigned h[4], l[4];
  split_bf16x2(a.x, a.y, h[0], l[0]);
  split_bf16x2(a.z, a.w, h[1], l[1]);
  split_bf16x2(b.x, b.y, h[2], l[2]);
  split_bf16x2(b.z, b.w, h[3], l[3]);
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(hi_addr),
               "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3])
               : "memory");
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(lo_addr),
               "r"(l[0]), "r"(l[1]), "r"(l[2]), "r"(l[3])
               : "memory");
}

// ============================================================ X^T X, 256 x 256
// Factor builds (C = alpha X^T X + beta C, lower tiles, mirrored) use a CTA
// tile of 256 x 256: two 128-row accumulators that share one staged set of
// 256 B rows, so a k-block needs 512 operand rows for 65536 outputs instead of
// 384 for 32768; on diagonal tiles the A rows are the B rows and only those
// are staged.  Operands are split into two bf16 terms (see above).  A stage
// holds 32 k as 64-byte rows under the 64-byte swizzle ([A hi][B hi][A lo]
// [B lo], 16 KB each), three stages are in flight, and each 128 x 256
// accumulator takes 256 of the 512 tensor-memory columns (cross terms and
// hi*hi go into the same accumulator, cross terms first).  Partial tiles of
// split contractions keep the 128 x 256 numbering of tc_tri_tile, so
// tc_reduce_kernel serves both kernels.
constexpr int PK_BK = 32;
constexpr int PK_ROWS = 256;                         // rows per operand tile
constexpr int PK_TILE_BYTES = PK_ROWS * PK_BK * 2;   // 16 KB of bf16
constexpr int PK_LO_OFF = 2 * PK_TILE_BYTES;
constexpr int PK_STAGE_BYTES = 4 * PK_TILE_BYTES;    // 64 KB
constexpr int PK_STAGES = 3;
constexpr int PK_PRODUCERS = 512;
constexpr int PK_PWARPS = PK_PRODUCERS / 32;
constexpr int PK_THREADS = PK_PRODUCERS + 32;
constexpr int PK_NTASK = 2 * PK_ROWS * (PK_BK / 8) / PK_PRODUCERS;   // 4

struct __align__(16) PkControl {
  unsigned long long full[PK_STAGES];
  unsigned long long empty[PK_STAGES];
  unsigned long long accum;
  unsigned tmem_base;
  volatile int abort_flag;
  int found;
  GemmDesc desc;
};
constexpr int PK_SMEM_BYTES =
    PK_STAGES * PK_STAGE_BYTES + ((int)sizeof(PkControl) + 1023) / 1024 * 1024 +
    1024;
static_assert(PK_SMEM_BYTES <= 227 * 1024, "pair kernel shared memory");
static_assert(TC_BM * TC_EPI_PITCH * 4 <= PK_STAGES * PK_STAGE_BYTES,
              "epilogue staging tile");

__device__ __forceinline__ unsigned long long pk_smem_desc(unsigned addr) {
  // K-major, 64-byte swizzle: 8-row groups 512 bytes apart.
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFF) >> 4);         // start address
  d |= (unsigned long long)1 << 16;                         // LBO (unused)
  d |= (unsigned long long)(512 >> 4) << 32;                // SBO
  d |= (unsigned long long)1 << 46;                         // descriptor version
  d |= (unsigned long long)4 << 61;                         // SWIZZLE_64B
  return d;
}

// Pair (Bi, Bj), Bj <= Bi, of 256-row blocks from its index Bi(Bi+1)/2 + Bj.
__device__ __forceinline__ void pk_pair(int t, int& Bi, int& Bj) {
  int a = (int)((sqrtf(8.f * (float)t + 1.f) - 1.f) * 0.5f);
  while ((a + 1) * (a + 2) / 2 <= t) ++a;
  while (a * (a + 1) / 2 > t) --a;
  Bi = a;
  Bj = t - a * (a + 1) / 2;
}

// STAGED: the operand comes from the bf16 planes of the staging pass through
// TMA: one thread issues, per k-block, a 32 k x 256 row box of each plane for
// the B rows (and the A rows off the diagonal) straight into the stage, in
// the 64-byte-swizzled K-major layout; rows past d and k past K arrive as
// zeros.  The other producer warps wait for the epilogue.
__device__ __forceinline__ void tma_load_2d(unsigned dst, const void* tmap,
                                            int x, int y, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::"
      "complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

template <bool IM2COL, bool TAILS, bool STAGED = false>
__global__ void __launch_bounds__(PK_THREADS, 1)
tc_pair_kernel(const GemmDesc* __restrict__ descs, int ndesc,
               const __grid_constant__ GemmDesc inline_desc) {
  extern __shared__ unsigned char tc_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
  PkControl* ctl =
      reinterpret_cast<PkControl*>(smem + PK_STAGES * PK_STAGE_BYTES);
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x;
  {
    const GemmDesc* src = &inline_desc;
    if (descs != nullptr) {
      for (int i = tid; i < ndesc; i += PK_THREADS) {
        const int lo = descs[i].tile_begin;
        const int hi = (i + 1 < ndesc) ? descs[i + 1].tile_begin : 0x7fffffff;
        if (lo <= tile && tile < hi) ctl->found = i;
      }
      __syncthreads();
      src = descs + ctl->found;
    }
    const int* s = reinterpret_cast<const int*>(src);
    int* d = reinterpret_cast<int*>(&ctl->desc);
    for (int i = tid; i < (int)(sizeof(GemmDesc) / sizeof(int)); i += PK_THREADS)
      d[i] = s[i];
  }
  if (tid == 0) {
    for (int s = 0; s < PK_STAGES; ++s) {
      mbar_init(&ctl->full[s], STAGED ? 1 : PK_PWARPS);
      mbar_init(&ctl->empty[s], 1);
    }
    mbar_init(&ctl->accum, 1);
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == PK_PWARPS) {
    asm volatile(
        "tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
        ::"r"(smem_u32(&ctl->tmem_base)), "r"(TC_TMEM_COLS)
        : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;"
                 ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

  const GemmDesc& g = ctl->desc;
  const unsigned tmem = ctl->tmem_base;
  const int nblk = (g.M + PK_ROWS - 1) / PK_ROWS;   // 256-row blocks
  const int npairs = nblk * (nblk + 1) / 2;
  int lt = tile - g.tile_begin, split = 0;
  if (g.splits > 1) {
    split = lt / npairs;
    lt -= split * npairs;
  }
  int Bi, Bj;
  pk_pair(lt, Bi, Bj);
  const int m0 = Bi * PK_ROWS, n0 = Bj * PK_ROWS;
  const bool share = Bi == Bj;
  const int n_valid = min(PK_ROWS, g.N - n0);
  const int n_inst = (n_valid + 15) & ~15;
  const int rows_a = min(PK_ROWS, g.M - m0);
  const bool two = rows_a > TC_BM;                  // second accumulator used
  long long kbeg = 0, kend = g.K;
  if (g.splits > 1) {
    kbeg = (long long)split * g.k_per_split;
    kend = min(g.K, kbeg + g.k_per_split);
  }
  const int nkb = kend > kbeg ? (int)((kend - kbeg + PK_BK - 1) / PK_BK) : 0;

  if (STAGED && warp < PK_PWARPS) {
    // ===================== TMA producer =====================
    if (tid == 0) {
      // the tensor maps were written to device memory by a copy that
      // precedes this launch in the stream
      asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;"
                   ::"l"(g.tmap_hi) : "memory");
      asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;"
                   ::"l"(g.tmap_lo) : "memory");
      const unsigned bytes = (share ? 2u : 4u) * PK_TILE_BYTES;
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % PK_STAGES;
        if (kb >= PK_STAGES) {
          if (!mbar_wait(&ctl->empty[s], ((kb / PK_STAGES) - 1) & 1,
                         &ctl->abort_flag))
            break;
        }
        const unsigned bar = smem_u32(&ctl->full[s]);
        asm volatile(
            "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
            ::"r"(bar), "r"(bytes) : "memory");
        const unsigned st = smem_u32(smem + s * PK_STAGE_BYTES);
        const int k0 = (int)kbeg + kb * PK_BK;
        tma_load_2d(st + PK_TILE_BYTES, g.tmap_hi, k0, n0, bar);
        tma_load_2d(st + PK_LO_OFF + PK_TILE_BYTES, g.tmap_lo, k0, n0, bar);
        if (!share) {
          tma_load_2d(st, g.tmap_hi, k0, m0, bar);
          tma_load_2d(st + PK_LO_OFF, g.tmap_lo, k0, m0, bar);
        }
      }
    }
  } else if (warp < PK_PWARPS) {
    // ===================== producers =====================
    const Operand X = g.A;                          // A and B are the same
    if (IM2COL) {
      // ---- im2col gather: lanes walk k.  Half a warp reads 32 consecutive
      // output pixels (16 lanes x 2) of one patch-matrix column, the other
      // half the same pixels of the next column: a load instruction touches
      // two to four cache lines instead of up to 32 sectors.  Warp w owns
      // rows 2w + 32 j + h (j = 0..15, h = lane / 16; j < 8: A rows) of the
      // 512 staged rows; a thread keeps the 16 row offsets in registers for
      // the whole tile, loads pixels (k, k+1) of each row per k-block and
      // packs them into one bf16x2 word per tile, so a warp's store covers
      // 128 contiguous bytes.  Rows past the operand's edge read column 0:
      // their products are never stored.  The appended ones column is
      // patched in after the loads.
      const int h = lane >> 4, kp = lane & 15;
      int off[16];
      unsigned ones = 0;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int R = 2 * warp + 32 * j + h;
        const bool is_a = j < 8;
        const int c = (is_a ? m0 : n0 - PK_ROWS) + R;
        int o = 0;
        if (c < X.ncols) {
          const int kk = X.ks * X.ks;
          const int ch = c / kk;
          const int r = c - ch * kk;
          const int ky = r / X.ks;
          const int kx = r - ky * X.ks;
          o = ch * X.H * X.W + ky * X.W + kx;
        } else if (c == X.extra_idx) {
          ones |= 1u << j;
        }
        off[j] = o;
      }
      const int kend_i = (int)kend;
      KState ks;
      kstate_init<true>(X, kbeg + 2 * kp, ks);
      const int chw = X.C * X.H * X.W, sw = X.st * X.W;
      const unsigned lane_off = (unsigned)((((kp >> 2) ^ (warp & 3)) << 4) +
                                           4 * (kp & 3) + h * 64 + warp * 128);
      // offset of the 1024-byte-aligned stage area inside the dynamic array
      const unsigned smem_skew = smem_u32(smem) - smem_u32(tc_smem_raw);
      const int j0 = share ? 8 : 0;
      float x[32];
      for (int kb = 0; kb <= nkb; ++kb) {
        if (kb > 0) {
          const int pb = kb - 1;
          const int s = pb % PK_STAGES;
          if (pb >= PK_STAGES) {
            if (!mbar_wait(&ctl->empty[s], ((pb / PK_STAGES) - 1) & 1,
                           &ctl->abort_flag))
              break;
          }
          // plain stores through a pointer into the shared array: the
          // per-row offsets (2048 j) fold into the instruction's immediate
          unsigned* st = reinterpret_cast<unsigned*>(
              tc_smem_raw + smem_skew + s * PK_STAGE_BYTES + lane_off);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (j < j0) continue;
            unsigned hi, lo;
            split_bf16x2(x[2 * j], x[2 * j + 1], hi, lo);
            st[512 * j] = hi;
            st[PK_LO_OFF / 4 + 512 * j] = lo;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->full[s]);
        }
        if (kb < nkb) {
          // pixel offsets of k and k + 1 (k + 1 may start the next image row)
          const bool live0 = !TAILS || ks.k < kend_i;
          const bool live1 = !TAILS || ks.k + 1 < kend_i;
          int o0 = ks.a * chw + ks.b * sw + ks.c * X.st;
          int o1 = o0 + X.st;
          if (ks.c + 1 >= X.Wo) {
            o1 = (ks.b + 1 >= X.Ho) ? (ks.a + 1) * chw
                                    : ks.a * chw + (ks.b + 1) * sw;
          }
          if (!live0) o0 = 0;
          if (!live1) o1 = 0;
          const float* p0 = X.base + o0;
          const float* p1 = X.base + o1;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (j < j0) continue;
            x[2 * j] = p0[off[j]];
            x[2 * j + 1] = p1[off[j]];
          }
          if (ones) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (ones & (1u << j)) x[2 * j] = x[2 * j + 1] = 1.f;
          }
          if (TAILS && !live1) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (!live0) x[2 * j] = 0.f;
              x[2 * j + 1] = 0.f;
            }
          }
          kstate_advance<true, PK_BK>(X, ks);
        }
      }
    } else {
      const bool kf = IM2COL || X.kfast;
      // per task: 128 of the 512 (A then B) rows; a warp covers 8 rows x 4
      // chunks of a k-contiguous operand, or one chunk of 32 rows of a
      // column-contiguous one
      PTask task[PK_NTASK];
  #pragma unroll
      for (int t = 0; t < PK_NTASK; ++t) {
        const bool is_a = t < PK_NTASK / 2;
        const int band_row = kf ? warp * 8 + (lane >> 2) : 32 * (warp >> 2) + lane;
        const int row = 128 * t + band_row - (is_a ? 0 : PK_ROWS);
        const int rows = is_a ? (share ? 0 : rows_a) : n_inst;
        const int chunk = kf ? (lane & 3) : (warp & 3);
        PTask v;
        v.soff = row < rows
                     ? (unsigned)((is_a ? 0 : PK_TILE_BYTES) + row * 64 +
                                  ((chunk ^ ((row >> 1) & 3)) << 4))
                     : ~0u;
        const float* p = g_zero_page;
        int m = 0;
        if (row < rows) {
          const int c = (is_a ? m0 : n0) + row;
          if (c < X.ncols) {
            p = X.base + (long long)c * X.s_col;
            m = X.period == 1 ? (int)X.s_outer : 1;
          } else if (c == X.extra_idx) {
            if (X.extra) { p = X.extra; m = 1; }
            else p = g_ones_page;
          }
        }
        v.p = reinterpret_cast<const char*>(p);
        v.m = m * 4;
        task[t] = v;
      }
      const int kend_i = (int)kend;
      KState ks;
      kstate_init<IM2COL>(X, kbeg + 8 * (kf ? (lane & 3) : (warp & 3)), ks);
      const unsigned smem_base = smem_u32(smem);
      const bool vec = !IM2COL && tc_operand_vec(X, kbeg);
      // a task is 8 consecutive k of one row: 16 bytes of each bf16 tile
      float4 v[PK_NTASK][2];
      for (int kb = 0; kb <= nkb; ++kb) {
        if (kb > 0) {
          const int pb = kb - 1;
          const int s = pb % PK_STAGES;
          if (pb >= PK_STAGES) {
            if (!mbar_wait(&ctl->empty[s], ((pb / PK_STAGES) - 1) & 1,
                           &ctl->abort_flag))
              break;
          }
          const unsigned st = smem_base + s * PK_STAGE_BYTES;
  #pragma unroll
          for (int t = 0; t < PK_NTASK; ++t)
            if (task[t].soff != ~0u)
              store_split_bf16(st + task[t].soff, st + PK_LO_OFF + task[t].soff,
                               v[t][0], v[t][1]);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->full[s]);
        }
        if (kb < nkb) {
          int o[8];
          tc_koffsets<IM2COL, TAILS, 8>(X, ks, kend_i, o);
          const int k = ks.k;
          const bool tail = TAILS && (k + 7 >= kend_i);
          if (vec && !tail) {
  #pragma unroll
            for (int t = 0; t < PK_NTASK; ++t)
              if (task[t].soff != ~0u) {
                v[t][0] = *reinterpret_cast<const float4*>(
                    task[t].p + (long long)o[0] * task[t].m);
                v[t][1] = *reinterpret_cast<const float4*>(
                    task[t].p + (long long)o[4] * task[t].m);
              }
          } else {
  #pragma unroll
            for (int t = 0; t < PK_NTASK; ++t) {
              if (task[t].soff == ~0u) continue;
              v[t][0].x = *reinterpret_cast<const float*>(task[t].p + (long long)o[0] * task[t].m);
              v[t][0].y = *reinterpret_cast<const float*>(task[t].p + (long long)o[1] * task[t].m);
              v[t][0].z = *reinterpret_cast<const float*>(task[t].p + (long long)o[2] * task[t].m);
              v[t][0].w = *reinterpret_cast<const float*>(task[t].p + (long long)o[3] * task[t].m);
              v[t][1].x = *reinterpret_cast<const float*>(task[t].p + (long long)o[4] * task[t].m);
              v[t][1].y = *reinterpret_cast<const float*>(task[t].p + (long long)o[5] * task[t].m);
              v[t][1].z = *reinterpret_cast<const float*>(task[t].p + (long long)o[6] * task[t].m);
              v[t][1].w = *reinterpret_cast<const float*>(task[t].p + (long long)o[7] * task[t].m);
            }
          }
          if (tail) {
  #pragma unroll
            for (int t = 0; t < PK_NTASK; ++t) {
              if (k + 0 >= kend_i) v[t][0].x = 0.f;
              if (k + 1 >= kend_i) v[t][0].y = 0.f;
              if (k + 2 >= kend_i) v[t][0].z = 0.f;
              if (k + 3 >= kend_i) v[t][0].w = 0.f;
              if (k + 4 >= kend_i) v[t][1].x = 0.f;
              if (k + 5 >= kend_i) v[t][1].y = 0.f;
              if (k + 6 >= kend_i) v[t][1].z = 0.f;
              if (k + 7 >= kend_i) v[t][1].w = 0.f;
            }
          }
          kstate_advance<IM2COL, PK_BK>(X, ks);
        }
      }
    }
  } else {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      const unsigned idesc = tc_instr_desc_bf16(n_inst);
      const unsigned a_off = share ? (unsigned)PK_TILE_BYTES : 0u;
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % PK_STAGES;
        if (!mbar_wait(&ctl->full[s], (kb / PK_STAGES) & 1, &ctl->abort_flag))
          break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned sa = smem_u32(smem + s * PK_STAGE_BYTES);
        const unsigned long long a_hi = pk_smem_desc(sa + a_off);
        const unsigned long long a_lo = pk_smem_desc(sa + PK_LO_OFF + a_off);
        const unsigned long long b_hi = pk_smem_desc(sa + PK_TILE_BYTES);
        const unsigned long long b_lo =
            pk_smem_desc(sa + PK_LO_OFF + PK_TILE_BYTES);
        // second accumulator: A rows 128..255 start 128 * 64 bytes later
        const unsigned long long up = (unsigned long long)(TC_BM * 64 >> 4);
#pragma unroll
        for (int kk = 0; kk < PK_BK / 16; ++kk) {
          // 16 bf16 = 32 bytes per MMA along k
          const unsigned long long adv = (unsigned long long)(kk * 32 >> 4);
          const unsigned acc = (kb | kk) != 0;
          tc_mma_bf16(tmem, a_lo + adv, b_hi + adv, idesc, acc);
          tc_mma_bf16(tmem, a_hi + adv, b_lo + adv, idesc, 1);
          tc_mma_bf16(tmem, a_hi + adv, b_hi + adv, idesc, 1);
          if (two) {
            tc_mma_bf16(tmem + TC_BN, a_lo + up + adv, b_hi + adv, idesc, acc);
            tc_mma_bf16(tmem + TC_BN, a_hi + up + adv, b_lo + adv, idesc, 1);
            tc_mma_bf16(tmem + TC_BN, a_hi + up + adv, b_hi + adv, idesc, 1);
          }
        }
        tc_commit(&ctl->empty[s]);
      }
      tc_commit(&ctl->accum);
    }
    __syncwarp();
  }

  // ===================== epilogue =====================
  if (warp < PK_PWARPS) {
    float* stage = reinterpret_cast<float*>(smem);
    if (nkb > 0) {
      mbar_wait(&ctl->accum, 0, &ctl->abort_flag);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    asm volatile("bar.sync 1, %0;" ::"r"(PK_PRODUCERS) : "memory");
    const bool dead = ctl->abort_flag != 0;        // uniform after the barrier
    const float alpha = g.alpha, beta = g.beta;
    const int q = warp & 3, h = warp >> 2;
    for (int tt = 0; tt < (two ? 2 : 1) && !dead; ++tt) {
      const int m0t = m0 + TC_BM * tt;
      const int m_valid = min(TC_BM, g.M - m0t);
      const int nv = min(n_valid, m0t + TC_BM - n0);   // lower triangle
      const int row = q * 32 + lane;
      for (int c0 = h * 16; c0 < n_inst; c0 += 16 * (PK_PWARPS / 4)) {
        float v[16];
        if (nkb > 0) {
          tc_ld16(tmem + ((unsigned)(q * 32) << 16) + (unsigned)(TC_BN * tt + c0), v);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) stage[row * TC_EPI_PITCH + c0 + i] = v[i];
      }
      asm volatile("bar.sync 1, %0;" ::"r"(PK_PRODUCERS) : "memory");
      if (g.splits > 1) {
        // 128 x 256 numbering: row block 2 Bi + tt, column block Bj
        const int lt128 = (tt == 0 ? Bi * (Bi + 1) : (Bi + 1) * (Bi + 1)) + Bj;
        float* p = g.partial +
                   ((long long)split * g.ntiles + lt128) * (TC_BM * TC_BN);
        for (int r = warp; r < TC_BM; r += PK_PWARPS)
          for (int c = lane; c < n_inst; c += 32)
            p[r * TC_BN + c] = stage[r * TC_EPI_PITCH + c];
      } else {
        for (int r = warp; r < m_valid; r += PK_PWARPS) {
          const int gr = m0t + r;
          float* crow = g.C + (long long)gr * g.ldc + n0;
          const int cend = min(nv, gr - n0 + 1);
          float old[TC_BN / 32];
          if (beta != 0.f) {
#pragma unroll
            for (int i = 0; i < TC_BN / 32; ++i) {
              const int c = lane + 32 * i;
              old[i] = c < cend ? crow[c] : 0.f;
            }
          }
#pragma unroll
          for (int i = 0; i < TC_BN / 32; ++i) {
            const int c = lane + 32 * i;
            if (c < cend) {
              float v = alpha * stage[r * TC_EPI_PITCH + c];
              if (beta != 0.f) v += beta * old[i];
              crow[c] = v;
              stage[r * TC_EPI_PITCH + c] = v;
            }
          }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(PK_PRODUCERS) : "memory");
        for (int c = warp; c < nv; c += PK_PWARPS) {
          const int gc = n0 + c;
          for (int r = lane; r < m_valid; r += 32) {
            const int gr = m0t + r;
            if (gc < gr)
              g.C[(long long)gc * g.ldc + gr] = stage[r * TC_EPI_PITCH + c];
          }
        }
      }
      // the second accumulator reuses the staging tile
      asm volatile("bar.sync 1, %0;" ::"r"(PK_PRODUCERS) : "memory");
    }
  }
  if (STAGED && tid == 0 && ctl->abort_flag != 0) {
    // a wait ran out: give the copies already issued time to land before
    // the shared memory is handed back (bounded: 64 us)
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == PK_PWARPS) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                 ::"r"(tmem), "r"(TC_TMEM_COLS)
                 : "memory");
  }
}


// Copies of NCHW tensors into buffers with a zero border of `pad` pixels.
// The zero-bordered copies of a grouped factor build in one launch: a work
// item is a run of whole planes of one job (about 4096 output elements),
// items are numbered job after job, and a block finds its job by bisection in
// a shared-memory copy of the first item of every job.
struct PadJob {
  const float* src;
  float* dst;
  long long planes;
  int h, w, pad;
  int group;        // planes per work item (NCHW source)
  int item_begin;   // first work item of this job
  int nhwc;         // source is channels-last: items are 32 x 32 transposes
  int C;            // channels (channels-last source)
};

constexpr int kPadJobsMax = 256;

__global__ void __launch_bounds__(256)
pad_copy_group_kernel(const PadJob* __restrict__ jobs, int njobs,
                      int total_items) {
  __shared__ int s_begin[kPadJobsMax];
  __shared__ float tile[32][33];
  for (int i = threadIdx.x; i < njobs; i += blockDim.x)
    s_begin[i] = jobs[i].item_begin;
  __syncthreads();
  for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
    int lo = 0, hi = njobs - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s_begin[mid] <= item) lo = mid; else hi = mid - 1;
    }
    const PadJob j = jobs[lo];
    const int wp = j.w + 2 * j.pad, per = (j.h + 2 * j.pad) * wp;
    if (j.nhwc) {
      // (n, h, w, c) -> zero-bordered (n, c, h + 2p, w + 2p): a 32-pixel x
      // 32-channel tile is read along c and written along the pixels; the
      // border was cleared before the launch
      const int hw = j.h * j.w;
      const int ct = (j.C + 31) >> 5, qt = (hw + 31) >> 5;
      int t = item - j.item_begin;
      const int n = t / (ct * qt);
      t -= n * ct * qt;
      const int c0 = (t / qt) << 5, q0 = (t % qt) << 5;
      const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int q = q0 + ty + 8 * i, c = c0 + tx;
        if (q < hw && c < j.C)
          tile[ty + 8 * i][tx] = j.src[((long long)n * hw + q) * j.C + c];
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = c0 + ty + 8 * i, q = q0 + tx;
        if (c < j.C && q < hw) {
          const int y = q / j.w, x = q - y * j.w;
          j.dst[((long long)n * j.C + c) * per + (y + j.pad) * wp + x + j.pad] =
              tile[tx][ty + 8 * i];
        }
      }
      __syncthreads();
      continue;
    }
    const long long p0 = (long long)(item - j.item_begin) * j.group;
    const long long p1 = min(j.planes, p0 + j.group);
    for (long long plane = p0; plane < p1; ++plane) {
      const float* src = j.src + plane * j.h * j.w;
      float* dst = j.dst + plane * per;
      for (int i = threadIdx.x; i < per; i += blockDim.x) {
        const int yy = i / wp;
        const int y = yy - j.pad, xx = i - yy * wp - j.pad;
        float v = 0.f;
        if ((unsigned)y < (unsigned)j.h && (unsigned)xx < (unsigned)j.w)
          v = src[y * j.w + xx];
        dst[i] = v;
      }
    }
  }
}

struct ReduceItem {     // one output tile whose split partials are summed
  const float* partial; // first split's copy of this tile
  float* out;
  long long sstride;    // elements between consecutive splits
  int d, tile, splits;
  float alpha, beta;
};

// `items` == nullptr: every block works on `single`, the item of tile 0 of one
// factor, and takes tile blockIdx.x of it (a lone factor needs no table in
// device memory, so the call neither allocates nor copies one).
__global__ void __launch_bounds__(256)
tc_reduce_kernel(const ReduceItem* __restrict__ items,
                 const __grid_constant__ ReduceItem single) {
  // Four lanes share one output element: lane q sums the splits
  // q, q+4, q+8, ... (always in that order), then the four sums are added in
  // a fixed tree, so the result does not depend on scheduling.
  ReduceItem it = items != nullptr ? items[blockIdx.x] : single;
  if (items == nullptr) {
    it.tile = (int)blockIdx.x;
    it.partial += (long long)blockIdx.x * (TC_BM * TC_BN);
  }
  int bi, bj;
  tc_tri_tile(it.tile, bi, bj);
  const int d = it.d;
  const int m0 = bi * TC_BM, n0 = bj * TC_BN;
  const int rows = min(TC_BM, d - m0);
  const int cols = min(min(TC_BN, d - n0), m0 + TC_BM - n0);
  const int q = threadIdx.x & 3;
  const int total = rows * cols;
  for (int e = blockIdx.y * 1024 + (threadIdx.x >> 2);
       e < min(total, (int)(blockIdx.y + 1) * 1024); e += 64) {
    const int r = e / cols, c = e - r * cols;
    const float* p = it.partial + r * TC_BN + c;
    float s0 = 0.f, s1 = 0.f;
    int sp = q;
    for (; sp + 4 < it.splits; sp += 8) {
      s0 += p[sp * it.sstride];
      s1 += p[(sp + 4) * it.sstride];
    }
    if (sp < it.splits) s0 += p[sp * it.sstride];
    float s = s0 + s1;
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    const int gr = m0 + r, gc = n0 + c;
    if (q != 0 || gc > gr) continue;
    float* o = it.out + (long long)gr * d + gc;
    float v = it.alpha * s;
    if (it.beta != 0.f) v += it.beta * (*o);
    *o = v;
    if (gc < gr) it.out[(long long)gc * d + gr] = v;
  }
}

// ------------------------------------------------------------------ host side
static int g_engine = 1;

int tc_tiles(GemmDesc& g) {
  g.tiles_m = (g.M + TC_BM - 1) / TC_BM;
  g.tiles_n = (g.N + TC_BN - 1) / TC_BN;
  if (g.flags & G_LOWER) {
    int nt = g.tiles_m, a = nt / 2;
    return (nt & 1) ? (a + 1) * (a + 1) : a * (a + 1);
  }
  return g.tiles_m * g.tiles_n;
}

int tc_prepare() {
  static std::mutex mu;
  static bool done[64] = {false};
  int dev = 0;
  KFAC_CUDA(cudaGetDevice(&dev));
  KFAC_REQUIRE(dev >= 0 && dev < 64, "device index %d unsupported", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!done[dev]) {
    KFAC_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<false, false, TC_PW_STRIDED>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   TC_SMEM_BYTES));
    KFAC_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<false, true, TC_PW_STRIDED>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   TC_SMEM_BYTES));
    KFAC_CUDA(cudaFuncSetAttribute(tc_pair_kernel<false, false, true>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   PK_SMEM_BYTES));
    KFAC_CUDA(cudaFuncSetAttribute(tc_pair_kernel<false, false>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   PK_SMEM_BYTES));
    KFAC_CUDA(cudaFuncSetAttribute(tc_pair_kernel<false, true>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   PK_SMEM_BYTES));
    KFAC_CUDA(cudaFuncSetAttribute(tc_pair_kernel<true, false>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   PK_SMEM_BYTES));
    KFAC_CUDA(cudaFuncSetAttribute(tc_pair_kernel<true, true>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   PK_SMEM_BYTES));
    done[dev] = true;
  }
  return KFAC_OK;
}

int launch_tc_grouped(const GemmDesc* descs_dev, int ndesc, int total_tiles,
                      float lr, float momentum, bool tails,
                      cudaStream_t stream) {
  if (ndesc <= 0 || total_tiles <= 0) return KFAC_OK;
  int rc = tc_prepare();
  if (rc != KFAC_OK) return rc;
  GemmDesc dummy = {};
  if (tails)
    tc_gemm_kernel<false, true, TC_PW_STRIDED><<<total_tiles, TcMap<TC_PW_STRIDED>::kThreads, TC_SMEM_BYTES,
                                  stream>>>(descs_dev, ndesc, dummy, lr,
                                            momentum);
  else
    tc_gemm_kernel<false, false, TC_PW_STRIDED><<<total_tiles, TcMap<TC_PW_STRIDED>::kThreads, TC_SMEM_BYTES,
                                   stream>>>(descs_dev, ndesc, dummy, lr,
                                             momentum);
  KFAC_LAUNCH_CHECK("tc_gemm_kernel");
  return KFAC_OK;
}

// True when some k-block of the problem can be cut by the end of its
// contraction range (ranges start at multiples of 128 or of k_per_split, both
// multiples of the k-block).
bool tc_desc_has_tails(const GemmDesc& g) {
  if (g.K % TC_BK != 0) return true;
  if (g.splits > 1 && g.k_per_split % TC_BK != 0) return true;
  return false;
}

struct TcFactorSplit {
  int tiles, splits;
  long long k_per_split;
};

// CTAs that cover the lower tiles of a d x d output once.
static int tc_factor_ctas(int d) {
  const int nblk = (d + PK_ROWS - 1) / PK_ROWS;
  return nblk * (nblk + 1) / 2;
}

static int tc_lower_tiles(int d) {
  GemmDesc g = {};
  g.M = g.N = d;
  g.flags = G_LOWER;
  return tc_tiles(g);
}

// Relative duration of one k-block of a CTA of a d x d factor, in 1/512: a
// CTA stages up to 512 operand rows per k-block, d of them when d <= 256; a
// k-block with few rows still costs about a memory round trip.
static long long tc_block_cost(int d) {
  const int rows = d < 512 ? d : 512;
  return rows < 256 ? 256 : rows;
}

// Split of one factor's contraction.  `chunk` is the cost (k-blocks x
// tc_block_cost) a CTA should own; a CTA keeps at least 16 k-blocks so that
// prologue and epilogue stay amortised, and a contraction is only cut when
// that brings its CTAs closer to the target than leaving it whole (partial
// tiles cost a write, a read and the reduce kernel).
// The tensor core adds each MMA's products into the fp32 accumulator with
// truncation, so a sum of N MMAs drifts by up to about N * 2^-25 of its
// magnitude, all in one direction when the addends share a sign (activation
// factors: products of non-negative values; three MMAs per 16 rows here).
// Measured relative error of 100 352-row factors: 2e-4 when one CTA
// accumulates 1500 k-blocks, 4.7e-5 at 256, 2e-5 at 128.  A CTA therefore
// never accumulates more than this many k-blocks (of 32 rows); the partial
// tiles of longer contractions are summed in fp32 by the reduce kernel, with
// rounding to nearest.  256 keeps the drift at half the 1e-4 bound and costs
// nothing measurable; 128 costs 15 % of the factor stage.
static long long tc_max_kblocks() {
  static const long long v = [] {
    const char* e = getenv("KFAC_TC_MAX_KBLOCKS");
    const long long k = e ? atoll(e) : 256;
    return k >= 16 ? k : 256;
  }();
  return v;
}

static TcFactorSplit tc_split_for(long long rows, int d, long long chunk) {
  TcFactorSplit s;
  s.tiles = tc_lower_tiles(d);
  chunk /= tc_block_cost(d);
  if (chunk < 16) chunk = 16;
  if (chunk > tc_max_kblocks()) chunk = tc_max_kblocks();
  const long long kblocks = (rows + TC_BK - 1) / TC_BK;
  long long sp = (kblocks + chunk / 2) / chunk;
  if (sp < 1) sp = 1;
  long long kps = (kblocks + sp - 1) / sp * TC_BK;
  s.splits = (int)((rows + kps - 1) / kps);
  if (s.splits < 1) s.splits = 1;
  s.k_per_split = kps;
  return s;
}

static TcFactorSplit tc_factor_split(long long rows, int d) {
  // a factor built on its own: aim at two waves of CTAs
  const int tiles = tc_factor_ctas(d);
  const long long kblocks = (rows + TC_BK - 1) / TC_BK;
  long long want = (2LL * sm_count() + tiles - 1) / tiles;   // splits wanted
  if (tiles >= sm_count()) want = 1;
  long long chunk = (kblocks + want - 1) / want;
  return tc_split_for(rows, d, chunk * tc_block_cost(d));
}

// Factor builds read their operands from the staged bf16 planes through TMA
// (stage.cu) when this is on (kfac_set_factor_staging, initial value from
// KFAC_TC_STAGED, default off) and the caller gives workspace; otherwise the
// producer warps gather and split the operands themselves.
static int g_staged = -1;
bool tc_staged() {
  if (g_staged < 0) {
    const char* e = getenv("KFAC_TC_STAGED");
    g_staged = (e != nullptr && atoi(e) != 0) ? 1 : 0;
  }
  return g_staged != 0;
}

size_t tc_factor_workspace_bytes(long long rows, int d, bool staged) {
  TcFactorSplit s = tc_factor_split(rows, d);
  size_t bytes = (staged && tc_staged()) ? tc_stage_bytes(rows, d) : 0;
  if (s.splits > 1)
    bytes += (size_t)s.splits * s.tiles * TC_BM * TC_BN * sizeof(float);
  return bytes;
}

size_t tc_pad_bytes(const Operand& X, int n, int nhwc) {
  // a staging copy is made for a zero border and / or to turn a channels-last
  // tensor into the NCHW planes the gather walks
  if (X.mode != 1 || (X.pd == 0 && !nhwc)) return 0;
  size_t e = (size_t)n * X.C * (X.H + 2 * X.pd) * (X.W + 2 * X.pd);
  return (e * sizeof(float) + 255) & ~(size_t)255;
}

// k-blocks per CTA for a group of factors: total work spread over ~4 waves.
static long long tc_group_chunk(int count, const FactorJob* jobs) {
  long long work = 0;
  for (int i = 0; i < count; ++i)
    work += (long long)tc_factor_ctas(jobs[i].d) *
            ((jobs[i].rows + TC_BK - 1) / TC_BK) * tc_block_cost(jobs[i].d);
  static const long long waves = [] {
    const char* e = getenv("KFAC_TC_WAVES");
    const long long w = e ? atoll(e) : 4;
    return w > 0 ? w : 4;
  }();
  return work / (waves * sm_count());
}

size_t tc_factor_group_workspace_bytes(int count, const FactorJob* jobs,
                                       bool staged) {
  const long long chunk = tc_group_chunk(count, jobs);
  staged = staged && tc_staged();
  size_t total = 0;
  for (int i = 0; i < count; ++i) {
    total += staged ? tc_stage_bytes(jobs[i].rows, jobs[i].d)
                    : tc_pad_bytes(jobs[i].X, jobs[i].n, jobs[i].nhwc);
    TcFactorSplit s = count == 1 ? tc_factor_split(jobs[i].rows, jobs[i].d)
                                 : tc_split_for(jobs[i].rows, jobs[i].d, chunk);
    if (s.splits > 1)
      total += (size_t)s.splits * s.tiles * TC_BM * TC_BN * sizeof(float);
  }
  return total;
}

// Per-device helper stream: the strided and the im2col launch of a grouped
// factor build do not depend on each other, and each has a tail of CTAs that
// leaves SMs idle, so they run side by side (fork / join with events).
struct SideStream {
  cudaStream_t stream;
  cudaEvent_t fork, join;
};

static int tc_side_stream(SideStream** out) {
  static std::mutex mu;
  static SideStream side[64];
  static bool made[64] = {false};
  int dev = 0;
  KFAC_CUDA(cudaGetDevice(&dev));
  KFAC_REQUIRE(dev >= 0 && dev < 64, "device index %d unsupported", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!made[dev]) {
    KFAC_CUDA(cudaStreamCreateWithFlags(&side[dev].stream, cudaStreamNonBlocking));
    KFAC_CUDA(cudaEventCreateWithFlags(&side[dev].fork, cudaEventDisableTiming));
    KFAC_CUDA(cudaEventCreateWithFlags(&side[dev].join, cudaEventDisableTiming));
    made[dev] = true;
  }
  *out = &side[dev];
  return KFAC_OK;
}

struct alignas(64) TmapBlob {     // a CUtensorMap, opaque here
  unsigned char b[128];
};

int run_factor_group_tc(int count, const FactorJob* jobs, void* workspace,
                        size_t workspace_bytes, cudaStream_t main_stream,
                        bool staged) {
  cudaStream_t stream = main_stream;
  int rc = tc_prepare();
  if (rc != KFAC_OK) return rc;
  staged = staged && tc_staged();
  const size_t need = tc_factor_group_workspace_bytes(count, jobs, staged);
  if (need > 0 && (workspace == nullptr || workspace_bytes < need))
    return fail(KFAC_ERR_WORKSPACE,
                "factor: workspace of %zu bytes needed, %zu given", need,
                workspace_bytes);
  const long long chunk = tc_group_chunk(count, jobs);
  char* ws = static_cast<char*>(workspace);

  std::vector<GemmDesc> descs[2];       // [0] strided, [1] im2col
  std::vector<ReduceItem> reduces;
  std::vector<PadJob> pads;
  int pad_items = 0;
  for (int i = 0; i < count; ++i) {
    KFAC_REQUIRE(jobs[i].out != nullptr && jobs[i].X.base != nullptr,
                 "factor: null pointer");
    KFAC_REQUIRE(jobs[i].rows > 0 && jobs[i].d > 0 &&
                     jobs[i].rows < (1LL << 31),
                 "factor: rows=%lld d=%d out of range", jobs[i].rows,
                 jobs[i].d);
  }
  const TmapBlob* dev_maps = nullptr;
  if (staged) {
    // staging pass: X^T of every job as two bf16 planes, two tensor maps each
    std::vector<TmapBlob> maps(2 * (size_t)count);
    rc = tc_stage_group(count, jobs, ws, maps.data(), stream);
    if (rc != KFAC_OK) return rc;
    for (int i = 0; i < count; ++i)
      ws += tc_stage_bytes(jobs[i].rows, jobs[i].d);
    void* dev = nullptr;
    rc = ring_alloc(maps.size() * sizeof(TmapBlob), &dev);
    if (rc != KFAC_OK) return rc;
    KFAC_CUDA(cudaMemcpyAsync(dev, maps.data(), maps.size() * sizeof(TmapBlob),
                              cudaMemcpyHostToDevice, stream));
    dev_maps = static_cast<const TmapBlob*>(dev);
  }
  for (int i = 0; i < count; ++i) {
    const FactorJob& job = jobs[i];
    Operand X = job.X;
    if (!staged && X.mode == 1 && (X.pd > 0 || job.nhwc)) {
      // zero-bordered NCHW copy first; the gather then needs no bounds checks
      const size_t pad_bytes = tc_pad_bytes(X, job.n, job.nhwc);
      float* padded = reinterpret_cast<float*>(ws);
      ws += pad_bytes;
      const long long planes = (long long)job.n * X.C;
      const long long total = planes * (X.H + 2 * X.pd) * (X.W + 2 * X.pd);
      KFAC_REQUIRE(total < (1LL << 31), "factor: padded input too large");
      const int per = (X.H + 2 * X.pd) * (X.W + 2 * X.pd);
      PadJob pj;
      pj.src = X.base;
      pj.dst = padded;
      pj.planes = planes;
      pj.h = X.H;
      pj.w = X.W;
      pj.pad = X.pd;
      pj.group = per >= 4096 ? 1 : 4096 / per;
      pj.item_begin = pad_items;
      pj.nhwc = job.nhwc;
      pj.C = X.C;
      if (job.nhwc) {
        if (X.pd > 0)
          KFAC_CUDA(cudaMemsetAsync(padded, 0, pad_bytes, stream));
        pad_items += job.n * ((X.C + 31) / 32) * ((X.H * X.W + 31) / 32);
      } else {
        pad_items += (int)((planes + pj.group - 1) / pj.group);
      }
      pads.push_back(pj);
      X.base = padded;
      X.H += 2 * X.pd;
      X.W += 2 * X.pd;
      X.pd = 0;
    }
    TcFactorSplit s = count == 1 ? tc_factor_split(job.rows, job.d)
                                 : tc_split_for(job.rows, job.d, chunk);
    GemmDesc g = {};
    g.A = X;
    g.B = X;
    g.C = job.out;
    g.ldc = job.d;
    g.K = job.rows;
    g.M = job.d;
    g.N = job.d;
    g.alpha = job.alpha;
    g.beta = job.beta;
    g.flags = G_LOWER | G_MIRROR | G_SAME_AB;
    g.ntiles = tc_tiles(g);
    g.splits = s.splits;
    g.k_per_split = s.k_per_split;
    g.partial = nullptr;
    if (staged) {
      g.tmap_hi = dev_maps + 2 * i;
      g.tmap_lo = dev_maps + 2 * i + 1;
    }
    if (s.splits > 1) {
      g.partial = reinterpret_cast<float*>(ws);
      ws += (size_t)s.splits * s.tiles * TC_BM * TC_BN * sizeof(float);
      for (int t = 0; t < s.tiles; ++t) {
        ReduceItem it;
        it.partial = g.partial + (long long)t * (TC_BM * TC_BN);
        it.out = job.out;
        it.sstride = (long long)s.tiles * (TC_BM * TC_BN);
        it.d = job.d;
        it.tile = t;
        it.splits = s.splits;
        it.alpha = job.alpha;
        it.beta = job.beta;
        reduces.push_back(it);
      }
    }
    descs[(X.mode == 1 && !staged) ? 1 : 0].push_back(g);
  }
  for (size_t b = 0; b < pads.size(); b += kPadJobsMax) {
    // (more than kPadJobsMax padded inputs in one group: several launches)
    const int nj = (int)std::min<size_t>(kPadJobsMax, pads.size() - b);
    std::vector<PadJob> part(pads.begin() + b, pads.begin() + b + nj);
    const int first = part[0].item_begin;
    for (PadJob& pj : part) pj.item_begin -= first;
    const int items =
        (b + nj < pads.size() ? pads[b + nj].item_begin : pad_items) - first;
    void* dev = nullptr;
    rc = ring_alloc(part.size() * sizeof(PadJob), &dev);
    if (rc != KFAC_OK) return rc;
    KFAC_CUDA(cudaMemcpyAsync(dev, part.data(), part.size() * sizeof(PadJob),
                              cudaMemcpyHostToDevice, stream));
    const int grid = std::min(items, sm_count() * 8);
    pad_copy_group_kernel<<<grid, 256, 0, stream>>>(
        static_cast<const PadJob*>(dev), nj, items);
    KFAC_LAUNCH_CHECK("pad_copy_group_kernel");
  }
  SideStream* side = nullptr;
  if (!descs[0].empty() && !descs[1].empty()) {
    rc = tc_side_stream(&side);
    if (rc != KFAC_OK) return rc;
    KFAC_CUDA(cudaEventRecord(side->fork, main_stream));
    KFAC_CUDA(cudaStreamWaitEvent(side->stream, side->fork, 0));
  }
  for (int m = 0; m < 2; ++m) {
    std::vector<GemmDesc>& v = descs[m];
    if (v.empty()) continue;
    // strided problems on the helper stream when there are both kinds
    stream = (m == 0 && side != nullptr) ? side->stream : main_stream;
    // long-running CTAs first
    // (duration of a CTA ~ its k-blocks times the operand rows it stages)
    std::stable_sort(v.begin(), v.end(), [](const GemmDesc& a, const GemmDesc& b) {
      long long ka = (a.splits > 1 ? a.k_per_split : a.K) * tc_block_cost(a.M);
      long long kb = (b.splits > 1 ? b.k_per_split : b.K) * tc_block_cost(b.M);
      return ka > kb;
    });
    int total = 0;
    for (GemmDesc& g : v) {
      g.tile_begin = total;
      total += tc_factor_ctas(g.M) * (g.splits > 1 ? g.splits : 1);
    }
    bool tails = false;
    for (const GemmDesc& g : v) tails = tails || tc_desc_has_tails(g);
    const GemmDesc* dev_descs = nullptr;
    GemmDesc inl = {};
    if (v.size() == 1) {
      inl = v[0];
    } else {
      void* dev = nullptr;
      rc = ring_alloc(v.size() * sizeof(GemmDesc), &dev);
      if (rc != KFAC_OK) return rc;
      KFAC_CUDA(cudaMemcpyAsync(dev, v.data(), v.size() * sizeof(GemmDesc),
                                cudaMemcpyHostToDevice, stream));
      dev_descs = static_cast<const GemmDesc*>(dev);
    }
    const int nd = (int)v.size();
    if (staged)
      tc_pair_kernel<false, false, true>
          <<<total, PK_THREADS, PK_SMEM_BYTES, stream>>>(dev_descs, nd, inl);
    else if (m == 1 && tails)
      tc_pair_kernel<true, true><<<total, PK_THREADS, PK_SMEM_BYTES, stream>>>(
          dev_descs, nd, inl);
    else if (m == 1)
      tc_pair_kernel<true, false><<<total, PK_THREADS, PK_SMEM_BYTES, stream>>>(
          dev_descs, nd, inl);
    else if (tails)
      tc_pair_kernel<false, true><<<total, PK_THREADS, PK_SMEM_BYTES, stream>>>(
          dev_descs, nd, inl);
    else
      tc_pair_kernel<false, false><<<total, PK_THREADS, PK_SMEM_BYTES, stream>>>(
          dev_descs, nd, inl);
    KFAC_LAUNCH_CHECK("tc_pair_kernel");
  }
  stream = main_stream;
  if (side != nullptr) {
    KFAC_CUDA(cudaEventRecord(side->join, side->stream));
    KFAC_CUDA(cudaStreamWaitEvent(main_stream, side->join, 0));
  }
  if (!reduces.empty()) {
    void* dev = nullptr;
    if (count > 1) {
      rc = ring_alloc(reduces.size() * sizeof(ReduceItem), &dev);
      if (rc != KFAC_OK) return rc;
      KFAC_CUDA(cudaMemcpyAsync(dev, reduces.data(),
                                reduces.size() * sizeof(ReduceItem),
                                cudaMemcpyHostToDevice, stream));
    }
    int dmax = 0;
    for (const ReduceItem& it : reduces) dmax = it.d > dmax ? it.d : dmax;
    const int rmax = dmax < TC_BM ? dmax : TC_BM;
    const int cmax = dmax < TC_BN ? dmax : TC_BN;
    dim3 rgrid((unsigned)reduces.size(), (rmax * cmax + 1023) / 1024);
    // a lone factor: its items are consecutive tiles of one output, passed
    // by value (reduces[0] is tile 0)
    tc_reduce_kernel<<<rgrid, 256, 0, stream>>>(
        static_cast<const ReduceItem*>(dev), reduces[0]);
    KFAC_LAUNCH_CHECK("tc_reduce_kernel");
  }
  return KFAC_OK;
}

int run_factor_tc(const Operand& X, long long rows, int d, float alpha,
                  float beta, float* out, void* workspace,
                  size_t workspace_bytes, cudaStream_t stream, bool staged) {
  FactorJob job;
  job.X = X;
  job.rows = rows;
  job.d = d;
  job.n = X.mode == 1 ? (int)(rows / ((long long)X.Ho * X.Wo)) : 0;
  job.nhwc = 0;
  job.alpha = alpha;
  job.beta = beta;
  job.out = out;
  return run_factor_group_tc(1, &job, workspace, workspace_bytes, stream,
                             staged);
}

int engine() { return g_engine; }

}  // namespace kfac

extern "C" int kfac_set_engine(int engine) {
  if (engine != 0 && engine != 1)
    return kfac::fail(KFAC_ERR_INVALID, "set_engine: engine must be 0 or 1");
  kfac::g_engine = engine;
  return KFAC_OK;
}

extern "C" int kfac_get_engine(void) { return kfac::g_engine; }

extern "C" int kfac_set_factor_staging(int on) {
  kfac::g_staged = on ? 1 : 0;
  return KFAC_OK;
}

extern "C" int kfac_get_factor_staging(void) {
  return kfac::tc_staged() ? 1 : 0;
}

#ifdef KFAC_TC_TRACE
extern "C" int kfac_tc_trace(long long* buf_dev, int capacity) {
  KFAC_CUDA(cudaMemcpyToSymbol(kfac::g_tc_trace, &buf_dev, sizeof(buf_dev)));
  KFAC_CUDA(cudaMemcpyToSymbol(kfac::g_tc_trace_cap, &capacity, sizeof(int)));
  return KFAC_OK;
}
#endif

namespace kfac {
// Self-test of the bounded barrier wait every tile kernel relies on: one warp
// waits on a barrier that nothing will ever arrive at, with a short limit.
// The wait must give up, raise the status word it was given and let the
// kernel return.
__global__ void wait_expiry_selftest_kernel(int* status, int* returned) {
  __shared__ unsigned long long bar;
  __shared__ volatile int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  const bool ok = mbar_wait_status(&bar, 0, &abort_flag, status, 1u << 10);
  if (threadIdx.x == 0) *returned = ok ? 1 : 2;
}
}  // namespace kfac

extern "C" int kfac_selftest_wait_expiry(int* status_out, int* returned_out) {
  KFAC_REQUIRE(status_out != nullptr && returned_out != nullptr,
               "selftest_wait_expiry: null pointer");
  int* dev = nullptr;
  KFAC_CUDA(cudaMalloc(&dev, 2 * sizeof(int)));
  cudaError_t e = cudaMemset(dev, 0, 2 * sizeof(int));
  if (e == cudaSuccess) {
    kfac::wait_expiry_selftest_kernel<<<1, 32>>>(dev, dev + 1);
    kfac::count_launch();
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  int host[2] = {-1, -1};
  if (e == cudaSuccess)
    e = cudaMemcpy(host, dev, sizeof(host), cudaMemcpyDeviceToHost);
  cudaFree(dev);
  if (e != cudaSuccess)
    return kfac::fail(KFAC_ERR_CUDA, "selftest_wait_expiry: %s",
                      cudaGetErrorString(e));
  *status_out = host[0];
  *returned_out = host[1];
  return KFAC_OK;
}

extern "C" int kfac_tc_status(int* status_out) {
  KFAC_REQUIRE(status_out != nullptr, "tc_status: null pointer");
  KFAC_CUDA(cudaDeviceSynchronize());
  int v = 0;
  KFAC_CUDA(cudaMemcpyFromSymbol(&v, kfac::g_tc_status, sizeof(int)));
  int w = 0;
  int rc = kfac::diag_status_read(&w);
  if (rc != KFAC_OK) return rc;
  *status_out = v | w;
  return KFAC_OK;
}
