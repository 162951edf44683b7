// Batched damped inverse of symmetric positive definite factors.
//
//   W = F + add * I                     (copy; the running average F is kept)
//   W = L L^T                           blocked right-looking Cholesky, NB = 128
//   X = L^-1                            diagonal blocks in the factor kernel,
//                                       off-diagonal blocks by recursive doubling
//   inv = X^T X                         symmetric product, lower tiles mirrored
//
// A plan precomputes, for a fixed set of matrices, the descriptor lists of
// every grouped-GEMM launch; running it replays ~3 launches per 128-column
// panel of the largest matrix plus 2 per doubling level, each launch covering
// all matrices that are still active.
#include <vector>
#include <algorithm>

#include "gemm_simt.cuh"
#include "tc_common.cuh"

namespace kfac {

constexpr int DB = 128;        // diagonal block
constexpr int PW = 512;        // Cholesky panel width (outer blocking)
// floats of the diagonal kernel's shared memory: Lt, Pt, Xr, Tk
constexpr int kDiagBaseFloats = DB * (DB + 4) + 24 * DB + 16 * 64;

struct MatInfo {
  const float* F;
  float* inv;
  float* W;
  float* X;
  int d;
  int partner;
  int role;
  float l2;
  float scale;
  float l2b;      // role 2: floor of the second half of the diagonal
};

// Per-run arguments, kept in device memory so that a captured CUDA graph of
// the plan's launches can be replayed with new values: a one-thread kernel
// ahead of the graph writes them.
struct RunParams {
  float damping;
  int use_pi;
  int refine_max_dim;
  float refine_threshold;
  // CUDA graph of one run (captured on first use)
  RunParams* params_dev;
  std::vector<cudaEvent_t> events;   // edges between the two streams
  cudaEvent_t fork_ev, join_ev[2];
  cudaStream_t side_stream[2];       // bulk / far stream of plain runs
  cudaStream_t cap_side[2];          // the same during capture
  bool look;
  cudaStream_t cap_stream;
  cudaGraphExec_t graph_exec;
  int* graph_info;
  float* graph_diag;
  long long graph_launches;
  bool graph_ok;
};

__global__ void set_run_params_kernel(RunParams* prm, float damping,
                                      int use_pi, int refine_max_dim,
                                      float refine_threshold) {
  prm->damping = damping;
  prm->use_pi = use_pi;
  prm->refine_max_dim = refine_max_dim;
  prm->refine_threshold = refine_threshold;
}

__global__ void trace_kernel(const MatInfo* __restrict__ mats,
                             float* __restrict__ trace, int* __restrict__ info) {
  const MatInfo mi = mats[blockIdx.x];
  float s = 0.f;
  for (int i = threadIdx.x; i < mi.d; i += blockDim.x)
    s += mi.F[(long long)i * mi.d + i];
  __shared__ float sh[32];
  for (int o = 16; o > 0; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    for (int o = 16; o > 0; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) {
      trace[blockIdx.x] = s;
      info[blockIdx.x] = 0;
    }
  }
}

__global__ void damping_kernel(const MatInfo* __restrict__ mats, int count,
                               const float* __restrict__ trace,
                               const RunParams* __restrict__ prm,
                               float* __restrict__ add,
                               float* __restrict__ add2,
                               float* __restrict__ add_out) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const float damping = prm->damping;
  const int use_pi = prm->use_pi;
  const MatInfo mi = mats[i];
  float g = fmaxf(mi.l2, damping);
  float v, v2;
  if (mi.role == 2) {
    // first half of the diagonal (scale parameters) and second half (shift
    // parameters) have their own floors
    v = g * mi.scale;
    v2 = fmaxf(mi.l2b, damping) * mi.scale;
  } else {
    float r = sqrtf(g);
    float pi = 1.f;
    if (use_pi && mi.partner >= 0) {
      const MatInfo mp = mats[mi.partner];
      // pi = sqrt(tr(A) dim(G) / (tr(G) dim(A))) with A the forward factor
      float tA = mi.role == 0 ? trace[i] : trace[mi.partner];
      float tG = mi.role == 0 ? trace[mi.partner] : trace[i];
      float dA = (float)(mi.role == 0 ? mi.d : mp.d);
      float dG = (float)(mi.role == 0 ? mp.d : mi.d);
      pi = sqrtf((tA * dG) / (tG * dA));
    }
    v = mi.role == 0 ? pi * r : (1.f / pi) * r;
    v2 = v;
  }
  add[i] = v;
  add2[i] = v2;
  if (add_out) add_out[i] = v;
}

// W = F + add * I, blockIdx.y = matrix, blockIdx.x strides over rows.  Only
// the lower triangle and the rest of each diagonal 128-block (which the
// trailing updates read-modify-write) is ever used, so only that is copied.
// With `dual` the first block column below the first diagonal block is also
// stored in the inverse's output buffer (see the look-ahead of the Cholesky).
__global__ void damp_copy_kernel(const MatInfo* __restrict__ mats,
                                 const float* __restrict__ add,
                                 const float* __restrict__ add2, int dual) {
  const MatInfo mi = mats[blockIdx.y];
  const float a_first = add[blockIdx.y], a_second = add2[blockIdx.y];
  const int d = mi.d;
  const bool vec = (d & 3) == 0 &&
                   ((reinterpret_cast<uintptr_t>(mi.F) |
                     reinterpret_cast<uintptr_t>(mi.W) |
                     reinterpret_cast<uintptr_t>(mi.inv)) & 15) == 0;
  for (int r = blockIdx.x; r < d; r += gridDim.x) {
    const float a = (mi.role == 2 && 2 * r >= d) ? a_second : a_first;
    const int cend = min(d, (r | (DB - 1)) + 1);
    const float* src = mi.F + (long long)r * d;
    float* dst = mi.W + (long long)r * d;
    if (vec) {
      // cend is a multiple of 128 or equals d, itself a multiple of 4 here
      const float4* s4 = reinterpret_cast<const float4*>(src);
      float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll 4
      for (int c4 = threadIdx.x; c4 < (cend >> 2); c4 += blockDim.x) {
        float4 v = s4[c4];
        if ((r >> 2) == c4) {
          if ((r & 3) == 0) v.x += a;
          else if ((r & 3) == 1) v.y += a;
          else if ((r & 3) == 2) v.z += a;
          else v.w += a;
        }
        d4[c4] = v;
        if (dual && r >= DB && c4 < DB / 4)
          reinterpret_cast<float4*>(mi.inv + (long long)r * d)[c4] = v;
      }
    } else {
      for (int c = threadIdx.x; c < cend; c += blockDim.x) {
        float v = src[c];
        if (r == c) v += a;
        dst[c] = v;
        if (dual && r >= DB && c < DB) mi.inv[(long long)r * d + c] = v;
      }
    }
  }
}


// ------------------------------------------------ look-ahead of the Cholesky
constexpr int DLD = DB + 4;   // shared-memory row pitch of a 128 x 128 block
constexpr int kLookTile = DB * 32 * 4;          // one 128 x 32 fp32 operand tile
constexpr int kLookStage = 4 * kLookTile;       // [A hi][A lo][B hi][B lo]
constexpr int kLookCols = 2 * DB;               // tensor-memory columns

static __device__ int g_diag_status = 0;

struct LookControl {
  unsigned long long bar[2];   // a stage's MMAs have finished reading it
  unsigned long long done;     // all MMAs of the second product have finished
  unsigned tmem_base;
  volatile int abort_flag;
};

// Issue the three split-TF32 MMAs of one 32-k operand block: D(128 x 128) +=
// A B^T with A, B given as hi / lo tile addresses (K-major, 128-byte
// swizzle).  hi*hi goes to columns [0, 128) of the tensor memory, the cross
// terms to [128, 256).
__device__ __forceinline__ void look_mma_block(unsigned tmem, unsigned a_hi,
                                               unsigned a_lo, unsigned b_hi,
                                               unsigned b_lo, bool first) {
  const unsigned idesc = tc_instr_desc(DB);
  const unsigned long long dah = tc_smem_desc(a_hi), dal = tc_smem_desc(a_lo);
  const unsigned long long dbh = tc_smem_desc(b_hi), dbl = tc_smem_desc(b_lo);
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    const unsigned long long adv = (unsigned long long)(kk * 32 >> 4);
    const unsigned acc = (first && kk == 0) ? 0u : 1u;
    tc_mma(tmem + DB, dal + adv, dbh + adv, idesc, acc);
    tc_mma(tmem + DB, dah + adv, dbl + adv, idesc, 1u);
    tc_mma(tmem, dah + adv, dbh + adv, idesc, acc);
  }
}

// The diagonal block of step k has received the updates of all steps before
// k - 1; the update of step k - 1,
//   D = W_kk - L' L'^T,  L' = A' X_pp^T,
// is computed here from A' (block (k, k-1) as it was before step k-1's panel
// solve overwrote it; the updates keep a second copy of it in the inverse's
// output buffer) and X_pp (inverse of the previous diagonal block's factor),
// so that this kernel does not have to wait for the panel solve and panel
// update of step k - 1.  Both products run on the tensor cores (tcgen05,
// split TF32, accumulators in tensor memory).  Result: D in Sa (rows and
// columns below `bs` are meaningful).  256 threads.  Returns false if a
// bounded wait ran out (the status word is set; the caller stores nothing).
__device__ __forceinline__ bool diag_lookahead(const MatInfo& mi, int o, int bs,
                                               float* Sa, unsigned char* stage,
                                               LookControl* ctl) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long ld = mi.d;
  const float* Ap = mi.inv + (long long)o * ld + (o - DB);
  const float* Xp = mi.X + (long long)(o - DB) * ld + (o - DB);
  const float* Wd = mi.W + (long long)o * ld + o;
  const bool vec = (ld & 3) == 0 && (o & 3) == 0 &&
                   ((reinterpret_cast<uintptr_t>(mi.inv) |
                     reinterpret_cast<uintptr_t>(mi.X) |
                     reinterpret_cast<uintptr_t>(mi.W)) & 15) == 0;
  if (tid == 0) {
    mbar_init(&ctl->bar[0], 1);
    mbar_init(&ctl->bar[1], 1);
    mbar_init(&ctl->done, 1);
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile(
        "tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
        ::"r"(smem_u32(&ctl->tmem_base)), "r"(kLookCols)
        : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;"
                 ::: "memory");
  }
  // W_kk into Sa (the update is subtracted from it at the end)
  for (int idx = tid; idx < DB * (DB / 4); idx += 256) {
    const int r = idx >> 5, c = (idx & 31) * 4;
    float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < bs) {
      if (vec && c + 3 < bs) {
        w = *reinterpret_cast<const float4*>(&Wd[r * ld + c]);
      } else {
        if (c < bs) w.x = Wd[r * ld + c];
        if (c + 1 < bs) w.y = Wd[r * ld + c + 1];
        if (c + 2 < bs) w.z = Wd[r * ld + c + 2];
        if (c + 3 < bs) w.w = Wd[r * ld + c + 3];
      }
    }
    *reinterpret_cast<float4*>(&Sa[r * DLD + c]) = w;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem = ctl->tmem_base;
  const unsigned sbase = smem_u32(stage);
  bool ok = true;

  // ---- L' = A' X_pp^T: four operand blocks of 32 k through two stages; the
  // global loads of block kb + 1 are in flight while block kb is split,
  // stored and multiplied
  float4 va[4], vx[4];
  auto load_block = [&](int kb) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = tid + 256 * j, row = c >> 3, col = 32 * kb + 4 * (c & 7);
      va[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (vec) {
        if (row < bs) va[j] = *reinterpret_cast<const float4*>(&Ap[row * ld + col]);
        vx[j] = *reinterpret_cast<const float4*>(&Xp[row * ld + col]);
      } else {
        if (row < bs) {
          va[j].x = Ap[row * ld + col]; va[j].y = Ap[row * ld + col + 1];
          va[j].z = Ap[row * ld + col + 2]; va[j].w = Ap[row * ld + col + 3];
        }
        vx[j].x = Xp[row * ld + col]; vx[j].y = Xp[row * ld + col + 1];
        vx[j].z = Xp[row * ld + col + 2]; vx[j].w = Xp[row * ld + col + 3];
      }
    }
  };
  load_block(0);
#pragma unroll
  for (int kb = 0; kb < 4; ++kb) {
    const int s = kb & 1;
    if (kb >= 2) ok = mbar_wait_status(&ctl->bar[s], 0, &ctl->abort_flag,
                                       &g_diag_status) && ok;
    const unsigned st = sbase + s * kLookStage;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = tid + 256 * j;
      const unsigned off = (unsigned)sw128_chunk_off(c >> 3, c & 7);
      store_split(st + off, st + kLookTile + off, va[j]);
      store_split(st + 2 * kLookTile + off, st + 3 * kLookTile + off, vx[j]);
    }
    if (kb + 1 < 4) load_block(kb + 1);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (tid == 0 && !ctl->abort_flag) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      look_mma_block(tmem, st, st + kLookTile, st + 2 * kLookTile,
                     st + 3 * kLookTile, kb == 0);
      tc_commit(&ctl->bar[s]);
    }
  }
  ok = mbar_wait_status(&ctl->bar[0], 1, &ctl->abort_flag, &g_diag_status) && ok;
  ok = mbar_wait_status(&ctl->bar[1], 1, &ctl->abort_flag, &g_diag_status) && ok;
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

  // ---- L' out of tensor memory, split, into the operand blocks of the second
  // product (A and B are the same matrix: [hi][lo] per 32 k, four blocks)
  const int q = warp & 3, h = warp >> 2;
  const int row = 32 * q + lane;
  ok = __all_sync(0xffffffffu, ok);     // the loads below are warp-wide
  if (ok) {
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      const int c0 = 64 * h + 16 * cc;
      float v[16], w[16];
      tc_ld16(tmem + ((unsigned)(32 * q) << 16) + (unsigned)c0, v);
      tc_ld16(tmem + ((unsigned)(32 * q) << 16) + (unsigned)(DB + c0), w);
      const unsigned blk = sbase + (unsigned)(c0 >> 5) * (2 * kLookTile);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 x = make_float4(v[4 * i] + w[4 * i], v[4 * i + 1] + w[4 * i + 1],
                                     v[4 * i + 2] + w[4 * i + 2],
                                     v[4 * i + 3] + w[4 * i + 3]);
        const unsigned off =
            (unsigned)sw128_chunk_off(row, ((c0 & 31) >> 2) + i);
        store_split(blk + off, blk + kLookTile + off, x);
      }
    }
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  // ---- L' L'^T
  if (tid == 0 && !ctl->abort_flag) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {
      const unsigned blk = sbase + (unsigned)kb * (2 * kLookTile);
      look_mma_block(tmem, blk, blk + kLookTile, blk, blk + kLookTile, kb == 0);
    }
    tc_commit(&ctl->done);
  }
  ok = mbar_wait_status(&ctl->done, 0, &ctl->abort_flag, &g_diag_status) && ok;
  ok = __all_sync(0xffffffffu, ok);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (ok) {
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      const int c0 = 64 * h + 16 * cc;
      float v[16], w[16];
      tc_ld16(tmem + ((unsigned)(32 * q) << 16) + (unsigned)c0, v);
      tc_ld16(tmem + ((unsigned)(32 * q) << 16) + (unsigned)(DB + c0), w);
#pragma unroll
      for (int i = 0; i < 16; ++i) Sa[row * DLD + c0 + i] -= v[i] + w[i];
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                 ::"r"(tmem), "r"(kLookCols)
                 : "memory");
  }
  return ctl->abort_flag == 0;
}

// Factor one diagonal block (<= 128 x 128) of W and invert the resulting
// triangle: W_jj <- L_jj (lower), X_jj <- L_jj^-1 (lower, upper part zero).
// One CTA of 256 threads per matrix that still has a block at `step`; thread
// (br, bc) = (tid / 16, tid % 16) keeps the 8 x 8 block (br, bc) in registers
// (consecutive lanes hold consecutive column blocks, so that rows of W and X
// are read and written as contiguous 32-byte pieces).
// Both sweeps advance by block columns of 8 with two barriers (Cholesky) or
// one (inverse) per block column instead of one per column:
//   Cholesky, block column kb: thread (kb, kb) factors its 8 x 8 block and
//   inverts the small triangle, all in registers; the threads below multiply
//   their blocks by that inverse (panel solve); every remaining block takes
//   a rank-8 update from the panel, read from shared memory.
//   Inverse, block row kb: the threads of block row kb apply the stored 8 x 8
//   inverse to their blocks of the running right-hand side (rows kb of X are
//   then final); the rows below take a rank-8 update.
template <bool LOOK>
__global__ void __launch_bounds__(256)
chol_diag_kernel(const MatInfo* __restrict__ mats, const int* __restrict__ ids,
                 int step, int* __restrict__ info) {
  extern __shared__ __align__(16) float dsm[];
  float (*Lt)[DB + 4] = reinterpret_cast<float (*)[DB + 4]>(dsm);  // L^T
  float (*Pt)[DB] = reinterpret_cast<float (*)[DB]>(dsm + DB * (DB + 4));
  float (*Xr)[8][DB] =
      reinterpret_cast<float (*)[8][DB]>(dsm + DB * (DB + 4) + 8 * DB);
  float (*Tk)[64] =
      reinterpret_cast<float (*)[64]>(dsm + DB * (DB + 4) + 24 * DB);
  const int id = ids[blockIdx.x];
  const MatInfo mi = mats[id];
  const int tid = threadIdx.x, br = tid >> 4, bc = tid & 15;
  const int o = step * DB;
  const int bs = min(DB, mi.d - o);
  const int nkb = (bs + 7) >> 3;
  const long long ld = mi.d;
  float* Wd = mi.W + (long long)o * ld + o;
  float* Xd = mi.X + (long long)o * ld + o;

  // blocks strictly below the diagonal move as two 16-byte pieces per row
  const bool vec = (ld & 3) == 0 && (o & 3) == 0 &&
                   ((reinterpret_cast<uintptr_t>(mi.W) |
                     reinterpret_cast<uintptr_t>(mi.X)) & 15) == 0;
  float a[8][8];
  if (LOOK) {
    // the block with step - 1's update applied comes out of the look-ahead
    // in shared memory (aliasing Lt, which is written only after the
    // Cholesky sweep's barriers)
    float* Sa = dsm;
    unsigned char* stage = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(dsm + kDiagBaseFloats) + 1023) &
        ~(uintptr_t)1023);
    LookControl* ctl = reinterpret_cast<LookControl*>(stage + 2 * kLookStage);
    if (!diag_lookahead(mi, o, bs, Sa, stage, ctl)) return;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int gi = 8 * br + i;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int gj = 8 * bc + j;
        float v = (gi == gj) ? 1.f : 0.f;
        if (gi < bs && gj <= gi) v = Sa[gi * DLD + gj];
        a[i][j] = v;
      }
    }
    __syncthreads();
  } else
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gi = 8 * br + i;
    if (vec && bc < br && gi < bs) {
      const float4 v0 = *reinterpret_cast<const float4*>(&Wd[gi * ld + 8 * bc]);
      const float4 v1 = *reinterpret_cast<const float4*>(&Wd[gi * ld + 8 * bc + 4]);
      a[i][0] = v0.x; a[i][1] = v0.y; a[i][2] = v0.z; a[i][3] = v0.w;
      a[i][4] = v1.x; a[i][5] = v1.y; a[i][6] = v1.z; a[i][7] = v1.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int gj = 8 * bc + j;
        float v = (gi == gj) ? 1.f : 0.f;        // identity beyond the block
        if (gi < bs && gj <= gi) v = Wd[gi * ld + gj];
        a[i][j] = v;
      }
    }
  }

  // ---- Cholesky by block columns
  for (int kb = 0; kb < nkb; ++kb) {
    if (br == kb && bc == kb) {
      // 8 x 8 Cholesky in registers; rl[c] = 1 / l_cc
      float rl[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float piv = a[c][c];
        if (!(piv > 0.f)) {
          atomicCAS(&info[id], 0, o + 8 * kb + c + 1);
          piv = 1.f;
        }
        // rsqrt + one Newton step: full fp32 accuracy without the slow IEEE
        // square root and division
        float r = rsqrtf(piv);
        r = r * (1.5f - 0.5f * piv * r * r);
        rl[c] = r;
        a[c][c] = piv * r;
#pragma unroll
        for (int i = c + 1; i < 8; ++i) a[i][c] *= r;
#pragma unroll
        for (int j = c + 1; j < 8; ++j)
#pragma unroll
          for (int i = j; i < 8; ++i) a[i][j] = fmaf(-a[i][c], a[j][c], a[i][j]);
      }
      // T = L_kk^-1 (lower), column by column: T[c][c] = rl[c],
      // T[i][c] = -rl[i] * sum_{m=c}^{i-1} L[i][m] T[m][c]
      float t[8][8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        t[c][c] = rl[c];
#pragma unroll
        for (int i = c + 1; i < 8; ++i) {
          float acc = 0.f;
#pragma unroll
          for (int m = c; m < i; ++m) acc = fmaf(a[i][m], t[m][c], acc);
          t[i][c] = -rl[i] * acc;
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) Tk[kb][8 * i + j] = (j <= i) ? t[i][j] : 0.f;
    }
    __syncthreads();
    if (bc == kb && br > kb) {
      // panel solve: L_blk = A_blk T^T, L[i][c] = sum_{m<=c} A[i][m] T[c][m]
      float t[8][8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 t0 = *reinterpret_cast<const float4*>(&Tk[kb][8 * i]);
        const float4 t1 = *reinterpret_cast<const float4*>(&Tk[kb][8 * i + 4]);
        t[i][0] = t0.x; t[i][1] = t0.y; t[i][2] = t0.z; t[i][3] = t0.w;
        t[i][4] = t1.x; t[i][5] = t1.y; t[i][6] = t1.z; t[i][7] = t1.w;
      }
      float l[8][8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float acc = 0.f;
#pragma unroll
          for (int m = 0; m <= c; ++m) acc = fmaf(a[i][m], t[c][m], acc);
          l[i][c] = acc;
        }
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        *reinterpret_cast<float4*>(&Pt[c][8 * br]) =
            make_float4(l[0][c], l[1][c], l[2][c], l[3][c]);
        *reinterpret_cast<float4*>(&Pt[c][8 * br + 4]) =
            make_float4(l[4][c], l[5][c], l[6][c], l[7][c]);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i][c] = l[i][c];
      }
    }
    __syncthreads();
    if (bc > kb && bc <= br) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float4 r0 = *reinterpret_cast<const float4*>(&Pt[c][8 * br]);
        const float4 r1 = *reinterpret_cast<const float4*>(&Pt[c][8 * br + 4]);
        const float4 c0 = *reinterpret_cast<const float4*>(&Pt[c][8 * bc]);
        const float4 c1 = *reinterpret_cast<const float4*>(&Pt[c][8 * bc + 4]);
        const float pr[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
        const float pc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int j = 0; j < 8; ++j) a[i][j] = fmaf(-pr[i], pc[j], a[i][j]);
      }
    }
  }

  // ---- L to global memory (lower part) and, transposed, to shared memory
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gi = 8 * br + i;
    if (vec && bc < br && gi < bs) {
      *reinterpret_cast<float4*>(&Wd[gi * ld + 8 * bc]) =
          make_float4(a[i][0], a[i][1], a[i][2], a[i][3]);
      *reinterpret_cast<float4*>(&Wd[gi * ld + 8 * bc + 4]) =
          make_float4(a[i][4], a[i][5], a[i][6], a[i][7]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int gj = 8 * bc + j;
        if (gi < bs && gj <= gi) Wd[gi * ld + gj] = a[i][j];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int gj = 8 * bc + j;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (8 * br + i > gj) ? a[i][j] : 0.f;
    *reinterpret_cast<float4*>(&Lt[gj][8 * br]) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(&Lt[gj][8 * br + 4]) = make_float4(v[4], v[5], v[6], v[7]);
  }
  // ---- inverse of the triangle by block rows: R starts as I; the rows of
  // block kb become X = T_kb R, every block row below subtracts L_blk X
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) a[i][j] = (8 * br + i == 8 * bc + j) ? 1.f : 0.f;
  __syncthreads();
  for (int kb = 0; kb < nkb; ++kb) {
    const int buf = kb & 1;
    if (br == kb && bc <= kb) {
      float t[8][8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 t0 = *reinterpret_cast<const float4*>(&Tk[kb][8 * i]);
        const float4 t1 = *reinterpret_cast<const float4*>(&Tk[kb][8 * i + 4]);
        t[i][0] = t0.x; t[i][1] = t0.y; t[i][2] = t0.z; t[i][3] = t0.w;
        t[i][4] = t1.x; t[i][5] = t1.y; t[i][6] = t1.z; t[i][7] = t1.w;
      }
      float x[8][8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float acc = 0.f;
#pragma unroll
          for (int m = 0; m <= i; ++m) acc = fmaf(t[i][m], a[m][j], acc);
          x[i][j] = acc;
        }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        *reinterpret_cast<float4*>(&Xr[buf][i][8 * bc]) =
            make_float4(x[i][0], x[i][1], x[i][2], x[i][3]);
        *reinterpret_cast<float4*>(&Xr[buf][i][8 * bc + 4]) =
            make_float4(x[i][4], x[i][5], x[i][6], x[i][7]);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[i][j] = x[i][j];
      }
    }
    __syncthreads();
    if (br > kb && bc <= kb) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float4 l0 = *reinterpret_cast<const float4*>(&Lt[8 * kb + c][8 * br]);
        const float4 l1 = *reinterpret_cast<const float4*>(&Lt[8 * kb + c][8 * br + 4]);
        const float4 x0 = *reinterpret_cast<const float4*>(&Xr[buf][c][8 * bc]);
        const float4 x1 = *reinterpret_cast<const float4*>(&Xr[buf][c][8 * bc + 4]);
        const float lc[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
        const float xr[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int j = 0; j < 8; ++j) a[i][j] = fmaf(-lc[i], xr[j], a[i][j]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gi = 8 * br + i;
    if (vec && bc != br && gi < bs && 8 * bc + 7 < bs) {
      const bool low = bc < br;
      *reinterpret_cast<float4*>(&Xd[gi * ld + 8 * bc]) =
          low ? make_float4(a[i][0], a[i][1], a[i][2], a[i][3])
              : make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4*>(&Xd[gi * ld + 8 * bc + 4]) =
          low ? make_float4(a[i][4], a[i][5], a[i][6], a[i][7])
              : make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int gj = 8 * bc + j;
        if (gi < bs && gj < bs) Xd[gi * ld + gj] = (gj <= gi) ? a[i][j] : 0.f;
      }
    }
  }
}


// ---------------------------------------------------------------- refinement
// One step of iterative refinement for factors whose fp32 inverse is visibly
// off (ill-conditioned factors: the error of any fp32 inverse grows with the
// condition number).  With R = I - (F + add I) X accumulated in fp64 from the
// fp32 data, X <- X + X R has the error of X squared (times the condition
// number), so one step is enough.  Whether a factor needs the step is decided
// on the device from a probe: for a fixed +-1 vector v,
//   t = X v,  r = v - (F + add I) t,  e = X r   (fp64 accumulation)
// e estimates (X - A^-1) v, so |e| / |t| estimates the relative error of X;
// the step runs when that exceeds `threshold` and d <= `max_dim`.
constexpr int kRefineDimCap = 1024;   // workspace is reserved up to this size

struct RefineItem {
  int mat;          // index into the plan's matrices
  int d;
  int tile_begin;   // first 64 x 64 tile of this matrix in the residual grid
  int pad_;
  float* Y;         // d x d scratch for X R
  double* vec;      // 2 d doubles: t, r
};

__device__ __forceinline__ float probe_sign(int i) {
  unsigned h = (unsigned)i * 2654435761u;
  h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
  return (h & 1u) ? 1.f : -1.f;
}

__device__ __forceinline__ float damp_of_row(const MatInfo& mi, float add,
                                             float add2, int row) {
  return (mi.role == 2 && 2 * row >= mi.d) ? add2 : add;
}

// stage 0: t = X v; stage 1: r = v - (F + add I) t; stage 2: e = X r and
// sums[item] += (|e|^2, |t|^2).  One warp per row, blockIdx.y = item.
__global__ void __launch_bounds__(256)
refine_probe_kernel(const MatInfo* __restrict__ mats,
                    const RefineItem* __restrict__ items,
                    const float* __restrict__ add,
                    const float* __restrict__ add2, double* __restrict__ sums,
                    const RunParams* __restrict__ prm, int stage) {
  if (prm->refine_max_dim <= 0) return;
  const RefineItem it = items[blockIdx.y];
  const MatInfo mi = mats[it.mat];
  const int d = it.d;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (stage == 1 && blockIdx.x == 0 && threadIdx.x == 0) {
    sums[2 * blockIdx.y] = 0.0;
    sums[2 * blockIdx.y + 1] = 0.0;
  }
  if (row >= d) return;
  double* t = it.vec;
  double* r = it.vec + d;
  const float* mrow = (stage == 1 ? mi.F : mi.inv) + (long long)row * d;
  double s = 0.0;
  if (stage == 0) {
    for (int c = lane; c < d; c += 32) s += (double)mrow[c] * probe_sign(c);
  } else {
    const double* x = stage == 1 ? t : r;
    for (int c = lane; c < d; c += 32) s += (double)mrow[c] * x[c];
  }
  for (int o = 16; o > 0; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
  if (lane != 0) return;
  if (stage == 0) {
    t[row] = s;
  } else if (stage == 1) {
    const float a = damp_of_row(mi, add[it.mat], add2[it.mat], row);
    r[row] = (double)probe_sign(row) - (s + (double)a * t[row]);
  } else {
    atomicAdd(&sums[2 * blockIdx.y], s * s);
    atomicAdd(&sums[2 * blockIdx.y + 1], t[row] * t[row]);
  }
}

__global__ void refine_gate_kernel(const RefineItem* __restrict__ items, int n,
                                   const double* __restrict__ sums,
                                   const RunParams* __restrict__ prm,
                                   int* __restrict__ gate,
                                   int* __restrict__ refined_count) {
  const int max_dim = prm->refine_max_dim;
  const float threshold = prm->refine_threshold;
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) *refined_count = 0;
  __syncthreads();
  if (i >= n) return;
  const double e2 = sums[2 * i], t2 = sums[2 * i + 1];
  const double thr = (double)threshold;
  // a NaN estimate (broken factorisation) is left alone: info reports it
  const int on = items[i].d <= max_dim && e2 > thr * thr * t2;
  gate[i] = on;
  if (on) atomicAdd(refined_count, 1);
}

// R = I - (F + add I) X for a 64 x 64 tile, fp64 accumulation, R stored as
// fp32 into the matrix's W scratch.  256 threads, 4 x 4 outputs each.
__global__ void __launch_bounds__(256)
refine_residual_kernel(const MatInfo* __restrict__ mats,
                       const RefineItem* __restrict__ items, int nitems,
                       const float* __restrict__ add,
                       const float* __restrict__ add2,
                       const int* __restrict__ gate) {
  __shared__ double As[16][64 + 2];   // As[k][i] = A[i0 + i][k0 + k]
  __shared__ double Bs[16][64 + 2];   // Bs[k][j] = X[k0 + k][j0 + j]
  __shared__ int s_item;
  const int tid = threadIdx.x;
  if (tid == 0) {
    int lo = 0, hi = nitems - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (items[mid].tile_begin <= (int)blockIdx.x) lo = mid; else hi = mid - 1;
    }
    s_item = lo;
  }
  __syncthreads();
  const int item = s_item;
  if (gate[item] == 0) return;
  const RefineItem it = items[item];
  const MatInfo mi = mats[it.mat];
  const int d = it.d;
  const int nt = (d + 63) >> 6;
  const int lt = blockIdx.x - it.tile_begin;
  const int i0 = (lt / nt) * 64, j0 = (lt % nt) * 64;
  const float a1 = add[it.mat], a2 = add2[it.mat];
  const int ty = tid >> 4, tx = tid & 15;
  double acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0;
  // loaders: A tile 64 rows x 16 k (thread: row tid / 4, k 4 (tid % 4) ..+3);
  // X tile 16 k x 64 cols (thread: k tid / 16, cols 4 (tid % 16) ..+3)
  const int ar = tid >> 2, ak = (tid & 3) * 4;
  const int bk = tid >> 4, bc = (tid & 15) * 4;
  for (int k0 = 0; k0 < d; k0 += 16) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int gi = i0 + ar, gk = k0 + ak + q;
      double v = 0.0;
      if (gi < d && gk < d) {
        v = (double)mi.F[(long long)gi * d + gk];
        if (gi == gk) v += (double)damp_of_row(mi, a1, a2, gi);
      }
      As[ak + q][ar] = v;
      const int gk2 = k0 + bk, gj = j0 + bc + q;
      Bs[bk][bc + q] =
          (gk2 < d && gj < d) ? (double)mi.inv[(long long)gk2 * d + gj] : 0.0;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      double a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fma(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gi = i0 + ty * 4 + i;
    if (gi >= d) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gj = j0 + tx * 4 + j;
      if (gj < d)
        mi.W[(long long)gi * d + gj] =
            (float)((gi == gj ? 1.0 : 0.0) - acc[i][j]);
    }
  }
}

// inv += Y for the refined matrices; blockIdx.y = item.
__global__ void __launch_bounds__(256)
refine_apply_kernel(const MatInfo* __restrict__ mats,
                    const RefineItem* __restrict__ items,
                    const int* __restrict__ gate) {
  if (gate[blockIdx.y] == 0) return;
  const RefineItem it = items[blockIdx.y];
  float* inv = mats[it.mat].inv;
  const long long n = (long long)it.d * it.d;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    inv[i] += it.Y[i];
}

constexpr size_t kDiagSmemBytes =
    kDiagBaseFloats * sizeof(float);                        // Lt, Pt, Xr, Tk
constexpr size_t kDiagLookSmemBytes =
    kDiagBaseFloats * sizeof(float) + 1024 + 2 * kLookStage + 256;
static_assert(kDiagLookSmemBytes <= 227 * 1024, "diagonal kernel shared memory");

struct Launch {
  int tails;     // grouped gemm: some contraction is not a multiple of 32
  int kind;      // 0 diag kernel, 1 grouped gemm, 2 join of the side stream
  int off;       // offset into ids / descs
  int n;         // number of ids / descs
  int tiles;     // grouped gemm: total tiles
  int step;      // diag kernel: panel index
  // A run uses two streams: the chain (0) and a side stream (1) for work
  // that is off the critical path.  A launch may wait for an event first and
  // record one afterwards (indices into the plan's events, -1: none).
  int stream;
  int wait_ev;
  int rec_ev;
  int wait_ev2;
  bool look;     // diag kernel: with the look-ahead prologue
};

// Status word of the diagonal kernel's bounded waits (read by kfac_tc_status).
int diag_status_read(int* out) {
  KFAC_CUDA(cudaMemcpyFromSymbol(out, g_diag_status, sizeof(int)));
  return KFAC_OK;
}

}  // namespace kfac

using namespace kfac;

struct kfac_inverse_plan {
  int count;
  int device;
  MatInfo* mats_dev;
  float* trace_dev;
  float* add_dev;
  int* info_dev;
  int* ids_dev;
  GemmDesc* descs_dev;
  std::vector<Launch> launches;
  long long total_elems;
  bool use_tc;
  // refinement (see refine_* kernels)
  float* add2_dev;
  int n_refine;
  int refine_dmax;
  int refine_tiles;
  Launch refine_prod;
  RefineItem* refine_items_dev;
  double* refine_sums_dev;
  double* refine_vec_dev;
  int* refine_gate_dev;
  int* refine_count_dev;
  int refine_max_dim;
  float refine_threshold;
  // CUDA graph of one run (captured on first use)
  RunParams* params_dev;
  std::vector<cudaEvent_t> events;   // edges between the two streams
  cudaEvent_t fork_ev, join_ev[2];
  cudaStream_t side_stream[2];       // bulk / far stream of plain runs
  cudaStream_t cap_side[2];          // the same during capture
  bool look;
  cudaStream_t cap_stream;
  cudaGraphExec_t graph_exec;
  int* graph_info;
  float* graph_diag;
  long long graph_launches;
  bool graph_ok;
};

static size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

extern "C" size_t kfac_inverse_workspace_bytes(int count, const int* dims) {
  size_t total = 0;
  for (int i = 0; i < count; ++i) {
    if (dims[i] <= 0) return 0;
    const size_t bytes = align256((size_t)dims[i] * dims[i] * sizeof(float));
    total += 2 * bytes;                              // W, X
    if (dims[i] <= kRefineDimCap) total += bytes;    // Y of the refinement
  }
  return total;
}

extern "C" int kfac_inverse_plan_create(
    int count, const int* dims, const float* const* factors,
    float* const* inverses, const int* partner, const int* role,
    const float* l2_coef, const float* scale, void* workspace,
    size_t workspace_bytes, kfac_inverse_plan** out) {
  KFAC_REQUIRE(out != nullptr, "inverse_plan_create: null plan pointer");
  *out = nullptr;
  KFAC_REQUIRE(count > 0 && dims && factors && inverses && role,
               "inverse_plan_create: null argument or count=%d", count);
  for (int i = 0; i < count; ++i) {
    KFAC_REQUIRE(dims[i] > 0 && dims[i] <= 32768,
                 "inverse_plan_create: dims[%d]=%d out of range", i, dims[i]);
    KFAC_REQUIRE(factors[i] && inverses[i],
                 "inverse_plan_create: null matrix pointer at %d", i);
    KFAC_REQUIRE(role[i] >= 0 && role[i] <= 2,
                 "inverse_plan_create: role[%d]=%d", i, role[i]);
    if (role[i] != 2 && partner && partner[i] >= 0)
      KFAC_REQUIRE(partner[i] < count && role[partner[i]] == 1 - role[i],
                   "inverse_plan_create: partner[%d]=%d is not the other "
                   "factor of a pair", i, partner[i]);
  }
  size_t need = kfac_inverse_workspace_bytes(count, dims);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(KFAC_ERR_WORKSPACE,
                "inverse_plan_create: workspace of %zu bytes needed, %zu given",
                need, workspace_bytes);

  // Blocks of X above the diagonal blocks are never written and are read as
  // zeros by the wide tiles of the triangular-inverse products.
  KFAC_CUDA(cudaMemset(workspace, 0, need));
  std::vector<MatInfo> mats(count);
  std::vector<float*> ybuf(count, nullptr);
  char* ws = static_cast<char*>(workspace);
  int dmax = 0;
  long long total_elems = 0;
  for (int i = 0; i < count; ++i) {
    MatInfo& m = mats[i];
    size_t bytes = align256((size_t)dims[i] * dims[i] * sizeof(float));
    m.F = factors[i];
    m.inv = inverses[i];
    m.W = reinterpret_cast<float*>(ws); ws += bytes;
    m.X = reinterpret_cast<float*>(ws); ws += bytes;
    if (dims[i] <= kRefineDimCap) {
      ybuf[i] = reinterpret_cast<float*>(ws); ws += bytes;
    }
    m.d = dims[i];
    m.partner = partner ? partner[i] : -1;
    m.role = role[i];
    m.l2 = l2_coef ? l2_coef[i] : 0.f;
    m.scale = scale ? scale[i] : 1.f;
    m.l2b = m.l2;
    dmax = std::max(dmax, dims[i]);
    total_elems += (long long)dims[i] * dims[i];
  }
  // large matrices first: their tiles are scheduled first
  std::vector<int> order(count);
  for (int i = 0; i < count; ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(),
                   [&](int a, int b) { return dims[a] > dims[b]; });

  std::vector<GemmDesc> descs;
  std::vector<int> ids;
  std::vector<Launch> launches;
  const bool use_tc = engine() == 1;

  int n_events = 0;
  const bool look = use_tc && [] {
    const char* env = getenv("KFAC_INVERSE_LOOKAHEAD");
    return !(env && env[0] == '0');
  }();
  std::vector<int> diag_ev((dmax + DB - 1) / DB + 1, -1);
  std::vector<int> upd_ev((dmax + DB - 1) / DB + 1, -1);
  auto begin_gemm = [&]() {
    Launch l = {0, 1, (int)descs.size(), 0, 0, 0, 0, -1, -1, -1, false};
    return l;
  };
  auto push_desc = [&](Launch& l, GemmDesc g) {
    g.tile_begin = l.tiles;
    l.tiles += use_tc ? tc_tiles(g) : gemm_desc_tiles(g);
    if (tc_desc_has_tails(g)) l.tails = 1;
    g.kfW = g.kfb = g.pW = g.pb = g.vW = g.vb = nullptr;
    g.dW = 0;
    g.splits = 1;
    g.ntiles = 0;
    g.k_per_split = 0;
    g.partial = nullptr;
    descs.push_back(g);
    l.n += 1;
  };
  auto end_gemm = [&](Launch& l) {
    if (l.n > 0) launches.push_back(l);
  };

  int prev_far_ev = -1;
  // Two-level right-looking Cholesky: panels of PW columns are factored by
  // 128-wide inner steps whose updates stay inside the panel (short
  // contractions, little work); the bulk of the flops is the update of the
  // trailing matrix with the whole panel (contraction length PW).
  //
  // With look-ahead (default) a run uses three streams.  The chain (0)
  // carries the diagonal kernels; inside a panel the diagonal kernel of step
  // k applies step k-1's update to its own block itself (diag_lookahead), so
  // it only waits for the panel update of step k-2.  The panel solves and
  // panel updates of the steps run on the bulk stream (1) behind the chain,
  // and the part of a panel's trailing update that the next panel does not
  // need runs on the far stream (2).  Panel updates (and the near part of a
  // trailing update, and the damped copy for the first block column) store
  // their results a second time in the inverse's output buffer: that copy of
  // block (k, k-1) is what diag_lookahead reads while the panel solve of
  // step k-1 overwrites the original.
  for (int po = 0; po < dmax; po += PW) {
    const int inner = std::min(PW, dmax - po);
    int last_solve_ev = -1;
    for (int o = po; o < po + inner; o += DB) {
      const bool lk = look && o > po;
      Launch dl = {0, 0, (int)ids.size(), 0, 0, o / DB, 0, -1, -1, -1, lk};
      for (int i : order)
        if (dims[i] > o) { ids.push_back(i); dl.n += 1; }
      if (lk && o - 2 * DB >= po) dl.wait_ev = upd_ev[(o - 2 * DB) / DB];
      if (look) dl.rec_ev = diag_ev[o / DB] = n_events++;
      launches.push_back(dl);

      Launch trsm = begin_gemm();
      for (int i : order) {
        const int d = dims[i];
        const int M = d - o - DB;
        if (M <= 0) continue;
        const MatInfo& m = mats[i];
        GemmDesc g = {};
        float* panel = m.W + (long long)(o + DB) * d + o;
        g.A = strided_operand(panel, 1, d, M);
        g.B = strided_operand(m.X + (long long)o * d + o, 1, d, DB);
        g.C = panel; g.ldc = d; g.M = M; g.N = DB; g.K = DB;
        g.alpha = 1.f; g.beta = 0.f; g.flags = 0;
        push_desc(trsm, g);
      }
      if (look && trsm.n > 0) {
        trsm.stream = 1;
        trsm.wait_ev = diag_ev[o / DB];
        trsm.rec_ev = last_solve_ev = n_events++;
      }
      end_gemm(trsm);

      // update the rest of this panel's columns (full rectangle; entries
      // above the diagonal are written but never read).  With look-ahead the
      // next diagonal block is left to the next diagonal kernel.
      const int skip = (look && o + DB < po + inner) ? DB : 0;
      Launch upd = begin_gemm();
      for (int i : order) {
        const int d = dims[i];
        const int M = d - o - DB - skip;
        const int N = std::min(po + PW, d) - (o + DB);
        if (M <= 0 || N <= 0) continue;
        const MatInfo& m = mats[i];
        GemmDesc g = {};
        float* panel = m.W + (long long)(o + DB + skip) * d + o;
        const long long coff = (long long)(o + DB + skip) * d + (o + DB);
        g.A = strided_operand(panel, 1, d, M);
        g.B = strided_operand(m.W + (long long)(o + DB) * d + o, 1, d, N);
        g.C = m.W + coff;
        g.ldc = d; g.M = M; g.N = N; g.K = DB;
        g.alpha = -1.f; g.beta = 1.f; g.flags = 0;
        if (look) g.C2 = m.inv + coff;
        push_desc(upd, g);
      }
      if (look) {
        upd.stream = 1;
        if (upd.n > 0) upd.rec_ev = upd_ev[o / DB] = n_events++;
      }
      end_gemm(upd);
    }

    // Update of the trailing matrix with the finished panel, in two parts:
    // the columns of the next panel (needed before the chain can go on) on
    // the chain's stream, the columns beyond them on the far stream, next to
    // the next panel's chain.  Both parts of one panel touch disjoint tiles;
    // parts of successive panels that touch the same tiles are ordered by
    // events (next-panel part p+1 after far part p) or by stream order.
    Launch near = begin_gemm(), far = begin_gemm();
    std::vector<GemmDesc> far_descs;
    for (int i : order) {
      const int d = dims[i];
      const int M = d - po - PW;
      if (M <= 0) continue;
      const int N1 = std::min(PW, M);
      const MatInfo& m = mats[i];
      const float* panel = m.W + (long long)(po + PW) * d + po;
      {
        GemmDesc g = {};     // square block on the diagonal: lower tiles
        const long long coff = (long long)(po + PW) * d + (po + PW);
        g.A = strided_operand(panel, 1, d, N1);
        g.B = g.A;
        g.C = m.W + coff;
        g.ldc = d; g.M = N1; g.N = N1; g.K = PW;
        g.alpha = -1.f; g.beta = 1.f; g.flags = G_LOWER | G_SAME_AB;
        if (look) g.C2 = m.inv + coff;
        push_desc(near, g);
      }
      if (M > N1) {
        const float* below = panel + (long long)N1 * d;
        GemmDesc g = {};     // rectangle below it
        const long long coff = (long long)(po + PW + N1) * d + (po + PW);
        g.A = strided_operand(below, 1, d, M - N1);
        g.B = strided_operand(panel, 1, d, N1);
        g.C = m.W + coff;
        g.ldc = d; g.M = M - N1; g.N = N1; g.K = PW;
        g.alpha = -1.f; g.beta = 1.f; g.flags = 0;
        if (look) g.C2 = m.inv + coff;
        push_desc(near, g);
        GemmDesc h = {};     // everything beyond the next panel's columns
        h.A = strided_operand(below, 1, d, M - N1);
        h.B = h.A;
        h.C = m.W + (long long)(po + PW + N1) * d + (po + PW + N1);
        h.ldc = d; h.M = M - N1; h.N = M - N1; h.K = PW;
        h.alpha = -1.f; h.beta = 1.f; h.flags = G_LOWER | G_SAME_AB;
        far_descs.push_back(h);
      }
    }
    far.off = (int)descs.size();
    for (auto& h : far_descs) push_desc(far, h);
    int panel_ev = look ? last_solve_ev : -1;
    if (!look && far.n > 0) {
      // the far part needs the finished panel: an event recorded on the
      // chain right before the near part
      panel_ev = n_events++;
      launches.back().rec_ev = panel_ev;   // last launch of the panel's chain
    }
    if (near.n > 0) {
      near.wait_ev = prev_far_ev;          // far part of the previous panel
      near.wait_ev2 = look ? panel_ev : -1;  // the bulk stream's last solve
      prev_far_ev = -1;
    }
    if (far.n > 0) {
      far.stream = 2;
      far.wait_ev = panel_ev;
      far.rec_ev = n_events++;
      prev_far_ev = far.rec_ev;
    }
    end_gemm(near);
    end_gemm(far);
  }
  {
    // the triangular inverse reads all of L: join the side stream
    Launch join = {0, 2, 0, 0, 0, 0, 0, -1, -1, -1, false};
    launches.push_back(join);
  }

  for (long long b = DB; b < dmax; b *= 2) {
    Launch g1 = begin_gemm(), g2 = begin_gemm();
    std::vector<GemmDesc> second;
    for (int i : order) {
      const int d = dims[i];
      if (d <= b) continue;
      const MatInfo& m = mats[i];
      for (long long s = 0; s + b < d; s += 2 * b) {
        const int r = (int)std::min<long long>(b, d - s - b);
        GemmDesc g = {};
        // T = L21 * X11, parked in the output matrix
        g.A = strided_operand(m.W + (s + b) * d + s, 1, d, r);
        g.B = strided_operand(m.X + s * d + s, d, 1, (int)b);
        g.C = m.inv + (s + b) * d + s;
        g.ldc = d; g.M = r; g.N = (int)b; g.K = b;
        g.alpha = 1.f; g.beta = 0.f; g.flags = G_KBEG_N0;
        push_desc(g1, g);
        // X21 = -X22 * T
        GemmDesc h = {};
        h.A = strided_operand(m.X + (s + b) * d + s + b, 1, d, r);
        h.B = strided_operand(m.inv + (s + b) * d + s, d, 1, (int)b);
        h.C = m.X + (s + b) * d + s;
        h.ldc = d; h.M = r; h.N = (int)b; h.K = r;
        h.alpha = -1.f; h.beta = 0.f; h.flags = G_KEND_M0;
        second.push_back(h);
      }
    }
    end_gemm(g1);
    g2.off = (int)descs.size();
    for (auto& h : second) push_desc(g2, h);
    end_gemm(g2);
  }

  {
    Launch prod = begin_gemm();
    for (int i : order) {
      const int d = dims[i];
      const MatInfo& m = mats[i];
      GemmDesc g = {};
      g.A = strided_operand(m.X, d, 1, d);
      g.B = g.A;
      g.C = m.inv; g.ldc = d; g.M = d; g.N = d; g.K = d;
      g.alpha = 1.f; g.beta = 0.f;
      g.flags = G_LOWER | G_MIRROR | G_KBEG_M0 | G_SAME_AB;
      push_desc(prod, g);
    }
    end_gemm(prod);
  }

  // refinement of the matrices of up to kRefineDimCap rows: Y = X R on the
  // tile engine (Y is symmetric: lower tiles, mirrored), gated per matrix
  std::vector<RefineItem> ritems;
  int refine_tiles = 0, refine_dmax = 0;
  long long vec_elems = 0;
  for (int i : order) {
    if (dims[i] > kRefineDimCap) continue;
    RefineItem it;
    it.mat = i;
    it.d = dims[i];
    it.tile_begin = refine_tiles;
    it.pad_ = 0;
    it.Y = ybuf[i];
    it.vec = reinterpret_cast<double*>(vec_elems);   // offset, fixed up below
    const int nt = (dims[i] + 63) / 64;
    refine_tiles += nt * nt;
    refine_dmax = std::max(refine_dmax, dims[i]);
    vec_elems += 2LL * dims[i];
    ritems.push_back(it);
  }
  Launch refine_prod = begin_gemm();

  kfac_inverse_plan* p = new kfac_inverse_plan();
  p->count = count;
  p->total_elems = total_elems;
  p->launches = launches;
  p->use_tc = use_tc;
  p->mats_dev = nullptr; p->trace_dev = nullptr; p->add_dev = nullptr;
  p->info_dev = nullptr; p->ids_dev = nullptr; p->descs_dev = nullptr;
  p->add2_dev = nullptr; p->refine_items_dev = nullptr;
  p->refine_sums_dev = nullptr; p->refine_vec_dev = nullptr;
  p->refine_gate_dev = nullptr; p->refine_count_dev = nullptr;
  p->n_refine = (int)ritems.size();
  p->refine_dmax = refine_dmax;
  p->refine_tiles = refine_tiles;
  p->refine_max_dim = kRefineDimCap;
  p->refine_threshold = 3e-5f;
  p->params_dev = nullptr;
  p->fork_ev = p->join_ev[0] = p->join_ev[1] = nullptr;
  p->side_stream[0] = p->side_stream[1] = nullptr;
  p->cap_side[0] = p->cap_side[1] = nullptr;
  p->look = look;
  p->cap_stream = nullptr;
  p->graph_exec = nullptr;
  p->graph_info = nullptr;
  p->graph_diag = nullptr;
  p->graph_launches = 0;
  {
    const char* env = getenv("KFAC_INVERSE_GRAPH");
    p->graph_ok = !(env && env[0] == '0');
  }
  cudaError_t e = cudaGetDevice(&p->device);
  if (e == cudaSuccess) e = cudaMalloc(&p->params_dev, sizeof(RunParams));
  // the chain is latency-bound and uses few SMs: it gets the higher
  // priority, the side stream's tiles fill the rest
  int prio_lo = 0, prio_hi = 0;
  if (e == cudaSuccess) e = cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi);
  if (e == cudaSuccess)
    e = cudaStreamCreateWithPriority(&p->cap_stream, cudaStreamNonBlocking,
                                     prio_hi);
  for (int k = 0; k < 2 && e == cudaSuccess; ++k) {
    e = cudaStreamCreateWithPriority(&p->cap_side[k], cudaStreamNonBlocking,
                                     prio_lo);
    if (e == cudaSuccess)
      e = cudaStreamCreateWithPriority(&p->side_stream[k],
                                       cudaStreamNonBlocking, prio_lo);
  }
  if (e == cudaSuccess)
    e = cudaEventCreateWithFlags(&p->fork_ev, cudaEventDisableTiming);
  for (int k = 0; k < 2 && e == cudaSuccess; ++k)
    e = cudaEventCreateWithFlags(&p->join_ev[k], cudaEventDisableTiming);
  for (int k = 0; k < n_events + 1 && e == cudaSuccess; ++k) {
    cudaEvent_t ev = nullptr;
    e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    if (e == cudaSuccess) p->events.push_back(ev);
  }
  if (e == cudaSuccess) e = cudaMalloc(&p->add2_dev, sizeof(float) * count);
  if (e == cudaSuccess) e = cudaMalloc(&p->refine_count_dev, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(p->refine_count_dev, 0, sizeof(int));
  if (e == cudaSuccess && !ritems.empty()) {
    const size_t nr = ritems.size();
    e = cudaMalloc(&p->refine_items_dev, sizeof(RefineItem) * nr);
    if (e == cudaSuccess) e = cudaMalloc(&p->refine_sums_dev, sizeof(double) * 2 * nr);
    if (e == cudaSuccess) e = cudaMalloc(&p->refine_vec_dev, sizeof(double) * vec_elems);
    if (e == cudaSuccess) e = cudaMalloc(&p->refine_gate_dev, sizeof(int) * nr);
    if (e == cudaSuccess) {
      for (size_t r = 0; r < nr; ++r) {
        RefineItem& it = ritems[r];
        it.vec = p->refine_vec_dev + reinterpret_cast<long long>(it.vec);
        const int d = it.d;
        const MatInfo& m = mats[it.mat];
        GemmDesc g = {};
        g.A = strided_operand(m.inv, 1, d, d);     // A(k, m) = X[m][k]
        g.B = strided_operand(m.W, d, 1, d);       // B(k, n) = R[k][n]
        g.C = it.Y; g.ldc = d; g.M = d; g.N = d; g.K = d;
        g.alpha = 1.f; g.beta = 0.f; g.flags = G_LOWER | G_MIRROR;
        g.gate = p->refine_gate_dev + r;
        push_desc(refine_prod, g);
      }
      e = cudaMemcpy(p->refine_items_dev, ritems.data(),
                     sizeof(RefineItem) * nr, cudaMemcpyHostToDevice);
    }
  }
  p->refine_prod = refine_prod;
  if (e == cudaSuccess) e = cudaMalloc(&p->mats_dev, sizeof(MatInfo) * count);
  if (e == cudaSuccess) e = cudaMalloc(&p->trace_dev, sizeof(float) * count);
  if (e == cudaSuccess) e = cudaMalloc(&p->add_dev, sizeof(float) * count);
  if (e == cudaSuccess) e = cudaMalloc(&p->info_dev, sizeof(int) * count);
  if (e == cudaSuccess) e = cudaMalloc(&p->ids_dev, sizeof(int) * std::max<size_t>(ids.size(), 1));
  if (e == cudaSuccess) e = cudaMalloc(&p->descs_dev, sizeof(GemmDesc) * std::max<size_t>(descs.size(), 1));
  if (e == cudaSuccess) e = cudaMemcpy(p->mats_dev, mats.data(), sizeof(MatInfo) * count, cudaMemcpyHostToDevice);
  if (e == cudaSuccess && !ids.empty()) e = cudaMemcpy(p->ids_dev, ids.data(), sizeof(int) * ids.size(), cudaMemcpyHostToDevice);
  if (e == cudaSuccess && !descs.empty()) e = cudaMemcpy(p->descs_dev, descs.data(), sizeof(GemmDesc) * descs.size(), cudaMemcpyHostToDevice);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(chol_diag_kernel<false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)kDiagSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(chol_diag_kernel<true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)kDiagLookSmemBytes);
  if (e != cudaSuccess) {
    kfac_inverse_plan_destroy(p);
    return fail(KFAC_ERR_CUDA, "inverse_plan_create: %s", cudaGetErrorString(e));
  }
  if (use_tc) {
    const int rc = tc_prepare();
    if (rc != KFAC_OK) {
      kfac_inverse_plan_destroy(p);
      return rc;
    }
  }
  *out = p;
  return KFAC_OK;
}

// Issue every launch of one run into `st` (a real stream, or one that is
// being captured into a graph).
static int plan_enqueue(kfac_inverse_plan* p, int* info, float* diag_dev,
                        cudaStream_t main_st, cudaStream_t* side_st) {
  cudaStream_t st = main_st;
  cudaStream_t sts[3] = {main_st, side_st[0], side_st[1]};
  // fork: the side streams start after what precedes this run
  KFAC_CUDA(cudaEventRecord(p->fork_ev, main_st));
  KFAC_CUDA(cudaStreamWaitEvent(side_st[0], p->fork_ev, 0));
  KFAC_CUDA(cudaStreamWaitEvent(side_st[1], p->fork_ev, 0));
  trace_kernel<<<p->count, 256, 0, st>>>(p->mats_dev, p->trace_dev, info);
  KFAC_LAUNCH_CHECK("trace_kernel");
  damping_kernel<<<ceil_div(p->count, 128), 128, 0, st>>>(
      p->mats_dev, p->count, p->trace_dev, p->params_dev, p->add_dev,
      p->add2_dev, diag_dev);
  KFAC_LAUNCH_CHECK("damping_kernel");
  {
    dim3 grid(512, p->count);
    damp_copy_kernel<<<grid, 256, 0, st>>>(p->mats_dev, p->add_dev,
                                           p->add2_dev, p->look ? 1 : 0);
    KFAC_LAUNCH_CHECK("damp_copy_kernel");
  }
  for (const Launch& l : p->launches) {
    if (l.kind == 2) {
      for (int k = 0; k < 2; ++k) {
        KFAC_CUDA(cudaEventRecord(p->join_ev[k], side_st[k]));
        KFAC_CUDA(cudaStreamWaitEvent(main_st, p->join_ev[k], 0));
      }
      continue;
    }
    st = sts[l.stream];
    if (l.wait_ev >= 0)
      KFAC_CUDA(cudaStreamWaitEvent(st, p->events[l.wait_ev], 0));
    if (l.wait_ev2 >= 0)
      KFAC_CUDA(cudaStreamWaitEvent(st, p->events[l.wait_ev2], 0));
    if (l.kind == 0) {
      if (l.look)
        chol_diag_kernel<true><<<l.n, 256, kDiagLookSmemBytes, st>>>(
            p->mats_dev, p->ids_dev + l.off, l.step, info);
      else
        chol_diag_kernel<false><<<l.n, 256, kDiagSmemBytes, st>>>(
            p->mats_dev, p->ids_dev + l.off, l.step, info);
      KFAC_LAUNCH_CHECK("chol_diag_kernel");
    } else {
      int rc = p->use_tc
                   ? launch_tc_grouped(p->descs_dev + l.off, l.n, l.tiles, 0.f,
                                       0.f, l.tails != 0, st)
                   : launch_grouped_gemm(p->descs_dev + l.off, l.n, l.tiles,
                                         0.f, 0.f, st);
      if (rc != KFAC_OK) return rc;
    }
    if (l.rec_ev >= 0) KFAC_CUDA(cudaEventRecord(p->events[l.rec_ev], st));
  }
  st = main_st;
  if (p->n_refine > 0) {
    const dim3 pgrid(ceil_div(p->refine_dmax, 8), p->n_refine);
    for (int stage = 0; stage < 3; ++stage) {
      refine_probe_kernel<<<pgrid, 256, 0, st>>>(
          p->mats_dev, p->refine_items_dev, p->add_dev, p->add2_dev,
          p->refine_sums_dev, p->params_dev, stage);
      KFAC_LAUNCH_CHECK("refine_probe_kernel");
    }
    refine_gate_kernel<<<ceil_div(p->n_refine, 256), 256, 0, st>>>(
        p->refine_items_dev, p->n_refine, p->refine_sums_dev, p->params_dev,
        p->refine_gate_dev, p->refine_count_dev);
    KFAC_LAUNCH_CHECK("refine_gate_kernel");
    refine_residual_kernel<<<p->refine_tiles, 256, 0, st>>>(
        p->mats_dev, p->refine_items_dev, p->n_refine, p->add_dev,
        p->add2_dev, p->refine_gate_dev);
    KFAC_LAUNCH_CHECK("refine_residual_kernel");
    const Launch& l = p->refine_prod;
    int rc = p->use_tc
                 ? launch_tc_grouped(p->descs_dev + l.off, l.n, l.tiles, 0.f,
                                     0.f, l.tails != 0, st)
                 : launch_grouped_gemm(p->descs_dev + l.off, l.n, l.tiles, 0.f,
                                       0.f, st);
    if (rc != KFAC_OK) return rc;
    const dim3 agrid(64, p->n_refine);
    refine_apply_kernel<<<agrid, 256, 0, st>>>(p->mats_dev, p->refine_items_dev,
                                               p->refine_gate_dev);
    KFAC_LAUNCH_CHECK("refine_apply_kernel");
  }
  return KFAC_OK;
}

static void plan_drop_graph(kfac_inverse_plan* p) {
  if (p->graph_exec != nullptr) cudaGraphExecDestroy(p->graph_exec);
  p->graph_exec = nullptr;
}

// Capture one run into a graph (on the plan's own stream: nothing executes
// during capture).  On any failure the plan falls back to plain launches.
static void plan_capture(kfac_inverse_plan* p, int* info, float* diag_dev) {
  plan_drop_graph(p);
  const long long before = launch_count_now();
  if (cudaStreamBeginCapture(p->cap_stream, cudaStreamCaptureModeRelaxed) !=
      cudaSuccess) {
    cudaGetLastError();
    p->graph_ok = false;
    return;
  }
  const int rc = plan_enqueue(p, info, diag_dev, p->cap_stream, p->cap_side);
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(p->cap_stream, &graph);
  const long long captured = launch_count_now() - before;
  count_launches(-captured);          // nothing ran yet
  if (rc == KFAC_OK && e == cudaSuccess && graph != nullptr)
    e = cudaGraphInstantiate(&p->graph_exec, graph, 0);
  if (graph != nullptr) cudaGraphDestroy(graph);
  if (rc != KFAC_OK || e != cudaSuccess || p->graph_exec == nullptr) {
    cudaGetLastError();
    plan_drop_graph(p);
    p->graph_ok = false;
    return;
  }
  p->graph_info = info;
  p->graph_diag = diag_dev;
  p->graph_launches = captured;
}

extern "C" int kfac_inverse_plan_run(kfac_inverse_plan* p, float damping,
                                     int use_pi, int* info_dev,
                                     float* diag_dev, void* stream) {
  KFAC_REQUIRE(p != nullptr, "inverse_plan_run: null plan");
  cudaStream_t st = (cudaStream_t)stream;
  int* info = info_dev ? info_dev : p->info_dev;
  set_run_params_kernel<<<1, 1, 0, st>>>(p->params_dev, damping, use_pi,
                                         p->refine_max_dim,
                                         p->refine_threshold);
  KFAC_LAUNCH_CHECK("set_run_params_kernel");
  if (p->graph_ok) {
    // a caller that is itself capturing gets plain launches in its capture
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) {
      cudaGetLastError();
      cs = cudaStreamCaptureStatusNone;
    }
    if (cs == cudaStreamCaptureStatusNone) {
      if (p->graph_exec == nullptr || p->graph_info != info ||
          p->graph_diag != diag_dev)
        plan_capture(p, info, diag_dev);
      if (p->graph_exec != nullptr) {
        KFAC_CUDA(cudaGraphLaunch(p->graph_exec, st));
        count_launches(p->graph_launches);
        return KFAC_OK;
      }
    }
  }
  return plan_enqueue(p, info, diag_dev, st, p->side_stream);
}

extern "C" int kfac_inverse_plan_set_refine(kfac_inverse_plan* p, int max_dim,
                                            float threshold) {
  KFAC_REQUIRE(p != nullptr, "inverse_plan_set_refine: null plan");
  KFAC_REQUIRE(max_dim >= 0 && threshold >= 0.f,
               "inverse_plan_set_refine: max_dim=%d threshold=%g", max_dim,
               (double)threshold);
  p->refine_max_dim = max_dim < kRefineDimCap ? max_dim : kRefineDimCap;
  p->refine_threshold = threshold;
  return KFAC_OK;
}

extern "C" int kfac_inverse_plan_refined(kfac_inverse_plan* p,
                                         int* refined_out) {
  KFAC_REQUIRE(p != nullptr && refined_out != nullptr,
               "inverse_plan_refined: null argument");
  KFAC_CUDA(cudaDeviceSynchronize());
  KFAC_CUDA(cudaMemcpy(refined_out, p->refine_count_dev, sizeof(int),
                       cudaMemcpyDeviceToHost));
  return KFAC_OK;
}

extern "C" int kfac_inverse_plan_error_estimates(kfac_inverse_plan* p,
                                                 float* estimates_out) {
  KFAC_REQUIRE(p != nullptr && estimates_out != nullptr,
               "inverse_plan_error_estimates: null argument");
  for (int i = 0; i < p->count; ++i) estimates_out[i] = -1.f;
  if (p->n_refine == 0) return KFAC_OK;
  std::vector<RefineItem> items(p->n_refine);
  std::vector<double> sums(2 * (size_t)p->n_refine);
  KFAC_CUDA(cudaDeviceSynchronize());
  KFAC_CUDA(cudaMemcpy(items.data(), p->refine_items_dev,
                       sizeof(RefineItem) * p->n_refine,
                       cudaMemcpyDeviceToHost));
  KFAC_CUDA(cudaMemcpy(sums.data(), p->refine_sums_dev,
                       sizeof(double) * 2 * p->n_refine,
                       cudaMemcpyDeviceToHost));
  for (int r = 0; r < p->n_refine; ++r)
    estimates_out[items[r].mat] =
        sums[2 * r + 1] > 0.0 ? (float)sqrt(sums[2 * r] / sums[2 * r + 1])
                              : -1.f;
  return KFAC_OK;
}

extern "C" int kfac_inverse_plan_set_second_floor(kfac_inverse_plan* p,
                                                  const float* l2_coef_second) {
  KFAC_REQUIRE(p != nullptr && l2_coef_second != nullptr,
               "inverse_plan_set_second_floor: null argument");
  std::vector<MatInfo> mats(p->count);
  KFAC_CUDA(cudaDeviceSynchronize());
  KFAC_CUDA(cudaMemcpy(mats.data(), p->mats_dev, sizeof(MatInfo) * p->count,
                       cudaMemcpyDeviceToHost));
  for (int i = 0; i < p->count; ++i) mats[i].l2b = l2_coef_second[i];
  KFAC_CUDA(cudaMemcpy(p->mats_dev, mats.data(), sizeof(MatInfo) * p->count,
                       cudaMemcpyHostToDevice));
  return KFAC_OK;
}

extern "C" int kfac_inverse_plan_destroy(kfac_inverse_plan* p) {
  if (p == nullptr) return KFAC_OK;
  plan_drop_graph(p);
  if (p->cap_stream != nullptr) cudaStreamDestroy(p->cap_stream);
  for (int k = 0; k < 2; ++k) {
    if (p->cap_side[k] != nullptr) cudaStreamDestroy(p->cap_side[k]);
    if (p->side_stream[k] != nullptr) cudaStreamDestroy(p->side_stream[k]);
    if (p->join_ev[k] != nullptr) cudaEventDestroy(p->join_ev[k]);
  }
  if (p->fork_ev != nullptr) cudaEventDestroy(p->fork_ev);
  for (cudaEvent_t ev : p->events) cudaEventDestroy(ev);
  cudaFree(p->params_dev);
  cudaFree(p->add2_dev);
  cudaFree(p->refine_items_dev);
  cudaFree(p->refine_sums_dev);
  cudaFree(p->refine_vec_dev);
  cudaFree(p->refine_gate_dev);
  cudaFree(p->refine_count_dev);
  cudaFree(p->mats_dev);
  cudaFree(p->trace_dev);
  cudaFree(p->add_dev);
  cudaFree(p->info_dev);
  cudaFree(p->ids_dev);
  cudaFree(p->descs_dev);
  delete p;
  return KFAC_OK;
}
