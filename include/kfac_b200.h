/*
 * kfac_b200 -- C ABI of the B200 (sm_100a) K-FAC curvature kernels.
 *
 * Every pointer named *_dev / documented "device" is a raw device pointer on
 * the current CUDA device; matrices are fp32, row-major, dense unless stated.
 * `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 * Every function returns 0 on success and a non-zero code otherwise; the
 * message for the calling thread's last failure is kfac_last_error().  No
 * function synchronises the device or the stream unless it says so.  There is
 * no CPU implementation behind this interface.
 *
 * Grouped entry points (one call for many layers) copy their per-layer tables
 * to the device through an 8 MiB ring per device, allocated on first use (the
 * one exception is kfac_factor_dense_noalloc, which allocates nothing).  A
 * table is read by the kernels of its own call, in stream order; the ring
 * has no in-flight tracking, so a region is handed out again once 8 MiB of
 * later tables have been requested (a ResNet-50 step with 161 factors
 * requests about 0.3 MiB): a caller whose host runs that far ahead of the
 * device must synchronise.  A
 * workspace passed to a call is scratch of that call's kernels: calls that
 * may run at the same time (different streams) need different workspaces.
 *
 * The reference (chainerkfac) has no native boundary: each entry point names
 * the Python function(s) of the reference whose arithmetic it replaces, by
 * path inside the chainerkfac project.
 */
#ifndef KFAC_B200_H_
#define KFAC_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KFAC_OK 0
#define KFAC_ERR_INVALID 1   /* bad argument                              */
#define KFAC_ERR_CUDA 2      /* a CUDA runtime call or launch failed      */
#define KFAC_ERR_WORKSPACE 3 /* workspace missing or too small            */

/* Version of this interface (bumped on incompatible change). */
int kfac_abi_version(void);
/* Message of the calling thread's most recent failure ("" if none). */
const char* kfac_last_error(void);
/* Number of kernels this library has launched in this process so far. */
int64_t kfac_launch_count(void);

/* Arithmetic engine of the factor / inverse / precondition products.
 * 1 (default, the product): tcgen05 tensor cores with fp32 operands split into
 * two terms, three MMAs per product, fp32 accumulation: two bf16 terms (16
 * significant bits) for the factor builds, two TF32 terms (22 bits) for the
 * inverse and precondition products.  Relative Frobenius error of a factor
 * stays below 1e-5 (bound of the reference comparison: 1e-4).
 * 0: fp32 FFMA tiles on the CUDA cores.  Not a supported product path: it is
 * the accuracy yardstick the parity tests run beside the tensor-core engine
 * (several times slower, no look-ahead, NCHW inputs only) and may go away.
 * The choice is read when a call is made or a plan is created. */
int kfac_set_engine(int engine);
int kfac_get_engine(void);

/* Operand feed of the tensor-core factor builds (no counterpart in the
 * reference).  0 (default): producer warps gather the operand from the
 * caller's arrays (strided rows, implicit im2col) and split it into bf16
 * terms on the way into shared memory.  1: a staging pass first writes X^T as
 * two bf16 planes into the workspace, and the X^T X kernel fetches 32 k x 256
 * row boxes of them with TMA (cp.async.bulk.tensor, 64-byte swizzle); needs
 * 4 * d * roundup(rows, 8) more workspace bytes per factor (the *_workspace_
 * bytes functions account for it) and is not used by
 * kfac_factor_dense_noalloc.  Same results; measured slower on B200 (the
 * 64-byte box rows arrive at about 16 bytes per clock per SM), hence off.
 * The environment variable KFAC_TC_STAGED sets the initial value. */
int kfac_set_factor_staging(int on);
int kfac_get_factor_staging(void);
/* Synchronises the device and returns in *status_out the tensor-core engine's
 * status word: 0, or 1 if a bounded barrier wait inside a kernel ran out (the
 * results of that launch are then invalid). */
int kfac_tc_status(int* status_out);

/* Self-test of that mechanism (failure detection without a fault): launches
 * one warp that waits, with a limit of about a thousand polls, on a barrier
 * nothing arrives at.  On return *status_out is the status word the wait
 * raised (1) and *returned_out is 2 when the wait reported its expiry to the
 * kernel, which then returned normally.  Uses its own status word: the one
 * behind kfac_tc_status is not touched.  Synchronises the device. */
int kfac_selftest_wait_expiry(int* status_out, int* returned_out);

/* ------------------------------------------------------------------ factors
 * out(d x d) = alpha * X^T X + beta * out, X a (rows x d) matrix that is never
 * materialised.  Only one triangle of tiles is computed; both triangles of
 * `out` are written, bit-identical mirror images.  beta == 0 never reads
 * `out`.  alpha carries the reference's scale (1/n, n, n/(ho*wo)); beta != 0
 * fuses the running average (alpha = r*scale, beta = 1-r) or the accumulation
 * over micro-steps.  Work is split along `rows`; partial tiles go to
 * `workspace` (device, at least kfac_factor_workspace_bytes(rows, d) bytes,
 * contents undefined on return).
 */
size_t kfac_factor_workspace_bytes(int64_t rows, int d);

/* X = [x, 1]: x is (rows x d_in) with leading dimension ld; a column of ones
 * is appended when add_ones_col != 0 (bias folded into the factor).
 * Replaces FisherBlockLinear.compute_A / compute_G,
 * optimizers/fisher_blocks/connections/linear.py:14-46. */
int kfac_factor_dense(const float* x, int64_t rows, int d_in, int64_t ld,
                      int add_ones_col, float alpha, float beta, float* out,
                      void* workspace, size_t workspace_bytes, void* stream);

/* X = im2col patches of an NCHW input: rows = n*ho*wo, columns ordered
 * (c, ky, kx) with c slowest, zero padding, square kernel, then the optional
 * ones column.  Replaces FisherBlockConvolution2D.compute_A,
 * optimizers/fisher_blocks/connections/convolution_2d.py:19-41 (including the
 * chainer.functions.im2col call, the NHWC transpose and column_stack).
 * Workspace: kfac_factor_conv_workspace_bytes (partial tiles plus, on the
 * tensor-core engine, a zero-bordered copy of the input when pad > 0, which
 * lets the gather run without bounds checks). */
size_t kfac_factor_conv_workspace_bytes(int n, int c, int h, int w, int ksize,
                                        int stride, int pad,
                                        int add_ones_col);
int kfac_factor_conv_input(const float* x, int n, int c, int h, int w,
                           int ksize, int stride, int pad, int add_ones_col,
                           float alpha, float beta, float* out,
                           void* workspace, size_t workspace_bytes,
                           void* stream);

/* X = output gradient viewed as (n*ho*wo, c) from NCHW storage.
 * Replaces FisherBlockConvolution2D.compute_G,
 * optimizers/fisher_blocks/connections/convolution_2d.py:43-72. */
int kfac_factor_conv_grad(const float* gy, int n, int c, int ho, int wo,
                          float alpha, float beta, float* out,
                          void* workspace, size_t workspace_bytes,
                          void* stream);

/* Same result as kfac_factor_dense, for callers that can neither allocate
 * device memory nor pass a workspace: code that runs inside a framework whose
 * own pool has taken all of the device's memory, so that a cudaMalloc would
 * fail, or on a path where an allocation's implicit device-wide wait is not
 * acceptable.  No counterpart in the reference (which allocates freely through
 * CuPy's pool).  The partial tiles go to a fixed array inside the library
 * (kfac_factor_noalloc_max_bytes() bytes, 32 MiB, held by every GPU context
 * that loads the library until it exits); the call performs no cudaMalloc,
 * cudaFree or other allocating routine.  Shapes whose split needs more than
 * that (kfac_factor_workspace_bytes(rows, d) > the maximum) are rejected with
 * KFAC_ERR_WORKSPACE.  The first call on each device looks up the array's
 * device address; make that first call outside any stream capture.  All calls
 * on a device share the one array, which keeps the previous call's partial
 * tiles (none need clearing: each is rewritten before it is read); two calls
 * whose kernels can overlap on the GPU (different streams) race on it. */
size_t kfac_factor_noalloc_max_bytes(void);
int kfac_factor_dense_noalloc(const float* x, int64_t rows, int d_in,
                              int64_t ld, int add_ones_col, float alpha,
                              float beta, float* out, void* stream);

/* Grouped build: all factors of a step in one call, so that the tiles of small
 * layers fill the GPU together (the reference builds one factor per hook
 * call; results are identical).  Each item is one of the three builds above
 * with the same meaning of its fields; conv gradients pass ho, wo in h, w.
 * `layout` (conv inputs only, tensor-core engine only): 0 = NCHW as in the
 * reference; 1 = the same logical (n, c, h, w) tensor stored channels-last
 * (n, h, w, c), which the zero-bordered staging copy then reads directly.
 * `items` is a host array read during the call; outputs must not alias. */
#define KFAC_FACTOR_DENSE 0
#define KFAC_FACTOR_CONV_INPUT 1
#define KFAC_FACTOR_CONV_GRAD 2
#define KFAC_FACTOR_DENSE_T 3   /* x is (d_in x rows) row-major, pitch ld:
                                   out = alpha x x^T + beta out */
typedef struct kfac_factor_item {
  int kind;
  int add_ones_col;
  const float* x;
  int64_t rows;   /* dense */
  int64_t ld;     /* dense */
  int d_in;       /* dense */
  int n, c, h, w, ksize, stride, pad; /* conv */
  float alpha, beta;
  float* out;
  int layout;     /* conv input: 0 NCHW, 1 channels-last */
} kfac_factor_item;

size_t kfac_factor_group_workspace_bytes(int count,
                                         const kfac_factor_item* items);
int kfac_factor_group(int count, const kfac_factor_item* items,
                      void* workspace, size_t workspace_bytes, void* stream);

/* Per-sample BatchNormalization gradients: out is (n x 2c),
 * out[s, j] = scale * sum_hw gy[s,j,:] * xhat[s,j,:] and
 * out[s, c+j] = scale * sum_hw gy[s,j,:], xhat = x normalised with the batch
 * mean and biased variance (+eps).  hw = 1 for 2-D inputs.  `stats` is a
 * device scratch of 2*c + 4*n*c floats (mean, 1/sqrt(var + eps), then per-
 * sample partial sums in double precision), 8-byte aligned.  Followed by kfac_factor_dense(out, n, 2c, ..)
 * it replaces FisherBlockBatchNormalization.compute_F,
 * optimizers/fisher_blocks/normalizations/batch_normalization.py:78-131. */
int kfac_bn_sample_grads(const float* x, const float* gy, int n, int c, int hw,
                         float eps, float scale, float* out, float* stats,
                         void* stream);

/* kfac_bn_sample_grads for all BatchNormalization layers of a step in two
 * launches (the reference computes them layer by layer inside its backward
 * hook, normalizations/batch_normalization.py:78-124).  `layout` 1: x and gy
 * are stored channels-last, (n, hw, c); 0: (n, c, hw) as in the reference.
 * `items` is a host array (<= 256 entries) read during the call. */
typedef struct kfac_bn_item {
  const float* x;
  const float* gy;
  float* out;      /* (n, 2c) */
  float* stats;    /* scratch, 2c + 4nc floats, 8-byte aligned */
  int n, c, hw;
  int layout;
  float eps, scale;
} kfac_bn_item;
int kfac_bn_sample_grads_group(int count, const kfac_bn_item* items,
                               void* stream);

/* out = a * x + b * y elementwise over `count` floats (out may alias y).
 * Replaces the running-average expression of FisherBlock.update_cov_emas,
 * optimizers/fisher_block.py:155-163, and KFAC.accumulate_grads /
 * accumulate_covs, optimizers/kfac.py:286-304. */
int kfac_axpby(int64_t count, float a, const float* x, float b, const float* y,
               float* out, void* stream);

/* kfac_axpby over `n_arrays` (<= 1024) arrays in one launch: out[i] = a * x[i]
 * + b * y[i] over counts[i] floats each (out[i] may alias y[i]); y may be NULL
 * when b == 0.  The running averages of all factors of a step
 * (FisherBlock.update_cov_emas called block by block in
 * optimizers/kfac.py:306-311).  Pointer/size arrays are host arrays read
 * during the call. */
int kfac_axpby_group(int n_arrays, const int64_t* counts, float a,
                     const float* const* x, float b, const float* const* y,
                     float* const* out, void* stream);

/* ------------------------------------------------------------------ inverse
 * Batched damped inverse of `count` symmetric positive definite factors:
 * inverses[i] = (factors[i] + add_i * I)^-1, dense symmetric, by blocked
 * Cholesky, triangular inverse and symmetric product (d^3 flops per factor).
 * The factors are read-only: the running average stays undamped.
 *
 * role[i] selects add_i with g_i = max(l2_coef[i], damping):
 *   0  forward factor A of a connection:  pi * sqrt(g_i)
 *   1  backward factor G of a connection: sqrt(g_i) / pi
 *   2  full block (BatchNormalization):   g_i * scale[i]
 * pi = sqrt(tr(A) dim(G) / (tr(G) dim(A))) from the factor and its
 * partner[i] (index of the other factor of the pair) when use_pi != 0, else 1.
 * Replaces FisherBlock.update_invs, compute_pi_tracenorm and get_diagval
 * (optimizers/fisher_block.py:14-49,165-179), FisherBlockConnection.
 * get_diagvals (optimizers/fisher_blocks/connection.py:66-77),
 * FisherBlockBatchNormalization.get_diagvals
 * (optimizers/fisher_blocks/normalizations/batch_normalization.py:133-157)
 * and inverse() (optimizers/cholesky_inverse.py:16-102).
 *
 * The plan records device pointers, so the factor and inverse buffers must
 * stay where they are for the plan's lifetime.  `workspace` (device,
 * kfac_inverse_workspace_bytes bytes) is owned by the caller and must outlive
 * the plan; plans that run concurrently need distinct workspaces.
 */
typedef struct kfac_inverse_plan kfac_inverse_plan;

size_t kfac_inverse_workspace_bytes(int count, const int* dims);

int kfac_inverse_plan_create(int count, const int* dims,
                             const float* const* factors,
                             float* const* inverses, const int* partner,
                             const int* role, const float* l2_coef,
                             const float* scale, void* workspace,
                             size_t workspace_bytes,
                             kfac_inverse_plan** plan);

/* info_dev: `count` ints on the device, 0 where the factorisation succeeded,
 * else 1 + index of the first non-positive pivot (the reference never reads
 * cuSOLVER's dev_info; here it is always produced).  diag_dev: `count` floats
 * on the device receiving add_i (the reference's diag_val_forward/backward).
 * Either may be NULL. */
int kfac_inverse_plan_run(kfac_inverse_plan* plan, float damping, int use_pi,
                          int* info_dev, float* diag_dev, void* stream);

/* Iterative refinement of ill-conditioned factors (not in the reference,
 * whose NumPy path reaches the same accuracy through LAPACK): after the
 * inverse X of a factor of at most `max_dim` rows (capped at 1024, the size
 * the workspace reserves room for) a probe estimates its relative error; where
 * that exceeds `threshold`, one step X <- X + X (I - (F + add I) X) runs with
 * the residual accumulated in fp64.  Defaults of a new plan: max_dim = 1024,
 * threshold = 3e-5; max_dim = 0 switches the step off.  Takes effect at the
 * next run. */
int kfac_inverse_plan_set_refine(kfac_inverse_plan* plan, int max_dim,
                                 float threshold);
/* Synchronises the device; *refined_out = number of factors the last run
 * refined. */
int kfac_inverse_plan_refined(kfac_inverse_plan* plan, int* refined_out);

/* Synchronises the device; estimates_out (host, `count` floats) receives the
 * probe's estimate of the relative error each inverse had before refinement
 * in the last run (-1 for factors above the size cap or before any run). */
int kfac_inverse_plan_error_estimates(kfac_inverse_plan* plan,
                                      float* estimates_out);

/* Role-2 blocks only (others ignore it): the rows of the second half of the
 * diagonal (the shift parameters of a BatchNormalization block) are damped
 * with max(l2_coef_second[i], damping) * scale[i] instead of the first half's
 * floor; FisherBlockBatchNormalization.get_diagvals
 * (normalizations/batch_normalization.py:133-157) floors gamma and beta
 * separately.  `l2_coef_second` is a host array of `count` floats.
 * Synchronises the device. */
int kfac_inverse_plan_set_second_floor(kfac_inverse_plan* plan,
                                       const float* l2_coef_second);

int kfac_inverse_plan_destroy(kfac_inverse_plan* plan);

/* ------------------------------------------------------------ precondition
 * For `count` layers: kf = G_inv * [grad_W, grad_b] * A_inv with grad_W viewed
 * as (dG x dW); the first dW columns go to kf_W, the last to kf_b (layers with
 * grad_b[i] == NULL have no bias column and A_inv is dW x dW).  When
 * param_W[i] != NULL the momentum rule is fused into the same epilogue:
 * v = momentum * v - lr * kf; param += v (mom_W / mom_b are the velocity
 * buffers).  Replaces compute_kfgrads (connections/linear.py:48-61,
 * connections/convolution_2d.py:74-90), FisherBlockConnection.update_kfgrads
 * (fisher_blocks/connection.py:51-61) and, when fused, KFACUpdateRule.
 * update_core (optimizers/kfac.py:87-116).
 *
 * All pointer arrays are host arrays of device pointers, read during the
 * call.  `workspace`: device, kfac_precond_workspace_bytes bytes.
 */
size_t kfac_precond_workspace_bytes(int count, const int* dG, const int* dW,
                                    const int* has_bias);

int kfac_precondition(int count, const int* dG, const int* dW,
                      const float* const* G_inv, const float* const* A_inv,
                      const float* const* grad_W, const float* const* grad_b,
                      float* const* kf_W, float* const* kf_b,
                      float* const* param_W, float* const* param_b,
                      float* const* mom_W, float* const* mom_b, float lr,
                      float momentum, void* workspace, size_t workspace_bytes,
                      void* stream);

/* y = M x for a (d x d) matrix, one launch per call: the BatchNormalization
 * preconditioning F_inv * [grad_gamma; grad_beta]
 * (normalizations/batch_normalization.py:175-191). x is given in two pieces
 * (x0 of length d0, then x1 of length d - d0; x1 may be NULL when d0 == d);
 * y likewise.  nan_flag_dev (two device ints, zero-initialised by the caller;
 * may be NULL): when any output is NaN the whole of y is replaced by x, which
 * is the reference's raw-gradient fallback (_check_nan,
 * normalizations/batch_normalization.py:14-31,165-166), done on the device by
 * a second small launch; nan_flag_dev[0] is scratch (0 again afterwards),
 * nan_flag_dev[1] counts the fallbacks taken so far. */
int kfac_symv_split(const float* m, int d, int d0, const float* x0,
                    const float* x1, float* y0, float* y1, int* nan_flag_dev,
                    void* stream);

/* kfac_symv_split for `count` (<= 256) BatchNormalization blocks in two
 * launches: kf = F_inv [grad_gamma; grad_beta] per block (F_inv is 2c x 2c),
 * the NaN fallback to the raw gradients (nan_flags[i]: two device ints per
 * block as in kfac_symv_split), and, for blocks whose param_gamma[i] is not
 * NULL, the fused update v = momentum * v - lr * kf; param += v
 * (normalizations/batch_normalization.py:159-191 and optimizers/kfac.py:
 * 87-116).  param_* / mom_* may be NULL when no block is fused.  All pointer
 * arrays are host arrays of device pointers, read during the call. */
int kfac_bn_precondition_group(
    int count, const int* channels, const float* const* F_inv,
    const float* const* grad_gamma, const float* const* grad_beta,
    float* const* kf_gamma, float* const* kf_beta, float* const* param_gamma,
    float* const* param_beta, float* const* mom_gamma, float* const* mom_beta,
    int* const* nan_flags, float lr, float momentum, void* stream);

/* Low-rank form of the BatchNormalization blocks (an addition: the reference
 * always forms and inverts the dense 2c x 2c factor,
 * normalizations/batch_normalization.py:126-191).  The factor of such a block
 * is F = sum_s w_s U_s^T U_s over the per-sample gradient matrices U_s
 * (rows_per_slot x 2c, as kfac_bn_sample_grads writes them) of the last
 * `slots` steps, so its rank is at most m = slots * rows_per_slot.  With the
 * damping D = diag(damp_gamma ... damp_beta ...)
 *   (F + D)^-1 g = D^-1/2 (g' - Hs^T (I + Hs Hs^T)^-1 Hs g'),
 *   Hs = rows sqrt(w_s) u D^-1/2,  g' = D^-1/2 g.
 * kfac_bn_lowrank_scale writes Hs (`scaled`, m x 2c) from the stored rows
 * (`hist`, m x 2c, slot after slot; slot_weight[s] <= 0: slot unused, rows
 * become zero).  The caller then forms Hs Hs^T with kfac_factor_group
 * (KFAC_FACTOR_DENSE_T) and inverts I + Hs Hs^T with an inverse plan (role 2,
 * damping 1, scale 1).  kfac_bn_lowrank_apply evaluates the formula with that
 * inverse (`m_inv`, m x m) for every block (four grouped launches: rows of
 * Hs, rows of the inverse, columns, finish), with the NaN fallback and the optional fused momentum update of
 * kfac_bn_precondition_group.  `items` is a host array (<= 256 entries). */
typedef struct kfac_bn_lowrank_item {
  const float* hist;
  float* scaled;
  const float* m_inv;                 /* apply only */
  const float* grad_gamma;            /* apply only, as are the next ten */
  const float* grad_beta;
  float* kf_gamma;
  float* kf_beta;
  float* param_gamma;                 /* NULL: no fused update */
  float* param_beta;
  float* mom_gamma;
  float* mom_beta;
  int* nan_flag;                      /* two device ints */
  int c, rows_per_slot, slots;        /* slots <= 32 */
  float damp_gamma, damp_beta;
  float slot_weight[32];
} kfac_bn_lowrank_item;
int kfac_bn_lowrank_scale(int count, const kfac_bn_lowrank_item* items,
                          void* stream);
int kfac_bn_lowrank_apply(int count, const kfac_bn_lowrank_item* items,
                          float lr, float momentum, void* stream);

/* v = momentum * v - lr * grad; param += v over `count` floats.
 * Replaces KFACUpdateRule.update_core_gpu, optimizers/kfac.py:101-116. */
int kfac_momentum_update(int64_t count, const float* grad, float* param,
                         float* v, float lr, float momentum, void* stream);

/* w *= target_norm / (|w|_2 + eps) when that factor is below 1 (`count`
 * floats), without a host synchronisation: the post-update weight rescaling
 * NormalizeWeightUR._normalize_weight of the reference's ImageNet recipe
 * (examples/imagenet/train.py:56-115) with skip_scale_comp off.  `scratch`:
 * two device floats; on return scratch[0] = |w|^2 before scaling,
 * scratch[1] = the factor. */
int kfac_normalize_weight(int64_t count, float* w, float target_norm,
                          float eps, float* scratch, void* stream);

/* ------------------------------------------------------- wire pack / unpack
 * Wire format of the reference's collectives: the arrays concatenated in the
 * given order, a square factor (tri_dim[i] > 0) as its packed row-major lower
 * triangle incl. diagonal (dst[r(r+1)/2 + c] = a[r][c], c <= r), anything else
 * (tri_dim[i] == 0) as its `nelems[i]` elements.  Arrays with select[i] == 0
 * are skipped (pack leaves their slot untouched; zero_skipped != 0 clears it).
 * unpack mirrors triangles back to full symmetric matrices and multiplies by
 * `scale` (1/size for the mean); with ema_r >= 0 the unpacked value is blended
 * into the destination as ema_r * value + (1 - ema_r) * dst.
 * Replaces _pack_arrays_to_buffer / _unpack_arrays_from_buffer and the three
 * NVRTC kernels of communicators/pure_nccl_communicator.py:110-147,300-471.
 * Pointer/size arrays are host arrays read during the call.
 */
int64_t kfac_wire_nelems(int n_arrays, const int64_t* nelems,
                         const int* tri_dim);

int kfac_wire_pack(int n_arrays, const float* const* arrays,
                   const int64_t* nelems, const int* tri_dim,
                   const int* select, int zero_skipped, float* wire,
                   void* stream);

int kfac_wire_unpack(int n_arrays, float* const* arrays, const int64_t* nelems,
                     const int* tri_dim, const int* select, float scale,
                     float ema_r, const float* wire, void* stream);

/* kfac_wire_unpack over `n_wires` (1..16) wire buffers of the same layout:
 * each unpacked element is wires[0][w] + wires[1][w] + ... in that order,
 * then scaled and blended as above.  The buffers may be peer mappings of other
 * GPUs' wire buffers (plain loads over NVLink); with every rank's buffer
 * listed in rank order and scale = 1/size this is the reduction of the
 * reference's reduce_scatter_v for the selected (owned) arrays, fused with the
 * unpack (communicators/pure_nccl_communicator.py:47-108 does allreduce, then
 * unpack).  The caller orders the launch after the peers' packs and keeps the
 * peers from repacking until it has finished (a barrier on either side).
 * `wires` is a host array read during the call. */
int kfac_wire_unpack_sum(int n_arrays, float* const* arrays,
                         const int64_t* nelems, const int* tri_dim,
                         const int* select, float scale, float ema_r,
                         const float* const* wires, int n_wires, void* stream);

/* The same two calls with a reduced-precision wire buffer, halving the bytes
 * that cross NVLink: values are rounded to `wire_dtype` when packed and
 * widened to fp32 when unpacked (sums over wire buffers are formed in fp32).
 * The arrays stay fp32.  The reference's pack / unpack kernels carry the same
 * casts (communicators/pure_nccl_communicator.py:354-375,438-461) but its
 * communicator fixes the wire type to fp32 (:32-33); here the type is the
 * caller's choice, fp32 by default.  A 16-bit wire cannot hold a factor to
 * the 1e-4 bound (bf16: 4e-3, fp16: 5e-4 relative per element). */
#define KFAC_WIRE_F32 0
#define KFAC_WIRE_F16 1
#define KFAC_WIRE_BF16 2
int kfac_wire_pack_as(int wire_dtype, int n_arrays, const float* const* arrays,
                      const int64_t* nelems, const int* tri_dim,
                      const int* select, int zero_skipped, void* wire,
                      void* stream);
int kfac_wire_unpack_sum_as(int wire_dtype, int n_arrays, float* const* arrays,
                            const int64_t* nelems, const int* tri_dim,
                            const int* select, float scale, float ema_r,
                            const void* const* wires, int n_wires,
                            void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KFAC_B200_H_ */
