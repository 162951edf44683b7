"""CPU oracle for the K-FAC curvature path: TEST INFRASTRUCTURE ONLY.

This module restates, in plain NumPy, the arithmetic that chainerkfac's
``--no_cuda`` path performs for one K-FAC step (factor build, running average,
pi-split damping, Cholesky inverse, preconditioning, momentum update) and the
semantics of its two collectives.  It is the checker the parity tests, the
smoke test and the CPU-baseline leg of the benchmark compare the CUDA path
with.  Nothing in the shipped package imports it and it is never a fallback:
the product path raises when the CUDA library is missing.

Pinning: the reference repository ships no tests, golden vectors or
known-answer fixtures for this path.  The restatement is therefore pinned
against outputs of the reference's own functions, executed in a container
where the reference source was available, under a small stand-in for the
``chainer``/``cupy`` modules it imports (``tests/golden/make_golden.py``);
the resulting input/output vectors are committed under ``tests/golden/`` and
``tests/test_oracle_golden.py`` checks every function here against them.

Each function cites the reference file and lines it follows (paths inside the
chainerkfac project).
"""

import numpy as np


# --------------------------------------------------------------------------
# Third-party pieces the reference calls but does not vendor (Chainer).
# --------------------------------------------------------------------------

def conv_out_size(size, k, s, p):
    """Output extent of a convolution without ``cover_all`` and dilation."""
    return (size + 2 * p - k) // s + 1


def im2col(x, ksize, stride, pad):
    """``chainer.functions.im2col`` as consumed by
    ``optimizers/fisher_blocks/connections/convolution_2d.py:25-29``:
    NCHW input -> (n, c*kh*kw, ho, wo) with the channel index slowest inside
    the second axis, zero padding, no dilation, ``cover_all=False``.
    """
    n, c, h, w = x.shape
    k, s, p = int(ksize), int(stride), int(pad)
    ho, wo = conv_out_size(h, k, s, p), conv_out_size(w, k, s, p)
    xp = np.zeros((n, c, h + 2 * p, w + 2 * p), dtype=x.dtype)
    xp[:, :, p:p + h, p:p + w] = x
    col = np.empty((n, c, k, k, ho, wo), dtype=x.dtype)
    for ky in range(k):
        for kx in range(k):
            col[:, :, ky, kx] = xp[:, :, ky:ky + s * ho:s, kx:kx + s * wo:s]
    return col.reshape(n, c * k * k, ho, wo)


def batch_normalize(x, eps):
    """Training-mode ``chainer.functions.batch_normalization`` with gamma=1 and
    beta=0, the only way the reference calls it
    (``fisher_blocks/normalizations/batch_normalization.py:92-96``): per
    channel, subtract the batch mean and divide by sqrt(biased variance + eps).
    """
    axes = (0,) if x.ndim == 2 else (0, 2, 3)
    mean = x.mean(axis=axes, keepdims=True)
    var = x.var(axis=axes, keepdims=True)
    return ((x - mean) / np.sqrt(var + x.dtype.type(eps))).astype(x.dtype)


# --------------------------------------------------------------------------
# Kronecker factors.
# --------------------------------------------------------------------------

def linear_A(x, has_bias):
    """``connections/linear.py:14-27``: A = [x,1]^T [x,1] / n."""
    n = x.shape[0]
    if has_bias:
        x = np.column_stack((x, np.ones(n, dtype=x.dtype)))
    return x.T.dot(x) * (1 / n)


def linear_G(gy, loss_scale=None):
    """``connections/linear.py:29-46``: G = (n gy)^T (n gy) / n."""
    n = gy.shape[0]
    gy_scale = n
    if loss_scale is not None:
        gy_scale *= 1.0 / loss_scale
    gy = gy_scale * gy
    return gy.T.dot(gy) * (1 / n)


def conv_patches(x, ksize, stride, pad, has_bias):
    """Rows of the patch matrix of ``connections/convolution_2d.py:25-32``:
    (n*ho*wo, c*k*k [+1]), columns ordered (c, ky, kx), ones column last."""
    col = im2col(x, ksize, stride, pad).transpose(0, 2, 3, 1)
    n, ho, wo, _ = col.shape
    col = col.reshape(n * ho * wo, -1)
    if has_bias:
        col = np.column_stack((col, np.ones(col.shape[0], dtype=col.dtype)))
    return col


def conv_A(x, ksize, stride, pad, has_bias):
    """``connections/convolution_2d.py:19-41``: A = P^T P / n (divided by the
    batch size, not by the number of patch rows)."""
    n = x.shape[0]
    p = conv_patches(x, ksize, stride, pad, has_bias)
    return p.T.dot(p) * (1 / n)


def conv_G(gy, loss_scale=None):
    """``connections/convolution_2d.py:43-72`` (non-diagonal branch):
    G = g^T g * n^2 / (n*ho*wo), g = gy as (n*ho*wo, c_out)."""
    g = gy.transpose(0, 2, 3, 1)
    n, ho, wo, _ = g.shape
    g = g.reshape(n * ho * wo, -1)
    gy_scale = n
    if loss_scale is not None:
        gy_scale *= 1.0 / loss_scale
    g_scale = 1 / (n * ho * wo) * (gy_scale ** 2)
    return g.T.dot(g) * g_scale


def bn_sample_grads(x, gy, eps, has_gamma=True, has_beta=True,
                    loss_scale=None):
    """Per-sample gradients of ``normalizations/batch_normalization.py:78-123``:
    rows [sum_hw n*gy*xhat, sum_hw n*gy] of shape (n, 2C)."""
    n = x.shape[0]
    gy_scale = n
    if loss_scale is not None:
        gy_scale *= 1.0 / loss_scale
    h = batch_normalize(x, eps)
    if x.ndim == 2:
        g = gy_scale * gy
        gyh = g * h
    else:
        h = h.transpose(0, 2, 3, 1)
        g = gy.transpose(0, 2, 3, 1) * gy_scale
        gyh = (g * h).sum(axis=(1, 2))
        g = g.sum(axis=(1, 2))
    if not has_beta:
        return gyh
    if not has_gamma:
        return g
    return np.hstack((gyh, g))


def bn_F(x, gy, eps, has_gamma=True, has_beta=True, loss_scale=None):
    """``normalizations/batch_normalization.py:124-131``: F = grad^T grad / n."""
    grad = bn_sample_grads(x, gy, eps, has_gamma, has_beta, loss_scale)
    return grad.T.dot(grad) * (1 / x.shape[0])


# --------------------------------------------------------------------------
# Running average, damping, inverse.
# --------------------------------------------------------------------------

def update_cov_ema(cov, cov_ema, decay):
    """``fisher_block.py:155-163``: the decay weights the NEW sample; the first
    step (no previous average) or decay == 1 takes the sample itself."""
    if decay == 1.0 or cov_ema is None:
        return cov
    return decay * cov + (1 - decay) * cov_ema


def pi_tracenorm(A, G):
    """``fisher_block.py:23-42``: sqrt(tr(A) dim(G) / (tr(G) dim(A))), fp32."""
    lnorm = A.trace() * G.shape[0]
    rnorm = G.trace() * A.shape[0]
    return np.sqrt(lnorm / rnorm, dtype=np.float32)


def connection_damping(A, G, damping, l2_coef=0.0, pi_type='tracenorm'):
    """``fisher_blocks/connection.py:66-77`` with ``fisher_block.py:14-20``:
    returns (pi, value added to diag(A), value added to diag(G))."""
    rW = max(l2_coef, damping) ** 0.5
    pi = pi_tracenorm(A, G) if pi_type == 'tracenorm' else 1.0
    return pi, pi * rW, (1 / pi) * rW


def bn_damping(damping, stab_coeff, l2_coef=0.0):
    """``normalizations/batch_normalization.py:133-157``."""
    return max(l2_coef, damping) * stab_coeff


def inverse(a):
    """NumPy branch of ``cholesky_inverse.py:19-25``."""
    la = np.linalg.cholesky(a)
    la_inv = np.linalg.inv(la)
    return np.matmul(la_inv.T, la_inv)


def damped_inverse(cov_ema, diag_add):
    """``fisher_block.py:165-179`` without its in-place write to the running
    average: inverse of (cov_ema + diag_add * I)."""
    a = cov_ema.copy()
    d = a.shape[0]
    a[np.arange(d), np.arange(d)] = np.diagonal(cov_ema) + diag_add
    return inverse(a.astype(cov_ema.dtype))


# --------------------------------------------------------------------------
# Preconditioning and the update rule.
# --------------------------------------------------------------------------

def connection_kfgrads(A_inv, G_inv, grad_W, grad_b=None):
    """``connections/linear.py:48-61`` / ``convolution_2d.py:74-90`` and the
    split of ``fisher_blocks/connection.py:51-61``: returns (W.kfgrad,
    b.kfgrad or None)."""
    grad = grad_W.reshape(grad_W.shape[0], -1)
    if grad_b is not None:
        grad = np.column_stack([grad, grad_b])
    kf = np.dot(np.dot(G_inv, grad), A_inv).astype(grad_W.dtype)
    if grad_b is not None:
        return kf[:, :-1].reshape(grad_W.shape), kf[:, -1].reshape(grad_b.shape)
    return kf.reshape(grad_W.shape), None


def bn_kfgrads(F_inv, grad_gamma, grad_beta):
    """``normalizations/batch_normalization.py:159-191`` incl. the NaN rule:
    returns (gamma.kfgrad, beta.kfgrad)."""
    grad = np.hstack((grad_gamma, grad_beta))
    kf = np.dot(F_inv, grad).astype(grad.dtype)
    if np.any(np.isnan(kf)):
        return grad_gamma, grad_beta
    c = len(grad_gamma)
    return kf[:c], kf[c:]


def momentum_update(param, v, grad, lr, momentum, lr_pre=None,
                    adjust_momentum=False):
    """``kfac.py:87-99``: v = m v - lr grad; param += v (in place)."""
    if adjust_momentum and lr_pre is not None and lr < lr_pre:
        momentum = momentum * lr / lr_pre
    v *= momentum
    v -= lr * grad
    param += v


def connection_step(A, G, grad_W, grad_b, damping, ema_A=None, ema_G=None,
                    decay=1.0, l2_coef=0.0, pi_type='tracenorm'):
    """One ``update_cov_emas -> update_invs -> update_kfgrads`` pass for a
    Linear/Convolution2D block (``kfac.py:306-310``) from clean state."""
    ema_A = update_cov_ema(A, ema_A, decay)
    ema_G = update_cov_ema(G, ema_G, decay)
    pi, dA, dG = connection_damping(ema_A, ema_G, damping, l2_coef, pi_type)
    A_inv = damped_inverse(ema_A, dA)
    G_inv = damped_inverse(ema_G, dG)
    kfW, kfb = connection_kfgrads(A_inv, G_inv, grad_W, grad_b)
    return dict(ema_A=ema_A, ema_G=ema_G, pi=pi, diag_A=dA, diag_G=dG,
                A_inv=A_inv, G_inv=G_inv, kfgrad_W=kfW, kfgrad_b=kfb)


# --------------------------------------------------------------------------
# Wire format and collectives (communicators/pure_nccl_communicator.py).
# --------------------------------------------------------------------------

def accumulate(samples, acc_iters):
    """``KFAC.accumulate_grads`` / ``accumulate_covs``
    (``optimizers/kfac.py:286-304``): the running sum of ``x * (1 /
    acc_iters)`` over the micro-steps, in the arrays' own precision and in
    arrival order."""
    acc = None
    for x in samples:
        new = x * (1 / acc_iters)
        if acc is None:
            acc = new
        else:
            acc += new
    return acc


def pack_lower(a):
    """Packed row-major lower triangle incl. diagonal:
    dst[r(r+1)/2 + c] = a[r, c], c <= r (``pure_nccl_communicator.py:343-349``).
    """
    r, c = np.tril_indices(a.shape[0])
    return a[r, c].copy()


def unpack_lower(buf, d, divisor=1.0):
    """Mirror a packed lower triangle into a full symmetric matrix and divide
    (``pure_nccl_communicator.py:423-432,448-461``)."""
    out = np.empty((d, d), dtype=buf.dtype)
    r, c = np.tril_indices(d)
    vals = buf / buf.dtype.type(divisor)
    out[r, c] = vals
    out[c, r] = vals
    return out


def wire_nelems(arrays):
    """``communicators/_utility.py:72-83``."""
    n = 0
    for local in arrays:
        for a, tri in local:
            n += a.shape[0] * (a.shape[0] + 1) // 2 if tri else a.size
    return n


def pack_arrays(arrays, only_rank=-1):
    """Wire buffer of ``_pack_arrays_to_buffer``
    (``pure_nccl_communicator.py:110-127,300-377``): concatenation in
    (rank, array) order; arrays of other ranks stay zero when ``only_rank``
    selects one."""
    buf = np.zeros(wire_nelems(arrays), dtype=np.float32)
    off = 0
    for rank, local in enumerate(arrays):
        for a, tri in local:
            flat = pack_lower(a) if tri else a.reshape(-1)
            if only_rank < 0 or rank == only_rank:
                buf[off:off + flat.size] = flat
            off += flat.size
    return buf


def unpack_arrays(arrays, buf, only_rank=-1, divisor=1.0):
    """``_unpack_arrays_from_buffer`` (``pure_nccl_communicator.py:129-147,
    380-463``): writes into the given arrays in place."""
    off = 0
    for rank, local in enumerate(arrays):
        for a, tri in local:
            n = a.shape[0] * (a.shape[0] + 1) // 2 if tri else a.size
            if only_rank < 0 or rank == only_rank:
                if tri:
                    a[...] = unpack_lower(buf[off:off + n], a.shape[0], divisor)
                else:
                    a[...] = (buf[off:off + n] /
                              np.float32(divisor)).reshape(a.shape)
            off += n


def reduce_scatter_v_sim(per_rank_arrays):
    """Semantics of ``reduce_scatter_v_arrays``
    (``pure_nccl_communicator.py:47-108``) for ``size`` simulated ranks:
    ``per_rank_arrays[q]`` is rank q's nested ``arrays`` list.  Every rank packs
    everything, the buffers are summed, rank r unpacks only arrays[r], divided
    by the number of ranks.  Modifies the arrays in place."""
    size = len(per_rank_arrays)
    total = sum(pack_arrays(a).astype(np.float32) for a in per_rank_arrays)
    for r, arrays in enumerate(per_rank_arrays):
        unpack_arrays(arrays, total, only_rank=r, divisor=size)


def all_gather_v_sim(per_rank_arrays):
    """Semantics of ``all_gather_v_arrays``
    (``pure_nccl_communicator.py:150-218``): each rank contributes only its own
    arrays (zeros elsewhere), buffers are summed, everyone unpacks all."""
    total = sum(pack_arrays(a, only_rank=r)
                for r, a in enumerate(per_rank_arrays))
    for arrays in per_rank_arrays:
        unpack_arrays(arrays, total, only_rank=-1, divisor=1.0)


def split_indices(n_blocks, size):
    """Ownership of ``kfac.py:344-348``: contiguous ``np.array_split``."""
    return [idx.tolist() for idx in np.array_split(np.arange(n_blocks), size)]


# --------------------------------------------------------------------------
# Training-recipe pieces of the ImageNet example.
# --------------------------------------------------------------------------

def lr_polynomial_decay(epoch, ref_lr, epoch_start, epoch_end, p=2):
    """``LrPolynomialDecay.lr`` (``examples/imagenet/train.py:37-45``)."""
    if epoch < epoch_start:
        rate = 1.0
    elif epoch < epoch_end:
        rate = (1.0 - (epoch - epoch_start) / (epoch_end - epoch_start)) ** p
    else:
        rate = 0.0
    return ref_lr * rate


def normalize_weight(w, eps=1e-9):
    """``NormalizeWeightUR`` with ``skip_scale_comp`` off
    (``examples/imagenet/train.py:68-115``): scale down to the norm
    sqrt(2 * w.shape[0]) if larger.  Returns the new array."""
    target = np.sqrt(2.0 * w.shape[0])
    scale = target / (np.linalg.norm(w) + eps)
    return w * np.float32(scale) if scale < 1 else w.copy()


def soft_target_cross_entropy(x, t, tt=None, ignore_label=-1):
    """Loss and gradient of ``examples/imagenet/softmax_cross_entropy.py``
    (forward ``:76-118`` with normalize=True, reduce='mean'; backward
    ``:235-291``): the loss uses the hard labels, the gradient the soft
    targets when given."""
    x64 = x.astype(np.float64)
    m = x64.max(axis=1, keepdims=True)
    log_y = x64 - m - np.log(np.exp(x64 - m).sum(axis=1, keepdims=True))
    valid = t != ignore_label
    count = max(int(valid.sum()), 1)
    picked = log_y[np.arange(len(t)), np.maximum(t, 0)]
    loss = -(picked * valid).sum() / count
    y = np.exp(log_y)
    if tt is not None:
        gx = (y - tt) / count
    else:
        onehot = np.zeros_like(y)
        onehot[np.arange(len(t)), np.maximum(t, 0)] = 1.0
        gx = (y - onehot) * valid[:, None] / count
    return loss, gx
