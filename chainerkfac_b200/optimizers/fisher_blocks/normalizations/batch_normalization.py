"""Full (2C x 2C) block of a BatchNormalization layer's scale and shift;
mirrors ``chainerkfac/optimizers/fisher_blocks/normalizations/
batch_normalization.py``."""

import math
import warnings

import torch

from chainerkfac_b200 import ops
from chainerkfac_b200.optimizers.fisher_block import FisherBlock


LOWRANK_MAX_SLOTS = 32      # slots of kfac_bn_lowrank_item
LOWRANK_FORGET = 1e-8       # weight below which a past step is forgotten


def lowrank_window(cov_ema_decay):
    """Number of past steps whose per-sample gradients the running average
    F <- decay * F_new + (1 - decay) * F still holds with a relative weight
    above LOWRANK_FORGET (below fp32 resolution of the sum): 1 when the
    running average is switched off (decay 1.0), 0 when the window would
    not fit the history slots of the low-rank form, which then is not used.
    A factor that is the weighted sum of w steps of n per-sample gradient
    rows has rank <= w * n, and (F + D)^-1 g needs only the inverse of a
    (w n) x (w n) matrix (Woodbury)."""
    rest = 1.0 - float(cov_ema_decay)
    if rest <= 0.0:
        return 1
    if rest >= 1.0:
        return 0
    w = int(math.ceil(math.log(LOWRANK_FORGET) / math.log(rest) - 1e-9))
    return w if w <= LOWRANK_MAX_SLOTS else 0


class BatchNormalizationFunction(object):
    """Marks a call of a batch-normalization layer in the hook protocol."""


class FisherBlockBatchNormalization(FisherBlock):

    def __init__(self, *args, **kwargs):
        self._F = None
        self._nan_flag = None
        super(FisherBlockBatchNormalization, self).__init__(*args, **kwargs)
        if self.link.gamma is None or self.link.beta is None:
            raise NotImplementedError(
                'BatchNormalization blocks need both gamma and beta')

    @property
    def funcclass(self):
        return BatchNormalizationFunction

    cov_forward = property(lambda self: None)
    cov_backward = property(lambda self: self.covs[0])
    inv_forward = property(lambda self: None)
    inv_backward = property(lambda self: self.invs[0])

    def is_mine(self, func, in_data, out_grad_data=None):
        if not isinstance(func, self.funcclass):
            return False
        return in_data[1] is self.link.gamma.data or \
            in_data[2] is self.link.beta.data

    # With ``deferred`` set (by the optimizer) the hook only remembers its
    # arguments; the optimizer then computes the per-sample gradients of all
    # BatchNormalization layers in one grouped call and builds their factors
    # together with the other layers' (``pending_item`` / ``factor_item``).
    deferred = False

    def forward_postprocess(self, func, in_data):
        pass  # F needs the output gradient

    def backward_preprocess(self, func, in_data, out_grad_data):
        if self.deferred:
            self._pending = (in_data, out_grad_data)
            return
        self._F = self.compute_F(in_data, out_grad_data)
        self.covs = [self._F]

    def _check_dims(self, x):
        if x.dim() not in (2, 4):
            raise RuntimeError(
                'len(x.shape) must be 2 or 4, not {}.'.format(x.dim()))

    def factor_buffer(self, c, device):
        out = self._F
        if out is None or out.shape[0] != 2 * c or out.device != device:
            out = torch.empty((2 * c, 2 * c), dtype=torch.float32,
                              device=device)
        return out

    def pending_item(self):
        """Item of ``ops.bn_sample_grads_group`` for the pending hook
        arguments (None if there are none)."""
        pend = getattr(self, '_pending', None)
        if pend is None:
            return None
        self._pending = None
        x, gy = pend[0][0], pend[1][0]
        self._check_dims(x)
        self._grads_item = ops.bn_item(
            x, gy, float(self.link.eps), self.gy_scale(x.shape[0]),
            getattr(self, '_grads', None))
        self._grads = self._grads_item.result
        return self._grads_item

    def factor_item(self):
        """Grouped-build item F = grads^T grads / n for the gradients of the
        last ``pending_item``; sets ``covs``."""
        grads = self._grads
        n, c2 = grads.shape
        self._F = self.factor_buffer(c2 // 2, grads.device)
        self.covs = [self._F]
        return ops.dense_item(grads, False, 1.0 / n, 0.0, self._F)

    def compute_F(self, in_data, out_grad_data):
        # batch_normalization.py:78-131: per-sample gradients of (gamma, beta)
        # with xhat from batch statistics, F = grad^T grad / n
        x, gy = in_data[0], out_grad_data[0]
        self._check_dims(x)
        n, c = x.shape[0], x.shape[1]
        grads = ops.bn_sample_grads(x, gy, float(self.link.eps),
                                    self.gy_scale(n))
        return ops.factor_dense(grads, False, alpha=1.0 / n,
                                out=self.factor_buffer(c, x.device))

    def plan_entries(self):
        # batch_normalization.py:133-157: max(l2_coef, damping) * stab_coeff,
        # with gamma's l2_coef for the first half of the diagonal and beta's
        # for the second
        l2_gamma = getattr(self.link.gamma, 'l2_coef', 0.0) or 0.0
        l2_beta = getattr(self.link.beta, 'l2_coef', 0.0) or 0.0
        return [(2, l2_gamma, float(self.stab_coeff), l2_beta)]

    def set_diag_vals(self, diag):
        self.diag_val_backward = diag[0]

    def get_diagvals(self):
        if self._plan is None:
            self.update_invs()
        return [self.diag_val_backward.expand(self.cov_emas[0].shape[0])]

    def kfgrad_args(self):
        """(F_inv, grad_gamma, grad_beta, kf_gamma, kf_beta, nan_flag) for
        ``ops.bn_precondition_group``."""
        self.check_attr('invs')
        gamma, beta = self.link.gamma, self.link.beta
        for p in (gamma, beta):
            if getattr(p, 'kfgrad', None) is None or p.kfgrad is p.grad:
                p.kfgrad = torch.empty_like(p.data)
        if self._nan_flag is None:
            self._nan_flag = torch.zeros(2, dtype=torch.int32,
                                         device=gamma.data.device)
            self._nan_seen = 0
        return (self.invs[0], gamma.grad.contiguous(), beta.grad.contiguous(),
                gamma.kfgrad, beta.kfgrad, self._nan_flag)

    def update_kfgrads(self):
        # batch_normalization.py:159-191: F_inv [grad_gamma; grad_beta]; on
        # NaN the raw gradients are used instead (the reference checks on the
        # host with xp.any(xp.isnan(..)); here the library substitutes them
        # on the device, without a synchronisation)
        a = self.kfgrad_args()
        ops.bn_precondition_group([a[0]], [a[1]], [a[2]], [a[3]], [a[4]],
                                  [a[5]])

    def check_nan(self):
        """True (with the reference's warning) when a step since the last
        check fell back to the raw gradients because its preconditioned
        gradients contained NaN.  Reads a device counter: synchronises."""
        if self._nan_flag is None:
            return False
        count = int(self._nan_flag[1].item())
        if count != self._nan_seen:
            self._nan_seen = count
            warnings.warn(
                'Detected NaN in the kfgrads of the batch normalization layer'
                'Substitue ``grad`` as ``kfgrad`` to avoid crashing')
            return True
        return False

    def extract_for_reduce_scatter_v(self):
        arrays = self.extract_attr_from_params('grad')
        arrays.append((self.cov_backward, True))
        return arrays
