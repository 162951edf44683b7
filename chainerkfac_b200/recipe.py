"""Training-recipe pieces of the reference's ImageNet example, for use with
``KFAC`` / ``DistributedKFAC``: the polynomial learning-rate schedule that
feeds ``adjust_momentum``, the post-update weight rescaling, and the
cross-entropy loss whose gradient takes soft (mixed) targets.

Reference: ``examples/imagenet/train.py:28-115`` and
``examples/imagenet/softmax_cross_entropy.py:121-174,235-291``.
"""

import math

import torch

from chainerkfac_b200 import ops


class LrPolynomialDecay(object):
    """``train.py:28-53``: lr = ref_lr * (1 - (e - e0) / (e1 - e0)) ** p for
    e0 <= e < e1, ref_lr before and 0 after.  Calling it with the optimizer
    and the current (fractional) epoch stores the previous rate in
    ``optimizer.lr_pre`` and the new one in ``optimizer.lr``, which is what
    ``adjust_momentum`` of the update rule compares (``kfac.py:94-95``)."""

    def __init__(self, ref_lr, epoch_start, epoch_end, p=2, start_rate=2e-5):
        self.ref_lr = ref_lr
        self.epoch_start = epoch_start
        self.epoch_end = epoch_end
        self.p = p
        self.start_rate = start_rate

    def lr(self, epoch):
        if epoch < self.epoch_start:
            rate = 1.0
        elif epoch < self.epoch_end:
            rate = 1.0 - (epoch - self.epoch_start) / \
                (self.epoch_end - self.epoch_start)
            rate = rate ** self.p
        else:
            rate = 0.0
        return self.ref_lr * rate

    def __call__(self, optimizer, epoch):
        lr = self.lr(epoch)
        optimizer.lr_pre = optimizer.lr
        optimizer.lr = lr
        return lr


class NormalizeWeightUR(object):
    """Update-rule hook of ``train.py:56-115`` (``timing = 'post'``): after
    each update the weight is scaled down to the norm sqrt(2 * out_channels)
    when it exceeds it.  Attach with
    ``param.update_rule.add_hook(NormalizeWeightUR(), timing='post')``.

    With ``skip_scale_comp`` off (the default) norm and scaling run on the
    device in two small launches and nothing is read back.  With it on the
    reference's schedule is followed: the norm is recomputed (and read back)
    only every few steps, the interval growing up to ``max_skip`` while the
    per-step scale stays predictable, and the remembered per-step scale is
    applied in between."""

    name = 'NormalizeWeightUR'
    timing = 'post'

    def __init__(self, skip_scale_comp=False):
        self.skip_scale_comp = skip_scale_comp
        self.warmup_len = 2
        self.max_skip = 10
        self.tolerance = 0.98
        self.eps = 1e-9

    def _normalize_weight(self, rule, param, target_norm=1.0):
        w = param.data
        if not self.skip_scale_comp:
            param._nw_scratch = ops.normalize_weight(
                w, target_norm, self.eps, getattr(param, '_nw_scratch', None))
            return
        calc_scale = calc_interval = False
        pre_interval = 1
        if rule.t < self.warmup_len:
            calc_scale = True
        elif rule.t >= param._t_next:
            calc_scale = calc_interval = True
            pre_interval = param._t_next - param._t
        if calc_scale:
            w_norm = float(torch.linalg.vector_norm(w))
            scale = target_norm / (w_norm + self.eps)
            if calc_interval:
                right_scale = math.pow(
                    scale * param._scale ** (pre_interval - 1),
                    1 / pre_interval)
                error_rate = param._scale / right_scale
                if error_rate > 1:
                    error_rate = 1 / error_rate
                if error_rate < 1:
                    max_interval = min(
                        self.max_skip,
                        math.log(self.tolerance, error_rate) + 1)
                else:
                    max_interval = self.max_skip
                interval = int(min(max_interval, pre_interval + 1))
                param._scale = right_scale
            else:
                interval = 1
                param._scale = scale
            param._t = rule.t
            param._t_next = rule.t + interval
        else:
            scale = param._scale
        if scale < 1:
            w.mul_(scale)

    def __call__(self, rule, param):
        w = param.data
        if w is None:
            return
        self._normalize_weight(rule, param, math.sqrt(2.0 * w.shape[0]))


class _SoftTargetCrossEntropy(torch.autograd.Function):
    """Loss value from the hard labels ``t`` (mean over the samples whose
    label is not ``ignore_label``); gradient coeff * (softmax(x) - tt) from
    the soft targets ``tt`` when they are given, else from the one-hot labels
    (``softmax_cross_entropy.py:121-174,235-291``)."""

    @staticmethod
    def forward(ctx, x, t, tt, ignore_label):
        log_y = torch.log_softmax(x, dim=1)
        valid = t != ignore_label
        count = max(int(valid.sum()), 1)
        picked = log_y.gather(1, t.clamp(min=0).unsqueeze(1)).squeeze(1)
        loss = -(picked * valid).sum() / count
        ctx.save_for_backward(log_y, t, tt if tt is not None else x.new_empty(0))
        ctx.has_tt = tt is not None
        ctx.coeff = 1.0 / count
        ctx.ignore_label = ignore_label
        return loss

    @staticmethod
    def backward(ctx, gloss):
        log_y, t, tt = ctx.saved_tensors
        y = log_y.exp()
        if ctx.has_tt:
            gx = y - tt
        else:
            gx = y.clone()
            gx.scatter_add_(1, t.clamp(min=0).unsqueeze(1),
                            -torch.ones_like(gx[:, :1]))
            gx = gx * (t != ctx.ignore_label).unsqueeze(1)
        return gx * (gloss * ctx.coeff), None, None, None


def softmax_cross_entropy(x, t, tt=None, ignore_label=-1):
    """Cross entropy of logits ``x`` (n, classes) with labels ``t``; with soft
    targets ``tt`` (n, classes; mixup) the gradient uses them."""
    return _SoftTargetCrossEntropy.apply(x, t, tt, ignore_label)
