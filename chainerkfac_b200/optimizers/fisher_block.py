"""Base class of the per-layer curvature blocks; mirrors
``chainerkfac/optimizers/fisher_block.py`` (state ``covs`` / ``cov_emas`` /
``invs``, running average, damped inverse, extraction of the arrays the
collectives move).  All arithmetic is done by the CUDA library through
``chainerkfac_b200.ops``."""

import torch

from chainerkfac_b200 import ops

PI_TYPE_TRACENORM = 'tracenorm'


def get_diagval(link, attrname, damping):
    """``fisher_block.py:14-20``: max(param.l2_coef or 0, damping)."""
    param = getattr(link, attrname, None)
    if param is None:
        return
    r = getattr(param, 'l2_coef', 0.0)
    return max(r, damping)


class FisherBlock(object):

    def __init__(self, linkname, link, cov_ema_decay, damping,
                 communicate_after_forward=False, pi_type=PI_TYPE_TRACENORM,
                 use_cholesky=True, stab_coeff=64.0, loss_scale=None):
        if not use_cholesky:
            raise NotImplementedError(
                'use_cholesky=False (LU inverse) is not part of this build')
        self._link = link
        self._linkname = linkname
        self._linkclass = link.__class__
        self._communicate_after_forward = communicate_after_forward
        self._pi_type = pi_type
        self._use_cholesky = use_cholesky
        self._loss_scale = loss_scale
        self.cov_ema_decay = cov_ema_decay
        self.damping = damping
        self.stab_coeff = stab_coeff
        self.xp = torch
        self.covs = None
        self.invs = None
        self.cov_emas = None
        self.diagonalize = False
        self._plan = None

    linkname = property(lambda self: self._linkname)
    link = property(lambda self: self._link)

    @property
    def funcclass(self):
        raise NotImplementedError

    def is_mine(self, func, in_data, out_grad_data=None):
        raise NotImplementedError

    def forward_postprocess(self, func, in_data):
        raise NotImplementedError

    def backward_preprocess(self, func, in_data, out_grad_data):
        raise NotImplementedError

    def check_attr(self, name):
        if getattr(self, name) is None:
            raise RuntimeError(
                '{} is None:\nlinkname: {}\nlinkclass: {}'.format(
                    name, self._linkname, self._linkclass))

    def get_diagval(self, attr):
        return get_diagval(self._link, attr, self.damping)

    low_rank_active = False

    def has_state(self):
        """A running average exists."""
        return self.cov_emas is not None

    def plan_factors(self):
        """The factors the optimizer's batched inverse plan covers."""
        return self.cov_emas

    def max_side(self):
        return max(int(c.shape[0]) for c in self.covs)

    def gy_scale(self, n):
        s = float(n)
        if self._loss_scale is not None:
            s *= 1.0 / self._loss_scale
        return s

    # -- running average (fisher_block.py:155-163) ------------------------
    def update_cov_emas(self):
        self.check_attr('covs')
        r = self.cov_ema_decay
        first = self.cov_emas is None
        if first:
            self.cov_emas = [torch.empty_like(c) for c in self.covs]
        for cov, ema in zip(self.covs, self.cov_emas):
            if r == 1.0 or first:
                ops.axpby(1.0, cov, 0.0, ema, ema)
            else:
                ops.axpby(r, cov, 1.0 - r, ema, ema)

    # -- damped inverse (fisher_block.py:165-179) -------------------------
    def plan_entries(self):
        """(role, l2_coef, scale[, l2_coef_second]) for each factor, see
        kfac_inverse_plan_create / kfac_inverse_plan_set_second_floor."""
        raise NotImplementedError

    def ensure_invs(self):
        if self.invs is None:
            self.invs = [torch.empty_like(e) for e in self.cov_emas]
        return self.invs

    def update_invs(self):
        self.check_attr('cov_emas')
        self.ensure_invs()
        if self._plan is None:
            entries = self.plan_entries()
            k = len(entries)
            partner = [1, 0] if k == 2 else [-1]
            self._plan = ops.InversePlan(
                self.cov_emas, self.invs, partner,
                [e[0] for e in entries], [e[1] for e in entries],
                [e[2] for e in entries],
                [e[3] if len(e) > 3 else e[1] for e in entries])
        self._plan.run(self.damping, self._pi_type == PI_TYPE_TRACENORM)
        self.set_diag_vals(self._plan.diag)

    def set_diag_vals(self, diag):
        raise NotImplementedError

    def update_kfgrads(self):
        raise NotImplementedError

    # -- arrays moved by the collectives (fisher_block.py:187-216) --------
    def extract_attr_from_params(self, attrname, triangular=False):
        arrays = []
        for _, param in sorted(self.link.namedparams()):
            x = getattr(param, attrname, None)
            if x is not None:
                arrays.append((x, triangular))
        return arrays

    def extract_for_reduce_scatter_v_after_forward(self):
        if self._communicate_after_forward:
            return [(self.cov_forward, True)]
        return []

    def extract_for_reduce_scatter_v(self):
        arrays = self.extract_attr_from_params('grad')
        if not self._communicate_after_forward:
            arrays.append((self.cov_forward, True))
        arrays.append((self.cov_backward, True))
        return arrays

    def extract_for_all_gather_v(self, target='kfgrad'):
        return self.extract_attr_from_params(target)
