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
    """Besides the reference's dense 2C x 2C factor this block has a
    low-rank form (no counterpart in the reference; same results up to the
    forgotten tail of the running average, see ``lowrank_window``): while
    the running average remembers w steps of n per-sample gradient rows on
    each of ``world`` ranks and w * n * world <= C, the block stores those
    rows instead of F, and applies (F + D)^-1 through the inverse of a
    (w n world)-sided matrix.  The optimizer switches it on by setting
    ``low_rank_world`` (the number of ranks; None: dense only); the block
    falls back to the dense factor for good when the batch size or the decay
    changes.  ``cov_emas`` then is the dense running average formed from the
    stored rows on request; ``invs`` stays None."""

    low_rank_world = None     # set by the optimizer: ranks whose rows arrive
    low_rank_rank = 0         # this rank's position among them
    keeps_history = True      # False on ranks that do not own the block

    def __init__(self, *args, **kwargs):
        self._F = None
        self._nan_flag = None
        self._lr = None
        self._cov_emas = None
        super(FisherBlockBatchNormalization, self).__init__(*args, **kwargs)
        if self.link.gamma is None or self.link.beta is None:
            raise NotImplementedError(
                'BatchNormalization blocks need both gamma and beta')

    # -- low-rank form -------------------------------------------------------
    @property
    def low_rank_active(self):
        return self._lr is not None

    @property
    def cov_emas(self):
        if self._lr is not None:
            if not self.keeps_history or not any(self._lr['w']):
                return None
            return [self._dense_from_history()]
        return self._cov_emas

    @cov_emas.setter
    def cov_emas(self, value):
        self._cov_emas = value

    def has_state(self):
        """A running average exists (dense, or as stored rows)."""
        if self._lr is not None:
            return any(self._lr['w'])
        return self._cov_emas is not None

    def plan_factors(self):
        """The factors the optimizer's batched inverse plan covers."""
        return [] if self._lr is not None else self._cov_emas

    def max_side(self):
        if self._lr is not None:
            return self._lr['slots'] * self._lr['rows']
        return 2 * self.link.gamma.data.numel()

    def _low_rank_wanted(self, n, c):
        world = self.low_rank_world
        if world is None or not self.deferred:
            return None
        slots = lowrank_window(self.cov_ema_decay)
        if slots == 0 or slots * n * world > c:
            return None
        return (n, slots, world, float(self.cov_ema_decay))

    def _low_rank_setup(self, key, c, device):
        n, slots, world, _ = key
        rows, d = n * world, 2 * c
        own = self.keeps_history
        m = slots * rows
        z = dict(dtype=torch.float32, device=device)
        self._lr = dict(
            key=key, rows=rows, slots=slots, c=c,
            hist=torch.zeros(((m if own else rows), d), **z),
            Hs=torch.empty((m, d), **z) if own else None,
            M=torch.empty((m, m), **z) if own else None,
            Minv=torch.empty((m, m), **z) if own else None,
            w=[0.0] * slots, pos=-1, plan=None)

    def _next_slot(self):
        st = self._lr
        k = (st['pos'] + 1) % st['slots'] if self.keeps_history else 0
        return st['hist'][k * st['rows']:(k + 1) * st['rows']]

    def _row_factor(self):
        # F = sum_s w_s (sum over ranks of U^T U) / (n world); after the mean
        # over ranks of the exchange a slot holds every rank's rows / world
        n, _, world, _ = self._lr['key']
        return float(world) / n

    def _dense_from_history(self, out=None):
        st = self._lr
        d = st['hist'].shape[1]
        if out is None:
            out = torch.empty((d, d), dtype=torch.float32,
                              device=st['hist'].device)
        beta, fac = 0.0, self._row_factor()
        for k, w in enumerate(st['w']):
            if w > 0.0:
                rows = st['hist'][k * st['rows']:(k + 1) * st['rows']]
                ops.factor_group([ops.dense_item(rows, False, w * fac, beta,
                                                 out)], out.device)
                beta = 1.0
        if beta == 0.0:
            out.zero_()
        return out

    def _to_dense(self):
        """Leave the low-rank form for good: the running average becomes the
        dense factor formed from the stored rows."""
        st = self._lr
        dense = None
        if self.keeps_history and any(st['w']):
            dense = [self._dense_from_history()]
        self._lr = None
        self._cov_emas = dense
        self._grads = None

    def commit_rows(self):
        """The running-average step of the low-rank form: the rows written
        by the last backward pass become the newest slot with the decay's
        weight, older slots fade (first step: weight 1, as the reference's
        first running average is a copy)."""
        st = self._lr
        r = self._lr['key'][3]
        first = not any(st['w'])
        st['pos'] = (st['pos'] + 1) % st['slots']
        rest = 0.0 if (first or r == 1.0) else 1.0 - r
        st['w'] = [w * rest for w in st['w']]
        st['w'][st['pos']] = 1.0 if (first or r == 1.0) else r

    def low_rank_item(self, with_grads=False):
        """struct kfac_bn_lowrank_item of this block (``with_grads``: the
        fields kfac_bn_lowrank_apply needs as well).  One struct per block,
        refreshed in place: the history, its scaled copy and the inverse keep
        their addresses."""
        st = self._lr
        it = st.get('item')
        if it is None:
            it = st['item'] = ops.bn_lowrank_item(
                st['hist'], st['Hs'], st['c'], st['rows'],
                [0.0] * st['slots'], 0.0, 0.0, st['Minv'])
        fac = self._row_factor()
        for k, w in enumerate(st['w']):
            it.slot_weight[k] = w * fac
        l2g = getattr(self.link.gamma, 'l2_coef', 0.0) or 0.0
        l2b = getattr(self.link.beta, 'l2_coef', 0.0) or 0.0
        it.damp_gamma = max(l2g, self.damping) * float(self.stab_coeff)
        it.damp_beta = max(l2b, self.damping) * float(self.stab_coeff)
        if with_grads:
            a = self.kfgrad_args(low_rank=True)
            it.grad_gamma, it.grad_beta = a[1].data_ptr(), a[2].data_ptr()
            it.kf_gamma, it.kf_beta = a[3].data_ptr(), a[4].data_ptr()
            it.nan_flag = a[5].data_ptr()
            it.param_gamma = it.param_beta = None     # no fused update
            it.mom_gamma = it.mom_beta = None
            it._grads_keep = a
        return it

    def low_rank_matrix_item(self):
        """Grouped-build item M = Hs Hs^T."""
        st = self._lr
        return ops.dense_t_item(st['Hs'], 1.0, 0.0, st['M'])

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
        if self._lr is not None:
            self._to_dense()
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

    def resolve_form(self):
        """Decide between the dense and the low-rank form for the pending
        hook arguments: low-rank from a block's first step while the stored
        rows stay fewer than C; dense for good once the batch size, the
        decay or the number of ranks changes."""
        pend = getattr(self, '_pending', None)
        if pend is None:
            return
        x = pend[0][0]
        self._check_dims(x)
        n, c = x.shape[0], x.shape[1]
        want = self._low_rank_wanted(n, c)
        if self._lr is not None and self._lr['key'] != want:
            self._to_dense()
        elif self._lr is None and want is not None and \
                self._cov_emas is None:
            self._low_rank_setup(want, c, x.device)

    def pending_item(self):
        """Item of ``ops.bn_sample_grads_group`` for the pending hook
        arguments (None if there are none).  The item of the last step is
        used again when the arrays have the same addresses and geometry (see
        ``FisherBlockConnection._memo_item``)."""
        pend = getattr(self, '_pending', None)
        if pend is None:
            return None
        self.resolve_form()
        self._pending = None
        x, gy = pend[0][0], pend[1][0]
        n = x.shape[0]
        out = getattr(self, '_grads', None)
        if self._lr is not None:
            slot = self._next_slot()
            if self._lr['key'][2] > 1:
                slot.zero_()      # the other ranks' rows arrive by the sum
            out = slot[self.low_rank_rank * n:(self.low_rank_rank + 1) * n]
            self.covs = None
        # (the output moves from slot to slot of the history ring in the
        # low-rank form: it is not part of the key but patched in)
        key = (x.data_ptr(), gy.data_ptr(), x.shape, x.stride(), gy.stride(),
               self._loss_scale)
        memo = getattr(self, '_item_memo', None)
        self._keep_x, self._keep_gy = x, gy
        if memo is not None and memo[0] == key and out is not None and \
                out.shape == memo[1].result.shape:
            it = memo[1]
            it.out = out.data_ptr()
            it.result = out
            it._keep = (out, it._keep[-1])
        else:
            it = ops.bn_item(x, gy, float(self.link.eps), self.gy_scale(n),
                             out, getattr(self, '_stats', None))
            self._stats = it._keep[3]
            self._item_memo = None
            if it.x == x.data_ptr() and it.gy == gy.data_ptr():
                it._keep = it._keep[2:]   # output and statistics only
                self._item_memo = (key, it)
        self._grads_item = it
        self._grads = it.result
        return it

    def factor_item(self):
        """Grouped-build item F = grads^T grads / n for the gradients of the
        last ``pending_item``; sets ``covs``.  None in the low-rank form (the
        rows themselves are the state)."""
        if self._lr is not None:
            return None
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
        if self._lr is not None:
            return []           # no dense factor to invert
        l2_gamma = getattr(self.link.gamma, 'l2_coef', 0.0) or 0.0
        l2_beta = getattr(self.link.beta, 'l2_coef', 0.0) or 0.0
        return [(2, l2_gamma, float(self.stab_coeff), l2_beta)]

    def set_diag_vals(self, diag):
        self.diag_val_backward = diag[0]

    def get_diagvals(self):
        if self._lr is not None:
            it = self.low_rank_item()
            c = self._lr['c']
            dev = self._lr['hist'].device
            return [torch.cat([torch.full((c,), it.damp_gamma, device=dev),
                               torch.full((c,), it.damp_beta, device=dev)])]
        if self._plan is None:
            self.update_invs()
        return [self.diag_val_backward.expand(self.cov_emas[0].shape[0])]

    def update_cov_emas(self):
        if self._lr is not None:
            self.commit_rows()
            return
        super(FisherBlockBatchNormalization, self).update_cov_emas()

    def update_invs(self):
        if self._lr is None:
            return super(FisherBlockBatchNormalization, self).update_invs()
        st = self._lr
        ops.bn_lowrank_scale([self.low_rank_item()])
        ops.factor_group([self.low_rank_matrix_item()], st['M'].device)
        if st['plan'] is None:
            st['plan'] = ops.InversePlan([st['M']], [st['Minv']], [-1], [2],
                                         scale=[1.0])
        st['plan'].run(1.0, False)

    def kfgrad_args(self, low_rank=False):
        """(F_inv, grad_gamma, grad_beta, kf_gamma, kf_beta, nan_flag) for
        ``ops.bn_precondition_group``."""
        if not low_rank:
            self.check_attr('invs')
        gamma, beta = self.link.gamma, self.link.beta
        for p in (gamma, beta):
            if getattr(p, 'kfgrad', None) is None or p.kfgrad is p.grad:
                p.kfgrad = torch.empty_like(p.data)
        if self._nan_flag is None:
            self._nan_flag = torch.zeros(2, dtype=torch.int32,
                                         device=gamma.data.device)
            self._nan_seen = 0
        return (None if low_rank else self.invs[0], gamma.grad.contiguous(),
                beta.grad.contiguous(), gamma.kfgrad, beta.kfgrad,
                self._nan_flag)

    def update_kfgrads(self):
        # batch_normalization.py:159-191: F_inv [grad_gamma; grad_beta]; on
        # NaN the raw gradients are used instead (the reference checks on the
        # host with xp.any(xp.isnan(..)); here the library substitutes them
        # on the device, without a synchronisation)
        if self._lr is not None:
            ops.bn_lowrank_apply([self.low_rank_item(with_grads=True)])
            return
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
        if self._lr is not None:
            # the slot with this rank's rows in place and zeros elsewhere:
            # the mean over ranks is the stack of all ranks' rows / world
            arrays.append((self._next_slot(), False))
        else:
            arrays.append((self.cov_backward, True))
        return arrays
