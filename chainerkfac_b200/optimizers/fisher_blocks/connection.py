"""Kronecker-factored block of a layer with a weight matrix; mirrors
``chainerkfac/optimizers/fisher_blocks/connection.py``."""

import torch

from chainerkfac_b200 import ops
from chainerkfac_b200.optimizers.fisher_block import FisherBlock


class FisherBlockConnection(FisherBlock):

    def __init__(self, *args, **kwargs):
        self._A = None
        self._G = None
        super(FisherBlockConnection, self).__init__(*args, **kwargs)

    @property
    def cov_forward(self):
        return self.covs[0]

    @property
    def cov_backward(self):
        return self.covs[1]

    @property
    def inv_forward(self):
        return self.invs[0]

    @property
    def inv_backward(self):
        return self.invs[1]

    def is_mine(self, func, in_data, out_grad_data=None):
        if not isinstance(func, self.funcclass):
            return False
        if in_data[1] is not self.link.W.data:
            return False
        return True

    # With ``deferred`` set (by the optimizer) the hooks only remember their
    # arguments; the optimizer then builds the factors of all blocks in one
    # grouped launch (``flush_items``) before anything reads ``covs``.
    deferred = False

    def forward_postprocess(self, func, in_data):
        if self.deferred:
            self._pending_A = in_data
            return
        self._A = self.compute_A(in_data)
        self.covs = [self._A, self._G]

    def backward_preprocess(self, func, in_data, out_grad_data):
        if self.deferred:
            self._pending_G = (in_data, out_grad_data)
            return
        self._G = self.compute_G(in_data, out_grad_data)
        self.covs = [self._A, self._G]

    def item_A(self, in_data):
        """Grouped-build item equivalent to compute_A; sets ``_A``."""
        raise NotImplementedError

    def item_G(self, in_data, out_grad_data):
        raise NotImplementedError

    def _memo_item(self, which, tensor, build):
        """The grouped-build item of the last step again when this step's
        array has the same address and geometry (the caching allocator hands
        activations of a steady training loop the same addresses every
        step); built anew otherwise.  The remembered item holds no reference
        to the array (that would keep its memory from being reused): the
        block's ``_keep_x`` / ``_keep_gy`` do until the launch is queued."""
        key = (tensor.data_ptr(), tensor.shape, tensor.stride(),
               self._loss_scale)
        memo = self.__dict__.setdefault('_item_memo', {})
        hit = memo.get(which)
        if hit is not None and hit[0] == key:
            if which == 0:
                self._keep_x = tensor
            else:
                self._keep_gy = tensor
            return hit[1]
        it = build()
        if it.x == tensor.data_ptr():     # read in place, not from a copy
            it._keep = it._keep[-1:]      # the factor buffer only
            memo[which] = (key, it)
        else:
            memo.pop(which, None)
        return it

    def flush_items(self, forward_only=False):
        """Items for the factors whose hook arguments are pending."""
        items = []
        pend = getattr(self, '_pending_A', None)
        if pend is not None:
            items.append(self._memo_item(0, pend[0],
                                         lambda: self.item_A(pend)))
            self._pending_A = None
        pend = getattr(self, '_pending_G', None)
        if pend is not None and not forward_only:
            items.append(self._memo_item(1, pend[1][0],
                                         lambda: self.item_G(*pend)))
            self._pending_G = None
        if items:
            self.covs = [self._A, self._G]
        return items

    def compute_A(self, in_data):
        raise NotImplementedError

    def compute_G(self, in_data, out_grad_data):
        raise NotImplementedError

    def dims(self):
        W = self.link.W
        dG = W.shape[0]
        dA = W.size // dG + (0 if self.link.b is None else 1)
        return dA, dG

    def factor_buffer(self, which, d, device):
        """Factor buffers are reused from step to step (the reference
        allocates new arrays; the values are the same)."""
        cur = self._A if which == 0 else self._G
        if cur is None or cur.shape[0] != d or cur.device != device:
            cur = torch.empty((d, d), dtype=torch.float32, device=device)
        return cur

    def plan_entries(self):
        # connection.py:66-77: A gets pi*sqrt(g), G gets sqrt(g)/pi,
        # g = max(W.l2_coef or 0, damping)
        l2 = getattr(self.link.W, 'l2_coef', 0.0) or 0.0
        return [(0, l2, 1.0), (1, l2, 1.0)]

    def set_diag_vals(self, diag):
        self.diag_val_forward = diag[0]
        self.diag_val_backward = diag[1]

    def get_diagvals(self):
        """Vectors added to the diagonals (connection.py:66-77), as views of
        the values the last damped inverse used."""
        if self._plan is None:
            self.update_invs()
        A, G = self.cov_emas
        return [self.diag_val_forward.expand(A.shape[0]),
                self.diag_val_backward.expand(G.shape[0])]

    def kfgrad_buffers(self):
        W, b = self.link.W, self.link.b
        if getattr(W, 'kfgrad', None) is None:
            W.kfgrad = torch.empty_like(W.data)
        if b is not None and getattr(b, 'kfgrad', None) is None:
            b.kfgrad = torch.empty_like(b.data)
        return W.kfgrad, (None if b is None else b.kfgrad)

    def update_kfgrads(self):
        # connection.py:51-61 with compute_kfgrads of linear.py:48-61 /
        # convolution_2d.py:74-90: kf = G_inv [grad_W, grad_b] A_inv
        self.check_attr('invs')
        W, b = self.link.W, self.link.b
        kfW, kfb = self.kfgrad_buffers()
        A_inv, G_inv = self.invs
        ops.precondition([G_inv], [A_inv], [W.grad.contiguous()],
                         [None if b is None else b.grad.contiguous()],
                         [kfW], [kfb])
