"""Block of a fully connected layer; mirrors
``chainerkfac/optimizers/fisher_blocks/connections/linear.py``."""

from chainerkfac_b200 import ops
from chainerkfac_b200.optimizers.fisher_blocks.connection import \
    FisherBlockConnection


class LinearFunction(object):
    """Marks a call of a fully connected layer in the hook protocol."""


class FisherBlockLinear(FisherBlockConnection):

    @property
    def funcclass(self):
        return LinearFunction

    def compute_A(self, in_data):
        # linear.py:14-27: A = [x,1]^T [x,1] / n
        x = in_data[0]
        x = x.reshape(-1, x.shape[-1]).contiguous()
        n = x.shape[0]
        bias = self.link.b is not None
        out = self.factor_buffer(0, x.shape[1] + int(bias), x.device)
        return ops.factor_dense(x, bias, alpha=1.0 / n, out=out)

    def compute_G(self, in_data, out_grad_data):
        # linear.py:29-46: G = (s gy)^T (s gy) / n, s = n / loss_scale
        gy = out_grad_data[0]
        gy = gy.reshape(-1, gy.shape[-1]).contiguous()
        n = gy.shape[0]
        s = self.gy_scale(n)
        out = self.factor_buffer(1, gy.shape[1], gy.device)
        return ops.factor_dense(gy, False, alpha=s * s / n, out=out)

    def item_A(self, in_data):
        x = in_data[0]
        x = x.reshape(-1, x.shape[-1]).contiguous()
        bias = self.link.b is not None
        self._A = self.factor_buffer(0, x.shape[1] + int(bias), x.device)
        self._keep_x = x
        return ops.dense_item(x, bias, 1.0 / x.shape[0], 0.0, self._A)

    def item_G(self, in_data, out_grad_data):
        gy = out_grad_data[0]
        gy = gy.reshape(-1, gy.shape[-1]).contiguous()
        n = gy.shape[0]
        s = self.gy_scale(n)
        self._G = self.factor_buffer(1, gy.shape[1], gy.device)
        self._keep_gy = gy
        return ops.dense_item(gy, False, s * s / n, 0.0, self._G)
