"""Block of a 2-D convolution; mirrors
``chainerkfac/optimizers/fisher_blocks/connections/convolution_2d.py``.  The
im2col patch matrix of the reference is never built: the factor kernel
gathers patches while it multiplies."""

import torch

from chainerkfac_b200 import ops
from chainerkfac_b200.optimizers.fisher_blocks.connection import \
    FisherBlockConnection


def _dense_layout(t):
    """NCHW-contiguous tensors as they are; channels-last tensors too (the
    factor calls read them in place where they can); anything else is copied."""
    if t.is_contiguous() or \
            t.is_contiguous(memory_format=torch.channels_last):
        return t
    return t.contiguous()


class Convolution2DFunction(object):
    """Marks a call of a convolution layer in the hook protocol."""


class FisherBlockConvolution2D(FisherBlockConnection):

    @property
    def funcclass(self):
        return Convolution2DFunction

    def compute_A(self, in_data):
        # convolution_2d.py:19-41: A = P^T P / n, P = patches (+ ones column)
        x = _dense_layout(in_data[0])
        ksize, stride, pad = \
            self._link.ksize, self._link.stride[0], self._link.pad[0]
        n, c = x.shape[0], x.shape[1]
        bias = self._link.b is not None
        out = self.factor_buffer(0, c * ksize * ksize + int(bias), x.device)
        return ops.factor_conv_input(x, ksize, stride, pad, bias,
                                     alpha=1.0 / n, out=out)

    def compute_G(self, in_data, out_grad_data):
        # convolution_2d.py:43-72: G = g^T g * s^2 / (n ho wo), s = n/loss_scale
        gy = _dense_layout(out_grad_data[0])
        n, c, ho, wo = gy.shape
        s = self.gy_scale(n)
        out = self.factor_buffer(1, c, gy.device)
        return ops.factor_conv_grad(gy, alpha=s * s / float(n * ho * wo),
                                    out=out)

    def item_A(self, in_data):
        x = _dense_layout(in_data[0])
        ksize, stride, pad = \
            self._link.ksize, self._link.stride[0], self._link.pad[0]
        n, c = x.shape[0], x.shape[1]
        bias = self._link.b is not None
        self._A = self.factor_buffer(0, c * ksize * ksize + int(bias),
                                     x.device)
        self._keep_x = x
        return ops.conv_input_item(x, ksize, stride, pad, bias, 1.0 / n, 0.0,
                                   self._A)

    def item_G(self, in_data, out_grad_data):
        gy = _dense_layout(out_grad_data[0])
        n, c, ho, wo = gy.shape
        s = self.gy_scale(n)
        self._G = self.factor_buffer(1, c, gy.device)
        self._keep_gy = gy
        return ops.conv_grad_item(gy, s * s / float(n * ho * wo), 0.0,
                                  self._G)
