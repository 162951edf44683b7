"""Link / Parameter protocol of the host framework, over ``torch.nn`` modules.

The reference optimizer is written against Chainer's duck types: a link tree
with ``namedlinks()`` / ``namedparams()`` / ``params()`` / ``cleargrads()``,
layers exposing ``W``, ``b`` (Linear, Convolution2D), ``ksize``, ``stride``,
``pad`` (Convolution2D), ``gamma``, ``beta``, ``avg_mean``, ``eps``
(BatchNormalization), and parameters exposing ``data`` / ``grad`` / ``update()``
(chainerkfac ``optimizers/kfac.py:192-203``, ``fisher_blocks/connections/
convolution_2d.py:21-22``, ``normalizations/batch_normalization.py:93-96``).
Chainer is not a dependency here; these classes give a ``torch.nn.Module`` the
same face so the optimizer code reads like the reference's.
"""

import torch
from torch import nn


class Parameter(object):
    """Chainer-style view of one ``torch.nn.Parameter``."""

    def __init__(self, tparam, name):
        self._p = tparam
        self._data = tparam.detach()   # alias of the storage, stable identity
        self.name = name
        self.update_rule = None
        self._loss_scale = None

    @property
    def data(self):
        return self._data

    @data.setter
    def data(self, value):
        self._p.data = value
        self._data = self._p.detach()

    array = data

    @property
    def grad(self):
        return self._p.grad

    @grad.setter
    def grad(self, value):
        self._p.grad = value

    @property
    def dtype(self):
        return self._p.dtype

    @property
    def shape(self):
        return tuple(self._p.shape)

    @property
    def size(self):
        return self._p.numel()

    def cleargrad(self):
        self._p.grad = None

    def update(self):
        if self.update_rule is not None:
            self.update_rule.update(self)


class Link(object):
    """Generic node of the link tree (a Chain when it has children)."""

    param_names = ()     # (chainer name, torch attribute) pairs

    def __init__(self, module):
        self.module = module
        self._params = []
        self._children = []
        self._flat_params = None     # params() of the finished tree
        for cname, tname in self.param_names:
            tp = getattr(module, tname, None)
            p = None if tp is None else Parameter(tp, cname)
            setattr(self, cname, p)
            if p is not None:
                self._params.append(cname)
        if not self.param_names:
            for tname, tp in module.named_parameters(recurse=False):
                setattr(self, '_param_' + tname, Parameter(tp, tname))
                self._params.append('_param_' + tname)

    @property
    def xp(self):
        return torch

    def add_child(self, name, link):
        self._children.append((name, link))
        self._flat_params = None

    def namedlinks(self, skipself=False, _prefix=''):
        if not skipself:
            yield (_prefix or '/'), self
        for name, child in self._children:
            for item in child.namedlinks(_prefix=_prefix + '/' + name):
                yield item

    def namedparams(self, include_uninit=True, _prefix=''):
        for attr in self._params:
            p = getattr(self, attr)
            yield _prefix + '/' + p.name, p
        for name, child in self._children:
            for item in child.namedparams(include_uninit,
                                          _prefix + '/' + name):
                yield item

    def params(self, include_uninit=True):
        # the tree is built once (wrap), bottom-up: the flat list is kept
        if self._flat_params is None:
            self._flat_params = [p for _, p in self.namedparams()]
        return iter(self._flat_params)

    def links(self, skipself=False):
        for _, l in self.namedlinks(skipself):
            yield l

    def cleargrads(self):
        for p in self.params():
            p.cleargrad()

    def zerograds(self):
        for p in self.params():
            if p.grad is None:
                p.grad = torch.zeros_like(p.data)
            else:
                p.grad.zero_()

    def __call__(self, *args, **kwargs):
        return self.module(*args, **kwargs)


class Linear(Link):
    param_names = (('W', 'weight'), ('b', 'bias'))


class Convolution2D(Link):
    param_names = (('W', 'weight'), ('b', 'bias'))

    def __init__(self, module):
        super(Convolution2D, self).__init__(module)
        self.ksize = module.kernel_size[0]
        self.stride = tuple(module.stride)
        self.pad = tuple(module.padding)


class BatchNormalization(Link):
    param_names = (('gamma', 'weight'), ('beta', 'bias'))

    def __init__(self, module):
        super(BatchNormalization, self).__init__(module)
        self.eps = module.eps

    @property
    def avg_mean(self):
        return self.module.running_mean


def _supported_conv(m):
    return (isinstance(m, nn.Conv2d) and m.groups == 1 and
            tuple(m.dilation) == (1, 1) and
            m.kernel_size[0] == m.kernel_size[1] and
            m.stride[0] == m.stride[1] and
            isinstance(m.padding, tuple) and m.padding[0] == m.padding[1] and
            m.padding_mode == 'zeros')


def wrap(module):
    """Build (once) the link tree of ``module``; children are visited in
    registration order and named as in ``module.named_children()``."""
    cached = getattr(module, '_kfac_link', None)
    if cached is not None:
        return cached
    if isinstance(module, nn.Linear):
        link = Linear(module)
    elif _supported_conv(module):
        link = Convolution2D(module)
    elif isinstance(module, (nn.BatchNorm1d, nn.BatchNorm2d)) and module.affine:
        link = BatchNormalization(module)
    else:
        link = Link(module)
        for name, child in module.named_children():
            link.add_child(name, wrap(child))
    object.__setattr__(module, '_kfac_link', link)
    return link
