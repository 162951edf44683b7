"""Minimal optimizer scaffolding with the shape of Chainer's
``GradientMethod`` / ``UpdateRule`` / ``Hyperparameter`` -- just what
``optimizers/kfac.py`` of the reference relies on (hyper-parameter proxies that
can be changed at run time, per-parameter update rules with state, pre/post
hooks, the iteration counter ``t``)."""

import collections

import torch
from torch import nn

from chainerkfac_b200 import links


class Hyperparameter(object):
    def __init__(self, parent=None):
        self._parent = parent

    def __getattr__(self, name):
        parent = self.__dict__.get('_parent')
        if name.startswith('_') or parent is None:
            raise AttributeError(name)
        return getattr(parent, name)

    def get_dict(self):
        d = {} if self._parent is None else self._parent.get_dict()
        d.update({k: v for k, v in self.__dict__.items() if k != '_parent'})
        return d


class HyperparameterProxy(object):
    def __init__(self, attr_name):
        self._attr_name = attr_name

    def __get__(self, obj, type=None):
        if obj is None:
            return self
        return getattr(obj.hyperparam, self._attr_name)

    def __set__(self, obj, value):
        setattr(obj.hyperparam, self._attr_name, value)


class UpdateRule(object):
    def __init__(self, parent_hyperparam=None):
        self.hyperparam = Hyperparameter(parent_hyperparam)
        self.enabled = True
        self.t = 0
        self._state = None
        self._use_fp32_update = False
        self._fp32_param = None
        self._pre_update_hooks = collections.OrderedDict()
        self._post_update_hooks = collections.OrderedDict()

    @property
    def state(self):
        return self._state

    def add_hook(self, hook, name=None, timing='pre'):
        name = name or getattr(hook, 'name', repr(hook))
        (self._pre_update_hooks if timing == 'pre'
         else self._post_update_hooks)[name] = hook

    def init_state(self, param):
        pass

    def update(self, param):
        if not self.enabled:
            return
        self.t += 1
        if self._state is None:
            self._state = {}
            self.init_state(param)
        # gradients of a scaled loss are un-scaled here, as in Chainer's
        # UpdateRule.update
        if getattr(param, '_loss_scale', None) is not None and \
                param.grad is not None:
            param.grad /= param._loss_scale
        for hook in self._pre_update_hooks.values():
            hook(self, param)
        self.update_core(param)
        for hook in self._post_update_hooks.values():
            hook(self, param)

    def update_core(self, param):
        raise NotImplementedError


class GradientMethod(object):
    def __init__(self):
        self.hyperparam = Hyperparameter()
        self.target = None
        self.t = 0
        self._pre_update_hooks = collections.OrderedDict()
        self._post_update_hooks = collections.OrderedDict()
        self._use_cleargrads = True

    def setup(self, link):
        if isinstance(link, nn.Module):
            link = links.wrap(link)
        self.target = link
        self.t = 0
        for param in link.params():
            param.update_rule = self.create_update_rule()
        return self

    def create_update_rule(self):
        raise NotImplementedError

    def add_hook(self, hook, name=None, timing='pre'):
        name = name or getattr(hook, 'name', repr(hook))
        (self._pre_update_hooks if timing == 'pre'
         else self._post_update_hooks)[name] = hook

    def call_hooks(self, timing='pre'):
        hooks = self._pre_update_hooks if timing == 'pre' \
            else self._post_update_hooks
        for hook in hooks.values():
            hook(self)

    def use_cleargrads(self, use=True):
        self._use_cleargrads = use

    def reallocate_cleared_grads(self):
        for param in self.target.params(False):
            if param.grad is None:
                param.grad = torch.zeros_like(param.data)
