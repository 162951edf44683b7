"""K-FAC optimizers with the interface of ``chainerkfac/optimizers/kfac.py``.

``KFAC`` / ``DistributedKFAC`` keep the reference's constructor arguments,
run-time mutable hyper-parameters (``lr``, ``lr_pre``, ``momentum``,
``cov_ema_decay``, ``damping``), public state (``fblocks``, ``kfhook``,
``acc_*``, ``indices`` / ``local_indices`` / ``local_fblocks``) and call
sequence.  Differences in mechanism, not in results: the per-block loop of
``update_kfgrads`` (``kfac.py:306-310``) becomes three batched device stages
(running averages, one inverse plan over every owned factor, one grouped
preconditioning launch pair, optionally with the momentum update fused in),
and hook dispatch is a dictionary lookup instead of a scan.
"""

import numpy as np
import torch
from torch import nn

from chainerkfac_b200 import links as L
from chainerkfac_b200 import ops
from chainerkfac_b200.optimizers import _base
from chainerkfac_b200.optimizers import fisher_blocks as FB
from chainerkfac_b200.optimizers.fisher_block import PI_TYPE_TRACENORM

_default_hyperparam = _base.Hyperparameter()
_default_hyperparam.lr = 0.001
_default_hyperparam.lr_pre = 0.001
_default_hyperparam.momentum = 0.9
_default_hyperparam.cov_ema_decay = 0.99
_default_hyperparam.damping = 0.03


def fblock_constructor(sub_linkname, sub_link, **kwargs):
    """``kfac.py:19-30``."""
    args = (sub_linkname, sub_link)
    if isinstance(sub_link, L.Linear):
        return FB.FisherBlockLinear(*args, **kwargs)
    elif isinstance(sub_link, L.Convolution2D):
        return FB.FisherBlockConvolution2D(*args, **kwargs)
    elif isinstance(sub_link, L.BatchNormalization):
        if sub_link.gamma is None and sub_link.beta is None:
            return None
        return FB.FisherBlockBatchNormalization(*args, **kwargs)
    else:
        return None


def connection_only_constructor(sub_linkname, sub_link, **kwargs):
    """Constructor that leaves BatchNormalization layers to the plain momentum
    rule (the ``constructor`` hook point of ``kfac.py:151,196-199``)."""
    if isinstance(sub_link, L.BatchNormalization):
        return None
    return fblock_constructor(sub_linkname, sub_link, **kwargs)


class KFACHook(object):
    """Function hook of ``kfac.py:33-48`` on top of torch module hooks: inside
    the ``with`` block every forward call of a layer that owns a block fires
    ``forward_postprocess(func, in_data)`` and, when the gradient of its
    output arrives, ``backward_preprocess(func, in_data, out_grad_data)``."""

    name = 'KFACHook'

    def __init__(self, fblocks):
        self.fblocks = fblocks
        self._handles = []
        self._by_array = None
        # optional observers fb -> None, called after the block's own hook
        self.on_forward = None
        self.on_backward = None

    def _lookup(self, func, in_data, out_grad_data=None):
        if self._by_array is None or len(self._by_array) != len(self.fblocks):
            self._by_array = {}
            for fb in self.fblocks:
                first = fb.link.W if hasattr(fb.link, 'W') else fb.link.gamma
                self._by_array[id(first.data)] = fb
        fb = self._by_array.get(id(in_data[1]))
        if fb is not None and fb.is_mine(func, in_data, out_grad_data):
            return fb
        for fb in self.fblocks:
            if fb.is_mine(func, in_data, out_grad_data):
                return fb
        return None

    def forward_postprocess(self, func, in_data):
        fblock = self._lookup(func, in_data)
        if fblock is not None:
            fblock.forward_postprocess(func, in_data)
            if self.on_forward is not None:
                self.on_forward(fblock)

    def backward_preprocess(self, func, in_data, out_grad_data):
        fblock = self._lookup(func, in_data, out_grad_data)
        if fblock is not None:
            fblock.backward_preprocess(func, in_data, out_grad_data)
            if self.on_backward is not None:
                self.on_backward(fblock)

    def _make_forward_hook(self, fblock):
        link = fblock.link

        def hook(module, inputs, output):
            if not (torch.is_grad_enabled() and output.requires_grad):
                return
            if isinstance(link, L.BatchNormalization):
                if not module.training:
                    return
                in_data = (inputs[0].detach(), link.gamma.data, link.beta.data)
            else:
                in_data = (inputs[0].detach(), link.W.data) + (
                    () if link.b is None else (link.b.data,))
            func = fblock.funcclass()
            self.forward_postprocess(func, in_data)
            output.register_hook(
                lambda g: self.backward_preprocess(func, in_data,
                                                   (g.detach(),)))
        return hook

    def __enter__(self):
        for fb in self.fblocks:
            self._handles.append(
                fb.link.module.register_forward_hook(
                    self._make_forward_hook(fb)))
        return self

    def __exit__(self, *exc):
        for h in self._handles:
            h.remove()
        self._handles = []
        return False


class KFACUpdateRule(_base.UpdateRule):
    """``kfac.py:51-116``: momentum SGD on ``param.kfgrad`` (falling back to
    ``param.grad``), one fused kernel per parameter."""

    def __init__(self, parent_hyperparam=None, adjust_momentum=False):
        super(KFACUpdateRule, self).__init__(
            parent_hyperparam or _default_hyperparam)
        self.adjust_momentum = adjust_momentum

    def init_state(self, param):
        self.state['v'] = torch.zeros_like(param.data)

    def velocity(self, param):
        if self._state is None:
            self._state = {}
            self.init_state(param)
        return self.state['v']

    def effective_momentum(self):
        lr, lr_pre = self.hyperparam.lr, self.hyperparam.lr_pre
        momentum = self.hyperparam.momentum
        if self.adjust_momentum and lr < lr_pre:
            momentum *= lr / lr_pre
        return momentum

    def update(self, param):
        if getattr(param, '_kfac_applied', False):
            # the preconditioning epilogue already applied this step's update
            param._kfac_applied = False
            self.t += 1
            return
        if param._loss_scale is not None and \
                getattr(param, 'kfgrad', None) is not None:
            param.kfgrad /= param._loss_scale
        super(KFACUpdateRule, self).update(param)

    def update_core(self, param):
        grad = getattr(param, 'kfgrad', None)
        if grad is None:
            grad = param.grad
        if grad is None:
            return
        ops.momentum_update(grad.contiguous(), param.data, self.state['v'],
                            self.hyperparam.lr, self.effective_momentum())

    update_core_gpu = update_core


def update_cov_emas_grouped(blocks):
    """``FisherBlock.update_cov_emas`` for a list of blocks with the running
    averages of all their factors in one launch.  Blocks without a running
    average yet, or with decay 1 (plain copy), take the per-block path."""
    xs, outs, r = [], [], None
    for fb in blocks:
        if fb.low_rank_active:
            fb.update_cov_emas()     # stored rows: a host-side step
            continue
        fb.check_attr('covs')
        decay = fb.cov_ema_decay
        if fb.cov_emas is None or decay == 1.0 or (r is not None and decay != r):
            fb.update_cov_emas()
            continue
        r = decay
        xs += list(fb.covs)
        outs += list(fb.cov_emas)
    if xs:
        ops.axpby_group(r, xs, 1.0 - r, outs, outs)


def pending_factor_items(blocks, forward_only=False):
    """Grouped-build items for every factor of ``blocks`` whose hook arguments
    are pending.  The per-sample gradients of all BatchNormalization blocks
    among them are computed here, in one grouped call, because their factors
    are built from those."""
    items, bn = [], []
    for fb in blocks:
        if isinstance(fb, FB.FisherBlockConnection):
            items += fb.flush_items(forward_only)
        elif isinstance(fb, FB.FisherBlockBatchNormalization) and \
                not forward_only:
            it = fb.pending_item()
            if it is not None:
                bn.append((fb, it))
    if bn:
        ops.bn_sample_grads_group([it for _, it in bn])
        items += [it for it in (fb.factor_item() for fb, _ in bn)
                  if it is not None]
    return items


def lowrank_build(blocks, device):
    """Scaled history Hs and M = Hs Hs^T of BatchNormalization blocks in
    their low-rank form (after the running-average step of this update)."""
    if blocks:
        ops.bn_lowrank_scale([fb.low_rank_item() for fb in blocks])
        ops.factor_group([fb.low_rank_matrix_item() for fb in blocks],
                         device)


class KFAC(_base.GradientMethod):
    """K-FAC optimizer (``kfac.py:119-310``); same arguments and defaults."""

    def __init__(self, lr=_default_hyperparam.lr,
                 momentum=_default_hyperparam.momentum,
                 cov_ema_decay=_default_hyperparam.cov_ema_decay,
                 damping=_default_hyperparam.damping, stab_coeff=16.0,
                 constructor=fblock_constructor, pi_type='tracenorm',
                 use_cholesky=True, loss_scale=None, adjust_momentum=False,
                 acc_iters=1, bn_low_rank=True):
        super(KFAC, self).__init__()
        # BatchNormalization blocks may keep their running average as the
        # per-sample gradient rows it is made of (see
        # FisherBlockBatchNormalization); False keeps the dense 2C x 2C
        # factor everywhere
        self.bn_low_rank = bn_low_rank
        self.hyperparam.lr = lr
        self.hyperparam.lr_pre = lr
        self.hyperparam.momentum = momentum
        self.hyperparam.cov_ema_decay = cov_ema_decay
        self.hyperparam.damping = damping
        self.pi_type = pi_type
        self.constructor = constructor
        self.adjust_momentum = adjust_momentum
        self.stab_coeff = stab_coeff
        self.fblocks = []
        self.kfhook = None
        self._loss_scale = loss_scale
        self.constructor_kwargs = {
            'cov_ema_decay': self.hyperparam.cov_ema_decay,
            'damping': self.hyperparam.damping,
            'use_cholesky': use_cholesky,
            'pi_type': self.pi_type,
            'stab_coeff': self.stab_coeff,
            'loss_scale': self._loss_scale,
        }
        assert acc_iters >= 1, 'Accumulation iterations should be 1 or larger'
        self.acc_iters = acc_iters
        self.acc_count = 0
        self.acc_aware_iterations = 0
        self.only_pic_update_weight = False  # True only if in DistributedKFAC
        # apply v = m v - lr kf; W += v inside the preconditioning epilogue
        self.fuse_update = True
        # build the factors of all layers in one grouped launch after
        # backward instead of one launch per hook call (same values)
        self.group_factors = True
        self._factors_pending = False
        self._emas_done = False
        self._accumulated = False    # accumulate() already ran for this call
        self._plans = {}
        self._lr_plans = {}
        self._lr_built = False       # a pipelined path already built M
        # start the inverses of a size class during the backward pass, as
        # soon as the output gradients of all its layers exist (the large
        # classes sit in the last layers, whose gradients come first): their
        # long serial chains then run beside the rest of the backward pass.
        # Off by default: on ResNet-50 at batch 32 the backward pass keeps
        # the GPU busy by itself and the early inverses slow it down by more
        # than they save afterwards (33.4 ms per step against 29.8 ms).
        self.eager_inverses = False
        self._eager = None
        self._eager_stream = None
        # Let update() return while size classes still run on their side
        # streams (the serial chains of the largest factors outlast
        # everything else): the next forward pass then overlaps them, and
        # every layer waits for its own class right before it is called
        # (forward pre-hooks installed by setup()).  Off by default: code that
        # reads weights other than by calling the layers (checkpoints,
        # parameter statistics) must call join() first.  Single process, one
        # damping group, every update fused into the preconditioning.
        self.defer_join = False
        self._pending_classes = {}      # class index -> event
        self._block_class = {}          # id(fblock) -> class index
        self._deferred_refs = None      # gradients the side streams still read
        self.observation = {}

    lr = _base.HyperparameterProxy('lr')
    lr_pre = _base.HyperparameterProxy('lr_pre')
    momentum = _base.HyperparameterProxy('momentum')
    cov_ema_decay = _base.HyperparameterProxy('cov_ema_decay')
    damping = _base.HyperparameterProxy('damping')

    def setup(self, link):
        super(KFAC, self).setup(link)
        self.fblocks = []
        for sub_linkname, sub_link in sorted(self.target.namedlinks(),
                                             key=lambda kv: kv[0]):
            fblock = self.constructor(sub_linkname, sub_link,
                                      **self.constructor_kwargs)
            if fblock is None:
                continue
            self.fblocks.append(fblock)
        self._set_low_rank(1, 0, None)
        self.kfhook = KFACHook(self.fblocks)
        for fb in self.fblocks:
            module = getattr(fb.link, 'module', None)
            if module is not None:
                module.register_forward_pre_hook(
                    lambda m, inp, fb=fb: self._wait_for_block(fb))
        return self

    def _wait_for_block(self, fb):
        """Forward pre-hook of a layer: its weights may still be being
        updated on a side stream (defer_join)."""
        if not self._pending_classes:
            return
        ev = self._pending_classes.pop(self._block_class.get(id(fb)), None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    def join(self):
        """Order the current stream after every size class still running
        on a side stream (see defer_join)."""
        if self._pending_classes:
            cur = torch.cuda.current_stream()
            for ev in self._pending_classes.values():
                cur.wait_event(ev)
            self._pending_classes = {}
        self._deferred_refs = None

    def _set_low_rank(self, world, rank, owned):
        on = self.bn_low_rank and self.acc_iters == 1
        for i, fb in enumerate(self.fblocks):
            if isinstance(fb, FB.FisherBlockBatchNormalization):
                fb.low_rank_world = world if on else None
                fb.low_rank_rank = rank
                fb.keeps_history = owned is None or i in owned

    def reallocate_cleared_grads(self):
        for param in self.target.params(include_uninit=False):
            if hasattr(param, 'kfgrad') and param.kfgrad is None:
                param.kfgrad = torch.zeros_like(param.data)
        super(KFAC, self).reallocate_cleared_grads()

    def create_update_rule(self):
        return KFACUpdateRule(self.hyperparam,
                              adjust_momentum=self.adjust_momentum)

    def flush_factors(self, forward_only=False):
        """Grouped build of every factor whose hook arguments are pending."""
        items = pending_factor_items(self.fblocks, forward_only)
        if items:
            dev = next(self.target.params()).data.device
            ops.factor_group(items, dev)
        if not forward_only:
            for fb in self.fblocks:
                fb._keep_x = fb._keep_gy = None

    def _forward_backward(self, lossfun, args, kwargs, after_forward=None):
        for fb in self.fblocks:
            fb.deferred = self.group_factors
        self._eager_begin()
        with self.kfhook:
            loss = lossfun(*args, **kwargs)
            if after_forward is not None:
                after_forward()
            if self._use_cleargrads:
                self.target.cleargrads()
            else:
                self.target.zerograds()
            if self._loss_scale is not None:
                loss.backward(torch.full_like(loss, self._loss_scale))
            else:
                loss.backward()
        self.kfhook.on_forward = self.kfhook.on_backward = None
        # what Chainer's backward(loss_scale=) leaves on every parameter: the
        # update rules divide the (scaled) gradients by it
        for param in self.target.params():
            param._loss_scale = self._loss_scale
        for fb in self.fblocks:
            if isinstance(fb, FB.FisherBlockBatchNormalization):
                fb.resolve_form()
        # with a valid inverse plan the factor build is pipelined with the
        # inverses inside update_kfgrads; otherwise build everything now
        # (a class already started during the backward pass keeps the step
        # on that path)
        self._factors_pending = self._pipeline_ready() or bool(
            self._eager is not None and self._eager['started'])
        if not self._factors_pending:
            self._eager = None
            self.flush_factors()
        self.loss = loss.detach()

    # -- size classes started during the backward pass -----------------------
    def _eager_begin(self):
        self._eager = None
        if type(self) is not KFAC or not self.eager_inverses or \
                not torch.cuda.is_available() or not self._pipeline_ready():
            return
        plan = self._plans[tuple(id(fb) for fb in self.fblocks)][0]
        owner = [fb for fb in self.fblocks for _ in fb.plan_factors()]
        blocks_of, cls = [], {}
        # the last class is built and started after the backward pass
        for c, idx in enumerate(plan.classes()[:-1]):
            blocks = []
            for i in idx:
                if id(owner[i]) not in cls:
                    cls[id(owner[i])] = c
                    blocks.append(owner[i])
            blocks_of.append(blocks)
        if not blocks_of:
            return
        if self._eager_stream is None:
            self._eager_stream = torch.cuda.Stream(priority=-1)
        self._eager = dict(
            plan=plan, blocks=blocks_of, cls=cls, calls={},
            waiting=[{id(fb) for fb in b} for b in blocks_of],
            started={}, ema_done=set(), keep=[])
        self.kfhook.on_forward = self._eager_forward
        self.kfhook.on_backward = self._eager_backward

    def _eager_forward(self, fb):
        calls = self._eager['calls']
        calls[id(fb)] = calls.get(id(fb), 0) + 1

    def _eager_backward(self, fb):
        e = self._eager
        c = e['cls'].get(id(fb))
        if c is None or c in e['started']:
            return
        if e['calls'].get(id(fb), 0) != 1:
            return      # a layer called twice: its class waits for the end
        if isinstance(fb, FB.FisherBlockBatchNormalization):
            dense = not fb.low_rank_active
            fb.resolve_form()
            if dense == fb.low_rank_active:
                return  # the block changed form: no early start
        e['waiting'][c].discard(id(fb))
        if e['waiting'][c]:
            return
        # every layer of class c has its output gradient: build its factors
        # and running averages on a side stream and start its inverses
        blocks = e['blocks'][c]
        first = blocks[0]
        cur = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(cur)
        side = self._eager_stream
        side.wait_event(ready)
        with torch.cuda.stream(side):
            items = pending_factor_items(blocks)
            # the activations and gradients behind the items stay referenced
            # until the main stream has waited for this build
            e['keep'].append(items)
            if items:
                ops.factor_group(items, first.link.W.data.device
                                 if hasattr(first.link, 'W')
                                 else first.link.gamma.data.device)
            update_cov_emas_grouped(blocks)
            e['plan'].start_class(c, first.damping,
                                  first._pi_type == PI_TYPE_TRACENORM)
            built = torch.cuda.Event()
            built.record(side)
        e['started'][c] = built
        e['ema_done'].update(id(fb) for fb in blocks)
        self.observation['classes_started_in_backward'] = \
            self.observation.get('classes_started_in_backward', 0) + 1

    def update(self, lossfun=None, *args, **kwargs):
        if lossfun is not None:
            self._forward_backward(lossfun, args, kwargs)

        if self.acc_iters > 1 and not self._accumulated:
            if self.accumulate():
                return
        self._accumulated = False

        self.reallocate_cleared_grads()
        self.call_hooks('pre')
        self.t += 1
        self.update_kfgrads(self.fblocks)

        if not self.only_pic_update_weight:
            for param in self.target.params():
                param.update()

        self.reallocate_cleared_grads()
        self.call_hooks('post')
        self.acc_aware_iterations += 1
        self.observation['acc_aware_iterations'] = self.acc_aware_iterations

    # -- accumulation over micro-steps (kfac.py:259-304) -------------------
    def accumulate(self):
        if self.acc_count == 0:
            for param in self.target.params():
                param.acc_grad = None
            for fblock in self.fblocks:
                fblock.acc_covs = None
        self.accumulate_grads()
        self.accumulate_covs()
        self.acc_count += 1
        if self.acc_count == self.acc_iters:
            self.acc_count = 0
            for param in self.target.params():
                param.grad = param.acc_grad
            for fblock in self.fblocks:
                fblock.covs = fblock.acc_covs
            return False
        elif self.acc_count < self.acc_iters:
            return True
        raise ValueError(
            'acc_count {} should not be larger than acc_iters {}'.format(
                self.acc_count, self.acc_iters))

    def _accumulate_group(self, pairs):
        """acc += x / acc_iters for (x, acc) pairs, acc = x / acc_iters for
        (x, None); one grouped launch each for the new and for the existing
        accumulators.  Returns the accumulators in order."""
        s = 1.0 / self.acc_iters
        accs, first, rest = [], [], []
        for x, acc in pairs:
            if acc is None:
                acc = torch.empty_like(x)
                first.append((x, acc))
            else:
                rest.append((x, acc))
            accs.append(acc)
        for group, b in ((first, 0.0), (rest, 1.0)):
            for k in range(0, len(group), 1024):
                part = group[k:k + 1024]
                xs = [x for x, _ in part]
                outs = [a for _, a in part]
                ops.axpby_group(s, xs, b, outs, outs)
        return accs

    def accumulate_grads(self):
        """``kfac.py:286-293``."""
        params = [p for p in self.target.params() if p.grad is not None]
        accs = self._accumulate_group(
            [(p.grad.contiguous(), getattr(p, 'acc_grad', None))
             for p in params])
        for p, a in zip(params, accs):
            p.acc_grad = a

    def accumulate_covs(self):
        """``kfac.py:295-304``."""
        pairs = []
        for fblock in self.fblocks:
            fblock.check_attr('covs')
            old = getattr(fblock, 'acc_covs', None)
            for j, c in enumerate(fblock.covs):
                pairs.append((c, None if old is None else old[j]))
        accs = self._accumulate_group(pairs)
        k = 0
        for fblock in self.fblocks:
            n = len(fblock.covs)
            fblock.acc_covs = accs[k:k + n]
            k += n

    # -- curvature stages (kfac.py:306-310), batched over blocks ------------
    def _plan_for(self, fblocks):
        key = tuple(id(fb) for fb in fblocks)
        entry = self._plans.get(key)
        bufs = tuple(e.data_ptr() for fb in fblocks
                     for e in fb.plan_factors())
        if entry is not None and entry[1] == bufs:
            return entry[0]
        if entry is not None and entry[0] is not None:
            entry[0].close()
        if not bufs:
            self._plans[key] = (None, bufs)
            return None
        factors, inverses, partner, role, l2, scale = [], [], [], [], [], []
        l2_second = []
        for fb in fblocks:
            ents = fb.plan_entries()
            base = len(factors)
            if ents:
                fb.ensure_invs()
            for j, ent in enumerate(ents):
                rl, l2c, sc = ent[:3]
                l2_second.append(ent[3] if len(ent) > 3 else l2c)
                factors.append(fb.plan_factors()[j])
                inverses.append(fb.invs[j])
                partner.append(base + 1 - j if len(ents) == 2 else -1)
                role.append(rl)
                l2.append(l2c)
                scale.append(sc)
        plan = ops.InversePlanSet(factors, inverses, partner, role, l2, scale,
                                  l2_coef_second=l2_second)
        self._plans[key] = (plan, bufs)
        return plan

    def _lr_plan_for(self, blocks):
        """Batched inverse of the matrices I + Hs Hs^T of low-rank blocks
        (role 2, damping 1, scale 1: the added diagonal is the identity)."""
        key = tuple(id(fb) for fb in blocks)
        entry = self._lr_plans.get(key)
        bufs = tuple(fb._lr['M'].data_ptr() for fb in blocks)
        if entry is not None and entry[1] == bufs:
            return entry[0]
        if entry is not None:
            entry[0].close()
        k = len(blocks)
        plan = ops.InversePlanSet([fb._lr['M'] for fb in blocks],
                                  [fb._lr['Minv'] for fb in blocks],
                                  [-1] * k, [2] * k, scale=[1.0] * k)
        self._lr_plans[key] = (plan, bufs)
        return plan

    def _pipeline_ready(self):
        """True when the factor build may be pipelined with the inverses: a
        single process, no accumulation, grouped factors, one (damping, pi)
        group, and the inverse plans of an earlier step still valid."""
        if type(self) is not KFAC or self.acc_iters != 1 or \
                not self.group_factors or not self.fblocks:
            return False
        first = self.fblocks[0]
        if any(not fb.has_state() or
               (fb.damping, fb._pi_type) != (first.damping, first._pi_type)
               for fb in self.fblocks):
            return False
        entry = self._plans.get(tuple(id(fb) for fb in self.fblocks))
        return entry is not None and entry[0] is not None

    def _pipelined_factors_and_emas(self, fblocks, plan):
        """Build factors and running averages size class by size class,
        largest first, and start each class's inverses on a side stream as
        soon as its factors are final: the long serial chains of the largest
        factors then run next to the factor build of the other layers."""
        owner = []
        for fb in fblocks:
            owner += [fb] * len(fb.plan_factors())
        classes = plan.classes()
        dev = next(self.target.params()).data.device
        first = fblocks[0]
        eager, self._eager = self._eager, None
        started, ema_done = {}, set()
        if eager is not None:
            # classes started during the backward pass: the builds on the
            # side stream come before anything queued here (shared build
            # workspaces; the hook arguments are released below)
            main = torch.cuda.current_stream()
            for ev in eager['started'].values():
                main.wait_event(ev)
            ema_done = eager['ema_done']
            if eager['plan'] is plan:
                started = eager['started']
        low = [fb for fb in fblocks if fb.low_rank_active]
        if low:
            # the low-rank blocks first: their small inverses run beside
            # everything else
            pending_factor_items(low)
            update_cov_emas_grouped(low)
            lowrank_build(low, dev)
            self._lr_plan_for(low).start_class(0, 1.0, False)
            self._lr_built = True
        for c, idx in enumerate(classes):
            if c in started:
                continue
            blocks, seen = [], set()
            for i in idx:
                if id(owner[i]) not in seen:
                    seen.add(id(owner[i]))
                    if id(owner[i]) not in ema_done:
                        blocks.append(owner[i])
            items = pending_factor_items(blocks)
            if items:
                ops.factor_group(items, dev)
            update_cov_emas_grouped(blocks)
            if c + 1 < len(classes):
                plan.start_class(c, first.damping,
                                 first._pi_type == PI_TYPE_TRACENORM)
        for fb in fblocks:
            fb._keep_x = fb._keep_gy = None

    def update_kfgrads(self, fblocks):
        fblocks = list(fblocks)
        if not fblocks:
            return
        self.join()        # classes left over from the previous update
        if self._factors_pending:
            self._factors_pending = False
            plan = self._plan_for(fblocks)
            self._pipelined_factors_and_emas(fblocks, plan)
        elif self._emas_done:
            self._emas_done = False      # a pipelined exchange already did it
        else:
            update_cov_emas_grouped(fblocks)
        low = [fb for fb in fblocks if fb.low_rank_active]
        if low:
            if not self._lr_built:
                lowrank_build(low, next(self.target.params()).data.device)
            self._lr_built = False
            self._lr_plan_for(low).run(1.0, False)
        # one batched damped inverse per (damping, pi rule) group
        groups = {}
        for fb in fblocks:
            groups.setdefault((fb.damping, fb._pi_type), []).append(fb)
        done = set()
        defer = (self.defer_join and type(self) is KFAC and
                 len(groups) == 1 and not self._post_update_hooks)
        for (damping, pi_type), group in groups.items():
            plan = self._plan_for(group)
            if plan is None:
                continue                 # low-rank blocks only
            after = None
            if len(groups) == 1:
                # precondition the layers of a size class on that class's
                # stream as soon as its inverses are done
                owner = []
                for fb in group:
                    owner += [fb] * len(fb.plan_factors())
                classes = plan.classes()

                def after(c, owner=owner, classes=classes):
                    part, part_bn, seen = [], [], set()
                    for i in classes[c]:
                        fb = owner[i]
                        if id(fb) in seen:
                            continue
                        seen.add(id(fb))
                        if isinstance(fb, FB.FisherBlockConnection):
                            part.append(fb)
                        elif defer:
                            part_bn.append(fb)
                    if part:
                        self._precondition(part, ws_key=c)
                    if part_bn:
                        self._precondition_bn(part_bn)
                    done.update(id(fb) for fb in part + part_bn)
            pending = plan.run(damping, pi_type == PI_TYPE_TRACENORM,
                               after_class=after, join=not defer)
            if defer:
                # (the damping values stay on the device, unread: gathering
                # them would wait for every class)
                self._pending_classes = pending
                self._block_class = {}
                owner_cls = {}
                for c, idx in enumerate(plan.classes()):
                    for i in idx:
                        owner_cls[i] = c
                k = 0
                for fb in group:
                    n = len(fb.plan_factors())
                    if n:
                        self._block_class[id(fb)] = owner_cls[k]
                    k += n
                continue
            diag = plan.diag
            k = 0
            for fb in group:
                n = len(fb.plan_factors())
                if n:
                    fb.set_diag_vals(diag[k:k + n])
                k += n
        conn = [fb for fb in fblocks
                if isinstance(fb, FB.FisherBlockConnection) and
                id(fb) not in done]
        if conn:
            self._precondition(conn)
        bn = [fb for fb in fblocks
              if isinstance(fb, FB.FisherBlockBatchNormalization) and
              id(fb) not in done]
        if bn:
            self._precondition_bn(bn)
        if self._pending_classes:
            # the side streams still read this step's gradients: keep them
            # from being handed out again until the classes are joined; a
            # parameter whose update was not fused needs its class now
            params = [p for fb in fblocks for p in fb.link.params()]
            if all(getattr(p, '_kfac_applied', False) for p in params):
                self._deferred_refs = [p.grad for p in params]
            else:
                self.join()

    def _precondition_bn(self, blocks):
        """All BatchNormalization blocks in one grouped call, with the
        momentum update fused in where the update rule allows it."""
        cols = [[] for _ in range(6)]
        pg, pb, vg, vb, fused_params = [], [], [], [], []
        mom, any_fused = None, False
        low_items = []
        # dense blocks first, then the low-rank ones (same per-block logic)
        blocks = [fb for fb in blocks if not fb.low_rank_active] + \
            [fb for fb in blocks if fb.low_rank_active]
        n_dense = sum(1 for fb in blocks if not fb.low_rank_active)
        for fb in blocks:
            if fb.low_rank_active:
                low_items.append(fb.low_rank_item(with_grads=True))
            else:
                for col, a in zip(cols, fb.kfgrad_args()):
                    col.append(a)
            gamma, beta = fb.link.gamma, fb.link.beta
            fuse = self._can_fuse(gamma) and self._can_fuse(beta)
            if fuse:
                m = gamma.update_rule.effective_momentum()
                mom = m if mom is None else mom
                fuse = (m == mom)
            if fuse:
                any_fused = True
                pg.append(gamma.data)
                pb.append(beta.data)
                vg.append(gamma.update_rule.velocity(gamma))
                vb.append(beta.update_rule.velocity(beta))
                fused_params += [gamma, beta]
            else:
                pg.append(None)
                pb.append(None)
                vg.append(None)
                vb.append(None)
        k = n_dense
        extra = dict(param_gamma=pg[:k], param_beta=pb[:k], mom_gamma=vg[:k],
                     mom_beta=vb[:k], lr=self.hyperparam.lr,
                     momentum=mom) if any_fused else {}
        if k:
            ops.bn_precondition_group(*cols, **extra)
        for j, it in enumerate(low_items):
            if pg[k + j] is not None:
                it.param_gamma = pg[k + j].data_ptr()
                it.param_beta = pb[k + j].data_ptr()
                it.mom_gamma = vg[k + j].data_ptr()
                it.mom_beta = vb[k + j].data_ptr()
        if low_items:
            ops.bn_lowrank_apply(low_items, self.hyperparam.lr,
                                 mom if mom is not None else 0.0)
        for p in fused_params:
            p._kfac_applied = True

    def _can_fuse(self, param):
        rule = param.update_rule
        return (self.fuse_update and isinstance(rule, KFACUpdateRule) and
                rule.enabled and param._loss_scale is None and
                rule.hyperparam.lr == self.hyperparam.lr and
                not rule._pre_update_hooks and not rule._post_update_hooks)

    def _precondition(self, conn, ws_key=None):
        Gi, Ai, gW, gb, kW, kb = [], [], [], [], [], []
        pW, pb, vW, vb = [], [], [], []
        fused_params = []
        lr = self.hyperparam.lr
        mom = None
        for fb in conn:
            W, b = fb.link.W, fb.link.b
            kfW, kfb = fb.kfgrad_buffers()
            Ai.append(fb.invs[0])
            Gi.append(fb.invs[1])
            gW.append(W.grad.contiguous())
            gb.append(None if b is None else b.grad.contiguous())
            kW.append(kfW)
            kb.append(kfb)
            fuse = self._can_fuse(W) and (b is None or self._can_fuse(b))
            if fuse:
                m = W.update_rule.effective_momentum()
                mom = m if mom is None else mom
                fuse = (m == mom)
            if fuse:
                pW.append(W.data)
                vW.append(W.update_rule.velocity(W))
                pb.append(None if b is None else b.data)
                vb.append(None if b is None else b.update_rule.velocity(b))
                fused_params += [W] + ([] if b is None else [b])
            else:
                pW.append(None)
                vW.append(None)
                pb.append(None)
                vb.append(None)
        ops.precondition(Gi, Ai, gW, gb, kW, kb, pW, pb, vW, vb, lr=lr,
                         momentum=mom if mom is not None else 0.0,
                         ws_key=ws_key)
        for p in fused_params:
            p._kfac_applied = True


class DistributedKFAC(KFAC):
    """K-FAC with layer-ownership partition (``kfac.py:313-453``): every rank
    builds factors from its local batch, factors and gradients are
    reduce-scattered to the block's owner, the owner inverts, preconditions
    and (by default) updates its layers, and the updated weights are
    all-gathered."""

    def __init__(self, comm, *args, communicate_after_forward=False,
                 only_pic_update_weight=True, ownership='reference',
                 exchange_every_micro_step=False, **kwargs):
        super(DistributedKFAC, self).__init__(*args, **kwargs)
        # With acc_iters > 1 the reference reduce-scatters gradients and
        # factors in every micro-step and accumulates the reduced values
        # (kfac.py:356-382 with :259-304).  The reduction is linear, so
        # accumulating locally and exchanging the accumulated arrays once per
        # update gives the owners the same values with 1/acc_iters of the
        # traffic; that is the default here.  True restores the reference's
        # schedule (also used when the forward factors travel early).
        self.exchange_every_micro_step = exchange_every_micro_step
        if ownership not in ('reference', 'balanced'):
            raise ValueError("ownership must be 'reference' or 'balanced'")
        # 'reference': contiguous split of the name-sorted block list by count
        # (kfac.py:344-348).  'balanced': longest-processing-time assignment
        # by inverse cost (sum of d^3), which evens out the owners' work.
        self.ownership = ownership
        self.comm = comm
        self.only_pic_update_weight = only_pic_update_weight
        cuda = torch.cuda.is_available()
        self.stream = torch.cuda.Stream() \
            if cuda and communicate_after_forward else None
        self.cuda_event = torch.cuda.Event(blocking=True) \
            if cuda and communicate_after_forward else None
        self.target_params = []
        self.constructor_kwargs['communicate_after_forward'] = \
            communicate_after_forward
        self.communicate_after_forward = communicate_after_forward
        self._real_updates = 0
        self._exchange_stream = None

    def setup(self, link):
        super(DistributedKFAC, self).setup(link)
        local_size = self.comm.size
        local_rank = self.comm.rank
        if self.ownership == 'balanced':
            indices = balanced_split(
                [block_cost(fb) for fb in self.fblocks], local_size)
        else:
            indices = np.array_split(np.arange(len(self.fblocks)), local_size)
            indices = [local_indices.tolist() for local_indices in indices]
        local_indices = indices[local_rank]
        self.indices = indices
        self.local_indices = local_indices
        self.local_fblocks = [self.fblocks[i] for i in local_indices]
        setattr(self.comm, 'indices', indices)
        self._set_low_rank(local_size, local_rank, set(local_indices))
        return self

    def update(self, lossfun=None, *args, **kwargs):
        if lossfun is not None:
            self._forward_backward(
                lossfun, args, kwargs,
                after_forward=self.reduce_scatter_v_after_forward)
        if self.is_changed(self.target):
            self.comm.bcast_data(self.target)
        elif self.acc_iters > 1 and not self.exchange_every_micro_step and \
                not self.communicate_after_forward:
            # accumulate this rank's own gradients and factors; on the last
            # micro-step exchange the accumulated arrays once
            if self.accumulate():
                return
            self._accumulated = True
            self.reduce_scatter_v_after_backward()
            super(DistributedKFAC, self).update()
            self._real_updates += 1
        else:
            if self._factors_pending:
                self._factors_pending = False
                self._pipelined_exchange()
                self._emas_done = True
            else:
                self.reduce_scatter_v_after_backward()
            super(DistributedKFAC, self).update()
            self._real_updates += 1

    def _pipeline_ready(self):
        """Whether this step builds, exchanges and averages the factors size
        class by size class (largest first) and starts the owners' inverses
        of a class while the next class is built and exchanged.  The answer
        only depends on state that is the same on every rank: the ranks must
        issue the same sequence of collectives."""
        return (self._real_updates >= 1 and
                not self.communicate_after_forward and
                self.acc_iters == 1 and self.group_factors and
                all(len(ix) > 0 for ix in self.indices) and
                len({(fb.damping, fb._pi_type) for fb in self.fblocks}) == 1)

    def _pipelined_exchange(self):
        plan = self._plan_for(self.local_fblocks)   # None: low-rank only
        bounds = ops.class_bounds()
        class_keys = plan.class_keys if plan is not None else []

        def key_of(fb):
            # covs exist on every rank from the first full update on
            return sum(fb.max_side() > b for b in bounds)
        keys = [key_of(fb) for fb in self.fblocks]
        dev = next(self.target.params()).data.device
        main = torch.cuda.current_stream()
        if self._exchange_stream is None:
            self._exchange_stream = torch.cuda.Stream(priority=-1)
        side = self._exchange_stream
        local = set(self.local_indices)
        first = self.local_fblocks[0]
        order = sorted(set(keys), reverse=True)
        for n, key in enumerate(order):
            members = [i for i, k in enumerate(keys) if k == key]
            items = pending_factor_items([self.fblocks[i] for i in members])
            if items:
                ops.factor_group(items, dev)
            built = torch.cuda.Event()
            built.record(main)
            side.wait_event(built)
            with torch.cuda.stream(side):
                member_set = set(members)
                arrays = extract(
                    self.fblocks,
                    [[i for i in ix if i in member_set] for ix in self.indices],
                    lambda block: block.extract_for_reduce_scatter_v())
                self.comm.reduce_scatter_v_arrays(arrays)
                mine = [self.fblocks[i] for i in members if i in local]
                update_cov_emas_grouped(mine)
                # every rank's rows have arrived in the owner's slot
                lowrank_build([fb for fb in mine if fb.low_rank_active], dev)
                if n + 1 < len(order) and key in class_keys:
                    plan.start_class(class_keys.index(key), first.damping,
                                     first._pi_type == PI_TYPE_TRACENORM)
        done = torch.cuda.Event()
        done.record(side)
        main.wait_event(done)
        self._lr_built = True
        for fb in self.fblocks:
            fb._keep_x = fb._keep_gy = None

    def reduce_scatter_v_after_forward(self):
        if not self.communicate_after_forward:
            return
        self.flush_factors(forward_only=True)
        if self.cuda_event is not None:
            self.cuda_event.record(torch.cuda.current_stream())
            self.stream.wait_event(self.cuda_event)
        arrays = extract(
            self.fblocks, self.indices,
            lambda block: block.extract_for_reduce_scatter_v_after_forward())
        self.comm.reduce_scatter_v_arrays(arrays, self.stream)

    def reduce_scatter_v_after_backward(self):
        if self.cuda_event is not None:
            self.cuda_event.record(self.stream)
            torch.cuda.current_stream().wait_event(self.cuda_event)
        arrays = extract(self.fblocks, self.indices,
                         lambda block: block.extract_for_reduce_scatter_v())
        self.comm.reduce_scatter_v_arrays(arrays)

    def is_changed(self, target):
        previous_params = self.target_params
        self.target_params = [(name, param.data is not None)
                              for name, param in sorted(target.namedparams(),
                                                        key=lambda kv: kv[0])]
        if len(previous_params) != len(self.target_params):
            return True
        for param1, param2 in zip(self.target_params, previous_params):
            if (param1[0] != param2[0]) or param1[1] != param2[1]:
                return True
        return False

    def allocate_asgrad(self, attr):
        for block in self.fblocks:
            for _, param in sorted(block.link.namedparams()):
                if getattr(param, attr, None) is None:
                    setattr(param, attr, torch.zeros_like(param.data))

    def update_kfgrads(self, fblocks):
        # owners run the curvature stages for their blocks; with
        # only_pic_update_weight the momentum update rides in the
        # preconditioning epilogue of the owner
        self.allocate_asgrad('kfgrad')
        super(DistributedKFAC, self).update_kfgrads(self.local_fblocks)

        if self.only_pic_update_weight:
            for fblock in self.local_fblocks:
                for param in fblock.link.params():
                    param.update()
            arrays = extract(fblocks, self.indices,
                             lambda block:
                             block.extract_for_all_gather_v('data'))
        else:
            # every rank applies the gathered kfgrads itself
            arrays = extract(fblocks, self.indices,
                             lambda block:
                             block.extract_for_all_gather_v('kfgrad'))
        self.comm.all_gather_v_arrays(arrays)

    def _can_fuse(self, param):
        # when kfgrads are gathered and applied by every rank, the owner must
        # not apply its update early
        if not self.only_pic_update_weight:
            return False
        return super(DistributedKFAC, self)._can_fuse(param)


def block_cost(fblock):
    """Inverse cost of a block: sum of d^3 over its factors."""
    link = fblock.link
    if hasattr(link, 'W'):
        dG = link.W.shape[0]
        dA = link.W.size // dG + (0 if link.b is None else 1)
        return float(dA) ** 3 + float(dG) ** 3
    return float(2 * link.gamma.size) ** 3


def balanced_split(costs, size):
    """Longest-processing-time assignment of blocks to `size` owners; each
    owner's list is ascending.  Deterministic, so every rank computes the same
    partition."""
    loads = [0.0] * size
    owned = [[] for _ in range(size)]
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    for i in order:
        r = min(range(size), key=lambda q: (loads[q], q))
        owned[r].append(i)
        loads[r] += costs[i]
    return [sorted(o) for o in owned]


def extract(blocks, indices, extractor):
    """``kfac.py:456-464``: arrays[rank] = [(array, triangular), ...]."""
    arrays = []
    for local_indices in indices:
        local_arrays = []
        for index in local_indices:
            for array in extractor(blocks[index]):
                local_arrays.append(array)
        arrays.append(local_arrays)
    return arrays
