"""Generate the golden vectors under tests/golden/ by EXECUTING the reference.

Run once, where a checkout of the chainerkfac sources is available, with its
location in ``CHAINERKFAC_SRC`` (the directory that holds ``chainerkfac/``):

    CHAINERKFAC_SRC=<checkout> python tests/golden/make_golden.py

The reference's NumPy (``--no_cuda``) arithmetic is imported unmodified and run
on seeded inputs.  Chainer, CuPy and ChainerMN are not installed, so a small
stand-in provides only the names the reference imports: array-module helpers
that return NumPy, placeholder function/link classes, a minimal optimizer /
update-rule / parameter protocol, and the three Chainer functions the path
calls (``im2col``, ``batch_normalization`` in training mode, ``cast``), which
are third-party code restated in ``oracle/kfac_oracle.py``.

The vectors are small on purpose (committed fixtures); the tests that consume
them never need the reference sources.
"""

import contextlib
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import kfac_oracle as orc  # noqa: E402

SRC = os.environ.get('CHAINERKFAC_SRC')
if not SRC or not os.path.isdir(os.path.join(SRC, 'chainerkfac')):
    raise SystemExit('set CHAINERKFAC_SRC to a checkout of chainerkfac')


# ---------------------------------------------------------------- stand-ins
def _module(name, **attrs):
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    sys.modules[name] = m
    return m


class _Data(object):
    def __init__(self, data):
        self.data = data


class Hyperparameter(object):
    def __init__(self, parent=None):
        self._parent = parent

    def __getattr__(self, name):
        if '_parent' not in self.__dict__ or self._parent is None:
            raise AttributeError(name)
        return getattr(self._parent, name)


class HyperparameterProxy(object):
    def __init__(self, name):
        self._name = name

    def __get__(self, obj, objtype=None):
        return getattr(obj.hyperparam, self._name)

    def __set__(self, obj, value):
        setattr(obj.hyperparam, self._name, value)


class UpdateRule(object):
    def __init__(self, parent_hyperparam=None):
        self.hyperparam = Hyperparameter(parent_hyperparam)
        self.state = None
        self._use_fp32_update = False
        self._fp32_param = None

    def update(self, param):
        if self.state is None:
            self.state = {}
            self.init_state(param)
        self.update_core_cpu(param)


class GradientMethod(object):
    def __init__(self):
        self.hyperparam = Hyperparameter()
        self.t = 0

    def setup(self, link):
        self.target = link
        for param in link.params():
            param.update_rule = self.create_update_rule()
        return self

    def reallocate_cleared_grads(self):
        for _, param in self.target.namedparams(False):
            if param.grad is None:
                param.grad = np.zeros_like(param.data)

    def call_hooks(self, timing='pre'):
        pass


class FunctionHook(object):
    def __enter__(self):
        return self

    def __exit__(self, *a):
        pass


class Parameter(object):
    def __init__(self, data, name):
        self.data = data
        self.grad = None
        self.name = name
        self.update_rule = None
        self._loss_scale = None

    array = property(lambda self: self.data)
    dtype = property(lambda self: self.data.dtype)
    shape = property(lambda self: self.data.shape)
    size = property(lambda self: self.data.size)

    def update(self):
        if self.update_rule is not None:
            self.update_rule.update(self)


class Link(object):
    xp = np

    def __init__(self):
        self._params = []
        self._children = []

    def add_param(self, name, data):
        p = None if data is None else Parameter(data, name)
        setattr(self, name, p)
        if p is not None:
            self._params.append(name)
        return p

    def add_link(self, name, link):
        setattr(self, name, link)
        self._children.append(name)

    def namedlinks(self, prefix=''):
        yield (prefix or '/'), self
        for c in self._children:
            for item in getattr(self, c).namedlinks(prefix + '/' + c):
                yield item

    def namedparams(self, include_uninit=True, prefix=''):
        for n in self._params:
            yield prefix + '/' + n, getattr(self, n)
        for c in self._children:
            for item in getattr(self, c).namedparams(include_uninit,
                                                     prefix + '/' + c):
                yield item

    def params(self, include_uninit=True):
        for _, p in self.namedparams(include_uninit):
            yield p

    def cleargrads(self):
        for p in self.params():
            p.grad = None


class Linear(Link):
    def __init__(self, W, b=None):
        super(Linear, self).__init__()
        self.add_param('W', W)
        self.add_param('b', b)


class Convolution2D(Link):
    def __init__(self, W, b, ksize, stride, pad):
        super(Convolution2D, self).__init__()
        self.add_param('W', W)
        self.add_param('b', b)
        self.ksize, self.stride, self.pad = ksize, (stride, stride), (pad, pad)


class BatchNormalization(Link):
    def __init__(self, gamma, beta, eps=2e-5):
        super(BatchNormalization, self).__init__()
        self.add_param('gamma', gamma)
        self.add_param('beta', beta)
        self.avg_mean = np.zeros(gamma.shape, dtype=gamma.dtype)
        self.eps = eps


class LinearFunction(object):
    pass


class Convolution2DFunction(object):
    pass


class BatchNormalizationFunction(object):
    pass


def install_standins():
    cuda = _module(
        'chainer.backends.cuda',
        get_array_module=lambda *a: np,
        get_device_from_array=lambda *a: contextlib.nullcontext(),
        available=False)
    backends = _module('chainer.backends', cuda=cuda)
    functions = _module(
        'chainer.functions',
        cast=lambda x, dt: _Data(np.asarray(x).astype(dt)),
        im2col=lambda x, k, s, p: _Data(orc.im2col(x, k, s, p)))
    _module('chainer.functions.connection')
    _module('chainer.functions.connection.linear',
            LinearFunction=LinearFunction)
    _module('chainer.functions.connection.convolution_2d',
            Convolution2DFunction=Convolution2DFunction)
    _module('chainer.functions.normalization')
    _module(
        'chainer.functions.normalization.batch_normalization',
        BatchNormalization=BatchNormalizationFunction,
        batch_normalization=lambda x, g, b, eps=2e-5: _Data(
            orc.batch_normalize(x, eps) * g.reshape(
                (1, -1) + (1,) * (x.ndim - 2)) + b.reshape(
                (1, -1) + (1,) * (x.ndim - 2))))
    links = _module('chainer.links', Linear=Linear,
                    Convolution2D=Convolution2D,
                    BatchNormalization=BatchNormalization)
    optimizer = _module('chainer.optimizer', Hyperparameter=Hyperparameter,
                        HyperparameterProxy=HyperparameterProxy,
                        UpdateRule=UpdateRule, GradientMethod=GradientMethod)
    function_hook = _module('chainer.function_hook',
                            FunctionHook=FunctionHook)
    variable = _module('chainer.variable', Variable=Parameter)
    _module('chainer', backends=backends, functions=functions, links=links,
            optimizer=optimizer, function_hook=function_hook,
            variable=variable, cuda=cuda, report=lambda *a, **k: None)
    _module('cupy.cuda', cublas=None, cusolver=None, device=None)
    _module('cupy', cuda=sys.modules['cupy.cuda'])
    # Enter the package below chainerkfac/__init__.py, which imports the
    # ChainerMN-based communicators.
    pkg = _module('chainerkfac')
    pkg.__path__ = [os.path.join(SRC, 'chainerkfac')]


# ---------------------------------------------------------------- cases
def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def gen_linear(rng, n, din, dout, bias):
    x = f32(rng.random((n, din)))
    gy = f32(rng.standard_normal((n, dout)) / n)
    W = f32(rng.standard_normal((dout, din)) * 0.1)
    b = f32(rng.standard_normal(dout) * 0.1) if bias else None
    gW = f32(rng.standard_normal((dout, din)))
    gb = f32(rng.standard_normal(dout)) if bias else None
    return x, gy, W, b, gW, gb


def gen_conv(rng, n, cin, cout, hw, k, bias):
    x = f32(rng.standard_normal((n, cin, hw, hw)))
    W = f32(rng.standard_normal((cout, cin, k, k)) * 0.1)
    b = f32(rng.standard_normal(cout) * 0.1) if bias else None
    gW = f32(rng.standard_normal(W.shape))
    gb = f32(rng.standard_normal(cout)) if bias else None
    return x, W, b, gW, gb


def run_connection_block(FB, kind, link, x, gy, damping, decay, steps=1):
    """Drive one reference block exactly as KFACHook/KFAC.update_kfgrads do."""
    cls = FB.FisherBlockLinear if kind == 'linear' \
        else FB.FisherBlockConvolution2D
    blk = cls('/l', link, cov_ema_decay=decay, damping=damping)
    out = {}
    for step in range(steps):
        in_data = (x[step], link.W.data) + (
            (link.b.data,) if link.b is not None else ())
        blk.forward_postprocess(None, in_data)
        blk.backward_preprocess(None, in_data, (gy[step],))
        out['A%d' % step] = blk.cov_forward.copy()
        out['G%d' % step] = blk.cov_backward.copy()
        blk.update_cov_emas()
        blk.update_invs()
        # update_invs wrote the damped diagonal into the running average
        out['ema_A_damped%d' % step] = blk.cov_emas[0].copy()
        out['ema_G_damped%d' % step] = blk.cov_emas[1].copy()
        out['diag_A%d' % step] = np.float32(blk.diag_val_forward)
        out['diag_G%d' % step] = np.float32(blk.diag_val_backward)
        out['A_inv%d' % step] = blk.inv_forward.copy()
        out['G_inv%d' % step] = blk.inv_backward.copy()
        blk.update_kfgrads()
        out['kfgrad_W%d' % step] = link.W.kfgrad.copy()
        if link.b is not None:
            out['kfgrad_b%d' % step] = link.b.kfgrad.copy()
    return out


def main():
    install_standins()
    import chainerkfac.optimizers as KO  # the reference, unmodified
    from chainerkfac.optimizers import fisher_blocks as FB
    from chainerkfac.optimizers import kfac as KF
    from chainerkfac.optimizers.cholesky_inverse import inverse as ref_inverse

    cases = {}

    # -- Linear blocks (with and without bias; two steps to pin the EMA) ----
    for name, (n, din, dout, bias, decay, steps) in {
            'linear_bias': (16, 12, 7, True, 0.9, 2),
            'linear_nobias': (8, 20, 10, False, 1.0, 1),
            'linear_odd': (33, 37, 19, True, 0.5, 2)}.items():
        rng = np.random.default_rng(sum(map(ord, name)))
        xs, gys = [], []
        for _ in range(steps):
            x, gy, W, b, gW, gb = gen_linear(rng, n, din, dout, bias)
            xs.append(x)
            gys.append(gy)
        link = Linear(W, b)
        link.W.grad = gW
        if bias:
            link.b.grad = gb
        out = run_connection_block(FB, 'linear', link, xs, gys, 1e-3, decay,
                                   steps)
        out.update(dict(W=W, gW=gW, damping=np.float32(1e-3),
                        decay=np.float32(decay), steps=np.int32(steps)))
        if bias:
            out.update(b=b, gb=gb)
        for s in range(steps):
            out['x%d' % s] = xs[s]
            out['gy%d' % s] = gys[s]
        cases[name] = out

    # -- Convolution blocks -------------------------------------------------
    for name, (n, cin, cout, hw, k, s, p, bias, decay, steps) in {
            'conv3x3_bias': (4, 3, 5, 8, 3, 1, 1, True, 0.9, 2),
            'conv3x3_s2': (3, 4, 6, 9, 3, 2, 1, False, 1.0, 1),
            'conv1x1_s2': (2, 6, 8, 8, 1, 2, 0, False, 1.0, 1),
            'conv7x7_s2': (2, 3, 4, 16, 7, 2, 3, True, 1.0, 1)}.items():
        rng = np.random.default_rng(sum(map(ord, name)))
        ho = orc.conv_out_size(hw, k, s, p)
        xs, gys = [], []
        for _ in range(steps):
            x, W, b, gW, gb = gen_conv(rng, n, cin, cout, hw, k, bias)
            xs.append(x)
            gys.append(f32(rng.standard_normal((n, cout, ho, ho)) / n))
        link = Convolution2D(W, b, k, s, p)
        link.W.grad = gW
        if bias:
            link.b.grad = gb
        out = run_connection_block(FB, 'conv', link, xs, gys, 2.5e-4, decay,
                                   steps)
        out.update(dict(W=W, gW=gW, damping=np.float32(2.5e-4),
                        decay=np.float32(decay), steps=np.int32(steps),
                        ksize=np.int32(k), stride=np.int32(s),
                        pad=np.int32(p)))
        if bias:
            out.update(b=b, gb=gb)
        for st in range(steps):
            out['x%d' % st] = xs[st]
            out['gy%d' % st] = gys[st]
        cases[name] = out

    # -- BatchNormalization block ---------------------------------------------
    for name, (shape, stab) in {'bn_4d': ((6, 5, 4, 4), 16.0),
                                'bn_2d': ((12, 7), 64.0)}.items():
        rng = np.random.default_rng(sum(map(ord, name)))
        c = shape[1]
        x = f32(rng.standard_normal(shape) * 2 + 0.5)
        gy = f32(rng.standard_normal(shape) / shape[0])
        link = BatchNormalization(f32(rng.random(c) + 0.5),
                                  f32(rng.standard_normal(c)))
        link.gamma.grad = f32(rng.standard_normal(c))
        link.beta.grad = f32(rng.standard_normal(c))
        blk = FB.FisherBlockBatchNormalization(
            '/bn', link, cov_ema_decay=1.0, damping=1e-3, stab_coeff=stab)
        in_data = (x, link.gamma.data, link.beta.data)
        blk.backward_preprocess(None, in_data, (gy,))
        F = blk.cov_backward.copy()
        blk.update_cov_emas()
        blk.update_invs()
        blk.update_kfgrads()
        cases[name] = dict(
            x=x, gy=gy, eps=np.float32(link.eps), stab_coeff=np.float32(stab),
            damping=np.float32(1e-3), g_gamma=link.gamma.grad,
            g_beta=link.beta.grad, F=F,
            diag=np.float32(blk.diag_val_backward),
            F_inv=blk.inv_backward.copy(),
            kf_gamma=link.gamma.kfgrad.copy(),
            kf_beta=link.beta.kfgrad.copy())

    # -- the inverse alone, on a config-4-style SPD matrix ----------------------
    rng = np.random.default_rng(4)
    for d in (10, 65):
        X = f32(rng.standard_normal((256, d)))
        a = f32(X.T.dot(X) / 256 + 1e-3 * np.eye(d))
        cases['inverse_%d' % d] = dict(a=a, inv=ref_inverse(a.copy()))

    # -- a whole optimizer step on a small MLP (KFAC.update, lossfun=None) --
    rng = np.random.default_rng(1)
    n, dims = 16, (12, 9, 9, 5)

    class MLP(Link):
        def __init__(self):
            super(MLP, self).__init__()
            for i in range(3):
                self.add_link('l%d' % (i + 1), Linear(
                    f32(rng.standard_normal((dims[i + 1], dims[i])) * 0.3),
                    f32(rng.standard_normal(dims[i + 1]) * 0.1)))

    model = MLP()
    opt = KF.KFAC(lr=0.01, momentum=0.9, cov_ema_decay=1.0, damping=1e-3)
    opt.setup(model)
    out = {}
    for nm, p in model.namedparams():
        out['init' + nm.replace('/', '.')] = p.data.copy()
    x = f32(rng.random((n, dims[0])))
    t = rng.integers(0, dims[3], n)
    for step in range(2):
        # forward/backward of the MLP in NumPy, firing the hook like Chainer
        hs, acts = x, []
        lins = [model.l1, model.l2, model.l3]
        for i, l in enumerate(lins):
            in_data = (hs, l.W.data, l.b.data)
            opt.kfhook.forward_postprocess(LinearFunction(), in_data)
            z = hs.dot(l.W.data.T) + l.b.data
            acts.append((in_data, z))
            hs = np.maximum(z, 0) if i < 2 else z
        z = hs - hs.max(axis=1, keepdims=True)
        prob = np.exp(z) / np.exp(z).sum(axis=1, keepdims=True)
        gz = prob.copy()
        gz[np.arange(n), t] -= 1
        gz = f32(gz / n)
        model.cleargrads()
        for i in (2, 1, 0):
            in_data, z = acts[i]
            if i < 2:
                gz = f32(gz * (z > 0))
            opt.kfhook.backward_preprocess(LinearFunction(), in_data, (gz,))
            lins[i].W.grad = f32(gz.T.dot(in_data[0]))
            lins[i].b.grad = f32(gz.sum(axis=0))
            gz = f32(gz.dot(lins[i].W.data))
        for nm, p in model.namedparams():
            out['grad%d' % step + nm.replace('/', '.')] = p.grad.copy()
        opt.update()
        for nm, p in model.namedparams():
            out['kfgrad%d' % step + nm.replace('/', '.')] = p.kfgrad.copy()
            out['param%d' % step + nm.replace('/', '.')] = p.data.copy()
    out.update(x=x, t=t.astype(np.int64), lr=np.float32(0.01),
               momentum=np.float32(0.9), damping=np.float32(1e-3))
    cases['mlp_two_steps'] = out

    for name, arrays in cases.items():
        np.savez_compressed(os.path.join(HERE, name + '.npz'), **arrays)
        print('wrote', name, sum(np.asarray(v).nbytes
                                 for v in arrays.values()), 'bytes')


if __name__ == '__main__':
    main()
