"""Thin torch-tensor front end of the C ABI.

Every function takes CUDA fp32 tensors, passes their raw device pointers and
the current CUDA stream to ``libkfac_b200.so`` and returns torch tensors that
own the outputs.  Tensors are plumbing only: all arithmetic happens in the
library's kernels.
"""

import ctypes
import os

import torch

from . import _lib


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _chk(t, name):
    if t is None:
        return
    if not t.is_cuda:
        raise _lib.KfacLibraryError(
            '%s must be a CUDA tensor: this package has no CPU path' % name)
    if t.dtype != torch.float32:
        raise TypeError('%s must be float32, got %s' % (name, t.dtype))
    if not t.is_contiguous():
        raise ValueError('%s must be contiguous' % name)


class Workspace(object):
    """Grow-only device scratch buffers, one per (device, CUDA stream): two
    calls that run on different streams at the same time (a factor build on
    the exchange stream beside one on the main stream) must not share their
    partial tiles."""

    def __init__(self):
        self.bufs = {}

    def get(self, nbytes, device):
        nbytes = max(int(nbytes), 256)
        device = torch.device(device)
        key = (device, torch.cuda.current_stream(device).cuda_stream
               if device.type == 'cuda' else 0)
        buf = self.bufs.get(key)
        if buf is None or buf.numel() < nbytes:
            # allocated under the calling stream: the caching allocator
            # hands the old buffer on in that stream's order
            buf = self.bufs[key] = torch.empty(nbytes, dtype=torch.uint8,
                                               device=device)
        return buf


_factor_ws = Workspace()

def _is_nhwc(t):
    """4-D tensor stored channels-last (and not also plain NCHW-contiguous)."""
    return (t.dim() == 4 and not t.is_contiguous() and
            t.is_contiguous(memory_format=torch.channels_last))


def _nhwc_rows(t):
    """(n*h*w, c) view of a channels-last tensor: no copy."""
    n, c, h, w = t.shape
    return t.permute(0, 2, 3, 1).reshape(n * h * w, c)


def _conv_input_as_dense(x, ksize, stride, pad):
    """A channels-last input of a 1x1, stride-1, unpadded convolution is its
    own patch matrix."""
    return _is_nhwc(x) and ksize == 1 and stride == 1 and pad == 0



def _factor_out(d, out, beta, device):
    if out is None:
        if beta != 0.0:
            raise ValueError('beta != 0 needs an existing `out`')
        out = torch.empty((d, d), dtype=torch.float32, device=device)
    _chk(out, 'out')
    if tuple(out.shape) != (d, d):
        raise ValueError('out must be %dx%d' % (d, d))
    return out


def factor_dense(x, add_ones_col=False, alpha=1.0, beta=0.0, out=None):
    """out = alpha * [x,1]^T [x,1] + beta * out for a 2-D ``x``."""
    lib = _lib.load()
    _chk(x, 'x')
    rows, d_in = x.shape
    d = d_in + int(bool(add_ones_col))
    out = _factor_out(d, out, beta, x.device)
    nbytes = lib.kfac_factor_workspace_bytes(rows, d)
    ws = _factor_ws.get(nbytes, x.device)
    _lib.check(lib.kfac_factor_dense(
        _p(x), rows, d_in, x.stride(0), int(bool(add_ones_col)), alpha, beta,
        _p(out), _p(ws), ws.numel(), _stream()), 'kfac_factor_dense')
    return out


def factor_conv_input(x, ksize, stride, pad, add_ones_col=False, alpha=1.0,
                      beta=0.0, out=None):
    """out = alpha * P^T P + beta * out, P the im2col patches of ``x`` (NCHW;
    a channels-last tensor is read in place when it is its own patch matrix
    and copied to NCHW otherwise)."""
    lib = _lib.load()
    if _conv_input_as_dense(x, ksize, stride, pad):
        return factor_dense(_nhwc_rows(x), add_ones_col, alpha, beta, out)
    if _is_nhwc(x):
        x = x.contiguous()
    _chk(x, 'x')
    n, c, h, w = x.shape
    ho = (h + 2 * pad - ksize) // stride + 1
    wo = (w + 2 * pad - ksize) // stride + 1
    d = c * ksize * ksize + int(bool(add_ones_col))
    out = _factor_out(d, out, beta, x.device)
    nbytes = lib.kfac_factor_conv_workspace_bytes(
        n, c, h, w, ksize, stride, pad, int(bool(add_ones_col)))
    ws = _factor_ws.get(nbytes, x.device)
    _lib.check(lib.kfac_factor_conv_input(
        _p(x), n, c, h, w, ksize, stride, pad, int(bool(add_ones_col)), alpha,
        beta, _p(out), _p(ws), ws.numel(), _stream()),
        'kfac_factor_conv_input')
    return out


def factor_conv_grad(gy, alpha=1.0, beta=0.0, out=None):
    """out = alpha * g^T g + beta * out, g = ``gy`` as (n*ho*wo, c); NCHW, or
    channels-last (then g is the tensor itself, read in place)."""
    lib = _lib.load()
    if _is_nhwc(gy):
        return factor_dense(_nhwc_rows(gy), False, alpha, beta, out)
    _chk(gy, 'gy')
    n, c, ho, wo = gy.shape
    out = _factor_out(c, out, beta, gy.device)
    nbytes = lib.kfac_factor_workspace_bytes(n * ho * wo, c)
    ws = _factor_ws.get(nbytes, gy.device)
    _lib.check(lib.kfac_factor_conv_grad(
        _p(gy), n, c, ho, wo, alpha, beta, _p(out), _p(ws), ws.numel(),
        _stream()), 'kfac_factor_conv_grad')
    return out


def dense_item(x, add_ones_col, alpha, beta, out):
    _chk(x, 'x')
    _chk(out, 'out')
    it = _lib.FactorItem()
    it.kind, it.add_ones_col = 0, int(bool(add_ones_col))
    it.x, it.rows, it.ld, it.d_in = x.data_ptr(), x.shape[0], x.stride(0), \
        x.shape[1]
    it.alpha, it.beta, it.out = alpha, beta, out.data_ptr()
    it._keep = (locals().get('x', None), locals().get('gy', None), out)
    return it


def dense_t_item(x, alpha, beta, out):
    """Item for out = alpha * x x^T + beta * out with ``x`` (d, rows)
    row-major: the contraction runs along x's rows."""
    _chk(x, 'x')
    _chk(out, 'out')
    it = _lib.FactorItem()
    it.kind, it.add_ones_col = 3, 0
    it.x, it.d_in, it.rows, it.ld = x.data_ptr(), x.shape[0], x.shape[1], \
        x.stride(0)
    it.alpha, it.beta, it.out = alpha, beta, out.data_ptr()
    it._keep = (x, out)
    return it


def conv_input_item(x, ksize, stride, pad, add_ones_col, alpha, beta, out):
    if _conv_input_as_dense(x, ksize, stride, pad):
        return dense_item(_nhwc_rows(x), add_ones_col, alpha, beta, out)
    layout = 0
    if _is_nhwc(x):
        if _lib.load().kfac_get_engine() == 1:
            layout = 1       # the staging copy reads channels-last directly
        else:
            x = x.contiguous()
    if layout == 0:
        _chk(x, 'x')
    elif not x.is_cuda or x.dtype != torch.float32:
        raise TypeError('x must be a float32 CUDA tensor')
    _chk(out, 'out')
    it = _lib.FactorItem()
    it.layout = layout
    it.kind, it.add_ones_col = 1, int(bool(add_ones_col))
    it.x = x.data_ptr()
    it.n, it.c, it.h, it.w = x.shape
    it.ksize, it.stride, it.pad = ksize, stride, pad
    it.alpha, it.beta, it.out = alpha, beta, out.data_ptr()
    it._keep = (locals().get('x', None), locals().get('gy', None), out)
    return it


def conv_grad_item(gy, alpha, beta, out):
    if _is_nhwc(gy):
        return dense_item(_nhwc_rows(gy), False, alpha, beta, out)
    _chk(gy, 'gy')
    _chk(out, 'out')
    it = _lib.FactorItem()
    it.kind = 2
    it.x = gy.data_ptr()
    it.n, it.c, it.h, it.w = gy.shape
    it.alpha, it.beta, it.out = alpha, beta, out.data_ptr()
    it._keep = (locals().get('x', None), locals().get('gy', None), out)
    return it


_group_ws = Workspace()


def factor_group(items, device):
    """Build all given factors (see *_item) in one grouped call."""
    lib = _lib.load()
    arr = (_lib.FactorItem * len(items))(*items)
    nbytes = lib.kfac_factor_group_workspace_bytes(len(items), arr)
    ws = _group_ws.get(nbytes, device)
    _lib.check(lib.kfac_factor_group(len(items), arr, _p(ws), ws.numel(),
                                     _stream()), 'kfac_factor_group')


def bn_item(x, gy, eps, scale, out=None, stats=None):
    """Item of ``bn_sample_grads_group`` for one BatchNormalization layer:
    ``x`` / ``gy`` are (n, c) or (n, c, h, w) tensors, NCHW-contiguous or
    channels-last (both must have the same layout)."""
    if not (x.is_cuda and x.dtype == torch.float32 and
            gy.dtype == torch.float32):
        raise TypeError('x and gy must be float32 CUDA tensors')
    n, c = x.shape[0], x.shape[1]
    hw = 1
    for s in x.shape[2:]:
        hw *= s
    layout = 0
    if _is_nhwc(x) or _is_nhwc(gy):
        # one common layout: channels-last if either is
        x = x.contiguous(memory_format=torch.channels_last)
        gy = gy.contiguous(memory_format=torch.channels_last)
        layout = 1
    else:
        _chk(x, 'x')
        _chk(gy, 'gy')
    if out is None or tuple(out.shape) != (n, 2 * c) or out.device != x.device:
        out = torch.empty((n, 2 * c), dtype=torch.float32, device=x.device)
    it = _lib.BnItem()
    it.x, it.gy, it.out = x.data_ptr(), gy.data_ptr(), out.data_ptr()
    need = 2 * c + 4 * n * c     # statistics, then per-sample double sums
    if stats is None or stats.numel() != need or stats.device != x.device:
        stats = torch.empty(need, dtype=torch.float32, device=x.device)
    it.stats = stats.data_ptr()
    it.n, it.c, it.hw, it.layout = n, c, hw, layout
    it.eps, it.scale = eps, scale
    it._keep = (x, gy, out, stats)
    it.result = out
    return it


def bn_sample_grads_group(items):
    """Per-sample gradients of all given layers (see bn_item), two launches."""
    if not items:
        return
    lib = _lib.load()
    for k in range(0, len(items), 256):
        part = items[k:k + 256]
        arr = (_lib.BnItem * len(part))(*part)
        _lib.check(lib.kfac_bn_sample_grads_group(len(part), arr, _stream()),
                   'kfac_bn_sample_grads_group')


def bn_sample_grads(x, gy, eps, scale):
    """(n, 2c) per-sample gradients of the BatchNormalization scale/shift."""
    it = bn_item(x, gy, eps, scale)
    bn_sample_grads_group([it])
    return it.result


def bn_precondition_group(F_inv, grad_gamma, grad_beta, kf_gamma, kf_beta,
                          nan_flags, param_gamma=None, param_beta=None,
                          mom_gamma=None, mom_beta=None, lr=0.0, momentum=0.0):
    """kf = F_inv [grad_gamma; grad_beta] for lists of blocks, with the NaN
    fallback and the optional fused momentum update (kfac_b200.h)."""
    if not F_inv:
        return
    lib = _lib.load()

    def ptrs(lst, lo, hi):
        if lst is None:
            return None
        return _lib.ptr_array([None if t is None else t.data_ptr()
                               for t in lst[lo:hi]])
    for lst in (F_inv, grad_gamma, grad_beta, kf_gamma, kf_beta):
        for t in lst:
            _chk(t, 'bn_precondition_group argument')
    for lo in range(0, len(F_inv), 256):
        hi = min(lo + 256, len(F_inv))
        _lib.check(lib.kfac_bn_precondition_group(
            hi - lo, _lib.int_array([g.numel() for g in grad_gamma[lo:hi]]),
            ptrs(F_inv, lo, hi), ptrs(grad_gamma, lo, hi),
            ptrs(grad_beta, lo, hi), ptrs(kf_gamma, lo, hi),
            ptrs(kf_beta, lo, hi), ptrs(param_gamma, lo, hi),
            ptrs(param_beta, lo, hi), ptrs(mom_gamma, lo, hi),
            ptrs(mom_beta, lo, hi), ptrs(nan_flags, lo, hi), lr, momentum,
            _stream()), 'kfac_bn_precondition_group')


def bn_lowrank_item(hist, scaled, c, rows_per_slot, slot_weights, damp_gamma,
                    damp_beta, m_inv=None, grad_gamma=None, grad_beta=None,
                    kf_gamma=None, kf_beta=None, nan_flag=None,
                    param_gamma=None, param_beta=None, mom_gamma=None,
                    mom_beta=None):
    """struct kfac_bn_lowrank_item for one BatchNormalization block (see
    include/kfac_b200.h)."""
    it = _lib.BnLowRankItem()
    keep = []
    for name, t in (('hist', hist), ('scaled', scaled), ('m_inv', m_inv),
                    ('grad_gamma', grad_gamma), ('grad_beta', grad_beta),
                    ('kf_gamma', kf_gamma), ('kf_beta', kf_beta),
                    ('param_gamma', param_gamma), ('param_beta', param_beta),
                    ('mom_gamma', mom_gamma), ('mom_beta', mom_beta),
                    ('nan_flag', nan_flag)):
        if t is not None:
            if name != 'nan_flag':
                _chk(t, name)
            setattr(it, name, t.data_ptr())
            keep.append(t)
    it.c, it.rows_per_slot, it.slots = c, rows_per_slot, len(slot_weights)
    it.damp_gamma, it.damp_beta = damp_gamma, damp_beta
    for k, w in enumerate(slot_weights):
        it.slot_weight[k] = w
    it._keep = keep
    return it


def bn_lowrank_scale(items):
    if not items:
        return
    lib = _lib.load()
    arr = (_lib.BnLowRankItem * len(items))(*items)
    _lib.check(lib.kfac_bn_lowrank_scale(len(items), arr, _stream()),
               'kfac_bn_lowrank_scale')


def bn_lowrank_apply(items, lr=0.0, momentum=0.0):
    if not items:
        return
    lib = _lib.load()
    arr = (_lib.BnLowRankItem * len(items))(*items)
    _lib.check(lib.kfac_bn_lowrank_apply(len(items), arr, lr, momentum,
                                         _stream()), 'kfac_bn_lowrank_apply')


def axpby(a, x, b, y, out):
    """out = a*x + b*y (out may be y)."""
    lib = _lib.load()
    for t, nm in ((x, 'x'), (y, 'y'), (out, 'out')):
        _chk(t, nm)
    _lib.check(lib.kfac_axpby(x.numel(), a, _p(x), b, _p(y), _p(out),
                              _stream()), 'kfac_axpby')
    return out


def axpby_group(a, xs, b, ys, outs):
    """outs[i] = a*xs[i] + b*ys[i] for lists of tensors, in one launch."""
    if not xs:
        return
    lib = _lib.load()
    for lst in (xs, ys, outs):
        for t in lst:
            _chk(t, 'axpby_group argument')
    counts = (ctypes.c_int64 * len(xs))(*[int(t.numel()) for t in xs])
    _lib.check(lib.kfac_axpby_group(
        len(xs), counts, a, _lib.ptr_array([t.data_ptr() for t in xs]), b,
        _lib.ptr_array([t.data_ptr() for t in ys]),
        _lib.ptr_array([t.data_ptr() for t in outs]), _stream()),
        'kfac_axpby_group')


class InversePlan(object):
    """Batched damped inverse of a fixed set of factor buffers."""

    def __init__(self, factors, inverses, partner, role, l2_coef=None,
                 scale=None, l2_coef_second=None):
        lib = _lib.load()
        self._lib = lib
        self.count = len(factors)
        for t in list(factors) + list(inverses):
            _chk(t, 'factor/inverse')
        dims = [int(f.shape[0]) for f in factors]
        self.dims = dims
        self.factors, self.inverses = list(factors), list(inverses)
        device = factors[0].device
        dims_c = _lib.int_array(dims)
        nbytes = lib.kfac_inverse_workspace_bytes(self.count, dims_c)
        self.workspace = torch.empty(max(nbytes, 256), dtype=torch.uint8,
                                     device=device)
        self.info = torch.zeros(self.count, dtype=torch.int32, device=device)
        self.diag = torch.zeros(self.count, dtype=torch.float32, device=device)
        handle = ctypes.c_void_p()
        _lib.check(lib.kfac_inverse_plan_create(
            self.count, dims_c,
            _lib.ptr_array([f.data_ptr() for f in factors]),
            _lib.ptr_array([f.data_ptr() for f in inverses]),
            _lib.int_array(partner), _lib.int_array(role),
            _lib.float_array(l2_coef if l2_coef is not None
                             else [0.0] * self.count),
            _lib.float_array(scale if scale is not None
                             else [1.0] * self.count),
            _p(self.workspace), self.workspace.numel(),
            ctypes.byref(handle)), 'kfac_inverse_plan_create')
        self._handle = handle
        if l2_coef_second is not None and any(r == 2 for r in role):
            _lib.check(lib.kfac_inverse_plan_set_second_floor(
                handle, _lib.float_array(l2_coef_second)),
                'kfac_inverse_plan_set_second_floor')
        refine = os.environ.get('KFAC_REFINE_MAX_DIM')
        if refine is not None:
            self.set_refine(int(refine))

    def set_refine(self, max_dim, threshold=3e-5):
        """Refinement of ill-conditioned factors of up to ``max_dim`` rows
        (0: off); see kfac_inverse_plan_set_refine."""
        _lib.check(self._lib.kfac_inverse_plan_set_refine(
            self._handle, int(max_dim), float(threshold)),
            'kfac_inverse_plan_set_refine')

    def error_estimates(self):
        """Probe estimate of each inverse's relative error before refinement
        in the last run (-1: not probed).  Synchronises."""
        out = (ctypes.c_float * self.count)()
        _lib.check(self._lib.kfac_inverse_plan_error_estimates(
            self._handle, out), 'kfac_inverse_plan_error_estimates')
        return list(out)

    def refined(self):
        """Number of factors the last run refined (synchronises)."""
        n = ctypes.c_int(0)
        _lib.check(self._lib.kfac_inverse_plan_refined(
            self._handle, ctypes.byref(n)), 'kfac_inverse_plan_refined')
        return n.value

    def run(self, damping, use_pi=True):
        _lib.check(self._lib.kfac_inverse_plan_run(
            self._handle, damping, int(bool(use_pi)),
            ctypes.c_void_p(self.info.data_ptr()),
            ctypes.c_void_p(self.diag.data_ptr()), _stream()),
            'kfac_inverse_plan_run')

    def close(self):
        if getattr(self, '_handle', None) is not None and self._handle:
            self._lib.kfac_inverse_plan_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def class_bounds():
    """Sides that separate the size classes of an InversePlanSet (environment
    variable KFAC_CLASS_BOUNDS, default 1024,3000)."""
    return tuple(int(b) for b in os.environ.get(
        'KFAC_CLASS_BOUNDS', '1024,3000').split(','))


class InversePlanSet(object):
    """Several InversePlans over disjoint subsets of (factor, inverse) pairs,
    run on separate CUDA streams.  The long serial chain of diagonal-block
    steps of the largest matrices leaves most SMs idle; running the other
    size classes next to it fills them.  Pairs (forward/backward factor of one
    layer) stay in one plan so that pi sees both traces."""

    def __init__(self, factors, inverses, partner, role, l2_coef=None,
                 scale=None, bounds=None, l2_coef_second=None):
        n = len(factors)
        if bounds is None:
            bounds = class_bounds()
        l2_coef = l2_coef if l2_coef is not None else [0.0] * n
        scale = scale if scale is not None else [1.0] * n
        second = l2_coef_second if l2_coef_second is not None else l2_coef

        def size_class(i):
            d = max(factors[i].shape[0],
                    factors[partner[i]].shape[0] if partner[i] >= 0 else 0)
            return sum(d > b for b in bounds)
        groups = {}
        for i in range(n):
            groups.setdefault(size_class(i), []).append(i)
        self.plans, self.index, self.class_keys = [], [], []
        self.bounds = tuple(bounds)
        for key, idx in sorted(groups.items(), reverse=True):
            self.class_keys.append(key)
            pos = {g: j for j, g in enumerate(idx)}
            self.plans.append(InversePlan(
                [factors[i] for i in idx], [inverses[i] for i in idx],
                [pos[partner[i]] if partner[i] >= 0 else -1 for i in idx],
                [role[i] for i in idx], [l2_coef[i] for i in idx],
                [scale[i] for i in idx], [second[i] for i in idx]))
            self.index.append(idx)
        self.streams = [torch.cuda.Stream() for _ in self.plans[1:]]
        # optional early start of a class (see start_class)
        self.early_streams = [torch.cuda.Stream(priority=-1)
                              for _ in self.plans]
        self._early = {}
        self.count = n
        dev = factors[0].device
        self._perm = [torch.tensor(idx, device=dev) for idx in self.index]

    def classes(self):
        """Index lists (caller's order) of the size classes, largest first."""
        return [list(idx) for idx in self.index]

    def start_class(self, c, damping, use_pi=True):
        """Start the plan of size class ``c`` now, on its own high-priority
        side stream, ordered after the work queued so far on the current
        stream.  The long serial chains of the large classes then overlap
        whatever the caller queues next (typically the factor build of the
        other layers); ``run`` later skips started classes and joins their
        streams.  Only legal once the factors of that class are final."""
        cur = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(cur)
        st = self.early_streams[c]
        st.wait_event(ready)
        with torch.cuda.stream(st):
            self.plans[c].run(damping, use_pi)
            ev = torch.cuda.Event()
            ev.record(st)
        self._early[c] = ev

    def run(self, damping, use_pi=True, after_class=None, join=True):
        """Run every class not started yet and join all of them.
        ``after_class(c)``, if given, is called on class c's stream right
        after its plan (its kernels then overlap the other classes'
        inverses); it must only touch data of that class.  With
        ``join=False`` the current stream does not wait for the classes on
        side streams: the call returns {class: event} for them and the
        caller orders later work after those events itself."""
        cur = torch.cuda.current_stream()
        start = torch.cuda.Event()
        start.record(cur)
        rest = [c for c in range(len(self.plans)) if c not in self._early]
        for c, st in zip(rest[1:], self.streams):
            st.wait_event(start)
            with torch.cuda.stream(st):
                self.plans[c].run(damping, use_pi)
                if after_class is not None:
                    after_class(c)
        if after_class is not None:
            for c in self._early:
                # what the caller queued on the current stream since the
                # class was started (optimizer pre-hooks on the gradients,
                # for instance) comes before the class's follow-up work
                self.early_streams[c].wait_event(start)
                with torch.cuda.stream(self.early_streams[c]):
                    after_class(c)
                    ev = torch.cuda.Event()
                    ev.record(self.early_streams[c])
                self._early[c] = ev
        if rest:
            self.plans[rest[0]].run(damping, use_pi)
            if after_class is not None:
                after_class(rest[0])
        pending = {}
        for c, st in zip(rest[1:], self.streams):
            done = torch.cuda.Event()
            done.record(st)
            pending[c] = done
        pending.update(self._early)
        self._early = {}
        if not join:
            return pending
        for ev in pending.values():
            cur.wait_event(ev)
        return {}

    def set_refine(self, max_dim, threshold=3e-5):
        for p in self.plans:
            p.set_refine(max_dim, threshold)

    def refined(self):
        return sum(p.refined() for p in self.plans)

    def gather(self, attr):
        """Per-factor values (info / diag) in the caller's original order."""
        first = getattr(self.plans[0], attr)
        out = torch.empty(self.count, dtype=first.dtype, device=first.device)
        for plan, idx in zip(self.plans, self.index):
            out[self._perm[self.plans.index(plan)]] = getattr(plan, attr)
        return out

    @property
    def info(self):
        return self.gather('info')

    @property
    def diag(self):
        return self.gather('diag')

    def close(self):
        for p in self.plans:
            p.close()


_precond_ws = {}


def precondition(G_inv, A_inv, grad_W, grad_b, kf_W=None, kf_b=None,
                 param_W=None, param_b=None, mom_W=None, mom_b=None, lr=0.0,
                 momentum=0.0, ws_key=None):
    """Grouped kf = G_inv [grad_W, grad_b] A_inv over lists of layers, with
    the optional fused momentum update (see include/kfac_b200.h)."""
    lib = _lib.load()
    count = len(G_inv)
    dG = [int(g.shape[0]) for g in G_inv]
    dW = [int(w.numel() // w.shape[0]) for w in grad_W]
    hb = [0 if b is None else 1 for b in grad_b]

    def ptrs(lst):
        if lst is None:
            return None
        for t in lst:
            _chk(t, 'precondition argument')
        return _lib.ptr_array([None if t is None else t.data_ptr()
                               for t in lst])
    nbytes = lib.kfac_precond_workspace_bytes(
        count, _lib.int_array(dG), _lib.int_array(dW), _lib.int_array(hb))
    # calls that may overlap on different streams pass different keys
    ws = _precond_ws.setdefault(ws_key, Workspace()).get(
        nbytes, G_inv[0].device)
    _lib.check(lib.kfac_precondition(
        count, _lib.int_array(dG), _lib.int_array(dW), ptrs(G_inv),
        ptrs(A_inv), ptrs(grad_W), ptrs(grad_b), ptrs(kf_W), ptrs(kf_b),
        ptrs(param_W), ptrs(param_b), ptrs(mom_W), ptrs(mom_b), lr, momentum,
        _p(ws), ws.numel(), _stream()), 'kfac_precondition')


def symv_split(m, x0, x1, y0, y1, nan_flag=None):
    lib = _lib.load()
    d = int(m.shape[0])
    _lib.check(lib.kfac_symv_split(
        _p(m), d, x0.numel(), _p(x0), _p(x1), _p(y0), _p(y1),
        None if nan_flag is None else ctypes.c_void_p(nan_flag.data_ptr()),
        _stream()), 'kfac_symv_split')


def momentum_update(grad, param, v, lr, momentum):
    lib = _lib.load()
    for t, nm in ((grad, 'grad'), (param, 'param'), (v, 'v')):
        _chk(t, nm)
    _lib.check(lib.kfac_momentum_update(param.numel(), _p(grad), _p(param),
                                        _p(v), lr, momentum, _stream()),
               'kfac_momentum_update')


def normalize_weight(w, target_norm, eps=1e-9, scratch=None):
    """In-place w *= target_norm / (|w| + eps) if that is below 1; returns the
    two-float device scratch (|w|^2 before, factor)."""
    lib = _lib.load()
    _chk(w, 'w')
    if scratch is None:
        scratch = torch.empty(2, dtype=torch.float32, device=w.device)
    _lib.check(lib.kfac_normalize_weight(w.numel(), _p(w), target_norm, eps,
                                         _p(scratch), _stream()),
               'kfac_normalize_weight')
    return scratch


def _wire_args(arrays, tri, select):
    nelems = [int(a.numel()) for a in arrays]
    tri_dim = [int(a.shape[0]) if t else 0 for a, t in zip(arrays, tri)]
    sel = None if select is None else _lib.int_array(select)
    return (len(arrays), _lib.ptr_array([a.data_ptr() for a in arrays]),
            _lib.i64_array(nelems), _lib.int_array(tri_dim), sel)


def wire_nelems(arrays, tri):
    lib = _lib.load()
    n, _, nelems, tri_dim, _ = _wire_args(arrays, tri, None)
    return int(lib.kfac_wire_nelems(n, nelems, tri_dim))


WIRE_DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def wire_pack(arrays, tri, wire, select=None, zero_skipped=False):
    """Pack into ``wire`` (fp32, or fp16 / bf16 for a reduced-precision
    wire)."""
    lib = _lib.load()
    n, ptrs, nelems, tri_dim, sel = _wire_args(arrays, tri, select)
    _lib.check(lib.kfac_wire_pack_as(
        WIRE_DTYPES[wire.dtype], n, ptrs, nelems, tri_dim, sel,
        int(bool(zero_skipped)), ctypes.c_void_p(wire.data_ptr()), _stream()),
        'kfac_wire_pack_as')


def wire_unpack_sum(arrays, tri, wire_ptrs, select=None, scale=1.0,
                    ema_r=-1.0, wire_dtype=torch.float32):
    """Unpack the sum of several wire buffers given as raw device addresses
    (this GPU's buffer and peer mappings of the other ranks' buffers)."""
    lib = _lib.load()
    n, ptrs, nelems, tri_dim, sel = _wire_args(arrays, tri, select)
    _lib.check(lib.kfac_wire_unpack_sum_as(
        WIRE_DTYPES[wire_dtype], n, ptrs, nelems, tri_dim, sel, scale, ema_r,
        _lib.ptr_array([int(q) for q in wire_ptrs]), len(wire_ptrs),
        _stream()), 'kfac_wire_unpack_sum_as')


def wire_unpack(arrays, tri, wire, select=None, scale=1.0, ema_r=-1.0):
    wire_unpack_sum(arrays, tri, [wire.data_ptr()], select, scale, ema_r,
                    wire_dtype=wire.dtype)
