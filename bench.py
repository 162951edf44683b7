#!/usr/bin/env python
"""Benchmark of the K-FAC curvature hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload resnet50|config1|config2|config4|config5]

Default workload (``config.workload`` = resnet50_kfac_step_b32_224): one K-FAC
step of a vanilla ResNet-50 at batch 32 per GPU, 224x224 inputs -- for each of
its 54 convolution / fully-connected layers the two Kronecker factors are built
from the layer's input activations and output gradients with the running
average fused in (decay 0.9), all 108 factors are inverted with pi-split
damping 2.5e-4, and the gradients are preconditioned and applied with
momentum.  Activations and gradients are synthetic (seeded) tensors of the
real shapes; ImageNet is not used.  The other workloads are the remaining
benchmark configurations with the same stages: the MNIST-shaped MLP (config1),
the CIFAR ResNet-18 at batch 128 (config2), the isolated curvature microbench
of 54 prebuilt factor pairs (config4: inverse + precondition only) and
ResNet-50 with 16 accumulation micro-steps per update (config5).

``value`` is images/sec with activations/gradients resident in HBM; ``e2e`` is
images/sec of the optimizer's public ``update(lossfun, x, t)`` call with the
image batch coming from pinned host memory and the loss read back.  Rank 0
prints one JSON line.  ``--impl reference`` times the reference's CPU (NumPy)
arithmetic for the same stages through the oracle restatement on the host
cores, whole passes over all layers until a time budget is used.
"""

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import bench_workloads as bw  # noqa: E402

LR = 0.01
MOMENTUM = 0.9
COMMUNICATOR = 'peer_memory'   # or 'pure_nccl' (NCCL reduce / broadcast)
OVERLAP = True           # start the largest factors' inverse during the factor build
OWNERSHIP = 'balanced'   # layer ownership at N > 1 ('reference': by count)

# name -> layer table, per-GPU batch, running-average decay (r on the new
# sample), damping, accumulation micro-steps per update
WORKLOADS = {
    'resnet50': dict(name='resnet50_kfac_step_b32_224',
                     layers=lambda: bw.resnet50_layers(batch=32), batch=32,
                     decay=0.9, damping=2.5e-4, acc=1, bn=True),
    'config1': dict(name='mlp_784_1000_1000_10_kfac_step_b128',
                    layers=lambda: bw.mlp_layers(batch=128), batch=128,
                    decay=0.99, damping=1e-3, acc=1),
    'config2': dict(name='cifar_resnet18_kfac_step_b128_32',
                    layers=lambda: bw.resnet18_cifar_layers(batch=128),
                    batch=128, decay=0.99, damping=1e-3, acc=1, bn=True),
    'config4': dict(name='curvature_microbench_54_pairs_m8192',
                    layers=lambda: bw.resnet50_layers(batch=32), batch=32,
                    decay=1.0, damping=0.0, acc=1, prebuilt=8192),
    'config5': dict(name='resnet50_kfac_acc16_b32_224',
                    layers=lambda: bw.resnet50_layers(batch=32), batch=32,
                    decay=0.9, damping=2.5e-4, acc=16, bn=True),
}

# DRAM bytes of single launches measured with ncu on small cases (the
# full-size grouped launches are too large for a multi-pass capture); the
# bench scales them by the algorithmic work of its own launches.
# stage: (case, measured bytes, algorithmic bytes, algorithmic flops)
TRAFFIC_CASES = {
    'factor': ('conv3x3_c256_hw14 (tc_pair_kernel)', 33.9e6, 29.4e6,
               32 * 14 * 14 * 2304 * 2305.0),
    'inverse': None,
    'precondition': None,
}


def algorithmic_flops(layers, prebuilt=False, lowrank=None):
    """Flops per step per GPU: one triangle of each factor, d^3 per inverse,
    two products per preconditioned gradient (one matrix-vector product for a
    BatchNormalization block).  `lowrank` maps the index of a
    BatchNormalization block held in low-rank form to its history rows m:
    the triangle of the m x m matrix Hs Hs^T over 2c columns, m^3 for its
    inverse, two m x 2c matrix-vector products to apply it."""
    factor = inverse = precond = 0.0
    for i, l in enumerate(layers):
        if lowrank and i in lowrank:
            m, d = lowrank[i], 2 * l['c']
            factor += float(d) * m * (m + 1)
            inverse += float(m) ** 3
            precond += 4.0 * m * d + 2.0 * m * m
            continue
        for d, rows in bw.block_factors(l):
            if not prebuilt:
                factor += float(rows) * d * (d + 1)
            inverse += float(d) ** 3
        if l['kind'] == 'bn':
            precond += 2.0 * (2 * l['c']) ** 2
        else:
            dA, dG, _, _ = bw.layer_dims(l)
            precond += 2.0 * dG * dG * dA + 2.0 * dG * dA * dA
    return dict(factor=factor, inverse=inverse, precondition=precond)


def algorithmic_bytes(layers, prebuilt=False, lowrank=None):
    """Minimum DRAM bytes per step per GPU: each un-expanded input once and
    each factor written once (plus read for the running average); factor read
    + inverse written; inverses, gradient, result.  A low-rank
    BatchNormalization block (`lowrank`: index -> history rows m) reads its
    input, writes n new history rows, writes and reads the scaled history and
    writes the m x m matrix; its inverse reads and writes m x m; applying it
    reads the inverse and the scaled history twice."""
    factor = inverse = precond = 0.0
    for i, l in enumerate(layers):
        if lowrank and i in lowrank:
            m, d = lowrank[i], 2 * l['c']
            factor += 4.0 * (2 * l['n'] * l['c'] * l['h'] ** 2 + l['n'] * d +
                             3 * m * d + m * m)
            inverse += 4.0 * 2 * m * m
            precond += 4.0 * (m * m + 2 * m * d + 4 * l['c'])
            continue
        sides = [d for d, _ in bw.block_factors(l)]
        sq = sum(d * d for d in sides)
        if not prebuilt:
            if l['kind'] == 'bn':
                src = 2 * l['n'] * l['c'] * l['h'] ** 2
            elif l['kind'] == 'conv':
                src = l['n'] * (l['cin'] * l['hin'] ** 2 +
                                l['cout'] * l['hout'] ** 2)
            else:
                src = l['n'] * (l['cin'] + l['cout'])
            factor += 4.0 * (src + 2 * sq)
        inverse += 4.0 * 2 * sq
        if l['kind'] == 'bn':
            precond += 4.0 * (sq + 4 * l['c'])
        else:
            dA, dG, _, _ = bw.layer_dims(l)
            precond += 4.0 * (sq + 3 * dG * dA)
    return dict(factor=factor, inverse=inverse, precondition=precond)


def measure_tf32_peak(device):
    """Dense TF32 matmul throughput (8192^3, best of 10), measured the way the
    bf16 figure of MEASURED_PEAKS.json was: the fp32 data of this path can at
    best run at this rate (a third of it with the split-TF32 scheme)."""
    import torch
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.randn(8192, 8192, device=device)
        b = torch.randn(8192, 8192, device=device)
        torch.matmul(a, b)
        best = float('inf')
        for _ in range(10):
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2 * 8192 ** 3 / (best * 1e-3) / 1e12
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


def measured_peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p['hbm_gbs'], tflops=p['bf16_tflops_sustained'],
                    tflops_burst=p['bf16_tflops'], source='measured')
    return dict(hbm_gbs=6650.0, tflops=1400.0, tflops_burst=1590.0,
                source='fallback')


# ---------------------------------------------------------------- clocks
class ClockSampler(object):
    """nvidia-smi clock / throttle-reason samples during the timed region."""

    QUERY = ('clocks.sm,clocks.max.sm,power.draw,'
             'clocks_event_reasons.hw_slowdown,'
             'clocks_event_reasons.hw_thermal_slowdown,'
             'clocks_event_reasons.sw_thermal_slowdown,'
             'clocks_event_reasons.sw_power_cap')

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ['nvidia-smi', '-i', str(self.index),
                 '--query-gpu=' + self.QUERY, '--format=csv,noheader,nounits',
                 '-lms', '50'], stdout=subprocess.PIPE,
                stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, t0, t1, label):
        """Summary of the samples read between host times t0 and t1."""
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=['unsampled'])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, smax, power, reasons = [], [], [], set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown',
                 'sw_power_cap']
        for ts, line in self.lines:
            if not (t0 <= ts <= t1):
                continue
            parts = [p.strip() for p in line.split(',')]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[3:7]):
                if val.lower().startswith('active'):
                    reasons.add(nm)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=['unsampled'])
        return dict(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(smax)),
                    power_w_max=float(max(power)), samples=len(sm),
                    window=label, reasons=sorted(reasons))


# ------------------------------------------------------------- GPU workload
STAB_COEFF = 16.0      # BatchNormalization blocks: damping * stab_coeff


class DeviceWorkload(object):
    """Synthetic per-layer activations, output gradients, weights and K-FAC
    state of one benchmark configuration, resident on one GPU.

    A *block* is a layer with curvature: a convolution / fully-connected layer
    (two factors A, G; parameters W [, b]) or a BatchNormalization layer (one
    factor F of side 2c; parameters gamma, beta).  Factors live in flat lists
    (`ema`, `inv`, ...); `fidx[i]` lists the factor indices of block i."""

    def __init__(self, device, seed, spec, bn_blocks=True, bn_lowrank=True,
                 world=1, rank=0):
        import torch
        from chainerkfac_b200 import ops
        from chainerkfac_b200.optimizers.fisher_blocks.normalizations \
            .batch_normalization import lowrank_window
        self.torch, self.ops, self.spec = torch, ops, spec
        self.world, self.rank = world, rank
        self.layers = spec['layers']()
        self.decay, self.damping = spec['decay'], spec['damping']
        self.acc = spec['acc']
        self.prebuilt = spec.get('prebuilt')
        if bn_blocks and spec.get('bn') and not self.prebuilt:
            self.layers = self.layers + bw.bn_layers_of(self.layers)
        self.dims = [bw.layer_dims(l) for l in self.layers]
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        nl = len(self.layers)
        self.x, self.gy = [None] * nl, [None] * nl
        # parameters, gradients, velocities per block: [W, b] or [gamma, beta]
        self.P, self.gP, self.vP = [], [], []
        self.ema, self.inv, self.fidx = [], [], []
        self.bn_grads, self.bn_kf = [None] * nl, [None] * nl
        self.bn_stats = {}
        # low-rank form of a BatchNormalization block (kfac_bn_lowrank_*):
        # when the per-sample gradients of the steps the running average
        # still remembers number fewer than half the factor's side
        self.lr_slots = lowrank_window(self.decay) if (
            bn_lowrank and self.acc == 1) else 0
        self.lowrank = [False] * nl
        self.lr = {}
        for i, l in enumerate(self.layers):
            n = l['n']
            if l['kind'] == 'bn':
                xs = gs = (n, l['c'], l['h'], l['h'])
                shapes = [(l['c'],), (l['c'],)]
                sides = [2 * l['c']]
                m = self.lr_slots * n * world
                if self.lr_slots and m <= l['c']:
                    self.lowrank[i] = True
                    sides = []
            elif l['kind'] == 'conv':
                xs = (n, l['cin'], l['hin'], l['hin'])
                gs = (n, l['cout'], l['hout'], l['hout'])
                shapes = [(l['cout'], l['cin'], l['k'], l['k'])]
                sides = list(self.dims[i][:2])
            else:
                xs, gs = (n, l['cin']), (n, l['cout'])
                shapes = [(l['cout'], l['cin'])]
                sides = list(self.dims[i][:2])
            if l['kind'] != 'bn':
                shapes.append((shapes[0][0],) if l['bias'] else None)
            if not self.prebuilt:
                x = torch.randn(xs, device=device, generator=g)
                if i > 0 and l['kind'] != 'bn':
                    x.clamp_(min=0)          # post-ReLU activations
                self.x[i] = x
                # output gradients of a mean loss; a BatchNormalization layer
                # sums them over h x h positions per sample, so they are
                # drawn smaller there by h (keeps F + damping well inside
                # fp32 range of a Cholesky factorisation)
                self.gy[i] = torch.randn(gs, device=device, generator=g) / (
                    n * l['h'] if l['kind'] == 'bn' else n)
            P, gP, vP = [], [], []
            for shp in shapes:
                if shp is None:
                    P.append(None); gP.append(None); vP.append(None)
                    continue
                fan = 1
                for v in shp[1:]:
                    fan *= v
                P.append(torch.randn(shp, device=device, generator=g) /
                         fan ** 0.5)
                gP.append(torch.randn(shp, device=device, generator=g) * 1e-2)
                vP.append(torch.zeros(shp, device=device))
            self.P.append(P); self.gP.append(gP); self.vP.append(vP)
            self.fidx.append(list(range(len(self.ema),
                                        len(self.ema) + len(sides))))
            for d in sides:
                self.ema.append(torch.zeros((d, d), device=device))
                self.inv.append(torch.empty((d, d), device=device))
            if l['kind'] == 'bn':
                self.bn_kf[i] = [torch.empty_like(t) for t in P]
                if self.lowrank[i]:
                    m, d = self.lr_slots * n * world, 2 * l['c']
                    self.lr[i] = dict(
                        hist=torch.zeros((m, d), device=device),
                        Hs=torch.empty((m, d), device=device),
                        M=torch.empty((m, m), device=device),
                        Minv=torch.empty((m, m), device=device),
                        w=[0.0] * self.lr_slots, pos=-1, rows=n * world)
                else:
                    self.bn_grads[i] = torch.empty((n, 2 * l['c']),
                                                   device=device)
        self.bn_flags = torch.zeros((nl, 2), dtype=torch.int32, device=device)
        if self.prebuilt:
            # factors X^T X / m + 1e-3 I from X ~ N(0,1) with m rows, built
            # once; the timed step only inverts and preconditions
            m = self.prebuilt
            for f in self.ema:
                d = f.shape[0]
                X = torch.randn((m, d), device=device, generator=g)
                ops.factor_dense(X, False, alpha=1.0 / m, out=f)
                f.diagonal().add_(1e-3)
        if self.acc > 1:
            self.cov = [torch.zeros_like(e) for e in self.ema]
            self.acc_cov = [torch.zeros_like(e) for e in self.ema]
            self.acc_g = [[None if t is None else torch.zeros_like(t)
                           for t in gp] for gp in self.gP]
            self.micro = 0
        self.make_plan(list(range(nl)))
        self.make_lr_plan(list(range(nl)))
        self.first = True
        self.input_bytes = sum(t.numel() * 4 for t in self.x + self.gy
                               if t is not None)

    def is_bn(self, i):
        return self.layers[i]['kind'] == 'bn'

    def make_plan(self, own, bounds=None):
        factors, inverses, partner, role, scale = [], [], [], [], []
        for i in own:
            base = len(factors)
            ks = self.fidx[i]
            for j, k in enumerate(ks):
                factors.append(self.ema[k])
                inverses.append(self.inv[k])
                if self.prebuilt:
                    # the 1e-3 I inside the factors is the damping
                    partner.append(-1); role.append(2); scale.append(0.0)
                elif len(ks) == 2:
                    partner.append(base + 1 - j); role.append(j)
                    scale.append(1.0)
                else:
                    partner.append(-1); role.append(2)
                    scale.append(STAB_COEFF)
        self.plan = self.ops.InversePlanSet(factors, inverses, partner, role,
                                            scale=scale, bounds=bounds)
        self.plan_layers = own
        owner_of = [i for i in own for _ in self.fidx[i]]
        self.class_layers = [sorted({owner_of[q] for q in idx})
                             for idx in self.plan.classes()]

    def make_lr_plan(self, own):
        """Inverse plan of the m x m matrices I + Hs Hs^T of the owned
        low-rank BatchNormalization blocks (damping 1 adds the identity)."""
        self.lr_layers = [i for i in own if self.lowrank[i]]
        self.lr_plan = None
        if self.lr_layers:
            k = len(self.lr_layers)
            self.lr_plan = self.ops.InversePlanSet(
                [self.lr[i]['M'] for i in self.lr_layers],
                [self.lr[i]['Minv'] for i in self.lr_layers],
                [-1] * k, [2] * k, scale=[1.0] * k)

    def lr_slot(self, i):
        """View of block i's current history slot (rows of all ranks)."""
        st = self.lr[i]
        return st['hist'][st['pos'] * st['rows']:(st['pos'] + 1) * st['rows']]

    def lr_advance(self, i, r, rest):
        """Start a step for low-rank block i: older slots fade by `rest`, the
        next slot of the ring takes weight r."""
        st = self.lr[i]
        st['pos'] = (st['pos'] + 1) % self.lr_slots
        st['w'] = [w * rest for w in st['w']]
        st['w'][st['pos']] = r

    def lr_item(self, i, grads=None):
        st, l = self.lr[i], self.layers[i]
        # F = sum_s w_s * (sum over ranks of U^T U) / (n * world); after the
        # mean-reduce of the exchange a slot holds every rank's rows / world
        fac = float(self.world) / l['n']
        g = grads if grads is not None else self.grads()
        d = max(self.damping, 0.0) * STAB_COEFF
        return self.ops.bn_lowrank_item(
            st['hist'], st['Hs'], l['c'], st['rows'],
            [w * fac for w in st['w']], d, d, st['Minv'], g[i][0], g[i][1],
            self.bn_kf[i][0], self.bn_kf[i][1], self.bn_flags[i],
            self.P[i][0], self.P[i][1], self.vP[i][0], self.vP[i][1])

    def lr_build(self, layers):
        """Hs and Hs Hs^T of the low-rank blocks among `layers` (their
        history slots must hold this step's rows)."""
        lr = [i for i in layers if self.lowrank[i]]
        if not lr:
            return
        self.ops.bn_lowrank_scale([self.lr_item(i) for i in lr])
        self.ops.factor_group(
            [self.ops.dense_t_item(self.lr[i]['Hs'], 1.0, 0.0,
                                   self.lr[i]['M']) for i in lr],
            self.ema[0].device)

    def layer_items(self, i, outs, r, rest):
        """Grouped-build items of block i's factors into `outs` (one tensor
        per factor).  BatchNormalization blocks need their per-sample
        gradients first (bn_prepare)."""
        ops, l = self.ops, self.layers[i]
        n = l['n']
        if l['kind'] == 'bn':
            return [ops.dense_item(self.bn_grads[i], False, r / n, rest,
                                   outs[0])]
        if l['kind'] == 'conv':
            return [ops.conv_input_item(self.x[i], l['k'], l['stride'],
                                        l['pad'], l['bias'], r / n, rest,
                                        outs[0]),
                    ops.conv_grad_item(self.gy[i],
                                       r * n / float(l['hout'] ** 2), rest,
                                       outs[1])]
        return [ops.dense_item(self.x[i], l['bias'], r / n, rest, outs[0]),
                ops.dense_item(self.gy[i], False, r * n, rest, outs[1])]

    def bn_prepare(self, layers):
        """Per-sample gradients of the BatchNormalization blocks among
        `layers`, one grouped call."""
        items = []
        for i in layers:
            if not self.is_bn(i):
                continue
            n = self.layers[i]['n']
            out = self.bn_grads[i]
            if self.lowrank[i]:
                slot = self.lr_slot(i)
                if self.world > 1:
                    slot.zero_()         # the other ranks' rows arrive by sum
                out = slot[self.rank * n:(self.rank + 1) * n]
            it = self.ops.bn_item(self.x[i], self.gy[i], 2e-5, float(n), out,
                                  self.bn_stats.get(i))
            self.bn_stats[i] = it._keep[3]      # scratch kept across steps
            items.append(it)
        self.ops.bn_sample_grads_group(items)

    def build(self, layers, outs, r, rest):
        """Factors of `layers` into the flat list `outs`, one grouped call
        (plus the grouped per-sample gradients of BatchNormalization)."""
        if not layers:
            return
        for i in layers:
            if self.lowrank[i]:
                self.lr_advance(i, r, rest)
        self.bn_prepare(layers)
        items = []
        for i in layers:
            if not self.lowrank[i]:
                items += self.layer_items(
                    i, [outs[k] for k in self.fidx[i]], r, rest)
        if items:
            self.ops.factor_group(items, self.ema[0].device)
        if self.world == 1:
            self.lr_build(layers)       # else after the exchange

    # -- stages timed alone (nothing else on the device) --------------------
    def factors_alone(self):
        """Every factor in one grouped call, no inverse started beside it."""
        self.build(list(range(len(self.layers))), self.ema, self.decay,
                   1.0 - self.decay)

    def inverses_alone(self):
        if self.lr_plan is not None:
            self.lr_plan.run(1.0, False)
        self.plan.run(self.damping, not self.prebuilt)

    def precondition_alone(self):
        self.precondition_layers(self.plan_layers, lr=0.0, momentum=1.0,
                                 grads=self.gP)

    # -- the step ------------------------------------------------------------
    def flat(self, per_block):
        return [t for blk in per_block for t in blk if t is not None]

    def accumulate(self):
        """Micro-step of an accumulated update: build this micro-batch's
        factors and add 1/acc of them (and of the gradients) to the
        accumulators in one launch."""
        self.build(list(range(len(self.layers))), self.cov, 1.0, 0.0)
        s, keep = 1.0 / self.acc, (0.0 if self.micro == 0 else 1.0)
        acc = self.acc_cov + self.flat(self.acc_g)
        self.ops.axpby_group(s, self.cov + self.flat(self.gP), keep, acc, acc)
        self.micro += 1

    def ema_weights(self):
        w = (1.0, 0.0) if self.first else (self.decay, 1.0 - self.decay)
        self.first = False
        return w

    def factors(self):
        # all factors in one grouped call per size class, running average
        # fused in, largest class first: its inverse (a long serial chain that
        # uses few SMs) starts on a side stream while the other layers'
        # factors are still being built
        if self.prebuilt:
            return
        if self.acc > 1:
            self.accumulate()
            if self.micro == self.acc:
                r, rest = self.ema_weights()
                self.ops.axpby_group(r, self.acc_cov, rest, self.ema, self.ema)
            return
        r, rest = self.ema_weights()
        classes = self.class_layers if OVERLAP else []
        done = set()
        if OVERLAP and self.lr_plan is not None:
            # the low-rank BatchNormalization blocks first: their small
            # inverses run beside everything else
            self.build(self.lr_layers, self.ema, r, rest)
            self.lr_plan.start_class(0, 1.0, False)
            done.update(self.lr_layers)
        for c, layers in enumerate(classes[:-1]):
            self.build(layers, self.ema, r, rest)
            self.plan.start_class(c, self.damping, True)
            done.update(layers)
        self.build([i for i in range(len(self.layers)) if i not in done],
                   self.ema, r, rest)

    def update_due(self):
        if self.acc > 1:
            if self.micro < self.acc:
                return False
            self.micro = 0
        return True

    def inverses(self):
        # the layers of a size class are preconditioned (and updated) on that
        # class's stream as soon as its inverses are done, next to the
        # remaining classes' inverses
        if self.lr_plan is not None:
            self.lr_plan.run(
                1.0, False, after_class=(lambda c: self.precondition_layers(
                    self.lr_layers)) if OVERLAP else None)
        self.plan.run(self.damping, not self.prebuilt,
                      after_class=self.precondition_class if OVERLAP else None)

    def grads(self):
        return self.acc_g if self.acc > 1 else self.gP

    def precondition_layers(self, layers, ws_key=None, lr=LR,
                            momentum=MOMENTUM, grads=None):
        g = grads if grads is not None else self.grads()
        conn = [i for i in layers if not self.is_bn(i)]
        bn = [i for i in layers if self.is_bn(i) and not self.lowrank[i]]
        low = [i for i in layers if self.lowrank[i]]
        if low:
            self.ops.bn_lowrank_apply([self.lr_item(i, g) for i in low], lr,
                                      momentum)
        if conn:
            self.ops.precondition(
                [self.inv[self.fidx[i][1]] for i in conn],
                [self.inv[self.fidx[i][0]] for i in conn],
                [g[i][0] for i in conn], [g[i][1] for i in conn], None, None,
                [self.P[i][0] for i in conn], [self.P[i][1] for i in conn],
                [self.vP[i][0] for i in conn], [self.vP[i][1] for i in conn],
                lr=lr, momentum=momentum, ws_key=ws_key)
        if bn:
            self.ops.bn_precondition_group(
                [self.inv[self.fidx[i][0]] for i in bn],
                [g[i][0] for i in bn], [g[i][1] for i in bn],
                [self.bn_kf[i][0] for i in bn],
                [self.bn_kf[i][1] for i in bn],
                [self.bn_flags[i] for i in bn],
                param_gamma=[self.P[i][0] for i in bn],
                param_beta=[self.P[i][1] for i in bn],
                mom_gamma=[self.vP[i][0] for i in bn],
                mom_beta=[self.vP[i][1] for i in bn], lr=lr,
                momentum=momentum)

    def precondition_class(self, c):
        self.precondition_layers(self.class_layers[c], ws_key=c)

    def precondition(self):
        if not OVERLAP:          # else done per class inside inverses()
            self.precondition_layers(self.plan_layers)

    def micro_step(self, events=None):
        self.factors()
        if events is not None:
            events[1].record()
        if self.update_due():
            self.inverses()
            if events is not None:
                events[2].record()
            self.precondition()
        elif events is not None:
            events[2].record()

    def step(self, events=None):
        """One update: `acc` micro-steps (1 without accumulation)."""
        for m in range(self.acc):
            self.micro_step(events if m == self.acc - 1 else None)


class DistributedWorkload(DeviceWorkload):
    """The same per-GPU work as DeviceWorkload for the factor build (every rank
    builds all factors from its own batch), then the reference's two
    exchanges: gradients and packed factors are reduce-scattered to the
    layer's owner, the owner averages them into its running average, inverts
    and preconditions/updates only its own layers, and the updated weights
    are all-gathered.  Ownership is cost-balanced by default (OWNERSHIP);
    'reference' is the reference's contiguous split of the layer list by
    count.  With accumulation the factors and gradients are accumulated
    locally and exchanged once per update (the reduction is linear).

    The first exchange runs size class by size class, largest first: as soon
    as a class is reduced its owners start its inverses on a side stream, next
    to the factor build and exchange of the remaining classes."""

    def __init__(self, device, seed, spec, comm, bn_blocks=True,
                 bn_lowrank=True):
        super(DistributedWorkload, self).__init__(
            device, seed, spec, bn_blocks, bn_lowrank, world=comm.size,
            rank=comm.rank)
        import torch
        self.comm = comm
        from chainerkfac_b200.optimizers.kfac import balanced_split
        cnt = len(self.layers)
        # a low-rank block costs its m x m inverse
        sides = [[self.ema[k].shape[0] for k in ks] if ks else
                 ([self.lr[i]['M'].shape[0]] if self.lowrank[i] else [1])
                 for i, ks in enumerate(self.fidx)]
        if OWNERSHIP == 'balanced':
            self.indices = balanced_split(
                [sum(float(d) ** 3 for d in sd) for sd in sides], comm.size)
        else:
            # the reference's contiguous split of the layer list by count
            self.indices = [ix.tolist() for ix in
                            np.array_split(np.arange(cnt), comm.size)]
        self.mine = self.indices[comm.rank]
        if self.acc == 1 and not self.prebuilt:
            self.cov = [torch.zeros_like(e) for e in self.ema]
        bounds = self.plan.bounds
        self.plan.close()
        self.make_plan(self.mine, bounds)
        if self.lr_plan is not None:
            self.lr_plan.close()
        self.make_lr_plan(self.mine)
        # size classes over all layers, largest first, as the plan forms them
        key_of = [sum(max(sd) > b for b in bounds) for sd in sides]
        pipelined = OVERLAP and self.acc == 1 and not self.prebuilt
        keys = sorted(set(key_of), reverse=True) if pipelined else [None]
        src = None if self.prebuilt else (
            self.acc_cov if self.acc > 1 else self.cov)
        self.xsrc = src
        self.xclass_layers, self.class_plan = [], []
        for key in keys:
            layers = [i for i in range(cnt) if key is None or key_of[i] == key]
            self.xclass_layers.append(layers)
            self.class_plan.append(
                self.plan.class_keys.index(key)
                if key in self.plan.class_keys else None)
        self.ag_arrays = [[(t, False) for i in idx for t in self.P[i]
                           if t is not None] for idx in self.indices]
        self.comm_stream = torch.cuda.Stream(priority=-1)
        if hasattr(comm, 'reserve'):
            from chainerkfac_b200.communicators import _utility
            for st in self.lr.values():
                st['pos'] = 0
            comm.reserve(max([_utility.get_nelems(self.class_rs(c))
                              for c in range(len(self.xclass_layers))]
                             + [_utility.get_nelems(self.ag_arrays)]), device)
            for st in self.lr.values():
                st['pos'] = -1

    def class_rs(self, c):
        """Arrays of exchange 1 for size class c, by owner: gradients (sorted
        parameter names), then the factors -- or, for a low-rank
        BatchNormalization block, the current history slot with this rank's
        rows in place and zeros elsewhere, whose mean over ranks is the stack
        of all ranks' rows divided by the number of ranks."""
        layers = set(self.xclass_layers[c])
        gsrc = self.grads()
        rs = []
        for idx in self.indices:
            loc = []
            for i in idx:
                if i not in layers:
                    continue
                loc += [(t, False) for t in gsrc[i] if t is not None]
                if self.lowrank[i]:
                    loc.append((self.lr_slot(i), False))
                elif self.xsrc is not None:
                    loc += [(self.xsrc[k], True) for k in self.fidx[i]]
            rs.append(loc)
        return rs

    def own_factors(self, layers=None):
        mine = set(self.mine)
        return [k for i in (layers if layers is not None else self.mine)
                if i in mine for k in self.fidx[i]]

    def factors(self):
        torch = self.torch
        if self.prebuilt:
            # only the gradients travel to the owners
            self.comm.reduce_scatter_v_arrays(self.class_rs(0))
            return
        if self.acc > 1:
            self.accumulate()
            if self.micro == self.acc:
                # one exchange per update: accumulated factors and gradients
                self.comm.reduce_scatter_v_arrays(self.class_rs(0))
                r, rest = self.ema_weights()
                own = self.own_factors()
                emas = [self.ema[k] for k in own]
                self.ops.axpby_group(r, [self.acc_cov[k] for k in own], rest,
                                     emas, emas)
            return
        r, rest = self.ema_weights()
        last = len(self.xclass_layers) - 1
        main = torch.cuda.current_stream()
        for c, layers in enumerate(self.xclass_layers):
            self.build(layers, self.cov, 1.0, 0.0)
            # exchange 1 for this class and the owner's running average run
            # on the exchange stream: the factor build of the next class does
            # not wait for the other ranks
            # (every exchange on the same stream: the communicator's buffer
            # reuse relies on its calls being ordered with one another)
            side = self.comm_stream if (OVERLAP and last > 0) else main
            if side is not main:
                built = torch.cuda.Event()
                built.record(main)
                side.wait_event(built)
            with torch.cuda.stream(side):
                self.comm.reduce_scatter_v_arrays(self.class_rs(c))
                own = self.own_factors(layers)
                if own:
                    emas = [self.ema[k] for k in own]
                    self.ops.axpby_group(r, [self.cov[k] for k in own], rest,
                                         emas, emas)
                mine = set(self.mine)
                low = [i for i in layers if self.lowrank[i] and i in mine]
                if low:
                    # every rank's rows have arrived in the owner's slot
                    self.lr_build(low)
                    if OVERLAP:
                        self.lr_plan.start_class(0, 1.0, False)
                if c < last and self.class_plan[c] is not None:
                    self.plan.start_class(self.class_plan[c], self.damping,
                                          True)
            if side is not main:
                done = torch.cuda.Event()
                done.record(side)
                self._exchanged = done
        if OVERLAP and last > 0:
            # later work on the main stream (and the next step's factor build,
            # which overwrites cov) comes after the exchanges
            main.wait_event(self._exchanged)

    def precondition(self):
        super(DistributedWorkload, self).precondition()
        # exchange 2: updated weights to everyone
        self.comm.all_gather_v_arrays(self.ag_arrays)

    def check(self):
        """One extra update from a clean state (running average = this
        update's mean factor) whose results are checked across ranks: the
        owner's averaged factors of one small layer against the mean of the
        factors every rank built, the owner's inverses of them against fp64
        inverses of that mean with the reference's damping rule, and the
        gathered weights of all layers for equality on every rank."""
        import torch.distributed as dist
        torch = self.torch
        if self.prebuilt:
            return None
        world = self.comm.size
        small = [i for i, l in enumerate(self.layers)
                 if l['kind'] != 'bn' and max(self.dims[i][:2]) <= 600]
        i = small[len(small) // 2] if small else 0
        owner = [r for r, ix in enumerate(self.indices) if i in ix][0]
        self.first = True
        self.step()
        torch.cuda.synchronize()
        # the factors this rank contributed (every micro-step of an
        # accumulated update saw the same synthetic batch)
        mine = [torch.empty_like(self.ema[k]) for k in self.fidx[i]]
        self.ops.factor_group(self.layer_items(i, mine, 1.0, 0.0),
                              mine[0].device)
        worst_f = worst_i = 0.0
        means = []
        for j, k in enumerate(self.fidx[i]):
            parts = [torch.empty_like(mine[j]) for _ in range(world)]
            dist.all_gather(parts, mine[j])
            mean = sum(p.double() for p in parts) / world
            got = self.ema[k].clone()
            dist.broadcast(got, src=owner)
            worst_f = max(worst_f, float((got.double() - mean).norm() /
                                         mean.norm()))
            means.append(mean)
        A, G = means
        pi = float(((A.trace() * G.shape[0]) /
                    (G.trace() * A.shape[0])).sqrt())
        adds = (pi * self.damping ** 0.5, self.damping ** 0.5 / pi)
        for k, m, add in zip(self.fidx[i], (A, G), adds):
            want = torch.linalg.inv(
                m + add * torch.eye(m.shape[0], device=m.device,
                                    dtype=torch.float64))
            got = self.inv[k].clone()
            dist.broadcast(got, src=owner)
            worst_i = max(worst_i, float((got.double() - want).norm() /
                                         want.norm()))
        # every rank's weights against rank 0's, element by element (a NaN
        # counts as a difference), the layers that differ, and what the
        # owners' inverse plans reported
        dev0 = mine[0].device
        bad = torch.zeros(len(self.layers), device=dev0, dtype=torch.float64)
        nonfinite = torch.zeros(1, device=dev0, dtype=torch.float64)
        for li, blk in enumerate(self.P):
            for w in blk:
                if w is None:
                    continue
                ref = w.clone()
                dist.broadcast(ref, src=0)
                bad[li] += (w != ref).sum().double()
                nonfinite += (~torch.isfinite(w)).sum().double()
        pivots = (self.plan.info != 0).sum().double().reshape(1)
        for t in (bad, nonfinite, pivots):
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        differing = [self.layers[li]['name'] for li in
                     torch.nonzero(bad).flatten().tolist()]
        return dict(layer=self.layers[i]['name'], owner=owner,
                    factor_rel=worst_f, inverse_rel=worst_i,
                    weights_equal=not differing,
                    weights_differing_layers=differing[:8],
                    weights_nonfinite=int(nonfinite.item()),
                    nonpositive_pivots_all_ranks=int(pivots.item()))


def time_alone(torch, fn, reps):
    fn()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


STAGE_KERNELS = {
    'factor': 'tc_pair_kernel (grouped strided and im2col launches over all '
              'factors, plus staging copies and the split reduce)',
    'inverse': 'tc_gemm_kernel + chol_diag_kernel (batched blocked Cholesky, '
               'triangular inverse and symmetric product of every factor, '
               'three size classes on three streams)',
    'precondition': 'tc_gemm_kernel (two grouped launches over all layers, '
                    'update fused)'}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from chainerkfac_b200 import _lib

    spec = WORKLOADS[args.workload]
    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device (no CPU fallback)')
    torch.cuda.set_device(local_rank)
    device = torch.device('cuda', local_rank)
    if world > 1:
        dist.init_process_group('nccl', device_id=device)
    lib = _lib.load()
    batch, acc = spec['batch'], spec['acc']
    if args.only_e2e:
        # the end-to-end steps alone (what a profiler run wants to see)
        e2e = run_e2e(args, device, world, rank, spec, profile=True)
        if rank == 0:
            print(json.dumps({'e2e': e2e, 'n_gpus': world,
                              'workload': spec['name']}))
        if world > 1:
            dist.destroy_process_group()
        return
    prebuilt = bool(spec.get('prebuilt'))

    if world > 1:
        from chainerkfac_b200.communicators import create_communicator
        wl = DistributedWorkload(device, 1234 + rank, spec,
                                 create_communicator(COMMUNICATOR),
                                 bn_blocks=not args.no_bn_blocks,
                                 bn_lowrank=not args.bn_dense)
    else:
        wl = DeviceWorkload(device, 1234 + rank, spec,
                            bn_blocks=not args.no_bn_blocks,
                            bn_lowrank=not args.bn_dense)
    low = {i: wl.lr[i]['M'].shape[0] for i in wl.lr}
    flops = algorithmic_flops(wl.layers, prebuilt, low)
    abytes = algorithmic_bytes(wl.layers, prebuilt, low)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        wl.step()
    barrier()

    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)]
          for _ in range(args.steps)]
    launches0 = lib.kfac_launch_count()
    barrier()
    # (a profiler started with its capture off sees exactly the timed steps)
    torch.cuda.profiler.start()
    t_begin = time.perf_counter()
    for s in range(args.steps):
        ev[s][0].record()
        wl.step(ev[s])
        ev[s][3].record()
    barrier()
    torch.cuda.profiler.stop()
    t_end = time.perf_counter()
    launches = lib.kfac_launch_count() - launches0
    total_ms = ev[0][0].elapsed_time(ev[-1][3])
    phase = np.zeros(3)
    for s in range(args.steps):
        for j in range(3):
            phase[j] += ev[s][j].elapsed_time(ev[s][j + 1])
    phase /= args.steps
    t = torch.tensor([total_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    # the same steps go on, untimed, until two seconds of load have been
    # sampled: a 0.2 s timed region sees only a few clock samples (the count
    # comes from the reduced time, so every rank runs the same number)
    soak = int(max(0.0, 2000.0 - total_ms) / max(ms_per_step, 0.05))
    for _ in range(min(soak, 4000)):
        wl.step()
    barrier()
    clocks = sampler.stop(
        t_begin, time.perf_counter(),
        'timed region and the same steps repeated, untimed, until 2 s of '
        'load were sampled') if rank == 0 else None
    if prebuilt:
        # strong scaling: the set of pairs is fixed
        value, unit = len(wl.layers) / (ms_per_step * 1e-3), 'factor pairs/sec'
    else:
        value, unit = batch * acc * world / (ms_per_step * 1e-3), 'images/sec'

    info_bad = int((wl.plan.info != 0).sum().item())
    refined = wl.plan.refined()

    # The step overlaps its stages, so the stage events above do not isolate
    # them.  Each stage is therefore also timed alone: the same launches,
    # nothing beside them, CUDA events on the launching stream.  At N > 1 a
    # rank times the stages of the layers it owns (the factor build is the
    # same on every rank) and the slowest rank counts.
    reps = max(3, min(args.steps, 10))
    alone = {}
    if not prebuilt:
        alone['factor'] = time_alone(torch, wl.factors_alone, reps)
    alone['inverse'] = time_alone(torch, wl.inverses_alone, reps)
    alone['precondition'] = time_alone(torch, wl.precondition_alone, reps)
    if world > 1:
        names = sorted(alone)
        tt = torch.tensor([alone[k] for k in names], device=device,
                          dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        alone = {k: float(v) for k, v in zip(names, tt.tolist())}
    all_layers = None
    if world > 1 and rank == 0:
        # the owner-partitioned stages over ALL layers on one GPU, for their
        # parallel efficiency: alone(all layers) / (N * slowest owner alone)
        own, cls, plan = wl.plan_layers, wl.class_layers, wl.plan
        wl.make_plan(list(range(len(wl.layers))), plan.bounds)
        all_layers = {
            'inverse': time_alone(torch, wl.inverses_alone, reps),
            'precondition': time_alone(torch, wl.precondition_alone, reps)}
        wl.plan.close()
        wl.plan, wl.plan_layers, wl.class_layers = plan, own, cls
    barrier()

    dist_check = wl.check() if world > 1 else None

    e2e = None
    if not args.no_e2e and args.workload in ('resnet50', 'config5'):
        e2e = run_e2e(args, device, world, rank, spec)

    if rank == 0:
        peaks = measured_peaks()
        tf32 = measure_tf32_peak(device)
        names = ['factor', 'inverse', 'precondition']
        stage = {nm: dict(ms=float(ms)) for nm, ms in zip(names, phase)}
        if OVERLAP:
            stage['inverse']['includes'] = 'precondition'
        for nm in alone:
            stage[nm]['alone_ms'] = float(alone[nm])
            stage[nm]['algorithmic_gflop'] = flops[nm] / 1e9
            stage[nm]['algorithmic_mbytes'] = abytes[nm] / 1e6
            if world == 1 or nm == 'factor':
                stage[nm]['alone_tflops'] = float(
                    flops[nm] / (alone[nm] * 1e-3) / 1e12)
        if all_layers:
            for nm, ms in all_layers.items():
                stage[nm]['alone_all_layers_one_gpu_ms'] = float(ms)
                stage[nm]['parallel_efficiency'] = float(
                    ms / (world * alone[nm]))
        # the roofline entry is the stage that takes longest alone
        dom = max(alone, key=lambda k: alone[k])
        if world == 1 or dom == 'factor':
            dom_flops = flops[dom]
            dom_ms = alone[dom]
        else:
            # an owner-partitioned stage: all layers on one GPU
            dom_flops = flops[dom]
            dom_ms = all_layers[dom]
        achieved = dom_flops / (dom_ms * 1e-3) / 1e12
        traffic = None
        tcase = TRAFFIC_CASES.get(dom)
        if tcase is not None:
            # measured bytes of the small case, scaled by algorithmic flops
            traffic = tcase[1] * dom_flops / tcase[3]
        cpu = None
        if not args.no_cpu_baseline and world == 1:
            cpu = cpu_baseline(spec, budget_s=25.0, min_passes=1,
                               bn_blocks=not args.no_bn_blocks)
        line = {
            'metric': 'ResNet-50 K-FAC images/sec (factor+inverse+'
                      'precondition step)' if not prebuilt else
                      'curvature microbench factor pairs/sec (inverse+'
                      'precondition)',
            'value': value, 'unit': unit, 'n_gpus': world,
            'steps': args.steps, 'warmup': warmup,
            'ms_per_step': ms_per_step, 'higher_is_better': True,
            'scaling': 'strong' if prebuilt else 'weak', 'vs_baseline': None,
            'dtype': 'f32', 'data': 'synthetic',
            'config': {'workload': spec['name'], 'batch_per_gpu': batch,
                       'layers': len(wl.layers),
                       'bn_blocks': sum(1 for l in wl.layers
                                        if l['kind'] == 'bn'),
                       'bn_blocks_low_rank': len(wl.lr),
                       'cov_ema_decay': spec['decay'],
                       'damping': spec['damping'], 'acc_iters': acc,
                       'l2_flush': ('inputs larger than L2 (%.2f GB of '
                                    'activations and gradients per step)'
                                    % (wl.input_bytes / 1e9))
                       if wl.input_bytes > 126e6 else
                       ('factor and inverse buffers of %.2f GB per step'
                        % (sum(e.numel() for e in wl.ema) * 8 / 1e9)),
                       'parallelism': 'dp%d' % world,
                       'ownership': OWNERSHIP if world > 1 else None,
                       'communicator': COMMUNICATOR if world > 1 else None},
            # 'ms': stage boundaries on the main stream of the overlapped
            # step (the inverses of the larger size classes run on side
            # streams during 'factor'); 'alone_ms': the stage by itself
            'stages': stage,
            'stages_overlap': bool(OVERLAP),
            'factor_inverse_ms': float(phase[0] + phase[1]),
            'ms_per_micro_step': ms_per_step / acc,
            'roofline': {
                'bound': 'tensor',
                'stage': dom,
                'kernel': STAGE_KERNELS[dom],
                'achieved': achieved, 'peak': peaks['tflops_burst'],
                'unit': 'TFLOP/s', 'frac': achieved / peaks['tflops_burst'],
                'peak_source': 'of %s: dense bf16 burst from '
                               'MEASURED_PEAKS.json (stage timed alone)'
                               % peaks['source'],
                # fp32 operands are split into two terms and every product
                # costs three MMAs: bf16 terms for the factors, TF32 terms
                # for the inverse and precondition products
                'frac_of_split_ceiling': achieved / (
                    (peaks['tflops_burst'] if dom == 'factor' else tf32) / 3.0),
                'tf32_tflops_measured_here': tf32,
                'step_tflops': (float(sum(flops.values()) * acc /
                                      (ms_per_step * 1e-3) / 1e12)
                                if world == 1 and acc == 1 else None),
                'traffic': traffic,
                'traffic_case': None if tcase is None else {
                    'case': tcase[0], 'dram_bytes': tcase[1],
                    'algorithmic_bytes': tcase[2]}},
            'cpu_baseline': cpu,
            'gpu_launches': int(launches),
            'clocks': clocks,
            'e2e': e2e,
            'dist_check': dist_check,
            'nonpositive_pivots': info_bad,
            'inverses_refined_last_step': refined,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_e2e(args, device, world, rank, spec, profile=False):
    """images/sec of KFAC.update(lossfun, x, t) on a torch ResNet-50 with the
    batch copied from pinned host memory and the loss read back every step."""
    import torch
    from bench_model import build_training_step
    acc = spec['acc']
    step, h2d, d2h = build_training_step(
        device, spec['batch'], world, rank, cov_ema_decay=spec['decay'],
        damping=spec['damping'], lr=LR, momentum=MOMENTUM,
        communicator=COMMUNICATOR, acc_iters=acc,
        bn_blocks=not args.no_bn_blocks, bn_low_rank=not args.bn_dense)
    steps = args.steps * acc
    for _ in range(max(args.warmup, 3) * acc):
        step()
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    if profile:
        torch.cuda.profiler.start()
    t0.record()
    for _ in range(steps):
        step()
    t1.record()
    torch.cuda.synchronize()
    if profile:
        torch.cuda.profiler.stop()
    ms = torch.tensor([t0.elapsed_time(t1)], device=device, dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(ms, op=torch.distributed.ReduceOp.MAX)
    per = float(ms.item()) / steps
    return dict(value=spec['batch'] * world / (per * 1e-3), unit='images/sec',
                ms_per_step=per * acc, ms_per_micro_step=per,
                h2d_bytes_per_step=h2d * acc, d2h_bytes_per_step=d2h * acc,
                bn_blocks=not args.no_bn_blocks)


# ------------------------------------------------------------- CPU baseline
def use_all_host_threads():
    """The BLAS behind NumPy follows OMP_NUM_THREADS, which torchrun sets to 1
    for its workers: raise the limit of the loaded BLAS to every host core.
    Returns the thread count in force."""
    n = os.cpu_count() or 1
    try:
        import threadpoolctl
        threadpoolctl.threadpool_limits(limits=n)
        got = max([p.get('num_threads', 1)
                   for p in threadpoolctl.threadpool_info()] or [1])
        return int(got)
    except Exception:
        return 1


def cpu_layer_inputs(l, rng):
    n = l['n']
    if l['kind'] == 'bn':
        shp = (n, l['c'], l['h'], l['h'])
        return (rng.standard_normal(shp, dtype=np.float32),
                rng.standard_normal(shp, dtype=np.float32) /
                np.float32(n * l['h']),
                rng.standard_normal(l['c'], dtype=np.float32),
                rng.standard_normal(l['c'], dtype=np.float32))
    if l['kind'] == 'conv':
        x = rng.standard_normal((n, l['cin'], l['hin'], l['hin']), dtype=np.float32)
        gy = rng.standard_normal((n, l['cout'], l['hout'], l['hout']), dtype=np.float32) / np.float32(n)
        gW = rng.standard_normal((l['cout'], l['cin'], l['k'], l['k']), dtype=np.float32)
    else:
        x = rng.standard_normal((n, l['cin']), dtype=np.float32)
        gy = rng.standard_normal((n, l['cout']), dtype=np.float32) / np.float32(n)
        gW = rng.standard_normal((l['cout'], l['cin']), dtype=np.float32)
    gb = rng.standard_normal(l['cout'], dtype=np.float32) if l['bias'] else None
    return x, gy, gW, gb


def cpu_layer_pass(orc, l, inputs, spec, prebuilt_AG=None):
    """The reference's --no_cuda stages for one layer, via the oracle."""
    x, gy, gW, gb = inputs
    W, v = np.zeros_like(gW), np.zeros_like(gW)
    t0 = time.perf_counter()
    if l['kind'] == 'bn':
        # batch_normalization.py:78-191 (gW, gb hold the gradients of gamma
        # and beta)
        F = orc.bn_F(x, gy, 2e-5)
        t1 = time.perf_counter()
        Finv = orc.damped_inverse(
            F, np.float32(orc.bn_damping(spec['damping'], STAB_COEFF)))
        kg, kb = orc.bn_kfgrads(Finv, gW, gb)
        orc.momentum_update(W, v, kg, LR, MOMENTUM)
        orc.momentum_update(np.zeros_like(gb), np.zeros_like(gb), kb, LR,
                            MOMENTUM)
        return t1 - t0, time.perf_counter() - t1
    if prebuilt_AG is not None:
        A, G = prebuilt_AG
    elif l['kind'] == 'conv':
        A = orc.conv_A(x, l['k'], l['stride'], l['pad'], l['bias'])
        G = orc.conv_G(gy)
    else:
        A = orc.linear_A(x, l['bias'])
        G = orc.linear_G(gy)
    t1 = time.perf_counter()
    if prebuilt_AG is not None:
        kW, _ = orc.connection_kfgrads(orc.inverse(A), orc.inverse(G), gW, gb)
    else:
        out = orc.connection_step(A, G, gW, gb, spec['damping'], None, None,
                                  spec['decay'])
        kW = out['kfgrad_W']
    orc.momentum_update(W, v, kW, LR, MOMENTUM)
    t2 = time.perf_counter()
    return t1 - t0, t2 - t1


def cpu_baseline(spec, budget_s, min_passes=1, max_passes=None,
                 bn_blocks=True):
    """Whole passes of the oracle (the reference's --no_cuda arithmetic) over
    the workload: one layer of each distinct shape is timed and counted once
    per layer of that shape.  Passes repeat until `budget_s` seconds are used
    (at least `min_passes`, at most `max_passes`)."""
    from oracle import kfac_oracle as orc
    threads = use_all_host_threads()
    layers = spec['layers']()
    if bn_blocks and spec.get('bn') and not spec.get('prebuilt'):
        layers = layers + bw.bn_layers_of(layers)
    groups = bw.distinct_shapes(layers)
    rng = np.random.default_rng(7)
    inputs = [cpu_layer_inputs(l, rng) for l, _ in groups]
    prebuilt = None
    if spec.get('prebuilt'):
        prebuilt = []
        for l, _ in groups:
            dA, dG, _, _ = bw.layer_dims(l)
            pair = []
            for d in (dA, dG):
                X = rng.standard_normal((2048, d), dtype=np.float32)
                pair.append((X.T @ X / 2048 + 1e-3 * np.eye(d)).astype(np.float32))
            prebuilt.append(pair)
    acc = spec['acc']
    times, t_start = [], time.perf_counter()
    while True:
        tf = ti = 0.0
        for k, ((l, mult), inp) in enumerate(zip(groups, inputs)):
            a, b = cpu_layer_pass(orc, l, inp, spec,
                                  None if prebuilt is None else prebuilt[k])
            # with accumulation the factors are built in every micro-step,
            # the inverse and preconditioning once per update
            tf += a * mult * acc
            ti += b * mult
        times.append((tf, ti))
        used = time.perf_counter() - t_start
        if len(times) >= min_passes and (
                used + used / len(times) > budget_s or
                (max_passes and len(times) >= max_passes)):
            break
    tf = float(np.mean([t[0] for t in times]))
    ti = float(np.mean([t[1] for t in times]))
    if spec.get('prebuilt'):
        value, unit = len(layers) / (tf + ti), 'factor pairs/sec'
    else:
        value, unit = spec['batch'] * acc / (tf + ti), 'images/sec'
    return dict(value=value, unit=unit, cores=threads,
                host_cpus=os.cpu_count(), kind='port', layers=len(layers),
                bn_blocks=sum(1 for l in layers if l['kind'] == 'bn'),
                factor_s=tf, inverse_precondition_s=ti,
                passes_timed=len(times), wall_s=time.perf_counter() - t_start,
                sample='NumPy oracle (the reference --no_cuda arithmetic '
                       'restated; %d BLAS threads) on one layer of each of '
                       'the %d distinct layer shapes of %s, each time counted '
                       'once per layer of that shape (%d layers): %d whole '
                       'pass(es)' % (threads, len(groups), spec['name'],
                                     len(layers), len(times)))


def run_reference(args):
    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    if rank != 0:
        return
    spec = WORKLOADS[args.workload]
    # one warm-up pass, then whole passes for about a minute and a half;
    # `steps` is the number of passes really timed
    bn = not args.no_bn_blocks
    warm = cpu_baseline(spec, budget_s=0.0, min_passes=1, max_passes=1,
                        bn_blocks=bn)
    want = max(1, min(args.steps, int(90.0 / max(warm['wall_s'], 1e-3))))
    cpu = cpu_baseline(spec, budget_s=1e9, min_passes=want, max_passes=want,
                       bn_blocks=bn)
    value = cpu['value']
    line = {
        'impl': 'reference',
        'metric': 'ResNet-50 K-FAC images/sec (factor+inverse+'
                  'precondition step)' if not spec.get('prebuilt') else
                  'curvature microbench factor pairs/sec (inverse+'
                  'precondition)',
        'value': value, 'unit': cpu['unit'], 'n_gpus': world,
        'steps': cpu['passes_timed'], 'warmup': 1,
        'steps_requested': args.steps,
        'ms_per_step': 1e3 * (cpu['factor_s'] + cpu['inverse_precondition_s']),
        'higher_is_better': True,
        'scaling': 'strong' if spec.get('prebuilt') else 'weak',
        'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': spec['name'], 'batch_per_gpu': spec['batch'],
                   'layers': cpu['layers'], 'bn_blocks': cpu['bn_blocks'],
                   'cov_ema_decay': spec['decay'], 'damping': spec['damping'],
                   'acc_iters': spec['acc'],
                   'parallelism': 'cpu (rank 0 only, %d BLAS threads)'
                                  % cpu['cores']},
        'cpu_baseline': cpu,
        'e2e': {'value': value, 'unit': cpu['unit'],
                'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))


MICRO_CASES = {
    # name: (kind, parameters) -- single-kernel cases for profiling
    'conv_grad_c256_hw56': ('conv_grad', dict(n=32, c=256, hw=56)),
    'conv_grad_c64_hw56': ('conv_grad', dict(n=32, c=64, hw=56)),
    'conv3x3_c64_hw56': ('conv_input', dict(n=32, c=64, hw=56, k=3, s=1, p=1)),
    'conv3x3_c64_hw128': ('conv_input', dict(n=32, c=64, hw=128, k=3, s=1, p=1)),
    'conv3x3_c256_hw14': ('conv_input', dict(n=32, c=256, hw=14, k=3, s=1, p=1)),
    'conv3x3_c512_hw7': ('conv_input', dict(n=32, c=512, hw=7, k=3, s=1, p=1)),
    'conv7x7_c3_hw224': ('conv_input', dict(n=32, c=3, hw=224, k=7, s=2, p=3)),
    'dense_rows8192_d4608': ('dense', dict(rows=8192, d=4608)),
    'inverse_d1024': ('inverse', dict(dims=[1024])),
    'inverse_d2304': ('inverse', dict(dims=[2304])),
    'inverse_d4608': ('inverse', dict(dims=[4608])),
    'inverse_d4608x3': ('inverse', dict(dims=[4608, 4608, 4608])),
    'precondition_dG512_dA4608': ('precondition', dict(dG=512, dA=4608)),
    # wire format of the exchange: every factor of ResNet-50 (308 MB packed,
    # 615 MB dense); the sum reads 4 rank buffers, all on this GPU here
    'wire_pack_resnet50': ('wire_pack', dict()),
    'wire_unpack_sum4_resnet50': ('wire_unpack', dict(ranks=4)),
}


def run_micro(args):
    """Time one small case with CUDA events (the cases the ncu captures
    use)."""
    import torch
    from chainerkfac_b200 import ops
    kind, p = MICRO_CASES[args.micro]
    torch.manual_seed(0)
    if kind == 'conv_grad':
        x = torch.randn(p['n'], p['c'], p['hw'], p['hw'], device='cuda')
        out = torch.empty(p['c'], p['c'], device='cuda')
        fn = lambda: ops.factor_conv_grad(x, alpha=1.0, out=out)
        flops = p['n'] * p['hw'] ** 2 * p['c'] * (p['c'] + 1)
    elif kind == 'conv_input':
        x = torch.randn(p['n'], p['c'], p['hw'], p['hw'], device='cuda')
        d = p['c'] * p['k'] ** 2
        out = torch.empty(d, d, device='cuda')
        fn = lambda: ops.factor_conv_input(x, p['k'], p['s'], p['p'], False,
                                           alpha=1.0, out=out)
        ho = (p['hw'] + 2 * p['p'] - p['k']) // p['s'] + 1
        flops = p['n'] * ho * ho * d * (d + 1)
    elif kind == 'dense':
        x = torch.randn(p['rows'], p['d'], device='cuda')
        out = torch.empty(p['d'], p['d'], device='cuda')
        fn = lambda: ops.factor_dense(x, False, alpha=1.0, out=out)
        flops = p['rows'] * p['d'] * (p['d'] + 1)
    elif kind == 'precondition':
        dG, dA = p['dG'], p['dA']
        Gi = torch.randn(dG, dG, device='cuda')
        Ai = torch.randn(dA, dA, device='cuda')
        gW = torch.randn(dG, dA, device='cuda')
        kW = torch.empty_like(gW)
        fn = lambda: ops.precondition([Gi], [Ai], [gW], [None], [kW], [None])
        flops = 2 * dG * dG * dA + 2 * dG * dA * dA
    elif kind in ('wire_pack', 'wire_unpack'):
        dims = [bw.layer_dims(l) for l in bw.resnet50_layers(batch=32)]
        sides = [d for dA, dG, _, _ in dims for d in (dA, dG)]
        arrs = [torch.randn(d, d, device='cuda') for d in sides]
        tri = [True] * len(arrs)
        n = ops.wire_nelems(arrs, tri)
        dense = sum(d * d for d in sides)
        if kind == 'wire_pack':
            wire = torch.empty(n, device='cuda')
            fn = lambda: ops.wire_pack(arrs, tri, wire)
            nbytes = 4 * 2 * n                 # triangle read + packed write
        else:
            wires = [torch.randn(n, device='cuda') for _ in range(p['ranks'])]
            ptrs = [w.data_ptr() for w in wires]
            fn = lambda: ops.wire_unpack_sum(arrs, tri, ptrs,
                                             scale=1.0 / p['ranks'])
            nbytes = 4 * (p['ranks'] * n + dense)
        flops = None
    else:
        F = []
        for d in p['dims']:
            X = torch.randn(2 * d, d, device='cuda')
            F.append((X.T @ X) / (2 * d) + 1e-3 * torch.eye(d, device='cuda'))
        inv = [torch.empty_like(f) for f in F]
        plan = ops.InversePlan(F, inv, [-1] * len(F), [2] * len(F),
                               scale=[0.0] * len(F))
        fn = lambda: plan.run(0.0)
        flops = sum(d ** 3 for d in p['dims'])
    for _ in range(max(args.warmup, 1)):
        fn()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    if flops is None:
        print(json.dumps({'micro': args.micro, 'ms': ms, 'bytes': nbytes,
                          'gbs': nbytes / (ms * 1e-3) / 1e9}))
    else:
        print(json.dumps({'micro': args.micro, 'ms': ms,
                          'tflops': flops / (ms * 1e-3) / 1e12}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--workload', default='resnet50', choices=sorted(WORKLOADS))
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--only-e2e', action='store_true',
                    help='run only the end-to-end steps (KFAC.update on the '
                         'torch model), bracketed by cudaProfilerStart/Stop')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-bn-blocks', action='store_true',
                    help='leave the BatchNormalization layers to the plain '
                         'momentum rule (convolution / fully-connected '
                         'blocks only)')
    ap.add_argument('--bn-dense', action='store_true',
                    help='keep every BatchNormalization block as a dense '
                         '2c x 2c factor (no low-rank form)')
    ap.add_argument('--no-overlap', action='store_true',
                    help='do not start the largest inverses during the '
                         'factor build')
    ap.add_argument('--ownership', default=None,
                    choices=['balanced', 'reference'])
    ap.add_argument('--communicator', default=None,
                    choices=['peer_memory', 'pure_nccl'])
    ap.add_argument('--micro', choices=sorted(MICRO_CASES), default=None,
                    help='time one single-kernel case instead of the step')
    args = ap.parse_args()
    global OWNERSHIP, OVERLAP, COMMUNICATOR
    if args.communicator:
        COMMUNICATOR = args.communicator
    if args.ownership:
        OWNERSHIP = args.ownership
    if args.no_overlap:
        OVERLAP = False
    if args.micro:
        run_micro(args)
    elif args.impl == 'reference':
        run_reference(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
