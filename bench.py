#!/usr/bin/env python
"""Benchmark of the K-FAC curvature hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (``config.workload``): one K-FAC step of a vanilla ResNet-50 at batch
32 per GPU, 224x224 inputs -- for each of its 54 convolution / fully-connected
layers the two Kronecker factors are built from the layer's input activations
and output gradients with the running average fused in (decay 0.9), all 108
factors are inverted with pi-split damping 2.5e-4, and the gradients are
preconditioned and applied with momentum.  Activations and gradients are
synthetic (seeded) tensors of the real shapes; ImageNet is not used.

``value`` is images/sec with activations/gradients resident in HBM; ``e2e`` is
images/sec of the optimizer's public ``update(lossfun, x, t)`` call with the
image batch coming from pinned host memory and the loss read back.  Rank 0
prints one JSON line.  ``--impl reference`` times the reference's CPU (NumPy)
arithmetic for the same stages through the oracle restatement on the host
cores, on one layer per distinct layer shape (times multiplied by the number of
layers of that shape).
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

BATCH = 32
DECAY = 0.9
DAMPING = 2.5e-4
LR = 0.01
MOMENTUM = 0.9
WORKLOAD = 'resnet50_kfac_step_b32_224'
# DRAM traffic of one factor measured with ncu (profiles/), bytes: measured,
# algorithmic (padded input once + factor written once)
TRAFFIC_CASE = (33.9e6, 8.2e6 + 21.2e6)
COMMUNICATOR = 'peer_memory'   # or 'pure_nccl' (NCCL reduce / broadcast)
OVERLAP = True           # start the largest factors' inverse during the factor build
OWNERSHIP = 'balanced'   # layer ownership at N > 1 ('reference': by count)


def layer_table():
    import bench_workloads as bw
    layers = bw.resnet50_layers(batch=BATCH)
    return layers, [bw.layer_dims(l) for l in layers]


def algorithmic_flops(dims):
    """Flops per step per GPU: one triangle of each factor, d^3 per inverse,
    two products per preconditioned gradient."""
    factor = sum(rA * dA * (dA + 1) + rG * dG * (dG + 1)
                 for dA, dG, rA, rG in dims)
    inverse = sum(dA ** 3 + dG ** 3 for dA, dG, _, _ in dims)
    precond = sum(2 * dG * dG * dA + 2 * dG * dA * dA for dA, dG, _, _ in dims)
    return dict(factor=float(factor), inverse=float(inverse),
                precondition=float(precond))


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

    def stop(self, t0=None, t1=None):
        """Summary of the samples read between host times t0 and t1 (the
        timed region); the sampler is started before the warm-up steps, which
        run the same work, and their samples are used (and said so) when the
        timed region was too short to catch one."""
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=['unsampled'])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, smax, reasons = [], [], set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown',
                 'sw_power_cap']
        window = 'timed region'
        lines = [l for ts, l in self.lines
                 if t0 is None or (t0 <= ts <= t1)]
        if not lines:
            window = 'warm-up and timed region'
            lines = [l for ts, l in self.lines if t1 is None or ts <= t1]
        for line in lines:
            parts = [p.strip() for p in line.split(',')]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[3:7]):
                if val.lower().startswith('active'):
                    reasons.add(nm)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=['unsampled'])
        return dict(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(smax)),
                    samples=len(sm), window=window, reasons=sorted(reasons))


# ------------------------------------------------------------- GPU workload
class DeviceWorkload(object):
    """Synthetic per-layer activations, output gradients, weights and K-FAC
    state of ResNet-50 at batch 32, resident on one GPU."""

    def __init__(self, device, seed):
        import torch
        from chainerkfac_b200 import ops
        self.torch, self.ops = torch, ops
        self.layers, self.dims = layer_table()
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        self.x, self.gy, self.W, self.b = [], [], [], []
        self.gW, self.gb, self.vW, self.vb = [], [], [], []
        self.ema, self.inv = [], []
        for i, (l, (dA, dG, _, _)) in enumerate(zip(self.layers, self.dims)):
            n = l['n']
            if l['kind'] == 'conv':
                xs = (n, l['cin'], l['hin'], l['hin'])
                gs = (n, l['cout'], l['hout'], l['hout'])
                ws = (l['cout'], l['cin'], l['k'], l['k'])
            else:
                xs, gs, ws = (n, l['cin']), (n, l['cout']), (l['cout'], l['cin'])
            x = torch.randn(xs, device=device, generator=g)
            if i > 0:
                x.clamp_(min=0)          # post-ReLU activations
            self.x.append(x)
            self.gy.append(torch.randn(gs, device=device, generator=g) / n)
            fan = ws[1] * (ws[2] * ws[3] if len(ws) == 4 else 1)
            self.W.append(torch.randn(ws, device=device, generator=g) / fan ** 0.5)
            self.gW.append(torch.randn(ws, device=device, generator=g) * 1e-2)
            self.vW.append(torch.zeros(ws, device=device))
            if l['bias']:
                self.b.append(torch.zeros(ws[0], device=device))
                self.gb.append(torch.randn(ws[0], device=device, generator=g) * 1e-2)
                self.vb.append(torch.zeros(ws[0], device=device))
            else:
                self.b.append(None)
                self.gb.append(None)
                self.vb.append(None)
            self.ema += [torch.zeros((dA, dA), device=device),
                         torch.zeros((dG, dG), device=device)]
            self.inv += [torch.empty((dA, dA), device=device),
                         torch.empty((dG, dG), device=device)]
        cnt = len(self.layers)
        partner = [j ^ 1 for j in range(2 * cnt)]
        role = [j & 1 for j in range(2 * cnt)]
        self.plan = ops.InversePlanSet(self.ema, self.inv, partner, role)
        self.class_layers = [sorted({i // 2 for i in idx})
                             for idx in self.plan.classes()]
        self.first = True
        self.input_bytes = sum(t.numel() * 4 for t in self.x + self.gy)

    def factor_items(self, outs, r, rest):
        ops, items = self.ops, []
        for i, l in enumerate(self.layers):
            n = l['n']
            A, G = outs[2 * i], outs[2 * i + 1]
            if l['kind'] == 'conv':
                items.append(ops.conv_input_item(
                    self.x[i], l['k'], l['stride'], l['pad'], l['bias'],
                    r / n, rest, A))
                items.append(ops.conv_grad_item(
                    self.gy[i], r * n / float(l['hout'] ** 2), rest, G))
            else:
                items.append(ops.dense_item(self.x[i], l['bias'], r / n, rest,
                                            A))
                items.append(ops.dense_item(self.gy[i], False, r * n, rest, G))
        return items

    def factors_alone(self):
        """The factor stage with nothing else on the device: every factor in
        one grouped call, no inverse started beside it."""
        items = self.factor_items(self.ema, DECAY, 1.0 - DECAY)
        self.ops.factor_group(items, self.ema[0].device)

    def factors(self):
        # all 108 factors in one grouped call per size class, running average
        # fused in, largest class first: its inverse (a long serial chain that
        # uses few SMs) starts on a side stream while the other layers'
        # factors are still being built
        r, rest = (1.0, 0.0) if self.first else (DECAY, 1.0 - DECAY)
        items = self.factor_items(self.ema, r, rest)
        dev = self.ema[0].device
        classes = self.plan.classes() if OVERLAP else []
        done = set()
        for c, idx in enumerate(classes[:-1]):
            self.ops.factor_group([items[i] for i in idx], dev)
            self.plan.start_class(c, DAMPING, True)
            done.update(idx)
        self.ops.factor_group([it for i, it in enumerate(items)
                               if i not in done], dev)
        self.first = False

    def inverses(self):
        # the layers of a size class are preconditioned (and updated) on that
        # class's stream as soon as its inverses are done, next to the
        # remaining classes' inverses
        self.plan.run(DAMPING, True,
                      after_class=self.precondition_class if OVERLAP else None)

    def precondition_class(self, c):
        layers = self.class_layers[c]
        self.ops.precondition(
            [self.inv[2 * i + 1] for i in layers],
            [self.inv[2 * i] for i in layers],
            [self.gW[i] for i in layers], [self.gb[i] for i in layers],
            None, None,
            [self.W[i] for i in layers], [self.b[i] for i in layers],
            [self.vW[i] for i in layers], [self.vb[i] for i in layers],
            lr=LR, momentum=MOMENTUM, ws_key=c)

    def precondition(self):
        if OVERLAP:
            return               # done per class inside inverses()
        cnt = len(self.layers)
        self.ops.precondition(
            [self.inv[2 * i + 1] for i in range(cnt)],
            [self.inv[2 * i] for i in range(cnt)], self.gW, self.gb,
            None, None, self.W, self.b, self.vW, self.vb, lr=LR,
            momentum=MOMENTUM)

    def step(self, events=None):
        self.factors()
        if events is not None:
            events[1].record()
        self.inverses()
        if events is not None:
            events[2].record()
        self.precondition()


class DistributedWorkload(DeviceWorkload):
    """The same per-GPU work as DeviceWorkload for the factor build (every rank
    builds all factors from its own batch), then the reference's two
    exchanges: gradients and packed factors are reduce-scattered to the
    layer's owner, the owner averages them into its running average, inverts
    and preconditions/updates only its own layers, and the updated weights
    are all-gathered.  Ownership is cost-balanced by default (OWNERSHIP);
    'reference' is the reference's contiguous split of the layer list by
    count.

    The first exchange runs size class by size class, largest first: as soon
    as a class is reduced its owners start its inverses on a side stream, next
    to the factor build and exchange of the remaining classes."""

    def __init__(self, device, seed, comm):
        super(DistributedWorkload, self).__init__(device, seed)
        import torch
        self.comm = comm
        from chainerkfac_b200.optimizers.kfac import balanced_split
        cnt = len(self.layers)
        if OWNERSHIP == 'balanced':
            self.indices = balanced_split(
                [float(dA) ** 3 + float(dG) ** 3
                 for dA, dG, _, _ in self.dims], comm.size)
        else:
            # the reference's contiguous split of the layer list by count
            self.indices = [ix.tolist() for ix in
                            np.array_split(np.arange(cnt), comm.size)]
        self.mine = self.indices[comm.rank]
        self.cov = [torch.zeros_like(e) for e in self.ema]
        bounds = self.plan.bounds
        self.plan.close()
        own = self.mine
        self.plan = self.ops.InversePlanSet(
            [self.ema[2 * i + j] for i in own for j in (0, 1)],
            [self.inv[2 * i + j] for i in own for j in (0, 1)],
            [k ^ 1 for k in range(2 * len(own))],
            [k & 1 for k in range(2 * len(own))], bounds=bounds)
        self.own_class_layers = [sorted({own[i // 2] for i in idx})
                                 for idx in self.plan.classes()]
        # size classes over all layers, largest first, as the plan forms them
        key_of = [sum(max(dA, dG) > b for b in bounds)
                  for dA, dG, _, _ in self.dims]
        keys = sorted(set(key_of), reverse=True) if OVERLAP else [None]
        self.class_layers, self.class_rs, self.class_plan = [], [], []
        for key in keys:
            layers = [i for i in range(cnt) if key is None or key_of[i] == key]
            rs = []
            for idx in self.indices:
                loc = []
                for i in idx:
                    if i not in layers:
                        continue
                    # sorted parameter names: W before b
                    loc.append((self.gW[i], False))
                    if self.gb[i] is not None:
                        loc.append((self.gb[i], False))
                    loc.append((self.cov[2 * i], True))
                    loc.append((self.cov[2 * i + 1], True))
                rs.append(loc)
            self.class_layers.append(layers)
            self.class_rs.append(rs)
            self.class_plan.append(
                self.plan.class_keys.index(key)
                if key in self.plan.class_keys else None)
        self.ag_arrays = []
        for idx in self.indices:
            ag = []
            for i in idx:
                ag.append((self.W[i], False))
                if self.b[i] is not None:
                    ag.append((self.b[i], False))
            self.ag_arrays.append(ag)
        self.comm_stream = torch.cuda.Stream(priority=-1)
        if hasattr(comm, 'reserve'):
            from chainerkfac_b200.communicators import _utility
            comm.reserve(max([_utility.get_nelems(rs) for rs in self.class_rs]
                             + [_utility.get_nelems(self.ag_arrays)]), device)

    def factors(self):
        torch = self.torch
        r, rest = (1.0, 0.0) if self.first else (DECAY, 1.0 - DECAY)
        items = self.factor_items(self.cov, 1.0, 0.0)
        dev = self.cov[0].device
        mine = set(self.mine)
        last = len(self.class_layers) - 1
        main = torch.cuda.current_stream()
        for c, layers in enumerate(self.class_layers):
            self.ops.factor_group(
                [items[2 * i + j] for i in layers for j in (0, 1)], dev)
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
                self.comm.reduce_scatter_v_arrays(self.class_rs[c])
                own = [2 * i + j for i in layers if i in mine for j in (0, 1)]
                if own:
                    emas = [self.ema[k] for k in own]
                    self.ops.axpby_group(r, [self.cov[k] for k in own], rest,
                                         emas, emas)
                if c < last and self.class_plan[c] is not None:
                    self.plan.start_class(self.class_plan[c], DAMPING, True)
            if side is not main:
                done = torch.cuda.Event()
                done.record(side)
                self._exchanged = done
        if OVERLAP and last > 0:
            # later work on the main stream (and the next step's factor build,
            # which overwrites cov) comes after the exchanges
            main.wait_event(self._exchanged)
        self.first = False

    def inverses(self):
        self.plan.run(DAMPING, True,
                      after_class=self.precondition_class if OVERLAP else None)

    def precondition_class(self, c):
        own = self.own_class_layers[c]
        self.ops.precondition(
            [self.inv[2 * i + 1] for i in own], [self.inv[2 * i] for i in own],
            [self.gW[i] for i in own], [self.gb[i] for i in own], None, None,
            [self.W[i] for i in own], [self.b[i] for i in own],
            [self.vW[i] for i in own], [self.vb[i] for i in own], lr=LR,
            momentum=MOMENTUM, ws_key=c)

    def precondition(self):
        if OVERLAP:
            # owned layers were updated per size class inside inverses()
            self.comm.all_gather_v_arrays(self.ag_arrays)
            return
        own = self.mine
        self.ops.precondition(
            [self.inv[2 * i + 1] for i in own], [self.inv[2 * i] for i in own],
            [self.gW[i] for i in own], [self.gb[i] for i in own], None, None,
            [self.W[i] for i in own], [self.b[i] for i in own],
            [self.vW[i] for i in own], [self.vb[i] for i in own], lr=LR,
            momentum=MOMENTUM)
        # exchange 2: updated weights to everyone
        self.comm.all_gather_v_arrays(self.ag_arrays)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from chainerkfac_b200 import _lib

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

    if world > 1:
        from chainerkfac_b200.communicators import create_communicator
        wl = DistributedWorkload(device, 1234 + rank,
                                 create_communicator(COMMUNICATOR))
    else:
        wl = DeviceWorkload(device, seed=1234 + rank)
    flops = algorithmic_flops(wl.dims)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        wl.step()
    barrier()

    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)]
          for _ in range(args.steps)]
    launches0 = lib.kfac_launch_count()
    barrier()
    t_begin = time.perf_counter()
    for s in range(args.steps):
        ev[s][0].record()
        wl.step(ev[s])
        ev[s][3].record()
    barrier()
    t_end = time.perf_counter()
    launches = lib.kfac_launch_count() - launches0
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None

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
    value = BATCH * world / (ms_per_step * 1e-3)

    info_bad = int((wl.plan.info != 0).sum().item())

    # The step overlaps the factor build with the first inverses, so the
    # stage events above do not isolate the dominant kernel.  Time the factor
    # stage alone for the roofline: the same grouped launches, nothing beside
    # them, inputs larger than L2, CUDA events on the launching stream.
    factor_alone_ms = None
    if rank == 0 and world == 1:
        reps = max(3, min(args.steps, 10))
        wl.factors_alone()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            wl.factors_alone()
        e1.record()
        torch.cuda.synchronize()
        factor_alone_ms = e0.elapsed_time(e1) / reps

    e2e = None
    if not args.no_e2e:
        try:
            e2e = run_e2e(args, device, world, rank)
        except ImportError as exc:     # API layer not built yet
            e2e = dict(value=None, unit='images/sec', error=str(exc))

    if rank == 0:
        peaks = measured_peaks()
        tf32 = measure_tf32_peak(device)
        names = ['factor', 'inverse', 'precondition']
        # the factor stage is the grouped launches of tc_gemm_kernel, the
        # kernel that also carries the inverse and precondition products
        dom = 0
        dom_ms = factor_alone_ms if factor_alone_ms else phase[dom]
        achieved = flops[names[dom]] / (dom_ms * 1e-3) / 1e12
        stage = {nm: dict(ms=float(ms), tflops=float(flops[nm] / (ms * 1e-3) / 1e12))
                 for nm, ms in zip(names, phase)}
        if OVERLAP and world == 1:
            # each size class is preconditioned on its own stream right after
            # its inverses: that work is inside the 'inverse' interval
            stage['inverse']['tflops'] = float(
                (flops['inverse'] + flops['precondition']) /
                (phase[1] * 1e-3) / 1e12)
            stage['inverse']['includes'] = 'precondition'
            stage['precondition'] = dict(ms=float(phase[2]), tflops=None)
        cpu = None if args.no_cpu_baseline else cpu_baseline_sample(steps=1, warmup=0)
        line = {
            'metric': 'ResNet-50 K-FAC images/sec (factor+inverse+precondition step)',
            'value': value, 'unit': 'images/sec', 'n_gpus': world,
            'steps': args.steps, 'warmup': max(args.warmup, 3),
            'ms_per_step': ms_per_step, 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32',
            'data': 'synthetic',
            'config': {'workload': WORKLOAD, 'batch_per_gpu': BATCH,
                       'layers': len(wl.layers), 'cov_ema_decay': DECAY,
                       'damping': DAMPING,
                       'l2_flush': 'inputs larger than L2 (%.1f GB of '
                                   'activations and gradients per step)'
                                   % (wl.input_bytes / 1e9),
                       'parallelism': 'dp%d' % world,
                       'ownership': OWNERSHIP if world > 1 else None,
                       'communicator': COMMUNICATOR if world > 1 else None},
            # stage boundaries on the main stream; at one GPU the inverses of
            # the larger size classes run on side streams during 'factor', so
            # the per-stage rates there are not isolated kernel rates
            'stages': stage,
            'stages_overlap': bool(OVERLAP and world == 1),
            'factor_alone_ms': factor_alone_ms,
            'factor_inverse_ms': float(phase[0] + phase[1]),
            'roofline': {
                'bound': 'tensor',
                'kernel': 'tc_pair_kernel (factor stage: grouped strided and '
                          'im2col launches over all 108 factors, plus pad '
                          'copies and split reduce)',
                # the factor stage is timed alone (a few launches, tens of
                # ms): the burst figure is its denominator
                'achieved': achieved, 'peak': peaks['tflops_burst'],
                'unit': 'TFLOP/s', 'frac': achieved / peaks['tflops_burst'],
                'peak_source': 'of %s: dense bf16 burst from '
                               'MEASURED_PEAKS.json (kernel timed alone)'
                               % peaks['source'],
                # fp32 operands are split into two bf16 terms: three MMAs per
                # algorithmic product, so a third of the bf16 rate is the
                # ceiling of this scheme
                'frac_of_split_bf16_ceiling':
                    achieved / (peaks['tflops_burst'] / 3.0),
                # the inverse and precondition products run as split TF32
                'tf32_tflops_measured_here': tf32,
                'step_tflops': float(sum(flops.values()) /
                                     (ms_per_step * 1e-3) / 1e12),
                # full-size launches are too large for a multi-pass capture;
                # profiles/ holds DRAM traffic of single factors
                'traffic': None,
                'traffic_case': {'case': 'conv3x3_c256_hw14 (tc_pair_kernel)',
                                 'dram_bytes': TRAFFIC_CASE[0],
                                 'algorithmic_bytes': TRAFFIC_CASE[1]}},
            'cpu_baseline': cpu,
            'gpu_launches': int(launches),
            'clocks': clocks,
            'e2e': e2e,
            'nonpositive_pivots': info_bad,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_e2e(args, device, world, rank):
    """images/sec of KFAC.update(lossfun, x, t) on a torch ResNet-50 with the
    batch copied from pinned host memory and the loss read back every step."""
    import torch
    from bench_model import build_training_step
    step, h2d, d2h = build_training_step(device, BATCH, world, rank,
                                         cov_ema_decay=DECAY, damping=DAMPING,
                                         lr=LR, momentum=MOMENTUM,
                                         communicator=COMMUNICATOR)
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        step()
    t1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([t0.elapsed_time(t1)], device=device, dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(ms, op=torch.distributed.ReduceOp.MAX)
    per = float(ms.item()) / args.steps
    return dict(value=BATCH * world / (per * 1e-3), unit='images/sec',
                ms_per_step=per, h2d_bytes_per_step=h2d,
                d2h_bytes_per_step=d2h)


# ------------------------------------------------------------- CPU baseline
def cpu_layer_inputs(l, rng):
    n = l['n']
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


def cpu_layer_pass(orc, l, inputs):
    """The reference's --no_cuda stages for one layer, via the oracle."""
    x, gy, gW, gb = inputs
    W, v = np.zeros_like(gW), np.zeros_like(gW)
    t0 = time.perf_counter()
    if l['kind'] == 'conv':
        A = orc.conv_A(x, l['k'], l['stride'], l['pad'], l['bias'])
        G = orc.conv_G(gy)
    else:
        A = orc.linear_A(x, l['bias'])
        G = orc.linear_G(gy)
    t1 = time.perf_counter()
    out = orc.connection_step(A, G, gW, gb, DAMPING, None, None, DECAY)
    orc.momentum_update(W, v, out['kfgrad_W'], LR, MOMENTUM)
    t2 = time.perf_counter()
    return t1 - t0, t2 - t1


def cpu_baseline_sample(steps=1, warmup=0, budget_s=150.0):
    """Time the oracle on one layer per distinct shape; scale by multiplicity.
    Stops early (and says so) once `budget_s` seconds of passes have run."""
    from oracle import kfac_oracle as orc
    layers, dims = layer_table()
    groups = {}
    for l, d in zip(layers, dims):
        key = (l['kind'], l.get('k'), l.get('stride'), l['cin'], l['cout'],
               l.get('hin'), l['bias'])
        groups.setdefault(key, [l, 0])[1] += 1
    rng = np.random.default_rng(7)
    inputs = [cpu_layer_inputs(l, rng) for l, _ in groups.values()]
    times, t_start, done = [], time.perf_counter(), 0
    for it in range(warmup + steps):
        tf = ti = 0.0
        for (l, mult), inp in zip(groups.values(), inputs):
            a, b = cpu_layer_pass(orc, l, inp)
            tf += a * mult
            ti += b * mult
        done += 1
        if it >= warmup:
            times.append((tf, ti))
        if time.perf_counter() - t_start > budget_s and times:
            break
    tf = float(np.mean([t[0] for t in times]))
    ti = float(np.mean([t[1] for t in times]))
    return dict(value=BATCH / (tf + ti), unit='images/sec',
                cores=os.cpu_count(), kind='port',
                factor_s=tf, inverse_precondition_s=ti,
                passes_timed=len(times), passes_run=done,
                sample='NumPy oracle (reference --no_cuda arithmetic, all '
                       'host cores through the BLAS threads) on one layer of '
                       'each of the %d distinct ResNet-50 layer shapes, batch '
                       '32; each time multiplied by the number of layers of '
                       'that shape (54 layers in total)' % len(groups))


def run_reference(args):
    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    if rank != 0:
        return
    t0 = time.perf_counter()
    cpu = cpu_baseline_sample(steps=max(args.steps, 1), warmup=args.warmup)
    wall = time.perf_counter() - t0
    value = cpu['value']
    line = {
        'impl': 'reference',
        'metric': 'ResNet-50 K-FAC images/sec (factor+inverse+precondition step)',
        'value': value, 'unit': 'images/sec', 'n_gpus': world,
        'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': 1e3 * BATCH / value, 'higher_is_better': True,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32',
        'data': 'synthetic',
        'config': {'workload': WORKLOAD, 'batch_per_gpu': BATCH,
                   'layers': 54, 'cov_ema_decay': DECAY, 'damping': DAMPING,
                   'parallelism': 'cpu (rank 0 only)'},
        'cpu_baseline': cpu,
        'e2e': {'value': value, 'unit': 'images/sec',
                'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0, 'wall_s': wall,
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
    'inverse_d2304': ('inverse', dict(dims=[2304])),
    'inverse_d4608': ('inverse', dict(dims=[4608])),
    # wire format of the exchange: every factor of ResNet-50 (308 MB packed,
    # 615 MB dense); the sum reads 4 rank buffers, all on this GPU here
    'wire_pack_resnet50': ('wire_pack', dict()),
    'wire_unpack_sum4_resnet50': ('wire_unpack', dict(ranks=4)),
}


def run_micro(args):
    """Time one small case (CUDA events); the command line used for the ncu
    captures summarised under profiles/."""
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
    elif kind in ('wire_pack', 'wire_unpack'):
        _, dims = layer_table()
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
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--no-cpu-baseline', action='store_true')
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
