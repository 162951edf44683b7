"""The optimizer classes (the reference's public interface) on the GPU against
the reference-generated golden trajectory and the oracle."""

import numpy as np
import pytest
import torch
from torch import nn
import torch.nn.functional as F

from oracle import kfac_oracle as orc

pytestmark = pytest.mark.gpu

KFGRAD_TOL = 1e-3
FACTOR_TOL = 1e-4


def rel(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


def host(t):
    return t.detach().cpu().numpy()


class MLP(nn.Module):
    def __init__(self, dims):
        super(MLP, self).__init__()
        self.l1 = nn.Linear(dims[0], dims[1])
        self.l2 = nn.Linear(dims[1], dims[2])
        self.l3 = nn.Linear(dims[2], dims[3])

    def forward(self, x):
        return self.l3(F.relu(self.l2(F.relu(self.l1(x)))))


@pytest.mark.parametrize('fuse', [True, False])
def test_kfac_update_matches_reference_trajectory(golden, fuse):
    import chainerkfac_b200 as ck
    g = golden('mlp_two_steps')
    model = MLP((12, 9, 9, 5)).cuda()
    with torch.no_grad():
        for nm in ('l1', 'l2', 'l3'):
            getattr(model, nm).weight.copy_(torch.from_numpy(g['init.%s.W' % nm]))
            getattr(model, nm).bias.copy_(torch.from_numpy(g['init.%s.b' % nm]))
    opt = ck.KFAC(lr=float(g['lr']), momentum=float(g['momentum']),
                  cov_ema_decay=1.0, damping=float(g['damping']))
    opt.setup(model)
    opt.fuse_update = fuse
    assert [fb.linkname for fb in opt.fblocks] == ['/l1', '/l2', '/l3']
    x = torch.from_numpy(g['x']).cuda()
    t = torch.from_numpy(g['t']).cuda()

    def lossfun(x, t):
        return F.cross_entropy(model(x), t)
    for step in range(2):
        opt.update(lossfun, x, t)
        for nm in ('l1', 'l2', 'l3'):
            link = getattr(opt.target, '_kfac_dummy', None)
        for name, param in opt.target.namedparams():
            key = name.replace('/', '.')
            assert rel(host(param.grad), g['grad%d%s' % (step, key)]) < 1e-4
            assert rel(host(param.kfgrad), g['kfgrad%d%s' % (step, key)]) \
                < KFGRAD_TOL, (step, name)
            assert rel(host(param.data), g['param%d%s' % (step, key)]) < 1e-5
    assert opt.t == 2 and opt.acc_aware_iterations == 2


class SmallNet(nn.Module):
    def __init__(self):
        super(SmallNet, self).__init__()
        self.conv1 = nn.Conv2d(3, 8, 3, 1, 1, bias=True)
        self.bn1 = nn.BatchNorm2d(8)
        self.conv2 = nn.Conv2d(8, 12, 3, 2, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(12)
        self.fc = nn.Linear(12, 7)

    def forward(self, x):
        h = F.relu(self.bn1(self.conv1(x)))
        h = F.relu(self.bn2(self.conv2(h)))
        return self.fc(F.adaptive_avg_pool2d(h, 1).flatten(1))


def capture(model, x, t):
    """Layer inputs / output gradients / parameter gradients by plain autograd."""
    rec, handles = {}, []
    for name, m in model.named_modules():
        if isinstance(m, (nn.Conv2d, nn.Linear, nn.BatchNorm2d)):
            def fwd(mod, inp, out, name=name):
                rec[name + '.x'] = inp[0].detach().cpu().numpy()
                out.register_hook(lambda gr, name=name: rec.__setitem__(
                    name + '.gy', gr.detach().cpu().numpy()))
            handles.append(m.register_forward_hook(fwd))
    model.zero_grad(set_to_none=True)
    F.cross_entropy(model(x), t).backward()
    for h in handles:
        h.remove()
    for name, p in model.named_parameters():
        rec[name + '.grad'] = p.grad.detach().cpu().numpy()
        rec[name] = p.detach().cpu().numpy().copy()
    return rec


def test_kfac_convnet_with_bn_blocks_matches_oracle():
    import chainerkfac_b200 as ck
    torch.manual_seed(0)
    model = SmallNet().cuda()
    x = torch.randn(6, 3, 10, 10, device='cuda')
    t = torch.randint(0, 7, (6,), device='cuda')
    rec = capture(model, x, t)
    # capture() ran a forward pass in train mode: BN running stats moved, the
    # parameters did not.
    damping, lr, mom, stab = 1e-3, 0.05, 0.9, 16.0
    opt = ck.KFAC(lr=lr, momentum=mom, cov_ema_decay=0.9, damping=damping,
                  stab_coeff=stab)
    opt.setup(model)
    assert [type(fb).__name__ for fb in opt.fblocks] == [
        'FisherBlockBatchNormalization', 'FisherBlockBatchNormalization',
        'FisherBlockConvolution2D', 'FisherBlockConvolution2D',
        'FisherBlockLinear']
    opt.update(lambda a, b: F.cross_entropy(model(a), b), x, t)
    blocks = {fb.linkname: fb for fb in opt.fblocks}

    for name, k, s, p, bias in (('conv1', 3, 1, 1, True),
                                ('conv2', 3, 2, 1, False)):
        fb = blocks['/' + name]
        A = orc.conv_A(rec[name + '.x'], k, s, p, bias)
        G = orc.conv_G(rec[name + '.gy'])
        assert rel(host(fb.cov_forward), A) < FACTOR_TOL
        assert rel(host(fb.cov_backward), G) < FACTOR_TOL
        want = orc.connection_step(
            A, G, rec[name + '.weight.grad'],
            rec[name + '.bias.grad'] if bias else None, damping)
        assert rel(host(fb.inv_forward), want['A_inv']) < 1e-4
        assert rel(host(fb.inv_backward), want['G_inv']) < 1e-4
        assert abs(float(fb.diag_val_forward) - want['diag_A']) < \
            1e-5 * want['diag_A']
        assert rel(host(fb.link.W.kfgrad), want['kfgrad_W']) < KFGRAD_TOL
        W = rec[name + '.weight'].copy()
        v = np.zeros_like(W)
        orc.momentum_update(W, v, want['kfgrad_W'], lr, mom)
        assert rel(host(fb.link.W.data), W) < 1e-5

    fb = blocks['/fc']
    A = orc.linear_A(rec['fc.x'], True)
    G = orc.linear_G(rec['fc.gy'])
    want = orc.connection_step(A, G, rec['fc.weight.grad'],
                               rec['fc.bias.grad'], damping)
    assert rel(host(fb.link.W.kfgrad), want['kfgrad_W']) < KFGRAD_TOL
    assert rel(host(fb.link.b.kfgrad), want['kfgrad_b']) < KFGRAD_TOL

    for name in ('bn1', 'bn2'):
        fb = blocks['/' + name]
        Fm = orc.bn_F(rec[name + '.x'], rec[name + '.gy'], model.bn1.eps)
        assert rel(host(fb.cov_backward), Fm) < FACTOR_TOL
        Finv = orc.damped_inverse(Fm, np.float32(orc.bn_damping(damping, stab)))
        assert rel(host(fb.inv_backward), Finv) < 1e-4
        kg, kb = orc.bn_kfgrads(Finv, rec[name + '.weight.grad'],
                                rec[name + '.bias.grad'])
        assert rel(host(fb.link.gamma.kfgrad), kg) < KFGRAD_TOL
        assert rel(host(fb.link.beta.kfgrad), kb) < KFGRAD_TOL
        gam = rec[name + '.weight'].copy()
        v = np.zeros_like(gam)
        orc.momentum_update(gam, v, kg, lr, mom)
        assert rel(host(fb.link.gamma.data), gam) < 1e-5
        assert fb.check_nan() is False


class WideBNNet(nn.Module):
    def __init__(self, c=64):
        super(WideBNNet, self).__init__()
        self.conv1 = nn.Conv2d(3, c, 3, 1, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(c)
        self.conv2 = nn.Conv2d(c, c, 3, 2, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(c)
        self.fc = nn.Linear(c, 5)

    def forward(self, x):
        h = F.relu(self.bn1(self.conv1(x)))
        h = F.relu(self.bn2(self.conv2(h)))
        return self.fc(F.adaptive_avg_pool2d(h, 1).flatten(1))


@pytest.mark.parametrize('decay', [0.9, 1.0])
def test_bn_low_rank_form_gives_the_dense_steps(decay):
    """BatchNormalization blocks kept as stored per-sample gradient rows
    (8 steps x 4 samples <= 64 channels at decay 0.9) against the dense
    2C x 2C factor of the reference, step by step from the same weights, over
    more steps than the history ring has slots; then a batch-size change,
    after which the block must carry on with the dense factor formed from
    its rows."""
    import chainerkfac_b200 as ck
    from chainerkfac_b200.optimizers.fisher_blocks.normalizations \
        .batch_normalization import FisherBlockBatchNormalization as BNB
    models, opts, bns = [], [], []
    for low in (True, False):
        torch.manual_seed(5)
        model = WideBNNet().cuda()
        opt = ck.KFAC(lr=0.02, momentum=0.9, cov_ema_decay=decay,
                      damping=1e-2, bn_low_rank=low)
        opt.setup(model)
        models.append(model)
        opts.append(opt)
        bns.append([fb for fb in opt.fblocks if isinstance(fb, BNB)])
        assert len(bns[-1]) == 2
    g = torch.Generator(device='cuda').manual_seed(11)
    for step in range(14):
        n = 4 if step < 11 else 6
        x = torch.randn(n, 3, 8, 8, device='cuda', generator=g)
        t = torch.randint(0, 5, (n,), device='cuda', generator=g)
        # the dense run restarts every step from the low-rank run's weights,
        # batch statistics and velocities: differences do not compound
        models[1].load_state_dict(models[0].state_dict())
        for p0, p1 in zip(opts[0].target.params(), opts[1].target.params()):
            p1.update_rule.velocity(p1).copy_(p0.update_rule.velocity(p0))
        for model, opt in zip(models, opts):
            opt.update(lambda a, b, m=model: F.cross_entropy(m(a), b), x, t)
        assert all(fb.low_rank_active == (step < 11) for fb in bns[0])
        assert not any(fb.low_rank_active for fb in bns[1])
        if step < 11:
            assert all(fb.invs is None for fb in bns[0])
        for f0, f1 in zip(bns[0], bns[1]):
            assert rel(host(f0.cov_emas[0]), host(f1.cov_emas[0])) < 1e-4, step
            for nm in ('gamma', 'beta'):
                a = host(getattr(f0.link, nm).kfgrad)
                b = host(getattr(f1.link, nm).kfgrad)
                assert rel(a, b) < KFGRAD_TOL, (step, nm, rel(a, b))
        for p0, p1 in zip(models[0].parameters(), models[1].parameters()):
            assert rel(host(p0.data), host(p1.data)) < 1e-5, step
        if step == 5:
            # the reference's per-block calls on a low-rank block give what
            # the optimizer's grouped calls gave (same history, same
            # gradients; no update applied by these)
            for fb in bns[0]:
                want = [host(fb.link.gamma.kfgrad), host(fb.link.beta.kfgrad)]
                fb.link.gamma.kfgrad.zero_()
                fb.link.beta.kfgrad.zero_()
                fb.update_invs()
                fb.update_kfgrads()
                assert rel(host(fb.link.gamma.kfgrad), want[0]) < 1e-5
                assert rel(host(fb.link.beta.kfgrad), want[1]) < 1e-5
                assert len(fb.get_diagvals()[0]) == 128
    assert all(fb.check_nan() is False for fb in bns[0] + bns[1])


def test_classes_started_during_backward_give_the_same_steps(monkeypatch):
    """With several size classes the optimizer starts the inverses of the
    large classes from the backward hooks; the result must not depend on
    that schedule."""
    import chainerkfac_b200 as ck
    monkeypatch.setenv('KFAC_CLASS_BOUNDS', '20,60')
    finals = {}
    for eager in (True, False):
        torch.manual_seed(3)
        model = SmallNet().cuda()       # sides 28/8, 72/12, 16, 24, 13/7
        opt = ck.KFAC(lr=0.05, momentum=0.9, cov_ema_decay=0.9, damping=1e-2)
        opt.eager_inverses = eager
        opt.setup(model)
        g = torch.Generator(device='cuda').manual_seed(4)
        for _ in range(5):
            x = torch.randn(6, 3, 10, 10, device='cuda', generator=g)
            t = torch.randint(0, 7, (6,), device='cuda', generator=g)
            opt.update(lambda a, b: F.cross_entropy(model(a), b), x, t)
        started = opt.observation.get('classes_started_in_backward', 0)
        assert (started > 0) == eager
        finals[eager] = [host(p.data) for p in model.parameters()]
    for a, b in zip(finals[True], finals[False]):
        assert rel(a, b) < 1e-6


def test_deferred_join_gives_the_same_steps(monkeypatch):
    """With defer_join the update returns while size classes still run on
    side streams; every layer waits for its class in a forward pre-hook.
    The trajectory must not change, join() must make the weights readable,
    and a layer that is never called again is joined by the next update."""
    import chainerkfac_b200 as ck
    monkeypatch.setenv('KFAC_CLASS_BOUNDS', '20,60')
    finals = {}
    for defer in (True, False):
        torch.manual_seed(3)
        model = SmallNet().cuda()
        opt = ck.KFAC(lr=0.05, momentum=0.9, cov_ema_decay=0.9, damping=1e-2)
        opt.defer_join = defer
        opt.setup(model)
        g = torch.Generator(device='cuda').manual_seed(4)
        seen_pending = 0
        for _ in range(6):
            x = torch.randn(6, 3, 10, 10, device='cuda', generator=g)
            t = torch.randint(0, 7, (6,), device='cuda', generator=g)
            opt.update(lambda a, b: F.cross_entropy(model(a), b), x, t)
            seen_pending += len(opt._pending_classes)
        assert (seen_pending > 0) == defer
        opt.join()
        assert not opt._pending_classes
        finals[defer] = [host(p.data) for p in model.parameters()]
    for a, b in zip(finals[True], finals[False]):
        assert rel(a, b) < 1e-6


def test_running_average_over_steps_stays_undamped():
    import chainerkfac_b200 as ck
    torch.manual_seed(1)
    model = MLP((6, 5, 5, 3)).cuda()
    opt = ck.KFAC(lr=0.0, momentum=0.0, cov_ema_decay=0.5, damping=1e-2)
    opt.setup(model)
    xs = [torch.rand(8, 6, device='cuda') for _ in range(2)]
    t = torch.randint(0, 3, (8,), device='cuda')
    As = []
    for x in xs:
        opt.update(lambda a, b: F.cross_entropy(model(a), b), x, t)
        As.append(orc.linear_A(host(x), True))
    fb = opt.fblocks[0]
    want = orc.update_cov_ema(As[1], As[0], 0.5)
    assert rel(host(fb.cov_emas[0]), want) < FACTOR_TOL


def _capture_mlp(model, x, t):
    """Per-layer inputs, output gradients and parameter gradients of one
    micro-batch by plain autograd (no optimizer involved)."""
    rec, handles = {}, []
    for name in ('l1', 'l2', 'l3'):
        def fwd(mod, inp, out, name=name):
            rec[name + '.x'] = host(inp[0])
            out.register_hook(lambda gr, name=name: rec.__setitem__(
                name + '.gy', host(gr)))
        handles.append(getattr(model, name).register_forward_hook(fwd))
    model.zero_grad(set_to_none=True)
    F.cross_entropy(model(x), t).backward()
    for h in handles:
        h.remove()
    for name in ('l1', 'l2', 'l3'):
        m = getattr(model, name)
        rec[name + '.gW'] = host(m.weight.grad)
        rec[name + '.gb'] = host(m.bias.grad)
        rec[name + '.W'] = host(m.weight).copy()
    model.zero_grad(set_to_none=True)
    return rec


def test_accumulation_matches_oracle():
    """acc_iters micro-steps on different micro-batches against the
    reference's accumulation rule (kfac.py:259-304) restated in the oracle:
    accumulated factors and gradients, then one K-FAC step on them."""
    import chainerkfac_b200 as ck
    torch.manual_seed(2)
    acc_iters, damping, lr = 3, 1e-2, 0.1
    model = MLP((6, 5, 5, 3)).cuda()
    xs = [torch.rand(8, 6, device='cuda') for _ in range(acc_iters)]
    ts = [torch.randint(0, 3, (8,), device='cuda') for _ in range(acc_iters)]
    recs = [_capture_mlp(model, x, t) for x, t in zip(xs, ts)]
    opt = ck.KFAC(lr=lr, momentum=0.0, cov_ema_decay=1.0, damping=damping,
                  acc_iters=acc_iters)
    opt.setup(model)
    for i, (x, t) in enumerate(zip(xs, ts)):
        opt.update(lambda a, b: F.cross_entropy(model(a), b), x, t)
        assert opt.acc_count == (i + 1) % acc_iters
        assert opt.t == (1 if i + 1 == acc_iters else 0)
    blocks = {fb.linkname: fb for fb in opt.fblocks}
    for name in ('l1', 'l2', 'l3'):
        A = orc.accumulate([orc.linear_A(r[name + '.x'], True) for r in recs],
                           acc_iters)
        G = orc.accumulate([orc.linear_G(r[name + '.gy']) for r in recs],
                           acc_iters)
        gW = orc.accumulate([r[name + '.gW'] for r in recs], acc_iters)
        gb = orc.accumulate([r[name + '.gb'] for r in recs], acc_iters)
        fb = blocks['/' + name]
        assert rel(host(fb.cov_forward), A) < FACTOR_TOL
        assert rel(host(fb.cov_backward), G) < FACTOR_TOL
        assert rel(host(fb.link.W.grad), gW) < 1e-5
        want = orc.connection_step(A, G, gW, gb, damping)
        assert rel(host(fb.link.W.kfgrad), want['kfgrad_W']) < KFGRAD_TOL
        assert rel(host(fb.link.b.kfgrad), want['kfgrad_b']) < KFGRAD_TOL
        W = recs[0][name + '.W'].copy()
        orc.momentum_update(W, np.zeros_like(W), want['kfgrad_W'], lr, 0.0)
        assert rel(host(fb.link.W.data), W) < 1e-5


@pytest.mark.parametrize('fuse', [True, False])
def test_loss_scale_gives_the_unscaled_trajectory(fuse):
    """``KFAC(loss_scale=s)`` scales the backward seed, un-scales the output
    gradients inside the factors (linear.py:34-36) and divides the
    preconditioned gradients by s before the update (kfac.py:72-78): the
    weights must follow the trajectory of the run without a scale."""
    import chainerkfac_b200 as ck
    x = torch.rand(16, 12, device='cuda',
                   generator=torch.Generator(device='cuda').manual_seed(3))
    t = torch.randint(0, 5, (16,), device='cuda',
                      generator=torch.Generator(device='cuda').manual_seed(4))
    finals = []
    for scale in (None, 128.0):
        torch.manual_seed(7)
        model = MLP((12, 9, 9, 5)).cuda()
        opt = ck.KFAC(lr=0.05, momentum=0.9, cov_ema_decay=0.9, damping=1e-2,
                      loss_scale=scale)
        opt.setup(model)
        opt.fuse_update = fuse
        init = [host(p).copy() for p in model.parameters()]
        for _ in range(3):
            opt.update(lambda a, b: F.cross_entropy(model(a), b), x, t)
        finals.append([host(p) - w for p, w in zip(model.parameters(), init)])
    for a, b in zip(*finals):
        assert rel(b, a) < KFGRAD_TOL


def test_normalize_weight_hook_matches_restatement():
    """NormalizeWeightUR as a post-update hook (train.py:56-115): weights
    whose norm exceeds sqrt(2 * out) are scaled down to it on the device,
    others are left alone; the skip_scale_comp schedule gives the same
    weights while it recomputes the norm every step (warm-up)."""
    import chainerkfac_b200 as ck
    from chainerkfac_b200 import recipe
    torch.manual_seed(4)
    model = MLP((12, 9, 9, 5)).cuda()
    with torch.no_grad():
        model.l1.weight.mul_(20.0)          # far above its target norm
    opt = ck.KFAC(lr=0.05, momentum=0.0, cov_ema_decay=1.0, damping=1e-2)
    opt.setup(model)
    opt.fuse_update = False                 # hooks run in the plain rule
    links = dict(opt.target.namedlinks())
    for p in (links['/l1'].W, links['/l2'].W):
        p.update_rule.add_hook(recipe.NormalizeWeightUR(), timing='post')
    x = torch.rand(16, 12, device='cuda')
    t = torch.randint(0, 5, (16,), device='cuda')
    ref = MLP((12, 9, 9, 5)).cuda()
    ref.load_state_dict(model.state_dict())
    o2 = ck.KFAC(lr=0.05, momentum=0.0, cov_ema_decay=1.0, damping=1e-2)
    o2.setup(ref)
    o2.fuse_update = False
    opt.update(lambda a, b: F.cross_entropy(model(a), b), x, t)
    o2.update(lambda a, b: F.cross_entropy(ref(a), b), x, t)
    for name in ('l1', 'l2'):
        got = host(getattr(model, name).weight)
        want = orc.normalize_weight(host(getattr(ref, name).weight))
        assert rel(got, want) < 1e-6
    n1 = float(np.linalg.norm(host(model.l1.weight)))
    assert abs(n1 - np.sqrt(2.0 * 9)) < 1e-4      # clipped
    assert rel(host(model.l3.weight), host(ref.l3.weight)) < 1e-7
    # the interval schedule, during its warm-up, computes the same scale
    w = torch.randn(9, 30, device='cuda') * 3
    p = type('P', (), {})()
    p.data = w.clone()
    rule = type('R', (), {'t': 0})()
    recipe.NormalizeWeightUR(skip_scale_comp=True)(rule, p)
    assert rel(host(p.data), orc.normalize_weight(host(w))) < 1e-6


def test_driver_smoke_entry_point():
    """The driver's smoke() (one small pass of the hot path checked against
    the oracle) stays green."""
    import __graft_entry__
    __graft_entry__.smoke()


def test_bench_resnet50_step_runs():
    from bench_model import build_training_step
    step, h2d, d2h = build_training_step(
        torch.device('cuda', 0), 2, 1, 0, cov_ema_decay=0.9, damping=2.5e-4,
        lr=0.01, momentum=0.9, image=64, classes=10)
    l0 = step()
    l1 = step()
    assert np.isfinite(l0) and np.isfinite(l1)
    assert h2d == 2 * 3 * 64 * 64 * 4 + 2 * 8 and d2h == 4


def test_channels_last_activations_give_the_same_update():
    """The same model and batch with channels-last activations (weights keep
    their layout): factors are read in place from the (n*h*w, c) tensors and
    the update must match the NCHW run."""
    import chainerkfac_b200 as ck

    def make():
        torch.manual_seed(11)
        return nn.Sequential(nn.Conv2d(3, 16, 3, 1, 1), nn.ReLU(),
                             nn.Conv2d(16, 24, 1, 1, 0, bias=False), nn.ReLU(),
                             nn.Conv2d(24, 8, 3, 2, 1), nn.ReLU(),
                             nn.AdaptiveAvgPool2d(1), nn.Flatten(),
                             nn.Linear(8, 5)).cuda()
    g = torch.Generator().manual_seed(5)
    x = torch.randn(6, 3, 12, 12, generator=g).cuda()
    t = torch.randint(0, 5, (6,), generator=g).cuda()
    results = []
    # fp32 convolutions: with TF32 the NCHW and NHWC algorithms of the
    # library differ by 1e-3, which would hide a layout mistake
    tf32 = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    for fmt in (torch.contiguous_format, torch.channels_last):
        m = make()
        opt = ck.KFAC(lr=0.05, momentum=0.9, cov_ema_decay=0.9, damping=1e-2)
        opt.setup(m)
        xin = x.contiguous(memory_format=fmt)
        for _ in range(3):
            opt.update(lambda a, b: F.cross_entropy(m(a), b), xin, t)
        results.append([host(p) for p in m.parameters()])
    torch.backends.cudnn.allow_tf32 = tf32
    errs = [rel(b, a) for a, b in zip(*results)]
    assert max(errs) < 1e-3, errs
