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


def test_accumulation_matches_one_big_step():
    import chainerkfac_b200 as ck
    torch.manual_seed(2)
    m1 = MLP((6, 5, 5, 3)).cuda()
    m2 = MLP((6, 5, 5, 3)).cuda()
    m2.load_state_dict(m1.state_dict())
    x = torch.rand(8, 6, device='cuda')
    t = torch.randint(0, 3, (8,), device='cuda')
    o1 = ck.KFAC(lr=0.1, cov_ema_decay=1.0, damping=1e-2, acc_iters=2)
    o1.setup(m1)
    for _ in range(2):       # same micro-batch twice == one step on it
        o1.update(lambda a, b: F.cross_entropy(m1(a), b), x, t)
    assert o1.t == 1 and o1.acc_count == 0
    o2 = ck.KFAC(lr=0.1, cov_ema_decay=1.0, damping=1e-2)
    o2.setup(m2)
    o2.update(lambda a, b: F.cross_entropy(m2(a), b), x, t)
    for p1, p2 in zip(m1.parameters(), m2.parameters()):
        assert rel(host(p1), host(p2)) < 1e-5


def test_bench_resnet50_step_runs():
    from chainerkfac_b200.bench_model import build_training_step
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
