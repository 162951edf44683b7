"""Factor parity at the full sizes of the benchmark configurations.

Every distinct layer shape of ResNet-50 at batch 32 (rows up to 401 408) and
of the CIFAR ResNet-18 at batch 128 (rows up to 131 072) is built by the CUDA
path (through the C ABI) and compared with an fp64 product of the explicitly
unfolded patch matrix, computed on the device with plain torch.  That fp64
construction is itself checked against the oracle's ``conv_A`` / ``conv_G`` on
a small case, so the chain is CUDA kernel -> fp64 unfold -> oracle ->
reference-generated golden vectors.  Tolerance: relative Frobenius error
<= 1e-4, the bound stated for factors.
"""

import zlib

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import bench_workloads as bw
from oracle import kfac_oracle as orc

pytestmark = pytest.mark.gpu

FACTOR_TOL = 1e-4


def rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm())


def factor_A_fp64(x, k, s, p, bias, chunk=4):
    """A = P^T P / n in fp64, P = patches (n*ho*wo, c*k*k [+1]), columns in
    (c, ky, kx) order, accumulated over chunks of images."""
    n, c = x.shape[0], x.shape[1]
    d = c * k * k + int(bias)
    A = torch.zeros((d, d), dtype=torch.float64, device=x.device)
    for i in range(0, n, chunk):
        cols = F.unfold(x[i:i + chunk].double(), k, padding=p, stride=s)
        P = cols.transpose(1, 2).reshape(-1, c * k * k)
        if bias:
            P = torch.cat([P, torch.ones_like(P[:, :1])], 1)
        A += P.T @ P
    return A / n


def factor_G_fp64(gy):
    """G = g^T g * n / (ho*wo), g = gy as (n*ho*wo, c), in fp64."""
    n, c, ho, wo = gy.shape
    g = gy.double().permute(0, 2, 3, 1).reshape(-1, c)
    return (g.T @ g) * (float(n) / (ho * wo))


def test_fp64_construction_matches_oracle():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 5, 9, 9)).astype(np.float32)
    gy = rng.standard_normal((3, 7, 5, 5)).astype(np.float32)
    for k, s, p, bias in ((3, 2, 1, True), (1, 1, 0, False), (3, 1, 1, False)):
        got = factor_A_fp64(torch.from_numpy(x).cuda(), k, s, p, bias, chunk=2)
        want = orc.conv_A(x.astype(np.float64), k, s, p, bias)
        assert rel(got, torch.from_numpy(want).cuda()) < 1e-12
    got = factor_G_fp64(torch.from_numpy(gy).cuda())
    # the oracle scales gy by n before the product and divides by n*ho*wo
    want = orc.conv_G(gy.astype(np.float64))
    assert rel(got, torch.from_numpy(want).cuda()) < 1e-12


def _cases():
    out = []
    for tag, layers in (('resnet50_b32', bw.resnet50_layers(batch=32)),
                        ('resnet18_cifar_b128',
                         bw.resnet18_cifar_layers(batch=128))):
        for l, _ in bw.distinct_shapes(layers):
            out.append(pytest.param(l, id='%s-%s' % (tag, l['name'])))
    return out


@pytest.mark.parametrize('layer', _cases())
def test_factors_at_full_size(layer):
    from chainerkfac_b200 import ops
    g = torch.Generator(device='cuda').manual_seed(
        zlib.crc32(layer['name'].encode()) % 1000 + layer['n'])
    n = layer['n']
    if layer['kind'] == 'linear':
        x = torch.randn((n, layer['cin']), device='cuda', generator=g).relu_()
        gy = torch.randn((n, layer['cout']), device='cuda', generator=g) / n
        A = ops.factor_dense(x, layer['bias'], alpha=1.0 / n)
        G = ops.factor_dense(gy, False, alpha=float(n))
        x64 = x.double()
        if layer['bias']:
            x64 = torch.cat([x64, torch.ones_like(x64[:, :1])], 1)
        assert rel(A, x64.T @ x64 / n) < FACTOR_TOL
        assert rel(G, gy.double().T @ gy.double() * n) < FACTOR_TOL
        return
    k, s, p = layer['k'], layer['stride'], layer['pad']
    x = torch.randn((n, layer['cin'], layer['hin'], layer['hin']),
                    device='cuda', generator=g)
    if layer['cin'] > 3:
        x.relu_()                       # post-ReLU activations
    gy = torch.randn((n, layer['cout'], layer['hout'], layer['hout']),
                     device='cuda', generator=g) / n
    A64 = factor_A_fp64(x, k, s, p, layer['bias'])
    G64 = factor_G_fp64(gy)
    dA, dG, _, _ = bw.layer_dims(layer)
    for fmt in (torch.contiguous_format, torch.channels_last):
        xin = x.contiguous(memory_format=fmt)
        gin = gy.contiguous(memory_format=fmt)
        A = torch.empty((dA, dA), device='cuda')
        G = torch.empty((dG, dG), device='cuda')
        # the grouped entry point is the one the optimizer uses
        ops.factor_group(
            [ops.conv_input_item(xin, k, s, p, layer['bias'], 1.0 / n, 0.0, A),
             ops.conv_grad_item(gin, float(n) / layer['hout'] ** 2, 0.0, G)],
            x.device)
        assert rel(A, A64) < FACTOR_TOL, (fmt, rel(A, A64))
        assert rel(G, G64) < FACTOR_TOL, (fmt, rel(G, G64))
        assert torch.equal(A, A.T) and torch.equal(G, G.T)


@pytest.mark.parametrize('c,h', [(256, 14), (1024, 14), (2048, 7)])
def test_batch_normalization_block_at_resnet50_sizes(c, h):
    """The BatchNormalization block (batch_normalization.py:78-191) at the
    channel counts of ResNet-50's later stages, batch 32, 4-D inputs in both
    layouts: per-sample gradients and factor against the oracle, the damped
    inverse and the preconditioned gradients against the oracle applied to
    the same factor."""
    from chainerkfac_b200 import ops
    n, eps, damping, stab = 32, 2e-5, 2.5e-4, 16.0
    rng = np.random.default_rng(c + h)
    x = rng.standard_normal((n, c, h, h)).astype(np.float32)
    # gradients of a mean-reduced loss shrink with batch and feature-map
    # size; with this scale the damped factors have condition numbers of
    # 1e2..1e3 (refinement covers sides up to 1024; the 2048- and 4096-row
    # factors here are taken as the blocked fp32 algorithm leaves them)
    gy = (rng.standard_normal((n, c, h, h)) * (1.0 / (n * h * h))).astype(
        np.float32)
    gg = rng.standard_normal(c).astype(np.float32)
    gb = rng.standard_normal(c).astype(np.float32)
    want_grads = orc.bn_sample_grads(x, gy, eps)
    want_F = orc.bn_F(x, gy, eps)

    def rel_np(a, b):
        a = np.asarray(a, np.float64)
        b = np.asarray(b, np.float64)
        return np.linalg.norm(a - b) / np.linalg.norm(b)
    xd, gd = torch.from_numpy(x).cuda(), torch.from_numpy(gy).cuda()
    Fs = []
    for fmt in (torch.contiguous_format, torch.channels_last):
        it = ops.bn_item(xd.contiguous(memory_format=fmt),
                         gd.contiguous(memory_format=fmt), eps, float(n))
        ops.bn_sample_grads_group([it])
        assert rel_np(it.result.cpu().numpy(), want_grads) < FACTOR_TOL
        F = torch.empty((2 * c, 2 * c), device='cuda')
        ops.factor_group([ops.dense_item(it.result, False, 1.0 / n, 0.0, F)],
                         F.device)
        assert rel_np(F.cpu().numpy(), want_F) < FACTOR_TOL
        assert torch.equal(F, F.T)
        Fs.append(F)
    F = Fs[0]
    inv = torch.empty_like(F)
    plan = ops.InversePlan([F], [inv], [-1], [2], l2_coef=[0.0], scale=[stab])
    plan.run(damping)
    add = np.float32(orc.bn_damping(damping, stab))
    want_inv = orc.damped_inverse(F.cpu().numpy(), add)
    err = rel_np(inv.cpu().numpy(), want_inv)
    assert err < 1e-4, (err, np.linalg.cond(
        F.cpu().numpy().astype(np.float64) + float(add) * np.eye(2 * c)))
    assert int(plan.info.cpu()[0]) == 0
    kg = torch.empty(c, device='cuda')
    kb = torch.empty(c, device='cuda')
    flag = torch.zeros(2, dtype=torch.int32, device='cuda')
    ops.bn_precondition_group([inv], [torch.from_numpy(gg).cuda()],
                              [torch.from_numpy(gb).cuda()], [kg], [kb],
                              [flag])
    wg, wb = orc.bn_kfgrads(want_inv, gg, gb)
    assert rel_np(kg.cpu().numpy(), wg) < 1e-3
    assert rel_np(kb.cpu().numpy(), wb) < 1e-3
    assert flag.tolist() == [0, 0]
    plan.close()


def test_grouped_build_of_all_resnet50_factors():
    """All 108 factors of ResNet-50 at batch 32 in ONE grouped call, as the
    optimizer and the benchmark issue them.  A grouped call gives each CTA a
    longer stretch of the contraction than a call for one layer does, and the
    tensor core's truncating accumulation drifts with that length, so the
    single-layer cases above do not cover it."""
    import bench
    dev = torch.device('cuda', 0)
    wl = bench.DeviceWorkload(dev, 1234, bench.WORKLOADS['resnet50'],
                              bn_blocks=False)
    outs = [torch.empty_like(e) for e in wl.ema]
    wl.build(list(range(len(wl.layers))), outs, 1.0, 0.0)
    torch.cuda.synchronize()
    worst = 0.0
    for i, l in enumerate(wl.layers):
        if l['name'] not in ('conv1', 'res1.0.conv2', 'res1.1.conv1',
                             'res2.2.conv3', 'res3.5.conv1', 'res4.1.conv2',
                             'fc'):
            continue
        if l['kind'] == 'conv':
            A64 = factor_A_fp64(wl.x[i], l['k'], l['stride'], l['pad'],
                                l['bias'])
            G64 = factor_G_fp64(wl.gy[i])
        else:
            x = wl.x[i].double()
            x = torch.cat([x, torch.ones_like(x[:, :1])], 1)
            A64 = x.T @ x / l['n']
            g = wl.gy[i].double()
            G64 = g.T @ g * l['n']
        eA = rel(outs[wl.fidx[i][0]], A64)
        eG = rel(outs[wl.fidx[i][1]], G64)
        assert eA < FACTOR_TOL and eG < FACTOR_TOL, (l['name'], eA, eG)
        worst = max(worst, eA, eG)
    assert worst < 7e-5, worst      # drift stays well inside the bound
    wl.plan.close()


@pytest.mark.parametrize('c,rows,slots', [(256, 32, 8), (1024, 64, 8),
                                          (2048, 256, 8)])
def test_bn_low_rank_form_at_full_size(c, rows, slots):
    """The low-rank form of a BatchNormalization block at ResNet-50 sizes
    (C up to 2048; 8 slots of 32 rows on one GPU, of 256 rows on eight)
    against the same formula in fp64: two blocks in one grouped call, a ring
    whose newest slot is in the middle, one slot still unused, the fused
    momentum update."""
    from chainerkfac_b200 import ops

    def dev(a):
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()

    def host(t):
        return t.detach().cpu().numpy()

    def rel(a, b):
        return float(np.linalg.norm(a.astype(np.float64) - b) /
                     np.linalg.norm(b))

    rng = np.random.default_rng(c + rows)
    m, d = rows * slots, 2 * c
    dg, db = 16.0 * 2.5e-4, 16.0 * 1e-3
    lr, mom = 0.05, 0.9
    items, wants, outs = [], [], []
    plans = []
    for blk in range(2):
        hist = (rng.standard_normal((m, d)) * 0.5).astype(np.float32)
        age = [(3 - s) % slots for s in range(slots)]      # newest: slot 3
        w = [0.9 * 0.1 ** a * 8.0 / rows for a in age]
        w[5] = 0.0                                           # unused slot
        gg = rng.standard_normal(c).astype(np.float32)
        gb = rng.standard_normal(c).astype(np.float32)
        dinv = np.concatenate([np.full(c, dg ** -0.5), np.full(c, db ** -0.5)])
        scale = np.repeat(np.sqrt(np.array(w, np.float64)), rows)
        Hs64 = hist.astype(np.float64) * scale[:, None] * dinv[None, :]
        gp = np.concatenate([gg, gb]).astype(np.float64) * dinv
        y = np.linalg.solve(np.eye(m) + Hs64 @ Hs64.T, Hs64 @ gp)
        want = (gp - Hs64.T @ y) * dinv
        wants.append(want)
        hist_d = dev(hist)
        Hs = torch.empty_like(hist_d)
        M0 = torch.empty((m, m), device='cuda')
        Minv = torch.empty_like(M0)
        kg, kb = torch.empty(c, device='cuda'), torch.empty(c, device='cuda')
        pg, pb = torch.ones(c, device='cuda'), torch.ones(c, device='cuda')
        vg, vb = torch.zeros(c, device='cuda'), torch.zeros(c, device='cuda')
        flag = torch.zeros(2, dtype=torch.int32, device='cuda')
        items.append(ops.bn_lowrank_item(hist_d, Hs, c, rows, w, dg, db, Minv,
                                         dev(gg), dev(gb), kg, kb, flag,
                                         pg, pb, vg, vb))
        outs.append((Hs, M0, Minv, kg, kb, pg, flag))
    ops.bn_lowrank_scale(items)
    ops.factor_group([ops.dense_t_item(o[0], 1.0, 0.0, o[1]) for o in outs],
                     outs[0][1].device)
    plan = ops.InversePlanSet([o[1] for o in outs], [o[2] for o in outs],
                              [-1, -1], [2, 2], scale=[1.0, 1.0])
    plan.run(1.0, False)
    ops.bn_lowrank_apply(items, lr, mom)
    torch.cuda.synchronize()
    assert plan.info.cpu().tolist() == [0, 0]
    for (Hs, M0, Minv, kg, kb, pg, flag), want in zip(outs, wants):
        got = np.concatenate([host(kg), host(kb)])
        assert rel(got, want) < 1e-3, rel(got, want)
        assert flag.cpu().tolist() == [0, 0]
        # fused update: v = -lr * kf, gamma = 1 + v
        assert rel(host(pg) - 1.0, -lr * want[:c]) < 1e-3
        assert float(Hs[5 * rows:6 * rows].abs().max()) == 0.0
    plan.close()
