"""The NumPy oracle against vectors produced by executing the reference
(tests/golden/make_golden.py).  CPU only."""

import numpy as np
import pytest

from oracle import kfac_oracle as orc
import bench_workloads as bw

TOL = 2e-6


def rel(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


LINEAR = ['linear_bias', 'linear_nobias', 'linear_odd']
CONV = ['conv3x3_bias', 'conv3x3_s2', 'conv1x1_s2', 'conv7x7_s2']


@pytest.mark.parametrize('name', LINEAR + CONV)
def test_connection_block(golden, name):
    g = golden(name)
    bias = 'b' in g
    is_conv = name in CONV
    ema_A = ema_G = None
    for s in range(int(g['steps'])):
        x, gy = g['x%d' % s], g['gy%d' % s]
        if is_conv:
            A = orc.conv_A(x, int(g['ksize']), int(g['stride']),
                           int(g['pad']), bias)
            G = orc.conv_G(gy)
        else:
            A = orc.linear_A(x, bias)
            G = orc.linear_G(gy)
        assert rel(A, g['A%d' % s]) < TOL
        assert rel(G, g['G%d' % s]) < TOL
        assert A.dtype == np.float32 and G.dtype == np.float32
        out = orc.connection_step(A, G, g['gW'], g['gb'] if bias else None,
                                  float(g['damping']), ema_A, ema_G,
                                  float(g['decay']))
        assert abs(out['diag_A'] - g['diag_A%d' % s]) < TOL * g['diag_A%d' % s]
        assert abs(out['diag_G'] - g['diag_G%d' % s]) < TOL * g['diag_G%d' % s]
        # the reference leaves the damped diagonal in its running average
        d = np.arange(A.shape[0])
        damped = out['ema_A'].copy()
        damped[d, d] += out['diag_A']
        assert rel(damped, g['ema_A_damped%d' % s]) < TOL
        assert rel(out['A_inv'], g['A_inv%d' % s]) < 1e-4
        assert rel(out['G_inv'], g['G_inv%d' % s]) < 1e-4
        assert rel(out['kfgrad_W'], g['kfgrad_W%d' % s]) < 1e-4
        assert out['kfgrad_W'].shape == g['W'].shape
        if bias:
            assert rel(out['kfgrad_b'], g['kfgrad_b%d' % s]) < 1e-4
        # next step starts from the state the reference actually kept
        ema_A = g['ema_A_damped%d' % s]
        ema_G = g['ema_G_damped%d' % s]


@pytest.mark.parametrize('name', ['bn_4d', 'bn_2d'])
def test_bn_block(golden, name):
    g = golden(name)
    F = orc.bn_F(g['x'], g['gy'], float(g['eps']))
    assert rel(F, g['F']) < TOL
    diag = orc.bn_damping(float(g['damping']), float(g['stab_coeff']))
    assert abs(diag - g['diag']) < TOL * g['diag']
    F_inv = orc.damped_inverse(F, diag)
    assert rel(F_inv, g['F_inv']) < 1e-4
    kg, kb = orc.bn_kfgrads(F_inv, g['g_gamma'], g['g_beta'])
    assert rel(kg, g['kf_gamma']) < 1e-4
    assert rel(kb, g['kf_beta']) < 1e-4


@pytest.mark.parametrize('d', [10, 65])
def test_inverse(golden, d):
    g = golden('inverse_%d' % d)
    assert rel(orc.inverse(g['a']), g['inv']) < TOL
    assert rel(orc.inverse(g['a']).dot(g['a']), np.eye(d)) < 1e-4


def test_mlp_two_steps(golden):
    """Whole KFAC.update trajectory (cov_ema_decay=1, so no carried state)."""
    g = golden('mlp_two_steps')
    names = ['.l1', '.l2', '.l3']
    P = {n + s: g['init' + n + s].copy() for n in names for s in ('.W', '.b')}
    V = {k: np.zeros_like(v) for k, v in P.items()}
    x, t = g['x'], g['t']
    n = x.shape[0]
    for step in range(2):
        h, acts = x, []
        for i, nm in enumerate(names):
            z = h.dot(P[nm + '.W'].T) + P[nm + '.b']
            acts.append((h, z))
            h = np.maximum(z, 0) if i < 2 else z
        z = h - h.max(axis=1, keepdims=True)
        prob = np.exp(z) / np.exp(z).sum(axis=1, keepdims=True)
        gz = prob.copy()
        gz[np.arange(n), t] -= 1
        gz = (gz / n).astype(np.float32)
        res = {}
        for i in (2, 1, 0):
            h, z = acts[i]
            if i < 2:
                gz = (gz * (z > 0)).astype(np.float32)
            A = orc.linear_A(h, True)
            G = orc.linear_G(gz)
            gW = gz.T.dot(h).astype(np.float32)
            gb = gz.sum(axis=0).astype(np.float32)
            assert rel(gW, g['grad%d' % step + names[i] + '.W']) < TOL
            res[names[i]] = orc.connection_step(A, G, gW, gb,
                                                float(g['damping']))
            gz = gz.dot(P[names[i] + '.W']).astype(np.float32)
        for nm in names:
            for s, key in (('.W', 'kfgrad_W'), ('.b', 'kfgrad_b')):
                kf = res[nm][key]
                assert rel(kf, g['kfgrad%d' % step + nm + s]) < 1e-4
                orc.momentum_update(P[nm + s], V[nm + s], kf,
                                    float(g['lr']), float(g['momentum']))
                assert rel(P[nm + s], g['param%d' % step + nm + s]) < 1e-5


def test_pack_layout_known_answer():
    """3x3 known answer derived from the reference's pack kernel index rule
    dst = r(r+1)/2 + c for c <= r."""
    a = np.arange(9, dtype=np.float32).reshape(3, 3)
    assert orc.pack_lower(a).tolist() == [0, 3, 4, 6, 7, 8]
    s = a + a.T
    assert np.array_equal(orc.unpack_lower(orc.pack_lower(s), 3), s)
    assert np.array_equal(orc.unpack_lower(orc.pack_lower(s), 3, 2.0), s / 2)


def test_collective_semantics():
    rng = np.random.default_rng(0)
    size = 3
    shapes = [[((4, 4), True), ((5,), False)], [((3, 3), True)],
              [((2, 6), False), ((6, 6), True)]]

    def make():
        out = []
        for local in shapes:
            row = []
            for shp, tri in local:
                a = rng.standard_normal(shp).astype(np.float32)
                if tri:
                    a = a + a.T
                row.append((a, tri))
            out.append(row)
        return out
    ranks = [make() for _ in range(size)]
    before = [[[a.copy() for a, _ in loc] for loc in r] for r in ranks]
    orc.reduce_scatter_v_sim(ranks)
    for r in range(size):
        for owner in range(size):
            for j, (a, tri) in enumerate(ranks[r][owner]):
                if owner == r:
                    mean = sum(before[q][owner][j] for q in range(size)) / size
                    assert rel(a, mean) < 1e-6
                else:
                    assert np.array_equal(a, before[r][owner][j])
    owned = [[a.copy() for a, _ in ranks[r][r]] for r in range(size)]
    orc.all_gather_v_sim(ranks)
    for r in range(size):
        for owner in range(size):
            for j, (a, tri) in enumerate(ranks[r][owner]):
                assert rel(a, owned[owner][j]) < 1e-6
    assert orc.split_indices(7, 3) == [[0, 1, 2], [3, 4], [5, 6]]


def test_resnet50_table():
    layers = bw.resnet50_layers()
    assert len(layers) == 54
    dims = [bw.layer_dims(l) for l in layers]
    assert dims[0] == (148, 64, 401408, 401408)
    assert dims[-1] == (2049, 1000, 32, 32)
    assert max(d[0] for d in dims) == 4608
    assert sum(1 for d in dims if d[0] == 4608) == 3
    syrk = sum(r * d * (d + 1) for dA, dG, rA, rG in dims
               for d, r in ((dA, rA), (dG, rG)))
    assert 7.5e11 < syrk < 8.5e11
    inv = sum(dA ** 3 + dG ** 3 for dA, dG, _, _ in dims)
    assert 4.4e11 < inv < 4.7e11
