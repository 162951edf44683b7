"""Parity of the CUDA kernels (called through the C ABI) with the oracle.

Tolerances are the ones the project states for this path: relative Frobenius
error <= 1e-4 on factors and inverses, <= 1e-3 on preconditioned gradients.
Pack/unpack is bit-exact.
"""

import numpy as np
import pytest
import torch

from oracle import kfac_oracle as orc
import bench_workloads as bw

pytestmark = pytest.mark.gpu

FACTOR_TOL = 1e-4
INVERSE_TOL = 1e-4
KFGRAD_TOL = 1e-3


@pytest.fixture(scope='module')
def ops():
    from chainerkfac_b200 import ops as _ops
    return _ops


@pytest.fixture(autouse=True, params=[1, 0], ids=['tcgen05', 'fp32'])
def engine(request):
    """Every test runs on both arithmetic engines: tcgen05 split-TF32 tensor
    cores (the default) and the fp32 FFMA tiles.  After a tensor-core run the
    engine's status word must be clean (no barrier wait ran out)."""
    import ctypes
    from chainerkfac_b200 import _lib
    lib = _lib.load()
    _lib.check(lib.kfac_set_engine(request.param), 'kfac_set_engine')
    yield request.param
    status = ctypes.c_int(-1)
    _lib.check(lib.kfac_tc_status(ctypes.byref(status)), 'kfac_tc_status')
    _lib.check(lib.kfac_set_engine(1), 'kfac_set_engine')
    assert status.value == 0


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def rel(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


def check_symmetric(m):
    assert np.array_equal(m, m.T), 'factor is not bit-symmetric'


# ------------------------------------------------------------------ factors
@pytest.mark.parametrize('name', ['linear_bias', 'linear_nobias', 'linear_odd'])
def test_factor_linear_golden(ops, golden, name):
    g = golden(name)
    bias = 'b' in g
    x, gy = g['x0'], g['gy0']
    n = x.shape[0]
    A = host(ops.factor_dense(dev(x), bias, alpha=1.0 / n))
    G = host(ops.factor_dense(dev(gy), False, alpha=float(n)))
    assert rel(A, g['A0']) < FACTOR_TOL
    assert rel(G, g['G0']) < FACTOR_TOL
    check_symmetric(A)
    check_symmetric(G)


@pytest.mark.parametrize('name', ['conv3x3_bias', 'conv3x3_s2', 'conv1x1_s2',
                                  'conv7x7_s2'])
def test_factor_conv_golden(ops, golden, name):
    g = golden(name)
    bias = 'b' in g
    x, gy = g['x0'], g['gy0']
    n, _, ho, wo = gy.shape
    A = host(ops.factor_conv_input(dev(x), int(g['ksize']), int(g['stride']),
                                   int(g['pad']), bias, alpha=1.0 / n))
    G = host(ops.factor_conv_grad(dev(gy), alpha=n / float(ho * wo)))
    assert rel(A, g['A0']) < FACTOR_TOL
    assert rel(G, g['G0']) < FACTOR_TOL
    check_symmetric(A)


@pytest.mark.parametrize('rows,d,bias', [
    (32, 10, False), (128, 27, True), (128, 784, True), (128, 1000, True),
    (5000, 64, False), (40000, 147, True), (3000, 513, False), (1, 5, True),
    (17, 129, True), (2049, 300, False),
    # 256-row tile pairs: odd number of 128-row blocks with a bias column and
    # a cut contraction; six 256-row blocks, the last with 20 rows
    (70000, 600, True), (6272, 1300, False)])
def test_factor_dense_sweep(ops, rows, d, bias):
    rng = np.random.default_rng(rows * 131 + d)
    x = np.maximum(rng.standard_normal((rows, d)), 0).astype(np.float32)
    want = orc.linear_A(x.astype(np.float64), bias) * rows / 7.0
    got = host(ops.factor_dense(dev(x), bias, alpha=1.0 / 7.0))
    assert got.shape == want.shape
    assert rel(got, want) < FACTOR_TOL
    check_symmetric(got)


def test_factor_dense_strided_rows(ops):
    rng = np.random.default_rng(5)
    big = dev(rng.standard_normal((300, 96)).astype(np.float32))
    x = big[:, :50]                      # leading dimension 96
    from chainerkfac_b200 import _lib
    import ctypes
    lib = _lib.load()
    out = torch.empty((50, 50), device='cuda')
    ws = torch.empty(max(lib.kfac_factor_workspace_bytes(300, 50), 256),
                     dtype=torch.uint8, device='cuda')
    _lib.check(lib.kfac_factor_dense(
        ctypes.c_void_p(x.data_ptr()), 300, 50, 96, 0, 1.0, 0.0,
        ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(ws.data_ptr()),
        ws.numel(), None), 'strided')
    torch.cuda.synchronize()
    xs = host(big)[:, :50].astype(np.float64)
    assert rel(host(out), xs.T @ xs) < FACTOR_TOL


def test_factor_running_average_and_accumulation(ops):
    rng = np.random.default_rng(9)
    x1 = rng.random((64, 33)).astype(np.float32)
    x2 = rng.random((64, 33)).astype(np.float32)
    r = 0.9
    ema = ops.factor_dense(dev(x1), True, alpha=1.0 / 64)
    ops.factor_dense(dev(x2), True, alpha=r / 64, beta=1 - r, out=ema)
    want = orc.update_cov_ema(orc.linear_A(x2, True), orc.linear_A(x1, True), r)
    assert rel(host(ema), want) < FACTOR_TOL
    check_symmetric(host(ema))
    # long contraction (split across CTAs) with beta
    x3 = rng.random((9000, 33)).astype(np.float32)
    acc = ops.factor_dense(dev(x1), True, alpha=0.5 / 64)
    ops.factor_dense(dev(x3), True, alpha=0.5 / 9000, beta=1.0, out=acc)
    want = 0.5 * orc.linear_A(x1, True) + 0.5 * orc.linear_A(x3, True)
    assert rel(host(acc), want) < FACTOR_TOL


@pytest.mark.parametrize('n,c,h,k,s,p,bias', [
    (2, 3, 32, 7, 2, 3, True),      # stem-like
    (2, 64, 14, 3, 1, 1, False),    # 3x3, 576 columns
    (3, 16, 15, 3, 2, 1, False),    # strided 3x3, odd extent
    (2, 40, 9, 1, 1, 0, False),     # 1x1 (strided view path)
    (2, 24, 10, 1, 2, 0, True),     # 1x1 stride 2 (gather path)
    (1, 5, 6, 5, 1, 0, True),       # no padding
    (4, 512, 7, 3, 1, 1, False)])   # 4608 columns
def test_factor_conv_input_sweep(ops, n, c, h, k, s, p, bias):
    rng = np.random.default_rng(n * 7 + c + h + k)
    x = rng.standard_normal((n, c, h, h)).astype(np.float32)
    want = orc.conv_A(x.astype(np.float64), k, s, p, bias)
    got = host(ops.factor_conv_input(dev(x), k, s, p, bias, alpha=1.0 / n))
    assert got.shape == want.shape
    assert rel(got, want) < FACTOR_TOL
    check_symmetric(got)


@pytest.mark.parametrize('n,c,hw', [(2, 5, 3), (4, 64, 28), (3, 130, 7),
                                    (32, 256, 14), (2, 2048, 7)])
def test_factor_conv_grad_sweep(ops, n, c, hw):
    rng = np.random.default_rng(n + c + hw)
    gy = (rng.standard_normal((n, c, hw, hw)) / n).astype(np.float32)
    want = orc.conv_G(gy.astype(np.float64))
    got = host(ops.factor_conv_grad(dev(gy), alpha=n / float(hw * hw)))
    assert rel(got, want) < FACTOR_TOL
    check_symmetric(got)


def test_factor_group_matches_single_calls(ops):
    rng = np.random.default_rng(21)
    xd = dev(rng.random((300, 70)).astype(np.float32))
    xc = dev(rng.standard_normal((3, 16, 12, 12)).astype(np.float32))
    xs = dev(rng.standard_normal((2, 24, 10, 10)).astype(np.float32))
    gy = dev(rng.standard_normal((3, 40, 12, 12)).astype(np.float32))
    big = dev(rng.standard_normal((2, 8, 40, 40)).astype(np.float32))
    prev = dev(np.eye(71, dtype=np.float32))
    want = [
        ops.factor_dense(xd, True, alpha=0.5, beta=0.25, out=prev.clone()),
        ops.factor_conv_input(xc, 3, 1, 1, False, alpha=1 / 3.),
        ops.factor_conv_input(xs, 1, 2, 0, True, alpha=0.5),
        ops.factor_conv_grad(gy, alpha=2.0),
        ops.factor_conv_input(big, 3, 1, 1, True, alpha=1.0),
    ]
    outs = [prev.clone()] + [torch.empty_like(w) for w in want[1:]]
    items = [
        ops.dense_item(xd, True, 0.5, 0.25, outs[0]),
        ops.conv_input_item(xc, 3, 1, 1, False, 1 / 3., 0.0, outs[1]),
        ops.conv_input_item(xs, 1, 2, 0, True, 0.5, 0.0, outs[2]),
        ops.conv_grad_item(gy, 2.0, 0.0, outs[3]),
        ops.conv_input_item(big, 3, 1, 1, True, 1.0, 0.0, outs[4]),
    ]
    ops.factor_group(items, xd.device)
    for w, o in zip(want, outs):
        assert rel(host(o), host(w)) < 1e-5
        check_symmetric(host(o))
    assert rel(host(outs[1]), orc.conv_A(host(xc).astype(np.float64), 3, 1, 1,
                                         False)) < FACTOR_TOL


def test_scratch_buffers_are_per_stream(ops):
    """Factor builds issued on different CUDA streams may run at the same
    time (the exchange stream builds a low-rank block's matrix while the main
    stream builds the next size class): their partial-tile scratch must not
    be the same memory."""
    ws = ops.Workspace()
    dev0 = torch.device('cuda', torch.cuda.current_device())
    a = ws.get(1 << 20, dev0)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        b = ws.get(1 << 20, dev0)
        assert ws.get(1 << 10, dev0) is b          # grow-only, reused
    assert a.data_ptr() != b.data_ptr()
    assert ws.get(1 << 20, dev0) is a
    # and a grouped build on a side stream beside one on the main stream
    rng = np.random.default_rng(5)
    x1 = dev(rng.standard_normal((90000, 200)).astype(np.float32))
    x2 = dev(rng.standard_normal((80000, 150)).astype(np.float32))
    o1 = torch.empty((200, 200), device='cuda')
    o2 = torch.empty((150, 150), device='cuda')
    torch.cuda.synchronize()
    for _ in range(3):
        ops.factor_group([ops.dense_item(x1, False, 1.0 / 90000, 0.0, o1)],
                         dev0)
        with torch.cuda.stream(side):
            ops.factor_group([ops.dense_item(x2, False, 1.0 / 80000, 0.0, o2)],
                             dev0)
    torch.cuda.synchronize()
    w1 = host(x1).astype(np.float64)
    w2 = host(x2).astype(np.float64)
    assert rel(host(o1), w1.T @ w1 / 90000) < FACTOR_TOL
    assert rel(host(o2), w2.T @ w2 / 80000) < FACTOR_TOL


def test_factor_builds_from_staged_operands(ops, engine):
    """The optional operand feed of the factor builds (staging pass that
    writes X^T as two bf16 planes, TMA boxes into the tile kernel) against the
    oracle and against the default feed: every operand kind and layout,
    ragged sizes, a cut contraction, the appended ones column."""
    from chainerkfac_b200 import _lib
    if engine == 0:
        pytest.skip('the staged feed belongs to the tensor-core engine')
    lib = _lib.load()
    rng = np.random.default_rng(77)

    def arr(*shape):
        return dev(rng.standard_normal(shape).astype(np.float32))

    xd, xs = arr(5000, 300), arr(70, 33)
    xl = arr(70000, 130)                      # several splits
    xc, x2, x7 = arr(4, 16, 14, 14), arr(2, 8, 15, 15), arr(2, 3, 30, 30)
    xn = arr(4, 32, 8, 8).contiguous(memory_format=torch.channels_last)
    x1 = arr(3, 24, 6, 6).contiguous(memory_format=torch.channels_last)
    gy = arr(3, 40, 12, 12)
    gn = arr(3, 40, 5, 5).contiguous(memory_format=torch.channels_last)
    xt = arr(48, 1000)
    cases = [
        lambda o: ops.dense_item(xd, True, 1 / 5000., 0.0, o),
        lambda o: ops.dense_item(xs, False, 1.0, 0.0, o),
        lambda o: ops.dense_item(xl, True, 1 / 70000., 0.0, o),
        lambda o: ops.conv_input_item(xc, 3, 1, 1, True, 0.25, 0.0, o),
        lambda o: ops.conv_input_item(x2, 3, 2, 1, False, 0.5, 0.0, o),
        lambda o: ops.conv_input_item(x7, 7, 2, 3, True, 0.5, 0.0, o),
        lambda o: ops.conv_input_item(xn, 3, 1, 1, True, 0.25, 0.0, o),
        lambda o: ops.conv_input_item(x1, 1, 1, 0, False, 1.0, 0.0, o),
        lambda o: ops.conv_grad_item(gy, 2.0, 0.0, o),
        lambda o: ops.conv_grad_item(gn, 2.0, 0.0, o),
        lambda o: ops.dense_t_item(xt, 1.0, 0.0, o),
    ]
    sides = [301, 33, 131, 145, 72, 148, 289, 24, 40, 40, 48]
    results = {}
    for staged in (0, 1):
        lib.kfac_set_factor_staging(staged)
        try:
            outs = [torch.full((d, d), 7.0, device='cuda') for d in sides]
            ops.factor_group([c(o) for c, o in zip(cases, outs)], xd.device)
            # a lone factor takes the by-value descriptor path
            lone = ops.factor_conv_input(xc, 3, 1, 1, True, alpha=0.25)
            torch.cuda.synchronize()
            results[staged] = [host(o) for o in outs] + [host(lone)]
        finally:
            lib.kfac_set_factor_staging(0)
    for k, (a, b) in enumerate(zip(results[1], results[0])):
        assert rel(a, b) < 2e-6, (k, rel(a, b))
        check_symmetric(a)
    want = orc.conv_A(host(xc).astype(np.float64), 3, 1, 1, True)
    assert rel(results[1][3], want) < FACTOR_TOL
    want = orc.conv_A(host(xn).astype(np.float64), 3, 1, 1, True)
    assert rel(results[1][6], want) < FACTOR_TOL
    want = host(xl).astype(np.float64)
    want = np.concatenate([want, np.ones((70000, 1))], 1)
    assert rel(results[1][2], want.T @ want / 70000.) < FACTOR_TOL
    assert rel(results[1][10],
               host(xt).astype(np.float64) @ host(xt).astype(np.float64).T) \
        < FACTOR_TOL


@pytest.mark.parametrize('name', ['bn_4d', 'bn_2d'])
def test_bn_factor_golden(ops, golden, name):
    g = golden(name)
    x, gy = g['x'], g['gy']
    n = x.shape[0]
    grads = ops.bn_sample_grads(dev(x), dev(gy), float(g['eps']), float(n))
    want = orc.bn_sample_grads(x, gy, float(g['eps']))
    assert rel(host(grads), want) < FACTOR_TOL
    F = host(ops.factor_dense(grads, False, alpha=1.0 / n))
    assert rel(F, g['F']) < FACTOR_TOL


def test_bounded_wait_expires_and_reports(ops):
    """A barrier wait that can never be satisfied gives up after its poll
    limit, raises its status word and lets the kernel return (the mechanism
    every tile kernel's waits use); the context stays usable."""
    import ctypes
    from chainerkfac_b200 import _lib
    lib = _lib.load()
    status, returned = ctypes.c_int(-1), ctypes.c_int(-1)
    _lib.check(lib.kfac_selftest_wait_expiry(ctypes.byref(status),
                                             ctypes.byref(returned)),
               'kfac_selftest_wait_expiry')
    assert status.value == 1 and returned.value == 2
    x = torch.ones(4, 3, device='cuda')
    assert float(ops.factor_dense(x, False, alpha=1.0).sum()) == 36.0


# ------------------------------------------------------------------ inverse
def spd(rng, d, m=None):
    m = m or max(2 * d, 64)
    X = rng.standard_normal((m, d)).astype(np.float32)
    return (X.T @ X / m + 1e-3 * np.eye(d)).astype(np.float32)


def run_pairs(ops, dimsA, dimsG, damping, use_pi=True, seed=0):
    rng = np.random.default_rng(seed)
    mats, partner, role = [], [], []
    for i, (da, dg) in enumerate(zip(dimsA, dimsG)):
        mats += [spd(rng, da), spd(rng, dg)]
        partner += [2 * i + 1, 2 * i]
        role += [0, 1]
    F = [dev(m) for m in mats]
    inv = [torch.empty_like(f) for f in F]
    plan = ops.InversePlan(F, inv, partner, role)
    plan.run(damping, use_pi)
    torch.cuda.synchronize()
    assert host(plan.info).tolist() == [0] * len(mats)
    diag = host(plan.diag)
    for i in range(len(dimsA)):
        A, G = mats[2 * i], mats[2 * i + 1]
        pi, dA, dG = orc.connection_damping(
            A, G, damping, 0.0, 'tracenorm' if use_pi else 'none')
        assert abs(diag[2 * i] - dA) <= 1e-5 * dA
        assert abs(diag[2 * i + 1] - dG) <= 1e-5 * dG
        for m, add, got in ((A, dA, inv[2 * i]), (G, dG, inv[2 * i + 1])):
            want = orc.damped_inverse(m, np.float32(add))
            truth = np.linalg.inv(m.astype(np.float64) +
                                  float(add) * np.eye(m.shape[0]))
            got = host(got)
            assert rel(got, want) < INVERSE_TOL, (m.shape, rel(got, want))
            assert rel(got, truth) < INVERSE_TOL
            assert np.array_equal(got, got.T)
        # the factors themselves stay undamped
        assert np.array_equal(host(F[2 * i]), A)
    plan.close()


def test_inverse_small_batch(ops):
    run_pairs(ops, [10, 27, 65, 148, 300], [7, 64, 128, 129, 257], 1e-3)


def test_inverse_no_pi(ops):
    run_pairs(ops, [33, 200], [16, 130], 2.5e-4, use_pi=False, seed=3)


def test_inverse_mlp_shapes(ops):
    run_pairs(ops, [785, 1001], [1000, 10], 1e-3, seed=1)


def test_inverse_large(ops):
    run_pairs(ops, [1152, 2304], [128, 513], 2.5e-4, seed=2)


@pytest.mark.parametrize('d', [10, 65])
def test_inverse_golden(ops, golden, d):
    g = golden('inverse_%d' % d)
    F = [dev(g['a'])]
    inv = [torch.empty_like(F[0])]
    plan = ops.InversePlan(F, inv, [-1], [2], l2_coef=[0.0], scale=[0.0])
    plan.run(0.0)
    assert rel(host(inv[0]), g['inv']) < INVERSE_TOL
    plan.close()


def test_inverse_bn_role_and_repeat(ops, golden):
    g = golden('bn_4d')
    F = [dev(g['F'])]
    inv = [torch.empty_like(F[0])]
    plan = ops.InversePlan(F, inv, [-1], [2], scale=[float(g['stab_coeff'])])
    for _ in range(2):          # a plan is reusable
        plan.run(float(g['damping']))
        assert abs(host(plan.diag)[0] - g['diag']) < 1e-6 * g['diag']
        assert rel(host(inv[0]), g['F_inv']) < INVERSE_TOL
    plan.close()


def test_inverse_bn_block_floors_each_half_separately(ops):
    """gamma and beta carry their own l2_coef floors
    (batch_normalization.py:141-157): the first half of the diagonal gets
    max(l2_gamma, damping) * stab_coeff, the second max(l2_beta, damping) *
    stab_coeff."""
    rng = np.random.default_rng(21)
    c, damping, stab = 9, 1e-2, 4.0
    F = spd(rng, 2 * c)
    Fd = [dev(F)]
    inv = [torch.empty_like(Fd[0])]
    plan = ops.InversePlan(Fd, inv, [-1], [2], l2_coef=[0.05], scale=[stab],
                           l2_coef_second=[0.002])
    plan.run(damping)
    add = np.concatenate([np.full(c, max(0.05, damping) * stab),
                          np.full(c, max(0.002, damping) * stab)])
    want = np.linalg.inv(F.astype(np.float64) + np.diag(add))
    assert rel(host(inv[0]), want) < INVERSE_TOL
    assert abs(host(plan.diag)[0] - 0.05 * stab) < 1e-6
    plan.close()


def test_inverse_reports_non_spd(ops):
    a = np.eye(40, dtype=np.float32)
    a[17, 17] = -1.0
    F = [dev(a), dev(np.eye(6, dtype=np.float32))]
    inv = [torch.empty_like(f) for f in F]
    plan = ops.InversePlan(F, inv, [-1, -1], [2, 2], scale=[0.0, 0.0])
    plan.run(0.0)
    assert host(plan.info).tolist() == [18, 0]
    assert rel(host(inv[1]), np.eye(6)) < 1e-6
    plan.close()


# ------------------------------------------------------------- precondition
def precond_case(rng, dG, dW, bias):
    dA = dW + int(bias)
    Gi = spd(rng, dG)
    Ai = spd(rng, dA)
    gW = rng.standard_normal((dG, dW)).astype(np.float32)
    gb = rng.standard_normal(dG).astype(np.float32) if bias else None
    return Gi, Ai, gW, gb


def test_precondition_matches_oracle(ops):
    rng = np.random.default_rng(11)
    shapes = [(10, 1000, True), (64, 147, True), (300, 129, False),
              (1000, 784, True), (7, 5, False), (256, 2304, False)]
    cases = [precond_case(rng, *s) for s in shapes]
    Gi = [dev(c[0]) for c in cases]
    Ai = [dev(c[1]) for c in cases]
    gW = [dev(c[2]) for c in cases]
    gb = [None if c[3] is None else dev(c[3]) for c in cases]
    kW = [torch.empty_like(t) for t in gW]
    kb = [None if t is None else torch.empty_like(t) for t in gb]
    ops.precondition(Gi, Ai, gW, gb, kW, kb)
    for c, w, b in zip(cases, kW, kb):
        wantW, wantb = orc.connection_kfgrads(c[1], c[0], c[2], c[3])
        assert rel(host(w), wantW) < KFGRAD_TOL
        if b is not None:
            assert rel(host(b), wantb) < KFGRAD_TOL


def test_precondition_conv_shape_and_fused_update(ops):
    rng = np.random.default_rng(12)
    Gi, Ai, gW2, gb = precond_case(rng, 20, 3 * 3 * 6, True)
    gW = gW2.reshape(20, 6, 3, 3)
    W = rng.standard_normal(gW.shape).astype(np.float32)
    b = rng.standard_normal(20).astype(np.float32)
    vW = rng.standard_normal(gW.shape).astype(np.float32)
    vb = rng.standard_normal(20).astype(np.float32)
    dW_, db_, dvW, dvb = dev(W), dev(b), dev(vW), dev(vb)
    kW, kb = torch.empty_like(dW_), torch.empty_like(db_)
    ops.precondition([dev(Gi)], [dev(Ai)], [dev(gW)], [dev(gb)], [kW], [kb],
                     [dW_], [db_], [dvW], [dvb], lr=0.05, momentum=0.9)
    wantW, wantb = orc.connection_kfgrads(Ai, Gi, gW, gb)
    assert rel(host(kW), wantW) < KFGRAD_TOL
    assert rel(host(kb), wantb) < KFGRAD_TOL
    orc.momentum_update(W, vW, wantW, 0.05, 0.9)
    orc.momentum_update(b, vb, wantb, 0.05, 0.9)
    assert rel(host(dW_), W) < 1e-5
    assert rel(host(db_), b) < 1e-5
    assert rel(host(dvW), vW) < KFGRAD_TOL


def test_momentum_update_and_axpby(ops):
    rng = np.random.default_rng(13)
    p = rng.standard_normal(100003).astype(np.float32)
    v = rng.standard_normal(100003).astype(np.float32)
    g = rng.standard_normal(100003).astype(np.float32)
    dp, dv = dev(p), dev(v)
    ops.momentum_update(dev(g), dp, dv, 0.01, 0.9)
    orc.momentum_update(p, v, g, 0.01, 0.9)
    assert rel(host(dp), p) < 1e-6 and rel(host(dv), v) < 1e-6
    y = dev(g)
    ops.axpby(0.25, dev(p), 0.75, y, y)
    assert rel(host(y), 0.25 * p + 0.75 * g) < 1e-6


def test_bn_kfgrad(ops, golden):
    g = golden('bn_4d')
    c = g['g_gamma'].shape[0]
    y0 = torch.empty(c, device='cuda')
    y1 = torch.empty(c, device='cuda')
    flag = torch.zeros(2, dtype=torch.int32, device='cuda')
    ops.symv_split(dev(g['F_inv']), dev(g['g_gamma']), dev(g['g_beta']), y0, y1,
                   flag)
    assert rel(host(y0), g['kf_gamma']) < KFGRAD_TOL
    assert rel(host(y1), g['kf_beta']) < KFGRAD_TOL
    assert flag.tolist() == [0, 0]
    # a NaN anywhere in the product: the raw gradients come back instead
    # (the reference's _check_nan fallback), the counter goes up, and the
    # next clean call is unaffected
    bad = g['F_inv'].copy()
    bad[2, 3] = np.nan
    ops.symv_split(dev(bad), dev(g['g_gamma']), dev(g['g_beta']), y0, y1, flag)
    assert flag.tolist() == [0, 1]
    assert np.array_equal(host(y0), g['g_gamma'])
    assert np.array_equal(host(y1), g['g_beta'])
    ops.symv_split(dev(g['F_inv']), dev(g['g_gamma']), dev(g['g_beta']), y0, y1,
                   flag)
    assert flag.tolist() == [0, 1]
    assert rel(host(y0), g['kf_gamma']) < KFGRAD_TOL


def test_bn_lowrank_form_matches_dense_oracle(ops):
    """The low-rank form of a BatchNormalization block -- (D + sum_s w_s
    U_s^T U_s)^-1 g through the m x m matrix I + Hs Hs^T -- against the dense
    path of the oracle: running average of three steps' factors (decay 0.9),
    separate damping of the gamma and beta halves, damped inverse, product
    with the gradient."""
    rng = np.random.default_rng(31)
    n, c, steps, r = 8, 20, 3, 0.9
    d_gamma, d_beta = 16.0 * 1e-3, 16.0 * 5e-3
    Us = [(rng.standard_normal((n, 2 * c)) * 0.3).astype(np.float32)
          for _ in range(steps)]
    # oracle: F_t = r U^T U / n + (1 - r) F_{t-1}, first step plain
    F = None
    for U in Us:
        cov = (U.T @ U / n).astype(np.float32)
        F = cov if F is None else orc.update_cov_ema(cov, F, r)
    add = np.concatenate([np.full(c, d_gamma), np.full(c, d_beta)])
    Finv = np.linalg.inv(F.astype(np.float64) + np.diag(add))
    gg = rng.standard_normal(c).astype(np.float32)
    gb = rng.standard_normal(c).astype(np.float32)
    want = Finv @ np.concatenate([gg, gb])
    # weights of the slots, oldest first: (1-r)^2, r(1-r), r; each over n
    w = [(1 - r) ** 2 / n, r * (1 - r) / n, r / n, 0.0]    # one unused slot
    hist = dev(np.concatenate(Us + [np.full((n, 2 * c), 7.0, np.float32)]))
    m = 4 * n
    Hs = torch.empty_like(hist)
    M0 = torch.empty((m, m), device='cuda')
    Minv = torch.empty_like(M0)
    kg, kb = torch.empty(c, device='cuda'), torch.empty(c, device='cuda')
    flag = torch.zeros(2, dtype=torch.int32, device='cuda')
    item = ops.bn_lowrank_item(hist, Hs, c, n, w, d_gamma, d_beta, Minv,
                               dev(gg), dev(gb), kg, kb, flag)
    ops.bn_lowrank_scale([item])
    ops.factor_group([ops.dense_t_item(Hs, 1.0, 0.0, M0)], M0.device)
    plan = ops.InversePlan([M0], [Minv], [-1], [2], scale=[1.0])
    plan.run(1.0, use_pi=False)
    ops.bn_lowrank_apply([item])
    got = np.concatenate([host(kg), host(kb)])
    assert rel(got, want) < KFGRAD_TOL
    assert rel(got, want) < 1e-4        # and in fact far inside it
    assert flag.tolist() == [0, 0]
    # the unused slot contributes nothing: its rows are zero in Hs
    assert float(Hs[3 * n:].abs().max()) == 0.0
    plan.close()


# -------------------------------------------------------------- wire format
@pytest.mark.parametrize('n,c,h,k,s,p,bias', [
    (2, 40, 9, 1, 1, 0, True),      # its own patch matrix: read in place
    (2, 64, 14, 3, 1, 1, False),    # staged as zero-bordered NCHW planes
    (2, 24, 10, 1, 2, 0, False),    # staged without a border
    (2, 3, 32, 7, 2, 3, True),      # few channels, bias column
    (3, 40, 9, 3, 1, 1, True)])     # sizes that are no multiples of 32
def test_factor_conv_channels_last(ops, n, c, h, k, s, p, bias):
    """Channels-last activations and gradients give the factors of the same
    logical NCHW tensors."""
    rng = np.random.default_rng(7 * n + c + h + k)
    x = np.maximum(rng.standard_normal((n, c, h, h)), 0).astype(np.float32)
    want = orc.conv_A(x.astype(np.float64), k, s, p, bias)
    xd = dev(x).contiguous(memory_format=torch.channels_last)
    got = host(ops.factor_conv_input(xd, k, s, p, bias, alpha=1.0 / n))
    assert rel(got, want) < FACTOR_TOL
    out = torch.empty_like(dev(got))
    ops.factor_group([ops.conv_input_item(xd, k, s, p, bias, 1.0 / n, 0.0,
                                          out)], out.device)
    assert rel(host(out), want) < FACTOR_TOL
    gy = (rng.standard_normal((n, c, h, h)) / n).astype(np.float32)
    wantg = orc.conv_G(gy.astype(np.float64))
    gd = dev(gy).contiguous(memory_format=torch.channels_last)
    gotg = host(ops.factor_conv_grad(gd, alpha=n / float(h * h)))
    assert rel(gotg, wantg) < FACTOR_TOL
    outg = torch.empty_like(dev(gotg))
    ops.factor_group([ops.conv_grad_item(gd, n / float(h * h), 0.0, outg)],
                     outg.device)
    assert rel(host(outg), wantg) < FACTOR_TOL


def test_axpby_group_matches_single_calls(ops):
    rng = np.random.default_rng(77)
    shapes = [(3, 3), (8192,), (100, 130), (1,), (8193, 2)]
    xs = [dev(rng.standard_normal(s).astype(np.float32)) for s in shapes]
    ys = [dev(rng.standard_normal(s).astype(np.float32)) for s in shapes]
    want = [ops.axpby(0.9, x, 0.1, y, torch.empty_like(y))
            for x, y in zip(xs, ys)]
    outs = [y.clone() for y in ys]
    ops.axpby_group(0.9, xs, 0.1, outs, outs)        # in place on y
    for o, w in zip(outs, want):
        assert torch.equal(o, w)
    outs = [torch.full_like(y, 7.0) for y in ys]
    ops.axpby_group(1.0, xs, 0.0, ys, outs)          # plain copy
    for o, x in zip(outs, xs):
        assert torch.equal(o, x)


def test_wire_pack_unpack_bit_exact(ops):
    rng = np.random.default_rng(14)
    shapes = [((37, 37), True), ((11,), False), ((1, 1), True),
              ((300, 300), True), ((4, 9), False)]
    arrs = []
    for shp, tri in shapes:
        a = rng.standard_normal(shp).astype(np.float32)
        if tri:
            a = (a + a.T).astype(np.float32)
        arrs.append(a)
    tri = [t for _, t in shapes]
    d_arrs = [dev(a) for a in arrs]
    n = ops.wire_nelems(d_arrs, tri)
    nested = [[(a, t) for a, t in zip(arrs, tri)]]
    assert n == orc.wire_nelems(nested)
    wire = torch.full((n,), 7.0, device='cuda')
    ops.wire_pack(d_arrs, tri, wire)
    assert np.array_equal(host(wire), orc.pack_arrays(nested))
    # selective pack with zero fill (all-gather send side)
    sel = [1, 0, 1, 0, 1]
    ops.wire_pack(d_arrs, tri, wire, select=sel, zero_skipped=True)
    want = orc.pack_arrays(nested)
    off = 0
    for a, t, s in zip(arrs, tri, sel):
        m = a.shape[0] * (a.shape[0] + 1) // 2 if t else a.size
        if not s:
            want[off:off + m] = 0
        off += m
    assert np.array_equal(host(wire), want)
    # unpack with mean scaling mirrors the triangles
    ops.wire_pack(d_arrs, tri, wire)
    outs = [torch.zeros_like(t) for t in d_arrs]
    ops.wire_unpack(outs, tri, wire, scale=0.25)
    for a, o in zip(arrs, outs):
        assert np.array_equal(host(o), a * np.float32(0.25))
    # fused running average on unpack
    prev = [dev(np.ones_like(a)) for a in arrs]
    ops.wire_unpack(prev, tri, wire, scale=1.0, ema_r=0.5)
    for a, o in zip(arrs, prev):
        assert rel(host(o), 0.5 * a + 0.5) < 1e-6


@pytest.mark.parametrize('wdt', [torch.float16, torch.bfloat16])
def test_wire_reduced_precision(ops, wdt):
    """A 16-bit wire buffer holds each value rounded to the wire type (the
    cast of pure_nccl_communicator.py:354-375); the sum over several wire
    buffers is formed in fp32 from the widened values (:438-461)."""
    rng = np.random.default_rng(15)
    shapes = [((70, 70), True), ((1000,), False), ((129, 129), True)]
    arrs = []
    for shp, tri in shapes:
        a = rng.standard_normal(shp).astype(np.float32)
        arrs.append((a + a.T).astype(np.float32) if tri else a)
    tri = [t for _, t in shapes]
    nested = [[(a, t) for a, t in zip(arrs, tri)]]
    n = orc.wire_nelems(nested)
    ranks = 3
    wires, want = [], np.zeros(n, np.float32)
    for r in range(ranks):
        scaled = [dev(a * np.float32(r + 1)) for a in arrs]
        w = torch.zeros(n, dtype=wdt, device='cuda')
        ops.wire_pack(scaled, tri, w)
        exp = torch.from_numpy(orc.pack_arrays(
            [[(a * np.float32(r + 1), t) for a, t in zip(arrs, tri)]])).to(wdt)
        assert torch.equal(w.cpu(), exp)          # rounded to nearest
        want += exp.float().numpy()
        wires.append(w)
    outs = [torch.zeros_like(dev(a)) for a in arrs]
    ops.wire_unpack_sum(outs, tri, [w.data_ptr() for w in wires],
                        scale=1.0 / ranks, wire_dtype=wdt)
    ref = [np.zeros_like(a) for a in arrs]
    orc.unpack_arrays([[(a, t) for a, t in zip(ref, tri)]], want,
                      divisor=float(ranks))
    for o, a in zip(outs, ref):
        assert rel(host(o), a) < 1e-6
        if a.ndim == 2:
            assert np.array_equal(host(o), host(o).T)


def test_wire_unpack_sum_of_rank_buffers(ops):
    """The owner's side of the peer-memory reduce-scatter: the same slot of
    several wire buffers (one per rank; here all on this GPU) summed in rank
    order, scaled to the mean and mirrored.  Sizes straddle the 64-wide tiles
    and the 8192-element runs; unselected arrays must stay untouched and must
    not shift the offsets of the others."""
    rng = np.random.default_rng(41)
    shapes = [((130, 130), True), ((8192 + 77,), False), ((64, 64), True),
              ((5, 7), False), ((513, 513), True), ((0,), False),
              ((65, 65), True)]
    tri = [t for _, t in shapes]
    ranks = 5
    per_rank, wires = [], []
    for q in range(ranks):
        arrs = []
        for shp, t in shapes:
            a = rng.standard_normal(shp).astype(np.float32)
            if t:
                a = (a + a.T).astype(np.float32)
            arrs.append(a)
        per_rank.append(arrs)
        d = [dev(a) for a in arrs]
        w = torch.empty(ops.wire_nelems(d, tri), device='cuda')
        ops.wire_pack(d, tri, w)
        assert np.array_equal(
            host(w), orc.pack_arrays([[(a, t) for a, t in zip(arrs, tri)]]))
        wires.append(w)
    sel = [1, 1, 0, 1, 1, 1, 1]
    outs = [torch.full(shp, 3.0, device='cuda') for shp, _ in shapes]
    ops.wire_unpack_sum(outs, tri, [w.data_ptr() for w in wires], select=sel,
                        scale=1.0 / ranks)
    for i, (o, s) in enumerate(zip(outs, sel)):
        if not s:
            assert np.array_equal(host(o), np.full(shapes[i][0], 3.0, np.float32))
            continue
        acc = np.zeros(shapes[i][0], np.float32)
        for q in range(ranks):         # rank order, fp32, as the kernel sums
            acc = acc + per_rank[q][i]
        want = acc * np.float32(1.0 / ranks)
        assert np.array_equal(host(o), want), i
        if tri[i]:
            assert np.array_equal(host(o), host(o).T)
    with pytest.raises(Exception):
        ops.wire_unpack_sum(outs, tri, [wires[0].data_ptr()] * 17)


# ------------------------------------------- full-size, size-independent checks
def test_config4_full_size_inverse_property(ops, engine):
    """The isolated curvature microbench at its full sizes: factors with the
    dimensions of every ResNet-50 layer, each X^T X / m + 1e-3 I with m = 8192
    rows of N(0,1), built by the factor kernel, inverted in one batch (three
    streams by size class).  Checked through inv * F ~ I, which needs no CPU
    inverse of a 4608 x 4608 matrix."""
    if engine == 0:
        pytest.skip('full-size sweep runs on the tensor-core engine only')
    dims = sorted({d for l in bw.resnet50_layers()
                   for d in bw.layer_dims(l)[:2]})
    g = torch.Generator(device='cuda')
    g.manual_seed(4)
    m = 8192
    F = []
    for d in dims:
        X = torch.randn((m, d), device='cuda', generator=g)
        eye = torch.eye(d, device='cuda') * 1e-3
        F.append(ops.factor_dense(X, False, alpha=1.0 / m, beta=1.0, out=eye))
        del X
    inv = [torch.empty_like(f) for f in F]
    plan = ops.InversePlanSet(F, inv, [-1] * len(F), [2] * len(F),
                              scale=[0.0] * len(F))
    plan.run(0.0)
    torch.cuda.synchronize()
    assert int(plan.info.abs().sum()) == 0
    for d, f, i in zip(dims, F, inv):
        resid = (i.double() @ f.double() -
                 torch.eye(d, device='cuda', dtype=torch.float64))
        err = float(resid.norm() / d ** 0.5)
        assert err < INVERSE_TOL, (d, err)
        assert torch.equal(i, i.T)
    plan.close()


def test_config1_mlp_shapes_step(ops):
    """One K-FAC pass at the MNIST-MLP shapes (784-1000-1000-10, batch 128,
    damping 1e-3) against the oracle, all three layers in grouped calls."""
    rng = np.random.default_rng(1)
    dims = [(784, 1000), (1000, 1000), (1000, 10)]
    xs = [rng.random((128, di)).astype(np.float32) for di, _ in dims]
    gys = [(rng.standard_normal((128, do)) / 128).astype(np.float32)
           for _, do in dims]
    gWs = [rng.standard_normal((do, di)).astype(np.float32) for di, do in dims]
    gbs = [rng.standard_normal(do).astype(np.float32) for _, do in dims]
    F, items = [], []
    for (di, do), x, gy in zip(dims, xs, gys):
        A = torch.empty((di + 1, di + 1), device='cuda')
        G = torch.empty((do, do), device='cuda')
        F += [A, G]
        items.append(ops.dense_item(dev(x), True, 1.0 / 128, 0.0, A))
        items.append(ops.dense_item(dev(gy), False, 128.0, 0.0, G))
    ops.factor_group(items, F[0].device)
    inv = [torch.empty_like(f) for f in F]
    plan = ops.InversePlan(F, inv, [1, 0, 3, 2, 5, 4], [0, 1] * 3)
    plan.run(1e-3)
    assert plan.refined() >= 2      # at least the two large A factors
    kW = [torch.empty(w.shape, device='cuda') for w in gWs]
    kb = [torch.empty(b.shape, device='cuda') for b in gbs]
    ops.precondition([inv[1], inv[3], inv[5]], [inv[0], inv[2], inv[4]],
                     [dev(w) for w in gWs], [dev(b) for b in gbs], kW, kb)
    for i in range(3):
        want = orc.connection_step(orc.linear_A(xs[i], True),
                                   orc.linear_G(gys[i]), gWs[i], gbs[i], 1e-3)
        assert rel(host(F[2 * i]), want['ema_A']) < FACTOR_TOL
        # These factors are ill-conditioned (uniform[0,1) inputs: cond ~ 6e3
        # to 1.4e4 with damping 1e-3); the plan's probe sees that and runs
        # the fp64-residual refinement step on them.  The inverse stage is
        # compared on identical inputs: the oracle inverts the factor this
        # stage was given (a factor that differs by 2e-6 moves the inverse
        # by up to cond * 2e-6, whoever computes it), with the damping the
        # oracle derives from it.
        for j, key in ((0, 'A_inv'), (1, 'G_inv')):
            f = host(F[2 * i + j])
            _, dA, dG = orc.connection_damping(host(F[2 * i]),
                                               host(F[2 * i + 1]), 1e-3)
            add = np.float32(dA if j == 0 else dG)
            oracle_inv = orc.damped_inverse(f, add)
            truth = np.linalg.inv(f.astype(np.float64) +
                                  float(add) * np.eye(len(f)))
            got = host(inv[2 * i + j])
            assert rel(got, oracle_inv) < INVERSE_TOL, (i, key)
            assert rel(got, truth) < INVERSE_TOL, (i, key)
        assert rel(host(kW[i]), want['kfgrad_W']) < KFGRAD_TOL
        assert rel(host(kb[i]), want['kfgrad_b']) < KFGRAD_TOL
    plan.close()
