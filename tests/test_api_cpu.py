"""Host-side logic of the optimizer / communicator classes (no GPU): the
reference's interface, ownership split, wire layout and the two collectives
over gloo with two processes."""

import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

from oracle import kfac_oracle as orc
import bench_workloads as bw

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def small_model():
    return nn.Sequential(nn.Conv2d(3, 4, 3, 1, 1), nn.BatchNorm2d(4),
                         nn.ReLU(), nn.Flatten(), nn.Linear(4 * 4 * 4, 5))


def test_public_interface_and_defaults():
    import chainerkfac_b200 as ck
    from chainerkfac_b200.optimizers import fisher_blocks as FB
    opt = ck.KFAC()
    assert (opt.lr, opt.momentum, opt.cov_ema_decay, opt.damping) == \
        (0.001, 0.9, 0.99, 0.03)
    assert opt.stab_coeff == 16.0 and opt.acc_iters == 1
    assert opt.pi_type == 'tracenorm'
    opt.lr = 0.5                       # run-time mutable proxies
    assert opt.hyperparam.lr == 0.5 and opt.lr_pre == 0.001
    opt.setup(small_model())
    kinds = [type(fb) for fb in opt.fblocks]
    assert kinds == [FB.FisherBlockConvolution2D,
                     FB.FisherBlockBatchNormalization, FB.FisherBlockLinear]
    assert [fb.linkname for fb in opt.fblocks] == ['/0', '/1', '/4']
    fb = opt.fblocks[0]
    assert fb.link.ksize == 3 and fb.link.stride == (1, 1) and fb.link.pad == (1, 1)
    assert fb.covs is None and fb.cov_emas is None and fb.invs is None
    with pytest.raises(RuntimeError):
        fb.update_cov_emas()           # 'covs is None', as in the reference
    names = [n for n, _ in opt.target.namedparams()]
    assert names == ['/0/W', '/0/b', '/1/gamma', '/1/beta', '/4/W', '/4/b']
    rule = opt.target.__dict__['_children'][0][1].W.update_rule
    assert rule.hyperparam.lr == 0.5   # rules see the optimizer's values
    with pytest.raises(ValueError):
        ck.create_communicator('mpi')
    with pytest.raises(NotImplementedError):
        ck.KFAC(use_cholesky=False).setup(small_model())


def test_bn_low_rank_history_weights_follow_the_running_average():
    """Host logic of the low-rank form of a BatchNormalization block: which
    blocks take it, how the history ring rotates, and that the slot weights
    reproduce the reference's running average (fisher_block.py:155-163)
    F <- decay * F_new + (1 - decay) * F up to the forgotten tail."""
    import chainerkfac_b200 as ck
    from chainerkfac_b200.optimizers.fisher_blocks.normalizations \
        .batch_normalization import lowrank_window
    assert [lowrank_window(d) for d in (1.0, 0.9, 0.99, 0.5)] == [1, 8, 4, 27]
    assert lowrank_window(0.05) == 0          # window longer than the ring
    model = nn.Sequential(nn.Conv2d(3, 64, 3), nn.BatchNorm2d(64))
    opt = ck.KFAC(cov_ema_decay=0.9).setup(model)
    fb = opt.fblocks[1]
    assert fb.low_rank_world == 1 and not fb.low_rank_active
    fb.deferred = True
    # 8 slots x 8 samples = 64 rows <= 64 channels: low rank; 9 samples: dense
    assert fb._low_rank_wanted(8, 64) == (8, 8, 1, 0.9)
    assert fb._low_rank_wanted(9, 64) is None
    assert ck.KFAC(acc_iters=2).setup(model).fblocks[1].low_rank_world is None
    assert ck.KFAC(bn_low_rank=False).setup(model).fblocks[1] \
        .low_rank_world is None
    fb._low_rank_setup((8, 8, 1, 0.9), 64, torch.device('cpu'))
    assert fb.low_rank_active and fb.plan_entries() == [] and \
        fb.plan_factors() == [] and not fb.has_state()
    assert fb._lr['hist'].shape == (64, 128) and fb.max_side() == 64
    rng = np.random.default_rng(0)
    dense = None
    for step in range(12):                    # more steps than slots
        rows = rng.standard_normal((8, 128)).astype(np.float32)
        slot = fb._next_slot()
        assert slot.data_ptr() == fb._lr['hist'][
            ((step % 8) * 8):].data_ptr()
        slot.copy_(torch.from_numpy(rows))
        fb.commit_rows()
        f_new = rows.astype(np.float64).T @ rows / 8
        dense = f_new if dense is None else 0.9 * f_new + 0.1 * dense
        hist = fb._lr['hist'].numpy().astype(np.float64)
        got = sum(w * fb._row_factor() * hist[8 * k:8 * k + 8].T @
                  hist[8 * k:8 * k + 8] for k, w in enumerate(fb._lr['w']))
        assert np.linalg.norm(got - dense) <= 2e-8 * np.linalg.norm(dense)
    assert fb.has_state()
    # a rank that does not own the block keeps one slot only
    other = ck.KFAC(cov_ema_decay=0.9).setup(model).fblocks[1]
    other.keeps_history, other.low_rank_world, other.low_rank_rank = \
        False, 2, 1
    other._low_rank_setup((4, 8, 2, 0.9), 64, torch.device('cpu'))
    assert other._lr['hist'].shape == (8, 128) and other._lr['M'] is None
    assert other._next_slot().shape == (8, 128) and other.cov_emas is None


def test_balanced_ownership_is_deterministic_and_even():
    from chainerkfac_b200.optimizers.kfac import balanced_split
    dims = [bw.layer_dims(l) for l in bw.resnet50_layers()]
    costs = [float(a) ** 3 + float(g) ** 3 for a, g, _, _ in dims]
    for size in (2, 4, 8):
        owned = balanced_split(costs, size)
        assert sorted(i for o in owned for i in o) == list(range(54))
        loads = [sum(costs[i] for i in o) for o in owned]
        ref = [sum(costs[i] for i in o) for o in orc.split_indices(54, size)]
        assert max(loads) <= max(ref)
        assert owned == balanced_split(costs, size)
    two = [sum(costs[i] for i in o) for o in balanced_split(costs, 2)]
    assert max(two) / (sum(two) / 2) < 1.02


def test_adjust_momentum_rule():
    from chainerkfac_b200.optimizers.kfac import KFACUpdateRule, _base
    hp = _base.Hyperparameter()
    hp.lr, hp.lr_pre, hp.momentum = 0.05, 0.1, 0.9
    assert KFACUpdateRule(hp, adjust_momentum=True).effective_momentum() == \
        pytest.approx(0.45)
    assert KFACUpdateRule(hp).effective_momentum() == 0.9


def test_recipe_schedule_and_soft_target_loss():
    """LrPolynomialDecay and the soft-target cross entropy of the ImageNet
    recipe against their restatements (host-side glue: runs on the CPU)."""
    from chainerkfac_b200 import recipe
    sched = recipe.LrPolynomialDecay(0.8, 2, 10, p=2)
    for e in (0.0, 1.99, 2.0, 5.5, 9.99, 10.0, 12.0):
        assert sched.lr(e) == pytest.approx(
            orc.lr_polynomial_decay(e, 0.8, 2, 10, 2))

    class Opt(object):
        lr, lr_pre = 0.8, 0.8
    opt = Opt()
    sched(opt, 6.0)
    assert opt.lr_pre == 0.8 and opt.lr == pytest.approx(0.8 * 0.25)
    rng = np.random.default_rng(3)
    x = rng.standard_normal((7, 5)).astype(np.float32)
    t = np.array([0, 4, -1, 2, 2, 1, 3])
    tt = rng.random((7, 5)).astype(np.float32)
    tt /= tt.sum(axis=1, keepdims=True)
    for soft in (None, tt):
        xt = torch.from_numpy(x).requires_grad_(True)
        loss = recipe.softmax_cross_entropy(
            xt, torch.from_numpy(t), None if soft is None
            else torch.from_numpy(soft))
        loss.backward()
        want_loss, want_gx = orc.soft_target_cross_entropy(x, t, soft)
        assert float(loss) == pytest.approx(want_loss, rel=1e-5)
        assert np.allclose(xt.grad.numpy(), want_gx, rtol=1e-4, atol=1e-6)


class NumpyWire(object):
    """Pack/unpack of the wire format with the oracle (CPU stand-in for the
    library kernels, injected by these tests only)."""

    def _pack(self, flat, tri, wire, select):
        off = 0
        for i, (a, t) in enumerate(zip(flat, tri)):
            p = orc.pack_lower(a.numpy()) if t else a.numpy().reshape(-1)
            if select is None or select[i]:
                wire[off:off + p.size] = torch.from_numpy(p.copy())
            off += p.size

    def _unpack(self, flat, tri, wire, select, scale):
        off = 0
        for i, (a, t) in enumerate(zip(flat, tri)):
            n = a.shape[0] * (a.shape[0] + 1) // 2 if t else a.numel()
            if select is None or select[i]:
                seg = wire[off:off + n].numpy() * np.float32(scale)
                if t:
                    a.copy_(torch.from_numpy(orc.unpack_lower(seg, a.shape[0])))
                else:
                    a.copy_(torch.from_numpy(seg.reshape(a.shape)))
            off += n


class FakePeerMemory(NumpyWire):
    """CPU stand-in for the mapped wire buffers of the peer-memory
    communicator: a 'device address' is a (buffer, rank) token, and the
    barrier copies every rank's buffers to every rank (what peer loads would
    see afterwards)."""

    def _map_wire(self, nelems, device):
        if not hasattr(self, '_bufs'):
            self._bufs, self._seen = [], []
        k = len(self._bufs)
        t = torch.zeros(nelems)
        self._bufs.append(t)
        self._seen.append(None)
        return t, [(k, r) for r in range(self.size)]

    def _barrier(self, device):
        dist.barrier()
        for k, t in enumerate(self._bufs):
            got = [torch.empty_like(t) for _ in range(self.size)]
            dist.all_gather(got, t)
            self._seen[k] = got

    def _unpack_sum(self, flat, tri, ptrs, select, scale):
        total = None
        for k, r in ptrs:
            w = self._seen[k][r]
            total = w.clone() if total is None else total + w
        self._unpack(flat, tri, total, select, scale)


def make_arrays(rng, size):
    shapes = [[((4, 4), True), ((5,), False)], [((3, 3), True), ((2, 6), False)],
              [((6, 6), True)]][:size]
    out = []
    for local in shapes:
        row = []
        for shp, tri in local:
            a = rng.standard_normal(shp).astype(np.float32)
            if tri:
                a = (a + a.T).astype(np.float32)
            row.append((a, tri))
        out.append(row)
    return out


def check_single_exchange_accumulation(ck, comm, rank, size):
    """acc_iters micro-steps of DistributedKFAC: every rank accumulates its
    own gradients and factors (kfac.py:286-304) and the owners receive, in
    ONE reduce-scatter per update, the mean over ranks of the accumulated
    arrays -- what the reference obtains by exchanging in every micro-step.
    The device arithmetic is replaced by torch on the CPU; the sequencing,
    the arrays handed to the communicator and the values the curvature
    stages then see are what is checked."""
    from chainerkfac_b200 import ops
    from chainerkfac_b200.optimizers import kfac as kfac_mod

    def axpby_group(a, xs, b, ys, outs):
        for x, y, o in zip(xs, ys, outs):
            o.copy_(a * x + (b * y if b != 0.0 else 0.0))
    old = ops.axpby_group
    ops.axpby_group = axpby_group
    try:
        acc = 3
        torch.manual_seed(0)
        model = nn.Sequential(nn.Linear(6, 5), nn.ReLU(), nn.Linear(5, 4),
                              nn.ReLU(), nn.Linear(4, 3))
        opt = ck.DistributedKFAC(comm, lr=0.1, acc_iters=acc)
        opt.setup(model)
        opt.update()                   # first call only broadcasts
        calls, seen = [], {}
        orig_rs = comm.reduce_scatter_v_arrays
        comm.reduce_scatter_v_arrays = lambda arrays, stream=None: (
            calls.append(1), orig_rs(arrays, stream))[1]

        def fake_update_kfgrads(fblocks):
            for i in opt.local_indices:
                fb = opt.fblocks[i]
                seen[i] = ([c.clone() for c in fb.covs],
                           fb.link.W.grad.clone())
        opt.update_kfgrads = fake_update_kfgrads
        opt.comm.all_gather_v_arrays = lambda arrays, stream=None: None
        for p in opt.target.params():
            p.update = lambda: None
        rngs = [np.random.default_rng(500 + q) for q in range(size)]
        per_rank = []                  # [rank][micro][block] -> (A, G, gW)
        for q in range(size):
            micro = []
            for m in range(acc):
                blocks = []
                for fb in opt.fblocks:
                    dG = fb.link.W.shape[0]
                    dA = fb.link.W.size // dG + 1
                    A = rngs[q].standard_normal((dA, dA)).astype(np.float32)
                    G = rngs[q].standard_normal((dG, dG)).astype(np.float32)
                    gW = rngs[q].standard_normal(
                        tuple(fb.link.W.shape)).astype(np.float32)
                    blocks.append(((A + A.T) / 2, (G + G.T) / 2, gW))
                micro.append(blocks)
            per_rank.append(micro)
        for m in range(acc):
            for fb, (A, G, gW) in zip(opt.fblocks, per_rank[rank][m]):
                fb.covs = [torch.from_numpy(A.copy()),
                           torch.from_numpy(G.copy())]
                fb.link.W.grad = torch.from_numpy(gW.copy())
                fb.link.b.grad = torch.zeros(tuple(fb.link.b.shape))
            opt.update()
            assert len(calls) == (1 if m == acc - 1 else 0)
        assert opt.t == 1 and opt.acc_count == 0
        for i in opt.local_indices:
            for j in (0, 1, 2):
                want = np.mean(
                    [orc.accumulate([per_rank[q][m][i][j]
                                     for m in range(acc)], acc)
                     for q in range(size)], axis=0)
                got = (seen[i][0][j] if j < 2 else seen[i][1]).numpy()
                assert np.allclose(got, want, rtol=1e-5, atol=1e-6), (i, j)
    finally:
        ops.axpby_group = old


def _worker(rank, size, port, tmp):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port),
                      RANK=str(rank), WORLD_SIZE=str(size))
    dist.init_process_group('gloo', rank=rank, world_size=size)
    import chainerkfac_b200 as ck
    from chainerkfac_b200.communicators.pure_nccl_communicator import \
        PureNcclCommunicator

    class TestComm(NumpyWire, PureNcclCommunicator):
        pass
    from chainerkfac_b200.communicators.peer_memory_communicator import \
        PeerMemoryCommunicator

    class TestPeerComm(FakePeerMemory, PeerMemoryCommunicator):
        pass
    # same collectives through the peer-memory sequencing, twice, so that
    # both alternating wire buffers are reused
    peer = TestPeerComm()
    for rep in range(2):
        per_rank = [make_arrays(np.random.default_rng(70 + rep * 10 + q), size)
                    for q in range(size)]
        mine = [[(torch.from_numpy(a.copy()), t) for a, t in loc]
                for loc in per_rank[rank]]
        peer.reduce_scatter_v_arrays(mine)
        want = [[[(a.copy(), t) for a, t in loc] for loc in r]
                for r in per_rank]
        orc.reduce_scatter_v_sim(want)
        for o in range(size):
            for (a, _), (w, _) in zip(mine[o], want[rank][o]):
                assert np.allclose(a.numpy(), w, rtol=1e-6, atol=1e-7)
        peer.all_gather_v_arrays(mine)
        orc.all_gather_v_sim(want)
        for o in range(size):
            for (a, _), (w, _) in zip(mine[o], want[rank][o]):
                assert np.allclose(a.numpy(), w, rtol=1e-6, atol=1e-7)
    assert len(peer._bufs) == 2

    comm = TestComm()
    assert comm.rank == rank and comm.size == size
    # every rank's local values (seeded per rank), same nested structure
    per_rank = [make_arrays(np.random.default_rng(10 + q), size)
                for q in range(size)]
    mine = [[(torch.from_numpy(a.copy()), t) for a, t in loc]
            for loc in per_rank[rank]]
    comm.reduce_scatter_v_arrays(mine)
    want = [[[(a.copy(), t) for a, t in loc] for loc in r] for r in per_rank]
    orc.reduce_scatter_v_sim(want)
    for o in range(size):
        for (a, _), (w, _) in zip(mine[o], want[rank][o]):
            assert np.allclose(a.numpy(), w, rtol=1e-6, atol=1e-7), (rank, o)
    comm.all_gather_v_arrays(mine)
    orc.all_gather_v_sim(want)
    for o in range(size):
        for (a, _), (w, _) in zip(mine[o], want[rank][o]):
            assert np.allclose(a.numpy(), w, rtol=1e-6, atol=1e-7), (rank, o)
    # ownership split and first-call broadcast of DistributedKFAC
    torch.manual_seed(rank)            # different initial weights per rank
    model = small_model()
    opt = ck.DistributedKFAC(comm, lr=0.1)
    opt.setup(model)
    assert opt.indices == orc.split_indices(3, size)
    assert opt.local_indices == opt.indices[rank]
    assert comm.indices == opt.indices
    assert opt.only_pic_update_weight is True
    opt.update()                       # first call: parameters changed -> bcast
    assert opt.t == 0
    flat = torch.cat([p.data.reshape(-1) for p in opt.target.params()])
    gathered = [torch.empty_like(flat) for _ in range(size)]
    dist.all_gather(gathered, flat)
    assert all(torch.equal(gathered[0], g) for g in gathered)
    with pytest.warns(UserWarning):
        comm.allreduce_grad()
    check_single_exchange_accumulation(ck, comm, rank, size)
    open(os.path.join(tmp, 'ok%d' % rank), 'w').close()
    dist.destroy_process_group()


@pytest.mark.parametrize('size', [2, 3])
def test_collectives_and_ownership_over_gloo(tmp_path, size):
    port = 29500 + (os.getpid() + size) % 2000
    mp.spawn(_worker, args=(size, port, str(tmp_path)), nprocs=size, join=True)
    assert all(os.path.exists(str(tmp_path / ('ok%d' % r)))
               for r in range(size))
