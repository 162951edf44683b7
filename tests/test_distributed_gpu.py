"""DistributedKFAC on two GPUs (one process each, NCCL) against single-process
KFAC on the concatenated batch.  Skipped where fewer than two GPUs exist."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys
sys.path.insert(0, %(root)r)
import numpy as np, torch, torch.distributed as dist
import torch.nn.functional as F
from torch import nn
import chainerkfac_b200 as ck

rank = int(os.environ['RANK']); world = int(os.environ['WORLD_SIZE'])
torch.cuda.set_device(rank)
dist.init_process_group('nccl', device_id=torch.device('cuda', rank))

def make():
    torch.manual_seed(7)
    return nn.Sequential(nn.Conv2d(3, 6, 3, 1, 1), nn.ReLU(),
                         nn.Conv2d(6, 8, 3, 2, 1, bias=False), nn.ReLU(),
                         nn.AdaptiveAvgPool2d(1), nn.Flatten(),
                         nn.Linear(8, 5)).cuda()

g = torch.Generator().manual_seed(3)
X = torch.randn(8, 3, 8, 8, generator=g).cuda()
T = torch.randint(0, 5, (8,), generator=g).cuda()
half = 8 // world
xs, ts = X[rank * half:(rank + 1) * half], T[rank * half:(rank + 1) * half]

# one communicator of each kind for the whole run: the peer-memory one maps
# its wire buffers once and reuses them across optimizers
comms = {name: ck.create_communicator(name)
         for name in ('pure_nccl', 'peer_memory')}

# the two communicators must deliver identical arrays for identical input
gen = torch.Generator().manual_seed(100 + rank)
def arrays():
    out = []
    for o in range(world):
        f = torch.randn(70 + o, 70 + o, generator=gen)
        out.append([((f + f.T).cuda(), True),
                    (torch.randn(9000 + o, generator=gen).cuda(), False)])
    return out
a_nccl = arrays()
a_peer = [[(t.clone(), tri) for t, tri in loc] for loc in a_nccl]
for rep in range(3):
    comms['pure_nccl'].reduce_scatter_v_arrays(a_nccl)
    comms['peer_memory'].reduce_scatter_v_arrays(a_peer)
    for (x, _), (y, _) in zip(a_nccl[rank], a_peer[rank]):
        assert float((x - y).abs().max()) <= 1e-6 * float(x.abs().max()), rep
        y.copy_(x)
    comms['pure_nccl'].all_gather_v_arrays(a_nccl)
    comms['peer_memory'].all_gather_v_arrays(a_peer)
    for o in range(world):
        for (x, _), (y, _) in zip(a_nccl[o], a_peer[o]):
            assert torch.equal(x, y), (rep, o)

# a bf16 wire: the exchanged arrays arrive rounded to bf16 (2^-9 relative)
half = ck.create_communicator('peer_memory', wire_dtype='bfloat16')
a_half = [[(t.clone(), tri) for t, tri in loc] for loc in a_nccl]
a_full = [[(t.clone(), tri) for t, tri in loc] for loc in a_nccl]
half.reduce_scatter_v_arrays(a_half)
comms['peer_memory'].reduce_scatter_v_arrays(a_full)
for (x, _), (y, _) in zip(a_full[rank], a_half[rank]):
    err = float((x - y).norm() / x.norm())
    assert 0 < err < 4e-3, err

for pic, early, own, cname, decay, acc in (
        (True, False, 'reference', 'pure_nccl', 1.0, 1),
        (False, False, 'reference', 'pure_nccl', 1.0, 1),
        (True, True, 'balanced', 'pure_nccl', 1.0, 1),
        (True, False, 'balanced', 'peer_memory', 1.0, 1),
        (False, True, 'reference', 'peer_memory', 1.0, 1),
        # running averages blended on the exchange stream of the pipelined
        # exchange, several steps
        (True, False, 'balanced', 'peer_memory', 0.9, 1),
        (True, False, 'reference', 'pure_nccl', 0.9, 1),
        # accumulation over micro-steps with a single exchange per update
        (True, False, 'balanced', 'peer_memory', 0.9, 2)):
    model = make()
    comm = comms[cname]
    opt = ck.DistributedKFAC(comm, lr=0.05, momentum=0.9, cov_ema_decay=decay,
                             damping=1e-2, only_pic_update_weight=pic,
                             communicate_after_forward=early, ownership=own,
                             acc_iters=acc)
    opt.setup(model)
    lossfun = lambda a, b: F.cross_entropy(model(a), b)
    opt.update(lossfun, xs, ts)          # first call: broadcast only
    assert opt.t == 0
    opt.update(lossfun, xs, ts)
    # further steps take the pipelined exchange (size class by size class)
    # when the configuration allows it
    steps = (4 if decay < 1.0 else 3) if not early else 1
    if acc > 1:
        # the call above was the first micro-step of the first update
        assert opt.t == 0 and opt.acc_count == 1
        for _ in range(acc * steps - 1):
            opt.update(lossfun, xs, ts)
        assert opt.t == steps
    else:
        assert opt.t == 1
        for _ in range(steps - 1):
            opt.update(lossfun, xs, ts)
    assert opt._real_updates == steps
    if not early and acc == 1:
        assert opt._pipeline_ready()
    # every rank holds the same weights afterwards
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    other = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(other, flat)
    assert all(torch.equal(other[0], o) for o in other), 'ranks diverged'
    if rank == 0:
        # reference: one process, whole batch.  Gradients of the mean loss
        # average exactly; factors of the halves average to the whole-batch
        # factor for A (scaled 1/n_local) and G (per-rank n_local * gy^T gy).
        ref = make()
        o1 = ck.KFAC(lr=0.05, momentum=0.9, cov_ema_decay=decay, damping=1e-2,
                     acc_iters=acc)
        o1.setup(ref)
        for _ in range(steps * acc):
            o1.update(lambda a, b: F.cross_entropy(ref(a), b), X, T)
        for (n1, p1), (n2, p2) in zip(ref.named_parameters(),
                                      model.named_parameters()):
            err = float((p1 - p2).norm() / p1.norm())
            assert err < 2e-3, (pic, early, own, cname, decay, acc, n1, err)
# BatchNormalization blocks in their low-rank form (every rank's per-sample
# gradient rows travel to the owner instead of a dense factor) against the
# dense form on the same ranks.  (A single-process run is no reference here:
# batch statistics are per rank.)
def make_bn():
    torch.manual_seed(9)
    return nn.Sequential(nn.Conv2d(3, 64, 3, 1, 1, bias=False),
                         nn.BatchNorm2d(64), nn.ReLU(),
                         nn.Conv2d(64, 64, 3, 2, 1, bias=False),
                         nn.BatchNorm2d(64), nn.ReLU(),
                         nn.AdaptiveAvgPool2d(1), nn.Flatten(),
                         nn.Linear(64, 5)).cuda()

for own, cname, decay in (('balanced', 'peer_memory', 0.9),
                          ('reference', 'pure_nccl', 1.0)):
    pair = []
    for low in (True, False):
        model = make_bn()
        opt = ck.DistributedKFAC(comms[cname], lr=0.02, momentum=0.9,
                                 cov_ema_decay=decay, damping=1e-2,
                                 ownership=own, bn_low_rank=low)
        opt.setup(model)
        pair.append((model, opt))
    gb = torch.Generator().manual_seed(50 + rank)
    for step in range(11):
        xb = torch.randn(4, 3, 8, 8, generator=gb).cuda()
        tb = torch.randint(0, 5, (4,), generator=gb).cuda()
        # the dense run restarts every step from the low-rank run's state:
        # differences do not compound over the steps
        pair[1][0].load_state_dict(pair[0][0].state_dict())
        for p0, p1 in zip(pair[0][1].target.params(),
                          pair[1][1].target.params()):
            p1.update_rule.velocity(p1).copy_(p0.update_rule.velocity(p0))
        for model, opt in pair:
            opt.update(lambda a, b, m=model: F.cross_entropy(m(a), b), xb, tb)
        flats = []
        for (model, opt), low in zip(pair, (True, False)):
            bn = [fb for fb in opt.fblocks if hasattr(fb.link, 'gamma')]
            assert len(bn) == 2
            if step > 0:            # (the first call only broadcasts)
                assert all(fb.low_rank_active == low for fb in bn)
            flat = torch.cat([p.detach().reshape(-1)
                              for p in model.parameters()])
            other = [torch.empty_like(flat) for _ in range(world)]
            dist.all_gather(other, flat)
            assert all(torch.equal(other[0], o) for o in other), \
                'ranks diverged'
            flats.append(flat)
        err = float((flats[0] - flats[1]).norm() / flats[1].norm())
        assert err < 1e-4, (own, cname, decay, step, err)
dist.barrier()
if rank == 0:
    print('DISTRIBUTED_OK')
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs 2 GPUs')
def test_distributed_kfac_two_gpus(tmp_path):
    script = tmp_path / 'worker.py'
    script.write_text(WORKER % {'root': ROOT})
    # small class bounds: the three layers fall into three size classes, so
    # the pipelined exchange runs one collective per class
    env = dict(os.environ, NCCL_NVLS_ENABLE='0', KFAC_CLASS_BOUNDS='20,40')
    res = subprocess.run(
        [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1',
         '--nproc-per-node=2', '--master-addr', '127.0.0.1', '--master-port',
         '29671', str(script)], env=env, stdout=subprocess.PIPE,
        stderr=subprocess.STDOUT, text=True, timeout=600)
    assert 'DISTRIBUTED_OK' in res.stdout, res.stdout[-3000:]
