"""Vanilla ResNet-50 (bottleneck 3-4-6-3, stride on the 3x3 convolution,
fc 2048->1000) as a plain ``torch.nn`` model, and the training step the
benchmark times through the optimizer's public ``update`` call.  The model is
host-framework plumbing (cuDNN convolutions); the K-FAC work in the step runs
in this package's kernels."""

import torch
from torch import nn
import torch.nn.functional as F


class Bottleneck(nn.Module):
    def __init__(self, cin, mid, stride):
        super(Bottleneck, self).__init__()
        cout = mid * 4
        self.conv1 = nn.Conv2d(cin, mid, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(mid)
        self.conv2 = nn.Conv2d(mid, mid, 3, stride, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(mid)
        self.conv3 = nn.Conv2d(mid, cout, 1, bias=False)
        self.bn3 = nn.BatchNorm2d(cout)
        self.short = None
        if stride != 1 or cin != cout:
            self.short = nn.Conv2d(cin, cout, 1, stride, bias=False)
            self.bn_short = nn.BatchNorm2d(cout)

    def forward(self, x):
        h = F.relu(self.bn1(self.conv1(x)))
        h = F.relu(self.bn2(self.conv2(h)))
        h = self.bn3(self.conv3(h))
        s = x if self.short is None else self.bn_short(self.short(x))
        return F.relu(h + s)


class ResNet50(nn.Module):
    def __init__(self, classes=1000):
        super(ResNet50, self).__init__()
        self.conv1 = nn.Conv2d(3, 64, 7, 2, 3, bias=True)
        self.bn1 = nn.BatchNorm2d(64)
        blocks, cin = [], 64
        for stage, (n, mid) in enumerate([(3, 64), (4, 128), (6, 256),
                                          (3, 512)]):
            for b in range(n):
                stride = 2 if (b == 0 and stage > 0) else 1
                blocks.append(Bottleneck(cin, mid, stride))
                cin = mid * 4
        self.blocks = nn.Sequential(*blocks)
        self.fc = nn.Linear(cin, classes)

    def forward(self, x):
        h = F.max_pool2d(F.relu(self.bn1(self.conv1(x))), 3, 2, 1)
        h = self.blocks(h)
        h = F.adaptive_avg_pool2d(h, 1).flatten(1)
        return self.fc(h)


def build_training_step(device, batch, world, rank, cov_ema_decay, damping,
                        lr, momentum, image=224, classes=1000,
                        bn_blocks=True, communicator='peer_memory',
                        channels_last=True, acc_iters=1, bn_low_rank=True):
    """Returns (step, h2d_bytes, d2h_bytes).  ``step()`` copies one pinned
    host batch to the device, runs ``optimizer.update(lossfun, x, t)``
    (forward, backward, K-FAC factors / inverses / preconditioned update) and
    returns the step's loss, read back to the host as soon as the forward
    pass has produced it."""
    import chainerkfac_b200 as ck
    from chainerkfac_b200.optimizers.kfac import connection_only_constructor
    from chainerkfac_b200.optimizers.kfac import fblock_constructor

    torch.manual_seed(1234)
    model = ResNet50(classes).to(device)
    model.train()
    ctor = fblock_constructor if bn_blocks else connection_only_constructor
    kwargs = dict(lr=lr, momentum=momentum, cov_ema_decay=cov_ema_decay,
                  damping=damping, constructor=ctor, acc_iters=acc_iters,
                  bn_low_rank=bn_low_rank)
    if world > 1:
        comm = ck.create_communicator(communicator)
        opt = ck.DistributedKFAC(comm, ownership='balanced', **kwargs)
    else:
        opt = ck.KFAC(**kwargs)
    opt.setup(model)

    g = torch.Generator().manual_seed(99 + rank)
    hx = torch.randn((batch, 3, image, image), generator=g)
    if channels_last:
        # channels-last activations (weights keep their layout): cuDNN's NHWC
        # kernels run the model, and the factor builds read the (n*h*w, c)
        # activations and gradients in place
        hx = hx.contiguous(memory_format=torch.channels_last)
    hx = hx.pin_memory()
    ht = torch.randint(0, classes, (batch,), generator=g).pin_memory()
    hloss = torch.empty((), dtype=torch.float32).pin_memory()

    have_loss = torch.cuda.Event()

    def lossfun(x, t):
        loss = F.cross_entropy(model(x), t)
        # the loss goes to the host right behind the forward pass; the
        # backward pass and the K-FAC stages are queued after this copy
        hloss.copy_(loss.detach(), non_blocking=True)
        have_loss.record()
        return loss

    def step():
        x = hx.to(device, non_blocking=True)
        if channels_last:
            x = x.contiguous(memory_format=torch.channels_last)
        t = ht.to(device, non_blocking=True)
        opt.update(lossfun, x, t)
        # wait for this step's loss only: the host then prepares the next
        # batch while the device finishes this update (the caller's timed
        # region ends with a full synchronisation)
        have_loss.synchronize()
        return float(hloss)

    h2d = hx.numel() * hx.element_size() + ht.numel() * ht.element_size()
    return step, h2d, hloss.element_size()
