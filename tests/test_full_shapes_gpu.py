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
