"""kfac_factor_dense_noalloc against kfac_factor_dense, through the C ABI.

The no-allocation entry point serves callers that may not allocate device
memory themselves and have no workspace to lend (for instance code running
under a framework whose pool already owns the whole device).  Its partial
tiles live in a fixed array inside the library, shared by every call, so the
test makes two calls in a row with different shapes and checks each against
the regular entry point.  The file name keeps it last in collection order.
"""

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

FACTOR_TOL = 1e-4   # relative Frobenius error, as for the other factor tests


def rel(a, b):
    a = a.double()
    b = b.double()
    return float((a - b).norm() / b.norm())


def vp(t):
    return ctypes.c_void_p(t.data_ptr())


def both(lib, check, x, ones, alpha, beta, prev):
    rows, d_in = x.shape
    d = d_in + ones
    ref = prev.clone()
    out = prev.clone()
    nbytes = lib.kfac_factor_workspace_bytes(rows, d)
    ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device='cuda')
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    check(lib.kfac_factor_dense(vp(x), rows, d_in, x.stride(0), ones, alpha,
                                beta, vp(ref), vp(ws), ws.numel(), stream),
          'kfac_factor_dense')
    check(lib.kfac_factor_dense_noalloc(vp(x), rows, d_in, x.stride(0), ones,
                                        alpha, beta, vp(out), stream),
          'kfac_factor_dense_noalloc')
    torch.cuda.synchronize()
    return nbytes, ref, out


def test_noalloc_matches_regular_entry_point_twice():
    from chainerkfac_b200 import _lib
    lib = _lib.load()
    assert lib.kfac_factor_noalloc_max_bytes() == 32 << 20
    g = torch.Generator(device='cuda')
    g.manual_seed(3)
    # call 1: long contraction, split across CTAs -> uses the built-in scratch
    x1 = torch.rand((60000, 200), device='cuda', generator=g)
    prev1 = torch.zeros((201, 201), device='cuda')
    need1, ref1, out1 = both(lib, _lib.check, x1, 1, 1.0 / 60000, 0.0, prev1)
    assert need1 > 0
    assert rel(out1, ref1) < FACTOR_TOL
    # call 2: other shape, blended into an existing factor; the scratch still
    # holds call 1's partial tiles
    x2 = torch.randn((9000, 64), device='cuda', generator=g)
    prev2 = torch.eye(64, device='cuda')
    need2, ref2, out2 = both(lib, _lib.check, x2, 0, 0.9 / 9000, 0.1, prev2)
    assert need2 > 0
    assert rel(out2, ref2) < FACTOR_TOL
    truth = 0.9 / 9000 * (x2.double().T @ x2.double()) + \
        0.1 * torch.eye(64, device='cuda', dtype=torch.float64)
    assert rel(out2, truth) < FACTOR_TOL
    # and the first shape again gives the first answer again
    _, _, out1b = both(lib, _lib.check, x1, 1, 1.0 / 60000, 0.0, prev1)
    assert torch.equal(out1b, out1)


def test_noalloc_rejects_shapes_beyond_the_built_in_scratch():
    from chainerkfac_b200 import _lib
    lib = _lib.load()
    rows, d = 400000, 576
    assert lib.kfac_factor_workspace_bytes(rows, d) > \
        lib.kfac_factor_noalloc_max_bytes()
    x = torch.zeros((8, d), device='cuda')       # never read: call must refuse
    out = torch.zeros((d, d), device='cuda')
    rc = lib.kfac_factor_dense_noalloc(vp(x), rows, d, d, 0, 1.0, 0.0, vp(out),
                                       None)
    assert rc == 3
    msg = lib.kfac_last_error().decode()
    assert 'scratch' in msg and str(32 << 20) in msg


_FIRST_CALL_SCRIPT = r'''
import ctypes, sys
import torch
from chainerkfac_b200 import _lib

lib = _lib.load()
vp = lambda t: ctypes.c_void_p(t.data_ptr())
g = torch.Generator(device='cuda'); g.manual_seed(5)
x = torch.rand((60000, 200), device='cuda', generator=g)
out = torch.zeros((201, 201), device='cuda')
ref = torch.zeros((201, 201), device='cuda')
need = lib.kfac_factor_workspace_bytes(60000, 201)
ws = torch.empty(max(need, 256), dtype=torch.uint8, device='cuda')
status = ctypes.c_int(-1)
# loads the library's device code (and with it the built-in scratch array)
# without touching any of its allocating paths
_lib.check(lib.kfac_tc_status(ctypes.byref(status)), 'kfac_tc_status')
torch.cuda.synchronize()
free0, _ = torch.cuda.mem_get_info()
_lib.check(lib.kfac_factor_dense_noalloc(vp(x), 60000, 200, 200, 1,
                                         1.0 / 60000, 0.0, vp(out), None),
           'kfac_factor_dense_noalloc')
torch.cuda.synchronize()
free1, _ = torch.cuda.mem_get_info()
_lib.check(lib.kfac_factor_dense(vp(x), 60000, 200, 200, 1, 1.0 / 60000, 0.0,
                                 vp(ref), vp(ws), ws.numel(), None),
           'kfac_factor_dense')
torch.cuda.synchronize()
err = float((out.double() - ref.double()).norm() / ref.double().norm())
print('RESULT', need, free0 - free1, err)
'''


def test_noalloc_as_first_call_of_a_process_leaves_free_memory_unchanged():
    """The entry point must not allocate even when nothing has warmed the
    library up: in a fresh process, with the library's device code loaded
    eagerly so that code loading cannot be mistaken for an allocation, the
    device's free memory is the same before and after the first call."""
    import os
    import subprocess
    import sys
    env = dict(os.environ)
    env['CUDA_MODULE_LOADING'] = 'EAGER'
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env['PYTHONPATH'] = root + os.pathsep + env.get('PYTHONPATH', '')
    r = subprocess.run([sys.executable, '-c', _FIRST_CALL_SCRIPT], env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    line = [l for l in r.stdout.splitlines() if l.startswith('RESULT')][-1]
    need, drop, err = line.split()[1:]
    assert int(need) > 0                 # the shape does use the scratch
    assert int(drop) < (1 << 20), 'free memory fell by %s bytes' % drop
    assert float(err) < FACTOR_TOL
