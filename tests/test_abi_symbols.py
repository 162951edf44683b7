"""The shared library loads on a machine without a GPU and exports every
function that include/kfac_b200.h declares (no compute calls here)."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope='module')
def lib():
    from chainerkfac_b200 import _build, _lib
    _build.build()
    return _lib.load()


def declared_functions():
    text = open(os.path.join(ROOT, 'include', 'kfac_b200.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(kfac_[a-z0-9_]+)\s*\(', text)))


def test_header_declares_what_the_binding_binds(lib):
    from chainerkfac_b200 import _lib
    assert declared_functions() == sorted(_lib.SIGNATURES)


def test_every_declared_symbol_is_exported(lib):
    names = declared_functions()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), name


def test_pure_host_entry_points(lib):
    from chainerkfac_b200 import _lib
    assert lib.kfac_abi_version() == 2
    # sizes are host arithmetic: no device needed
    dims = _lib.int_array([10, 300])
    need = lib.kfac_inverse_workspace_bytes(2, dims)
    assert need >= 3 * 4 * (10 * 10 + 300 * 300)
    n = lib.kfac_wire_nelems(2, _lib.i64_array([16, 5]),
                             _lib.int_array([4, 0]))
    assert n == 10 + 5
    assert lib.kfac_get_factor_staging() == 0
    assert lib.kfac_factor_workspace_bytes(32, 2049) == 0
    # with the staging pass on: the two bf16 planes of the transposed operand
    # (rows of 32 k, 256-byte aligned); a short contraction needs no more
    lib.kfac_set_factor_staging(1)
    try:
        plane = (2049 * 32 * 2 + 255) // 256 * 256
        assert lib.kfac_factor_workspace_bytes(32, 2049) == 2 * plane
    finally:
        lib.kfac_set_factor_staging(0)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from chainerkfac_b200 import _lib
    monkeypatch.setattr(_lib, '_lib', None)
    monkeypatch.setattr(_lib, 'LIB_PATH', str(tmp_path / 'absent.so'))
    with pytest.raises(_lib.KfacLibraryError):
        _lib.load()


def test_cpu_tensors_are_rejected(lib):
    import torch
    from chainerkfac_b200 import _lib, ops
    with pytest.raises(_lib.KfacLibraryError):
        ops.factor_dense(torch.zeros(4, 3))
