"""ctypes binding of ``libkfac_b200.so`` (the C ABI of include/kfac_b200.h).

The library is the only compute path of this package: if it cannot be loaded
the import of anything that computes fails with an explicit error; there is no
NumPy or PyTorch fallback.
"""

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, 'libkfac_b200.so')

c_float_p = ctypes.POINTER(ctypes.c_float)
c_int_p = ctypes.POINTER(ctypes.c_int)
c_i64_p = ctypes.POINTER(ctypes.c_int64)
c_void_pp = ctypes.POINTER(ctypes.c_void_p)
VP = ctypes.c_void_p
I = ctypes.c_int
I64 = ctypes.c_int64
F = ctypes.c_float
SZ = ctypes.c_size_t

class FactorItem(ctypes.Structure):
    """struct kfac_factor_item of include/kfac_b200.h."""
    _fields_ = [('kind', ctypes.c_int), ('add_ones_col', ctypes.c_int),
                ('x', ctypes.c_void_p), ('rows', ctypes.c_int64),
                ('ld', ctypes.c_int64), ('d_in', ctypes.c_int),
                ('n', ctypes.c_int), ('c', ctypes.c_int), ('h', ctypes.c_int),
                ('w', ctypes.c_int), ('ksize', ctypes.c_int),
                ('stride', ctypes.c_int), ('pad', ctypes.c_int),
                ('alpha', ctypes.c_float), ('beta', ctypes.c_float),
                ('out', ctypes.c_void_p), ('layout', ctypes.c_int)]


class BnItem(ctypes.Structure):
    """struct kfac_bn_item of include/kfac_b200.h."""
    _fields_ = [('x', ctypes.c_void_p), ('gy', ctypes.c_void_p),
                ('out', ctypes.c_void_p), ('stats', ctypes.c_void_p),
                ('n', ctypes.c_int), ('c', ctypes.c_int), ('hw', ctypes.c_int),
                ('layout', ctypes.c_int), ('eps', ctypes.c_float),
                ('scale', ctypes.c_float)]


class BnLowRankItem(ctypes.Structure):
    """struct kfac_bn_lowrank_item of include/kfac_b200.h."""
    _fields_ = [(nm, ctypes.c_void_p) for nm in (
        'hist', 'scaled', 'm_inv', 'grad_gamma', 'grad_beta', 'kf_gamma',
        'kf_beta', 'param_gamma', 'param_beta', 'mom_gamma', 'mom_beta',
        'nan_flag')] + [
        ('c', ctypes.c_int), ('rows_per_slot', ctypes.c_int),
        ('slots', ctypes.c_int), ('damp_gamma', ctypes.c_float),
        ('damp_beta', ctypes.c_float), ('slot_weight', ctypes.c_float * 32)]


# name -> (restype, argtypes); mirrors include/kfac_b200.h one to one.
SIGNATURES = {
    'kfac_abi_version': (I, []),
    'kfac_last_error': (ctypes.c_char_p, []),
    'kfac_launch_count': (I64, []),
    'kfac_set_engine': (I, [I]),
    'kfac_get_engine': (I, []),
    'kfac_set_factor_staging': (I, [I]),
    'kfac_get_factor_staging': (I, []),
    'kfac_tc_status': (I, [c_int_p]),
    'kfac_selftest_wait_expiry': (I, [c_int_p, c_int_p]),
    'kfac_factor_workspace_bytes': (SZ, [I64, I]),
    'kfac_factor_dense': (I, [VP, I64, I, I64, I, F, F, VP, VP, SZ, VP]),
    'kfac_factor_noalloc_max_bytes': (SZ, []),
    'kfac_factor_dense_noalloc': (I, [VP, I64, I, I64, I, F, F, VP, VP]),
    'kfac_factor_conv_workspace_bytes': (SZ, [I, I, I, I, I, I, I, I]),
    'kfac_factor_conv_input': (I, [VP, I, I, I, I, I, I, I, I, F, F, VP, VP,
                                   SZ, VP]),
    'kfac_factor_conv_grad': (I, [VP, I, I, I, I, F, F, VP, VP, SZ, VP]),
    'kfac_factor_group_workspace_bytes': (SZ, [I, ctypes.POINTER(FactorItem)]),
    'kfac_factor_group': (I, [I, ctypes.POINTER(FactorItem), VP, SZ, VP]),
    'kfac_bn_sample_grads': (I, [VP, VP, I, I, I, F, F, VP, VP, VP]),
    'kfac_bn_sample_grads_group': (I, [I, ctypes.POINTER(BnItem), VP]),
    'kfac_bn_precondition_group': (I, [I, c_int_p] + [c_void_pp] * 10 +
                                   [F, F, VP]),
    'kfac_bn_lowrank_scale': (I, [I, ctypes.POINTER(BnLowRankItem), VP]),
    'kfac_bn_lowrank_apply': (I, [I, ctypes.POINTER(BnLowRankItem), F, F,
                                  VP]),
    'kfac_axpby': (I, [I64, F, VP, F, VP, VP, VP]),
    'kfac_axpby_group': (I, [I, c_i64_p, F, c_void_pp, F, c_void_pp,
                             c_void_pp, VP]),
    'kfac_inverse_workspace_bytes': (SZ, [I, c_int_p]),
    'kfac_inverse_plan_create': (I, [I, c_int_p, c_void_pp, c_void_pp,
                                     c_int_p, c_int_p, c_float_p, c_float_p,
                                     VP, SZ, c_void_pp]),
    'kfac_inverse_plan_run': (I, [VP, F, I, VP, VP, VP]),
    'kfac_inverse_plan_set_refine': (I, [VP, I, F]),
    'kfac_inverse_plan_refined': (I, [VP, c_int_p]),
    'kfac_inverse_plan_error_estimates': (I, [VP, c_float_p]),
    'kfac_inverse_plan_set_second_floor': (I, [VP, c_float_p]),
    'kfac_inverse_plan_destroy': (I, [VP]),
    'kfac_precond_workspace_bytes': (SZ, [I, c_int_p, c_int_p, c_int_p]),
    'kfac_precondition': (I, [I, c_int_p, c_int_p] + [c_void_pp] * 10 +
                          [F, F, VP, SZ, VP]),
    'kfac_symv_split': (I, [VP, I, I, VP, VP, VP, VP, VP, VP]),
    'kfac_momentum_update': (I, [I64, VP, VP, VP, F, F, VP]),
    'kfac_normalize_weight': (I, [I64, VP, F, F, VP, VP]),
    'kfac_wire_nelems': (I64, [I, c_i64_p, c_int_p]),
    'kfac_wire_pack': (I, [I, c_void_pp, c_i64_p, c_int_p, c_int_p, I, VP,
                           VP]),
    'kfac_wire_unpack': (I, [I, c_void_pp, c_i64_p, c_int_p, c_int_p, F, F,
                             VP, VP]),
    'kfac_wire_unpack_sum': (I, [I, c_void_pp, c_i64_p, c_int_p, c_int_p, F,
                                 F, c_void_pp, I, VP]),
    'kfac_wire_pack_as': (I, [I, I, c_void_pp, c_i64_p, c_int_p, c_int_p, I,
                              VP, VP]),
    'kfac_wire_unpack_sum_as': (I, [I, I, c_void_pp, c_i64_p, c_int_p,
                                    c_int_p, F, F, c_void_pp, I, VP]),
}

_lib = None


class KfacLibraryError(RuntimeError):
    pass


def load():
    """Load the shared library (once) and declare every prototype."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise KfacLibraryError(
            '%s is missing: build it with `python -m chainerkfac_b200._build` '
            '(nvcc, sm_100a). This package has no CPU fallback.' % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError if the symbol is missing
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc, what):
    if rc != 0:
        msg = load().kfac_last_error().decode('utf-8', 'replace')
        raise KfacLibraryError('%s failed (code %d): %s' % (what, rc, msg))


def int_array(values):
    return (ctypes.c_int * len(values))(*[int(v) for v in values])


def i64_array(values):
    return (ctypes.c_int64 * len(values))(*[int(v) for v in values])


def float_array(values):
    return (ctypes.c_float * len(values))(*[float(v) for v in values])


def ptr_array(values):
    return (ctypes.c_void_p * len(values))(*[
        (None if v is None else int(v)) for v in values])
