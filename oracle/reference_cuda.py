"""ctypes binding of the reference's own kernels built by ``oracle/build_ref.py``
(TEST INFRASTRUCTURE ONLY; needs a GPU).  Arrays are numpy fp32.

Limits inherited from the reference: forward Rank in {1,2,4,8,16} and
(T+C+Y+X)*Rank <= 16384 (Cuda_kernels/cp4Conv2dForward.cu:24,254-310); backward-data
(T+C+Y+X)*Rank <= 4096 and filter size in {1,3,..,17} (cp4Conv2dBackwardData.cu:22,174-266),
and only tile-aligned images (W % 16 == 0, H % 4 == 0) are free of its barrier hazard
(cp4Conv2dBackwardData.cu:71-72).
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_libs = {}


def available():
    return all(os.path.exists(os.path.join(_HERE, "_ref", f"libcp4ref_{n}.so")) for n in ("fwd", "bwd"))


def _lib(n):
    if n not in _libs:
        name = f"libtvmref_{n[4:]}.so" if n.startswith("tvm_") else f"libcp4ref_{n}.so"
        _libs[n] = C.CDLL(os.path.join(_HERE, "_ref", name))
    return _libs[n]


def tvm_available():
    return all(os.path.exists(os.path.join(_HERE, "_ref", f"libtvmref_{n}.so")) for n in ("rcp", "dense", "cp3", "cp4"))


# the one shape each TensorFlow-op kernel of the reference is compiled for (Kernels/*.cc):
# inputs in launcher order, then the output
TVM_SHAPES = {
    "rcp": ([(1, 4, 4, 32, 32), (4, 4, 11), (4, 4, 11), (3, 3, 11)], (1, 4, 4, 32, 32)),
    "dense": ([(1, 16, 16, 16), (16, 4, 137), (16, 4, 137), (16, 4, 137)], (1, 4, 4, 4)),
    "cp3": ([(1, 16, 32, 32), (16, 6), (3, 3, 6), (6, 16)], (1, 16, 32, 32)),
    "cp4": ([(1, 16, 32, 32), (16, 6), (3, 6), (3, 6), (16, 6)], (1, 16, 32, 32)),
}


def tvm_inputs(op, seed):
    """Seeded inputs of the op's compiled shape, uniform in [0, 1) like the reference's tests
    (test/test_conv2d_rcp.py:22-25, test_dense_cp.py:22-25, test_conv2d_cp.py:12-15, test_conv2d_cp4.py:13-17)."""
    rng = np.random.default_rng(seed)
    return [rng.uniform(0, 1, size=s).astype(np.float32) for s in TVM_SHAPES[op][0]]


def tvm_run(op, arrays):
    """Run ``Conv2dRcpFusedNchwKernelLauncher`` (Kernels/rcp_fused_nchw.cu:80), ``DenseCpKernelLauncher``
    (dense_cp.cu:48), ``Conv2dCpFusedNchwKernelLauncher`` (cp_fused_nchw.cu:454) or
    ``Cp4Conv2dFusedNchwKernelLauncher`` (cp4_conv_nchw.cu:88) on host arrays of the compiled shape."""
    shapes, oshape = TVM_SHAPES[op]
    arrs = [_f(a) for a in arrays]
    assert [a.shape for a in arrs] == [tuple(s) for s in shapes], "this kernel takes one literal shape"
    lib = _lib("tvm_" + op)
    out = np.zeros(oshape, np.float32)
    ptrs = (C.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])
    rc = lib.ref_tvm_run(ptrs, _p(out))
    assert rc == 0, rc
    return out


def forward_time(X, K0, K1, KH, KW, pad, profcount=47):
    """Mean microseconds of the reference's own forward kernel over ``profcount`` launches, as its launcher measures
    them (cp4_conv2d_forward_gpu's PROFCOUNT loop, Cuda_kernels/cp4Conv2dForward.cu:245-327)."""
    X, K0, K1, KH, KW = map(_f, (X, K0, K1, KH, KW))
    N, C_, H, W = X.shape
    T, R = K0.shape
    assert R in (1, 2, 4, 8, 16) and (T + C_ + KH.shape[0] + KW.shape[0]) * R <= 16384
    fn = _lib("fwd").ref_cp4_forward_time
    fn.restype = C.c_float
    return float(fn(_shape(N, C_, T, H, W, KH.shape[0], KW.shape[0], R, pad), _p(X), _p(K0), _p(K1), _p(KH), _p(KW),
                    C.c_uint(profcount)))


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _shape(N, C_, T, H, W, Y, X, R, pad):
    return (C.c_uint * 9)(N, H, W, pad, T, C_, Y, X, R)


def forward(X, K0, K1, KH, KW, pad):
    X, K0, K1, KH, KW = map(_f, (X, K0, K1, KH, KW))
    N, C_, H, W = X.shape
    T, R = K0.shape
    assert R in (1, 2, 4, 8, 16) and (T + C_ + KH.shape[0] + KW.shape[0]) * R <= 16384
    out = np.zeros((N, T, H, W), np.float32)
    rc = _lib("fwd").ref_cp4_forward(_shape(N, C_, T, H, W, KH.shape[0], KW.shape[0], R, pad), _p(X), _p(K0), _p(K1),
                                     _p(KH), _p(KW), _p(out))
    assert rc == 0, rc
    return out


def backward_data(dU, K0, K1, KH, KW, pad):
    dU, K0, K1, KH, KW = map(_f, (dU, K0, K1, KH, KW))
    N, T, H, W = dU.shape
    C_, R = K1.shape
    assert (T + C_ + KH.shape[0] + KW.shape[0]) * R <= 4096 and W % 16 == 0 and H % 4 == 0
    assert R in (1, 2, 4, 8, 16)
    out = np.zeros((N, C_, H, W), np.float32)
    rc = _lib("bwd").ref_cp4_backward_data(_shape(N, C_, T, H, W, KH.shape[0], KW.shape[0], R, pad), _p(dU), _p(K0),
                                           _p(K1), _p(KH), _p(KW), _p(out))
    assert rc == 0, rc
    return out


def backward_filter(X, dU, K0, K1, KH, KW, pad):
    X, dU, K0, K1, KH, KW = map(_f, (X, dU, K0, K1, KH, KW))
    N, C_, H, W = X.shape
    T, R = K0.shape
    Y, Xf = KH.shape[0], KW.shape[0]
    assert 2 * pad >= Y - 1 and 2 * pad >= Xf - 1
    g = [np.zeros((d, R), np.float32) for d in (T, C_, Y, Xf)]
    rc = _lib("bwd").ref_cp4_backward_filter(_shape(N, C_, T, H, W, Y, Xf, R, pad), _p(X), _p(dU), _p(K0), _p(K1),
                                             _p(KH), _p(KW), *[_p(a) for a in g])
    assert rc == 0, rc
    return tuple(g)
