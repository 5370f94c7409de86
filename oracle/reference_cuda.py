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
        _libs[n] = C.CDLL(os.path.join(_HERE, "_ref", f"libcp4ref_{n}.so"))
    return _libs[n]


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
