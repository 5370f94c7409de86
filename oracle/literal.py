"""ctypes binding of ``oracle/cp_literal.c`` (TEST INFRASTRUCTURE ONLY).

``build()`` compiles the C file with gcc into ``oracle/_build/``; the functions
take and return numpy fp32 arrays.  Used on small shapes to pin the float64
restatement in ``cp_oracle.py`` to the reference's literal loop nests.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libcp_literal.so")
_lib = None


class Shape(ctypes.Structure):
    _fields_ = [(k, ctypes.c_uint) for k in ("N", "H", "W", "pad", "T", "C", "Y", "X", "Rank")]


def build(force=False):
    src = os.path.join(_HERE, "cp_literal.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        os.makedirs(os.path.dirname(_SO), exist_ok=True)
        subprocess.check_call(["gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-o", _SO, src])
    return _SO


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _shape(N, C, T, H, W, Y, X, R, pad):
    return Shape(N=N, H=H, W=W, pad=pad, T=T, C=C, Y=Y, X=X, Rank=R)


def forward(X, K0, K1, KH, KW, pad):
    X, K0, K1, KH, KW = map(_c, (X, K0, K1, KH, KW))
    N, C, H, W = X.shape
    T, R = K0.shape
    s = _shape(N, C, T, H, W, KH.shape[0], KW.shape[0], R, pad)
    out = np.zeros((N, T, H, W), np.float32)
    lib().cp4lit_forward(ctypes.byref(s), _p(X), _p(K0), _p(K1), _p(KH), _p(KW), _p(out))
    return out


def backward_data(dU, K0, K1, KH, KW, pad):
    dU, K0, K1, KH, KW = map(_c, (dU, K0, K1, KH, KW))
    N, T, H, W = dU.shape
    C, R = K1.shape
    s = _shape(N, C, T, H, W, KH.shape[0], KW.shape[0], R, pad)
    out = np.zeros((N, C, H, W), np.float32)
    lib().cp4lit_backward_data(ctypes.byref(s), _p(dU), _p(K0), _p(K1), _p(KH), _p(KW), _p(out))
    return out


def backward_filter(X, dU, K0, K1, KH, KW, pad):
    """Four literal nests; requires 2*pad >= F-1 like the reference."""
    X, dU, K0, K1, KH, KW = map(_c, (X, dU, K0, K1, KH, KW))
    N, C, H, W = X.shape
    T, R = K0.shape
    Y, Xf = KH.shape[0], KW.shape[0]
    assert 2 * pad >= Y - 1 and 2 * pad >= Xf - 1
    s = _shape(N, C, T, H, W, Y, Xf, R, pad)
    dK0 = np.zeros((T, R), np.float32)
    dK1 = np.zeros((C, R), np.float32)
    dKH = np.zeros((Y, R), np.float32)
    dKW = np.zeros((Xf, R), np.float32)
    L = lib()
    L.cp4lit_backward_filter_t(ctypes.byref(s), _p(dK0), _p(X), _p(dU), _p(K1), _p(KH), _p(KW))
    L.cp4lit_backward_filter_c(ctypes.byref(s), _p(dK1), _p(X), _p(dU), _p(K0), _p(KH), _p(KW))
    L.cp4lit_backward_filter_y(ctypes.byref(s), _p(dKH), _p(X), _p(dU), _p(K0), _p(K1), _p(KW))
    L.cp4lit_backward_filter_x(ctypes.byref(s), _p(dKW), _p(X), _p(dU), _p(K0), _p(K1), _p(KH))
    return dK0, dK1, dKH, dKW


def backward_filter_full(X, dU, Y, Xf, pad):
    X, dU = map(_c, (X, dU))
    N, C, H, W = X.shape
    T = dU.shape[1]
    s = _shape(N, C, T, H, W, Y, Xf, 1, pad)
    FF = np.zeros((T, C, Y, Xf), np.float32)
    lib().cp4lit_backward_filter_full(ctypes.byref(s), _p(FF), _p(X), _p(dU))
    return FF
