"""Operator-level mirror of the reference's entry points.

C++ order (``Cuda_kernels/cp4Conv2d.cuh:8-28``): ``cp4_conv2d_forward(Input, FT, FC, FY, FX, pad)``
and the backward pair.  TF custom-op order (``Kernels/cp4_conv_nchw.cc:6-13``,
``test/test_conv2d_cp4.py:13-25``): ``cp4_conv2d_nchw(U, K0[C,R], K1[FH,R], K2[FW,R], K3[T,R])``;
``conv2d_rcp_fused_nchw(U, K0, K1, ..., KC)`` (``Kernels/rcp_fused_nchw.cc:6-12``) and
``dense_cp(U, K0, K1, ...)`` (``Kernels/dense_cp.cc:6-12``), generalised from the single shape
each reference op was compiled for.  Arguments are fp32 CUDA tensors; errors raise, like
the reference ops' ``OP_REQUIRES``.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import TensorShape, check, int_array, lib, ptr_array


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dev(t, name):
    if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dtype != torch.float32:
        raise TypeError(f"{name} must be a float32 CUDA tensor")
    return t.contiguous()


def _p(t):
    return C.c_void_p(t.data_ptr())


def tensor_shape(N, C_, H, W, T, Y, X, Rank, pad):
    return TensorShape(N=N, H=H, W=W, pad=pad, T=T, C=C_, Y=Y, X=X, Rank=Rank)


def _shape_from(inp, FT, FC, FY, FX, pad, in_is_upstream=False):
    if inp.dim() != 4:
        raise ValueError("input must be a rank-4 NCHW tensor")
    for f, nm in ((FT, "FT"), (FC, "FC"), (FY, "FY"), (FX, "FX")):
        if f.dim() != 2 or f.shape[1] != FT.shape[1]:
            raise ValueError(f"{nm} must be [dim, rank] with the same rank as FT")
    ch = FT.shape[0] if in_is_upstream else FC.shape[0]
    if inp.shape[1] != ch:
        raise ValueError(f"input has {inp.shape[1]} channels, the factor has {ch}")
    return tensor_shape(inp.shape[0], FC.shape[0], inp.shape[2], inp.shape[3], FT.shape[0], FY.shape[0],
                        FX.shape[0], FT.shape[1], pad)


# ---- CP4, C++ order ---------------------------------------------------------
def cp4_conv2d_forward(Input, FT, FC, FY, FX, pad=1, flags=0):
    """``CP::Conv2dForward`` (Cuda_kernels/cp4Conv2d.cu:14-43): returns Out [N,T,H,W]."""
    Input, FT, FC, FY, FX = (_dev(t, n) for t, n in ((Input, "Input"), (FT, "FT"), (FC, "FC"), (FY, "FY"), (FX, "FX")))
    s = _shape_from(Input, FT, FC, FY, FX, pad)
    out = torch.empty((s.N, s.T, s.H, s.W), device=Input.device, dtype=torch.float32)
    with torch.cuda.device(Input.device):
        check(lib.b200cp_cp4_fwd(C.byref(s), _p(Input), _p(FT), _p(FC), _p(FY), _p(FX), _p(out), _stream(), flags))
    return out


def cp4_conv2d_backward_data(Upstream, FT, FC, FY, FX, pad=1, flags=0):
    """``CP::Conv2dBackwardData`` (Cuda_kernels/cp4Conv2d.cu:48-77): returns dX [N,C,H,W]."""
    Upstream, FT, FC, FY, FX = (_dev(t, n) for t, n in
                                ((Upstream, "Upstream"), (FT, "FT"), (FC, "FC"), (FY, "FY"), (FX, "FX")))
    s = _shape_from(Upstream, FT, FC, FY, FX, pad, in_is_upstream=True)
    out = torch.empty((s.N, s.C, s.H, s.W), device=Upstream.device, dtype=torch.float32)
    with torch.cuda.device(Upstream.device):
        check(lib.b200cp_cp4_bwd_data(C.byref(s), _p(Upstream), _p(FT), _p(FC), _p(FY), _p(FX), _p(out), _stream(),
                                      flags))
    return out


def cp4_conv2d_forward_backward_data(Input, Upstream, FT, FC, FY, FX, pad=1, flags=0, save=False):
    """Forward of ``Input`` and backward-data of ``Upstream`` in one call (one launch where the shape allows it): the
    two convolutions of a training step with frozen factors.  Returns ``(Out, dInput)``, with ``save`` also the rank
    planes ``(P, Q)`` for ``cp4_conv2d_backward_filter_saved``."""
    Input, Upstream = _dev(Input, "Input"), _dev(Upstream, "Upstream")
    FT, FC, FY, FX = (_dev(t, n) for t, n in ((FT, "FT"), (FC, "FC"), (FY, "FY"), (FX, "FX")))
    s = _shape_from(Input, FT, FC, FY, FX, pad)
    if tuple(Upstream.shape) != (s.N, s.T, s.H, s.W):
        raise ValueError("Upstream must be [N, T, H, W]")
    U = torch.empty((s.N, s.T, s.H, s.W), device=Input.device, dtype=torch.float32)
    dX = torch.empty_like(Input)
    Pl = torch.empty((s.N, s.Rank, s.H, s.W), device=Input.device, dtype=torch.float32) if save else None
    Ql = torch.empty_like(Pl) if save else None
    with torch.cuda.device(Input.device):
        check(lib.b200cp_cp4_fwd_bwd_data(C.byref(s), _p(Input), _p(Upstream), _p(FT), _p(FC), _p(FY), _p(FX), _p(U),
                                          _p(dX), _p(Pl) if save else None, _p(Ql) if save else None, _stream(), flags))
    return (U, dX, Pl, Ql) if save else (U, dX)


def cp4_conv2d_backward_filter(dLdO, In, FT, FC, FY, FX, pad=1, flags=0, packed=False):
    """The four factor gradients of ``CP::Conv2dBackwardFilter``
    (Cuda_kernels/cp4Conv2d.cu:83-153): returns (dFT, dFC, dFY, dFX), or the
    packed buffer [dFT|dFC|dFY|dFX] with ``packed=True`` (the allreduce unit)."""
    dLdO, In, FT, FC, FY, FX = (_dev(t, n) for t, n in
                                ((dLdO, "dLdO"), (In, "In"), (FT, "FT"), (FC, "FC"), (FY, "FY"), (FX, "FX")))
    s = _shape_from(In, FT, FC, FY, FX, pad)
    if tuple(dLdO.shape) != (s.N, s.T, s.H, s.W):
        raise ValueError("dLdO must be [N,T,H,W]")
    R = s.Rank
    nT, nC, nY, nX = s.T * R, s.C * R, s.Y * R, s.X * R
    dK = torch.empty(nT + nC + nY + nX, device=In.device, dtype=torch.float32)
    with torch.cuda.device(In.device):
        wsb = lib.b200cp_cp4_bwd_filter_workspace_bytes(C.byref(s), flags)
        ws = torch.empty(max(wsb, 4) // 4, device=In.device, dtype=torch.float32)
        check(lib.b200cp_cp4_bwd_filter(C.byref(s), _p(In), _p(dLdO), _p(FT), _p(FC), _p(FY), _p(FX), _p(dK), _p(ws),
                                        ws.numel() * 4, _stream(), flags))
    if packed:
        return dK
    return (dK[:nT].view(s.T, R), dK[nT:nT + nC].view(s.C, R), dK[nT + nC:nT + nC + nY].view(s.Y, R),
            dK[nT + nC + nY:].view(s.X, R))


def cp4_conv2d_backward_filter_full(dLdO, In, Y, X, pad=1):
    """``cp4_conv2d_backward_filter_full_gpu`` (Cuda_kernels/cp4Conv2dBackwardFilter.cu:23-59): dK [T,C,Y,X]."""
    dLdO, In = _dev(dLdO, "dLdO"), _dev(In, "In")
    s = tensor_shape(In.shape[0], In.shape[1], In.shape[2], In.shape[3], dLdO.shape[1], Y, X, 1, pad)
    dK = torch.empty((s.T, s.C, Y, X), device=In.device, dtype=torch.float32)
    with torch.cuda.device(In.device):
        check(lib.b200cp_cp4_bwd_filter_full(C.byref(s), _p(In), _p(dLdO), _p(dK), _stream()))
    return dK


def cp4recom(FT, FC, FY, FX):
    """``cp4recom`` (Cuda_kernels/Utils.cu:67-98): dense K [T,C,Y,X]."""
    FT, FC, FY, FX = (_dev(t, n) for t, n in ((FT, "FT"), (FC, "FC"), (FY, "FY"), (FX, "FX")))
    s = tensor_shape(1, FC.shape[0], 1, 1, FT.shape[0], FY.shape[0], FX.shape[0], FT.shape[1], 0)
    K = torch.empty((s.T, s.C, s.Y, s.X), device=FT.device, dtype=torch.float32)
    with torch.cuda.device(FT.device):
        check(lib.b200cp_cp4_recompose(C.byref(s), _p(FT), _p(FC), _p(FY), _p(FX), _p(K), _stream()))
    return K


def allclose(A, B, tolerance=1e-3):
    """``AllClose`` (Cuda_kernels/Utils.cu:159-180): True when no element's relative difference
    max(|a-b|/|a|, |a-b|/|b|) exceeds ``tolerance``; the count runs on the device."""
    A, B = _dev(A, "A"), _dev(B, "B")
    if A.numel() != B.numel():
        return False
    n = C.c_ulonglong(0)
    with torch.cuda.device(A.device):
        check(lib.b200cp_allclose_count(_p(A), _p(B), A.numel(), C.c_float(tolerance), C.byref(n), _stream()))
    return n.value == 0


def cp4_conv2d_step(X, dU, FT, FC, FY, FX, pad=1, flags=0):
    """One training step on device tensors (``b200cp_cp4_step``): returns (U, dX, dK_packed); the work forward,
    backward-data and backward-filter share is done once."""
    X, dU, FT, FC, FY, FX = (_dev(t, n) for t, n in
                             ((X, "X"), (dU, "dU"), (FT, "FT"), (FC, "FC"), (FY, "FY"), (FX, "FX")))
    s = _shape_from(X, FT, FC, FY, FX, pad)
    if tuple(dU.shape) != (s.N, s.T, s.H, s.W):
        raise ValueError("dU must be [N,T,H,W]")
    U = torch.empty((s.N, s.T, s.H, s.W), device=X.device, dtype=torch.float32)
    dX = torch.empty_like(X)
    dK = torch.empty((s.T + s.C + s.Y + s.X) * s.Rank, device=X.device, dtype=torch.float32)
    with torch.cuda.device(X.device):
        wsb = lib.b200cp_cp4_step_workspace_bytes(C.byref(s), flags)
        ws = torch.empty(max(wsb, 4) // 4, device=X.device, dtype=torch.float32)
        check(lib.b200cp_cp4_step(C.byref(s), _p(X), _p(dU), _p(FT), _p(FC), _p(FY), _p(FX), _p(U), _p(dX), _p(dK),
                                  _p(ws), ws.numel() * 4, _stream(), flags))
    return U, dX, dK


def _shares_planes(s, flags):
    """The library's own rule (``b200cp_cp4_shares_planes``): shape, path flags and its environment switches."""
    return bool(lib.b200cp_cp4_shares_planes(C.byref(s), flags))


def cp4_conv2d_forward_save(Input, FT, FC, FY, FX, pad=1, flags=0):
    """Forward that also returns its rank plane ``P = FC^T Input`` [N,R,H,W] (``b200cp_cp4_fwd_save``)."""
    Input, FT, FC, FY, FX = (_dev(t, n) for t, n in ((Input, "Input"), (FT, "FT"), (FC, "FC"), (FY, "FY"), (FX, "FX")))
    s = _shape_from(Input, FT, FC, FY, FX, pad)
    out = torch.empty((s.N, s.T, s.H, s.W), device=Input.device, dtype=torch.float32)
    P = torch.empty((s.N, s.Rank, s.H, s.W), device=Input.device, dtype=torch.float32)
    with torch.cuda.device(Input.device):
        check(lib.b200cp_cp4_fwd_save(C.byref(s), _p(Input), _p(FT), _p(FC), _p(FY), _p(FX), _p(out), _p(P), _stream(),
                                      flags))
    return out, P


def cp4_conv2d_backward_data_save(Upstream, FT, FC, FY, FX, pad=1, flags=0):
    """Backward-data that also returns its rank plane ``Q = FT^T Upstream`` (``b200cp_cp4_bwd_data_save``)."""
    Upstream, FT, FC, FY, FX = (_dev(t, n) for t, n in
                                ((Upstream, "Upstream"), (FT, "FT"), (FC, "FC"), (FY, "FY"), (FX, "FX")))
    s = _shape_from(Upstream, FT, FC, FY, FX, pad, in_is_upstream=True)
    out = torch.empty((s.N, s.C, s.H, s.W), device=Upstream.device, dtype=torch.float32)
    Q = torch.empty((s.N, s.Rank, s.H, s.W), device=Upstream.device, dtype=torch.float32)
    with torch.cuda.device(Upstream.device):
        check(lib.b200cp_cp4_bwd_data_save(C.byref(s), _p(Upstream), _p(FT), _p(FC), _p(FY), _p(FX), _p(out), _p(Q),
                                           _stream(), flags))
    return out, Q


def cp4_conv2d_backward_filter_saved(dLdO, In, P, Q, FT, FC, FY, FX, pad=1, flags=0):
    """The four factor gradients from the saved rank planes (``b200cp_cp4_bwd_filter_saved``)."""
    dLdO, In, P, Q, FY, FX = (_dev(t, n) for t, n in
                              ((dLdO, "dLdO"), (In, "In"), (P, "P"), (Q, "Q"), (FY, "FY"), (FX, "FX")))
    s = _shape_from(In, FT, FC, FY, FX, pad)
    R = s.Rank
    nT, nC, nY, nX = s.T * R, s.C * R, s.Y * R, s.X * R
    dK = torch.empty(nT + nC + nY + nX, device=In.device, dtype=torch.float32)
    with torch.cuda.device(In.device):
        wsb = lib.b200cp_cp4_bwd_filter_saved_workspace_bytes(C.byref(s), flags)
        ws = torch.empty(max(wsb, 4) // 4, device=In.device, dtype=torch.float32)
        check(lib.b200cp_cp4_bwd_filter_saved(C.byref(s), _p(In), _p(dLdO), _p(P), _p(Q), _p(FY), _p(FX), _p(dK), _p(ws),
                                              ws.numel() * 4, _stream(), flags))
    return (dK[:nT].view(s.T, R), dK[nT:nT + nC].view(s.C, R), dK[nT + nC:nT + nC + nY].view(s.Y, R),
            dK[nT + nC + nY:].view(s.X, R))


def cp4_conv2d_step_host(X, dU, FT, FC, FY, FX, pad=1, flags=0, out=None):
    """Forward + both backward passes through the host-buffer entry point
    (``b200cp_cp4_step_host``): CPU tensors in, CPU tensors out, transfers included.
    ``out`` may hold preallocated (pinned) ``(U, dX, dK_packed)``."""
    ts = [X, dU, FT, FC, FY, FX]
    for t in ts:
        if t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous():
            raise TypeError("host entry point takes contiguous float32 CPU tensors")
    s = tensor_shape(X.shape[0], FC.shape[0], X.shape[2], X.shape[3], FT.shape[0], FY.shape[0], FX.shape[0],
                     FT.shape[1], pad)
    R = s.Rank
    if out is None:
        out = (torch.empty((s.N, s.T, s.H, s.W)), torch.empty((s.N, s.C, s.H, s.W)),
               torch.empty((s.T + s.C + s.Y + s.X) * R))
    U, dX, dK = out
    check(lib.b200cp_cp4_step_host(C.byref(s), _p(X), _p(dU), _p(FT), _p(FC), _p(FY), _p(FX), _p(U), _p(dX), _p(dK),
                                   flags))
    return U, dX, dK


def cp4_conv2d_step_host_submit(X, dU, FT, FC, FY, FX, out, pad=1, flags=0, slot=0):
    """Queue one step on ``slot`` (0 .. 3) through ``b200cp_cp4_step_host_submit``; ``out`` holds the pinned
    ``(U, dX, dK_packed)`` that ``cp4_conv2d_step_host_wait(slot)`` fills.  Inputs and outputs must stay
    alive and untouched until that wait returns."""
    ts = [X, dU, FT, FC, FY, FX] + list(out)
    for t in ts:
        if t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous():
            raise TypeError("host entry point takes contiguous float32 CPU tensors")
    s = tensor_shape(X.shape[0], FC.shape[0], X.shape[2], X.shape[3], FT.shape[0], FY.shape[0], FX.shape[0],
                     FT.shape[1], pad)
    U, dX, dK = out
    if U.numel() != s.N * s.T * s.H * s.W or dX.numel() != X.numel() or dK.numel() != (s.T + s.C + s.Y + s.X) * s.Rank:
        raise ValueError("out must be (U [N,T,H,W], dX [N,C,H,W], dK_packed [(T+C+Y+X)*R])")
    check(lib.b200cp_cp4_step_host_submit(C.byref(s), _p(X), _p(dU), _p(FT), _p(FC), _p(FY), _p(FX), _p(U), _p(dX),
                                          _p(dK), flags, slot))


def cp4_conv2d_step_host_wait(slot=0):
    """Block until the step queued on ``slot`` has its results in the host tensors."""
    check(lib.b200cp_cp4_step_host_wait(slot))


def device_status():
    """Synchronise and raise if a tensor-path kernel gave up a bounded wait (``b200cp_device_status``)."""
    check(lib.b200cp_device_status())


def set_band_rows(rows):
    """Test hook: force the band height of the row-band CP4 kernel (0: the planner chooses)."""
    lib.b200cp_test_set_band_rows(int(rows))


def set_band_tensor_loads(on):
    """Test hook: the row-band kernel loads its input with 4-D tensor-map boxes (True) or 1-D bulk copies (False)."""
    lib.b200cp_test_set_band_tensor_loads(1 if on else 0)


def set_band_tcgen05(on):
    """Test hook: the row-band kernel's output contraction on tcgen05 (True) or mma.sync (False, default)."""
    lib.b200cp_test_set_band_tcgen05(1 if on else 0)


def set_stream(on):
    """Test hook: the row-stream convolution kernel off (0 / False), on (1 / True) or as the environment says (-1)."""
    lib.b200cp_test_set_stream(int(on))


def debug_cp4_tc(Input, FT, FC, FY, FX, pad=1, terms=3, p_floats=0):
    """Diagnostic forward on the tensor path; also returns the first CTA's rank-R intermediate."""
    Input, FT, FC, FY, FX = (_dev(t, n) for t, n in ((Input, "Input"), (FT, "FT"), (FC, "FC"), (FY, "FY"), (FX, "FX")))
    s = _shape_from(Input, FT, FC, FY, FX, pad)
    out = torch.empty((s.N, s.T, s.H, s.W), device=Input.device, dtype=torch.float32)
    P = torch.zeros(max(p_floats, 1), device=Input.device, dtype=torch.float32)
    with torch.cuda.device(Input.device):
        check(lib.b200cp_debug_cp4_tc(C.byref(s), _p(Input), _p(FT), _p(FC), _p(FY), _p(FX), _p(out),
                                      _p(P) if p_floats else None, terms, _stream()))
    return out, P


# ---- three-factor CP conv -----------------------------------------------------
def _shape3(inp, KT, KCin, KC, pad, in_is_upstream=False):
    if inp.dim() != 4 or KT.dim() != 2 or KCin.dim() != 2 or KC.dim() != 3:
        raise ValueError("expected input [N,ch,H,W], KT [T,R], KCin [C,R], KC [Y,X,R]")
    R = KT.shape[1]
    if KCin.shape[1] != R or KC.shape[2] != R:
        raise ValueError("all factors must have the same rank")
    if inp.shape[1] != (KT.shape[0] if in_is_upstream else KCin.shape[0]):
        raise ValueError("channel count of the input does not match the factor")
    return tensor_shape(inp.shape[0], KCin.shape[0], inp.shape[2], inp.shape[3], KT.shape[0], KC.shape[0], KC.shape[1],
                        R, pad)


def cp3_conv2d_forward(Input, KT, KCin, KC, pad=1, flags=0):
    """Three-factor CP conv (``b200cp_cp3_fwd``): ``KT [T,R]``, ``KCin [C,R]``, free core ``KC [Y,X,R]``."""
    Input, KT, KCin, KC = (_dev(t, n) for t, n in ((Input, "Input"), (KT, "KT"), (KCin, "KCin"), (KC, "KC")))
    s = _shape3(Input, KT, KCin, KC, pad)
    out = torch.empty((s.N, s.T, s.H, s.W), device=Input.device, dtype=torch.float32)
    with torch.cuda.device(Input.device):
        check(lib.b200cp_cp3_fwd(C.byref(s), _p(Input), _p(KT), _p(KCin), _p(KC), _p(out), _stream(), flags))
    return out


def cp3_conv2d_backward_data(Upstream, KT, KCin, KC, pad=1, flags=0):
    Upstream, KT, KCin, KC = (_dev(t, n) for t, n in ((Upstream, "Upstream"), (KT, "KT"), (KCin, "KCin"), (KC, "KC")))
    s = _shape3(Upstream, KT, KCin, KC, pad, in_is_upstream=True)
    out = torch.empty((s.N, s.C, s.H, s.W), device=Upstream.device, dtype=torch.float32)
    with torch.cuda.device(Upstream.device):
        check(lib.b200cp_cp3_bwd_data(C.byref(s), _p(Upstream), _p(KT), _p(KCin), _p(KC), _p(out), _stream(), flags))
    return out


def cp3_conv2d_backward_filter(dLdO, In, KT, KCin, KC, pad=1, flags=0):
    """Factor gradients (dKT, dKCin, dKC) of the three-factor CP conv; 3x3 cores with pad 1."""
    dLdO, In, KT, KCin, KC = (_dev(t, n) for t, n in
                              ((dLdO, "dLdO"), (In, "In"), (KT, "KT"), (KCin, "KCin"), (KC, "KC")))
    s = _shape3(In, KT, KCin, KC, pad)
    R = s.Rank
    nT, nC, nS = s.T * R, s.C * R, s.Y * s.X * R
    dK = torch.empty(nT + nC + nS, device=In.device, dtype=torch.float32)
    with torch.cuda.device(In.device):
        wsb = lib.b200cp_cp3_bwd_filter_workspace_bytes(C.byref(s), flags)
        ws = torch.empty(max(wsb, 4) // 4, device=In.device, dtype=torch.float32)
        check(lib.b200cp_cp3_bwd_filter(C.byref(s), _p(In), _p(dLdO), _p(KT), _p(KCin), _p(KC), _p(dK), _p(ws),
                                        ws.numel() * 4, _stream(), flags))
    return dK[:nT].view(s.T, R), dK[nT:nT + nC].view(s.C, R), dK[nT + nC:].view(s.Y, s.X, R)


def conv2d_cp_fused_nchw(U, K0, K1, K2, flags=0):
    """``Conv2dCpFusedNchw`` (Kernels/cp_fused_nchw.cc): K0 [C,R], K1 [FH,FW,R], K2 [R,T], SAME padding
    (test/test_conv2d_cp.py:33-38)."""
    return cp3_conv2d_forward(U, K2.t().contiguous(), K0, K1, pad=(K1.shape[0] - 1) // 2, flags=flags)


class CP3Conv2dFunction(torch.autograd.Function):
    """y = three-factor CP conv2d(x; KT, KCin, KC) with the fused backward kernels."""

    @staticmethod
    def forward(ctx, x, KT, KCin, KC, pad=1):
        ctx.save_for_backward(x, KT, KCin, KC)
        ctx.pad = pad
        return cp3_conv2d_forward(x, KT, KCin, KC, pad)

    @staticmethod
    def backward(ctx, dy):
        x, KT, KCin, KC = ctx.saved_tensors
        dy = dy.contiguous()
        dx = cp3_conv2d_backward_data(dy, KT, KCin, KC, ctx.pad) if ctx.needs_input_grad[0] else None
        g = (None,) * 3
        if any(ctx.needs_input_grad[1:4]):
            g = cp3_conv2d_backward_filter(dy, x, KT, KCin, KC, ctx.pad)
        return (dx, *g, None)


# ---- TF custom-op order -----------------------------------------------------
def cp4_conv2d_nchw(U, K0, K1, K2, K3, flags=0):
    """``Cp4Conv2dNchw`` (Kernels/cp4_conv_nchw.cc:6-13): K0 [C,R], K1 [FH,R], K2 [FW,R], K3 [T,R],
    SAME padding (test/test_conv2d_cp4.py:25-33)."""
    return cp4_conv2d_forward(U, K3, K0, K1, K2, pad=(K1.shape[0] - 1) // 2, flags=flags)


def _modes(factors, what):
    a, b = [], []
    R = factors[0].shape[2]
    for k, f in enumerate(factors):
        if f.dim() != 3 or f.shape[2] != R:
            raise ValueError(f"{what}: kernel {k} must be [in, out, rank] with a common rank")
        a.append(f.shape[0])
        b.append(f.shape[1])
    return a, b, R


def conv2d_rcp_fused_nchw(U, *kernels, flags=0):
    """``Conv2dRcpFusedNchw`` (Kernels/rcp_fused_nchw.cc:6-12): ``(U[N,S0..,H,W], K0[S0,T0,R], ..., KC[FH,FW,R])``
    -> ``V[N,T0..,H,W]``.  ``U`` may also be given as [N,C,H,W]."""
    *A, KC = kernels
    U = _dev(U, "input")
    A = [_dev(a, f"kernel{k}") for k, a in enumerate(A)]
    KC = _dev(KC, "kernelc")
    cd, td, R = _modes(A, "conv2d_rcp_fused_nchw")
    if KC.dim() != 3 or KC.shape[2] != R:
        raise ValueError("kernelc must be [FH, FW, rank]")
    Cc = 1
    for c in cd:
        Cc *= c
    folded = U.dim() == 4
    if not folded and tuple(U.shape[1:-2]) != tuple(cd):
        raise ValueError("input modes do not match the kernels")
    N, H, W = U.shape[0], U.shape[-2], U.shape[-1]
    if U.numel() != N * Cc * H * W:
        raise ValueError("input channel count does not match the kernels")
    Tc = 1
    for t in td:
        Tc *= t
    V = torch.empty((N, Tc, H, W), device=U.device, dtype=torch.float32)
    with torch.cuda.device(U.device):
        check(lib.b200cp_rcp_fwd(N, H, W, len(A), int_array(cd), int_array(td), R, KC.shape[0], KC.shape[1], _p(U),
                                 ptr_array([a.data_ptr() for a in A]), _p(KC), _p(V), _stream(), flags))
    return V if folded else V.view(N, *td, H, W)


def rcp_conv2d_backward(U, dV, *kernels, flags=0, need_dx=True, need_dw=True):
    """Gradients of ``conv2d_rcp_fused_nchw``: (dU, [dK_k], dKC)."""
    *A, KC = kernels
    U, dV = _dev(U, "input"), _dev(dV, "dV")
    A = [_dev(a, f"kernel{k}") for k, a in enumerate(A)]
    KC = _dev(KC, "kernelc")
    cd, td, R = _modes(A, "rcp_conv2d_backward")
    N, H, W = U.shape[0], U.shape[-2], U.shape[-1]
    dU = torch.empty_like(U) if need_dx else None
    dA = [torch.empty_like(a) for a in A] if need_dw else None
    dS = torch.empty_like(KC) if need_dw else None
    with torch.cuda.device(U.device):
        wsb = lib.b200cp_rcp_bwd_workspace_bytes(N, H, W, len(A), int_array(cd), int_array(td), R, KC.shape[0],
                                                 KC.shape[1], flags)
        ws = torch.empty(max(wsb, 4) // 4, device=U.device, dtype=torch.float32)
        check(lib.b200cp_rcp_bwd(N, H, W, len(A), int_array(cd), int_array(td), R, KC.shape[0], KC.shape[1], _p(U),
                                 _p(dV), ptr_array([a.data_ptr() for a in A]), _p(KC),
                                 _p(dU) if need_dx else None,
                                 ptr_array([a.data_ptr() for a in dA]) if need_dw else None,
                                 _p(dS) if need_dw else None, _p(ws), ws.numel() * 4, _stream(), flags))
    return dU, dA, dS


def dense_cp(U, *kernels, flags=0):
    """``DenseCp`` (Kernels/dense_cp.cc:6-12): ``(U[N,S0,S1,..], K0[S0,T0,R], ...)`` -> ``V[N,T0,T1,..]``
    (output dims are ``kernel_k.dim(1)``, Kernels/dense_cp.cc:86-91).  ``U`` may also be [N, I]."""
    U = _dev(U, "input")
    Fk = [_dev(f, f"kernel{k}") for k, f in enumerate(kernels)]
    idims, odims, R = _modes(Fk, "dense_cp")
    I = 1
    for d in idims:
        I *= d
    O = 1
    for d in odims:
        O *= d
    B = U.shape[0]
    if U.numel() != B * I:
        raise ValueError("input size does not match the kernels")
    flat = U.dim() == 2
    Y = torch.empty((B, O), device=U.device, dtype=torch.float32)
    with torch.cuda.device(U.device):
        check(lib.b200cp_dense_fwd(B, len(Fk), int_array(idims), int_array(odims), R, _p(U),
                                   ptr_array([f.data_ptr() for f in Fk]), _p(Y), _stream(), flags))
    return Y if flat else Y.view(B, *odims)


def dense_cp_backward(U, dV, *kernels, flags=0, need_dx=True, need_dw=True):
    """Gradients of ``dense_cp``: (dU, [dK_k])."""
    U, dV = _dev(U, "input"), _dev(dV, "dV")
    Fk = [_dev(f, f"kernel{k}") for k, f in enumerate(kernels)]
    idims, odims, R = _modes(Fk, "dense_cp_backward")
    B = U.shape[0]
    dU = torch.empty_like(U) if need_dx else None
    dF = [torch.empty_like(f) for f in Fk] if need_dw else None
    with torch.cuda.device(U.device):
        wsb = lib.b200cp_dense_bwd_workspace_bytes(B, len(Fk), int_array(idims), int_array(odims), R, flags)
        ws = torch.empty(max(wsb, 4) // 4, device=U.device, dtype=torch.float32)
        check(lib.b200cp_dense_bwd(B, len(Fk), int_array(idims), int_array(odims), R, _p(U), _p(dV),
                                   ptr_array([f.data_ptr() for f in Fk]), _p(dU) if need_dx else None,
                                   ptr_array([f.data_ptr() for f in dF]) if need_dw else None, _p(ws),
                                   ws.numel() * 4, _stream(), flags))
    return dU, dF


# ---- the reference's "rebuild" variants: the undecomposed layer with the recomposed weight --------------------

def conv2d_dense_forward(Input, K, pad=1):
    """Ordinary conv2d with a dense filter ``K [T,C,Y,X]``, H x W output: the ``tf.nn.conv2d(U, K, ..., 'SAME')`` of
    test/benchmark_conv2d_cp4.py:41."""
    Input, K = _dev(Input, "Input"), _dev(K, "K")
    if K.dim() != 4 or K.shape[1] != Input.shape[1]:
        raise ValueError("K must be [T, C, Y, X] with C the input's channel count")
    s = tensor_shape(Input.shape[0], Input.shape[1], Input.shape[2], Input.shape[3], K.shape[0], K.shape[2],
                     K.shape[3], 1, pad)
    U = torch.empty((s.N, s.T, s.H, s.W), device=Input.device, dtype=torch.float32)
    with torch.cuda.device(Input.device):
        wsb = lib.b200cp_conv2d_dense_fwd_workspace_bytes(C.byref(s))
        ws = torch.empty(max(wsb, 4) // 4, device=Input.device, dtype=torch.float32)
        check(lib.b200cp_conv2d_dense_fwd(C.byref(s), _p(Input), _p(K), _p(U), _p(ws), ws.numel() * 4, _stream()))
    return U


def cp4_conv2d_rebuild_forward(Input, FT, FC, FY, FX, pad=1):
    """The CP4 layer's "rebuild" line (test/benchmark_conv2d_cp4.py:35-42): ``cp4recom`` then an ordinary conv2d."""
    Input = _dev(Input, "Input")
    FT, FC, FY, FX = (_dev(t, n) for t, n in ((FT, "FT"), (FC, "FC"), (FY, "FY"), (FX, "FX")))
    s = _shape_from(Input, FT, FC, FY, FX, pad)
    U = torch.empty((s.N, s.T, s.H, s.W), device=Input.device, dtype=torch.float32)
    with torch.cuda.device(Input.device):
        wsb = lib.b200cp_cp4_rebuild_fwd_workspace_bytes(C.byref(s))
        ws = torch.empty(max(wsb, 4) // 4, device=Input.device, dtype=torch.float32)
        check(lib.b200cp_cp4_rebuild_fwd(C.byref(s), _p(Input), _p(FT), _p(FC), _p(FY), _p(FX), _p(U), _p(ws),
                                         ws.numel() * 4, _stream()))
    return U


def rcp_recompose(*kernels):
    """Dense filter ``[T, C, FH, FW]`` of the reshaped-CP conv from ``(K0[S0,T0,R], ..., KC[FH,FW,R])``."""
    *A, KC = kernels
    A = [_dev(a, f"kernel{k}") for k, a in enumerate(A)]
    KC = _dev(KC, "kernelc")
    cd, td, R = _modes(A, "rcp_recompose")
    if KC.dim() != 3 or KC.shape[2] != R:
        raise ValueError("kernelc must be [FH, FW, rank]")
    Cc, Tc = 1, 1
    for c, t in zip(cd, td):
        Cc *= c
        Tc *= t
    K = torch.empty((Tc, Cc, KC.shape[0], KC.shape[1]), device=KC.device, dtype=torch.float32)
    with torch.cuda.device(KC.device):
        check(lib.b200cp_rcp_recompose(len(A), int_array(cd), int_array(td), R, KC.shape[0], KC.shape[1],
                                       ptr_array([a.data_ptr() for a in A]), _p(KC), _p(K), _stream()))
    return K


def conv2d_rcp_rebuild_nchw(U, *kernels):
    """The reshaped-CP layer's "rebuild" line: recompose the filter, then an ordinary same-size conv2d."""
    K = rcp_recompose(*kernels)
    U = _dev(U, "input")
    N, H, W = U.shape[0], U.shape[-2], U.shape[-1]
    return conv2d_dense_forward(U.reshape(N, K.shape[1], H, W), K, pad=(K.shape[2] - 1) // 2)


def dense_cp_recompose(*kernels):
    """``M [I, O]`` of the CP dense layer (the einsum + reshape of test/benchmark_dense_cp.py:43-44)."""
    Fk = [_dev(f, f"kernel{k}") for k, f in enumerate(kernels)]
    idims, odims, R = _modes(Fk, "dense_cp_recompose")
    I, O = 1, 1
    for a, b in zip(idims, odims):
        I *= a
        O *= b
    M = torch.empty((I, O), device=Fk[0].device, dtype=torch.float32)
    with torch.cuda.device(M.device):
        wsb = lib.b200cp_dense_recompose_workspace_bytes(len(Fk), int_array(idims), int_array(odims), R)
        ws = torch.empty(max(wsb, 4) // 4, device=M.device, dtype=torch.float32)
        check(lib.b200cp_dense_recompose(len(Fk), int_array(idims), int_array(odims), R,
                                         ptr_array([f.data_ptr() for f in Fk]), _p(M), _p(ws), ws.numel() * 4,
                                         _stream()))
    return M


def dense_matmul(U, M):
    """``U [B, I] @ M [I, O]`` with fp32-grade results (test/benchmark_dense_cp.py:45-48)."""
    U, M = _dev(U, "input"), _dev(M, "M")
    B = U.shape[0]
    I, O = M.shape
    if U.numel() != B * I:
        raise ValueError("input size does not match M")
    Y = torch.empty((B, O), device=U.device, dtype=torch.float32)
    with torch.cuda.device(U.device):
        wsb = lib.b200cp_dense_matmul_workspace_bytes(B, I, O)
        ws = torch.empty(max(wsb, 4) // 4, device=U.device, dtype=torch.float32)
        check(lib.b200cp_dense_matmul(B, I, O, _p(U), _p(M), _p(Y), _p(ws), ws.numel() * 4, _stream()))
    return Y


def dense_cp_rebuild(U, *kernels):
    """The CP dense layer's "rebuild" line: recompose ``M``, then one matmul."""
    return dense_matmul(U, dense_cp_recompose(*kernels))


# ---- autograd wrappers ----------------------------------------------------------
class CP4Conv2dFunction(torch.autograd.Function):
    """y = CP4 conv2d(x; FT, FC, FY, FX) with the fused backward kernels."""

    @staticmethod
    def forward(ctx, x, FT, FC, FY, FX, pad=1, flags=0):
        ctx.pad, ctx.flags = pad, flags
        # with 3x3 filters the forward keeps its rank plane for the factor gradients (a quarter of x at C = 4R)
        ctx.shared = (any(t.requires_grad for t in (FT, FC, FY, FX)) and x.dim() == 4 and
                      _shares_planes(_shape_from(x, FT, FC, FY, FX, pad), flags))
        if ctx.shared:
            y, P = cp4_conv2d_forward_save(x, FT, FC, FY, FX, pad, flags)
            ctx.save_for_backward(x, FT, FC, FY, FX, P)
            return y
        ctx.save_for_backward(x, FT, FC, FY, FX)
        return cp4_conv2d_forward(x, FT, FC, FY, FX, pad, flags)

    @staticmethod
    def backward(ctx, dy):
        dy = dy.contiguous()
        if ctx.shared:
            x, FT, FC, FY, FX, P = ctx.saved_tensors
            dx, Q = cp4_conv2d_backward_data_save(dy, FT, FC, FY, FX, ctx.pad, ctx.flags)
            g = cp4_conv2d_backward_filter_saved(dy, x, P, Q, FT, FC, FY, FX, ctx.pad, ctx.flags)
            return (dx if ctx.needs_input_grad[0] else None, *g, None, None)
        x, FT, FC, FY, FX = ctx.saved_tensors
        dx = cp4_conv2d_backward_data(dy, FT, FC, FY, FX, ctx.pad, ctx.flags) if ctx.needs_input_grad[0] else None
        g = (None,) * 4
        if any(ctx.needs_input_grad[1:5]):
            g = cp4_conv2d_backward_filter(dy, x, FT, FC, FY, FX, ctx.pad, ctx.flags)
        return (dx, *g, None, None)


class RCPConv2dFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, KC, *A):
        ctx.save_for_backward(x, KC, *A)
        return conv2d_rcp_fused_nchw(x, *A, KC)

    @staticmethod
    def backward(ctx, dy):
        x, KC, *A = ctx.saved_tensors
        dx, dA, dS = rcp_conv2d_backward(x, dy.contiguous().view(x.shape[0], -1, x.shape[-2], x.shape[-1]), *A, KC)
        return (dx, dS, *dA)


class CPDenseFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, *Fk):
        ctx.save_for_backward(x, *Fk)
        return dense_cp(x, *Fk)

    @staticmethod
    def backward(ctx, dy):
        x, *Fk = ctx.saved_tensors
        dx, dF = dense_cp_backward(x.reshape(x.shape[0], -1), dy.contiguous().reshape(x.shape[0], -1), *Fk)
        return (dx.view_as(x), *dF)
