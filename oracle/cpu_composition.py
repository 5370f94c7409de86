"""The reference's unfused CP-layer composition, restated for PyTorch-CPU.
TEST INFRASTRUCTURE / CPU BASELINE ONLY.

``test/layers.py:265-283`` (``conv2d_cp``) composes
    conv2d 1x1 [C->R]  ->  depthwise conv2d FHxFW over the R channels  ->  conv2d 1x1 [R->T];
with the depthwise kernel [i,j,r] = KH[i,r]*KW[j,r] that equals the CP4 layer.
TensorFlow is not installed, so the three ops are the torch.nn.functional
equivalents; backward is torch.autograd of the same composition, which is what
a TF user of the unfused layer gets.  rCP and dense-CP follow
``test/layers.py:716-773`` and ``test/layers.py:445-465`` (mode-by-mode
contraction per rank, then sum over ranks).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def cp4_forward(X, K0, K1, KH, KW, pad):
    T, R = K0.shape
    C = K1.shape[0]
    FH, FW = KH.shape[0], KW.shape[0]
    t = F.conv2d(X, K1.t().reshape(R, C, 1, 1))
    dw = torch.einsum("ir,jr->rij", KH, KW).reshape(R, 1, FH, FW)
    # output stays HxW for every pad: pad (pad, F-1-pad) like the reference's window
    t = F.pad(t, (pad, max(FW - 1 - pad, 0), pad, max(FH - 1 - pad, 0)))
    t = F.conv2d(t, dw, groups=R)
    return F.conv2d(t, K0.reshape(T, R, 1, 1))


def cp4_step(X, K0, K1, KH, KW, dU, pad):
    """forward + backward-data + backward-filter, as one autograd step."""
    X = X.detach().requires_grad_(True)
    fs = [k.detach().requires_grad_(True) for k in (K0, K1, KH, KW)]
    U = cp4_forward(X, *fs, pad)
    g = torch.autograd.grad(U, [X] + fs, dU)
    return U.detach(), g[0], g[1:]


def rcp_forward(X, A, S, pad=None):
    """X [N,C,H,W]; A_k [c_k,t_k,R]; S [FH,FW,R]."""
    N, C, H, W = X.shape
    R = S.shape[2]
    FH, FW = S.shape[0], S.shape[1]
    if pad is None:
        pad = (FH - 1) // 2
    cd = [a.shape[0] for a in A]
    td = [a.shape[1] for a in A]
    m = len(A)
    t = X.reshape(N, *cd, H, W)
    # first mode for every rank, then the remaining modes rank by rank
    t = torch.tensordot(t, A[0], dims=([1], [0]))          # [N, c2.., H, W, t1, R]
    t = t.movedim(-1, 0)                                    # [R, N, c2.., H, W, t1]
    for k in range(1, m):
        # contract mode c_k (now axis 2) with A_k[:, :, r] per rank
        t = torch.einsum("rnc...,ctr->rn...t", t, A[k])
    # t: [R, N, H, W, t1..tm] -> [N, R, T, H, W]
    T = 1
    for d in td:
        T *= d
    t = t.reshape(R, N, H, W, T).permute(1, 0, 4, 2, 3)
    t = F.pad(t, (pad, max(FW - 1 - pad, 0), pad, max(FH - 1 - pad, 0)))
    k3 = S.permute(2, 0, 1).reshape(1, R, 1, FH, FW)
    return F.conv3d(t, k3).reshape(N, T, H, W)


def dense_cp_forward(X, Fk):
    """X [B, I]; F_k [i_k, o_k, R]."""
    B = X.shape[0]
    idims = [f.shape[0] for f in Fk]
    m = len(Fk)
    t = X.reshape(B, *idims)
    t = torch.tensordot(t, Fk[0], dims=([1], [0]))          # [B, i2.., o1, R]
    t = t.movedim(-1, 0)                                    # [R, B, i2.., o1]
    for k in range(1, m):
        t = torch.einsum("rbi...,ior->rb...o", t, Fk[k])
    return t.sum(0).reshape(B, -1)
