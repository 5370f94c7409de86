"""The reference's "rebuild" variants (recomposed weight + the ordinary layer) against the float64 oracle."""
import numpy as np
import pytest
import torch

from oracle import cp_oracle as O
from tests.gpu_util import check, dev

pytestmark = pytest.mark.gpu

CONV_CASES = [
    # seed, N, C, T, H, W, FH, FW, R, pad
    (300, 1, 16, 16, 32, 32, 3, 3, 6, 1),    # BASELINE config 1
    (301, 2, 64, 64, 56, 56, 3, 3, 16, 1),   # config 2 layer at a reduced batch
    (302, 2, 12, 70, 9, 13, 3, 3, 5, 1),     # ragged channels, 117-pixel image (one tile, partly empty)
    (303, 1, 3, 20, 55, 55, 11, 11, 2, 5),   # the reference's 11 x 11 first layer
    (304, 3, 24, 40, 7, 7, 3, 3, 4, 1),      # 49 pixels
    (305, 2, 8, 8, 17, 130, 1, 5, 3, 2),     # wide rows: a tile inside one image row; 1 x 5 filter
    (306, 1, 130, 136, 14, 14, 3, 3, 8, 1),  # three channel tiles, last one ragged
    (307, 2, 16, 16, 12, 10, 3, 3, 4, 0),    # pad 0: zero ring on the bottom / right only
]


@pytest.mark.parametrize("case", CONV_CASES, ids=lambda c: "s%d" % c[0])
def test_cp4_rebuild_forward(case):
    import paralleltnnlayers_b200 as P
    seed, N, C, T, H, W, FH, FW, R, pad = case
    X, K0, K1, KH, KW, _ = O.make_cp4_inputs(seed, N, C, T, H, W, FH, FW, R)
    dX, d0, d1, dH, dW = dev(X, K0, K1, KH, KW)
    K = P.cp4recom(d0, d1, dH, dW)
    Kref = O.cp4_recompose(K0, K1, KH, KW)
    check(K, Kref, "recomposed filter", atol=1e-6 * max(1.0, float(np.abs(Kref).max())))
    ref = O.dense_conv2d(X, Kref, pad)
    tol = 1e-5 * max(1.0, float(np.abs(ref).max()))
    check(P.conv2d_dense_forward(dX, K, pad), ref, "dense conv2d", atol=tol)
    U = P.cp4_conv2d_rebuild_forward(dX, d0, d1, dH, dW, pad)
    check(U, ref, "rebuild forward", atol=tol)
    check(U, O.cp4_forward(X, K0, K1, KH, KW, pad), "rebuild against the factored formula", atol=tol)
    P.device_status()


def test_rcp_rebuild_forward():
    import paralleltnnlayers_b200 as P
    for seed, N, cd, td, H, W, F, R in [(310, 2, (2, 3, 2), (3, 2, 2), 6, 5, 3, 4), (311, 2, (4, 8, 8), (4, 8, 8), 14, 14, 3, 16),
                                        (312, 1, (6,), (10,), 7, 7, 5, 3)]:
        X, A, S, _ = O.make_rcp_inputs(seed, N, cd, td, H, W, F, F, R)
        dX_, dS_ = dev(X, S)
        dA_ = dev(*A)
        Kref = O.rcp_recompose(A, S)
        check(P.rcp_recompose(*dA_, dS_), Kref, "rcp filter", atol=1e-6 * max(1.0, float(np.abs(Kref).max())))
        ref = O.rcp_forward(X, A, S)
        V = P.conv2d_rcp_rebuild_nchw(dX_, *dA_, dS_)
        check(V, ref, "rcp rebuild forward", atol=1e-5 * max(1.0, float(np.abs(ref).max())))
        check(V, P.conv2d_rcp_fused_nchw(dX_, *dA_, dS_).cpu().numpy(), "rebuild against the fused kernel",
              atol=1e-4 * max(1.0, float(np.abs(ref).max())))


@pytest.mark.parametrize("case", [(320, 5, (3, 4), (2, 5), 3), (321, 64, (8, 8, 8), (8, 8, 8), 4),
                                  (322, 300, (4, 8, 8), (8, 8, 6), 7), (323, 7, (2, 2, 2, 2), (3, 2, 2, 2), 2)],
                         ids=lambda c: "s%d" % c[0])
def test_dense_rebuild_forward(case):
    """Small shapes take the CUDA-core product, 300 x 256 x 384 the tcgen05 one."""
    import paralleltnnlayers_b200 as P
    seed, B, idims, odims, R = case
    X, F, _ = O.make_dense_inputs(seed, B, idims, odims, R)
    dX_ = dev(X)[0]
    dF_ = dev(*F)
    Mref = O.dense_cp_weight(F)
    M = P.dense_cp_recompose(*dF_)
    check(M, Mref, "recomposed matrix", atol=1e-6 * max(1.0, float(np.abs(Mref).max())))
    ref = O.dense_cp_forward(X, F)
    Y = P.dense_cp_rebuild(dX_.reshape(B, -1), *dF_)
    check(Y, ref, "dense rebuild forward", atol=1e-5 * max(1.0, float(np.abs(ref).max())))
    P.device_status()


def test_rebuild_errors_are_status_codes():
    import paralleltnnlayers_b200 as P
    X = torch.zeros(1, 8, 8, 8, device="cuda")
    with pytest.raises(ValueError):
        P.conv2d_dense_forward(X, torch.zeros(8, 4, 3, 3, device="cuda"))
    with pytest.raises(P.B200CPError):      # a row of 40 000 pixels and an 11-wide filter do not fit shared memory
        P.conv2d_dense_forward(torch.zeros(1, 1, 1, 40000, device="cuda"), torch.zeros(1, 1, 1, 11, device="cuda"), pad=5)
