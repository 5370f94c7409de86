"""Parity of the three-factor CP conv (free 3x3 core) with the float64 oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import cp_oracle as O
from tests.gpu_util import check, dev

pytestmark = pytest.mark.gpu

# seed, N, C, T, H, W, F, R, pad
CASES = [
    (500, 1, 16, 16, 32, 32, 3, 6, 1),      # the reference op's shape (test/test_conv2d_cp.py:12-15)
    (501, 2, 40, 24, 19, 23, 3, 12, 1),     # ragged tiles, odd channel counts
    (502, 2, 64, 64, 28, 28, 3, 16, 1),
    (503, 1, 24, 24, 8, 8, 3, 80, 1),       # rank > 64
    (504, 2, 9, 7, 10, 12, 5, 3, 2),        # 5x5 core: forward and data gradient only
]


def _inputs(case):
    seed, N, C, T, H, W, F, R, pad = case
    rng = np.random.default_rng(seed)
    X = rng.uniform(-1, 1, size=(N, C, H, W)).astype(np.float32)
    KT = rng.normal(0, 0.3, size=(T, R)).astype(np.float32)
    KCin = rng.normal(0, 0.3, size=(C, R)).astype(np.float32)
    KC = rng.normal(0, 0.3, size=(F, F, R)).astype(np.float32)
    dU = rng.normal(0, 1, size=(N, T, H, W)).astype(np.float32)
    return X, KT, KCin, KC, dU, pad


@pytest.mark.parametrize("case", CASES, ids=lambda c: "s%d" % c[0])
def test_cp3_forward_backward(case):
    import paralleltnnlayers_b200 as P
    X, KT, KCin, KC, dU, pad = _inputs(case)
    dX_, dKT, dKCin, dKC, ddU = dev(X, KT, KCin, KC, dU)
    U = P.cp3_conv2d_forward(dX_, dKT, dKCin, dKC, pad)
    ref = O.cp3_forward(X, KT, KCin, KC, pad)
    check(U, ref, "cp3 forward", atol=1e-5 * max(1.0, float(np.abs(ref).max())))
    rX, rKT, rKCin, rKC = O.cp3_backward(X, dU, KT, KCin, KC, pad)
    gX = P.cp3_conv2d_backward_data(ddU, dKT, dKCin, dKC, pad)
    check(gX, rX, "cp3 dX", atol=1e-5 * max(1.0, float(np.abs(rX).max())))
    if KC.shape[0] == 3:
        g = P.cp3_conv2d_backward_filter(ddU, dX_, dKT, dKCin, dKC, pad)
        for a, r, nm in zip(g, (rKT, rKCin, rKC), ("dKT", "dKCin", "dKC")):
            check(a, r, "cp3 " + nm, rtol=1e-4, atol=1e-5 * max(1.0, float(np.abs(r).max())))
    else:
        with pytest.raises(P.B200CPError):
            P.cp3_conv2d_backward_filter(ddU, dX_, dKT, dKCin, dKC, pad)


def test_cp3_tf_op_argument_order_and_autograd():
    """conv2d_cp_fused_nchw(U, K0[C,R], K1[3,3,R], K2[R,T]) as in test/test_conv2d_cp.py:12-38."""
    import paralleltnnlayers_b200 as P
    rng = np.random.default_rng(7)
    U = rng.uniform(size=(1, 16, 32, 32)).astype(np.float32)
    K0 = rng.uniform(size=(16, 6)).astype(np.float32)
    K1 = rng.uniform(size=(3, 3, 6)).astype(np.float32)
    K2 = rng.uniform(size=(6, 16)).astype(np.float32)
    Kcp = np.einsum("ar,ijr,rx->ijax", *[k.astype(np.float64) for k in (K0, K1, K2)])   # HWIO, the test's filter
    ref = O.dense_conv2d(U, Kcp.transpose(3, 2, 0, 1), 1)
    got = P.conv2d_cp_fused_nchw(*dev(U, K0, K1, K2))
    check(got, ref, "Conv2dCpFusedNchw", rtol=1e-4, atol=1e-4)
    t = [a.requires_grad_(True) for a in dev(U, K2.T.copy(), K0, K1)]
    y = P.CP3Conv2dFunction.apply(*t, 1)
    dy = torch.ones_like(y)
    y.backward(dy)
    rX, rKT, rKCin, rKC = O.cp3_backward(U, np.ones_like(ref, dtype=np.float32), K2.T, K0, K1, 1)
    check(t[0].grad, rX, "autograd dX", atol=1e-3)
    check(t[3].grad, rKC, "autograd dKC", rtol=1e-4, atol=1e-5 * float(np.abs(rKC).max()))
