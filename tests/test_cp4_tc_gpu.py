"""The tcgen05 / TMA path of the CP4 conv2d: parity with the float64 oracle.
3-term tf32 split: the fp32 tolerance (rtol 1e-4, atol 1e-5).  Single tf32 pass: rtol 5e-3 of the output scale."""
import os

import numpy as np
import pytest
import torch

from oracle import cp_oracle as O
from tests.gpu_util import check, dev

pytestmark = pytest.mark.gpu

# (seed, N, C, T, H, W, F, R, pad, std)
TC_SHAPES = [
    (0, 1, 16, 16, 32, 32, 3, 8, 1, 0.5),       # BASELINE config 1
    (200, 2, 64, 64, 56, 56, 3, 16, 1, None),   # config 2 channels / image, small batch
    (201, 2, 128, 128, 28, 28, 3, 32, 1, None),  # config 3 (128 @ 28^2)
    (202, 3, 64, 64, 14, 14, 3, 64, 1, None),   # 14^2: one band per image, rank 64
    (203, 2, 40, 24, 12, 20, 3, 6, 1, 0.2),     # channels not multiples of the MMA K step, odd rank
    (204, 1, 16, 48, 16, 24, 5, 16, 2, 0.1),    # 5x5 filter
    (205, 2, 32, 32, 20, 20, 1, 16, 0, 0.2),    # 1x1 filter
    (206, 1, 256, 256, 14, 14, 3, 16, 1, None),  # config 3 (256 @ 14^2)
]


def _inputs(case):
    seed, N, C, T, H, W, F, R, pad, std = case
    return O.make_cp4_inputs(seed, N, C, T, H, W, F, F, R, factor_std=std), pad


@pytest.mark.parametrize("mode", [0, 1])
def test_tc_selftest_single_mma(mode):
    """One tcgen05.mma on operands staged in each of the two shared-memory layouts the kernel uses."""
    import ctypes as C
    import paralleltnnlayers_b200 as P
    rng = np.random.default_rng(mode)
    A = rng.integers(-8, 9, size=(128, 8)).astype(np.float32)     # exactly representable in tf32
    B = rng.integers(-8, 9, size=(16, 8)).astype(np.float32)
    dA, dB = dev(A, B)
    D = torch.full((128, 16), -777.0, device="cuda")
    st = torch.full((1,), -1, device="cuda", dtype=torch.int32)
    p = lambda t: C.c_void_p(t.data_ptr())
    P._lib.check(P._lib.lib.b200cp_debug_tc_selftest(mode, p(dA), p(dB), p(D), p(st), None))
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    ref = A.astype(np.float64) @ B.astype(np.float64).T
    got = D.cpu().numpy()
    print("mode", mode, "nonzero", int((got != 0).sum()), "max|got|", float(np.abs(got).max()), "max|ref|", float(np.abs(ref).max()))
    np.testing.assert_array_equal(got, ref)


def test_tc_intermediate_of_first_band():
    """GEMM 1 alone: the rank-R intermediate P of the first CTA against sum_c K1[c,r] X[0,c,flat]."""
    import paralleltnnlayers_b200 as P
    os.environ["B200CP_TC_TH"] = "4"
    try:
        (X, K0, K1, KH, KW, dU), pad = _inputs((210, 2, 32, 32, 16, 16, 3, 16, 1, 0.3))
        H = W = 16
        TH, Y, Xf, RP = 4, 3, 3, 16
        Mmax = ((TH + Y - 1) * W + Xf - 1 + 3 + 127) // 128 * 128
        U, Pd = P.debug_cp4_tc(*dev(X, K0, K1, KH, KW), pad, 3, RP * Mmax + 64)
        P.device_status()
        Pd = Pd[:RP * Mmax]
        ha = -pad * W - pad
        s0 = ha - ((ha % 4) + 4) % 4
        hb = TH * W + (Y - 1 - pad) * W + (Xf - 1 - pad)
        MB = (hb - s0 + 127) // 128
        Pref = np.zeros((RP, Mmax))
        Pfull = np.einsum("cp,cr->rp", X[0].reshape(32, -1).astype(np.float64), K1.astype(np.float64))
        for m in range(MB * 128):
            f = s0 + m
            if 0 <= f < H * W:
                Pref[:, m] = Pfull[:, f]
        got = Pd.cpu().numpy().reshape(RP, Mmax)[:, :MB * 128]
        check(got, Pref[:, :MB * 128], "P of block 0")
        check(U, O.cp4_forward(X, K0, K1, KH, KW, pad), "forward through the debug entry")
    finally:
        del os.environ["B200CP_TC_TH"]


@pytest.mark.parametrize("case", TC_SHAPES, ids=lambda c: "s%d" % c[0])
def test_tc_forward_and_backward_data(case):
    import paralleltnnlayers_b200 as P
    (X, K0, K1, KH, KW, dU), pad = _inputs(case)
    t = dev(X, K0, K1, KH, KW, dU)
    U = P.cp4_conv2d_forward(*t[:5], pad, flags=P.PATH_TC3X)
    P.device_status()
    check(U, O.cp4_forward(X, K0, K1, KH, KW, pad), "tc forward")
    dX = P.cp4_conv2d_backward_data(t[5], *t[1:5], pad, flags=P.PATH_TC3X)
    P.device_status()
    check(dX, O.cp4_backward_data(dU, K0, K1, KH, KW, pad), "tc backward-data")


def test_tc_single_pass_tolerance():
    import paralleltnnlayers_b200 as P
    (X, K0, K1, KH, KW, dU), pad = _inputs(TC_SHAPES[1])
    ref = O.cp4_forward(X, K0, K1, KH, KW, pad)
    U = P.cp4_conv2d_forward(*dev(X, K0, K1, KH, KW), pad, flags=P.PATH_TC1X)
    P.device_status()
    check(U, ref, "tc single tf32 pass", rtol=5e-3, atol=5e-3 * float(np.abs(ref).max()))


def test_tc_rejects_unsupported_shapes():
    import paralleltnnlayers_b200 as P
    (X, K0, K1, KH, KW, dU), pad = _inputs((220, 1, 8, 8, 7, 7, 3, 4, 1, 0.3))     # 49 pixels: H*W % 4 != 0
    with pytest.raises(P.B200CPError) as e:
        P.cp4_conv2d_forward(*dev(X, K0, K1, KH, KW), pad, flags=P.PATH_TC3X)
    assert e.value.status == -2
    # the automatic path falls back to the CUDA-core kernel for the same shape
    check(P.cp4_conv2d_forward(*dev(X, K0, K1, KH, KW), pad), O.cp4_forward(X, K0, K1, KH, KW, pad), "auto path")
