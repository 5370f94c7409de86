"""Parity of the reshaped-CP conv2d and CP dense kernels with the float64 oracle."""
import numpy as np
import pytest
import torch

from oracle import cp_oracle as O
from tests.gpu_util import check, dev

pytestmark = pytest.mark.gpu

RCP_CASES = [
    # seed, N, cdims, tdims, H, W, F, R
    (4, 1, (4, 4), (4, 4), 32, 32, 3, 11),        # the reference op's shape (test/test_conv2d_rcp.py:17-20)
    (70, 2, (2, 3, 2), (3, 2, 2), 6, 5, 3, 4),
    (71, 2, (4, 8), (8, 2), 9, 13, 3, 5),
    (72, 1, (6,), (10,), 7, 7, 5, 3),
    (73, 2, (2, 2, 2, 2), (2, 3, 2, 2), 8, 8, 1, 6),
    (74, 2, (4, 8, 8), (4, 8, 8), 14, 14, 3, 16),  # BASELINE config 4 channels at a reduced image
    (75, 1, (4, 8, 8), (4, 8, 8), 10, 12, 3, 5),   # same modes, tiles ragged in both directions
    (76, 6, (4, 8, 8), (4, 8, 8), 14, 12, 3, 6),   # dense gradient on the tensor cores (padded-pixel GEMM, 9 taps, split K)
    (77, 8, (4, 8, 10), (4, 6, 8), 9, 11, 3, 4),   # ... tiles ragged in T (192) and C (320), odd image
    (78, 5, (8, 16), (16, 8), 12, 12, 5, 3),       # ... 5x5 core: 25 taps, two-pixel zero ring
]


@pytest.mark.parametrize("case", RCP_CASES, ids=lambda c: "s%d" % c[0])
def test_rcp_forward_backward(case):
    import paralleltnnlayers_b200 as P
    seed, N, cd, td, H, W, F, R = case
    X, A, S, dV = O.make_rcp_inputs(seed, N, cd, td, H, W, F, F, R)
    dX_, dS_, ddV = dev(X, S, dV)
    dA_ = dev(*A)
    V = P.conv2d_rcp_fused_nchw(dX_, *dA_, dS_)
    check(V, O.rcp_forward(X, A, S), "rcp forward", atol=1e-4)
    gX, gA, gS = P.rcp_conv2d_backward(dX_, ddV, *dA_, dS_)
    rX, rA, rS = O.rcp_backward(X, dV, A, S)
    check(gX, rX, "rcp dX", atol=1e-4)
    for k, (a, b) in enumerate(zip(gA, rA)):
        check(a, b, f"rcp dA{k}", atol=1e-5 * max(1.0, float(np.abs(b).max())))
    check(gS, rS, "rcp dS", atol=1e-5 * max(1.0, float(np.abs(rS).max())))


@pytest.mark.parametrize("tile", ["7", "8"])
def test_rcp_register_tiled_kernel_tiles(tile, monkeypatch):
    """Both tile sizes of the register-tiled order-3 kernel, forward and data gradient, against the chain kernel."""
    import paralleltnnlayers_b200 as P
    X, A, S, dV = O.make_rcp_inputs(76, 2, (4, 8, 8), (4, 8, 8), 17, 9, 3, 3, 3)
    dX_, dS_, ddV = dev(X, S, dV)
    dA_ = dev(*A)
    monkeypatch.setenv("B200CP_RCP_TILE", tile)
    V = P.conv2d_rcp_fused_nchw(dX_, *dA_, dS_)
    gX, _, _ = P.rcp_conv2d_backward(dX_, ddV, *dA_, dS_, need_dw=False)
    monkeypatch.delenv("B200CP_RCP_TILE")
    monkeypatch.setenv("B200CP_NO_FAST", "1")
    V0 = P.conv2d_rcp_fused_nchw(dX_, *dA_, dS_)
    g0, _, _ = P.rcp_conv2d_backward(dX_, ddV, *dA_, dS_, need_dw=False)
    check(V, O.rcp_forward(X, A, S), "rcp forward", atol=1e-4)
    check(gX, O.rcp_backward(X, dV, A, S)[0], "rcp dX", atol=1e-4)
    assert float((V - V0).abs().max()) < 1e-4 and float((gX - g0).abs().max()) < 1e-4


def test_rcp_reference_op_layout():
    """5-D input [N,S0,S1,H,W] and 5-D output, as the TF op is called (test/test_conv2d_rcp.py:47)."""
    import paralleltnnlayers_b200 as P
    X, A, S, _ = O.make_rcp_inputs(4, 1, (4, 4), (4, 4), 32, 32, 3, 3, 11)
    dX_, dS_ = dev(X, S)
    V = P.conv2d_rcp_fused_nchw(dX_.view(1, 4, 4, 32, 32), *dev(*A), dS_)
    assert tuple(V.shape) == (1, 4, 4, 32, 32)
    check(V.reshape(1, 16, 32, 32), O.rcp_forward(X, A, S), "rcp op layout", atol=1e-4)


DENSE_CASES = [
    # seed, B, idims, odims, R
    (6, 1, (16, 16, 16), (4, 4, 4), 137),          # the reference op's shape (test/test_dense_cp.py:15-20)
    (80, 5, (2, 3, 4, 2), (3, 2, 2, 3), 5),
    (81, 33, (8, 8), (4, 16), 7),
    (82, 7, (12,), (9,), 3),
    (83, 64, (8, 8, 8, 8), (8, 8, 8, 8), 4),       # BASELINE config 5 modes at reduced batch and rank
    (84, 5, (8, 8, 8, 8), (8, 8, 8, 8), 3),        # same modes, odd batch (half-empty last CTA)
    (86, 300, (4, 8, 8), (4, 8, 8), 8),            # gradient GEMM on the tensor cores: one 128x256 tile column, ragged K
    (87, 333, (4, 8, 10), (4, 6, 8), 5),           # ... tiles ragged in M (192) and N (320)
    (88, 1024, (8, 8, 8), (8, 8, 8), 4),           # ... several tiles, 64 K stages (the ring wraps 16 times)
]


@pytest.mark.parametrize("case", DENSE_CASES, ids=lambda c: "s%d" % c[0])
def test_dense_forward_backward(case):
    import paralleltnnlayers_b200 as P
    seed, B, idims, odims, R = case
    X, F, dY = O.make_dense_inputs(seed, B, idims, odims, R)
    dX_, ddY = dev(X, dY)
    dF_ = dev(*F)
    Y = P.dense_cp(dX_, *dF_)
    ref = O.dense_cp_forward(X, F)
    check(Y, ref, "dense forward", atol=1e-5 * max(1.0, float(np.abs(ref).max())))
    gX, gF = P.dense_cp_backward(dX_, ddY, *dF_)
    rX, rF = O.dense_cp_backward(X, dY, F)
    check(gX, rX, "dense dX", atol=1e-5 * max(1.0, float(np.abs(rX).max())))
    for k, (a, b) in enumerate(zip(gF, rF)):
        check(a, b, f"dense dF{k}", atol=1e-5 * max(1.0, float(np.abs(b).max())))


def test_dense_register_tiled_kernel_matches_chain_kernel(monkeypatch):
    import paralleltnnlayers_b200 as P
    X, F, dY = O.make_dense_inputs(85, 9, (8, 8, 8, 8), (8, 8, 8, 8), 6)
    dX_, ddY = dev(X, dY)
    dF_ = dev(*F)
    Y = P.dense_cp(dX_, *dF_)
    gX, _ = P.dense_cp_backward(dX_, ddY, *dF_, need_dw=False)
    monkeypatch.setenv("B200CP_NO_FAST", "1")
    Y0 = P.dense_cp(dX_, *dF_)
    g0, _ = P.dense_cp_backward(dX_, ddY, *dF_, need_dw=False)
    scale = float(Y0.abs().max())
    assert float((Y - Y0).abs().max()) < 1e-5 * scale and float((gX - g0).abs().max()) < 1e-5 * float(g0.abs().max())


def test_dense_gradient_gemm_tensor_path_matches_cuda_core_path(monkeypatch):
    """The tcgen05 three-term GEMM and the fp32 CUDA-core GEMM give the same factor gradients to fp32 accuracy."""
    import paralleltnnlayers_b200 as P
    X, F, dY = O.make_dense_inputs(89, 512, (4, 8, 8), (8, 8, 8), 6)
    dX_, ddY = dev(X, dY)
    dF_ = dev(*F)
    _, g1 = P.dense_cp_backward(dX_, ddY, *dF_, need_dx=False)
    monkeypatch.setenv("B200CP_GEMM_TC", "0")
    _, g0 = P.dense_cp_backward(dX_, ddY, *dF_, need_dx=False)
    P.device_status()
    for a, b in zip(g1, g0):
        assert float((a - b).abs().max()) < 2e-5 * float(b.abs().max())


def test_dense_reference_op_layout():
    import paralleltnnlayers_b200 as P
    X, F, _ = O.make_dense_inputs(6, 1, (16, 16, 16), (4, 4, 4), 137)
    V = P.dense_cp(dev(X)[0].view(1, 16, 16, 16), *dev(*F))
    assert tuple(V.shape) == (1, 4, 4, 4)
    ref = O.dense_cp_forward_einsum3(X.reshape(1, 16, 16, 16), *F)
    check(V, ref, "DenseCp", atol=1e-5 * float(np.abs(ref).max()))


def test_autograd_functions():
    import paralleltnnlayers_b200 as P
    X, K0, K1, KH, KW, dU = O.make_cp4_inputs(90, 2, 6, 5, 8, 8, 3, 3, 4, factor_std=0.4)
    t = [a.requires_grad_(True) for a in dev(X, K0, K1, KH, KW)]
    U = P.CP4Conv2dFunction.apply(*t, 1, 0)
    U.backward(dev(dU)[0])
    check(t[0].grad, O.cp4_backward_data(dU, K0, K1, KH, KW, 1), "autograd dX")
    for a, b in zip(t[1:], O.cp4_backward_filter(X, dU, K0, K1, KH, KW, 1)):
        check(a.grad, b, "autograd dK", atol=1e-4)
