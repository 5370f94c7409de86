"""CPU checks of the oracle itself: its formulations against each other, against the
literal C restatement of the reference loops, against torch autograd, and against the
golden outputs of the reference's own kernels (tests/golden/)."""
import os

import numpy as np
import pytest
import torch

from oracle import cp_oracle as O
from oracle import cpu_composition as CC
from oracle import literal as L

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "cp4_reference_golden.npz")


def t64(*a):
    return [torch.from_numpy(np.asarray(x)).double() for x in a]


@pytest.mark.parametrize("pad", [0, 1, 2])
def test_cp4_forward_formulations_agree(pad):
    X, K0, K1, KH, KW, dU = O.make_cp4_inputs(0, 2, 5, 6, 9, 7, 3, 3, 4, factor_std=0.5)
    U = O.cp4_forward(X, K0, K1, KH, KW, pad)
    # recompose + dense cross-correlation: the reference test's formula (test_cp4Conv.cpp.cu:26-43)
    np.testing.assert_allclose(U, O.dense_conv2d(X, O.cp4_recompose(K0, K1, KH, KW), pad), atol=1e-12)
    # literal fp32 loops of the reference kernel
    np.testing.assert_allclose(L.forward(X, K0, K1, KH, KW, pad), U, rtol=1e-4, atol=1e-5)
    # the unfused composition of test/layers.py:265-283
    np.testing.assert_allclose(CC.cp4_forward(*t64(X, K0, K1, KH, KW), pad).numpy(), U, atol=1e-12)
    np.testing.assert_allclose(L.backward_data(dU, K0, K1, KH, KW, pad), O.cp4_backward_data(dU, K0, K1, KH, KW, pad),
                               rtol=1e-4, atol=1e-5)


def test_cp4_tf_op_formula():
    # test/test_conv2d_cp4.py:25: Kcp = einsum('ir,hr,wr,or->hwio', K0, K1, K2, K3), SAME, NCHW
    rng = np.random.default_rng(5)
    U = rng.uniform(size=(1, 16, 32, 32)); K0 = rng.uniform(size=(16, 6)); K1 = rng.uniform(size=(3, 6))
    K2 = rng.uniform(size=(3, 6)); K3 = rng.uniform(size=(16, 6))
    Kcp = np.einsum("ir,hr,wr,or->hwio", K0, K1, K2, K3)
    ref = O.dense_conv2d(U, Kcp.transpose(3, 2, 0, 1), 1)
    np.testing.assert_allclose(O.cp4_forward(U, K3, K0, K1, K2, 1), ref, atol=1e-11)


def test_cp4_backward_filter_forms():
    X, K0, K1, KH, KW, dU = O.make_cp4_inputs(1, 2, 4, 3, 6, 5, 3, 3, 4, factor_std=0.5)
    g = O.cp4_backward_filter(X, dU, K0, K1, KH, KW, 1)
    for a, b in zip(g, O.cp4_backward_filter_via_full(X, dU, K0, K1, KH, KW, 1)):
        np.testing.assert_allclose(a, b, atol=1e-11)
    for a, b in zip(L.backward_filter(X, dU, K0, K1, KH, KW, 1), g):
        np.testing.assert_allclose(a, b, rtol=1e-3, atol=1e-4)   # fp32 loop-order sums of the reference
    np.testing.assert_allclose(L.backward_filter_full(X, dU, 3, 3, 1), O.cp4_backward_filter_full(X, dU, 3, 3, 1),
                               rtol=1e-4, atol=1e-4)
    # chain rule of the composition
    _, dX, gf = CC.cp4_step(*t64(X, K0, K1, KH, KW, dU), 1)
    np.testing.assert_allclose(dX.numpy(), O.cp4_backward_data(dU, K0, K1, KH, KW, 1), atol=1e-11)
    for a, b in zip(gf, g):
        np.testing.assert_allclose(a.numpy(), b, atol=1e-10)


def test_cp4_backward_filter_5x5():
    X, K0, K1, KH, KW, dU = O.make_cp4_inputs(2, 1, 3, 2, 7, 6, 5, 5, 2, factor_std=0.5)
    g = O.cp4_backward_filter(X, dU, K0, K1, KH, KW, 2)
    _, _, gf = CC.cp4_step(*t64(X, K0, K1, KH, KW, dU), 2)
    for a, b in zip(gf, g):
        np.testing.assert_allclose(a.numpy(), b, atol=1e-10)


def test_rcp_reference_test_formula():
    # test/test_conv2d_rcp.py:17-45
    X, A, S, dV = O.make_rcp_inputs(4, 1, (4, 4), (4, 4), 8, 8, 3, 3, 11)
    Kh = np.einsum("axr,byr,hwr->hwabxy", *[a.astype(np.float64) for a in A], S.astype(np.float64)).reshape(3, 3, 16, 16)
    np.testing.assert_allclose(O.dense_conv2d(X, Kh.transpose(3, 2, 0, 1), 1), O.rcp_forward(X, A, S), atol=1e-12)


def test_rcp_forward_and_backward():
    X, A, S, dV = O.make_rcp_inputs(3, 2, (2, 3, 2), (3, 2, 2), 6, 5, 3, 3, 4)
    V = O.rcp_forward(X, A, S)
    np.testing.assert_allclose(O.rcp_forward_factored(X, A, S), V, atol=1e-12)
    Xt, St = t64(X, S)
    At = t64(*A)
    for t in [Xt, St] + At:
        t.requires_grad_(True)
    Vt = CC.rcp_forward(Xt, At, St)
    np.testing.assert_allclose(Vt.detach().numpy(), V, atol=1e-12)
    gr = torch.autograd.grad(Vt, [Xt] + At + [St], t64(dV)[0])
    dX, dA, dS = O.rcp_backward(X, dV, A, S)
    np.testing.assert_allclose(dX, gr[0].numpy(), atol=1e-11)
    for a, b in zip(dA, gr[1:4]):
        np.testing.assert_allclose(a, b.numpy(), atol=1e-10)
    np.testing.assert_allclose(dS, gr[4].numpy(), atol=1e-10)


def test_dense_cp_forms():
    # test/test_dense_cp.py:39
    X3, F3, _ = O.make_dense_inputs(6, 2, (4, 4, 4), (2, 2, 2), 7)
    np.testing.assert_allclose(O.dense_cp_forward(X3, F3).reshape(2, 2, 2, 2),
                               O.dense_cp_forward_einsum3(X3.reshape(2, 4, 4, 4), *F3), atol=1e-12)
    X, F, dY = O.make_dense_inputs(5, 3, (2, 3, 4, 2), (3, 2, 2, 3), 5)
    Xt = t64(X)[0].requires_grad_(True)
    Ft = [f.requires_grad_(True) for f in t64(*F)]
    Yt = CC.dense_cp_forward(Xt, Ft)
    np.testing.assert_allclose(Yt.detach().numpy(), O.dense_cp_forward(X, F), atol=1e-12)
    gr = torch.autograd.grad(Yt, [Xt] + Ft, t64(dY)[0])
    dX, dF = O.dense_cp_backward(X, dY, F)
    np.testing.assert_allclose(dX, gr[0].numpy(), atol=1e-11)
    for a, b in zip(dF, gr[1:]):
        np.testing.assert_allclose(a, b.numpy(), atol=1e-10)


def test_linearity_and_shift_properties():
    X, K0, K1, KH, KW, dU = O.make_cp4_inputs(7, 1, 3, 4, 8, 8, 3, 3, 2, factor_std=0.5)
    U = O.cp4_forward(X, K0, K1, KH, KW, 1)
    np.testing.assert_allclose(O.cp4_forward(2.5 * X.astype(np.float64), K0, K1, KH, KW, 1), 2.5 * U, atol=1e-12)
    # <dU, fwd(X)> == <bwd_data(dU), X>  (adjoint identity, same padding)
    lhs = float((dU.astype(np.float64) * U).sum())
    rhs = float((O.cp4_backward_data(dU, K0, K1, KH, KW, 1) * X).sum())
    assert abs(lhs - rhs) < 1e-9 * max(1.0, abs(lhs))


@pytest.mark.skipif(not os.path.exists(GOLDEN), reason="golden file not generated yet")
def test_oracle_matches_reference_golden():
    """The float64 restatement against fp32 outputs of the reference's own kernels."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("mk", os.path.join(os.path.dirname(GOLDEN), "make_reference_golden.py"))
    mk = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mk)
    gold = np.load(GOLDEN)
    for name, (seed, N, C, T, H, W, F, R, pad, std) in mk.FWD_CASES.items():
        X, K0, K1, KH, KW, dU = O.make_cp4_inputs(seed, N, C, T, H, W, F, F, R, factor_std=std)
        np.testing.assert_allclose(gold[name], O.cp4_forward(X, K0, K1, KH, KW, pad), rtol=1e-4, atol=1e-5, err_msg=name)
    for name, (seed, N, C, T, H, W, F, R, pad, std) in mk.BWD_DATA_CASES.items():
        X, K0, K1, KH, KW, dU = O.make_cp4_inputs(seed, N, C, T, H, W, F, F, R, factor_std=std)
        np.testing.assert_allclose(gold[name], O.cp4_backward_data(dU, K0, K1, KH, KW, pad), rtol=1e-4, atol=1e-5,
                                   err_msg=name)
    for name, (seed, N, C, T, H, W, F, R, pad, std) in mk.BWD_FILTER_CASES.items():
        X, K0, K1, KH, KW, dU = O.make_cp4_inputs(seed, N, C, T, H, W, F, F, R, factor_std=std)
        g = O.cp4_backward_filter(X, dU, K0, K1, KH, KW, pad)
        for nm, a in zip(("dK0", "dK1", "dKH", "dKW"), g):
            np.testing.assert_allclose(gold[f"{name}_{nm}"], a, rtol=1e-3, atol=1e-4, err_msg=f"{name}_{nm}")
    # The four fixed-shape TensorFlow-op kernels (reshaped-CP conv, CP dense, three-factor CP conv, CP4 conv).  The
    # three convolutions agree with float64 to 3e-6 relative.  The dense kernel adds 137 * 4096 positive products one
    # after the other in fp32 and is 2.2e-4 off (the reference's own test allows 1e-2, test/test_dense_cp.py:43):
    # it is pinned at 1e-3.
    from oracle import reference_cuda as RC
    for name, (op, seed) in mk.TVM_CASES.items():
        assert name in gold.files, f"{name} is missing from the golden file"
        want = mk.tvm_oracle(op, RC.tvm_inputs(op, seed))
        np.testing.assert_allclose(gold[name], want, rtol=1e-3 if op == "dense" else 2e-5, atol=1e-5, err_msg=name)


def test_cp3_oracle_matches_the_reference_formula_and_autograd():
    """The three-factor filter of test/test_conv2d_cp.py:19, evaluated with the reference's own einsum string,
    and float64 autograd of the dense conv for the gradients."""
    import torch
    rng = np.random.default_rng(11)
    K0 = rng.uniform(size=(1, 1, 16, 6)); K1 = rng.uniform(size=(3, 3, 6, 1)); K2 = rng.uniform(size=(1, 1, 6, 16))
    Kcp = np.einsum('llar,ijrl,llrx->ijax', K0, K1, K2)                       # HWIO, as the reference builds it
    mine = O.cp3_recompose(K2.reshape(6, 16).T, K0.reshape(16, 6), K1.reshape(3, 3, 6))   # [T,C,Y,X]
    np.testing.assert_allclose(mine, Kcp.transpose(3, 2, 0, 1), rtol=1e-12, atol=1e-12)
    X = rng.normal(size=(2, 5, 7, 6)); KT = rng.normal(size=(4, 3)); KCin = rng.normal(size=(5, 3))
    KC = rng.normal(size=(3, 3, 3)); dU = rng.normal(size=(2, 4, 7, 6))
    t = [torch.tensor(a, dtype=torch.float64, requires_grad=True) for a in (X, KT, KCin, KC)]
    y = torch.nn.functional.conv2d(t[0], torch.einsum('tr,cr,yxr->tcyx', t[1], t[2], t[3]), padding=1)
    np.testing.assert_allclose(y.detach().numpy(), O.cp3_forward(X, KT, KCin, KC, 1), rtol=1e-10, atol=1e-10)
    y.backward(torch.tensor(dU))
    for a, b in zip([x.grad.numpy() for x in t], O.cp3_backward(X, dU, KT, KCin, KC, 1)):
        np.testing.assert_allclose(a, b, rtol=1e-10, atol=1e-10)
