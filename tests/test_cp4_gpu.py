"""Parity of the CP4 conv2d kernels with the float64 oracle, through the C ABI.
fp32 tolerance: rtol 1e-4, atol 1e-5 (the tolerance the task states for fp32)."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import cp_oracle as O
from tests.gpu_util import check, dev

pytestmark = pytest.mark.gpu

# (seed, N, C, T, H, W, F, R, pad, std) -- the reference's own test shapes have odd sizes (55, 27, 13, 7)
FWD_SHAPES = [
    (0, 1, 16, 16, 32, 32, 3, 8, 1, 0.5),      # BASELINE config 1
    (40, 1, 16, 16, 32, 32, 3, 6, 1, 0.5),     # the TF op's shape, R = 6 (test/test_conv2d_cp4.py:10-17)
    (41, 1, 48, 256, 55, 55, 11, 16, 5, 0.05),  # Cuda_kernels/test/test_cp4Conv.cpp.cu:16-22
    (42, 1, 192, 384, 13, 13, 3, 16, 1, 0.05),  # AlexNet conv4 (bench/tensors_alexnet.txt:24)
    (43, 2, 48, 64, 27, 27, 5, 4, 2, 0.1),
    (44, 3, 7, 5, 7, 7, 3, 1, 1, 0.5),
    (45, 2, 9, 11, 10, 70, 3, 2, 1, 0.3),
    (46, 1, 20, 12, 12, 130, 3, 12, 1, 0.2),   # W > 96: column tiles
    (47, 2, 12, 10, 9, 8, 1, 5, 0, 0.4),       # 1x1 filter
    (48, 1, 8, 8, 9, 9, 3, 3, 0, 0.4),         # pad 0 with a 3x3 filter
    (49, 1, 8, 8, 9, 9, 3, 3, 2, 0.4),         # pad 2 with a 3x3 filter
    (50, 2, 32, 32, 14, 14, 3, 32, 1, 0.1),
    (51, 2, 64, 48, 7, 7, 3, 64, 1, 0.1),
    (52, 1, 24, 24, 8, 8, 3, 80, 1, 0.1),      # rank > 64: two rank chunks
]


def _inputs(case):
    seed, N, C, T, H, W, F, R, pad, std = case
    return O.make_cp4_inputs(seed, N, C, T, H, W, F, F, R, factor_std=std), pad


@pytest.mark.parametrize("case", FWD_SHAPES, ids=lambda c: "s%d" % c[0])
def test_forward_and_backward_data(case):
    import paralleltnnlayers_b200 as P
    (X, K0, K1, KH, KW, dU), pad = _inputs(case)
    dX_, dK0, dK1, dKH, dKW, ddU = dev(X, K0, K1, KH, KW, dU)
    n0 = P.launch_count()
    U = P.cp4_conv2d_forward(dX_, dK0, dK1, dKH, dKW, pad, flags=P.PATH_SIMT)
    assert P.launch_count() > n0
    check(U, O.cp4_forward(X, K0, K1, KH, KW, pad), "forward")
    dX = P.cp4_conv2d_backward_data(ddU, dK0, dK1, dKH, dKW, pad, flags=P.PATH_SIMT)
    check(dX, O.cp4_backward_data(dU, K0, K1, KH, KW, pad), "backward-data")


BWDF_SHAPES = [c for c in FWD_SHAPES if c[8] == (c[6] - 1) // 2 and c[0] != 41] + [
    (60, 4, 16, 24, 28, 28, 3, 16, 1, 0.1),
    (61, 2, 6, 10, 20, 12, 7, 4, 3, 0.2),
]


@pytest.mark.parametrize("case", BWDF_SHAPES, ids=lambda c: "s%d" % c[0])
def test_backward_filter(case):
    import paralleltnnlayers_b200 as P
    (X, K0, K1, KH, KW, dU), pad = _inputs(case)
    dX_, dK0, dK1, dKH, dKW, ddU = dev(X, K0, K1, KH, KW, dU)
    got = P.cp4_conv2d_backward_filter(ddU, dX_, dK0, dK1, dKH, dKW, pad, flags=P.PATH_SIMT)
    ref = O.cp4_backward_filter(X, dU, K0, K1, KH, KW, pad)
    for g, r, nm in zip(got, ref, ("dK0", "dK1", "dKH", "dKW")):
        # gradient entries are sums of N*H*W*... signed terms: the absolute floor scales with the typical magnitude
        check(g, r, nm, rtol=1e-4, atol=1e-5 * max(1.0, float(np.abs(r).max())))
    # bitwise reproducible
    again = P.cp4_conv2d_backward_filter(ddU, dX_, dK0, dK1, dKH, dKW, pad, flags=P.PATH_SIMT)
    for a, b in zip(got, again):
        assert torch.equal(a, b)


def test_backward_filter_full_and_recompose():
    import paralleltnnlayers_b200 as P
    (X, K0, K1, KH, KW, dU), pad = _inputs((62, 2, 5, 6, 9, 10, 3, 4, 1, 0.5))
    dX_, dK0, dK1, dKH, dKW, ddU = dev(X, K0, K1, KH, KW, dU)
    check(P.cp4_conv2d_backward_filter_full(ddU, dX_, 3, 3, pad), O.cp4_backward_filter_full(X, dU, 3, 3, pad), "dK full",
          atol=1e-4)
    check(P.cp4recom(dK0, dK1, dKH, dKW), O.cp4_recompose(K0, K1, KH, KW), "cp4recom")


def test_tf_op_argument_order():
    """cp4_conv2d_nchw(U, K0[C,R], K1[FH,R], K2[FW,R], K3[T,R]) as in test/test_conv2d_cp4.py:19-34."""
    import paralleltnnlayers_b200 as P
    rng = np.random.default_rng(3)
    U = rng.uniform(size=(1, 16, 32, 32)).astype(np.float32)
    K0 = rng.uniform(size=(16, 6)).astype(np.float32); K1 = rng.uniform(size=(3, 6)).astype(np.float32)
    K2 = rng.uniform(size=(3, 6)).astype(np.float32); K3 = rng.uniform(size=(16, 6)).astype(np.float32)
    Kcp = np.einsum("ir,hr,wr,or->hwio", *[k.astype(np.float64) for k in (K0, K1, K2, K3)])
    ref = O.dense_conv2d(U, Kcp.transpose(3, 2, 0, 1), 1)
    got = P.cp4_conv2d_nchw(*dev(U, K0, K1, K2, K3))
    check(got, ref, "Cp4Conv2dNchw", rtol=1e-4, atol=1e-4)


def test_config2_full_size_parity_and_properties():
    """BASELINE config 2 (N=32, C=T=64, 56x56, R=16): oracle parity plus the adjoint identity
    <dU, fwd(X)> == <bwd_data(dU), X> and Euler's identity <K, dK> == <dU, U> for each factor."""
    import paralleltnnlayers_b200 as P
    (X, K0, K1, KH, KW, dU), pad = _inputs((1, 32, 64, 64, 56, 56, 3, 16, 1, None))
    t = dev(X, K0, K1, KH, KW, dU)
    U = P.cp4_conv2d_forward(*t[:5], pad)
    dX = P.cp4_conv2d_backward_data(t[5], *t[1:5], pad)
    g = P.cp4_conv2d_backward_filter(t[5], t[0], *t[1:5], pad)
    check(U, O.cp4_forward(X, K0, K1, KH, KW, pad), "forward cfg2")
    check(dX, O.cp4_backward_data(dU, K0, K1, KH, KW, pad), "backward-data cfg2")
    ref = O.cp4_backward_filter(X, dU, K0, K1, KH, KW, pad)
    for a, r, nm in zip(g, ref, ("dK0", "dK1", "dKH", "dKW")):
        check(a, r, nm + " cfg2", rtol=1e-4, atol=1e-5 * max(1.0, float(np.abs(r).max())))
    lhs = float((t[5].double() * U.double()).sum())
    rhs = float((dX.double() * t[0].double()).sum())
    assert abs(lhs - rhs) <= 1e-4 * abs(lhs) + 1e-2
    for k, a in zip(t[1:5], g):   # U is linear in each factor: <K, dK> = <dU, U>
        assert abs(float((k.double() * a.double()).sum()) - lhs) <= 1e-4 * abs(lhs) + 1e-2


def test_host_entry_point():
    import paralleltnnlayers_b200 as P
    (X, K0, K1, KH, KW, dU), pad = _inputs((63, 2, 8, 6, 12, 12, 3, 4, 1, 0.3))
    ts = [torch.from_numpy(a).pin_memory() for a in (X, dU, K0, K1, KH, KW)]
    U, dX, dK = P.cp4_conv2d_step_host(*ts, pad=pad)
    check(U, O.cp4_forward(X, K0, K1, KH, KW, pad), "host fwd")
    check(dX, O.cp4_backward_data(dU, K0, K1, KH, KW, pad), "host bwd-data")
    ref = np.concatenate([a.ravel() for a in O.cp4_backward_filter(X, dU, K0, K1, KH, KW, pad)])
    check(dK, ref, "host dK", atol=1e-4)


def test_host_entry_point_two_slots_in_flight():
    """Three different steps queued on alternating slots; every result must belong to its own inputs."""
    import paralleltnnlayers_b200 as P
    cases = [_inputs((64 + k, 3, 8, 6, 12, 12, 3, 4, 1, 0.3)) for k in range(3)]
    pins, outs = [], []
    for (X, K0, K1, KH, KW, dU), pad in cases:
        pins.append([torch.from_numpy(a).pin_memory() for a in (X, dU, K0, K1, KH, KW)])
        outs.append((torch.empty(X.shape[0], K0.shape[0], 12, 12).pin_memory(), torch.empty(X.shape).pin_memory(),
                     torch.empty((K0.shape[0] + K1.shape[0] + 6) * 4).pin_memory()))
    for k in range(3):
        P.cp4_conv2d_step_host_submit(*pins[k], outs[k], pad=1, slot=k % 2)
        if k >= 1:
            P.cp4_conv2d_step_host_wait((k - 1) % 2)
    P.cp4_conv2d_step_host_wait(0)
    for ((X, K0, K1, KH, KW, dU), pad), (U, dX, dK) in zip(cases, outs):
        check(U, O.cp4_forward(X, K0, K1, KH, KW, pad), "queued fwd")
        check(dX, O.cp4_backward_data(dU, K0, K1, KH, KW, pad), "queued bwd-data")
        ref = np.concatenate([a.ravel() for a in O.cp4_backward_filter(X, dU, K0, K1, KH, KW, pad)])
        check(dK, ref, "queued dK", atol=1e-4)


def test_host_entry_point_four_slots_in_flight():
    """Six steps over the four slots, three or four in flight at a time; a slot outside 0 .. 3 is refused."""
    import paralleltnnlayers_b200 as P
    cases = [_inputs((80 + k, 2, 8, 16, 9, 24, 3, 5, 1, 0.3)) for k in range(6)]
    pins, outs = [], []
    for (X, K0, K1, KH, KW, dU), pad in cases:
        pins.append([torch.from_numpy(a).pin_memory() for a in (X, dU, K0, K1, KH, KW)])
        outs.append((torch.empty(X.shape[0], K0.shape[0], X.shape[2], X.shape[3]).pin_memory(),
                     torch.empty(X.shape).pin_memory(), torch.empty((K0.shape[0] + K1.shape[0] + 6) * K0.shape[1]).pin_memory()))
    for k in range(6):
        P.cp4_conv2d_step_host_submit(*pins[k], outs[k], pad=1, slot=k % 4)
        if k >= 3:
            P.cp4_conv2d_step_host_wait((k - 3) % 4)
    for k in range(3, 6):
        P.cp4_conv2d_step_host_wait(k % 4)
    for ((X, K0, K1, KH, KW, dU), pad), (U, dX, dK) in zip(cases, outs):
        check(U, O.cp4_forward(X, K0, K1, KH, KW, pad), "queued fwd")
        check(dX, O.cp4_backward_data(dU, K0, K1, KH, KW, pad), "queued bwd-data")
        ref = np.concatenate([a.ravel() for a in O.cp4_backward_filter(X, dU, K0, K1, KH, KW, pad)])
        check(dK, ref, "queued dK", atol=1e-4)
    with pytest.raises(P.B200CPError):
        P.cp4_conv2d_step_host_submit(*pins[0], outs[0], pad=1, slot=4)


def test_errors_are_status_codes():
    import paralleltnnlayers_b200 as P
    x = torch.zeros(1, 4, 8, 8, device="cuda")
    f = lambda d, r=3: torch.zeros(d, r, device="cuda")
    with pytest.raises(ValueError):
        P.cp4_conv2d_forward(x, f(5), f(3), f(3), f(3))          # C mismatch
    with pytest.raises(P.B200CPError) as e:
        P.cp4_conv2d_backward_filter(torch.zeros(1, 5, 8, 8, device="cuda"), x, f(5), f(4), f(3), f(3), pad=0)
    assert e.value.status == -2
    with pytest.raises(P.B200CPError) as e:
        P._lib.check(P._lib.lib.b200cp_cp4_fwd(None, None, None, None, None, None, None, None, 0))
    assert e.value.status == -1
