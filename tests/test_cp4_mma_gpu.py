"""Parity of the CP4 kernels on the warp-level tensor path (mma.sync, three tf32 terms) with the float64 oracle,
at the fp32 tolerance: rtol 1e-4, atol 1e-5."""
import numpy as np
import pytest
import torch

from oracle import cp_oracle as O
from tests.gpu_util import check, dev
from tests.test_cp4_gpu import FWD_SHAPES, _inputs

pytestmark = pytest.mark.gpu

MMA_SHAPES = FWD_SHAPES + [
    (53, 2, 64, 64, 56, 56, 3, 16, 1, 1.0 / 24),   # BASELINE config 2 at N = 2
    (54, 2, 128, 128, 28, 28, 3, 32, 1, 0.03),     # config 3 shapes at a reduced batch
    (55, 2, 256, 256, 14, 14, 3, 64, 1, 0.02),
    (56, 2, 512, 512, 7, 7, 3, 8, 1, 0.015),       # more channels than one staged factor chunk
]


@pytest.mark.parametrize("case", MMA_SHAPES, ids=lambda c: "s%d" % c[0])
def test_forward_and_backward_data_mma(case):
    import paralleltnnlayers_b200 as P
    (X, K0, K1, KH, KW, dU), pad = _inputs(case)
    dX_, dK0, dK1, dKH, dKW, ddU = dev(X, K0, K1, KH, KW, dU)
    n0 = P.launch_count()
    U = P.cp4_conv2d_forward(dX_, dK0, dK1, dKH, dKW, pad, flags=P.PATH_MMA)
    assert P.launch_count() > n0
    check(U, O.cp4_forward(X, K0, K1, KH, KW, pad), "forward (mma)")
    dX = P.cp4_conv2d_backward_data(ddU, dK0, dK1, dKH, dKW, pad, flags=P.PATH_MMA)
    check(dX, O.cp4_backward_data(dU, K0, K1, KH, KW, pad), "backward-data (mma)")


SLICE_SHAPES = [
    (56, 2, 512, 512, 7, 7, 3, 8, 1, 0.015),       # config 3's smallest image: whole image per tile
    (55, 2, 256, 256, 14, 14, 3, 64, 1, 0.02),
    (58, 3, 40, 72, 19, 23, 3, 24, 1, 0.05),       # channel counts that do not divide into equal slices of 8
    (43, 2, 48, 64, 27, 27, 5, 4, 2, 0.1),         # 5x5 filter
    (59, 2, 24, 24, 8, 8, 3, 80, 1, 0.1),          # rank > 64: two rank chunks accumulate into the output
]


@pytest.mark.parametrize("slices", [2, 4, 8])
@pytest.mark.parametrize("case", SLICE_SHAPES, ids=lambda c: "s%d" % c[0])
def test_channel_slices_over_a_cluster(case, slices, monkeypatch):
    """The S CTAs of a cluster split the channels of one tile and exchange partial rank planes through
    distributed shared memory; forced here, chosen by the planner for small images with many channels."""
    import paralleltnnlayers_b200 as P
    monkeypatch.setenv("B200CP_MMA_SLICES", str(slices))
    (X, K0, K1, KH, KW, dU), pad = _inputs(case)
    dX_, dK0, dK1, dKH, dKW, ddU = dev(X, K0, K1, KH, KW, dU)
    U = P.cp4_conv2d_forward(dX_, dK0, dK1, dKH, dKW, pad, flags=P.PATH_MMA)
    check(U, O.cp4_forward(X, K0, K1, KH, KW, pad), "forward (mma, %d slices)" % slices)
    dX = P.cp4_conv2d_backward_data(ddU, dK0, dK1, dKH, dKW, pad, flags=P.PATH_MMA)
    check(dX, O.cp4_backward_data(dU, K0, K1, KH, KW, pad), "backward-data (mma, %d slices)" % slices)
    if case[6] == 3 and pad == 1:   # the step saves the summed rank planes for the gradient kernel
        U2, gX2, dK = P.cp4_conv2d_step(dX_, ddU, dK0, dK1, dKH, dKW, pad)
        monkeypatch.setenv("B200CP_MMA_SLICES", "1")
        U1, gX1, dK1_ = P.cp4_conv2d_step(dX_, ddU, dK0, dK1, dKH, dKW, pad)
        assert float((U2 - U1).abs().max()) <= 1e-5 * max(1.0, float(U1.abs().max()))
        assert float((gX2 - gX1).abs().max()) <= 1e-5 * max(1.0, float(gX1.abs().max()))
        assert float((dK - dK1_).abs().max()) <= 1e-5 * max(1.0, float(dK1_.abs().max()))
    P.device_status()


def test_mma_path_close_to_exact_path():
    """The three-term tf32 products stay within a few fp32 ulps of the FFMA path."""
    import paralleltnnlayers_b200 as P
    (X, K0, K1, KH, KW, dU), pad = _inputs((57, 2, 64, 64, 28, 28, 3, 16, 1, 1.0 / 24))
    t = dev(X, K0, K1, KH, KW)
    a = P.cp4_conv2d_forward(*t, pad, flags=P.PATH_MMA)
    b = P.cp4_conv2d_forward(*t, pad, flags=P.PATH_SIMT)
    assert float((a - b).abs().max()) <= 2e-6 * float(b.abs().max())


BWDF_MMA_SHAPES = [c for c in MMA_SHAPES if c[6] == 3 and c[8] == 1] + [
    (60, 4, 16, 24, 28, 28, 3, 16, 1, 0.1),
    (58, 3, 40, 72, 19, 23, 3, 24, 1, 0.05),     # ragged tiles, channel counts that are not multiples of 16
    (59, 2, 24, 24, 8, 8, 3, 80, 1, 0.1),        # rank > 64: two rank chunks
]


@pytest.mark.parametrize("case", BWDF_MMA_SHAPES, ids=lambda c: "s%d" % c[0])
def test_backward_filter_mma(case):
    import paralleltnnlayers_b200 as P
    (X, K0, K1, KH, KW, dU), pad = _inputs(case)
    dX_, dK0, dK1, dKH, dKW, ddU = dev(X, K0, K1, KH, KW, dU)
    got = P.cp4_conv2d_backward_filter(ddU, dX_, dK0, dK1, dKH, dKW, pad, flags=P.PATH_MMA)
    ref = O.cp4_backward_filter(X, dU, K0, K1, KH, KW, pad)
    for g, r, nm in zip(got, ref, ("dK0", "dK1", "dKH", "dKW")):
        check(g, r, nm + " (mma)", rtol=1e-4, atol=1e-5 * max(1.0, float(np.abs(r).max())))
    again = P.cp4_conv2d_backward_filter(ddU, dX_, dK0, dK1, dKH, dKW, pad, flags=P.PATH_MMA)
    for a, b in zip(got, again):   # bitwise reproducible
        assert torch.equal(a, b)


STEP_SHAPES = [
    (53, 2, 64, 64, 56, 56, 3, 16, 1, 1.0 / 24),   # BASELINE config 2 at N = 2
    (58, 3, 40, 72, 19, 23, 3, 24, 1, 0.05),       # ragged tiles, odd channel counts
    (59, 2, 24, 24, 8, 8, 3, 80, 1, 0.1),          # rank > 64
    (56, 2, 512, 512, 7, 7, 3, 8, 1, 0.015),
    (43, 2, 48, 64, 27, 27, 5, 4, 2, 0.1),         # 5x5: the step runs the three kernels as they are
]


@pytest.mark.parametrize("case", STEP_SHAPES, ids=lambda c: "s%d" % c[0])
def test_step_shares_the_rank_planes(case):
    """b200cp_cp4_step gives what the three entry points give on the same inputs."""
    import paralleltnnlayers_b200 as P
    (X, K0, K1, KH, KW, dU), pad = _inputs(case)
    dX_, dK0, dK1, dKH, dKW, ddU = dev(X, K0, K1, KH, KW, dU)
    U, gX, dK = P.cp4_conv2d_step(dX_, ddU, dK0, dK1, dKH, dKW, pad)
    check(U, O.cp4_forward(X, K0, K1, KH, KW, pad), "step forward")
    check(gX, O.cp4_backward_data(dU, K0, K1, KH, KW, pad), "step backward-data")
    ref = O.cp4_backward_filter(X, dU, K0, K1, KH, KW, pad)
    off = 0
    for r, nm in zip(ref, ("dK0", "dK1", "dKH", "dKW")):
        check(dK[off:off + r.size].view(*r.shape), r, "step " + nm, rtol=1e-4, atol=1e-5 * max(1.0, float(np.abs(r).max())))
        off += r.size
    U2, gX2, dK2 = P.cp4_conv2d_step(dX_, ddU, dK0, dK1, dKH, dKW, pad)
    assert torch.equal(dK, dK2) and torch.equal(U, U2)     # bitwise reproducible
