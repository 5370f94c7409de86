"""Parity of the row-band CP4 kernel (TMA band loads, mma.sync contractions) with the float64 oracle at the fp32
tolerance (rtol 1e-4, atol 1e-5), on the shapes that exercise its planner: both n-block modes, ragged last bands,
channel counts that are not multiples of 8 or 16, ranks up to 32, the three-factor core, and the two-convolution
launch of the training step with its saved rank planes."""
import numpy as np
import pytest
import torch

from oracle import cp_oracle as O
from tests.gpu_util import check, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _row_bands_only():
    """The row-stream kernel is tried first on the shapes it takes; these tests are about the row bands."""
    import paralleltnnlayers_b200 as P
    P.set_stream(0)
    P._lib.lib.b200cp_test_set_band_max_rank(32)     # by default ranks above 16 go to the tile kernel
    yield
    P._lib.lib.b200cp_test_set_band_max_rank(16)
    P.set_stream(-1)

# (seed, N, C, T, H, W, R, factor std)
BAND_SHAPES = [
    (70, 2, 64, 64, 56, 56, 16, 1.0 / 24),    # BASELINE config 2 at N = 2: bands of 7 rows, consecutive n-blocks
    (71, 2, 128, 128, 28, 28, 16, 0.03),      # config 3, 128 @ 28x28: n-blocks as two runs of four
    (72, 2, 128, 128, 28, 28, 32, 0.03),      # 32 ranks: two rank m-blocks
    (73, 3, 20, 36, 19, 24, 11, 0.08),        # ragged last band, channels not multiples of 8 / 16, odd rank
    (74, 2, 8, 8, 5, 8, 3, 0.2),              # tiny image, fewer n-blocks than warps
    (75, 1, 40, 24, 33, 12, 20, 0.06),        # narrow rows, rank padded to 32
    (76, 2, 16, 16, 32, 32, 8, 0.5),          # BASELINE config 1 shape (batch 2)
    (77, 2, 72, 48, 40, 64, 16, 0.04),        # wide rows
]


def _inputs(case):
    seed, N, C, T, H, W, R, std = case
    return O.make_cp4_inputs(seed, N, C, T, H, W, 3, 3, R, factor_std=std)


@pytest.mark.parametrize("tcgen05", [True, False], ids=["tcgen05", "mmasync"])
@pytest.mark.parametrize("tensor_loads", [False, True], ids=["bulk", "tensormap"])
@pytest.mark.parametrize("case", BAND_SHAPES, ids=lambda c: "s%d" % c[0])
def test_band_forward_and_backward_data(case, tensor_loads, tcgen05):
    """Both ways of loading the band -- one 1-D bulk copy per channel (default; the padding rows are zeroed by the
    CTA), or one 4-D tensor-map box per stage (the padding rows are the map's out-of-range fill) -- and both forms of
    the output contraction: mma.sync with the output staged in shared memory (default), or tcgen05.mma with the
    accumulators in tensor memory."""
    import paralleltnnlayers_b200 as P
    X, K0, K1, KH, KW, dU = _inputs(case)
    t = dev(X, K0, K1, KH, KW, dU)
    P.set_band_tensor_loads(tensor_loads)
    P.set_band_tcgen05(tcgen05)
    try:
        U = P.cp4_conv2d_forward(*t[:5], 1)
        dX = P.cp4_conv2d_backward_data(t[5], *t[1:5], 1)
    finally:
        P.set_band_tensor_loads(False)
        P.set_band_tcgen05(False)
    check(U, O.cp4_forward(X, K0, K1, KH, KW, 1), "forward (band)")
    check(dX, O.cp4_backward_data(dU, K0, K1, KH, KW, 1), "backward-data (band)")
    P.device_status()


@pytest.mark.parametrize("rows", [1, 3, 4, 5])
def test_band_heights(rows):
    """Every band height the planner may pick gives the same result (heights whose halo pitch would collide in
    shared memory are refused by the planner and the next allowed one is used)."""
    import paralleltnnlayers_b200 as P
    case = (78, 2, 24, 40, 21, 28, 16, 0.07)
    X, K0, K1, KH, KW, dU = _inputs(case)
    t = dev(X, K0, K1, KH, KW, dU)
    P.set_band_rows(rows)
    try:
        U = P.cp4_conv2d_forward(*t[:5], 1)
        dX = P.cp4_conv2d_backward_data(t[5], *t[1:5], 1)
    finally:
        P.set_band_rows(0)
    check(U, O.cp4_forward(X, K0, K1, KH, KW, 1), "forward (band rows %d)" % rows)
    check(dX, O.cp4_backward_data(dU, K0, K1, KH, KW, 1), "backward-data (band rows %d)" % rows)


def test_band_matches_exact_path():
    """The three-term tf32 products stay within a few fp32 ulps of the FFMA kernels."""
    import paralleltnnlayers_b200 as P
    X, K0, K1, KH, KW, dU = _inputs((79, 2, 64, 64, 28, 28, 16, 1.0 / 24))
    t = dev(X, K0, K1, KH, KW)
    a = P.cp4_conv2d_forward(*t, 1)
    b = P.cp4_conv2d_forward(*t, 1, flags=P.PATH_SIMT)
    assert float((a - b).abs().max()) <= 2e-6 * float(b.abs().max())


@pytest.mark.parametrize("case", BAND_SHAPES[:4], ids=lambda c: "s%d" % c[0])
def test_band_step(case):
    """b200cp_cp4_step: both convolutions in one launch, rank planes saved for the factor gradients."""
    import paralleltnnlayers_b200 as P
    X, K0, K1, KH, KW, dU = _inputs(case)
    t = dev(X, K0, K1, KH, KW, dU)
    U, gX, dK = P.cp4_conv2d_step(t[0], t[5], *t[1:5], 1)
    check(U, O.cp4_forward(X, K0, K1, KH, KW, 1), "step forward")
    check(gX, O.cp4_backward_data(dU, K0, K1, KH, KW, 1), "step backward-data")
    off = 0
    for r, nm in zip(O.cp4_backward_filter(X, dU, K0, K1, KH, KW, 1), ("dK0", "dK1", "dKH", "dKW")):
        check(dK[off:off + r.size].view(*r.shape), r, "step " + nm, rtol=1e-4, atol=1e-5 * max(1.0, float(np.abs(r).max())))
        off += r.size
    U2, gX2, dK2 = P.cp4_conv2d_step(t[0], t[5], *t[1:5], 1)
    assert torch.equal(U, U2) and torch.equal(gX, gX2) and torch.equal(dK, dK2)
    P.device_status()
