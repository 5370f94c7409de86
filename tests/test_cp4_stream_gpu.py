"""Parity of the row-stream CP4 kernel (one persistent CTA per SM, rows handed from warp group to warp group) with
the float64 oracle at the fp32 tolerance (rtol 1e-4, atol 1e-5): row lists shorter and longer than the grid, ranges
that start and end inside images, ranks below 16, channel counts that leave output m-blocks unused, the three-factor
core, accumulation into the output, and the two-convolution launch of the training step with its saved rank planes."""
import numpy as np
import pytest
import torch

from oracle import cp_oracle as O
from tests.gpu_util import check, dev

pytestmark = pytest.mark.gpu

# (seed, N, C, T, H, W, R, factor std): W is 8, 24, 40 or 56; C and T multiples of 8 (each is the input channel
# count of one of the two convolutions)
STREAM_SHAPES = [
    (170, 2, 64, 64, 56, 56, 16, 1.0 / 24),   # BASELINE config 2 at N = 2: 112 rows, fewer than CTAs
    (171, 9, 64, 64, 56, 56, 16, 1.0 / 24),   # 504 rows: ranges of 3-4 rows that cross image borders
    (172, 3, 16, 32, 5, 24, 7, 0.2),          # short images, rank padded to 16, half of an m-block group unused
    (173, 5, 24, 48, 3, 8, 16, 0.15),         # one pixel block per row
    (174, 2, 40, 16, 9, 40, 3, 0.1),
    (175, 1, 8, 24, 1, 8, 1, 0.5),            # a single row; 8 output channels in one direction
    (176, 4, 16, 16, 100, 24, 8, 0.3),        # tall images
    (177, 2, 128, 80, 30, 56, 12, 0.03),      # 80 output channels: 5 m-blocks
]


def _inputs(case):
    seed, N, C, T, H, W, R, std = case
    return O.make_cp4_inputs(seed, N, C, T, H, W, 3, 3, R, factor_std=std)


@pytest.fixture(autouse=True)
def _stream_on():
    import paralleltnnlayers_b200 as P
    P.set_stream(1)
    yield
    P.set_stream(-1)


@pytest.mark.parametrize("case", STREAM_SHAPES, ids=lambda c: "s%d" % c[0])
def test_stream_forward_and_backward_data(case):
    import paralleltnnlayers_b200 as P
    X, K0, K1, KH, KW, dU = _inputs(case)
    t = dev(X, K0, K1, KH, KW, dU)
    before = P._lib.lib.b200cp_test_stream_launches()
    U = P.cp4_conv2d_forward(*t[:5], 1)
    dX = P.cp4_conv2d_backward_data(t[5], *t[1:5], 1)
    assert P._lib.lib.b200cp_test_stream_launches() == before + 2     # the kernel under test ran, not another path
    P.device_status()
    check(U, O.cp4_forward(X, K0, K1, KH, KW, 1), "forward (stream)")
    check(dX, O.cp4_backward_data(dU, K0, K1, KH, KW, 1), "backward-data (stream)")
    # the row bands compute the same sums in another order
    P.set_stream(0)
    U2 = P.cp4_conv2d_forward(*t[:5], 1)
    assert float((U - U2).abs().max()) <= 4e-6 * float(U2.abs().max())


@pytest.mark.parametrize("case", [STREAM_SHAPES[0], STREAM_SHAPES[1], STREAM_SHAPES[6]], ids=lambda c: "s%d" % c[0])
def test_stream_step(case):
    """b200cp_cp4_step: both convolutions as one row list, rank planes saved for the factor gradients."""
    import paralleltnnlayers_b200 as P
    X, K0, K1, KH, KW, dU = _inputs(case)
    t = dev(X, K0, K1, KH, KW, dU)
    before = P._lib.lib.b200cp_test_stream_launches()
    U, gX, dK = P.cp4_conv2d_step(t[0], t[5], *t[1:5], 1)
    assert P._lib.lib.b200cp_test_stream_launches() == before + 1     # both convolutions in one launch
    P.device_status()
    check(U, O.cp4_forward(X, K0, K1, KH, KW, 1), "step forward")
    check(gX, O.cp4_backward_data(dU, K0, K1, KH, KW, 1), "step backward-data")
    off = 0
    for r, nm in zip(O.cp4_backward_filter(X, dU, K0, K1, KH, KW, 1), ("dK0", "dK1", "dKH", "dKW")):
        check(dK[off:off + r.size].view(*r.shape), r, "step " + nm, rtol=1e-4, atol=1e-5 * max(1.0, float(np.abs(r).max())))
        off += r.size
    U2, gX2, dK2 = P.cp4_conv2d_step(t[0], t[5], *t[1:5], 1)
    assert torch.equal(U, U2) and torch.equal(gX, gX2) and torch.equal(dK, dK2)


def test_stream_random_shapes_against_the_exact_kernels():
    """Forty seeded random shapes the row stream takes (any batch and height, W in {8, 24, 40, 56}, channels in
    multiples of 8 up to 136, ranks 1..16): forward, backward-data and the stand-alone backward-filter (plane-only
    convolutions + gradient bands) against the exact-fp32 CUDA-core kernels of the same library."""
    import paralleltnnlayers_b200 as P
    rng = np.random.default_rng(4242)
    lib = P._lib.lib
    for k in range(40):
        N = int(rng.integers(1, 7)); H = int(rng.integers(1, 40)); W = int(rng.choice([8, 24, 40, 56]))
        C = 8 * int(rng.integers(1, 18)); T = 8 * int(rng.integers(1, 18)); R = int(rng.integers(1, 17))
        g = torch.Generator(device="cuda").manual_seed(1000 + k)
        X = torch.rand(N, C, H, W, device="cuda", generator=g) * 2 - 1
        dU = torch.randn(N, T, H, W, device="cuda", generator=g)
        K0 = torch.randn(T, R, device="cuda", generator=g) * 0.2
        K1 = torch.randn(C, R, device="cuda", generator=g) * 0.2
        KH = torch.randn(3, R, device="cuda", generator=g) * 0.5
        KW = torch.randn(3, R, device="cuda", generator=g) * 0.5
        what = f"case {k}: N={N} C={C} T={T} H={H} W={W} R={R}"
        before = lib.b200cp_test_stream_launches()
        U = P.cp4_conv2d_forward(X, K0, K1, KH, KW, 1)
        dX = P.cp4_conv2d_backward_data(dU, K0, K1, KH, KW, 1)
        assert lib.b200cp_test_stream_launches() == before + 2, what
        dK = P.cp4_conv2d_backward_filter(dU, X, K0, K1, KH, KW, 1)
        Ue = P.cp4_conv2d_forward(X, K0, K1, KH, KW, 1, flags=P.PATH_SIMT)
        dXe = P.cp4_conv2d_backward_data(dU, K0, K1, KH, KW, 1, flags=P.PATH_SIMT)
        dKe = P.cp4_conv2d_backward_filter(dU, X, K0, K1, KH, KW, 1, flags=P.PATH_SIMT)
        for a, b, nm in [(U, Ue, "forward"), (dX, dXe, "backward-data")] + [(x, y, "dK%d" % i) for i, (x, y) in enumerate(zip(dK, dKe))]:
            scale = float(b.abs().max()) + 1e-30
            assert float((a - b).abs().max()) <= 2e-5 * scale, f"{what}: {nm}"
    P.device_status()


def test_forward_and_backward_data_in_one_call():
    """``b200cp_cp4_fwd_bwd_data``: one row-stream launch for both convolutions (with and without the rank planes),
    two launches of other kernels where the stream does not take the shape; results as the separate calls give."""
    import paralleltnnlayers_b200 as P
    lib = P._lib.lib
    for k, (N, C, T, H, W, R, one) in enumerate([(3, 64, 64, 20, 56, 16, True), (2, 24, 40, 9, 24, 5, True),
                                                 (2, 16, 16, 12, 12, 6, False), (1, 128, 128, 28, 28, 32, False)]):
        g = torch.Generator(device="cuda").manual_seed(77 + k)
        X = torch.rand(N, C, H, W, device="cuda", generator=g) * 2 - 1
        dU = torch.randn(N, T, H, W, device="cuda", generator=g)
        K0 = torch.randn(T, R, device="cuda", generator=g) * 0.2
        K1 = torch.randn(C, R, device="cuda", generator=g) * 0.2
        KH = torch.randn(3, R, device="cuda", generator=g) * 0.5
        KW = torch.randn(3, R, device="cuda", generator=g) * 0.5
        Ue = P.cp4_conv2d_forward(X, K0, K1, KH, KW, 1)
        dXe = P.cp4_conv2d_backward_data(dU, K0, K1, KH, KW, 1)
        before = lib.b200cp_test_stream_launches()
        U, dX = P.cp4_conv2d_forward_backward_data(X, dU, K0, K1, KH, KW, 1)
        assert lib.b200cp_test_stream_launches() - before == (1 if one else 0)
        U2, dX2, Pl, Ql = P.cp4_conv2d_forward_backward_data(X, dU, K0, K1, KH, KW, 1, save=True)
        for a, b, nm in ((U, Ue, "forward"), (dX, dXe, "backward-data"), (U2, Ue, "forward + plane"), (dX2, dXe, "backward-data + plane")):
            assert float((a - b).abs().max()) <= 2e-5 * (float(b.abs().max()) + 1e-30), f"case {k}: {nm}"
        dK = P.cp4_conv2d_backward_filter_saved(dU, X, Pl, Ql, K0, K1, KH, KW, 1)
        dKe = P.cp4_conv2d_backward_filter(dU, X, K0, K1, KH, KW, 1, flags=P.PATH_SIMT)
        for i, (a, b) in enumerate(zip(dK, dKe)):
            assert float((a - b).abs().max()) <= 3e-5 * (float(b.abs().max()) + 1e-30), f"case {k}: dK{i} from the planes"
    # one plane without the other is an argument error, reported as a status
    import ctypes
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    sh = P.tensor_shape(N, C, H, W, T, 3, 3, R, 1)
    rc = lib.b200cp_cp4_fwd_bwd_data(ctypes.byref(sh), vp(X), vp(dU), vp(K0), vp(K1), vp(KH), vp(KW), vp(U), vp(dX), vp(Pl),
                                     None, None, 0)
    assert rc == -1
    P.device_status()
