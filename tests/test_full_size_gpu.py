"""Parity at the full sizes of the benchmark configurations, on the calls the benchmark times.

Config 2 and every (shape, rank) pair of config 3 run ``b200cp_cp4_step`` (forward, backward-data and the factor
gradients in one call) at their full batch and are compared with the float64 oracle: every output element, every
gradient.  Config 4 (reshaped-CP conv) and config 5 (CP dense) run their forward and backward ops at full size.
Tolerance everywhere: |got - ref| <= rtol * |ref| + atol * scale with rtol 1e-4, atol 1e-5 and scale = the largest
magnitude of the reference tensor (for outputs of magnitude 1e-3, as config 2's are, an unscaled atol of 1e-5 would
accept 1 % errors; for gradients that are sums of 10^5 .. 10^7 fp32 products it would ask for more than fp32 has).
One exception, stated where it is used: the factor gradients of config 5 are sums of 1.07e9 products and get
atol 2e-5.  The measured worst error / bound of every case is written to the file named by B200CP_PARITY_REPORT
when that is set.
"""
import json
import os

import numpy as np
import pytest
import torch

from oracle import cp_oracle as O
from tests.gpu_util import check, dev

pytestmark = pytest.mark.gpu

_report = {}


def _note(case, what, worst):
    _report.setdefault(case, {})[what] = round(float(worst), 4)
    path = os.environ.get("B200CP_PARITY_REPORT")
    if path:
        with open(path, "w") as f:
            json.dump(_report, f, indent=1, sort_keys=True)


def _check(got, ref, what, atol=1e-5):
    return check(got, ref, what, rtol=1e-4, atol=atol * float(np.abs(ref).max()))


def _cp4_step_case(name, seed, N, C, H, R):
    import paralleltnnlayers_b200 as P
    X, K0, K1, KH, KW, dU = O.make_cp4_inputs(seed, N, C, C, H, H, 3, 3, R)
    t = dev(X, K0, K1, KH, KW, dU)
    U, dX, dK = P.cp4_conv2d_step(t[0], t[5], *t[1:5], 1)
    P.device_status()
    _note(name, "U", _check(U, O.cp4_forward(X, K0, K1, KH, KW, 1), name + " forward"))
    _note(name, "dX", _check(dX, O.cp4_backward_data(dU, K0, K1, KH, KW, 1), name + " backward-data"))
    off = 0
    for r, nm in zip(O.cp4_backward_filter(X, dU, K0, K1, KH, KW, 1), ("dK0", "dK1", "dKH", "dKW")):
        w = _check(dK[off:off + r.size].view(*r.shape), r, f"{name} {nm}")
        _note(name, nm, w)
        off += r.size


def test_config2_step_full_batch():
    """N=32, C=T=64, 56x56, R=16: the benchmark's step."""
    _cp4_step_case("cfg2", 1, 32, 64, 56, 16)


@pytest.mark.parametrize("k,C,H,R", [(k, C, H, R) for k, (C, H, R) in enumerate(
    (C, H, R) for (C, H) in ((128, 28), (256, 14), (512, 7)) for R in (8, 16, 32, 64))],
    ids=lambda v: str(v))
def test_config3_step_full_batch(k, C, H, R):
    """N=64, (C=T, H=W) in {(128,28), (256,14), (512,7)} x R in {8,16,32,64}, seeds 2+k: on the tile / slice / band
    choice the planner makes at the full batch."""
    _cp4_step_case(f"cfg3_{C}x{H}_R{R}", 2 + k, 64, C, H, R)


def test_config4_rcp_full_size():
    """N=32, 256 = 4*8*8 channels, 28x28, 3x3, R=16: forward, data gradient and factor gradients."""
    import paralleltnnlayers_b200 as P
    X, A, S, dV = O.make_rcp_inputs(20, 32, (4, 8, 8), (4, 8, 8), 28, 28, 3, 3, 16)
    tX, tS, tdV = dev(X, S, dV)
    tA = dev(*A)
    V = P.conv2d_rcp_fused_nchw(tX, *tA, tS)
    dX, dA, dS = P.rcp_conv2d_backward(tX, tdV, *tA, tS)
    P.device_status()
    _note("cfg4", "V", _check(V.reshape(X.shape[0], -1, 28, 28), O.rcp_forward(X, A, S), "cfg4 forward"))
    rX, rA, rS = O.rcp_backward(X, dV, A, S)
    _note("cfg4", "dX", _check(dX.reshape(rX.shape), rX, "cfg4 data gradient"))
    for k, (g, r) in enumerate(zip(list(dA) + [dS], list(rA) + [rS])):
        _note("cfg4", f"dA{k}" if k < 3 else "dS", _check(g, r, f"cfg4 factor gradient {k}"))


def test_config5_dense_full_size():
    """Batch 4096, 8^4 -> 8^4, R=32: forward, data gradient and factor gradients."""
    import paralleltnnlayers_b200 as P
    X, F, dY = O.make_dense_inputs(30, 4096, (8, 8, 8, 8), (8, 8, 8, 8), 32)
    tX, tdY = dev(X, dY)
    tF = dev(*F)
    Y = P.dense_cp(tX, *tF)
    dX, dF = P.dense_cp_backward(tX, tdY, *tF)
    P.device_status()
    ref = O.dense_cp_forward(X, F)
    _note("cfg5", "Y", _check(Y.reshape(ref.shape), ref, "cfg5 forward"))
    rX, rF = O.dense_cp_backward(X, dY, F)
    _note("cfg5", "dX", _check(dX.reshape(rX.shape), rX, "cfg5 data gradient"))
    for k, (g, r) in enumerate(zip(dF, rF)):
        # every entry sums 4096 * 8^6 = 1.07e9 fp32 products (three tf32 terms each): atol 2e-5 of the largest entry
        _note("cfg5", f"dF{k}", _check(g, r, f"cfg5 factor gradient {k}", atol=2e-5))


def test_allclose_counts_on_the_device():
    """``AllClose`` (Cuda_kernels/Utils.cu:143-180): relative differences counted by a device kernel."""
    import paralleltnnlayers_b200 as P
    a = torch.rand(100003, device="cuda") + 0.5
    b = a * (1 + 5e-4)
    assert P.allclose(a, b, 1e-3) and not P.allclose(a, b, 1e-4)
    c = a.clone()
    c[77] = 0.0                                   # a zero switches that element to the absolute difference
    assert not P.allclose(a, c, 1e-3)
    assert P.allclose(a, a.clone(), 0.0)
