"""The reference's own kernels (compiled unmodified into oracle/_ref) run on the GPU and are
compared with the float64 oracle -- this is what pins the oracle -- and with this library."""
import numpy as np
import pytest

from oracle import cp_oracle as O
from oracle import reference_cuda as RC
from tests.gpu_util import check, dev

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not RC.available(), reason="oracle/_ref not built")]


@pytest.mark.parametrize("case", [
    (0, 1, 16, 16, 32, 32, 3, 8, 1, 0.5),
    (41, 1, 48, 256, 55, 55, 11, 16, 5, 0.05),
    (100, 2, 40, 24, 13, 27, 3, 16, 1, 0.2),
    (101, 1, 3, 8, 20, 20, 5, 4, 2, 0.3),
], ids=lambda c: "s%d" % c[0])
def test_reference_forward_matches_oracle_and_library(case):
    import paralleltnnlayers_b200 as P
    seed, N, C, T, H, W, F, R, pad, std = case
    X, K0, K1, KH, KW, dU = O.make_cp4_inputs(seed, N, C, T, H, W, F, F, R, factor_std=std)
    ref = RC.forward(X, K0, K1, KH, KW, pad)
    orc = O.cp4_forward(X, K0, K1, KH, KW, pad)
    check(ref, orc, "reference kernel vs oracle")
    check(P.cp4_conv2d_forward(*dev(X, K0, K1, KH, KW), pad), ref, "library vs reference kernel", rtol=2e-4, atol=2e-5)


@pytest.mark.parametrize("case", [
    (21, 1, 6, 8, 8, 16, 3, 4, 1, 0.5),
    (102, 2, 12, 20, 12, 32, 3, 8, 1, 0.3),
    (103, 1, 5, 3, 4, 32, 5, 2, 2, 0.5),
], ids=lambda c: "s%d" % c[0])
def test_reference_backward_data_matches_oracle(case):
    import paralleltnnlayers_b200 as P
    seed, N, C, T, H, W, F, R, pad, std = case
    X, K0, K1, KH, KW, dU = O.make_cp4_inputs(seed, N, C, T, H, W, F, F, R, factor_std=std)
    ref = RC.backward_data(dU, K0, K1, KH, KW, pad)
    check(ref, O.cp4_backward_data(dU, K0, K1, KH, KW, pad), "reference bwd-data vs oracle")
    check(P.cp4_conv2d_backward_data(*dev(dU, K0, K1, KH, KW), pad), ref, "library vs reference bwd-data",
          rtol=2e-4, atol=2e-5)


def test_reference_backward_filter_matches_oracle():
    import paralleltnnlayers_b200 as P
    X, K0, K1, KH, KW, dU = O.make_cp4_inputs(31, 1, 3, 4, 6, 5, 3, 3, 2, factor_std=0.5)
    ref = RC.backward_filter(X, dU, K0, K1, KH, KW, 1)
    orc = O.cp4_backward_filter(X, dU, K0, K1, KH, KW, 1)
    t = dev(X, K0, K1, KH, KW, dU)
    got = P.cp4_conv2d_backward_filter(t[5], t[0], *t[1:5], 1)
    for a, b, c in zip(ref, orc, got):
        check(a, b, "reference bwd-filter vs oracle", rtol=1e-3, atol=1e-4)
        check(c, b, "library bwd-filter vs oracle", rtol=1e-4, atol=1e-4)


@pytest.mark.skipif(not RC.tvm_available(), reason="oracle/_ref TVM-kernel libraries not built")
@pytest.mark.parametrize("op", ["rcp", "dense", "cp3", "cp4"])
def test_reference_op_kernels_match_oracle_and_library(op):
    """The reference's fixed-shape TensorFlow-op kernels (Kernels/rcp_fused_nchw.cu, dense_cp.cu, cp_fused_nchw.cu,
    cp4_conv_nchw.cu) run here on their one compiled shape: reference == oracle == this library's op of the same name."""
    import importlib.util
    import os
    import paralleltnnlayers_b200 as P
    spec = importlib.util.spec_from_file_location(
        "mk", os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "make_reference_golden.py"))
    mk = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mk)
    arrs = RC.tvm_inputs(op, 300 + len(op))
    ref = RC.tvm_run(op, arrs)
    orc = mk.tvm_oracle(op, arrs)
    # the dense kernel's own sequential fp32 sum is 2e-4 off float64 (its test allows 1e-2, test/test_dense_cp.py:43)
    loose = 1e-3 if op == "dense" else 2e-5
    check(ref, orc, f"reference {op} kernel vs oracle", rtol=loose, atol=1e-5)
    t = dev(*arrs)
    got = {"rcp": P.conv2d_rcp_fused_nchw, "dense": P.dense_cp, "cp3": P.conv2d_cp_fused_nchw, "cp4": P.cp4_conv2d_nchw}[op](*t)
    check(got.reshape(ref.shape), orc, f"library {op} op vs oracle", rtol=1e-4, atol=1e-5 * max(1.0, float(np.abs(orc).max())))
    check(got.reshape(ref.shape), ref, f"library {op} op vs reference kernel", rtol=max(loose, 1e-4),
          atol=1e-5 * max(1.0, float(np.abs(orc).max())))
