"""Generate tests/golden/cp4_reference_golden.npz by running the reference's OWN
kernels (oracle/_ref, built from the reference sources by oracle/build_ref.py)
on seeded inputs.  Needs a GPU; run from the repository root:

    python tests/golden/make_reference_golden.py out.npz

Inputs are not stored: each case is (seed, shape) and is regenerated with
oracle.cp_oracle.make_cp4_inputs (the CP4 kernels of Cuda_kernels/) or
oracle.reference_cuda.tvm_inputs (the four fixed-shape TensorFlow-op kernels of
Kernels/).  The outputs are the reference's fp32 results.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import cp_oracle as O  # noqa: E402
from oracle import reference_cuda as RC  # noqa: E402

# name: (seed, N, C, T, H, W, F, R, pad, factor_std)
FWD_CASES = {
    "fwd_cfg1": (0, 1, 16, 16, 32, 32, 3, 8, 1, 0.5),       # BASELINE config 1
    "fwd_odd": (11, 2, 5, 7, 13, 9, 3, 4, 1, 0.5),
    "fwd_5x5": (12, 1, 6, 4, 11, 12, 5, 2, 2, 0.5),
    "fwd_r16_c40": (13, 1, 40, 24, 8, 10, 3, 16, 1, 0.3),   # C >= 32 -> the reference's 8-lane channel split
    "fwd_r1": (14, 1, 3, 5, 6, 7, 3, 1, 1, 0.5),
}
BWD_DATA_CASES = {
    "bwdd_a": (21, 1, 6, 8, 8, 16, 3, 4, 1, 0.5),
    "bwdd_b": (22, 2, 5, 3, 4, 32, 5, 2, 2, 0.5),
}
BWD_FILTER_CASES = {
    "bwdf_a": (31, 1, 3, 4, 6, 5, 3, 2, 1, 0.5),
    "bwdf_b": (32, 2, 2, 3, 4, 4, 3, 4, 1, 0.5),
}


# the fixed-shape TensorFlow-op kernels: name -> (op, seed); shapes in oracle.reference_cuda.TVM_SHAPES
TVM_CASES = {"tvm_rcp": ("rcp", 201), "tvm_dense": ("dense", 202), "tvm_cp3": ("cp3", 203), "tvm_cp4": ("cp4", 204)}


def tvm_oracle(op, arrs):
    """What the float64 oracle gives for the op's inputs, in the op's own output shape."""
    if op == "rcp":      # test/test_conv2d_rcp.py:41-45
        U, K0, K1, KC = arrs
        return O.rcp_forward(U.reshape(1, 16, 32, 32), [K0, K1], KC).reshape(1, 4, 4, 32, 32)
    if op == "dense":    # test/test_dense_cp.py:39
        U, K0, K1, K2 = arrs
        return O.dense_cp_forward_einsum3(U, K0, K1, K2)
    if op == "cp3":      # test/test_conv2d_cp.py:19,33-38: K0 [C,R], K1 [FH,FW,R], K2 [R,T]
        U, K0, K1, K2 = arrs
        return O.cp3_forward(U, K2.T, K0, K1, 1)
    U, K0, K1, K2, K3 = arrs   # test/test_conv2d_cp4.py:25: K0 [C,R], K1 [FH,R], K2 [FW,R], K3 [T,R]
    return O.cp4_forward(U, K3, K0, K1, K2, 1)


def main(out):
    assert RC.available(), "oracle/_ref libraries are missing (python -m oracle.build_ref)"
    res = {}
    if RC.tvm_available():
        for name, (op, seed) in TVM_CASES.items():
            res[name] = RC.tvm_run(op, RC.tvm_inputs(op, seed))
    for name, (seed, N, C, T, H, W, F, R, pad, std) in FWD_CASES.items():
        X, K0, K1, KH, KW, dU = O.make_cp4_inputs(seed, N, C, T, H, W, F, F, R, factor_std=std)
        res[name] = RC.forward(X, K0, K1, KH, KW, pad)
    for name, (seed, N, C, T, H, W, F, R, pad, std) in BWD_DATA_CASES.items():
        X, K0, K1, KH, KW, dU = O.make_cp4_inputs(seed, N, C, T, H, W, F, F, R, factor_std=std)
        res[name] = RC.backward_data(dU, K0, K1, KH, KW, pad)
    for name, (seed, N, C, T, H, W, F, R, pad, std) in BWD_FILTER_CASES.items():
        X, K0, K1, KH, KW, dU = O.make_cp4_inputs(seed, N, C, T, H, W, F, F, R, factor_std=std)
        g = RC.backward_filter(X, dU, K0, K1, KH, KW, pad)
        for nm, a in zip(("dK0", "dK1", "dKH", "dKW"), g):
            res[f"{name}_{nm}"] = a
    np.savez_compressed(out, **res)
    for k, v in res.items():
        print(k, v.shape, float(np.abs(v).max()))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
