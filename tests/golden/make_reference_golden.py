"""Generate tests/golden/cp4_reference_golden.npz by running the reference's OWN
kernels (oracle/_ref, built from the reference sources by oracle/build_ref.py)
on seeded inputs.  Needs a GPU; run from the repository root:

    python tests/golden/make_reference_golden.py [out.npz]

Inputs are not stored: each case is (seed, shape) and is regenerated with
oracle.cp_oracle.make_cp4_inputs.  The outputs are the reference's fp32 results.
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


def main(out):
    assert RC.available(), "oracle/_ref libraries are missing (python -m oracle.build_ref)"
    res = {}
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
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "gpurun_out", "cp4_reference_golden.npz"))
