"""The allocation-free factor-gradient entry point, called through the C ABI.

Some hosts of this library cannot call cudaMalloc where they call us (a plugin slot inside
another framework's stream-ordered region, a control loop with a fixed memory budget) and have no
scratch buffer of their own to pass.  b200cp_cp4_bwd_filter_noalloc keeps its partial sums in a
fixed array inside the library instead.  It runs the CUDA-core kernels and must give exactly what
b200cp_cp4_bwd_filter gives on that path (B200CP_PATH_SIMT) with a caller-provided workspace, call after call, although the array still holds the previous call's
partial sums.  This file is collected last on purpose: it has to pass both on its own and after
every other test has used the library."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import cp_oracle as O

pytestmark = pytest.mark.gpu


def _both(P, case):
    seed, N, Cc, T, H, W, F, R, pad = case
    X, K0, K1, KH, KW, dU = O.make_cp4_inputs(seed, N, Cc, T, H, W, F, F, R, factor_std=0.2)
    t = [torch.from_numpy(a).cuda() for a in (X, dU, K0, K1, KH, KW)]
    s = P.tensor_shape(N, Cc, H, W, T, F, F, R, pad)
    lib = P._lib.lib
    p = lambda a: C.c_void_p(a.data_ptr())
    nK = (T + Cc + 2 * F) * R
    wsb = lib.b200cp_cp4_bwd_filter_workspace_bytes(C.byref(s), P.PATH_SIMT)
    ws = torch.empty(max(wsb, 4) // 4, device="cuda")
    ref = torch.full((nK,), float("nan"), device="cuda")
    got = torch.full((nK,), float("nan"), device="cuda")
    P._lib.check(lib.b200cp_cp4_bwd_filter(C.byref(s), *[p(a) for a in t], p(ref), p(ws), wsb, None, P.PATH_SIMT))
    P._lib.check(lib.b200cp_cp4_bwd_filter_noalloc(C.byref(s), *[p(a) for a in t], p(got), None))
    torch.cuda.synchronize()
    oracle = np.concatenate([g.ravel() for g in O.cp4_backward_filter(X, dU, K0, K1, KH, KW, pad)])
    return got.cpu().numpy(), ref.cpu().numpy(), oracle


def test_noalloc_matches_workspace_entry_point_twice_in_a_row():
    import paralleltnnlayers_b200 as P
    # two different shapes back to back: the second call finds the first call's partial sums in the array
    for case in [(301, 4, 16, 24, 28, 28, 3, 16, 1), (302, 2, 10, 6, 12, 20, 5, 4, 2), (301, 4, 16, 24, 28, 28, 3, 16, 1)]:
        got, ref, oracle = _both(P, case)
        assert np.isfinite(got).all()
        # same kernels, same tiles, same fixed summation order: the two entry points agree to the last bit,
        # which is well inside the fp32 tolerance the other tests use (rtol 1e-4, atol 1e-5 of the scale)
        np.testing.assert_array_equal(got, ref)
        scale = max(1.0, float(np.abs(oracle).max()))
        assert np.all(np.abs(got - oracle) <= 1e-5 * scale + 1e-4 * np.abs(oracle))


def test_noalloc_refuses_shapes_beyond_the_built_in_array():
    import paralleltnnlayers_b200 as P
    s = P.tensor_shape(256, 128, 56, 56, 128, 3, 3, 64, 1)     # partial sums far beyond 8 MiB
    lib = P._lib.lib
    # sized the way the call sizes it: the exact-fp32 kernels' partial sums
    assert lib.b200cp_cp4_bwd_filter_workspace_bytes(C.byref(s), P.PATH_SIMT) > (8 << 20)
    one = torch.zeros(1, device="cuda")
    p = C.c_void_p(one.data_ptr())
    rc = lib.b200cp_cp4_bwd_filter_noalloc(C.byref(s), p, p, p, p, p, p, p, None)
    assert rc == -2
    assert b"built-in array" in lib.b200cp_last_error_string()
