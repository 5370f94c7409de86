"""ctypes binding of libb200cp.so (the C ABI declared in include/b200cp.h).

The library is the product: there is no Python or CPU fallback.  Importing this
module without the built shared object raises immediately.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200cp.so")

# flags (include/b200cp.h)
PATH_AUTO, PATH_SIMT, PATH_TC3X, PATH_TC1X, PATH_MMA = 0, 1, 2, 3, 4


class TensorShape(C.Structure):
    """Same fields, order and types as the reference's ``struct tensor_shape``
    (Cuda_kernels/Tensor.cuh:10-19)."""
    _fields_ = [(k, C.c_uint) for k in ("N", "H", "W", "pad", "T", "C", "Y", "X", "Rank")]


class B200CPError(RuntimeError):
    def __init__(self, status, msg):
        super().__init__(f"b200cp status {status}: {msg}")
        self.status = status


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m paralleltnnlayers_b200.build` "
            "(nvcc, sm_100a).  There is no fallback implementation.")
    lib = C.CDLL(LIB_PATH)
    vp, fp, i, sz = C.c_void_p, C.c_void_p, C.c_int, C.c_size_t
    sp = C.POINTER(TensorShape)
    ip = C.POINTER(C.c_int)
    pp = C.POINTER(C.c_void_p)
    sig = {
        "b200cp_cp4_fwd": (i, [sp, fp, fp, fp, fp, fp, fp, vp, i]),
        "b200cp_cp4_bwd_data": (i, [sp, fp, fp, fp, fp, fp, fp, vp, i]),
        "b200cp_cp4_bwd_filter_workspace_bytes": (sz, [sp, i]),
        "b200cp_cp4_bwd_filter": (i, [sp, fp, fp, fp, fp, fp, fp, fp, vp, sz, vp, i]),
        "b200cp_cp4_bwd_filter_noalloc": (i, [sp, fp, fp, fp, fp, fp, fp, fp, vp]),
        "b200cp_cp4_bwd_filter_full": (i, [sp, fp, fp, fp, vp]),
        "b200cp_cp4_recompose": (i, [sp, fp, fp, fp, fp, fp, vp]),
        "b200cp_allclose_count": (i, [fp, fp, sz, C.c_float, C.POINTER(C.c_ulonglong), vp]),
        "b200cp_cp4_shares_planes": (i, [sp, i]),
        "b200cp_cp4_step_workspace_bytes": (sz, [sp, i]),
        "b200cp_cp4_step": (i, [sp, fp, fp, fp, fp, fp, fp, fp, fp, fp, vp, sz, vp, i]),
        "b200cp_cp4_step_allreduce": (i, [vp, sp, fp, fp, fp, fp, fp, fp, fp, fp, fp, vp, sz, vp, i]),
        "b200cp_cp4_step_allreduce_pipelined": (i, [vp, sp, fp, fp, fp, fp, fp, fp, fp, fp, fp, fp, vp, sz, vp, i]),
        "b200cp_p2p_flush": (i, [vp, fp, vp]),
        "b200cp_cp4_fwd_bwd_data": (i, [sp, fp, fp, fp, fp, fp, fp, fp, fp, fp, fp, vp, i]),
        "b200cp_cp4_fwd_save": (i, [sp, fp, fp, fp, fp, fp, fp, fp, vp, i]),
        "b200cp_cp4_bwd_data_save": (i, [sp, fp, fp, fp, fp, fp, fp, fp, vp, i]),
        "b200cp_cp4_bwd_filter_saved_workspace_bytes": (sz, [sp, i]),
        "b200cp_cp4_bwd_filter_saved": (i, [sp, fp, fp, fp, fp, fp, fp, fp, vp, sz, vp, i]),
        "b200cp_cp3_fwd": (i, [sp, fp, fp, fp, fp, fp, vp, i]),
        "b200cp_cp3_bwd_data": (i, [sp, fp, fp, fp, fp, fp, vp, i]),
        "b200cp_cp3_bwd_filter_workspace_bytes": (sz, [sp, i]),
        "b200cp_cp3_bwd_filter": (i, [sp, fp, fp, fp, fp, fp, fp, vp, sz, vp, i]),
        "b200cp_cp4_fwd_host": (i, [sp, fp, fp, fp, fp, fp, fp, i]),
        "b200cp_cp4_step_host": (i, [sp, fp, fp, fp, fp, fp, fp, fp, fp, fp, i]),
        "b200cp_cp4_step_host_submit": (i, [sp, fp, fp, fp, fp, fp, fp, fp, fp, fp, i, i]),
        "b200cp_cp4_step_host_wait": (i, [i]),
        "b200cp_rcp_fwd": (i, [i, i, i, i, ip, ip, i, i, i, fp, pp, fp, fp, vp, i]),
        "b200cp_rcp_bwd_workspace_bytes": (sz, [i, i, i, i, ip, ip, i, i, i, i]),
        "b200cp_rcp_bwd": (i, [i, i, i, i, ip, ip, i, i, i, fp, fp, pp, fp, fp, pp, fp, vp, sz, vp, i]),
        "b200cp_dense_fwd": (i, [i, i, ip, ip, i, fp, pp, fp, vp, i]),
        "b200cp_conv2d_dense_fwd_workspace_bytes": (sz, [sp]),
        "b200cp_conv2d_dense_fwd": (i, [sp, fp, fp, fp, vp, sz, vp]),
        "b200cp_cp4_rebuild_fwd_workspace_bytes": (sz, [sp]),
        "b200cp_cp4_rebuild_fwd": (i, [sp, fp, fp, fp, fp, fp, fp, vp, sz, vp]),
        "b200cp_rcp_recompose": (i, [i, ip, ip, i, i, i, pp, fp, fp, vp]),
        "b200cp_dense_recompose_workspace_bytes": (sz, [i, ip, ip, i]),
        "b200cp_dense_recompose": (i, [i, ip, ip, i, pp, fp, vp, sz, vp]),
        "b200cp_dense_matmul_workspace_bytes": (sz, [i, i, i]),
        "b200cp_dense_matmul": (i, [i, i, i, fp, fp, fp, vp, sz, vp]),
        "b200cp_dense_bwd_workspace_bytes": (sz, [i, i, ip, ip, i, i]),
        "b200cp_dense_bwd": (i, [i, i, ip, ip, i, fp, fp, pp, fp, pp, vp, sz, vp, i]),
        "b200cp_device_status": (i, []),
        "b200cp_last_error_string": (C.c_char_p, []),
        "b200cp_status_string": (C.c_char_p, [i]),
        "b200cp_p2p_init": (i, [i, i, sz, vp, pp]),
        "b200cp_p2p_connect": (i, [vp, vp]),
        "b200cp_p2p_allreduce": (i, [vp, fp, fp, sz, vp]),
        "b200cp_p2p_status": (i, [vp]),
        "b200cp_p2p_destroy": (i, [vp]),
        "b200cp_launch_count": (C.c_ulonglong, []),
        "b200cp_version": (i, []),
    }
    # test and diagnostic entry points (include/b200cp_test.h)
    test_sig = {
        "b200cp_debug_cp4_tc": (i, [sp, fp, fp, fp, fp, fp, fp, fp, i, vp]),
        "b200cp_debug_tc_selftest": (i, [i, fp, fp, fp, vp, vp]),
        "b200cp_test_set_band_rows": (None, [i]),
        "b200cp_test_set_band_trace": (None, [vp]),
        "b200cp_test_set_band_tensor_loads": (None, [i]),
        "b200cp_test_set_band_tcgen05": (None, [i]),
        "b200cp_test_set_band_max_rank": (None, [i]),
        "b200cp_test_set_stream": (None, [i]),
        "b200cp_test_stream_launches": (C.c_longlong, []),
        "b200cp_test_set_p2p_wait_cycles": (None, [C.c_longlong]),
        "b200cp_test_p2p_connect_local": (i, [vp, pp]),
    }
    for table in (sig, test_sig):
        for name, (res, args) in table.items():
            fn = getattr(lib, name)      # AttributeError if the ABI and the library disagree
            fn.restype = res
            fn.argtypes = args
    return lib, tuple(sig), tuple(test_sig)


lib, EXPORTS, TEST_EXPORTS = _load()


def check(status):
    if status != 0:
        raise B200CPError(status, lib.b200cp_last_error_string().decode() or
                          lib.b200cp_status_string(status).decode())


def int_array(vals):
    return (C.c_int * len(vals))(*[int(v) for v in vals])


def ptr_array(ptrs):
    return (C.c_void_p * len(ptrs))(*[C.c_void_p(int(p)) for p in ptrs])


def launch_count():
    return int(lib.b200cp_launch_count())
