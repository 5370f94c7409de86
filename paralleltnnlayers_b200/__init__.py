"""B200-native fused CP-decomposed layers (CP4 conv2d, reshaped-CP conv2d, CP dense).

Host-side mirror of the reference's operator interface over the C ABI of
``libb200cp.so``; tensors are torch CUDA tensors used as device-memory handles.

The shared library is loaded on first use of any operator (so that
``paralleltnnlayers_b200.build`` can be imported to build it); a missing or stale
library raises at that point -- there is no fallback implementation.
"""
import importlib

_LIB_NAMES = ("B200CPError", "LIB_PATH", "PATH_AUTO", "PATH_MMA", "PATH_SIMT", "PATH_TC1X", "PATH_TC3X", "TensorShape",
              "launch_count")
_OPS_NAMES = ("allclose", "CP3Conv2dFunction", "conv2d_cp_fused_nchw", "cp3_conv2d_backward_data", "cp3_conv2d_backward_filter",
              "cp3_conv2d_forward", "CP4Conv2dFunction", "CPDenseFunction", "RCPConv2dFunction", "conv2d_rcp_fused_nchw",
              "cp4_conv2d_backward_data", "cp4_conv2d_backward_filter", "cp4_conv2d_backward_filter_full",
              "cp4_conv2d_forward", "cp4_conv2d_nchw", "cp4_conv2d_step", "cp4_conv2d_step_host", "cp4_conv2d_step_host_submit",
              "cp4_conv2d_step_host_wait", "cp4recom", "dense_cp",
              "dense_cp_backward", "debug_cp4_tc", "device_status", "set_band_rows", "set_band_tcgen05", "set_stream", "set_band_tensor_loads", "rcp_conv2d_backward", "tensor_shape",
              "conv2d_dense_forward", "cp4_conv2d_forward_backward_data", "cp4_conv2d_backward_filter_saved",
              "cp4_conv2d_forward_save", "cp4_conv2d_backward_data_save", "cp4_conv2d_rebuild_forward", "rcp_recompose", "conv2d_rcp_rebuild_nchw",
              "dense_cp_recompose", "dense_matmul", "dense_cp_rebuild")
__all__ = list(_LIB_NAMES + _OPS_NAMES)


def __getattr__(name):
    if name in _LIB_NAMES or name == "_lib":
        mod = importlib.import_module("._lib", __name__)
        return mod if name == "_lib" else getattr(mod, name)
    if name in _OPS_NAMES or name == "ops":
        mod = importlib.import_module(".ops", __name__)
        return mod if name == "ops" else getattr(mod, name)
    if name in ("build", "dist", "layers", "sweep"):
        return importlib.import_module("." + name, __name__)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
