"""B200-native fused CP-decomposed layers (CP4 conv2d, reshaped-CP conv2d, CP dense).

Host-side mirror of the reference's operator interface over the C ABI of
``libb200cp.so``; tensors are torch CUDA tensors used as device-memory handles.
"""
from ._lib import (B200CPError, LIB_PATH, PATH_AUTO, PATH_SIMT, PATH_TC1X, PATH_TC3X, TensorShape,
                   launch_count)
from .ops import (CP4Conv2dFunction, CPDenseFunction, RCPConv2dFunction, conv2d_rcp_fused_nchw,
                  cp4_conv2d_backward_data, cp4_conv2d_backward_filter, cp4_conv2d_backward_filter_full,
                  cp4_conv2d_forward, cp4_conv2d_nchw, cp4_conv2d_step_host, cp4recom, dense_cp,
                  dense_cp_backward, rcp_conv2d_backward, tensor_shape)

__all__ = [n for n in dir() if not n.startswith("_")]
