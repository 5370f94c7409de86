"""``torch.nn`` layers on top of the fused kernels, with the reference's rank-from-compression-rate rules.

The reference builds its layers with ``conv2d_tensor`` / ``dense_tensor`` (test/layers.py:63-101,147-175): a
compression ``rate`` is turned into a CP rank by ``generate_params_*`` (pure integer arithmetic, restated here),
factor variables are created, and the layer is the sequential or the fused op.  These modules keep that
interface for the three CP layer families of the hot path; weights live in the layout the C ABI takes
(``[dim, R]`` factors for CP4, ``[c_k, t_k, R]`` for rCP, ``[i_k, o_k, R]`` for the dense layer).
"""
from __future__ import annotations

import math

import torch
from torch import nn

DEFAULT_COMPRESSION_RATE = 0.1        # test/layers.py:16
DEFAULT_FACTORIZATION_BASE = 16       # test/layers.py:17


def generate_shape(number, order=None, base=None, reverse=False):
    """Mode sizes of a power of two ``number = 2**e``, the rule of the reference's ``generate_shape``
    (test/layers.py:22-48), stated on the exponents.

    ``base = 2**b``: ``e = q*b + s`` gives ``q`` modes of size ``base``; the left-over ``2**s`` becomes a mode of its
    own when it is at least ``sqrt(base)`` (``2*s >= b``) or when there is no other mode, else it is folded into the
    first mode.  ``order``: the ``e`` twos are dealt to ``order`` modes in turn, so the first ``e % order`` modes get
    one more.  ``reverse`` flips the list.
    """
    if number <= 0 or number & (number - 1):
        raise ValueError("generate_shape supports powers of two only")
    if (order is None) == (base is None):
        raise ValueError("give either order or base")
    e = number.bit_length() - 1
    if order is not None:
        shape = [1 << (e // order + (1 if k < e % order else 0)) for k in range(order)]
    else:
        if base < 2 or base & (base - 1):
            raise ValueError("base must be a power of two")
        b = base.bit_length() - 1
        q, s = divmod(e, b)
        shape = [base] * q
        if q == 0 or 2 * s >= b:
            shape.append(1 << s)
        else:
            shape[0] <<= s
    return shape[::-1] if reverse else shape


def params_conv2d_cp4(in_channels, out_channels, kernel_size, rate=DEFAULT_COMPRESSION_RATE):
    """Rank of the four-factor CP conv: the rule of ``generate_params_conv2d_cp`` (test/layers.py:296-304) with the
    spatial factor counted as two separable vectors (2k parameters per rank instead of k*k)."""
    original = kernel_size * kernel_size * in_channels * out_channels
    unit = 2 * kernel_size + in_channels + out_channels
    return {"rank": int(math.ceil(rate * original / unit))}


def params_conv2d_cp(in_channels, out_channels, kernel_size, rate=DEFAULT_COMPRESSION_RATE):
    """``generate_params_conv2d_cp`` (test/layers.py:296-304): the three-factor CP conv, k*k + C + T parameters per rank."""
    original = kernel_size * kernel_size * in_channels * out_channels
    unit = kernel_size * kernel_size + in_channels + out_channels
    return {"rank": int(math.ceil(rate * original / unit))}


def params_conv2d_rcp(in_channels, out_channels, kernel_size, rate=DEFAULT_COMPRESSION_RATE, order=2):
    """``generate_params_conv2d_rcp`` (test/layers.py:816-851); the reference fixes ``order = 2``."""
    ishape = generate_shape(in_channels, order=order)
    oshape = generate_shape(out_channels, order=order)
    original = kernel_size ** 2 * in_channels * out_channels
    unit = (2 * kernel_size if kernel_size > 1 else 0) + sum(ishape) + sum(oshape)
    return {"input_shape": ishape, "output_shape": oshape, "rank": int(math.ceil(rate * original / unit))}


def params_dense_cp(in_features, out_features, rate=DEFAULT_COMPRESSION_RATE):
    """``generate_params_dense_cp`` (test/layers.py:491-507)."""
    ishape = generate_shape(in_features, base=DEFAULT_FACTORIZATION_BASE)
    if len(ishape) < 2:
        raise ValueError("in_features is too small to be factorized further")
    oshape = generate_shape(out_features, order=len(ishape), reverse=True)
    unit = sum(i * o for i, o in zip(ishape, oshape))
    return {"input_shape": ishape, "output_shape": oshape,
            "rank": int(math.ceil(in_features * out_features * rate / unit))}


class CP4Conv2d(nn.Module):
    """Rank-R CP4 conv2d, stride 1, same padding: ``K[t,c,y,x] = sum_r FT[t,r] FC[c,r] FY[y,r] FX[x,r]``
    (Cuda_kernels/Utils.cu:51-62) without ever forming ``K``."""

    def __init__(self, in_channels, out_channels, kernel_size=3, rank=None, rate=DEFAULT_COMPRESSION_RATE, bias=False,
                 flags=0):
        super().__init__()
        if kernel_size % 2 == 0:
            raise ValueError("same padding needs an odd kernel size")
        self.rank = rank or params_conv2d_cp4(in_channels, out_channels, kernel_size, rate)["rank"]
        self.pad, self.flags = (kernel_size - 1) // 2, flags
        # every factor gets the fourth root of the variance a dense filter of this fan-in would have per rank term
        std4 = (1.0 / (in_channels * kernel_size * kernel_size * self.rank)) ** 0.125
        mk = lambda d: nn.Parameter(torch.randn(d, self.rank) * std4)
        self.FT, self.FC, self.FY, self.FX = mk(out_channels), mk(in_channels), mk(kernel_size), mk(kernel_size)
        self.bias = nn.Parameter(torch.zeros(out_channels)) if bias else None

    def forward(self, x):
        from .ops import CP4Conv2dFunction
        y = CP4Conv2dFunction.apply(x.contiguous(), self.FT, self.FC, self.FY, self.FX, self.pad, self.flags)
        return y if self.bias is None else y + self.bias.view(1, -1, 1, 1)


class CPConv2d(nn.Module):
    """Three-factor CP conv2d, the layer ``conv2d_cp`` defines (test/layers.py:265-291): 1x1 conv C->R, per-rank k x k
    filter, 1x1 conv R->T, as one fused kernel; stride 1, same padding.  Training needs a 3x3 filter."""

    def __init__(self, in_channels, out_channels, kernel_size=3, rank=None, rate=DEFAULT_COMPRESSION_RATE, bias=False):
        super().__init__()
        if kernel_size % 2 == 0:
            raise ValueError("same padding needs an odd kernel size")
        self.rank = rank or params_conv2d_cp(in_channels, out_channels, kernel_size, rate)["rank"]
        self.pad = (kernel_size - 1) // 2
        std3 = (1.0 / (in_channels * kernel_size * kernel_size * self.rank)) ** (1.0 / 6.0)
        self.KT = nn.Parameter(torch.randn(out_channels, self.rank) * std3)
        self.KCin = nn.Parameter(torch.randn(in_channels, self.rank) * std3)
        self.KC = nn.Parameter(torch.randn(kernel_size, kernel_size, self.rank) * std3)
        self.bias = nn.Parameter(torch.zeros(out_channels)) if bias else None

    def forward(self, x):
        from .ops import CP3Conv2dFunction
        y = CP3Conv2dFunction.apply(x.contiguous(), self.KT, self.KCin, self.KC, self.pad)
        return y if self.bias is None else y + self.bias.view(1, -1, 1, 1)


class RCPConv2d(nn.Module):
    """Reshaped-CP conv2d (test/layers.py:687-789): channels factored into modes, one ``[c_k, t_k, R]`` factor per
    mode and a ``[k, k, R]`` spatial core; stride 1, same padding."""

    def __init__(self, in_channels, out_channels, kernel_size=3, rank=None, rate=DEFAULT_COMPRESSION_RATE,
                 input_shape=None, output_shape=None, bias=False):
        super().__init__()
        p = params_conv2d_rcp(in_channels, out_channels, kernel_size, rate)
        self.input_shape = list(input_shape or p["input_shape"])
        self.output_shape = list(output_shape or p["output_shape"])
        if math.prod(self.input_shape) != in_channels or math.prod(self.output_shape) != out_channels:
            raise ValueError("mode sizes must multiply to the channel counts")
        if len(self.input_shape) != len(self.output_shape):
            raise ValueError("input_shape and output_shape need the same number of modes")
        self.rank = rank or p["rank"]
        m = len(self.input_shape)
        std = (1.0 / (in_channels * kernel_size * kernel_size * self.rank)) ** (0.5 / (m + 1))
        self.factors = nn.ParameterList([nn.Parameter(torch.randn(c, t, self.rank) * std)
                                         for c, t in zip(self.input_shape, self.output_shape)])
        self.core = nn.Parameter(torch.randn(kernel_size, kernel_size, self.rank) * std)
        self.bias = nn.Parameter(torch.zeros(out_channels)) if bias else None

    def forward(self, x):
        from .ops import RCPConv2dFunction
        y = RCPConv2dFunction.apply(x.contiguous(), self.core, *self.factors)
        return y if self.bias is None else y + self.bias.view(1, -1, 1, 1)


class CPDense(nn.Module):
    """CP dense layer (test/layers.py:430-469): ``W[i, o] = sum_r prod_k F_k[i_k, o_k, r]`` without forming ``W``."""

    def __init__(self, in_features, out_features, rank=None, rate=DEFAULT_COMPRESSION_RATE, input_shape=None,
                 output_shape=None, bias=False):
        super().__init__()
        if input_shape is None or output_shape is None:
            p = params_dense_cp(in_features, out_features, rate)
            input_shape, output_shape = p["input_shape"], p["output_shape"]
            rank = rank or p["rank"]
        self.input_shape, self.output_shape = list(input_shape), list(output_shape)
        if math.prod(self.input_shape) != in_features or math.prod(self.output_shape) != out_features:
            raise ValueError("mode sizes must multiply to the feature counts")
        if rank is None:
            rank = params_dense_cp(in_features, out_features, rate)["rank"]
        self.rank = rank
        m = len(self.input_shape)
        std = (1.0 / (in_features * self.rank)) ** (0.5 / m)
        self.factors = nn.ParameterList([nn.Parameter(torch.randn(i, o, self.rank) * std)
                                         for i, o in zip(self.input_shape, self.output_shape)])
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None

    def forward(self, x):
        from .ops import CPDenseFunction
        lead = x.shape[:-1]
        y = CPDenseFunction.apply(x.reshape(-1, x.shape[-1]).contiguous(), *self.factors)
        y = y.reshape(*lead, -1)
        return y if self.bias is None else y + self.bias
