"""Batch-sharded data parallelism for the CP layers: one process per GPU.

Forward and backward-data are independent per image, so ranks never talk during them.  The factor
gradients are sums over the batch: each rank reduces its own shard on its GPU and the packed
buffers ``[dK0 | dK1 | dKH | dKW]`` are added with ONE allreduce (NCCL over NVLink on GPUs; gloo in
the CPU tests).  The reference itself is single-GPU (``cudaSetDevice``, Cuda_kernels/cp4Conv2d.cu:210).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_batch(n, rank, world):
    """Contiguous slice [start, start + count) of a batch of n for `rank` of `world`; NCHW makes a
    slice of images one contiguous range of memory.  The first n % world ranks get one image more."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    base, extra = divmod(n, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def allreduce_factor_grads(packed, group=None):
    """Sum the packed factor-gradient buffer over all ranks, in place, on the current stream."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
    return packed


def cp4_data_parallel_step(X, dU, FT, FC, FY, FX, pad=1, flags=0, group=None):
    """forward, backward-data and backward-filter on this rank's shard, then the gradient allreduce.
    Returns (U, dX, (dFT, dFC, dFY, dFX)) with the gradients summed over every rank's shard."""
    from . import ops
    U = ops.cp4_conv2d_forward(X, FT, FC, FY, FX, pad, flags)
    dX = ops.cp4_conv2d_backward_data(dU, FT, FC, FY, FX, pad, flags)
    packed = ops.cp4_conv2d_backward_filter(dU, X, FT, FC, FY, FX, pad, packed=True)
    allreduce_factor_grads(packed, group)
    R = FT.shape[1]
    sizes = [FT.shape[0] * R, FC.shape[0] * R, FY.shape[0] * R, FX.shape[0] * R]
    parts = torch.split(packed, sizes)
    grads = tuple(p.view(-1, R) for p in parts)
    return U, dX, grads
