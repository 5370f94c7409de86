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


def bind_host_to_gpu(device=None):
    """Best effort: restrict this process to the CPUs of the NUMA node its GPU hangs off, so that the pinned host
    buffers it allocates afterwards (first touch) and the threads that fill them are local to the GPU's PCIe root.
    With one process per GPU on a two-socket host this keeps the host-to-device traffic of half the ranks off the
    socket interconnect.  Returns the node number, or None when it cannot be found (no sysfs, one node, no rights)."""
    import os
    try:
        dev = torch.cuda.current_device() if device is None else int(device)
        pr = torch.cuda.get_device_properties(dev)
        path = "/sys/bus/pci/devices/%04x:%02x:%02x.0/numa_node" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
        node = int(open(path).read().strip())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            a, _, b = part.partition("-")
            cpus.update(range(int(a), int(b or a) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception:
        return None


class P2PAllreduce:
    """The gradient allreduce as one small kernel over NVLink peer memory (``b200cp_p2p_*``), one process per GPU.

    Set-up (collective, outside the hot path): every rank allocates its exchange region, the 64-byte CUDA IPC
    handles go round with ``all_gather`` and every rank maps the others' regions.  ``__call__`` then sums a float32
    CUDA tensor over the ranks in place, asynchronously on the current stream; it can be captured in a CUDA graph.
    All ranks get bitwise the same sums (rows added in rank order)."""

    HANDLE_BYTES = 64

    def __init__(self, max_floats, group=None):
        import ctypes as C
        from . import _lib
        self._lib, self._C = _lib, C
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.max_floats = int(max_floats)
        handle = (C.c_ubyte * self.HANDLE_BYTES)()
        ctx = C.c_void_p()
        self._ctx = None
        err = None
        try:
            _lib.check(_lib.lib.b200cp_p2p_init(self.rank, self.world, self.max_floats, handle, C.byref(ctx)))
            self._ctx = ctx
        except Exception as e:          # keep taking part in the collectives below: all ranks fail together
            err = e
        if self.world > 1:
            backend = dist.get_backend(group)
            dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
            mine = torch.tensor(list(handle), dtype=torch.uint8, device=dev)
            every = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(every, mine, group=group)
            if err is None:
                try:
                    flat = bytes(torch.cat(every).cpu().tolist())
                    buf = (C.c_ubyte * len(flat)).from_buffer_copy(flat)
                    _lib.check(_lib.lib.b200cp_p2p_connect(self._ctx, buf))
                except Exception as e:
                    err = e
            # every rank has mapped its peers before anyone starts an exchange; a failure anywhere fails everywhere
            ok = torch.tensor([0 if err is not None else 1], dtype=torch.int32, device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok.item()) == 0:
                self.close()
                raise RuntimeError(f"peer-memory allreduce set-up failed on some rank (this rank: {err})")
        else:
            if err is not None:
                raise err
            _lib.check(_lib.lib.b200cp_p2p_connect(self._ctx, None))

    def __call__(self, t, out=None):
        out = t if out is None else out
        assert t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() and out.is_contiguous()
        assert out.numel() == t.numel() <= self.max_floats
        st = torch.cuda.current_stream().cuda_stream
        self._lib.check(self._lib.lib.b200cp_p2p_allreduce(self._ctx, t.data_ptr(), out.data_ptr(), t.numel(), st))
        return out

    def cp4_step(self, X, dU, K0, K1, KH, KW, pad=1, flags=0):
        """``b200cp_cp4_step_allreduce``: forward, backward-data and the factor gradients of this rank's shard with the
        packed gradients summed over the ranks; where the step runs as its fused kernel chain the exchange is the tail
        of the kernel that adds the partial gradients.  Returns (U, dX, dK_packed)."""
        C = self._C
        lib = self._lib.lib
        N, Cc, H, W = X.shape
        T, R = K0.shape
        s = self._lib.TensorShape(N=N, H=H, W=W, pad=pad, T=T, C=Cc, Y=KH.shape[0], X=KW.shape[0], Rank=R)
        U = torch.empty(N, T, H, W, device=X.device, dtype=torch.float32)
        dX = torch.empty_like(X)
        dK = torch.empty((T + Cc + KH.shape[0] + KW.shape[0]) * R, device=X.device, dtype=torch.float32)
        nb = lib.b200cp_cp4_step_workspace_bytes(C.byref(s), flags)
        ws = torch.empty(max(nb, 4) // 4, device=X.device, dtype=torch.float32)
        st = torch.cuda.current_stream().cuda_stream
        self._lib.check(lib.b200cp_cp4_step_allreduce(self._ctx, C.byref(s), X.data_ptr(), dU.data_ptr(), K0.data_ptr(),
                                                      K1.data_ptr(), KH.data_ptr(), KW.data_ptr(), U.data_ptr(),
                                                      dX.data_ptr(), dK.data_ptr(), ws.data_ptr(), nb, st, flags))
        return U, dX, dK

    def cp4_step_pipelined(self, X, dU, K0, K1, KH, KW, dK_prev, pad=1, flags=0):
        """``b200cp_cp4_step_allreduce_pipelined``: posts this step's gradients to the peers and completes the previous
        pipelined step's exchange into ``dK_prev`` (a float32 CUDA tensor of (T+C+Y+X)*R entries; untouched by the
        first call).  Returns (U, dX).  ``flush(dK_last)`` completes the last step's exchange."""
        C = self._C
        lib = self._lib.lib
        N, Cc, H, W = X.shape
        T, R = K0.shape
        s = self._lib.TensorShape(N=N, H=H, W=W, pad=pad, T=T, C=Cc, Y=KH.shape[0], X=KW.shape[0], Rank=R)
        U = torch.empty(N, T, H, W, device=X.device, dtype=torch.float32)
        dX = torch.empty_like(X)
        scratch = torch.empty((T + Cc + KH.shape[0] + KW.shape[0]) * R, device=X.device, dtype=torch.float32)
        assert dK_prev.is_cuda and dK_prev.dtype == torch.float32 and dK_prev.numel() == scratch.numel()
        nb = lib.b200cp_cp4_step_workspace_bytes(C.byref(s), flags)
        ws = torch.empty(max(nb, 4) // 4, device=X.device, dtype=torch.float32)
        st = torch.cuda.current_stream().cuda_stream
        self._lib.check(lib.b200cp_cp4_step_allreduce_pipelined(
            self._ctx, C.byref(s), X.data_ptr(), dU.data_ptr(), K0.data_ptr(), K1.data_ptr(), KH.data_ptr(), KW.data_ptr(),
            U.data_ptr(), dX.data_ptr(), scratch.data_ptr(), dK_prev.data_ptr(), ws.data_ptr(), nb, st, flags))
        return U, dX

    def flush(self, dK_last):
        """Completes the last posted pipelined exchange into ``dK_last`` (nothing happens when none is pending)."""
        st = torch.cuda.current_stream().cuda_stream
        self._lib.check(self._lib.lib.b200cp_p2p_flush(self._ctx, dK_last.data_ptr(), st))
        return dK_last

    def status(self):
        """Synchronises the device; raises if a wait for a peer's flag ran out."""
        self._lib.check(self._lib.lib.b200cp_p2p_status(self._ctx))

    def close(self):
        if self._ctx is not None:
            self._lib.lib.b200cp_p2p_destroy(self._ctx)
            self._ctx = None


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


def _pack(ts):
    return torch.cat([t.reshape(-1) for t in ts])


def _unpack(packed, like):
    out, o = [], 0
    for t in like:
        out.append(packed[o:o + t.numel()].view_as(t))
        o += t.numel()
    return out


def rcp_data_parallel_step(X, dV, A, S, allreduce=None, group=None):
    """Reshaped-CP conv on this rank's batch shard: forward, data gradient and factor gradients, then ONE allreduce of
    the packed factor gradients ``[dA_1 | ... | dA_m | dS]`` (sum_k c_k t_k R + FH FW R floats).  ``allreduce`` is a
    callable on the packed buffer (e.g. a ``P2PAllreduce``); default: ``allreduce_factor_grads``.
    Returns (V, dX, [dA_k], dS) with the gradients summed over all ranks."""
    from . import ops
    V = ops.conv2d_rcp_fused_nchw(X, *A, S)
    dX, dA, dS = ops.rcp_conv2d_backward(X, dV, *A, S)
    packed = _pack(list(dA) + [dS])
    (allreduce or (lambda t: allreduce_factor_grads(t, group)))(packed)
    *dA, dS = _unpack(packed, list(dA) + [dS])
    return V, dX, dA, dS


def dense_data_parallel_step(X, dY, F, allreduce=None, group=None):
    """CP dense layer on this rank's batch shard: forward, data gradient and factor gradients, then ONE allreduce of
    the packed factor gradients (sum_k i_k o_k R floats: 8 192 at 8^4 -> 8^4, R = 32).
    Returns (Y, dX, [dF_k]) with the gradients summed over all ranks."""
    from . import ops
    Y = ops.dense_cp(X, *F)
    dX, dF = ops.dense_cp_backward(X, dY, *F)
    packed = _pack(dF)
    (allreduce or (lambda t: allreduce_factor_grads(t, group)))(packed)
    return Y, dX, _unpack(packed, dF)
