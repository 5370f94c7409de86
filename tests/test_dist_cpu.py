"""Host-side logic of the data-parallel path with 2 gloo ranks on CPU: contiguous batch shards, one allreduce of
the packed factor gradients, every rank ending with the full-batch gradient.  (The per-shard gradients come from
the CPU oracle here; on GPUs they come from the kernels -- tests/test_cp4_gpu.py.)"""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import cp_oracle as O
from paralleltnnlayers_b200 import dist as D


def test_shard_batch_partitions_the_batch():
    for n in (1, 7, 32, 33):
        for world in (1, 2, 3, 8):
            got = []
            for r in range(world):
                s, c = D.shard_batch(n, r, world)
                got += list(range(s, s + c))
            assert got == list(range(n))
    try:
        D.shard_batch(4, 2, 2)
        assert False
    except ValueError:
        pass


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        N = 5
        X, K0, K1, KH, KW, dU = O.make_cp4_inputs(77, N, 3, 4, 6, 5, 3, 3, 2, factor_std=0.5)
        s, c = D.shard_batch(N, rank, world)
        g = O.cp4_backward_filter(X[s:s + c], dU[s:s + c], K0, K1, KH, KW, 1)
        packed = torch.from_numpy(np.concatenate([a.ravel() for a in g]))
        D.allreduce_factor_grads(packed)
        full = np.concatenate([a.ravel() for a in O.cp4_backward_filter(X, dU, K0, K1, KH, KW, 1)])
        q.put((rank, float(np.abs(packed.numpy() - full).max())))
    finally:
        dist.destroy_process_group()


def test_two_ranks_reduce_to_the_full_batch_gradient():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r for r, _ in res) == [0, 1]
    assert all(e < 1e-10 for _, e in res)


def _worker_layers(rank, world, port, q):
    """The packed-gradient helpers of the reshaped-CP and dense layers: pack, one allreduce, unpack."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        errs = []
        # dense: per-shard oracle gradients, packed like dense_data_parallel_step packs them
        B = 6
        X, F, dY = O.make_dense_inputs(3, B, (2, 3), (3, 2), 4)
        s, c = D.shard_batch(B, rank, world)
        _, dF = O.dense_cp_backward(X[s:s + c], dY[s:s + c], F)
        like = [torch.from_numpy(np.ascontiguousarray(a)) for a in dF]
        packed = D._pack(like)
        D.allreduce_factor_grads(packed)
        _, full = O.dense_cp_backward(X, dY, F)
        for a, b in zip(D._unpack(packed, like), full):
            errs.append(float(np.abs(a.numpy() - b).max()))
        # reshaped-CP conv
        N = 4
        Xr, A, S, dV = O.make_rcp_inputs(4, N, (2, 2), (2, 3), 5, 4, 3, 3, 3)
        s, c = D.shard_batch(N, rank, world)
        _, dA, dS = O.rcp_backward(Xr[s:s + c], dV[s:s + c], A, S)
        like = [torch.from_numpy(np.ascontiguousarray(a)) for a in list(dA) + [dS]]
        packed = D._pack(like)
        assert packed.numel() == sum(a.size for a in A) + S.size
        D.allreduce_factor_grads(packed)
        _, fA, fS = O.rcp_backward(Xr, dV, A, S)
        for a, b in zip(D._unpack(packed, like), list(fA) + [fS]):
            errs.append(float(np.abs(a.numpy() - b).max()))
        q.put((rank, max(errs)))
    finally:
        dist.destroy_process_group()


def test_two_ranks_reduce_the_dense_and_rcp_gradients():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker_layers, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(e < 1e-9 for _, e in res), res
