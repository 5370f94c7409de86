"""The peer-memory allreduce of the packed factor gradients (b200cp_p2p_*).

One GPU: a single rank exchanges with itself, which runs the whole kernel (stores, flags, the bounded wait, the
sum) and the slot / sequence logic over many launches and CUDA-graph replays.  Two or more GPUs: one process per
GPU compares it with the NCCL allreduce."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_single_rank_exchange_and_graph_replay():
    from paralleltnnlayers_b200.dist import P2PAllreduce
    ar = P2PAllreduce(5000)
    for n in (1, 3, 2144, 5000):
        v = torch.randn(n, device="cuda")
        out = torch.empty_like(v)
        ar(v, out)
        assert torch.equal(out, v)
    v = torch.randn(2144, device="cuda")
    w = v.clone()
    ar(w)                               # in place
    assert torch.equal(w, v)
    # captured: the sequence number lives on the device, so replays keep alternating the slots
    src, dst = torch.randn(2144, device="cuda"), torch.zeros(2144, device="cuda")
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for _ in range(3):
                ar(src, dst)
        for _ in range(4):
            src.normal_()
            g.replay()
            torch.cuda.synchronize()
            assert torch.equal(dst, src)
    ar.status()
    with pytest.raises(Exception):
        ar(torch.zeros(5001, device="cuda"))
    ar.close()


def test_single_rank_step_with_the_exchange_fused_into_the_gradient_reduction():
    """``b200cp_cp4_step_allreduce`` with one rank: the reduction kernel's exchange tail runs against itself (stores,
    flags, wait, sum, sequence numbers over repeated calls and graph replays) and must give the plain step's bits;
    a shape outside the fused kernel chain takes the stand-alone exchange kernel after the step."""
    import paralleltnnlayers_b200 as P
    from oracle import cp_oracle as O
    from paralleltnnlayers_b200.dist import P2PAllreduce
    from tests.gpu_util import dev
    for shape in ((3, 64, 64, 56, 56, 16), (2, 16, 24, 9, 24, 5), (2, 12, 20, 7, 10, 3)):    # the last: not a fused shape
        N, Cc, T, H, W, R = shape
        X, K0, K1, KH, KW, dU = O.make_cp4_inputs(900 + H, N, Cc, T, H, W, 3, 3, R, factor_std=0.1)
        t = dev(X, K0, K1, KH, KW, dU)
        ar = P2PAllreduce((T + Cc + 6) * R)
        ref = P.cp4_conv2d_step(t[0], t[5], *t[1:5], 1)
        for _ in range(3):
            got = ar.cp4_step(t[0], t[5], *t[1:5], 1)
            for a, b in zip(got, ref):
                assert torch.equal(a, b)
        # pipelined: the gradients of a call arrive with the next call, the last ones with flush()
        ref2 = P.cp4_conv2d_step(t[0], 2 * t[5], *t[1:5], 1)
        prev = [torch.full_like(ref[2], 7.0) for _ in range(3)]
        U0, dX0 = ar.cp4_step_pipelined(t[0], t[5], *t[1:5], prev[0], 1)
        U1, dX1 = ar.cp4_step_pipelined(t[0], 2 * t[5], *t[1:5], prev[1], 1)
        with pytest.raises(Exception):
            ar.cp4_step(t[0], t[5], *t[1:5], 1)            # an exchange is pending: the unpipelined call is refused
        ar.flush(prev[2])
        ar.flush(prev[2])                                   # nothing pending: a no-op
        assert torch.equal(U0, ref[0]) and torch.equal(dX0, ref[1]) and torch.equal(dX1, ref2[1])
        assert torch.all(prev[0] == 7.0)                    # the first call had nothing to complete
        assert torch.equal(prev[1], ref[2]) and torch.equal(prev[2], ref2[2])
        got = ar.cp4_step(t[0], t[5], *t[1:5], 1)          # and the context is free again
        assert torch.equal(got[2], ref[2])
        ar.status()
        ar.close()


def test_a_wait_that_runs_out_is_reported_and_the_exchange_recovers():
    """Two ranks of one process on one GPU, driven one after the other with a wait limit of about a millisecond.
    The rank launched first stores its vector and raises its flags, finds its peer's flag missing, gives up within
    the limit (the kernel returns by itself: nothing is trapped or left spinning), fills its result with NaN and
    records the time-out; the rank launched second finds the first one's data in place and gets the correct sum.
    The next exchange, in the opposite order, behaves the same way: the contexts stay usable."""
    import ctypes as C
    import paralleltnnlayers_b200 as P
    lib = P._lib.lib
    n = 777
    ctxs = []
    handle = (C.c_ubyte * 64)()
    for r in range(2):
        c = C.c_void_p()
        P._lib.check(lib.b200cp_p2p_init(r, 2, 1024, handle, C.byref(c)))
        ctxs.append(c)
    arr = (C.c_void_p * 2)(*[c.value for c in ctxs])
    for c in ctxs:
        P._lib.check(lib.b200cp_test_p2p_connect_local(c, arr))
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    lib.b200cp_test_set_p2p_wait_cycles(2_000_000)          # about a millisecond
    try:
        for order in ((1, 0), (0, 1)):
            v = [torch.randn(n, device="cuda") for _ in range(2)]
            out = [torch.zeros(n, device="cuda") for _ in range(2)]
            first, second = order
            P._lib.check(lib.b200cp_p2p_allreduce(ctxs[first], v[first].data_ptr(), out[first].data_ptr(), n, st))
            torch.cuda.synchronize()                          # the kernel came back by itself
            assert lib.b200cp_p2p_status(ctxs[first]) == -5   # B200CP_ERR_TIMEOUT
            assert b"waited in vain" in lib.b200cp_last_error_string()
            assert torch.isnan(out[first]).all()              # a missed exchange cannot pass for a sum
            P._lib.check(lib.b200cp_p2p_allreduce(ctxs[second], v[second].data_ptr(), out[second].data_ptr(), n, st))
            torch.cuda.synchronize()
            P._lib.check(lib.b200cp_p2p_status(ctxs[second]))
            assert torch.equal(out[second], v[0] + v[1])
            assert lib.b200cp_p2p_status(ctxs[first]) == 0    # the record was cleared when it was read
    finally:
        lib.b200cp_test_set_p2p_wait_cycles(0)
        for c in ctxs:
            lib.b200cp_p2p_destroy(c)


def _worker_free_running(rank, world, port, q):
    """A few hundred exchanges with nothing between them -- eager, then as a replayed CUDA graph -- so that a rank
    can run ahead of its peer by the one exchange the two slots allow.  Inputs with sums known in closed form."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from paralleltnnlayers_b200.dist import P2PAllreduce
    n = 2144
    ar = P2PAllreduce(n)
    base = torch.arange(n, device="cuda", dtype=torch.float32)
    ok = True
    src = torch.empty(n, device="cuda")
    outs = [torch.empty(n, device="cuda") for _ in range(300)]
    for it in range(300):                                  # eager, no collective in between
        src.copy_(base * (rank + 1) + it)
        ar(src, outs[it])
    torch.cuda.synchronize()
    tri = world * (world + 1) // 2
    for it in range(300):
        ok = ok and torch.equal(outs[it], base * tri + world * it)
    # a captured sequence, replayed: every replay advances the device-side sequence numbers by its 50 exchanges
    step = torch.zeros(1, device="cuda")
    acc = torch.zeros(n, device="cuda")
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for _ in range(50):
                src.copy_(base * (rank + 1) + step)
                ar(src, outs[0])
                acc.add_(outs[0])
                step.add_(1)
        for _ in range(4):
            g.replay()
        torch.cuda.synchronize()
    k = 200
    ok = ok and torch.allclose(acc, base * tri * k + world * (k * (k - 1) / 2), rtol=1e-6, atol=1e-3)
    ar.status()
    q.put((rank, bool(ok)))
    torch.cuda.synchronize()
    dist.barrier()
    ar.close()
    dist.destroy_process_group()


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from paralleltnnlayers_b200.dist import P2PAllreduce
    ar = P2PAllreduce(4096)
    ok = True
    for it in range(20):
        torch.manual_seed(100 * it + rank)
        v = torch.randn(2144 if it % 2 else 4096, device="cuda")
        want = v.clone()
        dist.all_reduce(want)
        got = ar(v.clone())
        ok = ok and torch.allclose(got, want, rtol=1e-5, atol=1e-6)
        every = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(every, got)
        ok = ok and all(torch.equal(e, every[0]) for e in every)     # bitwise the same on every rank
    # the exchange fused into the gradient reduction of a training step against the plain step + NCCL
    import paralleltnnlayers_b200 as P
    g = torch.Generator(device="cuda").manual_seed(7 + rank)
    X = torch.rand(4, 64, 56, 56, device="cuda", generator=g) * 2 - 1
    dU = torch.randn(4, 64, 56, 56, device="cuda", generator=g)
    f = torch.Generator(device="cuda").manual_seed(5)                  # the factors are the same on every rank
    K0, K1 = torch.randn(64, 16, device="cuda", generator=f) / 24, torch.randn(64, 16, device="cuda", generator=f) / 24
    KH, KW = torch.randn(3, 16, device="cuda", generator=f) / 3, torch.randn(3, 16, device="cuda", generator=f) / 3
    ar2 = P2PAllreduce((64 + 64 + 6) * 16)
    for _ in range(5):
        U, dX, dK = ar2.cp4_step(X, dU, K0, K1, KH, KW, 1)
        U1, dX1, dK1 = P.cp4_conv2d_step(X, dU, K0, K1, KH, KW, 1)
        dist.all_reduce(dK1)
        ok = ok and torch.equal(U, U1) and torch.equal(dX, dX1)
        ok = ok and torch.allclose(dK, dK1, rtol=1e-5, atol=1e-6 * float(dK1.abs().max()))
        every = [torch.empty_like(dK) for _ in range(world)]
        dist.all_gather(every, dK)
        ok = ok and all(torch.equal(e, every[0]) for e in every)
    prev = [torch.zeros_like(dK1) for _ in range(4)]
    for k in range(3):
        ar2.cp4_step_pipelined(X, (k + 1) * dU, K0, K1, KH, KW, prev[k], 1)
    ar2.flush(prev[3])
    for k in range(3):
        want = P.cp4_conv2d_step(X, (k + 1) * dU, K0, K1, KH, KW, 1)[2]
        dist.all_reduce(want)
        ok = ok and torch.allclose(prev[k + 1], want, rtol=1e-5, atol=1e-6 * float(want.abs().max()))
    ar2.status()
    ar.status()
    q.put((rank, bool(ok)))
    torch.cuda.synchronize()
    dist.barrier()
    ar2.close()
    ar.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("worker,port", [(_worker, 29533), (_worker_free_running, 29534)], ids=["vs_nccl", "free_running"])
def test_two_ranks_match_nccl(worker, port):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world = 2
    procs = [ctx.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert all(ok for _, ok in res), res
