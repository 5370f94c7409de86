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
    ar.status()
    q.put((rank, bool(ok)))
    torch.cuda.synchronize()
    dist.barrier()
    ar.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_match_nccl():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world = 2
    procs = [ctx.Process(target=_worker, args=(r, world, 29533, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert all(ok for _, ok in res), res
