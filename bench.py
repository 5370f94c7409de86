#!/usr/bin/env python
"""CP4 conv2d forward + backward-data + backward-filter throughput (images/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: the configuration the headline metric is quoted on -- N=32 images per GPU,
C=T=64, 56x56, 3x3 filter, rank 16, same padding, fp32, seeded synthetic inputs.
One step = forward, backward-data and backward-filter over one batch (plus the allreduce
of the packed factor gradients when more than one GPU runs).  Batches are sharded across
ranks (weak scaling: every rank owns N=32 images).

Timing: the K steps are captured once as a CUDA graph and replayed REPLAYS times inside the timed
region (a barrier + synchronize on both sides); every replay has its own pair of CUDA events on the
launching stream and the reported time per step is the median replay (maximum over ranks).  Every
step uses the next of several distinct buffer sets so that a set is evicted from L2 before it is
used again.  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(N=32, C=64, T=64, H=56, W=56, F=3, R=16, pad=1)
WORKLOAD = "cp4_conv2d fwd+bwd_data+bwd_filter N=32/GPU C=T=64 56x56 3x3 R=16 same-pad fp32"
METRIC = "CP4 conv fwd+bwd images/sec"
FALLBACK_HBM_GBS = 6650.0
REPLAYS = 10          # replays of the K-step graph inside the timed region; the median is reported


def make_inputs(seed, n):
    from oracle.cp_oracle import make_cp4_inputs  # seeded generator shared with the tests
    return make_cp4_inputs(seed, n, CFG["C"], CFG["T"], CFG["H"], CFG["W"], CFG["F"], CFG["F"], CFG["R"])


def synth_inputs(seed, n):
    """Same distributions as the test generator, without importing the oracle (used by the GPU arm)."""
    rng = np.random.default_rng(seed)
    c = CFG
    std = 1.0 / np.sqrt(c["C"] * c["F"] * c["F"])
    X = rng.uniform(-1, 1, size=(n, c["C"], c["H"], c["W"])).astype(np.float32)
    K0 = rng.normal(0, std, size=(c["T"], c["R"])).astype(np.float32)
    K1 = rng.normal(0, std, size=(c["C"], c["R"])).astype(np.float32)
    KH = rng.normal(0, std, size=(c["F"], c["R"])).astype(np.float32)
    KW = rng.normal(0, std, size=(c["F"], c["R"])).astype(np.float32)
    dU = rng.normal(0, 1, size=(n, c["T"], c["H"], c["W"])).astype(np.float32)
    return X, K0, K1, KH, KW, dU


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled during the timed region."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for nm, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def cpu_step_fn(n):
    """The reference's CPU path: its unfused CP-layer composition (test/layers.py:265-283) restated for
    torch-CPU, forward + autograd backward, on all host threads."""
    from oracle import cpu_composition as CC
    X, K0, K1, KH, KW, dU = [torch.from_numpy(a) for a in make_inputs(1, n)]

    def step():
        CC.cp4_step(X, K0, K1, KH, KW, dU, CFG["pad"])
    return step


def time_cpu(n, steps, warmup, budget_s):
    step = cpu_step_fn(n)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    done = 0
    while done < steps and (time.perf_counter() - t0 < budget_s or done == 0):
        step()
        done += 1
    dt = (time.perf_counter() - t0) / done
    return n / dt, dt, done


def run_reference(args, rank, world):
    """--impl reference: the reference's CPU path on this box's host cores (rank 0 only)."""
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    n = CFG["N"]
    ips, dt, done = time_cpu(n, args.steps, args.warmup, budget_s=120.0)
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": ips, "unit": "images/s", "n_gpus": args.gpus,
        "steps": done, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded; X~U[-1,1], factors~N(0,1/sqrt(9C)), dU~N(0,1))",
        "config": {"workload": WORKLOAD, "images_per_step": n},
        "cpu_baseline": {"value": ips, "unit": "images/s", "cores": cores, "kind": "port",
                         "sample": f"{done} full steps of N={n} (torch-CPU restatement of the unfused composition)"},
        "e2e": {"value": ips, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def graph_time_us(fn, reps, replays=3):
    """fn(i) launched `reps` times inside one CUDA graph; microseconds per call, best of `replays` replays."""
    for i in range(2):
        fn(i)
    torch.cuda.synchronize()
    st = torch.cuda.Stream()
    best = float("inf")
    with torch.cuda.stream(st):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for i in range(reps):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        for _ in range(replays):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            g.replay()
            e1.record(st)
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) / reps * 1e3)
        del g
    return best


def extra_configs(P, world, rank, reduce_fn, max_over_ranks):
    """Step times of the other benchmark configurations at a FIXED global batch (strong scaling: every rank owns
    1 / world of it), each step followed by the allreduce of its packed factor gradients on the same stream:
    config 3 at (C=T=128, 28x28, R=16) and (C=T=512, 7x7, R=64), global N = 64; config 5, global batch 4096."""
    out = {"scaling": "strong", "world": world}
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()
    for (C, H, R, seed) in ((128, 28, 16, 3), (512, 7, 64, 13)):
        n = max(1, 64 // world)
        rng = np.random.default_rng(seed * 100 + rank)
        std = 1.0 / np.sqrt(9 * C)
        K = [dev(rng.normal(0, std, size=(d, R))) for d in (C, C, 3, 3)]
        nsets = int(min(12, max(2, 300e6 // (4 * n * C * H * H * 4) + 1)))
        Xs = [dev(rng.uniform(-1, 1, size=(n, C, H, H))) for _ in range(nsets)]
        dUs = [dev(rng.normal(0, 1, size=(n, C, H, H))) for _ in range(nsets)]

        def step(i):
            U, dX, dK = P.cp4_conv2d_step(Xs[i % nsets], dUs[i % nsets], *K, 1)
            reduce_fn(dK)
        us = max_over_ranks(graph_time_us(step, 12))
        key = f"cfg3_C{C}_{H}x{H}_R{R}"
        out[key] = {"images_per_rank": n, "step_us": us, "images_per_s": world * n / (us * 1e-6),
                    "grad_floats": (2 * C + 6) * R}
        del Xs, dUs
        torch.cuda.empty_cache()
    B = max(1, 4096 // world)
    rng = np.random.default_rng(3000 + rank)
    F = [dev(rng.normal(0, 0.35, size=(8, 8, 32))) for _ in range(4)]
    Xs = [dev(rng.normal(0, 1, size=(B, 4096))) for _ in range(3)]
    dYs = [dev(rng.normal(0, 1, size=(B, 4096))) for _ in range(3)]

    def dstep(i):
        Y = P.dense_cp(Xs[i % 3], *F)
        dX, dF = P.dense_cp_backward(Xs[i % 3], dYs[i % 3], *F)
        reduce_fn(torch.cat([g.reshape(-1) for g in dF]))
    us = max_over_ranks(graph_time_us(dstep, 4))
    out["cfg5_dense_8x8x8x8_R32"] = {"samples_per_rank": B, "step_us": us, "samples_per_s": world * B / (us * 1e-6),
                                    "grad_floats": 4 * 8 * 8 * 32}
    return out


def reference_gpu_forward_us():
    """The reference's own forward kernel (compiled unmodified for this GPU by oracle/build_ref.py) timed by its own
    PROFCOUNT loop (47 launches, Cuda_kernels/cp4Conv2dForward.cu:245-327; bench/BenchBothTime.cu:90) at config 1 and
    config 2.  Forward only; part of the CPU-baseline leg: it is the checker's code, not the product's."""
    try:
        from oracle import cp_oracle as O
        from oracle import reference_cuda as RC
        if not RC.available():
            return {"unavailable": "oracle/_ref is not built"}
        out = {}
        for name, (seed, N, C, T, H, R, std) in {"config1": (0, 1, 16, 16, 32, 8, 0.5), "config2": (1, 32, 64, 64, 56, 16, None)}.items():
            X, K0, K1, KH, KW, _ = O.make_cp4_inputs(seed, N, C, T, H, H, 3, 3, R, factor_std=std)
            out[name] = RC.forward_time(X, K0, K1, KH, KW, 1, 47)
        return out
    except Exception as e:     # the baseline leg never takes the product's numbers down with it
        return {"unavailable": str(e)[:200]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--path", default="auto", choices=["auto", "simt", "tc3x", "mma"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the step times of the other configurations")
    ap.add_argument("--allreduce", default="p2p", choices=["p2p", "nccl"],
                    help="gradient allreduce of the multi-GPU step: the library's peer-memory kernel, or NCCL")
    ap.add_argument("--exchange", default="fused", choices=["pipelined", "fused", "inline", "overlap"],
                    help="N > 1: the allreduce of the factor gradients as the tail of the step's gradient reduction "
                         "kernel, completed by the next step's (pipelined: b200cp_cp4_step_allreduce_pipelined, the "
                         "last one by b200cp_p2p_flush inside the timed region) or by the same kernel (fused: "
                         "b200cp_cp4_step_allreduce) -- both need --allreduce p2p; as its own kernel on the step's "
                         "stream (inline), or on a communication stream overlapped with the next step (overlap)")
    ap.add_argument("--separate", action="store_true",
                    help="step = the three entry points one after the other instead of b200cp_cp4_step")
    ap.add_argument("--watchdog", type=int, default=420, help="seconds after which a stuck run dumps its stacks and exits")
    args = ap.parse_args()
    import faulthandler
    faulthandler.dump_traceback_later(args.watchdog, exit=True)
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import paralleltnnlayers_b200 as P   # raises if libb200cp.so is missing: there is no fallback
    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(local)
    # one process per GPU: keep this rank's host threads and the pinned buffers it allocates on the GPU's NUMA node
    from paralleltnnlayers_b200.dist import bind_host_to_gpu
    numa_node = bind_host_to_gpu(local) if world > 1 else None
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    flags = {"auto": P.PATH_AUTO, "simt": P.PATH_SIMT, "tc3x": P.PATH_TC3X, "mma": P.PATH_MMA}[args.path]
    flags_f = P.PATH_AUTO if flags == P.PATH_TC3X else flags   # the factor-gradient kernel has no forced tensor path

    c = CFG
    n = c["N"]
    HW = c["H"] * c["W"]
    X, K0, K1, KH, KW, dU = synth_inputs(1000 + rank, n)
    fac = [torch.from_numpy(a).cuda() for a in (K0, K1, KH, KW)]
    # distinct buffer sets: (X, dU, U, dX) = 4 * 25.7 MB each; 6 sets = 617 MB >> 126 MB of L2
    NSETS = 6
    Xd, dUd = torch.from_numpy(X).cuda(), torch.from_numpy(dU).cuda()
    sets = []
    for i in range(NSETS):
        sets.append((Xd.clone() if i else Xd, dUd.clone() if i else dUd,
                     torch.empty((n, c["T"], c["H"], c["W"]), device="cuda"),
                     torch.empty((n, c["C"], c["H"], c["W"]), device="cuda")))
    nK = (c["T"] + c["C"] + 2 * c["F"]) * c["R"]
    dK = torch.empty(nK, device="cuda")
    import ctypes as C
    s = P.tensor_shape(n, c["C"], c["H"], c["W"], c["T"], c["F"], c["F"], c["R"], c["pad"])
    lib = P._lib.lib
    wsb = lib.b200cp_cp4_bwd_filter_workspace_bytes(C.byref(s), flags_f)
    ws = torch.empty(wsb // 4, device="cuda")
    ptr = lambda t: C.c_void_p(t.data_ptr())
    fp = [ptr(f) for f in fac]

    def cur_stream():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def k_fwd(i, st):
        x, du, u, dx = sets[i % NSETS]
        P._lib.check(lib.b200cp_cp4_fwd(C.byref(s), ptr(x), *fp, ptr(u), st, flags))

    def k_bwdd(i, st):
        x, du, u, dx = sets[i % NSETS]
        P._lib.check(lib.b200cp_cp4_bwd_data(C.byref(s), ptr(du), *fp, ptr(dx), st, flags))

    def k_bwdf(i, st):
        x, du, u, dx = sets[i % NSETS]
        P._lib.check(lib.b200cp_cp4_bwd_filter(C.byref(s), ptr(x), ptr(du), *fp, ptr(dK), ptr(ws), wsb, st, flags_f))

    # b200cp_cp4_step: the same three results from one call; the two convolutions leave their rank planes in the
    # workspace and the factor gradients start from those (3x3 filters on the default path)
    shared = not args.separate and args.path in ("auto", "mma")
    wsb_step = lib.b200cp_cp4_step_workspace_bytes(C.byref(s), flags)
    ws_step = torch.empty(max(wsb_step, 4) // 4, device="cuda")
    plane_floats = n * c["R"] * HW
    Pp, Qp = ws_step[:plane_floats], ws_step[plane_floats + 64:2 * plane_floats + 64]   # scratch for the per-kernel runs
    wsb_sv = lib.b200cp_cp4_bwd_filter_saved_workspace_bytes(C.byref(s), flags) if shared else 0
    ws_sv = torch.empty(max(wsb_sv, 4) // 4, device="cuda")

    def k_fwd_save(i, st):
        x, du, u, dx = sets[i % NSETS]
        P._lib.check(lib.b200cp_cp4_fwd_save(C.byref(s), ptr(x), *fp, ptr(u), ptr(Pp), st, flags))

    def k_bwdd_save(i, st):
        x, du, u, dx = sets[i % NSETS]
        P._lib.check(lib.b200cp_cp4_bwd_data_save(C.byref(s), ptr(du), *fp, ptr(dx), ptr(Qp), st, flags))

    def k_convs_save(i, st):
        # the first launch of the timed step: forward and backward-data in one launch, both rank planes saved
        x, du, u, dx = sets[i % NSETS]
        P._lib.check(lib.b200cp_cp4_fwd_bwd_data(C.byref(s), ptr(x), ptr(du), *fp, ptr(u), ptr(dx), ptr(Pp), ptr(Qp), st, flags))

    def k_bwdf_saved(i, st):
        x, du, u, dx = sets[i % NSETS]
        P._lib.check(lib.b200cp_cp4_bwd_filter_saved(C.byref(s), ptr(x), ptr(du), ptr(Pp), ptr(Qp), fp[2], fp[3], ptr(dK),
                                                     ptr(ws_sv), wsb_sv, st, flags))

    # Data parallel: the allreduce of step i's packed gradients runs on a communication stream while step i+1
    # computes (two gradient buffers; a buffer is reused only after its allreduce has finished); every allreduce is
    # joined back before the timed region ends.
    dKs = [dK, torch.empty_like(dK)] if dist is not None else [dK]
    comm = torch.cuda.Stream() if dist is not None else None
    ar_done = [None, None]
    p2p = None
    if dist is not None and args.allreduce == "p2p":
        # the library's own exchange kernel over NVLink peer memory; checked once against NCCL before it is used
        from paralleltnnlayers_b200.dist import P2PAllreduce
        try:
            p2p = P2PAllreduce(dK.numel())          # fails on all ranks together or on none
        except Exception as e:
            sys.stderr.write(f"[bench] peer-memory allreduce unavailable ({e}); using NCCL\n")
            p2p = None
        if p2p is not None:
            probe = torch.randn(dK.numel(), device="cuda")
            want = probe.clone()
            dist.all_reduce(want)
            good = 1
            try:
                got = p2p(probe.clone())
                p2p.status()
                good = int(torch.allclose(got, want, rtol=1e-5, atol=1e-6))
            except Exception as e:
                sys.stderr.write(f"[bench] peer-memory allreduce failed its check ({e})\n")
                good = 0
            flag = torch.tensor([good], device="cuda", dtype=torch.int32)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag.item()) == 0:               # all ranks take the same decision
                sys.stderr.write("[bench] peer-memory allreduce disagrees with NCCL on some rank; using NCCL\n")
                p2p = None

    fused_exchange = p2p is not None and shared and args.exchange in ("fused", "pipelined")
    pipelined = fused_exchange and args.exchange == "pipelined"
    if dist is not None and args.exchange in ("fused", "pipelined") and not fused_exchange:
        args.exchange = "inline"                    # NCCL, or a path without the fused kernel chain
    dk_scratch = torch.empty_like(dK) if pipelined else None

    def step(i, st):
        dk = dKs[i % len(dKs)]
        if dist is not None and ar_done[i % 2] is not None:
            torch.cuda.current_stream().wait_event(ar_done[i % 2])
        if shared and pipelined:
            # step i posts its gradients and completes step i-1's exchange into the other gradient buffer
            x, du, u, dx = sets[i % NSETS]
            P._lib.check(lib.b200cp_cp4_step_allreduce_pipelined(
                p2p._ctx, C.byref(s), ptr(x), ptr(du), *fp, ptr(u), ptr(dx), ptr(dk_scratch), ptr(dKs[(i + 1) % len(dKs)]),
                ptr(ws_step), wsb_step, st, flags))
            return
        if shared and fused_exchange:
            x, du, u, dx = sets[i % NSETS]
            P._lib.check(lib.b200cp_cp4_step_allreduce(p2p._ctx, C.byref(s), ptr(x), ptr(du), *fp, ptr(u), ptr(dx), ptr(dk),
                                                       ptr(ws_step), wsb_step, st, flags))
            return
        if shared:
            x, du, u, dx = sets[i % NSETS]
            P._lib.check(lib.b200cp_cp4_step(C.byref(s), ptr(x), ptr(du), *fp, ptr(u), ptr(dx), ptr(dk), ptr(ws_step),
                                             wsb_step, st, flags))
        else:
            x, du, u, dx = sets[i % NSETS]
            k_fwd(i, st)
            k_bwdd(i, st)
            P._lib.check(lib.b200cp_cp4_bwd_filter(C.byref(s), ptr(x), ptr(du), *fp, ptr(dk), ptr(ws), wsb, st, flags_f))
        if dist is not None and args.exchange == "inline":
            # The step's kernels are persistent (one CTA per SM, nearly all of its registers): an exchange kernel on
            # another stream either waits for them to leave or takes the room of the next step's CTAs, and both
            # measured slower than the exchange's own few microseconds on the step's stream.
            if p2p is not None:
                p2p(dk)
            else:
                dist.all_reduce(dk)
        elif dist is not None:
            ready = torch.cuda.Event()
            ready.record()
            comm.wait_event(ready)
            with torch.cuda.stream(comm):
                if p2p is not None:
                    p2p(dk)
                else:
                    dist.all_reduce(dk)
                done = torch.cuda.Event()
                done.record()
            ar_done[i % 2] = done

    def join_comm(*_):
        if pipelined:                       # the last step's exchange, inside the timed region
            P._lib.check(lib.b200cp_p2p_flush(p2p._ctx, ptr(dKs[0]), cur_stream()))
        for k in range(2):
            if ar_done[k] is not None:
                torch.cuda.current_stream().wait_event(ar_done[k])
                ar_done[k] = None

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def many(fn, k, tail=None):
        """k consecutive calls of fn as one CUDA graph (no host launch gaps); falls back to an eager loop."""
        g = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(g):
                st = cur_stream()
                for i in range(k):
                    fn(i, st)
                if tail:
                    tail()
            return g.replay, True
        except Exception as e:  # capture not possible: time the eager loop instead
            sys.stderr.write(f"[bench] graph capture failed ({e}); timing eager launches\n")
            torch.cuda.synchronize()

            def eager():
                for i in range(k):
                    fn(i, cur_stream())
                if tail:
                    tail()
            return eager, False

    for i in range(args.warmup):
        step(i, cur_stream())
    join_comm()
    barrier()
    K = args.steps
    l0 = P.launch_count()
    run_steps, graphed = many(step, K, join_comm)
    launches = P.launch_count() - l0 if graphed else None
    run_steps()                      # one untimed replay (graph upload, caches)
    barrier()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(REPLAYS)]
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    if launches is None:
        l0 = P.launch_count()
    for a, b in evs:
        a.record()
        run_steps()
        b.record()
    barrier()
    if launches is None:
        launches = (P.launch_count() - l0) // REPLAYS
    replay_ms = sorted(a.elapsed_time(b) for a, b in evs)
    ms = float(np.median(replay_ms))
    if p2p is not None:
        p2p.status()        # raises if an exchange gave up waiting for a peer: the timed steps would not be valid
    # the three kernels on their own, K back-to-back launches each, same rotating buffers, same run
    kt = []
    kernels = [("cp4_fwd", k_fwd, 0), ("cp4_bwd_data", k_bwdd, 0), ("cp4_bwd_filter", k_bwdf, 0)]
    if shared:   # the kernels of the step; third entry: bytes of rank planes they move on top of the algorithmic bytes
        kernels += [("cp4_fwd_save", k_fwd_save, 4 * plane_floats), ("cp4_bwd_data_save", k_bwdd_save, 4 * plane_floats),
                    ("cp4_bwd_filter_saved", k_bwdf_saved, 8 * plane_floats),
                    ("cp4_fwd_bwd_data_save", k_convs_save, 8 * plane_floats)]
        k_fwd_save(0, cur_stream())      # the planes the saved-plane kernel reads
        k_bwdd_save(0, cur_stream())
    for _, fn, _ in kernels:
        run_k, _ = many(fn, K)
        run_k()
        torch.cuda.synchronize()
        reps = []
        for _ in range(5):
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            run_k()
            a1.record()
            torch.cuda.synchronize()
            reps.append(a0.elapsed_time(a1) / K)
        kt.append(float(np.median(reps)))
        del run_k
    clocks = sampler.stop() if rank == 0 else None
    mean_ms = np.array(kt)
    if dist is not None:
        tms = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = float(tms.item())
        tl = torch.tensor([launches], device="cuda", dtype=torch.int64)
        dist.all_reduce(tl)
        launches = int(tl.item())
    value = world * n * K / (ms * 1e-3)

    # ---- end to end: host buffers through the C ABI's host entry point ------------------------
    Ks = max(8, min(K, 60))                     # steps of the end-to-end loop: its fill and drain cost one step's copies
    hX, hdU = torch.from_numpy(X).pin_memory(), torch.from_numpy(dU).pin_memory()
    hf = [torch.from_numpy(a).pin_memory() for a in (K0, K1, KH, KW)]
    # NSLOT sets of pinned result buffers: steps i+1 .. i+NSLOT-1 are queued while step i drains (the slots of the host
    # entry point), so that the copy-in runs ahead of the copy-out by more than a kernel time
    NSLOT = 4
    houts = [(torch.empty((n, c["T"], c["H"], c["W"])).pin_memory(), torch.empty((n, c["C"], c["H"], c["W"])).pin_memory(),
              torch.empty(nK).pin_memory()) for _ in range(NSLOT)]

    def finish(slot):
        P.cp4_conv2d_step_host_wait(slot)
        if dist is not None:   # the gradient exchange of a data-parallel step, on the host-visible result
            g = houts[slot][2].cuda(non_blocking=True)
            dist.all_reduce(g)
            houts[slot][2].copy_(g, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        return float(houts[slot][2][0])   # the host reads the step's result

    def run_e2e(steps):
        for i in range(steps):
            P.cp4_conv2d_step_host_submit(hX, hdU, *hf, houts[i % NSLOT], pad=c["pad"], flags=flags, slot=i % NSLOT)
            if i >= NSLOT - 1:
                finish((i - (NSLOT - 1)) % NSLOT)
        for i in range(max(0, steps - (NSLOT - 1)), steps):
            finish(i % NSLOT)

    run_e2e(NSLOT + 1)
    barrier()
    t0 = time.perf_counter()
    run_e2e(Ks)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    # the copies alone (same bytes, both directions at once on two streams, no kernels): what the host link gives
    # this rank while every other rank does the same
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    dbuf = [torch.empty_like(Xd), torch.empty_like(dUd)]
    barrier()
    t0 = time.perf_counter()
    for _ in range(Ks):
        with torch.cuda.stream(s_in):
            dbuf[0].copy_(hX, non_blocking=True)
            dbuf[1].copy_(hdU, non_blocking=True)
        with torch.cuda.stream(s_out):
            houts[0][0].copy_(dbuf[0], non_blocking=True)
            houts[0][1].copy_(dbuf[1], non_blocking=True)
    torch.cuda.synchronize()
    copy_s = time.perf_counter() - t0
    if dist is not None:
        te = torch.tensor([e2e_s, copy_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_s, copy_s = float(te[0].item()), float(te[1].item())
    h2d = 4 * (X.size + dU.size + sum(a.numel() for a in hf))
    d2h = 4 * sum(a.numel() for a in houts[0])
    e2e = world * n * Ks / e2e_s
    copy_gbs = (h2d + d2h) * Ks / copy_s / 1e9          # per rank, both directions together
    e2e_gbs = (h2d + d2h) * Ks / e2e_s / 1e9

    # ---- the other configurations, strong scaling, in the same run --------------------------------------------
    extra = None
    if not args.no_extra:
        def reduce_fn(t):
            if dist is not None:
                dist.all_reduce(t)

        def max_over_ranks(v):
            if dist is None:
                return v
            tv = torch.tensor([v], device="cuda", dtype=torch.float64)
            dist.all_reduce(tv, op=dist.ReduceOp.MAX)
            return float(tv.item())
        extra = extra_configs(P, world, rank, reduce_fn, max_over_ranks)
        # what a caller without a CUDA graph pays per step of the headline configuration (host launch path included)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(K):
            step(i, cur_stream())
        join_comm()
        torch.cuda.synchronize()
        extra["cfg2_eager_step_us"] = max_over_ranks((time.perf_counter() - t0) / K * 1e6)
        extra["cfg2_graph_step_us"] = ms / K * 1e3

    def leave():
        # release everything that holds the communicator (captured graphs, the exchange regions), then tear down
        sys.stdout.flush()
        sys.stderr.flush()
        if dist is not None:
            torch.cuda.synchronize()
            if p2p is not None:
                p2p.close()
            dist.barrier()
            dist.destroy_process_group()

    del run_steps          # the captured graphs go before the process group does
    if rank != 0:
        leave()
        return

    # ---- roofline of the dominant kernel ---------------------------------------------------------
    names = [k[0] for k in kernels]
    # algorithmic bytes of every kernel: input + output tensor once, the factors once; the rank planes a kernel
    # of the step writes or reads on top of that are traffic, not algorithmic bytes
    base_bytes = 4 * n * HW * (c["C"] + c["T"]) + 4 * c["R"] * (c["T"] + c["C"] + 2 * c["F"])
    kbytes = [base_bytes for k in kernels]
    if shared:
        kbytes[6] = 2 * base_bytes                         # one launch that is two of the path's kernels
    # The launches of the timed step: with shared planes forward and backward-data are one launch (entry 6) followed
    # by the gradient kernels (entry 5); entries 3 and 4 are that launch's two halves run on their own.
    in_step = (6, 5) if shared else range(0, 3)
    dom = max(in_step, key=lambda i: mean_ms[i])
    alg_bytes = kbytes[dom]
    peak, peak_kind = hbm_peak()
    achieved = alg_bytes / (mean_ms[dom] * 1e-3) / 1e9
    traffic = None
    try:
        traffic = json.load(open(os.path.join(ROOT, "profiles", "dram_traffic.json"))).get(names[dom])
    except Exception:
        pass
    step_us = ms / K * 1e3
    roofline = {"bound": "hbm", "kernel": names[dom], "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": traffic, "peak_kind": f"of {peak_kind}",
                "algorithmic_bytes_per_launch": alg_bytes,
                "plane_bytes_per_launch": {k[0]: k[2] for k in kernels if k[2]},
                "step": {"bytes": 3 * base_bytes, "us": step_us, "frac": 3 * base_bytes / (step_us * 1e-6) / 1e9 / peak},
                "per_kernel_us": {nm: float(v * 1e3) for nm, v in zip(names, mean_ms)},
                "per_kernel_frac": {nm: float(b / (v * 1e-3) / 1e9 / peak) for nm, v, b in zip(names, mean_ms, kbytes)},
                "kernels_in_step": [names[i] for i in in_step],
                "launches_in_step": [{"kernel": names[i], "us": float(mean_ms[i] * 1e3), "algorithmic_bytes": kbytes[i],
                                      "frac": float(kbytes[i] / (mean_ms[i] * 1e-3) / 1e9 / peak)} for i in in_step]}

    cpu = None
    if not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)
        ips, dt, done = time_cpu(n, 1000, 1, budget_s=15.0)
        cpu = {"value": ips, "unit": "images/s", "cores": torch.get_num_threads(), "kind": "port",
               "sample": f"{done} full steps of N={n} in {dt * done:.1f} s (torch-CPU restatement of the reference's "
                         "unfused composition, forward + autograd backward)"}
        if world == 1:
            cpu["reference_gpu_forward_us"] = reference_gpu_forward_us()

    line = {
        "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world, "steps": K, "warmup": args.warmup,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic (seeded; X~U[-1,1], factors~N(0,1/sqrt(9C)), dU~N(0,1))",
        "config": {"workload": WORKLOAD, "images_per_step_per_gpu": n, "path": args.path,
                   "step": "b200cp_cp4_step: forward, backward-data and backward-filter in one call, rank planes shared"
                           if shared else "b200cp_cp4_fwd + b200cp_cp4_bwd_data + b200cp_cp4_bwd_filter",
                   "timing": (f"K steps captured as one CUDA graph, replayed {REPLAYS} times, each replay between its own two "
                              "events; median replay") if graphed else f"K eager steps, {REPLAYS} times; median",
                   "replay_ms": [round(x, 4) for x in replay_ms],
                   "l2": f"{NSETS} rotating buffer sets ({NSETS * 4 * n * HW * 64 * 4 / 1e6:.0f} MB) > 126 MB L2",
                   "collective": ("allreduce of %d packed factor-gradient floats per step (%s), %s"
                                  % (nK, "b200cp_p2p_allreduce: one kernel over NVLink peer memory" if p2p is not None
                                     else "NCCL",
                                     "posted by the step's gradient reduction kernel and completed by the next step's "
                                     "(b200cp_cp4_step_allreduce_pipelined; the last one by b200cp_p2p_flush, timed)"
                                     if pipelined else
                                     "as the tail of the step's gradient reduction kernel (b200cp_cp4_step_allreduce)"
                                     if fused_exchange else "on the step's stream" if args.exchange == "inline" else
                                     "on a communication stream, overlapped with the next step")) if world > 1 else "none"},
        "roofline": roofline, "cpu_baseline": cpu,
        "e2e": {"value": e2e, "unit": "images/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": Ks,
                "copy_gbs_per_rank": e2e_gbs, "copy_only_gbs_per_rank": copy_gbs, "numa_node_rank0": numa_node,
                "note": "host buffers through b200cp_cp4_step_host_submit / _wait (b200cp_cp4_step inside); the copies "
                        "alone, both directions at once, reach copy_only_gbs_per_rank on this host"},
        "extra": extra,
        "gpu_launches": launches, "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    leave()


if __name__ == "__main__":
    main()
