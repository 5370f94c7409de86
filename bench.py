#!/usr/bin/env python
"""CP4 conv2d forward + backward-data + backward-filter throughput (images/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: the configuration the headline metric is quoted on -- N=32 images per GPU,
C=T=64, 56x56, 3x3 filter, rank 16, same padding, fp32, seeded synthetic inputs.
One step = forward, backward-data and backward-filter over one batch (plus the allreduce
of the packed factor gradients when more than one GPU runs).  Batches are sharded across
ranks (weak scaling: every rank owns N=32 images).

Timing: CUDA events on the launching stream; a barrier + synchronize on both sides; the
maximum over ranks.  Every step uses the next of several distinct buffer sets so that a set
is evicted from L2 before it is used again.  Rank 0 prints one JSON line.
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--path", default="auto", choices=["auto", "simt", "tc3x", "mma"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--allreduce", default="p2p", choices=["p2p", "nccl"],
                    help="gradient allreduce of the multi-GPU step: the library's peer-memory kernel, or NCCL")
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

    def step(i, st):
        dk = dKs[i % len(dKs)]
        if dist is not None and ar_done[i % 2] is not None:
            torch.cuda.current_stream().wait_event(ar_done[i % 2])
        if shared:
            x, du, u, dx = sets[i % NSETS]
            P._lib.check(lib.b200cp_cp4_step(C.byref(s), ptr(x), ptr(du), *fp, ptr(u), ptr(dx), ptr(dk), ptr(ws_step),
                                             wsb_step, st, flags))
        else:
            x, du, u, dx = sets[i % NSETS]
            k_fwd(i, st)
            k_bwdd(i, st)
            P._lib.check(lib.b200cp_cp4_bwd_filter(C.byref(s), ptr(x), ptr(du), *fp, ptr(dk), ptr(ws), wsb, st, flags_f))
        if dist is not None:
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
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    if launches is None:
        l0 = P.launch_count()
    e0.record()
    run_steps()
    e1.record()
    barrier()
    if launches is None:
        launches = P.launch_count() - l0
    ms = e0.elapsed_time(e1)
    if p2p is not None:
        p2p.status()        # raises if an exchange gave up waiting for a peer: the timed steps would not be valid
    # the three kernels on their own, K back-to-back launches each, same rotating buffers, same run
    kt = []
    kernels = [("cp4_fwd", k_fwd, 0), ("cp4_bwd_data", k_bwdd, 0), ("cp4_bwd_filter", k_bwdf, 0)]
    if shared:   # the kernels of the step: extra bytes = the rank planes written / read
        kernels += [("cp4_fwd_save", k_fwd_save, 4 * plane_floats), ("cp4_bwd_data_save", k_bwdd_save, 4 * plane_floats),
                    ("cp4_bwd_filter_saved", k_bwdf_saved, 8 * plane_floats)]
        k_fwd_save(0, cur_stream())      # the planes the saved-plane kernel reads
        k_bwdd_save(0, cur_stream())
    for _, fn, _ in kernels:
        run_k, _ = many(fn, K)
        run_k()
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        run_k()
        a1.record()
        torch.cuda.synchronize()
        kt.append(a0.elapsed_time(a1) / K)
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
    Ks = max(4, min(K, 20))
    hX, hdU = torch.from_numpy(X).pin_memory(), torch.from_numpy(dU).pin_memory()
    hf = [torch.from_numpy(a).pin_memory() for a in (K0, K1, KH, KW)]
    # two sets of pinned result buffers: step i+1 is queued while step i drains (two slots of the host entry point)
    houts = [(torch.empty((n, c["T"], c["H"], c["W"])).pin_memory(), torch.empty((n, c["C"], c["H"], c["W"])).pin_memory(),
              torch.empty(nK).pin_memory()) for _ in range(2)]

    def finish(slot):
        P.cp4_conv2d_step_host_wait(slot)
        if dist is not None:   # the gradient exchange of a data-parallel step, on the host-visible result
            g = houts[slot][2].cuda(non_blocking=True)
            dist.all_reduce(g)
            houts[slot][2].copy_(g)
        return float(houts[slot][2][0])   # the host reads the step's result

    def run_e2e(steps):
        for i in range(steps):
            P.cp4_conv2d_step_host_submit(hX, hdU, *hf, houts[i % 2], pad=c["pad"], flags=flags, slot=i % 2)
            if i >= 1:
                finish((i - 1) % 2)
        finish((steps - 1) % 2)

    run_e2e(3)
    barrier()
    t0 = time.perf_counter()
    run_e2e(Ks)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if dist is not None:
        te = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_s = float(te.item())
    h2d = 4 * (X.size + dU.size + sum(a.numel() for a in hf))
    d2h = 4 * sum(a.numel() for a in houts[0])
    e2e = world * n * Ks / e2e_s

    def leave():
        # CUDA graphs that captured NCCL work keep the communicator busy and make destroy_process_group() wait for
        # ever; all results are out, so leave without tearing NCCL down
        sys.stdout.flush()
        sys.stderr.flush()
        if dist is not None:
            torch.cuda.synchronize()
            os._exit(0)

    if rank != 0:
        leave()
        return

    # ---- roofline of the dominant kernel ---------------------------------------------------------
    names = [k[0] for k in kernels]
    base_bytes = 4 * n * HW * (c["C"] + c["T"]) + 4 * c["R"] * (c["T"] + c["C"] + 2 * c["F"])
    kbytes = [base_bytes + k[2] for k in kernels]
    in_step = range(3, 6) if shared else range(0, 3)      # the kernels the timed step launches
    dom = max(in_step, key=lambda i: mean_ms[i])
    alg_bytes = kbytes[dom]
    peak, peak_kind = hbm_peak()
    achieved = alg_bytes / (mean_ms[dom] * 1e-3) / 1e9
    traffic = None
    try:
        traffic = json.load(open(os.path.join(ROOT, "profiles", "dram_traffic.json"))).get(names[dom])
    except Exception:
        pass
    roofline = {"bound": "hbm", "kernel": names[dom], "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": traffic, "peak_kind": f"of {peak_kind}",
                "algorithmic_bytes_per_launch": alg_bytes,
                "per_kernel_us": {nm: float(v * 1e3) for nm, v in zip(names, mean_ms)},
                "per_kernel_frac": {nm: float(b / (v * 1e-3) / 1e9 / peak) for nm, v, b in zip(names, mean_ms, kbytes)},
                "kernels_in_step": [names[i] for i in in_step]}

    cpu = None
    if not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)
        ips, dt, done = time_cpu(n, 1000, 1, budget_s=15.0)
        cpu = {"value": ips, "unit": "images/s", "cores": torch.get_num_threads(), "kind": "port",
               "sample": f"{done} full steps of N={n} in {dt * done:.1f} s (torch-CPU restatement of the reference's "
                         "unfused composition, forward + autograd backward)"}

    line = {
        "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world, "steps": K, "warmup": args.warmup,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic (seeded; X~U[-1,1], factors~N(0,1/sqrt(9C)), dU~N(0,1))",
        "config": {"workload": WORKLOAD, "images_per_step_per_gpu": n, "path": args.path,
                   "step": "b200cp_cp4_step: forward, backward-data and backward-filter in one call, rank planes shared"
                           if shared else "b200cp_cp4_fwd + b200cp_cp4_bwd_data + b200cp_cp4_bwd_filter",
                   "timing": "K steps replayed as one CUDA graph between two events" if graphed else "K eager steps between two events",
                   "l2": f"{NSETS} rotating buffer sets ({NSETS * 4 * n * HW * 64 * 4 / 1e6:.0f} MB) > 126 MB L2",
                   "collective": ("allreduce of %d packed factor-gradient floats per step (%s), on a communication stream, "
                                  "overlapped with the next step"
                                  % (nK, "b200cp_p2p_allreduce: one kernel over NVLink peer memory" if p2p is not None
                                     else "NCCL")) if world > 1 else "none"},
        "roofline": roofline, "cpu_baseline": cpu,
        "e2e": {"value": e2e, "unit": "images/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": Ks},
        "gpu_launches": launches, "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    leave()


if __name__ == "__main__":
    main()
