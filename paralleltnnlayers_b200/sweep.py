"""Kernel timings of every layer family at the sizes of the benchmark configurations.

    python -m paralleltnnlayers_b200.sweep [cp4] [rcp] [dense] [--reps 12] [--json]
    python -m paralleltnnlayers_b200.sweep --shapes FILE [--ranks 1,2,4,8,16] [--reps 47] [--out results.csv] [--mem]

The second form reads a shape list in the reference's format (``N C H W pad T Y X`` per line, ``#`` comments;
Cuda_kernels/bench/tensors*.txt) and writes the CSV its ``BenchBothTime`` writes (bench/BenchBothTime.cu:84-104):
the shape, then the mean forward time in microseconds for each CP rank (the cuDNN column is left out).  With
``--mem`` it writes the table of ``BenchBothMem`` instead (bench/BenchBothMem.cu:84-106): the KiB of device memory
the forward call touches per rank, input + output + factors (``CP::run_convolution``, cp4Conv2d.cu:176-178); that
mode needs no device.

Inputs live on the device; every call of a timed kernel uses the next of several distinct buffer sets (more
than the L2 holds), the calls of one measurement are captured in one CUDA graph so that there are no host gaps,
and the time is the best of three replays, taken with CUDA events on the launching stream.  Seeded synthetic
inputs with the value distributions of the benchmark configurations: X ~ U[-1,1], CP4 factors ~ N(0, 1/sqrt(9C)),
rCP factors ~ N(0, 0.3), dense factors ~ N(0, 0.35), upstream gradients ~ N(0,1).
"""
from __future__ import annotations

import argparse
import json
import sys

import numpy as np
import torch

CP4_SHAPES = [(32, 64, 56, 16)] + [(64, c, h, r) for (c, h) in ((128, 28), (256, 14), (512, 7)) for r in (8, 16, 32, 64)]
RCP = dict(N=32, cdims=(4, 8, 8), tdims=(4, 8, 8), H=28, W=28, F=3, R=16)
DENSE = dict(B=4096, idims=(8, 8, 8, 8), odims=(8, 8, 8, 8), R=32)


def timeit(fn, reps):
    """fn(i) launched `reps` times inside one CUDA graph, replayed three times; microseconds per call (best replay)."""
    for i in range(2):
        fn(i)
    torch.cuda.synchronize()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for i in range(reps):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            g.replay()
            e1.record(st)
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) / reps * 1e3)
    return best


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def _sets(t, total_bytes=300e6, most=12):
    n = int(min(most, max(2, total_bytes // (2 * t.numel() * 4) + 1)))
    return [t.clone() for _ in range(n)]


def sweep_cp4(P, reps, rows):
    paths = (("simt", P.PATH_SIMT), ("tc3x", P.PATH_TC3X), ("mma", P.PATH_MMA))
    for (N, C, H, R) in CP4_SHAPES:
        rng = np.random.default_rng(1)
        std = 1.0 / np.sqrt(9 * C)
        X = _dev(rng.uniform(-1, 1, size=(N, C, H, H)))
        K = [_dev(rng.normal(0, std, size=(d, R))) for d in (C, C, 3, 3)]
        dU = _dev(rng.normal(0, 1, size=(N, C, H, H)))
        Xs, dUs = _sets(X), _sets(dU)
        n = len(Xs)
        row = {"layer": "cp4", "N": N, "C=T": C, "H=W": H, "R": R, "hbm_floor_us": 2 * X.numel() * 4 / 6.45e12 * 1e6}
        for name, fl in paths:
            try:
                row["fwd_" + name] = timeit(lambda i: P.cp4_conv2d_forward(Xs[i % n], *K, 1, flags=fl), reps)
            except P.B200CPError:
                row["fwd_" + name] = None      # the path does not take this shape
        # the reference's comparison line: recomposed filter + ordinary conv2d (and the conv2d alone, filter kept)
        row["fwd_rebuild"] = timeit(lambda i: P.cp4_conv2d_rebuild_forward(Xs[i % n], *K, 1), reps)
        Kd = P.cp4recom(*K)
        row["fwd_dense_conv"] = timeit(lambda i: P.conv2d_dense_forward(Xs[i % n], Kd, 1), reps)
        row["bwd_data"] = timeit(lambda i: P.cp4_conv2d_backward_data(dUs[i % n], *K, 1), reps)
        for name, fl in (("simt", P.PATH_SIMT), ("mma", P.PATH_MMA)):
            row["bwd_filter_" + name] = timeit(
                lambda i: P.cp4_conv2d_backward_filter(dUs[i % n], Xs[i % n], *K, 1, flags=fl, packed=True), reps)
        # the whole training step in one call (rank planes shared between the three kernels)
        row["step"] = timeit(lambda i: P.cp4_conv2d_step(Xs[i % n], dUs[i % n], *K, 1), reps)
        rows.append(row)
        del Xs, dUs
        torch.cuda.empty_cache()
    P.device_status()


def sweep_rcp(P, reps, rows):
    c = RCP
    rng = np.random.default_rng(20)
    Cc, Tc = int(np.prod(c["cdims"])), int(np.prod(c["tdims"]))
    X = _dev(rng.uniform(-1, 1, size=(c["N"], Cc, c["H"], c["W"])))
    A = [_dev(rng.normal(0, 0.3, size=(a, b, c["R"]))) for a, b in zip(c["cdims"], c["tdims"])]
    S = _dev(rng.normal(0, 0.3, size=(c["F"], c["F"], c["R"])))
    dV = _dev(rng.normal(0, 1, size=(c["N"], Tc, c["H"], c["W"])))
    Xs, dVs = _sets(X, most=8), _sets(dV, most=8)
    n = len(Xs)
    rows.append({"layer": "rcp", **{k: v for k, v in c.items()},
                 "fwd": timeit(lambda i: P.conv2d_rcp_fused_nchw(Xs[i % n], *A, S), reps),
                 "fwd_rebuild": timeit(lambda i: P.conv2d_rcp_rebuild_nchw(Xs[i % n], *A, S), reps),
                 "bwd_data": timeit(lambda i: P.rcp_conv2d_backward(Xs[i % n], dVs[i % n], *A, S, need_dw=False), reps),
                 "bwd_factors": timeit(lambda i: P.rcp_conv2d_backward(Xs[i % n], dVs[i % n], *A, S, need_dx=False), reps),
                 "hbm_floor_us": 2 * X.numel() * 4 / 6.45e12 * 1e6})


def sweep_dense(P, reps, rows):
    c = DENSE
    rng = np.random.default_rng(30)
    I, O = int(np.prod(c["idims"])), int(np.prod(c["odims"]))
    X = _dev(rng.normal(0, 1, size=(c["B"], I)))
    F = [_dev(rng.normal(0, 0.35, size=(a, b, c["R"]))) for a, b in zip(c["idims"], c["odims"])]
    dY = _dev(rng.normal(0, 1, size=(c["B"], O)))
    Xs, dYs = _sets(X, most=4), _sets(dY, most=4)
    n = len(Xs)
    reps = max(2, reps // 3)
    rows.append({"layer": "dense", **{k: v for k, v in c.items()},
                 "fwd": timeit(lambda i: P.dense_cp(Xs[i % n], *F), reps),
                 "fwd_rebuild": timeit(lambda i: P.dense_cp_rebuild(Xs[i % n], *F), reps),
                 "fwd_matmul": timeit(lambda i, M=P.dense_cp_recompose(*F): P.dense_matmul(Xs[i % n], M), reps),
                 "bwd_data": timeit(lambda i: P.dense_cp_backward(Xs[i % n], dYs[i % n], *F, need_dw=False), reps),
                 "bwd_factors": timeit(lambda i: P.dense_cp_backward(Xs[i % n], dYs[i % n], *F, need_dx=False), reps),
                 "hbm_floor_us": 2 * X.numel() * 4 / 6.45e12 * 1e6})


def read_shapes(path):
    """Unique shapes of a reference-format list, in the order ``tensor_shape::operator<`` gives them
    (Cuda_kernels/Tensor.cuh:10-25: lexicographic over N, C, H, W, pad, T, Y, X)."""
    shapes = set()
    with open(path) as f:
        for line in f:
            line = line.split("#", 1)[0].strip()
            if not line:
                continue
            v = [int(x) for x in line.replace("|", " ").split()]
            if len(v) < 8:
                raise ValueError(f"shape line needs N C H W pad T Y X: {line!r}")
            shapes.add(tuple(v[:8]))
    return sorted(shapes)


def footprint_bytes(N, C, H, W, T, Y, X, R):
    """Bytes the forward call touches: input, output and the four factors (cp4Conv2d.cu:176-178)."""
    return 4 * (N * T * H * W + N * C * H * W + R * (T + C + X + Y))


def mem_shapes(path, ranks, out):
    lines = [f"{N} {C} {H} {W} {pad} {T} {Y} {X}, "
             + ", ".join(str(footprint_bytes(N, C, H, W, T, Y, X, R) // 1024) for R in ranks)
             for (N, C, H, W, pad, T, Y, X) in read_shapes(path)]
    text = "\n".join(lines) + "\n"
    if out:
        with open(out, "w") as f:
            f.write(text)
    else:
        sys.stdout.write(text)


def bench_shapes(P, path, ranks, reps, out):
    lines = []
    for (N, C, H, W, pad, T, Y, X) in read_shapes(path):
        rng = np.random.default_rng(1234)     # the reference seeds its generator with 1234 (test_cp4Conv.cpp.cu)
        x = _dev(rng.uniform(0, 1, size=(N, C, H, W)))
        xs = _sets(x)
        n = len(xs)
        cols = []
        for R in ranks:
            K = [_dev(rng.uniform(0, 1, size=(d, R))) for d in (T, C, Y, X)]
            try:
                cols.append("%.3f" % timeit(lambda i: P.cp4_conv2d_forward(xs[i % n], *K, pad), reps))
            except P.B200CPError as e:
                cols.append("nan")
                sys.stderr.write(f"[sweep] {N} {C} {H} {W} {pad} {T} {Y} {X} rank {R}: {e}\n")
        lines.append(f"{N} {C} {H} {W} {pad} {T} {Y} {X}, " + ", ".join(cols))
        del xs
        torch.cuda.empty_cache()
    text = "\n".join(lines) + "\n"
    if out:
        with open(out, "w") as f:
            f.write(text)
    else:
        sys.stdout.write(text)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("which", nargs="*", help="any of cp4, rcp, dense (default: all)")
    ap.add_argument("--reps", type=int, default=12)
    ap.add_argument("--json", action="store_true", help="one JSON object per line instead of text")
    ap.add_argument("--shapes", help="shape list in the reference's format: time the CP4 forward per shape and rank")
    ap.add_argument("--ranks", default="1,2,4,8,16", help="CP ranks of the --shapes run (the reference's 1..16)")
    ap.add_argument("--out", help="CSV file of the --shapes run (default: stdout)")
    ap.add_argument("--mem", action="store_true", help="with --shapes: KiB touched per rank instead of timings")
    args = ap.parse_args(argv)
    if args.shapes and args.mem:
        mem_shapes(args.shapes, [int(r) for r in args.ranks.split(",")], args.out)
        return 0
    if args.shapes:
        import paralleltnnlayers_b200 as P
        assert torch.cuda.is_available(), "the sweep needs a CUDA device"
        bench_shapes(P, args.shapes, [int(r) for r in args.ranks.split(",")], 47 if args.reps == 12 else args.reps,
                     args.out)
        return 0
    args.which = args.which or ["cp4", "rcp", "dense"]
    for w in args.which:
        if w not in ("cp4", "rcp", "dense"):
            ap.error(f"unknown layer family {w!r}")
    import paralleltnnlayers_b200 as P   # raises if libb200cp.so is missing
    assert torch.cuda.is_available(), "the sweep needs a CUDA device"
    rows = []
    for w in args.which:
        {"cp4": sweep_cp4, "rcp": sweep_rcp, "dense": sweep_dense}[w](P, args.reps, rows)
    for r in rows:
        if args.json:
            print(json.dumps(r))
        else:
            print("  ".join(f"{k}={v:.1f}" if isinstance(v, float) else f"{k}={v}" for k, v in r.items()))
    return 0


if __name__ == "__main__":
    sys.exit(main())
