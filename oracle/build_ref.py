"""Compile the reference's own CP4 sources (where they lie, unmodified) plus
``oracle/ref_shim.cu`` into ``oracle/_ref/libcp4ref_{fwd,bwd}.so`` for sm_100a.

TEST INFRASTRUCTURE ONLY.  Needs the reference checkout; on a machine without
it (the GPU box) the prebuilt libraries that travelled with the repository are
used.  ``oracle/_ref/`` is git-ignored: no reference code enters the history.

    python -m oracle.build_ref [/path/to/reference]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
DEFAULT_REF = "/root/reference"


def build(ref=DEFAULT_REF, force=False):
    ck = os.path.join(ref, "Cuda_kernels")
    libs = {n: os.path.join(OUT, f"libcp4ref_{n}.so") for n in ("fwd", "bwd")}
    if not os.path.isdir(ck):
        return {n: p for n, p in libs.items() if os.path.exists(p)}
    os.makedirs(OUT, exist_ok=True)
    srcs = {
        "fwd": ["Tensor.cu", "cp4Conv2dForward.cu"],
        "bwd": ["Tensor.cu", "cp4Conv2dBackwardData.cu", "cp4Conv2dBackwardFilter.cu"],
    }
    shim = os.path.join(HERE, "ref_shim.cu")
    for n, files in srcs.items():
        if not force and os.path.exists(libs[n]) and os.path.getmtime(libs[n]) > os.path.getmtime(shim):
            continue
        cmd = ["nvcc", "-shared", "-o", libs[n], "-std=c++14", "-O2", "-w", "-gencode",
               "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", f"-DREF_{n.upper()}", "-I", ck, shim]
        cmd += [os.path.join(ck, f) for f in files]
        subprocess.check_call(cmd)
    return libs


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REF, force=True))
