"""Compile the reference's own CUDA sources (where they lie, unmodified) plus the shims of this directory
into ``oracle/_ref/`` for sm_100a:

    libcp4ref_fwd.so / libcp4ref_bwd.so   Cuda_kernels/{Tensor,cp4Conv2dForward,cp4Conv2dBackwardData,
                                          cp4Conv2dBackwardFilter}.cu + ref_shim.cu
    libtvmref_{rcp,dense,cp3,cp4}.so      Kernels/{rcp_fused_nchw,dense_cp,cp_fused_nchw,cp4_conv_nchw}.cu
                                          (-DGOOGLE_CUDA=1; the files include nothing) + ref_tvm_shim.cu

TEST INFRASTRUCTURE ONLY.  Needs the reference checkout; on a machine without it (the GPU box) the prebuilt
libraries that travelled with the repository are used.  ``oracle/_ref/`` is git-ignored: no reference code
enters the history.

    python -m oracle.build_ref [/path/to/reference]

Without an argument the checkout is looked for in ``$B200CP_REFERENCE_DIR`` and then in a directory named
``reference`` beside the repository.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
TVM = {"rcp": "rcp_fused_nchw.cu", "dense": "dense_cp.cu", "cp3": "cp_fused_nchw.cu", "cp4": "cp4_conv_nchw.cu"}
NVCC = ["nvcc", "-shared", "-O2", "-w", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]


def default_reference():
    env = os.environ.get("B200CP_REFERENCE_DIR")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref=None, force=False):
    ref = ref or default_reference()
    ck, kn = os.path.join(ref, "Cuda_kernels"), os.path.join(ref, "Kernels")
    libs = {n: os.path.join(OUT, f"libcp4ref_{n}.so") for n in ("fwd", "bwd")}
    libs.update({"tvm_" + n: os.path.join(OUT, f"libtvmref_{n}.so") for n in TVM})
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
        cmd = NVCC + ["-o", libs[n], "-std=c++14", f"-DREF_{n.upper()}", "-I", ck, shim]
        cmd += [os.path.join(ck, f) for f in files]
        subprocess.check_call(cmd)
    tshim = os.path.join(HERE, "ref_tvm_shim.cu")
    for n, f in TVM.items():
        lib = libs["tvm_" + n]
        if not force and os.path.exists(lib) and os.path.getmtime(lib) > os.path.getmtime(tshim):
            continue
        subprocess.check_call(NVCC + ["-o", lib, "-DGOOGLE_CUDA=1", f"-DREF_TVM_{n.upper()}", tshim, os.path.join(kn, f)])
    return libs


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None, force=True))
