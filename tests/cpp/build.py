"""Build tests/cpp/test_hpp (the C++ mirror of the reference API over libb200cp) with g++."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "_build", "test_hpp")


def build():
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    from paralleltnnlayers_b200 import build as b
    lib = b.build()
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    src = os.path.join(HERE, "test_hpp.cpp")
    hdr = os.path.join(ROOT, "include", "b200cp.hpp")
    if os.path.exists(OUT) and os.path.getmtime(OUT) > max(os.path.getmtime(src), os.path.getmtime(hdr), os.path.getmtime(lib)):
        return OUT
    libdir = os.path.dirname(lib)
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-o", OUT, src, "-I", os.path.join(ROOT, "include"),
                           "-I", "/usr/local/cuda/include", "-L", libdir, "-lb200cp", "-L", "/usr/local/cuda/lib64",
                           "-lcudart", f"-Wl,-rpath,{libdir}", "-Wl,-rpath,/usr/local/cuda/lib64"])
    return OUT


if __name__ == "__main__":
    print(build())
