"""Builds libzepp_b200.so in-tree with nvcc for sm_100a:  python -m zepp_b200.build"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc", "runtime.cu")
OUT = os.path.join(HERE, "lib", "libzepp_b200.so")
DEPS = [os.path.join(HERE, "csrc", f) for f in os.listdir(os.path.join(HERE, "csrc"))] + \
       [os.path.join(os.path.dirname(HERE), "include", "zepp_b200.h")]


def build(force=False, verbose=False):
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    if not force and os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(d) for d in DEPS):
        return OUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--shared",
           "-Xcompiler", "-fPIC", "-o", OUT, SRC]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    extra = os.environ.get("ZEPP_B200_NVCC_FLAGS", "").split()     # e.g. -DZEPP_FINE_TRACE, -DZEPP_GEMM_PROFILE
    if extra:
        cmd[1:1] = extra
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
