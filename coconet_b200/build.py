"""Builds libcoconet_rt.so (the C-ABI runtime + sm_100a kernels) in-tree."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libcoconet_rt.so")
SOURCES = ["fused_step.cu", "runtime.cu", "bootstrap.cpp", "no_alloc.cu"]
HEADERS = ["fused_step.cuh", "bootstrap.h", os.path.join(ROOT, "include", "coconet_rt.h")]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + [
        h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force=False, verbose=False):
    """Compile for sm_100a only; returns the path of the shared library."""
    if not force and not _stale():
        return LIB
    cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-shared", "-cudart", "shared", "-Xcompiler", "-fPIC",
           "-I" + os.path.join(ROOT, "include"), "-I" + CSRC, "-o", LIB]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build_library(force=True, verbose="-v" in os.sys.argv))
