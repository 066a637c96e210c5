"""Builds a program emitted by the DSL into an executable (nvcc, sm_100a),
linked against the in-tree runtime library.  Shared by the GPU tests."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DSL = os.path.join(ROOT, "coconet_b200", "dsl")
LIBDIR = os.path.join(ROOT, "coconet_b200")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

SCALARS = {"COCONET_SCALAR_lr": "0.01", "COCONET_SCALAR_beta1": "0.9", "COCONET_SCALAR_beta2": "0.999",
           "COCONET_SCALAR_decay": "0.01", "COCONET_SCALAR_mu": "0.9",
           "COCONET_SCALAR_inv_scale": "0.125"}


def build_program(opt, schedule, workdir):
    subprocess.check_call(["make", "-C", DSL, "-s"])
    src = os.path.join(workdir, f"{opt}-{schedule}.cu")
    subprocess.check_call([os.path.join(DSL, "build", "optimizers"), opt, schedule, src])
    exe = os.path.join(workdir, f"{opt}-{schedule}")
    libs = ["-lcoconet_rt", "-lcurand"]
    if "COCONET_USE_NCCL" in open(src).read():
        libs.append("-lnccl")
    subprocess.check_call([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O2",
                           "-I", os.path.join(DSL, "rt"), "-I", os.path.join(ROOT, "include"), src,
                           "-L", LIBDIR, "-Xlinker", "-rpath", "-Xlinker", LIBDIR, "-o", exe] + libs)
    return exe
