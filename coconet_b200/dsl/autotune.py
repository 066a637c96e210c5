#!/usr/bin/env python
"""Measuring autotuner for the data-parallel schedules of a DSL program.

The reference's Autotuner enumerates schedules and prints them
(src/pipeline.cpp:1062-1192); this one builds what the emitter generates for
each schedule, runs it on the GPUs of this node and reports the fastest:

    python -m coconet_b200.dsl.autotune adam --gpus 8 --log2 26 --epochs 20

With --derive the three programs come from ONE DSL program written with
AllReduce: the C++ `Autotuner` (pipeline.hpp) derives RS_C_AG and fuse_RS_C_AG
from it with split / reorder / asSlice / fuse and emits all three; without it
each schedule is the hand-written variant in dsl/examples/optimizers.cpp.

Every schedule runs as plain C++ processes (one per GPU, started by
torch.distributed.run --no-python); times are the programs' own CUDA-event
totals from their "{SZ: .., Total: ..}" report line.
"""
import argparse
import json
import os
import re
import socket
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
SCHEDULES = ["AR_C", "RS_C_AG", "fuse_RS_C_AG"]


def build(opt, schedule, workdir, derive=False):
    subprocess.check_call(["make", "-C", HERE, "-s"])
    src = os.path.join(workdir, f"{opt}-{schedule}.cu")
    if not derive:
        subprocess.check_call([os.path.join(HERE, "build", "optimizers"), opt, schedule, src])
    elif not os.path.exists(src):   # one call emits all three schedules
        subprocess.check_call([os.path.join(HERE, "build", "optimizers"), opt, "autotune", workdir],
                              stdout=subprocess.DEVNULL)
    exe = os.path.join(workdir, f"{opt}-{schedule}")
    libdir = os.path.join(ROOT, "coconet_b200")
    libs = ["-lcoconet_rt", "-lcurand"] + (["-lnccl"] if "COCONET_USE_NCCL" in open(src).read() else [])
    subprocess.check_call([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-I",
                           os.path.join(HERE, "rt"), "-I", os.path.join(ROOT, "include"), src, "-L",
                           libdir, "-Xlinker", "-rpath", "-Xlinker", libdir, "-o", exe] + libs)
    return exe


def run(exe, gpus, log2, epochs, env):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--no-python", "--nnodes=1",
           f"--nproc-per-node={gpus}", "--master-addr", "127.0.0.1", "--master-port", str(port),
           exe, str(epochs), str(log2), str(log2 + 1)]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    if out.returncode != 0:
        raise RuntimeError(out.stdout[-2000:] + out.stderr[-2000:])
    m = re.search(r"\{SZ: (\d+), Epochs: (\d+), (.*)Total: ([0-9.]+)\}", out.stdout)
    if not m:
        raise RuntimeError("no report line in:\n" + out.stdout[-2000:])
    stages = dict((k, float(v)) for k, v in re.findall(r"(\w+): ([0-9.]+), ", m.group(3)))
    return float(m.group(4)), stages


def autotune(opt, gpus, log2, epochs, scalars=None, derive=False):
    env = dict(os.environ)
    env.update({f"COCONET_SCALAR_{k}": str(v) for k, v in (scalars or {}).items()})
    results = []
    with tempfile.TemporaryDirectory() as work:
        for schedule in SCHEDULES:
            exe = build(opt, schedule, work, derive)
            run(exe, gpus, log2, 2, env)                       # warm-up: first-call costs
            total, stages = run(exe, gpus, log2, epochs, env)
            results.append({"schedule": schedule, "ms_per_step": total / epochs, "stages_ms": stages})
    best = min(results, key=lambda r: r["ms_per_step"])
    return {"program": opt, "gpus": gpus, "elements": 1 << log2, "epochs": epochs, "results": results,
            "best": best["schedule"], "schedules": "derived" if derive else "hand-written"}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("program", choices=["sgd", "adam", "lamb", "nesterov"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--log2", type=int, default=24, help="log2 of the element count")
    ap.add_argument("--epochs", type=int, default=20)
    ap.add_argument("--derive", action="store_true",
                    help="derive the schedules from the AllReduce program with the C++ Autotuner")
    a = ap.parse_args()
    print(json.dumps(autotune(a.program, a.gpus, a.log2, a.epochs,
                              {"beta1": 0.9, "beta2": 0.999, "lr": 0.01, "decay": 0.01, "mu": 0.9},
                              derive=a.derive)))
