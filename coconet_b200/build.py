"""Builds libcoconet_rt.so (the C-ABI runtime + sm_100a kernels) in-tree."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libcoconet_rt.so")
SOURCES = ["fused_step.cu", "runtime.cu", "bootstrap.cpp", "no_alloc.cu", "symm_mem.cu", "collectives.cu",
           "link_probe.cu"]
HEADERS = ["fused_step.cuh", "bootstrap.h", os.path.join(ROOT, "include", "coconet_rt.h"),
           os.path.join(ROOT, "include", "coconet_device.h"),
           os.path.join(ROOT, "include", "coconet_fused_generic.cuh")]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + [
        h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force=False, verbose=False, checked=False):
    """Compile for sm_100a only; returns the path of the shared library.  The
    kernel file is compiled as four parts in parallel (see COCO_PART in
    fused_step.cu).  `checked` builds libcoconet_rt_checked.so beside it: the
    same library with per-unit bounds and alignment checks in the kernels that
    record cocoInternalError in the status word (load it with
    COCO_RT_LIBRARY=<that file>)."""
    if checked:
        return _build(os.path.join(HERE, "libcoconet_rt_checked.so"), os.path.join(HERE, "build", "checked"),
                      ["-DCOCO_CHECKED=1"], verbose)
    if not force and not _stale():
        return LIB
    return _build(LIB, os.path.join(HERE, "build"), [], verbose)


def _build(lib, objdir, extra, verbose):
    from concurrent.futures import ThreadPoolExecutor
    os.makedirs(objdir, exist_ok=True)
    base = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
            "-Xcompiler", "-fPIC", "-diag-suppress", "177", "-I" + os.path.join(ROOT, "include"), "-I" + CSRC] + extra
    if verbose:
        base += ["-Xptxas", "-v"]
    jobs = []
    for part in range(4):
        obj = os.path.join(objdir, f"fused_step_{part}.o")
        jobs.append((base + [f"-DCOCO_PART={part}", "-c", os.path.join(CSRC, "fused_step.cu"), "-o", obj], obj))
    for src in SOURCES:
        if src == "fused_step.cu":
            continue
        obj = os.path.join(objdir, os.path.splitext(src)[0] + ".o")
        jobs.append((base + ["-c", os.path.join(CSRC, src), "-o", obj], obj))
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        list(pool.map(lambda j: subprocess.check_call(j[0]), jobs))
    subprocess.check_call([NVCC, "-shared", "-cudart", "shared", "-Wno-deprecated-gpu-targets", "-o", lib] + [j[1] for j in jobs])
    return lib


if __name__ == "__main__":
    print(build_library(force=True, verbose="-v" in os.sys.argv, checked="--checked" in os.sys.argv))
