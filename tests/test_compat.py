"""include/coconet_compat.h: the forked NCCL's `AllReduce_pipe` in the four
arities the fork and its frozen test programs use, as overloads over the C
ABI.  tests/compat_prog.cu is written like those programs (host check after
every call).  CPU: it compiles for sm_100a.  GPU: it runs and every check
passes."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
LIBDIR = os.path.join(ROOT, "coconet_b200")


def _build(tmp_path, link):
    # links against the in-tree library as it is (never rebuilt from a test: the
    # test process may have it loaded)
    assert os.path.exists(os.path.join(LIBDIR, "libcoconet_rt.so")), "build the library first"
    out = str(tmp_path / ("compat_prog" if link else "compat_prog.o"))
    cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17",
           "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "compat_prog.cu"), "-o", out]
    cmd += (["-L", LIBDIR, "-lcoconet_rt", "-Xlinker", "-rpath", "-Xlinker", LIBDIR] if link else ["-c"])
    subprocess.check_call(cmd)
    return out


def test_frozen_style_program_compiles_against_the_compat_header(tmp_path):
    _build(tmp_path, link=False)
    _build(tmp_path, link=True)      # every overload resolves to an exported entry point


@pytest.mark.gpu
def test_frozen_style_program_passes_its_host_checks(tmp_path):
    exe = _build(tmp_path, link=True)
    env = dict(os.environ, RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", MASTER_ADDR="127.0.0.1",
               MASTER_PORT="29879")
    r = subprocess.run([exe, "10007"], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.split() == ["PASSED", "sgd", "PASSED", "adam", "PASSED", "adam-mixed",
                                "PASSED", "lamb"], r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("R", [2, 3])
def test_frozen_style_program_with_virtual_ranks_on_one_gpu(tmp_path, R):
    # the four arities at more than one rank without more than one GPU: all R
    # ranks live in the process (cocoCommInitAll, device 0 listed R times) and
    # each AllReduce_pipe round is one grouped launch
    exe = _build(tmp_path, link=True)
    env = dict(os.environ, COMPAT_VIRTUAL_RANKS=str(R))
    r = subprocess.run([exe, "10007"], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.split() == ["PASSED", "sgd", "PASSED", "adam", "PASSED", "adam-mixed",
                                "PASSED", "lamb"], r.stdout
