"""Multi-process parity: one process per GPU over CUDA IPC peer memory, the
product path for R > 1.  Needs at least two GPUs; skipped otherwise (the same
kernel code runs in tests/test_fused_gpu.py with virtual ranks on one GPU)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _why(r):
    k = r.stdout.find("WORKER FAILURE")
    return (r.stdout[k:k + 4000] if k >= 0 else r.stdout[-3000:]) + r.stderr[-1500:]


def _launch(case, world, timeout=600, extra_env=None):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ)
    # plain peer loads only; no NVLS anywhere in these child processes
    env.update(NCCL_NVLS_ENABLE="0", COCO_TIMEOUT_MS=env.get("COCO_TIMEOUT_MS", "5000"))
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(HERE, "mp_worker.py"), case]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)


@pytest.mark.skipif(_ngpu() < 2, reason="needs >= 2 GPUs")
def test_parity_all_gpus():
    world = min(_ngpu(), 8)
    r = _launch("parity", world)
    assert r.returncode == 0, _why(r)
    assert r.stdout.count("ok ") >= 8, r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs >= 2 GPUs")
def test_parity_through_the_warp_rings_all_gpus():
    # the same cases with the gradients staged by bulk copies out of the peers'
    # IPC-mapped memory (COCO_PIPELINE=1): bit-exact like the register-staged path
    world = min(_ngpu(), 8)
    r = _launch("parity", world, extra_env={"COCO_PIPELINE": "1"})
    assert r.returncode == 0, _why(r)
    assert r.stdout.count("ok ") >= 8, r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs >= 2 GPUs")
def test_absent_rank_times_out_cleanly():
    r = _launch("timeout", 2)
    assert r.returncode == 0, _why(r)
    assert "ok timeout" in r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs >= 2 GPUs")
def test_nvls_multicast_path():
    world = min(_ngpu(), 8)
    r = _launch("nvls", world)
    assert r.returncode == 0, _why(r)
    assert "ok nvls_lamb_fp32" in r.stdout or "skip nvls" in r.stdout, r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs >= 2 GPUs")
@pytest.mark.parametrize("opt,schedule", [("adam", "fuse_RS_C_AG"), ("lamb", "fuse_RS_C_AG"),
                                          ("sgd", "RS_C_AG"), ("nesterov", "fuse_RS_C_AG"),
                                          ("lamb", "RS_C_AG"), ("adam", "AR_C"),
                                          ("adam_derived", "RS_C_AG"),
                                          ("adam_derived", "fuse_RS_C_AG"),
                                          ("adam_mixed", "fuse_RS_C_AG")])
def test_emitted_program_multi_rank(tmp_path, opt, schedule):
    """A DSL-emitted C++ program, one process per GPU, started without MPI."""
    import dsl_build_util as B
    exe = B.build_program(opt, schedule, str(tmp_path))
    world = min(_ngpu(), 8)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **B.SCALARS)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--no-python", "--nnodes=1",
           f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", str(port),
           exe, "3", "12", "20", "check"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert r.stdout.count("PASSED") == 8 * world and "FAILED" not in r.stdout
    assert "{SZ: 524288, Epochs: 3" in r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs >= 2 GPUs")
def test_runtime_symmetric_memory_and_multicast():
    world = min(_ngpu(), 8)
    r = _launch("symm", world)
    assert r.returncode == 0, _why(r)
    assert "ok symm_p2p" in r.stdout and "ok symm_free_realloc" in r.stdout, r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs >= 2 GPUs")
def test_scattered_tensor_lists_across_processes():
    r = _launch("scattered", min(_ngpu(), 8))
    assert r.returncode == 0, _why(r)
    assert "ok scattered" in r.stdout and "ok scattered_lamb" in r.stdout, r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs >= 2 GPUs")
def test_stand_alone_collectives():
    r = _launch("collectives", min(_ngpu(), 8))
    assert r.returncode == 0, _why(r)
    assert "ok collectives" in r.stdout, r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs >= 2 GPUs")
def test_topology_table_and_link_probe():
    r = _launch("probe", min(_ngpu(), 8))
    assert r.returncode == 0, _why(r)
    assert "ok probe" in r.stdout, r.stdout
