"""CPU-only checks of the host side: the C-ABI library loads and exports every
declared entry point, slice bounds, argument validation that needs no device,
and the TCP rendezvous with 2-4 processes (including its failure modes)."""
import multiprocessing as mp
import os
import re
import socket
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import coconet_b200 as coco  # noqa: E402
from coconet_b200 import runtime as rt  # noqa: E402


def test_library_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "coconet_rt.h")).read()
    declared = set(re.findall(r"^(?:int|const char \*)\s*(coco[A-Za-z]+)\(", hdr, re.M))
    assert len(declared) >= 25
    L = coco.lib()
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} declared in coconet_rt.h but not exported"
    assert declared == set(rt._SIGNATURES), declared ^ set(rt._SIGNATURES)


def test_version_and_error_strings():
    import ctypes as C
    v = C.c_int()
    assert coco.lib().cocoGetVersion(C.byref(v)) == 0 and v.value == 100
    assert rt.error_string(0) == "success"
    assert "timed out" in rt.error_string(5)
    assert "unknown" in rt.error_string(1234)


@pytest.mark.parametrize("n,R", [(0, 1), (1, 8), (10, 4), (334_000_000, 8), (1 << 20, 2), (4099, 3)])
def test_slice_bounds_partition(n, R):
    S = -(-n // R) if n else 0
    prev = 0
    for r in range(R):
        lo, hi = coco.slice_bounds(n, R, r)
        assert lo == min(n, r * S) and hi == min(n, lo + S) and lo == prev
        prev = hi
    assert prev == n
    with pytest.raises(coco.CocoError):
        coco.slice_bounds(n, R, R)


@pytest.mark.parametrize("R", [1, 2, 3, 8])
def test_scattered_layout_places_every_tensor(R):
    # the flat layout of a list of tensors: 8-element alignment per tensor, slices a
    # multiple of 8, every element of every tensor on exactly one rank
    counts = [1000, 8, 3, 0, 4096, 70001, 2, 1, (1 << 19) + 5, 24]
    S = coco.scattered_slice_elems(counts, R)
    at = 0
    owned = [0] * R
    for b, c in enumerate(counts):
        off, r0, r1 = coco.scattered_tensor_place(counts, R, b)
        assert off == at and off % 8 == 0
        if c == 0:
            assert (r0, r1) == (-1, -1)
        else:
            assert (r0, r1) == (off // S, (off + c - 1) // S) and 0 <= r0 <= r1 < R
            for r in range(r0, r1 + 1):
                owned[r] += max(0, min(off + c, (r + 1) * S) - max(off, r * S))
        at += (c + 7) // 8 * 8
    assert S % 8 == 0 and S * R >= at and sum(owned) == sum(counts) and max(owned) <= S
    with pytest.raises(coco.CocoError):
        coco.scattered_tensor_place(counts, R, len(counts))


def test_null_handles_are_rejected_not_dereferenced():
    import ctypes as C
    L = coco.lib()
    assert L.cocoCommDestroy(None) == 1
    assert L.cocoBarrier(None) == 1
    assert L.cocoFusedSGD(None, None, 7, None, None, 6, 16, 0.1, 1.0, None) == 1
    assert L.cocoGroupEnd() == 2  # no matching cocoGroupStart
    st = rt._Status()
    assert L.cocoGetStatus(None, C.byref(st)) == 1
    assert L.cocoCommInitRank(None, 2, 0, None) == 1
    h = C.c_void_p()
    assert L.cocoCommInitRank(C.byref(h), 9, 0, None) == 1  # more than COCO_MAX_RANKS
    assert L.cocoCommInitRank(C.byref(h), 2, 2, None) == 1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _bs_worker(world, rank, port, q, mode):
    try:
        if mode == "late" and rank == 1:
            time.sleep(1.0)
        if mode == "absent" and rank == world - 1:
            q.put((rank, "skipped"))
            return
        bs = coco.HostBootstrap(world, rank, f"127.0.0.1:{port}", timeout_ms=1500 if mode == "absent" else 20000)
        if mode in ("size_mismatch", "kind_mismatch"):
            bs.barrier()
            try:  # rank 1 is in another collective than the rest: every rank must be told
                if mode == "size_mismatch":
                    bs.all_gather(bytes(64 if rank == 1 else 8))
                elif rank == 1:
                    bs.all_gather(b"x")
                else:
                    bs.barrier()
                first = "passed"
            except coco.CocoError as e:
                first = f"error {e.code}"
            try:  # and the connection stays refused afterwards
                bs.barrier()
                second = "passed"
            except coco.CocoError as e:
                second = f"error {e.code}"
            bs.close()
            q.put((rank, (first, second)))
            return
        out = []
        for rnd in range(3):
            blob = bytes([rank, rnd]) * 50
            got = bs.all_gather(blob)
            out.append(all(got[r] == bytes([r, rnd]) * 50 for r in range(world)))
            bs.barrier()
        big = bytes([rank]) * (1 << 20)
        got = bs.all_gather(big)
        out.append(all(got[r] == bytes([r]) * (1 << 20) for r in range(world)))
        bs.close()
        q.put((rank, all(out)))
    except coco.CocoError as e:
        q.put((rank, f"error {e.code}"))


def _run(world, mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_bs_worker, args=(world, r, port, q, mode)) for r in range(world)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=60) for _ in ps)
    for p in ps:
        p.join(timeout=30)
    return res


@pytest.mark.parametrize("world", [2, 4])
def test_bootstrap_all_gather_and_barrier(world):
    assert _run(world, "normal") == {r: True for r in range(world)}


def test_bootstrap_tolerates_a_late_rank():
    assert _run(2, "late") == {0: True, 1: True}


def test_bootstrap_times_out_when_a_rank_never_joins():
    res = _run(3, "absent")
    assert res[2] == "skipped"
    assert res[0] == "error 5"  # rank 0 gives up in accept()
    assert res[1].startswith("error")  # connected, then the root went away


@pytest.mark.parametrize("mode", ["size_mismatch", "kind_mismatch"])
def test_bootstrap_refuses_ranks_that_are_out_of_step(mode):
    # a rank in a different collective (other size, or an all-gather against a
    # barrier) must not have its bytes taken for the others': invalid usage (2)
    # on every rank, then and afterwards
    res = _run(3, mode)
    assert res == {r: ("error 2", "error 2") for r in range(3)}


def test_topology_rule_on_fake_tables():
    # what cocoCommInitRank applies to the gathered cudaDeviceGetP2PAttribute rows
    R = 4
    full = [[1] * R for _ in range(R)]
    flat_perf = [[0] * R for _ in range(R)]
    assert coco.topology_check(R, full, flat_perf) == (0, True)           # NVSwitch: all equal
    ring = [[0 if a == b else (0 if abs(a - b) in (1, R - 1) else 1) for b in range(R)] for a in range(R)]
    assert coco.topology_check(R, full, ring) == (0, False)               # unequal performance ranks
    cut = [row[:] for row in full]
    cut[2][3] = 0
    assert coco.topology_check(R, cut, flat_perf)[0] == 6                 # cocoPeerError
    unknown = [row[:] for row in full]
    unknown[0][1] = -1
    assert coco.topology_check(R, unknown, flat_perf) == (0, False)       # the driver did not say
    assert coco.topology_check(1, [[1]], [[0]]) == (0, True)
    assert coco.lib().cocoTopologyCheck(9, None, None, None) == 1


# ---- world-size-2 host path under torch.distributed (gloo, CPU) --------------

def _gloo_worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        addr = coco.rendezvous_address()           # rank 0 picks a port, everyone learns it
        bs = coco.HostBootstrap(world, rank, addr, timeout_ms=20000)
        # every rank computes every rank's slice; the shards must tile [0, count)
        count = 334_000_000
        mine = "%d:%d" % coco.slice_bounds(count, world, rank)
        got = [b.decode().rstrip("\0") for b in bs.all_gather(mine.encode().ljust(32, b"\0"))]
        bs.barrier()
        bs.close()
        q.put((rank, addr, got))
    finally:
        dist.destroy_process_group()


def test_gloo_world_2_rendezvous_and_sharding():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = sorted(q.get(timeout=120) for _ in ps)
    for p in ps:
        p.join(timeout=30)
    assert res[0][1] == res[1][1]                      # the same address on both ranks
    assert res[0][2] == res[1][2] == ["0:167000000", "167000000:334000000"]
