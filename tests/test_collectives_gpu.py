"""Stand-alone collectives (cocoAllReduce / cocoReduceScatter / cocoAllGather:
what the unfused schedules of a generated program call where the reference
emits ncclAllReduce / ncclReduceScatter / ncclAllGather, src/codegen.cpp:
4146-4189) with R virtual ranks on ONE GPU: the R calls of a round are grouped
into one cooperative launch.  fp32 sums in rank order, so results equal numpy's
left-to-right sum bit for bit."""
import numpy as np
import pytest
import torch

import cases as K

pytestmark = pytest.mark.gpu

import coconet_b200 as coco  # noqa: E402


@pytest.mark.parametrize("R", [2, 3, 8])
@pytest.mark.parametrize("n", [5, 4099, (1 << 18) + 8])
def test_collectives_with_virtual_ranks(R, n):
    comms = coco.Communicator.init_all(R, [0] * R)
    try:
        rng = np.random.default_rng((R, n))
        xs = [rng.standard_normal(n).astype(np.float32) for _ in range(R)]
        want = xs[0].copy()
        for r in range(1, R):
            want = want + xs[r]
        S = (n + R - 1) // R
        # all-reduce in place
        bufs = [torch.from_numpy(x.copy()).cuda() for x in xs]
        with coco.group():
            for r, c in enumerate(comms):
                c.all_reduce(bufs[r])
        torch.cuda.synchronize()
        for r in range(R):
            assert np.array_equal(bufs[r].cpu().numpy(), want), f"all_reduce rank {r}"
        # reduce-scatter: recv[0 .. S_r) = sum of the ranks' send[lo_r .. hi_r)
        sends = [torch.from_numpy(x.copy()).cuda() for x in xs]
        recvs = [torch.full((S,), -7.0, device="cuda") for _ in range(R)]
        with coco.group():
            for r, c in enumerate(comms):
                c.reduce_scatter(sends[r], recvs[r])
        torch.cuda.synchronize()
        for r in range(R):
            lo, hi = K.slice_bounds(n, R, r)
            got = recvs[r].cpu().numpy()
            assert np.array_equal(got[: hi - lo], want[lo:hi]), f"reduce_scatter rank {r}"
            assert np.all(got[hi - lo:] == -7.0)                      # nothing written past the slice
            assert np.array_equal(sends[r].cpu().numpy(), xs[r])      # the input is only read
        # all-gather of those slices gives the whole sum everywhere
        fulls = [torch.zeros(n, device="cuda") for _ in range(R)]
        with coco.group():
            for r, c in enumerate(comms):
                c.all_gather(recvs[r], fulls[r])
        torch.cuda.synchronize()
        for r in range(R):
            assert np.array_equal(fulls[r].cpu().numpy(), want), f"all_gather rank {r}"
        for c in comms:
            assert c.status()["code"] == 0
    finally:
        for c in comms:
            c.destroy()


def test_collective_rounds_must_agree_across_ranks():
    comms = coco.Communicator.init_all(2, [0, 0])
    try:
        a = torch.zeros(64, device="cuda")
        b = torch.zeros(64, device="cuda")
        with pytest.raises(coco.CocoError) as e:
            with coco.group():
                comms[0].all_reduce(a)
                comms[1].all_gather(b[:32], b)     # another collective than rank 0's
        assert e.value.code == 2                   # invalid usage, nothing launched
        with coco.group():                         # the communicators stay usable
            comms[0].all_reduce(a)
            comms[1].all_reduce(b)
        torch.cuda.synchronize()
    finally:
        for c in comms:
            c.destroy()
