"""CPU restatement of the index arithmetic of the single-rank 8-element units
(direct_step in coconet_b200/csrc/fused_step.cu): a warp's 32 units are 256
consecutive elements, lane t takes 4t..4t+3 and 128+4t..128+4t+3; the last,
partial warp of units falls back to 8 consecutive elements per lane; one
4-element unit may remain.  Every element must be touched exactly once, every
access must start on a 16-byte boundary relative to `first`, and a warp's
access must be one contiguous run."""
import numpy as np
import pytest


def units_8(nelems, nth):
    """(thread, [element offsets of its accesses, each 4 long]) as the kernel issues them."""
    assert nelems % 4 == 0 and nth % 32 == 0
    nunits = nelems // 8
    nfull = nunits // 32 * 32
    out = []
    for tid in range(nth):
        u = tid
        while u < nfull:
            i = u * 8 - (u & 31) * 4
            out.append((tid, u, [i, i + 128]))
            u += nth
        u = nfull + tid
        while u < nunits:
            out.append((tid, u, [u * 8, u * 8 + 4]))
            u += nth
        if (nelems & 4) and tid == 0:
            out.append((tid, -1, [nunits * 8]))
    return out


@pytest.mark.parametrize("nelems", [0, 4, 8, 252, 256, 260, 1024 + 8 * 31 + 4, 8 * 32 * 7, 100000])
@pytest.mark.parametrize("nth", [32, 64, 512 * 3])
def test_every_element_once_and_aligned(nelems, nth):
    seen = np.zeros(nelems, np.int32)
    for _, _, starts in units_8(nelems, nth):
        for s in starts:
            assert s % 4 == 0 and 0 <= s and s + 4 <= nelems
            seen[s:s + 4] += 1
    assert (seen == 1).all()


def test_full_warps_access_contiguous_runs():
    nelems, nth = 8 * 32 * 5, 64
    by_unit = {u: starts for _, u, starts in units_8(nelems, nth) if u >= 0}
    for warp_first in range(0, 32 * 5, 32):
        first_half = sorted(by_unit[warp_first + lane][0] for lane in range(32))
        second_half = sorted(by_unit[warp_first + lane][1] for lane in range(32))
        assert first_half == list(range(warp_first * 8, warp_first * 8 + 128, 4))
        assert second_half == list(range(warp_first * 8 + 128, warp_first * 8 + 256, 4))


def test_rotated_start_of_a_shared_piece_keeps_lanes():
    # the list kernels start a shared piece at thread (tid + piece * 37 * blockDim) % nth:
    # the lane of a thread must not change, or u & 31 would not be the lane
    block, grid = 512, 296
    nth = block * grid
    for piece in (0, 1, 5, 397):
        for tid in (0, 31, 32, 511, 512, nth - 1):
            assert ((tid + piece * 37 * block) % nth) % 32 == tid % 32
