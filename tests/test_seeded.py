"""The counter-based input generator: torch and numpy must produce the same
bits (the benchmark fills buffers on the device and its parity checker
regenerates windows of them on the host), with the stated distributions."""
import numpy as np
import pytest
import torch

import seeded as S


@pytest.mark.parametrize("tdt,ndt", [(torch.float16, np.float16), (torch.float32, np.float32)])
def test_normal_torch_cpu_equals_numpy_bit_for_bit(tdt, ndt):
    n, first = 200_003, 333_900_000
    t = torch.empty(n, dtype=tdt)
    S.fill_normal_(t, 5, 3, 17, 1.024, first=first, chunk=1 << 16)
    h = S.normal_np(np.arange(first, first + n), 5, 3, 17, 1.024, ndt)
    bits = np.uint16 if ndt == np.float16 else np.uint32
    assert np.array_equal(t.numpy().view(bits), h.view(bits))


def test_uniform_torch_cpu_equals_numpy_and_range():
    n = 1 << 18
    t = torch.empty(n)
    S.fill_uniform_(t, 1, 0, 2)
    h = S.uniform_np(np.arange(n), 1, 0, 2)
    assert np.array_equal(t.numpy(), h)
    assert h.min() >= -1.0 and h.max() < 1.0 and abs(float(h.mean())) < 0.01
    assert abs(float(h.std()) - 1 / np.sqrt(3)) < 0.01


def test_normal_moments_and_independence_of_streams():
    idx = np.arange(1 << 20)
    a = S.normal_np(idx, 9, 0, 0, 1e-3).astype(np.float64)
    b = S.normal_np(idx, 9, 1, 0, 1e-3).astype(np.float64)
    c = S.normal_np(idx, 9, 0, 1, 1e-3).astype(np.float64)
    for x in (a, b, c):
        assert abs(x.mean()) < 1e-5 and abs(x.std() - 1e-3) < 2e-5
        assert abs(((x / 1e-3) ** 4).mean() - 3.0) < 0.2      # kurtosis close to a normal's
    assert abs(np.corrcoef(a, b)[0, 1]) < 0.01 and abs(np.corrcoef(a, c)[0, 1]) < 0.01
    # a window of a tensor equals the same elements of the whole
    w = S.normal_np(idx[1000:2000], 9, 0, 0, 1e-3)
    assert np.array_equal(w, S.normal_np(idx, 9, 0, 0, 1e-3)[1000:2000])


@pytest.mark.gpu
def test_device_fill_equals_host_windows():
    n = (1 << 22) + 5
    t = torch.empty(n, dtype=torch.float16, device="cuda")
    S.fill_normal_(t, 20240229, 6, 3, 1.024)
    idx = np.concatenate([np.arange(0, 4096), np.arange(n - 4096, n)])
    h = S.normal_np(idx, 20240229, 6, 3, 1.024, np.float16)
    got = t[torch.from_numpy(idx).cuda()].cpu().numpy()
    assert np.array_equal(got.view(np.uint16), h.view(np.uint16))
    u = torch.empty(n, device="cuda")
    S.fill_uniform_(u, 20240229, 0, 0)
    assert np.array_equal(u[:4096].cpu().numpy(), S.uniform_np(np.arange(4096), 20240229, 0, 0))
