"""Counter-based synthetic inputs that a GPU and the host produce bit for bit.

The benchmark fills 334 M-element gradient buffers on the device; its parity
checker must know a few windows of them on the host without copying gigabytes
back or replaying a stateful generator.  So every element is a pure function of
(seed, stream, step, index): a 64-bit mix of the index, cut into 16-bit
fields whose sum approximates a normal variate (Irwin-Hall, 8 uniforms), then
ONE float32 multiplication and (for 16-bit tensors) ONE rounding -- integer
arithmetic plus two IEEE operations, identical in torch on the device and in
numpy on the host.  No transcendental function is involved: those differ in
the last bit between libraries.

  normal(...)   ~ N(0, std) to a good approximation (|x| <= 4.9 std)
  uniform(...)  ~ U[-1, 1) on a 2^-23 grid
"""
import numpy as np

_M64 = (1 << 64) - 1
_C1, _C2 = 0xBF58476D1CE4E5B9, 0x94D049BB133111EB
_GOLD = 0x9E3779B97F4A7C15
# sum of 8 uniform 16-bit integers: mean 8 * 65535 / 2, variance 8 * (65536^2 - 1) / 12
_IH_MEAN = 4 * 65535
_IH_STD = float(np.sqrt(8.0 * (65536.0 ** 2 - 1.0) / 12.0))


def _key(seed, stream, step, salt):
    """64-bit key of one tensor: splitmix64 over the identifying integers."""
    x = (seed * _GOLD + stream * _C1 + step * _C2 + salt * 0xD6E8FEB86659FD93) & _M64
    x ^= x >> 30
    x = (x * _C1) & _M64
    x ^= x >> 27
    x = (x * _C2) & _M64
    x ^= x >> 31
    return x


def _signed(x):
    return x - (1 << 64) if x >= (1 << 63) else x


# ---- numpy (host) -------------------------------------------------------------------
def _mix_np(idx, key):
    x = idx.astype(np.uint64) ^ np.uint64(key)
    with np.errstate(over="ignore"):
        x ^= x >> np.uint64(30)
        x *= np.uint64(_C1)
        x ^= x >> np.uint64(27)
        x *= np.uint64(_C2)
        x ^= x >> np.uint64(31)
    return x


def _fields_np(x):
    m = np.uint64(0xFFFF)
    return ((x & m) + ((x >> np.uint64(16)) & m) + ((x >> np.uint64(32)) & m)
            + (x >> np.uint64(48))).astype(np.int64)


def normal_np(idx, seed, stream, step, std, dtype=np.float32):
    """Elements `idx` (integer array of global indices) of the tensor."""
    s = _fields_np(_mix_np(idx, _key(seed, stream, step, 1))) + \
        _fields_np(_mix_np(idx, _key(seed, stream, step, 2)))
    c = (s - _IH_MEAN).astype(np.float32)                 # exact: |c| < 2^19
    return (c * np.float32(std / _IH_STD)).astype(dtype)  # one multiply, one rounding


def uniform_np(idx, seed, stream, step, dtype=np.float32):
    x = _mix_np(idx, _key(seed, stream, step, 3))
    c = ((x & np.uint64(0xFFFFFF)).astype(np.int64) - (1 << 23)).astype(np.float32)
    return (c * np.float32(2.0 ** -23)).astype(dtype)


# ---- torch (device) -----------------------------------------------------------------
def _lsr(x, k):
    """Logical shift right of an int64 tensor (torch's >> is arithmetic)."""
    return (x >> k) & ((1 << (64 - k)) - 1)


def _mix_t(idx, key):
    x = idx ^ _signed(key)
    x = x ^ _lsr(x, 30)
    x = x * _signed(_C1)          # wraps modulo 2^64
    x = x ^ _lsr(x, 27)
    x = x * _signed(_C2)
    x = x ^ _lsr(x, 31)
    return x


def _fields_t(x):
    return (x & 0xFFFF) + ((x >> 16) & 0xFFFF) + ((x >> 32) & 0xFFFF) + _lsr(x, 48)


def fill_normal_(t, seed, stream, step, std, first=0, chunk=1 << 25):
    """Fills the 1-D torch tensor `t` (fp32 / fp16 / bf16, any device) with
    elements first .. first + len(t) - 1 of the tensor (seed, stream, step)."""
    import torch
    scale = float(np.float32(std / _IH_STD))
    k1, k2 = _key(seed, stream, step, 1), _key(seed, stream, step, 2)
    n = t.numel()
    for a in range(0, n, chunk):
        b = min(n, a + chunk)
        idx = torch.arange(first + a, first + b, dtype=torch.int64, device=t.device)
        s = _fields_t(_mix_t(idx, k1)) + _fields_t(_mix_t(idx, k2))
        c = (s - _IH_MEAN).to(torch.float32)
        t[a:b] = (c * scale).to(t.dtype)
    return t


def fill_uniform_(t, seed, stream, step, first=0, chunk=1 << 25):
    import torch
    k = _key(seed, stream, step, 3)
    n = t.numel()
    for a in range(0, n, chunk):
        b = min(n, a + chunk)
        idx = torch.arange(first + a, first + b, dtype=torch.int64, device=t.device)
        c = ((_mix_t(idx, k) & 0xFFFFFF) - (1 << 23)).to(torch.float32)
        t[a:b] = (c * float(2.0 ** -23)).to(t.dtype)
    return t
