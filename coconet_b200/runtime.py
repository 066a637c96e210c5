"""ctypes host layer over libcoconet_rt.so (see include/coconet_rt.h).

Tensors are torch CUDA tensors; only their device pointers cross the C ABI.
"""
import contextlib
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))

VARIANT_OVERLAP, VARIANT_DSL, VARIANT_NCCL = 0, 1, 2
LAMB_REF_QUIRK = 0x1
_F16, _F32, _BF16 = 6, 7, 9


class CocoError(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        super().__init__(f"{what}: {error_string(code)} ({code})")


class _Topology(C.Structure):
    _fields_ = [("world", C.c_int), ("access", (C.c_int * 8) * 8), ("perf_rank", (C.c_int * 8) * 8),
                ("native_atomics", (C.c_int * 8) * 8), ("uniform", C.c_int)]


class _Status(C.Structure):
    _fields_ = [("code", C.c_int), ("rank", C.c_int), ("phase", C.c_int), ("peer", C.c_int),
                ("seq", C.c_uint64)]


def library_path():
    """The in-tree library; COCO_RT_LIBRARY points at another build (A/B runs)."""
    return os.environ.get("COCO_RT_LIBRARY") or os.path.join(HERE, "libcoconet_rt.so")


_lib = None

# name -> (restype, argtypes); also the list the symbol-export test checks.
_SIGNATURES = {
    "cocoGetVersion": (C.c_int, [C.POINTER(C.c_int)]),
    "cocoErrorString": (C.c_char_p, [C.c_int]),
    "cocoCommInitRank": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_char_p]),
    "cocoCommInitAll": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.POINTER(C.c_int)]),
    "cocoCommDestroy": (C.c_int, [C.c_void_p]),
    "cocoCommCount": (C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
    "cocoCommUserRank": (C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
    "cocoCommCuDevice": (C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
    "cocoCommTopology": (C.c_int, [C.c_void_p, C.POINTER(_Topology)]),
    "cocoTopologyCheck": (C.c_int, [C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int),
                                    C.POINTER(C.c_int)]),
    "cocoBarrier": (C.c_int, [C.c_void_p]),
    "cocoAllGatherHost": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "cocoBootstrapInit": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_char_p, C.c_int]),
    "cocoBootstrapAllGather": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "cocoBootstrapBarrier": (C.c_int, [C.c_void_p]),
    "cocoBootstrapDestroy": (C.c_int, [C.c_void_p]),
    "cocoEnvRank": (C.c_int, [C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "cocoGroupStart": (C.c_int, []),
    "cocoGroupEnd": (C.c_int, []),
    "cocoRegister": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "cocoDeregister": (C.c_int, [C.c_void_p, C.c_void_p]),
    "cocoRegisterMapped": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p),
                                     C.c_void_p]),
    "cocoSetAlgo": (C.c_int, [C.c_void_p, C.c_int]),
    "cocoMemAlloc": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.c_size_t]),
    "cocoMemFree": (C.c_int, [C.c_void_p, C.c_void_p]),
    "cocoMemHasMulticast": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int)]),
    "cocoFusedSGD": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                               C.c_size_t, C.c_float, C.c_float, C.c_void_p]),
    "cocoFusedAdam": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                                C.c_void_p, C.c_void_p, C.c_size_t, C.c_float, C.c_float,
                                C.c_float, C.c_float, C.c_int, C.c_float, C.c_int, C.c_void_p]),
    "cocoFusedLAMB": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                                C.c_void_p, C.c_void_p, C.c_size_t, C.c_float, C.c_float,
                                C.c_float, C.c_float, C.c_float, C.c_int, C.c_float, C.c_int,
                                C.c_uint, C.c_void_p]),
    "cocoLambStepNoAlloc": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                                      C.c_void_p, C.c_void_p, C.c_size_t, C.c_float, C.c_float,
                                      C.c_float, C.c_float, C.c_float, C.c_int, C.c_float,
                                      C.c_void_p]),
    "cocoScatteredSliceElems": (C.c_int, [C.c_size_t, C.POINTER(C.c_size_t), C.c_int,
                                          C.POINTER(C.c_size_t)]),
    "cocoScatteredTensorPlace": (C.c_int, [C.c_size_t, C.POINTER(C.c_size_t), C.c_int, C.c_size_t,
                                           C.POINTER(C.c_size_t), C.POINTER(C.c_int),
                                           C.POINTER(C.c_int)]),
    "cocoFusedSGDScattered": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p), C.c_int,
                                        C.POINTER(C.c_void_p), C.POINTER(C.c_size_t), C.c_float,
                                        C.c_float, C.c_void_p]),
    "cocoFusedAdamScattered": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p), C.c_int,
                                         C.POINTER(C.c_void_p), C.POINTER(C.c_size_t), C.c_void_p,
                                         C.c_void_p, C.c_float, C.c_float, C.c_float, C.c_float,
                                         C.c_int, C.c_float, C.c_int, C.c_void_p]),
    "cocoFusedLAMBScattered": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p), C.c_int,
                                         C.POINTER(C.c_void_p), C.POINTER(C.c_size_t), C.c_void_p,
                                         C.c_void_p, C.c_float, C.c_float, C.c_float, C.c_float,
                                         C.c_float, C.c_int, C.c_float, C.c_int, C.c_uint,
                                         C.c_void_p]),
    "cocoAllReduce": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "cocoReduceScatter": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "cocoAllGather": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "cocoFusedGenericPlan": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_size_t,
                                       C.c_float, C.c_void_p, C.c_void_p]),
    "cocoLinkProbe": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_int,
                                C.POINTER(C.c_double), C.c_void_p]),
    "cocoLastLambNorms": (C.c_int, [C.c_void_p, C.POINTER(C.c_double)]),
    "cocoLastPhaseTimes": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "cocoLastCtaSpread": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "cocoGetStatus": (C.c_int, [C.c_void_p, C.POINTER(_Status)]),
    "cocoSliceBounds": (C.c_int, [C.c_size_t, C.c_int, C.c_int, C.POINTER(C.c_size_t),
                                  C.POINTER(C.c_size_t)]),
    "cocoSetTunables": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "cocoLaunchCount": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64)]),
}


def lib():
    """The loaded C-ABI library.  Raises if it has not been built: there is no
    fallback path."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise ImportError(
                f"{path} is missing: build it with `python -m coconet_b200.build` "
                "(or __graft_entry__.build()); coconet_b200 has no fallback path")
        L = C.CDLL(path)
        for name, (res, args) in _SIGNATURES.items():
            if os.environ.get("COCO_RT_LIBRARY") and not hasattr(L, name):
                continue  # an older build under comparison
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def error_string(code):
    return lib().cocoErrorString(code).decode()


def _check(code, what):
    if code != 0:
        raise CocoError(code, what)


def scattered_tensor_place(counts, world, tensor):
    """(flat_offset, first_rank, last_rank) of one tensor of a list in the flat
    Sliced moments of the scattered calls."""
    arr = (C.c_size_t * len(counts))(*counts)
    off, r0, r1 = C.c_size_t(), C.c_int(), C.c_int()
    _check(lib().cocoScatteredTensorPlace(len(counts), arr, world, tensor, C.byref(off),
                                          C.byref(r0), C.byref(r1)), "cocoScatteredTensorPlace")
    return off.value, r0.value, r1.value


def scattered_slice_elems(counts, world):
    """Elements of m / v each rank holds for a list of tensors of these sizes."""
    arr = (C.c_size_t * len(counts))(*counts)
    out = C.c_size_t()
    _check(lib().cocoScatteredSliceElems(len(counts), arr, world, C.byref(out)), "cocoScatteredSliceElems")
    return out.value


def topology_check(world, access, perf_rank):
    """The rule communicators apply to the peer-access table at creation, on a
    table of the caller's (lists of lists; no GPU needed).  Returns (result
    code, uniform)."""
    flat_a = (C.c_int * (world * world))(*[x for row in access for x in row])
    flat_p = (C.c_int * (world * world))(*[x for row in perf_rank for x in row])
    uni = C.c_int()
    rc = lib().cocoTopologyCheck(world, flat_a, flat_p, C.byref(uni))
    return rc, bool(uni.value)


def slice_bounds(count, world, rank):
    lo, hi = C.c_size_t(), C.c_size_t()
    _check(lib().cocoSliceBounds(count, world, rank, C.byref(lo), C.byref(hi)), "cocoSliceBounds")
    return lo.value, hi.value


@contextlib.contextmanager
def group():
    """Fused calls issued inside are launched together on exit (needed when
    several ranks of a single-process communicator share one GPU)."""
    _check(lib().cocoGroupStart(), "cocoGroupStart")
    try:
        yield
    finally:
        _check(lib().cocoGroupEnd(), "cocoGroupEnd")


def _dtype_code(t):
    import torch
    return {torch.float32: _F32, torch.float16: _F16, torch.bfloat16: _BF16}[t.dtype]


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _stream(stream):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def rendezvous_address(pg=None):
    """"host:port" for the runtime's TCP rendezvous, agreed through an
    initialised torch.distributed group (any backend): rank 0 picks a free port
    and broadcasts it."""
    import socket
    import torch.distributed as dist
    box = [None]
    if dist.get_rank(pg) == 0:
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        box[0] = s.getsockname()[1]
        s.close()
    dist.broadcast_object_list(box, src=0, group=pg)
    host = os.environ.get("MASTER_ADDR", "127.0.0.1")
    return f"{host}:{box[0]}"


class HostBootstrap:
    """The runtime's TCP rendezvous on its own (no GPU needed)."""

    def __init__(self, world, rank, addr=None, timeout_ms=0):
        h = C.c_void_p()
        _check(lib().cocoBootstrapInit(C.byref(h), world, rank, addr.encode() if addr else None,
                                       timeout_ms), "cocoBootstrapInit")
        self._h, self.world, self.rank = h, world, rank

    def all_gather(self, blob: bytes):
        recv = C.create_string_buffer(len(blob) * self.world)
        _check(lib().cocoBootstrapAllGather(self._h, blob, recv, len(blob)), "cocoBootstrapAllGather")
        return [recv.raw[i * len(blob):(i + 1) * len(blob)] for i in range(self.world)]

    def barrier(self):
        _check(lib().cocoBootstrapBarrier(self._h), "cocoBootstrapBarrier")

    def close(self):
        if self._h:
            lib().cocoBootstrapDestroy(self._h)
            self._h = None


class TensorList:
    """The pointer and size arrays of a list of (gradient, weight) tensors, made
    once: what a C caller of the `...Scattered` entry points builds before its
    training loop.  Pass it as `gs` (with `ws=None`) to the `fused_*_scattered`
    methods; converting a few hundred tensors on every call costs more host
    time than the step takes on the device."""

    def __init__(self, gs, ws):
        assert len(gs) == len(ws) and len(gs) > 0
        self.tensors = (list(gs), list(ws))   # keeps the memory alive
        self.n = len(gs)
        self.g = (C.c_void_p * self.n)(*[t.data_ptr() for t in gs])
        self.w = (C.c_void_p * self.n)(*[t.data_ptr() for t in ws])
        self.counts = (C.c_size_t * self.n)(*[t.numel() for t in ws])
        self.dtype = _dtype_code(gs[0])


def _list_dtype(gs):
    return gs.dtype if isinstance(gs, TensorList) else _dtype_code(gs[0])


class Communicator:
    """One rank of a fused-step communicator (wraps cocoComm_t)."""

    def __init__(self, handle, world, rank):
        self._h = C.c_void_p(handle)
        self.world = world
        self.rank = rank

    # ---- construction ----
    @classmethod
    def init_rank(cls, world, rank, bootstrap=None):
        """One process per GPU; the current CUDA device becomes the rank's."""
        h = C.c_void_p()
        addr = bootstrap.encode() if bootstrap else None
        _check(lib().cocoCommInitRank(C.byref(h), world, rank, addr), "cocoCommInitRank")
        return cls(h.value, world, rank)

    @classmethod
    def init_all(cls, n, devices=None):
        """All ranks in this process; a device listed twice hosts virtual ranks."""
        hs = (C.c_void_p * n)()
        devs = (C.c_int * n)(*devices) if devices is not None else None
        _check(lib().cocoCommInitAll(hs, n, devs), "cocoCommInitAll")
        return [cls(hs[r], n, r) for r in range(n)]

    @classmethod
    def from_torch_distributed(cls, pg=None):
        """Rendezvous through an initialised torch.distributed group."""
        import torch.distributed as dist
        return cls.init_rank(dist.get_world_size(pg), dist.get_rank(pg), rendezvous_address(pg))

    def destroy(self):
        if self._h:
            lib().cocoCommDestroy(self._h)
            self._h = None

    # ---- host-side collectives ----
    def barrier(self):
        _check(lib().cocoBarrier(self._h), "cocoBarrier")

    def all_gather_host(self, blob: bytes):
        """Every rank's `blob` (same length everywhere), in rank order."""
        recv = C.create_string_buffer(len(blob) * self.world)
        _check(lib().cocoAllGatherHost(self._h, blob, recv, len(blob)), "cocoAllGatherHost")
        return [recv.raw[i * len(blob):(i + 1) * len(blob)] for i in range(self.world)]

    def register(self, t):
        _check(lib().cocoRegister(self._h, _ptr(t), t.numel() * t.element_size()), "cocoRegister")

    def register_mapped(self, t, peer_ptrs, multicast_ptr=0):
        """Register a tensor whose peer mappings (and optional NVLS multicast
        address) the caller already holds, e.g. torch symmetric memory."""
        arr = (C.c_void_p * self.world)(*peer_ptrs)
        _check(lib().cocoRegisterMapped(self._h, _ptr(t), t.numel() * t.element_size(), arr,
                                        C.c_void_p(multicast_ptr or None)), "cocoRegisterMapped")

    def mem_alloc(self, numel, dtype):
        """Collective: a torch tensor over runtime-made symmetric memory (peer
        mappings and, where supported, an NVSwitch multicast mapping).  Free it
        with mem_free before destroying the communicator."""
        import torch
        esize = torch.empty(0, dtype=dtype).element_size()
        p = C.c_void_p()
        _check(lib().cocoMemAlloc(self._h, C.byref(p), numel * esize), "cocoMemAlloc")
        typestr = {torch.float32: "<f4", torch.float16: "<f2", torch.uint8: "|u1"}.get(dtype)
        view_dtype = dtype
        if typestr is None:  # e.g. bfloat16: expose as 16-bit integers, then reinterpret
            typestr, view_dtype = "<i2", torch.int16

        class _Raw:
            __cuda_array_interface__ = {"shape": (numel,), "typestr": typestr,
                                        "data": (p.value, False), "version": 2}
        t = torch.as_tensor(_Raw(), device=torch.device("cuda", torch.cuda.current_device()))
        if view_dtype != dtype:
            t = t.view(dtype)
        self._allocs = getattr(self, "_allocs", {})
        self._allocs[t.data_ptr()] = p.value
        return t

    def mem_free(self, t):
        base = getattr(self, "_allocs", {}).pop(t.data_ptr())
        _check(lib().cocoMemFree(self._h, C.c_void_p(base)), "cocoMemFree")

    def has_multicast(self, t):
        yes = C.c_int()
        _check(lib().cocoMemHasMulticast(self._h, _ptr(t), C.byref(yes)), "cocoMemHasMulticast")
        return bool(yes.value)

    def set_algo(self, algo):
        """0 / False / "p2p", 1 / True / "nvls", 2 / "auto"."""
        code = {"p2p": 0, "nvls": 1, "auto": 2}.get(algo, algo)
        _check(lib().cocoSetAlgo(self._h, int(code)), "cocoSetAlgo")

    def set_tunables(self, ctas_per_sm=0, threads=0, timeout_ms=0):
        _check(lib().cocoSetTunables(self._h, ctas_per_sm, threads, timeout_ms), "cocoSetTunables")

    # ---- the fused step ----
    def _lp(self, w_lp):
        return (_ptr(w_lp), _dtype_code(w_lp)) if w_lp is not None else (None, _F16)

    def fused_sgd(self, g, w, lr, w_lp=None, grad_scale=1.0, stream=None):
        lp, lpt = self._lp(w_lp)
        _check(lib().cocoFusedSGD(self._h, _ptr(g), _dtype_code(g), _ptr(w), lp, lpt, w.numel(),
                                  lr, grad_scale, _stream(stream)), "cocoFusedSGD")

    def fused_adam(self, g, w, m, v, lr, beta1, beta2, eps, step, w_lp=None, grad_scale=1.0,
                   variant=VARIANT_OVERLAP, stream=None):
        lp, lpt = self._lp(w_lp)
        _check(lib().cocoFusedAdam(self._h, _ptr(g), _dtype_code(g), _ptr(w), lp, lpt, _ptr(m),
                                   _ptr(v), w.numel(), lr, beta1, beta2, eps, step, grad_scale,
                                   variant, _stream(stream)), "cocoFusedAdam")

    def fused_lamb(self, g, w, m, v, lr, beta1, beta2, eps, weight_decay, step, w_lp=None,
                   grad_scale=1.0, variant=VARIANT_OVERLAP, flags=0, stream=None):
        lp, lpt = self._lp(w_lp)
        _check(lib().cocoFusedLAMB(self._h, _ptr(g), _dtype_code(g), _ptr(w), lp, lpt, _ptr(m),
                                   _ptr(v), w.numel(), lr, beta1, beta2, eps, weight_decay, step,
                                   grad_scale, variant, flags, _stream(stream)), "cocoFusedLAMB")

    # ---- stand-alone collectives (fp32 sum; count = total elements) ----
    def all_reduce(self, buf, stream=None):
        _check(lib().cocoAllReduce(self._h, _ptr(buf), buf.numel(), _stream(stream)), "cocoAllReduce")

    def reduce_scatter(self, send, recv, stream=None):
        _check(lib().cocoReduceScatter(self._h, _ptr(send), _ptr(recv), send.numel(), _stream(stream)),
               "cocoReduceScatter")

    def all_gather(self, send, recv, stream=None):
        _check(lib().cocoAllGather(self._h, _ptr(send), _ptr(recv), recv.numel(), _stream(stream)),
               "cocoAllGather")

    # ---- lists of tensors ----
    @staticmethod
    def _lists(gs, ws):
        if isinstance(gs, TensorList):
            return gs.n, gs.g, gs.w, gs.counts
        n = len(gs)
        ga = (C.c_void_p * n)(*[t.data_ptr() for t in gs])
        wa = (C.c_void_p * n)(*[t.data_ptr() for t in ws])
        ca = (C.c_size_t * n)(*[t.numel() for t in ws])
        return n, ga, wa, ca

    def fused_sgd_scattered(self, gs, ws, lr, grad_scale=1.0, stream=None):
        n, ga, wa, ca = self._lists(gs, ws)
        _check(lib().cocoFusedSGDScattered(self._h, n, ga, _list_dtype(gs), wa, ca, lr,
                                           grad_scale, _stream(stream)), "cocoFusedSGDScattered")

    def fused_adam_scattered(self, gs, ws, m, v, lr, beta1, beta2, eps, step, grad_scale=1.0,
                             variant=VARIANT_OVERLAP, stream=None):
        n, ga, wa, ca = self._lists(gs, ws)
        _check(lib().cocoFusedAdamScattered(self._h, n, ga, _list_dtype(gs), wa, ca, _ptr(m),
                                            _ptr(v), lr, beta1, beta2, eps, step, grad_scale,
                                            variant, _stream(stream)), "cocoFusedAdamScattered")

    def fused_lamb_scattered(self, gs, ws, m, v, lr, beta1, beta2, eps, weight_decay, step,
                             grad_scale=1.0, variant=VARIANT_OVERLAP, flags=0, stream=None):
        """LAMB over a list of tensors with one trust ratio PER TENSOR."""
        n, ga, wa, ca = self._lists(gs, ws)
        _check(lib().cocoFusedLAMBScattered(self._h, n, ga, _list_dtype(gs), wa, ca, _ptr(m),
                                            _ptr(v), lr, beta1, beta2, eps, weight_decay, step,
                                            grad_scale, variant, flags, _stream(stream)),
               "cocoFusedLAMBScattered")

    def link_probe(self, buf, mode, unroll=1, iters=5, stream=None):
        """GB/s per direction per GPU of a pull ("pull"), push ("push"), pull +
        push ("both") kernel with the fused step's access shape, of the copy
        engine ("copy"), or of the same through the NVSwitch ("switch_reduce",
        "switch_store", "switch_both"; `buf` from mem_alloc), over `buf`
        (overwritten).  Collective; synchronises."""
        code = {"pull": 0, "push": 1, "both": 2, "copy": 3, "switch_reduce": 4,
                "switch_store": 5, "switch_both": 6, "hybrid": 7}[mode]
        out = C.c_double()
        _check(lib().cocoLinkProbe(self._h, _ptr(buf), buf.numel() * buf.element_size(), code,
                                   unroll, iters, C.byref(out), _stream(stream)), "cocoLinkProbe")
        return out.value

    # ---- introspection ----
    def topology(self):
        """Peer access and relative P2P performance between the ranks' GPUs as
        found at creation: dict with world, access, perf_rank (lists of lists,
        -1 = unknown) and uniform."""
        t = _Topology()
        _check(lib().cocoCommTopology(self._h, C.byref(t)), "cocoCommTopology")
        n = t.world
        return {"world": n, "uniform": bool(t.uniform),
                "access": [[t.access[a][b] for b in range(n)] for a in range(n)],
                "perf_rank": [[t.perf_rank[a][b] for b in range(n)] for a in range(n)],
                "native_atomics": [[t.native_atomics[a][b] for b in range(n)] for a in range(n)]}

    def status(self):
        """First device-side failure since the last call, as a dict (code 0 =
        none).  Synchronise the stream first."""
        s = _Status()
        _check(lib().cocoGetStatus(self._h, C.byref(s)), "cocoGetStatus")
        return {"code": s.code, "rank": s.rank, "phase": s.phase, "peer": s.peer, "seq": s.seq}

    def last_lamb_norms(self):
        out = (C.c_double * 2)()
        _check(lib().cocoLastLambNorms(self._h, out), "cocoLastLambNorms")
        return out[0], out[1]

    def last_phase_times(self):
        """(first data phase, norm exchange, last data phase) of the last fused call
        in microseconds, as CTA 0 of this rank saw them.  Synchronise first."""
        out = (C.c_uint64 * 3)()
        _check(lib().cocoLastPhaseTimes(self._h, out), "cocoLastPhaseTimes")
        return tuple(x / 1e3 for x in out)

    def last_cta_spread(self):
        """Microseconds from the start barrier to the end of the data of the first,
        the median and the last CTA of this rank in the last fused call."""
        out = (C.c_uint64 * 3)()
        _check(lib().cocoLastCtaSpread(self._h, out), "cocoLastCtaSpread")
        return tuple(x / 1e3 for x in out)

    def launch_count(self):
        n = C.c_uint64()
        _check(lib().cocoLaunchCount(self._h, C.byref(n)), "cocoLaunchCount")
        return n.value
