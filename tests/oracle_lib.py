"""ctypes view of the CPU oracle (oracle/liboracle.so) and, when built, of the
reference's own host checkers (oracle/_ref/*.so).  Test infrastructure only."""
import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")

OVERLAP, DSL, NCCL = 0, 1, 2
LAMB_REF_QUIRK = 1

_f32p = C.POINTER(C.c_float)
_u16p = C.POINTER(C.c_uint16)


def _fp(a):
    if a is None:
        return None
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(_f32p)


def _hp(a):
    if a is None:
        return None
    assert a.dtype in (np.uint16, np.float16) and a.flags.c_contiguous
    return a.ctypes.data_as(_u16p)


def _ptr_array(arrs):
    arr = (C.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])
    return arr


_lib = None


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(os.path.join(ORACLE_DIR, "liboracle.so"))
        L.oracle_reduce_f32.argtypes = [C.c_void_p, C.c_int, C.c_size_t, _f32p]
        L.oracle_reduce_f16.argtypes = [C.c_void_p, C.c_int, C.c_size_t, C.c_float, _f32p]
        L.oracle_reduce_f16_ring.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_size_t, _u16p]
        L.oracle_sgd.argtypes = [_f32p, _f32p, C.c_size_t, C.c_float]
        L.oracle_adam.argtypes = [_f32p, _f32p, _f32p, _u16p, _f32p, _u16p, C.c_size_t,
                                  C.c_float, C.c_float, C.c_float, C.c_float, C.c_int, C.c_int]
        L.oracle_adam.restype = C.c_int
        L.oracle_lamb.argtypes = [_f32p, _f32p, _f32p, _u16p, _f32p, C.c_size_t, C.c_float,
                                  C.c_float, C.c_float, C.c_float, C.c_float, C.c_int, C.c_int,
                                  C.c_uint, C.POINTER(C.c_double)]
        L.oracle_lamb.restype = C.c_int
        L.oracle_cpu_step_adam.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, _f32p, _f32p,
                                           _f32p, _u16p, C.c_size_t, C.c_float, C.c_float,
                                           C.c_float, C.c_float, C.c_int]
        L.oracle_cpu_step_adam.restype = C.c_int
        L.oracle_cpu_step_adam_mt.argtypes = L.oracle_cpu_step_adam.argtypes + [C.c_int]
        L.oracle_cpu_step_adam_mt.restype = C.c_int
        L.oracle_threads_available.restype = C.c_int
        L.oracle_f32_to_f16.argtypes = [C.c_float]
        L.oracle_f32_to_f16.restype = C.c_uint16
        _lib = L
    return _lib


def reduce_f32(grads):
    out = np.empty_like(grads[0])
    lib().oracle_reduce_f32(_ptr_array(grads), len(grads), out.size, _fp(out))
    return out


def reduce_f16(grads, inv_scale=1.0):
    out = np.empty(grads[0].shape, np.float32)
    lib().oracle_reduce_f16(_ptr_array(grads), len(grads), out.size, inv_scale, _fp(out))
    return out


def reduce_f16_ring(grads, owner):
    out = np.empty(grads[0].shape, np.float16)
    lib().oracle_reduce_f16_ring(_ptr_array(grads), len(grads), owner, out.size, _hp(out))
    return out


def sgd(w, gsum, lr):
    lib().oracle_sgd(_fp(w), _fp(gsum), w.size, lr)


def adam(w, m, v, gsum, lr, b1, b2, eps, step, variant=OVERLAP, w_lp=None, gsum_h=None):
    rc = lib().oracle_adam(_fp(w), _fp(m), _fp(v), _hp(w_lp), _fp(gsum), _hp(gsum_h), w.size,
                           lr, b1, b2, eps, step, variant)
    assert rc == 0


def lamb(w, m, v, gsum, lr, b1, b2, eps, wd, step, variant=OVERLAP, flags=0, w_lp=None):
    norms = (C.c_double * 2)()
    rc = lib().oracle_lamb(_fp(w), _fp(m), _fp(v), _hp(w_lp), _fp(gsum), w.size, lr, b1, b2,
                           eps, wd, step, variant, flags, norms)
    assert rc == 0
    return norms[0], norms[1]


def cpu_step_adam(grads, w, m, v, lr, b1, b2, eps, step, inv_scale=1.0, w_lp=None, threads=1):
    is16 = grads[0].dtype == np.float16
    if threads == 1:
        rc = lib().oracle_cpu_step_adam(_ptr_array(grads), len(grads), int(is16), inv_scale, _fp(w),
                                        _fp(m), _fp(v), _hp(w_lp), w.size, lr, b1, b2, eps, step)
    else:
        rc = lib().oracle_cpu_step_adam_mt(_ptr_array(grads), len(grads), int(is16), inv_scale,
                                           _fp(w), _fp(m), _fp(v), _hp(w_lp), w.size, lr, b1, b2,
                                           eps, step, threads)
    assert rc == 0


def threads_available():
    return int(lib().oracle_threads_available())


# ---- the reference's own host checkers, compiled by `make -C oracle ref` ----

def ref_available():
    return all(os.path.exists(os.path.join(ORACLE_DIR, "_ref", f"libref_{n}.so"))
               for n in ("sgd", "adam", "overlap"))


_ref = {}


def ref(name):
    if name not in _ref:
        L = C.CDLL(os.path.join(ORACLE_DIR, "_ref", f"libref_{name}.so"))
        if name == "sgd":
            L.ref_sgd_check.argtypes = [C.c_void_p, C.c_int, _f32p, C.c_float, _f32p, C.c_size_t]
        elif name == "adam":
            L.ref_adam_dsl_check.argtypes = [C.c_void_p, C.c_int, _f32p, _f32p, _f32p, C.c_float,
                                             C.c_float, C.c_float, _f32p, C.c_size_t]
        else:
            for fn in (L.ref_overlap_adam_check, L.ref_overlap_lamb_check):
                fn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_size_t, _f32p, _f32p, _f32p,
                               _f32p, C.c_float, C.c_float, C.c_float, C.c_float]
        _ref[name] = L
    return _ref[name]


def ref_sgd_check(grads, w_old, lr, w_new):
    return bool(ref("sgd").ref_sgd_check(_ptr_array(grads), len(grads), _fp(w_old), lr,
                                         _fp(w_new), w_old.size))


def ref_adam_dsl_check(grads, w_old, m_old, v_old, lr, b1, b2, w_new):
    return bool(ref("adam").ref_adam_dsl_check(_ptr_array(grads), len(grads), _fp(w_old),
                                               _fp(m_old), _fp(v_old), lr, b1, b2, _fp(w_new),
                                               w_old.size))


def ref_overlap_check(kind, grads, epoch, w_old, w_new, cpu_m, cpu_v, b1, b2, stepsize, eps):
    fn = getattr(ref("overlap"), f"ref_overlap_{kind}_check")
    return bool(fn(_ptr_array(grads), len(grads), epoch, w_old.size, _fp(w_old), _fp(w_new),
                   _fp(cpu_m), _fp(cpu_v), b1, b2, stepsize, eps))
