"""cocoLambStepNoAlloc: the LAMB step for callers that cannot allocate device
memory while stepping the optimizer (a frozen or fully reserved pool, a device
near its memory limit, a loop that avoids the driver's allocation locks).  It must give what the
communicator-based entry point gives.  Collected last on purpose: it shares a
library-resident scratch array, and a failure here must not hide other tests.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import cases as K

pytestmark = pytest.mark.gpu

import coconet_b200 as coco  # noqa: E402

_F16, _F32 = 6, 7


def _no_alloc_step(g, w, m, v, step, w_lp=None, grad_scale=1.0):
    h = K.HYPER
    rc = coco.lib().cocoLambStepNoAlloc(
        C.c_void_p(g.data_ptr()), _F16 if g.dtype == torch.float16 else _F32,
        C.c_void_p(w.data_ptr()), C.c_void_p(w_lp.data_ptr()) if w_lp is not None else None, _F16,
        C.c_void_p(m.data_ptr()), C.c_void_p(v.data_ptr()), w.numel(), h["lr"], h["beta1"],
        h["beta2"], h["eps"], h["weight_decay"], step, grad_scale,
        C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, coco.runtime.error_string(rc)


@pytest.mark.parametrize("n,mixed", [(100003, False), (1 << 20, True)])
def test_no_alloc_matches_communicator_entry_point_twice_in_a_row(n, mixed):
    comm = coco.Communicator.init_all(1, [0])[0]
    try:
        w0 = torch.from_numpy(K.make_weights(n, 31)).cuda()
        wa, wb = w0.clone(), w0.clone()
        ma, va, mb, vb = (torch.zeros(n, device="cuda") for _ in range(4))
        la = lb = None
        if mixed:
            la = torch.zeros(n, dtype=torch.float16, device="cuda")
            lb = torch.zeros(n, dtype=torch.float16, device="cuda")
        h = K.HYPER
        for step in range(2):  # two calls in a row share the scratch array
            grads = K.make_grads(1, n, 31, step, dtype=np.float16 if mixed else np.float32,
                                 loss_scale=1024.0 if mixed else 1.0)
            g = torch.from_numpy(grads[0]).cuda()
            gs = 1 / 1024.0 if mixed else 1.0
            comm.fused_lamb(g, wa, ma, va, h["lr"], h["beta1"], h["beta2"], h["eps"],
                            h["weight_decay"], step, w_lp=la, grad_scale=gs)
            torch.cuda.synchronize()
            # the driver's own count of free device memory also sees a raw
            # cudaMalloc made behind torch's back (the first call is left out:
            # loading the kernel image may take memory once)
            free_before = torch.cuda.mem_get_info()[0]
            _no_alloc_step(g, wb, mb, vb, step, w_lp=lb, grad_scale=gs)
            torch.cuda.synchronize()
            if step > 0:
                assert torch.cuda.mem_get_info()[0] == free_before
            assert comm.status()["code"] == 0
            # same kernel, same arithmetic; only the number of CTAs (hence the
            # summation tree of the norms) may differ: fp32 tolerance of the suite
            K.assert_close(wb.cpu().numpy(), wa.cpu().numpy(), 1e-5, f"w step {step}")
            assert torch.equal(mb, ma) and torch.equal(vb, va)
            if mixed:
                K.assert_close(lb.float().cpu().numpy(), la.float().cpu().numpy(), 1e-3, "w_lp")
    finally:
        comm.destroy()


def test_no_alloc_rejects_oversize_and_bad_arguments():
    L = coco.lib()
    t = torch.zeros(16, device="cuda")
    p = C.c_void_p(t.data_ptr())
    too_many = (1 << 31) + 1
    assert L.cocoLambStepNoAlloc(p, _F32, p, None, _F16, p, p, too_many, 1e-3, 0.9, 0.999, 1e-6,
                                 0.01, 0, 1.0, None) == 1
    assert L.cocoLambStepNoAlloc(None, _F32, p, None, _F16, p, p, 16, 1e-3, 0.9, 0.999, 1e-6,
                                 0.01, 0, 1.0, None) == 1
    assert L.cocoLambStepNoAlloc(p, 3, p, None, _F16, p, p, 16, 1e-3, 0.9, 0.999, 1e-6,
                                 0.01, 0, 1.0, None) == 1
