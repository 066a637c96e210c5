"""One rank of a multi-process parity case (one process per GPU).  Launched by
tests/test_multigpu.py through torch.distributed.run; exits non-zero on any
mismatch with the CPU oracle.  Every rank regenerates all ranks' seeded
gradients on the host, so each can evaluate the oracle for itself."""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)

import cases as K  # noqa: E402
import coconet_b200 as coco  # noqa: E402


def run_case(comm, name, opt, n, steps, g_dtype=np.float32, lp=None, loss_scale=1.0, hyper=None,
             dist="normal", exact_w=True):
    R, rank = comm.world, comm.rank
    h = dict(K.HYPER)
    if hyper:
        h.update(hyper)
    ora = K.OracleState(opt, n, seed=77, lp=lp is not None, hyper=hyper)
    w = torch.from_numpy(ora.w.copy()).cuda()
    w_lp = torch.zeros(n, dtype=lp, device="cuda") if lp else None
    S = (n + R - 1) // R
    m = torch.zeros(S, device="cuda")
    v = torch.zeros(S, device="cuda")
    g = torch.zeros(n, dtype=torch.float16 if g_dtype == np.float16 else torch.float32, device="cuda")
    lo, hi = K.slice_bounds(n, R, rank)
    for step in range(steps):
        grads = K.make_grads(R, n, 77, step, dtype=g_dtype, dist=dist, loss_scale=loss_scale)
        g.copy_(torch.from_numpy(grads[rank]))
        torch.cuda.synchronize()
        gs = 1.0 / loss_scale
        if opt == K.SGD:
            comm.fused_sgd(g, w, h["lr"], w_lp=w_lp, grad_scale=gs)
        elif opt == K.ADAM:
            comm.fused_adam(g, w, m, v, h["lr"], h["beta1"], h["beta2"], h["eps"], step, w_lp=w_lp,
                            grad_scale=gs)
        else:
            comm.fused_lamb(g, w, m, v, h["lr"], h["beta1"], h["beta2"], h["eps"],
                            h["weight_decay"], step, w_lp=w_lp, grad_scale=gs)
        torch.cuda.synchronize()
        st = comm.status()
        assert st["code"] == 0, f"{name}: device status {st}"
        ora.step(grads, step, inv_scale=gs)
        wh = w.cpu().numpy()
        if lp is None:
            K.assert_close(wh, ora.w, 1e-5, f"{name} step {step} w")
            if exact_w:
                assert np.array_equal(wh, ora.w), f"{name} step {step}: w not bit-exact"
        else:
            K.assert_close(wh[lo:hi], ora.w[lo:hi], 1e-5, f"{name} step {step} master slice")
            got = w_lp.float().cpu().numpy()
            K.assert_close(got, ora.w_lp.astype(np.float32), 1e-3, f"{name} step {step} w_lp")
            if exact_w:
                assert np.array_equal(w_lp.cpu().numpy().view(np.uint16), ora.w_lp.view(np.uint16))
        if opt != K.SGD:
            assert np.array_equal(m.cpu().numpy()[: hi - lo], ora.m[lo:hi]), f"{name}: m"
            assert np.array_equal(v.cpu().numpy()[: hi - lo], ora.v[lo:hi]), f"{name}: v"
    comm.barrier()
    if rank == 0:
        print(f"ok {name} R={R} n={n} steps={steps}", flush=True)


def case_parity(comm):
    run_case(comm, "sgd_cfg0", K.SGD, 1 << 20, 2, hyper=dict(lr=0.01), dist="uniform")
    run_case(comm, "sgd_ragged", K.SGD, 4099, 2, hyper=dict(lr=0.01), dist="uniform")
    run_case(comm, "adam_fp32", K.ADAM, (1 << 22), 3)
    run_case(comm, "adam_fp32_ragged", K.ADAM, (1 << 20) + 3, 3)
    run_case(comm, "adam_mixed", K.ADAM, 1 << 22, 3, g_dtype=np.float16, lp=torch.float16,
             loss_scale=1024.0)
    run_case(comm, "adam_mixed_ragged", K.ADAM, 100003, 2, g_dtype=np.float16, lp=torch.float16,
             loss_scale=1024.0)
    run_case(comm, "lamb_fp32", K.LAMB, (1 << 21) + 8, 3, exact_w=False)
    run_case(comm, "lamb_mixed", K.LAMB, 1 << 20, 2, g_dtype=np.float16, lp=torch.float16,
             loss_scale=1024.0, exact_w=False)


def case_timeout(comm):
    """Rank 1 skips one fused call: the others' bounded start wait must give
    up with a status, leave the weights untouched and keep the context alive."""
    n = 1 << 16
    g = torch.ones(n, device="cuda")
    w = torch.zeros(n, device="cuda")
    comm.register(g)
    comm.register(w)
    comm.set_tunables(timeout_ms=700)
    comm.barrier()
    if comm.rank != 1:
        comm.fused_sgd(g, w, 1.0)
    torch.cuda.synchronize()
    comm.barrier()
    if comm.rank != 1:
        st = comm.status()
        assert st["code"] == 5 and st["phase"] == 1 and st["peer"] == 1, st
        assert float(w.abs().max()) == 0.0
        assert comm.status()["code"] == 0  # cleared by the read
    # the context is still usable
    assert float((g + 1).sum()) == 2.0 * n
    comm.barrier()
    if comm.rank == 0:
        print("ok timeout", flush=True)


if __name__ == "__main__":
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    comm = coco.Communicator.init_rank(world, rank)
    try:
        {"parity": case_parity, "timeout": case_timeout}[sys.argv[1]](comm)
    finally:
        comm.destroy()
