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


def symmetric_buffers(comm, shapes):
    """torch symmetric memory as plumbing: peer pointers + NVLS multicast
    address of each buffer, registered with the communicator."""
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem
    out = []
    for numel, dtype in shapes:
        t = symm_mem.empty(numel, dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()))
        h = symm_mem.rendezvous(t, dist.group.WORLD)
        mc = int(h.multicast_ptr)
        comm.register_mapped(t, [int(p) for p in h.buffer_ptrs], mc)
        out.append((t, mc, h))
    return out


def case_nvls(comm):
    """NVSwitch multicast path (multimem.ld_reduce / multimem.st).  The in-switch
    sum has its own order and 16-bit sums arrive rounded to 16 bits, so parity
    is to tolerance: rel 1e-5 for fp32 gradients, rel 2e-3 for fp16 gradients."""
    import torch.distributed as dist
    R, rank = comm.world, comm.rank
    h = K.HYPER
    for name, opt, n, g16, lp in [("nvls_adam_mixed", K.ADAM, 1 << 22, True, True),
                                  ("nvls_adam_fp32", K.ADAM, (1 << 21) + 64, False, False),
                                  ("nvls_sgd_fp32", K.SGD, 1 << 20, False, False),
                                  ("nvls_lamb_fp32", K.LAMB, 1 << 21, False, False)]:
        gdt = torch.float16 if g16 else torch.float32
        shapes = [(n, gdt), (n, torch.float16 if lp else torch.float32)]
        (g, mc_g, _h1), (out, mc_o, _h2) = symmetric_buffers(comm, shapes)
        if not (mc_g and mc_o):
            if rank == 0:
                print("skip nvls: no multicast support", flush=True)
            return
        comm.set_algo(True)
        ora = K.OracleState(opt, n, seed=55, lp=lp)
        if lp:
            w, w_lp = torch.from_numpy(ora.w.copy()).cuda(), out
        else:
            out.copy_(torch.from_numpy(ora.w))
            w, w_lp = out, None
        S = (n + R - 1) // R
        m, v = torch.zeros(S, device="cuda"), torch.zeros(S, device="cuda")
        lo, hi = K.slice_bounds(n, R, rank)
        ls = 1024.0 if g16 else 1.0
        rtol = 2e-3 if g16 else 1e-5
        for step in range(3):
            grads = K.make_grads(R, n, 55, step, dtype=np.float16 if g16 else np.float32, loss_scale=ls)
            g.copy_(torch.from_numpy(grads[rank]))
            torch.cuda.synchronize()
            dist.barrier()
            if opt == K.SGD:
                comm.fused_sgd(g, w, h["lr"], w_lp=w_lp, grad_scale=1 / ls)
            elif opt == K.ADAM:
                comm.fused_adam(g, w, m, v, h["lr"], h["beta1"], h["beta2"], h["eps"], step,
                                w_lp=w_lp, grad_scale=1 / ls)
            else:
                comm.fused_lamb(g, w, m, v, h["lr"], h["beta1"], h["beta2"], h["eps"],
                                h["weight_decay"], step, w_lp=w_lp, grad_scale=1 / ls)
            torch.cuda.synchronize()
            st = comm.status()
            assert st["code"] == 0, f"{name}: {st}"
            ora.step(grads, step, inv_scale=1 / ls)
            wh = w.cpu().numpy()
            if lp:
                K.assert_close_most(wh[lo:hi], ora.w[lo:hi], rtol, f"{name} master", rtol_all=4e-3)
                K.assert_close(w_lp.float().cpu().numpy(), ora.w_lp.astype(np.float32), 4e-3, f"{name} w_lp")
            else:
                K.assert_close_most(wh, ora.w, rtol, f"{name} w")
            if opt != K.SGD:
                # v = (1-b2) g^2 doubles the relative error of g
                K.assert_close_most(m.cpu().numpy()[: hi - lo], ora.m[lo:hi], rtol, f"{name} m")
                K.assert_close(v.cpu().numpy()[: hi - lo], ora.v[lo:hi], 3 * rtol, f"{name} v")
            dist.barrier()
        comm.set_algo(False)
        if rank == 0:
            print(f"ok {name} R={R} n={n}", flush=True)


def case_symm(comm):
    """Symmetric memory made by the runtime itself (cuMemCreate + fd exchange +
    cuMulticast): the peer-to-peer path on it is bit-exact as on IPC-mapped
    memory, the NVSwitch path within tolerance; then everything is freed."""
    R, rank = comm.world, comm.rank
    n = 1 << 22
    h = K.HYPER
    g = comm.mem_alloc(n, torch.float16)
    w_lp = comm.mem_alloc(n, torch.float16)
    mc = comm.has_multicast(g) and comm.has_multicast(w_lp)
    S = (n + R - 1) // R
    lo, hi = K.slice_bounds(n, R, rank)
    for algo, exact in (("p2p", True), ("nvls", False)):
        if algo == "nvls" and not mc:
            if rank == 0:
                print("skip symm nvls: no multicast support", flush=True)
            continue
        comm.set_algo(algo)
        ora = K.OracleState(K.ADAM, n, seed=66, lp=True)
        w = torch.from_numpy(ora.w.copy()).cuda()
        m, v = torch.zeros(S, device="cuda"), torch.zeros(S, device="cuda")
        for step in range(2):
            grads = K.make_grads(R, n, 66, step, dtype=np.float16, loss_scale=1024.0)
            g.copy_(torch.from_numpy(grads[rank]))
            torch.cuda.synchronize()
            comm.barrier()
            comm.fused_adam(g, w, m, v, h["lr"], h["beta1"], h["beta2"], h["eps"], step, w_lp=w_lp,
                            grad_scale=1 / 1024.0)
            torch.cuda.synchronize()
            assert comm.status()["code"] == 0
            ora.step(grads, step, inv_scale=1 / 1024.0)
            if exact:
                assert np.array_equal(w.cpu().numpy()[lo:hi], ora.w[lo:hi])
                assert np.array_equal(w_lp.cpu().numpy().view(np.uint16), ora.w_lp.view(np.uint16))
                assert np.array_equal(m.cpu().numpy()[: hi - lo], ora.m[lo:hi])
            else:
                K.assert_close_most(w.cpu().numpy()[lo:hi], ora.w[lo:hi], 2e-3, "symm nvls master", rtol_all=4e-3)
                K.assert_close(w_lp.float().cpu().numpy(), ora.w_lp.astype(np.float32), 4e-3, "symm nvls w_lp")
            comm.barrier()
        if rank == 0:
            print(f"ok symm_{algo} R={R} multicast={mc}", flush=True)
    comm.set_algo("auto")
    comm.mem_free(g)
    comm.mem_free(w_lp)
    # a second allocation after a free reuses the side channel names
    t = comm.mem_alloc(1000, torch.float32)
    t.fill_(float(rank))
    torch.cuda.synchronize()
    comm.barrier()
    comm.mem_free(t)
    if rank == 0:
        print("ok symm_free_realloc", flush=True)


def case_scattered(comm):
    """Lists of tensors across processes: every tensor is peer-mapped over CUDA
    IPC on first use; results per tensor against the oracle, bit for bit."""
    R, rank = comm.world, comm.rank
    counts = [1000, 8, 3, 4096, 70001, 2, (1 << 20) + 5, 24]
    S = coco.scattered_slice_elems(counts, R)
    h = K.HYPER
    w0 = [K.make_weights(c, 800 + b) for b, c in enumerate(counts)]
    w = [torch.from_numpy(x.copy()).cuda() for x in w0]
    g = [torch.zeros(c, device="cuda") for c in counts]
    m, v = torch.zeros(S, device="cuda"), torch.zeros(S, device="cuda")
    ow = [x.copy() for x in w0]
    om = [np.zeros(c, np.float32) for c in counts]
    ov = [np.zeros(c, np.float32) for c in counts]
    off, at = [], 0
    for c in counts:
        off.append(at)
        at += (c + 7) // 8 * 8
    for step in range(3):
        grads = [K.make_grads(R, c, 900 + b, step) for b, c in enumerate(counts)]
        for b in range(len(counts)):
            g[b].copy_(torch.from_numpy(grads[b][rank]))
        torch.cuda.synchronize()
        comm.barrier()
        comm.fused_adam_scattered(g, w, m, v, h["lr"], h["beta1"], h["beta2"], h["eps"], step)
        torch.cuda.synchronize()
        assert comm.status()["code"] == 0
        mh, vh = m.cpu().numpy(), v.cpu().numpy()
        for b, cnt in enumerate(counts):
            O_ = __import__("oracle_lib")
            O_.adam(ow[b], om[b], ov[b], O_.reduce_f32(grads[b]), h["lr"], h["beta1"], h["beta2"],
                    h["eps"], step)
            assert np.array_equal(w[b].cpu().numpy(), ow[b]), f"scattered w tensor {b} step {step}"
            # the part of this tensor's moments that lives on this rank
            lo, hi = rank * S, (rank + 1) * S
            a, z = max(off[b], lo), min(off[b] + cnt, hi)
            if a < z:
                assert np.array_equal(mh[a - lo:z - lo], om[b][a - off[b]:z - off[b]])
                assert np.array_equal(vh[a - lo:z - lo], ov[b][a - off[b]:z - off[b]])
        comm.barrier()
    # LAMB with one trust ratio per tensor: the per-tensor norm partials cross
    # processes through the table behind each rank's flag page
    O_ = __import__("oracle_lib")
    lw = [torch.from_numpy(x.copy()).cuda() for x in w0]
    lm, lv = torch.zeros(S, device="cuda"), torch.zeros(S, device="cuda")
    low = [x.copy() for x in w0]
    lom = [np.zeros(c, np.float32) for c in counts]
    lov = [np.zeros(c, np.float32) for c in counts]
    for step in range(3):
        grads = [K.make_grads(R, c, 950 + b, step) for b, c in enumerate(counts)]
        for b in range(len(counts)):
            g[b].copy_(torch.from_numpy(grads[b][rank]))
        torch.cuda.synchronize()
        comm.barrier()
        comm.fused_lamb_scattered(g, lw, lm, lv, h["lr"], h["beta1"], h["beta2"], h["eps"],
                                  h["weight_decay"], step)
        torch.cuda.synchronize()
        assert comm.status()["code"] == 0
        mh = lm.cpu().numpy()
        for b, cnt in enumerate(counts):
            O_.lamb(low[b], lom[b], lov[b], O_.reduce_f32(grads[b]), h["lr"], h["beta1"],
                    h["beta2"], h["eps"], h["weight_decay"], step)
            got = lw[b].cpu().numpy()
            K.assert_close(got, low[b], 1e-5, f"scattered lamb w tensor {b} step {step}")
            low[b] = got.copy()
            lo, hi = rank * S, (rank + 1) * S
            a, z = max(off[b], lo), min(off[b] + cnt, hi)
            if a < z:
                assert np.array_equal(mh[a - lo:z - lo], lom[b][a - off[b]:z - off[b]])
        # replicas agree bit for bit: compare a checksum of all weights across ranks
        digest = np.array([float(np.sum(x.cpu().numpy().astype(np.float64))) for x in lw])
        all_d = comm.all_gather_host(digest.tobytes())
        assert all(d == all_d[0] for d in all_d), "scattered lamb: replicas differ"
        comm.barrier()
    if rank == 0:
        print(f"ok scattered R={R} tensors={len(counts)}", flush=True)
        print(f"ok scattered_lamb R={R}", flush=True)


def case_collectives(comm):
    """cocoAllReduce / cocoReduceScatter / cocoAllGather against numpy, sums in
    rank order (bit-exact), aligned and ragged sizes."""
    R, rank = comm.world, comm.rank
    for n in (1 << 20, 100003, 5):
        xs = [np.random.default_rng((n, r)).standard_normal(n).astype(np.float32) for r in range(R)]
        want = xs[0].copy()
        for r in range(1, R):
            want = want + xs[r]
        lo, hi = K.slice_bounds(n, R, rank)
        S = (n + R - 1) // R
        buf = torch.from_numpy(xs[rank].copy()).cuda()
        comm.all_reduce(buf)
        torch.cuda.synchronize()
        assert np.array_equal(buf.cpu().numpy(), want), f"all_reduce n={n}"
        send = torch.from_numpy(xs[rank].copy()).cuda()
        recv = torch.zeros(S, device="cuda")
        comm.barrier()
        comm.reduce_scatter(send, recv)
        torch.cuda.synchronize()
        assert np.array_equal(recv.cpu().numpy()[: hi - lo], want[lo:hi]), f"reduce_scatter n={n}"
        full = torch.zeros(n, device="cuda")
        comm.barrier()
        comm.all_gather(recv, full)
        torch.cuda.synchronize()
        assert np.array_equal(full.cpu().numpy(), want), f"all_gather n={n}"
        assert comm.status()["code"] == 0
        comm.barrier()
    if rank == 0:
        print(f"ok collectives R={R}", flush=True)


def case_probe(comm):
    """Topology table and link yardstick across processes: every pair reachable,
    every mode of the probe gives a positive rate and leaves no device status."""
    R, rank = comm.world, comm.rank
    topo = comm.topology()
    assert topo["world"] == R
    for a in range(R):
        for b in range(R):
            assert topo["access"][a][b] in (1, -1), topo      # 0 would have failed creation
    assert topo["access"][rank][rank] == 1
    buf = torch.zeros(1 << 24, dtype=torch.float32, device="cuda")   # 64 MiB
    comm.register(buf)
    rates = {m: comm.link_probe(buf, m, unroll=u, iters=2)
             for m, u in (("copy", 1), ("pull", 1), ("push", 2), ("both", 4))}
    assert all(v > 1.0 for v in rates.values()), rates
    sym = comm.mem_alloc(1 << 24, torch.float32)
    sym.zero_()
    torch.cuda.synchronize()
    if comm.has_multicast(sym):
        for m in ("switch_reduce", "switch_store", "switch_both"):
            assert comm.link_probe(sym, m, unroll=2, iters=2) > 1.0
        assert comm.link_probe(sym, "hybrid", unroll=8, iters=2) > 0.0    # microseconds
    assert comm.status()["code"] == 0
    torch.cuda.synchronize()
    comm.mem_free(sym)
    comm.barrier()
    if rank == 0:
        print(f"ok probe R={R} uniform={topo['uniform']} {rates}", flush=True)


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
    failed = False
    if sys.argv[1] == "nvls":
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    comm = coco.Communicator.init_rank(world, rank)
    try:
        {"parity": case_parity, "timeout": case_timeout, "nvls": case_nvls, "symm": case_symm, "scattered": case_scattered, "collectives": case_collectives, "probe": case_probe}[sys.argv[1]](comm)
    except Exception:  # keep this rank alive until its peers are done with its memory
        import traceback
        print("WORKER FAILURE rank %d\n%s" % (rank, traceback.format_exc()), flush=True)
        failed = True
    try:
        comm.barrier()
    except Exception:
        pass
    torch.cuda.synchronize()
    comm.destroy()
    if sys.argv[1] == "nvls":
        dist.barrier()
        dist.destroy_process_group()
    sys.exit(1 if failed else 0)
