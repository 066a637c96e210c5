#!/usr/bin/env python
"""Benchmark of the fused AllReduce optimizer step.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE config 2): mixed-precision Adam on one flattened buffer of
334,000,000 parameters -- fp16 Local gradients (loss scale 1024, removed in the
kernel), fp32 master weights, fp32 Sliced m/v, fp16 Replicated weight copy that
is all-gathered -- at world size N.  Synthetic seeded inputs.

A "step" is one fused call per rank: reduce-scatter of the gradients, the Adam
update of the rank's slice, all-gather of the updated weights; one kernel.
`value` counts gradient elements reduced and applied per second over the whole
job (N ranks x count / step time), inputs resident in HBM.  `e2e` is the same
with the gradients arriving from pinned host memory and the updated fp16
weights read back to the host every step.

For N > 1 launch with torchrun (one rank per GPU); rank 0 prints ONE JSON line.
`--impl reference` times the reference's CPU path (single-threaded host loops)
on a bounded sample instead.
"""
import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

COUNT = 334_000_000
LOSS_SCALE = 1024.0
HYPER = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-6)
NVLINK_PEER_GBS = 770.0  # measured peer copy per direction on this pool (900 nominal)
METRIC = "fused_allreduce_adam_grad_elems_per_s"
UNIT = "Gelem/s"


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 50 ms by one
    streaming nvidia-smi process while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc = index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i",
                 str(self.index), "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
            time.sleep(0.3)  # let the first samples arrive before the region starts
        except Exception:
            self.proc = None

    def stop(self):
        samples = []
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()  # our own child, by handle
            try:
                out, _ = self.proc.communicate(timeout=5)
            except Exception:
                out = ""
            for line in out.splitlines():
                f = [x.strip() for x in line.split(",")]
                if len(f) >= 9:
                    samples.append(f)

        def num(x):
            try:
                return float(x)
            except ValueError:
                return None
        sm = sorted(v for v in (num(s[1]) for s in samples) if v is not None)
        mx = [v for v in (num(s[2]) for s in samples) if v is not None]
        pw = [v for v in (num(s[3]) for s in samples) if v is not None]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in samples for n, v in zip(names, s[5:9])
                          if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "reasons": reasons, "samples": len(samples)}


def cpu_baseline(count_sample, world, reps=2, threads=1):
    """The reference's CPU path (host sum of `world` gradient arrays + the
    per-element passes) on a bounded sample: single-threaded like the
    reference's loops by default, or on `threads` host threads."""
    import numpy as np
    import oracle_lib as O
    so = os.path.join(ROOT, "oracle", "liboracle.so")
    if not os.path.exists(so):
        subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "-s"])
    n = count_sample
    rng = np.random.default_rng(0)
    grads = [(rng.standard_normal(n, dtype=np.float32) * 1e-3 * LOSS_SCALE).astype(np.float16)
             for _ in range(world)]
    w = (rng.standard_normal(n, dtype=np.float32) * 0.02).astype(np.float32)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    wl = np.zeros(n, np.float16)
    best = None
    for step in range(reps):
        t0 = time.perf_counter()
        O.cpu_step_adam(grads, w, m, v, HYPER["lr"], HYPER["beta1"], HYPER["beta2"], HYPER["eps"],
                        step, inv_scale=1.0 / LOSS_SCALE, w_lp=wl, threads=threads)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": world * n / best / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{n} of {COUNT} elements x {world} gradient arrays, best of {reps}, "
                      f"{best * 1e3:.1f} ms per step on {threads} thread(s); host has "
                      f"{os.cpu_count()} cores"}


def run_reference(args, rank, world):
    if rank != 0:
        return
    # Every host thread the box offers (the elements are independent: contiguous
    # ranges, one thread each); the sample grows with the thread count so that a
    # step stays long enough to time.
    import oracle_lib as O
    threads = max(1, min(O.threads_available(), os.cpu_count() or 1))
    n = min(COUNT, (1 << 24) * max(1, threads // 4))
    steps = max(1, min(args.steps, 3))
    cb = cpu_baseline(n, world, reps=steps + min(args.warmup, 1), threads=threads)
    one = cpu_baseline(1 << 24, world, reps=1, threads=1)
    cb["sample"] += f"; one thread: {one['value']:.4f} {UNIT}"
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT,
            "n_gpus": world, "steps": steps, "warmup": min(args.warmup, 1),
            "ms_per_step": world * n / (cb["value"] * 1e9) * 1e3 * (COUNT / n),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "mixed_adam_334M", "count": COUNT, "world": world,
                       "note": "CPU loops timed on a sample and reported as a rate; ms_per_step "
                               "is that rate scaled to the full count"},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_sweep(args, rank, world, local_rank):
    """Message-size sweep (BASELINE config 4) plus the named configs: fused SGD,
    fp32 Adam, mixed-precision Adam and fp32 LAMB at N = 4^k elements, each next
    to stock NCCL all-reduce + the update kernel over all elements.  L2 is
    flushed (a 256 MB memset) between timed iterations; every iteration is
    timed with its own CUDA event pair."""
    import torch
    import torch.distributed as dist
    import coconet_b200 as coco

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        comm = coco.Communicator.from_torch_distributed()
    else:
        comm = coco.Communicator.init_all(1, [local_rank])[0]
    local = coco.Communicator.init_all(1, [local_rank])[0]
    R = world
    use_nvls = world > 1 and (args.algo == "nvls" or (args.algo == "auto" and world >= 4))
    max_n = max(1 << args.sweep_max_log, COUNT, 340_000_000)  # also holds the BERT-large-shaped list
    keep = []

    def comm_buffer(numel, dtype):
        if not use_nvls:
            t = torch.empty(numel, dtype=dtype, device=dev)
            comm.register(t)
            return t
        t = comm.mem_alloc(numel, dtype)
        keep.append(t)
        return t

    # one set of maximum-size buffers; smaller points use leading views of them
    g32 = comm_buffer(max_n, torch.float32)
    g16 = comm_buffer(max_n, torch.float16)
    w32 = comm_buffer(max_n, torch.float32)
    w16 = comm_buffer(max_n, torch.float16)
    g32.normal_(0, 1e-3)
    g16.copy_(g32 * LOSS_SCALE)
    w32.normal_(0, 0.02)
    Smax = (max_n + R - 1) // R
    m = torch.zeros(Smax, device=dev)
    v = torch.zeros(Smax, device=dev)
    mf = torch.zeros(max_n, device=dev)     # un-sharded state of the baseline
    vf = torch.zeros(max_n, device=dev)
    gb32 = torch.empty(max_n, dtype=torch.float32, device=dev)
    gb16 = torch.empty(max_n, dtype=torch.float16, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    if use_nvls:
        comm.set_algo("nvls")

    def time_back_to_back(fn, steps, warmup):
        """Steps enqueued one after the other as a training loop would (no L2
        flush, one event pair around all of them): the latency a small
        message sees once the ranks run in step."""
        for i in range(warmup):
            fn(i)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(warmup + i)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def time_ms(fn, steps, warmup):
        for i in range(warmup):
            fn(i)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        total = 0.0
        for i in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if world > 1:
                dist.barrier()
            e0.record()
            fn(warmup + i)
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        t = torch.tensor([total / steps], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    hbm_peak, _ = measured_peaks()
    points = [("sgd", "f32", 4 ** k) for k in range(5, args.sweep_max_log // 2 + 1)]
    points += [("adam", "f32", 4 ** k) for k in range(5, args.sweep_max_log // 2 + 1)]
    points += [("adam", "f16", 4 ** k) for k in range(5, args.sweep_max_log // 2 + 1)]
    points += [("adam", "f16", COUNT), ("lamb", "f32", COUNT), ("lamb", "f32", 1 << 26)]
    out = []
    for opt, gt, n in points:
        if n > max_n:
            continue
        g = (g16 if gt == "f16" else g32)[:n]
        gb = (gb16 if gt == "f16" else gb32)[:n]
        w = w32[:n]
        lp = w16[:n] if gt == "f16" else None
        gs = 1.0 / LOSS_SCALE if gt == "f16" else 1.0
        S = (n + R - 1) // R
        h = HYPER

        def fused(i, c=comm, mm=m[:S], vv=v[:S], gg=g):
            if opt == "sgd":
                c.fused_sgd(gg, w, 1e-3, w_lp=lp, grad_scale=gs)
            elif opt == "adam":
                c.fused_adam(gg, w, mm, vv, h["lr"], h["beta1"], h["beta2"], h["eps"], i, w_lp=lp,
                             grad_scale=gs)
            else:
                c.fused_lamb(gg, w, mm, vv, h["lr"], h["beta1"], h["beta2"], h["eps"], 0.01, i,
                             w_lp=lp, grad_scale=gs)

        def stock(i):
            gb.copy_(g)
            if world > 1:
                dist.all_reduce(gb)
            fused(i, c=local, mm=mf[:n], vv=vf[:n], gg=gb)

        def stock_copy_only(i):
            gb.copy_(g)

        steps = 5 if n >= (1 << 26) else 10
        ms = time_ms(fused, steps, 3)
        base = time_ms(stock, steps, 3) - time_ms(stock_copy_only, steps, 3)
        s_g = 2 if gt == "f16" else 4
        s_o = 2 if gt == "f16" else 4
        state = {"sgd": 8, "adam": 24, "lamb": 36}[opt] + (s_o if gt == "f16" else 0)
        b_bus = (R - 1) * S * (s_g + s_o)
        b_hbm = n * s_g + S * state + (R - 1) * S * s_o
        t_roof = max(b_bus / (NVLINK_PEER_GBS * 1e9), b_hbm / (hbm_peak * 1e9))
        b2b = time_back_to_back(fused, 50, 5) if n <= (1 << 22) else None
        out.append({"opt": opt, "grad": gt, "count": n, "world": R, "ms_back_to_back": b2b,
                    "algo": "nvls" if use_nvls else "p2p", "ms": ms, "bus_gbs": b_bus / ms / 1e6,
                    "hbm_gbs": b_hbm / ms / 1e6, "roof_frac": t_roof / (ms * 1e-3),
                    "stock_nccl_plus_update_ms": base, "speedup": base / ms})
        if rank == 0:
            p = out[-1]
            print(f"# {opt:5s} {gt} n={n:>11d} fused {ms:9.4f} ms  bus {p['bus_gbs']:7.1f} GB/s  "
                  f"hbm {p['hbm_gbs']:7.1f} GB/s  roof {p['roof_frac']:.3f}  stock {base:9.4f} ms  "
                  f"x{p['speedup']:.2f}" + (f"  back-to-back {b2b * 1e3:7.1f} us" if b2b else ""), flush=True)
    # ---- a list of tensors shaped like BERT-large (24 layers, hidden 1024, FFN 4096,
    # vocabulary 30522, 512 positions: 398 tensors, 336 M elements) through the scattered
    # call, next to the flat call on the same number of elements
    shapes = [30522 * 1024, 512 * 1024, 2 * 1024, 1024, 1024]
    for _ in range(24):
        shapes += [1024 * 1024, 1024] * 4 + [1024, 1024]
        shapes += [1024 * 4096, 4096, 4096 * 1024, 1024, 1024, 1024]
    shapes += [1024 * 1024, 1024, 1024 * 1024, 1024, 1024, 1024, 30522, 2 * 1024, 2]
    tot = sum(shapes)
    if tot <= max_n and not use_nvls:
        gl, wl, at = [], [], 0
        for c in shapes:
            gl.append(g32[at:at + c])
            wl.append(w32[at:at + c])
            at += (c + 7) // 8 * 8       # keep every tensor 16-byte aligned inside the big buffers
        if at <= max_n:
            Ssc = coco.scattered_slice_elems(shapes, R)
            msc, vsc = torch.zeros(Ssc, device=dev), torch.zeros(Ssc, device=dev)

            def scattered(i):
                comm.fused_adam_scattered(gl, wl, msc, vsc, HYPER["lr"], HYPER["beta1"],
                                          HYPER["beta2"], HYPER["eps"], i)

            tot_f = tot // (8 * R) * (8 * R)   # keeps every rank's flat slice 16-byte aligned

            def flat(i):
                comm.fused_adam(g32[:tot_f], w32[:tot_f], m[:tot_f // R], v[:tot_f // R],
                                HYPER["lr"], HYPER["beta1"], HYPER["beta2"], HYPER["eps"], i)

            ms_sc, ms_fl = time_ms(scattered, 5, 3), time_ms(flat, 5, 3)
            out.append({"opt": "adam", "grad": "f32", "count": tot, "world": R, "tensors": len(shapes),
                        "scattered_ms": ms_sc, "flat_ms": ms_fl})
            if rank == 0:
                print(f"# adam  f32 scattered over {len(shapes)} BERT-large-shaped tensors, {tot} elements: "
                      f"{ms_sc:.4f} ms  (flat call on as many elements: {ms_fl:.4f} ms)", flush=True)

            # LAMB with one trust ratio per tensor, next to the flat call (one ratio overall)
            def scattered_lamb(i):
                comm.fused_lamb_scattered(gl, wl, msc, vsc, HYPER["lr"], HYPER["beta1"],
                                          HYPER["beta2"], HYPER["eps"], 0.01, i)

            def flat_lamb(i):
                comm.fused_lamb(g32[:tot_f], w32[:tot_f], m[:tot_f // R], v[:tot_f // R],
                                HYPER["lr"], HYPER["beta1"], HYPER["beta2"], HYPER["eps"],
                                0.01, i)

            ms_sc, ms_fl = time_ms(scattered_lamb, 5, 3), time_ms(flat_lamb, 5, 3)
            out.append({"opt": "lamb", "grad": "f32", "count": tot, "world": R, "tensors": len(shapes),
                        "scattered_ms": ms_sc, "flat_ms": ms_fl})
            if rank == 0:
                print(f"# lamb  f32 scattered (per-tensor trust ratios) over {len(shapes)} tensors: "
                      f"{ms_sc:.4f} ms  (flat call on as many elements: {ms_fl:.4f} ms)", flush=True)
    st = comm.status()
    if rank == 0:
        line = {"sweep": out, "n_gpus": R, "status": st["code"],
                "timing": "CUDA events per iteration, L2 flushed between iterations, max over ranks"}
        print(json.dumps(line), flush=True)
    torch.cuda.synchronize()
    for t in keep:
        comm.mem_free(t)
    local.destroy()
    comm.destroy()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--count", type=int, default=COUNT, help="elements (default: the 334M workload)")
    ap.add_argument("--no-baseline", action="store_true", help="skip the stock NCCL comparison (N > 1)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--symm", default="runtime", choices=["runtime", "torch"],
                    help="who makes the symmetric memory of the NVLS path")
    ap.add_argument("--sweep", action="store_true", help="message-size sweep instead of the headline workload")
    ap.add_argument("--sweep-max-log", type=int, default=30)
    ap.add_argument("--algo", default=os.environ.get("COCO_BENCH_ALGO", "auto"),
                    choices=["auto", "p2p", "nvls"],
                    help="nvls: gradients and fp16 weights in symmetric memory with an NVSwitch "
                         "multicast mapping; reduce-scatter and all-gather go through the switch")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1 and args.gpus > 1:
        print(f"bench.py --gpus {args.gpus} must be launched with torchrun (one rank per GPU)",
              file=sys.stderr)
        sys.exit(2)

    if args.impl == "reference":
        run_reference(args, rank, max(world, args.gpus))
        return

    if args.sweep:
        run_sweep(args, rank, world, local_rank)
        return

    import torch
    import torch.distributed as dist
    import coconet_b200 as coco

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        comm = coco.Communicator.from_torch_distributed()
    else:
        comm = coco.Communicator.init_all(1, [local_rank])[0]

    N, R = args.count, world
    lo, hi = coco.slice_bounds(N, R, rank)
    S = (N + R - 1) // R
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    # two gradient buffers, alternated, each far larger than L2 (126 MB)
    # auto: the NVSwitch path from 4 ranks on (fewer bytes per link), else peer-to-peer
    use_nvls = world > 1 and (args.algo == "nvls" or (args.algo == "auto" and world >= 4))
    symm = []

    runtime_allocs = []

    def comm_buffer(numel):
        """A buffer peers touch: plain device memory (peer-mapped by the runtime
        over CUDA IPC), or symmetric memory with an NVSwitch multicast mapping --
        made by the runtime (cocoMemAlloc, default) or, with --symm torch, by
        torch's symmetric memory and handed over with cocoRegisterMapped."""
        if not use_nvls:
            return torch.empty(numel, dtype=torch.float16, device=dev)
        if args.symm == "runtime":
            t = comm.mem_alloc(numel, torch.float16)
            runtime_allocs.append(t)
            return t
        import torch.distributed._symmetric_memory as symm_mem
        t = symm_mem.empty(numel, dtype=torch.float16, device=dev)
        h = symm_mem.rendezvous(t, dist.group.WORLD)
        mc = int(h.multicast_ptr)
        if not mc and args.algo == "nvls":
            raise SystemExit("--algo nvls: this node exposes no NVLS multicast")
        comm.register_mapped(t, [int(p) for p in h.buffer_ptrs], mc)
        symm.append(h)
        return t

    g = []
    for _ in range(2):
        t = comm_buffer(N)
        chunk = 1 << 26
        for a in range(0, N, chunk):
            b = min(N, a + chunk)
            t[a:b] = (torch.randn(b - a, device=dev, generator=gen) * (1e-3 * LOSS_SCALE)).half()
        g.append(t)
    wgen = torch.Generator(device=dev).manual_seed(7)
    w = torch.randn(N, device=dev, generator=wgen) * 0.02
    w_lp = comm_buffer(N)
    w_lp.copy_(w)
    m = torch.zeros(S, device=dev)
    v = torch.zeros(S, device=dev)
    if use_nvls:
        comm.set_algo("nvls")
        # without a multicast mapping the runtime falls back to peer-to-peer
        use_nvls = (all(comm.has_multicast(t) for t in runtime_allocs) if args.symm == "runtime"
                    else all(int(h.multicast_ptr) != 0 for h in symm))
    else:
        for t in g:
            comm.register(t)
        comm.register(w_lp)

    step_no = [0]

    def fused_step(gbuf):
        comm.fused_adam(gbuf, w, m, v, HYPER["lr"], HYPER["beta1"], HYPER["beta2"], HYPER["eps"],
                        step_no[0], w_lp=w_lp, grad_scale=1.0 / LOSS_SCALE)
        step_no[0] += 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup, finish=None):
        """ms per step, max over ranks (CUDA events on the launching stream).
        `finish` makes the launching stream wait for work `fn` put on other
        streams, so that the closing event comes after all of it."""
        for i in range(warmup):
            fn(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(warmup + i)
        if finish:
            finish()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        barrier()
        return float(ms.item())

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    l0 = comm.launch_count()
    ms = timed(lambda i: fused_step(g[i & 1]), args.steps, args.warmup)
    launches = comm.launch_count() - l0 - args.warmup
    clocks = sampler.stop() if sampler else None
    st = comm.status()
    if st["code"] != 0:
        time.sleep(3.0 if use_nvls else 0.0)  # let the peers finish with this rank's memory
        raise SystemExit(f"device-side failure during the benchmark: {st}")

    # ---- end to end: host gradients in, host fp16 weights out ------------------
    e2e = None
    if not args.no_e2e:
        hg = torch.empty(N, dtype=torch.float16).pin_memory()
        hg.copy_(g[0])
        hout = torch.empty(N, dtype=torch.float16).pin_memory()

        # Every step copies its gradients in from pinned host memory and its fp16
        # weights out to pinned host memory.  The copies run on two side streams:
        # step i's gradients (double-buffered on the device) travel while step
        # i-1's weights are still on their way out; the kernel of step i waits for
        # both (it overwrites the weights the outgoing copy reads).
        cur = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event(), torch.cuda.Event()]
        ev_kernel = [torch.cuda.Event(), torch.cuda.Event()]
        ev_out = torch.cuda.Event()

        def e2e_step(i):
            b = i & 1
            s_in.wait_event(ev_kernel[b])      # the kernel two steps back is done with g[b]
            with torch.cuda.stream(s_in):
                g[b].copy_(hg, non_blocking=True)
                ev_in[b].record(s_in)
            cur.wait_event(ev_in[b])
            cur.wait_event(ev_out)             # the previous weights have left w_lp
            fused_step(g[b])
            ev_kernel[b].record(cur)
            s_out.wait_event(ev_kernel[b])
            with torch.cuda.stream(s_out):
                hout.copy_(w_lp, non_blocking=True)
                ev_out.record(s_out)

        def e2e_step_serial(i):  # everything on the launching stream
            g[i & 1].copy_(hg, non_blocking=True)
            fused_step(g[i & 1])
            hout.copy_(w_lp, non_blocking=True)

        k = max(3, min(args.steps, 10))
        # The overlapped form has been run on one GPU only; with more ranks the
        # serial form (measured at 2 and 8 GPUs) is used.
        if world == 1:
            ems = timed(e2e_step, k, 2, finish=lambda: cur.wait_event(ev_out))
            how = "copies on two side streams, gradients double-buffered"
        else:
            ems = timed(e2e_step_serial, k, 2)
            how = "none: copies and kernel on one stream"
        e2e = {"value": R * N / (ems * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": ems,
               "h2d_bytes_per_step": N * 2, "d2h_bytes_per_step": N * 2, "overlap": how}
        del hg, hout

    # ---- stock NCCL all-reduce + separate update kernel (the AR_C schedule) ---
    nccl = None
    if world > 1 and not args.no_baseline:
        local = coco.Communicator.init_all(1, [local_rank])[0]
        mf = torch.zeros(N, device=dev)
        vf = torch.zeros(N, device=dev)
        gb = g[0].clone()
        bstep = [0]

        def nccl_step(i):
            dist.all_reduce(gb)
            local.fused_adam(gb, w, mf, vf, HYPER["lr"], HYPER["beta1"], HYPER["beta2"],
                             HYPER["eps"], bstep[0], w_lp=w_lp, grad_scale=1.0 / LOSS_SCALE)
            bstep[0] += 1

        k = max(3, min(args.steps, 10))
        bms = timed(nccl_step, k, 3)
        nccl = {"what": "torch.distributed.all_reduce (NCCL) on fp16 gradients + one update "
                        "kernel over all elements", "ms_per_step": bms, "speedup": bms / ms}
        local.destroy()
        del mf, vf, gb

    if rank == 0:
        hbm_peak, peak_kind = measured_peaks()
        s_g, s_o = 2, 2
        # algorithmic bytes per launch (per GPU)
        b_hbm = N * s_g + (hi - lo) * 24 + (hi - lo) * s_o + (R - 1) * S * s_o
        b_nv = (R - 1) * S * (s_g + s_o)
        b_bus = b_nv  # bus GB/s always by the peer-to-peer formula, whatever the algorithm
        t = ms * 1e-3
        if R == 1:
            # dram read+write of an ncu capture of this kernel on 64 Mi elements
            # (profiles/fused_step_adam_mixed_1gpu.md): 1830.9 MB, i.e. 27.283 B per element;
            # traffic grows in proportion to the element count
            roof = {"bound": "hbm", "achieved": b_hbm / t / 1e9, "peak": hbm_peak, "unit": "GB/s",
                    "frac": b_hbm / t / 1e9 / hbm_peak, "traffic": 1830.9e6 / 67108864 * N,
                    "peak_kind": peak_kind, "algorithmic_bytes": b_hbm}
        else:
            # The roof is defined by the peer-to-peer algorithmic bytes per direction,
            # (R-1)/R * N * (s_g + s_o), whatever path the bytes take: the NVSwitch path
            # moves fewer bytes per link (each slice leaves a GPU once, each updated slice
            # arrives once) and may therefore exceed 1.0 of this roof.
            t_roof = max(b_nv / (NVLINK_PEER_GBS * 1e9), b_hbm / (hbm_peak * 1e9))
            roof = {"bound": "nvlink", "achieved": b_nv / t / 1e9, "peak": NVLINK_PEER_GBS,
                    "unit": "GB/s", "frac": t_roof / t, "traffic": None,
                    "peak_kind": "measured peer copy per direction (900 nominal)",
                    "algorithmic_bytes": b_nv, "hbm_bytes": b_hbm,
                    "frac_of_nominal_900": max(b_nv / 900e9, b_hbm / 8e12) / t}
            if use_nvls:
                link = N * s_g + (hi - lo) * s_o
                roof["nvls_link_bytes"] = link
                roof["nvls_link_gbs"] = link / t / 1e9
        line = {"metric": METRIC, "value": R * N / t / 1e9, "unit": UNIT, "n_gpus": R,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic",
                "config": {"workload": "mixed_adam_334M" if N == COUNT else f"mixed_adam_{N}",
                           "count": N, "world": R, "algo": "nvls" if use_nvls else "p2p", "grad": "f16", "state": "f32", "gathered": "f16",
                           "l2": "inputs larger than L2 (two 668 MB gradient buffers alternated)"},
                "bus_gbs": b_bus / t / 1e9, "roofline": roof, "clocks": clocks,
                "gpu_launches": int(launches), "e2e": e2e}
        if nccl:
            line["nccl_baseline"] = nccl
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(1 << 24, 1)
        print(json.dumps(line), flush=True)

    torch.cuda.synchronize()
    for t in runtime_allocs:
        comm.mem_free(t)
    comm.destroy()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
