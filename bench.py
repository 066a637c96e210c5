#!/usr/bin/env python
"""Benchmark of the fused AllReduce optimizer step.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--config 0|1|2|3] [--impl ours|reference]

Workloads (seeded synthetic inputs; --config, default 2):
  0  SGD, 1,048,576 fp32 parameters, lr 0.01, gradients ~ U[-1, 1)
  1  Adam fp32, 2^26 parameters, gradients ~ N(0, 1e-3)
  2  mixed-precision Adam on one flattened buffer of 334,000,000 parameters:
     fp16 Local gradients (loss scale 1024, removed in the kernel), fp32 master
     weights, fp32 Sliced m/v, fp16 Replicated weight copy that is all-gathered
  3  LAMB fp32, 334,000,000 parameters, weight decay 0.01
each at world size N, weights ~ N(0, 0.02), m = v = 0 at step 0, a fresh seeded
gradient every step (a pool of distinct buffers, reused in order once it is
exhausted).

A "step" is one fused call per rank: reduce-scatter of the gradients, the
update of the rank's slice, all-gather of the updated weights; one kernel.
`value` counts gradient elements reduced and applied per second over the whole
job (N ranks x count / step time), inputs resident in HBM.  `e2e` is the same
with the gradients arriving from pinned host memory and the updated weights
read back to the host every step.  After the timed region every rank checks
windows of the state the steps left behind against the CPU oracle (`parity`)
and the job exits non-zero if that fails.

For N > 1 launch with torchrun (one rank per GPU); rank 0 prints ONE JSON line.
`--impl reference` times the reference's CPU path on the host cores instead.
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
HYPER = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-6, weight_decay=0.01)
NVLINK_NOMINAL_GBS = 900.0   # per direction per GPU (18 links x 50 GB/s)
UNIT = "Gelem/s"
SEED = 20240229
WEIGHT_STREAM = 255          # generator stream of the weights (ranks use 0 .. R-1)
GRAD_POOL_BYTES = 24e9       # distinct gradient buffers kept on the device, per rank

CONFIGS = {
    0: dict(workload="sgd_fp32_1M", opt="sgd", grad="f32", lp=None, count=1 << 20, lr=0.01,
            dist="uniform"),
    1: dict(workload="adam_fp32_64M", opt="adam", grad="f32", lp=None, count=1 << 26, dist="normal"),
    2: dict(workload="mixed_adam_334M", opt="adam", grad="f16", lp="f16", count=COUNT, dist="normal",
            loss_scale=LOSS_SCALE),
    3: dict(workload="lamb_fp32_334M", opt="lamb", grad="f32", lp=None, count=COUNT, dist="normal"),
}


def workload_of(args):
    cfg = dict(CONFIGS[args.config])
    if args.count:
        cfg["count"] = args.count
        cfg["workload"] = f"{cfg['workload'].rsplit('_', 1)[0]}_{args.count}"
    cfg.setdefault("loss_scale", 1.0)
    cfg.setdefault("lr", HYPER["lr"])
    return cfg


def config_block(cfg, world, l2):
    """`config` of the JSON line: the same keys in both arms.  `l2` says how the
    timed steps were kept from running out of the last-level cache."""
    return {"workload": cfg["workload"], "count": cfg["count"], "world": world, "grad": cfg["grad"],
            "state": "f32", "gathered": cfg["lp"] or "f32", "l2": l2}


def metric_of(cfg):
    return f"fused_allreduce_{cfg['opt']}_grad_elems_per_s"


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def ncu_traffic_per_element(cfg, world):
    """DRAM bytes per element of the dominant kernel from the committed ncu
    capture of this workload's kernel, if there is one (traffic grows in
    proportion to the element count)."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
            for row in json.load(f)["captures"]:
                if row["workload"] == CONFIGS[2]["workload"] and cfg["opt"] == "adam" and \
                        cfg["grad"] == "f16" and world == row["world"]:
                    return row["dram_bytes"] / row["elements"], row["capture"]
    except Exception:
        pass
    return None, None


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



# ---- seeded inputs (device) and their host twins --------------------------------------
def grad_std(cfg):
    return 1e-3 * cfg["loss_scale"]


def fill_grad_(t, cfg, rank, k):
    import seeded
    if cfg["dist"] == "uniform":
        seeded.fill_uniform_(t, SEED, rank, k)
    else:
        seeded.fill_normal_(t, SEED, rank, k, grad_std(cfg))


def host_grad(idx, cfg, rank, k):
    import numpy as np
    import seeded
    dt = np.float16 if cfg["grad"] == "f16" else np.float32
    if cfg["dist"] == "uniform":
        return seeded.uniform_np(idx, SEED, rank, k, dt)
    return seeded.normal_np(idx, SEED, rank, k, grad_std(cfg), dt)


def cpu_baseline(cfg, count_sample, world, reps=2, threads=1, warmup=0, time_cap_s=120.0):
    """The reference's CPU path (host sum of `world` gradient arrays + the
    per-element passes) on a bounded sample: single-threaded like the
    reference's loops by default, or on `threads` host threads (Adam)."""
    import numpy as np
    import oracle_lib as O
    so = os.path.join(ROOT, "oracle", "liboracle.so")
    if not os.path.exists(so):
        subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "-s"])
    n = count_sample
    idx = np.arange(n, dtype=np.int64)
    grads = [host_grad(idx, cfg, r, 0) for r in range(world)]
    import seeded
    w = seeded.normal_np(idx, SEED, WEIGHT_STREAM, 0, 0.02)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    wl = np.zeros(n, np.float16) if cfg["lp"] else None
    inv = 1.0 / cfg["loss_scale"]
    h = HYPER
    best, done, t_begin = None, 0, time.perf_counter()
    for step in range(warmup + reps):
        t0 = time.perf_counter()
        if cfg["opt"] == "adam":
            O.cpu_step_adam(grads, w, m, v, cfg["lr"], h["beta1"], h["beta2"], h["eps"], step,
                            inv_scale=inv, w_lp=wl, threads=threads)
        else:
            gsum = O.reduce_f16(grads, inv) if cfg["grad"] == "f16" else O.reduce_f32(grads)
            if cfg["opt"] == "sgd":
                O.sgd(w, gsum, cfg["lr"])
            else:
                O.lamb(w, m, v, gsum, cfg["lr"], h["beta1"], h["beta2"], h["eps"],
                       h["weight_decay"], step, w_lp=wl)
        dt = time.perf_counter() - t0
        if step >= warmup:
            best = dt if best is None else min(best, dt)
            done += 1
        if time.perf_counter() - t_begin > time_cap_s and done >= 1:
            break
    used = threads if cfg["opt"] == "adam" else 1
    return {"value": world * n / best / 1e9, "unit": UNIT, "cores": used, "kind": "port",
            "steps_run": done,
            "sample": f"{n} of {cfg['count']} elements x {world} gradient arrays, best of {done}, "
                      f"{best * 1e3:.1f} ms per step on {used} thread(s); host has "
                      f"{os.cpu_count()} cores"}


def run_reference(args, rank, world):
    if rank != 0:
        return
    # Every host thread the box offers (the elements are independent: contiguous
    # ranges, one thread each); the sample grows with the thread count so that a
    # step stays long enough to time.  --steps / --warmup are honoured up to a
    # time cap of two minutes.
    import oracle_lib as O
    cfg = workload_of(args)
    threads = max(1, min(O.threads_available(), os.cpu_count() or 1))
    n = min(cfg["count"], (1 << 24) * max(1, threads // 4))
    cb = cpu_baseline(cfg, n, world, reps=max(1, args.steps), threads=threads,
                      warmup=max(0, args.warmup))
    one = cpu_baseline(cfg, min(cfg["count"], 1 << 24), world, reps=1, threads=1)
    cb["sample"] += f"; one thread: {one['value']:.4f} {UNIT}"
    steps = cb.pop("steps_run")
    line = {"impl": "reference", "metric": metric_of(cfg), "value": cb["value"], "unit": UNIT,
            "n_gpus": world, "steps": steps, "warmup": max(0, args.warmup),
            "ms_per_step": world * n / (cb["value"] * 1e9) * 1e3 * (cfg["count"] / n),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": config_block(cfg, world, "CPU arm: every step streams a sample far larger than "
                                               "the host's last-level cache"),
            "note": "CPU loops timed on a sample and reported as a rate; ms_per_step is that "
                    "rate scaled to the full count",
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_sweep(args, rank, world, local_rank):
    """Message-size sweep plus the named workloads: fused SGD,
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
    # RS_C_AG arm: the reduced slice, the gather's input and output
    gsl32 = torch.empty(Smax, dtype=torch.float32, device=dev)
    gsl16 = torch.empty(Smax, dtype=torch.float16, device=dev)
    ag32 = torch.zeros(Smax, dtype=torch.float32, device=dev)
    ag16 = torch.zeros(Smax, dtype=torch.float16, device=dev)
    agf32 = torch.empty(Smax * R, dtype=torch.float32, device=dev)
    agf16 = torch.empty(Smax * R, dtype=torch.float16, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    if use_nvls:
        # `auto` is the runtime's own choice: the switch for 16-bit gradients only
        comm.set_algo("nvls" if args.algo == "nvls" else "auto")

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
        times = []
        for i in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if world > 1:
                dist.barrier()
            e0.record()
            fn(warmup + i)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        # every iteration's time is the slowest rank's; the point is the median iteration
        # (these boxes share their switch and host: one iteration in ten runs long)
        t = torch.tensor(times, device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.median().item())

    hbm_peak, _ = measured_peaks()
    # per-direction link rate of this box: the copy engine's peer copy, measured here
    peer_gbs = comm.link_probe(g32, "copy") if world > 1 and not use_nvls else 0.0
    if not peer_gbs:
        peer_gbs = NVLINK_NOMINAL_GBS
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

        # RS_C_AG: reduce-scatter, update of the slice, all-gather of the updated slice
        # (the gather's input is a stand-in of the slice's size and type: timing only)
        SR = S * R
        even = SR == n
        out_t = (lp if lp is not None else w)
        gsl = (gsl16 if gt == "f16" else gsl32)[:S]
        ag_in = (ag16 if gt == "f16" else ag32)[:S]
        ag_out = (agf16 if gt == "f16" else agf32)[:SR]
        lo_r = min(n, rank * S)
        w_own = w[lo_r:lo_r + S] if even else None      # ragged counts: the arm is skipped
        lp_own = out_t[lo_r:lo_r + S] if (even and lp is not None) else None

        def stock_rs(i):
            gb.copy_(g)
            if world > 1:
                dist.reduce_scatter_tensor(gsl, gb)
            if opt == "sgd":
                local.fused_sgd(gsl, w_own, 1e-3, w_lp=lp_own, grad_scale=gs)
            elif opt == "adam":
                local.fused_adam(gsl, w_own, m[:S], v[:S], h["lr"], h["beta1"], h["beta2"], h["eps"], i,
                                 w_lp=lp_own, grad_scale=gs)
            else:
                local.fused_lamb(gsl, w_own, m[:S], v[:S], h["lr"], h["beta1"], h["beta2"], h["eps"],
                                 0.01, i, w_lp=lp_own, grad_scale=gs)
            if world > 1:
                dist.all_gather_into_tensor(ag_out, ag_in)

        steps = 5 if n >= (1 << 26) else 10
        ms = time_ms(fused, steps, 3)
        t_copy = time_ms(stock_copy_only, steps, 3)
        base = time_ms(stock, steps, 3) - t_copy
        base_rs = (time_ms(stock_rs, steps, 3) - t_copy) if world > 1 and even else None
        s_g = 2 if gt == "f16" else 4
        s_o = 2 if gt == "f16" else 4
        state = {"sgd": 8, "adam": 24, "lamb": 36}[opt] + (s_o if gt == "f16" else 0)
        b_bus = (R - 1) * S * (s_g + s_o)
        b_hbm = n * s_g + S * state + (R - 1) * S * s_o
        t_roof = max(b_bus / (peer_gbs * 1e9), b_hbm / (hbm_peak * 1e9))
        b2b = time_back_to_back(fused, 50, 5) if n <= (1 << 22) else None
        out.append({"opt": opt, "grad": gt, "count": n, "world": R, "ms_back_to_back": b2b,
                    "algo": "nvls" if use_nvls and (args.algo == "nvls" or gt == "f16") else "p2p",
                    "ms": ms, "bus_gbs": b_bus / ms / 1e6,
                    "hbm_gbs": b_hbm / ms / 1e6, "roof_frac": t_roof / (ms * 1e-3),
                    "stock_nccl_plus_update_ms": base, "stock_rs_update_ag_ms": base_rs,
                    "speedup": min(base, base_rs or base) / ms})
        if rank == 0:
            p = out[-1]
            print(f"# {opt:5s} {gt} n={n:>11d} fused {ms:9.4f} ms  bus {p['bus_gbs']:7.1f} GB/s  "
                  f"hbm {p['hbm_gbs']:7.1f} GB/s  roof {p['roof_frac']:.3f}  AR_C {base:9.4f} ms  "
                  f"RS_C_AG {(base_rs if base_rs is not None else float('nan')):9.4f} ms  "
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
            tlist = coco.TensorList(gl, wl)   # the pointer arrays, made once like a C caller's

            def time_queued_ms(fn, steps):
                # `steps` calls enqueued behind 0.7 ms of memsets, one event pair around them:
                # the device never waits for the host, whose work per call (a few hundred
                # tensors' pieces) would otherwise be timed too.  Every call streams 5 GB,
                # far more than L2 holds.
                fn(0)
                if world > 1:
                    dist.barrier()
                torch.cuda.synchronize()
                for _ in range(8):
                    flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for i in range(steps):
                    fn(1 + i)
                e1.record()
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
                if world > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                return float(t.item())

            def scattered(i):
                comm.fused_adam_scattered(tlist, None, msc, vsc, HYPER["lr"], HYPER["beta1"],
                                          HYPER["beta2"], HYPER["eps"], i)

            tot_f = tot // (8 * R) * (8 * R)   # keeps every rank's flat slice 16-byte aligned

            def flat(i):
                comm.fused_adam(g32[:tot_f], w32[:tot_f], m[:tot_f // R], v[:tot_f // R],
                                HYPER["lr"], HYPER["beta1"], HYPER["beta2"], HYPER["eps"], i)

            ms_sc, ms_fl = time_queued_ms(scattered, 10), time_queued_ms(flat, 10)
            out.append({"opt": "adam", "grad": "f32", "count": tot, "world": R, "tensors": len(shapes),
                        "scattered_ms": ms_sc, "flat_ms": ms_fl, "timing": "10 calls queued back to back"})
            if rank == 0:
                print(f"# adam  f32 scattered over {len(shapes)} BERT-large-shaped tensors, {tot} elements: "
                      f"{ms_sc:.4f} ms  (flat call on as many elements: {ms_fl:.4f} ms)", flush=True)

            # LAMB with one trust ratio per tensor, next to the flat call (one ratio overall)
            def scattered_lamb(i):
                comm.fused_lamb_scattered(tlist, None, msc, vsc, HYPER["lr"], HYPER["beta1"],
                                          HYPER["beta2"], HYPER["eps"], 0.01, i)

            def flat_lamb(i):
                comm.fused_lamb(g32[:tot_f], w32[:tot_f], m[:tot_f // R], v[:tot_f // R],
                                HYPER["lr"], HYPER["beta1"], HYPER["beta2"], HYPER["eps"],
                                0.01, i)

            ms_sc, ms_fl = time_queued_ms(scattered_lamb, 10), time_queued_ms(flat_lamb, 10)
            out.append({"opt": "lamb", "grad": "f32", "count": tot, "world": R, "tensors": len(shapes),
                        "scattered_ms": ms_sc, "flat_ms": ms_fl, "timing": "10 calls queued back to back"})
            if rank == 0:
                print(f"# lamb  f32 scattered (per-tensor trust ratios) over {len(shapes)} tensors: "
                      f"{ms_sc:.4f} ms  (flat call on as many elements: {ms_fl:.4f} ms)", flush=True)
    st = comm.status()
    if rank == 0:
        line = {"sweep": out, "n_gpus": R, "status": st["code"], "peer_copy_gbs": peer_gbs,
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



# ---- parity of the state the timed steps left behind ------------------------------------
def parity_windows(count, world, rank):
    """Global indices checked on `rank`: the first and last 64 Ki elements of its
    slice and a 512 Ki window at a seeded position (the same on every run)."""
    import numpy as np
    S = (count + world - 1) // world
    lo = min(count, rank * S)
    hi = min(count, lo + S)
    L = hi - lo
    if L <= (1 << 20):
        return np.arange(lo, hi, dtype=np.int64)
    k = 1 << 16
    mid_len = 1 << 19
    start = lo + k + int(np.random.default_rng((SEED, rank, world)).integers(0, L - 2 * k - mid_len))
    return np.concatenate([np.arange(lo, lo + k), np.arange(start, start + mid_len),
                           np.arange(hi - k, hi)]).astype(np.int64)


def oracle_windows(cfg, world, rank, idx, steps_run, nbuf):
    """The CPU oracle on the window `idx` of rank's slice for the steps that ran:
    returns w, m, v, w_lp (numpy) after `steps_run` steps.  LAMB needs the global
    norms, which a window cannot give: its weights are not produced (None)."""
    import numpy as np
    import oracle_lib as O
    import seeded
    h = HYPER
    w = seeded.normal_np(idx, SEED, WEIGHT_STREAM, 0, 0.02)
    m = np.zeros(idx.size, np.float32)
    v = np.zeros(idx.size, np.float32)
    wl = np.zeros(idx.size, np.float16) if cfg["lp"] else None
    inv = 1.0 / cfg["loss_scale"]
    for s in range(steps_run):
        grads = [np.ascontiguousarray(host_grad(idx, cfg, r, s % nbuf)) for r in range(world)]
        if cfg["grad"] == "f16":
            gsum = O.reduce_f16(grads, inv)
        else:
            gsum = O.reduce_f32(grads)
            if inv != 1.0:
                gsum = (gsum * np.float32(inv)).astype(np.float32)
        if cfg["opt"] == "sgd":
            O.sgd(w, gsum, cfg["lr"])
            if wl is not None:
                wl[:] = w.astype(np.float16)
        elif cfg["opt"] == "adam":
            O.adam(w, m, v, gsum, cfg["lr"], h["beta1"], h["beta2"], h["eps"], s, w_lp=wl)
        else:
            # moments only (they do not depend on the trust ratio): the update of
            # m and v is Adam's
            scratch = w.copy()
            O.adam(scratch, m, v, gsum, cfg["lr"], h["beta1"], h["beta2"], h["eps"], s)
    if cfg["opt"] == "lamb":
        return None, m, v, None
    return w, m, v, wl


def rel_err(a, b, floor):
    """max |a - b| / (max(|a|, |b|) + floor): relative where the values are
    large against `floor`, absolute (in units of floor) where they nearly cancel."""
    import numpy as np
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b) / (np.maximum(np.abs(a), np.abs(b)) + floor))) if a.size else 0.0


def rms(x):
    import numpy as np
    return float(np.sqrt(np.mean(np.asarray(x, np.float64) ** 2))) if x.size else 0.0


def numa_bind(local_rank):
    """Run this process (and so its pinned-memory allocations) on the host cores
    next to its GPU.  Returns the NUMA node, or None when the box has one node
    or does not say."""
    try:
        import torch
        p = torch.cuda.get_device_properties(local_rank)
        bus = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                a, _, b = part.partition("-")
                cpus.update(range(int(a), int(b or a) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return node
    except Exception:
        pass
    # the device does not say (containers often hide it): spread the ranks over the
    # host's memory nodes in order, as GPUs are usually numbered socket by socket
    try:
        import glob
        nodes = sorted(int(p.rsplit("node", 1)[1]) for p in glob.glob("/sys/devices/system/node/node[0-9]*"))
        world = int(os.environ.get("LOCAL_WORLD_SIZE", os.environ.get("WORLD_SIZE", "1")))
        if len(nodes) > 1 and world > 1:
            node = nodes[min(len(nodes) - 1, local_rank * len(nodes) // world)]
            with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
                cpus = set()
                for part in f.read().strip().split(","):
                    a, _, b = part.partition("-")
                    cpus.update(range(int(a), int(b or a) + 1))
            cpus &= os.sched_getaffinity(0)
            if cpus:
                os.sched_setaffinity(0, cpus)
                return node
    except Exception:
        pass
    return None


def run_probe(args, rank, world, local_rank):
    """The link yardstick alone: every mode and unroll of cocoLinkProbe over a
    1 GiB buffer (GB/s per direction per GPU), plus, where the node has an
    NVSwitch multicast mapping, the same through the switch and the time of the
    hybrid split (part of the slice through the switch, the rest peer to peer)."""
    import torch
    import torch.distributed as dist
    import coconet_b200 as coco

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world < 2:
        raise SystemExit("--probe measures links: launch it with torchrun on 2 or more GPUs")
    dist.init_process_group("nccl", device_id=dev)
    comm = coco.Communicator.from_torch_distributed()
    out = {}
    try:
        buf = torch.zeros(1 << 28, dtype=torch.float32, device=dev)
        comm.register(buf)
        out["copy_engine"] = round(comm.link_probe(buf, "copy"), 1)
        for mode in ("pull", "push", "both"):
            for u in (1, 2, 4):
                out[f"{mode}_u{u}"] = round(comm.link_probe(buf, mode, unroll=u), 1)
        sym = comm.mem_alloc(1 << 28, torch.float32)
        sym.zero_()
        torch.cuda.synchronize()
        if comm.has_multicast(sym):
            for mode in ("switch_reduce", "switch_store", "switch_both"):
                for u in (1, 2, 4):
                    out[f"{mode}_u{u}"] = round(comm.link_probe(sym, mode, unroll=u), 1)
            out["hybrid_us_by_sixteenths_through_switch"] = {
                str(k): round(comm.link_probe(sym, "hybrid", unroll=k), 1) for k in (0, 4, 8, 10, 12, 14, 16)}
        st = comm.status()
        if rank == 0:
            print(json.dumps({"link_probe": out, "n_gpus": world, "unit": "GB/s per direction per GPU",
                              "buffer_bytes": 1 << 30, "status": st["code"],
                              "topology": comm.topology()}), flush=True)
        torch.cuda.synchronize()
        comm.mem_free(sym)
    finally:
        comm.destroy()
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=sorted(CONFIGS),
                    help="workload: 0 SGD 1M, 1 Adam fp32 64M, 2 mixed Adam 334M (default), 3 LAMB 334M")
    ap.add_argument("--count", type=int, default=0, help="override the workload's element count")
    ap.add_argument("--no-baseline", action="store_true", help="skip the stock NCCL arms (N > 1)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-probe", action="store_true", help="skip the link probe (N > 1)")
    ap.add_argument("--symm", default="runtime", choices=["runtime", "torch"],
                    help="who makes the symmetric memory of the NVLS path")
    ap.add_argument("--sweep", action="store_true", help="message-size sweep instead of one workload")
    ap.add_argument("--sweep-max-log", type=int, default=30)
    ap.add_argument("--probe", action="store_true", help="the link yardstick alone (N > 1)")
    ap.add_argument("--algo", default=os.environ.get("COCO_BENCH_ALGO", "auto"),
                    choices=["auto", "p2p", "nvls"],
                    help="nvls: gradients and gathered weights in symmetric memory with an NVSwitch "
                         "multicast mapping; reduce-scatter and all-gather go through the switch. "
                         "auto: nvls from 4 ranks on for 16-bit gradients, else p2p")
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
    if args.probe:
        run_probe(args, rank, world, local_rank)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    import coconet_b200 as coco
    import seeded

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    cfg = workload_of(args)
    numa = numa_bind(local_rank)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        comm = coco.Communicator.from_torch_distributed()
    else:
        comm = coco.Communicator.init_all(1, [local_rank])[0]

    N, R = cfg["count"], world
    lo, hi = coco.slice_bounds(N, R, rank)
    S = (N + R - 1) // R
    gdt = torch.float16 if cfg["grad"] == "f16" else torch.float32
    s_g = 2 if cfg["grad"] == "f16" else 4
    s_o = 2 if cfg["lp"] else 4
    T = args.warmup + args.steps                     # fused steps of the main timed call
    stride = (N + 7) // 8 * 8                        # keeps every pooled buffer 16-byte aligned
    nbuf = int(max(2, min(T, GRAD_POOL_BYTES // (stride * s_g))))
    # auto: the NVSwitch path from 4 ranks on for 16-bit gradients (fewer bytes per link; fp32
    # gradients keep the fixed-order path and its 1e-5 contract), else peer-to-peer
    use_nvls = world > 1 and (args.algo == "nvls" or
                              (args.algo == "auto" and world >= 4 and cfg["grad"] == "f16"))
    symm, runtime_allocs = [], []

    def comm_buffer(numel, dtype):
        """A buffer peers touch: plain device memory (peer-mapped by the runtime
        over CUDA IPC), or symmetric memory with an NVSwitch multicast mapping --
        made by the runtime (cocoMemAlloc, default) or, with --symm torch, by
        torch's symmetric memory and handed over with cocoRegisterMapped."""
        if not use_nvls:
            t = torch.empty(numel, dtype=dtype, device=dev)
            if world > 1:
                comm.register(t)
            return t
        if args.symm == "runtime":
            t = comm.mem_alloc(numel, dtype)
            runtime_allocs.append(t)
            return t
        import torch.distributed._symmetric_memory as symm_mem
        t = symm_mem.empty(numel, dtype=dtype, device=dev)
        h = symm_mem.rendezvous(t, dist.group.WORLD)
        mc = int(h.multicast_ptr)
        if not mc and args.algo == "nvls":
            raise SystemExit("--algo nvls: this node exposes no NVLS multicast")
        comm.register_mapped(t, [int(p) for p in h.buffer_ptrs], mc)
        symm.append(h)
        return t

    failed, crashed = None, False
    try:
        # ---- seeded inputs, generated on the device (untimed) ----------------------------
        pool = comm_buffer(nbuf * stride, gdt)
        g = [pool[k * stride:k * stride + N] for k in range(nbuf)]
        for k in range(nbuf):
            fill_grad_(g[k], cfg, rank, k)
        if cfg["lp"]:
            w = torch.empty(N, dtype=torch.float32, device=dev)
            w_lp = comm_buffer(N, torch.float16)
        else:
            w = comm_buffer(N, torch.float32)
            w_lp = None
        seeded.fill_normal_(w, SEED, WEIGHT_STREAM, 0, 0.02)
        if w_lp is not None:
            w_lp.copy_(w)
        out = w_lp if w_lp is not None else w        # what the all-gather fills on every rank
        m = torch.zeros(S, device=dev)
        v = torch.zeros(S, device=dev)
        if use_nvls:
            comm.set_algo("nvls")
            # without a multicast mapping the runtime falls back to peer-to-peer
            use_nvls = (all(comm.has_multicast(t) for t in runtime_allocs) if args.symm == "runtime"
                        else all(int(h.multicast_ptr) != 0 for h in symm))
        elif world > 1:
            comm.set_algo("p2p")
        torch.cuda.synchronize()

        step_no = [0]
        h = HYPER
        gs = 1.0 / cfg["loss_scale"]

        def fused_on(c, gbuf, ww, mm, vv, lp, step):
            if cfg["opt"] == "sgd":
                c.fused_sgd(gbuf, ww, cfg["lr"], w_lp=lp, grad_scale=gs)
            elif cfg["opt"] == "adam":
                c.fused_adam(gbuf, ww, mm, vv, cfg["lr"], h["beta1"], h["beta2"], h["eps"], step,
                             w_lp=lp, grad_scale=gs)
            else:
                c.fused_lamb(gbuf, ww, mm, vv, cfg["lr"], h["beta1"], h["beta2"], h["eps"],
                             h["weight_decay"], step, w_lp=lp, grad_scale=gs)

        def fused_step(gbuf):
            fused_on(comm, gbuf, w, m, v, w_lp, step_no[0])
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

        small = N * s_g * nbuf <= 256e6      # the whole gradient pool would sit in L2 (126 MB)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if small else None

        def timed_flushed(fn, steps, warmup):
            """For workloads smaller than L2: a 256 MB memset before every step pushes
            the previous step's lines out, and every step is timed by its own event
            pair (the flush is outside the pairs); mean over steps, max over ranks."""
            for i in range(warmup):
                fn(i)
            barrier()
            total = 0.0
            for i in range(steps):
                flush.zero_()
                if world > 1:
                    dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn(warmup + i)
                e1.record()
                torch.cuda.synchronize()
                total += e0.elapsed_time(e1)
            ms = torch.tensor([total / steps], device=dev)
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            barrier()
            return float(ms.item())

        sampler = ClockSampler(local_rank) if rank == 0 else None
        if sampler:
            sampler.start()
        l0 = comm.launch_count()
        ms = (timed_flushed if small else timed)(lambda i: fused_step(g[i % nbuf]), args.steps, args.warmup)
        launches = comm.launch_count() - l0 - args.warmup
        clocks = sampler.stop() if sampler else None
        # the last timed step as CTA 0 of rank 0 saw it (GPU timer): first data phase, norm
        # exchange, last data phase (everything but LAMB has only the last)
        phases_us = [round(x, 1) for x in comm.last_phase_times()]
        # ... and how evenly its work was spread: first, median and last CTA of rank 0
        spread_us = [round(x, 1) for x in comm.last_cta_spread()] \
            if hasattr(coco.lib(), "cocoLastCtaSpread") else None
        st = comm.status()
        if st["code"] != 0:
            raise RuntimeError(f"device-side failure during the benchmark: {st}")

        # ---- parity: windows of the state those T steps left, against the CPU oracle ------
        parity = None
        if not args.no_parity:
            idx = parity_windows(N, R, rank)
            didx = torch.from_numpy(idx).to(dev)
            got_w = w[didx].cpu().numpy()
            got_m = m[didx - lo].cpu().numpy()
            got_v = v[didx - lo].cpu().numpy()
            got_out = out[didx].cpu().numpy()
            # the all-gather: every rank's copy of the gathered tensor must hold, at every
            # rank's windows, the bits that rank holds itself; and the copies must agree as
            # wholes (64-bit sum of the raw bits, compared over the ranks)
            gather_ok, replicas_ok = True, True
            if world > 1:
                mine = out[didx].contiguous()
                sizes = [parity_windows(N, R, q).size for q in range(R)]
                bufs = [torch.empty(sizes[q], dtype=out.dtype, device=dev) for q in range(R)]
                dist.all_gather(bufs, mine)
                ibits = torch.int16 if out.dtype == torch.float16 else torch.int32
                for q in range(R):
                    qi = torch.from_numpy(parity_windows(N, R, q)).to(dev)
                    gather_ok = gather_ok and bool(torch.equal(out[qi].view(ibits), bufs[q].view(ibits)))
                csum = out.view(ibits).sum(dtype=torch.int64).reshape(1)
                sums = [torch.empty_like(csum) for _ in range(R)]
                dist.all_gather(sums, csum)
                replicas_ok = all(int(x.item()) == int(sums[0].item()) for x in sums)
            t0 = time.perf_counter()
            ow, om, ov, owl = oracle_windows(cfg, R, rank, idx, T, nbuf)
            exact_mv = bool(np.array_equal(got_m, om) and np.array_equal(got_v, ov)) \
                if cfg["opt"] != "sgd" else True
            fixed_order = not use_nvls
            tol_w = 1e-5 if cfg["grad"] == "f32" and fixed_order else 2e-3
            # Every quantity is compared relative to its own scale: |got - want| / (max(|got|,
            # |want|) + rms(want)).  A plain relative error is meaningless for the elements of
            # w and m that lie near zero, and the switch path's 16-bit-rounded sums move every
            # element by about 2^-12 of the typical gradient per step.
            detail = {}
            exact_w = None
            if ow is not None:
                detail["w"] = rel_err(got_w, ow, rms(ow))
                exact_w = bool(np.array_equal(got_w, ow))
                if owl is not None:
                    detail["gathered"] = rel_err(got_out.astype(np.float32), owl.astype(np.float32), rms(ow))
                    exact_w = exact_w and bool(np.array_equal(got_out.view(np.uint16), owl.view(np.uint16)))
                else:
                    detail["gathered"] = rel_err(got_out, ow, rms(ow))
            if cfg["opt"] != "sgd":
                detail["m"] = rel_err(got_m, om, rms(om))
                detail["v"] = rel_err(got_v, ov, rms(ov))
            # The stated tolerance is on the results, the weights.  The moments are
            # intermediates whose every step's contribution carries the 16-bit rounding of
            # that step's sum: m may be off by twice, v (g squared) by three times as much.
            max_rel = max([detail[k] for k in ("w", "gathered") if k in detail] or [0.0])
            moments_ok = detail.get("m", 0.0) <= 2 * tol_w and detail.get("v", 0.0) <= 3 * tol_w
            ok = max_rel <= tol_w and moments_ok and gather_ok and replicas_ok
            if fixed_order:  # fixed summation order: the moments match a CPU evaluation bit for bit
                ok = ok and exact_mv
                if cfg["opt"] != "lamb":
                    ok = ok and bool(exact_w)
            flags = torch.tensor([1 if ok else 0, 1 if exact_mv else 0, 1 if (exact_w or exact_w is None) else 0],
                                 device=dev)
            worst = torch.tensor([max_rel], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(flags, op=dist.ReduceOp.MIN)
                dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            parity = {"checked": int(idx.size) * R, "steps": T, "path": "nvls" if use_nvls else "p2p",
                      "max_rel": float(worst.item()), "tolerance": tol_w, "rank0_detail": detail,
                      "exact_mv": bool(flags[1].item()), "exact_w": bool(flags[2].item()),
                      "gather_ok": gather_ok, "replicas_identical": replicas_ok,
                      "ok": bool(flags[0].item()),
                      "what": "oracle on 64 Ki + 512 Ki + 64 Ki elements of every rank's slice after all "
                              "timed and warm-up steps: master weights, m, v, gathered copy; every "
                              "rank's copy compared with the owners' bits; every difference as |got - want| / "
                              "(max(|got|, |want|) + rms(want)); max_rel = the weights' and the gathered "
                              "copy's (<= tolerance), the moments' may be 2x (m) and 3x (v) that"
                              + ("; LAMB: moments only (the weights need the global norms)"
                                 if cfg["opt"] == "lamb" else ""),
                      "oracle_s": round(time.perf_counter() - t0, 2)}

        # ---- end to end: host gradients in, updated weights out to the host ---------------
        e2e = None
        if not args.no_e2e:
            hg = torch.empty(N, dtype=gdt).pin_memory()
            hg.copy_(g[0])
            hout = torch.empty(N, dtype=out.dtype).pin_memory()
            # Every step copies its gradients in from pinned host memory and the gathered
            # weights out to pinned host memory.  The copies run on two side streams and
            # both ends are double-buffered on the device: step i+1's gradients travel in
            # while step i computes, and step i's weights -- copied aside on the device
            # right after its kernel (0.2 ms) -- travel out while step i+1 computes.
            cur = torch.cuda.current_stream()
            s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
            ev_in = [torch.cuda.Event(), torch.cuda.Event()]
            ev_kernel = [torch.cuda.Event(), torch.cuda.Event()]
            ev_staged = torch.cuda.Event()
            ev_out = torch.cuda.Event()
            stage = torch.empty_like(out)

            def e2e_step(i):
                b = i & 1
                s_in.wait_event(ev_kernel[b])      # the kernel two steps back is done with g[b]
                with torch.cuda.stream(s_in):
                    g[b].copy_(hg, non_blocking=True)
                    ev_in[b].record(s_in)
                cur.wait_event(ev_in[b])
                fused_step(g[b])
                ev_kernel[b].record(cur)
                cur.wait_event(ev_out)             # the previous weights have left the staging copy
                stage.copy_(out, non_blocking=True)
                ev_staged.record(cur)
                s_out.wait_event(ev_staged)
                with torch.cuda.stream(s_out):
                    hout.copy_(stage, non_blocking=True)
                    ev_out.record(s_out)

            k = max(3, min(args.steps, 10))
            ems = timed(e2e_step, k, 2, finish=lambda: cur.wait_event(ev_out))
            e2e = {"value": R * N / (ems * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": ems,
                   "h2d_bytes_per_step": N * s_g, "d2h_bytes_per_step": N * s_o,
                   "overlap": "copies on two side streams, gradients and outgoing weights double-buffered",
                   "host_gbs_all_ranks": R * N * (s_g + s_o) / (ems * 1e-3) / 1e9,
                   "numa_node": numa}
            del hg, hout, stage

        # ---- stock NCCL arms: AR_C (all-reduce + update over all elements) and RS_C_AG
        # (reduce-scatter + update of the slice + all-gather), the reference's two unfused
        # schedules.  The gradient copy is refilled before every step outside the events;
        # every part is timed with its own event pair.
        nccl = None
        if world > 1 and not args.no_baseline:
            local = coco.Communicator.init_all(1, [local_rank])[0]
            k = max(3, min(args.steps, 10))
            SR = S * R
            gb = torch.zeros(SR, dtype=gdt, device=dev)
            gsl = torch.empty(S, dtype=gdt, device=dev)
            mf = torch.zeros(N, device=dev)
            vf = torch.zeros(N, device=dev)
            m2 = torch.zeros(S, device=dev)
            v2 = torch.zeros(S, device=dev)
            # the slice update works on this rank's slice of the real state when the count
            # divides evenly, else on stand-ins of the same sizes; the all-gather moves a
            # buffer of the slice's size and type into a full-size one (timing only)
            even = SR == N
            w_own = w[lo:lo + S] if even else torch.zeros(S, device=dev)
            lp_own = (out[lo:lo + S] if even else torch.zeros(S, dtype=out.dtype, device=dev)) \
                if cfg["lp"] else None
            ag_in = torch.zeros(S, dtype=out.dtype, device=dev)
            out_full = torch.empty(SR, dtype=out.dtype, device=dev)

            def timed_parts(parts, steps, warmup):
                """parts: list of callables run in order each step; returns ms per part
                (mean over steps, max over ranks) and their sum."""
                tot = [0.0] * len(parts)
                for i in range(warmup + steps):
                    gb[:N].copy_(g[i % nbuf])
                    if world > 1:
                        dist.barrier()
                    ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(parts) + 1)]
                    ev[0].record()
                    for j, part in enumerate(parts):
                        part(i)
                        ev[j + 1].record()
                    torch.cuda.synchronize()
                    if i >= warmup:
                        for j in range(len(parts)):
                            tot[j] += ev[j].elapsed_time(ev[j + 1])
                t = torch.tensor([x / steps for x in tot] + [sum(tot) / steps], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                return [float(x) for x in t.tolist()]

            bstep = [0]

            def upd_full(i):
                fused_on(local, gb[:N], w, mf, vf, w_lp, bstep[0])
                bstep[0] += 1

            ar, up, tot_ar = timed_parts([lambda i: dist.all_reduce(gb), upd_full], k, 3)
            bstep[0] = 0

            def upd_slice(i):
                fused_on(local, gsl, w_own, m2, v2, lp_own, bstep[0])
                bstep[0] += 1

            rs, us, ag, tot_rs = timed_parts(
                [lambda i: dist.reduce_scatter_tensor(gsl, gb),
                 upd_slice,
                 lambda i: dist.all_gather_into_tensor(out_full, ag_in)], k, 3)
            best = min(tot_ar, tot_rs)
            nccl = {"ar_c": {"what": "torch.distributed.all_reduce (NCCL) on the gradients + one update "
                                     "kernel over all elements", "allreduce_ms": ar, "update_ms": up,
                             "ms_per_step": tot_ar},
                    "rs_c_ag": {"what": "reduce_scatter_tensor + update kernel on the slice + "
                                        "all_gather_into_tensor of the updated slice"
                                        + (" (LAMB: the slice's own norms, no norm exchange)"
                                           if cfg["opt"] == "lamb" else ""),
                                "rs_ms": rs, "update_ms": us, "ag_ms": ag, "ms_per_step": tot_rs},
                    "ms_per_step": best, "faster_arm": "ar_c" if tot_ar <= tot_rs else "rs_c_ag",
                    "speedup": best / ms,
                    "timing": "per part CUDA events, gradient copy refilled outside the events, "
                              "mean over steps, max over ranks"}
            local.destroy()
            del mf, vf, gb, gsl, m2, v2, ag_in, out_full

        # ---- what the links give a kernel of this shape (untimed, after everything else) ----
        probe = None
        if world > 1 and not args.no_probe:
            # on (at most 1 GiB of) the gradient pool, whose contents are no longer needed;
            # a workload with a small pool gets a buffer of its own
            pb = pool[:min(pool.numel(), (1 << 30) // s_g)]
            if pb.numel() * s_g < (256 << 20):
                pb = comm_buffer(1 << 26, torch.float32)
            pool = pb
            probe = {"copy_engine": comm.link_probe(pool, "copy"),
                     "pull": comm.link_probe(pool, "pull", unroll=2),
                     "push": comm.link_probe(pool, "push", unroll=2),
                     "pull_and_push": comm.link_probe(pool, "both", unroll=2),
                     "unit": "GB/s per direction per GPU",
                     "what": "16-byte peer loads / stores with the fused step's slice pattern and no "
                             "update; copy_engine = cudaMemcpyAsync from the next rank"}
            if use_nvls and args.symm == "runtime":
                probe["switch_reduce_and_store"] = comm.link_probe(pool, "switch_both", unroll=2)

        if rank == 0:
            hbm_peak, peak_kind = measured_peaks()
            L = hi - lo
            state = {"sgd": 8, "adam": 24, "lamb": 36}[cfg["opt"]]
            # algorithmic bytes per launch (per GPU)
            b_hbm = N * s_g + L * state + (L * s_o if cfg["lp"] else 0) + (R - 1) * S * s_o
            b_nv = (R - 1) * S * (s_g + s_o)
            t = ms * 1e-3
            if R == 1:
                per_elem, capture = ncu_traffic_per_element(cfg, R)
                roof = {"bound": "hbm", "achieved": b_hbm / t / 1e9, "peak": hbm_peak, "unit": "GB/s",
                        "frac": b_hbm / t / 1e9 / hbm_peak,
                        "traffic": per_elem * N if per_elem else None, "traffic_from": capture,
                        "peak_kind": peak_kind, "algorithmic_bytes": b_hbm}
            else:
                # The link bytes of the algorithm that ran, per GPU and direction: peer to peer
                # (R-1)/R * N * (s_g + s_o); through the switch the whole gradient buffer
                # leaves once and the whole gathered buffer arrives once, plus the slice the
                # other way.  The peak is the copy-engine peer copy measured in this run.
                link_bytes = max(N * s_g + L * s_o, L * s_g + N * s_o) if use_nvls else b_nv
                peak = probe["copy_engine"] if probe and probe["copy_engine"] > 0 else NVLINK_NOMINAL_GBS
                kind = "measured in this run: copy-engine peer copy, per direction" if probe \
                    else "constant: nominal NVLink rate per direction"
                t_link, t_hbm = link_bytes / (peak * 1e9), b_hbm / (hbm_peak * 1e9)
                roof = {"bound": "nvlink" if t_link >= t_hbm else "hbm",
                        "achieved": link_bytes / t / 1e9, "peak": peak, "unit": "GB/s",
                        "frac": max(t_link, t_hbm) / t, "traffic": None, "peak_kind": kind,
                        "algorithmic_bytes": link_bytes, "hbm_bytes": b_hbm, "hbm_peak": hbm_peak,
                        "frac_of_nominal_900": max(link_bytes / (NVLINK_NOMINAL_GBS * 1e9),
                                                   b_hbm / 8e12) / t,
                        "p2p_formula_bytes": b_nv,
                        "frac_of_p2p_roof_at_900": max(b_nv / (NVLINK_NOMINAL_GBS * 1e9),
                                                       b_hbm / 8e12) / t}
            line = {"metric": metric_of(cfg), "value": R * N / t / 1e9, "unit": UNIT, "n_gpus": R,
                    "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                    "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                    "data": "synthetic",
                    "config": config_block(
                        cfg, R, f"inputs larger than L2 ({nbuf} gradient buffers of "
                                f"{N * s_g / 1e6:.0f} MB used in turn, no flush)" if N * s_g * nbuf > 256e6
                        else "small workload: L2 flushed (a 256 MB memset) before every timed step, "
                             "every step under its own event pair"),
                    "algo": "nvls" if use_nvls else "p2p",
                    "bus_gbs": b_nv / t / 1e9, "roofline": roof, "clocks": clocks,
                    "gpu_launches": int(launches), "e2e": e2e, "parity": parity,
                    "phases_us": {"first_data_phase": phases_us[0], "norm_exchange": phases_us[1],
                                  "last_data_phase": phases_us[2],
                                  "cta_end_first_median_last": spread_us,
                                  "what": "the last timed step inside the kernel, CTA 0 of rank 0, GPU timer"}}
            if probe:
                line["link_probe"] = probe
            if nccl:
                line["nccl_baseline"] = nccl
            if world == 1 and not args.no_cpu:
                cb = cpu_baseline(cfg, min(N, 1 << 24), 1)
                cb.pop("steps_run", None)
                line["cpu_baseline"] = cb
            print(json.dumps(line), flush=True)
        if parity is not None and not parity["ok"]:
            failed = f"parity check failed: {parity}"
    except Exception as e:
        failed = f"{type(e).__name__}: {e}"
        crashed = True
    else:
        crashed = False
    # Release what peers have mapped before the process goes away: symmetric allocations
    # (unbound from the multicast object, unmapped) and the communicator, behind a barrier
    # so that no peer still works on this rank's memory.  After an exception on this rank
    # alone the collective release could wait for peers that are elsewhere: then only what
    # is local is released (the runtime's own waits are bounded).
    try:
        torch.cuda.synchronize()
        if not crashed:
            if world > 1:
                dist.barrier()
            for t in runtime_allocs:
                comm.mem_free(t)
            comm.destroy()
            if world > 1:
                dist.barrier()
                dist.destroy_process_group()
        elif world == 1:
            comm.destroy()
    except Exception as e:
        failed = failed or f"cleanup: {type(e).__name__}: {e}"
    if failed:
        print(failed, file=sys.stderr)
        sys.exit(1)


if __name__ == "__main__":
    main()
