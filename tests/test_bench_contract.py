"""The benchmark's reference arm runs without a GPU: its JSON line must carry
the keys the contract names, rank 0 alone prints, other ranks exit quietly."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(env_extra, gpus):
    env = dict(os.environ, **env_extra)
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                           "--gpus", str(gpus), "--steps", "1", "--warmup", "0"],
                          env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    r = _run({}, 1)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for k in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step",
              "higher_is_better", "scaling", "vs_baseline", "dtype", "data", "config",
              "cpu_baseline", "e2e"):
        assert k in d, k
    assert d["impl"] == "reference" and d["n_gpus"] == 1 and d["higher_is_better"] is True
    assert d["value"] > 0 and d["config"]["workload"] == "mixed_adam_334M"
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}


def test_reference_arm_other_ranks_exit_without_work():
    r = _run({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1", "MASTER_ADDR": "127.0.0.1",
              "MASTER_PORT": "29555"}, 2)
    assert r.returncode == 0, r.stderr[-2000:]
    assert not [ln for ln in r.stdout.splitlines() if ln.startswith("{")]


def test_parity_windows_and_host_oracle_are_self_consistent():
    """The benchmark's checker on the host: windows lie inside the rank's slice,
    are the same on every call, and the window oracle equals the full-tensor
    oracle restricted to the window (Adam, mixed precision, 3 steps, 2 ranks)."""
    import sys
    import numpy as np
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import bench
    import oracle_lib as O
    import seeded

    count, world = 5_000_000, 2
    for r in range(world):
        idx = bench.parity_windows(count, world, r)
        S = (count + world - 1) // world
        assert idx.min() >= r * S and idx.max() < min(count, (r + 1) * S)
        assert idx.size == (1 << 16) * 2 + (1 << 19) and np.array_equal(idx, bench.parity_windows(count, world, r))
    small = bench.parity_windows(1 << 20, 2, 1)
    assert np.array_equal(small, np.arange(1 << 19, 1 << 20))          # a short slice is checked whole

    cfg = dict(bench.CONFIGS[2], count=200_000, lr=1e-3)
    cfg.setdefault("loss_scale", 1024.0)
    steps, nbuf = 3, 2
    idx = np.arange(50_000, 60_000, dtype=np.int64)
    w, m, v, wl = bench.oracle_windows(cfg, world, 0, idx, steps, nbuf)
    # the same on the whole tensor
    full = np.arange(cfg["count"], dtype=np.int64)
    W = seeded.normal_np(full, bench.SEED, bench.WEIGHT_STREAM, 0, 0.02)
    M, V = np.zeros_like(W), np.zeros_like(W)
    WL = np.zeros(W.size, np.float16)
    for s in range(steps):
        grads = [bench.host_grad(full, cfg, r, s % nbuf) for r in range(world)]
        gsum = O.reduce_f16(grads, 1.0 / 1024.0)
        O.adam(W, M, V, gsum, 1e-3, 0.9, 0.999, 1e-6, s, w_lp=WL)
    assert np.array_equal(w, W[idx]) and np.array_equal(m, M[idx]) and np.array_equal(v, V[idx])
    assert np.array_equal(wl.view(np.uint16), WL[idx].view(np.uint16))
    assert bench.rel_err(w, W[idx], bench.rms(W[idx])) == 0.0
    assert bench.config_block(cfg, 2, "x")["workload"] == "mixed_adam_334M"
