"""Pins the CPU oracle: closed-form known answers taken from the reference's
frozen test programs, and the reference's own host checkers compiled from the
reference tree (oracle/_ref, built by `make -C oracle ref`)."""
import numpy as np
import pytest

import oracle_lib as O

needs_ref = pytest.mark.skipif(not O.ref_available(), reason="oracle/_ref not built")


def _grads(R, n, seed, scale=1.0, dtype=np.float32):
    return [(np.random.default_rng((seed, r)).standard_normal(n) * scale).astype(dtype)
            for r in range(R)]


# ---- known answers ----------------------------------------------------------

@pytest.mark.parametrize("R", [1, 2, 4, 8, 16])
def test_sgd_identical_inputs(R):
    # examples/test-sgd.cu: g and w come from the same generator with the same
    # seed on every rank and lr = 1, so w' = w - R*w.
    w0 = np.random.default_rng(1234).random(1000, dtype=np.float32)
    g = [w0.copy() for _ in range(R)]
    w = w0.copy()
    O.sgd(w, O.reduce_f32(g), 1.0)
    np.testing.assert_allclose(w, w0 * (1 - R), rtol=1e-6)


@pytest.mark.parametrize("R", [1, 2, 3, 8])
def test_adam_constant_inputs(R):
    # examples/test-adam.cu:73-88: g = 1 on every rank, w = m = v = 0,
    # lr = 1, beta1 = beta2 = 0.5.
    n = 257
    g = [np.ones(n, np.float16) for _ in range(R)]
    # forked-NCCL functors: m = R/2, m_ = R, v = R^2/2, v_ = R^2 -> w' = -1.
    gh = O.reduce_f16_ring(g, owner=0)
    assert np.all(gh == np.float16(R))
    w, m, v = (np.zeros(n, np.float32) for _ in range(3))
    wl = np.zeros(n, np.float16)
    O.adam(w, m, v, None, 1.0, 0.5, 0.5, 0.0, 0, O.NCCL, w_lp=wl, gsum_h=gh)
    assert np.all(w == -1.0) and np.all(wl == np.float16(-1.0))
    assert np.all(m == R / 2) and np.all(v == R * R / 2)
    # DSL program: w' = 0 - (R)/(R^2) = -1/R.
    w, m, v = (np.zeros(n, np.float32) for _ in range(3))
    O.adam(w, m, v, O.reduce_f32([x.astype(np.float32) for x in g]), 1.0, 0.5, 0.5, 0.0, 0, O.DSL)
    np.testing.assert_allclose(w, -1.0 / R, rtol=1e-7)
    # bias-corrected form at t = 1: m^ = g, v^ = g^2 -> w' = -g/(|g| + eps).
    w, m, v = (np.zeros(n, np.float32) for _ in range(3))
    O.adam(w, m, v, np.full(n, R, np.float32), 1.0, 0.5, 0.5, 1e-6, 0, O.OVERLAP)
    np.testing.assert_allclose(w, -R / (R + 1e-6), rtol=1e-6)


def test_reduce_f16_ring_order_and_rounding():
    # 2048 + 1 is not representable in fp16: the ring order decides the result.
    g = [np.array([2048.0], np.float16), np.array([1.0], np.float16), np.array([1.0], np.float16)]
    assert O.reduce_f16_ring(g, owner=0)[0] == np.float16(2050.0)   # (1+1)+2048
    assert O.reduce_f16_ring(g, owner=2)[0] == np.float16(2048.0)   # (2048+1)+1 -> ties to even
    assert O.reduce_f16(g)[0] == 2050.0                              # fp32 accumulate


def test_lamb_trust_ratio_guards():
    n = 64
    g = np.zeros(n, np.float32)
    # w = 0 -> ||w|| = 0 -> trust ratio 1; g = 0 -> r = 0 -> step 0.
    w, m, v = (np.zeros(n, np.float32) for _ in range(3))
    wn, rn = O.lamb(w, m, v, g, 1e-3, 0.9, 0.999, 1e-6, 0.01, 0)
    assert wn == 0 and rn == 0 and np.all(w == 0)
    # constant case, t = 1: m^ = g, v^ = g^2 -> r = g/(|g|+eps) + wd*w
    w = np.full(n, 2.0, np.float32); m = np.zeros(n, np.float32); v = np.zeros(n, np.float32)
    g = np.full(n, 3.0, np.float32)
    wn, rn = O.lamb(w, m, v, g, 0.5, 0.9, 0.999, 0.0, 0.25, 0)
    r = 1.0 + 0.25 * 2.0
    np.testing.assert_allclose([wn, rn], [2.0 * 8, r * 8], rtol=1e-6)
    np.testing.assert_allclose(w, 2.0 - 0.5 * (2.0 / r) * r, rtol=1e-6)


def test_cpu_step_matches_elementwise_adam():
    R, n = 4, 4099
    w0 = (np.random.default_rng(7).standard_normal(n) * 0.02).astype(np.float32)
    w1, m1, v1 = w0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    w2, m2, v2 = w0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    for step in range(3):
        g = _grads(R, n, 100 + step, 1e-3)
        O.adam(w1, m1, v1, O.reduce_f32(g), 1e-3, 0.9, 0.999, 1e-6, step)
        O.cpu_step_adam(g, w2, m2, v2, 1e-3, 0.9, 0.999, 1e-6, step)
    assert np.array_equal(w1, w2) and np.array_equal(m1, m2) and np.array_equal(v1, v2)
    # fp16 gradients with loss scale
    gh = [(x * 1024).astype(np.float16) for x in _grads(R, n, 5, 1e-3)]
    wl1, wl2 = np.zeros(n, np.float16), np.zeros(n, np.float16)
    O.adam(w1, m1, v1, O.reduce_f16(gh, 1 / 1024), 1e-3, 0.9, 0.999, 1e-6, 3, w_lp=wl1)
    O.cpu_step_adam(gh, w2, m2, v2, 1e-3, 0.9, 0.999, 1e-6, 3, inv_scale=1 / 1024, w_lp=wl2)
    assert np.array_equal(w1, w2) and np.array_equal(wl1, wl2)
    assert np.array_equal(wl1, w1.astype(np.float16))
    # the multi-threaded form (the benchmark's reference arm) gives the same bits
    w3, m3, v3, wl3 = w0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros(n, np.float16)
    w4, m4, v4, wl4 = w0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros(n, np.float16)
    for step in range(2):
        O.cpu_step_adam(gh, w3, m3, v3, 1e-3, 0.9, 0.999, 1e-6, step, inv_scale=1 / 1024, w_lp=wl3)
        O.cpu_step_adam(gh, w4, m4, v4, 1e-3, 0.9, 0.999, 1e-6, step, inv_scale=1 / 1024, w_lp=wl4,
                        threads=5)
    assert np.array_equal(w3, w4) and np.array_equal(m3, m4) and np.array_equal(v3, v4)
    assert np.array_equal(wl3, wl4) and O.threads_available() >= 1


# ---- the reference's own host checkers --------------------------------------

@needs_ref
@pytest.mark.parametrize("R", [1, 2, 8])
def test_ref_checker_accepts_oracle_sgd(R):
    n = 5000
    g = [np.random.default_rng((3, r)).uniform(-1, 1, n).astype(np.float32) for r in range(R)]
    w0 = (np.random.default_rng(9).standard_normal(n) * 0.02).astype(np.float32)
    w = w0.copy()
    O.sgd(w, O.reduce_f32(g), 0.01)
    assert O.ref_sgd_check(g, w0, 0.01, w)
    bad = w.copy(); bad[n // 2] *= 1.01
    assert not O.ref_sgd_check(g, w0, 0.01, bad)


@needs_ref
@pytest.mark.parametrize("R", [2, 8])
def test_ref_checker_accepts_oracle_adam_dsl(R):
    n = 3000
    rng = np.random.default_rng(11)
    g = _grads(R, n, 21)
    w0 = rng.standard_normal(n).astype(np.float32)
    m0 = rng.standard_normal(n).astype(np.float32)
    v0 = rng.random(n).astype(np.float32) + 0.1
    w, m, v = w0.copy(), m0.copy(), v0.copy()
    O.adam(w, m, v, O.reduce_f32(g), 0.5, 0.9, 0.999, 0.0, 0, O.DSL)
    assert O.ref_adam_dsl_check(g, w0, m0, v0, 0.5, 0.9, 0.999, w)
    bad = w.copy(); bad[7] *= 1.01
    assert not O.ref_adam_dsl_check(g, w0, m0, v0, 0.5, 0.9, 0.999, bad)


@needs_ref
@pytest.mark.parametrize("kind", ["adam", "lamb"])
@pytest.mark.parametrize("betas", [(0.5, 0.5), (0.9, 0.999)])
def test_ref_checker_accepts_oracle_overlap(kind, betas):
    # multi-process-adam-scattered.cpp runs 25 epochs with running moments and
    # compares at rel 1e-5; feed it the oracle's weights epoch by epoch.  The
    # checker advances its own m/v: they must equal the oracle's bit for bit.
    R, n, lr, eps = 4, 4096, 1e-3, 1e-6
    b1, b2 = betas
    w = (np.random.default_rng(5).standard_normal(n) * 0.02).astype(np.float32)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    rm, rv = np.zeros(n, np.float32), np.zeros(n, np.float32)
    for epoch in range(25):
        g = _grads(R, n, 1000 + epoch, 1e-3)
        w_old = w.copy()
        if kind == "adam":
            O.adam(w, m, v, O.reduce_f32(g), lr, b1, b2, eps, epoch)
            stepsize = -lr          # the sample adds stepsize * m^/(sqrt(v^)+eps)
        else:
            # the sample's LAMB has weight decay 1.0 and its own scale formula
            O.lamb(w, m, v, O.reduce_f32(g), lr, b1, b2, eps, 1.0, epoch,
                   flags=O.LAMB_REF_QUIRK)
            stepsize = lr
        assert O.ref_overlap_check(kind, g, epoch, w_old, w, rm, rv, b1, b2, stepsize, eps), epoch
        assert np.array_equal(rm, m) and np.array_equal(rv, v)
    bad = w.copy(); bad[3] = bad[3] * 1.001 + 1e-3
    g = _grads(R, n, 1, 1e-3)
    assert not O.ref_overlap_check(kind, g, 25, w, bad, rm, rv, b1, b2, -lr, eps)


def test_lamb_nccl_variant_known_answer_and_decay_constant():
    # reduce_kernel.h:391-452 / common_kernel.h:2699 on the frozen tests' constants:
    # r = 1 everywhere, ||w|| = 0 -> scale = 1/sqrt(n), w' = -1/sqrt(n) for any R
    n = 4096
    for R in (1, 2, 8):
        gsum = np.full(n, float(R), np.float32)       # fp16 ring sum of R ones
        w, m, v = np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros(n, np.float32)
        wl = np.zeros(n, np.float16)
        wn, rn = O.lamb(w, m, v, gsum, 1.0, 0.5, 0.5, 0.0, 0.01, 0, O.NCCL, w_lp=wl)
        assert np.all(w == np.float32(-1.0 / 64.0)) and np.all(wl == np.float16(-1.0 / 64.0))
        assert np.all(m == R / 2) and np.all(v == R * R / 2)
        assert wn == 0.0 and rn == 64.0
    # the decay factor is the constant 1.0: weight_decay and eps are ignored
    rng = np.random.default_rng(3)
    g = rng.standard_normal(1000).astype(np.float16).astype(np.float32)
    outs = []
    for wd, eps in ((0.01, 1e-6), (0.5, 0.0)):
        w = (rng.standard_normal(1000) * 0 + np.linspace(-0.05, 0.05, 1000)).astype(np.float32)
        m, v = np.zeros(1000, np.float32), np.zeros(1000, np.float32)
        O.lamb(w, m, v, g, 1e-3, 0.9, 0.999, eps, wd, 0, O.NCCL)
        outs.append(w)
    assert np.array_equal(outs[0], outs[1])
    # against the formula written out in numpy (fp32 throughout)
    w0 = np.linspace(-0.05, 0.05, 1000).astype(np.float32)
    f = np.float32
    gg = (g * g).astype(np.float16).astype(np.float32)
    vn = gg * (f(1) - f(0.999))
    mn = g * (f(1) - f(0.9))
    r = (mn / f(0.9)) / np.sqrt(vn / f(0.999)) + f(1.0) * w0
    w2, r2 = f(0), f(0)
    for a, b in zip(w0, r):
        w2 = f(w2 + a * a)
        r2 = f(r2 + b * b)
    wn, rn = np.sqrt(w2), np.sqrt(r2)
    scale = f(f(wn / rn) / rn)
    want = (w0 - f(f(1e-3) * scale) * r).astype(np.float32)
    assert np.array_equal(outs[0], want)
