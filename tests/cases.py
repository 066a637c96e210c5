"""Seeded inputs and oracle evaluation shared by the GPU parity tests and the
benchmark checker.  numpy + the CPU oracle only (test infrastructure)."""
import numpy as np

import oracle_lib as O

SGD, ADAM, LAMB = "sgd", "adam", "lamb"

HYPER = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-6, weight_decay=0.01)


def make_grads(R, n, seed, step, dtype=np.float32, dist="normal", loss_scale=1.0):
    out = []
    for r in range(R):
        rng = np.random.default_rng((seed, r, step))
        if dist == "uniform":
            x = rng.uniform(-1.0, 1.0, n)
        else:
            x = rng.standard_normal(n) * 1e-3
        out.append((x * loss_scale).astype(dtype))
    return out


def make_weights(n, seed):
    return (np.random.default_rng((seed, 12345)).standard_normal(n) * 0.02).astype(np.float32)


def slice_bounds(n, R, r):
    S = (n + R - 1) // R
    lo = min(n, r * S)
    return lo, min(n, lo + S)


class OracleState:
    """Full-tensor oracle state advanced one step at a time."""

    def __init__(self, opt, n, seed, lp=False, variant=O.OVERLAP, lamb_flags=0, hyper=None):
        self.opt, self.n, self.variant, self.lamb_flags = opt, n, variant, lamb_flags
        self.h = dict(HYPER)
        if hyper:
            self.h.update(hyper)
        self.w = make_weights(n, seed)
        self.m = np.zeros(n, np.float32)
        self.v = np.zeros(n, np.float32)
        self.w_lp = np.zeros(n, np.float16) if lp else None
        self.norms = None

    def step(self, grads, step, inv_scale=1.0):
        h = self.h
        if grads[0].dtype == np.float16:
            gsum = O.reduce_f16(grads, inv_scale)
        else:
            gsum = O.reduce_f32(grads)
            if inv_scale != 1.0:
                gsum = (gsum * np.float32(inv_scale)).astype(np.float32)
        if self.opt == SGD:
            O.sgd(self.w, gsum, h["lr"])
            if self.w_lp is not None:
                self.w_lp[:] = self.w.astype(np.float16)
        elif self.opt == ADAM:
            O.adam(self.w, self.m, self.v, gsum, h["lr"], h["beta1"], h["beta2"], h["eps"], step,
                   self.variant, w_lp=self.w_lp)
        else:
            self.norms = O.lamb(self.w, self.m, self.v, gsum, h["lr"], h["beta1"], h["beta2"],
                                h["eps"], h["weight_decay"], step, self.variant, self.lamb_flags,
                                w_lp=self.w_lp)


def assert_close(actual, expect, rtol, what):
    """|a-b| <= rtol*max(|a|,|b|) + atol, atol = rtol * 1e-3 (weights are O(1e-2))."""
    a = np.asarray(actual, np.float64)
    b = np.asarray(expect, np.float64)
    # e.g. 0/0 in the DSL's LAMB when a gradient is 0, x/0 where a formulation without
    # epsilon meets v = 0: NaN against NaN and equal infinities agree
    same = (np.isnan(a) & np.isnan(b)) | (a == b)
    with np.errstate(invalid="ignore"):
        err = np.where(same, 0.0, np.abs(a - b))
        tol = np.where(same, 0.0, rtol * np.maximum(np.abs(a), np.abs(b)) + rtol * 1e-3)
        bad = (~(err <= tol) | np.isinf(a) | np.isinf(b)) & ~same
    if bad.any():
        i = int(np.flatnonzero(bad)[0])
        raise AssertionError(f"{what}: {int(bad.sum())} of {a.size} outside rtol {rtol}; "
                             f"worst at [{i}]: got {a[i]!r}, want {b[i]!r}")


def assert_close_most(actual, expect, rtol, what, frac=1e-3, rtol_all=2e-3):
    """For sums whose order is not fixed (in-switch reduction): all but a
    fraction `frac` of the elements within rtol, every element within
    rtol_all.  The outliers are elements whose gradient sum nearly cancels, on
    which Adam's m/sqrt(v) amplifies the last-bit difference of the sum."""
    assert_close(actual, expect, rtol_all, what + " (all elements)")
    a = np.asarray(actual, np.float64)
    b = np.asarray(expect, np.float64)
    tol = rtol * np.maximum(np.abs(a), np.abs(b)) + rtol * 1e-3
    bad = int((np.abs(a - b) > tol).sum())
    assert bad <= frac * a.size, f"{what}: {bad} of {a.size} outside rtol {rtol}"
