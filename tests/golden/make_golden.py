"""Generates tests/golden/golden_v1.npz.

Run it where the reference tree is present and `make -C oracle ref` has
compiled the reference's own host checkers into oracle/_ref (its sources:
examples/test-sgd.cu, examples/test-adam.cu and
nccl-overlap/samples/multi-process-adam-scattered.cpp):

    python tests/golden/make_golden.py

For seeded inputs it stores
  * the inputs (per-rank gradients, initial weights),
  * the weights / moments the CPU oracle computes from them, kept ONLY IF the
    reference's checker accepted them when this script ran, and
  * for the bias-corrected Adam and LAMB of the second NCCL fork, the first and
    second moments the REFERENCE's checker computed itself (it carries them in
    the arrays it is given), epoch by epoch.
tests/test_golden.py then needs neither the reference tree nor oracle/_ref: it
recomputes the oracle and compares bit for bit with what is stored here.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as O  # noqa: E402

OUT = os.path.join(HERE, "golden_v1.npz")
N = 257          # ragged: not a multiple of 4 or 8
EPOCHS = 4


def grads(R, n, seed, epoch, scale=1e-3):
    return [(np.random.default_rng((seed, r, epoch)).standard_normal(n) * scale).astype(np.float32)
            for r in range(R)]


def main():
    assert O.ref_available(), "build oracle/_ref first (make -C oracle ref)"
    out = {}

    # SGD, the DSL program's check (examples/test-sgd.cu:17-23)
    for R in (2, 3):
        g = [np.random.default_rng((11, r)).uniform(-1, 1, N).astype(np.float32) for r in range(R)]
        w0 = (np.random.default_rng(12).standard_normal(N) * 0.02).astype(np.float32)
        w = w0.copy()
        O.sgd(w, O.reduce_f32(g), 0.01)
        assert O.ref_sgd_check(g, w0, 0.01, w), "reference checker rejected the oracle's SGD"
        out[f"sgd_R{R}_g"] = np.stack(g)
        out[f"sgd_R{R}_w0"] = w0
        out[f"sgd_R{R}_w"] = w

    # Adam as the DSL program writes it (examples/test-adam.cu:14-43)
    for R in (2, 3):
        g = grads(R, N, 21, 0, scale=1.0)
        w0 = (np.random.default_rng(22).standard_normal(N) * 0.02).astype(np.float32)
        m0 = (np.random.default_rng(23).standard_normal(N) * 0.1).astype(np.float32)
        v0 = np.abs(np.random.default_rng(24).standard_normal(N)).astype(np.float32)
        w, m, v = w0.copy(), m0.copy(), v0.copy()
        O.adam(w, m, v, O.reduce_f32(g), 1e-3, 0.9, 0.999, 0.0, 0, O.DSL)
        assert O.ref_adam_dsl_check(g, w0, m0, v0, 1e-3, 0.9, 0.999, w), \
            "reference checker rejected the oracle's DSL Adam"
        for k, a in (("g", np.stack(g)), ("w0", w0), ("m0", m0), ("v0", v0), ("w", w), ("m", m), ("v", v)):
            out[f"adam_dsl_R{R}_{k}"] = a

    # bias-corrected Adam and LAMB of the second fork, several epochs with carried state
    # (nccl-overlap/samples/multi-process-adam-scattered.cpp:112-136, 402-435)
    for kind in ("adam", "lamb"):
        for R in (2, 4):
            w = (np.random.default_rng(32).standard_normal(N) * 0.02).astype(np.float32)
            m, v = np.zeros(N, np.float32), np.zeros(N, np.float32)
            rm, rv = np.zeros(N, np.float32), np.zeros(N, np.float32)
            out[f"{kind}_R{R}_w0"] = w.copy()
            for e in range(EPOCHS):
                g = grads(R, N, 31, e)
                w_old = w.copy()
                gsum = O.reduce_f32(g)
                if kind == "adam":
                    O.adam(w, m, v, gsum, 1e-3, 0.9, 0.999, 1e-6, e)
                else:
                    O.lamb(w, m, v, gsum, 1e-3, 0.9, 0.999, 1e-6, 1.0, e, flags=O.LAMB_REF_QUIRK)
                # the sample ADDS stepsize * m^/(sqrt(v^)+eps) for Adam, subtracts for LAMB
                stepsize = -1e-3 if kind == "adam" else 1e-3
                assert O.ref_overlap_check(kind, g, e, w_old, w, rm, rv, 0.9, 0.999, stepsize, 1e-6), \
                    f"reference checker rejected the oracle's {kind} at epoch {e}"
                out[f"{kind}_R{R}_e{e}_g"] = np.stack(g)
                out[f"{kind}_R{R}_e{e}_w"] = w.copy()
                out[f"{kind}_R{R}_e{e}_m"] = m.copy()
                out[f"{kind}_R{R}_e{e}_v"] = v.copy()
                out[f"{kind}_R{R}_e{e}_ref_m"] = rm.copy()   # computed by the reference itself
                out[f"{kind}_R{R}_e{e}_ref_v"] = rv.copy()
    np.savez_compressed(OUT, **out)
    print(f"wrote {OUT}: {len(out)} arrays, {os.path.getsize(OUT)} bytes")


if __name__ == "__main__":
    main()
