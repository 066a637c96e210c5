"""The committed golden vectors (tests/golden/golden_v1.npz, made by
tests/golden/make_golden.py with the reference's own host checkers compiled
from the reference tree): the oracle must reproduce them bit for bit, with or
without the reference tree at hand, and the moments the REFERENCE computed
must equal the oracle's.  The GPU test runs the same inputs through the C ABI."""
import os

import numpy as np
import pytest

import oracle_lib as O

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_v1.npz"))
EPOCHS = 4


@pytest.mark.parametrize("R", [2, 3])
def test_oracle_sgd_matches_golden(R):
    g = list(G[f"sgd_R{R}_g"])
    w = G[f"sgd_R{R}_w0"].copy()
    O.sgd(w, O.reduce_f32(g), 0.01)
    assert np.array_equal(w, G[f"sgd_R{R}_w"])


@pytest.mark.parametrize("R", [2, 3])
def test_oracle_dsl_adam_matches_golden(R):
    k = f"adam_dsl_R{R}_"
    w, m, v = G[k + "w0"].copy(), G[k + "m0"].copy(), G[k + "v0"].copy()
    O.adam(w, m, v, O.reduce_f32(list(G[k + "g"])), 1e-3, 0.9, 0.999, 0.0, 0, O.DSL)
    assert np.array_equal(w, G[k + "w"]) and np.array_equal(m, G[k + "m"]) and np.array_equal(v, G[k + "v"])


@pytest.mark.parametrize("kind", ["adam", "lamb"])
@pytest.mark.parametrize("R", [2, 4])
def test_oracle_bias_corrected_matches_golden_and_reference_moments(kind, R):
    k = f"{kind}_R{R}_"
    w = G[k + "w0"].copy()
    m, v = np.zeros_like(w), np.zeros_like(w)
    for e in range(EPOCHS):
        gsum = O.reduce_f32(list(G[f"{k}e{e}_g"]))
        if kind == "adam":
            O.adam(w, m, v, gsum, 1e-3, 0.9, 0.999, 1e-6, e)
        else:
            O.lamb(w, m, v, gsum, 1e-3, 0.9, 0.999, 1e-6, 1.0, e, flags=O.LAMB_REF_QUIRK)
        assert np.array_equal(w, G[f"{k}e{e}_w"]), e
        assert np.array_equal(m, G[f"{k}e{e}_m"]) and np.array_equal(v, G[f"{k}e{e}_v"]), e
        # what the reference's own checker computed for its moments
        assert np.array_equal(m, G[f"{k}e{e}_ref_m"]) and np.array_equal(v, G[f"{k}e{e}_ref_v"]), e


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["sgd", "adam_dsl", "adam", "lamb"])
def test_cuda_path_matches_golden(kind):
    import torch

    import cases as K
    import coconet_b200 as coco

    R = 2
    n = G["sgd_R2_w0"].size
    S = (n + R - 1) // R
    comms = coco.Communicator.init_all(R, [0] * R)
    try:
        if kind == "sgd":
            w = [torch.from_numpy(G["sgd_R2_w0"].copy()).cuda() for _ in range(R)]
            g = [torch.from_numpy(G["sgd_R2_g"][r].copy()).cuda() for r in range(R)]
            with coco.group():
                for r, c in enumerate(comms):
                    c.fused_sgd(g[r], w[r], 0.01)
            torch.cuda.synchronize()
            for r in range(R):
                assert np.array_equal(w[r].cpu().numpy(), G["sgd_R2_w"])   # fixed sum order: exact
            return
        if kind == "adam_dsl":
            k = "adam_dsl_R2_"
            w = [torch.from_numpy(G[k + "w0"].copy()).cuda() for _ in range(R)]
            g = [torch.from_numpy(G[k + "g"][r].copy()).cuda() for r in range(R)]
            m, v = [], []
            for r in range(R):
                lo, hi = K.slice_bounds(n, R, r)
                ms, vs = np.zeros(S, np.float32), np.zeros(S, np.float32)
                ms[: hi - lo], vs[: hi - lo] = G[k + "m0"][lo:hi], G[k + "v0"][lo:hi]
                m.append(torch.from_numpy(ms).cuda())
                v.append(torch.from_numpy(vs).cuda())
            with coco.group():
                for r, c in enumerate(comms):
                    c.fused_adam(g[r], w[r], m[r], v[r], 1e-3, 0.9, 0.999, 0.0, 0,
                                 variant=coco.VARIANT_DSL)
            torch.cuda.synchronize()
            for r in range(R):
                lo, hi = K.slice_bounds(n, R, r)
                assert np.array_equal(m[r].cpu().numpy()[: hi - lo], G[k + "m"][lo:hi])
                assert np.array_equal(v[r].cpu().numpy()[: hi - lo], G[k + "v"][lo:hi])
                K.assert_close(w[r].cpu().numpy(), G[k + "w"], 1e-5, "w")
            return
        k = f"{kind}_R2_"
        w = [torch.from_numpy(G[k + "w0"].copy()).cuda() for _ in range(R)]
        m = [torch.zeros(S, device="cuda") for _ in range(R)]
        v = [torch.zeros(S, device="cuda") for _ in range(R)]
        for e in range(EPOCHS):
            g = [torch.from_numpy(G[f"{k}e{e}_g"][r].copy()).cuda() for r in range(R)]
            with coco.group():
                for r, c in enumerate(comms):
                    if kind == "adam":
                        c.fused_adam(g[r], w[r], m[r], v[r], 1e-3, 0.9, 0.999, 1e-6, e)
                    else:
                        c.fused_lamb(g[r], w[r], m[r], v[r], 1e-3, 0.9, 0.999, 1e-6, 1.0, e,
                                     flags=coco.LAMB_REF_QUIRK)
            torch.cuda.synchronize()
            for r in range(R):
                lo, hi = K.slice_bounds(n, R, r)
                assert np.array_equal(m[r].cpu().numpy()[: hi - lo], G[f"{k}e{e}_ref_m"][lo:hi]), e
                assert np.array_equal(v[r].cpu().numpy()[: hi - lo], G[f"{k}e{e}_ref_v"][lo:hi]), e
                K.assert_close(w[r].cpu().numpy(), G[f"{k}e{e}_w"], 1e-5, f"w at epoch {e}")
            # continue from the golden weights, so that a last-bit difference in one
            # epoch is not carried into the next comparison
            for r in range(R):
                w[r].copy_(torch.from_numpy(G[f"{k}e{e}_w"]))
    finally:
        for c in comms:
            c.destroy()
