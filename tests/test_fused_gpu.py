"""Parity of the CUDA fused step with the CPU oracle, through the C ABI.

These run on ONE GPU: the R ranks of a communicator are virtual ranks of a
single cooperative launch (cocoCommInitAll with one device listed R times), so
the same kernel code, flags and barriers run as on R GPUs.

Tolerances (stated by the task): fp32 paths rel 1e-5; fp16-gradient paths rel
2e-3 (measured far tighter; the assertion uses 1e-5 on fp32 state and exact
equality on the fp16 copy of an fp32-identical weight).  m and v must match the
oracle bit for bit.
"""
import numpy as np
import pytest
import torch

import cases as K
import oracle_lib as O

pytestmark = pytest.mark.gpu

import coconet_b200 as coco  # noqa: E402

RTOL_FP32 = 1e-5


def _dev(a):
    return torch.from_numpy(a).cuda()


class Ranks:
    """Device state of R virtual ranks on cuda:0."""

    def __init__(self, opt, R, n, seed, lp_dtype=None):
        self.opt, self.R, self.n = opt, R, n
        self.comms = coco.Communicator.init_all(R, [0] * R)
        w0 = K.make_weights(n, seed)
        self.w = [_dev(w0.copy()) for _ in range(R)]
        self.lp = [torch.zeros(n, dtype=lp_dtype, device="cuda") for _ in range(R)] if lp_dtype else None
        S = (n + R - 1) // R
        self.m = [torch.zeros(S, device="cuda") for _ in range(R)]
        self.v = [torch.zeros(S, device="cuda") for _ in range(R)]

    def step(self, grads, step, grad_scale=1.0, variant=coco.VARIANT_OVERLAP, flags=0, hyper=None):
        h = dict(K.HYPER)
        if hyper:
            h.update(hyper)
        g = [_dev(x) for x in grads]
        with coco.group():
            for r, c in enumerate(self.comms):
                lp = self.lp[r] if self.lp else None
                if self.opt == K.SGD:
                    c.fused_sgd(g[r], self.w[r], h["lr"], w_lp=lp, grad_scale=grad_scale)
                elif self.opt == K.ADAM:
                    c.fused_adam(g[r], self.w[r], self.m[r], self.v[r], h["lr"], h["beta1"],
                                 h["beta2"], h["eps"], step, w_lp=lp, grad_scale=grad_scale,
                                 variant=variant)
                else:
                    c.fused_lamb(g[r], self.w[r], self.m[r], self.v[r], h["lr"], h["beta1"],
                                 h["beta2"], h["eps"], h["weight_decay"], step, w_lp=lp,
                                 grad_scale=grad_scale, variant=variant, flags=flags)
        torch.cuda.synchronize()
        for c in self.comms:
            st = c.status()
            assert st["code"] == 0, st
        return g

    def close(self):
        for c in self.comms:
            c.destroy()


def _check_against(ranks, ora, rtol=RTOL_FP32, exact_state=True, exact_w=False):
    R, n = ranks.R, ranks.n
    for r in range(R):
        lo, hi = K.slice_bounds(n, R, r)
        w = ranks.w[r].cpu().numpy()
        if ranks.lp is None:
            K.assert_close(w, ora.w, rtol, f"w on rank {r}")
            if exact_w:
                assert np.array_equal(w, ora.w), f"w on rank {r} not bit-exact"
            assert np.array_equal(w, ranks.w[0].cpu().numpy()), "replicas differ"
        else:
            K.assert_close(w[lo:hi], ora.w[lo:hi], rtol, f"master w slice on rank {r}")
            if exact_w:
                assert np.array_equal(w[lo:hi], ora.w[lo:hi]), f"master w on rank {r} not bit-exact"
                assert np.array_equal(ranks.lp[r].cpu().numpy().view(np.uint16),
                                      ora.w_lp.view(np.uint16)), "w_lp not bit-exact"
            lp = ranks.lp[r].float().cpu().numpy()
            # half(w') of weights that agree to 1e-5 may differ by one fp16 ulp
            K.assert_close(lp, ora.w_lp.astype(np.float32), 1e-3, f"w_lp on rank {r}")
            assert torch.equal(ranks.lp[r].view(torch.int16), ranks.lp[0].view(torch.int16)), \
                "low-precision replicas differ"
            own = ranks.w[r][lo:hi].to(ranks.lp[r].dtype)
            got = ranks.lp[r][lo:hi]
            same = (got == own) | (got.isnan() & own.isnan())
            if not bool(same.all()):
                bad = torch.nonzero(~same).flatten()
                k = int(bad[0])
                raise AssertionError(
                    f"w_lp is not the rounding of the master on rank {r}: {bad.numel()} elements, "
                    f"first at slice index {k}: lp={float(ranks.lp[r][lo + k])!r} "
                    f"master={float(ranks.w[r][lo + k])!r} oracle={float(ora.w[lo + k])!r}")
        if ranks.opt != K.SGD:
            m = ranks.m[r].cpu().numpy()[: hi - lo]
            v = ranks.v[r].cpu().numpy()[: hi - lo]
            if exact_state:
                assert np.array_equal(m, ora.m[lo:hi]), f"m on rank {r} not bit-exact"
                assert np.array_equal(v, ora.v[lo:hi]), f"v on rank {r} not bit-exact"
            else:
                K.assert_close(m, ora.m[lo:hi], rtol, f"m on rank {r}")
                K.assert_close(v, ora.v[lo:hi], rtol, f"v on rank {r}")


SIZES = [1, 5, 257, 4099, 65536, (1 << 20) + 3]


@pytest.mark.parametrize("R", [1, 2, 3, 8])
@pytest.mark.parametrize("n", SIZES)
def test_sgd_fp32(R, n):
    ranks = Ranks(K.SGD, R, n, seed=1)
    ora = K.OracleState(K.SGD, n, seed=1, hyper=dict(lr=0.01))
    try:
        for step in range(2):
            grads = K.make_grads(R, n, 1, step, dist="uniform")
            ranks.step(grads, step, hyper=dict(lr=0.01))
            ora.step(grads, step)
            _check_against(ranks, ora)
        # the reduction order is fixed, so SGD is bit-exact
        assert np.array_equal(ranks.w[0].cpu().numpy(), ora.w)
    finally:
        ranks.close()


def test_sgd_config0_reference_checker():
    # the repo's sgd-fuse-rs-c-ag program: N = 2^20, world 2, lr = 0.01,
    # checked by the oracle and, when built, by the reference's own mpiRef.
    R, n = 2, 1 << 20
    ranks = Ranks(K.SGD, R, n, seed=2)
    try:
        w0 = K.make_weights(n, 2)
        grads = K.make_grads(R, n, 2, 0, dist="uniform")
        ranks.step(grads, 0, hyper=dict(lr=0.01))
        w = ranks.w[1].cpu().numpy()
        ref = w0.copy()
        O.sgd(ref, O.reduce_f32(grads), 0.01)
        assert np.array_equal(w, ref)
        if O.ref_available():
            assert O.ref_sgd_check(grads, w0, 0.01, w)
    finally:
        ranks.close()


@pytest.mark.parametrize("R", [1, 2, 4, 8])
@pytest.mark.parametrize("n", [7, 4099, 65536, 1 << 20, (1 << 20) + 3])
def test_adam_fp32(R, n):
    ranks = Ranks(K.ADAM, R, n, seed=3)
    ora = K.OracleState(K.ADAM, n, seed=3)
    try:
        for step in range(3):
            grads = K.make_grads(R, n, 3, step)
            ranks.step(grads, step)
            ora.step(grads, step)
            # every operation is individually rounded in the oracle's order
            _check_against(ranks, ora, exact_w=True)
    finally:
        ranks.close()


def test_adam_fp32_ten_steps_reference_checker():
    # 10 consecutive steps with fresh gradients; the reference's own host
    # checker (nccl-overlap sample) must accept every step.
    R, n = 8, 50000
    ranks = Ranks(K.ADAM, R, n, seed=4)
    ora = K.OracleState(K.ADAM, n, seed=4)
    rm, rv = np.zeros(n, np.float32), np.zeros(n, np.float32)
    try:
        for step in range(10):
            grads = K.make_grads(R, n, 4, step)
            w_old = ranks.w[0].cpu().numpy().copy()
            ranks.step(grads, step)
            ora.step(grads, step)
            _check_against(ranks, ora)
            if O.ref_available():
                h = K.HYPER
                assert O.ref_overlap_check("adam", grads, step, w_old, ranks.w[0].cpu().numpy(),
                                           rm, rv, h["beta1"], h["beta2"], -h["lr"], h["eps"])
    finally:
        ranks.close()


@pytest.mark.parametrize("R", [1, 2, 8])
@pytest.mark.parametrize("n", [9, 4099, 1 << 20, (1 << 20) + 8])
@pytest.mark.parametrize("lp", [torch.float16, torch.bfloat16])
def test_adam_mixed_precision(R, n, lp):
    # fp16 gradients scaled by 1024, unscaled in the kernel; fp32 master slice;
    # fp16/bf16 copy gathered to every rank.
    ranks = Ranks(K.ADAM, R, n, seed=5, lp_dtype=lp)
    ora = K.OracleState(K.ADAM, n, seed=5, lp=True)
    try:
        for step in range(3):
            grads = K.make_grads(R, n, 5, step, dtype=np.float16, loss_scale=1024.0)
            ranks.step(grads, step, grad_scale=1.0 / 1024.0)
            ora.step(grads, step, inv_scale=1.0 / 1024.0)
            if lp == torch.bfloat16:
                ora.w_lp = None
                saved = ranks.lp
                # compare the bf16 copy against the rounding of the oracle's fp32 weights
                want = torch.from_numpy(ora.w).to(torch.bfloat16).float().numpy()
                for r in range(R):
                    K.assert_close(saved[r].float().cpu().numpy(), want, 1e-2, "bf16 copy")
                ranks.lp = None
                # master slices + moments
                for r in range(R):
                    lo, hi = K.slice_bounds(n, R, r)
                    K.assert_close(ranks.w[r].cpu().numpy()[lo:hi], ora.w[lo:hi], RTOL_FP32, "w")
                    assert np.array_equal(ranks.m[r].cpu().numpy()[: hi - lo], ora.m[lo:hi])
                ranks.lp = saved
                ora.w_lp = np.zeros(n, np.float16)
            else:
                _check_against(ranks, ora, exact_w=True)
    finally:
        ranks.close()


@pytest.mark.parametrize("gdt", [np.float32, np.float16])
def test_adam_bf16_and_f16_grads_fp32_gather(gdt):
    # 16-bit gradients with the fp32 weights themselves gathered (no copy)
    R, n = 4, 10007
    ranks = Ranks(K.ADAM, R, n, seed=6)
    ora = K.OracleState(K.ADAM, n, seed=6)
    try:
        grads = K.make_grads(R, n, 6, 0, dtype=gdt, loss_scale=1.0)
        ranks.step(grads, 0)
        ora.step(grads, 0)
        _check_against(ranks, ora)
    finally:
        ranks.close()


def test_adam_bf16_grads():
    R, n = 4, 4100
    ranks = Ranks(K.ADAM, R, n, seed=7)
    ora = K.OracleState(K.ADAM, n, seed=7)
    try:
        g32 = K.make_grads(R, n, 7, 0)
        gb = [torch.from_numpy(x).to(torch.bfloat16) for x in g32]
        # oracle on the bf16-rounded values (exactly representable in fp32)
        ora.step([x.float().numpy() for x in gb], 0)
        g = [x.cuda() for x in gb]
        with coco.group():
            for r, c in enumerate(ranks.comms):
                h = K.HYPER
                c.fused_adam(g[r], ranks.w[r], ranks.m[r], ranks.v[r], h["lr"], h["beta1"],
                             h["beta2"], h["eps"], 0)
        torch.cuda.synchronize()
        _check_against(ranks, ora)
    finally:
        ranks.close()


@pytest.mark.parametrize("R", [1, 2, 8])
def test_adam_reference_known_answers(R):
    # examples/test-adam.cu:73-88: g = 1, w = m = v = 0, lr = 1, beta = 0.5.
    n = 1000
    hyper = dict(lr=1.0, beta1=0.5, beta2=0.5, eps=0.0)
    ones16 = [np.ones(n, np.float16) for _ in range(R)]
    ones32 = [np.ones(n, np.float32) for _ in range(R)]
    # forked-NCCL formulation -> -1 for any R; fp16 copy too
    ranks = Ranks(K.ADAM, R, n, seed=0, lp_dtype=torch.float16)
    try:
        for r in range(R):
            ranks.w[r].zero_()
        ranks.step(ones16, 0, variant=coco.VARIANT_NCCL, hyper=hyper)
        for r in range(R):
            lo, hi = K.slice_bounds(n, R, r)
            assert torch.all(ranks.w[r][lo:hi] == -1.0)
            assert torch.all(ranks.lp[r] == -1.0)
            assert torch.all(ranks.m[r][: hi - lo] == R / 2) and torch.all(ranks.v[r][: hi - lo] == R * R / 2)
    finally:
        ranks.close()
    # DSL formulation -> -1/R
    ranks = Ranks(K.ADAM, R, n, seed=0)
    try:
        for r in range(R):
            ranks.w[r].zero_()
        ranks.step(ones32, 0, variant=coco.VARIANT_DSL, hyper=hyper)
        np.testing.assert_allclose(ranks.w[0].cpu().numpy(), -1.0 / R, rtol=1e-7)
    finally:
        ranks.close()


def test_adam_nccl_variant_matches_oracle_ring_sum():
    # fp16 ring-order sums differ from fp32 sums; the oracle reproduces the ring.
    R, n = 4, 4096
    ranks = Ranks(K.ADAM, R, n, seed=8, lp_dtype=torch.float16)
    try:
        grads = K.make_grads(R, n, 8, 0, dtype=np.float16, loss_scale=512.0)
        w0 = K.make_weights(n, 8)
        ranks.step(grads, 0, variant=coco.VARIANT_NCCL, hyper=dict(lr=1e-3, beta1=0.9, beta2=0.999))
        for r in range(R):
            lo, hi = K.slice_bounds(n, R, r)
            gh = O.reduce_f16_ring([x[lo:hi].copy() for x in grads], owner=r)
            w, m, v = w0[lo:hi].copy(), np.zeros(hi - lo, np.float32), np.zeros(hi - lo, np.float32)
            wl = np.zeros(hi - lo, np.float16)
            O.adam(w, m, v, None, 1e-3, 0.9, 0.999, 0.0, 0, O.NCCL, w_lp=wl, gsum_h=gh)
            assert np.array_equal(ranks.m[r].cpu().numpy()[: hi - lo], m)
            assert np.array_equal(ranks.v[r].cpu().numpy()[: hi - lo], v)
            K.assert_close(ranks.w[r].cpu().numpy()[lo:hi], w, RTOL_FP32, "w")
    finally:
        ranks.close()


@pytest.mark.parametrize("R", [1, 2, 8])
def test_lamb_nccl_variant_known_answer(R):
    # forked-NCCL LAMB functors on the constants of the reference's frozen tests
    # (g = 1 per rank, w = m = v = 0, beta = 0.5, lr = 1): S0 = R, v^ = R^2,
    # m^ = R, r = 1 everywhere, ||w|| = 0 so scale = 1/||r|| = 1/sqrt(n), and
    # w' = -1/sqrt(n) for any R (reduce_kernel.h:391-452, common_kernel.h:2699)
    n = 4096
    ranks = Ranks(K.LAMB, R, n, seed=0, lp_dtype=torch.float16)
    try:
        for r in range(R):
            ranks.w[r].zero_()
        ones16 = [np.ones(n, np.float16) for _ in range(R)]
        ranks.step(ones16, 0, variant=coco.VARIANT_NCCL, hyper=dict(lr=1.0, beta1=0.5, beta2=0.5))
        for r in range(R):
            lo, hi = K.slice_bounds(n, R, r)
            assert torch.all(ranks.w[r][lo:hi] == -1.0 / 64.0)
            assert torch.all(ranks.lp[r] == -1.0 / 64.0)
            assert torch.all(ranks.m[r][: hi - lo] == R / 2) and torch.all(ranks.v[r][: hi - lo] == R * R / 2)
    finally:
        ranks.close()


@pytest.mark.parametrize("R,n", [(1, 5000), (4, 1 << 16), (8, (1 << 18) + 24)])
def test_lamb_nccl_variant_matches_oracle(R, n):
    # fp16 ring sum per slice owner, beta1 for m, decay factor 1.0 whatever the
    # caller passes, float norms, scale = (||w||/||r||)/||r||; two steps
    ranks = Ranks(K.LAMB, R, n, seed=14, lp_dtype=torch.float16)
    w = K.make_weights(n, 14)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    wl = np.zeros(n, np.float16)
    try:
        for step in range(2):
            # gradients in [0.5, 1.5): this formulation has no epsilon and squares the sum in
            # half precision, so a sum that cancels or is below 2.4e-4 gives v = 0 and a
            # non-finite r, which would make the check vacuous
            grads = [(np.abs(x) + 0.5).astype(np.float16)
                     for x in K.make_grads(R, n, 14, step, dtype=np.float32, dist="uniform")]
            ranks.step(grads, step, variant=coco.VARIANT_NCCL,
                       hyper=dict(lr=1e-3, beta1=0.9, beta2=0.999, weight_decay=0.01))
            gsum = np.empty(n, np.float32)
            for r in range(R):
                lo, hi = K.slice_bounds(n, R, r)
                gsum[lo:hi] = O.reduce_f16_ring([x[lo:hi].copy() for x in grads], owner=r).astype(np.float32)
            norms = O.lamb(w, m, v, gsum, 1e-3, 0.9, 0.999, 0.0, 0.01, step, O.NCCL, w_lp=wl)
            for r in range(R):
                lo, hi = K.slice_bounds(n, R, r)
                assert np.array_equal(ranks.m[r].cpu().numpy()[: hi - lo], m[lo:hi])
                assert np.array_equal(ranks.v[r].cpu().numpy()[: hi - lo], v[lo:hi])
                K.assert_close(ranks.w[r].cpu().numpy()[lo:hi], w[lo:hi], RTOL_FP32, f"w step {step}")
                K.assert_close(ranks.lp[r].float().cpu().numpy(), wl.astype(np.float32), 1e-3, "w_lp")
            wn, rn = ranks.comms[0].last_lamb_norms()
            assert np.isfinite(norms).all() and np.isfinite(w).all()
            # the oracle adds the squares in fp32 in element order (the fork: fp32 atomics in
            # no fixed order), the kernel in double: they agree to fp32 summation error
            np.testing.assert_allclose([wn, rn], norms, rtol=2e-4)
    finally:
        ranks.close()


@pytest.mark.parametrize("R", [1, 2, 8])
@pytest.mark.parametrize("n", [11, 4099, 1 << 20, (1 << 20) + 3])
def test_lamb_fp32(R, n):
    ranks = Ranks(K.LAMB, R, n, seed=9)
    ora = K.OracleState(K.LAMB, n, seed=9)
    try:
        for step in range(3):
            grads = K.make_grads(R, n, 9, step)
            ranks.step(grads, step)
            ora.step(grads, step)
            _check_against(ranks, ora)
            for c in ranks.comms:
                wn, rn = c.last_lamb_norms()
                np.testing.assert_allclose([wn, rn], ora.norms, rtol=1e-9)
    finally:
        ranks.close()


def test_lamb_reference_checker_quirk():
    # The reference sample's LAMB (decay 1.0, scale = trust/||r|| on mean-square
    # norms) replayed through its own host checker.
    R, n = 4, 20000
    ranks = Ranks(K.LAMB, R, n, seed=10)
    ora = K.OracleState(K.LAMB, n, seed=10, lamb_flags=O.LAMB_REF_QUIRK, hyper=dict(weight_decay=1.0))
    rm, rv = np.zeros(n, np.float32), np.zeros(n, np.float32)
    try:
        for step in range(5):
            grads = K.make_grads(R, n, 10, step)
            w_old = ranks.w[0].cpu().numpy().copy()
            ranks.step(grads, step, flags=coco.LAMB_REF_QUIRK, hyper=dict(weight_decay=1.0))
            ora.step(grads, step)
            _check_against(ranks, ora)
            if O.ref_available():
                h = K.HYPER
                assert O.ref_overlap_check("lamb", grads, step, w_old, ranks.w[0].cpu().numpy(),
                                           rm, rv, h["beta1"], h["beta2"], h["lr"], h["eps"])
    finally:
        ranks.close()


def test_lamb_dsl_variant_and_mixed():
    R, n = 2, 30001
    ranks = Ranks(K.LAMB, R, n, seed=11, lp_dtype=torch.float16)
    ora = K.OracleState(K.LAMB, n, seed=11, lp=True, variant=O.DSL)
    try:
        for step in range(2):
            grads = K.make_grads(R, n, 11, step, dtype=np.float16, loss_scale=1024.0)
            ranks.step(grads, step, grad_scale=1 / 1024.0, variant=coco.VARIANT_DSL)
            ora.step(grads, step, inv_scale=1 / 1024.0)
            _check_against(ranks, ora)
    finally:
        ranks.close()


@pytest.mark.parametrize("opt,R,n", [(K.ADAM, 2, 1 << 20), (K.ADAM, 8, 1 << 20), (K.LAMB, 4, 1 << 20),
                                     (K.SGD, 2, (1 << 18) + 5), (K.ADAM, 1, (1 << 20) + 3),
                                     (K.ADAM, 3, (1 << 19) + 264), (K.LAMB, 8, (1 << 20) + 8),
                                     (K.SGD, 8, 1 << 16), (K.ADAM, 4, 300)])
def test_warp_ring_path(monkeypatch, opt, R, n):
    # the shared-memory staging path (COCO_PIPELINE=1: per-warp rings filled by bulk
    # copies) must give the same bits as the register-staged path: whole tiles
    # through the rings, ragged ends and slices shorter than a tile through the
    # scalar loop
    monkeypatch.setenv("COCO_PIPELINE", "1")
    ranks = Ranks(opt, R, n, seed=21, lp_dtype=torch.float16 if opt == K.ADAM else None)
    ora = K.OracleState(opt, n, seed=21, lp=opt == K.ADAM)
    try:
        for step in range(2):
            if opt == K.ADAM:
                grads = K.make_grads(R, n, 21, step, dtype=np.float16, loss_scale=1024.0)
                ranks.step(grads, step, grad_scale=1 / 1024.0)
                ora.step(grads, step, inv_scale=1 / 1024.0)
            else:
                grads = K.make_grads(R, n, 21, step)
                ranks.step(grads, step)
                ora.step(grads, step)
            _check_against(ranks, ora, exact_w=opt != K.LAMB)
    finally:
        ranks.close()


@pytest.mark.parametrize("stages", ["1", "2", "4"])
def test_warp_ring_depths_and_block_sizes(monkeypatch, stages):
    monkeypatch.setenv("COCO_PIPELINE", "1")
    monkeypatch.setenv("COCO_RING_STAGES", stages)
    monkeypatch.setenv("COCO_THREADS", "256" if stages == "2" else "512")
    R, n = 2, (1 << 21) + 40
    ranks = Ranks(K.ADAM, R, n, seed=23)          # fp32 gradients, fp32 weights gathered
    ora = K.OracleState(K.ADAM, n, seed=23)
    try:
        for step in range(3):
            grads = K.make_grads(R, n, 23, step)
            ranks.step(grads, step)
            ora.step(grads, step)
            _check_against(ranks, ora, exact_w=True)
    finally:
        ranks.close()


def test_warp_ring_path_forked_nccl_variant(monkeypatch):
    # the fp16 ring-order sum (owner + 1 first) read out of the staged tiles
    monkeypatch.setenv("COCO_PIPELINE", "1")
    R, n = 4, 1 << 16
    ranks = Ranks(K.ADAM, R, n, seed=8, lp_dtype=torch.float16)
    try:
        grads = K.make_grads(R, n, 8, 0, dtype=np.float16, loss_scale=512.0)
        w0 = K.make_weights(n, 8)
        ranks.step(grads, 0, variant=coco.VARIANT_NCCL, hyper=dict(lr=1e-3, beta1=0.9, beta2=0.999))
        for r in range(R):
            lo, hi = K.slice_bounds(n, R, r)
            gh = O.reduce_f16_ring([x[lo:hi].copy() for x in grads], owner=r)
            w, m, v = w0[lo:hi].copy(), np.zeros(hi - lo, np.float32), np.zeros(hi - lo, np.float32)
            wl = np.zeros(hi - lo, np.float16)
            O.adam(w, m, v, None, 1e-3, 0.9, 0.999, 0.0, 0, O.NCCL, w_lp=wl, gsum_h=gh)
            assert np.array_equal(ranks.m[r].cpu().numpy()[: hi - lo], m)
            assert np.array_equal(ranks.v[r].cpu().numpy()[: hi - lo], v)
            K.assert_close(ranks.w[r].cpu().numpy()[lo:hi], w, RTOL_FP32, "w")
    finally:
        ranks.close()


def test_unaligned_views_take_the_scalar_path():
    # pointers that are not 16-byte aligned (views at odd offsets)
    R, n = 2, 5001
    comms = coco.Communicator.init_all(R, [0] * R)
    try:
        w0 = K.make_weights(n, 12)
        grads = K.make_grads(R, n, 12, 0)
        S = (n + R - 1) // R
        gbuf = [torch.zeros(n + 1, device="cuda") for _ in range(R)]
        wbuf = [torch.zeros(n + 3, device="cuda") for _ in range(R)]
        g = [b[1:] for b in gbuf]
        w = [b[3:] for b in wbuf]
        m = [torch.zeros(S + 1, device="cuda")[1:] for _ in range(R)]
        v = [torch.zeros(S, device="cuda") for _ in range(R)]
        for r in range(R):
            g[r].copy_(torch.from_numpy(grads[r]))
            w[r].copy_(torch.from_numpy(w0))
        h = K.HYPER
        with coco.group():
            for r, c in enumerate(comms):
                c.fused_adam(g[r], w[r], m[r], v[r], h["lr"], h["beta1"], h["beta2"], h["eps"], 0)
        torch.cuda.synchronize()
        ora = K.OracleState(K.ADAM, n, seed=12)
        ora.step(grads, 0)
        for r in range(R):
            K.assert_close(w[r].cpu().numpy(), ora.w, RTOL_FP32, "w")
            lo, hi = K.slice_bounds(n, R, r)
            assert np.array_equal(m[r].cpu().numpy()[: hi - lo], ora.m[lo:hi])
    finally:
        for c in comms:
            c.destroy()


def test_fused_equals_single_rank_update_on_summed_gradient_full_size():
    # Size-independent property at the benchmark's full size (N = 334e6 mixed
    # precision would need ~6 GB per rank; two ranks of it fit easily): the
    # R-rank fused step equals the one-rank step on the pre-summed gradient,
    # bit for bit, because the reduction order is fixed.
    R, n = 2, 334_000_000 // 8  # one slice of the 334 M-element workload at eight ranks
    gen = torch.Generator(device="cuda").manual_seed(13)
    g = [(torch.randn(n, device="cuda", generator=gen) * 1e-3) for _ in range(R)]
    w0 = torch.randn(n, device="cuda", generator=gen) * 0.02
    comms = coco.Communicator.init_all(R, [0] * R)
    one = coco.Communicator.init_all(1, [0])[0]
    try:
        S = (n + R - 1) // R
        w = [w0.clone() for _ in range(R)]
        m = [torch.zeros(S, device="cuda") for _ in range(R)]
        v = [torch.zeros(S, device="cuda") for _ in range(R)]
        h = K.HYPER
        with coco.group():
            for r, c in enumerate(comms):
                c.fused_adam(g[r], w[r], m[r], v[r], h["lr"], h["beta1"], h["beta2"], h["eps"], 0)
        gs = g[0] + g[1]
        w1, m1, v1 = w0.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        one.fused_adam(gs, w1, m1, v1, h["lr"], h["beta1"], h["beta2"], h["eps"], 0)
        torch.cuda.synchronize()
        assert torch.equal(w[0], w1) and torch.equal(w[1], w1)
        assert torch.equal(torch.cat([m[0], m[1]])[:n], m1)
        assert torch.equal(torch.cat([v[0], v[1]])[:n], v1)
    finally:
        for c in comms + [one]:
            c.destroy()


def test_host_side_usage_errors():
    comms = coco.Communicator.init_all(2, [0, 0])
    try:
        g = torch.zeros(16, device="cuda")
        w = torch.zeros(16, device="cuda")
        # only one of two ranks called before the group closed
        with pytest.raises(coco.CocoError) as e:
            with coco.group():
                comms[0].fused_sgd(g, w, 0.1)
        assert e.value.code == 2
        # missing moments
        with pytest.raises(coco.CocoError):
            coco.lib().cocoFusedAdam  # symbol exists
            comms[0].fused_adam(g, w, None, None, 1e-3, 0.9, 0.999, 1e-6, 0)
    finally:
        for c in comms:
            c.destroy()


# ---- edge cases: empty, tiny and very large inputs ---------------------------------

@pytest.mark.parametrize("R", [1, 2, 8])
def test_empty_and_tiny_counts(R):
    # count 0: nothing is launched; count < R: some ranks own an empty slice
    comms = coco.Communicator.init_all(R, [0] * R)
    try:
        before = sum(c.launch_count() for c in comms)
        z = torch.zeros(8, device="cuda")
        with coco.group():
            for c in comms:
                coco.runtime._check(coco.lib().cocoFusedSGD(
                    c._h, z.data_ptr(), 7, z.data_ptr(), None, 6, 0, 0.1, 1.0, None), "count 0")
        assert sum(c.launch_count() for c in comms) == before
        for n in (1, 2, 3, 5):
            ranks = Ranks(K.ADAM, R, n, seed=40 + n)
            ora = K.OracleState(K.ADAM, n, seed=40 + n)
            try:
                grads = K.make_grads(R, n, 40 + n, 0)
                ranks.step(grads, 0)
                ora.step(grads, 0)
                _check_against(ranks, ora, exact_w=True)
            finally:
                ranks.close()
    finally:
        for c in comms:
            c.destroy()


def test_more_than_2_to_the_31_elements():
    # Index and byte-offset arithmetic beyond 32 bits: 2^31 + 2^20 + 24 elements,
    # two ranks (slice starts at byte offset > 2^32 in the fp32 arrays).  Checked
    # through a size-independent property: the two-rank fused SGD step equals the
    # one-rank step on the pre-summed gradient, bit for bit, everywhere.
    n = (1 << 31) + (1 << 20) + 24
    free, _ = torch.cuda.mem_get_info()
    if free < 70 * (1 << 30):
        pytest.skip("needs about 60 GB of free device memory")
    R = 2
    gen = torch.Generator(device="cuda").manual_seed(99)

    def big_randn(scale, dtype):
        t = torch.empty(n, dtype=dtype, device="cuda")
        step = 1 << 28
        for a in range(0, n, step):
            b = min(n, a + step)
            t[a:b] = (torch.randn(b - a, device="cuda", generator=gen) * scale).to(dtype)
        return t

    g = [big_randn(1.0, torch.float16) for _ in range(R)]
    w0 = big_randn(0.02, torch.float32)
    comms = coco.Communicator.init_all(R, [0] * R)
    one = coco.Communicator.init_all(1, [0])[0]
    try:
        w = [w0.clone() for _ in range(R)]
        with coco.group():
            for r, c in enumerate(comms):
                c.fused_sgd(g[r], w[r], 0.01)
        torch.cuda.synchronize()
        for c in comms:
            assert c.status()["code"] == 0
        assert torch.equal(w[0], w[1])
        w1 = w[1]
        del w[1]
        del w1
        gs = torch.empty(n, dtype=torch.float32, device="cuda")
        step = 1 << 28
        for a in range(0, n, step):
            b = min(n, a + step)
            gs[a:b] = g[0][a:b].float() + g[1][a:b].float()
        del g
        one.fused_sgd(gs, w0, 0.01)
        torch.cuda.synchronize()
        assert torch.equal(w[0], w0)
        # the last elements (past 2^31) did change and are finite
        assert bool(torch.isfinite(w0[-64:]).all())
    finally:
        for c in comms + [one]:
            c.destroy()


def test_phase_times_of_the_last_call():
    # cocoLastPhaseTimes: LAMB has two data phases with the exchange of the norms between
    # them, everything else one; the three add up to less than the call's event time
    comm = coco.Communicator.init_all(1, [0])[0]
    try:
        n = 1 << 24
        g = torch.full((n,), 1e-3, device="cuda")
        w = torch.full((n,), 0.5, device="cuda")
        m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        for step, lamb in ((0, True), (1, True), (2, False)):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if lamb:
                comm.fused_lamb(g, w, m, v, 1e-3, 0.9, 0.999, 1e-6, 0.01, step)
            else:
                comm.fused_adam(g, w, m, v, 1e-3, 0.9, 0.999, 1e-6, step)
            e1.record()
            torch.cuda.synchronize()
            first, exchange, last = comm.last_phase_times()
            assert last > 0
            assert (first > 0 and exchange > 0) if lamb else (first == 0 and exchange == 0)
            assert first + exchange + last <= e0.elapsed_time(e1) * 1e3 + 1.0
            # cocoLastCtaSpread: the first, the median and the last CTA to finish its data
            lo_us, mid_us, hi_us = comm.last_cta_spread()
            assert 0 < lo_us <= mid_us <= hi_us <= e0.elapsed_time(e1) * 1e3 + 1.0
        assert comm.status()["code"] == 0
    finally:
        comm.destroy()
