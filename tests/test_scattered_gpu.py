"""Lists of tensors ("scattered" calls): one fused kernel over per-layer
gradient and weight tensors, with flat Sliced moments.  Virtual ranks on one
GPU; every tensor is checked against the CPU oracle run on that tensor alone,
bit for bit (the arithmetic is the flat path's)."""
import numpy as np
import pytest
import torch

import cases as K
import oracle_lib as O

pytestmark = pytest.mark.gpu

import coconet_b200 as coco  # noqa: E402

# sizes that are not multiples of 8, tiny tensors, and one larger than a slice
SIZES = [1000, 8, 3, 4096, 70001, 2, 1, (1 << 19) + 5, 24]


def _layout(counts, R):
    off, at = [], 0
    for c in counts:
        off.append(at)
        at += (c + 7) // 8 * 8
    S = ((at + R - 1) // R + 7) // 8 * 8
    return off, at, S


@pytest.mark.parametrize("R,chunk_shift,as_list", [(1, 0, False), (2, 0, True), (3, 0, False), (8, 0, False),
                                                  (1, 16, True), (3, 14, False)])
@pytest.mark.parametrize("opt", ["sgd", "adam"])
def test_scattered_matches_per_tensor_oracle(R, opt, chunk_shift, as_list, monkeypatch):
    # chunk_shift: the walk's chunk size (0 = chosen by size: 8 Ki elements here, so the
    # half-million-element tensor is 65 chunks spread over the CTAs); as_list: the
    # pointer arrays made once (TensorList) instead of on every call
    if chunk_shift:
        monkeypatch.setenv("COCO_SEG_CHUNK_SHIFT", str(chunk_shift))
    counts = SIZES
    off, total, S = _layout(counts, R)
    assert coco.scattered_slice_elems(counts, R) == S
    comms = coco.Communicator.init_all(R, [0] * R)
    h = K.HYPER
    try:
        w0 = [K.make_weights(c, 500 + b) for b, c in enumerate(counts)]
        w = [[torch.from_numpy(x.copy()).cuda() for x in w0] for _ in range(R)]
        m = [torch.zeros(S, device="cuda") for _ in range(R)]
        v = [torch.zeros(S, device="cuda") for _ in range(R)]
        ow = [x.copy() for x in w0]
        om = [np.zeros(c, np.float32) for c in counts]
        ov = [np.zeros(c, np.float32) for c in counts]
        for step in range(3):
            grads = [[K.make_grads(R, c, 600 + b, step)[r] for b, c in enumerate(counts)]
                     for r in range(R)]
            if step == 0 or not as_list:
                g = [[torch.from_numpy(x).cuda() for x in grads[r]] for r in range(R)]
                lists = [coco.TensorList(g[r], w[r]) for r in range(R)] if as_list else None
            else:       # the list holds the gradient tensors' addresses: refill them in place
                for r in range(R):
                    for b in range(len(counts)):
                        g[r][b].copy_(torch.from_numpy(grads[r][b]))
            with coco.group():
                for r, c in enumerate(comms):
                    gs, ws = (lists[r], None) if as_list else (g[r], w[r])
                    if opt == "sgd":
                        c.fused_sgd_scattered(gs, ws, 0.01)
                    else:
                        c.fused_adam_scattered(gs, ws, m[r], v[r], h["lr"], h["beta1"],
                                               h["beta2"], h["eps"], step)
            torch.cuda.synchronize()
            for c in comms:
                assert c.status()["code"] == 0
            for b, cnt in enumerate(counts):
                gsum = O.reduce_f32([grads[r][b] for r in range(R)])
                if opt == "sgd":
                    O.sgd(ow[b], gsum, 0.01)
                else:
                    O.adam(ow[b], om[b], ov[b], gsum, h["lr"], h["beta1"], h["beta2"], h["eps"], step)
                for r in range(R):
                    assert np.array_equal(w[r][b].cpu().numpy(), ow[b]), (step, b, r)
            if opt == "adam":
                flat_m = np.concatenate([x.cpu().numpy() for x in m])[:total]
                flat_v = np.concatenate([x.cpu().numpy() for x in v])[:total]
                for b, cnt in enumerate(counts):
                    assert np.array_equal(flat_m[off[b]:off[b] + cnt], om[b]), (step, b)
                    assert np.array_equal(flat_v[off[b]:off[b] + cnt], ov[b]), (step, b)
    finally:
        for c in comms:
            c.destroy()


@pytest.mark.parametrize("R,chunk_shift", [(1, 0), (2, 0), (3, 0), (8, 0), (2, 15)])
@pytest.mark.parametrize("quirk", [False, True])
def test_scattered_lamb_has_one_trust_ratio_per_tensor(R, quirk, chunk_shift, monkeypatch):
    """Every tensor of the list against the oracle's LAMB run on that tensor
    alone (its own ||w||, ||r||): moments bit for bit, weights to 1e-5 (the
    norms are summed in another order), replicas bit-identical.  With the
    quirk flag the step is also replayed through the reference sample's own
    host checker, tensor by tensor.  With the default chunk size the largest
    tensor's norms are summed by a warp, the others' by a thread each."""
    if chunk_shift:
        monkeypatch.setenv("COCO_SEG_CHUNK_SHIFT", str(chunk_shift))
    counts = SIZES
    off, total, S = _layout(counts, R)
    comms = coco.Communicator.init_all(R, [0] * R)
    h = dict(K.HYPER)
    flags = coco.LAMB_REF_QUIRK if quirk else 0
    if quirk:
        h["weight_decay"] = 1.0
    try:
        w0 = [K.make_weights(c, 700 + b) for b, c in enumerate(counts)]
        w = [[torch.from_numpy(x.copy()).cuda() for x in w0] for _ in range(R)]
        m = [torch.zeros(S, device="cuda") for _ in range(R)]
        v = [torch.zeros(S, device="cuda") for _ in range(R)]
        ow = [x.copy() for x in w0]
        om = [np.zeros(c, np.float32) for c in counts]
        ov = [np.zeros(c, np.float32) for c in counts]
        rm = [np.zeros(c, np.float32) for c in counts]
        rv = [np.zeros(c, np.float32) for c in counts]
        for step in range(3):
            grads = [[K.make_grads(R, c, 800 + b, step)[r] for b, c in enumerate(counts)]
                     for r in range(R)]
            g = [[torch.from_numpy(x).cuda() for x in grads[r]] for r in range(R)]
            w_old = [x.cpu().numpy().copy() for x in w[0]]
            with coco.group():
                for r, c in enumerate(comms):
                    c.fused_lamb_scattered(g[r], w[r], m[r], v[r], h["lr"], h["beta1"], h["beta2"],
                                           h["eps"], h["weight_decay"], step, flags=flags)
            torch.cuda.synchronize()
            for c in comms:
                assert c.status()["code"] == 0
            flat_m = np.concatenate([x.cpu().numpy() for x in m])[:total]
            flat_v = np.concatenate([x.cpu().numpy() for x in v])[:total]
            for b, cnt in enumerate(counts):
                gsum = O.reduce_f32([grads[r][b] for r in range(R)])
                O.lamb(ow[b], om[b], ov[b], gsum, h["lr"], h["beta1"], h["beta2"], h["eps"],
                       h["weight_decay"], step, flags=O.LAMB_REF_QUIRK if quirk else 0)
                got = w[0][b].cpu().numpy()
                K.assert_close(got, ow[b], 1e-5, f"w of tensor {b} at step {step}")
                for r in range(1, R):
                    assert np.array_equal(w[r][b].cpu().numpy(), got), (step, b, r)
                assert np.array_equal(flat_m[off[b]:off[b] + cnt], om[b]), (step, b)
                assert np.array_equal(flat_v[off[b]:off[b] + cnt], ov[b]), (step, b)
                if quirk and O.ref_available() and cnt >= 8:
                    assert O.ref_overlap_check("lamb", [grads[r][b] for r in range(R)], step,
                                               w_old[b], got, rm[b], rv[b], h["beta1"], h["beta2"],
                                               h["lr"], h["eps"]), (step, b)
                # the oracle continues from the device's weights, so that a last-bit
                # difference of one step is not carried into the next comparison
                ow[b] = got.copy()
    finally:
        for c in comms:
            c.destroy()


def test_scattered_lamb_equals_flat_call_on_one_tensor():
    R, n = 4, 1 << 18
    comms = coco.Communicator.init_all(R, [0] * R)
    h = K.HYPER
    try:
        w0 = K.make_weights(n, 17)
        grads = K.make_grads(R, n, 17, 0)
        g = [torch.from_numpy(x).cuda() for x in grads]
        wa = [torch.from_numpy(w0.copy()).cuda() for _ in range(R)]
        wb = [torch.from_numpy(w0.copy()).cuda() for _ in range(R)]
        S = n // R
        ma, va, mb, vb = ([torch.zeros(S, device="cuda") for _ in range(R)] for _ in range(4))
        with coco.group():
            for r, c in enumerate(comms):
                c.fused_lamb(g[r], wa[r], ma[r], va[r], h["lr"], h["beta1"], h["beta2"], h["eps"],
                             h["weight_decay"], 0)
        with coco.group():
            for r, c in enumerate(comms):
                c.fused_lamb_scattered([g[r]], [wb[r]], mb[r], vb[r], h["lr"], h["beta1"],
                                       h["beta2"], h["eps"], h["weight_decay"], 0)
        torch.cuda.synchronize()
        for r in range(R):
            assert torch.equal(ma[r], mb[r]) and torch.equal(va[r], vb[r])
            # the flat call sums its norm partials per CTA over the whole slice, the
            # list call per piece: same values to the last bits of a double
            K.assert_close(wb[r].cpu().numpy(), wa[r].cpu().numpy(), 1e-6, "w")
            assert torch.equal(wb[r], wb[0])
    finally:
        for c in comms:
            c.destroy()


def test_scattered_equals_flat_call_on_one_tensor():
    # a list with a single tensor of a multiple-of-8R size is the flat call
    R, n = 4, 1 << 18
    comms = coco.Communicator.init_all(R, [0] * R)
    h = K.HYPER
    try:
        w0 = K.make_weights(n, 7)
        grads = K.make_grads(R, n, 7, 0)
        g = [torch.from_numpy(x).cuda() for x in grads]
        wa = [torch.from_numpy(w0.copy()).cuda() for _ in range(R)]
        wb = [torch.from_numpy(w0.copy()).cuda() for _ in range(R)]
        S = n // R
        ma, va, mb, vb = ([torch.zeros(S, device="cuda") for _ in range(R)] for _ in range(4))
        with coco.group():
            for r, c in enumerate(comms):
                c.fused_adam(g[r], wa[r], ma[r], va[r], h["lr"], h["beta1"], h["beta2"], h["eps"], 0)
        with coco.group():
            for r, c in enumerate(comms):
                c.fused_adam_scattered([g[r]], [wb[r]], mb[r], vb[r], h["lr"], h["beta1"],
                                       h["beta2"], h["eps"], 0)
        torch.cuda.synchronize()
        for r in range(R):
            assert torch.equal(wa[r], wb[r]) and torch.equal(ma[r], mb[r]) and torch.equal(va[r], vb[r])
    finally:
        for c in comms:
            c.destroy()


def test_scattered_rejects_what_is_not_built():
    c = coco.Communicator.init_all(1, [0])[0]
    try:
        g = [torch.zeros(16, device="cuda")]
        w = [torch.zeros(16, device="cuda")]
        with pytest.raises(coco.CocoError):     # moments are required
            c.fused_adam_scattered(g, w, None, None, 1e-3, 0.9, 0.999, 1e-6, 0)
        with pytest.raises(coco.CocoError):     # the forked-NCCL formulation is flat-only
            c.fused_adam_scattered(g, w, w[0], w[0], 1e-3, 0.9, 0.999, 1e-6, 0,
                                   variant=coco.VARIANT_NCCL)
        many = [torch.zeros(8, device="cuda") for _ in range(2049)]   # more tensors than the norm table holds
        with pytest.raises(coco.CocoError):
            c.fused_lamb_scattered(many, many, w[0], w[0], 1e-3, 0.9, 0.999, 1e-6, 0.01, 0)
    finally:
        c.destroy()


@pytest.mark.parametrize("opt", ["adam", "lamb"])
def test_scattered_more_pieces_than_the_shared_tables_hold(opt):
    """2000 small tensors on one rank: more pieces than the kernel keeps first-chunk
    numbers and trust ratios for in shared memory (1536), so the walk's lookups and
    the per-tensor ratios of the pieces beyond come from device memory.  Every
    tensor against the oracle's run on that tensor alone."""
    rng = np.random.default_rng(11)
    counts = [int(c) for c in rng.integers(1, 40, size=2000)]
    counts[1700] = 20000                     # one piece of several chunks among the late ones
    off, total, S = _layout(counts, 1)
    comm = coco.Communicator.init_all(1, [0])[0]
    h = K.HYPER
    try:
        w0 = [K.make_weights(c, 900 + b) for b, c in enumerate(counts)]
        grads = [K.make_grads(1, c, 950 + b, 0)[0] for b, c in enumerate(counts)]
        # all tensors inside two big buffers, every one at a multiple of 8 elements
        gbuf, wbuf = torch.zeros(total, device="cuda"), torch.zeros(total, device="cuda")
        g = [gbuf[o:o + c] for o, c in zip(off, counts)]
        w = [wbuf[o:o + c] for o, c in zip(off, counts)]
        gbuf.copy_(torch.from_numpy(np.concatenate(
            [np.pad(x, (0, (len(x) + 7) // 8 * 8 - len(x))) for x in grads])))
        wbuf.copy_(torch.from_numpy(np.concatenate(
            [np.pad(x, (0, (len(x) + 7) // 8 * 8 - len(x))) for x in w0])))
        m, v = torch.zeros(S, device="cuda"), torch.zeros(S, device="cuda")
        tl = coco.TensorList(g, w)
        if opt == "adam":
            comm.fused_adam_scattered(tl, None, m, v, h["lr"], h["beta1"], h["beta2"], h["eps"], 0)
        else:
            comm.fused_lamb_scattered(tl, None, m, v, h["lr"], h["beta1"], h["beta2"], h["eps"],
                                      h["weight_decay"], 0)
        torch.cuda.synchronize()
        assert comm.status()["code"] == 0
        got_w, got_m, got_v = wbuf.cpu().numpy(), m.cpu().numpy(), v.cpu().numpy()
        for b, c in enumerate(counts):
            ow, om, ov = w0[b].copy(), np.zeros(c, np.float32), np.zeros(c, np.float32)
            if opt == "adam":
                O.adam(ow, om, ov, grads[b], h["lr"], h["beta1"], h["beta2"], h["eps"], 0)
                assert np.array_equal(got_w[off[b]:off[b] + c], ow), b
            else:
                O.lamb(ow, om, ov, grads[b], h["lr"], h["beta1"], h["beta2"], h["eps"],
                       h["weight_decay"], 0)
                K.assert_close(got_w[off[b]:off[b] + c], ow, 1e-5, f"w of tensor {b}")
            assert np.array_equal(got_m[off[b]:off[b] + c], om), b
            assert np.array_equal(got_v[off[b]:off[b] + c], ov), b
    finally:
        comm.destroy()
