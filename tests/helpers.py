"""Shared helpers of the parity tests: seeded inputs, packing through the oracle, comparison rules."""
import numpy as np

import oracle

REL_TOL = 1e-3  # float scores: 1e-3 relative ...
FLOOR = 5e-2    # ... down to scores of FLOOR*|q||d|; below that the bound is absolute REL_TOL*FLOOR*|q||d|
# (5e-5*|q||d| absolute: the two int8 planes that carry the query hold max|q| * 2^-16 per element; the
# reference's own tests compare its device and host paths with 5e-4 absolute, ten times looser.)


def f16_round(x):
    """Values rounded to f16 and widened back (the canonical, f16-representable inputs)."""
    return oracle.half_to_float(oracle.float_to_half(np.asarray(x, np.float32)))


def make_rows(rng, n, d, normalised=True):
    x = rng.standard_normal((n, d))
    if normalised:
        x /= np.maximum(np.linalg.norm(x, axis=1, keepdims=True), 1e-30)
    return f16_round(x.astype(np.float32))


def pack(layout, x):
    """(data, scales, dequantised f32 rows) for a layout name."""
    if layout == "f16":
        return oracle.float_to_half(x), None, f16_round(x)
    if layout == "q8":
        codes, scales = oracle.pack_q8_rows(x)
        return codes, scales, oracle.unpack_q8_rows(codes, scales)
    codes, scales = oracle.pack_q4_b32(x)
    return codes, scales, oracle.unpack_q4_b32(codes, scales)


def score_scale(metric, q, deq):
    """|q||d| per (query,row): the magnitude relative tolerances are floored with."""
    qn = np.linalg.norm(np.atleast_2d(q).astype(np.float64), axis=1)
    dn = np.linalg.norm(deq.astype(np.float64), axis=1)
    if metric == "cosine":
        return np.ones((qn.shape[0], dn.shape[0]))
    if metric == "dot":
        return np.maximum(qn[:, None] * dn[None, :], 1e-30)
    return np.maximum(qn[:, None] + dn[None, :], 1e-30)


def tol_abs(metric, q, deq, ref):
    scale = score_scale(metric, q, deq)
    return REL_TOL * np.maximum(np.abs(np.atleast_2d(ref)), FLOOR * scale)


def assert_scores_close(metric, q, deq, got, ref):
    got2, ref2 = np.atleast_2d(got), np.atleast_2d(ref)
    tol = tol_abs(metric, q, deq, ref2)
    bad = np.abs(got2.astype(np.float64) - ref2) > tol
    assert not bad.any(), f"{metric}: {bad.sum()} scores out of tolerance, worst {np.abs(got2 - ref2).max()}"


def assert_topk_matches(metric, q, deq, ids, scores, k, smallest=False):
    """ids/scores [Q,k] from the device against the oracle on the de-quantised rows: scores within
    tolerance of the oracle's score of the same row, best-first order, ids identical to topKTensor's
    except where the two candidates' oracle scores differ by less than the tolerance."""
    q2 = np.atleast_2d(q)
    ids2, sc2 = np.atleast_2d(ids), np.atleast_2d(scores)
    ref_full = oracle.SCORE_FNS[metric](q2, deq)
    ref_ids = oracle.topk(ref_full, k, smallest)
    tol = tol_abs(metric, q2, deq, ref_full)
    nq = q2.shape[0]
    assert ids2.shape == (nq, k) and sc2.shape == (nq, k)
    for i in range(nq):
        assert len(set(ids2[i].tolist())) == k, "duplicate ids"
        assert ids2[i].min() >= 0 and ids2[i].max() < deq.shape[0]
        ref_at = ref_full[i, ids2[i]]
        assert np.all(np.abs(sc2[i] - ref_at) <= tol[i, ids2[i]]), (
            f"query {i}: returned scores differ from the oracle's, worst {np.abs(sc2[i] - ref_at).max()}")
        g = -sc2[i] if smallest else sc2[i]
        order_ok = (g[:-1] > g[1:]) | ((g[:-1] == g[1:]) & (ids2[i][:-1] < ids2[i][1:]))
        assert order_ok.all(), f"query {i}: result not ordered best first / lower id first"
        diff = ids2[i] != ref_ids[i]
        if diff.any():
            gap = np.abs(ref_full[i, ids2[i][diff]] - ref_full[i, ref_ids[i][diff]])
            lim = 2 * np.maximum(tol[i, ids2[i][diff]], tol[i, ref_ids[i][diff]])
            assert np.all(gap <= lim), f"query {i}: ids differ where the score gap {gap.max()} exceeds tolerance"
    return ref_full, ref_ids
