"""Shared helpers of the parity tests: seeded inputs, packing through the oracle, comparison rules."""
import numpy as np

import oracle

REL_TOL = 1e-3  # float scores: 1e-3 relative ...
FLOOR = 2e-2    # ... down to scores of FLOOR*|q||d|; below that the bound is absolute REL_TOL*FLOOR*|q||d| = 2e-5*|q||d|
# Why a floor at all: scores of random vectors cluster at 0 +- |q||d|/sqrt(D), where a relative bound means nothing.
# Why this one: on packed candidates the device carries the f16 query as two int8 planes, 16-bit fixed point against
# max|q|, i.e. up to max|q| * 2^-16 per element, so the deviation from the oracle grows with max|q| / |q|, which is
# largest for narrow rows.  Largest deviations seen: 1.6e-5*|q||d| at 31 columns (q8 dot / cosine), 1.3e-5 at 64 columns
# (q4), 4.5e-6 at 768 columns (q8 cosine, 1,000,000 rows x 256 queries), 1.5e-7 for f16 candidates at any width.  The
# absolute part of the bound sits just above the worst of these.  (The reference's own tests compare its device and
# host paths with 5e-4 absolute.)
EMBED_FLOOR = 5e-2
# End-to-end embed + score compares against an oracle that embeds on the CPU: the two pooled queries agree to a few
# 1e-7 relative, which flips the f16 rounding of a handful of query elements (1e-3 relative each); the scores then
# differ by up to 1.7e-5*|q||d| through no fault of the scoring pass, hence the wider floor for that comparison only.


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


def _row_norms(deq):
    deq = np.asarray(deq, np.float32)
    return np.sqrt(np.einsum("ij,ij->i", deq, deq, dtype=np.float64))


def score_scale(metric, q, deq, dn=None):
    """|q||d| per (query,row): the magnitude relative tolerances are floored with."""
    qn = np.linalg.norm(np.atleast_2d(q).astype(np.float64), axis=1)
    dn = _row_norms(deq) if dn is None else dn
    if metric == "cosine":
        return np.ones((qn.shape[0], dn.shape[0]))
    if metric == "dot":
        return np.maximum(qn[:, None] * dn[None, :], 1e-30)
    return np.maximum(qn[:, None] + dn[None, :], 1e-30)


def tol_abs(metric, q, deq, ref, floor=None):
    scale = score_scale(metric, q, deq)
    return REL_TOL * np.maximum(np.abs(np.atleast_2d(ref)), (FLOOR if floor is None else floor) * scale)


def assert_scores_close(metric, q, deq, got, ref):
    got2, ref2 = np.atleast_2d(got), np.atleast_2d(ref)
    tol = tol_abs(metric, q, deq, ref2)
    bad = np.abs(got2.astype(np.float64) - ref2) > tol
    assert not bad.any(), f"{metric}: {bad.sum()} scores out of tolerance, worst {np.abs(got2 - ref2).max()}"


def topk_parity_report(metric, q, deq, ids, scores, k, smallest=False, ref_full=None, floor=None):
    """Compares device ids/scores [Q,k] with the oracle on the de-quantised rows and returns a report instead of
    asserting.  The rule: returned scores within tolerance of the oracle's score of the same row; best-first order
    (equal scores: lower id first); ids identical to topKTensor's (runtime/backend/tensor_ops.go:1523-1592) except at
    positions where the two candidates' oracle scores differ by less than twice the tolerance (the gap rule).
    `worst_score_error` is the largest |device - oracle| in units of the tolerance (<= 1 passes);
    `worst_error_vs_scale` the same error relative to |q||d| (1 for cosine)."""
    q2 = np.atleast_2d(np.asarray(q, np.float32))
    ids2, sc2 = np.atleast_2d(ids), np.atleast_2d(scores)
    if ref_full is None:
        ref_full = oracle.SCORE_FNS[metric](q2, deq)
    ref_full = np.atleast_2d(ref_full)
    ref_ids = np.atleast_2d(oracle.topk(ref_full, k, smallest))
    nq, nrows = q2.shape[0], deq.shape[0]
    qn = np.linalg.norm(q2.astype(np.float64), axis=1)
    floor = FLOOR if floor is None else floor

    def tol_at(i, rows):
        ref = ref_full[i, rows].astype(np.float64)
        if metric == "cosine":
            scale = np.ones(len(rows))
        else:
            d = np.asarray(deq[rows], np.float64)
            dn = np.sqrt((d * d).sum(axis=1))
            scale = np.maximum(qn[i] * dn if metric == "dot" else qn[i] + dn, 1e-30)
        return REL_TOL * np.maximum(np.abs(ref), floor * scale), scale

    rep = {"queries": int(nq), "rows": int(nrows), "k": int(k), "shape_ok": ids2.shape == (nq, k) and sc2.shape == (nq, k),
           "ids_equal_oracle": True, "ids_within_gap_rule": True, "scores_within_tolerance": True, "ordered": True,
           "ids_valid": True, "mismatches": 0, "mismatches_outside_gap": 0, "worst_score_error": 0.0,
           "worst_error_vs_scale": 0.0, "worst_gap_over_limit": 0.0}
    if not rep["shape_ok"]:
        rep["ids_equal_oracle"] = rep["ids_within_gap_rule"] = False
        return rep
    for i in range(nq):
        mine, want = ids2[i].astype(np.int64), ref_ids[i].astype(np.int64)
        if len(set(mine.tolist())) != k or mine.min() < 0 or mine.max() >= nrows:
            rep["ids_valid"] = rep["ids_within_gap_rule"] = rep["ids_equal_oracle"] = False
            continue
        tol_m, scale_m = tol_at(i, mine)
        err = np.abs(sc2[i].astype(np.float64) - ref_full[i, mine])
        rep["worst_score_error"] = max(rep["worst_score_error"], float((err / tol_m).max()))
        rep["worst_error_vs_scale"] = max(rep["worst_error_vs_scale"], float((err / scale_m).max()))
        if (err > tol_m).any():
            rep["scores_within_tolerance"] = False
        g = -sc2[i] if smallest else sc2[i]
        if not ((g[:-1] > g[1:]) | ((g[:-1] == g[1:]) & (mine[:-1] < mine[1:]))).all():
            rep["ordered"] = False
        diff = mine != want
        if diff.any():
            rep["ids_equal_oracle"] = False
            rep["mismatches"] += int(diff.sum())
            tol_w, _ = tol_at(i, want[diff])
            gap = np.abs(ref_full[i, mine[diff]].astype(np.float64) - ref_full[i, want[diff]])
            lim = 2 * np.maximum(tol_m[diff], tol_w)
            rep["worst_gap_over_limit"] = max(rep["worst_gap_over_limit"], float((gap / lim).max()))
            outside = int((gap > lim).sum())
            rep["mismatches_outside_gap"] += outside
            if outside:
                rep["ids_within_gap_rule"] = False
    rep["ok"] = bool(rep["ids_valid"] and rep["ids_within_gap_rule"] and rep["scores_within_tolerance"] and rep["ordered"])
    return rep


def assert_topk_matches(metric, q, deq, ids, scores, k, smallest=False, floor=None):
    """ids/scores [Q,k] from the device against the oracle on the de-quantised rows (rule: topk_parity_report)."""
    q2 = np.atleast_2d(q)
    ref_full = np.atleast_2d(oracle.SCORE_FNS[metric](q2, deq))
    rep = topk_parity_report(metric, q2, deq, ids, scores, k, smallest, ref_full=ref_full, floor=floor)
    assert rep["shape_ok"], "ids / scores do not have shape [Q,k]"
    assert rep["ids_valid"], "duplicate or out-of-range ids"
    assert rep["scores_within_tolerance"], f"returned scores differ from the oracle's, worst {rep['worst_score_error']:.3g} x tolerance"
    assert rep["ordered"], "result not ordered best first / lower id first"
    assert rep["ids_within_gap_rule"], (
        f"{rep['mismatches_outside_gap']} ids differ where the score gap exceeds the tolerance (worst {rep['worst_gap_over_limit']:.3g} x limit)")
    return ref_full, np.atleast_2d(oracle.topk(ref_full, k, smallest))
