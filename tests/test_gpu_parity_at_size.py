"""Parity of the fused score + top-k pass at the sizes the benchmark configurations state, through the C ABI against
the CPU oracle on the same seeded rows (the generator of manta_b200/synth.py, the one bench.py uses):

  * batched f16 dot, whole: 1,000,000 x 384, 64 queries, k = 100 (tensor-core pass);
  * q8 cosine 768-wide on 1,000,000 rows, one query and 256 queries, k = 10;
  * q4 l2_distance 256-wide on 1,000,000 rows, one query and 32 queries, k = 1000 smallest;
  * embed -> q8 dot 384-wide on 500,000 rows, 128 token sequences, k = 50.

The oracle scores the de-quantised rows (what the reference's tensors hold) with the restated builtins and selects
with the restated topKTensor; the comparison is tests/helpers.py::topk_parity_report: returned scores within the
tolerance, ids identical except across score gaps below twice the tolerance.  Each case also prints the worst error
it saw, in units of the tolerance and relative to |q||d|.
"""
import numpy as np
import pytest

import oracle
from helpers import EMBED_FLOOR, topk_parity_report

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    from manta_b200 import native

    r = native.Runtime(0)
    yield r
    r.close()


def _dequantised(layout, rows, cols, normalise):
    """The seeded f16 rows as the oracle sees them after the layout's quantiser: float32 [rows, cols]."""
    from manta_b200 import synth

    x = synth.rows_f16(0, rows, cols, normalise=normalise).float().cpu().numpy()
    if layout == "q8":
        return oracle.unpack_q8_rows(*oracle.pack_q8_rows(x))
    if layout == "q4":
        return oracle.unpack_q4_b32(*oracle.pack_q4_b32(x))
    return np.ascontiguousarray(x)


def _check(rep, label):
    print(f"\n{label}: worst score error {rep['worst_score_error']:.4f} x tolerance, {rep['worst_error_vs_scale']:.3e} of |q||d|; "
          f"{rep['mismatches']} id mismatches, {rep['mismatches_outside_gap']} outside the gap rule "
          f"(worst gap {rep['worst_gap_over_limit']:.3f} x limit)")
    assert rep["ids_valid"] and rep["ordered"], rep
    assert rep["scores_within_tolerance"], rep
    assert rep["ids_within_gap_rule"], rep


CASES = [  # (label, layout, metric, rows, cols, queries, k, smallest, normalise)
    ("f16 dot 1M x 384, Q=64, k=100", "f16", "dot", 1_000_000, 384, 64, 100, False, True),
    ("q8 cosine 1M x 768, Q=1, k=10", "q8", "cosine", 1_000_000, 768, 1, 10, False, True),
    ("q8 cosine 1M x 768, Q=256, k=10", "q8", "cosine", 1_000_000, 768, 256, 10, False, True),
    ("q4 l2 1M x 256, Q=1, k=1000 smallest", "q4", "l2_distance", 1_000_000, 256, 1, 1000, True, False),
    ("q4 l2 1M x 256, Q=32, k=1000 smallest", "q4", "l2_distance", 1_000_000, 256, 32, 1000, True, False),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: c[0])
def test_fused_topk_at_stated_size(rt, case):
    from manta_b200 import synth

    label, layout, metric, rows, cols, nq, k, smallest, normalise = case
    data, scales = synth.packed_candidates(rt, layout, 0, rows, cols, normalise=normalise)
    cands = rt.bind(layout, data, scales, rows=rows, cols=cols)
    q = synth.queries_f16(nq, cols, normalise=normalise).float().cpu().numpy()
    ids, scores = rt.score_topk(cands, metric, q, k, smallest=smallest)
    cands.unbind()
    deq = _dequantised(layout, rows, cols, normalise)
    _check(topk_parity_report(metric, q, deq, np.asarray(ids).reshape(nq, k), np.asarray(scores).reshape(nq, k), k, smallest), label)


def test_embed_then_score_at_stated_size(rt):
    """Token batch -> embedding front end -> q8 dot + top-k on 500,000 x 384 rows, 128 sequences of 128 tokens, k = 50."""
    from manta_b200 import synth

    rows, cols, batch, seq, vocab, dim, k = 500_000, 384, 128, 128, 32000, 384, 50
    data, scales = synth.packed_candidates(rt, "q8", 0, rows, cols)
    cands = rt.bind("q8", data, scales, rows=rows, cols=cols)
    table, proj = synth.embed_weights_f16(vocab, dim, cols)
    tokens, mask = synth.token_batches(1, batch, seq, vocab)
    emb = rt.bind_embedder(table.cpu().numpy().view(np.uint16), proj.cpu().numpy().view(np.uint16))
    h_tok, h_mask = tokens[0].cpu().numpy(), mask[0].cpu().numpy()
    ids, scores = rt.embed_score_topk(emb, cands, h_tok, h_mask, "dot", k)
    rt.unbind_embedder(emb)
    cands.unbind()
    pooled = oracle.embed_pooled(table.float().cpu().numpy(), proj.float().cpu().numpy(), h_tok, h_mask, 0)
    q = oracle.half_to_float(oracle.float_to_half(pooled))  # the scan reads the pooled rows rounded to f16
    deq = _dequantised("q8", rows, cols, True)
    _check(topk_parity_report("dot", q, deq, ids, scores, k, floor=EMBED_FLOOR), "embed + q8 dot 500k x 384, Q=128, k=50")


# Long passes deal their tiles differently from short ones (runs of eight tiles per warp, then a round-robin remainder; a
# fused single-query top-k pass hands out its last quarter on demand): every row must still be scored exactly once.  Narrow
# rows keep the oracle cheap: 64-byte rows make 32-row tiles, so 1.3 M rows are 17 tiles for each of the 2,368 warps.
LONG = [("q8", "dot", 1_300_003, 64), ("f16", "cosine", 1_300_003, 64), ("q4", "l2_distance", 1_300_003, 128)]


@pytest.mark.parametrize("case", LONG, ids=lambda c: f"{c[0]}-{c[1]}-{c[2]}x{c[3]}")
def test_every_row_of_a_long_pass_is_scored_once(rt, case):
    from helpers import assert_scores_close, assert_topk_matches, make_rows, pack

    layout, metric, rows, cols = case
    rng = np.random.default_rng(rows + cols)
    x = make_rows(rng, rows, cols, normalised=(layout != "q4"))
    q = make_rows(rng, 2, cols)
    data, scales, deq = pack(layout, x)
    cands = rt.bind(layout, data, scales)
    try:
        got = rt.score(cands, metric, q)                      # all scores: fixed deal, runs + remainder
        ids1, sc1 = rt.score_topk(cands, metric, q[:1], 25)   # fused single-query pass: part of it on demand (f16 / q8)
        ids2, sc2 = rt.score_topk(cands, metric, q, 25, smallest=True)
    finally:
        cands.unbind()
    ref = oracle.SCORE_FNS[metric](q, deq)
    assert_scores_close(metric, q, deq, got, ref)
    assert_topk_matches(metric, q[:1], deq, ids1, sc1, 25)
    assert_topk_matches(metric, q, deq, ids2, sc2, 25, smallest=True)
