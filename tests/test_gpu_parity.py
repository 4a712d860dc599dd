"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle on the same seeded inputs.

Integer work (q8 accumulators, pack codes, ids on exact ties) must be bit-exact; float scores within 1e-3
relative (floored as tests/helpers.py states); top-k ids identical to topKTensor's except across score gaps
below that tolerance.
"""
import json
import os

import numpy as np
import pytest

import oracle
from helpers import assert_scores_close, assert_topk_matches, f16_round, make_rows, pack

pytestmark = pytest.mark.gpu

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kat.json")))


@pytest.fixture(scope="module")
def rt():
    from manta_b200 import native

    r = native.Runtime(0)
    yield r
    r.close()


def _bind(rt, layout, x, row_base=0):
    data, scales, deq = pack(layout, x)
    return rt.bind(layout, data, scales, row_base=row_base), deq


def _pad32(a):
    a = np.asarray(a, np.float32)
    pad = (-a.shape[-1]) % 32
    return np.pad(a, [(0, 0)] * (a.ndim - 1) + [(0, pad)])


# ---- the reference's own known-answer fixtures through the C ABI ------------------------------------------
@pytest.mark.parametrize("layout", ["f16", "q8", "q4"])
@pytest.mark.parametrize("case", GOLD["score"] + GOLD["direct_q4_ops"], ids=lambda c: c["op"])
def test_reference_score_fixtures(rt, layout, case):
    docs = np.array(case["docs"], np.float32)
    query = np.array(case["query"], np.float32)
    if layout == "q4":  # block layout needs 32 columns; zero columns change none of the three scores
        docs, query = _pad32(docs), _pad32(query)
    cands, _ = _bind(rt, layout, docs)
    out = rt.score(cands, case["op"], query)
    np.testing.assert_allclose(out, np.array(case["want"], np.float32), atol=GOLD["tolerance_abs"], rtol=0)


@pytest.mark.parametrize("layout", ["f16", "q8", "q4"])
@pytest.mark.parametrize("case", GOLD["pipelines"], ids=lambda c: c["name"])
def test_reference_pipeline_fixtures(rt, layout, case):
    docs = np.array(case["docs"], np.float32)
    query = np.array(case["query"], np.float32)
    cols = docs.shape[1]
    if layout == "q4":
        docs, query = _pad32(docs), _pad32(query)
    cands, _ = _bind(rt, layout, docs)
    ids, scores = rt.score_topk(cands, case["op"], query, case["k"])
    np.testing.assert_array_equal(ids, case["want_ids"])
    np.testing.assert_allclose(scores, np.array(case["want_scores"], np.float32), atol=GOLD["tolerance_abs"], rtol=0)
    if "want_docs" in case:
        rows = rt.gather_rows(cands, ids)[:, :cols]
        # real 4-bit blocks with an f16 scale store 1.0 as 7 * half(1/7) = 0.99976; the reference's q4 tensors
        # are float32 in disguise, so the comparison uses the reference's own 5e-4 tolerance there
        atol = GOLD["tolerance_abs"] if layout == "q4" else 0
        np.testing.assert_allclose(rows, np.array(case["want_docs"], np.float32), atol=atol, rtol=0)


def test_reference_topk_tie_fixture(rt):
    # topKTensor fixture [0.25, 0.9, 0.5, 0.9], k=3 -> [1, 3, 2]: rows whose dot with q=[1] are those scores
    case = GOLD["topk"][0]
    docs = np.array(case["scores"], np.float32)[:, None]
    cands, _ = _bind(rt, "f16", f16_round(docs))
    ids, _ = rt.score_topk(cands, "dot", np.array([1.0], np.float32), case["k"])
    ref = oracle.topk(oracle.dot_rows(np.array([1.0], np.float32), f16_round(docs)), case["k"])
    np.testing.assert_array_equal(ids, ref)
    np.testing.assert_array_equal(ids, case["want"])


# ---- seeded parity, all layouts x metrics ---------------------------------------------------------------------
SHAPES = [  # (rows, cols)
    (1, 32), (7, 32), (1000, 32), (4099, 64), (10000, 128), (3001, 256), (2500, 384), (2049, 768),
    (513, 1024), (300, 2048),
]
ODD_SHAPES = [(999, 1), (777, 2), (1234, 31), (555, 33), (800, 100), (257, 770)]  # f16 / q8 only


@pytest.mark.parametrize("metric", ["dot", "cosine", "l2_distance"])
@pytest.mark.parametrize("layout", ["f16", "q8", "q4"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: f"{s[0]}x{s[1]}")
def test_full_scores_match_oracle(rt, layout, metric, shape):
    rows, cols = shape
    if layout == "f16" and cols > 1024:
        cols = 1024
    rng = np.random.default_rng(rows * 131 + cols)
    x = make_rows(rng, rows, cols, normalised=(layout != "q4"))
    q = make_rows(rng, 3, cols)
    cands, deq = _bind(rt, layout, x)
    got = rt.score(cands, metric, q)
    ref = oracle.SCORE_FNS[metric](q, deq)
    assert got.shape == ref.shape
    assert_scores_close(metric, q, deq, got, ref)


@pytest.mark.parametrize("metric", ["dot", "cosine", "l2_distance"])
@pytest.mark.parametrize("layout", ["f16", "q8"])
@pytest.mark.parametrize("shape", ODD_SHAPES, ids=lambda s: f"{s[0]}x{s[1]}")
def test_ragged_widths(rt, layout, metric, shape):
    rows, cols = shape
    rng = np.random.default_rng(rows + cols)
    x = make_rows(rng, rows, cols)
    q = make_rows(rng, 2, cols)
    cands, deq = _bind(rt, layout, x)
    ref = oracle.SCORE_FNS[metric](q, deq)
    assert_scores_close(metric, q, deq, rt.score(cands, metric, q), ref)
    k = min(5, rows)
    ids, scores = rt.score_topk(cands, metric, q, k)
    assert_topk_matches(metric, q, deq, ids, scores, k)


TOPK_CASES = [  # (layout, metric, rows, cols, nq, k, smallest)
    ("q8", "cosine", 10000, 128, 1, 10, False),      # the CPU-runnable select configuration
    ("q8", "cosine", 200000, 768, 1, 10, False),
    ("q8", "cosine", 60000, 768, 3, 10, False),
    ("q8", "dot", 50000, 384, 4, 50, False),
    ("q8", "l2_distance", 30000, 256, 2, 100, True),
    ("f16", "dot", 100000, 384, 1, 100, False),
    ("f16", "dot", 40000, 384, 5, 100, False),
    ("f16", "cosine", 30000, 128, 2, 7, False),
    ("f16", "l2_distance", 20000, 64, 1, 33, True),
    ("q4", "l2_distance", 100000, 256, 1, 1000, True),
    ("q4", "l2_distance", 30000, 256, 3, 1000, True),
    ("q4", "cosine", 50000, 128, 2, 10, False),
    ("q4", "dot", 20000, 768, 1, 64, False),
    ("q8", "cosine", 5000, 768, 1, 2048, False),     # largest k
    ("q8", "dot", 17, 32, 1, 17, False),             # k == rows
    ("f16", "cosine", 1, 8, 1, 1, False),            # single row
]


@pytest.mark.parametrize("case", TOPK_CASES, ids=lambda c: "-".join(str(v) for v in c))
def test_fused_topk_matches_oracle(rt, case):
    layout, metric, rows, cols, nq, k, smallest = case
    rng = np.random.default_rng(1000 + TOPK_CASES.index(case))
    x = make_rows(rng, rows, cols, normalised=(layout != "q4"))
    q = make_rows(rng, nq, cols, normalised=(layout != "q4"))
    cands, deq = _bind(rt, layout, x)
    before = rt.stats()["mma_passes"]
    ids, scores = rt.score_topk(cands, metric, q, k, smallest=smallest)
    on_tensor_cores = rt.stats()["mma_passes"] > before   # two or more queries over f16 / q8 rows, eight over q4
    assert_topk_matches(metric, q, deq, ids, scores, k, smallest)
    # the fused pass returns gather(scores, ids) of the unfused one (the streaming kernel): exactly, except that the
    # tensor cores add the f32 products of f16 / q4 rows in another order than the streaming kernel's fma chain
    full = rt.score(cands, metric, q)
    at = np.take_along_axis(np.atleast_2d(full), np.atleast_2d(ids).astype(np.int64), 1)
    if on_tensor_cores and layout != "q8":
        np.testing.assert_allclose(scores, at, rtol=2e-4, atol=2e-5)
    else:
        np.testing.assert_array_equal(scores, at)
    # and it is deterministic
    ids2, scores2 = rt.score_topk(cands, metric, q, k, smallest=smallest)
    np.testing.assert_array_equal(ids, ids2)
    np.testing.assert_array_equal(scores, scores2)


def test_single_query_rank1_form(rt):
    rng = np.random.default_rng(5)
    x = make_rows(rng, 3000, 128)
    q = make_rows(rng, 1, 128)[0]
    cands, deq = _bind(rt, "q8", x)
    ids, scores = rt.score_topk(cands, "cosine", q, 10)
    assert ids.shape == (10,) and scores.shape == (10,)
    rid, rsc = oracle.score_topk("cosine", q, deq, 10)
    np.testing.assert_array_equal(ids, rid)
    np.testing.assert_allclose(scores, rsc, rtol=1e-3)


# ---- integer work is bit-exact ---------------------------------------------------------------------------------
@pytest.mark.parametrize("cols", [32, 128, 384, 768, 1000])
def test_q8_integer_accumulators_bit_exact(rt, cols):
    rng = np.random.default_rng(cols)
    x = make_rows(rng, 5003, cols)
    q = make_rows(rng, 1, cols)[0]
    codes, scales = oracle.pack_q8_rows(x)
    cands = rt.bind("q8", codes, scales)
    acc = rt.q8_accumulators(cands, q)
    for metric in ("dot", "cosine", "l2_distance"):
        model, macc = oracle.q8_model_scores(q, codes, scales, metric, want_acc=True)
        np.testing.assert_array_equal(acc, macc)
        got = rt.score(cands, metric, q)
        np.testing.assert_array_equal(got.view(np.uint32), model.view(np.uint32))


def test_pack_kernels_bit_exact(rt):
    rng = np.random.default_rng(21)
    x = (rng.standard_normal((1237, 96)) * rng.uniform(0.01, 30, (1237, 1))).astype(np.float32)
    x[11] = 0
    x[12, :32] = 0
    codes, scales = rt.pack_q8_rows(x)
    rc, rs = oracle.pack_q8_rows(x)
    np.testing.assert_array_equal(codes, rc)
    np.testing.assert_array_equal(scales.view(np.uint32), rs.view(np.uint32))
    c4, s4 = rt.pack_q4_b32(x)
    r4, rs4 = oracle.pack_q4_b32(x)
    np.testing.assert_array_equal(c4, r4)
    np.testing.assert_array_equal(s4, rs4)
    # half-away-from-zero on exact ties (q = 2.5 -> 3), the reference quantiser's rounding
    t = np.zeros((1, 32), np.float32)
    t[0, :4] = [127.0, 2.5, -2.5, 0.5]
    tc, ts = rt.pack_q8_rows(t)
    np.testing.assert_array_equal(tc[0, :4], [127, 3, -3, 1])


# ---- ties, zero rows, selection edge cases ------------------------------------------------------------------------
def test_ties_resolve_to_lower_row_id(rt):
    rng = np.random.default_rng(3)
    base = make_rows(rng, 50, 64)
    x = np.tile(base, (40, 1))  # every row appears 40 times -> 40-way exact ties
    q = make_rows(rng, 2, 64)
    for layout in ("f16", "q8"):
        cands, deq = _bind(rt, layout, x)
        ids, scores = rt.score_topk(cands, "dot", q, 100)
        full = rt.score(cands, "dot", q)
        want = oracle.topk(full, 100)  # the device's own scores, the oracle's ordering rule
        np.testing.assert_array_equal(ids, want)


def test_zero_rows_and_zero_query(rt):
    rng = np.random.default_rng(4)
    x = make_rows(rng, 500, 64)
    x[::7] = 0
    q = make_rows(rng, 2, 64)
    q[1] = 0
    for layout in ("f16", "q8", "q4"):
        cands, deq = _bind(rt, layout, x)
        got = rt.score(cands, "cosine", q)
        ref = oracle.cosine_rows(q, deq)
        assert np.all(got[:, ::7] == 0) and np.all(got[1] == 0)
        assert_scores_close("cosine", q, deq, got, ref)
        ids, scores = rt.score_topk(cands, "cosine", q, 500)
        np.testing.assert_array_equal(ids[1], np.arange(500))  # all-equal scores: pure id order


def test_pool_overflow_falls_back_to_chunks(rt):
    """Rows sorted so that every row beats all earlier ones: every row passes the filter, the candidate pool
    overflows and the pass is redone in chunks; the result must still be exact."""
    rows, cols = 900000, 128
    rng = np.random.default_rng(9)
    q = make_rows(rng, 1, cols)[0]
    x = rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(1e-4)
    x += (np.arange(rows, dtype=np.float32) / rows)[:, None] * q[None, :]
    x = f16_round(x)
    cands, deq = _bind(rt, "f16", x)
    before = rt.stats()["chunked_reruns"]
    ids, scores = rt.score_topk(cands, "dot", q, 10)
    assert_topk_matches("dot", q, deq, ids, scores, 10)
    assert rt.stats()["chunked_reruns"] == before + 1


def test_random_rows_never_need_the_chunked_rerun(rt):
    """On rows in random order the running threshold keeps the candidate pool far from overflowing: the fused
    pass must finish in its single optimistic launch (a rerun would still be exact, only slower)."""
    rows, cols = 1_500_000, 128
    rng = np.random.default_rng(123)
    codes = rng.integers(-127, 128, (rows, cols), dtype=np.int8)
    scales = np.full(rows, 0.01, np.float32)
    q = make_rows(rng, 2, cols)
    cands = rt.bind("q8", codes, scales)
    before = rt.stats()["chunked_reruns"]
    ids, scores = rt.score_topk(cands, "cosine", q, 10)
    assert rt.stats()["chunked_reruns"] == before
    model = np.stack([oracle.q8_model_scores(q[i], codes, scales, "cosine") for i in range(2)])
    np.testing.assert_array_equal(ids, oracle.topk(model, 10))
    np.testing.assert_array_equal(scores, np.take_along_axis(model, ids.astype(np.int64), 1))


# ---- errors mirror the reference's ---------------------------------------------------------------------------------
def test_error_messages(rt):
    from manta_b200.native import MantaError

    rng = np.random.default_rng(1)
    x = make_rows(rng, 10, 32)
    cands, _ = _bind(rt, "q8", x)
    q = make_rows(rng, 1, 32)[0]
    with pytest.raises(MantaError, match="topk limit 0 out of range for 10 scores"):
        rt.score_topk(cands, "cosine", q, 0)
    with pytest.raises(MantaError, match="topk limit 11 out of range for 10 scores"):
        rt.score_topk(cands, "cosine", q, 11)
    with pytest.raises(MantaError, match="score mismatch"):
        rt.score(cands, "cosine", np.zeros(16, np.float32))
    with pytest.raises(MantaError, match="gather index 10 out of range"):
        rt.gather_rows(cands, np.array([3, 10], np.int32))
    with pytest.raises(MantaError, match="gather index -1 out of range"):
        rt.gather_rows(cands, np.array([-1], np.int32))
    with pytest.raises(MantaError, match="cols % 32"):
        rt.bind("q4", np.zeros((4, 8), np.uint8), np.zeros((4, 1), np.uint16), cols=16)


def test_gather_rows_dequantises(rt):
    rng = np.random.default_rng(2)
    x = make_rows(rng, 300, 96, normalised=False)
    ids = np.array([299, 0, 17, 17, 128], np.int32)
    for layout in ("f16", "q8", "q4"):
        cands, deq = _bind(rt, layout, x, row_base=1000)
        got = rt.gather_rows(cands, ids + 1000)
        np.testing.assert_array_equal(got, oracle.gather(deq, ids))


# ---- shards -----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("layout,metric,smallest,k", [("q8", "cosine", False, 10), ("q4", "l2_distance", True, 1000),
                                                      ("f16", "dot", False, 100)])
def test_sharded_equals_unsharded(rt, layout, metric, smallest, k):
    import torch

    rows, cols, nq, shards = 40000, 256, 3, 3
    rng = np.random.default_rng(77)
    x = make_rows(rng, rows, cols, normalised=(layout != "q4"))
    q = make_rows(rng, nq, cols)
    whole, deq = _bind(rt, layout, x)
    ids_all, sc_all = rt.score_topk(whole, metric, q, k, smallest=smallest)
    bounds = [0, 9999, 27001, rows]
    lists_i, lists_s = [], []
    for s in range(shards):
        part, _ = _bind(rt, layout, x[bounds[s]:bounds[s + 1]], row_base=bounds[s])
        i, sc = rt.score_topk(part, metric, q, k, smallest=smallest)
        assert i.min() >= bounds[s] and i.max() < bounds[s + 1]
        lists_i.append(i)
        lists_s.append(sc)
    stream = torch.cuda.ExternalStream(rt.stream)
    with torch.cuda.stream(stream):
        d_i = torch.from_numpy(np.stack(lists_i)).cuda()
        d_s = torch.from_numpy(np.stack(lists_s)).cuda()
        o_i = torch.empty((nq, k), dtype=torch.int32, device="cuda")
        o_s = torch.empty((nq, k), dtype=torch.float32, device="cuda")
        rt.topk_merge_device(d_i, d_s, shards, nq, k, o_i, o_s, smallest=smallest, sync=True)
    np.testing.assert_array_equal(o_i.cpu().numpy(), ids_all)
    np.testing.assert_array_equal(o_s.cpu().numpy(), sc_all)
    assert_topk_matches(metric, q, deq, ids_all, sc_all, k, smallest)


def test_device_buffer_entry_point_and_adopt(rt):
    import torch

    rows, cols, nq, k = 50000, 768, 2, 10
    rng = np.random.default_rng(31)
    x = make_rows(rng, rows, cols)
    q = make_rows(rng, nq, cols)
    codes, scales = oracle.pack_q8_rows(x)
    deq = oracle.unpack_q8_rows(codes, scales)
    stream = torch.cuda.ExternalStream(rt.stream)
    with torch.cuda.stream(stream):
        d_codes = torch.from_numpy(codes).cuda()
        d_scales = torch.from_numpy(scales).cuda()
        d_q = torch.from_numpy(oracle.float_to_half(q).view(np.int16)).cuda()
        o_i = torch.empty((nq, k), dtype=torch.int32, device="cuda")
        o_s = torch.empty((nq, k), dtype=torch.float32, device="cuda")
    stream.synchronize()
    cands = rt.bind("q8", d_codes, d_scales, rows=rows, cols=cols)  # adopted in place
    assert cands.stored_bytes == rows * (cols + 4)
    rt.score_topk_device(cands, "cosine", d_q, nq, k, o_i, o_s, sync=False)
    rt.synchronize()
    assert_topk_matches("cosine", q, deq, o_i.cpu().numpy(), o_s.cpu().numpy(), k)
    # device-side quantiser from f16 rows gives the same codes as the oracle
    with torch.cuda.stream(stream):
        d_x = torch.from_numpy(oracle.float_to_half(x).view(np.int16)).cuda()
        c2 = torch.empty((rows, cols), dtype=torch.int8, device="cuda")
        s2 = torch.empty(rows, dtype=torch.float32, device="cuda")
    stream.synchronize()
    rt.pack_q8_rows_device(d_x, True, rows, cols, c2, s2)
    rt.synchronize()
    np.testing.assert_array_equal(c2.cpu().numpy(), codes)
    np.testing.assert_array_equal(s2.cpu().numpy(), scales)


def test_a_later_pass_never_sees_another_querys_old_threshold(rt):
    """A tensor-core pass leaves thresholds and fill counts behind for ALL its queries; a streaming pass over fewer
    queries cleans up, and a streaming pass over more queries after that must still start from a clean workspace."""
    rng = np.random.default_rng(2024)
    xf = make_rows(rng, 40000, 64)
    cf, _ = _bind(rt, "f16", xf)
    xq = make_rows(rng, 30000, 64, normalised=False)
    cq, deq = _bind(rt, "q4", xq)
    q = make_rows(rng, 3, 64)
    before = rt.stats()["mma_passes"]
    rt.score_topk(cf, "cosine", q, 7)                      # three queries over f16 rows: tensor cores, high thresholds stay behind
    assert rt.stats()["mma_passes"] == before + 1
    rt.score_topk(cq, "l2_distance", q[:1], 7, smallest=True)   # one query, streaming kernel
    ids, scores = rt.score_topk(cq, "l2_distance", q, 7, smallest=True)   # three queries, streaming kernel (q4 below eight)
    assert rt.stats()["mma_passes"] == before + 1
    assert_topk_matches("l2_distance", q, deq, ids, scores, 7, smallest=True)
