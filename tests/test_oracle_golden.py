"""Pins the CPU oracle against the reference's own known-answer fixtures (tests/golden/reference_kat.json,
values transcribed from the reference's Go tests) and checks the build-defined packed layouts."""
import json
import os

import numpy as np
import pytest

import oracle

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kat.json")))
TOL = GOLD["tolerance_abs"]


@pytest.mark.parametrize("case", GOLD["score"] + GOLD["direct_q4_ops"], ids=lambda c: c["op"])
def test_score_kat(case):
    out = oracle.SCORE_FNS[case["op"]](np.array(case["query"], np.float32), np.array(case["docs"], np.float32))
    assert out.shape == (len(case["want"]),)
    np.testing.assert_allclose(out, np.array(case["want"], np.float32), atol=TOL, rtol=0)


@pytest.mark.parametrize("case", GOLD["score_batched"], ids=lambda c: c["op"])
def test_score_batched_kat(case):
    out = oracle.SCORE_FNS[case["op"]](np.array(case["queries"], np.float32), np.array(case["docs"], np.float32))
    np.testing.assert_allclose(out, np.array(case["want"], np.float32), atol=TOL, rtol=0)


def test_score_shape_errors():
    with pytest.raises(oracle.OracleError, match="score expects query/docs"):
        oracle.dot_rows(np.zeros((2, 2, 2), np.float32), np.zeros((2, 2), np.float32))
    with pytest.raises(oracle.OracleError, match="score mismatch"):
        oracle.cosine_rows(np.zeros(3, np.float32), np.zeros((2, 2), np.float32))


@pytest.mark.parametrize("case", GOLD["topk"], ids=lambda c: str(c["k"]))
def test_topk_kat(case):
    out = oracle.topk(np.array(case["scores"], np.float32), case["k"])
    assert out.dtype == np.int32
    np.testing.assert_array_equal(out, np.array(case["want"], np.int32))


def test_topk_errors_and_smallest():
    s = np.array([0.25, 0.9, 0.5, 0.9], np.float32)
    with pytest.raises(oracle.OracleError, match="out of range"):
        oracle.topk(s, 0)
    with pytest.raises(oracle.OracleError, match="out of range"):
        oracle.topk(s, 5)
    np.testing.assert_array_equal(oracle.topk(s, 4), [1, 3, 2, 0])
    np.testing.assert_array_equal(oracle.topk(s, 3, smallest=True), [0, 2, 1])


@pytest.mark.parametrize("case", GOLD["gather"], ids=lambda c: c["dtype"])
def test_gather_kat(case):
    dt = {"f32": np.float32, "i32": np.int32, "i64": np.int64}[case["dtype"]]
    out = oracle.gather(np.array(case["table"], dt), np.array(case["indices"], np.int32))
    np.testing.assert_array_equal(out, np.array(case["want"], dt))
    with pytest.raises(oracle.OracleError, match="out of range"):
        oracle.gather(np.array(case["table"], dt), np.array([99], np.int32))


@pytest.mark.parametrize("case", GOLD["pipelines"], ids=lambda c: c["name"])
def test_pipeline_kat(case):
    q = np.array(case["query"], np.float32)
    docs = np.array(case["docs"], np.float32)
    ids, scores = oracle.score_topk(case["op"], q, docs, case["k"])
    np.testing.assert_array_equal(ids, case["want_ids"])
    np.testing.assert_allclose(scores, np.array(case["want_scores"], np.float32), atol=TOL, rtol=0)
    if "want_docs" in case:
        np.testing.assert_array_equal(oracle.gather(docs, ids), np.array(case["want_docs"], np.float32))
    if "candidate_ids" in case:
        got = oracle.gather(np.array(case["candidate_ids"], np.int64), ids)
        np.testing.assert_array_equal(got, case["want_candidate_ids"])


@pytest.mark.parametrize("case", GOLD["fake_quantize"], ids=lambda c: str(c["bits"]))
def test_fake_quantize_kat(case):
    data = np.array(case["data"], np.float32)
    out = oracle.fake_quantize(data, case["bits"])
    scale = np.float32(case["scale_num"]) / np.float32(case["levels"])
    want = np.array(case["want_codes"], np.float32) * scale
    np.testing.assert_array_equal(out, want)
    # the per-row q8 packing applies the same rule to one row
    codes, scales = oracle.pack_q8_rows(data[None, :])
    np.testing.assert_array_equal(codes[0], case["want_codes"])
    assert scales[0] == scale
    np.testing.assert_array_equal(oracle.unpack_q8_rows(codes, scales)[0], want)


def test_fake_quantize_half_away_from_zero_and_zero_slice():
    # 2.5/1 -> 3 (half away from zero), -2.5 -> -3; all-zero slices are left untouched
    data = np.array([127.0, 2.5, -2.5, 0.5, -0.5], np.float32)
    out = oracle.fake_quantize(data, 8)
    np.testing.assert_array_equal(out, [127.0, 3.0, -3.0, 1.0, -1.0])
    z = np.zeros(4, np.float32)
    np.testing.assert_array_equal(oracle.fake_quantize(z, 4), z)


def test_half_conversion_matches_numpy():
    bits = np.arange(0, 65536, dtype=np.uint32).astype(np.uint16)
    f = oracle.half_to_float(bits)
    ref = bits.view(np.float16).astype(np.float32)
    finite = np.isfinite(ref)
    np.testing.assert_array_equal(f[finite], ref[finite])
    assert np.all(np.isnan(f[np.isnan(ref)]))
    # f32 -> f16 RNE agrees with numpy on random values, ties and subnormals
    rng = np.random.default_rng(7)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32),
        (rng.standard_normal(50000) * 1e-6).astype(np.float32),
        (rng.standard_normal(1000) * 7e4).astype(np.float32),
        f[finite][:60000] + np.float32(0),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 2.98e-8, 2.9802325e-08, 5.96e-8], np.float32),
    ])
    mid = (f[finite][:-1].astype(np.float64) + f[finite][1:].astype(np.float64)) / 2  # exact ties
    mid = mid[np.isfinite(mid)].astype(np.float32)
    x = np.concatenate([x, mid])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    np.testing.assert_array_equal(oracle.float_to_half(x), want)


def test_q8_rows_pack_roundtrip_properties():
    rng = np.random.default_rng(11)
    x = rng.standard_normal((257, 96)).astype(np.float32)
    x[5] = 0.0
    codes, scales = oracle.pack_q8_rows(x)
    assert scales[5] == 0 and not codes[5].any()
    assert np.abs(codes.astype(np.int32)).max() == 127
    np.testing.assert_array_equal(scales, np.abs(x).max(axis=1) / np.float32(127))
    deq = oracle.unpack_q8_rows(codes, scales)
    for r in (0, 17, 256):
        np.testing.assert_array_equal(deq[r], oracle.fake_quantize(x[r], 8))
    # idempotent: re-packing the de-quantised rows gives the same codes
    c2, s2 = oracle.pack_q8_rows(deq)
    np.testing.assert_array_equal(c2, codes)


def test_q4_b32_pack_layout_and_roundtrip():
    rng = np.random.default_rng(12)
    x = rng.standard_normal((33, 64)).astype(np.float32)
    x[3, 32:] = 0.0
    codes, scales = oracle.pack_q4_b32(x)
    assert codes.shape == (33, 32) and scales.shape == (33, 2)
    assert scales[3, 1] == 0 and not codes[3, 16:].any()
    deq = oracle.unpack_q4_b32(codes, scales)
    # nibble order: element 2j in the low nibble of byte j, two's complement
    lo = (codes & 0x0F).astype(np.int8)
    hi = (codes >> 4).astype(np.int8)
    lo = np.where(lo >= 8, lo - 16, lo)
    hi = np.where(hi >= 8, hi - 16, hi)
    n = np.empty((33, 64), np.int8)
    n[:, 0::2] = lo
    n[:, 1::2] = hi
    assert np.abs(n).max() == 7
    sc = scales.view(np.float16).astype(np.float32)
    np.testing.assert_array_equal(deq, n.astype(np.float32) * np.repeat(sc, 32, axis=1))
    # error bound: half a step of the (f16-rounded) block scale, plus clamp slack from rounding the scale down
    step = np.repeat(sc, 32, axis=1)
    assert np.all(np.abs(deq - x) <= 0.5 * step + np.abs(x) * 2e-3 + 1e-12)
    with pytest.raises(oracle.OracleError):
        oracle.pack_q4_b32(np.zeros((2, 48), np.float32))


def test_q8_model_close_to_reference_float_path():
    """The packed-int arithmetic the device uses stays within 1e-3 relative (with the floor the score
    scale gives) of the reference's float path on de-quantised rows."""
    rng = np.random.default_rng(13)
    d = 768
    x = rng.standard_normal((2000, d))
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    x = oracle.half_to_float(oracle.float_to_half(x.astype(np.float32)))
    q = rng.standard_normal(d)
    q = oracle.half_to_float(oracle.float_to_half((q / np.linalg.norm(q)).astype(np.float32)))
    codes, scales = oracle.pack_q8_rows(x)
    deq = oracle.unpack_q8_rows(codes, scales)
    for metric in ("dot", "cosine", "l2_distance"):
        ref = oracle.SCORE_FNS[metric](q, deq)
        got, acc = oracle.q8_model_scores(q, codes, scales, metric, want_acc=True)
        # 1e-3 relative down to scores of 5e-2*|q||d| (|q||d| = 1 here); below that the bound is the
        # absolute 5e-5*|q||d|, 10x tighter than the reference's own 5e-4 absolute test tolerance
        floor = 5e-2
        err = np.abs(got - ref) / np.maximum(np.maximum(np.abs(got), np.abs(ref)), floor)
        assert err.max() < 1e-3, (metric, err.max())
        np.testing.assert_array_equal(acc[:, 2], (codes.astype(np.int32) ** 2).sum(axis=1))


@pytest.mark.parametrize("case", GOLD["embed"], ids=lambda c: c["source"].split()[1])
def test_embed_pooled_kat(case):
    out = oracle.embed_pooled(np.array(case["table"], np.float32), np.array(case["projection"], np.float32),
                              np.array(case["tokens"], np.int32), np.array(case["mask"], np.int32), case["order"])
    np.testing.assert_allclose(out, np.array(case["want"], np.float32), atol=TOL, rtol=0)


def test_embed_pooled_against_numpy():
    rng = np.random.default_rng(5)
    table = oracle.half_to_float(oracle.float_to_half(rng.normal(0, 0.02, (500, 48)).astype(np.float32)))
    proj = oracle.half_to_float(oracle.float_to_half(rng.normal(0, 0.05, (48, 40)).astype(np.float32)))
    tokens = rng.integers(0, 500, (6, 17)).astype(np.int32)
    lengths = np.array([17, 1, 9, 0, 16, 3])
    mask = (np.arange(17)[None, :] < lengths[:, None]).astype(np.int32)
    x = table[tokens].astype(np.float64) @ proj.astype(np.float64)
    m = mask[:, :, None].astype(np.float64)
    cnt = np.maximum(lengths, 1)[:, None]
    pooled = (x * m).sum(1) / cnt
    n = np.linalg.norm(pooled, axis=1, keepdims=True)
    want0 = np.where(n > 0, pooled / np.where(n > 0, n, 1), pooled)
    xn = x / np.linalg.norm(x, axis=2, keepdims=True)
    want1 = (xn * m).sum(1) / cnt
    np.testing.assert_allclose(oracle.embed_pooled(table, proj, tokens, mask, 0), want0, atol=2e-6)
    np.testing.assert_allclose(oracle.embed_pooled(table, proj, tokens, mask, 1), want1, atol=2e-6)
    assert not oracle.embed_pooled(table, proj, tokens, mask, 0)[3].any()  # an all-masked row pools to zeros
    bad = tokens.copy()
    bad[0, 0] = 500
    with pytest.raises(oracle.OracleError, match="out of range"):
        oracle.embed_pooled(table, proj, bad, mask, 0)
