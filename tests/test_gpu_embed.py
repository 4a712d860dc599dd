"""Embedding front end on the device (gather -> matmul -> masked mean_pool / normalize) against the CPU oracle and
the reference's own fixtures, and the fused embed -> score -> top-k call against the two-step path."""
import json
import os

import numpy as np
import pytest

import oracle
from helpers import EMBED_FLOOR, assert_topk_matches, f16_round, make_rows, pack
from manta_b200 import native

pytestmark = pytest.mark.gpu

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kat.json")))


@pytest.fixture(scope="module")
def rt():
    r = native.Runtime(0)
    yield r
    r.close()


def _weights(rng, vocab, dim, out_dim):
    table = oracle.half_to_float(oracle.float_to_half(rng.normal(0, 0.02, (vocab, dim)).astype(np.float32)))
    proj = oracle.half_to_float(oracle.float_to_half(rng.normal(0, 0.05, (dim, out_dim)).astype(np.float32)))
    return table, proj


def _ragged(rng, vocab, batch, seq, lo=1):
    tokens = rng.integers(0, vocab, (batch, seq)).astype(np.int32)
    lengths = rng.integers(lo, seq + 1, batch)
    mask = (np.arange(seq)[None, :] < lengths[:, None]).astype(np.int32)
    return tokens, mask


@pytest.mark.parametrize("case", GOLD["embed"], ids=lambda c: c["source"].split()[1])
def test_embed_reference_fixtures(rt, case):
    emb = rt.bind_embedder(np.array(case["table"], np.float32), np.array(case["projection"], np.float32))
    try:
        out = rt.embed_pooled(emb, 2, np.array(case["tokens"], np.int32), np.array(case["mask"], np.int32),
                              normalize_then_pool=bool(case["order"]))
    finally:
        rt.unbind_embedder(emb)
    np.testing.assert_allclose(out, np.array(case["want"], np.float32), atol=GOLD["tolerance_abs"], rtol=0)


def _on_tensor_cores(dim, out_dim):
    """Shapes whose per-token projection runs as tcgen05 MMAs (manta_b200/csrc/embed_mma.cu::embed_mma_supported)."""
    return dim >= 64 and dim % 64 == 0 and out_dim >= 16 and out_dim % 16 == 0 and out_dim <= 512


@pytest.mark.parametrize("vocab,dim,out_dim,batch,seq", [(1000, 64, 64, 5, 9), (32000, 384, 384, 16, 128), (777, 100, 300, 3, 33),
                                                        (50, 8, 1024, 2, 4), (5000, 128, 512, 9, 77), (3000, 256, 272, 4, 200),
                                                        (900, 64, 16, 3, 130)])
@pytest.mark.parametrize("order", [0, 1])
def test_embed_matches_oracle(rt, vocab, dim, out_dim, batch, seq, order):
    rng = np.random.default_rng(vocab + out_dim + order)
    table, proj = _weights(rng, vocab, dim, out_dim)
    tokens, mask = _ragged(rng, vocab, batch, seq)
    mask[-1, :] = 0  # one all-padding row pools to zeros
    emb = rt.bind_embedder(table, proj)
    try:
        got = rt.embed_pooled(emb, out_dim, tokens, mask, normalize_then_pool=bool(order))
    finally:
        rt.unbind_embedder(emb)
    want = oracle.embed_pooled(table, proj, tokens, mask, order)
    if order == 1 and _on_tensor_cores(dim, out_dim):
        # the token rows' norms come from f16 x f16 -> f32 tensor-core products and the pool is taken on the embedding
        # rows (weights 1/norm) before one projection per batch element: sums associate differently from the oracle's
        np.testing.assert_allclose(got, want, atol=2e-6, rtol=2e-5)
    elif order == 1:
        # same f32 operation order for the products and the pooling; the sums of squares are parallel f64 reductions
        np.testing.assert_allclose(got, want, atol=3e-7, rtol=1e-6)
    else:
        # the pool is taken before the projection (it is linear): f32 sums associate differently from the oracle's
        np.testing.assert_allclose(got, want, atol=2e-6, rtol=2e-5)
    assert not got[-1].any()


def test_embed_bad_token(rt):
    rng = np.random.default_rng(3)
    table, proj = _weights(rng, 100, 16, 16)
    tokens, mask = _ragged(rng, 100, 2, 5)
    tokens[1, 4] = 100
    mask[1, 4] = 0  # masked out, still rejected like the reference's gather
    emb = rt.bind_embedder(table, proj)
    try:
        with pytest.raises(native.MantaError, match="gather index 100 out of range"):
            rt.embed_pooled(emb, 16, tokens, mask)
        tokens[1, 4] = 5
        assert np.isfinite(rt.embed_pooled(emb, 16, tokens, mask)).all()  # the runtime stays usable
    finally:
        rt.unbind_embedder(emb)


@pytest.mark.parametrize("layout", ["q8", "f16", "q4"])
@pytest.mark.parametrize("metric,batch", [("dot", 1), ("cosine", 7), ("dot", 40)])
def test_embed_score_topk(rt, layout, metric, batch):
    rng = np.random.default_rng(batch)
    vocab, dim, out_dim, seq, rows, k = 2000, 96, 128, 24, 20000, 10
    table, proj = _weights(rng, vocab, dim, out_dim)
    tokens, mask = _ragged(rng, vocab, batch, seq)
    data, scales, deq = pack(layout, make_rows(rng, rows, out_dim, normalised=(layout != "q4")))
    cands = rt.bind(layout, data, scales)
    emb = rt.bind_embedder(table, proj)
    try:
        ids, scores = rt.embed_score_topk(emb, cands, tokens, mask, metric, k)
        pooled = rt.embed_pooled(emb, out_dim, tokens, mask)
        ids2, scores2 = rt.score_topk(cands, metric, pooled, k)
    finally:
        rt.unbind_embedder(emb)
    # the fused call rounds the pooled rows to f16 on the device exactly as the host path does before its upload
    np.testing.assert_array_equal(ids, ids2)
    np.testing.assert_array_equal(scores, scores2)
    q16 = f16_round(oracle.embed_pooled(table, proj, tokens, mask, 0))
    assert_topk_matches(metric, q16, deq, ids, scores, k, floor=EMBED_FLOOR)
    cands.unbind()


def test_embed_score_topk_normalize_first_on_tensor_cores(rt):
    """mean_pool(normalize(x @ P)) with the per-token projection on the tensor cores, fused with the scoring pass."""
    rng = np.random.default_rng(77)
    vocab, dim, out_dim, batch, seq, rows, k = 2000, 128, 128, 9, 40, 20000, 10
    assert _on_tensor_cores(dim, out_dim)
    table, proj = _weights(rng, vocab, dim, out_dim)
    tokens, mask = _ragged(rng, vocab, batch, seq)
    data, scales, deq = pack("q8", make_rows(rng, rows, out_dim, normalised=True))
    cands = rt.bind("q8", data, scales)
    emb = rt.bind_embedder(table, proj)
    try:
        ids, scores = rt.embed_score_topk(emb, cands, tokens, mask, "dot", k, normalize_then_pool=True)
        pooled = rt.embed_pooled(emb, out_dim, tokens, mask, normalize_then_pool=True)
        ids2, scores2 = rt.score_topk(cands, "dot", pooled, k)
    finally:
        rt.unbind_embedder(emb)
    np.testing.assert_array_equal(ids, ids2)
    np.testing.assert_array_equal(scores, scores2)
    want = oracle.embed_pooled(table, proj, tokens, mask, 1)
    np.testing.assert_allclose(pooled, want, atol=2e-6, rtol=2e-5)
    assert_topk_matches("dot", f16_round(want), deq, ids, scores, k, floor=EMBED_FLOOR)
    cands.unbind()
