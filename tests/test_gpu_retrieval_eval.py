"""manta_b200_retrieval_quality (device score + top-k, host metrics) against the oracle's restatement of
computeRetrievalQuality and the reference's own test values."""
import numpy as np
import pytest

import oracle
from retrieval_eval_cases import bounded_top_k, perfect_ranking, seeded_with_ties

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    from manta_b200 import native

    r = native.Runtime(0)
    yield r
    r.close()


@pytest.mark.parametrize("case", [perfect_ranking, bounded_top_k], ids=lambda f: f.__name__)
def test_reference_values(rt, case):
    from manta_b200.retrieval_eval import retrieval_quality

    args, want = case()
    got = retrieval_quality(rt, *args)
    for name, v in want.items():
        if name == "quality":
            for m, x in v.items():
                assert got["quality"][m] == pytest.approx(x, abs=1e-12), m
        else:
            assert got[name] == v, name


@pytest.mark.parametrize("top_k", [100, 250])
def test_matches_oracle_with_ties(rt, top_k):
    from manta_b200.retrieval_eval import retrieval_quality

    args = seeded_with_ties()
    got = retrieval_quality(rt, *args[:5], top_k)
    want = oracle.retrieval_quality(*args[:5], top_k)
    for name in ("evaluated_queries", "relevant_pairs", "skipped_relevant_docs", "skipped_no_relevant", "scored_pairs", "top_k"):
        assert got[name] == want[name], name
    for m, x in want["quality"].items():
        # exact small-integer scores: the rankings, ties included, are identical, so the metrics agree to rounding
        assert got["quality"][m] == pytest.approx(x, abs=1e-12), m


def test_small_corpus_and_errors(rt):
    from manta_b200 import native
    from manta_b200.retrieval_eval import retrieval_quality

    docs = np.eye(3, dtype=np.float32)
    got = retrieval_quality(rt, docs[:1], ["q"], docs, ["b", "a", "c"], {"q": {"b": 2}}, 100)
    assert got["top_k"] == 3 and got["quality"]["mrr_at_10"] == 1.0
    with pytest.raises(native.MantaError, match="do not match"):
        retrieval_quality(rt, np.zeros((1, 2), np.float32), ["q"], docs, ["a", "b", "c"], {}, 100)
