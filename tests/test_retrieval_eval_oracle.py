"""The oracle's restatement of the eval-retrieval quality computation against the reference's own test values."""
import pytest

import oracle
from retrieval_eval_cases import bounded_top_k, perfect_ranking, seeded_with_ties


@pytest.mark.parametrize("case", [perfect_ranking, bounded_top_k], ids=lambda f: f.__name__)
def test_reference_values(case):
    args, want = case()
    got = oracle.retrieval_quality(*args)
    for name, v in want.items():
        if name == "quality":
            for m, x in v.items():
                assert got["quality"][m] == pytest.approx(x, abs=1e-12), m
        else:
            assert got[name] == v, name


def test_seeded_case_counts():
    args = seeded_with_ties(n_docs=400, n_queries=10)
    got = oracle.retrieval_quality(*args)
    assert got["evaluated_queries"] == 9 and got["skipped_no_relevant"] == 1
    assert got["skipped_relevant_docs"] == 9 and got["relevant_pairs"] == 54
    assert 0 < got["quality"]["recall_at_100"] <= 1
