"""GPU parity of the tensor-core (tcgen05) pass that takes over for query batches of 8 and more on q8 and f16
candidates: same oracle, same tolerances, and for q8 the same bits as the streaming kernel (both finish the same
integer accumulators with the same epilogue)."""
import numpy as np
import pytest

import oracle
from helpers import assert_topk_matches, make_rows, pack

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    from manta_b200 import native

    r = native.Runtime(0)
    yield r
    r.close()


CASES = [  # (layout, metric, rows, cols, nq, k, smallest)
    ("q8", "cosine", 5000, 128, 8, 10, False),        # unfiltered (set smaller than the pool)
    ("q8", "cosine", 5000, 768, 33, 10, False),
    ("q8", "dot", 3000, 100, 16, 5, False),           # ragged width
    ("q8", "cosine", 120000, 128, 64, 10, False),     # filtered: observed tiles replayed at the end
    ("q8", "cosine", 100001, 256, 130, 10, False),    # two query groups, ragged last tile
    ("q8", "l2_distance", 60000, 128, 24, 100, True),
    ("q8", "dot", 70000, 384, 256, 50, False),
    ("q8", "cosine", 50000, 768, 8, 1000, False),     # large k: several observed tiles per CTA
    ("f16", "dot", 5000, 384, 64, 100, False),
    ("f16", "dot", 150000, 384, 64, 100, False),
    ("f16", "cosine", 80000, 128, 200, 10, False),
    ("f16", "l2_distance", 40000, 64, 16, 20, True),
    ("f16", "dot", 30000, 100, 9, 7, False),          # ragged width
    ("q8", "cosine", 90000, 128, 40, 10, True),       # "smallest" orders go through the pre-filter with the sign flipped
    ("f16", "dot", 90000, 96, 12, 10, True),
    ("q8", "l2_distance", 150000, 768, 130, 10, True),  # nearest neighbours, two query groups
    ("f16", "l2_distance", 120000, 384, 64, 10, False),  # farthest rows: no pre-filter, exact path throughout
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(str(v) for v in c))
def test_batched_topk_matches_oracle(rt, case):
    layout, metric, rows, cols, nq, k, smallest = case
    rng = np.random.default_rng(5000 + CASES.index(case))
    x = make_rows(rng, rows, cols)
    q = make_rows(rng, nq, cols)
    data, scales, deq = pack(layout, x)
    cands = rt.bind(layout, data, scales)
    before = rt.stats()
    ids, scores = rt.score_topk(cands, metric, q, k, smallest=smallest)
    after = rt.stats()
    assert after["mma_passes"] == before["mma_passes"] + 1, "the tensor-core pass did not run"
    assert after["chunked_reruns"] == before["chunked_reruns"]
    assert_topk_matches(metric, q, deq, ids, scores, k, smallest)
    full = rt.score(cands, metric, q)  # streaming kernel
    at = np.take_along_axis(full, ids.astype(np.int64), 1)
    if layout == "q8":
        np.testing.assert_array_equal(scores.view(np.uint32), at.view(np.uint32))
        np.testing.assert_array_equal(ids, oracle.topk(full, k, smallest))
    else:
        np.testing.assert_allclose(scores, at, rtol=2e-4, atol=2e-5)
    ids2, scores2 = rt.score_topk(cands, metric, q, k, smallest=smallest)
    np.testing.assert_array_equal(ids, ids2)
    np.testing.assert_array_equal(scores, scores2)


def test_batched_ties_resolve_to_lower_row_id(rt):
    rng = np.random.default_rng(42)
    base = make_rows(rng, 64, 128)
    x = np.tile(base, (400, 1))  # 25,600 rows, every row 400 times
    q = make_rows(rng, 16, 128)
    data, scales, deq = pack("q8", x)
    cands = rt.bind("q8", data, scales)
    ids, scores = rt.score_topk(cands, "cosine", q, 50)
    full = rt.score(cands, "cosine", q)
    np.testing.assert_array_equal(ids, oracle.topk(full, 50))
