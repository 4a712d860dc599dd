"""Inputs of the reference's retrieval-quality tests (runtime/retrieval_eval_test.go:16-72 of odvcencio/manta) and a
seeded case with exact score ties, shared by the oracle test and the GPU test."""
import numpy as np


def normalize(v):
    v = np.asarray(v, np.float32)
    s = float(np.sum(v.astype(np.float64) ** 2))
    return v if s == 0 else v * np.float32(1 / np.sqrt(s))


def perfect_ranking():
    # TestComputeRetrievalQualityPerfectRanking
    queries = np.stack([normalize([1, 0]), normalize([0, 1])])
    docs = np.stack([normalize([1, 0]), normalize([0, 1]), normalize([0.2, 0.1])])
    qrels = {"q1": {"d1": 1}, "q2": {"d2": 1}}
    want = {"quality": {"ndcg_at_10": 1, "mrr_at_10": 1, "recall_at_10": 1, "recall_at_100": 1}, "evaluated_queries": 2,
            "relevant_pairs": 2, "skipped_relevant_docs": 0, "skipped_no_relevant": 0}
    return (queries, ["q1", "q2"], docs, ["d1", "d2", "d3"], qrels, 100), want


def bounded_top_k():
    # TestComputeRetrievalQualityUsesBoundedTopK: 120 docs, score 200 - i, relevant d000 d009 d099 d100
    queries = np.array([[1]], np.float32)
    docs = np.array([[200 - i] for i in range(120)], np.float32)
    ids = ["d%03d" % i for i in range(120)]
    qrels = {"q": {"d000": 1, "d009": 1, "d099": 1, "d100": 1}}
    want = {"quality": {"mrr_at_10": 1, "recall_at_10": 0.5, "recall_at_100": 0.75}, "evaluated_queries": 1, "relevant_pairs": 4,
            "skipped_relevant_docs": 0, "skipped_no_relevant": 0}
    return (queries, ["q"], docs, ids, qrels, 100), want


def seeded_with_ties(n_docs=3000, n_queries=37, dim=32, seed=11):
    """f16-representable small-integer vectors, so every dot product is exact in any summation order and many
    documents tie; document ids are shuffled strings, so the ID tie-break differs from the row order."""
    rng = np.random.default_rng(seed)
    docs = rng.integers(-2, 3, (n_docs, dim)).astype(np.float32)
    queries = rng.integers(-2, 3, (n_queries, dim)).astype(np.float32)
    perm = rng.permutation(n_docs)
    doc_ids = ["doc-%05d" % p for p in perm]
    query_ids = ["query-%d" % i for i in range(n_queries)]
    qrels = {}
    for i, qid in enumerate(query_ids):
        if i % 9 == 8:
            continue  # a query without judgements
        best = np.argsort(-(docs @ queries[i]))[:40]
        picks = rng.choice(best, 6, replace=False)
        qrels[qid] = {doc_ids[int(p)]: int(rng.integers(1, 4)) for p in picks}
        qrels[qid]["missing-doc-%d" % i] = 1  # not in the corpus: counted as skipped
    qrels["query-unknown"] = {doc_ids[0]: 1}
    return (queries, query_ids, docs, doc_ids, qrels, 100)
