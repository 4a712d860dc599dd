"""ctypes front end of the CPU oracle (``manta_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.  The shipped package never imports it.

Function names follow the reference's Go helpers (``dotRows`` -> ``dot_rows`` and so on); each C
function cites the reference lines it restates.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmanta_oracle.so")

METRICS = {"dot": 0, "cosine": 1, "l2_distance": 2}


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "manta_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libmanta_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.mo_half_to_float.restype = ctypes.c_float
        _lib.mo_half_to_float.argtypes = [ctypes.c_uint16]
        _lib.mo_float_to_half.restype = ctypes.c_uint16
        _lib.mo_float_to_half.argtypes = [ctypes.c_float]
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def num_threads() -> int:
    return int(lib().mo_num_threads())


def set_threads(n: int) -> None:
    lib().mo_set_threads(int(n))


def half_to_float(bits) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, dtype=np.float32)
    lib().mo_half_to_float_n(_p(bits), _p(out), ctypes.c_int64(bits.size))
    return out


def float_to_half(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().mo_float_to_half_n(_p(x), _p(out), ctypes.c_int64(x.size))
    return out


class OracleError(ValueError):
    pass


def _score(fn, query, docs):
    """Shape contract of scoreLayout (runtime/backend/tensor_ops.go:1492-1521) plus the build's
    shared-candidate batch [Q,D] x [N,D]."""
    query = _f32(query)
    docs = _f32(docs)
    if query.ndim == 1 and docs.ndim == 2:
        if query.shape[0] != docs.shape[1]:
            raise OracleError(f"score mismatch {list(query.shape)} x {list(docs.shape)}")
        batches, rows, cols, shared, oshape = 1, docs.shape[0], docs.shape[1], 1, (docs.shape[0],)
    elif query.ndim == 2 and docs.ndim == 3:
        if query.shape[0] != docs.shape[0] or query.shape[1] != docs.shape[2]:
            raise OracleError(f"score mismatch {list(query.shape)} x {list(docs.shape)}")
        batches, rows, cols, shared = query.shape[0], docs.shape[1], docs.shape[2], 0
        oshape = (batches, rows)
    elif query.ndim == 2 and docs.ndim == 2:  # build extension: shared candidates
        if query.shape[1] != docs.shape[1]:
            raise OracleError(f"score mismatch {list(query.shape)} x {list(docs.shape)}")
        batches, rows, cols, shared = query.shape[0], docs.shape[0], docs.shape[1], 1
        oshape = (batches, rows)
    else:
        raise OracleError("score expects query/docs as [D] x [N,D] or [Q,D] x [Q,N,D]")
    out = np.empty(oshape, dtype=np.float32)
    rc = fn(_p(query), _p(docs), ctypes.c_int64(batches), ctypes.c_int64(rows), ctypes.c_int64(cols),
            ctypes.c_int(shared), _p(out))
    if rc != 0:
        raise OracleError(f"oracle score failed rc={rc}")
    return out


def dot_rows(query, docs):
    return _score(lib().mo_dot_rows, query, docs)


def cosine_rows(query, docs):
    return _score(lib().mo_cosine_rows, query, docs)


def l2_distance_rows(query, docs):
    return _score(lib().mo_l2_rows, query, docs)


SCORE_FNS = {"dot": dot_rows, "cosine": cosine_rows, "l2_distance": l2_distance_rows}


def topk(scores, k: int, smallest: bool = False) -> np.ndarray:
    """topKTensor: rank-1 [N] -> i32[k]; rank-2 [Q,N] -> i32[Q,k]."""
    scores = _f32(scores)
    if scores.ndim == 1:
        rows, cols, oshape = 1, scores.shape[0], (k,)
        what = f"{cols} scores"
    elif scores.ndim == 2:
        rows, cols, oshape = scores.shape[0], scores.shape[1], (scores.shape[0], k)
        what = f"row width {cols}"
    else:
        raise OracleError("topk expects rank-1 or rank-2 scores")
    if k <= 0 or k > cols:
        raise OracleError(f"topk limit {k} out of range for {what}")
    out = np.empty(oshape, dtype=np.int32)
    rc = lib().mo_topk(_p(scores), ctypes.c_int64(rows), ctypes.c_int64(cols), ctypes.c_int(k),
                       ctypes.c_int(1 if smallest else 0), _p(out))
    if rc != 0:
        raise OracleError(f"topk limit {k} out of range for {what}")
    return out


def dot_heap_topk(query, docs, k: int):
    query = _f32(query)
    docs = _f32(docs)
    kk = k if 0 < k <= docs.shape[0] else docs.shape[0]
    ids = np.empty(kk, dtype=np.int32)
    sc = np.empty(kk, dtype=np.float32)
    lib().mo_dot_heap_topk(_p(query), _p(docs), ctypes.c_int64(docs.shape[0]), ctypes.c_int64(docs.shape[1]),
                           ctypes.c_int(k), _p(ids), _p(sc))
    return ids, sc


def gather(table, indices) -> np.ndarray:
    """gatherTensor for rank-1/rank-2 tables with rank-1 i32 indices."""
    table = np.ascontiguousarray(table)
    indices = np.ascontiguousarray(indices, dtype=np.int32)
    if indices.ndim != 1:
        raise OracleError("gather expects indices rank 1 or 2")
    if table.dtype not in (np.float32, np.int32, np.int64):
        raise OracleError("unsupported table dtype")
    rows = table.shape[0]
    cols = 1 if table.ndim == 1 else table.shape[1]
    oshape = (indices.shape[0],) if table.ndim == 1 else (indices.shape[0], cols)
    out = np.empty(oshape, dtype=table.dtype)
    bad = ctypes.c_int32(0)
    rc = lib().mo_gather_rows(_p(table), ctypes.c_int64(rows), ctypes.c_int64(cols),
                              ctypes.c_int(table.dtype.itemsize), _p(indices), ctypes.c_int64(indices.shape[0]),
                              _p(out), ctypes.byref(bad))
    if rc != 0:
        raise OracleError(f"gather index {bad.value} out of range")
    return out


def fake_quantize(data, bits: int) -> np.ndarray:
    out = _f32(data).copy()
    lib().mo_fake_quantize(_p(out), ctypes.c_int64(out.size), ctypes.c_int(bits))
    return out


def pack_q8_rows(src):
    src = _f32(src)
    rows, cols = src.shape
    codes = np.empty((rows, cols), dtype=np.int8)
    scales = np.empty(rows, dtype=np.float32)
    lib().mo_pack_q8_rows(_p(src), ctypes.c_int64(rows), ctypes.c_int64(cols), _p(codes), _p(scales))
    return codes, scales


def unpack_q8_rows(codes, scales) -> np.ndarray:
    codes = np.ascontiguousarray(codes, dtype=np.int8)
    scales = _f32(scales)
    out = np.empty(codes.shape, dtype=np.float32)
    lib().mo_unpack_q8_rows(_p(codes), _p(scales), ctypes.c_int64(codes.shape[0]), ctypes.c_int64(codes.shape[1]),
                            _p(out))
    return out


def pack_q4_b32(src):
    src = _f32(src)
    rows, cols = src.shape
    if cols % 32:
        raise OracleError("q4 block32 needs cols % 32 == 0")
    codes = np.empty((rows, cols // 2), dtype=np.uint8)
    scales = np.empty((rows, cols // 32), dtype=np.uint16)
    lib().mo_pack_q4_b32(_p(src), ctypes.c_int64(rows), ctypes.c_int64(cols), _p(codes), _p(scales))
    return codes, scales


def unpack_q4_b32(codes, scales) -> np.ndarray:
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint16)
    rows, cols = codes.shape[0], codes.shape[1] * 2
    out = np.empty((rows, cols), dtype=np.float32)
    lib().mo_unpack_q4_b32(_p(codes), _p(scales), ctypes.c_int64(rows), ctypes.c_int64(cols), _p(out))
    return out


def q8_model_scores(query, codes, scales, metric: str, want_acc: bool = False):
    """Bit-exact model of the device's packed-q8 arithmetic (two int8 query planes, int32
    accumulators, fixed f32 epilogue).  Returns scores [N] (and int32 [N,3] = I_hi, I_lo, nn)."""
    query = _f32(query)
    codes = np.ascontiguousarray(codes, dtype=np.int8)
    scales = _f32(scales)
    rows, cols = codes.shape
    out = np.empty(rows, dtype=np.float32)
    acc = np.empty((rows, 3), dtype=np.int32) if want_acc else None
    lib().mo_q8_model_scores(_p(query), _p(codes), _p(scales), ctypes.c_int64(rows), ctypes.c_int64(cols),
                             ctypes.c_int(METRICS[metric]), _p(out), _p(acc) if want_acc else None)
    return (out, acc) if want_acc else out


def score_topk(metric: str, queries, docs_f32, k: int, smallest: bool = False):
    """Oracle for the fused path: score builtin -> topKTensor -> gatherTensor(scores, ids), on a
    shared candidate matrix.  queries [Q,D] (or [D]); returns ids i32[Q,k], scores f32[Q,k]."""
    queries = _f32(queries)
    one = queries.ndim == 1
    q2 = queries[None, :] if one else queries
    scores = SCORE_FNS[metric](q2, docs_f32)
    ids = topk(scores, k, smallest)
    top = np.take_along_axis(scores, ids.astype(np.int64), axis=1)
    return (ids[0], top[0]) if one else (ids, top)


def embed_pooled(table, proj, tokens, mask, order: int = 0) -> np.ndarray:
    """gather -> matmul -> masked mean_pool / normalize in the given order (0: normalize(mean_pool(x)),
    1: mean_pool(normalize(x))); table [V,D], proj [D,E], tokens/mask i32 [B,T] -> f32 [B,E]."""
    table, proj = _f32(table), _f32(proj)
    tokens = np.ascontiguousarray(tokens, dtype=np.int32)
    mask = np.ascontiguousarray(mask, dtype=np.int32)
    b, t = tokens.shape
    out = np.empty((b, proj.shape[1]), dtype=np.float32)
    rc = lib().mo_embed_pooled(_p(table), ctypes.c_int64(table.shape[0]), ctypes.c_int64(table.shape[1]), _p(proj),
                               ctypes.c_int64(proj.shape[1]), _p(tokens), _p(mask), ctypes.c_int64(b), ctypes.c_int64(t),
                               ctypes.c_int(order), _p(out))
    if rc != 0:
        raise OracleError("gather index out of range")
    return out


def retrieval_quality(query_vectors, query_ids, doc_vectors, doc_ids, qrels, top_k: int = 100) -> dict:
    """computeRetrievalQuality + topRetrievalScores + ndcgAt / mrrAt / recallAt of the reference's eval-retrieval
    command (runtime/retrieval_eval.go:541-726), restated in Python for small cases: f32 sequential dot per
    document (:649-659), ranking by score descending then document ID string ascending (:618-626), top_k raised to
    at least 100 (:546-548) and clamped to the corpus (:587-589)."""
    import math

    q = _f32(query_vectors)
    d = _f32(doc_vectors)
    doc_set = set(doc_ids)
    top_k = max(int(top_k), 100)
    k = min(top_k, len(doc_ids)) if top_k <= len(doc_ids) else len(doc_ids)
    totals = {"ndcg_at_10": 0.0, "mrr_at_10": 0.0, "recall_at_10": 0.0, "recall_at_100": 0.0}
    evaluated = relevant_pairs = skipped_docs = skipped_queries = 0
    for qi, qid in enumerate(query_ids):
        rels = {}
        for doc_id, rel in qrels.get(qid, {}).items():
            if doc_id in doc_set:
                rels[doc_id] = float(rel)
            else:
                skipped_docs += 1
        if not rels:
            skipped_queries += 1
            continue
        scores = dot_rows(q[qi], d)  # dotRetrievalVectors: f32 sequential
        ranked = sorted(range(len(doc_ids)), key=lambda i: (-float(scores[i]), doc_ids[i]))[:k]
        ids = [doc_ids[i] for i in ranked]
        evaluated += 1
        relevant_pairs += len(rels)
        dcg = sum(rels.get(ids[i], 0.0) / math.log2(i + 2) for i in range(min(10, len(ids))) if rels.get(ids[i], 0.0) > 0)
        ideal = sorted((r for r in rels.values() if r > 0), reverse=True)[:10]
        idcg = sum(r / math.log2(i + 2) for i, r in enumerate(ideal))
        totals["ndcg_at_10"] += dcg / idcg if idcg else 0.0
        totals["mrr_at_10"] += next((1.0 / (i + 1) for i in range(min(10, len(ids))) if rels.get(ids[i], 0.0) > 0), 0.0)
        totals["recall_at_10"] += sum(1 for i in ids[:10] if rels.get(i, 0.0) > 0) / len(rels)
        totals["recall_at_100"] += sum(1 for i in ids[:100] if rels.get(i, 0.0) > 0) / len(rels)
    if evaluated:
        totals = {name: v / evaluated for name, v in totals.items()}
    return {"quality": totals, "evaluated_queries": evaluated, "relevant_pairs": relevant_pairs,
            "skipped_relevant_docs": skipped_docs, "skipped_no_relevant": skipped_queries,
            "scored_pairs": evaluated * len(doc_ids), "top_k": k}
