"""Retrieval-quality scoring on the accelerated path (``manta_b200_retrieval_quality``).

Host-side mirror of ``computeRetrievalQuality`` (runtime/retrieval_eval.go:541-584 of odvcencio/manta): document
and query vectors with their string ids, qrels as ``{query_id: {doc_id: relevance}}``; returns the quality
metrics and the counts the reference's metrics JSON takes from them.
"""
from __future__ import annotations

import ctypes
import json
from ctypes import POINTER, byref, c_char_p, c_double, c_int, c_int64, c_void_p

import numpy as np

from . import native

_configured = False


def _lib():
    global _configured
    lib = native.load()
    if not _configured:
        lib.manta_b200_retrieval_quality.argtypes = [c_void_p, c_void_p, POINTER(c_char_p), c_int, c_void_p, POINTER(c_char_p), c_int64,
                                                     c_int, POINTER(c_char_p), POINTER(c_char_p), POINTER(c_double), c_int64, c_int,
                                                     POINTER(c_void_p), POINTER(c_char_p)]
        lib.manta_b200_retrieval_quality.restype = c_int
        _configured = True
    return lib


def _strings(items):
    arr = (c_char_p * max(len(items), 1))()
    for i, s in enumerate(items):
        arr[i] = s.encode()
    return arr


def retrieval_quality(rt: "native.Runtime", query_vectors, query_ids, doc_vectors, doc_ids, qrels, top_k: int = 100) -> dict:
    _lib()
    q = np.ascontiguousarray(query_vectors, dtype=np.float32)
    d = np.ascontiguousarray(doc_vectors, dtype=np.float32)
    if d.ndim != 2 or (q.size and (q.ndim != 2 or q.shape[1] != d.shape[1])):
        raise native.MantaError(f"retrieval_quality: vectors {list(q.shape)} x {list(d.shape)} do not match")
    if len(query_ids) != q.shape[0] or len(doc_ids) != d.shape[0]:
        raise native.MantaError("retrieval_quality: one id per vector is required")
    triples = [(qi, di, float(rel)) for qi, docs in qrels.items() for di, rel in docs.items()]
    vals = (c_double * max(len(triples), 1))(*[t[2] for t in triples])
    out = c_void_p()
    native.call("manta_b200_retrieval_quality", rt.handle, native._ptr(q), _strings(list(query_ids)), c_int(q.shape[0]), native._ptr(d),
                _strings(list(doc_ids)), c_int64(d.shape[0]), c_int(d.shape[1]), _strings([t[0] for t in triples]),
                _strings([t[1] for t in triples]), vals, c_int64(len(triples)), c_int(int(top_k)), byref(out))
    try:
        return json.loads(ctypes.string_at(out.value).decode())
    finally:
        native.load().manta_b200_free_cstring(out)
