"""Manifest-backed serving handles over a loaded plan: the host-side mirror of the reference's ``ScoreModel``
(runtime/score_model.go:10-330 of odvcencio/manta) and ``RetrievalModel`` (runtime/retrieval_model.go:14-345): same
manifest fields and defaults, same module-contract checks with the same error texts, same result checks.  The
entry points run through ``Program.run`` — the shared-candidate forms on the fused device pass, the batched
``[Q,D] x [Q,N,D]`` forms on the per-query kernel.  Manifests are plain JSON dicts here (the reference stores them in
its MLL container, whose codec is a separate module)."""
from __future__ import annotations

from dataclasses import asdict, dataclass, fields

import numpy as np

from .program import Program, Tensor


class ServingError(ValueError):
    pass


def _find_entry(module: dict, name: str) -> dict:
    if module is None:
        raise ServingError("nil module")
    for entry in module.get("entry_points", []):
        if entry.get("name") == name:
            return entry
    raise ServingError(f'unknown entrypoint "{name}"')  # findEntryPoint, runtime/embedding_model.go:828-838


def _require_tensor_input(entry: dict, name: str, dtype: str, rank: int) -> None:
    ename = entry["name"]
    binding = next((i for i in entry.get("inputs", []) if i.get("name") == name), None)
    if binding is None:
        raise ServingError(f'entrypoint "{ename}" does not declare input "{name}"')  # requireEntryInput, :840-847
    typ = binding.get("type", {})
    if typ.get("kind") != "tensor" or not typ.get("tensor"):
        raise ServingError(f'entrypoint "{ename}" input "{name}" is not a tensor')
    if dtype and typ["tensor"].get("dtype") != dtype:
        raise ServingError(f'entrypoint "{ename}" input "{name}" dtype = "{typ["tensor"].get("dtype")}", want "{dtype}"')
    got = len(typ["tensor"].get("shape", []))
    if got != rank:
        raise ServingError(f'entrypoint "{ename}" input "{name}" rank = {got}, want {rank}')


def _single_output(entry: dict, output_name: str) -> dict:
    outs = entry.get("outputs", [])
    if len(outs) != 1:
        raise ServingError(f'entrypoint "{entry["name"]}" output count = {len(outs)}, want 1')
    if output_name and outs[0].get("name") != output_name:
        raise ServingError(f'entrypoint "{entry["name"]}" output "{outs[0].get("name")}" does not match manifest "{output_name}"')
    return outs[0]


def _stack_rows(rows, what="doc") -> np.ndarray:
    """buildDocsTable (runtime/inference.go:259-285): rank-1 rows of one width into [N, D]."""
    if len(rows) == 0:
        raise ServingError("docs table is empty")
    first = np.asarray(rows[0], np.float32)
    if first.ndim != 1:
        raise ServingError("docs must be rank-1 tensors")
    out = np.empty((len(rows), first.shape[0]), np.float32)
    for i, r in enumerate(rows):
        a = np.asarray(r, np.float32)
        if a.ndim != 1 or a.shape[0] != first.shape[0]:
            raise ServingError(f"{what} {i} shape {list(a.shape)} does not match [{first.shape[0]}]")
        out[i] = a
    return out


def _stack_batches(batches) -> np.ndarray:
    """buildDocsTableBatched: [Q][N] rank-1 rows into [Q, N, D]; every query brings the same number of rows."""
    if len(batches) == 0:
        raise ServingError("docs batches are empty")
    tables = [_stack_rows(b) for b in batches]
    for i, t in enumerate(tables):
        if t.shape != tables[0].shape:
            raise ServingError(f"docs batch {i} shape {list(t.shape)} does not match {list(tables[0].shape)}")
    return np.stack(tables)


def _from_dict(cls, d: dict):
    names = {f.name for f in fields(cls)}
    return cls(**{k: v for k, v in (d or {}).items() if k in names})


# ---- score ----------------------------------------------------------------------------------------------------
@dataclass
class ScoreManifest:
    name: str = ""
    entry: str = ""
    batch_entry: str = ""
    query_input: str = ""
    batch_query_input: str = ""
    docs_input: str = ""
    output_name: str = ""
    batch_output_name: str = ""
    query_dtype: str = ""
    docs_dtype: str = ""
    output_dtype: str = ""

    def normalized(self) -> "ScoreManifest":  # score_model.go:211-235
        m = ScoreManifest(**asdict(self))
        m.entry = m.entry or "score"
        m.query_input = m.query_input or "query"
        m.batch_query_input = m.batch_query_input or "queries"
        m.docs_input = m.docs_input or "docs"
        m.query_dtype = m.query_dtype or "f16"
        m.docs_dtype = m.docs_dtype or "q4"
        m.output_dtype = m.output_dtype or "f32"
        return m

    def validate_module(self, module: dict) -> None:  # ValidateModule + validateScoreEntry, :238-251, 276-330
        self._validate_entry(module, self.entry, self.query_input, 1, 2, self.output_name, 1)
        if self.batch_entry:
            self._validate_entry(module, self.batch_entry, self.batch_query_input, 2, 3, self.batch_output_name, 2)

    def _validate_entry(self, module, entry_name, query_input, query_rank, docs_rank, output_name, output_rank):
        entry = _find_entry(module, entry_name)
        _require_tensor_input(entry, query_input, self.query_dtype, query_rank)
        _require_tensor_input(entry, self.docs_input, self.docs_dtype, docs_rank)
        out = _single_output(entry, output_name)
        typ = out.get("type", {})
        if typ.get("kind") != "tensor" or not typ.get("tensor"):
            raise ServingError(f'entrypoint "{entry_name}" output "{out.get("name")}" is not a tensor')
        if self.output_dtype and typ["tensor"].get("dtype") != self.output_dtype:
            raise ServingError(f'entrypoint "{entry_name}" output dtype = "{typ["tensor"].get("dtype")}", want "{self.output_dtype}"')
        got = len(typ["tensor"].get("shape", []))
        if got != output_rank:
            raise ServingError(f'entrypoint "{entry_name}" output rank = {got}, want {output_rank}')


@dataclass
class ScoreResult:
    output_name: str
    scores: np.ndarray
    dtype: str
    raw: object


class ScoreModel:
    """LoadScore (score_model.go:57-68): validates the module against the manifest, then loads the plan."""

    def __init__(self, rt, module: dict, manifest=None, weights: dict | None = None):
        self.manifest = (manifest if isinstance(manifest, ScoreManifest) else _from_dict(ScoreManifest, manifest)).normalized()
        self.manifest.validate_module(module)
        self.module = module
        self.program = Program(rt, module)
        for name, tensor in (weights or {}).items():
            self.program.bind_weight(name, tensor)

    def _run(self, entry, query_name, query, docs, batched) -> ScoreResult:
        m = self.manifest
        q = np.asarray(query, np.float32)
        res = self.program.run(entry, {query_name: Tensor(m.query_dtype, list(q.shape), q),
                                       m.docs_input: Tensor(m.docs_dtype, list(docs.shape), docs)})
        if len(res.outputs) != 1:
            raise ServingError(f"score entrypoint returned {len(res.outputs)} outputs, want 1")
        name, out = next(iter(res.outputs.items()))
        want = m.batch_output_name if batched else m.output_name
        if want and name != want:  # validateScoreResult, :253-274
            raise ServingError(f'score {"batch " if batched else ""}output name "{name}" does not match manifest "{want}"')
        if out.kind != "tensor":
            raise ServingError("score output tensor is nil")
        if m.output_dtype and out.dtype != m.output_dtype:
            raise ServingError(f'score output dtype "{out.dtype}" does not match manifest "{m.output_dtype}"')
        want_rank = 2 if batched else 1
        if out.data.ndim != want_rank:
            raise ServingError(f"score output rank {out.data.ndim} does not match expected {want_rank}")
        return ScoreResult(name, out.data, out.dtype, res)

    def score(self, query, docs) -> ScoreResult:
        """query [D], docs: N rank-1 rows -> scores [N]."""
        return self._run(self.manifest.entry, self.manifest.query_input, query, _stack_rows(docs), False)

    def score_batch(self, queries, batches) -> ScoreResult:
        """queries [Q, D], batches: Q lists of N rank-1 rows -> scores [Q, N]."""
        if not self.manifest.batch_entry:
            raise ServingError("score model does not declare a batch entrypoint")
        return self._run(self.manifest.batch_entry, self.manifest.batch_query_input, queries, _stack_batches(batches), True)


# ---- retrieval --------------------------------------------------------------------------------------------------
@dataclass
class RetrievalManifest:
    name: str = ""
    entry: str = ""
    batch_entry: str = ""
    query_input: str = ""
    batch_query_input: str = ""
    docs_input: str = ""
    candidate_ids_input: str = ""
    output_name: str = ""
    batch_output_name: str = ""
    query_dtype: str = ""
    docs_dtype: str = ""
    candidate_ids_dtype: str = ""

    def normalized(self) -> "RetrievalManifest":  # retrieval_model.go:217-243
        m = RetrievalManifest(**asdict(self))
        m.entry = m.entry or "rerank_candidates_packed"
        m.query_input = m.query_input or "query"
        m.batch_query_input = m.batch_query_input or "queries"
        m.docs_input = m.docs_input or "docs"
        m.candidate_ids_input = m.candidate_ids_input or "candidate_ids"
        m.query_dtype = m.query_dtype or "f16"
        m.docs_dtype = m.docs_dtype or "q4"
        m.candidate_ids_dtype = m.candidate_ids_dtype or "i64"
        return m

    def validate_module(self, module: dict) -> None:  # ValidateModule + validateRetrievalEntry, :246-345
        self._validate_entry(module, self.entry, self.query_input, 1, 2, 1, self.output_name, 2)
        if self.batch_entry:
            self._validate_entry(module, self.batch_entry, self.batch_query_input, 2, 3, 2, self.batch_output_name, 3)

    def _validate_entry(self, module, entry_name, query_input, query_rank, docs_rank, ids_rank, output_name, output_rank):
        entry = _find_entry(module, entry_name)
        _require_tensor_input(entry, query_input, self.query_dtype, query_rank)
        _require_tensor_input(entry, self.docs_input, self.docs_dtype, docs_rank)
        _require_tensor_input(entry, self.candidate_ids_input, self.candidate_ids_dtype, ids_rank)
        out = _single_output(entry, output_name)
        typ = out.get("type", {})
        if typ.get("kind") != "candidate_pack" or not typ.get("candidate_pack"):
            raise ServingError(f'entrypoint "{entry_name}" output "{out.get("name")}" is not a candidate_pack')
        got = len(typ["candidate_pack"].get("shape", []))
        if got != output_rank:
            raise ServingError(f'entrypoint "{entry_name}" candidate_pack rank = {got}, want {output_rank}')


@dataclass
class Candidate:  # runtime/retrieval.go:12-17
    id: int
    score: float
    doc: np.ndarray


@dataclass
class CandidateResult:  # runtime/retrieval.go:32-36
    output_name: str
    batches: list
    raw: object


class RetrievalModel:
    """LoadRetrieval (retrieval_model.go:58-69)."""

    def __init__(self, rt, module: dict, manifest=None, weights: dict | None = None):
        self.manifest = (manifest if isinstance(manifest, RetrievalManifest) else _from_dict(RetrievalManifest, manifest)).normalized()
        self.manifest.validate_module(module)
        self.module = module
        self.program = Program(rt, module)
        for name, tensor in (weights or {}).items():
            self.program.bind_weight(name, tensor)

    def _run(self, entry, query_name, query, docs, ids, batched) -> CandidateResult:
        m = self.manifest
        q = np.asarray(query, np.float32)
        res = self.program.run(entry, {query_name: Tensor(m.query_dtype, list(q.shape), q),
                                       m.docs_input: Tensor(m.docs_dtype, list(docs.shape), docs),
                                       m.candidate_ids_input: Tensor(m.candidate_ids_dtype, list(ids.shape), ids)})
        if len(res.outputs) != 1:
            raise ServingError(f"retrieval entrypoint returned {len(res.outputs)} outputs, want 1")
        name, out = next(iter(res.outputs.items()))
        want = m.batch_output_name if batched else m.output_name
        if want and name != want:  # validateCandidateResult, :262-273
            raise ServingError(f'retrieval {"batch " if batched else ""}output name "{name}" does not match manifest "{want}"')
        if out.kind != "candidate_pack":
            raise ServingError("retrieval output is not a candidate_pack")
        p_ids, p_scores, p_docs = out.data["ids"], out.data["scores"], out.data["docs"]
        if not batched:
            p_ids, p_scores, p_docs = p_ids[None], p_scores[None], p_docs[None]
        batches = [[Candidate(int(p_ids[b, i]), float(p_scores[b, i]), p_docs[b, i]) for i in range(p_ids.shape[1])]
                   for b in range(p_ids.shape[0])]
        if not batches:
            raise ServingError("retrieval output has no candidate batches")
        return CandidateResult(name, batches, res)

    def retrieve(self, query, candidates) -> CandidateResult:
        """query [D]; candidates: (id, rank-1 doc row) pairs."""
        if len(candidates) == 0:
            raise ServingError("docs table is empty")
        ids = np.asarray([c[0] for c in candidates], np.int64)
        return self._run(self.manifest.entry, self.manifest.query_input, query, _stack_rows([c[1] for c in candidates]), ids, False)

    def retrieve_batch(self, queries, batches) -> CandidateResult:
        """queries [Q, D]; batches: Q lists of (id, rank-1 doc row) pairs of one length."""
        if not self.manifest.batch_entry:
            raise ServingError("retrieval model does not declare a batch entrypoint")
        docs = _stack_batches([[c[1] for c in b] for b in batches])
        ids = np.asarray([[c[0] for c in b] for b in batches], np.int64)
        return self._run(self.manifest.batch_entry, self.manifest.batch_query_input, queries, docs, ids, True)
