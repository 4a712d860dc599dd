"""Serving manifests without a GPU: defaults and the module-contract checks of ScoreManifest / RetrievalManifest, with
the error texts of the reference (runtime/score_model.go:211-330, runtime/retrieval_model.go:217-345; cases after
runtime/score_model_test.go:40-53)."""
import copy
import json
import os

import pytest

from manta_b200.serving import RetrievalManifest, ScoreManifest, ServingError

MODS = os.path.join(os.path.dirname(__file__), "golden", "modules")


def load(name):
    return json.load(open(os.path.join(MODS, name + ".json")))


def test_defaults():
    m = ScoreManifest().normalized()
    assert (m.entry, m.query_input, m.batch_query_input, m.docs_input) == ("score", "query", "queries", "docs")
    assert (m.query_dtype, m.docs_dtype, m.output_dtype) == ("f16", "q4", "f32")
    r = RetrievalManifest().normalized()
    assert (r.entry, r.candidate_ids_input, r.candidate_ids_dtype) == ("rerank_candidates_packed", "candidate_ids", "i64")


def test_score_manifest_accepts_the_bundle_and_names_what_is_wrong():
    bundle = load("score_bundle")
    ok = ScoreManifest(entry="score", output_name="scores", batch_entry="score_batch", batch_output_name="scores").normalized()
    ok.validate_module(bundle)
    with pytest.raises(ServingError, match='unknown entrypoint "score"'):  # TestLoadScoreValidatesManifest
        ScoreManifest().normalized().validate_module(load("tiny_rerank"))
    with pytest.raises(ServingError, match='entrypoint "score" does not declare input "q"'):
        ScoreManifest(query_input="q").normalized().validate_module(bundle)
    with pytest.raises(ServingError, match='entrypoint "score" input "docs" dtype = "q4", want "q8"'):
        ScoreManifest(docs_dtype="q8").normalized().validate_module(bundle)
    with pytest.raises(ServingError, match='entrypoint "score_batch" input "queries" rank = 2, want 1'):
        ScoreManifest(entry="score_batch", query_input="queries").normalized().validate_module(bundle)
    with pytest.raises(ServingError, match='entrypoint "score" output "scores" does not match manifest "result"'):
        ScoreManifest(output_name="result").normalized().validate_module(bundle)
    two = copy.deepcopy(bundle)
    two["entry_points"][0]["outputs"].append(two["entry_points"][0]["outputs"][0])
    with pytest.raises(ServingError, match='entrypoint "score" output count = 2, want 1'):
        ScoreManifest().normalized().validate_module(two)
    with pytest.raises(ServingError, match='entrypoint "rerank" output count = 2, want 1'):
        ScoreManifest(entry="rerank").normalized().validate_module(load("tiny_rerank") | {"entry_points": [
            dict(load("tiny_rerank")["entry_points"][0], inputs=load("score_bundle")["entry_points"][0]["inputs"])]})


def test_retrieval_manifest_checks():
    bundle = load("retrieval_bundle")
    RetrievalManifest(output_name="candidates", batch_entry="rerank_candidates_packed_batch",
                      batch_output_name="candidates").normalized().validate_module(bundle)
    with pytest.raises(ServingError, match='entrypoint "rerank_candidates" output count = 3, want 1'):
        RetrievalManifest(entry="rerank_candidates").normalized().validate_module(load("tiny_candidates"))
    with pytest.raises(ServingError, match='input "candidate_ids" rank = 2, want 1'):
        RetrievalManifest(entry="rerank_candidates_packed_batch", query_input="queries").normalized().validate_module(
            {**bundle, "entry_points": [dict(bundle["entry_points"][1], inputs=[
                dict(bundle["entry_points"][1]["inputs"][0], type={"kind": "tensor", "tensor": {"dtype": "f16", "shape": ["D"]}}),
                dict(bundle["entry_points"][1]["inputs"][1], type={"kind": "tensor", "tensor": {"dtype": "q4", "shape": ["N", "D"]}}),
                bundle["entry_points"][1]["inputs"][2]])]})
    with pytest.raises(ServingError, match='candidate_pack rank = 2, want 3'):
        RetrievalManifest(entry="rerank_candidates_packed", batch_entry="rerank_candidates_packed_batch").normalized().validate_module(
            {**bundle, "entry_points": [bundle["entry_points"][0],
                                        dict(bundle["entry_points"][1], outputs=bundle["entry_points"][0]["outputs"])]})
    score = load("score_bundle")
    with pytest.raises(ServingError, match='does not declare input "candidate_ids"'):
        RetrievalManifest(entry="score").normalized().validate_module(score)
