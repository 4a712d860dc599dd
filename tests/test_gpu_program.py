"""End-to-end runs of the host executor on the GPU, written after the reference's own runtime tests
(runtime/runtime_test.go:483-678, 928-963, 1143-1184, 1356-1419 of odvcencio/manta): same tiny fixtures, same
outputs, producers, trace and metadata keys."""
import json
import os

import numpy as np
import pytest

import oracle
from helpers import assert_topk_matches, make_rows

pytestmark = pytest.mark.gpu

MODS = os.path.join(os.path.dirname(__file__), "golden", "modules")
TOL = 5e-4  # the reference's tolerance for these fixtures


def load(name):
    return json.load(open(os.path.join(MODS, name + ".json")))


@pytest.fixture(scope="module")
def rt():
    from manta_b200 import native

    r = native.Runtime(0)
    yield r
    r.close()


def T(*a):
    from manta_b200.program import Tensor

    return Tensor(*a)


def tiny_rerank_weights(prog):
    prog.bind_weight("docs", T("q4", [3, 2], [1, 0, 0, 1, 1, 1]))  # tinyRerankWeights, runtime_test.go:1585-1593


def test_run_tiny_score_entry_point(rt):
    from manta_b200.program import Program

    prog = Program(rt, load("tiny_score"))
    prog.bind_weight("docs", T("q4", [2, 2], [1, 0, 0, 1]))  # tinyScoreWeights
    res = prog.run("score", {"query": T("f16", [2], [1, 0])})
    out = res.outputs["scores"]
    assert out.producer == "kernel:cosine"
    assert out.kind == "tensor" and out.dtype == "f32"
    np.testing.assert_allclose(out.data, [1, 0], atol=TOL)
    assert out.metadata["variant_entry"] == "cosine_cuda"
    assert out.metadata["device_execution"] is True
    assert res.metadata["compiled_kernels"] == "1"
    assert res.metadata["entrypoint"] == "score"


def test_run_tiny_rerank_entry_point(rt):
    from manta_b200.program import Program

    prog = Program(rt, load("tiny_rerank"))
    tiny_rerank_weights(prog)
    res = prog.run("rerank", {"query": T("f16", [2], [1, 0])})
    assert res.outputs["top_ids"].producer == "topk:topk"
    np.testing.assert_array_equal(res.outputs["top_ids"].data, [0, 2])
    assert res.outputs["top_ids"].data.dtype == np.int32
    assert res.outputs["top_scores"].producer == "gather:gather"
    np.testing.assert_allclose(res.outputs["top_scores"].data, [1, 0.70710677], atol=TOL)
    assert res.metadata["entrypoint"] == "rerank"
    assert len(res.trace) == 4
    assert res.trace[1]["kind"] == "topk" and res.trace[2]["kind"] == "gather"
    assert res.trace[0]["variant"] == "cosine_cuda"
    assert res.metadata["fused_passes"] == "1"


def test_run_tiny_select_and_retrieve(rt):
    from manta_b200.program import Program

    prog = Program(rt, load("tiny_select"))
    tiny_rerank_weights(prog)
    res = prog.run("select_scores", {"query": T("f16", [2], [1, 0])})
    assert res.outputs["top_scores"].producer == "gather:gather"
    np.testing.assert_allclose(res.outputs["top_scores"].data, [1, 0.70710677], atol=TOL)
    assert len(res.trace) == 4 and res.trace[2]["kind"] == "gather"

    prog = Program(rt, load("tiny_retrieve"))
    tiny_rerank_weights(prog)
    res = prog.run("retrieve", {"query": T("f16", [2], [1, 0])})
    np.testing.assert_array_equal(res.outputs["top_ids"].data, [0, 2])
    np.testing.assert_allclose(res.outputs["top_scores"].data, [1, 0.70710677], atol=TOL)
    np.testing.assert_allclose(res.outputs["top_docs"].data, [[1, 0], [1, 1]], atol=TOL)
    assert res.outputs["top_docs"].dtype == "q4"
    assert len(res.trace) == 5 and res.trace[3]["kind"] == "gather"
    # a second run reuses the resident candidate set
    res2 = prog.run("retrieve", {"query": T("f16", [2], [0, 1])})
    np.testing.assert_array_equal(res2.outputs["top_ids"].data, [1, 2])


def test_run_tiny_candidates_and_packed(rt):
    from manta_b200.program import Program

    inputs = {"query": T("f16", [2], [1, 0]), "docs": T("q4", [3, 2], [1, 0, 0, 1, 1, 1]),
              "candidate_ids": T("i64", [3], [1001, 2002, 3003])}
    res = Program(rt, load("tiny_candidates")).run("rerank_candidates", inputs)
    np.testing.assert_array_equal(res.outputs["top_candidate_ids"].data, [1001, 3003])
    assert res.outputs["top_candidate_ids"].data.dtype == np.int64
    np.testing.assert_allclose(res.outputs["top_scores"].data, [1, 0.70710677], atol=TOL)
    np.testing.assert_allclose(res.outputs["top_docs"].data, [[1, 0], [1, 1]], atol=TOL)
    assert res.outputs["top_docs"].dtype == "q4"

    res = Program(rt, load("tiny_packed_candidates")).run("rerank_candidates_packed", inputs)
    out = res.outputs["candidates"]
    assert out.kind == "candidate_pack"
    np.testing.assert_array_equal(out.data["ids"], [1001, 3003])
    np.testing.assert_allclose(out.data["scores"], [1, 0.70710677], atol=TOL)
    np.testing.assert_allclose(out.data["docs"], [[1, 0], [1, 1]], atol=TOL)
    assert out.data["docs_dtype"] == "q4"


@pytest.mark.parametrize("op,want", [("dot", [1, 0, 1]), ("cosine", [1, 0, 0.70710677]), ("l2_distance", [0, 1.4142135, 1])])
def test_run_direct_quantized_builtin_score_ops(rt, op, want):
    from manta_b200.program import Program

    res = Program(rt, load("direct_" + op)).run("score", {"query": T("f16", [2], [1, 0]), "docs": T("q4", [3, 2], [1, 0, 0, 1, 1, 1])})
    out = res.outputs["scores"]
    assert out.producer == "kernel:" + op
    np.testing.assert_allclose(out.data, want, atol=TOL)
    assert out.metadata["device_execution"] is True


def test_request_validation_errors(rt):
    from manta_b200.program import MantaError, Program

    prog = Program(rt, load("tiny_rerank"))
    with pytest.raises(MantaError, match='missing weight binding for param "docs"'):
        prog.run("rerank", {"query": T("f16", [2], [1, 0])})
    tiny_rerank_weights(prog)
    with pytest.raises(MantaError, match='unknown entrypoint "nope"'):
        prog.run("nope", {})
    with pytest.raises(MantaError, match='entrypoint "rerank" missing input "query"'):
        prog.run("rerank", {})
    with pytest.raises(MantaError, match='entrypoint "rerank" does not declare input "extra"'):
        prog.run("rerank", {"query": T("f16", [2], [1, 0]), "extra": T("f16", [2], [1, 0])})
    with pytest.raises(MantaError, match='symbol "D" mismatch: expected 2, got 3'):
        prog.run("rerank", {"query": T("f16", [3], [1, 0, 0])})
    with pytest.raises(MantaError, match="tensor rank 2 does not match expected rank 1"):
        prog.run("rerank", {"query": T("f16", [1, 2], [1, 0])})
    with pytest.raises(MantaError, match='tensor dtype "i32" does not match expected "f16"'):
        prog.run("rerank", {"query": T("i32", [2], [1, 0])})
    # f32-labelled data is accepted where f16 is expected (runtime/backend/tensor.go:392-395)
    res = prog.run("rerank", {"query": T("f32", [2], [1, 0])})
    np.testing.assert_array_equal(res.outputs["top_ids"].data, [0, 2])
    # k larger than the candidate count is topKTensor's error, reported on the topk step
    mod = load("tiny_rerank")
    mod["steps"][1]["attributes"]["k"] = "5"
    prog5 = Program(rt, mod)
    tiny_rerank_weights(prog5)
    with pytest.raises(MantaError, match='step "topk": topk limit 5 out of range for 3 scores'):
        prog5.run("rerank", {"query": T("f16", [2], [1, 0])})


def test_rerank_at_size_against_oracle(rt):
    """The same plan on a real-sized q8 parameter and a query batch (shared-candidate extension)."""
    from manta_b200.program import Program

    rows, cols, nq, k = 30000, 128, 3, 10
    rng = np.random.default_rng(8)
    x = make_rows(rng, rows, cols)
    q = make_rows(rng, nq, cols)
    mod = load("tiny_rerank")
    mod["params"][0]["type"]["tensor"]["dtype"] = "q8"
    mod["kernels"][0]["inputs"][1]["type"]["tensor"]["dtype"] = "q8"
    mod["entry_points"][0]["inputs"][0]["type"]["tensor"]["shape"] = ["Q", "D"]
    mod["entry_points"][0]["outputs"][0]["type"]["tensor"]["shape"] = ["Q", str(k)]
    mod["entry_points"][0]["outputs"][1]["type"]["tensor"]["shape"] = ["Q", str(k)]
    mod["steps"][1]["attributes"]["k"] = str(k)
    prog = Program(rt, mod)
    prog.bind_weight("docs", T("q8", [rows, cols], x))
    res = prog.run("rerank", {"query": T("f16", [nq, cols], q)})
    deq = oracle.unpack_q8_rows(*oracle.pack_q8_rows(x))
    assert_topk_matches("cosine", q, deq, res.outputs["top_ids"].data, res.outputs["top_scores"].data, k)


def test_memory_plan_residency_is_honoured(rt):
    """A param the plan does not keep device_resident is bound for the run and released afterwards; results are
    the same (the reference's lazy_staged behaviour, runtime/runtime_test.go:223-271)."""
    from manta_b200.program import Program

    prog = Program(rt, load("tiny_retrieve"))
    tiny_rerank_weights(prog)
    plan = prog.memory_plan(1)  # nothing fits; docs is read by two steps (score, gather) -> host_pinned
    assert plan["weights"][0]["residency"] == "host_pinned" and plan["weights"][0]["access_count"] == 2
    prog.apply_memory_plan(plan)
    binds0 = rt.stats()["bind_calls"]
    for _ in range(2):
        res = prog.run("retrieve", {"query": T("f16", [2], [1, 0])})
        np.testing.assert_array_equal(res.outputs["top_ids"].data, [0, 2])
        np.testing.assert_allclose(res.outputs["top_docs"].data, [[1, 0], [1, 1]], atol=TOL)
        assert res.metadata["params_released"] == "1"
    assert rt.stats()["bind_calls"] == binds0 + 2
    prog.apply_memory_plan(prog.memory_plan())  # unbudgeted: resident again
    binds1 = rt.stats()["bind_calls"]
    for _ in range(2):
        res = prog.run("retrieve", {"query": T("f16", [2], [1, 0])})
        assert res.metadata["params_released"] == "0"
    assert rt.stats()["bind_calls"] == binds1 + 1


# ---- per-query candidate sets [Q,D] x [Q,N,D] -----------------------------------------------------------------
BATCH_Q = [1, 0, 0, 1]
BATCH_DOCS = [1, 0, 0, 1, 1, 1, 0, 1, 1, 0, 1, 1]


def test_score_bundle_score_batch(rt):
    # TestScoreModelScoreBatch, runtime/score_model_test.go:86-131
    from manta_b200.program import Program

    prog = Program(rt, load("score_bundle"))
    res = prog.run("score_batch", {"queries": T("f16", [2, 2], BATCH_Q), "docs": T("q4", [2, 3, 2], BATCH_DOCS)})
    out = res.outputs["scores"]
    assert out.producer == "kernel:cosine_batch" and out.dtype == "f32"
    assert list(out.data.shape) == [2, 3]
    np.testing.assert_allclose(out.data, [[1, 0, 0.70710677], [1, 0, 0.70710677]], atol=TOL)
    assert out.metadata["device_execution"] is True and out.metadata["candidate_sets"] == "per_query"
    # the rank-1 entry of the same bundle still runs
    res = prog.run("score", {"query": T("f16", [2], [1, 0]), "docs": T("q4", [2, 2], [1, 0, 0, 1])})
    np.testing.assert_allclose(res.outputs["scores"].data, [1, 0], atol=TOL)


def test_retrieval_bundle_packed_batch(rt):
    # TestRetrievalModelRetrieveBatch, runtime/retrieval_model_test.go:94-150
    from manta_b200.program import Program

    prog = Program(rt, load("retrieval_bundle"))
    res = prog.run("rerank_candidates_packed_batch", {
        "queries": T("f16", [2, 2], BATCH_Q), "docs": T("q4", [2, 3, 2], BATCH_DOCS),
        "candidate_ids": T("i64", [2, 3], [1001, 2002, 3003, 4004, 5005, 6006])})
    out = res.outputs["candidates"]
    assert out.kind == "candidate_pack"
    np.testing.assert_array_equal(out.data["ids"], [[1001, 3003], [4004, 6006]])
    np.testing.assert_allclose(out.data["scores"], [[1, 0.70710677], [1, 0.70710677]], atol=TOL)
    np.testing.assert_allclose(out.data["docs"], [[[1, 0], [1, 1]], [[0, 1], [1, 1]]], atol=TOL)
    assert res.metadata["fused_passes"] == "1"
    # the symbol Q is bound by the first input that carries it (symbolic.go:265-277)
    with pytest.raises(Exception, match='symbol "Q" mismatch: expected 3, got 2'):
        prog.run("rerank_candidates_packed_batch", {
            "queries": T("f16", [3, 2], [1, 0, 0, 1, 1, 1]), "docs": T("q4", [2, 3, 2], BATCH_DOCS),
            "candidate_ids": T("i64", [2, 3], [1, 2, 3, 4, 5, 6])})


@pytest.mark.parametrize("metric", ["dot", "cosine", "l2_distance"])
@pytest.mark.parametrize("shape", [(1, 1, 1), (3, 50, 7), (5, 300, 64), (16, 1000, 384), (2, 20000, 128)])
def test_batched_abi_matches_oracle(rt, metric, shape):
    nq, rows, cols = shape
    rng = np.random.default_rng(nq * 1000 + rows + cols)
    q = make_rows(rng, nq, cols)
    docs = make_rows(rng, nq * rows, cols, normalised=False).reshape(nq, rows, cols)
    docs[0, 0] = 0  # a zero row: cosine is exactly 0
    got = rt.score_batched(metric, q, docs)
    want = oracle.SCORE_FNS[metric](q, docs)
    np.testing.assert_allclose(got, want, rtol=2e-6, atol=2e-6 * np.abs(want).max())
    if metric == "cosine":
        assert got[0, 0] == 0.0
    k = min(10, rows)
    for smallest in (False, True):
        ids, sc = rt.score_topk_batched(metric, q, docs, k, smallest=smallest)
        for i in range(nq):
            ref_ids = oracle.topk(got[i], k, smallest)  # selection rule on the device's own scores: bit-exact
            np.testing.assert_array_equal(ids[i], ref_ids)
            np.testing.assert_array_equal(sc[i], got[i][ref_ids])


def test_batched_abi_errors(rt):
    from manta_b200 import native

    q = np.zeros((2, 4), np.float32)
    with pytest.raises(native.MantaError, match="score expects query/docs"):
        rt.score_batched("dot", q, np.zeros((3, 4), np.float32))
    with pytest.raises(native.MantaError, match="score mismatch"):
        rt.score_batched("dot", q, np.zeros((2, 3, 5), np.float32))
    with pytest.raises(native.MantaError, match="topk limit 4 out of range for row width 3"):
        rt.score_topk_batched("dot", q, np.zeros((2, 3, 4), np.float32), 4)


# ---- manifest-backed serving handles ------------------------------------------------------------------------------
def test_score_model_score_and_score_batch(rt):
    # TestScoreModelScore / TestScoreModelScoreBatch, runtime/score_model_test.go:55-131
    from manta_b200.serving import ScoreManifest, ScoreModel, ServingError

    model = ScoreModel(rt, load("score_bundle"), ScoreManifest(name="score_bundle", entry="score", output_name="scores",
                                                               batch_entry="score_batch", batch_output_name="scores"))
    res = model.score([1, 0], [[1, 0], [0, 1]])
    assert res.output_name == "scores" and res.dtype == "f32"
    np.testing.assert_allclose(res.scores, [1, 0], atol=TOL)
    res = model.score_batch([[1, 0], [0, 1]], [[[1, 0], [0, 1], [1, 1]], [[0, 1], [1, 0], [1, 1]]])
    np.testing.assert_allclose(res.scores, [[1, 0, 0.70710677], [1, 0, 0.70710677]], atol=TOL)
    with pytest.raises(ServingError, match="doc 1 shape"):
        model.score([1, 0], [[1, 0], [0, 1, 2]])
    single = ScoreModel(rt, load("score_bundle"), {"entry": "score"})
    with pytest.raises(ServingError, match="does not declare a batch entrypoint"):
        single.score_batch([[1, 0]], [[[1, 0]]])
    with pytest.raises(ServingError, match='unknown entrypoint "score"'):  # TestLoadScoreValidatesManifest
        ScoreModel(rt, load("tiny_rerank"), {})


def test_retrieval_model_retrieve_and_retrieve_batch(rt):
    # TestRetrievalModelRetrieve / RetrieveBatch, runtime/retrieval_model_test.go:55-150
    from manta_b200.serving import RetrievalManifest, RetrievalModel

    model = RetrievalModel(rt, load("retrieval_bundle"), RetrievalManifest(
        name="retrieval_bundle", output_name="candidates", batch_entry="rerank_candidates_packed_batch", batch_output_name="candidates"))
    res = model.retrieve([1, 0], [(1001, [1, 0]), (2002, [0, 1]), (3003, [1, 1])])
    assert len(res.batches) == 1
    assert [c.id for c in res.batches[0]] == [1001, 3003]
    np.testing.assert_allclose([c.score for c in res.batches[0]], [1, 0.70710677], atol=TOL)
    np.testing.assert_allclose(res.batches[0][1].doc, [1, 1], atol=TOL)
    res = model.retrieve_batch([[1, 0], [0, 1]], [[(1001, [1, 0]), (2002, [0, 1]), (3003, [1, 1])],
                                                  [(4004, [0, 1]), (5005, [1, 0]), (6006, [1, 1])]])
    assert len(res.batches) == 2
    assert res.batches[1][0].id == 4004
    assert [c.id for c in res.batches[0]] == [1001, 3003]


def test_dequant_step_keeps_docs_packed(rt):
    """score(query, dequant(docs_q)) (StepDequant, runtime/backend/tensor_ops.go:136-148: a clone relabelled f16): the
    fused pass binds docs_q itself, packed by its own label, and the result equals the plan without the dequant step."""
    import hashlib

    from manta_b200.program import Program

    rng = np.random.default_rng(77)
    x = make_rows(rng, 3000, 64)
    deq = oracle.unpack_q8_rows(*oracle.pack_q8_rows(x))  # what a q8-labelled float32 tensor of the reference holds
    q = make_rows(rng, 1, 64)[0]
    mod = load("dequant_rerank")
    prog = Program(rt, mod)
    prog.bind_weight("docs_q", T("q8", list(deq.shape), deq))
    res = prog.run("rerank", {"query": T("f16", [64], q)})
    assert [t["kind"] for t in res.trace] == ["dequant", "launch_kernel", "topk", "gather", "return"]
    ids, scores = res.outputs["top_ids"].data, res.outputs["top_scores"].data
    assert_topk_matches("cosine", q, deq, ids, scores, 2)
    plain_mod = load("tiny_rerank")
    plain_mod["params"][0]["type"]["tensor"]["dtype"] = "q8"
    plain = Program(rt, plain_mod)
    plain.bind_weight("docs", T("q8", list(deq.shape), deq))
    res2 = plain.run("rerank", {"query": T("f16", [64], q)})
    np.testing.assert_array_equal(ids, res2.outputs["top_ids"].data)
    np.testing.assert_array_equal(scores.view(np.uint32), res2.outputs["top_scores"].data.view(np.uint32))
    # CompileVariants' source hash (runtime/backend/backend.go:286-293) and the launch configuration of the kernel
    # that really ran, beside the plan-side keys of nativeLaunchConfig (runtime/backend/native_kernel.go:65-112)
    mod2 = load("tiny_score")
    prog = Program(rt, mod2)
    prog.bind_weight("docs", T("q4", [2, 2], [1, 0, 0, 1]))
    md = prog.run("score", {"query": T("f16", [2], [1, 0])}).outputs["scores"].metadata
    src = [v for v in mod2["kernels"][0]["variants"] if v["backend"] == "cuda"][0]["source"]
    assert md["source_hash"] == hashlib.sha256(src.encode()).hexdigest()
    assert md["dispatch_mode"] == "backend_native" and md["dispatch_backend"] == "cuda" and md["launch_entry"] == "cosine_cuda"
    assert md["launch_tile"] == "[128]" and md["launch_vector_width"] == "4" and md["launch_memory"] == "workgroup_local"
    assert md["plan_block_size"] == 128 and md["plan_shared_bytes"] == 128 * 4 * 3 * 4  # estimatedSharedBytes
    assert md["launch_grid"] == "1d" and md["launch_kernel"].endswith("_kernel")
    assert md["launch_block_size"] >= 32 and md["launch_grid_size"] >= 1 and md["launch_count"] >= 1
