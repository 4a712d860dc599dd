"""Host executor without a GPU: Module JSON parsing / validation errors and the fusion pre-pass over the step list
(which steps run as one device pass)."""
import json
import os

import pytest

from manta_b200.program import MantaError, Program

MODS = os.path.join(os.path.dirname(__file__), "golden", "modules")


def load(name):
    return json.load(open(os.path.join(MODS, name + ".json")))


def test_rerank_plan_fuses_score_topk_gather():
    prog = Program(None, load("tiny_rerank"))
    plan = prog.plan("rerank")
    assert [s["kind"] for s in plan] == ["launch_kernel", "topk", "gather", "return"]
    assert [s["execution"] for s in plan] == ["fused_pass", "fused_with_score", "fused_with_score", "host"]


def test_score_plan_materialises_full_scores():
    plan = Program(None, load("tiny_score")).plan("score")
    assert [s["execution"] for s in plan] == ["score_pass", "host"]


def test_retrieve_and_packed_plans():
    plan = Program(None, load("tiny_retrieve")).plan("retrieve")
    assert [s["execution"] for s in plan] == ["fused_pass", "fused_with_score", "fused_with_score", "device", "host"]
    plan = Program(None, load("tiny_packed_candidates")).plan("rerank_candidates_packed")
    assert [s["kind"] for s in plan][-2:] == ["pack_candidates", "return"]
    assert plan[0]["execution"] == "fused_pass" and plan[3]["execution"] == "fused_with_score"


def test_scores_returned_next_to_topk_forces_full_scores():
    mod = load("tiny_rerank")
    mod["steps"][-1]["outputs"].append("scores")
    plan = Program(None, mod).plan("rerank")
    assert plan[0]["execution"] == "fused_pass+full_scores"


def test_validation_errors():
    mod = load("tiny_rerank")
    bad = dict(mod, version="manta/v9")
    with pytest.raises(MantaError, match="unsupported artifact version"):
        Program(None, bad)
    bad = dict(mod, entry_points=[])
    with pytest.raises(MantaError, match="at least one entry point"):
        Program(None, bad)
    bad = json.loads(json.dumps(mod))
    bad["steps"][0]["kernel"] = "nope"
    with pytest.raises(MantaError, match='unknown kernel "nope"'):
        Program(None, bad)
    bad = json.loads(json.dumps(mod))
    bad["kernels"][0]["variants"] = [v for v in bad["kernels"][0]["variants"] if v["backend"] != "cuda"]
    with pytest.raises(MantaError, match="missing a cuda variant"):
        Program(None, bad)
    with pytest.raises(MantaError, match="json:"):
        Program(None, "{not json")
    prog = Program(None, mod)
    with pytest.raises(MantaError, match='unknown entrypoint "nope"'):
        prog.plan("nope")


def test_run_without_runtime_fails_loudly():
    from manta_b200.program import Tensor

    prog = Program(None, load("tiny_rerank"))
    with pytest.raises(MantaError, match="no host fallback"):
        prog.run("rerank", {"query": Tensor("f16", [2], [1, 0])})
