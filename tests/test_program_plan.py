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


def test_per_query_bundle_plans():
    # the [Q,D] x [Q,N,D] entries of the reference's score / retrieval bundles
    prog = Program(None, load("score_bundle"))
    assert [s["execution"] for s in prog.plan("score_batch")] == ["score_pass", "host"]
    assert [s["execution"] for s in prog.plan("score")] == ["score_pass", "host"]
    plan = Program(None, load("retrieval_bundle")).plan("rerank_candidates_packed_batch")
    assert [s["kind"] for s in plan] == ["launch_kernel", "topk", "gather", "gather", "gather", "pack_candidates", "return"]
    assert plan[0]["execution"] == "fused_pass" and plan[1]["execution"] == "fused_with_score"


def test_scores_returned_next_to_topk_forces_full_scores():
    mod = load("tiny_rerank")
    mod["steps"][-1]["outputs"].append("scores")
    plan = Program(None, mod).plan("rerank")
    assert plan[0]["execution"] == "fused_pass+full_scores"


def test_validation_errors():
    mod = load("tiny_rerank")
    bad = dict(mod, version="manta/v9")
    with pytest.raises(MantaError, match='module version "manta/v9" is not supported, want "manta/v0alpha1"'):
        Program(None, bad)
    bad = dict(mod, entry_points=[])
    with pytest.raises(MantaError, match="at least one entry point"):
        Program(None, bad)
    bad = json.loads(json.dumps(mod))
    bad["steps"][0]["kernel"] = "nope"
    with pytest.raises(MantaError, match='unknown kernel "nope"'):
        Program(None, bad)
    with pytest.raises(MantaError, match="json:"):
        Program(None, "{not json")
    prog = Program(None, mod)
    with pytest.raises(MantaError, match='unknown entrypoint "nope"'):
        prog.plan("nope")


def test_kernel_variant_rules():
    """validateKernelVariants (artifact/manta/module.go:426-449) and what loading on the CUDA backend adds."""
    mod = load("tiny_rerank")

    def broken(edit):
        bad = json.loads(json.dumps(mod))
        edit(bad)
        return bad

    # a compiler-made module supports five backends and every kernel carries all five variants
    assert sorted(v["backend"] for v in mod["kernels"][0]["variants"]) == ["cuda", "directml", "metal", "vulkan", "webgpu"]
    for backend in ("cuda", "metal", "vulkan", "directml", "webgpu"):
        bad = broken(lambda m: m["kernels"][0].__setitem__("variants", [v for v in m["kernels"][0]["variants"] if v["backend"] != backend]))
        with pytest.raises(MantaError, match=f'kernel "cosine" is missing variant for backend "{backend}"'):
            Program(None, bad)
    bad = broken(lambda m: m["kernels"][0]["variants"].append(dict(m["kernels"][0]["variants"][0])))
    with pytest.raises(MantaError, match='has duplicate variant for backend "cuda"'):
        Program(None, bad)
    bad = broken(lambda m: m["kernels"][0]["variants"][1].__setitem__("entry", ""))
    with pytest.raises(MantaError, match='variant entry is required for backend "metal"'):
        Program(None, bad)
    bad = broken(lambda m: m["kernels"][0]["variants"][2].__setitem__("source", ""))
    with pytest.raises(MantaError, match='variant source is required for backend "vulkan"'):
        Program(None, bad)
    bad = broken(lambda m: m["kernels"][0]["variants"][0].__setitem__("backend", ""))
    with pytest.raises(MantaError, match="variant backend is required"):
        Program(None, bad)
    bad = broken(lambda m: m["requirements"].__setitem__("supported_backends", []))
    with pytest.raises(MantaError, match="at least one supported backend is required"):
        Program(None, bad)
    bad = broken(lambda m: m["requirements"].__setitem__("supported_backends", ["cuda", "cuda"]))
    with pytest.raises(MantaError, match='duplicate supported backend "cuda"'):
        Program(None, bad)
    # a module that does not list cuda cannot load on this backend
    bad = broken(lambda m: m["requirements"].__setitem__("supported_backends", ["metal"]))
    with pytest.raises(MantaError, match="cuda: unsupported backend"):
        Program(None, bad)
    # the cuda variant's source must define its entry (validateCompiledKernelSource)
    bad = broken(lambda m: m["kernels"][0]["variants"][0].__setitem__("entry", "other_name"))
    with pytest.raises(MantaError, match='CUDA source does not define entry "other_name"'):
        Program(None, bad)
    # a module limited to cuda needs only the cuda variant
    ok = broken(lambda m: (m["requirements"].__setitem__("supported_backends", ["cuda"]),
                           m["kernels"][0].__setitem__("variants", m["kernels"][0]["variants"][:1])))
    Program(None, ok)


def test_dequant_step_is_seen_through():
    plan = Program(None, load("dequant_rerank")).plan("rerank")
    assert [s["kind"] for s in plan] == ["dequant", "launch_kernel", "topk", "gather", "return"]
    assert [s["execution"] for s in plan] == ["relabel", "fused_pass", "fused_with_score", "fused_with_score", "host"]


def test_run_without_runtime_fails_loudly():
    from manta_b200.program import Tensor

    prog = Program(None, load("tiny_rerank"))
    with pytest.raises(MantaError, match="no host fallback"):
        prog.run("rerank", {"query": Tensor("f16", [2], [1, 0])})


def test_memory_plan_budgeted_residency():
    """NewMemoryPlan's ordering and residency rule on the reference's own fixture shapes
    (runtime/memory_plan_test.go:60-86: q8 [32,16] embedding + q8 [16,16] projection, 300-byte budget)."""
    from manta_b200.program import Tensor

    mod = {"version": "manta/v0alpha1", "name": "tiny_embed_pooled",
           "params": [{"name": "token_embedding", "binding": "weights/token_embedding", "type": {"kind": "tensor", "tensor": {"dtype": "q8", "shape": ["V", "D"]}}},
                      {"name": "projection", "binding": "weights/projection", "type": {"kind": "tensor", "tensor": {"dtype": "q8", "shape": ["D", "E"]}}}],
           "entry_points": [{"name": "embed_pooled", "kind": "pipeline", "inputs": [], "outputs": []}],
           "requirements": {"supported_backends": ["cuda"]}, "kernels": [],
           "steps": [{"entry": "embed_pooled", "kind": "gather", "name": "gather", "inputs": ["token_embedding", "tokens"], "outputs": ["hidden"]},
                     {"entry": "embed_pooled", "kind": "matmul", "name": "matmul", "inputs": ["hidden", "projection"], "outputs": ["projected"]}]}
    prog = Program(None, mod)
    prog.bind_weight("token_embedding", Tensor("q8", [32, 16], [0.0] * 512))
    prog.bind_weight("projection", Tensor("q8", [16, 16], [0.0] * 256))
    plan = prog.memory_plan(300, shared_host_weights=True, accounting="logical")
    assert plan["version"] == "manta/memory/v0alpha1" and len(plan["weights"]) == 2
    res = {w["name"]: w for w in plan["weights"]}
    assert res["projection"]["bytes"] == 256 and res["token_embedding"]["bytes"] == 512  # tensorLogicalBytes
    assert res["projection"]["residency"] == "device_resident"
    assert res["token_embedding"]["residency"] == "host_shared"
    assert plan["device_resident_bytes"] == 256 and plan["host_resident_bytes"] == 512
    # without shared host weights a once-read weight is lazily staged
    plan = prog.memory_plan(300, accounting="logical")
    assert {w["name"]: w["residency"] for w in plan["weights"]}["token_embedding"] == "lazy_staged"
    # device accounting counts scales and the row statistic: 16*(16+4+4) = 384, 32*(16+4+4) = 768
    plan = prog.memory_plan(400, shared_host_weights=True)
    res = {w["name"]: w for w in plan["weights"]}
    assert res["projection"]["device_bytes_per_shard"] == 384 and res["token_embedding"]["device_bytes_per_shard"] == 768
    assert res["projection"]["residency"] == "device_resident" and res["token_embedding"]["residency"] == "host_shared"
    # sharding the rows over 8 GPUs divides what each device holds
    plan = prog.memory_plan(400, shared_host_weights=True, shards=8)
    assert {w["name"]: w["device_bytes_per_shard"] for w in plan["weights"]} == {"projection": 48, "token_embedding": 96}
    assert all(w["residency"] == "device_resident" for w in plan["weights"])
    # unbudgeted: everything resident
    assert all(w["residency"] == "device_resident" for w in prog.memory_plan()["weights"])
    with pytest.raises(MantaError, match="unknown residency"):
        prog.apply_memory_plan({"version": "manta/memory/v0alpha1", "weights": [{"name": "projection", "residency": "moon"}]})
