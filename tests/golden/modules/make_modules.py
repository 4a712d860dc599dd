"""Writes the Module JSON fixtures of this folder.

The documents have the structure the reference compiler emits for its example pipelines (examples/*.manta;
lowering rules compiler/compiler.go:1542-1585, 1628-1661, 1722-1747, 1792-1803 of odvcencio/manta): params,
entry points, one kernel per score builtin with a variant for each of the five backends, and the step list
launch_kernel -> topk -> gather ... -> return.  They are authored here because no Go toolchain is available to
run the compiler.  Run:  python tests/golden/modules/make_modules.py
"""
import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))


def ttype(dtype, shape):
    return {"kind": "tensor", "tensor": {"dtype": dtype, "shape": shape}}


def variants(op):
    src = ("extern \"C\" __global__ void %s_cuda(const float* query, const float* docs, float* out0, int rows, int cols) "
           "{ /* vestigial: replaced by AOT sm_100a kernels */ }" % op)
    meta = {"tile": "[128]", "vector_width": "4", "subgroup": "true", "memory": "workgroup_local"}
    return [{"backend": b, "entry": "%s_%s" % (op, b), "source": src if b == "cuda" else "// %s" % b, "meta": dict(meta)}
            for b in ["cuda", "metal", "vulkan", "directml", "webgpu"]]


def kernel(op, qshape, dshape, oshape):
    return {"name": op,
            "inputs": [{"name": "query", "type": ttype("f16", qshape)}, {"name": "docs", "type": ttype("q4", dshape)}],
            "outputs": [{"name": "result", "type": ttype("f32", oshape)}],
            "hints": {"tile": [128], "vector_width": 4, "subgroup": True, "memory": "workgroup_local"},
            "body": [{"kind": "reduce", "op": op, "inputs": ["query", "docs"], "outputs": ["result"]},
                     {"kind": "return", "op": "return", "outputs": ["result"]}],
            "variants": variants(op)}


def module(name, params, entries, kernels, steps):
    return {"version": "manta/v0alpha1", "name": name, "params": params, "entry_points": entries,
            "requirements": {"supported_backends": ["cuda", "metal", "vulkan", "directml", "webgpu"]},
            "buffers": [], "kernels": kernels, "steps": steps}


def step(entry, kind, name, inputs=None, outputs=None, kernel=None, attrs=None):
    s = {"entry": entry, "kind": kind, "name": name}
    if kernel:
        s["kernel"] = kernel
    if inputs:
        s["inputs"] = inputs
    if outputs:
        s["outputs"] = outputs
    if attrs:
        s["attributes"] = attrs
    return s


def build():
    docs_param = [{"name": "docs", "type": ttype("q4", ["N", "D"]), "binding": "weights/docs"}]
    q_in = [{"name": "query", "type": ttype("f16", ["D"])}]
    cos = [kernel("cosine", ["D"], ["N", "D"], ["N"])]
    mods = {}
    mods["tiny_score"] = module("tiny_score", docs_param,
        [{"name": "score", "kind": "pipeline", "inputs": q_in, "outputs": [{"name": "scores", "type": ttype("f32", ["N"])}]}], cos,
        [step("score", "launch_kernel", "cosine", ["query", "docs"], ["scores"], "cosine"), step("score", "return", "return", None, ["scores"])])
    mods["tiny_rerank"] = module("tiny_rerank", docs_param,
        [{"name": "rerank", "kind": "pipeline", "inputs": q_in,
          "outputs": [{"name": "top_ids", "type": ttype("i32", ["2"])}, {"name": "top_scores", "type": ttype("f32", ["2"])}]}], cos,
        [step("rerank", "launch_kernel", "cosine", ["query", "docs"], ["scores"], "cosine"),
         step("rerank", "topk", "topk", ["scores"], ["top_ids"], None, {"k": "2"}),
         step("rerank", "gather", "gather", ["scores", "top_ids"], ["top_scores"]),
         step("rerank", "return", "return", None, ["top_ids", "top_scores"])])
    mods["tiny_select"] = module("tiny_select", docs_param,
        [{"name": "select_scores", "kind": "pipeline", "inputs": q_in, "outputs": [{"name": "top_scores", "type": ttype("f32", ["2"])}]}], cos,
        [step("select_scores", "launch_kernel", "cosine", ["query", "docs"], ["scores"], "cosine"),
         step("select_scores", "topk", "topk", ["scores"], ["ids"], None, {"k": "2"}),
         step("select_scores", "gather", "gather", ["scores", "ids"], ["top_scores"]),
         step("select_scores", "return", "return", None, ["top_scores"])])
    mods["tiny_retrieve"] = module("tiny_retrieve", docs_param,
        [{"name": "retrieve", "kind": "pipeline", "inputs": q_in,
          "outputs": [{"name": "top_ids", "type": ttype("i32", ["2"])}, {"name": "top_scores", "type": ttype("f32", ["2"])},
                      {"name": "top_docs", "type": ttype("q4", ["2", "D"])}]}], cos,
        [step("retrieve", "launch_kernel", "cosine", ["query", "docs"], ["scores"], "cosine"),
         step("retrieve", "topk", "topk", ["scores"], ["top_ids"], None, {"k": "2"}),
         step("retrieve", "gather", "gather", ["scores", "top_ids"], ["top_scores"]),
         step("retrieve", "gather", "gather", ["docs", "top_ids"], ["top_docs"]),
         step("retrieve", "return", "return", None, ["top_ids", "top_scores", "top_docs"])])
    cand_inputs = q_in + [{"name": "docs", "type": ttype("q4", ["N", "D"])}, {"name": "candidate_ids", "type": ttype("i64", ["N"])}]

    def cand_steps(e):
        return [step(e, "launch_kernel", "cosine", ["query", "docs"], ["scores"], "cosine"),
                step(e, "topk", "topk", ["scores"], ["top_indices"], None, {"k": "2"}),
                step(e, "gather", "gather", ["candidate_ids", "top_indices"], ["top_candidate_ids"]),
                step(e, "gather", "gather", ["scores", "top_indices"], ["top_scores"]),
                step(e, "gather", "gather", ["docs", "top_indices"], ["top_docs"])]

    mods["tiny_candidates"] = module("tiny_candidates", [],
        [{"name": "rerank_candidates", "kind": "pipeline", "inputs": cand_inputs,
          "outputs": [{"name": "top_candidate_ids", "type": ttype("i64", ["2"])}, {"name": "top_scores", "type": ttype("f32", ["2"])},
                      {"name": "top_docs", "type": ttype("q4", ["2", "D"])}]}], cos,
        cand_steps("rerank_candidates") + [step("rerank_candidates", "return", "return", None, ["top_candidate_ids", "top_scores", "top_docs"])])
    mods["tiny_packed_candidates"] = module("tiny_packed_candidates", [],
        [{"name": "rerank_candidates_packed", "kind": "pipeline", "inputs": cand_inputs,
          "outputs": [{"name": "candidates", "type": {"kind": "candidate_pack", "candidate_pack": {"shape": ["2", "D"]}}}]}], cos,
        cand_steps("rerank_candidates_packed") +
        [step("rerank_candidates_packed", "pack_candidates", "pack_candidates", ["top_candidate_ids", "top_scores", "top_docs"], ["candidates"]),
         step("rerank_candidates_packed", "return", "return", None, ["candidates"])])
    # the per-query-docs entries of the reference's score / retrieval bundles (runtime/score_model_test.go:86-131,
    # runtime/retrieval_model_test.go:94-150)
    qb_in = [{"name": "queries", "type": ttype("f16", ["Q", "D"])}, {"name": "docs", "type": ttype("q4", ["Q", "N", "D"])}]
    cos_batch = dict(kernel("cosine", ["Q", "D"], ["Q", "N", "D"], ["Q", "N"]), name="cosine_batch")
    mods["score_bundle"] = module("score_bundle", [],
        [{"name": "score", "kind": "pipeline", "inputs": q_in + [{"name": "docs", "type": ttype("q4", ["N", "D"])}],
          "outputs": [{"name": "scores", "type": ttype("f32", ["N"])}]},
         {"name": "score_batch", "kind": "pipeline", "inputs": qb_in, "outputs": [{"name": "scores", "type": ttype("f32", ["Q", "N"])}]}],
        cos + [cos_batch],
        [step("score", "launch_kernel", "cosine", ["query", "docs"], ["scores"], "cosine"), step("score", "return", "return", None, ["scores"]),
         step("score_batch", "launch_kernel", "cosine_batch", ["queries", "docs"], ["scores"], "cosine_batch"),
         step("score_batch", "return", "return", None, ["scores"])])
    eb = "rerank_candidates_packed_batch"
    mods["retrieval_bundle"] = module("retrieval_bundle", [],
        [{"name": "rerank_candidates_packed", "kind": "pipeline", "inputs": cand_inputs,
          "outputs": [{"name": "candidates", "type": {"kind": "candidate_pack", "candidate_pack": {"shape": ["2", "D"]}}}]},
         {"name": eb, "kind": "pipeline", "inputs": qb_in + [{"name": "candidate_ids", "type": ttype("i64", ["Q", "N"])}],
          "outputs": [{"name": "candidates", "type": {"kind": "candidate_pack", "candidate_pack": {"shape": ["Q", "2", "D"]}}}]}],
        cos + [cos_batch],
        cand_steps("rerank_candidates_packed") +
        [step("rerank_candidates_packed", "pack_candidates", "pack_candidates", ["top_candidate_ids", "top_scores", "top_docs"], ["candidates"]),
         step("rerank_candidates_packed", "return", "return", None, ["candidates"]),
         step(eb, "launch_kernel", "cosine_batch", ["queries", "docs"], ["scores"], "cosine_batch"),
         step(eb, "topk", "topk", ["scores"], ["top_indices"], None, {"k": "2"}),
         step(eb, "gather", "gather", ["candidate_ids", "top_indices"], ["top_candidate_ids"]),
         step(eb, "gather", "gather", ["scores", "top_indices"], ["top_scores"]),
         step(eb, "gather", "gather", ["docs", "top_indices"], ["top_docs"]),
         step(eb, "pack_candidates", "pack_candidates", ["top_candidate_ids", "top_scores", "top_docs"], ["candidates"]),
         step(eb, "return", "return", None, ["candidates"])])
    # score(query, dequant(docs_q)): the dequant step only relabels, the pass still binds docs_q packed
    docs_q8 = [{"name": "docs_q", "type": ttype("q8", ["N", "D"]), "binding": "weights/docs_q"}]
    mods["dequant_rerank"] = module("dequant_rerank", docs_q8,
        [{"name": "rerank", "kind": "pipeline", "inputs": q_in,
          "outputs": [{"name": "top_ids", "type": ttype("i32", ["2"])}, {"name": "top_scores", "type": ttype("f32", ["2"])}]}], cos,
        [step("rerank", "dequant", "dequant", ["docs_q"], ["docs"]),
         step("rerank", "launch_kernel", "cosine", ["query", "docs"], ["scores"], "cosine"),
         step("rerank", "topk", "topk", ["scores"], ["top_ids"], None, {"k": "2"}),
         step("rerank", "gather", "gather", ["scores", "top_ids"], ["top_scores"]),
         step("rerank", "return", "return", None, ["top_ids", "top_scores"])])
    for op in ("dot", "cosine", "l2_distance"):
        mods["direct_" + op] = module(op, [],
            [{"name": "score", "kind": "pipeline",
              "inputs": q_in + [{"name": "docs", "type": ttype("q4", ["N", "D"])}], "outputs": [{"name": "scores", "type": ttype("f32", ["N"])}]}],
            [kernel(op, ["D"], ["N", "D"], ["N"])],
            [step("score", "launch_kernel", op, ["query", "docs"], ["scores"], op), step("score", "return", "return", None, ["scores"])])
    return mods


if __name__ == "__main__":
    for name, mod in build().items():
        with open(os.path.join(HERE, name + ".json"), "w") as f:
            json.dump(mod, f, indent=1)
        print("wrote", name)
