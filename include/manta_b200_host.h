/*
 * manta_b200_host.h -- host side of the score/select path above the kernels' C ABI: a plan (Module) loader and
 * step walker with the reference's Backend/Executor contract (reference paths are inside odvcencio/manta).
 *
 * In the reference this layer is Go: Runtime.Load / Program.Run (runtime/runtime.go:43-119), the plan
 * interpreter ExecuteSymbolic + executeStep (runtime/backend/symbolic.go:14-163, tensor_ops.go:13-135) and the
 * CUDA executor's dispatch (runtime/backends/cuda/cuda.go:222-429).  Go is not available to this build, so the
 * same contract is implemented in C++ inside libmanta_b200.so and exported with a C ABI; tests drive it through
 * ctypes (manta_b200/program.py).  What it keeps from the reference:
 *   - the Module JSON schema (artifact/manta/module.go:109-207, version "manta/v0alpha1");
 *   - tensors as (dtype label, shape, float32 / int32 / int64 data) (runtime/backend/tensor.go:11-19);
 *   - request validation, symbol binding (N, D, Q) and their error texts (symbolic.go:265-277, tensor.go:388-517);
 *   - Result.Outputs with Producer / Metadata, Result.Trace with one entry per ORIGINAL step, Result.Metadata
 *     (backend.go:12-36, symbolic.go:76-161);
 *   - error texts of topk / gather (tensor_ops.go:1532, 803).
 * What it changes: launch_kernel{dot|cosine|l2_distance} -> topk -> gather(scores, ids) is recognised at run time
 * and executed as ONE fused device pass; rank-2 q4/q8/f16 params feeding a score kernel are quantised into the
 * packed layouts and bound resident at load; nothing falls back to the CPU.
 */
#ifndef MANTA_B200_HOST_H_
#define MANTA_B200_HOST_H_

#include "manta_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct MantaB200Program MantaB200Program; /* backend.Executor + loaded Program, runtime/runtime.go:88-119 */
typedef struct MantaB200Result MantaB200Result;   /* backend.Result, runtime/backend/backend.go:250-254 */

/* backend.Tensor (runtime/backend/tensor.go:11-19): data is float32 for the labels f16, f32, q4, q8 (the
 * reference stores every float-like tensor widened to float32), int32 for i32, int64 for i64. */
typedef struct {
    const char* name;
    const char* dtype;
    int rank;
    const int64_t* shape;
    const void* data;
} MantaB200TensorArg;

/* Runtime.Load for one backend (runtime/runtime.go:43-86 + cuda.Backend.load, cuda.go:67-109): parses and
 * validates the Module JSON.  rt may be NULL: the program can then be inspected (manta_b200_program_plan) but
 * not run. */
int manta_b200_program_load(MantaB200Runtime* rt, const char* module_json, MantaB200Program** out, char** err);
/* WithWeight (runtime/runtime.go load options; fixtures at runtime/runtime_test.go:1576-1593). */
int manta_b200_program_bind_weight(MantaB200Program* prog, const MantaB200TensorArg* weight, char** err);
/* The steps of an entry point as this backend will execute them (which steps are fused), as JSON.  The string is
 * released with manta_b200_free_cstring. */
int manta_b200_program_plan(MantaB200Program* prog, const char* entry, char** out_json, char** err);
/* Program.Run (runtime/runtime.go:113-119 -> executor.Run, cuda.go:222-241 -> ExecuteSymbolic). */
int manta_b200_program_run(MantaB200Program* prog, const char* entry, const MantaB200TensorArg* inputs, int n_inputs,
                           MantaB200Result** out, char** err);
int manta_b200_program_destroy(MantaB200Program* prog, char** err);

/* NewMemoryPlan (runtime/memory_plan.go:59-138) over the bound weights: JSON document with version
 * "manta/memory/v0alpha1" (same fields as MemoryPlan / WeightMemoryPlan, :34-56).  accounting 0 budgets the
 * reference's logical bytes (tensorLogicalBytes, :381-406: codes only); accounting 1 budgets what one of `shards`
 * row shards really holds in HBM in the packed layouts (padded codes + scales + row statistic).  The string is
 * released with manta_b200_free_cstring. */
int manta_b200_program_memory_plan(MantaB200Program* prog, int64_t device_budget_bytes, int shared_host_weights, int shards,
                                   int accounting, char** out_json, char** err);
/* WithMemoryPlan (runtime/runtime.go:172-197): params whose residency is not device_resident are bound only for
 * the run that reads them and released afterwards (the reference honours lazy_staged the same way,
 * runtime/backend/symbolic.go:139-152, 165-171). */
int manta_b200_program_apply_memory_plan(MantaB200Program* prog, const char* plan_json, char** err);

/* Result as JSON: {"outputs": {name: {kind, dtype, shape, producer, inputs, metadata}}, "trace": [...],
 * "metadata": {...}}.  Owned by the result. */
const char* manta_b200_result_json(const MantaB200Result* res);
/* Borrowed view of an output tensor; field is "" for tensors and "ids" / "scores" / "docs" for a candidate_pack
 * (runtime/backend/tensor.go:26-31).  Valid until manta_b200_result_free. */
int manta_b200_result_tensor(const MantaB200Result* res, const char* output, const char* field, MantaB200TensorArg* view,
                             char** err);
void manta_b200_result_free(MantaB200Result* res);

/* computeRetrievalQuality of the eval-retrieval command (runtime/retrieval_eval.go:541-584, gate cmd/manta/main.go:
 * 2446-2452) with topRetrievalScores (:586-616) replaced by fused score + top-k passes: the document vectors
 * ([n_docs, dim] float32, rounded to f16) are bound once in document-ID order, so that the device's tie rule (lower
 * row first) is the reference's (smaller ID string first, :618-626); queries with a relevant document in the corpus
 * are scored 256 per pass with k = min(max(top_k, 100), n_docs).  qrels arrive as n_qrels (query id, doc id,
 * relevance) triples.  out_json (released with manta_b200_free_cstring):
 *   {"quality": {"ndcg_at_10", "mrr_at_10", "recall_at_10", "recall_at_100"}, "evaluated_queries",
 *    "relevant_pairs", "skipped_relevant_docs", "skipped_no_relevant", "scored_pairs", "top_k"}
 * -- the fields RetrievalEvalQualityMetrics / RetrievalEvalInputMetrics / RetrievalEvalSkippedCounts take from it
 * (:38-98). */
int manta_b200_retrieval_quality(MantaB200Runtime* rt, const float* query_vectors, const char* const* query_ids,
                                 int n_queries, const float* doc_vectors, const char* const* doc_ids, int64_t n_docs,
                                 int dim, const char* const* qrel_query_ids, const char* const* qrel_doc_ids,
                                 const double* qrel_values, int64_t n_qrels, int top_k, char** out_json, char** err);

#ifdef __cplusplus
}
#endif
#endif /* MANTA_B200_HOST_H_ */
