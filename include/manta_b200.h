/*
 * manta_b200.h -- C ABI of the B200-native score/select path for Manta's CUDA backend.
 *
 * This is the boundary the Go side binds with cgo in place of the C preamble of
 * runtime/backends/cuda/native_linux.go (reference paths are inside odvcencio/manta).
 * Conventions kept from that preamble (native_linux.go:30-75, 385-402, 620-624):
 *   - every call returns int: 0 = ok, 1 = failure;
 *   - on failure *err receives a malloc'd, NUL-terminated message that the caller releases with
 *     manta_b200_free_cstring (the reference's mantaCudaFreeCString); err may be NULL;
 *   - the device is made current at the top of every call (goroutines migrate between threads);
 *   - host pointers are borrowed for the duration of the call only; calls are synchronous unless
 *     the name ends in _device and sync == 0;
 *   - nothing aborts or traps; a runtime handle serialises its calls with an internal mutex.
 *
 * Differences from the reference's device path, by design:
 *   - candidates are bound once and stay resident in HBM in their packed form (the reference
 *     uploads all docs as fp32 on every call, native_linux.go:1705-1714);
 *   - score -> topk -> gather(scores, ids) runs as one fused device pass (the reference runs topk
 *     and gather on the host, runtime/backend/tensor_ops.go:119-135, 1523-1592);
 *   - a batch of queries against ONE shared candidate matrix is supported ([Q,D] x [N,D]).
 *
 * There is no CPU fallback behind any of these entry points.
 */
#ifndef MANTA_B200_H_
#define MANTA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct MantaB200Runtime MantaB200Runtime;       /* replaces MantaCudaRuntime, native_linux.go:16-23 */
typedef struct MantaB200Candidates MantaB200Candidates; /* replaces the per-call docs buffer, native_linux.go:1710 */

/* Candidate layouts.  Row-major [rows, cols].
 *   F16        : IEEE half bits, 2*cols bytes per row.
 *   Q8_ROW_F32 : int8 codes, cols bytes per row + one f32 scale per row; value = code * scale;
 *                scale = max|x|/127, code = round-half-away(x/scale) clamped to +-127
 *                (the rule of runtime/embedding_trainer.go:3730-3763 applied per row).
 *   Q4_B32_F16 : cols/32 blocks per row; block = 16 bytes, element 2j in the low nibble of byte j and
 *                element 2j+1 in the high nibble, 4-bit two's complement codes in [-7,7]; one f16
 *                scale per block (scales array [rows, cols/32]); value = code * scale; cols % 32 == 0.
 */
enum {
    MANTA_B200_LAYOUT_F16 = 0,
    MANTA_B200_LAYOUT_Q8_ROW_F32 = 1,
    MANTA_B200_LAYOUT_Q4_B32_F16 = 2
};

/* Score builtins of compiler/compiler.go:803-842 / runtime/backend/tensor_ops.go:1366-1490. */
enum {
    MANTA_B200_METRIC_DOT = 0,
    MANTA_B200_METRIC_COSINE = 1,
    MANTA_B200_METRIC_L2_DISTANCE = 2
};

/* LARGEST is topKTensor's order (value descending, ties to the lower row id,
 * runtime/backend/tensor_ops.go:1539-1552).  SMALLEST is the build's extension for
 * "k smallest distance": ascending value, ties to the lower row id. */
enum {
    MANTA_B200_ORDER_LARGEST = 0,
    MANTA_B200_ORDER_SMALLEST = 1
};

/* Where the pointers passed to manta_b200_candidates_bind live. */
enum {
    MANTA_B200_MEM_HOST = 0,        /* host memory: copied to the device */
    MANTA_B200_MEM_DEVICE_COPY = 1, /* device memory: copied into storage the set owns */
    MANTA_B200_MEM_DEVICE_ADOPT = 2 /* device memory: used in place, caller keeps it alive; needs 16-byte
                                       aligned base and a row size that is a multiple of 16 bytes */
};

typedef struct {
    uint64_t bind_calls;         /* counterparts of MatMulAcceleratorStats, runtime/backend/backend.go:92-107 */
    uint64_t bound_bytes;
    uint64_t score_calls;
    uint64_t score_topk_calls;
    uint64_t kernel_launches;    /* launches of this library's kernels */
    uint64_t h2d_bytes;
    uint64_t d2h_bytes;
    uint64_t chunked_reruns;     /* fused passes that overflowed the candidate pool and were redone in chunks */
    uint64_t mma_passes;         /* fused passes that ran on the tcgen05 tensor-core kernel */
    uint64_t gemv_passes;        /* fused passes that ran on the streaming (GEMV) kernel */
} MantaB200Stats;

/* mantaCudaRuntimeCreate, native_linux.go:108-169.  device: CUDA ordinal (the reference hard-codes 0).
 * stream: a cudaStream_t to launch on, or NULL to let the runtime create its own. */
int manta_b200_runtime_create(int device, void* stream, MantaB200Runtime** out, char** err);
/* mantaCudaRuntimeDestroy, native_linux.go:171-189. */
int manta_b200_runtime_destroy(MantaB200Runtime* rt, char** err);
/* mantaCudaFreeCString, native_linux.go:620-624. */
void manta_b200_free_cstring(char* s);
/* The stream all work of this runtime is issued on (cudaStream_t). */
int manta_b200_runtime_stream(MantaB200Runtime* rt, void** out_stream, char** err);
/* mantaCudaSynchronize-equivalent for the runtime's stream (native_linux.go:385-402 syncs after each launch).
 * Also reports, as a failure, a candidate-pool overflow of the last fused pass issued with sync == 0. */
int manta_b200_runtime_synchronize(MantaB200Runtime* rt, char** err);
int manta_b200_runtime_stats(MantaB200Runtime* rt, MantaB200Stats* out, char** err);
/* Device-time accounting of the scan kernels (the counterpart of RunNanos in MatMulAcceleratorStats,
 * runtime/backend/backend.go:92-107).  While enabled, every fused pass brackets its scan kernel(s) with CUDA
 * events on the runtime's stream (at most 256 passes are kept).  scan_time synchronises the stream, returns the
 * summed device milliseconds and the number of passes measured since the last call, and clears the record. */
int manta_b200_runtime_profile(MantaB200Runtime* rt, int enable, char** err);
int manta_b200_runtime_scan_time(MantaB200Runtime* rt, double* total_ms, int* passes, char** err);
/* Launch configuration of the scan kernel the runtime's last score / fused pass issued: the truthful counterpart of
 * nativeLaunchConfig's launch_* metadata (runtime/backend/native_kernel.go:65-112), which the host executor attaches
 * to the values a score step produces.  kernel is the __global__ function's name. */
typedef struct {
    char kernel[48];
    int grid;          /* thread blocks (one-dimensional grid) */
    int block;         /* threads per block */
    int shared_bytes;  /* dynamic shared memory per block */
    int launches;      /* scan launches of that pass (query groups, row chunks) */
} MantaB200LaunchInfo;
int manta_b200_runtime_last_launch(MantaB200Runtime* rt, MantaB200LaunchInfo* out, char** err);
/* Number of kernels this library has launched in this process (all runtimes). */
uint64_t manta_b200_kernel_launch_count(void);

/* Binds a packed candidate matrix: replaces uploadFloat32(docs.F32) of runScoreKernel
 * (native_linux.go:1710, 1775-1785) and bindResidentMatMulParams' residency (cuda.go:129-196).
 * data/scales are laid out as described at the layout enum; scales is NULL for F16.
 * row_base is added to local row numbers to form the ids a fused pass returns (shard offset);
 * row_base + rows must fit int32 (topKTensor returns int32 ids, tensor_ops.go:1553).
 * Row statistics (sum of squares per row) are computed on the device at bind time. */
int manta_b200_candidates_bind(MantaB200Runtime* rt, int layout, int64_t rows, int cols, const void* data,
                               const void* scales, int64_t row_base, int mem, MantaB200Candidates** out,
                               char** err);
int manta_b200_candidates_unbind(MantaB200Runtime* rt, MantaB200Candidates* set, char** err);
/* Stored bytes of a bound set (codes + scales), the figure memory planning budgets
 * (runtime/memory_plan.go:381-406 counts codes only). */
int64_t manta_b200_candidates_bytes(const MantaB200Candidates* set);

/* Quantisers for the packed layouts: quantizeBufferInPlace + manta_forward_quantize_in_place
 * (native_linux.go:2588-2619, 641-661) applied per row (q8) / per 32-element block (q4), codes kept
 * instead of being multiplied back.  Host in, host out; the work runs on the device. */
int manta_b200_pack_q8_rows(MantaB200Runtime* rt, const float* src, int64_t rows, int cols, int8_t* codes,
                            float* scales, char** err);
int manta_b200_pack_q4_b32(MantaB200Runtime* rt, const float* src, int64_t rows, int cols, uint8_t* codes,
                           uint16_t* scales, char** err);
/* Same, device in / device out, asynchronous on the runtime's stream. src_is_f16: rows are half bits. */
int manta_b200_pack_q8_rows_device(MantaB200Runtime* rt, const void* d_src, int src_is_f16, int64_t rows, int cols,
                                   int8_t* d_codes, float* d_scales, char** err);
int manta_b200_pack_q4_b32_device(MantaB200Runtime* rt, const void* d_src, int src_is_f16, int64_t rows, int cols,
                                  uint8_t* d_codes, uint16_t* d_scales, char** err);

/* Full score vector: runScoreKernel + mantaCudaLaunchScore (native_linux.go:1694-1732, 419-422).
 * queries: nq x cols IEEE half bits (nq == 1 is the reference's [D] x [N,D] form).
 * out_scores: host, nq x rows f32. */
int manta_b200_score(MantaB200Runtime* rt, const MantaB200Candidates* set, int metric, const uint16_t* queries,
                     int nq, float* out_scores, char** err);

/* Fused score -> topk -> gather(scores, ids): the three plan steps of compiler/compiler.go:1628-1661
 * executed as one device pass.  out_ids: host int32 [nq, k] (row_base + local row), out_scores: host f32
 * [nq, k], best first.  Fails like topKTensor (tensor_ops.go:1532) when k <= 0 or k > rows. */
int manta_b200_score_topk(MantaB200Runtime* rt, const MantaB200Candidates* set, int metric, int order,
                          const uint16_t* queries, int nq, int k, int32_t* out_ids, float* out_scores,
                          char** err);
/* Same with device buffers; asynchronous on the runtime's stream when sync == 0. */
int manta_b200_score_topk_device(MantaB200Runtime* rt, const MantaB200Candidates* set, int metric, int order,
                                 const void* d_queries, int nq, int k, int32_t* d_out_ids, float* d_out_scores,
                                 int sync, char** err);

/* Same pass as manta_b200_score_topk_device for callers that cannot allocate device memory when they score
 * (all HBM already handed out, a no-allocation rule after start-up, another stream being captured).  It has no
 * counterpart in the reference.  It never calls cudaMalloc/cudaFree or any allocating routine: all scratch lives in
 * one fixed array inside the library image (about 4.4 MB, held by every GPU that loads the library until exit).
 * Limits, rejected with an error beyond them: at most 4 queries, k <= 256, cols <= 4096 per call.  The candidate
 * pool holds 131072 keys per query, so rows are scanned in chunks of (131072 - k) rows with the pool compacted to
 * the best k between chunks: the result is exact for any row order, but large sets take more launches than the
 * allocating entry points need.
 * The first call on a device looks up the array's device address; make that call before any stream capture.
 * All calls share the array, which keeps the previous call's contents (what must start at zero is cleared by
 * the pass itself): two calls whose device work overlaps, from any runtimes or threads, race. */
int manta_b200_score_topk_static(MantaB200Runtime* rt, const MantaB200Candidates* set, int metric, int order,
                                 const void* d_queries, int nq, int k, int32_t* d_out_ids, float* d_out_scores,
                                 int sync, char** err);

/* Merges `lists` per-shard results (device memory) into the global best k per query with the same ordering
 * rule.  List l holds ids at d_ids + l*list_stride and scores at d_scores + l*list_stride, each [nq, k];
 * list_stride is in 4-byte elements and 0 means nq*k (lists back to back).  A stride lets one all-gather carry
 * both arrays: every shard fills [2, nq, k] (ids, then scores) and the gathered [lists, 2, nq, k] buffer is merged
 * with d_scores = d_ids + nq*k and list_stride = 2*nq*k.  Used after the shards' lists are gathered. */
int manta_b200_topk_merge_device(MantaB200Runtime* rt, int order, const int32_t* d_ids, const float* d_scores,
                                 int lists, int64_t list_stride, int nq, int k, int32_t* d_out_ids,
                                 float* d_out_scores, int sync, char** err);

/* gatherTensor on a rank-2 table (tensor_ops.go:794-827) for the bound set: de-quantised rows
 * out[i, :] = value(ids[i] - row_base, :) as f32 (the reference keeps them as float32 labelled q4).
 * Any id outside the set fails with "gather index %d out of range". */
int manta_b200_gather_rows(MantaB200Runtime* rt, const MantaB200Candidates* set, const int32_t* ids, int64_t n,
                           float* out, char** err);

/* ---- exchange of per-shard lists over peer memory (no counterpart in the reference, which runs on one device) ------
 * One process per GPU.  Every rank creates an exchange (an inbox on its own GPU), the 64-byte handles are passed to all
 * ranks by the host (any transport), and manta_b200_exchange_connect maps the peers' inboxes.
 * manta_b200_topk_exchange_merge_device then replaces "all-gather the [nq,k] lists + manta_b200_topk_merge_device":
 * on the runtime's stream it stores this rank's list into every rank's inbox with peer stores over NVLink, waits
 * (bounded, about two seconds) for the lists of all ranks and selects the global top k.  Ranks must issue the same
 * sequence of merges.  A list that does not arrive fails the call (sync != 0) or the next
 * manta_b200_runtime_synchronize (sync == 0); the context stays usable. */
typedef struct MantaB200Exchange MantaB200Exchange;
int manta_b200_exchange_create(MantaB200Runtime* rt, int world, int rank, int nq_max, int k_max, MantaB200Exchange** out,
                               unsigned char* handle_out /* 64 bytes */, char** err);
int manta_b200_exchange_connect(MantaB200Runtime* rt, MantaB200Exchange* ex, const unsigned char* handles /* world x 64 */,
                                char** err);
/* Same for ranks that live in ONE process (one process driving several GPUs, or several exchanges on one GPU): takes
 * the ranks' exchange handles (ranks[r] for every r != own rank) instead of IPC handles; peer access between the
 * devices is enabled when they differ. */
int manta_b200_exchange_connect_local(MantaB200Runtime* rt, MantaB200Exchange* ex, MantaB200Exchange* const* ranks, char** err);
/* How long a merge waits for a list that has not arrived, in naps of 200 ns (default 10,000,000: about two seconds). */
int manta_b200_exchange_set_wait_limit(MantaB200Exchange* ex, uint32_t naps_200ns, char** err);
/* Tear-down is two steps with a host barrier between them: EVERY rank first disconnects (synchronises its stream and
 * unmaps the peers' inboxes), the ranks meet at a barrier, and only then does each rank destroy its exchange, which
 * frees its own inbox.  Freeing an inbox a peer still has mapped is undefined behaviour of CUDA IPC.  destroy on an
 * exchange that was never disconnected unmaps first (correct for a single rank, and for peers known to be gone). */
int manta_b200_exchange_disconnect(MantaB200Runtime* rt, MantaB200Exchange* ex, char** err);
int manta_b200_exchange_destroy(MantaB200Runtime* rt, MantaB200Exchange* ex, char** err);
/* The whole sharded step on the runtime's stream: fused score + top-k over this rank's shard whose selection kernel
 * stores the lists straight into every rank's inbox (peer stores) and publishes the epoch, then the merge whose
 * selection kernel waits for all ranks' lists.  The shard pass is asynchronous: a pool overflow is reported by the next
 * synchronisation and the step must then be redone with manta_b200_score_topk_device(sync != 0) +
 * manta_b200_topk_exchange_merge_device. */
int manta_b200_score_topk_exchange_device(MantaB200Runtime* rt, MantaB200Exchange* ex, const MantaB200Candidates* set,
                                          int metric, int order, const void* d_queries, int nq, int k,
                                          int32_t* d_out_ids, float* d_out_scores, int sync, char** err);
int manta_b200_topk_exchange_merge_device(MantaB200Runtime* rt, MantaB200Exchange* ex, int order, const int32_t* d_ids,
                                          const float* d_scores, int nq, int k, int32_t* d_out_ids, float* d_out_scores,
                                          int sync, char** err);

/* ---- packed candidate files ------------------------------------------------------------------------------
 * The stored form of a bound set (codes + scales of its layout) on disk.  The reference exports q4 / q8 tensors
 * widened to float32 inside its MLL container (runtime/mll_export.go:833-866, read back by decodeTensorEntry,
 * runtime/weight_file.go:304-367; the container library github.com/odvcencio/mll is a separate module); this file
 * keeps the packed bytes, so a set is quantised once and a row shard [row_begin, row_end) of it can be bound per GPU
 * (row_end < 0: to the end; ids continue from the file's row_base).  verify != 0 checks the payload checksum. */
int manta_b200_candidates_save(MantaB200Runtime* rt, const MantaB200Candidates* set, const char* path, char** err);
int manta_b200_candidates_load(MantaB200Runtime* rt, const char* path, int64_t row_begin, int64_t row_end, int verify,
                               MantaB200Candidates** out, char** err);
int manta_b200_packed_file_info(const char* path, int* layout, int64_t* rows, int* cols, int64_t* row_base,
                                int64_t* stored_bytes, char** err);

/* ---- per-query candidate sets: queries [Q,D] x docs [Q,N,D] ----------------------------------------------
 * The second legal shape of the score builtins (scoreLayout, runtime/backend/tensor_ops.go:1492-1521), used by
 * ScoreModel.ScoreBatch / RetrievalModel.RetrieveBatch (runtime/score_model.go:238-324, retrieval_model.go:246-332).
 * The reference's CUDA backend computes it on the host (runtime/backends/cuda/cuda.go:961-976).  queries / docs are
 * float32 (the reference's tensor storage), host pointers for MANTA_B200_MEM_HOST, device pointers for
 * MANTA_B200_MEM_DEVICE_COPY (read in place); outputs live where the inputs live.  out: [Q,N] float32. */
int manta_b200_score_batched(MantaB200Runtime* rt, int metric, const float* queries, const float* docs, int nq,
                             int64_t rows, int cols, int mem, float* out, char** err);
/* Fused with topKTensor per query row (tensor_ops.go:1548-1590; error "topk limit %d out of range for row width
 * %d") and gather(scores, ids): out_ids int32 [Q,k] (row index within the query's own set), out_scores [Q,k]. */
int manta_b200_score_topk_batched(MantaB200Runtime* rt, int metric, int order, const float* queries, const float* docs,
                                  int nq, int64_t rows, int cols, int mem, int k, int32_t* out_ids, float* out_scores,
                                  char** err);

/* ---- embedding front end: the caller of the score path in the reference's embed pipelines ----------------
 * gather(token_embedding, tokens) -> @matmul(projection) -> masked mean_pool / normalize
 * (examples/embed_masked_pooled.manta; steps runtime/backend/tensor_ops.go:31-47, 83-118, 646-658; host math
 * :751-827 gather, :981-1011 matmul, :1210-1275 masked mean pool, :1114-1138 normalize).  In the reference every
 * one of these steps uploads and downloads its operands (native_linux.go:3608-3670, 1583-1622) and mean_pool has
 * no device kernel at all (:1734-1750); here the weights stay resident and the pooled query batch is handed to the
 * scoring kernels on the device. */
typedef struct MantaB200Embedder MantaB200Embedder;
enum {
    MANTA_B200_POOL_THEN_NORMALIZE = 0, /* normalize(mean_pool(x, mask)) */
    MANTA_B200_NORMALIZE_THEN_POOL = 1  /* mean_pool(normalize(x), mask), the order of embed_masked_pooled.manta */
};
/* table: [vocab, dim] half bits, projection: [dim, out_dim] half bits (row-major, as the reference's @matmul reads
 * its right operand); mem as for manta_b200_candidates_bind (HOST or DEVICE_COPY). */
int manta_b200_embedder_bind(MantaB200Runtime* rt, int vocab, int dim, int out_dim, const uint16_t* table,
                             const uint16_t* projection, int mem, MantaB200Embedder** out, char** err);
int manta_b200_embedder_unbind(MantaB200Runtime* rt, MantaB200Embedder* emb, char** err);
/* tokens, mask: host int32 [batch, seq] (mask != 0 keeps a position); out: host f32 [batch, out_dim].
 * A token outside the table fails with "gather index %d out of range" (tensor_ops.go:803). */
int manta_b200_embed_pooled(MantaB200Runtime* rt, const MantaB200Embedder* emb, const int32_t* tokens,
                            const int32_t* mask, int batch, int seq, int pool_order, float* out, char** err);
/* Device-resident form: tokens / mask are device int32 [batch, seq]; writes the pooled rows rounded to f16 into
 * d_out_queries [batch, out_dim], ready for manta_b200_score_topk_device on the runtime's stream.  With sync == 0 a
 * token outside the table is reported by the next manta_b200_runtime_synchronize. */
int manta_b200_embed_device(MantaB200Runtime* rt, const MantaB200Embedder* emb, const int32_t* d_tokens,
                            const int32_t* d_mask, int batch, int seq, int pool_order, void* d_out_queries, int sync,
                            char** err);
/* Embed, then fused score + top-k against a bound candidate set whose cols == out_dim; the pooled queries are
 * rounded to f16 on the device and never visit the host.  out_ids / out_scores: host [batch, k]. */
int manta_b200_embed_score_topk(MantaB200Runtime* rt, const MantaB200Embedder* emb, const MantaB200Candidates* set,
                                const int32_t* tokens, const int32_t* mask, int batch, int seq, int pool_order,
                                int metric, int order, int k, int32_t* out_ids, float* out_scores, char** err);

/* Integer accumulators of the packed q8 path for one query: out_acc int32 [rows, 3] =
 * (sum hi*code, sum lo*code, sum code*code) where hi/lo are the two int8 planes the query is split into.
 * Exists so that parity tests can demand bit equality of the integer work. */
int manta_b200_q8_accumulators(MantaB200Runtime* rt, const MantaB200Candidates* set, const uint16_t* query,
                               int32_t* out_acc, char** err);

#ifdef __cplusplus
}
#endif
#endif /* MANTA_B200_H_ */
