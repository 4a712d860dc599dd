// Host-side launchers of the kernels (one translation unit per kernel family).
#pragma once

#include "common.cuh"

namespace mb200 {

void count_launch();
// Records the configuration of a scan launch issued by the calling thread (read back by the runtime that issued it).
void note_scan_launch(const char* kernel, int grid, int block, size_t shared_bytes);

struct QueryPrep {
    const QueryHeader* headers;  // [nq]
    const float* qf32;           // [nq][cols]
    const int8_t* plane_hi;      // [nq][plane_stride]  (q8/q4 candidates)
    const int8_t* plane_lo;      // [nq][plane_stride]
    int plane_stride;            // bytes per query in a plane (multiple of 32)
    const float* lo_norm;        // [nq] norm of the low plane, rounded up a shade (q8/q4 candidates)
    const void* queries_f16;     // [nq][cols] the queries as they came
    int nq;
};

void launch_query_prep(cudaStream_t st, const void* d_queries_f16, int nq, int cols, int layout, int plane_stride, float* lo_norm,
                       QueryHeader* headers, float* qf32, int8_t* plane_hi, int8_t* plane_lo, const SelectWs& ws,
                       int reset_ws);
void launch_row_stats(cudaStream_t st, const CandView& cv, void* stats);
void launch_pack_q8(cudaStream_t st, const void* d_src, bool src_f16, int64_t rows, int cols, int dst_stride,
                    int8_t* d_codes, float* d_scales);
void launch_pack_q4(cudaStream_t st, const void* d_src, bool src_f16, int64_t rows, int cols, uint8_t* d_codes,
                    uint16_t* d_scales);
void launch_gather_rows(cudaStream_t st, const CandView& cv, const int32_t* d_ids, int64_t n, float* d_out,
                        int32_t* d_bad_id, uint32_t* d_bad_flag);

// Per-query candidate sets ([Q,D] x [Q,N,D], float32 docs): scores [Q,N] and / or the keys of every row in the
// selection pools (ws.cap >= rows).
cudaError_t launch_score_batched(cudaStream_t st, int sm_count, int metric, const float* d_queries, const float* d_docs, int nq,
                                 int64_t rows, int cols, int order, float* d_out_scores, const SelectWs& ws, int fill_pool);

// Embedding front end: gather -> matmul -> masked mean_pool / normalize (order 0: normalize(mean_pool(x)),
// 1: mean_pool(normalize(x))); writes the pooled rows as f32 and / or f16.
// d_token_norms (order 1 only, may be NULL): [batch*seq] norms of the tokens' projected rows from
// launch_embed_token_norms; with them the pool runs on the embedding rows and one row per batch element is projected.
cudaError_t launch_embed_pooled(cudaStream_t st, const void* table_f16, int vocab, int dim, const void* proj_f16, int out_dim,
                                const int32_t* d_tokens, const int32_t* d_mask, int batch, int seq, int order,
                                const float* d_token_norms, float* d_out_f32, void* d_out_f16, int32_t* d_bad_token,
                                uint32_t* d_bad_flag);
// Tensor-core projection of every token row, reduced to the row norms (embed_mma.cu).  proj_t is the projection
// transposed to [out_dim][dim].  A wait that runs out raises *d_flag to 2.
bool embed_mma_supported(int dim, int out_dim);
cudaError_t launch_transpose_f16(cudaStream_t st, const void* src, int rows, int cols, void* dst);
cudaError_t launch_embed_token_norms(cudaStream_t st, const void* table_f16, int vocab, int dim, const void* proj_t_f16, int out_dim,
                                     const int32_t* d_tokens, int64_t n_tokens, float* d_norms, uint32_t* d_flag);

// Streaming scoring kernel (stream_scan.cuh).  mode: what the epilogue does with a score.
enum { kModeScores = 0, kModeTopk = 1, kModeAccum = 2 };
// One query per launch runs 16 warps per block on a two-stage ring (one tile in flight per warp while one is consumed:
// 16 tiles per SM); two or four queries per launch need more registers per thread and run 8 warps on a three-stage
// ring.  Every warp owns one bucket (running maximum) per query, two when a block has 8 warps, so that a grid of one
// block per SM always offers more buckets than the largest k.
constexpr int scan_warps(int qt) { return qt == 1 ? 16 : 8; }
constexpr int scan_bucket_slots(int qt) { return qt == 1 ? 1 : 2; }
constexpr int kScanMaxBucketsPerBlock = 16;   // scan_warps * scan_bucket_slots for either form
constexpr int kScanClaimMinTiles = 16;  // tiles per warp from which the last part of a fused pass is dealt on demand
constexpr int kScanRefreshWords = 2560; // bucket maxima a threshold refresh can stage in shared memory
constexpr int kSelSmemKeys = 4096;      // keys the selection sorts in shared memory
// shared memory a block needs for select_block: keys, a 256-bin histogram, four scalars
constexpr size_t kSelSmemBytes = (size_t)kSelSmemKeys * 8 + 256 * 4 + 16;

// Where a shard's selection also stores its k results: slot [parity][rank] of every rank's exchange inbox (peer
// stores), followed by the status and epoch words of that slot once all queries are written.  world == 0: no sink.
struct ExchangeSink {
    unsigned char* inbox[16] = {};
    size_t slot_words = 0;
    int world = 0;
    int rank = 0;
    int parity = 0;
    uint32_t epoch = 0;
    uint32_t* done = nullptr;   // device counter of the queries that have been stored (returns to 0)
};

// Geometry of a launch, chosen on the host (stream_scan_geometry).
struct ScanGeometry {
    int rows_per_tile;   // R
    int lpr_shift;       // log2(32 / R)
    int cstride;         // row stride inside a stage, in 16-byte chunks (>= chunks, padded against bank conflicts)
    int stage_bytes;     // codes + per-row values, multiple of 16
    int scale_off;       // q4: byte offset of the block scales inside a stage
    int scale_unit;      // q4: 16 or 4 = size of the asynchronous copies that bring the block scales, 0 = read them from global memory
    int stat_off;        // byte offset of the R row statistics
    int rscale_off;      // q8: byte offset of the R row scales
    int q_bytes;         // shared memory per query (planes or f32 values), multiple of 128
    int warps;           // warps per block
    int stages;          // ring depth per warp (2..4): stages - 1 tiles in flight while one is consumed
};

struct StreamArgs {
    CandView cv;
    const __half* queries;   // [nq][cols] device, IEEE half
    int q0;                  // first query of this launch
    int qt;                  // queries in this launch (<= QT)
    int metric;
    int order;
    int k;
    int mode;                // kModeScores / kModeTopk / kModeAccum
    int64_t row_begin;       // rows [row_begin, row_end) of the set are scanned
    int64_t row_end;
    SelectWs ws;             // kModeTopk
    float* out_scores;       // kModeScores: [nq][rows]
    int32_t* out_acc;        // kModeAccum: [rows][3]
    ScanGeometry g;
    // tail of a fused pass (kModeTopk): the last block selects, stores and cleans the workspace
    int fused_select;
    int nq_total;            // queries of the whole pass (the exchange's epoch goes out after the last one)
    uint32_t* done_blocks;   // two device counters, zero between launches: [0] blocks that finished, [1] tiles dealt on demand
    uint32_t* host_flags;    // pinned host words that receive the pass's raised flags (sticky until the host clears them)
    int32_t* out_ids;        // [nq][k]
    float* out_topk_scores;  // [nq][k]
    ExchangeSink sink;
};

// Dynamic shared memory a block of the scan may ask for: the 227 KB a block can have, less 1 KB for the kernel's static
// shared variables.
constexpr size_t kScanSmemLimit = 232448 - 1024;

__host__ __device__ constexpr int scan_padded_stride(int chunks, int lpr) {
    if (lpr >= 8) return chunks;
    // the 8 lanes that share a shared-memory wavefront read rows r, r+1, ... at chunk offsets 0..lpr-1: they fall into
    // distinct 16-byte bank groups when the stride is congruent to lpr modulo 2*lpr
    return chunks + ((lpr - chunks % (2 * lpr)) + 2 * lpr) % (2 * lpr);
}

// Picks the tile geometry for a candidate layout and a launch of qt (1, 2 or 4) queries: as many rows per tile as the
// block's share of shared memory allows (up to 32), fewer warps only when a single row does not fit otherwise.
// Returns false when even one warp with one row per tile does not fit.
inline bool stream_scan_geometry(const CandView& cv, int qt, int64_t row_begin, ScanGeometry* g, size_t* smem_bytes) {
    const int C = cv.chunks;
    if (C <= 0) return false;
    (void)row_begin;   // a row's block scales start on a multiple of 2*C bytes, so any first row is aligned for the copy units below
    const int per_chunk = (cv.layout == MANTA_B200_LAYOUT_Q4_B32_F16) ? 64 : 32;   // q8: two planes of 16 bytes; q4: two of 32; f16: 8 floats
    g->q_bytes = (C * per_chunk + 127) / 128 * 128;
    const size_t fixed = 256 + (size_t)qt * g->q_bytes + (size_t)(kScanRefreshWords + 256) * 4;   // headers, queries, staged maxima + histogram
    if (fixed >= kScanSmemLimit) return false;
    auto stage_bytes_for = [&](int R, ScanGeometry* out) {
        const int lpr = 32 / R;
        int shift = 0;
        while ((1 << shift) < lpr) ++shift;
        out->rows_per_tile = R;
        out->lpr_shift = shift;
        out->cstride = scan_padded_stride(C, lpr);
        int off = R * out->cstride * 16;
        out->scale_off = 0;
        out->scale_unit = 0;
        if (cv.layout == MANTA_B200_LAYOUT_Q4_B32_F16) {
            const uintptr_t sp = (uintptr_t)cv.scales;
            if (C % 8 == 0 && (sp & 15) == 0) out->scale_unit = 16;
            else if (C % 2 == 0 && (sp & 3) == 0) out->scale_unit = 4;
            if (out->scale_unit) {
                out->scale_off = off;
                off += (R * C * 2 + 15) / 16 * 16;
            }
        }
        out->stat_off = off;
        off += (R * 4 + 15) / 16 * 16;
        out->rscale_off = off;
        if (cv.layout == MANTA_B200_LAYOUT_Q8_ROW_F32) off += (R * 4 + 15) / 16 * 16;
        out->stage_bytes = off;
    };
    // Measured on B200: what counts is the height of the tile (the per-tile work of a warp -- epilogue, bookkeeping,
    // one round trip of latency -- is paid once per tile whatever its size), not the depth of the ring, so the ring is
    // two stages deep (one tile in flight per warp while one is consumed, 16 warps per SM) and the tile as tall as the
    // block's shared memory allows.  Deeper rings with shorter tiles were 1.4x to 1.7x slower on every layout.
    for (int warps = scan_warps(qt); warps >= 1; warps >>= 1) {
        long best = -1;
        ScanGeometry pick{};
        const int S = (qt == 1) ? 2 : 3;
        const size_t budget = (kScanSmemLimit - fixed) / ((size_t)warps * S);
        for (int R = 32; R >= 1; R >>= 1) {
            ScanGeometry t = *g;
            stage_bytes_for(R, &t);
            if ((size_t)t.stage_bytes > budget) continue;
            best = (long)R;
            pick = t;
            pick.stages = S;
            break;
        }
        if (best < 0) continue;
        pick.warps = warps;
        *g = pick;
        size_t ring = (size_t)warps * pick.stages * pick.stage_bytes;
        if (ring < kSelSmemBytes) ring = kSelSmemBytes;   // the tail's selection reuses the ring
        *smem_bytes = fixed + ring;
        return true;
    }
    return false;
}

// Buckets (running maxima) per query the workspace must provide for any launch of the scan on this device.
inline int stream_bucket_count(int sm_count) { return sm_count * kScanMaxBucketsPerBlock; }
// Runs the scan for a.qt <= 4 queries; the geometry is filled in by the launcher.
cudaError_t launch_stream_scan(cudaStream_t st, int sm_count, const StreamArgs& a);
// Zeroes the selection workspace of nq queries (fill counts, thresholds, bucket maxima, flags, the block counter).
cudaError_t launch_ws_reset(cudaStream_t st, const SelectWs& ws, int nq, uint32_t* done_blocks);

// Final selection: best k keys of each query's pool, sorted best first.  With write_back the k keys are
// also written to the front of the pool, count becomes k and the threshold becomes the k-th goodness
// (used between row chunks).  pool_override/count_override select a different key source (merge of lists).
// Per-shard lists waiting in this rank's exchange inbox (exchange.cu); inbox == nullptr: the pool is already filled.
struct ExchangeSource {
    const unsigned char* inbox = nullptr;
    size_t slot_words = 0;   // int32 words per (parity, rank) slot
    int world = 0;
    int parity = 0;
    uint32_t epoch = 0;      // value every slot's word must carry before the lists are read
    uint32_t spin_limit = 0; // 200 ns naps before a missing list is reported
};

struct SelectArgs {
    SelectWs ws;
    int nq;
    int k;
    int order;
    int write_back;
    int32_t* out_ids;    // [nq][k] or null
    float* out_scores;   // [nq][k] or null
    ExchangeSource src;  // optional: fill the pool from the exchange inbox first
    ExchangeSink sink;   // optional: also store the results into every rank's inbox
    uint32_t* flags_out = nullptr;  // where this selection raises its flags (null: ws.flags); may be pinned host memory
    int reset_after = 0; // leave the query's fill count and threshold at zero (the workspace is clean for the next pass)
};
cudaError_t launch_select(cudaStream_t st, const SelectArgs& a);

// Builds keys from gathered per-shard lists: pool[q][l*k + i] = key(ids[l][q][i], scores[l][q][i]).
cudaError_t launch_lists_to_pool(cudaStream_t st, const int32_t* d_ids, const float* d_scores, int lists,
                                 int64_t list_stride, int nq, int k, int order, const SelectWs& ws);

}  // namespace mb200
