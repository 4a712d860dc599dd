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
    int nq;
};

void launch_query_prep(cudaStream_t st, const void* d_queries_f16, int nq, int cols, int layout, int plane_stride,
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
cudaError_t launch_embed_pooled(cudaStream_t st, const void* table_f16, int vocab, int dim, const void* proj_f16, int out_dim,
                                const int32_t* d_tokens, const int32_t* d_mask, int batch, int seq, int order, float* d_out_f32,
                                void* d_out_f16, int32_t* d_bad_token, uint32_t* d_bad_flag);

// Streaming (GEMV) scoring kernel.  mode: what the epilogue does with a score.
enum { kModeScores = 0, kModeTopk = 1, kModeAccum = 2 };
struct GemvArgs {
    CandView cv;
    QueryPrep qp;
    int q0;            // first query of this pass
    int qt;            // queries in this pass (1, 2 or 4)
    int metric;
    int order;
    int k;
    int64_t row_begin; // rows [row_begin, row_end) of the set are scanned
    int64_t row_end;
    SelectWs ws;       // kModeTopk
    float* out_scores; // kModeScores: [nq][rows]
    int32_t* out_acc;  // kModeAccum: [rows][3]
    int no_startup_wait; // debugging: do not wait for the first threshold after two unfiltered tiles
};
// How a row of `chunks` 16-byte chunks is split over lanes: lpr lanes per row, cpl chunks per lane, u rows in
// flight per lane group.  Smallest padded footprint first, then the wider group.
struct GemvShape {
    int lpr, cpl, u;
};
inline bool pick_gemv_shape(int chunks, GemvShape* out) {
    const int lprs[3] = {32, 16, 8};
    int best_cost = 1 << 30;
    GemvShape best{0, 0, 0};
    bool ok = false;
    for (int i = 0; i < 3; ++i) {
        int lpr = lprs[i];
        int cpl = (chunks + lpr - 1) / lpr;
        if (cpl > 4 && !(lpr == 32 && cpl <= 8)) continue;
        if (cpl > 4) cpl = 8;
        int cost = lpr * cpl;
        if (cost < best_cost) {
            best_cost = cost;
            best.lpr = lpr;
            best.cpl = cpl;
            ok = true;
        }
    }
    if (ok) {
        best.u = (best.cpl == 1) ? 8 : (best.cpl == 2) ? 4 : (best.cpl <= 4) ? 2 : 1;
        if (out) *out = best;
    }
    return ok;
}

// Number of buckets (running maxima) the kernel keeps per query for a given grid; the workspace must
// provide at least this many.
int gemv_grid_size(int sm_count);
int gemv_bucket_count(int sm_count);
// Rows that can be scanned before a useful threshold exists (every one of them is appended).
int gemv_first_burst_rows(int sm_count, int chunks);
cudaError_t launch_gemv(cudaStream_t st, int sm_count, const GemvArgs& a, int mode);

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

// Where a shard's selection also stores its k results: slot [parity][rank] of every rank's exchange inbox (peer
// stores), followed by the epoch word of that slot once all queries are written.  world == 0: no sink.
struct ExchangeSink {
    unsigned char* inbox[16] = {};
    size_t slot_words = 0;
    int world = 0;
    int rank = 0;
    int parity = 0;
    uint32_t epoch = 0;
    uint32_t* done = nullptr;   // device counter of the blocks that have stored their query (returns to 0)
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
};
cudaError_t launch_select(cudaStream_t st, const SelectArgs& a);

// Builds keys from gathered per-shard lists: pool[q][l*k + i] = key(ids[l][q][i], scores[l][q][i]).
cudaError_t launch_lists_to_pool(cudaStream_t st, const int32_t* d_ids, const float* d_scores, int lists,
                                 int64_t list_stride, int nq, int k, int order, const SelectWs& ws);

}  // namespace mb200
