// Per-query candidate sets: queries [Q,D] against docs [Q,N,D], the "batched" form of the score builtins
// (scoreLayout, runtime/backend/tensor_ops.go:1492-1521; the reference's CUDA backend runs it on the host,
// runtime/backends/cuda/cuda.go:961-976).  The docs of this form are request inputs, not bound parameters: they
// arrive as float32 (the reference's tensor storage) and are read once, so the kernel is a plain streaming pass --
// one warp per (query, row), float4 loads, f32 accumulation, the finishing arithmetic in f64 like the host math
// (:1405-1476) -- and optionally writes every row as a key of the query's selection pool for the fused top-k.
#include "common.cuh"
#include "kernels.h"

namespace mb200 {

constexpr int kBatchedThreads = 256;

template <int METRIC>
__global__ void __launch_bounds__(kBatchedThreads) score_batched_kernel(const float* __restrict__ queries, const float* __restrict__ docs,
                                                                        int nq, int64_t rows, int cols, int order,
                                                                        float* __restrict__ out_scores, SelectWs ws, int fill_pool) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (kBatchedThreads / 32);
    const int64_t total = (int64_t)nq * rows;
    const float sign = (order == MANTA_B200_ORDER_SMALLEST) ? -1.0f : 1.0f;
    const bool vec = (cols & 3) == 0 && (((uintptr_t)queries | (uintptr_t)docs) & 15) == 0;
    for (int64_t w = (int64_t)blockIdx.x * (kBatchedThreads / 32) + (threadIdx.x >> 5); w < total; w += warps) {
        const int q = (int)(w / rows);
        const int64_t r = w - (int64_t)q * rows;
        const float* qv = queries + (size_t)q * cols;
        const float* dv = docs + (size_t)w * cols;
        float acc = 0.0f, qq = 0.0f, dd = 0.0f;
        auto step = [&](float a, float b) {
            if (METRIC == MANTA_B200_METRIC_L2_DISTANCE) {
                const float diff = a - b;
                acc = fmaf(diff, diff, acc);
            } else {
                acc = fmaf(a, b, acc);
                if (METRIC == MANTA_B200_METRIC_COSINE) {
                    qq = fmaf(a, a, qq);
                    dd = fmaf(b, b, dd);
                }
            }
        };
        if (vec) {
            for (int c = lane * 4; c < cols; c += 128) {
                const float4 a = *reinterpret_cast<const float4*>(qv + c);
                const float4 b = __ldcs(reinterpret_cast<const float4*>(dv + c));
                step(a.x, b.x);
                step(a.y, b.y);
                step(a.z, b.z);
                step(a.w, b.w);
            }
        } else {
            for (int c = lane; c < cols; c += 32) step(qv[c], dv[c]);
        }
        for (int off = 16; off > 0; off >>= 1) {
            acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (METRIC == MANTA_B200_METRIC_COSINE) {
                qq += __shfl_xor_sync(0xffffffffu, qq, off);
                dd += __shfl_xor_sync(0xffffffffu, dd, off);
            }
        }
        if (lane == 0) {
            float score;
            if (METRIC == MANTA_B200_METRIC_DOT) {
                score = acc;
            } else if (METRIC == MANTA_B200_METRIC_COSINE) {
                // zero norm on either side scores exactly 0 (tensor_ops.go:1420-1424)
                score = (qq == 0.0f || dd == 0.0f) ? 0.0f : (float)((double)acc / (sqrt((double)qq) * sqrt((double)dd)));
            } else {
                score = (float)sqrt((double)acc);
            }
            if (out_scores) out_scores[w] = score;
            if (fill_pool) {
                ws.pool[(size_t)q * ws.cap + r] = make_key(score * sign + 0.0f, (int32_t)r);
                if (r == 0) {
                    ws.count[q] = (uint32_t)rows;
                    ws.thr[q] = 0;
                    if (q == 0)
                        for (int f = 0; f < kNumFlags; ++f) ws.flags[f] = 0;
                }
            }
        }
    }
}

cudaError_t launch_score_batched(cudaStream_t st, int sm_count, int metric, const float* d_queries, const float* d_docs, int nq,
                                 int64_t rows, int cols, int order, float* d_out_scores, const SelectWs& ws, int fill_pool) {
    const int64_t total = (int64_t)nq * rows;
    const int64_t want = (total + (kBatchedThreads / 32) - 1) / (kBatchedThreads / 32);
    const int64_t cap = (int64_t)sm_count * 8;  // eight resident CTAs per SM, grid-stride beyond that
    const int grid = (int)(want < cap ? want : cap);
    switch (metric) {
        case MANTA_B200_METRIC_DOT:
            score_batched_kernel<MANTA_B200_METRIC_DOT><<<grid, kBatchedThreads, 0, st>>>(d_queries, d_docs, nq, rows, cols, order,
                                                                                     d_out_scores, ws, fill_pool);
            break;
        case MANTA_B200_METRIC_COSINE:
            score_batched_kernel<MANTA_B200_METRIC_COSINE><<<grid, kBatchedThreads, 0, st>>>(d_queries, d_docs, nq, rows, cols, order,
                                                                                        d_out_scores, ws, fill_pool);
            break;
        default:
            score_batched_kernel<MANTA_B200_METRIC_L2_DISTANCE><<<grid, kBatchedThreads, 0, st>>>(d_queries, d_docs, nq, rows, cols, order,
                                                                                             d_out_scores, ws, fill_pool);
            break;
    }
    count_launch();
    note_scan_launch("score_batched_kernel", grid, kBatchedThreads, 0);
    return cudaGetLastError();
}

}  // namespace mb200
