// tcgen05 tensor-core scoring pass (query batches large enough to make the scan a dense contraction).
#pragma once

#include "kernels.h"

namespace mb200 {

struct MmaState;  // tensor maps and other per-runtime state of the tensor-core pass

struct MmaArgs {
    CandView cv;
    QueryPrep qp;
    int metric;
    int order;
    int k;
    int nq;
    int64_t row_begin;
    int64_t row_end;
    SelectWs ws;
};

// True when the tensor-core pass handles this candidate set, query count and metric.
bool mma_supported(const CandView& cv, int nq, int metric);
int mma_bucket_count(int sm_count);
int mma_first_burst_rows(int sm_count);
// Pool capacity per query of a filtered tensor-core pass.
int mma_pool_cap(int k);
cudaError_t launch_mma_topk(cudaStream_t st, int sm_count, MmaState** state, const MmaArgs& a, int* launches,
                            const char** why);
void mma_state_destroy(MmaState* s);

}  // namespace mb200
