// tcgen05 tensor-core scoring pass.
#include "mma.h"

namespace mb200 {

struct MmaState {
    int unused;
};

bool mma_supported(const CandView&, int) { return false; }
int mma_bucket_count(int) { return 0; }
int mma_first_burst_rows(int) { return 0; }
cudaError_t launch_mma_topk(cudaStream_t, int, MmaState**, const MmaArgs&, int* launches, const char** why) {
    *launches = 0;
    *why = "tensor-core pass not built";
    return cudaErrorNotSupported;
}
void mma_state_destroy(MmaState* s) { delete s; }

}  // namespace mb200
