// Accessors into the opaque handles of api.cu for the other translation units of the library.
#pragma once

#include <mutex>

#include "kernels.h"

namespace mb200 {

struct RuntimeInfo {
    int device;
    int sm_count;
    cudaStream_t stream;
    uint32_t* h_flags;  // 16 pinned host words owned by the runtime: 0..3 fused pass, 4..7 exchange merge, 8..9 row
                        // gather, 10..11 embedding front end, 12..15 the allocation-free entry point
    bool* static_flags_pending;  // set when an asynchronous allocation-free pass has copied its flags to words 12..15
    std::mutex* mu;
};
RuntimeInfo runtime_info(MantaB200Runtime* rt);
const CandView* candidates_view(const MantaB200Candidates* set);
int candidates_device(const MantaB200Candidates* set);

}  // namespace mb200
