// Accessors into the opaque handles of api.cu for the other translation units of the library.
#pragma once

#include <mutex>

#include "kernels.h"

namespace mb200 {

struct RuntimeInfo {
    int device;
    int sm_count;
    cudaStream_t stream;
    uint32_t* h_flags;  // 16 pinned host words owned by the runtime; words 4..7 are free for callers of this header
    std::mutex* mu;
};
RuntimeInfo runtime_info(MantaB200Runtime* rt);
const CandView* candidates_view(const MantaB200Candidates* set);
int candidates_device(const MantaB200Candidates* set);

}  // namespace mb200
