// Instantiations of the streaming scoring kernel for q4 candidates (one translation unit per layout so the
// three families compile in parallel).
#include "gemv.cuh"

namespace mb200 {
cudaError_t launch_gemv_q4(cudaStream_t st, int sm_count, const GemvArgs& a, int mode) {
    return launch_gemv_layout<MANTA_B200_LAYOUT_Q4_B32_F16>(st, sm_count, a, mode);
}
}  // namespace mb200
