// Instantiations of the streaming scoring kernel for f16 candidates (one translation unit per layout so the
// three families compile in parallel).
#include "gemv.cuh"

namespace mb200 {
cudaError_t launch_gemv_f16(cudaStream_t st, int sm_count, const GemvArgs& a, int mode) {
    return launch_gemv_layout<MANTA_B200_LAYOUT_F16>(st, sm_count, a, mode);
}
}  // namespace mb200
