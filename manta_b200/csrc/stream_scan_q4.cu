// Instantiations of the streaming scan for q4 candidate rows.
#include "stream_scan.cuh"

namespace mb200 {

cudaError_t launch_stream_scan_q4(cudaStream_t st, int sm_count, const StreamArgs& a) {
    return launch_stream_scan_layout<MANTA_B200_LAYOUT_Q4_B32_F16>(st, sm_count, a);
}

}  // namespace mb200
