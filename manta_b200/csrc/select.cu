// Stand-alone selection kernel (one block per query) and the conversion of gathered per-shard lists into pool keys.
#include "select.cuh"

namespace mb200 {

constexpr int kSelThreads = 1024;

__global__ void __launch_bounds__(kSelThreads) select_kernel(const SelectArgs a) {
    __shared__ __align__(16) unsigned char s_sel[kSelSmemBytes];
    select_block(a, blockIdx.x, s_sel);
}

__global__ void lists_to_pool_kernel(const int32_t* __restrict__ ids, const float* __restrict__ scores, int lists,
                                     int64_t list_stride, int nq, int k, int order, SelectWs ws) {
    const int q = blockIdx.x;
    const float sign = (order == MANTA_B200_ORDER_SMALLEST) ? -1.0f : 1.0f;
    const int per = lists * k;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        const int l = i / k, j = i % k;
        const size_t src = (size_t)l * list_stride + (size_t)q * k + j;
        const int32_t id = ids[src];
        // entries a shard could not fill (id < 0) rank below everything
        ws.pool[(size_t)q * ws.cap + i] = (id < 0) ? 0ull : make_key(scores[src] * sign + 0.0f, id);
    }
    if (threadIdx.x == 0) {
        ws.count[q] = (uint32_t)per;
        ws.thr[q] = 0;
        if (q == 0) {
            for (int f = 0; f < kNumFlags; ++f) ws.flags[f] = 0;
        }
    }
}

cudaError_t launch_select(cudaStream_t st, const SelectArgs& a) {
    select_kernel<<<a.nq, kSelThreads, 0, st>>>(a);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_lists_to_pool(cudaStream_t st, const int32_t* d_ids, const float* d_scores, int lists,
                                 int64_t list_stride, int nq, int k, int order, const SelectWs& ws) {
    lists_to_pool_kernel<<<nq, 256, 0, st>>>(d_ids, d_scores, lists, list_stride, nq, k, order, ws);
    count_launch();
    return cudaGetLastError();
}

}  // namespace mb200
