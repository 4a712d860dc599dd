// Final selection: exact best-k of each query's candidate pool, sorted best first (goodness descending,
// row id ascending -- the comparator of topKTensor, runtime/backend/tensor_ops.go:1539-1552).
#include "kernels.h"
#include "exchange.cuh"

namespace mb200 {

constexpr int kSelThreads = 1024;
constexpr int kSelSmemKeys = 4096;

// Bitonic sort of n2 (power of two) keys in shared memory, descending.
__device__ void bitonic_sort_desc(uint64_t* s, int n2) {
    for (int size = 2; size <= n2; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (int t = threadIdx.x; t < (n2 >> 1); t += blockDim.x) {
                int lo = 2 * t - (t & (stride - 1));
                int hi = lo + stride;
                bool desc = ((lo & size) == 0);
                uint64_t a = s[lo], b = s[hi];
                if ((a < b) == desc) {
                    s[lo] = b;
                    s[hi] = a;
                }
            }
        }
    }
    __syncthreads();
}

// One CTA per query.
//  1. keys whose goodness is not below the query's last threshold are compacted into shared memory (the
//     threshold is a lower bound of the k-th best, so nothing that matters is dropped);
//  2. if more than kSelSmemKeys survive, an 8-pass byte-wise radix select over the whole pool finds the
//     exact k-th largest key (keys are unique) and the k keys >= it are compacted instead;
//  3. bitonic sort, write ids and scores; optionally write the k keys back as the new pool.
__global__ void __launch_bounds__(kSelThreads) select_kernel(const SelectArgs a) {
    __shared__ uint64_t s_keys[kSelSmemKeys];
    __shared__ uint32_t s_hist[256];
    __shared__ uint32_t s_cnt;
    __shared__ uint32_t s_digit, s_krem;

    const int q = blockIdx.x;
    const int tid = threadIdx.x;
    if (a.src.inbox != nullptr) exchange_collect(a.src, q, a.nq, a.k, a.order, a.ws);   // sharded: lists arrive over peer memory
    const uint32_t total = min(a.ws.count[q], a.ws.cap);
    const uint64_t* pool = a.ws.pool + (size_t)q * a.ws.cap;
    const uint64_t floor_key = (uint64_t)a.ws.thr[q] << 32;
    const uint32_t k = (uint32_t)a.k;

    if (tid == 0) s_cnt = 0;
    __syncthreads();
    for (uint32_t i = tid; i < total; i += blockDim.x) {
        uint64_t key = pool[i];
        if (key >= floor_key) {
            uint32_t pos = atomicAdd(&s_cnt, 1u);
            if (pos < kSelSmemKeys) s_keys[pos] = key;
        }
    }
    __syncthreads();
    uint32_t n = s_cnt;
    __syncthreads();

    if (n > kSelSmemKeys) {
        // radix select of the k-th largest key over the whole pool
        uint64_t prefix = 0, mask = 0;
        if (tid == 0) s_krem = k;
        for (int pass = 7; pass >= 0; --pass) {
            const int shift = pass * 8;
            if (tid < 256) s_hist[tid] = 0;
            __syncthreads();
            for (uint32_t i = tid; i < total; i += blockDim.x) {
                uint64_t key = pool[i];
                if ((key & mask) == prefix) atomicAdd(&s_hist[(uint32_t)(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                uint32_t rem = s_krem, d = 255;
                for (;; --d) {
                    uint32_t c = s_hist[d];
                    if (c >= rem || d == 0) break;
                    rem -= c;
                }
                s_digit = d;
                s_krem = rem;
            }
            __syncthreads();
            prefix |= (uint64_t)s_digit << shift;
            mask |= (uint64_t)255u << shift;
            __syncthreads();
        }
        if (tid == 0) s_cnt = 0;
        __syncthreads();
        for (uint32_t i = tid; i < total; i += blockDim.x) {
            uint64_t key = pool[i];
            if (key >= prefix) {
                uint32_t pos = atomicAdd(&s_cnt, 1u);
                if (pos < kSelSmemKeys) s_keys[pos] = key;
            }
        }
        __syncthreads();
        n = min(s_cnt, (uint32_t)kSelSmemKeys);
        __syncthreads();
    }

    int n2 = 1;
    while ((uint32_t)n2 < n) n2 <<= 1;
    for (int i = n + tid; i < n2; i += blockDim.x) s_keys[i] = 0;
    bitonic_sort_desc(s_keys, n2);

    if (n < k && tid == 0) a.ws.flags[kFlagInternal] = 1u;
    const float sign = (a.order == MANTA_B200_ORDER_SMALLEST) ? -1.0f : 1.0f;
    for (uint32_t i = tid; i < k; i += blockDim.x) {
        const uint64_t key = (i < n) ? s_keys[i] : 0;
        const bool have = key != 0;
        const int32_t rid = have ? key_id(key) : -1;
        const float rsc = have ? (key_goodness(key) * sign + 0.0f) : 0.0f;
        if (a.out_ids) a.out_ids[(size_t)q * k + i] = rid;
        if (a.out_scores) a.out_scores[(size_t)q * k + i] = rsc;
        // sharded: the same pair goes straight into every rank's inbox over peer memory
        for (int r = 0; r < a.sink.world; ++r) {
            int32_t* dst = reinterpret_cast<int32_t*>(a.sink.inbox[r] + exchange_slot_offset(a.sink.slot_words, a.sink.world, a.sink.parity, a.sink.rank));
            dst[(size_t)q * k + i] = rid;
            dst[(size_t)a.nq * k + (size_t)q * k + i] = __float_as_int(rsc);
        }
    }
    if (a.sink.world > 0) {
        // the block that stores the last query publishes the epoch to every rank
        __threadfence_system();
        __syncthreads();
        if (tid == 0) {
            const uint32_t prev = atomicAdd(a.sink.done, 1u);
            if (prev + 1u == (uint32_t)a.nq) {
                *a.sink.done = 0u;
                __threadfence_system();
                for (int r = 0; r < a.sink.world; ++r)
                    st_release_sys_u32(reinterpret_cast<uint32_t*>(a.sink.inbox[r] + exchange_flag_offset(a.sink.slot_words, a.sink.world, a.sink.parity, a.sink.rank)),
                                       a.sink.epoch);
            }
        }
    }
    if (a.write_back) {
        __syncthreads();  // every read of the pool is done
        uint64_t* wpool = a.ws.pool + (size_t)q * a.ws.cap;
        const uint32_t keep = min(n, k);
        for (uint32_t i = tid; i < keep; i += blockDim.x) wpool[i] = s_keys[i];
        if (tid == 0) {
            a.ws.count[q] = keep;
            if (keep == k) a.ws.thr[q] = max(a.ws.thr[q], (uint32_t)(s_keys[k - 1] >> 32));
        }
    }
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
