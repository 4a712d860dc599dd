// Exact selection of the best k keys of one query's candidate pool by one thread block: the body shared by the
// stand-alone selection kernel (select.cu) and the tail of the streaming scan (stream_scan.cuh), where the last
// block to finish selects for the queries of its launch.  Order: goodness descending, row id ascending -- the
// comparator of topKTensor, runtime/backend/tensor_ops.go:1539-1552.
#pragma once

#include "exchange.cuh"
#include "kernels.h"

namespace mb200 {

// Bitonic sort of n2 (power of two) keys in shared memory, descending.
__device__ __forceinline__ void bitonic_sort_desc(uint64_t* s, int n2) {
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

// Called by every thread of a block (any block size) for query q of the pass.
//  1. keys whose goodness is not below the query's last threshold are compacted into shared memory (the
//     threshold is a lower bound of the k-th best, so nothing that matters is dropped);
//  2. if more than kSelSmemKeys survive, an 8-pass byte-wise radix select over the whole pool finds the
//     exact k-th largest key (keys are unique) and the k keys >= it are compacted instead;
//  3. sort (by rank when the survivors fit one per thread, else bitonic), write ids and scores (and, sharded, store them into every rank's inbox); optionally write the
//     k keys back as the new pool, or leave the query's fill count and threshold at zero for the next pass.
// smem: kSelSmemBytes bytes, 16-byte aligned.  Pool entries are read through L2 (other blocks wrote them).
__device__ __forceinline__ void select_block(const SelectArgs& a, int q, unsigned char* smem) {
    uint64_t* s_keys = reinterpret_cast<uint64_t*>(smem);
    uint32_t* s_hist = reinterpret_cast<uint32_t*>(smem + (size_t)kSelSmemKeys * 8);
    uint32_t* s_scal = s_hist + 256;   // [0] count, [1] digit, [2] remaining rank
    uint32_t* flags = a.flags_out ? a.flags_out : a.ws.flags;

    const int tid = threadIdx.x;
    if (a.src.inbox != nullptr) exchange_collect(a.src, q, a.nq, a.k, a.order, a.ws, flags);   // sharded: lists arrive over peer memory
    const uint32_t total = min(__ldcg(a.ws.count + q), a.ws.cap);
    const uint64_t* pool = a.ws.pool + (size_t)q * a.ws.cap;
    const uint64_t floor_key = (uint64_t)__ldcg(a.ws.thr + q) << 32;
    const uint32_t k = (uint32_t)a.k;

    __syncthreads();
    if (tid == 0) s_scal[0] = 0;
    __syncthreads();
    for (uint32_t i0 = tid; i0 < total; i0 += 4 * blockDim.x) {   // four independent loads at a time
        uint64_t key[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) key[u] = (i0 + u * blockDim.x < total) ? __ldcg(pool + i0 + u * blockDim.x) : 0ull;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (i0 + u * blockDim.x < total && key[u] >= floor_key) {
                uint32_t pos = atomicAdd(&s_scal[0], 1u);
                if (pos < kSelSmemKeys) s_keys[pos] = key[u];
            }
        }
    }
    __syncthreads();
    uint32_t n = s_scal[0];
    __syncthreads();

    if (n > kSelSmemKeys) {
        // radix select of the k-th largest key over the whole pool
        uint64_t prefix = 0, mask = 0;
        if (tid == 0) s_scal[2] = k;
        for (int pass = 7; pass >= 0; --pass) {
            const int shift = pass * 8;
            for (int b = tid; b < 256; b += blockDim.x) s_hist[b] = 0;
            __syncthreads();
            for (uint32_t i = tid; i < total; i += blockDim.x) {
                uint64_t key = __ldcg(pool + i);
                if ((key & mask) == prefix) atomicAdd(&s_hist[(uint32_t)(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                uint32_t rem = s_scal[2], d = 255;
                for (;; --d) {
                    uint32_t c = s_hist[d];
                    if (c >= rem || d == 0) break;
                    rem -= c;
                }
                s_scal[1] = d;
                s_scal[2] = rem;
            }
            __syncthreads();
            prefix |= (uint64_t)s_scal[1] << shift;
            mask |= (uint64_t)255u << shift;
            __syncthreads();
        }
        if (tid == 0) s_scal[0] = 0;
        __syncthreads();
        for (uint32_t i = tid; i < total; i += blockDim.x) {
            uint64_t key = __ldcg(pool + i);
            if (key >= prefix) {
                uint32_t pos = atomicAdd(&s_scal[0], 1u);
                if (pos < kSelSmemKeys) s_keys[pos] = key;
            }
        }
        __syncthreads();
        n = min(s_scal[0], (uint32_t)kSelSmemKeys);
        __syncthreads();
    }

    if (n <= blockDim.x) {
        // the usual case, a few hundred survivors at most: every thread ranks one key against all the others (keys are
        // unique) and stores it at its rank
        const uint64_t mine = ((uint32_t)tid < n) ? s_keys[tid] : 0ull;
        uint32_t rank = 0;
        if ((uint32_t)tid < n) {
#pragma unroll 4
            for (uint32_t j = 0; j < n; ++j) rank += (s_keys[j] > mine) ? 1u : 0u;
        }
        __syncthreads();
        if ((uint32_t)tid < n) s_keys[rank] = mine;
        __syncthreads();
    } else {
        int n2 = 1;
        while ((uint32_t)n2 < n) n2 <<= 1;
        for (int i = n + tid; i < n2; i += blockDim.x) s_keys[i] = 0;
        bitonic_sort_desc(s_keys, n2);
    }

    if (n < k && tid == 0) flags[kFlagInternal] = 1u;
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
        // the block that stores the last query publishes the step's status and epoch to every rank
        __threadfence_system();
        __syncthreads();
        if (tid == 0) {
            const uint32_t prev = atomicAdd(a.sink.done, 1u);
            if (prev + 1u == (uint32_t)a.nq) {
                *a.sink.done = 0u;
                // a shard pass whose pool overflowed holds an incomplete list: say so next to the epoch, so that every
                // rank's merge reports it
                const uint32_t status = __ldcg(a.ws.flags + kFlagOverflow) ? 1u : 0u;
                __threadfence_system();
                for (int r = 0; r < a.sink.world; ++r) {
                    uint32_t* word = reinterpret_cast<uint32_t*>(a.sink.inbox[r] + exchange_flag_offset(a.sink.slot_words, a.sink.world, a.sink.parity, a.sink.rank));
                    word[1] = status;
                    st_release_sys_u32(word, a.sink.epoch);
                }
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
    } else if (a.reset_after) {
        if (tid == 0) {
            a.ws.count[q] = 0;
            a.ws.thr[q] = 0;
        }
    }
    __syncthreads();
}

}  // namespace mb200
