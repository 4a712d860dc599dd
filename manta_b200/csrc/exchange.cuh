// Device side of the list exchange over peer memory: inbox layout, system-scope flag accesses, and the prologue
// of the selection kernel that waits for every rank's list and turns them into pool keys.
#pragma once

#include "common.cuh"
#include "kernels.h"

namespace mb200 {

__host__ __device__ inline size_t exchange_slot_offset(size_t slot_words, int world, int parity, int r) {
    return ((size_t)parity * world + r) * slot_words * 4;
}
__host__ __device__ inline size_t exchange_flag_offset(size_t slot_words, int world, int parity, int r) {
    return (size_t)2 * world * slot_words * 4 + ((size_t)parity * world + r) * 64;
}

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Called by all threads of the block that selects for query q.  Waits (bounded) until every rank's slot of this
// parity carries the epoch, then writes the keys of all lists into the query's pool (entries a shard could not
// fill, id < 0, rank below everything).  A list that does not arrive raises the time-out flag and empties the pool;
// a list whose sender marked it incomplete (its candidate pool overflowed) raises the peer-overflow flag.
__device__ __forceinline__ void exchange_collect(const ExchangeSource& src, int q, int nq, int k, int order, const SelectWs& ws,
                                                 uint32_t* flags) {
    __shared__ int ok_s, bad_s;
    if (threadIdx.x == 0) {
        ok_s = 1;
        bad_s = 0;
    }
    __syncthreads();
    if ((int)threadIdx.x < src.world) {
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(src.inbox + exchange_flag_offset(src.slot_words, src.world, src.parity, threadIdx.x));
        uint32_t spin = 0;
        bool arrived = true;
        while (ld_acquire_sys_u32(flag) != src.epoch) {
            if (++spin > src.spin_limit) {
                ok_s = 0;
                arrived = false;
                break;
            }
            __nanosleep(200);
        }
        if (arrived && __ldcv(flag + 1) != 0u) bad_s = 1;
    }
    __syncthreads();
    const float sign = (order == MANTA_B200_ORDER_SMALLEST) ? -1.0f : 1.0f;
    const int n = nq * k;
    const int per = src.world * k;
    if (ok_s) {
        for (int i = threadIdx.x; i < per; i += blockDim.x) {
            const int r = i / k, j = i % k;
            const int32_t* slot = reinterpret_cast<const int32_t*>(src.inbox + exchange_slot_offset(src.slot_words, src.world, src.parity, r));
            const int32_t id = __ldcv(slot + (size_t)q * k + j);
            const float sc = __int_as_float(__ldcv(slot + n + (size_t)q * k + j));
            ws.pool[(size_t)q * ws.cap + i] = (id < 0) ? 0ull : make_key(sc * sign + 0.0f, id);
        }
    }
    if (threadIdx.x == 0) {
        ws.count[q] = ok_s ? (uint32_t)per : 0u;
        ws.thr[q] = 0;
        if (!ok_s) flags[kFlagTimeout] = 1u;
        if (bad_s) flags[kFlagPeerOverflow] = 1u;
    }
    __threadfence();
    __syncthreads();
}

}  // namespace mb200
