// Exchange of per-shard top-k lists over peer memory (NVLink / NVSwitch), fused with the merge.
// Every rank owns an inbox on its GPU: two parities x world slots of (ids, scores) plus one epoch word per slot.  After
// its fused score + top-k pass a rank stores its list into slot [parity][rank] of EVERY rank's inbox with plain peer
// stores, fences, and writes the step's epoch into the slot's word; the merge kernel of a rank waits (bounded) until
// all of its own slots carry the epoch, then feeds them to the selection.  No collective library call and no host
// round trip sit between the shard pass and the merged result.  Two parities are enough: a rank can push step s+2
// only after it merged step s+1, which needs every peer's push of s+1, which a peer issues after its merge of step s.
// Every wait has an iteration limit; when it runs out the time-out flag is raised and the kernel returns.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "../../include/manta_b200.h"
#include "common.cuh"
#include "exchange.cuh"
#include "internal.h"
#include "kernels.h"

constexpr int kMaxWorld = 16;

struct MantaB200Exchange {
    int device = 0, world = 0, rank = 0, nq_max = 0, k_max = 0;
    size_t slot_words = 0;      // int32 words per slot: 2 * nq_max * k_max
    size_t inbox_bytes = 0;
    unsigned char* inbox = nullptr;           // [2][world] slots, then [2][world] epoch words (64-byte spaced)
    unsigned char* peer[kMaxWorld] = {};      // every rank's inbox as mapped into this process (peer[rank] == inbox)
    bool opened[kMaxWorld] = {};
    uint32_t epoch = 0;
    uint32_t spin_limit = 10000000u;   // 200 ns naps a merge waits for a missing list: about two seconds
    bool connected = false;
};

namespace {

int fail(char** err, const char* fmt, ...) {
    if (err) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        size_t n = strlen(buf) + 1;
        char* out = (char*)malloc(n);
        if (out) memcpy(out, buf, n);
        *err = out;
    }
    return 1;
}

struct PeerTable {
    unsigned char* inbox[kMaxWorld];
};

// Block p stores this rank's list into peer p's inbox slot [parity][rank], then publishes the status and the epoch.
__global__ void exchange_push_kernel(PeerTable peers, const int32_t* __restrict__ ids, const float* __restrict__ scores, int n,
                                     size_t slot_words, int world, int rank, int parity, uint32_t epoch) {
    unsigned char* box = peers.inbox[blockIdx.x];
    int32_t* dst = reinterpret_cast<int32_t*>(box + mb200::exchange_slot_offset(slot_words, world, parity, rank));
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        dst[i] = ids[i];
        dst[n + i] = __float_as_int(scores[i]);
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t* word = reinterpret_cast<uint32_t*>(box + mb200::exchange_flag_offset(slot_words, world, parity, rank));
        word[1] = 0u;   // status: a list handed over by the caller is complete
        mb200::st_release_sys_u32(word, epoch);
    }
}

}  // namespace

namespace mb200 {
int score_topk_into_sink(MantaB200Runtime* rt, const MantaB200Candidates* set, int metric, int order, const void* d_queries, int nq,
                         int k, const ExchangeSink& sink, char** err);  // api.cu
int exchange_select_ws(MantaB200Runtime* rt, int nq, uint32_t cap, SelectWs* ws, char** err);  // api.cu
void exchange_note_async_flags(MantaB200Runtime* rt, const SelectWs& ws, int sync, char** err, int* rc);  // api.cu
uint32_t* exchange_host_flags(MantaB200Runtime* rt);  // api.cu
}

extern "C" {

int manta_b200_exchange_create(MantaB200Runtime* rt, int world, int rank, int nq_max, int k_max, MantaB200Exchange** out,
                               unsigned char* handle_out, char** err) {
    if (!rt || !out || !handle_out) return fail(err, "exchange_create: NULL argument");
    *out = nullptr;
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) return fail(err, "exchange_create: rank %d of %d out of range (max %d ranks)", rank, world, kMaxWorld);
    if (nq_max <= 0 || k_max <= 0 || k_max > 1024) return fail(err, "exchange_create: bad list shape [%d,%d]", nq_max, k_max);
    mb200::RuntimeInfo ri = mb200::runtime_info(rt);
    std::lock_guard<std::mutex> lk(*ri.mu);
    cudaError_t e = cudaSetDevice(ri.device);
    if (e != cudaSuccess) return fail(err, "exchange_create: %s", cudaGetErrorString(e));
    MantaB200Exchange* ex = new (std::nothrow) MantaB200Exchange();
    if (!ex) return fail(err, "exchange_create: out of host memory");
    ex->device = ri.device;
    ex->world = world;
    ex->rank = rank;
    ex->nq_max = nq_max;
    ex->k_max = k_max;
    ex->slot_words = ((size_t)2 * nq_max * k_max + 63) / 64 * 64;
    ex->inbox_bytes = (size_t)2 * world * ex->slot_words * 4 + (size_t)2 * world * 64 + 64;   // slots, epoch words, block counter
    e = cudaMalloc((void**)&ex->inbox, ex->inbox_bytes);
    if (e == cudaSuccess) e = cudaMemset(ex->inbox, 0, ex->inbox_bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, ex->inbox);
    if (e != cudaSuccess) {
        if (ex->inbox) cudaFree(ex->inbox);
        delete ex;
        return fail(err, "exchange_create: %s", cudaGetErrorString(e));
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
    memcpy(handle_out, &h, 64);
    ex->peer[rank] = ex->inbox;
    *out = ex;
    return 0;
}

int manta_b200_exchange_connect(MantaB200Runtime* rt, MantaB200Exchange* ex, const unsigned char* handles, char** err) {
    if (!rt || !ex || !handles) return fail(err, "exchange_connect: NULL argument");
    mb200::RuntimeInfo ri = mb200::runtime_info(rt);
    std::lock_guard<std::mutex> lk(*ri.mu);
    cudaError_t e = cudaSetDevice(ri.device);
    if (e != cudaSuccess) return fail(err, "exchange_connect: %s", cudaGetErrorString(e));
    for (int r = 0; r < ex->world; ++r) {
        if (r == ex->rank || ex->opened[r]) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)r * 64, 64);
        void* p = nullptr;
        e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return fail(err, "exchange_connect: cannot map rank %d's inbox: %s", r, cudaGetErrorString(e));
        ex->peer[r] = (unsigned char*)p;
        ex->opened[r] = true;
    }
    ex->connected = true;
    return 0;
}

int manta_b200_exchange_connect_local(MantaB200Runtime* rt, MantaB200Exchange* ex, MantaB200Exchange* const* ranks, char** err) {
    if (!rt || !ex || !ranks) return fail(err, "exchange_connect_local: NULL argument");
    mb200::RuntimeInfo ri = mb200::runtime_info(rt);
    std::lock_guard<std::mutex> lk(*ri.mu);
    for (int r = 0; r < ex->world; ++r) {
        if (r == ex->rank) continue;
        const MantaB200Exchange* other = ranks[r];
        if (!other || !other->inbox) return fail(err, "exchange_connect_local: rank %d has no exchange", r);
        if (other->world != ex->world || other->rank != r || other->slot_words != ex->slot_words)
            return fail(err, "exchange_connect_local: rank %d's exchange was created with another shape", r);
        if (other->device != ex->device) {
            int can = 0;
            cudaError_t e = cudaDeviceCanAccessPeer(&can, ex->device, other->device);
            if (e != cudaSuccess || !can) return fail(err, "exchange_connect_local: device %d cannot store into device %d's memory", ex->device, other->device);
            e = cudaSetDevice(ex->device);
            if (e == cudaSuccess) e = cudaDeviceEnablePeerAccess(other->device, 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) {
                cudaGetLastError();
                e = cudaSuccess;
            }
            if (e != cudaSuccess) return fail(err, "exchange_connect_local: %s", cudaGetErrorString(e));
        }
        ex->peer[r] = other->inbox;   // same address space: no IPC mapping, nothing to close later
    }
    ex->connected = true;
    return 0;
}

int manta_b200_exchange_set_wait_limit(MantaB200Exchange* ex, uint32_t naps_200ns, char** err) {
    if (!ex) return fail(err, "exchange_set_wait_limit: NULL exchange");
    if (naps_200ns == 0) return fail(err, "exchange_set_wait_limit: the limit must be positive");
    ex->spin_limit = naps_200ns;
    return 0;
}

int manta_b200_exchange_disconnect(MantaB200Runtime* rt, MantaB200Exchange* ex, char** err) {
    if (!ex) return 0;
    if (!rt) return fail(err, "exchange_disconnect: NULL runtime");
    mb200::RuntimeInfo ri = mb200::runtime_info(rt);
    std::lock_guard<std::mutex> lk(*ri.mu);
    cudaSetDevice(ri.device);
    cudaError_t e = cudaStreamSynchronize(ri.stream);
    for (int r = 0; r < ex->world; ++r) {
        if (ex->opened[r]) {
            cudaError_t c = cudaIpcCloseMemHandle(ex->peer[r]);
            if (e == cudaSuccess) e = c;
            ex->opened[r] = false;
        }
        if (r != ex->rank) ex->peer[r] = nullptr;
    }
    ex->connected = false;
    if (e != cudaSuccess) return fail(err, "exchange_disconnect: %s", cudaGetErrorString(e));
    return 0;
}

int manta_b200_exchange_destroy(MantaB200Runtime* rt, MantaB200Exchange* ex, char** err) {
    if (!ex) return 0;
    if (!rt) return fail(err, "exchange_destroy: NULL runtime");
    // unmaps whatever is still mapped (a caller that skipped the disconnect step), then frees this rank's inbox
    int rc = manta_b200_exchange_disconnect(rt, ex, err);
    mb200::RuntimeInfo ri = mb200::runtime_info(rt);
    std::lock_guard<std::mutex> lk(*ri.mu);
    cudaSetDevice(ri.device);
    if (ex->inbox) cudaFree(ex->inbox);
    delete ex;
    return rc;
}

// Waits for the lists of this epoch and selects (shared by the two entry points below); the caller holds nothing.
static int exchange_merge_tail(MantaB200Runtime* rt, MantaB200Exchange* ex, const mb200::SelectWs& ws, int order, int nq, int k,
                               int parity, uint32_t epoch, int32_t* d_out_ids, float* d_out_scores, int sync, char** err) {
    mb200::RuntimeInfo ri = mb200::runtime_info(rt);
    std::lock_guard<std::mutex> lk(*ri.mu);
    cudaError_t e = cudaSetDevice(ri.device);
    if (e != cudaSuccess) return fail(err, "topk_exchange_merge: %s", cudaGetErrorString(e));
    mb200::SelectArgs sa{};
    sa.ws = ws;
    sa.nq = nq;
    sa.k = k;
    sa.order = order;
    sa.out_ids = d_out_ids;
    sa.out_scores = d_out_scores;
    sa.src.inbox = ex->inbox;   // the selection kernel waits for the lists of all ranks, then selects
    sa.src.slot_words = ex->slot_words;
    sa.src.world = ex->world;
    sa.src.parity = parity;
    sa.src.epoch = epoch;
    sa.src.spin_limit = ex->spin_limit;   // 200 ns naps before a missing list is reported
    sa.flags_out = mb200::exchange_host_flags(rt);   // pinned host words: no copy after the kernel
    sa.reset_after = 1;                               // the workspace is clean again for the next fused pass
    e = mb200::launch_select(ri.stream, sa);
    if (e != cudaSuccess) return fail(err, "topk_exchange_merge: select launch failed: %s", cudaGetErrorString(e));
    int rc = 0;
    mb200::exchange_note_async_flags(rt, ws, sync, err, &rc);
    return rc;
}

int manta_b200_score_topk_exchange_device(MantaB200Runtime* rt, MantaB200Exchange* ex, const MantaB200Candidates* set, int metric,
                                          int order, const void* d_queries, int nq, int k, int32_t* d_out_ids,
                                          float* d_out_scores, int sync, char** err) {
    if (!rt || !ex || !set || !d_queries || !d_out_ids || !d_out_scores) return fail(err, "score_topk_exchange: NULL argument");
    if (!ex->connected && ex->world > 1) return fail(err, "score_topk_exchange: the exchange is not connected to its peers");
    if (nq <= 0 || k <= 0 || nq > ex->nq_max || k > ex->k_max || (size_t)2 * nq * k > ex->slot_words)
        return fail(err, "score_topk_exchange: list shape [%d,%d] exceeds the exchange's [%d,%d]", nq, k, ex->nq_max, ex->k_max);
    mb200::RuntimeInfo ri = mb200::runtime_info(rt);
    if (ri.device != ex->device) return fail(err, "score_topk_exchange: the exchange lives on device %d, the runtime on %d", ex->device, ri.device);
    const uint32_t epoch = ex->epoch + 1;
    const int parity = (int)(epoch & 1u);
    mb200::ExchangeSink sink;
    for (int r = 0; r < ex->world; ++r) sink.inbox[r] = ex->peer[r];
    sink.slot_words = ex->slot_words;
    sink.world = ex->world;
    sink.rank = ex->rank;
    sink.parity = parity;
    sink.epoch = epoch;
    sink.done = reinterpret_cast<uint32_t*>(ex->inbox + ex->inbox_bytes - 64);
    // shard pass: the selection kernel stores this rank's lists into every inbox and publishes the epoch
    if (mb200::score_topk_into_sink(rt, set, metric, order, d_queries, nq, k, sink, err)) return 1;
    ex->epoch = epoch;
    // merge: the same workspace, stream-ordered behind the shard pass (world * k <= the shard pass's pool)
    mb200::SelectWs ws;
    if (mb200::exchange_select_ws(rt, nq, (uint32_t)(ex->world * k), &ws, err)) return 1;
    return exchange_merge_tail(rt, ex, ws, order, nq, k, parity, epoch, d_out_ids, d_out_scores, sync, err);
}

int manta_b200_topk_exchange_merge_device(MantaB200Runtime* rt, MantaB200Exchange* ex, int order, const int32_t* d_ids,
                                          const float* d_scores, int nq, int k, int32_t* d_out_ids, float* d_out_scores,
                                          int sync, char** err) {
    if (!rt || !ex || !d_ids || !d_scores || !d_out_ids || !d_out_scores) return fail(err, "topk_exchange_merge: NULL argument");
    if (!ex->connected && ex->world > 1) return fail(err, "topk_exchange_merge: the exchange is not connected to its peers");
    if (nq <= 0 || k <= 0 || nq > ex->nq_max || k > ex->k_max || (size_t)2 * nq * k > ex->slot_words)
        return fail(err, "topk_exchange_merge: list shape [%d,%d] exceeds the exchange's [%d,%d]", nq, k, ex->nq_max, ex->k_max);
    if (order != MANTA_B200_ORDER_LARGEST && order != MANTA_B200_ORDER_SMALLEST) return fail(err, "topk_exchange_merge: unknown order %d", order);
    mb200::RuntimeInfo ri = mb200::runtime_info(rt);
    if (ri.device != ex->device) return fail(err, "topk_exchange_merge: the exchange lives on device %d, the runtime on %d", ex->device, ri.device);
    mb200::SelectWs ws;
    if (mb200::exchange_select_ws(rt, nq, (uint32_t)(ex->world * k), &ws, err)) return 1;
    std::lock_guard<std::mutex> lk(*ri.mu);
    cudaError_t e = cudaSetDevice(ri.device);
    if (e != cudaSuccess) return fail(err, "topk_exchange_merge: %s", cudaGetErrorString(e));
    const uint32_t epoch = ++ex->epoch;
    const int parity = (int)(epoch & 1u);
    PeerTable pt;
    for (int r = 0; r < kMaxWorld; ++r) pt.inbox[r] = ex->peer[r];
    exchange_push_kernel<<<ex->world, 256, 0, ri.stream>>>(pt, d_ids, d_scores, nq * k, ex->slot_words, ex->world, ex->rank, parity, epoch);
    mb200::count_launch();
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(err, "topk_exchange_merge: launch failed: %s", cudaGetErrorString(e));
    mb200::SelectArgs sa{};
    sa.ws = ws;
    sa.nq = nq;
    sa.k = k;
    sa.order = order;
    sa.out_ids = d_out_ids;
    sa.out_scores = d_out_scores;
    sa.src.inbox = ex->inbox;   // the selection kernel waits for the lists of all ranks, then selects
    sa.src.slot_words = ex->slot_words;
    sa.src.world = ex->world;
    sa.src.parity = parity;
    sa.src.epoch = epoch;
    sa.src.spin_limit = ex->spin_limit;   // 200 ns naps before a missing list is reported
    sa.flags_out = mb200::exchange_host_flags(rt);   // pinned host words: no copy after the kernel
    sa.reset_after = 1;                               // the workspace is clean again for the next fused pass
    e = mb200::launch_select(ri.stream, sa);
    if (e != cudaSuccess) return fail(err, "topk_exchange_merge: select launch failed: %s", cudaGetErrorString(e));
    int rc = 0;
    mb200::exchange_note_async_flags(rt, ws, sync, err, &rc);
    return rc;
}

}  // extern "C"
