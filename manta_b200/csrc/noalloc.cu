// A fused score + top-k entry point that allocates nothing.
//
// Who needs it: callers that must not allocate device memory at the moment they score -- a serving loop that
// has handed all remaining HBM to another component, a host that forbids allocation after start-up, or code
// running while some other stream is being captured (cudaMalloc is not allowed then).  The regular entry
// points grow their scratch buffers with cudaMalloc on first use or when a larger request arrives; this one
// keeps all scratch (query planes, thresholds, bucket maxima, candidate pools) in one fixed array that is part
// of the library image, so every GPU that loads the library holds those bytes until the process exits.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "internal.h"

namespace {

using namespace mb200;

constexpr int kStaticMaxQueries = 4;
constexpr int kStaticMaxK = 256;
constexpr int kStaticMaxCols = 4096;
constexpr uint32_t kStaticPoolCap = 1u << 17;   // candidate keys per query
constexpr uint32_t kStaticBuckets = 8192;       // running maxima per query
// carve-up of the scratch array (every offset is a multiple of 256)
constexpr size_t kOffCount = 0;
constexpr size_t kOffThr = kOffCount + 256;
constexpr size_t kOffFlags = kOffThr + 256;      // [0..3] flags, [4] counter of finished blocks
constexpr size_t kOffBucket = kOffFlags + 256;
constexpr size_t kOffPool = kOffBucket + (size_t)kStaticMaxQueries * kStaticBuckets * 4;
constexpr size_t kScratchBytes = kOffPool + (size_t)kStaticMaxQueries * kStaticPoolCap * 8;  // about 4.3 MB

// The scratch itself.  In host code this name is only a handle for the runtime API, not a device address:
// the address is fetched per device with cudaGetSymbolAddress below and only that pointer goes to kernels.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
unsigned char* g_scratch_ptr[kMaxDevices];  // per device, filled on the first call on that device
std::mutex g_setup_mu;

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

}  // namespace

extern "C" int manta_b200_score_topk_static(MantaB200Runtime* rt, const MantaB200Candidates* set, int metric,
                                            int order, const void* d_queries, int nq, int k, int32_t* d_out_ids,
                                            float* d_out_scores, int sync, char** err) {
    if (!rt || !set || !d_queries || !d_out_ids || !d_out_scores) return fail(err, "score_topk_static: NULL argument");
    const RuntimeInfo ri = runtime_info(rt);
    const CandView cv = *candidates_view(set);
    if (candidates_device(set) != ri.device) return fail(err, "score_topk_static: candidate set and runtime are on different devices");
    if (metric < 0 || metric > 2) return fail(err, "score_topk_static: unknown metric %d", metric);
    if (order != MANTA_B200_ORDER_LARGEST && order != MANTA_B200_ORDER_SMALLEST) return fail(err, "score_topk_static: unknown order %d", order);
    if (nq <= 0 || nq > kStaticMaxQueries)
        return fail(err, "score_topk_static: %d queries exceed the fixed scratch (at most %d per call)", nq, kStaticMaxQueries);
    if (k <= 0 || k > cv.rows) return fail(err, "topk limit %d out of range for %lld scores", k, (long long)cv.rows);
    if (k > kStaticMaxK) return fail(err, "score_topk_static: k = %d exceeds the fixed scratch (at most %d)", k, kStaticMaxK);
    if (cv.cols > kStaticMaxCols) return fail(err, "score_topk_static: %d columns exceed the fixed scratch (at most %d)", cv.cols, kStaticMaxCols);
    if (stream_bucket_count(ri.sm_count) > (int)kStaticBuckets) return fail(err, "score_topk_static: this GPU needs more bucket slots than the fixed scratch holds");
    if (ri.device < 0 || ri.device >= kMaxDevices) return fail(err, "score_topk_static: device ordinal %d out of range", ri.device);
    {
        ScanGeometry geo;
        size_t smem = 0;
        if (!stream_scan_geometry(cv, nq <= 1 ? 1 : (nq <= 2 ? 2 : 4), 0, &geo, &smem)) return fail(err, "score_topk_static: row too wide");
    }

    std::lock_guard<std::mutex> lk(*ri.mu);
    cudaError_t e = cudaSetDevice(ri.device);
    if (e != cudaSuccess) return fail(err, "cudaSetDevice: %s", cudaGetErrorName(e));
    unsigned char* base = nullptr;
    {
        // Set-up, once per device, with that device current: ask the runtime for the array's device address.
        std::lock_guard<std::mutex> sk(g_setup_mu);
        if (!g_scratch_ptr[ri.device]) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_static_scratch);
            if (e != cudaSuccess) return fail(err, "cudaGetSymbolAddress(scratch): %s (%s)", cudaGetErrorName(e), cudaGetErrorString(e));
            g_scratch_ptr[ri.device] = (unsigned char*)p;
        }
        base = g_scratch_ptr[ri.device];
    }

    SelectWs ws;
    ws.pool = (uint64_t*)(base + kOffPool);
    ws.count = (uint32_t*)(base + kOffCount);
    ws.thr = (uint32_t*)(base + kOffThr);
    ws.bucket = (uint32_t*)(base + kOffBucket);
    ws.flags = (uint32_t*)(base + kOffFlags);
    ws.cap = kStaticPoolCap;
    ws.nb = kStaticBuckets;
    uint32_t* done_blocks = ws.flags + 4;
    // What must start at zero (fill counts, thresholds, bucket maxima, flags, the block counter) is cleared by a
    // small kernel; the pool itself may keep the previous call's keys, only the first `count` entries are ever read.
    // The queries are prepared inside the scan, in shared memory: no scratch for them.
    e = launch_ws_reset(ri.stream, ws, nq, done_blocks);
    if (e != cudaSuccess) return fail(err, "score_topk_static: workspace reset launch: %s", cudaGetErrorName(e));
    // Rows are scanned in chunks of (pool capacity - k) rows and the pool is compacted to the best k between
    // chunks, so the fixed pool cannot overflow whatever order the scores arrive in.
    const int64_t chunk = (int64_t)ws.cap - k > 0 ? (int64_t)ws.cap - k : cv.rows;
    for (int64_t r0 = 0; r0 < cv.rows; r0 += chunk) {
        const int64_t r1 = (r0 + chunk < cv.rows) ? r0 + chunk : cv.rows;
        for (int q0 = 0; q0 < nq;) {
            const int left = nq - q0;
            const int qt = left >= 4 ? 4 : (left >= 2 ? 2 : 1);
            StreamArgs a{};
            a.cv = cv;
            a.queries = (const __half*)d_queries;
            a.q0 = q0;
            a.qt = qt;
            a.metric = metric;
            a.order = order;
            a.k = k;
            a.mode = kModeTopk;
            a.row_begin = r0;
            a.row_end = r1;
            a.ws = ws;
            a.nq_total = nq;
            e = launch_stream_scan(ri.stream, ri.sm_count, a);
            if (e != cudaSuccess) return fail(err, "score_topk_static: scan launch: %s", cudaGetErrorName(e));
            q0 += qt;
        }
        const bool last = r1 >= cv.rows;
        SelectArgs sa{};
        sa.ws = ws;
        sa.nq = nq;
        sa.k = k;
        sa.order = order;
        sa.write_back = last ? 0 : 1;
        sa.out_ids = last ? d_out_ids : nullptr;
        sa.out_scores = last ? d_out_scores : nullptr;
        e = launch_select(ri.stream, sa);
        if (e != cudaSuccess) return fail(err, "score_topk_static: select launch: %s", cudaGetErrorName(e));
    }
    // The pass's flag words go to the runtime's pinned host words 12..15 (this entry point's own slot): read here
    // when the call is synchronous, by the next manta_b200_runtime_synchronize otherwise.
    e = cudaMemcpyAsync(ri.h_flags + 12, ws.flags, kNumFlags * 4, cudaMemcpyDeviceToHost, ri.stream);
    if (e != cudaSuccess) return fail(err, "score_topk_static: %s (%s)", cudaGetErrorName(e), cudaGetErrorString(e));
    if (!sync) {
        *ri.static_flags_pending = true;
        return 0;
    }
    e = cudaStreamSynchronize(ri.stream);
    if (e != cudaSuccess) return fail(err, "score_topk_static: %s (%s)", cudaGetErrorName(e), cudaGetErrorString(e));
    *ri.static_flags_pending = false;
    if (ri.h_flags[12 + kFlagTimeout]) return fail(err, "score_topk_static: a bounded device wait gave up");
    if (ri.h_flags[12 + kFlagOverflow] || ri.h_flags[12 + kFlagInternal]) return fail(err, "score_topk_static: selection found fewer than k candidates");
    return 0;
}
