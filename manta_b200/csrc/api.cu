// C ABI of the library (include/manta_b200.h): runtime, resident candidate sets, fused score/select.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>

#include "internal.h"
#include "kernels.h"
#include "mma.h"

namespace mb200 {

static std::atomic<uint64_t> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

static thread_local MantaB200LaunchInfo t_last_scan{};
void note_scan_launch(const char* kernel, int grid, int block, size_t shared_bytes) {
    snprintf(t_last_scan.kernel, sizeof t_last_scan.kernel, "%s", kernel);
    t_last_scan.grid = grid;
    t_last_scan.block = block;
    t_last_scan.shared_bytes = (int)shared_bytes;
    t_last_scan.launches++;
}

cudaError_t launch_stream_scan_f16(cudaStream_t st, int sm_count, const StreamArgs& a);
cudaError_t launch_stream_scan_q8(cudaStream_t st, int sm_count, const StreamArgs& a);
cudaError_t launch_stream_scan_q4(cudaStream_t st, int sm_count, const StreamArgs& a);

cudaError_t launch_stream_scan(cudaStream_t st, int sm_count, const StreamArgs& a) {
    switch (a.cv.layout) {
        case MANTA_B200_LAYOUT_F16: return launch_stream_scan_f16(st, sm_count, a);
        case MANTA_B200_LAYOUT_Q8_ROW_F32: return launch_stream_scan_q8(st, sm_count, a);
        case MANTA_B200_LAYOUT_Q4_B32_F16: return launch_stream_scan_q4(st, sm_count, a);
    }
    return cudaErrorInvalidValue;
}

}  // namespace mb200

using namespace mb200;

// ---- error plumbing (int rc + malloc'd message, as the reference's cgo preamble) -----------------------
static int fail(char** err, const char* fmt, ...) {
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

static int fail_cuda(char** err, const char* what, cudaError_t e) {
    return fail(err, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

#define CU_TRY(call)                                       \
    do {                                                   \
        cudaError_t e_ = (call);                           \
        if (e_ != cudaSuccess) return fail_cuda(err, #call, e_); \
    } while (0)

// ---- handles -----------------------------------------------------------------------------------------
struct DevBuf {
    void* p = nullptr;
    size_t bytes = 0;
};

struct MantaB200Runtime {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int sm_count = 0;
    std::mutex mu;
    MantaB200Stats stats{};
    // grow-only device buffers
    DevBuf queries, headers, qf32, plane_hi, plane_lo, pool, count, thr, bucket, flags, out_ids, out_scores, misc, embed_flag, batch_in, tok_norms, lo_norm;
    // pinned host staging
    void* h_stage = nullptr;
    size_t h_stage_bytes = 0;
    uint32_t* h_flags = nullptr;
    mb200::MmaState* mma = nullptr;
    // device-time accounting of the scan kernels
    bool profiling = false;
    static constexpr int kMaxProf = 256;
    cudaEvent_t prof_ev[2 * kMaxProf];
    int prof_created = 0;
    int prof_used = 0;
    bool async_exchange_pending = false;  // a sync == 0 exchange merge copied its flags to h_flags[4..7]
    bool async_embed_pending = false;  // a sync == 0 embed pass copied its bad-token word to h_flags[10..11]
    bool async_flags_pending = false;  // a sync == 0 pass copied its flags to h_flags; checked at synchronize
    bool async_static_pending = false;  // a sync == 0 allocation-free pass copied its flags to h_flags[12..15]
    MantaB200LaunchInfo last_launch{};  // configuration of the last pass's scan kernel
    bool ws_dirty = true;  // the selection workspace is not in the all-zero state a fused streaming pass starts from
    int ws_dirty_nq = 0;   // ... for this many queries (a later pass with fewer queries must not leave the others' state behind)
};

static void prof_mark(MantaB200Runtime* rt, int which) {
    if (!rt->profiling || rt->prof_used >= MantaB200Runtime::kMaxProf) return;
    const int idx = 2 * rt->prof_used + which;
    while (rt->prof_created <= idx) {
        if (cudaEventCreate(&rt->prof_ev[rt->prof_created]) != cudaSuccess) return;
        rt->prof_created++;
    }
    cudaEventRecord(rt->prof_ev[idx], rt->stream);
    if (which == 1) rt->prof_used++;
}

struct MantaB200Embedder {
    int device = 0;
    int vocab = 0, dim = 0, out_dim = 0;
    void* d_table = nullptr;
    void* d_proj = nullptr;
    void* d_proj_t = nullptr;   // [out_dim][dim], only for shapes the tensor-core projection takes
};

struct MantaB200Candidates {
    CandView cv{};
    void* owned_data = nullptr;
    void* owned_scales = nullptr;
    void* owned_stats = nullptr;
    int64_t stored_bytes = 0;
    int device = 0;
};

namespace mb200 {
RuntimeInfo runtime_info(MantaB200Runtime* rt) {
    return RuntimeInfo{rt->device, rt->sm_count, rt->stream, rt->h_flags, &rt->async_static_pending, &rt->mu};
}
const CandView* candidates_view(const MantaB200Candidates* set) { return &set->cv; }
int candidates_device(const MantaB200Candidates* set) { return set->device; }
}  // namespace mb200

static int ensure(MantaB200Runtime* rt, DevBuf& b, size_t bytes, char** err) {
    if (bytes <= b.bytes) return 0;
    if (b.p) {
        CU_TRY(cudaStreamSynchronize(rt->stream));
        CU_TRY(cudaFree(b.p));
        b.p = nullptr;
        b.bytes = 0;
    }
    size_t want = bytes + bytes / 4 + 256;
    CU_TRY(cudaMalloc(&b.p, want));
    b.bytes = want;
    // fresh memory is not the zeroed workspace a fused streaming pass expects: zero all of it once, whatever it is for
    CU_TRY(cudaMemsetAsync(b.p, 0, want, rt->stream));
    return 0;
}

static int ensure_host(MantaB200Runtime* rt, size_t bytes, char** err) {
    if (bytes <= rt->h_stage_bytes) return 0;
    if (rt->h_stage) {
        CU_TRY(cudaStreamSynchronize(rt->stream));
        CU_TRY(cudaFreeHost(rt->h_stage));
        rt->h_stage = nullptr;
        rt->h_stage_bytes = 0;
    }
    size_t want = bytes * 2 + 4096;
    CU_TRY(cudaMallocHost(&rt->h_stage, want));
    rt->h_stage_bytes = want;
    return 0;
}

static void free_buf(DevBuf& b) {
    if (b.p) cudaFree(b.p);
    b.p = nullptr;
    b.bytes = 0;
}

static const char* metric_name(int m) {
    return m == MANTA_B200_METRIC_DOT ? "dot" : m == MANTA_B200_METRIC_COSINE ? "cosine" : "l2_distance";
}

extern "C" {

void manta_b200_free_cstring(char* s) { free(s); }

uint64_t manta_b200_kernel_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int manta_b200_runtime_create(int device, void* stream, MantaB200Runtime** out, char** err) {
    if (!out) return fail(err, "runtime_create: out is NULL");
    *out = nullptr;
    int ndev = 0;
    CU_TRY(cudaGetDeviceCount(&ndev));
    if (device < 0 || device >= ndev) return fail(err, "runtime_create: device %d out of range (%d devices)", device, ndev);
    CU_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    CU_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        return fail(err, "runtime_create: device %d is sm_%d%d; this library carries sm_100a code only", device,
                    prop.major, prop.minor);
    }
    MantaB200Runtime* rt = new (std::nothrow) MantaB200Runtime();
    if (!rt) return fail(err, "runtime_create: out of host memory");
    rt->device = device;
    rt->sm_count = prop.multiProcessorCount;
    if (stream) {
        rt->stream = (cudaStream_t)stream;
    } else {
        cudaError_t e = cudaStreamCreateWithFlags(&rt->stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) {
            delete rt;
            return fail_cuda(err, "cudaStreamCreateWithFlags", e);
        }
        rt->owns_stream = true;
    }
    cudaError_t e = cudaMallocHost((void**)&rt->h_flags, 64);
    if (e != cudaSuccess) {
        if (rt->owns_stream) cudaStreamDestroy(rt->stream);
        delete rt;
        return fail_cuda(err, "cudaMallocHost", e);
    }
    *out = rt;
    return 0;
}

int manta_b200_runtime_destroy(MantaB200Runtime* rt, char** err) {
    if (!rt) return 0;
    cudaSetDevice(rt->device);
    cudaError_t e = cudaStreamSynchronize(rt->stream);
    DevBuf* bufs[] = {&rt->queries, &rt->headers, &rt->qf32, &rt->plane_hi, &rt->plane_lo, &rt->pool, &rt->count,
                      &rt->thr, &rt->bucket, &rt->flags, &rt->out_ids, &rt->out_scores, &rt->misc, &rt->embed_flag, &rt->batch_in, &rt->tok_norms, &rt->lo_norm};
    for (DevBuf* b : bufs) free_buf(*b);
    mma_state_destroy(rt->mma);
    for (int i = 0; i < rt->prof_created; ++i) cudaEventDestroy(rt->prof_ev[i]);
    if (rt->h_stage) cudaFreeHost(rt->h_stage);
    if (rt->h_flags) cudaFreeHost(rt->h_flags);
    if (rt->owns_stream) cudaStreamDestroy(rt->stream);
    delete rt;
    if (e != cudaSuccess) return fail_cuda(err, "cudaStreamSynchronize", e);
    return 0;
}

int manta_b200_runtime_stream(MantaB200Runtime* rt, void** out_stream, char** err) {
    if (!rt || !out_stream) return fail(err, "runtime_stream: NULL argument");
    *out_stream = (void*)rt->stream;
    return 0;
}

int manta_b200_runtime_synchronize(MantaB200Runtime* rt, char** err) {
    if (!rt) return fail(err, "runtime_synchronize: NULL runtime");
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    CU_TRY(cudaStreamSynchronize(rt->stream));
    // every pending report is read and cleared first, then the first failure (if any) is returned
    const char* msg = nullptr;
    if (rt->async_exchange_pending) {
        rt->async_exchange_pending = false;
        uint32_t fl[kNumFlags];
        for (int f = 0; f < kNumFlags; ++f) {
            fl[f] = rt->h_flags[4 + f];
            rt->h_flags[4 + f] = 0;
        }
        if (fl[kFlagTimeout]) msg = "runtime_synchronize: a peer's top-k list did not arrive within the wait limit of the exchange";
        else if (fl[kFlagPeerOverflow] || rt->h_flags[kFlagOverflow])
            msg = "runtime_synchronize: a shard's candidate pool overflowed during an exchange step, the merged result is incomplete on "
                  "every rank; redo the step with manta_b200_score_topk_device(sync != 0) + manta_b200_topk_exchange_merge_device";
        else if (fl[kFlagInternal]) msg = "runtime_synchronize: the exchange merge found fewer than k candidates";
    }
    if (rt->async_embed_pending) {
        rt->async_embed_pending = false;
        if (rt->h_flags[10] == 2u && !msg) return fail(err, "embed: a bounded wait of the tensor-core projection ran out");
        if (rt->h_flags[10] && !msg) return fail(err, "gather index %d out of range", (int32_t)rt->h_flags[11]);
    }
    if (rt->async_static_pending) {
        rt->async_static_pending = false;
        if (!msg) {
            if (rt->h_flags[12 + kFlagTimeout]) msg = "runtime_synchronize: a bounded device wait gave up in an allocation-free pass";
            else if (rt->h_flags[12 + kFlagOverflow] || rt->h_flags[12 + kFlagInternal])
                msg = "runtime_synchronize: the last allocation-free pass found fewer than k candidates";
        }
    }
    if (rt->async_flags_pending) {
        rt->async_flags_pending = false;
        uint32_t fl[kNumFlags];
        for (int f = 0; f < kNumFlags; ++f) {
            fl[f] = rt->h_flags[f];
            rt->h_flags[f] = 0;
        }
        if (!msg) {
            if (fl[kFlagTimeout]) msg = "runtime_synchronize: a bounded device wait gave up in an asynchronous pass";
            else if (fl[kFlagOverflow])
                msg = "runtime_synchronize: an asynchronous fused pass overflowed its candidate pool; its result is incomplete, reissue it "
                      "with sync != 0 (which redoes it in chunks)";
            else if (fl[kFlagInternal]) msg = "runtime_synchronize: selection found fewer than k candidates";
        }
    }
    if (msg) return fail(err, "%s", msg);
    return 0;
}

int manta_b200_runtime_stats(MantaB200Runtime* rt, MantaB200Stats* out, char** err) {
    if (!rt || !out) return fail(err, "runtime_stats: NULL argument");
    std::lock_guard<std::mutex> lk(rt->mu);
    *out = rt->stats;
    return 0;
}

int manta_b200_runtime_last_launch(MantaB200Runtime* rt, MantaB200LaunchInfo* out, char** err) {
    if (!rt || !out) return fail(err, "runtime_last_launch: NULL argument");
    std::lock_guard<std::mutex> lk(rt->mu);
    *out = rt->last_launch;
    return 0;
}

int manta_b200_runtime_profile(MantaB200Runtime* rt, int enable, char** err) {
    if (!rt) return fail(err, "runtime_profile: NULL runtime");
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    CU_TRY(cudaStreamSynchronize(rt->stream));
    rt->profiling = enable != 0;
    rt->prof_used = 0;
    return 0;
}

int manta_b200_runtime_scan_time(MantaB200Runtime* rt, double* total_ms, int* passes, char** err) {
    if (!rt || !total_ms || !passes) return fail(err, "runtime_scan_time: NULL argument");
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    CU_TRY(cudaStreamSynchronize(rt->stream));
    double sum = 0.0;
    for (int i = 0; i < rt->prof_used; ++i) {
        float ms = 0.0f;
        CU_TRY(cudaEventElapsedTime(&ms, rt->prof_ev[2 * i], rt->prof_ev[2 * i + 1]));
        sum += ms;
    }
    *total_ms = sum;
    *passes = rt->prof_used;
    rt->prof_used = 0;
    return 0;
}

// ---- candidates ------------------------------------------------------------------------------------------
static int layout_geometry(int layout, int cols, int* elem_row_bytes, int* chunks, int* scale_row_bytes, char** err) {
    if (cols <= 0 || cols > kMaxCols) return fail(err, "candidates: cols %d out of range (1..%d)", cols, kMaxCols);
    switch (layout) {
        case MANTA_B200_LAYOUT_F16:
            *elem_row_bytes = cols * 2;
            *chunks = (cols + 7) / 8;
            *scale_row_bytes = 0;
            return 0;
        case MANTA_B200_LAYOUT_Q8_ROW_F32:
            *elem_row_bytes = cols;
            *chunks = (cols + 15) / 16;
            *scale_row_bytes = 4;
            return 0;
        case MANTA_B200_LAYOUT_Q4_B32_F16:
            if (cols % 32) return fail(err, "candidates: q4 block32 layout needs cols %% 32 == 0, got %d", cols);
            *elem_row_bytes = cols / 2;
            *chunks = cols / 32;
            *scale_row_bytes = (cols / 32) * 2;
            return 0;
    }
    return fail(err, "candidates: unknown layout %d", layout);
}

int manta_b200_candidates_bind(MantaB200Runtime* rt, int layout, int64_t rows, int cols, const void* data,
                               const void* scales, int64_t row_base, int mem, MantaB200Candidates** out,
                               char** err) {
    if (!rt || !out) return fail(err, "candidates_bind: NULL argument");
    *out = nullptr;
    int elem_row_bytes = 0, chunks = 0, scale_row_bytes = 0;
    if (layout_geometry(layout, cols, &elem_row_bytes, &chunks, &scale_row_bytes, err)) return 1;
    if (rows < 0) return fail(err, "candidates_bind: negative row count");
    if (row_base < 0 || row_base + rows > (int64_t)INT32_MAX)
        return fail(err, "candidates_bind: row ids [%lld, %lld) do not fit int32", (long long)row_base,
                    (long long)(row_base + rows));
    if (rows > 0 && (!data || (scale_row_bytes && !scales))) return fail(err, "candidates_bind: NULL data or scales");
    {
        CandView probe{};
        probe.layout = layout;
        probe.chunks = chunks;
        ScanGeometry g;
        size_t smem = 0;
        if (!stream_scan_geometry(probe, 1, 0, &g, &smem))
            return fail(err, "candidates_bind: row of %d columns is wider than the kernels support for this layout", cols);
    }

    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    MantaB200Candidates* set = new (std::nothrow) MantaB200Candidates();
    if (!set) return fail(err, "candidates_bind: out of host memory");
    set->device = rt->device;
    CandView& cv = set->cv;
    cv.layout = layout;
    cv.rows = rows;
    cv.cols = cols;
    cv.row_base = row_base;
    cv.chunks = chunks;
    cv.row_bytes = chunks * 16;
    const size_t data_bytes = (size_t)rows * cv.row_bytes;
    const size_t scale_bytes = (size_t)rows * scale_row_bytes;
    set->stored_bytes = (int64_t)((size_t)rows * elem_row_bytes + scale_bytes);
    auto cleanup = [&]() {
        if (set->owned_data) cudaFree(set->owned_data);
        if (set->owned_scales) cudaFree(set->owned_scales);
        if (set->owned_stats) cudaFree(set->owned_stats);
        delete set;
    };
#define BIND_TRY(call)                                 \
    do {                                               \
        cudaError_t e_ = (call);                       \
        if (e_ != cudaSuccess) {                       \
            cleanup();                                 \
            return fail_cuda(err, #call, e_);          \
        }                                              \
    } while (0)

    if (rows > 0) {
        if (mem == MANTA_B200_MEM_DEVICE_ADOPT) {
            if (cv.row_bytes != elem_row_bytes || ((uintptr_t)data & 15)) {
                cleanup();
                return fail(err, "candidates_bind: adopt needs a 16-byte aligned base and a row size that is a multiple of 16 bytes");
            }
            cv.data = (const uint8_t*)data;
            cv.scales = scales;
        } else if (mem == MANTA_B200_MEM_HOST || mem == MANTA_B200_MEM_DEVICE_COPY) {
            const cudaMemcpyKind kind = (mem == MANTA_B200_MEM_HOST) ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice;
            BIND_TRY(cudaMalloc(&set->owned_data, data_bytes));
            if (cv.row_bytes != elem_row_bytes) BIND_TRY(cudaMemsetAsync(set->owned_data, 0, data_bytes, rt->stream));
            BIND_TRY(cudaMemcpy2DAsync(set->owned_data, cv.row_bytes, data, elem_row_bytes, elem_row_bytes, rows, kind,
                                       rt->stream));
            if (scale_bytes) {
                BIND_TRY(cudaMalloc(&set->owned_scales, scale_bytes));
                BIND_TRY(cudaMemcpyAsync(set->owned_scales, scales, scale_bytes, kind, rt->stream));
            }
            cv.data = (const uint8_t*)set->owned_data;
            cv.scales = set->owned_scales;
            if (mem == MANTA_B200_MEM_HOST) rt->stats.h2d_bytes += (uint64_t)rows * elem_row_bytes + scale_bytes;
        } else {
            cleanup();
            return fail(err, "candidates_bind: unknown mem kind %d", mem);
        }
        BIND_TRY(cudaMalloc(&set->owned_stats, (size_t)rows * 4));
        cv.stats = set->owned_stats;
        launch_row_stats(rt->stream, cv, set->owned_stats);
        rt->stats.kernel_launches++;
        BIND_TRY(cudaGetLastError());
        BIND_TRY(cudaStreamSynchronize(rt->stream));
    }
#undef BIND_TRY
    rt->stats.bind_calls++;
    rt->stats.bound_bytes += (uint64_t)set->stored_bytes;
    *out = set;
    return 0;
}

int manta_b200_candidates_unbind(MantaB200Runtime* rt, MantaB200Candidates* set, char** err) {
    if (!set) return 0;
    if (!rt) return fail(err, "candidates_unbind: NULL runtime");
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    CU_TRY(cudaStreamSynchronize(rt->stream));
    if (set->owned_data) cudaFree(set->owned_data);
    if (set->owned_scales) cudaFree(set->owned_scales);
    if (set->owned_stats) cudaFree(set->owned_stats);
    delete set;
    return 0;
}

int64_t manta_b200_candidates_bytes(const MantaB200Candidates* set) { return set ? set->stored_bytes : 0; }

// ---- quantisers --------------------------------------------------------------------------------------------
int manta_b200_pack_q8_rows_device(MantaB200Runtime* rt, const void* d_src, int src_is_f16, int64_t rows, int cols,
                                   int8_t* d_codes, float* d_scales, char** err) {
    if (!rt) return fail(err, "pack_q8_rows: NULL runtime");
    if (rows < 0 || cols <= 0) return fail(err, "pack_q8_rows: bad shape");
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    launch_pack_q8(rt->stream, d_src, src_is_f16 != 0, rows, cols, cols, d_codes, d_scales);
    rt->stats.kernel_launches++;
    CU_TRY(cudaGetLastError());
    return 0;
}

int manta_b200_pack_q4_b32_device(MantaB200Runtime* rt, const void* d_src, int src_is_f16, int64_t rows, int cols,
                                  uint8_t* d_codes, uint16_t* d_scales, char** err) {
    if (!rt) return fail(err, "pack_q4_b32: NULL runtime");
    if (rows < 0 || cols <= 0 || cols % 32) return fail(err, "pack_q4_b32: cols must be a positive multiple of 32");
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    launch_pack_q4(rt->stream, d_src, src_is_f16 != 0, rows, cols, d_codes, d_scales);
    rt->stats.kernel_launches++;
    CU_TRY(cudaGetLastError());
    return 0;
}

static int pack_host(MantaB200Runtime* rt, int which, const float* src, int64_t rows, int cols, void* codes,
                     void* scales, char** err) {
    if (!rt || !src || !codes || !scales) return fail(err, "pack: NULL argument");
    if (rows < 0 || cols <= 0 || (which == 4 && cols % 32)) return fail(err, "pack: bad shape");
    if (rows == 0) return 0;
    const size_t src_bytes = (size_t)rows * cols * 4;
    const size_t code_bytes = (which == 8) ? (size_t)rows * cols : (size_t)rows * cols / 2;
    const size_t scale_bytes = (which == 8) ? (size_t)rows * 4 : (size_t)rows * (cols / 32) * 2;
    void *d_src = nullptr, *d_codes = nullptr, *d_scales = nullptr;
    {
        std::lock_guard<std::mutex> lk(rt->mu);
        CU_TRY(cudaSetDevice(rt->device));
        cudaError_t e = cudaMalloc(&d_src, src_bytes);
        if (e == cudaSuccess) e = cudaMalloc(&d_codes, code_bytes);
        if (e == cudaSuccess) e = cudaMalloc(&d_scales, scale_bytes);
        if (e == cudaSuccess) e = cudaMemcpyAsync(d_src, src, src_bytes, cudaMemcpyHostToDevice, rt->stream);
        if (e == cudaSuccess) {
            if (which == 8)
                launch_pack_q8(rt->stream, d_src, false, rows, cols, cols, (int8_t*)d_codes, (float*)d_scales);
            else
                launch_pack_q4(rt->stream, d_src, false, rows, cols, (uint8_t*)d_codes, (uint16_t*)d_scales);
            rt->stats.kernel_launches++;
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = cudaMemcpyAsync(codes, d_codes, code_bytes, cudaMemcpyDeviceToHost, rt->stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(scales, d_scales, scale_bytes, cudaMemcpyDeviceToHost, rt->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(rt->stream);
        cudaFree(d_src);
        cudaFree(d_codes);
        cudaFree(d_scales);
        if (e != cudaSuccess) return fail_cuda(err, "pack", e);
        rt->stats.h2d_bytes += src_bytes;
        rt->stats.d2h_bytes += code_bytes + scale_bytes;
    }
    return 0;
}

int manta_b200_pack_q8_rows(MantaB200Runtime* rt, const float* src, int64_t rows, int cols, int8_t* codes,
                            float* scales, char** err) {
    return pack_host(rt, 8, src, rows, cols, codes, scales, err);
}

int manta_b200_pack_q4_b32(MantaB200Runtime* rt, const float* src, int64_t rows, int cols, uint8_t* codes,
                           uint16_t* scales, char** err) {
    return pack_host(rt, 4, src, rows, cols, codes, scales, err);
}

// ---- scoring ---------------------------------------------------------------------------------------------------
static int plane_stride_for(const CandView& cv) {
    int bytes = (cv.layout == MANTA_B200_LAYOUT_Q4_B32_F16) ? cv.chunks * 32 : cv.chunks * 16;
    return (bytes + 127) / 128 * 128;
}

// Pool capacity per query for the optimistic single-launch pass.
static uint32_t pool_cap_for(const MantaB200Runtime* rt, const CandView& cv, int nq, int k, int metric) {
    const int64_t rows = cv.rows;
    int64_t cap;
    if (mma_supported(cv, nq, metric)) {
        cap = mma_pool_cap(k);  // observed tiles are replayed, so nothing enters the pool unfiltered
        if (cap > rows) cap = rows;
        if (cap < k) cap = k;
        return (uint32_t)cap;
    } else {
        // The streaming scan appends only rows that pass the running threshold (tiles seen before a threshold exists
        // are observed and re-read), so the pool holds a small multiple of k; a set smaller than this is held whole.
        cap = 64ll * k;
    }
    if (cap < 32ll * k) cap = 32ll * k;
    if (cap < (1 << 16)) cap = 1 << 16;
    if (cap > rows) cap = rows;  // a pool as large as the set cannot overflow
    if (cap < k) cap = k;
    return (uint32_t)cap;
}

static int prepare_queries(MantaB200Runtime* rt, const CandView& cv, const void* d_queries, int nq, const SelectWs& ws,
                           int reset_ws, QueryPrep* qp, char** err) {
    const int ps = plane_stride_for(cv);
    if (ensure(rt, rt->headers, (size_t)nq * sizeof(QueryHeader), err)) return 1;
    if (ensure(rt, rt->qf32, (size_t)nq * cv.cols * 4, err)) return 1;
    if (ensure(rt, rt->plane_hi, (size_t)nq * ps, err)) return 1;
    if (ensure(rt, rt->plane_lo, (size_t)nq * ps, err)) return 1;
    if (ensure(rt, rt->lo_norm, (size_t)nq * 4, err)) return 1;
    launch_query_prep(rt->stream, d_queries, nq, cv.cols, cv.layout, ps, (float*)rt->lo_norm.p, (QueryHeader*)rt->headers.p, (float*)rt->qf32.p,
                      (int8_t*)rt->plane_hi.p, (int8_t*)rt->plane_lo.p, ws, reset_ws);
    rt->stats.kernel_launches++;
    CU_TRY(cudaGetLastError());
    qp->headers = (const QueryHeader*)rt->headers.p;
    qp->qf32 = (const float*)rt->qf32.p;
    qp->plane_hi = (const int8_t*)rt->plane_hi.p;
    qp->plane_lo = (const int8_t*)rt->plane_lo.p;
    qp->plane_stride = ps;
    qp->lo_norm = (const float*)rt->lo_norm.p;
    qp->queries_f16 = d_queries;
    qp->nq = nq;
    return 0;
}

static int ensure_select_ws(MantaB200Runtime* rt, int nq, uint32_t cap, uint32_t nb, SelectWs* ws, char** err) {
    if (ensure(rt, rt->pool, (size_t)nq * cap * 8, err)) return 1;
    if (ensure(rt, rt->count, (size_t)nq * 4, err)) return 1;
    if (ensure(rt, rt->thr, (size_t)nq * 4, err)) return 1;
    if (ensure(rt, rt->bucket, (size_t)nq * nb * 4, err)) return 1;
    if (ensure(rt, rt->flags, 64, err)) return 1;   // [0..3] flags, [4] blocks that have finished the current scan
    ws->pool = (uint64_t*)rt->pool.p;
    ws->count = (uint32_t*)rt->count.p;
    ws->thr = (uint32_t*)rt->thr.p;
    ws->bucket = (uint32_t*)rt->bucket.p;
    ws->flags = (uint32_t*)rt->flags.p;
    ws->cap = cap;
    ws->nb = nb;
    return 0;
}

// Reads and clears the sticky host flag words [first, first + 4); the stream must be synchronised.
static void take_host_flags(MantaB200Runtime* rt, int first, uint32_t out[kNumFlags]) {
    for (int f = 0; f < kNumFlags; ++f) {
        out[f] = rt->h_flags[first + f];
        rt->h_flags[first + f] = 0;
    }
}

extern "C++" {
namespace mb200 {
// Selection workspace for the exchange merge (exchange.cu); takes the runtime's lock itself.
int exchange_select_ws(MantaB200Runtime* rt, int nq, uint32_t cap, SelectWs* ws, char** err) {
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    rt->stats.kernel_launches += 2;
    return ensure_select_ws(rt, nq, cap, 1, ws, err);
}
// The exchange merge raises its flags in the pinned host words 4..7 (the fused pass keeps 0..3).
uint32_t* exchange_host_flags(MantaB200Runtime* rt) { return rt->h_flags + 4; }
// After the merge's selection kernel is queued: with sync the words are read (and cleared) here, otherwise by the next
// runtime_synchronize.  The caller holds the lock.
void exchange_note_async_flags(MantaB200Runtime* rt, const SelectWs& ws, int sync, char** err, int* rc) {
    (void)ws;
    *rc = 0;
    if (!sync) {
        rt->async_exchange_pending = true;
        return;
    }
    cudaError_t e = cudaStreamSynchronize(rt->stream);
    if (e != cudaSuccess) {
        *rc = fail_cuda(err, "topk_exchange_merge", e);
        return;
    }
    rt->async_exchange_pending = false;
    uint32_t fl[kNumFlags];
    take_host_flags(rt, 4, fl);
    const bool own_overflow = rt->h_flags[kFlagOverflow] != 0;   // this rank's shard pass (its words stay for the next synchronize)
    if (fl[kFlagTimeout]) *rc = fail(err, "topk_exchange_merge: a peer's top-k list did not arrive within the wait limit");
    else if (fl[kFlagPeerOverflow] || own_overflow)
        *rc = fail(err, "topk_exchange_merge: a shard's candidate pool overflowed, the merged result is incomplete on every rank; redo the "
                        "step with manta_b200_score_topk_device(sync != 0) + manta_b200_topk_exchange_merge_device");
    else if (fl[kFlagInternal]) *rc = fail(err, "topk_exchange_merge: selection found fewer than k candidates");
    if (*rc && own_overflow) {
        for (int f = 0; f < kNumFlags; ++f) rt->h_flags[f] = 0;   // reported here
        rt->async_flags_pending = false;
    }
}
}  // namespace mb200
}  // extern "C++"

static int check_score_args(const MantaB200Runtime* rt, const MantaB200Candidates* set, int metric, int nq, char** err) {
    if (!rt || !set) return fail(err, "score: NULL runtime or candidate set");
    if (set->device != rt->device) return fail(err, "score: candidate set lives on device %d, runtime on %d", set->device, rt->device);
    if (metric < 0 || metric > 2) return fail(err, "score: unknown metric %d", metric);
    if (nq <= 0) return fail(err, "score: query count %d out of range", nq);
    return 0;
}

// What the tail of a fused streaming pass does with the selected lists.
struct FusedTail {
    int32_t* d_out_ids = nullptr;
    float* d_out_scores = nullptr;
    const ExchangeSink* sink = nullptr;
};

// Streams the row range [r0, r1) through the streaming kernel for all queries, four at a time.  With a tail the
// last block of every launch selects its queries' top k (one launch per query group is the whole pass); without one
// the pools are left for a selection kernel.
static int stream_rows(MantaB200Runtime* rt, const CandView& cv, const void* d_queries, int metric, int order, int k, int64_t r0,
                       int64_t r1, const SelectWs& ws, int nq, const FusedTail* tail, char** err) {
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
        a.done_blocks = (uint32_t*)rt->flags.p + 4;
        a.host_flags = rt->h_flags;
        if (tail) {
            a.fused_select = 1;
            a.out_ids = tail->d_out_ids;
            a.out_topk_scores = tail->d_out_scores;
            if (tail->sink) a.sink = *tail->sink;
        }
        cudaError_t e = launch_stream_scan(rt->stream, rt->sm_count, a);
        rt->stats.kernel_launches++;
        if (e != cudaSuccess) return fail_cuda(err, "launch score kernel", e);
        q0 += qt;
    }
    rt->stats.gemv_passes++;
    return 0;
}

static int reset_ws(MantaB200Runtime* rt, const SelectWs& ws, int nq, char** err) {
    cudaError_t e = launch_ws_reset(rt->stream, ws, nq, (uint32_t*)rt->flags.p + 4);
    rt->stats.kernel_launches++;
    if (e != cudaSuccess) return fail_cuda(err, "launch workspace reset", e);
    return 0;
}

// The tensor-core pass: query preparation kernel, scan, selection kernel; flags copied to the host words.
static int mma_pass(MantaB200Runtime* rt, const CandView& cv, const void* d_queries, int metric, int order, int k, const SelectWs& ws,
                    int nq, int32_t* d_out_ids, float* d_out_scores, const ExchangeSink* sink, bool* declined, char** err) {
    *declined = false;
    QueryPrep qp;
    if (prepare_queries(rt, cv, d_queries, nq, ws, 1, &qp, err)) return 1;
    rt->ws_dirty = true;
    rt->ws_dirty_nq = std::max(rt->ws_dirty_nq, nq);
    MmaArgs m;
    m.cv = cv;
    m.qp = qp;
    m.metric = metric;
    m.order = order;
    m.k = k;
    m.row_begin = 0;
    m.row_end = cv.rows;
    m.ws = ws;
    m.nq = nq;
    int launches = 0;
    const char* why = nullptr;
    prof_mark(rt, 0);
    cudaError_t e = launch_mma_topk(rt->stream, rt->sm_count, &rt->mma, m, &launches, &why);
    rt->stats.kernel_launches += launches;
    if (e == cudaErrorNotSupported) {
        *declined = true;   // shapes the tensor-core pass declines go to the streaming kernel
        return 0;
    }
    if (e != cudaSuccess)
        return fail(err, "score_topk(%s): tensor-core pass: %s (%s)", metric_name(metric), why ? why : "launch failed", cudaGetErrorName(e));
    prof_mark(rt, 1);
    rt->stats.mma_passes++;
    SelectArgs sa{};
    sa.ws = ws;
    sa.nq = nq;
    sa.k = k;
    sa.order = order;
    sa.out_ids = d_out_ids;
    sa.out_scores = d_out_scores;
    if (sink) sa.sink = *sink;
    e = launch_select(rt->stream, sa);
    rt->stats.kernel_launches++;
    if (e != cudaSuccess) return fail_cuda(err, "launch select kernel", e);
    // the pass's flags join the sticky host words (the copy overwrites: an earlier unsynchronised pass's report in
    // these words is replaced, as before)
    CU_TRY(cudaMemcpyAsync(rt->h_flags, ws.flags, kNumFlags * 4, cudaMemcpyDeviceToHost, rt->stream));
    return 0;
}

static int score_topk_locked(MantaB200Runtime* rt, const MantaB200Candidates* set, int metric, int order,
                             const void* d_queries, int nq, int k, int32_t* d_out_ids, float* d_out_scores, int sync,
                             char** err, const ExchangeSink* sink = nullptr) {
    const CandView& cv = set->cv;
    // a multiple of four, so that every query's bucket row starts on a 16-byte boundary
    const uint32_t nb = ((uint32_t)std::max(stream_bucket_count(rt->sm_count), mma_bucket_count(rt->sm_count)) + 3u) & ~3u;
    uint32_t cap = pool_cap_for(rt, cv, nq, k, metric);
    SelectWs ws;
    if (ensure_select_ws(rt, nq, cap, nb, &ws, err)) return 1;
    t_last_scan = MantaB200LaunchInfo{};
    bool streamed = true;
    if (mma_supported(cv, nq, metric)) {
        bool declined = false;
        if (mma_pass(rt, cv, d_queries, metric, order, k, ws, nq, d_out_ids, d_out_scores, sink, &declined, err)) return 1;
        streamed = declined;
    }
    if (streamed) {
        // one launch per group of four queries does everything: query preparation, scan, selection, clean-up
        // every query a dirty pass touched, not only the ones of this call: a two-query tensor-core pass followed by a
        // one-query pass and then a two-query streaming pass must not find the second query's old threshold
        if (rt->ws_dirty && reset_ws(rt, ws, std::max(nq, rt->ws_dirty_nq), err)) return 1;
        rt->ws_dirty = false;
        rt->ws_dirty_nq = 0;
        FusedTail tail;
        tail.d_out_ids = d_out_ids;
        tail.d_out_scores = d_out_scores;
        tail.sink = sink;
        prof_mark(rt, 0);
        if (stream_rows(rt, cv, d_queries, metric, order, k, 0, cv.rows, ws, nq, &tail, err)) {
            rt->ws_dirty = true;
            rt->ws_dirty_nq = std::max(rt->ws_dirty_nq, nq);
            return 1;
        }
        prof_mark(rt, 1);
    }
    rt->last_launch = t_last_scan;
    if (!sync) {
        rt->async_flags_pending = true;
        return 0;
    }
    CU_TRY(cudaStreamSynchronize(rt->stream));
    rt->async_flags_pending = false;
    uint32_t fl[kNumFlags];
    take_host_flags(rt, 0, fl);
    if (fl[kFlagTimeout]) return fail(err, "score_topk(%s): a bounded device wait gave up", metric_name(metric));
    if (!fl[kFlagOverflow]) {
        if (fl[kFlagInternal]) return fail(err, "score_topk(%s): selection found fewer than k candidates", metric_name(metric));
        return 0;
    }
    // The candidate pool overflowed (scores arrive in an order that keeps beating the threshold).  Redo the
    // pass in row chunks that cannot overflow, compacting the pool to the best k between chunks.
    rt->stats.chunked_reruns++;
    int64_t chunk = std::min<int64_t>(cv.rows, (int64_t)1 << 20);
    cap = (uint32_t)(chunk + k);
    if (ensure_select_ws(rt, nq, cap, nb, &ws, err)) return 1;
    rt->ws_dirty = true;
    rt->ws_dirty_nq = std::max(rt->ws_dirty_nq, nq);
    if (reset_ws(rt, ws, nq, err)) return 1;
    SelectArgs sa{};
    sa.nq = nq;
    sa.k = k;
    sa.order = order;
    if (sink) sa.sink = *sink;
    for (int64_t r0 = 0; r0 < cv.rows; r0 += chunk) {
        int64_t r1 = std::min(cv.rows, r0 + chunk);
        if (stream_rows(rt, cv, d_queries, metric, order, k, r0, r1, ws, nq, nullptr, err)) return 1;
        sa.ws = ws;
        sa.write_back = (r1 < cv.rows) ? 1 : 0;
        sa.out_ids = sa.write_back ? nullptr : d_out_ids;
        sa.out_scores = sa.write_back ? nullptr : d_out_scores;
        ExchangeSink none;
        if (sa.write_back) sa.sink = none;
        else if (sink) sa.sink = *sink;
        cudaError_t e = launch_select(rt->stream, sa);
        rt->stats.kernel_launches++;
        if (e != cudaSuccess) return fail_cuda(err, "launch select kernel", e);
    }
    CU_TRY(cudaMemcpyAsync(rt->h_flags, ws.flags, kNumFlags * 4, cudaMemcpyDeviceToHost, rt->stream));
    CU_TRY(cudaStreamSynchronize(rt->stream));
    take_host_flags(rt, 0, fl);
    if (fl[kFlagOverflow] || fl[kFlagInternal])
        return fail(err, "score_topk(%s): chunked selection failed (flags %u %u)", metric_name(metric), fl[kFlagOverflow], fl[kFlagInternal]);
    return 0;
}

static int check_topk_args(const MantaB200Candidates* set, int order, int k, char** err) {
    if (order != MANTA_B200_ORDER_LARGEST && order != MANTA_B200_ORDER_SMALLEST) return fail(err, "score_topk: unknown order %d", order);
    // message of topKTensor, runtime/backend/tensor_ops.go:1532
    if (k <= 0 || k > set->cv.rows) return fail(err, "topk limit %d out of range for %lld scores", k, (long long)set->cv.rows);
    if (k > kMaxK) return fail(err, "topk limit %d exceeds the fused pass maximum %d", k, kMaxK);
    return 0;
}

extern "C++" {
namespace mb200 {
// The shard pass of a sharded step (exchange.cu): fused score + top-k whose selection stores the lists into every
// rank's inbox.  Always asynchronous: a pool overflow is reported by the next synchronisation, not redone in chunks
// (the peers would already hold the incomplete list).  Takes the runtime's lock itself.
int score_topk_into_sink(MantaB200Runtime* rt, const MantaB200Candidates* set, int metric, int order, const void* d_queries, int nq,
                         int k, const ExchangeSink& sink, char** err) {
    if (check_score_args(rt, set, metric, nq, err)) return 1;
    if (check_topk_args(set, order, k, err)) return 1;
    if (!d_queries) return fail(err, "score_topk: NULL buffer");
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    rt->stats.score_topk_calls++;
    return score_topk_locked(rt, set, metric, order, d_queries, nq, k, nullptr, nullptr, 0, err, &sink);
}
}  // namespace mb200
}  // extern "C++"

int manta_b200_score_topk_device(MantaB200Runtime* rt, const MantaB200Candidates* set, int metric, int order,
                                 const void* d_queries, int nq, int k, int32_t* d_out_ids, float* d_out_scores,
                                 int sync, char** err) {
    if (check_score_args(rt, set, metric, nq, err)) return 1;
    if (check_topk_args(set, order, k, err)) return 1;
    if (!d_queries || !d_out_ids || !d_out_scores) return fail(err, "score_topk: NULL buffer");
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    rt->stats.score_topk_calls++;
    return score_topk_locked(rt, set, metric, order, d_queries, nq, k, d_out_ids, d_out_scores, sync, err);
}

int manta_b200_score_topk(MantaB200Runtime* rt, const MantaB200Candidates* set, int metric, int order,
                          const uint16_t* queries, int nq, int k, int32_t* out_ids, float* out_scores, char** err) {
    if (check_score_args(rt, set, metric, nq, err)) return 1;
    if (check_topk_args(set, order, k, err)) return 1;
    if (!queries || !out_ids || !out_scores) return fail(err, "score_topk: NULL buffer");
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    rt->stats.score_topk_calls++;
    const size_t qbytes = (size_t)nq * set->cv.cols * 2;
    const size_t obytes = (size_t)nq * k * 4;
    if (ensure(rt, rt->queries, qbytes, err)) return 1;
    const size_t qpad = (qbytes + 255) / 256 * 256, opad = (obytes + 255) / 256 * 256;
    if (ensure_host(rt, qpad + 2 * opad, err)) return 1;
    char* hq = (char*)rt->h_stage;
    char* hi = hq + qpad;
    char* hs = hi + opad;
    memcpy(hq, queries, qbytes);
    CU_TRY(cudaMemcpyAsync(rt->queries.p, hq, qbytes, cudaMemcpyHostToDevice, rt->stream));
    rt->stats.h2d_bytes += qbytes;
    // The selection writes ids and scores straight into the pinned staging buffer (device-addressable host memory): the
    // synchronisation that reads the pass's flags is also the one that makes the results visible, no copy back, no second
    // synchronisation.
    int rc = score_topk_locked(rt, set, metric, order, rt->queries.p, nq, k, (int32_t*)hi, (float*)hs, 1, err);
    if (rc) return rc;
    memcpy(out_ids, hi, obytes);
    memcpy(out_scores, hs, obytes);
    rt->stats.d2h_bytes += 2 * obytes;
    return 0;
}

int manta_b200_score(MantaB200Runtime* rt, const MantaB200Candidates* set, int metric, const uint16_t* queries,
                     int nq, float* out_scores, char** err) {
    if (check_score_args(rt, set, metric, nq, err)) return 1;
    if (!queries || !out_scores) return fail(err, "score: NULL buffer");
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    rt->stats.score_calls++;
    const CandView& cv = set->cv;
    if (cv.rows == 0) return 0;
    const size_t qbytes = (size_t)nq * cv.cols * 2;
    const size_t obytes = (size_t)nq * cv.rows * 4;
    if (ensure(rt, rt->queries, qbytes, err)) return 1;
    if (ensure(rt, rt->misc, obytes, err)) return 1;
    CU_TRY(cudaMemcpyAsync(rt->queries.p, queries, qbytes, cudaMemcpyHostToDevice, rt->stream));
    t_last_scan = MantaB200LaunchInfo{};
    for (int q0 = 0; q0 < nq;) {
        const int left = nq - q0;
        const int qt = left >= 4 ? 4 : (left >= 2 ? 2 : 1);
        StreamArgs a{};
        a.cv = cv;
        a.queries = (const __half*)rt->queries.p;
        a.q0 = q0;
        a.qt = qt;
        a.metric = metric;
        a.mode = kModeScores;
        a.row_begin = 0;
        a.row_end = cv.rows;
        a.out_scores = (float*)rt->misc.p;
        cudaError_t e = launch_stream_scan(rt->stream, rt->sm_count, a);
        rt->stats.kernel_launches++;
        if (e != cudaSuccess) return fail_cuda(err, "launch score kernel", e);
        q0 += qt;
    }
    rt->last_launch = t_last_scan;
    CU_TRY(cudaMemcpyAsync(out_scores, rt->misc.p, obytes, cudaMemcpyDeviceToHost, rt->stream));
    CU_TRY(cudaStreamSynchronize(rt->stream));
    rt->stats.h2d_bytes += qbytes;
    rt->stats.d2h_bytes += obytes;
    return 0;
}

// ---- per-query candidate sets -----------------------------------------------------------------------------------
static int batched_common(MantaB200Runtime* rt, int metric, int order, const float* queries, const float* docs, int nq, int64_t rows,
                          int cols, int mem, int k, float* out_full, int32_t* out_ids, float* out_scores, char** err) {
    if (!rt || !queries || !docs) return fail(err, "score: NULL argument");
    if (metric < 0 || metric > 2) return fail(err, "score: unknown metric %d", metric);
    if (nq <= 0 || rows <= 0 || cols <= 0) return fail(err, "score mismatch [%d %d] x [%d %lld %d]", nq, cols, nq, (long long)rows, cols);
    if (mem != MANTA_B200_MEM_HOST && mem != MANTA_B200_MEM_DEVICE_COPY) return fail(err, "score: mem must be HOST or DEVICE_COPY");
    const bool topk = out_ids != nullptr;
    if (topk) {
        if (order != MANTA_B200_ORDER_LARGEST && order != MANTA_B200_ORDER_SMALLEST) return fail(err, "score_topk: unknown order %d", order);
        // message of topKTensor for rank-2 scores, runtime/backend/tensor_ops.go:1561
        if (k <= 0 || k > rows) return fail(err, "topk limit %d out of range for row width %lld", k, (long long)rows);
        if (k > kMaxK) return fail(err, "topk limit %d exceeds the fused pass maximum %d", k, kMaxK);
        if (rows > (int64_t)1 << 26) return fail(err, "score_topk: %lld rows per query exceed the per-query form's limit", (long long)rows);
    }
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    const bool host = mem == MANTA_B200_MEM_HOST;
    const size_t qbytes = (size_t)nq * cols * 4, dbytes = (size_t)nq * rows * cols * 4, sbytes = (size_t)nq * rows * 4;
    const float* d_q = queries;
    const float* d_d = docs;
    if (host) {
        if (ensure(rt, rt->batch_in, qbytes + 256 + dbytes, err)) return 1;
        float* bq = (float*)rt->batch_in.p;
        float* bd = (float*)((char*)rt->batch_in.p + (qbytes + 255) / 256 * 256);
        CU_TRY(cudaMemcpyAsync(bq, queries, qbytes, cudaMemcpyHostToDevice, rt->stream));
        CU_TRY(cudaMemcpyAsync(bd, docs, dbytes, cudaMemcpyHostToDevice, rt->stream));
        rt->stats.h2d_bytes += qbytes + dbytes;
        d_q = bq;
        d_d = bd;
    }
    float* d_full = nullptr;
    if (out_full) {
        d_full = out_full;
        if (host) {
            if (ensure(rt, rt->misc, sbytes, err)) return 1;
            d_full = (float*)rt->misc.p;
        }
    }
    SelectWs ws{};
    if (topk && ensure_select_ws(rt, nq, (uint32_t)rows, 1, &ws, err)) return 1;
    t_last_scan = MantaB200LaunchInfo{};
    cudaError_t e = launch_score_batched(rt->stream, rt->sm_count, metric, d_q, d_d, nq, rows, cols, order, d_full, ws, topk ? 1 : 0);
    rt->last_launch = t_last_scan;
    rt->stats.kernel_launches++;
    rt->stats.score_calls++;
    if (e != cudaSuccess) return fail_cuda(err, "launch batched score kernel", e);
    if (out_full && host) {
        CU_TRY(cudaMemcpyAsync(out_full, d_full, sbytes, cudaMemcpyDeviceToHost, rt->stream));
        rt->stats.d2h_bytes += sbytes;
    }
    if (topk) {
        const size_t obytes = (size_t)nq * k * 4;
        int32_t* d_ids = out_ids;
        float* d_sc = out_scores;
        if (host) {
            if (ensure(rt, rt->out_ids, obytes, err)) return 1;
            if (ensure(rt, rt->out_scores, obytes, err)) return 1;
            d_ids = (int32_t*)rt->out_ids.p;
            d_sc = (float*)rt->out_scores.p;
        }
        SelectArgs sa{};
        sa.ws = ws;
        sa.nq = nq;
        sa.k = k;
        sa.order = order;
        sa.out_ids = d_ids;
        sa.out_scores = d_sc;
        sa.reset_after = 1;
        e = launch_select(rt->stream, sa);
        rt->stats.kernel_launches++;
        if (e != cudaSuccess) return fail_cuda(err, "launch select kernel", e);
        if (host) {
            CU_TRY(cudaMemcpyAsync(out_ids, d_ids, obytes, cudaMemcpyDeviceToHost, rt->stream));
            CU_TRY(cudaMemcpyAsync(out_scores, d_sc, obytes, cudaMemcpyDeviceToHost, rt->stream));
            rt->stats.d2h_bytes += 2 * obytes;
        }
    }
    CU_TRY(cudaStreamSynchronize(rt->stream));
    return 0;
}

int manta_b200_score_batched(MantaB200Runtime* rt, int metric, const float* queries, const float* docs, int nq, int64_t rows,
                             int cols, int mem, float* out, char** err) {
    if (!out) return fail(err, "score: NULL output");
    return batched_common(rt, metric, MANTA_B200_ORDER_LARGEST, queries, docs, nq, rows, cols, mem, 0, out, nullptr, nullptr, err);
}

int manta_b200_score_topk_batched(MantaB200Runtime* rt, int metric, int order, const float* queries, const float* docs, int nq,
                                  int64_t rows, int cols, int mem, int k, int32_t* out_ids, float* out_scores, char** err) {
    if (!out_ids || !out_scores) return fail(err, "score_topk: NULL output");
    return batched_common(rt, metric, order, queries, docs, nq, rows, cols, mem, k, nullptr, out_ids, out_scores, err);
}

// ---- embedding front end ------------------------------------------------------------------------------------
int manta_b200_embedder_bind(MantaB200Runtime* rt, int vocab, int dim, int out_dim, const uint16_t* table,
                             const uint16_t* projection, int mem, MantaB200Embedder** out, char** err) {
    if (!rt || !table || !projection || !out) return fail(err, "embedder_bind: NULL argument");
    *out = nullptr;
    if (vocab <= 0 || dim <= 0 || out_dim <= 0 || out_dim > 1024 || dim > 4096)
        return fail(err, "embedder_bind: shape [%d,%d] x [%d,%d] out of range", vocab, dim, dim, out_dim);
    if (mem != MANTA_B200_MEM_HOST && mem != MANTA_B200_MEM_DEVICE_COPY) return fail(err, "embedder_bind: mem must be HOST or DEVICE_COPY");
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    MantaB200Embedder* e = new (std::nothrow) MantaB200Embedder();
    if (!e) return fail(err, "embedder_bind: out of host memory");
    e->device = rt->device;
    e->vocab = vocab;
    e->dim = dim;
    e->out_dim = out_dim;
    const cudaMemcpyKind kind = (mem == MANTA_B200_MEM_HOST) ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice;
    const size_t tb = (size_t)vocab * dim * 2, pb = (size_t)dim * out_dim * 2;
    cudaError_t ce = cudaMalloc(&e->d_table, tb);
    if (ce == cudaSuccess) ce = cudaMalloc(&e->d_proj, pb);
    if (ce == cudaSuccess) ce = cudaMemcpyAsync(e->d_table, table, tb, kind, rt->stream);
    if (ce == cudaSuccess) ce = cudaMemcpyAsync(e->d_proj, projection, pb, kind, rt->stream);
    if (ce == cudaSuccess && embed_mma_supported(dim, out_dim)) {
        ce = cudaMalloc(&e->d_proj_t, pb);
        if (ce == cudaSuccess) {
            ce = launch_transpose_f16(rt->stream, e->d_proj, dim, out_dim, e->d_proj_t);
            rt->stats.kernel_launches++;
        }
    }
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(rt->stream);
    if (ce != cudaSuccess) {
        if (e->d_table) cudaFree(e->d_table);
        if (e->d_proj) cudaFree(e->d_proj);
        if (e->d_proj_t) cudaFree(e->d_proj_t);
        delete e;
        return fail_cuda(err, "embedder_bind", ce);
    }
    rt->stats.bind_calls++;
    rt->stats.bound_bytes += tb + pb;
    if (mem == MANTA_B200_MEM_HOST) rt->stats.h2d_bytes += tb + pb;
    *out = e;
    return 0;
}

int manta_b200_embedder_unbind(MantaB200Runtime* rt, MantaB200Embedder* emb, char** err) {
    if (!emb) return 0;
    if (!rt) return fail(err, "embedder_unbind: NULL runtime");
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    CU_TRY(cudaStreamSynchronize(rt->stream));
    cudaFree(emb->d_table);
    cudaFree(emb->d_proj);
    if (emb->d_proj_t) cudaFree(emb->d_proj_t);
    delete emb;
    return 0;
}

// Runs the embed kernel on device tokens / mask into d_out_f32 and / or d_out_f16.  Caller holds the lock.  With
// sync the bad-token word is read back and reported here, otherwise at the next runtime_synchronize.
static int embed_device_locked(MantaB200Runtime* rt, const MantaB200Embedder* emb, const int32_t* d_tok, const int32_t* d_mask,
                               int batch, int seq, int pool_order, float* d_out_f32, void* d_out_f16, int sync, char** err) {
    if (ensure(rt, rt->embed_flag, 16, err)) return 1;
    uint32_t* d_flag = (uint32_t*)rt->embed_flag.p;
    int32_t* d_bad = (int32_t*)rt->embed_flag.p + 1;
    CU_TRY(cudaMemsetAsync(d_flag, 0, 8, rt->stream));
    // mean_pool(normalize(x @ P)) on shapes the tensor cores take: the per-token product only yields the row norms
    const float* d_norms = nullptr;
    if (pool_order != 0 && emb->d_proj_t != nullptr) {
        if (ensure(rt, rt->tok_norms, (size_t)batch * seq * 4, err)) return 1;
        cudaError_t en = launch_embed_token_norms(rt->stream, emb->d_table, emb->vocab, emb->dim, emb->d_proj_t, emb->out_dim, d_tok,
                                                  (int64_t)batch * seq, (float*)rt->tok_norms.p, d_flag);
        rt->stats.kernel_launches++;
        if (en != cudaSuccess) return fail_cuda(err, "launch embed projection kernel", en);
        d_norms = (const float*)rt->tok_norms.p;
    }
    cudaError_t e = launch_embed_pooled(rt->stream, emb->d_table, emb->vocab, emb->dim, emb->d_proj, emb->out_dim, d_tok, d_mask, batch,
                                        seq, pool_order, d_norms, d_out_f32, d_out_f16, d_bad, d_flag);
    rt->stats.kernel_launches++;
    if (e != cudaSuccess) return fail_cuda(err, "launch embed kernel", e);
    CU_TRY(cudaMemcpyAsync(&rt->h_flags[10], d_flag, 8, cudaMemcpyDeviceToHost, rt->stream));
    if (!sync) {
        rt->async_embed_pending = true;
        return 0;
    }
    CU_TRY(cudaStreamSynchronize(rt->stream));
    rt->async_embed_pending = false;
    if (rt->h_flags[10] == 2u) return fail(err, "embed: a bounded wait of the tensor-core projection ran out");
    if (rt->h_flags[10]) return fail(err, "gather index %d out of range", (int32_t)rt->h_flags[11]);  // tensor_ops.go:803
    return 0;
}

// Uploads host tokens + mask (staged in rt->out_ids), then embeds into rt->queries (f16) and optionally rt->misc (f32).
static int embed_locked(MantaB200Runtime* rt, const MantaB200Embedder* emb, const int32_t* tokens, const int32_t* mask, int batch,
                        int seq, int pool_order, bool want_f32, char** err, int sync = 1) {
    const size_t tb = (size_t)batch * seq * 4;
    if (ensure(rt, rt->out_ids, 2 * tb, err)) return 1;
    if (ensure(rt, rt->queries, (size_t)batch * emb->out_dim * 2, err)) return 1;
    if (want_f32 && ensure(rt, rt->misc, (size_t)batch * emb->out_dim * 4, err)) return 1;
    int32_t* d_tok = (int32_t*)rt->out_ids.p;
    int32_t* d_mask = d_tok + (size_t)batch * seq;
    CU_TRY(cudaMemcpyAsync(d_tok, tokens, tb, cudaMemcpyHostToDevice, rt->stream));
    CU_TRY(cudaMemcpyAsync(d_mask, mask, tb, cudaMemcpyHostToDevice, rt->stream));
    rt->stats.h2d_bytes += 2 * tb;
    return embed_device_locked(rt, emb, d_tok, d_mask, batch, seq, pool_order, want_f32 ? (float*)rt->misc.p : nullptr, rt->queries.p,
                               sync, err);
}

static int check_embed_args(const MantaB200Runtime* rt, const MantaB200Embedder* emb, const int32_t* tokens, const int32_t* mask,
                            int batch, int seq, int pool_order, char** err) {
    if (!rt || !emb || !tokens || !mask) return fail(err, "embed: NULL argument");
    if (emb->device != rt->device) return fail(err, "embed: embedder lives on device %d, runtime on %d", emb->device, rt->device);
    if (batch <= 0 || seq <= 0 || seq > 8192) return fail(err, "embed: tokens shape [%d,%d] out of range", batch, seq);
    if (pool_order != MANTA_B200_POOL_THEN_NORMALIZE && pool_order != MANTA_B200_NORMALIZE_THEN_POOL) return fail(err, "embed: unknown pool order %d", pool_order);
    return 0;
}

int manta_b200_embed_pooled(MantaB200Runtime* rt, const MantaB200Embedder* emb, const int32_t* tokens, const int32_t* mask,
                            int batch, int seq, int pool_order, float* out, char** err) {
    if (check_embed_args(rt, emb, tokens, mask, batch, seq, pool_order, err)) return 1;
    if (!out) return fail(err, "embed: NULL output");
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    if (embed_locked(rt, emb, tokens, mask, batch, seq, pool_order, true, err)) return 1;
    const size_t ob = (size_t)batch * emb->out_dim * 4;
    CU_TRY(cudaMemcpyAsync(out, rt->misc.p, ob, cudaMemcpyDeviceToHost, rt->stream));
    CU_TRY(cudaStreamSynchronize(rt->stream));
    rt->stats.d2h_bytes += ob;
    return 0;
}

int manta_b200_embed_device(MantaB200Runtime* rt, const MantaB200Embedder* emb, const int32_t* d_tokens, const int32_t* d_mask,
                            int batch, int seq, int pool_order, void* d_out_queries_f16, int sync, char** err) {
    if (check_embed_args(rt, emb, d_tokens, d_mask, batch, seq, pool_order, err)) return 1;
    if (!d_out_queries_f16) return fail(err, "embed: NULL output");
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    return embed_device_locked(rt, emb, d_tokens, d_mask, batch, seq, pool_order, nullptr, d_out_queries_f16, sync, err);
}

int manta_b200_embed_score_topk(MantaB200Runtime* rt, const MantaB200Embedder* emb, const MantaB200Candidates* set,
                                const int32_t* tokens, const int32_t* mask, int batch, int seq, int pool_order, int metric,
                                int order, int k, int32_t* out_ids, float* out_scores, char** err) {
    if (check_embed_args(rt, emb, tokens, mask, batch, seq, pool_order, err)) return 1;
    if (check_score_args(rt, set, metric, batch, err)) return 1;
    if (check_topk_args(set, order, k, err)) return 1;
    if (!out_ids || !out_scores) return fail(err, "embed_score_topk: NULL output");
    if (set->cv.cols != emb->out_dim) return fail(err, "score mismatch [%d %d] x [%lld %d]", batch, emb->out_dim, (long long)set->cv.rows, set->cv.cols);
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    rt->stats.score_topk_calls++;
    const size_t obytes = (size_t)batch * k * 4;
    // One synchronisation for the whole call: the embedding kernels are enqueued without one (their flag words are read
    // below), and the selection writes ids and scores straight into the pinned staging buffer.
    const size_t opad = (obytes + 255) / 256 * 256;
    if (ensure_host(rt, 2 * opad, err)) return 1;
    int32_t* h_ids = (int32_t*)rt->h_stage;
    float* h_sc = (float*)((char*)rt->h_stage + opad);
    if (embed_locked(rt, emb, tokens, mask, batch, seq, pool_order, false, err, 0)) return 1;
    int rc = score_topk_locked(rt, set, metric, order, rt->queries.p, batch, k, h_ids, h_sc, 1, err);
    // the stream is synchronised (or the pass failed to launch): the embedding kernels' report first
    const bool embed_pending = rt->async_embed_pending;
    rt->async_embed_pending = false;
    if (embed_pending && rc == 0) {
        if (rt->h_flags[10] == 2u) return fail(err, "embed: a bounded wait of the tensor-core projection ran out");
        if (rt->h_flags[10]) return fail(err, "gather index %d out of range", (int32_t)rt->h_flags[11]);  // tensor_ops.go:803
    }
    if (rc) return rc;
    memcpy(out_ids, h_ids, obytes);
    memcpy(out_scores, h_sc, obytes);
    rt->stats.d2h_bytes += 2 * obytes;
    return 0;
}

int manta_b200_q8_accumulators(MantaB200Runtime* rt, const MantaB200Candidates* set, const uint16_t* query,
                               int32_t* out_acc, char** err) {
    if (check_score_args(rt, set, MANTA_B200_METRIC_DOT, 1, err)) return 1;
    if (set->cv.layout != MANTA_B200_LAYOUT_Q8_ROW_F32) return fail(err, "q8_accumulators: candidate set is not q8");
    if (!query || !out_acc) return fail(err, "q8_accumulators: NULL buffer");
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    const CandView& cv = set->cv;
    if (cv.rows == 0) return 0;
    const size_t qbytes = (size_t)cv.cols * 2;
    const size_t obytes = (size_t)cv.rows * 12;
    if (ensure(rt, rt->queries, qbytes, err)) return 1;
    if (ensure(rt, rt->misc, obytes, err)) return 1;
    CU_TRY(cudaMemcpyAsync(rt->queries.p, query, qbytes, cudaMemcpyHostToDevice, rt->stream));
    StreamArgs a{};
    a.cv = cv;
    a.queries = (const __half*)rt->queries.p;
    a.q0 = 0;
    a.qt = 1;
    a.metric = MANTA_B200_METRIC_COSINE;
    a.mode = kModeAccum;
    a.row_begin = 0;
    a.row_end = cv.rows;
    a.out_acc = (int32_t*)rt->misc.p;
    cudaError_t e = launch_stream_scan(rt->stream, rt->sm_count, a);
    rt->stats.kernel_launches++;
    if (e != cudaSuccess) return fail_cuda(err, "launch score kernel", e);
    CU_TRY(cudaMemcpyAsync(out_acc, rt->misc.p, obytes, cudaMemcpyDeviceToHost, rt->stream));
    CU_TRY(cudaStreamSynchronize(rt->stream));
    return 0;
}

int manta_b200_topk_merge_device(MantaB200Runtime* rt, int order, const int32_t* d_ids, const float* d_scores,
                                 int lists, int64_t list_stride, int nq, int k, int32_t* d_out_ids,
                                 float* d_out_scores, int sync, char** err) {
    if (!rt || !d_ids || !d_scores || !d_out_ids || !d_out_scores) return fail(err, "topk_merge: NULL argument");
    if (lists <= 0 || nq <= 0 || k <= 0 || k > kMaxK) return fail(err, "topk_merge: bad shape (lists %d, nq %d, k %d)", lists, nq, k);
    if (list_stride == 0) list_stride = (int64_t)nq * k;
    if (list_stride < (int64_t)nq * k) return fail(err, "topk_merge: list stride %lld is smaller than one list", (long long)list_stride);
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    SelectWs ws;
    if (ensure_select_ws(rt, nq, (uint32_t)(lists * k), 1, &ws, err)) return 1;
    cudaError_t e = launch_lists_to_pool(rt->stream, d_ids, d_scores, lists, list_stride, nq, k, order, ws);
    rt->stats.kernel_launches++;
    if (e != cudaSuccess) return fail_cuda(err, "launch lists_to_pool", e);
    SelectArgs sa{};
    sa.ws = ws;
    sa.nq = nq;
    sa.k = k;
    sa.order = order;
    sa.out_ids = d_out_ids;
    sa.out_scores = d_out_scores;
    sa.reset_after = 1;
    sa.flags_out = rt->h_flags + 4;   // "fewer than k entries in the lists" is raised in the merge's host words
    e = launch_select(rt->stream, sa);
    rt->stats.kernel_launches++;
    if (e != cudaSuccess) return fail_cuda(err, "launch select kernel", e);
    if (!sync) {
        rt->async_exchange_pending = true;
        return 0;
    }
    CU_TRY(cudaStreamSynchronize(rt->stream));
    uint32_t fl[kNumFlags];
    take_host_flags(rt, 4, fl);
    if (fl[kFlagInternal]) return fail(err, "topk_merge: the lists hold fewer than k entries");
    return 0;
}

int manta_b200_gather_rows(MantaB200Runtime* rt, const MantaB200Candidates* set, const int32_t* ids, int64_t n,
                           float* out, char** err) {
    if (!rt || !set) return fail(err, "gather: NULL runtime or candidate set");
    if (n < 0 || (n > 0 && (!ids || !out))) return fail(err, "gather: NULL buffer");
    if (n == 0) return 0;
    std::lock_guard<std::mutex> lk(rt->mu);
    CU_TRY(cudaSetDevice(rt->device));
    const CandView& cv = set->cv;
    const size_t ibytes = (size_t)n * 4, obytes = (size_t)n * cv.cols * 4;
    if (ensure(rt, rt->out_ids, ibytes + 64, err)) return 1;
    if (ensure(rt, rt->misc, obytes, err)) return 1;
    if (ensure(rt, rt->embed_flag, 16, err)) return 1;
    // out_ids: [n ids][pad][bad id]; the "bad id seen" word is word 2 of the small flag buffer the embedding front
    // end keeps its own two words in
    int32_t* d_ids = (int32_t*)rt->out_ids.p;
    int32_t* d_bad = d_ids + n + 8;
    uint32_t* d_flag = (uint32_t*)rt->embed_flag.p + 2;
    CU_TRY(cudaMemcpyAsync(d_ids, ids, ibytes, cudaMemcpyHostToDevice, rt->stream));
    CU_TRY(cudaMemsetAsync(d_flag, 0, 4, rt->stream));
    launch_gather_rows(rt->stream, cv, d_ids, n, (float*)rt->misc.p, d_bad, d_flag);
    rt->stats.kernel_launches++;
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaMemcpyAsync(&rt->h_flags[8], d_flag, 4, cudaMemcpyDeviceToHost, rt->stream));
    CU_TRY(cudaMemcpyAsync(&rt->h_flags[9], d_bad, 4, cudaMemcpyDeviceToHost, rt->stream));
    CU_TRY(cudaMemcpyAsync(out, rt->misc.p, obytes, cudaMemcpyDeviceToHost, rt->stream));
    CU_TRY(cudaStreamSynchronize(rt->stream));
    if (rt->h_flags[8]) return fail(err, "gather index %d out of range", (int32_t)rt->h_flags[9]);  // tensor_ops.go:803
    rt->stats.h2d_bytes += ibytes;
    rt->stats.d2h_bytes += obytes;
    return 0;
}

}  // extern "C"
