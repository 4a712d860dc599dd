// tcgen05 tensor-core scoring pass: a batch of queries (two or more over f16 / q8 rows, eight or more over q4 rows)
// against packed candidate rows as a dense contraction.  One persistent CTA per SM; candidate tiles of 128 rows stream
// through a TMA-fed shared-memory ring, tcgen05.mma accumulates [128 rows x N columns] in tensor memory (int32 for q8:
// the columns are the high int8 planes of up to 256 queries, or both planes of up to 128; f32 for f16 and q4), and the
// epilogue warps read the accumulators back (tcgen05.ld), finish the scores with the same epilogue functions as the
// streaming kernel and filter them into the top-k pools.  Operand B is read where the queries already lie (the f16 rows
// as they came, the int8 planes of the query preparation); q4 rows get a built, permuted f16 operand.
//
// Warp roles: 0 = TMA producer, 1 = MMA issuer (owns the tensor-memory allocation), then SUBS = 2 or 4 epilogue warps per
// 32-lane quadrant of tensor memory (each taking every SUBS-th 16-query chunk), one threshold refresher, and for q4 rows
// four converter warps: 11 to 19 warps.  With four epilogue warps per quadrant (608 threads x 96 registers) the exact
// scoring of a chunk that passes the cheap filter re-reads its accumulators four queries at a time instead of keeping
// sixteen finished scores live.  The producer, the issuer and the converters are single threads (or one thread per row)
// on their own latency chains: their loops count stages and phases instead of dividing, and build descriptors from one
// base -- the issuer's own scalar instructions were what the tensor core used to wait for.
//
// Every wait in this file is bounded: a wait that runs out sets the abort flag of the CTA and the time-out flag
// of the pass, every role leaves its loop, tensor memory is released and the kernel returns; the host then
// reports the failure (and the streaming kernel can redo the pass).
#include <cuda.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>

#include "mma.h"
#include "tc.cuh"

namespace mb200 {

namespace {

constexpr int kTileRows = 128;
constexpr int kChunkBytes = 128;      // K extent of one pipeline stage, in bytes (one 128-byte swizzle span)
// SUBS (template parameter of the kernel) = epilogue warps per tensor-memory quadrant; warp s of a quadrant takes the
// 16-query chunks s, s + SUBS, ...
constexpr int kConvWarps = 4;          // q4 candidates: warps that unpack nibbles to f16 into the operand ring
constexpr int mma_threads(int subs, bool conv = false) { return 32 * (2 + 4 * subs + 1 + (conv ? kConvWarps : 0)); }
constexpr int kRawStages = 3;         // q4 candidates: ring of raw (packed) tiles in front of the converter warps
constexpr int kRawStageBytes = kTileRows * kChunkBytes;   // one swizzled 128 x 128-byte box of nibbles
constexpr int kQ4Blocks = 8;          // q4 rows the tensor-core pass takes are 256 columns = eight blocks = one raw chunk
constexpr int kMmaCols = 256;         // N of one MMA
constexpr int kBucketSlots = 4;       // bucket slots per epilogue warp (tiles rotate through them)
constexpr int kRefStage = 2560;       // bucket maxima per query the refresher looks at (20 merged values per lane)
constexpr size_t kSmemLimit = 232448; // dynamic shared memory one CTA may ask for (227 KB)

struct KernelArgs {
    CandView cv;
    const QueryHeader* headers;   // [nq] (global query index)
    SelectWs ws;
    uint32_t* ready;              // CTAs that have published their observed tiles
    int q0;                       // first query of this group
    int qn;                       // queries in this group
    int ncols;                    // N of the MMA (multiple of 16)
    int lo_off;                   // q8: column offset of the low planes
    int kchunks;                  // 128-byte chunks per row
    int stages;
    int epi_subs;                 // epilogue warps per tensor-memory quadrant (2 or 4): which instantiation runs
    int b_resident;               // operand B (all K chunks) is loaded once and stays in shared memory
    int b_second_rows;            // > 0: operand B is read from the query planes themselves and its low planes are a second
                                  // box of this many rows (map_b2) behind the high planes; 0: one box per chunk
    int metric;
    int order;
    int k;
    int filtered;                 // 0: everything enters the pool (small sets)
    int observe_tiles;            // tiles per CTA scored before the first bound exists (replayed at the end)
    int raw_chunks;               // q4: 128-byte chunks of packed nibbles per row (each becomes four f16 K chunks)
    int hi_first;                 // q8: only the high planes are contracted (ncols = queries); see the kernel's note
    const int8_t* plane_lo;       // q8, hi_first: low planes of this group's queries, [qn][plane_stride]
    const float* lo_norms;        // q8, hi_first: their norms, rounded up a shade (written by build_b_kernel)
    int plane_stride;
    int64_t row_begin;
    int64_t row_end;
};

// Exact int32 dot product of one q8 row with one low query plane (n16 16-byte pieces), computed by the whole warp: every
// lane takes pieces lane, lane + 32, ... so that all loads of a pair are in flight together.  Used for the rare
// (row, query) pair that passes the high-plane filter.
__device__ __forceinline__ int lo_plane_dot_warp(const uint4* __restrict__ row, const uint4* __restrict__ lo, int n16, int lane) {
    int acc = 0;
#pragma unroll 2
    for (int i = lane; i < n16; i += 32) {
        const uint4 r = __ldg(row + i), q = __ldg(lo + i);
        acc = __dp4a((int)r.x, (int)q.x, acc);
        acc = __dp4a((int)r.y, (int)q.y, acc);
        acc = __dp4a((int)r.z, (int)q.z, acc);
        acc = __dp4a((int)r.w, (int)q.w, acc);
    }
    return __reduce_add_sync(0xffffffffu, acc);
}

// Scores of N consecutive queries for one candidate row (one lane).  METRIC is a compile-time constant so that
// the evaluations are one basic block the compiler can interleave.
template <bool I8, int METRIC, int N>
__device__ __forceinline__ void score_n(const uint32_t (&vh)[N], const uint32_t (&vl)[N], uint32_t stat, float rinv, float sd,
                                        const QueryHeader* hdr_s, int c0, int qn, bool rv, float sign, float (&g)[N], uint32_t (&o)[N]) {
#pragma unroll
    for (int jj = 0; jj < N; ++jj) {
        const int j = min(c0 + jj, qn - 1);
        float score;
        if constexpr (I8)
            score = q8_finish(METRIC, (int)vh[jj], (int)vl[jj], (int)stat, rinv, sd, hdr_s[j]);
        else
            score = float_finish(METRIC, __uint_as_float(vh[jj]), __uint_as_float(stat), rinv, hdr_s[j], hdr_s[j].qn2d);
        g[jj] = score * sign + 0.0f;
        o[jj] = (rv && c0 + jj < qn) ? ord_from_float(g[jj]) : 0u;   // 0 never passes (bounds are >= 1)
    }
}

// Q4: the candidates are q4 rows of 256 columns (eight blocks of 32).  The TMA producer fills a ring of raw tiles (128
// rows x 128 bytes of nibbles, 128-byte swizzle) and four converter warps, one thread per row, unpack each raw tile
// into four f16 operand stages holding the CODES (small integers, exact in f16).  The MMA issuer gives every block its
// own accumulator columns (block b, query j -> column b * ncols + j; K = 32 per block, two instructions), so tensor
// memory holds the exact per-block sums of code * query, and the epilogue applies the row's eight block scales with
// eight fused multiply-adds per score -- the arithmetic of the streaming kernel with the exact f16 query.
// Within every group of eight elements the converter emits them in the order 0,4,1,5,2,6,3,7 (what the nibble
// unpack yields pairwise); operand B is built with the same order, and a contraction does not care.
template <bool I8, int METRIC, int SUBS, bool Q4>
__global__ void __launch_bounds__(mma_threads(SUBS, Q4), 1)
mma_scan_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_b2, const KernelArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = a.stages;
    constexpr int kEpiSubs = SUBS;
    constexpr int kEpiWarps = 4 * SUBS;
    const uint32_t b_stage_bytes = (uint32_t)a.ncols * kChunkBytes;
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sA = base;
    unsigned char* sB = sA + (size_t)S * kTileRows * kChunkBytes;
    unsigned char* sRaw = sB + (size_t)(a.b_resident ? a.kchunks : S) * b_stage_bytes;   // q4 only (1024-byte aligned: every stage is)
    unsigned char* p = sRaw + (Q4 ? (size_t)kRawStages * kRawStageBytes : 0);
    uint64_t* full = (uint64_t*)p;
    uint64_t* empty = full + 8;
    uint64_t* tfull = empty + 8;
    uint64_t* tempty = tfull + 2;
    uint64_t* bfull = tempty + 2;
    uint64_t* rfull = bfull + 1;          // [kRawStages]
    uint64_t* rempty = rfull + kRawStages;  // [kRawStages]
    uint32_t* tmem_slot = (uint32_t*)(rempty + kRawStages);
    volatile uint32_t* abort_s = tmem_slot + 1;
    volatile uint32_t* done_s = tmem_slot + 2;       // epilogue warps that have finished
    volatile uint32_t* thr_ready_s = tmem_slot + 3;  // set by the refresher once every query has a bound
    QueryHeader* hdr_s = (QueryHeader*)(p + 256);
    uint32_t* thr_s = (uint32_t*)(hdr_s + kMmaCols);
    uint32_t* bmax_s = thr_s + kMmaCols;                 // [qn][4]: maxima of the current tile per epilogue warp
    uint32_t* pub_s = bmax_s + kMmaCols * 4;             // [qn][4][kBucketSlots]: last published values
    // [kMmaCols] pairs: .x pre-filter bound per query (+inf past qn), .y (hi_first only) norm of the query's low plane, a
    // shade high -- side by side so that the filter fetches both with one shared-memory read
    float2* zl_s = (float2*)(pub_s + kMmaCols * 4 * kBucketSlots);
    float* wq_s = (float*)(zl_s + kMmaCols);                          // [kMmaCols]: l2 only, weight of ||row||^2 in the bound

    const int64_t nrows = a.row_end - a.row_begin;
    const int n_tiles = (int)((nrows + kTileRows - 1) / kTileRows);
    const int grid = gridDim.x, cta = blockIdx.x;
    const int n_my = (cta < n_tiles) ? (n_tiles - cta + grid - 1) / grid : 0;
    const int n_obs = a.filtered ? min(a.observe_tiles, n_my) : 0;
    const int n_iters = n_my + n_obs;   // observed tiles are replayed at the end in append mode
    const int active_ctas = min(grid, n_tiles);

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], Q4 ? kConvWarps : 1);   // q4: one arrival per converter warp instead of a TMA transaction
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < kRawStages; ++s) {
            mbar_init(&rfull[s], 1);
            mbar_init(&rempty[s], kConvWarps);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], kEpiWarps);
        }
        mbar_init(bfull, 1);
        *abort_s = 0;
        *done_s = 0;
        *thr_ready_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int j = threadIdx.x; j < a.qn; j += blockDim.x) {
        hdr_s[j] = a.headers[a.q0 + j];
        zl_s[j].x = -INFINITY;   // no bound yet: every chunk takes the exact path
        {
            // l2: 1 / (2 s_lo) for q8 (the filter works on T = dot / (row scale * s_lo)), 1/2 for f16, a shade low
            const float s2 = I8 ? 2.0f * hdr_s[j].s_lo : 2.0f;
            wq_s[j] = (s2 > 0.0f) ? (1.0f / s2) * (1.0f - 1e-6f) : 0.0f;
        }
        thr_s[j] = 1;
        for (int w = 0; w < 4; ++w) {
            bmax_s[j * 4 + w] = 0;
            for (int s = 0; s < kBucketSlots; ++s) pub_s[(j * 4 + w) * kBucketSlots + s] = 0;
        }
    }
    for (int j = a.qn + threadIdx.x; j < kMmaCols; j += blockDim.x) {   // padding columns never pass
        zl_s[j].x = INFINITY;
        wq_s[j] = 0.0f;
    }
    if constexpr (I8) {
        for (int j = threadIdx.x; j < kMmaCols; j += blockDim.x) zl_s[j].y = (a.hi_first && j < a.qn) ? a.lo_norms[j] : 0.0f;
    }
    if (warp == 1) tmem_alloc(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto tile_of = [&](int it) { return cta + ((it < n_my) ? it : it - n_my) * grid; };

    if (n_my > 0) {
        if (warp == 0) {
            // ---------------- TMA producer ----------------
            if (lane == 0) {
                if (a.b_resident) {
                    // the query operand fits beside the candidate ring: one load, then only candidates stream
                    mbar_expect_tx(bfull, (uint32_t)a.kchunks * b_stage_bytes);
                    for (int kc = 0; kc < a.kchunks; ++kc) {
                        tma_load_2d(sB + (size_t)kc * b_stage_bytes, &map_b, kc * kChunkBytes, 0, bfull);
                        if (a.b_second_rows > 0)
                            tma_load_2d(sB + (size_t)kc * b_stage_bytes + (size_t)a.b_second_rows * kChunkBytes, &map_b2, kc * kChunkBytes, 0, bfull);
                    }
                }
                if constexpr (Q4) {
                    // raw tiles: one 128 x 128-byte box of nibbles per tile; the converter warps make the operand stages
                    for (int it = 0; it < n_iters && !*abort_s; ++it) {
                        const int row0 = (int)(a.row_begin + (int64_t)tile_of(it) * kTileRows);
                        const int rs = it % kRawStages;
                        const uint32_t ph = (uint32_t)(it / kRawStages) & 1u;
                        if (!mbar_wait(&rempty[rs], ph ^ 1u, abort_s)) break;
                        mbar_expect_tx(&rfull[rs], (uint32_t)kRawStageBytes);
                        tma_load_2d(sRaw + (size_t)rs * kRawStageBytes, &map_a, 0, row0, &rfull[rs]);
                    }
                }
                const uint32_t stage_tx = (uint32_t)(kTileRows * kChunkBytes) + (a.b_resident ? 0u : b_stage_bytes);
                // (stage and phase are counted, not divided out of g: these single-thread loops are latency chains)
                int s = 0;
                uint32_t ph = 0;
                const int kchunks = a.kchunks;
                const bool b_res = a.b_resident != 0;
                bool ok = true;
                for (int it = 0; !Q4 && ok && it < n_iters && !*abort_s; ++it) {
                    const int row0 = (int)(a.row_begin + (int64_t)tile_of(it) * kTileRows);
                    for (int kc = 0; kc < kchunks; ++kc) {
                        if (!mbar_try_wait(&empty[s], ph ^ 1u) && !mbar_wait(&empty[s], ph ^ 1u, abort_s)) { ok = false; break; }
                        mbar_expect_tx(&full[s], stage_tx);
                        tma_load_2d(sA + (size_t)s * kTileRows * kChunkBytes, &map_a, kc * kChunkBytes, row0, &full[s]);
                        if (!b_res) {
                            tma_load_2d(sB + (size_t)s * b_stage_bytes, &map_b, kc * kChunkBytes, 0, &full[s]);
                            if (a.b_second_rows > 0)
                                tma_load_2d(sB + (size_t)s * b_stage_bytes + (size_t)a.b_second_rows * kChunkBytes, &map_b2, kc * kChunkBytes, 0, &full[s]);
                        }
                        if (++s == S) { s = 0; ph ^= 1u; }
                    }
                }
            }
        } else if (warp == 1) {
            // ---------------- MMA issuer ----------------
            if (lane == 0) {
                const uint32_t idesc = I8 ? ((2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(a.ncols >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24))
                                          : ((1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(a.ncols >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24));
                // The issuing thread is alone on its latency chain: between two MMAs nothing hides the latency of its own
                // scalar instructions (measured: 67 cycles per back-to-back tcgen05.mma of up to 128 columns, 127 at 256, but
                // 170 - 240 when every instruction is preceded by divisions, descriptor construction and a called wait).  So
                // stage and phase are counters, descriptors are one base plus a multiple of the stage stride, and a wait that
                // is already over costs one try_wait.
                const uint64_t desc_a0 = smem_desc_sw128(smem_u32(sA));
                const uint64_t desc_b0 = smem_desc_sw128(smem_u32(sB));
                const uint32_t a_step = (uint32_t)(kTileRows * kChunkBytes) >> 4;   // descriptor address units (16 bytes) per stage
                const uint32_t b_step = b_stage_bytes >> 4;
                const int kchunks = a.kchunks;
                const bool b_res = a.b_resident != 0;
                const uint32_t ncols = (uint32_t)a.ncols;
                int s = 0;
                uint32_t ph = 0;
                bool b_ok = true;
                if (b_res) {
                    b_ok = mbar_wait(bfull, 0u, abort_s);
                    tc_fence_after();
                }
                for (int it = 0; b_ok && it < n_iters && !*abort_s; ++it) {
                    const int acc = it & 1;
                    const uint32_t tph = ((uint32_t)(it >> 1) & 1u) ^ 1u;
                    if (!mbar_try_wait(&tempty[acc], tph) && !mbar_wait(&tempty[acc], tph, abort_s)) break;
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + (uint32_t)acc * kMmaCols;
                    bool ok = true;
                    for (int kc = 0; kc < kchunks; ++kc) {
                        if (!mbar_try_wait(&full[s], ph) && !mbar_wait(&full[s], ph, abort_s)) { ok = false; break; }
                        tc_fence_after();
                        const uint64_t da = desc_a0 + (uint64_t)((uint32_t)s * a_step);
                        const uint64_t db = desc_b0 + (uint64_t)((uint32_t)(b_res ? kc : s) * b_step);
#pragma unroll
                        for (int ks = 0; ks < kChunkBytes / 32; ++ks) {   // +2 descriptor units = 32 bytes of K
                            if constexpr (Q4) {
                                // 32 bytes = 16 codes: two steps per block, each block into its own columns
                                const uint32_t blk = (uint32_t)(kc * 2 + (ks >> 1));
                                tc_mma<I8>(d_tmem + blk * ncols, da + (uint64_t)(ks * 2), db + (uint64_t)(ks * 2), idesc, (ks & 1) ? 1u : 0u);
                            } else {
                                tc_mma<I8>(d_tmem, da + (uint64_t)(ks * 2), db + (uint64_t)(ks * 2), idesc, (ks > 0) ? 1u : (kc > 0 ? 1u : 0u));
                            }
                        }
                        tc_commit(&empty[s]);   // frees the stage when these MMAs have read it
                        if (++s == S) { s = 0; ph ^= 1u; }
                    }
                    if (!ok) break;
                    tc_commit(&tfull[acc]);     // accumulator complete
                }
            }
        } else if (warp < 2 + kEpiWarps) {
            // ---------------- epilogue ----------------
            // The epilogue warps never synchronise with each other: each reads one quadrant of tensor memory for
            // its share of the query chunks, owns the bucket maxima of (quadrant, those queries), and arrives on the
            // accumulator's "empty" barrier by itself.
            const int quad = warp & 3;              // tensor-memory lanes 32*quad .. 32*quad+31
            const int ew = quad;                    // bucket owner index 0..3 (rows of a quadrant are one bucket)
            const int sub = (warp - 2) >> 2;        // this warp takes the 16-query chunks sub, sub + kEpiSubs, ...
            const float sign = (a.order == MANTA_B200_ORDER_SMALLEST) ? -1.0f : 1.0f;
            const bool want_scale = I8 && METRIC != MANTA_B200_METRIC_COSINE;
            // High planes first (q8, a.hi_first).  With T = 254 * I_hi + I_lo, the low plane can move T by at most ||lo|| *
            // ||codes of the row|| (Cauchy-Schwarz; the row's sum of squared codes is its stored statistic).  The low planes
            // are not contracted at all (twice the queries per pass, half the MMAs): the pre-filter tests the upper bound of
            // T, and a (row, query) pair that passes gets its I_lo from lo_plane_dot_warp -- the same int32 the second
            // plane's MMA would have produced, so scores are unchanged.  While a warp only observes (no bound yet, nothing
            // appended) it scores every row with the low plane at its worst: lower bounds of the scores, hence valid
            // (slightly low) bucket maxima.  (Keeping both planes in the contraction and bounding the low one only in the
            // pre-filter, to halve its tensor-memory reads, measured 1 - 2 % slower than reading both: not built in.)
            const bool hf = I8 && a.hi_first;
            const bool want_stats = METRIC != MANTA_B200_METRIC_DOT || hf;
            // every (metric, order) has a pre-filter except "largest l2 distance", which takes the exact path throughout
            constexpr bool kL2 = METRIC == MANTA_B200_METRIC_L2_DISTANCE;
            const bool cheap = !(kL2 && a.order == MANTA_B200_ORDER_LARGEST);
            float nxt_sd = 0.0f;
            uint32_t nxt_stat = 0;
            uint4 nxt_sc = make_uint4(0u, 0u, 0u, 0u);
            auto load_row_consts = [&](int it2) {
                const int64_t r2 = a.row_begin + (int64_t)tile_of(it2) * kTileRows + quad * 32 + lane;
                nxt_sd = 0.0f;
                nxt_stat = 0;
                nxt_sc = make_uint4(0u, 0u, 0u, 0u);
                if (r2 < a.row_end) {
                    if (want_scale) nxt_sd = ((const float*)a.cv.scales)[r2];
                    if (want_stats) nxt_stat = ((const uint32_t*)a.cv.stats)[r2];
                    if constexpr (Q4) nxt_sc = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(a.cv.scales) + (size_t)r2 * kQ4Blocks));
                }
            };
            if (n_iters > 0) load_row_consts(0);
            for (int it = 0; it < n_iters; ++it) {
                const bool observe = it < n_obs;            // score and record maxima only
                const bool replay = it >= n_my;             // append only
                if (a.filtered && it == n_obs && n_obs > 0) {
                    // the first bounds must exist before anything is appended (bounded wait on the refresher)
                    for (uint32_t spin = 0; spin < 40000u && !*thr_ready_s && !*abort_s; ++spin) __nanosleep(100);
                }
                const int acc = it & 1;
                // Row constants (row scale, statistic, q4 block scales): the loads for the NEXT tile are issued now and
                // used one iteration later, so their latency (these rows are cold in L2) hides behind a whole tile.
                const int64_t row = a.row_begin + (int64_t)tile_of(it) * kTileRows + quad * 32 + lane;
                const bool rv = row < a.row_end;
                const float sd = nxt_sd;
                const uint32_t stat = nxt_stat;
                const uint4 sc = nxt_sc;
                if (it + 1 < n_iters) load_row_consts(it + 1);
                float bsc[kQ4Blocks];   // q4: the row's eight block scales
                if constexpr (Q4) {
                    const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
                    for (int b = 0; b < kQ4Blocks; ++b)
                        bsc[b] = __half2float(__ushort_as_half((unsigned short)((b & 1) ? (scw[b >> 1] >> 16) : (scw[b >> 1] & 0xffffu))));
                }
                float rinv = 0.0f;
                if (METRIC == MANTA_B200_METRIC_COSINE) rinv = I8 ? q8_row_inv_norm((int)stat) : float_row_inv_norm(__uint_as_float(stat));
                if (!mbar_wait(&tfull[acc], (uint32_t)(it >> 1) & 1u, abort_s)) break;
                tc_fence_after();
                const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)acc * kMmaCols;
                const int32_t my_id = (int32_t)(a.cv.row_base + row);
                // row factor of the pre-filter; NaN for rows past the end makes every comparison false
                float rowc = __int_as_float(0x7fc00000);
                if (rv) rowc = (METRIC == MANTA_B200_METRIC_COSINE) ? rinv : (I8 ? sd : 1.0f);
                // |T_f32 - T| and the 254 * s_lo != s_hi mismatch (and, high planes first, the rounding of 254 * row factor) are below 5e-7 * 254 * |I_hi|, |I_hi| <= 127^2 * cols
                const float srow = I8 ? rowc * (5e-7f * 254.0f * 16129.0f * (float)a.cv.cols) : 0.0f;
                // "smallest" orders compare -score; the smallest l2 distance asks for a LARGE dot product, see below
                const float rowcs = kL2 ? rowc : sign * rowc;
                const float rowcs254 = __fmul_rn(rowcs, 254.0f);
                // l2: ||row||^2 as the filter adds it to the per-query constant
                float dn2row = 0.0f;
                if constexpr (kL2) dn2row = I8 ? __fmul_rn(__fmul_rn(sd, sd), (float)(int)stat) : __uint_as_float(stat);
                // hi_first: what the low plane can add to T * rowcs for a query whose low plane has norm 1
                const float rnorm = (hf && rv) ? sqrtf((float)(int)stat) * 1.000002f : 0.0f;   // norm of the row's codes, a shade high
                const float rslack = rnorm * fabsf(rv ? rowc : 0.0f);
                const uint4* row_codes = reinterpret_cast<const uint4*>(a.cv.data + (size_t)(rv ? row : a.row_begin) * a.cv.row_bytes);
                // One finished score of this lane's row for query j: vote against the bound, keep the bucket maximum,
                // append the passing rows with one reservation per warp.
                auto offer = [&](int j, float g, uint32_t o) {
                    const uint32_t ballot = __ballot_sync(0xffffffffu, o >= thr_s[min(j, a.qn - 1)]);
                    if (ballot == 0) return;
                    const bool pass = (ballot >> lane) & 1u;
                    if (!replay) {
                        // only scores at or above the current bound can raise it, so the bucket maxima are
                        // maintained from the passing rows (all valid rows while no bound exists)
                        const uint32_t wmax = __reduce_max_sync(0xffffffffu, pass ? o : 0u);
                        if (lane == 0 && wmax > bmax_s[j * 4 + ew]) bmax_s[j * 4 + ew] = wmax;
                    }
                    if (observe) return;
                    uint32_t pos0 = 0;
                    if (lane == 0) pos0 = atomicAdd(a.ws.count + a.q0 + j, (uint32_t)__popc(ballot));
                    pos0 = __shfl_sync(0xffffffffu, pos0, 0);
                    if (pass) {
                        const uint32_t pos = pos0 + __popc(ballot & ((1u << lane) - 1u));
                        if (pos < a.ws.cap)
                            a.ws.pool[(size_t)(a.q0 + j) * a.ws.cap + pos] = make_key(g, my_id);
                        else
                            a.ws.flags[kFlagOverflow] = 1u;
                    }
                };
                // chunks of 16 queries for this lane's row
                for (int c0 = sub * 16; c0 < a.qn; c0 += 16 * kEpiSubs) {
                    uint32_t groups = 0xFu;   // four-query groups of the chunk that need the exact evaluation
                    uint32_t myhit = 0xFFFFu; // this lane's own row: queries of the chunk that passed the pre-filter
                    uint32_t vh[16], vl[16];
                    if (cheap) {
                        if constexpr (Q4) {
                            // dot = sum over the eight blocks of scale_b * (exact block sum), in block order; eight
                            // queries at a time, so that the eight block reads are in flight together behind one wait
#pragma unroll
                            for (int half = 0; half < 2; ++half) {
                                uint32_t pb[kQ4Blocks][8];
#pragma unroll
                                for (int b = 0; b < kQ4Blocks; ++b) tmem_ld8(t_row + (uint32_t)(b * a.ncols + c0 + 8 * half), pb[b]);
                                tmem_ld_wait();
#pragma unroll
                                for (int jj = 0; jj < 8; ++jj) {
                                    float dv = 0.0f;
#pragma unroll
                                    for (int b = 0; b < kQ4Blocks; ++b) dv = __fmaf_rn(bsc[b], __uint_as_float(pb[b][jj]), dv);
                                    vh[8 * half + jj] = __float_as_uint(dv);
                                    vl[8 * half + jj] = 0;
                                }
                            }
                        } else {
                            tmem_ld16(t_row + c0, vh);
                            if constexpr (I8) {
                                if (!hf) tmem_ld16(t_row + a.lo_off + c0, vl);
                            } else {
#pragma unroll
                                for (int jj = 0; jj < 16; ++jj) vl[jj] = 0;
                            }
                            tmem_ld_wait();
                        }
                    }
                    if (cheap) {
                        // Pre-filter without finishing the scores.  With s_hi = 254 * s_lo the unscaled dot product is
                        // s_lo * T, T = 254 * I_hi + I_lo, so score >= bound  <=>  T * rowc >= bound / (qinv * s_lo) =: z
                        // (kept per query by the refresher).  T is formed in f32; srow covers its rounding and the
                        // rounding of s_lo itself, z is lowered by a few ulps, so the test can only pass too often.
                        // Five arithmetic instructions per score; almost every chunk ends here.
                        uint32_t hit = 0;
                        if (I8 && hf) {
                            // high planes first: T's upper bound, 254 folded into the row factor (its rounding is inside srow)
#pragma unroll
                            for (int jj = 0; jj < 16; ++jj) {
                                const float2 zl = zl_s[c0 + jj];
                                float rhs = zl.x;
                                if constexpr (kL2) rhs = __fmaf_rn(dn2row, wq_s[c0 + jj], rhs);
                                hit |= (__fmaf_rn((float)(int)vh[jj], rowcs254, __fmaf_rn(zl.y, rslack, srow)) >= rhs) ? (1u << jj) : 0u;
                            }
                        } else {
#pragma unroll
                            for (int jj = 0; jj < 16; ++jj) {
                                float t;
                                if constexpr (I8)
                                    t = __fmaf_rn((float)(int)vh[jj], 254.0f, (float)(int)vl[jj]);
                                else
                                    t = __uint_as_float(vh[jj]);
                                // l2 (smallest): dist <= B  <=>  dot >= (||q||^2 - B^2 + ||row||^2) / 2, in the units of T
                                float rhs = zl_s[c0 + jj].x;
                                if constexpr (kL2) rhs = __fmaf_rn(dn2row, wq_s[c0 + jj], rhs);
                                hit |= (__fmaf_rn(t, rowcs, srow) >= rhs) ? (1u << jj) : 0u;
                            }
                        }
                        myhit = hit;
                        hit = __reduce_or_sync(0xffffffffu, hit);
                        if (hit == 0u) continue;
                        groups = ((hit & 0x000Fu) ? 1u : 0u) | ((hit & 0x00F0u) ? 2u : 0u) | ((hit & 0x0F00u) ? 4u : 0u) |
                                 ((hit & 0xF000u) ? 8u : 0u);
                    }
                    {
                        // The accumulators of a group that passed are re-read four queries at a time instead of keeping
                        // sixteen finished scores live: the epilogue stays under 104 registers, which is what lets four
                        // warps per quadrant fit, and it is also the faster form when passing chunks are frequent.
#pragma unroll 1
                        for (int gq = 0; gq < 4; ++gq) {
                            const int cg = c0 + 4 * gq;
                            if (cg >= a.qn) break;
                            if (!((groups >> gq) & 1u)) continue;
                            uint32_t h4[4], l4[4];
                            if constexpr (Q4) {
                                uint32_t pb[kQ4Blocks][4];
#pragma unroll
                                for (int b = 0; b < kQ4Blocks; ++b) tmem_ld4(t_row + (uint32_t)(b * a.ncols + cg), pb[b]);
                                tmem_ld_wait();
#pragma unroll
                                for (int jj = 0; jj < 4; ++jj) {
                                    float dv = 0.0f;
#pragma unroll
                                    for (int b = 0; b < kQ4Blocks; ++b) dv = __fmaf_rn(bsc[b], __uint_as_float(pb[b][jj]), dv);
                                    h4[jj] = __float_as_uint(dv);
                                    l4[jj] = 0;
                                }
                            } else {
                                tmem_ld4(t_row + cg, h4);
                                if constexpr (I8) {
                                    if (!hf) tmem_ld4(t_row + a.lo_off + cg, l4);
                                } else {
#pragma unroll
                                    for (int jj = 0; jj < 4; ++jj) l4[jj] = 0;
                                }
                                tmem_ld_wait();
                            }
                            uint32_t need = 0xFu;   // queries of the group this lane finishes for its row
                            if constexpr (I8) {
                                if (hf) {
                                    need = 0u;
#pragma unroll
                                    for (int jj = 0; jj < 4; ++jj) {
                                        l4[jj] = 0;
                                        if (cg + jj >= a.qn) continue;
                                        if (observe) {
                                            // no bound yet, nothing is appended: the score with the low plane at its worst
                                            // (finished by the same function, which is monotone in I_lo) is a valid lower
                                            // bound of the row's score and so of the bucket maximum
                                            const int worst = (int)ceilf(__fmul_rn(zl_s[cg + jj].y, rnorm)) + 1;
                                            l4[jj] = (uint32_t)((rowcs >= 0.0f) ? -worst : worst);
                                            need |= 1u << jj;
                                            continue;
                                        }
                                        const bool mine = rv && ((myhit >> (4 * gq + jj)) & 1u);
                                        // one pair at a time, the whole warp on each
                                        uint32_t pend = __ballot_sync(0xffffffffu, mine);
                                        const uint4* lo_q = reinterpret_cast<const uint4*>(a.plane_lo + (size_t)(cg + jj) * a.plane_stride);
                                        while (pend != 0u) {
                                            const int src = __ffs(pend) - 1;
                                            pend &= pend - 1u;
                                            const uint4* rsrc = reinterpret_cast<const uint4*>(__shfl_sync(0xffffffffu, (unsigned long long)row_codes, src));
                                            const int dot = lo_plane_dot_warp(rsrc, lo_q, a.cv.cols >> 4, lane);
                                            if (lane == src) l4[jj] = (uint32_t)dot;
                                        }
                                        if (mine) need |= 1u << jj;
                                    }
                                }
                            }
                            float g[4];
                            uint32_t o[4];
                            score_n<I8, METRIC, 4>(h4, l4, stat, rinv, sd, hdr_s, cg, a.qn, rv, sign, g, o);
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj)
                                if (cg + jj < a.qn) offer(cg + jj, g[jj], ((need >> jj) & 1u) ? o[jj] : 0u);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tempty[acc]);
                // ---- publish this warp's maxima of the tile (bucket slot it % kBucketSlots)
                // (every tile at first, while the bounds are still forming; every fourth tile afterwards -- the maxima
                // of the tiles in between stay accumulated in bmax_s and go out with the next publication)
                if (a.filtered && !replay && (it < 16 || (it & 3) == 3 || it + 1 == n_my)) {
                    const int slot = (it < 16 ? it : (it >> 2)) % kBucketSlots;
                    for (int j = lane; j < a.qn; j += 32) {
                        if (((j >> 4) % kEpiSubs) != sub) continue;   // another warp of the quadrant owns this query
                        const int i = j * 4 + ew;
                        const uint32_t v = bmax_s[i];
                        bmax_s[i] = 0;
                        if (v > pub_s[i * kBucketSlots + slot]) {
                            pub_s[i * kBucketSlots + slot] = v;
                            st_relaxed_u32(a.ws.bucket + (size_t)(a.q0 + j) * a.ws.nb + ((size_t)(cta * 4 + ew) * kBucketSlots + slot), v);
                        }
                    }
                    __syncwarp();
                    if (it + 1 == n_obs) {
                        // this warp's observed tiles are all published
                        __threadfence();
                        __syncwarp();
                        if (lane == 0) atomicAdd(a.ready, 1u);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) atomicAdd((uint32_t*)done_s, 1u);
        } else if (Q4 && warp >= 2 + kEpiWarps + 1) {
            // ---------------- q4 converter ----------------
            // Thread t of the four converter warps owns row t of the tile.  Per raw chunk (128 bytes of nibbles = 256
            // elements = 8 blocks) it reads its row from the swizzled raw stage and its eight block scales from global
            // memory, and writes four operand stages of 64 f16 each.
            const int t = (warp - (2 + kEpiWarps + 1)) * 32 + lane;
            const __half2 off2 = __floats2half2_rn(1032.0f, 1032.0f);
            int s = 0, rs = 0;
            uint32_t ph = 0, rph = 0;
            for (int it = 0; it < n_iters && !*abort_s; ++it) {
                if (!mbar_try_wait(&rfull[rs], rph) && !mbar_wait(&rfull[rs], rph, abort_s)) break;
                const unsigned char* raw = sRaw + (size_t)rs * kRawStageBytes + (size_t)t * kChunkBytes;
                bool ok = true;
                for (int kc = 0; kc < 4; ++kc) {
                    if (!mbar_try_wait(&empty[s], ph ^ 1u) && !mbar_wait(&empty[s], ph ^ 1u, abort_s)) { ok = false; break; }
                    unsigned char* dst = sA + (size_t)s * kTileRows * kChunkBytes + (size_t)t * kChunkBytes;
                    // 32 raw bytes = two 16-byte chunks (2kc, 2kc+1), each one block of 32 codes
#pragma unroll
                    for (int hb = 0; hb < 2; ++hb) {
                        const int rawc = 2 * kc + hb;
                        const uint4 w4 = *reinterpret_cast<const uint4*>(raw + ((rawc ^ (t & 7)) << 4));
                        const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                        for (int wi = 0; wi < 4; ++wi) {
                            // nibble n (two's complement) ^ 8 is n + 8; 0x6400 | u is the half 1024 + u: subtract 1032
                            const uint32_t x = w[wi] ^ 0x88888888u;
                            uint32_t o[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const uint32_t bits = ((x >> (4 * e)) & 0x000F000Fu) | 0x64006400u;
                                const __half2 code = __hsub2(*reinterpret_cast<const __half2*>(&bits), off2);
                                o[e] = *reinterpret_cast<const uint32_t*>(&code);
                            }
                            const int outc = 4 * hb + wi;   // 16-byte chunk of the 128-byte operand row
                            *reinterpret_cast<uint4*>(dst + ((outc ^ (t & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                        }
                    }
                    // make the generic-proxy stores visible to the tensor core's async proxy, then one arrival per warp
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&full[s]);
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(&rempty[rs]);
                if (++rs == kRawStages) { rs = 0; rph ^= 1u; }
            }
        } else if (a.filtered && warp == 2 + kEpiWarps) {
            // ---------------- threshold refresher ----------------
            // Waits until every epilogue warp of every active CTA has published its observed tiles, then keeps
            // recomputing, for one query per round, the k-th largest bucket maximum (top 20 bits; rounding a bound
            // down keeps it valid) and refreshing this CTA's copy of all bounds.
            uint32_t seen = 0;
            const uint32_t want = (uint32_t)active_ctas * (uint32_t)kEpiWarps;
            for (uint32_t spin = 0; spin < 100000u && seen < want && !*abort_s && *done_s < (uint32_t)kEpiWarps; ++spin) {
                seen = ld_relaxed_u32(a.ready);
                if (seen < want) __nanosleep(64);
            }
            const uint32_t nb = min(a.ws.nb, (uint32_t)kRefStage);
            for (uint32_t round = 0; *done_s < (uint32_t)kEpiWarps && !*abort_s; ++round) {
                const int j = (int)(((uint64_t)cta + (uint64_t)round * grid) % (uint64_t)a.qn);
                const uint32_t* b = a.ws.bucket + (size_t)(a.q0 + j) * a.ws.nb;
                // k-th largest bucket maximum of the query, top 20 bits.  The four slots of one (CTA, quadrant) are
                // adjacent, so one 16-byte load brings them; while 4k <= buckets their maximum is taken as ONE bucket
                // (a union of disjoint row sets is still disjoint from the others), which leaves 20 values per lane in
                // registers for the twenty counting passes.
                const uint32_t nb4 = nb >> 2;   // the bucket count is a multiple of four (sixteen per SM)
                const uint4* b4 = reinterpret_cast<const uint4*>(b);
                uint32_t t = 0;
                if ((uint32_t)a.k <= nb4) {
                    uint32_t m[kRefStage / 128];
#pragma unroll
                    for (int u0 = 0; u0 < kRefStage / 128; u0 += 5) {   // five independent loads in flight per lane
                        uint4 tmp[5];
#pragma unroll
                        for (int u = 0; u < 5; ++u) {
                            const uint32_t i = (uint32_t)(u0 + u) * 32u + lane;
                            tmp[u] = (i < nb4) ? __ldcg(b4 + i) : make_uint4(0u, 0u, 0u, 0u);
                        }
#pragma unroll
                        for (int u = 0; u < 5; ++u) m[u0 + u] = max(max(tmp[u].x, tmp[u].y), max(tmp[u].z, tmp[u].w));
                    }
                    for (int bit = 31; bit >= 12; --bit) {
                        const uint32_t cand = t | (1u << bit);
                        uint32_t c0 = 0, c1 = 0, c2 = 0, c3 = 0;
#pragma unroll
                        for (int u = 0; u < kRefStage / 128; u += 4) {
                            c0 += (m[u] >= cand) ? 1u : 0u;
                            c1 += (m[u + 1] >= cand) ? 1u : 0u;
                            c2 += (m[u + 2] >= cand) ? 1u : 0u;
                            c3 += (m[u + 3] >= cand) ? 1u : 0u;
                        }
                        const uint32_t cnt = __reduce_add_sync(0xffffffffu, (c0 + c1) + (c2 + c3));
                        if (cnt >= (uint32_t)a.k) t = cand;
                    }
                } else {
                    // k larger than a quarter of the buckets (rare: several hundred results per query): every bucket
                    // counts by itself, re-read from L2 in each pass
                    for (int bit = 31; bit >= 12; --bit) {
                        const uint32_t cand = t | (1u << bit);
                        uint32_t cnt = 0;
                        for (uint32_t i = lane; i < nb4; i += 32) {
                            const uint4 v = __ldcg(b4 + i);
                            cnt += (v.x >= cand ? 1u : 0u) + (v.y >= cand ? 1u : 0u) + (v.z >= cand ? 1u : 0u) + (v.w >= cand ? 1u : 0u);
                        }
                        cnt = __reduce_add_sync(0xffffffffu, cnt);
                        if (cnt >= (uint32_t)a.k) t = cand;
                    }
                }
                if (lane == 0 && t != 0) atomicMax(a.ws.thr + a.q0 + j, t);
                __syncwarp();
                bool allset = true;
                uint32_t tv[kMmaCols / 32];
#pragma unroll
                for (int u = 0; u < kMmaCols / 32; ++u) {   // all bounds of the group, loads in flight together
                    const int jj = u * 32 + lane;
                    tv[u] = (jj < a.qn) ? ld_relaxed_u32(a.ws.thr + a.q0 + jj) : 1u;
                }
#pragma unroll
                for (int u = 0; u < kMmaCols / 32; ++u) {
                    const int jj = u * 32 + lane;
                    if (jj >= a.qn) continue;
                    const uint32_t v = tv[u];
                    thr_s[jj] = max(v, 1u);
                    allset = allset && (v != 0u);
                    // pre-filter bound: bound / qinv for cosine, the bound itself for dot, lowered by a few ulps; for
                    // q8 divided by s_lo (the filter compares the integer combination T, see the epilogue)
                    float c = -INFINITY;
                    if (v > 1u) {
                        const float tf = float_from_ord(v);   // bound on the goodness (score, or -score for "smallest")
                        if constexpr (METRIC == MANTA_B200_METRIC_L2_DISTANCE) {
                            // smallest distance: dist <= B = -tf.  z = (||q||^2 - B^2) / (2 s_lo) (q8) or / 2 (f16), with
                            // B^2 raised and z lowered by a few ulps; the row's ||d||^2 is added in the epilogue.
                            const float bnd = fmaxf(-tf, 0.0f);
                            const double b2 = (double)bnd * (double)bnd * (1.0 + 4e-6) + 1e-30;
                            const double q2 = I8 ? hdr_s[jj].qhat2 : hdr_s[jj].qn2d;
                            const float s2 = I8 ? 2.0f * hdr_s[jj].s_lo : 2.0f;
                            c = (s2 > 0.0f) ? (float)((q2 - b2) / (double)s2) : -INFINITY;
                            c = c - fabsf(c) * 1e-6f - 1e-30f;
                        } else {
                            const float qi = hdr_s[jj].qinv;
                            c = (METRIC == MANTA_B200_METRIC_COSINE) ? ((qi > 0.0f) ? tf / qi : -INFINITY) : tf;
                            c = c - fabsf(c) * 2e-6f - 1e-30f;
                            if constexpr (I8) {
                                const float sl = hdr_s[jj].s_lo;
                                c = (sl > 0.0f) ? c / sl : -INFINITY;
                                c = c - fabsf(c) * 1e-6f;
                            }
                        }
                    }
                    zl_s[jj].x = c;
                }
                allset = __all_sync(0xffffffffu, allset);
                if (allset && lane == 0) *thr_ready_s = 1u;
                if (round > (uint32_t)(4 * a.qn)) __nanosleep(1000);   // steady state: refresh at a relaxed pace
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *abort_s) a.ws.flags[kFlagTimeout] = 1u;
}

// Operand B: [ncols][kpad] bytes, K-major.  q8: rows 0..qn-1 are the high planes, lo_off.. the low planes.
// f16: row j is query j as half bits.  Everything else is zero.
__global__ void build_b_kernel(unsigned char* __restrict__ out, int ncols, int kpad, int layout, QueryPrep qp, int q0,
                               int qn, int lo_off, int cols, float* __restrict__ lo_norms) {
    if (lo_norms != nullptr && layout == MANTA_B200_LAYOUT_Q8_ROW_F32) {
        // norms of the low planes (high-planes-first passes), one warp per query, rounded up a shade
        const int lane = threadIdx.x & 31;
        for (int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); n < qn; n += gridDim.x * (blockDim.x >> 5)) {
            const int8_t* lo = qp.plane_lo + (size_t)(q0 + n) * qp.plane_stride;
            int acc = 0;
            for (int c = lane; c < cols; c += 32) acc += (int)lo[c] * (int)lo[c];
            acc = __reduce_add_sync(0xffffffffu, acc);
            if (lane == 0) lo_norms[n] = sqrtf((float)acc) * 1.000002f;
        }
    }
    const size_t total = (size_t)ncols * kpad;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int n = (int)(i / kpad), kb = (int)(i % kpad);
        unsigned char v = 0;
        if (layout == MANTA_B200_LAYOUT_Q8_ROW_F32) {
            if (kb < qp.plane_stride) {
                if (n < qn)
                    v = (unsigned char)qp.plane_hi[(size_t)(q0 + n) * qp.plane_stride + kb];
                else if (n >= lo_off && n < lo_off + qn)
                    v = (unsigned char)qp.plane_lo[(size_t)(q0 + n - lo_off) * qp.plane_stride + kb];
            }
        } else if (n < qn) {
            // q4 candidates reach the MMA as f16 with every group of eight elements in the converter's order
            int e = kb >> 1;
            if (layout == MANTA_B200_LAYOUT_Q4_B32_F16) {
                const int j = e & 7;
                e = (e & ~7) + ((j & 1) ? 4 + (j >> 1) : (j >> 1));
            }
            if (e < cols) {
                const __half h = __float2half_rn(qp.qf32[(size_t)(q0 + n) * cols + e]);
                v = (unsigned char)((__half_as_ushort(h) >> ((kb & 1) * 8)) & 0xFF);
            }
        }
        out[i] = v;
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

struct MmaState {
    EncodeTiledFn encode = nullptr;
    unsigned char* d_b = nullptr;     // operand B staging
    size_t d_b_bytes = 0;
    uint32_t* d_ready = nullptr;
    bool attr_set[18] = {};
};

static int mma_group_queries(const CandView& cv) {
    if (cv.layout == MANTA_B200_LAYOUT_Q4_B32_F16) return kMmaCols / kQ4Blocks;   // every block has its own columns: 8 x 32 = 256
    return cv.layout == MANTA_B200_LAYOUT_Q8_ROW_F32 ? kMmaCols / 2 : kMmaCols;
}

bool mma_supported(const CandView& cv, int nq, int metric) {
    // From two queries up the contraction beats the streaming kernel on f16 and q8 rows by 2 - 4x (four queries over 10 M x
    // 768: 4.22 ms streamed, 1.12 ms here; the streaming kernel pays its dp4a work once per query, an MMA of up to 128
    // columns costs the same 67 cycles whatever the column count).  One query stays on the streaming kernel (one launch
    // per step, no start-up).  q4 rows pass through the converter warps, which bound the pass at about 1.35 ms per 12.5 M
    // rows: worth it from eight queries.
    if (nq < (cv.layout == MANTA_B200_LAYOUT_Q4_B32_F16 ? 8 : 2)) return false;
    if (cv.rows < kTileRows) return false;
    if (((uintptr_t)cv.data & 15) || (cv.row_bytes & 15)) return false;
    if (cv.layout == MANTA_B200_LAYOUT_Q4_B32_F16) {
        // q4 rows reach the tensor cores as f16 codes, one accumulator range per 32-element block, and the block scales
        // are applied to the exact per-block sums: rows of 256 columns (eight blocks, one 128-byte chunk of nibbles)
        // whose scale rows are 16-byte aligned.
        (void)metric;
        return cv.cols == 32 * kQ4Blocks && ((uintptr_t)cv.scales & 15) == 0;
    }
    return cv.layout == MANTA_B200_LAYOUT_Q8_ROW_F32 || cv.layout == MANTA_B200_LAYOUT_F16;
}
int mma_bucket_count(int sm_count) { return sm_count * 4 * kBucketSlots; }
int mma_first_burst_rows(int) { return 0; }
int mma_pool_cap(int k) {
    int cap = 64 * k;
    return cap < 16384 ? 16384 : cap;
}

void mma_state_destroy(MmaState* s) {
    if (!s) return;
    if (s->d_b) cudaFree(s->d_b);
    if (s->d_ready) cudaFree(s->d_ready);
    delete s;
}

static cudaError_t make_map(MmaState* st, CUtensorMap* map, const void* base, uint64_t inner_bytes, uint64_t rows,
                            uint64_t stride_bytes, uint32_t box_rows, const char** why) {
    cuuint64_t dims[2] = {inner_bytes, rows};
    cuuint64_t strides[1] = {stride_bytes};
    cuuint32_t box[2] = {(cuuint32_t)kChunkBytes, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = st->encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        *why = "cuTensorMapEncodeTiled failed";
        return cudaErrorInvalidValue;
    }
    return cudaSuccess;
}

template <bool I8, int METRIC, int SUBS, bool Q4>
static cudaError_t launch_scan_subs(MmaState* st, int slot, int grid, size_t smem, cudaStream_t stream, const CUtensorMap& map_a,
                                    const CUtensorMap& map_b, const CUtensorMap& map_b2, const KernelArgs& ka, const char** why) {
    const int idx = slot * 2 + (SUBS == 4 ? 1 : 0);
    if (!st->attr_set[idx]) {
        cudaError_t e = cudaFuncSetAttribute(mma_scan_kernel<I8, METRIC, SUBS, Q4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit);
        if (e != cudaSuccess) { *why = "cudaFuncSetAttribute"; return e; }
        st->attr_set[idx] = true;
    }
    mma_scan_kernel<I8, METRIC, SUBS, Q4><<<grid, mma_threads(SUBS, Q4), smem, stream>>>(map_a, map_b, map_b2, ka);
    note_scan_launch("mma_scan_kernel", grid, mma_threads(SUBS, Q4), smem);
    return cudaSuccess;
}

template <bool I8, int METRIC, bool Q4 = false>
static cudaError_t launch_scan_one(MmaState* st, int slot, int grid, size_t smem, cudaStream_t stream, const CUtensorMap& map_a,
                                   const CUtensorMap& map_b, const CUtensorMap& map_b2, const KernelArgs& ka, const char** why) {
    if (ka.epi_subs == 4) return launch_scan_subs<I8, METRIC, 4, Q4>(st, slot, grid, smem, stream, map_a, map_b, map_b2, ka, why);
    return launch_scan_subs<I8, METRIC, 2, Q4>(st, slot, grid, smem, stream, map_a, map_b, map_b2, ka, why);
}

// One instantiation per (layout, metric): the epilogue of each is straight-line code for its own metric.
static cudaError_t launch_scan_variant(MmaState* st, int layout, int metric, int grid, size_t smem, cudaStream_t stream,
                                       const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_b2, const KernelArgs& ka,
                                       const char** why) {
    if (layout == MANTA_B200_LAYOUT_Q4_B32_F16) {
        switch (metric) {
            case MANTA_B200_METRIC_DOT: return launch_scan_one<false, MANTA_B200_METRIC_DOT, true>(st, 6, grid, smem, stream, map_a, map_b, map_b2, ka, why);
            case MANTA_B200_METRIC_COSINE: return launch_scan_one<false, MANTA_B200_METRIC_COSINE, true>(st, 7, grid, smem, stream, map_a, map_b, map_b2, ka, why);
            default: return launch_scan_one<false, MANTA_B200_METRIC_L2_DISTANCE, true>(st, 8, grid, smem, stream, map_a, map_b, map_b2, ka, why);
        }
    }
    const int slot = (layout == MANTA_B200_LAYOUT_Q8_ROW_F32 ? 0 : 3) + metric;
    switch (slot) {
        case 0: return launch_scan_one<true, MANTA_B200_METRIC_DOT>(st, slot, grid, smem, stream, map_a, map_b, map_b2, ka, why);
        case 1: return launch_scan_one<true, MANTA_B200_METRIC_COSINE>(st, slot, grid, smem, stream, map_a, map_b, map_b2, ka, why);
        case 2: return launch_scan_one<true, MANTA_B200_METRIC_L2_DISTANCE>(st, slot, grid, smem, stream, map_a, map_b, map_b2, ka, why);
        case 3: return launch_scan_one<false, MANTA_B200_METRIC_DOT>(st, slot, grid, smem, stream, map_a, map_b, map_b2, ka, why);
        case 4: return launch_scan_one<false, MANTA_B200_METRIC_COSINE>(st, slot, grid, smem, stream, map_a, map_b, map_b2, ka, why);
        default: return launch_scan_one<false, MANTA_B200_METRIC_L2_DISTANCE>(st, slot, grid, smem, stream, map_a, map_b, map_b2, ka, why);
    }
}

cudaError_t launch_mma_topk(cudaStream_t stream, int sm_count, MmaState** state, const MmaArgs& a, int* launches, const char** why) {
    *launches = 0;
    *why = nullptr;
    if (!*state) {
        MmaState* s = new MmaState();
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess || !fn || qres != cudaDriverEntryPointSuccess) {
            delete s;
            *why = "cuTensorMapEncodeTiled is not available";
            return e != cudaSuccess ? e : cudaErrorNotSupported;
        }
        s->encode = (EncodeTiledFn)fn;
        e = cudaMalloc(&s->d_ready, 256);
        if (e != cudaSuccess) {
            delete s;
            *why = "cudaMalloc(ready)";
            return e;
        }
        *state = s;
    }
    MmaState* st = *state;
    const CandView& cv = a.cv;
    const bool i8 = cv.layout == MANTA_B200_LAYOUT_Q8_ROW_F32;
    const bool q4 = cv.layout == MANTA_B200_LAYOUT_Q4_B32_F16;
    // q4: a 128-byte chunk of nibbles (256 codes) becomes four 128-byte K chunks of f16
    const int raw_chunks = (cv.row_bytes + kChunkBytes - 1) / kChunkBytes;
    const int kchunks = q4 ? 4 * raw_chunks : raw_chunks;
    const int kpad = kchunks * kChunkBytes;
    const size_t b_bytes = (size_t)kMmaCols * kpad + kMmaCols * sizeof(float);   // operand B, then the low-plane norms
    if (st->d_b_bytes < b_bytes) {
        cudaError_t e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) return e;
        if (st->d_b) cudaFree(st->d_b);
        st->d_b = nullptr;
        st->d_b_bytes = 0;
        e = cudaMalloc(&st->d_b, b_bytes);
        if (e != cudaSuccess) {
            *why = "cudaMalloc(operand B)";
            return e;
        }
        st->d_b_bytes = b_bytes;
    }
    const int64_t nrows = a.row_end - a.row_begin;
    const int n_tiles = (int)((nrows + kTileRows - 1) / kTileRows);
    const int grid = sm_count < n_tiles ? sm_count : n_tiles;
    const int filtered = (nrows > (int64_t)a.ws.cap) ? 1 : 0;
    // q8: a filtered pass with a pre-filter contracts the high planes only (twice the queries per pass, half the MMAs
    // and tensor-memory reads); everything else carries both planes
    // It pays when pairs that pass the filter are rare next to the rows streamed: a pass appends on the order of
    // k * log(rows / k) keys per query, each of which now costs a round trip to L2 for the low plane's dot product.  Measured
    // on 768-byte cosine rows: 10 M rows, k = 10 wins from 64 queries up (1.6x at 256) and loses 2 - 3 % up to 32, where the
    // second plane's columns cost the tensor core nothing (an MMA of up to 128 columns takes the same 67 cycles); k = 100,
    // or 2 M rows, or C5's k = 50 on 5 M rows lose 3 - 15 %.  The more the second plane costs, the denser the appends may
    // be: up to 64 queries it costs nothing (threshold 30,000 rows per append), up to 128 it doubles the MMA time (8,000:
    // 128 queries, k = 50 over 10 M rows 2.11 -> 1.76 ms), beyond that it costs a second pass (3,000: 256 queries, k = 100
    // 4.42 -> 3.09 ms).
    const double rows_per_append = (double)nrows / ((double)a.k * log2((double)nrows / (double)a.k + 2.0));
    const int hi_first = (a.nq > 32 && i8 && filtered && !(a.metric == MANTA_B200_METRIC_L2_DISTANCE && a.order == MANTA_B200_ORDER_LARGEST) &&
                          rows_per_append >= (a.nq > kMmaCols / 2 ? 3000.0 : a.nq > kMmaCols / 4 ? 8000.0 : 30000.0))
                             ? 1 : 0;
    const int group = hi_first ? kMmaCols : mma_group_queries(cv);
    int observe = (a.k + grid * 4 - 1) / (grid * 4);
    if (filtered && observe > kBucketSlots) {
        *why = "k exceeds the bucket capacity of the tensor-core pass for this grid";
        return cudaErrorNotSupported;
    }

    CUtensorMap map_a;
    cudaError_t e = make_map(st, &map_a, cv.data, (uint64_t)cv.row_bytes, (uint64_t)cv.rows, (uint64_t)cv.row_bytes, kTileRows, why);
    if (e != cudaSuccess) return e;

    for (int q0 = 0; q0 < a.nq; q0 += group) {
        const int qn = (a.nq - q0 < group) ? a.nq - q0 : group;
        const int qpad = (qn + 15) / 16 * 16;
        const int ncols = (i8 && !hi_first) ? 2 * qpad : qpad;
        const int lo_off = hi_first ? ncols : qpad;   // hi_first: no row of operand B is a low plane
        // Operand B.  f16 and q8 queries are already K-major rows in memory (the queries as they came; the int8 planes of the
        // query preparation): the tensor maps read them where they lie, rows past the group and bytes past the row come
        // back as zeros, and two planes are two boxes per chunk.  q4 rows (permuted f16 operand) and rows the TMA cannot
        // address (pitch or base not a multiple of 16 bytes) go through build_b_kernel as before.
        const float* d_lo_norms = a.qp.lo_norm ? a.qp.lo_norm + q0 : nullptr;
        CUtensorMap map_b, map_b2;
        int b_second_rows = 0;
        const size_t f16_pitch = (size_t)cv.cols * 2;
        const bool direct = !q4 && (i8 ? (a.qp.plane_hi != nullptr && a.qp.lo_norm != nullptr)
                                       : (a.qp.queries_f16 != nullptr && (f16_pitch & 15) == 0 && ((uintptr_t)a.qp.queries_f16 & 15) == 0));
        if (direct) {
            if (i8) {
                const size_t ps = (size_t)a.qp.plane_stride;
                e = make_map(st, &map_b, a.qp.plane_hi + (size_t)q0 * ps, ps, (uint64_t)qn, ps, (uint32_t)(hi_first ? ncols : qpad), why);
                if (e != cudaSuccess) return e;
                if (!hi_first) {
                    e = make_map(st, &map_b2, a.qp.plane_lo + (size_t)q0 * ps, ps, (uint64_t)qn, ps, (uint32_t)qpad, why);
                    if (e != cudaSuccess) return e;
                    b_second_rows = qpad;
                } else {
                    map_b2 = map_b;
                }
            } else {
                e = make_map(st, &map_b, (const unsigned char*)a.qp.queries_f16 + (size_t)q0 * f16_pitch, f16_pitch, (uint64_t)qn, f16_pitch,
                             (uint32_t)ncols, why);
                if (e != cudaSuccess) return e;
                map_b2 = map_b;
            }
        } else {
            float* built_norms = reinterpret_cast<float*>(st->d_b + (size_t)kMmaCols * kpad);
            build_b_kernel<<<128, 256, 0, stream>>>(st->d_b, ncols, kpad, cv.layout, a.qp, q0, qn, lo_off, cv.cols, hi_first ? built_norms : nullptr);
            count_launch();
            ++*launches;
            e = cudaGetLastError();
            if (e != cudaSuccess) { *why = "operand B build launch"; return e; }
            if (hi_first) d_lo_norms = built_norms;
            e = make_map(st, &map_b, st->d_b, (uint64_t)kpad, (uint64_t)ncols, (uint64_t)kpad, (uint32_t)ncols, why);
            if (e != cudaSuccess) return e;
            map_b2 = map_b;
        }
        e = cudaMemsetAsync(st->d_ready, 0, 4, stream);
        if (e != cudaSuccess) { *why = "cudaMemsetAsync(ready)"; return e; }

        const size_t a_stage = (size_t)kTileRows * kChunkBytes, b_stage = (size_t)ncols * kChunkBytes;
        const size_t fixed = 1024 /*alignment slack*/ + 256 /*barriers*/ + sizeof(QueryHeader) * kMmaCols + 4 * kMmaCols +
                             16 * kMmaCols + 16 * kMmaCols * kBucketSlots + 12 * kMmaCols;
        const size_t raw_ring = q4 ? (size_t)kRawStages * kRawStageBytes : 0;
        const size_t budget = kSmemLimit - fixed - raw_ring;
        // Operand B stays resident when it leaves room for at least four candidate stages: the ring then carries
        // only candidate bytes instead of re-reading the queries from L2 for every tile.
        const int b_resident = (b_stage * kchunks + 4 * a_stage <= budget) ? 1 : 0;
        int stages = b_resident ? (int)((budget - b_stage * kchunks) / a_stage) : (int)(budget / (a_stage + b_stage));
        if (stages > 8) stages = 8;
        if (stages < 2) { *why = "not enough shared memory for two pipeline stages"; return cudaErrorInvalidValue; }
        if (q4 && !b_resident) { *why = "q4 rows this wide do not leave room for the resident query operand"; return cudaErrorNotSupported; }
        const size_t smem = fixed + raw_ring + (b_resident ? b_stage * kchunks + stages * a_stage : stages * (a_stage + b_stage));

        KernelArgs ka;
        ka.cv = cv;
        ka.headers = a.qp.headers;
        ka.ws = a.ws;
        ka.ready = st->d_ready;
        ka.q0 = q0;
        ka.qn = qn;
        ka.ncols = ncols;
        ka.lo_off = lo_off;
        ka.kchunks = kchunks;
        ka.stages = stages;
        ka.b_resident = b_resident;
        ka.b_second_rows = b_second_rows;
        // Four epilogue warps per quadrant pay off when a tile carries many 16-query chunks and few K chunks, and for f16
        // rows from 48 queries up (measured: C2 0.173 -> 0.165 ms, 256 queries 0.36 -> 0.29 ms); the q8 instantiations with
        // four are short of registers (96 per thread) and measured slower at 768-byte rows.
        ka.epi_subs = ((qn >= 96 && kchunks <= 4) || (!i8 && !q4 && qn >= 48)) ? 4 : 2;
        ka.metric = a.metric;
        ka.order = a.order;
        ka.k = a.k;
        ka.filtered = filtered;
        ka.observe_tiles = observe;
        ka.row_begin = a.row_begin;
        ka.row_end = a.row_end;
        ka.raw_chunks = raw_chunks;
        ka.hi_first = hi_first;
        ka.plane_lo = a.qp.plane_lo ? a.qp.plane_lo + (size_t)q0 * a.qp.plane_stride : nullptr;
        ka.plane_stride = a.qp.plane_stride;
        ka.lo_norms = d_lo_norms;
        e = launch_scan_variant(st, cv.layout, a.metric, grid, smem, stream, map_a, map_b, map_b2, ka, why);
        if (e != cudaSuccess) return e;
        count_launch();
        ++*launches;
        e = cudaGetLastError();
        if (e != cudaSuccess) { *why = "tensor-core scan launch"; return e; }
    }
    return cudaSuccess;
}

}  // namespace mb200
