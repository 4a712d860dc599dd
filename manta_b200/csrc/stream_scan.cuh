// Streaming scoring kernel: 1, 2 or 4 queries against packed candidate rows, every stored byte read once.
//
// Data movement.  A warp works on "tiles" of R consecutive rows (R a power of two, 1..32).  Short passes deal the tiles
// round robin; long ones give every warp runs of eight consecutive tiles, and a fused single-query pass over f16 or q8
// rows hands out its last quarter on demand from a device counter (see the kernel).
// The tile's bytes are contiguous in HBM; the 32 lanes copy them 16 bytes at a time, lane after lane, with
// asynchronous copies (cp.async.cg, no registers held in flight) into the warp's own ring in shared memory (two
// stages with 16 warps per block, three with 8), so every global access is a fully coalesced 512-byte warp request.
// The copy lays rows out with a padded stride chosen so that the reads below are free of bank conflicts.  The next
// tile(s) of a warp are in flight while one is consumed: 16 tiles per SM at any time.  The small per-row values (row
// scale, row statistic, q4 block scales) travel through the same ring.
//
// Arithmetic.  A row is consumed by LPR = 32/R adjacent lanes, each taking every LPR-th 16-byte chunk of the row
// from shared memory; the query (for q8/q4 two int8 planes q ~= s_hi*hi + s_lo*lo, for f16 candidates f32 values)
// is prepared by the block itself at start-up and read from shared memory as a broadcast.  q8/q4 accumulate with
// dp4a into int32 (exact, order-free), f16 with fma.  log2(LPR) shuffle steps finish a row, one lane per row runs
// the score epilogue.  Warps never synchronise with each other inside the loop.
//
// Top-k.  A row's score enters the query's pool when it is not below the query's threshold.  The threshold is the
// k-th largest of the per-warp running maxima ("buckets": disjoint row sets, so k bucket maxima >= t prove that k
// rows score >= t); it can only be too low, never too high, so the pool always contains the true top k.  Until a
// first threshold exists a warp only observes (scores, bucket maxima; with one query per launch it also keeps the
// keys of its first four tiles in registers); once it exists the held keys go through the filter, or, if more tiles
// were observed than are held, the warp re-reads them (still in L2) and appends what passes.  Nothing waits and the
// pool never sees an unfiltered burst.
// The last block to finish selects the exact top k of the launch's queries (select.cuh), stores them (sharded: also
// into every rank's exchange inbox) and leaves the workspace zeroed for the next pass: a fused step is one launch.
#pragma once

#include <type_traits>

#include "select.cuh"

namespace mb200 {


__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- query preparation inside the scan ------------------------------------------------------------------------
// The whole block prepares the launch's queries into shared memory: header, and either the two int8 planes in the
// order the consumer reads them (q8: element order; q4: per 32-element block, per 8-element group the even elements
// then the odd ones, matching the nibble unpack) or the f32 values (f16 candidates), zero padded to whole chunks.
//   1. all threads: max |x| of every query (any order: a maximum) -> the plane scales s_hi = max/127, s_lo = s_hi/254;
//   2. all threads: the planes, element by element (each element is independent of the others);
//   3. warp q: the sums of query q that must come out bit for bit on every path: ||q||^2 in f64 (lane l adds
//      elements l, l+32, ... in order, then the 32 partial sums meet in an xor butterfly 16, 8, 4, 2, 1) and, for
//      packed candidates, the squared norm of the query the planes represent, summed the same way.
// The stand-alone preparation kernel (prep.cu) and the CPU model of the packed path use the same arithmetic and order.
__device__ __forceinline__ void quantise_query_element(float v, float sh, float sl, bool zero, float* h, float* l) {
    *h = 0.0f;
    *l = 0.0f;
    if (zero) return;
    float hh = roundf(__fdiv_rn(v, sh));
    hh = fminf(fmaxf(hh, -127.0f), 127.0f);
    const float rem = __fmaf_rn(-hh, sh, v);
    float ll = 0.0f;
    if (sl != 0.0f) {
        ll = roundf(__fdiv_rn(rem, sl));
        ll = fminf(fmaxf(ll, -127.0f), 127.0f);
    }
    *h = hh;
    *l = ll;
}

// Storage position inside a plane of query element e (the inverse of the order described above).
template <int LAYOUT>
__device__ __forceinline__ int plane_index_of_element(int e) {
    if constexpr (LAYOUT == MANTA_B200_LAYOUT_Q4_B32_F16) {
        const int blk = e >> 5, j = e & 31, grp = j >> 3, pos = j & 7;
        return blk * 32 + (2 * grp + (pos & 1)) * 4 + (pos >> 1);
    }
    return e;
}

template <int LAYOUT, int QT>
__device__ __forceinline__ void prepare_queries_block(const __half* __restrict__ queries, int q0, int qt, int cols, int chunks, int q_bytes,
                                                      QueryHeader* hdr_s, unsigned char* q_s, float* s_red /* [QT][32] scratch */,
                                                      float* lo_norm_s /* [QT] out */) {
    constexpr bool kF16 = LAYOUT == MANTA_B200_LAYOUT_F16;
    constexpr bool kQ4 = LAYOUT == MANTA_B200_LAYOUT_Q4_B32_F16;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, W = blockDim.x >> 5;
    // 1. max |x| per query
#pragma unroll
    for (int q = 0; q < QT; ++q) {
        const __half* src = queries + (size_t)(q0 + ((q < qt) ? q : 0)) * cols;   // unused slots repeat query 0 of the launch
        float amax = 0.0f;
        for (int c = threadIdx.x; c < cols; c += blockDim.x) amax = fmaxf(amax, fabsf(__half2float(src[c])));
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        if (lane == 0) s_red[q * 32 + warp] = amax;
    }
    __syncthreads();
    float s_hi[QT], s_lo[QT];
    bool zero[QT];
#pragma unroll
    for (int q = 0; q < QT; ++q) {
        float amax = 0.0f;
        for (int w = 0; w < W; ++w) amax = fmaxf(amax, s_red[q * 32 + w]);
        zero[q] = !(amax > 0.0f);
        s_hi[q] = zero[q] ? 0.0f : __fdiv_rn(amax, 127.0f);
        s_lo[q] = zero[q] ? 0.0f : __fdiv_rn(s_hi[q], 254.0f);
    }
    // 2. planes / f32 values
#pragma unroll
    for (int q = 0; q < QT; ++q) {
        const __half* src = queries + (size_t)(q0 + ((q < qt) ? q : 0)) * cols;
        unsigned char* dst = q_s + (size_t)q * q_bytes;
        if constexpr (kF16) {
            float* qf = reinterpret_cast<float*>(dst);
            for (int c = threadIdx.x; c < chunks * 8; c += blockDim.x) qf[c] = (c < cols) ? __half2float(src[c]) : 0.0f;
        } else {
            const int plane = kQ4 ? chunks * 32 : chunks * 16;   // bytes of one plane
            int8_t* hi = reinterpret_cast<int8_t*>(dst);
            int8_t* lo = hi + plane;
            for (int c = threadIdx.x; c < plane; c += blockDim.x) {
                int e = c;   // c indexes the plane in storage order; e is the query element stored there
                if constexpr (kQ4) {
                    const int blk = c >> 5, w = (c >> 2) & 7, b = c & 3;
                    e = blk * 32 + (w >> 1) * 8 + 2 * b + (w & 1);
                }
                float hh = 0.0f, ll = 0.0f;
                if (e < cols) quantise_query_element(__half2float(src[e]), s_hi[q], s_lo[q], zero[q], &hh, &ll);
                hi[c] = (int8_t)hh;
                lo[c] = (int8_t)ll;
            }
        }
    }
    __syncthreads();
    // 3. the ordered sums, one warp per query
    for (int q = warp; q < QT; q += W) {
        const __half* src = queries + (size_t)(q0 + ((q < qt) ? q : 0)) * cols;
        double part = 0.0, p2 = 0.0, lo2 = 0.0;
        for (int c = lane; c < cols; c += 32) {
            const double v = (double)__half2float(src[c]);
            part = __dadd_rn(part, __dmul_rn(v, v));
        }
        if constexpr (!kF16) {
            const int plane = kQ4 ? chunks * 32 : chunks * 16;
            const int8_t* hi = reinterpret_cast<const int8_t*>(q_s + (size_t)q * q_bytes);
            const int8_t* lo = hi + plane;
            const double dh = (double)s_hi[q], dl = (double)s_lo[q];
            for (int c = lane; c < cols; c += 32) {
                const int idx = plane_index_of_element<LAYOUT>(c);
                const double vl = __dmul_rn((double)lo[idx], dl);
                const double v = __dadd_rn(__dmul_rn((double)hi[idx], dh), vl);
                p2 = __dadd_rn(p2, __dmul_rn(v, v));
                lo2 += vl * vl;
            }
        }
        for (int off = 16; off > 0; off >>= 1) {
            part = __dadd_rn(part, __shfl_xor_sync(0xffffffffu, part, off));
            p2 = __dadd_rn(p2, __shfl_xor_sync(0xffffffffu, p2, off));
            lo2 += __shfl_xor_sync(0xffffffffu, lo2, off);
        }
        if (lane == 0) {
            // norm of the low plane's part of the query, rounded up: |q_lo . d| <= lo_norm * ||d|| bounds what the low
            // plane can add to a dot product (used by the high-plane-first filter of the q4 scan)
            lo_norm_s[q] = (float)(sqrt(lo2) * 1.000001) + 1e-30f;
            QueryHeader h;
            h.qn = __double2float_rn(__dsqrt_rn(part));
            h.qinv = (h.qn > 0.0f) ? __fdiv_rn(1.0f, h.qn) : 0.0f;
            h.qn2d = part;
            h.qhat2 = kF16 ? part : p2;
            h.s_hi = s_hi[q];
            h.s_lo = s_lo[q];
            hdr_s[q] = h;
        }
    }
}

// LPR, CPL: lanes per row and 16-byte chunks per lane and row as compile-time constants (a row is exactly LPR * CPL
// chunks: the loops unroll and every shared-memory access is a base register plus an immediate), or LPR == 0 for the
// generic form that takes both from the launch geometry.
template <int LAYOUT, int QT, int LPR, int CPL>
__global__ void __launch_bounds__(scan_warps(QT) * 32, 1) stream_scan_kernel(const StreamArgs a) {
    constexpr bool kSpec = LPR > 0;
    constexpr bool kQ8 = LAYOUT == MANTA_B200_LAYOUT_Q8_ROW_F32;
    constexpr bool kQ4 = LAYOUT == MANTA_B200_LAYOUT_Q4_B32_F16;
    constexpr bool kF16 = LAYOUT == MANTA_B200_LAYOUT_F16;
    const int S = a.g.stages;

    extern __shared__ __align__(128) unsigned char smem[];
    QueryHeader* hdr_s = reinterpret_cast<QueryHeader*>(smem);                   // [QT], 256 bytes reserved
    unsigned char* q_s = smem + 256;                                             // [QT][q_bytes]
    uint32_t* s_stage = reinterpret_cast<uint32_t*>(q_s + (size_t)QT * a.g.q_bytes);   // [kScanRefreshWords]
    unsigned char* ring = reinterpret_cast<unsigned char*>(s_stage + kScanRefreshWords + 256);   // 256 histogram bins follow the staged maxima
    __shared__ int s_last;

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int W = blockDim.x >> 5;
    const CandView& cv = a.cv;
    const ScanGeometry& g = a.g;
    const int lpr = kSpec ? LPR : (1 << g.lpr_shift);
    const int R = kSpec ? 32 / (kSpec ? LPR : 1) : g.rows_per_tile;
    const int r_in = kSpec ? lane / (kSpec ? LPR : 1) : (lane >> g.lpr_shift);    // row of the tile this lane works on
    const int part = lane & (lpr - 1);       // which chunks of the row: part, part + lpr, ...
    const bool leader = part == 0;           // the lane that finishes the row
    const int C = kSpec ? LPR * CPL : cv.chunks;
    const int Cs = kSpec ? scan_padded_stride(LPR * CPL, kSpec ? LPR : 1) : g.cstride;
    unsigned char* my_ring = ring + (size_t)warp * S * g.stage_bytes;

    // tile numbers fit 32 bits: a candidate set has fewer than 2^31 rows
    const int n_tiles = (int)((a.row_end - a.row_begin + R - 1) / R);
    const int gw = (int)blockIdx.x * W + warp;
    const int nwarps = (int)gridDim.x * W;
    const bool topk = a.mode == kModeTopk;
    // How the tiles are dealt.  A long pass (kScanClaimMinTiles tiles per warp or more) gives every warp runs of kRun
    // consecutive tiles: run r of warp gw is tiles (r * nwarps + gw) * kRun ... + kRun - 1 (part A, `own_a` tiles per warp).
    // In a fused single-query top-k pass over f16 or q8 rows -- the passes bound by memory bandwidth, in which the SMs
    // advance unevenly -- part A ends after about three quarters of the tiles and the rest is claimed from a device
    // counter in runs of 8, 4, 2 and finally 1 tiles, so that the SMs the memory system serves more slowly end up with
    // fewer tiles and every warp finishes within a tile or two of the others.  (Runs, because one address takes well
    // under a billion atomic adds a second and the warps together finish more than a billion tiles a second.  The
    // passes bound by instruction issue, several queries or q4 rows, advance evenly and measured 3-4 % slower with
    // claimed tiles, whose runs scatter an SM's warps over the rows; they keep part A to the end.)  What part A
    // leaves of any other pass, and all of a short pass, goes round robin, one tile at a time (part B).  The tiles a warp
    // observes and reads again are always its own first ones.
    constexpr int kRun = 8;
    const int per_warp = n_tiles / nwarps;
    const bool long_pass = per_warp >= kScanClaimMinTiles;
    const bool claim_on = QT == 1 && !kQ4 && topk && a.fused_select && long_pass;
    const int own_a = !long_pass ? 0 : ((claim_on ? max(kScanClaimMinTiles - 4, per_warp - per_warp / 4) : per_warp) & ~(kRun - 1));
    const int a_end = own_a * nwarps;
    const int static_end = claim_on ? a_end : n_tiles;
    const int own_b = (gw < static_end - a_end) ? (static_end - a_end - gw + nwarps - 1) / nwarps : 0;
    const int my_tiles = own_a + own_b;
    const int n_claimable = n_tiles - static_end;
    uint32_t* claim_counter = a.done_blocks + 1;

    // ---- the asynchronous copy of one tile: lane l copies chunks l, l + 32, ... of the tile's contiguous bytes
    // chunk i of the tile lands at ((i / C) * Cs + i % C) * 16 = (i + (i / C) * (Cs - C)) * 16; the division is a
    // multiply-high by ceil(2^32 / C), exact for every chunk index a tile can have
    const uint32_t c_magic = (uint32_t)((0x100000000ull + (uint32_t)C - 1u) / (uint32_t)C);
    const int c_pad = Cs - C;
    auto issue = [&](int tile, int stage) {
        if (tile >= 0) {
            const int64_t first = a.row_begin + (int64_t)tile * R;
            const int rows_here = (int)min((int64_t)R, a.row_end - first);
            const int n_chunks = rows_here * C;
            const unsigned char* src = cv.data + (size_t)first * cv.row_bytes;
            unsigned char* dst = my_ring + (size_t)stage * g.stage_bytes;
            if constexpr (kSpec) {
                // a full tile is exactly CPL copies per lane
#pragma unroll
                for (int j = 0; j < CPL; ++j) {
                    const int i = lane + 32 * j;
                    const int rr = i / (LPR * CPL);
                    if (i < n_chunks) cp_async16(dst + (size_t)(i + rr * c_pad) * 16, src + (size_t)i * 16);
                }
            } else {
#pragma unroll 4
                for (int i = lane; i < n_chunks; i += 32) {
                    const int rr = (C == 1) ? i : (int)__umulhi((uint32_t)i, c_magic);
                    cp_async16(dst + (size_t)(i + rr * c_pad) * 16, src + (size_t)i * 16);
                }
            }
            if constexpr (kQ4) {
                if (g.scale_unit != 0) {
                    const unsigned char* ssrc = reinterpret_cast<const unsigned char*>(cv.scales) + (size_t)first * C * 2;
                    const int n_units = rows_here * C * 2 / g.scale_unit;
                    if (g.scale_unit == 16) {
                        for (int i = lane; i < n_units; i += 32) cp_async16(dst + g.scale_off + i * 16, ssrc + (size_t)i * 16);
                    } else {
                        for (int i = lane; i < n_units; i += 32) cp_async4(dst + g.scale_off + i * 4, ssrc + (size_t)i * 4);
                    }
                }
            }
            if (lane < rows_here) {
                if (cv.stats != nullptr) cp_async4(dst + g.stat_off + lane * 4, reinterpret_cast<const uint32_t*>(cv.stats) + first + lane);
                if constexpr (kQ8) cp_async4(dst + g.rscale_off + lane * 4, reinterpret_cast<const float*>(cv.scales) + first + lane);
            }
        }
        cp_async_commit();
    };
    // Tile processed in iteration i.  A warp observes its first T tiles (T unknown while it observes); when the first
    // threshold arrives at the top of iteration T the F = S - 1 tiles whose copies were already issued (T .. T+F-1) are
    // consumed in append mode, then the T observed tiles are read again and appended, then the scan goes on.
    const int F = S - 1;
    int T = topk ? 0x3fffffff : 0;
    // Position i of the warp's schedule: the warp's own tile number (>= 0), kNoTile, or kClaim (the tile comes from the
    // shared counter).  Claims start once the warp's own tiles are used up, always after observation and replay.
    constexpr int kNoTile = -1, kClaim = -2;
    auto slot_of = [&](int i) -> int {
        if (i < T + F) return (i < my_tiles) ? i : kNoTile;
        if (i < 2 * T + F) return i - (T + F);
        return (i - T < my_tiles) ? i - T : (claim_on ? kClaim : kNoTile);
    };
    // A warp works through its run, and takes the next run an iteration before the copy that needs it is issued.  The
    // length it asks for follows from where the counter will be by then: its last answer plus one run of every warp.
    int claimed = 0, run_next = 0, run_end = 0, run_len = 0, counter_guess = 0;
    bool claim_ready = false, dry = false;
    auto take_run = [&]() {
        const int left = n_claimable - counter_guess;
        run_len = (left >= 16 * nwarps) ? 8 : (left >= 8 * nwarps) ? 4 : (left >= nwarps) ? 2 : 1;
        if (lane == 0) claimed = (int)atomicAdd(claim_counter, (uint32_t)run_len);
        claim_ready = true;
    };
    auto claim_ahead = [&](int i) {
        if (claim_on && !claim_ready && !dry && run_next >= run_end && slot_of(i) == kClaim) take_run();
    };
    auto tile_at = [&](int i) -> int {
        const int sl = slot_of(i);
        if (sl >= 0) return (sl < own_a) ? (((sl / kRun) * nwarps + gw) * kRun + (sl % kRun)) : (a_end + gw + (sl - own_a) * nwarps);
        if (sl == kNoTile || dry) return -1;
        if (run_next >= run_end) {
            if (!claim_ready) take_run();
            claim_ready = false;
            const int start = __shfl_sync(0xffffffffu, claimed, 0);
            if (start < 0 || start >= n_claimable) {
                dry = true;   // the counter only rises: every later claim is past the end too
                return -1;
            }
            run_next = start;
            run_end = min(start + run_len, n_claimable);
            counter_guess = (int)min((int64_t)n_claimable, (int64_t)start + (int64_t)run_len * (1 + nwarps));
        }
        return static_end + run_next++;
    };
    // tiles in flight, oldest first (the ring holds S <= 3 stages)
    int pend0 = -1, pend1 = -1, pend2 = -1;
    auto push_tile = [&](int t) {
        if (S == 2) pend1 = t;
        else pend2 = t;
    };

    // start the stream before anything else, then prepare the queries while the first tiles are on their way
    for (int p = 0; p < S - 1; ++p) {
        const int t = tile_at(p);
        issue(t, p);
        if (p == 0) pend0 = t;
        else pend1 = t;
    }
    float* lo_norm_s = reinterpret_cast<float*>(hdr_s + QT);   // behind the headers, inside their 256 bytes
    prepare_queries_block<LAYOUT, QT>(a.queries, a.q0, a.qt, cv.cols, C, g.q_bytes, hdr_s, q_s, reinterpret_cast<float*>(s_stage), lo_norm_s);
    __syncthreads();
    QueryHeader hdr[QT];
    float q4_sh[QT], q4_sl[QT], lo_norm[QT];
#pragma unroll
    for (int q = 0; q < QT; ++q) {
        hdr[q] = hdr_s[q];
        lo_norm[q] = lo_norm_s[q];
        q4_sh[q] = hdr[q].s_hi * 0.0625f;  // the nibble unpack yields 16*code
        q4_sl[q] = hdr[q].s_lo * 0.0625f;
    }

    const float sign = (a.order == MANTA_B200_ORDER_SMALLEST) ? -1.0f : 1.0f;
    // Nearest-neighbour l2 on packed rows finishes a score in f64 (square root included).  In top-k mode a row is
    // first tested in f32: dist <= B  <=>  dot >= (||q||^2 - B^2 + ||row||^2) / 2, with B the current bound and a few
    // ulps of slack; a tile in which no row passes skips the exact evaluation.  Rows that do not pass are below the
    // bound, so leaving them out of the bucket maxima keeps those maxima valid lower bounds.
    const bool l2_pref = !kF16 && topk && a.metric == MANTA_B200_METRIC_L2_DISTANCE && a.order == MANTA_B200_ORDER_SMALLEST;
    constexpr int kSlots = scan_bucket_slots(QT);
    uint32_t thr[QT], bmax[QT][kSlots], published[QT][kSlots];
    float l2_ch[QT];   // (||q||^2 - B^2) / 2 per query, lowered; -inf while no bound exists
#pragma unroll
    for (int q = 0; q < QT; ++q) {
        thr[q] = 0;
        l2_ch[q] = -INFINITY;
#pragma unroll
        for (int s = 0; s < kSlots; ++s) bmax[q][s] = published[q][s] = 0;
    }
    auto load_bounds = [&]() {
#pragma unroll
        for (int q = 0; q < QT; ++q) {
            thr[q] = ld_relaxed_u32(a.ws.thr + a.q0 + ((q < a.qt) ? q : 0));
            float ch = -INFINITY;
            if (l2_pref && thr[q] > 1u) {
                const float bnd = fmaxf(-float_from_ord(thr[q]), 0.0f);
                const double b2 = (double)bnd * (double)bnd * (1.0 + 4e-6) + 1e-30;
                ch = (float)((hdr[q].qhat2 - b2) * 0.5);
                ch = ch - fabsf(ch) * 1e-6f - 1e-30f;
            }
            l2_ch[q] = ch;
        }
    };
    // one reservation per call for all lanes that pass
    auto append = [&](int q, bool pass, uint64_t key) {
        const uint32_t ballot = __ballot_sync(0xffffffffu, pass);
        if (ballot == 0) return;
        uint32_t base = 0;
        if (lane == 0) base = atomicAdd(a.ws.count + a.q0 + q, (uint32_t)__popc(ballot));
        base = __shfl_sync(0xffffffffu, base, 0);
        if (pass) {
            const uint32_t pos = base + __popc(ballot & ((1u << lane) - 1u));
            if (pos < a.ws.cap)
                a.ws.pool[(size_t)(a.q0 + q) * a.ws.cap + pos] = key;
            else
                a.ws.flags[kFlagOverflow] = 1u;
        }
    };

    int stage = 0;                 // ring slot of the tile consumed in this iteration
    int next_stage = S - 1;        // ring slot the copies issued in this iteration go to
    // One query per launch: the keys of the first kHeld observed tiles are held back in registers (one per lane and
    // tile), so the usual case -- a first threshold after two or three tiles -- needs no second read at all.
    constexpr bool kHold = QT == 1;
    constexpr int kHeld = 4;
    uint64_t held_key[kHeld];
    bool held_ok[kHeld];
#pragma unroll
    for (int e = 0; e < kHeld; ++e) {
        held_key[e] = 0;
        held_ok[e] = false;
    }
    bool observing = topk;
    int total = topk ? 0x3fffffff : max(my_tiles, F);
    uint32_t fresh = 0;            // fresh (not re-read) tiles consumed so far: drives the refresh duty
    uint32_t overflow_seen = 0;
    for (int i = 0; i < total || (claim_on && !(dry && pend0 < 0 && pend1 < 0)); ++i) {
        if (topk) {
            // the bounds move fast only at the start: reread them every tile early on, every eighth tile later
            if (observing || i <= 16 || (i & 7) == 0) load_bounds();
            if (observing) {
                bool have = true;
#pragma unroll
                for (int q = 0; q < QT; ++q) have = have && thr[q] != 0u;
                if (have || i >= my_tiles) {
                    observing = false;
                    T = min(i, my_tiles);
                    if (kHold && T <= kHeld) {
                        // every observed tile's keys are still in registers: they go through the filter now and
                        // nothing has to be read again
#pragma unroll
                        for (int e = 0; e < kHeld; ++e)
                            if (e < T) append(0, held_ok[e] && (uint32_t)(held_key[e] >> 32) >= thr[0], held_key[e]);
                        T = 0;
                    }
                    total = max(2 * T + F, my_tiles + T);
                }
            }
            // a pool that overflowed makes the host redo the pass in chunks: stop streaming.  The flag is loaded in
            // one check and tested in the next, so its latency never stalls the stream.
            if ((i & 63) == 63) {
                if (overflow_seen != 0) break;
                overflow_seen = ld_relaxed_u32(a.ws.flags + kFlagOverflow);
            }
        }
        // the copies of this iteration's tile have landed once at most S - 2 younger groups are still pending
        if (S == 2) cp_async_wait<0>();
        else if (S == 3) cp_async_wait<1>();
        else cp_async_wait<2>();
        __syncwarp();             // ... for every lane, and every lane is done with the stage refilled next
        {
            const int t = tile_at(i + S - 1);
            issue(t, next_stage);
            push_tile(t);
        }
        claim_ahead(i + S);
        next_stage = stage;       // the stage consumed now is refilled in the next iteration
        stage = (stage + 1 == S) ? 0 : stage + 1;
        const int cur_stage = next_stage;
        const int tile = pend0;
        pend0 = pend1;
        pend1 = pend2;
        pend2 = -1;
        if (tile < 0) continue;
        const bool observe = i < T;
        const bool replay = i >= T + F && i < 2 * T + F;
        const unsigned char* st = my_ring + (size_t)cur_stage * g.stage_bytes;
        const int64_t first = a.row_begin + (int64_t)tile * R;
        const int64_t my_row = first + r_in;
        const bool rv = leader && my_row < a.row_end;

        // ---- accumulate this lane's chunks of its row
        bool skip_tile = false;   // q4 high-plane filter: no row of the tile can pass, nothing to finish
        int ih[QT], il[QT];
        float fa[QT], fb[QT];
#pragma unroll
        for (int q = 0; q < QT; ++q) {
            ih[q] = il[q] = 0;
            fa[q] = fb[q] = 0.0f;
        }
        const uint4* rowp = reinterpret_cast<const uint4*>(st) + (size_t)r_in * Cs + part;
        // body(j) consumes chunk part + j * lpr of the row; compile-time j in the specialised form
        auto for_each_chunk = [&](auto&& body) {
            if constexpr (kSpec) {
#pragma unroll
                for (int j = 0; j < CPL; ++j) body(j * LPR);
            } else {
#pragma unroll 4
                for (int c = 0; part + c < C; c += lpr) body(c);
            }
        };
        if constexpr (kQ8) {
            // two independent accumulator chains per plane (.x/.z and .y/.w words) keep the integer pipe busy
            int ih2[QT], il2[QT];
#pragma unroll
            for (int q = 0; q < QT; ++q) ih2[q] = il2[q] = 0;
            const uint4* qbase = reinterpret_cast<const uint4*>(q_s) + part;
            const int q_stride = g.q_bytes / 16;
            for_each_chunk([&](int c) {
                const uint4 d = rowp[c];
#pragma unroll
                for (int q = 0; q < QT; ++q) {
                    const uint4 qh = qbase[q * q_stride + c];
                    const uint4 ql = qbase[q * q_stride + C + c];
                    ih[q] = __dp4a((int)d.x, (int)qh.x, ih[q]);
                    ih2[q] = __dp4a((int)d.y, (int)qh.y, ih2[q]);
                    il[q] = __dp4a((int)d.x, (int)ql.x, il[q]);
                    il2[q] = __dp4a((int)d.y, (int)ql.y, il2[q]);
                    ih[q] = __dp4a((int)d.z, (int)qh.z, ih[q]);
                    ih2[q] = __dp4a((int)d.w, (int)qh.w, ih2[q]);
                    il[q] = __dp4a((int)d.z, (int)ql.z, il[q]);
                    il2[q] = __dp4a((int)d.w, (int)ql.w, il2[q]);
                }
            });
#pragma unroll
            for (int q = 0; q < QT; ++q) {
                ih[q] += ih2[q];
                il[q] += il2[q];
            }
        } else if constexpr (kQ4) {
            const __half* srow = (g.scale_unit != 0) ? reinterpret_cast<const __half*>(st + g.scale_off) + (size_t)r_in * C + part
                                                     : reinterpret_cast<const __half*>(cv.scales) + (size_t)min(my_row, a.row_end - 1) * C + part;
            // a row of eight blocks handled by one lane: its eight block scales are one 16-byte read
            uint4 sc8 = make_uint4(0u, 0u, 0u, 0u);
            constexpr bool kRowScales = kSpec && LPR == 1 && CPL == 8;
            if constexpr (kRowScales) sc8 = *reinterpret_cast<const uint4*>(srow);
            const uint4* qbase = reinterpret_cast<const uint4*>(q_s) + 2 * part;
            const int q_stride = g.q_bytes / 16;
            // one pass over the lane's chunks for the high plane (DO_H), the low plane (DO_L) or both
            auto q4_pass = [&](auto do_h, auto do_l) {
                for_each_chunk([&](int c) {
                    const uint4 d = rowp[c];
                    const uint32_t w[4] = {d.x, d.y, d.z, d.w};
                    int ev[4], od[4];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        ev[t] = (int)((w[t] << 4) & 0xF0F0F0F0u);
                        od[t] = (int)(w[t] & 0xF0F0F0F0u);
                    }
                    float bs;
                    if constexpr (kRowScales) {
                        const uint32_t pair = (c < 2) ? sc8.x : (c < 4) ? sc8.y : (c < 6) ? sc8.z : sc8.w;
                        bs = __half2float(__ushort_as_half((unsigned short)((c & 1) ? (pair >> 16) : (pair & 0xffffu))));
                    } else {
                        bs = __half2float(srow[c]);
                    }
#pragma unroll
                    for (int q = 0; q < QT; ++q) {
                        const uint4* qh = qbase + q * q_stride + 2 * c;
                        const uint4* ql = qh + 2 * C;
                        if constexpr (decltype(do_h)::value) {
                            const uint4 h0 = qh[0], h1 = qh[1];
                            const uint32_t ph[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
                            int h = 0;
#pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                h = __dp4a(ev[t], (int)ph[2 * t], h);
                                h = __dp4a(od[t], (int)ph[2 * t + 1], h);
                            }
                            fa[q] = __fmaf_rn((float)h, bs, fa[q]);
                        }
                        if constexpr (decltype(do_l)::value) {
                            const uint4 l0 = ql[0], l1 = ql[1];
                            const uint32_t pl[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
                            int l = 0;
#pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                l = __dp4a(ev[t], (int)pl[2 * t], l);
                                l = __dp4a(od[t], (int)pl[2 * t + 1], l);
                            }
                            fb[q] = __fmaf_rn((float)l, bs, fb[q]);
                        }
                    }
                });
            };
            using yes = std::integral_constant<bool, true>;
            using no = std::integral_constant<bool, false>;
            if (l2_pref && !observe) {
                // High plane first.  The low plane can change a dot product by at most ||q_lo|| * ||row||, so a tile in
                // which no row passes the distance filter even with that much added is finished after half the work;
                // otherwise the low plane is accumulated as well and the exact filter and evaluation follow.
                q4_pass(yes{}, no{});
                bool maybe = false;
                const float dn2e = __uint_as_float((cv.stats != nullptr) ? reinterpret_cast<const uint32_t*>(st + g.stat_off)[r_in] : 0u);
                const float dnorm = sqrtf(dn2e) * 1.000001f;
#pragma unroll
                for (int q = 0; q < QT; ++q) {
                    float th = fa[q];
#pragma unroll
                    for (int off = lpr >> 1; off > 0; off >>= 1) th += __shfl_xor_sync(0xffffffffu, th, off);
                    const float dot_hi = __fmul_rn(th, q4_sh[q]);
                    const float slack = __fmaf_rn(lo_norm[q], dnorm, 1e-6f * fabsf(dot_hi));
                    maybe = maybe || (rv && dot_hi + slack >= __fmaf_rn(dn2e, 0.4999995f, l2_ch[q]));
                }
                if (!__any_sync(0xffffffffu, maybe)) {
                    skip_tile = true;
                } else {
                    q4_pass(no{}, yes{});
                }
            } else {
                q4_pass(yes{}, yes{});
            }
        } else {
            const bool l2 = a.metric == MANTA_B200_METRIC_L2_DISTANCE;
            const float4* qbase = reinterpret_cast<const float4*>(q_s) + 2 * part;
            const int q_stride = g.q_bytes / 16;
            for_each_chunk([&](int c) {
                const uint4 d = rowp[c];
                const __half2* hp = reinterpret_cast<const __half2*>(&d);
                float f[8];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const float2 p = __half22float2(hp[t]);
                    f[2 * t] = p.x;
                    f[2 * t + 1] = p.y;
                }
#pragma unroll
                for (int q = 0; q < QT; ++q) {
                    const float4* qf = qbase + q * q_stride + 2 * c;
                    const float4 q0 = qf[0], q1 = qf[1];
                    const float qv[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                    float acc = fa[q];
                    if (l2) {
                        // sum (q - d)^2 directly, as the reference does: no cancellation near zero distance
#pragma unroll
                        for (int t = 0; t < 8; ++t) {
                            const float df = __fsub_rn(qv[t], f[t]);
                            acc = __fmaf_rn(df, df, acc);
                        }
                    } else {
#pragma unroll
                        for (int t = 0; t < 8; ++t) acc = __fmaf_rn(f[t], qv[t], acc);
                    }
                    fa[q] = acc;
                }
            });
        }
        // ---- finish the row: log2(lpr) exchange steps, then the row's leader lane holds the sums
#pragma unroll
        for (int q = 0; q < QT && !skip_tile; ++q) {
#pragma unroll
            for (int off = lpr >> 1; off > 0; off >>= 1) {
                if constexpr (kQ8) {
                    ih[q] += __shfl_xor_sync(0xffffffffu, ih[q], off);
                    il[q] += __shfl_xor_sync(0xffffffffu, il[q], off);
                } else if constexpr (kQ4) {
                    fa[q] += __shfl_xor_sync(0xffffffffu, fa[q], off);
                    fb[q] += __shfl_xor_sync(0xffffffffu, fb[q], off);
                } else {
                    fa[q] += __shfl_xor_sync(0xffffffffu, fa[q], off);
                }
            }
        }
        const uint32_t stat = (cv.stats != nullptr) ? reinterpret_cast<const uint32_t*>(st + g.stat_off)[r_in] : 0u;
        const int nn = (int)stat;
        const float dn2 = __uint_as_float(stat);
        float sd = 0.0f;
        if constexpr (kQ8) sd = reinterpret_cast<const float*>(st + g.rscale_off)[r_in];
        float rinv = 0.0f;
        if (a.metric == MANTA_B200_METRIC_COSINE) rinv = kQ8 ? q8_row_inv_norm(nn) : float_row_inv_norm(dn2);
        const int slot = (int)(fresh & (kSlots - 1));
#pragma unroll
        for (int q = 0; q < QT && !skip_tile; ++q) {
            float score;
            if constexpr (kQ8) {
                if (a.mode == kModeAccum) {
                    if (rv && q == 0) {
                        int32_t* o = a.out_acc + (size_t)(my_row - a.row_begin) * 3;
                        o[0] = ih[q];
                        o[1] = il[q];
                        o[2] = nn;
                    }
                    continue;
                }
                if (l2_pref && !observe) {
                    const float t = __fmaf_rn((float)il[q], hdr[q].s_lo, __fmul_rn((float)ih[q], hdr[q].s_hi));
                    float dc = __fmul_rn(t, sd);
                    dc = dc + 4e-7f * fabsf(dc);   // the exact path forms this product in f64
                    const float dn2c = __fmul_rn(__fmul_rn(sd, sd), (float)nn);
                    const bool pass = rv && dc >= __fmaf_rn(dn2c, 0.4999995f, l2_ch[q]);
                    if (!__any_sync(0xffffffffu, pass)) continue;
                }
                score = q8_finish(a.metric, ih[q], il[q], nn, rinv, sd, hdr[q]);
            } else if constexpr (kQ4) {
                const float dotv = __fmaf_rn(fb[q], q4_sl[q], __fmul_rn(fa[q], q4_sh[q]));
                if (l2_pref && !observe) {
                    const bool pass = rv && dotv >= __fmaf_rn(dn2, 0.4999995f, l2_ch[q]);
                    if (!__any_sync(0xffffffffu, pass)) continue;
                }
                score = float_finish(a.metric, dotv, dn2, rinv, hdr[q], hdr[q].qhat2);
            } else {
                if (a.metric == MANTA_B200_METRIC_L2_DISTANCE)
                    score = __fsqrt_rn(fa[q]) + 0.0f;  // fa holds sum (q - d)^2 here
                else
                    score = float_finish(a.metric, fa[q], dn2, rinv, hdr[q], hdr[q].qn2d);
            }
            const bool mine = rv && q < a.qt;
            if (a.mode == kModeScores) {
                if (mine) a.out_scores[(size_t)(a.q0 + q) * cv.rows + my_row] = score;
            } else if (topk) {
                const float gd = score * sign + 0.0f;
                const uint32_t o = ord_from_float(gd);
                if (mine && !replay) bmax[q][slot] = max(bmax[q][slot], o);
                const uint64_t key = make_key(gd, (int32_t)(cv.row_base + my_row));
                if (!observe) {
                    append(q, mine && o >= thr[q], key);
                } else if (kHold) {
#pragma unroll
                    for (int e = 0; e < kHeld; ++e)
                        if (i == e) {
                            held_key[e] = key;
                            held_ok[e] = mine;
                        }
                }
            }
        }
        if (!topk || replay) continue;
        ++fresh;
        // ---- publish this warp's running maximum of the slot when it changed
#pragma unroll
        for (int q = 0; q < QT; ++q) {
            uint32_t m = bmax[q][slot];
            if (__any_sync(0xffffffffu, m > published[q][slot])) {
                m = __reduce_max_sync(0xffffffffu, m);
                published[q][slot] = m;
                bmax[q][slot] = m;
                if (lane == 0 && q < a.qt)
                    st_relaxed_u32(a.ws.bucket + (size_t)(a.q0 + q) * a.ws.nb + (size_t)gw * kSlots + slot, m);
            }
        }
        // ---- threshold refresh duty: warp 0, at power-of-two tile counts, one block in eight per count (plus tile
        // counts 3 and 6 early on); the blocks on duty at a count share the launch's queries among them, one query
        // each.  The bound is built from the top 20 bits only: rounding it down keeps it valid and costs a fraction of
        // a percent of selectivity.
        const bool duty_iter = (fresh & (fresh - 1)) == 0 || fresh == 3 || fresh == 6;
        if (warp == 0 && duty_iter && ((blockIdx.x & 7) == ((fresh == 3 || fresh == 6) ? 7 - (fresh / 3) : ((31 - __clz(fresh)) & 7)))) {
            const int q = (int)((blockIdx.x >> 3) % (unsigned)a.qt);
            const uint32_t* b = a.ws.bucket + (size_t)(a.q0 + q) * a.ws.nb;
            // A bound needs k buckets; for small k the first 256 buckets are plenty (any subset of buckets gives a
            // valid, slightly lower bound) and fit in eight registers per lane.
            const uint32_t nb_all = min(min(a.ws.nb, (uint32_t)kScanRefreshWords), (uint32_t)(nwarps * kSlots));
            uint32_t t = 0;
            if (2u * (uint32_t)a.k <= 256u) {
                const uint32_t nb = min(nb_all, 256u);
                uint32_t v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = ((uint32_t)(u * 32 + lane) < nb) ? __ldcg(b + u * 32 + lane) : 0u;
                for (int bit = 31; bit >= 12; --bit) {
                    const uint32_t cand = t | (1u << bit);
                    uint32_t cnt = 0;
#pragma unroll
                    for (int u = 0; u < 8; ++u) cnt += (v[u] >= cand) ? 1u : 0u;
                    cnt = __reduce_add_sync(0xffffffffu, cnt);
                    if (cnt >= (uint32_t)a.k) t = cand;
                }
            } else if (nb_all >= (uint32_t)a.k) {
                // Larger k: the maxima are staged in shared memory and the top 20 bits of the k-th largest are found by
                // a radix select (8 + 8 + 4 bits, one histogram pass each).
                const uint32_t nb = nb_all;
                for (uint32_t i0 = lane; i0 < nb; i0 += 256) {   // eight independent loads at a time
                    uint32_t v[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) v[u] = (i0 + u * 32 < nb) ? __ldcg(b + i0 + u * 32) : 0u;
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        if (i0 + u * 32 < nb) s_stage[i0 + u * 32] = v[u];
                }
                uint32_t* hist = s_stage + kScanRefreshWords;   // 256 bins behind the staged values
                uint32_t prefix = 0, mask = 0, need = (uint32_t)a.k;
                bool ok = true;
#pragma unroll 1
                for (int pass = 0; pass < 3 && ok; ++pass) {
                    const int shift = (pass == 0) ? 24 : (pass == 1) ? 16 : 12;
                    const uint32_t bin_mask = (pass == 2) ? 15u : 255u;
                    for (int h = lane; h < 256; h += 32) hist[h] = 0u;
                    __syncwarp();
                    for (uint32_t j = lane; j < nb; j += 32) {
                        const uint32_t v = s_stage[j];
                        if ((v & mask) == prefix) atomicAdd(&hist[(v >> shift) & bin_mask], 1u);
                    }
                    __syncwarp();
                    // lane l owns digits 8l .. 8l+7; counts of all higher digits come from a suffix sum over the lanes
                    uint32_t c[8], mine = 0;
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        c[u] = hist[lane * 8 + u];
                        mine += c[u];
                    }
                    uint32_t incl = mine;   // becomes the count of values whose digit is in this lane's range or above
#pragma unroll
                    for (int off = 1; off < 32; off <<= 1) {
                        const uint32_t up = __shfl_down_sync(0xffffffffu, incl, off);
                        if (lane + off < 32) incl += up;
                    }
                    int hit = -1;
                    uint32_t run = incl - mine, above_digit = 0;
#pragma unroll
                    for (int u = 7; u >= 0; --u) {
                        if (hit < 0) {
                            if (run + c[u] >= need) {
                                hit = u;
                                above_digit = run;
                            } else {
                                run += c[u];
                            }
                        }
                    }
                    const uint32_t ballot = __ballot_sync(0xffffffffu, hit >= 0);
                    if (ballot == 0u) {
                        ok = false;
                    } else {
                        const int src = 31 - __clz(ballot);   // the highest digit range that reaches the rank
                        const uint32_t digit = (uint32_t)__shfl_sync(0xffffffffu, lane * 8 + hit, src);
                        need -= __shfl_sync(0xffffffffu, above_digit, src);
                        prefix |= digit << shift;
                        mask |= bin_mask << shift;
                    }
                    __syncwarp();
                }
                if (ok) t = prefix;
            }
            if (lane == 0 && t != 0) atomicMax(a.ws.thr + a.q0 + q, t);
            __syncwarp();
        }
    }
    cp_async_wait<0>();

    // ---- tail of a fused pass: the last block to arrive selects the exact top k of this launch's queries
    if (!a.fused_select) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t prev = atomicAdd(a.done_blocks, 1u);
        s_last = (prev + 1u == gridDim.x) ? 1 : 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    SelectArgs sa{};
    sa.ws = a.ws;
    sa.nq = a.nq_total;
    sa.k = a.k;
    sa.order = a.order;
    sa.write_back = 0;
    sa.out_ids = a.out_ids;
    sa.out_scores = a.out_topk_scores;
    sa.sink = a.sink;
    for (int q = 0; q < a.qt; ++q) {
        select_block(sa, a.q0 + q, ring);   // the ring is free: every warp of this block has drained its copies
        // leave the query's workspace zeroed: the next pass starts from a clean state without a reset launch
        uint32_t* b = a.ws.bucket + (size_t)(a.q0 + q) * a.ws.nb;
        const uint32_t nb_used = min(a.ws.nb, (uint32_t)(nwarps * kSlots));
        for (uint32_t j = threadIdx.x; j < nb_used; j += blockDim.x) b[j] = 0u;
        if (threadIdx.x == 0) {
            a.ws.count[a.q0 + q] = 0u;
            a.ws.thr[a.q0 + q] = 0u;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        a.done_blocks[0] = 0u;
        a.done_blocks[1] = 0u;   // the tile counter
        static_assert(kNumFlags == 4, "the flag words are read as one 16-byte load");
        const uint4 fl = __ldcg(reinterpret_cast<const uint4*>(a.ws.flags));
        const uint32_t fw[4] = {fl.x, fl.y, fl.z, fl.w};
#pragma unroll
        for (int f = 0; f < kNumFlags; ++f) {
            if (fw[f] != 0u) {
                a.host_flags[f] = 1u;   // sticky on the host until it reads and clears them
                a.ws.flags[f] = 0u;
            }
        }
    }
}

// ---- host side ---------------------------------------------------------------------------------------------------
template <int LAYOUT, int QT, int LPR, int CPL>
cudaError_t launch_stream_scan_form(cudaStream_t st, int sm_count, const StreamArgs& a, size_t smem) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(stream_scan_kernel<LAYOUT, QT, LPR, CPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kScanSmemLimit);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    // one persistent block per SM; every warp is a bucket owner, so the grid is exactly what is resident at once
    const int grid = sm_count;
    stream_scan_kernel<LAYOUT, QT, LPR, CPL><<<grid, a.g.warps * 32, smem, st>>>(a);
    count_launch();
    note_scan_launch("stream_scan_kernel", grid, a.g.warps * 32, smem);
    return cudaGetLastError();
}

// One query per launch has specialised forms for the row shapes that matter most (768-byte rows: q8 x 768 and
// f16 x 384; 384-byte rows: q8 x 384; 128-byte rows: q4 x 256); everything else runs the generic form.
template <int LAYOUT, int QT>
cudaError_t launch_stream_scan_qt(cudaStream_t st, int sm_count, const StreamArgs& a, size_t smem) {
    if constexpr (QT == 1) {
        const int lpr = 1 << a.g.lpr_shift;
        const int C = a.cv.chunks;
        if (lpr == 4 && C == 48) return launch_stream_scan_form<LAYOUT, 1, 4, 12>(st, sm_count, a, smem);
        if (lpr == 2 && C == 24) return launch_stream_scan_form<LAYOUT, 1, 2, 12>(st, sm_count, a, smem);
        if (lpr == 1 && C == 8) return launch_stream_scan_form<LAYOUT, 1, 1, 8>(st, sm_count, a, smem);
    }
    return launch_stream_scan_form<LAYOUT, QT, 0, 0>(st, sm_count, a, smem);
}

template <int LAYOUT>
cudaError_t launch_stream_scan_layout(cudaStream_t st, int sm_count, StreamArgs a) {
    size_t smem = 0;
    const int qt_slots = a.qt <= 1 ? 1 : (a.qt <= 2 ? 2 : 4);
    if (!stream_scan_geometry(a.cv, qt_slots, a.row_begin, &a.g, &smem)) return cudaErrorInvalidValue;
    if (qt_slots == 1) return launch_stream_scan_qt<LAYOUT, 1>(st, sm_count, a, smem);
    if (qt_slots == 2) return launch_stream_scan_qt<LAYOUT, 2>(st, sm_count, a, smem);
    return launch_stream_scan_qt<LAYOUT, 4>(st, sm_count, a, smem);
}

cudaError_t launch_stream_scan_f16(cudaStream_t st, int sm_count, const StreamArgs& a);
cudaError_t launch_stream_scan_q8(cudaStream_t st, int sm_count, const StreamArgs& a);
cudaError_t launch_stream_scan_q4(cudaStream_t st, int sm_count, const StreamArgs& a);

}  // namespace mb200
