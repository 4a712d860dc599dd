// Streaming (GEMV) scoring kernel: 1, 2 or 4 queries against packed candidate rows, each row read once with
// 128-bit loads, de-quantised in registers, reduced with warp shuffles, score finished in the epilogue and
// either stored (full score vector) or filtered into the top-k candidate pool.
//
// Work split.  A row is covered by LPR lanes (LPR in {8,16,32}); lane l of the group reads 16-byte chunks
// l, l+LPR, ... (CPL of them), so a warp instruction reads 32/LPR adjacent rows, fully coalesced.  A warp
// owns "warp-tiles" of (32/LPR)*U rows and strides over the row range; U rows are loaded before any is
// consumed so that U*CPL 16-byte loads are in flight per lane.  Warps never synchronise with each other.
//
// The query lives in registers: for q8/q4 candidates as two int8 planes (q ~= s_hi*hi + s_lo*lo) consumed
// with dp4a into int32 accumulators; for f16 candidates as f32 consumed with fma.
//
// Top-k.  A row's score enters the query's pool when it is not below the query's threshold.  The threshold
// is the k-th largest of the per-warp running maxima ("buckets"; each warp sees a disjoint set of rows, so k
// bucket maxima >= t prove that k rows score >= t): it can only be too low, never too high, so the pool
// always contains the true top k.  Warp 0 of some CTAs recomputes it at power-of-two tile counts.
#pragma once

#include "kernels.h"

namespace mb200 {

template <int LAYOUT>
struct QChunk;  // the query registers that pair with one 16-byte chunk of a candidate row

template <>
struct QChunk<MANTA_B200_LAYOUT_Q8_ROW_F32> {
    uint4 hi, lo;
    __device__ __forceinline__ void load(const QueryPrep& qp, int q, int chunk, bool valid) {
        hi = lo = make_uint4(0, 0, 0, 0);
        if (valid) {
            hi = *(const uint4*)(qp.plane_hi + (size_t)q * qp.plane_stride + (size_t)chunk * 16);
            lo = *(const uint4*)(qp.plane_lo + (size_t)q * qp.plane_stride + (size_t)chunk * 16);
        }
    }
};
template <>
struct QChunk<MANTA_B200_LAYOUT_Q4_B32_F16> {
    uint4 hi[2], lo[2];
    __device__ __forceinline__ void load(const QueryPrep& qp, int q, int chunk, bool valid) {
        hi[0] = hi[1] = lo[0] = lo[1] = make_uint4(0, 0, 0, 0);
        if (valid) {
            const uint4* ph = (const uint4*)(qp.plane_hi + (size_t)q * qp.plane_stride + (size_t)chunk * 32);
            const uint4* pl = (const uint4*)(qp.plane_lo + (size_t)q * qp.plane_stride + (size_t)chunk * 32);
            hi[0] = ph[0];
            hi[1] = ph[1];
            lo[0] = pl[0];
            lo[1] = pl[1];
        }
    }
};
template <>
struct QChunk<MANTA_B200_LAYOUT_F16> {
    float v[8];
    __device__ __forceinline__ void load(const QueryPrep& qp, int q, int chunk, bool valid, int cols) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int e = chunk * 8 + j;
            v[j] = (valid && e < cols) ? qp.qf32[(size_t)q * cols + e] : 0.0f;
        }
    }
};

constexpr int kStages = 3;        // ring depth of the asynchronous copies (kStages-1 warp-tiles in flight)
constexpr int kStageWords = 2560; // bucket maxima a threshold refresh can stage in shared memory

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int LPR, typename T>
__device__ __forceinline__ T group_sum(T v) {
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// Sums v[0..V) over the LPR lanes of a row group and leaves the total of v[i] on the lanes whose position in
// the group, gl, satisfies gl / (LPR / V) == i (returned value).  Values are exchanged half at a time, so the
// whole reduction costs V - 1 + log2(LPR / V) shuffles instead of V * log2(LPR).
template <int LPR, int V, typename T>
__device__ __forceinline__ T reduce_scatter(T (&v)[V], int gl) {
    static_assert((V & (V - 1)) == 0 && V <= LPR, "V must be a power of two not above LPR");
    int off = LPR / 2;
#pragma unroll
    for (int n = V / 2; n >= 1; n >>= 1, off >>= 1) {
        const bool upper = (gl & off) != 0;
#pragma unroll
        for (int i = 0; i < n; ++i) {
            const T send = upper ? v[i] : v[i + n];
            const T keep = upper ? v[i + n] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
#pragma unroll
    for (; off > 0; off >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
    return v[0];
}

// L2P: instantiation for nearest-neighbour l2 on packed rows in top-k mode (an f32 pre-filter in front of the f64
// finish); kept out of the other instantiations so that their code is untouched by it.
template <int LAYOUT, int QT, int LPR, int CPL, int U, bool L2P>
__global__ void __launch_bounds__(kThreads, (QT == 1 && CPL <= 4) ? 2 : 1) gemv_kernel(const GemvArgs a, const int mode) {
    constexpr bool kQ8 = LAYOUT == MANTA_B200_LAYOUT_Q8_ROW_F32;
    constexpr bool kQ4 = LAYOUT == MANTA_B200_LAYOUT_Q4_B32_F16;
    constexpr bool kF16 = LAYOUT == MANTA_B200_LAYOUT_F16;
    constexpr int GPW = 32 / LPR;             // row groups per warp
    constexpr int ROWS_PER_WT = GPW * U;      // rows per warp-tile
    constexpr int OWN = LPR / U;              // lanes of a group that end up holding the same row's sums
    constexpr int SLOTS = U * CPL;

    const int lane = threadIdx.x & 31;
    const int warp_in_cta = threadIdx.x >> 5;
    const int gl = lane % LPR;
    const int grp = lane / LPR;
    const int own_u = gl / OWN;               // the row of the tile (within the group) this lane finishes
    const bool leader = (gl % OWN) == 0;
    const int own_off = own_u * GPW + grp;    // row offset inside the warp-tile
    const int64_t gw = (int64_t)blockIdx.x * kWarpsPerCta + warp_in_cta;
    const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerCta;
    const CandView& cv = a.cv;

    // query registers and per-query constants
    QChunk<LAYOUT> qr[QT][CPL];
    QueryHeader hdr[QT];
    bool cvalid[CPL];
#pragma unroll
    for (int j = 0; j < CPL; ++j) cvalid[j] = (j * LPR + gl) < cv.chunks;
#pragma unroll
    for (int q = 0; q < QT; ++q) {
        const int qi = a.q0 + ((q < a.qt) ? q : 0);  // unused slots repeat query 0 of the pass
        hdr[q] = a.qp.headers[qi];
#pragma unroll
        for (int j = 0; j < CPL; ++j) {
            const int chunk = j * LPR + gl;
            if constexpr (kF16)
                qr[q][j].load(a.qp, qi, chunk, cvalid[j], cv.cols);
            else
                qr[q][j].load(a.qp, qi, chunk, cvalid[j]);
        }
    }
    float q4_sh[QT], q4_sl[QT];
#pragma unroll
    for (int q = 0; q < QT; ++q) {
        q4_sh[q] = hdr[q].s_hi * 0.0625f;  // the nibble unpack yields 16*code
        q4_sl[q] = hdr[q].s_lo * 0.0625f;
    }

    const float sign = (a.order == MANTA_B200_ORDER_SMALLEST) ? -1.0f : 1.0f;
    uint32_t bmax[QT], published[QT];
#pragma unroll
    for (int q = 0; q < QT; ++q) bmax[q] = published[q] = 0;

    const int64_t nrows = a.row_end - a.row_begin;
    const int64_t n_wt = (nrows + ROWS_PER_WT - 1) / ROWS_PER_WT;
    const bool want_stats = (a.metric != MANTA_B200_METRIC_DOT || mode == kModeAccum) &&
                            !(kF16 && a.metric == MANTA_B200_METRIC_L2_DISTANCE);
    const bool want_scale = kQ8 && a.metric != MANTA_B200_METRIC_COSINE;

    // Candidate bytes travel global -> shared memory with 16-byte asynchronous copies (cp.async.cg, no registers
    // held while in flight): every lane copies exactly the chunks it will consume itself into its own slots of a
    // kStages-deep ring, so no barrier is needed; kStages-1 warp-tiles are in flight per lane while one is
    // consumed.  The small per-row values (scale, block scales, statistic) are prefetched one tile ahead in
    // registers, by the lane that will finish that row.
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    uint4* ring = reinterpret_cast<uint4*>(dyn_smem);
    uint32_t* s_stage = reinterpret_cast<uint32_t*>(dyn_smem + (size_t)kStages * SLOTS * kThreads * 16);
    auto slot = [&](int stage, int i) -> uint4* { return ring + ((size_t)(stage * SLOTS + i) * kThreads + threadIdx.x); };
    const size_t tile_stride = (size_t)ROWS_PER_WT * cv.row_bytes;
    // address of this lane's first chunk of row `grp` of warp-tile `gw`
    const uint8_t* lane_base = cv.data + (size_t)(a.row_begin + gw * ROWS_PER_WT + grp) * cv.row_bytes + (size_t)gl * 16;
    const size_t u_stride = (size_t)GPW * cv.row_bytes;
    auto issue_tile = [&](int64_t wt, int stage) {
        const int64_t left = nrows - wt * ROWS_PER_WT;  // rows of the range at or after this tile's first row
        const uint8_t* tp = lane_base + (size_t)(wt - gw) * tile_stride;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const bool rv = (int64_t)(u * GPW + grp) < left;
#pragma unroll
            for (int j = 0; j < CPL; ++j) {
                if (rv && cvalid[j])
                    cp_async16(slot(stage, u * CPL + j), tp + u * u_stride + (size_t)j * LPR * 16);
                else
                    *slot(stage, u * CPL + j) = make_uint4(0, 0, 0, 0);
            }
        }
        cp_async_commit();
    };
    struct Meta {
        float sd;             // q8: scale of the row this lane finishes
        uint32_t stat;        // statistic bits of that row
        __half q4s[U][CPL];   // q4: block scales of the chunks this lane accumulates
    };
    auto load_meta = [&](int64_t wt, Meta& t) {
        const int64_t first = a.row_begin + wt * ROWS_PER_WT;
        if constexpr (kQ4) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t r = first + u * GPW + grp;
                const bool rv = wt < n_wt && r < a.row_end;
#pragma unroll
                for (int j = 0; j < CPL; ++j) {
                    t.q4s[u][j] = __ushort_as_half((unsigned short)0);
                    if (rv && cvalid[j]) t.q4s[u][j] = ((const __half*)cv.scales)[(size_t)r * cv.chunks + j * LPR + gl];
                }
            }
        }
        const int64_t r = first + own_off;
        const bool rv = leader && wt < n_wt && r < a.row_end;
        t.sd = 0.0f;
        t.stat = 0u;
        if (rv && want_scale) t.sd = ((const float*)cv.scales)[r];
        if (rv && want_stats) t.stat = ((const uint32_t*)cv.stats)[r];
    };

#pragma unroll
    for (int p = 0; p < kStages - 1; ++p) issue_tile(gw + (int64_t)p * nwarps, p);
    Meta nxt;
    load_meta(gw, nxt);
    uint32_t iter = 0;
    uint32_t overflow_seen = 0;
    uint32_t thr[QT];
    // Nearest-neighbour l2 on packed rows finishes a score in f64 (square root included).  In top-k mode a row is
    // first tested in f32: dist <= B  <=>  dot >= (||q||^2 - B^2 + ||row||^2) / 2, with B the current bound and a few
    // ulps of slack; a warp-tile in which no row passes skips the exact evaluation.  Rows that do not pass are below
    // the bound, so leaving them out of the bucket maxima keeps those maxima valid lower bounds.
    constexpr bool l2_pref = L2P && (kQ8 || kQ4);   // the launcher picks this instantiation for (top-k, l2, smallest) only
    float l2_ch[QT];   // (||q||^2 - B^2) / 2 per query, lowered; -inf while no bound exists
#pragma unroll
    for (int q = 0; q < QT; ++q) l2_ch[q] = -INFINITY;
    auto update_l2_bounds = [&]() {
        if constexpr (l2_pref) {
#pragma unroll
        for (int q = 0; q < QT; ++q) {
            float ch = -INFINITY;
            if (thr[q] > 1u) {
                const float bnd = fmaxf(-float_from_ord(thr[q]), 0.0f);
                const double b2 = (double)bnd * (double)bnd * (1.0 + 4e-6) + 1e-30;
                ch = (float)((hdr[q].qhat2 - b2) * 0.5);
                ch = ch - fabsf(ch) * 1e-6f - 1e-30f;
            }
            l2_ch[q] = ch;
        }
        }
    };
    // Rows of the first two tiles are scored before any bound exists.  They are held back (one key per lane and
    // tile) and enter the pool, filtered, once the first bound has arrived, so the pool never sees a burst.
    uint64_t early_key[QT][2];
    bool early_ok[QT][2];
#pragma unroll
    for (int q = 0; q < QT; ++q) {
        thr[q] = 0;
        early_ok[q][0] = early_ok[q][1] = false;
        early_key[q][0] = early_key[q][1] = 0;
    }
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
    auto flush_early = [&]() {
#pragma unroll
        for (int q = 0; q < QT; ++q) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                if (__any_sync(0xffffffffu, early_ok[q][e])) {
                    append(q, early_ok[q][e] && (uint32_t)(early_key[q][e] >> 32) >= thr[q], early_key[q][e]);
                    early_ok[q][e] = false;
                }
            }
        }
    };
    int stage = 0;
    for (int64_t wt = gw; wt < n_wt; wt += nwarps) {
        ++iter;
        if (mode == kModeTopk) {
            // the bounds move fast only at the start: reread them every tile early on, every eighth tile later
            if (iter <= 16 || (iter & 7) == 0) {
#pragma unroll
                for (int q = 0; q < QT; ++q) thr[q] = ld_relaxed_u32(a.ws.thr + a.q0 + ((q < a.qt) ? q : 0));
                update_l2_bounds();
            }
            // a pool that overflowed makes the host redo the pass in chunks: stop streaming.  The flag is
            // loaded in one check and tested in the next, so its latency never stalls the stream.
            if ((iter & 63) == 0) {
                if (overflow_seen != 0) break;
                overflow_seen = ld_relaxed_u32(a.ws.flags + kFlagOverflow);
            }
            // Two tiles per warp have been scored without a bound and are held back.  Before streaming on, let
            // the first bound arrive (the warps on refresh duty at tile counts 2 and 3 are computing it), then
            // release the held rows through the filter.  The wait is bounded; giving up only costs pool space.
            if (iter == 3) {
                if (!a.no_startup_wait && !(warp_in_cta == 0 && (blockIdx.x & 7) == 6)) {
#pragma unroll
                    for (int q = 0; q < QT; ++q) {
                        for (int spin = 0; thr[q] == 0 && spin < 2000; ++spin) {
                            __nanosleep(32);
                            thr[q] = ld_relaxed_u32(a.ws.thr + a.q0 + ((q < a.qt) ? q : 0));
                        }
                    }
                    update_l2_bounds();
                }
                flush_early();
            }
        }
        cp_async_wait<kStages - 2>();  // the copies of this tile have landed
        // refill the stage that was consumed in the previous iteration
        issue_tile(wt + (int64_t)(kStages - 1) * nwarps, (stage == 0) ? kStages - 1 : stage - 1);
        uint4 data[U][CPL];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int j = 0; j < CPL; ++j) data[u][j] = *slot(stage, u * CPL + j);
        stage = (stage + 1 == kStages) ? 0 : stage + 1;
        const Meta cur = nxt;
        load_meta(wt + nwarps, nxt);

        // ---- accumulate: ih/il int32 (q8), fa/fb f32 (q4: hi/lo planes; f16: fa only)
        int ih[QT][U], il[QT][U];
        float fa[QT][U], fb[QT][U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
            for (int q = 0; q < QT; ++q) {
                ih[q][u] = il[q][u] = 0;
                fa[q][u] = fb[q][u] = 0.0f;
            }
#pragma unroll
            for (int j = 0; j < CPL; ++j) {
                const uint4 d = data[u][j];
                if constexpr (kQ8) {
#pragma unroll
                    for (int q = 0; q < QT; ++q) {
                        int h = ih[q][u], l = il[q][u];
                        h = __dp4a((int)d.x, (int)qr[q][j].hi.x, h);
                        h = __dp4a((int)d.y, (int)qr[q][j].hi.y, h);
                        h = __dp4a((int)d.z, (int)qr[q][j].hi.z, h);
                        h = __dp4a((int)d.w, (int)qr[q][j].hi.w, h);
                        l = __dp4a((int)d.x, (int)qr[q][j].lo.x, l);
                        l = __dp4a((int)d.y, (int)qr[q][j].lo.y, l);
                        l = __dp4a((int)d.z, (int)qr[q][j].lo.z, l);
                        l = __dp4a((int)d.w, (int)qr[q][j].lo.w, l);
                        ih[q][u] = h;
                        il[q][u] = l;
                    }
                } else if constexpr (kQ4) {
                    const uint32_t w[4] = {d.x, d.y, d.z, d.w};
                    int ev[4], od[4];
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        ev[g] = (int)((w[g] << 4) & 0xF0F0F0F0u);
                        od[g] = (int)(w[g] & 0xF0F0F0F0u);
                    }
                    const float bs = __half2float(cur.q4s[u][j]);
#pragma unroll
                    for (int q = 0; q < QT; ++q) {
                        const uint32_t* ph = (const uint32_t*)qr[q][j].hi;
                        const uint32_t* pl = (const uint32_t*)qr[q][j].lo;
                        int h = 0, l = 0;
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            h = __dp4a(ev[g], (int)ph[2 * g], h);
                            h = __dp4a(od[g], (int)ph[2 * g + 1], h);
                            l = __dp4a(ev[g], (int)pl[2 * g], l);
                            l = __dp4a(od[g], (int)pl[2 * g + 1], l);
                        }
                        fa[q][u] = __fmaf_rn((float)h, bs, fa[q][u]);
                        fb[q][u] = __fmaf_rn((float)l, bs, fb[q][u]);
                    }
                } else {
                    const __half2* hp = (const __half2*)&d;
                    float f[8];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        float2 p = __half22float2(hp[t]);
                        f[2 * t] = p.x;
                        f[2 * t + 1] = p.y;
                    }
                    if (a.metric == MANTA_B200_METRIC_L2_DISTANCE) {
                        // sum (q - d)^2 directly, as the reference does: no cancellation near zero distance
#pragma unroll
                        for (int q = 0; q < QT; ++q) {
                            float acc = fa[q][u];
#pragma unroll
                            for (int t = 0; t < 8; ++t) {
                                const float df = __fsub_rn(qr[q][j].v[t], f[t]);
                                acc = __fmaf_rn(df, df, acc);
                            }
                            fa[q][u] = acc;
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < QT; ++q) {
                            float acc = fa[q][u];
#pragma unroll
                            for (int t = 0; t < 8; ++t) acc = __fmaf_rn(f[t], qr[q][j].v[t], acc);
                            fa[q][u] = acc;
                        }
                    }
                }
            }
        }

        // ---- reduce over the lanes of a row; afterwards lane (own_u, leader) holds the sums of row own_u of its
        // group, so one pass of the epilogue finishes all GPW*U rows of the warp-tile at once
        const int64_t my_row = a.row_begin + wt * ROWS_PER_WT + own_off;
        const bool rv = leader && my_row < a.row_end;
        const int nn = (int)cur.stat;
        const float dn2 = __uint_as_float(cur.stat);
        float rinv = 0.0f;
        if (a.metric == MANTA_B200_METRIC_COSINE) rinv = kQ8 ? q8_row_inv_norm(nn) : float_row_inv_norm(dn2);
#pragma unroll
        for (int q = 0; q < QT; ++q) {
            float score;
            if constexpr (kQ8) {
                const int h = reduce_scatter<LPR, U>(ih[q], gl);
                const int l = reduce_scatter<LPR, U>(il[q], gl);
                if (mode == kModeAccum) {
                    if (rv && q == 0) {
                        int32_t* o = a.out_acc + (size_t)(my_row - a.row_begin) * 3;
                        o[0] = h;
                        o[1] = l;
                        o[2] = nn;
                    }
                    continue;
                }
                if constexpr (l2_pref) if (iter > 2) {
                    const float t = __fmaf_rn((float)l, hdr[q].s_lo, __fmul_rn((float)h, hdr[q].s_hi));
                    float dc = __fmul_rn(t, cur.sd);
                    dc = dc + 4e-7f * fabsf(dc);   // the exact path forms this product in f64
                    const float dn2c = __fmul_rn(__fmul_rn(cur.sd, cur.sd), (float)nn);
                    const bool pass = rv && dc >= __fmaf_rn(dn2c, 0.4999995f, l2_ch[q]);
                    if (!__any_sync(0xffffffffu, pass)) continue;
                }
                score = q8_finish(a.metric, h, l, nn, rinv, cur.sd, hdr[q]);
            } else if constexpr (kQ4) {
                const float th = reduce_scatter<LPR, U>(fa[q], gl);
                const float tl = reduce_scatter<LPR, U>(fb[q], gl);
                const float dotv = __fmaf_rn(tl, q4_sl[q], __fmul_rn(th, q4_sh[q]));
                if constexpr (l2_pref) if (iter > 2) {
                    const bool pass = rv && dotv >= __fmaf_rn(dn2, 0.4999995f, l2_ch[q]);
                    if (!__any_sync(0xffffffffu, pass)) continue;
                }
                score = float_finish(a.metric, dotv, dn2, rinv, hdr[q], hdr[q].qhat2);
            } else {
                const float dotv = reduce_scatter<LPR, U>(fa[q], gl);
                if (a.metric == MANTA_B200_METRIC_L2_DISTANCE)
                    score = __fsqrt_rn(dotv) + 0.0f;  // dotv holds sum (q - d)^2 here
                else
                    score = float_finish(a.metric, dotv, dn2, rinv, hdr[q], hdr[q].qn2d);
            }
            const bool mine = rv && q < a.qt;
            if (mode == kModeScores) {
                if (mine) a.out_scores[(size_t)(a.q0 + q) * cv.rows + my_row] = score;
            } else if (mode == kModeTopk) {
                const float g = score * sign + 0.0f;
                const uint32_t o = ord_from_float(g);
                if (mine) bmax[q] = max(bmax[q], o);
                const uint64_t key = make_key(g, (int32_t)(cv.row_base + my_row));
                if (iter == 1) {
                    early_key[q][0] = key;
                    early_ok[q][0] = mine;
                } else if (iter == 2) {
                    early_key[q][1] = key;
                    early_ok[q][1] = mine;
                } else {
                    append(q, mine && o >= thr[q], key);
                }
            }
        }
        if (mode != kModeTopk) continue;
        // ---- publish this warp's running maxima when they changed
#pragma unroll
        for (int q = 0; q < QT; ++q) {
            uint32_t m = bmax[q];
            if (__any_sync(0xffffffffu, m > published[q])) {
                m = __reduce_max_sync(0xffffffffu, m);
                published[q] = m;
                bmax[q] = m;
                if (lane == 0 && q < a.qt) st_relaxed_u32(a.ws.bucket + (size_t)(a.q0 + q) * a.ws.nb + gw, m);
            }
        }
        // ---- threshold refresh duty: warp 0, at power-of-two tile counts, one CTA in eight per count
        // (plus tile counts 3, 6 early on).  The bound is built from the top 20 bits only: rounding it down keeps
        // it valid and costs a fraction of a percent of selectivity.
        const bool duty_iter = (iter & (iter - 1)) == 0 || iter == 3 || iter == 6;
        if (warp_in_cta == 0 && duty_iter && ((blockIdx.x & 7) == ((iter == 3 || iter == 6) ? 7 - (iter / 3) : ((31 - __clz(iter)) & 7)))) {
            for (int q = 0; q < a.qt; ++q) {
                const uint32_t* b = a.ws.bucket + (size_t)(a.q0 + q) * a.ws.nb;
                // A bound needs k buckets; for small k the first 256 warps' maxima are plenty (any subset of
                // buckets gives a valid, slightly lower bound) and fit in eight registers per lane.
                const uint32_t nb_all = min(min(a.ws.nb, (uint32_t)kStageWords), (uint32_t)nwarps);
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
                } else {
                    const uint32_t nb = nb_all;
                    // eight independent loads at a time (a volatile load per element would serialise on its store)
                    for (uint32_t i0 = lane; i0 < nb; i0 += 256) {
                        uint32_t v[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u) v[u] = (i0 + u * 32 < nb) ? __ldcg(b + i0 + u * 32) : 0u;
#pragma unroll
                        for (int u = 0; u < 8; ++u)
                            if (i0 + u * 32 < nb) s_stage[i0 + u * 32] = v[u];
                    }
                    __syncwarp();
                    for (int bit = 31; bit >= 12; --bit) {
                        const uint32_t cand = t | (1u << bit);
                        uint32_t cnt = 0;
                        for (uint32_t i = lane; i < nb; i += 32) cnt += (s_stage[i] >= cand) ? 1u : 0u;
                        cnt = __reduce_add_sync(0xffffffffu, cnt);
                        if (cnt >= (uint32_t)a.k) t = cand;
                    }
                }
                if (lane == 0 && t != 0) atomicMax(a.ws.thr + a.q0 + q, t);
                __syncwarp();
            }
        }
    }
    if (mode == kModeTopk) {
        // warps that ran out of tiles before the release point: whatever they still hold goes through the
        // filter with the freshest bounds
#pragma unroll
        for (int q = 0; q < QT; ++q) thr[q] = ld_relaxed_u32(a.ws.thr + a.q0 + ((q < a.qt) ? q : 0));
        flush_early();
    }
    cp_async_wait<0>();
}

template <int LAYOUT, int QT, int LPR, int CPL, bool L2P>
cudaError_t launch_gemv_shape(cudaStream_t st, int grid, const GemvArgs& a, int mode) {
    constexpr int U = (CPL == 1) ? 8 : (CPL == 2) ? 4 : (CPL <= 4) ? 2 : 1;
    constexpr size_t smem = (size_t)kStages * U * CPL * kThreads * 16 + (size_t)kStageWords * 4;
    // One attribute call and one occupancy query per instantiation and device.  The grid is exactly what is
    // resident at once (every warp is a bucket and the start-up wait relies on all of them running).
    static int resident[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    int occ = (dev >= 0 && dev < 64) ? resident[dev] : 0;
    if (occ == 0) {
        cudaError_t e = cudaFuncSetAttribute(gemv_kernel<LAYOUT, QT, LPR, CPL, U, L2P>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, gemv_kernel<LAYOUT, QT, LPR, CPL, U, L2P>, kThreads, smem);
        if (e != cudaSuccess) return e;
        if (occ < 1) return cudaErrorLaunchOutOfResources;
        if (occ > 2) occ = 2;
        if (dev >= 0 && dev < 64) resident[dev] = occ;
    }
    grid = (grid / 2) * occ;  // the caller passes 2 CTAs per SM, the bucket layout's upper bound
    gemv_kernel<LAYOUT, QT, LPR, CPL, U, L2P><<<grid, kThreads, smem, st>>>(a, mode);
    count_launch();
    note_scan_launch("gemv_kernel", grid, kThreads, smem);
    return cudaGetLastError();
}

template <int LAYOUT, int QT, bool L2P>
cudaError_t launch_gemv_qt(cudaStream_t st, int grid, const GemvArgs& a, int mode, const GemvShape& s) {
#define MB200_SHAPE(L, C) \
    if (s.lpr == L && s.cpl == C) return launch_gemv_shape<LAYOUT, QT, L, C, L2P>(st, grid, a, mode);
    MB200_SHAPE(8, 1) MB200_SHAPE(8, 2) MB200_SHAPE(8, 3) MB200_SHAPE(8, 4)
    MB200_SHAPE(16, 1) MB200_SHAPE(16, 2) MB200_SHAPE(16, 3) MB200_SHAPE(16, 4)
    MB200_SHAPE(32, 1) MB200_SHAPE(32, 2) MB200_SHAPE(32, 3) MB200_SHAPE(32, 4)
    if constexpr (QT == 1) {
        MB200_SHAPE(32, 8)
    }
#undef MB200_SHAPE
    return cudaErrorInvalidValue;
}

template <int LAYOUT>
cudaError_t launch_gemv_layout(cudaStream_t st, int sm_count, const GemvArgs& a, int mode) {
    GemvShape s;
    if (!pick_gemv_shape(a.cv.chunks, &s)) return cudaErrorInvalidValue;
    const int grid = gemv_grid_size(sm_count);
    int qt = a.qt;
    if (s.cpl == 8 && qt != 1) return cudaErrorInvalidValue;
    if constexpr (LAYOUT != MANTA_B200_LAYOUT_F16) {
        if (mode == kModeTopk && a.metric == MANTA_B200_METRIC_L2_DISTANCE && a.order == MANTA_B200_ORDER_SMALLEST) {
            if (qt == 1) return launch_gemv_qt<LAYOUT, 1, true>(st, grid, a, mode, s);
            if (qt == 2) return launch_gemv_qt<LAYOUT, 2, true>(st, grid, a, mode, s);
            return launch_gemv_qt<LAYOUT, 4, true>(st, grid, a, mode, s);
        }
    }
    if (qt == 1) return launch_gemv_qt<LAYOUT, 1, false>(st, grid, a, mode, s);
    if (qt == 2) return launch_gemv_qt<LAYOUT, 2, false>(st, grid, a, mode, s);
    return launch_gemv_qt<LAYOUT, 4, false>(st, grid, a, mode, s);
}

cudaError_t launch_gemv_f16(cudaStream_t st, int sm_count, const GemvArgs& a, int mode);
cudaError_t launch_gemv_q8(cudaStream_t st, int sm_count, const GemvArgs& a, int mode);
cudaError_t launch_gemv_q4(cudaStream_t st, int sm_count, const GemvArgs& a, int mode);

}  // namespace mb200
