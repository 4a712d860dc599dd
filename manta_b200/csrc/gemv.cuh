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

template <int LPR, typename T>
__device__ __forceinline__ T group_sum(T v) {
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

template <int LAYOUT, int QT, int LPR, int CPL, int U>
__global__ void __launch_bounds__(kThreads, (QT == 1 && CPL <= 4) ? 2 : 1) gemv_kernel(const GemvArgs a, const int mode) {
    constexpr bool kQ8 = LAYOUT == MANTA_B200_LAYOUT_Q8_ROW_F32;
    constexpr bool kQ4 = LAYOUT == MANTA_B200_LAYOUT_Q4_B32_F16;
    constexpr bool kF16 = LAYOUT == MANTA_B200_LAYOUT_F16;
    constexpr int GPW = 32 / LPR;
    constexpr int ROWS_PER_WT = GPW * U;

    __shared__ uint32_t s_stage[4096];

    const int lane = threadIdx.x & 31;
    const int warp_in_cta = threadIdx.x >> 5;
    const int gl = lane % LPR;
    const int grp = lane / LPR;
    const int64_t gw = (int64_t)blockIdx.x * kWarpsPerCta + warp_in_cta;
    const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerCta;
    const CandView& cv = a.cv;

    // query registers and per-query constants
    QChunk<LAYOUT> qr[QT][CPL];
    QueryHeader hdr[QT];
#pragma unroll
    for (int q = 0; q < QT; ++q) {
        const int qi = a.q0 + ((q < a.qt) ? q : 0);  // unused slots repeat query 0 of the pass
        hdr[q] = a.qp.headers[qi];
#pragma unroll
        for (int j = 0; j < CPL; ++j) {
            const int chunk = j * LPR + gl;
            if constexpr (kF16)
                qr[q][j].load(a.qp, qi, chunk, chunk < cv.chunks, cv.cols);
            else
                qr[q][j].load(a.qp, qi, chunk, chunk < cv.chunks);
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

    // Everything one warp-tile needs from memory.  The loads of tile t+1 are issued before tile t is consumed
    // (software pipelining), so every lane keeps U*CPL 16-byte loads in flight while it computes.
    struct Tile {
        uint4 data[U][CPL];
        float sd[U];          // q8: row scale
        __half q4s[U][CPL];   // q4: block scales
        uint32_t stat[U];     // row statistic bits (leader lane only)
    };
    auto load_tile = [&](int64_t wt, Tile& t) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t r = a.row_begin + wt * ROWS_PER_WT + (int64_t)u * GPW + grp;
            const bool rv = wt < n_wt && r < a.row_end;
            const uint8_t* rp = cv.data + (size_t)(rv ? r : a.row_begin) * cv.row_bytes;
#pragma unroll
            for (int j = 0; j < CPL; ++j) {
                const int chunk = j * LPR + gl;
                if (rv && chunk < cv.chunks)
                    t.data[u][j] = ld_stream16(rp + (size_t)chunk * 16);
                else
                    t.data[u][j] = make_uint4(0, 0, 0, 0);
                if constexpr (kQ4) {
                    t.q4s[u][j] = __ushort_as_half((unsigned short)0);
                    if (rv && chunk < cv.chunks) t.q4s[u][j] = ((const __half*)cv.scales)[(size_t)r * cv.chunks + chunk];
                }
            }
            t.sd[u] = 0.0f;
            t.stat[u] = 0u;
            if (rv && want_scale) t.sd[u] = ((const float*)cv.scales)[r];
            if (rv && gl == 0 && want_stats) t.stat[u] = ((const uint32_t*)cv.stats)[r];
        }
    };

    Tile nxt;
    load_tile(gw, nxt);
    uint32_t iter = 0;
    for (int64_t wt = gw; wt < n_wt; wt += nwarps) {
        ++iter;
        uint32_t thr[QT];
        if (mode == kModeTopk) {
#pragma unroll
            for (int q = 0; q < QT; ++q) thr[q] = ld_relaxed_u32(a.ws.thr + a.q0 + ((q < a.qt) ? q : 0));
            // a pool that overflowed makes the host redo the pass in chunks: stop streaming
            if ((iter & 15) == 0 && ld_relaxed_u32(a.ws.flags + kFlagOverflow) != 0) break;
        }
        const Tile cur = nxt;
        load_tile(wt + nwarps, nxt);
        int64_t row[U];
#pragma unroll
        for (int u = 0; u < U; ++u) row[u] = a.row_begin + wt * ROWS_PER_WT + (int64_t)u * GPW + grp;
        const auto& data = cur.data;
        const auto& sd = cur.sd;
        // ---- accumulate
        int ih[U][QT], il[U][QT];
        float fa[U][QT], fb[U][QT];
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
            for (int q = 0; q < QT; ++q) {
                ih[u][q] = il[u][q] = 0;
                fa[u][q] = fb[u][q] = 0.0f;
            }
#pragma unroll
            for (int j = 0; j < CPL; ++j) {
                const uint4 d = data[u][j];
                if constexpr (kQ8) {
#pragma unroll
                    for (int q = 0; q < QT; ++q) {
                        int h = ih[u][q], l = il[u][q];
                        h = __dp4a((int)d.x, (int)qr[q][j].hi.x, h);
                        h = __dp4a((int)d.y, (int)qr[q][j].hi.y, h);
                        h = __dp4a((int)d.z, (int)qr[q][j].hi.z, h);
                        h = __dp4a((int)d.w, (int)qr[q][j].hi.w, h);
                        l = __dp4a((int)d.x, (int)qr[q][j].lo.x, l);
                        l = __dp4a((int)d.y, (int)qr[q][j].lo.y, l);
                        l = __dp4a((int)d.z, (int)qr[q][j].lo.z, l);
                        l = __dp4a((int)d.w, (int)qr[q][j].lo.w, l);
                        ih[u][q] = h;
                        il[u][q] = l;
                    }
                } else if constexpr (kQ4) {
                    const uint32_t w[4] = {d.x, d.y, d.z, d.w};
                    int ev[4], od[4];
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        ev[g] = (int)((w[g] << 4) & 0xF0F0F0F0u);
                        od[g] = (int)(w[g] & 0xF0F0F0F0u);
                    }
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
                        const float bs = __half2float(cur.q4s[u][j]);
                        fa[u][q] = __fmaf_rn((float)h, bs, fa[u][q]);
                        fb[u][q] = __fmaf_rn((float)l, bs, fb[u][q]);
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
                            float acc = fa[u][q];
#pragma unroll
                            for (int t = 0; t < 8; ++t) {
                                const float df = __fsub_rn(qr[q][j].v[t], f[t]);
                                acc = __fmaf_rn(df, df, acc);
                            }
                            fa[u][q] = acc;
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < QT; ++q) {
                            float acc = fa[u][q];
#pragma unroll
                            for (int t = 0; t < 8; ++t) acc = __fmaf_rn(f[t], qr[q][j].v[t], acc);
                            fa[u][q] = acc;
                        }
                    }
                }
            }
        }
        // ---- reduce over the lanes of a row, finish the score, store or filter
        int nnv[U];
        float dn2v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            nnv[u] = (int)cur.stat[u];
            dn2v[u] = __uint_as_float(cur.stat[u]);
        }
#pragma unroll
        for (int q = 0; q < QT; ++q) {
            uint64_t key[U];
            uint32_t ballots[U];
            uint32_t total = 0;
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const bool rv = row[u] < a.row_end;
                float score;
                if constexpr (kQ8) {
                    const int h = group_sum<LPR>(ih[u][q]);
                    const int l = group_sum<LPR>(il[u][q]);
                    if (mode == kModeAccum) {
                        if (rv && gl == 0 && q == 0) {
                            int32_t* o = a.out_acc + (size_t)(row[u] - a.row_begin) * 3;
                            o[0] = h;
                            o[1] = l;
                            o[2] = nnv[u];
                        }
                        ballots[u] = 0;
                        continue;
                    }
                    score = q8_finish(a.metric, h, l, nnv[u], sd[u], hdr[q]);
                } else if constexpr (kQ4) {
                    const float th = group_sum<LPR>(fa[u][q]);
                    const float tl = group_sum<LPR>(fb[u][q]);
                    const float dotv = __fmaf_rn(tl, q4_sl[q], __fmul_rn(th, q4_sh[q]));
                    score = float_finish(a.metric, dotv, dn2v[u], hdr[q], hdr[q].qhat2);
                } else {
                    const float dotv = group_sum<LPR>(fa[u][q]);
                    if (a.metric == MANTA_B200_METRIC_L2_DISTANCE)
                        score = __fsqrt_rn(dotv) + 0.0f;  // dotv holds sum (q - d)^2 here
                    else
                        score = float_finish(a.metric, dotv, dn2v[u], hdr[q], hdr[q].qn2d);
                }
                const bool mine = rv && gl == 0 && q < a.qt;
                bool pass = false;
                if (mode == kModeScores) {
                    if (mine) a.out_scores[(size_t)(a.q0 + q) * cv.rows + row[u]] = score;
                } else if (mode == kModeTopk) {
                    const float g = score * sign + 0.0f;
                    const uint32_t o = ord_from_float(g);
                    if (mine) {
                        bmax[q] = max(bmax[q], o);
                        pass = o >= thr[q];
                        key[u] = make_key(g, (int32_t)(cv.row_base + row[u]));
                    }
                }
                ballots[u] = __ballot_sync(0xffffffffu, pass);
                total += __popc(ballots[u]);
            }
            // one reservation per warp-tile and query for all rows that passed
            if (mode == kModeTopk && total != 0) {
                uint32_t base = 0;
                if (lane == 0) base = atomicAdd(a.ws.count + a.q0 + q, total);
                base = __shfl_sync(0xffffffffu, base, 0);
                uint64_t* pool = a.ws.pool + (size_t)(a.q0 + q) * a.ws.cap;
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (ballots[u] & (1u << lane)) {
                        const uint32_t pos = base + __popc(ballots[u] & ((1u << lane) - 1u));
                        if (pos < a.ws.cap)
                            pool[pos] = key[u];
                        else
                            a.ws.flags[kFlagOverflow] = 1u;
                    }
                    base += __popc(ballots[u]);
                }
            }
        }
        if (mode != kModeTopk) continue;
        // ---- publish this warp's running maxima when they changed
#pragma unroll
        for (int q = 0; q < QT; ++q) {
            uint32_t m = (gl == 0) ? bmax[q] : 0u;
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
                const uint32_t nb = min(a.ws.nb, 4096u);
                for (uint32_t i = lane; i < nb; i += 32) s_stage[i] = ld_relaxed_u32(b + i);
                __syncwarp();
                uint32_t t = 0;
                for (int bit = 31; bit >= 12; --bit) {
                    const uint32_t cand = t | (1u << bit);
                    uint32_t cnt = 0;
                    for (uint32_t i = lane; i < nb; i += 32) cnt += (s_stage[i] >= cand) ? 1u : 0u;
                    cnt = __reduce_add_sync(0xffffffffu, cnt);
                    if (cnt >= (uint32_t)a.k) t = cand;
                }
                if (lane == 0 && t != 0) atomicMax(a.ws.thr + a.q0 + q, t);
                __syncwarp();
            }
        }
    }
}

template <int LAYOUT, int QT, int LPR, int CPL>
cudaError_t launch_gemv_shape(cudaStream_t st, int grid, const GemvArgs& a, int mode) {
    constexpr int U = (CPL == 1) ? 8 : (CPL == 2) ? 4 : (CPL <= 4) ? 2 : 1;
    gemv_kernel<LAYOUT, QT, LPR, CPL, U><<<grid, kThreads, 0, st>>>(a, mode);
    count_launch();
    return cudaGetLastError();
}

template <int LAYOUT, int QT>
cudaError_t launch_gemv_qt(cudaStream_t st, int grid, const GemvArgs& a, int mode, const GemvShape& s) {
#define MB200_SHAPE(L, C) \
    if (s.lpr == L && s.cpl == C) return launch_gemv_shape<LAYOUT, QT, L, C>(st, grid, a, mode);
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
    if (qt == 1) return launch_gemv_qt<LAYOUT, 1>(st, grid, a, mode, s);
    if (qt == 2) return launch_gemv_qt<LAYOUT, 2>(st, grid, a, mode, s);
    return launch_gemv_qt<LAYOUT, 4>(st, grid, a, mode, s);
}

cudaError_t launch_gemv_f16(cudaStream_t st, int sm_count, const GemvArgs& a, int mode);
cudaError_t launch_gemv_q8(cudaStream_t st, int sm_count, const GemvArgs& a, int mode);
cudaError_t launch_gemv_q4(cudaStream_t st, int sm_count, const GemvArgs& a, int mode);

}  // namespace mb200
