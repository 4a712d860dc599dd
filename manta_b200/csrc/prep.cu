// Query preparation, bind-time row statistics, quantisers and row gather.
#include "kernels.h"

namespace mb200 {

// ---- query preparation ---------------------------------------------------------------------------------
// One CTA per query.  Produces the QueryHeader, the f32 copy of the query, and for q8/q4 candidates the
// two int8 planes q ~= s_hi*hi + s_lo*lo laid out chunk by chunk the way the scoring kernels consume them:
//   q8 : plane chunk c holds elements 16c..16c+15 in order;
//   q4 : plane chunk c (32 elements = one block) holds, per 8-element group g, the even elements
//        (8g, 8g+2, 8g+4, 8g+6) in word 2g and the odd elements in word 2g+1, matching the nibble unpack
//        ((w << 4) & 0xF0F0F0F0 -> even elements, w & 0xF0F0F0F0 -> odd elements).
// Also resets the selection workspace of its query (count, threshold, buckets).
//
// ||q||^2 is summed in f64: lane l of warp 0 adds elements l, l+32, ... in order, then the 32 partial sums
// are combined by an xor butterfly (16, 8, 4, 2, 1).  The CPU model of the packed path uses the same order.
__global__ void __launch_bounds__(256) query_prep_kernel(const __half* __restrict__ queries, int cols, int layout,
                                                         int plane_stride, QueryHeader* __restrict__ headers,
                                                         float* __restrict__ qf32, int8_t* __restrict__ plane_hi,
                                                         int8_t* __restrict__ plane_lo, float* __restrict__ lo_norm, SelectWs ws,
                                                         int reset_ws) {
    const int q = blockIdx.x;
    const int tid = threadIdx.x;
    const __half* src = queries + (size_t)q * cols;
    __shared__ float s_red[8];
    __shared__ int s_lsq[8];
    __shared__ float s_amax;
    __shared__ float s_sh, s_sl;

    float amax = 0.0f;
    for (int c = tid; c < cols; c += blockDim.x) {
        float v = __half2float(src[c]);
        qf32[(size_t)q * cols + c] = v;
        amax = fmaxf(amax, fabsf(v));
    }
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if ((tid & 31) == 0) s_red[tid >> 5] = amax;
    __syncthreads();
    if (tid < 32) {
        float m = (tid < 8) ? s_red[tid] : 0.0f;
        for (int off = 4; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        double part = 0.0;
        for (int c = tid; c < cols; c += 32) {
            double v = (double)__half2float(src[c]);
            part = __dadd_rn(part, __dmul_rn(v, v));
        }
        for (int off = 16; off > 0; off >>= 1) part = __dadd_rn(part, __shfl_xor_sync(0xffffffffu, part, off));
        if (tid == 0) {
            QueryHeader h;
            h.qn = __double2float_rn(__dsqrt_rn(part));
            h.qinv = (h.qn > 0.0f) ? __fdiv_rn(1.0f, h.qn) : 0.0f;
            h.qn2d = part;
            h.qhat2 = part;
            float sh = 0.0f, sl = 0.0f;
            if (m > 0.0f) {
                sh = __fdiv_rn(m, 127.0f);
                sl = __fdiv_rn(sh, 254.0f);
            }
            h.s_hi = sh;
            h.s_lo = sl;
            headers[q] = h;
            s_amax = m;
            s_sh = sh;
            s_sl = sl;
        }
    }
    __syncthreads();
    if (layout != MANTA_B200_LAYOUT_F16) {
        const float sh = s_sh, sl = s_sl;
        const bool zero = !(s_amax > 0.0f);
        int lsq = 0;   // sum of the squared low-plane codes of this thread's elements
        for (int c = tid; c < plane_stride; c += blockDim.x) {
            // c indexes the plane in storage order; e is the query element stored there
            int e = c;
            if (layout == MANTA_B200_LAYOUT_Q4_B32_F16) {
                int blk = c >> 5, w = (c >> 2) & 7, b = c & 3;
                e = blk * 32 + (w >> 1) * 8 + 2 * b + (w & 1);
            }
            int8_t hi = 0, lo = 0;
            if (!zero && e < cols) {
                float v = __half2float(src[e]);
                float h = roundf(__fdiv_rn(v, sh));
                h = fminf(fmaxf(h, -127.0f), 127.0f);
                float rem = __fmaf_rn(-h, sh, v);
                float l = 0.0f;
                if (sl != 0.0f) {
                    l = roundf(__fdiv_rn(rem, sl));
                    l = fminf(fmaxf(l, -127.0f), 127.0f);
                }
                hi = (int8_t)h;
                lo = (int8_t)l;
            }
            plane_hi[(size_t)q * plane_stride + c] = hi;
            plane_lo[(size_t)q * plane_stride + c] = lo;
            lsq += (int)lo * (int)lo;
        }
        // norm of the low plane, a shade high: what the plane can add to a dot product is at most this times the norm of
        // the row's codes (the tensor-core pass bounds it that way when it contracts the high planes only)
        lsq = __reduce_add_sync(0xffffffffu, lsq);
        if ((tid & 31) == 0) s_lsq[tid >> 5] = lsq;
        __syncthreads();
        if (tid == 0 && lo_norm != nullptr) {
            int tot = 0;
            for (int w = 0; w < 8; ++w) tot += s_lsq[w];
            lo_norm[q] = sqrtf((float)tot) * 1.000002f;
        }
    }
    if (layout != MANTA_B200_LAYOUT_F16) {
        // squared norm of the query the planes represent, same summation order as ||q||^2
        __syncthreads();
        if (tid < 32) {
            const float sh = s_sh, sl = s_sl;
            const bool zero = !(s_amax > 0.0f);
            double part = 0.0;
            for (int c = tid; c < cols; c += 32) {
                double v = 0.0;
                if (!zero) {
                    float x = __half2float(src[c]);
                    float h = roundf(__fdiv_rn(x, sh));
                    h = fminf(fmaxf(h, -127.0f), 127.0f);
                    float rem = __fmaf_rn(-h, sh, x);
                    float l = 0.0f;
                    if (sl != 0.0f) {
                        l = roundf(__fdiv_rn(rem, sl));
                        l = fminf(fmaxf(l, -127.0f), 127.0f);
                    }
                    v = __dadd_rn(__dmul_rn((double)h, (double)sh), __dmul_rn((double)l, (double)sl));
                }
                part = __dadd_rn(part, __dmul_rn(v, v));
            }
            for (int off = 16; off > 0; off >>= 1) part = __dadd_rn(part, __shfl_xor_sync(0xffffffffu, part, off));
            if (tid == 0) headers[q].qhat2 = part;
        }
    }
    if (reset_ws) {
        if (tid == 0) {
            ws.count[q] = 0;
            ws.thr[q] = 0;
        }
        for (uint32_t i = tid; i < ws.nb; i += blockDim.x) ws.bucket[(size_t)q * ws.nb + i] = 0;
        if (q == 0 && tid < kNumFlags) ws.flags[tid] = 0;
    }
}

// ---- bind-time row statistics ------------------------------------------------------------------------
// One warp per row.  q8: stat[r] = sum code^2 (int32, exact).  q4: stat[r] = sum_b s_b^2 * sum code^2 (f32).
// f16: stat[r] = f32 of the f64 sum of squares.  Lane l takes 16-byte chunks l, l+32, ... in order and the
// partial sums are combined by an xor butterfly.
__global__ void __launch_bounds__(256) row_stats_kernel(CandView cv, void* __restrict__ stats) {
    const int lane = threadIdx.x & 31;
    int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= cv.rows) return;
    const uint8_t* row = cv.data + (size_t)r * cv.row_bytes;
    if (cv.layout == MANTA_B200_LAYOUT_Q8_ROW_F32) {
        int nn = 0;
        for (int ch = lane; ch < cv.chunks; ch += 32) {
            uint4 v = *(const uint4*)(row + (size_t)ch * 16);
            nn = __dp4a((int)v.x, (int)v.x, nn);
            nn = __dp4a((int)v.y, (int)v.y, nn);
            nn = __dp4a((int)v.z, (int)v.z, nn);
            nn = __dp4a((int)v.w, (int)v.w, nn);
        }
        nn = __reduce_add_sync(0xffffffffu, nn);
        if (lane == 0) ((int32_t*)stats)[r] = nn;
    } else if (cv.layout == MANTA_B200_LAYOUT_Q4_B32_F16) {
        const __half* sc = (const __half*)cv.scales + (size_t)r * (cv.cols / 32);
        float acc = 0.0f;
        for (int b = lane; b < cv.chunks; b += 32) {
            uint4 v = *(const uint4*)(row + (size_t)b * 16);
            uint32_t w[4] = {v.x, v.y, v.z, v.w};
            int m = 0;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                int e = (int)((w[g] << 4) & 0xF0F0F0F0u), o = (int)(w[g] & 0xF0F0F0F0u);
                m = __dp4a(e, e, m);
                m = __dp4a(o, o, m);
            }
            float s = __half2float(sc[b]);
            acc = __fmaf_rn(__fmul_rn(s, s), (float)(m >> 8), acc);
        }
        for (int off = 16; off > 0; off >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
        if (lane == 0) ((float*)stats)[r] = acc;
    } else {
        double acc = 0.0;
        for (int ch = lane; ch < cv.chunks; ch += 32) {
            uint4 v = *(const uint4*)(row + (size_t)ch * 16);
            const __half2* h = (const __half2*)&v;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 f = __half22float2(h[j]);
                acc = __dadd_rn(acc, __dmul_rn((double)f.x, (double)f.x));
                acc = __dadd_rn(acc, __dmul_rn((double)f.y, (double)f.y));
            }
        }
        for (int off = 16; off > 0; off >>= 1) acc = __dadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
        if (lane == 0) ((float*)stats)[r] = __double2float_rn(acc);
    }
}

// ---- quantisers -------------------------------------------------------------------------------------------
template <bool SRC_F16>
__device__ __forceinline__ float load_src(const void* src, size_t i) {
    if (SRC_F16) return __half2float(((const __half*)src)[i]);
    return ((const float*)src)[i];
}

// One warp per row: max|x| by shuffle, scale = max/127 (f32 division), code = round-half-away(x/scale).
template <bool SRC_F16>
__global__ void __launch_bounds__(256) pack_q8_rows_kernel(const void* __restrict__ src, int64_t rows, int cols,
                                                           int dst_stride, int8_t* __restrict__ codes,
                                                           float* __restrict__ scales) {
    const int lane = threadIdx.x & 31;
    int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const size_t base = (size_t)r * cols;
    float amax = 0.0f;
    for (int c = lane; c < cols; c += 32) amax = fmaxf(amax, fabsf(load_src<SRC_F16>(src, base + c)));
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    float scale = __fdiv_rn(amax, 127.0f);
    bool zero = (amax == 0.0f) || (scale == 0.0f);
    if (lane == 0) scales[r] = zero ? 0.0f : scale;
    int8_t* dst = codes + (size_t)r * dst_stride;
    for (int c = lane; c < dst_stride; c += 32) {
        int8_t q = 0;
        if (!zero && c < cols) {
            float v = roundf(__fdiv_rn(load_src<SRC_F16>(src, base + c), scale));
            q = (int8_t)fminf(fmaxf(v, -127.0f), 127.0f);
        }
        dst[c] = q;
    }
}

// One thread per 32-element block: scale = half(max/7), codes against the rounded scale.
template <bool SRC_F16>
__global__ void __launch_bounds__(256) pack_q4_b32_kernel(const void* __restrict__ src, int64_t total_blocks,
                                                          uint8_t* __restrict__ codes, __half* __restrict__ scales) {
    int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= total_blocks) return;
    float x[32];
    float amax = 0.0f;
#pragma unroll
    for (int c = 0; c < 32; ++c) {
        x[c] = load_src<SRC_F16>(src, (size_t)b * 32 + c);
        amax = fmaxf(amax, fabsf(x[c]));
    }
    __half hs = __float2half_rn(__fdiv_rn(amax, 7.0f));
    float scale = __half2float(hs);
    bool zero = (amax == 0.0f) || (scale == 0.0f);
    scales[b] = zero ? __ushort_as_half((unsigned short)0) : hs;
    uint32_t words[4] = {0, 0, 0, 0};
    if (!zero) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            float v = roundf(__fdiv_rn(x[c], scale));
            int q = (int)fminf(fmaxf(v, -7.0f), 7.0f);
            words[c >> 3] |= (uint32_t)(q & 15) << (4 * (c & 7));
        }
    }
    ((uint4*)codes)[b] = make_uint4(words[0], words[1], words[2], words[3]);
}

// ---- gather of de-quantised rows ----------------------------------------------------------------------
// out[i, c] = value(ids[i] - row_base, c) as f32.  One CTA per output row.  Out-of-range ids are reported
// through bad_id (first one wins) and their rows are left untouched.
__global__ void __launch_bounds__(256) gather_rows_kernel(CandView cv, const int32_t* __restrict__ ids, int64_t n,
                                                          float* __restrict__ out, int32_t* __restrict__ bad_id,
                                                          uint32_t* __restrict__ bad_flag) {
    int64_t i = blockIdx.x;
    if (i >= n) return;
    int64_t r = (int64_t)ids[i] - cv.row_base;
    if (r < 0 || r >= cv.rows) {
        if (threadIdx.x == 0 && atomicExch(bad_flag, 1u) == 0u) *bad_id = ids[i];
        return;
    }
    const uint8_t* row = cv.data + (size_t)r * cv.row_bytes;
    float* dst = out + (size_t)i * cv.cols;
    for (int c = threadIdx.x; c < cv.cols; c += blockDim.x) {
        float v;
        if (cv.layout == MANTA_B200_LAYOUT_Q8_ROW_F32) {
            v = __fmul_rn((float)((const int8_t*)row)[c], ((const float*)cv.scales)[r]);
        } else if (cv.layout == MANTA_B200_LAYOUT_Q4_B32_F16) {
            int byte = row[c >> 1];
            int nib = (c & 1) ? (byte >> 4) : (byte & 15);
            nib = (nib >= 8) ? nib - 16 : nib;
            float s = __half2float(((const __half*)cv.scales)[(size_t)r * (cv.cols / 32) + (c >> 5)]);
            v = __fmul_rn((float)nib, s);
        } else {
            v = __half2float(((const __half*)row)[c]);
        }
        dst[c] = v;
    }
}

// ---- workspace reset ---------------------------------------------------------------------------------------------
// One block per query: fill count, threshold and bucket maxima to zero; block 0 also clears the flags and the counter
// of finished blocks.  The fused scan leaves its workspace clean by itself; this kernel runs only after a pass that
// did not (the tensor-core pass, a chunked rerun, an error).
__global__ void __launch_bounds__(256) ws_reset_kernel(SelectWs ws, uint32_t* done_blocks) {
    const int q = blockIdx.x;
    if (threadIdx.x == 0) {
        ws.count[q] = 0;
        ws.thr[q] = 0;
    }
    for (uint32_t i = threadIdx.x; i < ws.nb; i += blockDim.x) ws.bucket[(size_t)q * ws.nb + i] = 0;
    if (q == 0 && threadIdx.x < kNumFlags) ws.flags[threadIdx.x] = 0;
    if (q == 0 && threadIdx.x == 0 && done_blocks != nullptr) done_blocks[0] = done_blocks[1] = 0;
}

cudaError_t launch_ws_reset(cudaStream_t st, const SelectWs& ws, int nq, uint32_t* done_blocks) {
    ws_reset_kernel<<<nq, 256, 0, st>>>(ws, done_blocks);
    count_launch();
    return cudaGetLastError();
}

// ---- launchers ----------------------------------------------------------------------------------------------
void launch_query_prep(cudaStream_t st, const void* d_queries_f16, int nq, int cols, int layout, int plane_stride, float* lo_norm,
                       QueryHeader* headers, float* qf32, int8_t* plane_hi, int8_t* plane_lo, const SelectWs& ws,
                       int reset_ws) {
    query_prep_kernel<<<nq, 256, 0, st>>>((const __half*)d_queries_f16, cols, layout, plane_stride, headers, qf32,
                                           plane_hi, plane_lo, lo_norm, ws, reset_ws);
    count_launch();
}

void launch_row_stats(cudaStream_t st, const CandView& cv, void* stats) {
    if (cv.rows == 0) return;
    unsigned grid = (unsigned)((cv.rows + 7) / 8);
    row_stats_kernel<<<grid, 256, 0, st>>>(cv, stats);
    count_launch();
}

void launch_pack_q8(cudaStream_t st, const void* d_src, bool src_f16, int64_t rows, int cols, int dst_stride,
                    int8_t* d_codes, float* d_scales) {
    if (rows == 0) return;
    unsigned grid = (unsigned)((rows + 7) / 8);
    if (src_f16)
        pack_q8_rows_kernel<true><<<grid, 256, 0, st>>>(d_src, rows, cols, dst_stride, d_codes, d_scales);
    else
        pack_q8_rows_kernel<false><<<grid, 256, 0, st>>>(d_src, rows, cols, dst_stride, d_codes, d_scales);
    count_launch();
}

void launch_pack_q4(cudaStream_t st, const void* d_src, bool src_f16, int64_t rows, int cols, uint8_t* d_codes,
                    uint16_t* d_scales) {
    int64_t blocks = rows * (cols / 32);
    if (blocks == 0) return;
    unsigned grid = (unsigned)((blocks + 255) / 256);
    if (src_f16)
        pack_q4_b32_kernel<true><<<grid, 256, 0, st>>>(d_src, blocks, d_codes, (__half*)d_scales);
    else
        pack_q4_b32_kernel<false><<<grid, 256, 0, st>>>(d_src, blocks, d_codes, (__half*)d_scales);
    count_launch();
}

void launch_gather_rows(cudaStream_t st, const CandView& cv, const int32_t* d_ids, int64_t n, float* d_out,
                        int32_t* d_bad_id, uint32_t* d_bad_flag) {
    if (n == 0) return;
    gather_rows_kernel<<<(unsigned)n, 256, 0, st>>>(cv, d_ids, n, d_out, d_bad_id, d_bad_flag);
    count_launch();
}

}  // namespace mb200
