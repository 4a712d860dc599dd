// Embedding front end of the score path on the device: gather(token_embedding, tokens) -> @matmul(projection) ->
// masked mean_pool / normalize, producing the f16 query batch the scoring kernels consume without a host hop.
// Reference host math: runtime/backend/tensor_ops.go:751-827 gather, :981-1011 matmul (f32, k ascending),
// :1210-1275 masked mean pool (rows added in order, times 1/count), :1114-1138 normalize (f64 sum of squares, f32
// norm, f32 divide, zero rows untouched).
//
// Two kernels, one per step order:
//  - normalize(mean_pool(x @ P)): the pool is linear, so the kept token rows are summed first and ONE row is
//    multiplied with the projection per batch element (seq times less arithmetic than the step-by-step order; the
//    f32 sums associate differently from the reference's, a relative difference of a few 1e-7);
//  - mean_pool(normalize(x @ P)): every kept token row is projected (f32 products and sums rounded separately, k
//    ascending, as the reference's loop does), normalised, and added to the pool in token order.  Shapes the tensor
//    cores take (embed_mma.cu) go another way: that file computes the norm of every token's projected row, and the
//    first kernel, given those norms, pools the embedding rows weighted by 1/norm and projects one row per batch
//    element -- the same linearity, a relative difference of about 1e-6 from the step-by-step order.
#include "kernels.h"

namespace mb200 {

constexpr int kEmbThreads = 256;
constexpr int kEmbRows = 16;  // token rows multiplied per pass over the projection matrix (second kernel)
constexpr int kEmbColsPerThread = 4;

// Warp 0 compacts the token ids of the kept positions, in order, into valid[] and checks every token's range (the
// reference's gather rejects an out-of-range token whether or not the mask keeps it).
__device__ __forceinline__ void count_valid_tokens(const int32_t* __restrict__ tokens, const int32_t* __restrict__ mask, int seq,
                                                   int vocab, int32_t* valid, int* s_count, int32_t* bad_token, uint32_t* bad_flag,
                                                   int32_t* vpos = nullptr) {
    const int lane = threadIdx.x & 31;
    int n = 0;
    for (int t0 = 0; t0 < seq; t0 += 32) {
        const int t = t0 + lane;
        int32_t tok = 0;
        bool keep = false;
        if (t < seq) {
            tok = tokens[t];
            if (tok < 0 || tok >= vocab) {
                if (atomicExch(bad_flag, 1u) == 0u) *bad_token = tok;
            } else {
                keep = mask[t] != 0;
            }
        }
        const uint32_t m = __ballot_sync(0xffffffffu, keep);
        if (keep) {
            valid[n + __popc(m & ((1u << lane) - 1u))] = tok;
            if (vpos) vpos[n + __popc(m & ((1u << lane) - 1u))] = t;
        }
        n += __popc(m);
    }
    if (lane == 0) *s_count = n;
}

// Block-wide f64 sum of per-thread partials (xor butterfly within a warp, then warps in order).
__device__ __forceinline__ double block_sum(double ss, double* s_part) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int off = 16; off > 0; off >>= 1) ss = __dadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, off));
    if (lane == 0) s_part[warp] = ss;
    __syncthreads();
    double tot = 0.0;
    for (int w = 0; w < kEmbThreads / 32; ++w) tot = __dadd_rn(tot, s_part[w]);
    return tot;
}

// normalize(mean_pool(gather(table, tokens) @ proj, mask)).  One CTA per batch element; thread t owns hidden
// elements t, t+256, ... of the token-row sum and output columns t, t+256, ...
// WEIGHTED: token_norms[b][t] is the norm of token t's projected row; the rows are pooled with the weights 1/norm (1 for
// a zero norm, whose row projects to zero anyway) and the result is mean_pool(normalize(...)): no final normalisation.
template <bool WEIGHTED>
__global__ void __launch_bounds__(kEmbThreads) embed_pool_first_kernel(const __half* __restrict__ table, int vocab, int dim,
                                                                       const __half* __restrict__ proj, int out_dim,
                                                                       const int32_t* __restrict__ tokens,
                                                                       const int32_t* __restrict__ mask, int seq,
                                                                       const float* __restrict__ token_norms,
                                                                       float* __restrict__ out_f32, __half* __restrict__ out_f16,
                                                                       int32_t* __restrict__ bad_token, uint32_t* __restrict__ bad_flag) {
    extern __shared__ __align__(16) unsigned char emb_smem[];
    float* hsum = reinterpret_cast<float*>(emb_smem);              // [dim]
    int32_t* valid = reinterpret_cast<int32_t*>(hsum + dim);       // [seq]
    int32_t* vpos = valid + seq;                                   // [seq], WEIGHTED only: position of each kept token
    float* wts = reinterpret_cast<float*>(vpos + seq);             // [seq], WEIGHTED only
    __shared__ int s_count;
    __shared__ double s_part[kEmbThreads / 32];
    const int b = blockIdx.x, tid = threadIdx.x;
    if (tid < 32)
        count_valid_tokens(tokens + (size_t)b * seq, mask + (size_t)b * seq, seq, vocab, valid, &s_count, bad_token, bad_flag,
                           WEIGHTED ? vpos : nullptr);
    __syncthreads();
    const int count = s_count;
    if constexpr (WEIGHTED) {
        for (int n = tid; n < count; n += kEmbThreads) {
            const float nm = token_norms[(size_t)b * seq + vpos[n]];
            wts[n] = (nm != 0.0f) ? __fdiv_rn(1.0f, nm) : 1.0f;
        }
        __syncthreads();
    }

    // sum of the kept token rows, token order, eight independent loads in flight per thread
    for (int k = tid; k < dim; k += kEmbThreads) {
        float acc = 0.0f;
        int t = 0;
        for (; t + 8 <= count; t += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __half2float(table[(size_t)valid[t + u] * dim + k]);
#pragma unroll
            for (int u = 0; u < 8; ++u) acc = WEIGHTED ? fmaf(wts[t + u], v[u], acc) : __fadd_rn(acc, v[u]);
        }
        for (; t < count; ++t) {
            const float v = __half2float(table[(size_t)valid[t] * dim + k]);
            acc = WEIGHTED ? fmaf(wts[t], v, acc) : __fadd_rn(acc, v);
        }
        hsum[k] = acc;
    }
    __syncthreads();

    float pooled[kEmbColsPerThread];
    double ss = 0.0;
    const float inv = count > 0 ? __fdiv_rn(1.0f, (float)count) : 0.0f;
    if ((out_dim & 7) == 0) {
        // The [1, dim] x [dim, out_dim] product, split over the warps by k: warp w takes k = w, w + 8, ...; a lane owns eight
        // consecutive columns per group of 256 (one 16-byte load per k and group, a warp's loads contiguous), eight k in
        // flight: 128 bytes per thread, 32 KB per SM.  The eight partial rows meet in shared memory and are added in warp
        // order.  (One column per thread with a serial walk over k kept only eight 2-byte loads in flight per thread, and
        // four 8-byte loads were hardly better: 50 us of latency per batch element either way.)
        float* part = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(wts + seq) + 15) & ~(uintptr_t)15);   // [8][out_dim], 16-byte aligned
        const int lane = tid & 31, warp = tid >> 5;
        constexpr int kWarps = kEmbThreads / 32;
        constexpr int kGroups = kEmbThreads * kEmbColsPerThread / 256;   // column groups of 256 at the widest projection
        float acc[kGroups][8];
#pragma unroll
        for (int g = 0; g < kGroups; ++g)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[g][e] = 0.0f;
        const int groups = (out_dim + 255) / 256;
        for (int k0 = warp; k0 < dim; k0 += 8 * kWarps) {
#pragma unroll
            for (int g = 0; g < kGroups; ++g) {
                if (g < groups) {
                    const int c = g * 256 + lane * 8;
                    uint4 pv[8];
                    float hv[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int k = k0 + u * kWarps;
                        const bool in = k < dim && c < out_dim;
                        pv[u] = in ? __ldg(reinterpret_cast<const uint4*>(proj + (size_t)k * out_dim + c)) : make_uint4(0u, 0u, 0u, 0u);
                        hv[u] = (k < dim) ? hsum[k] : 0.0f;
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const uint32_t w4[4] = {pv[u].x, pv[u].y, pv[u].z, pv[u].w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 p2 = __half22float2(*reinterpret_cast<const __half2*>(&w4[e]));
                            acc[g][2 * e] = fmaf(hv[u], p2.x, acc[g][2 * e]);
                            acc[g][2 * e + 1] = fmaf(hv[u], p2.y, acc[g][2 * e + 1]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int g = 0; g < kGroups; ++g) {
            const int c = g * 256 + lane * 8;
            if (g < groups && c < out_dim) {
                float4* dst = reinterpret_cast<float4*>(part + (size_t)warp * out_dim + c);
                dst[0] = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
                dst[1] = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
            }
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < kEmbColsPerThread; ++j) {
            const int c = tid + j * kEmbThreads;
            float a = 0.0f;
            if (c < out_dim) {
#pragma unroll
                for (int w = 0; w < kEmbThreads / 32; ++w) a = __fadd_rn(a, part[(size_t)w * out_dim + c]);
            }
            pooled[j] = __fmul_rn(a, inv);
            ss = __dadd_rn(ss, __dmul_rn((double)pooled[j], (double)pooled[j]));  // columns past out_dim hold 0
        }
    } else {
#pragma unroll
        for (int j = 0; j < kEmbColsPerThread; ++j) {
            const int c = tid + j * kEmbThreads;
            float acc = 0.0f;
            if (c < out_dim) {
                int k = 0;
                for (; k + 8 <= dim; k += 8) {
                    float p[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) p[u] = __half2float(proj[(size_t)(k + u) * out_dim + c]);
#pragma unroll
                    for (int u = 0; u < 8; ++u) acc = fmaf(hsum[k + u], p[u], acc);
                }
                for (; k < dim; ++k) acc = fmaf(hsum[k], __half2float(proj[(size_t)k * out_dim + c]), acc);
            }
            pooled[j] = __fmul_rn(acc, inv);
            ss = __dadd_rn(ss, __dmul_rn((double)pooled[j], (double)pooled[j]));  // columns past out_dim hold 0
        }
    }
    const float norm = WEIGHTED ? 0.0f : __double2float_rn(__dsqrt_rn(block_sum(ss, s_part)));   // 0: values stay as they are
#pragma unroll
    for (int j = 0; j < kEmbColsPerThread; ++j) {
        const int c = tid + j * kEmbThreads;
        if (c >= out_dim) continue;
        const float v = (norm != 0.0f) ? __fdiv_rn(pooled[j], norm) : pooled[j];
        if (out_f32) out_f32[(size_t)b * out_dim + c] = v;
        if (out_f16) out_f16[(size_t)b * out_dim + c] = __float2half_rn(v);
    }
}

// mean_pool(normalize(gather(table, tokens) @ proj), mask).  One CTA per batch element; kept tokens are processed in
// order, sixteen at a time: their embedding rows are staged in shared memory as f32 and every thread walks k once per
// group for each of its output columns.
__global__ void __launch_bounds__(kEmbThreads) embed_normalize_first_kernel(const __half* __restrict__ table, int vocab, int dim,
                                                                            const __half* __restrict__ proj, int out_dim,
                                                                            const int32_t* __restrict__ tokens,
                                                                            const int32_t* __restrict__ mask, int seq,
                                                                            float* __restrict__ out_f32, __half* __restrict__ out_f16,
                                                                            int32_t* __restrict__ bad_token,
                                                                            uint32_t* __restrict__ bad_flag) {
    extern __shared__ __align__(16) unsigned char emb_smem[];
    float* h = reinterpret_cast<float*>(emb_smem);                                        // [kEmbRows][dim]
    float* proj_rows = h + (size_t)kEmbRows * dim;                                        // [kEmbRows][out_dim]
    int32_t* valid = reinterpret_cast<int32_t*>(proj_rows + (size_t)kEmbRows * out_dim);  // [seq]
    __shared__ int s_count;
    __shared__ float s_norm[kEmbRows];

    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid < 32) count_valid_tokens(tokens + (size_t)b * seq, mask + (size_t)b * seq, seq, vocab, valid, &s_count, bad_token, bad_flag);
    __syncthreads();
    const int count = s_count;
    float pooled[kEmbColsPerThread];
#pragma unroll
    for (int j = 0; j < kEmbColsPerThread; ++j) pooled[j] = 0.0f;

    for (int g0 = 0; g0 < count; g0 += kEmbRows) {
        const int rows = min(kEmbRows, count - g0);
        for (int i = tid; i < kEmbRows * dim; i += kEmbThreads) {
            const int r = i / dim, k = i % dim;
            h[i] = (r < rows) ? __half2float(table[(size_t)valid[g0 + r] * dim + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll 1
        for (int j = 0; j < kEmbColsPerThread; ++j) {
            const int c = tid + j * kEmbThreads;
            if (c >= out_dim) break;
            float sums[kEmbRows];
#pragma unroll
            for (int r = 0; r < kEmbRows; ++r) sums[r] = 0.0f;
            int k = 0;
            if ((dim & 3) == 0) {  // four k per shared-memory read of each staged row, the next four prefetched
                float p[4], pn[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) p[u] = __half2float(proj[(size_t)u * out_dim + c]);
                for (; k < dim; k += 4) {
                    const int kn = (k + 4 < dim) ? k + 4 : k;
#pragma unroll
                    for (int u = 0; u < 4; ++u) pn[u] = __half2float(proj[(size_t)(kn + u) * out_dim + c]);
#pragma unroll
                    for (int r = 0; r < kEmbRows; ++r) {
                        const float4 hv = *reinterpret_cast<const float4*>(h + r * dim + k);
                        sums[r] = __fadd_rn(sums[r], __fmul_rn(hv.x, p[0]));
                        sums[r] = __fadd_rn(sums[r], __fmul_rn(hv.y, p[1]));
                        sums[r] = __fadd_rn(sums[r], __fmul_rn(hv.z, p[2]));
                        sums[r] = __fadd_rn(sums[r], __fmul_rn(hv.w, p[3]));
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) p[u] = pn[u];
                }
            }
            for (; k < dim; ++k) {
                const float p = __half2float(proj[(size_t)k * out_dim + c]);
#pragma unroll
                for (int r = 0; r < kEmbRows; ++r) sums[r] = __fadd_rn(sums[r], __fmul_rn(h[r * dim + k], p));
            }
#pragma unroll
            for (int r = 0; r < kEmbRows; ++r) proj_rows[(size_t)r * out_dim + c] = sums[r];
        }
        __syncthreads();
        // norm of each projected row: warp w handles rows w, w + 8
        for (int r = warp; r < kEmbRows; r += kEmbThreads / 32) {
            double ss = 0.0;
            for (int c = lane; c < out_dim; c += 32) {
                const double v = (double)proj_rows[(size_t)r * out_dim + c];
                ss = __dadd_rn(ss, __dmul_rn(v, v));
            }
            for (int off = 16; off > 0; off >>= 1) ss = __dadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, off));
            if (lane == 0) s_norm[r] = __double2float_rn(__dsqrt_rn(ss));
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < kEmbColsPerThread; ++j) {
            const int c = tid + j * kEmbThreads;
            if (c >= out_dim) continue;
            for (int r = 0; r < rows; ++r) {
                float v = proj_rows[(size_t)r * out_dim + c];
                if (s_norm[r] != 0.0f) v = __fdiv_rn(v, s_norm[r]);
                pooled[j] = __fadd_rn(pooled[j], v);
            }
        }
        __syncthreads();
    }
    const float inv = count > 0 ? __fdiv_rn(1.0f, (float)count) : 0.0f;
#pragma unroll
    for (int j = 0; j < kEmbColsPerThread; ++j) {
        const int c = tid + j * kEmbThreads;
        if (c >= out_dim) continue;
        const float v = __fmul_rn(pooled[j], inv);
        if (out_f32) out_f32[(size_t)b * out_dim + c] = v;
        if (out_f16) out_f16[(size_t)b * out_dim + c] = __float2half_rn(v);
    }
}

cudaError_t launch_embed_pooled(cudaStream_t st, const void* table_f16, int vocab, int dim, const void* proj_f16, int out_dim,
                                const int32_t* d_tokens, const int32_t* d_mask, int batch, int seq, int order,
                                const float* d_token_norms, float* d_out_f32, void* d_out_f16, int32_t* d_bad_token,
                                uint32_t* d_bad_flag) {
    if (out_dim > kEmbThreads * kEmbColsPerThread) return cudaErrorInvalidValue;
    const bool weighted = order != 0 && d_token_norms != nullptr;
    // pool-first kernel: token-row sum [dim], kept tokens, their positions and weights ([seq] each), eight partial rows
    const size_t smem = (weighted || order == 0) ? (size_t)dim * 4 + (size_t)seq * 12 + (size_t)(kEmbThreads / 32) * out_dim * 4 + 16
                                                 : (size_t)kEmbRows * dim * 4 + (size_t)kEmbRows * out_dim * 4 + (size_t)seq * 4;
    constexpr size_t kMaxSmem = 220 * 1024;
    if (smem > kMaxSmem) return cudaErrorInvalidValue;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(embed_pool_first_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxSmem);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(embed_pool_first_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxSmem);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(embed_normalize_first_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxSmem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const __half* table = (const __half*)table_f16;
    const __half* proj = (const __half*)proj_f16;
    if (weighted)
        embed_pool_first_kernel<true><<<batch, kEmbThreads, smem, st>>>(table, vocab, dim, proj, out_dim, d_tokens, d_mask, seq,
                                                                      d_token_norms, d_out_f32, (__half*)d_out_f16, d_bad_token, d_bad_flag);
    else if (order == 0)
        embed_pool_first_kernel<false><<<batch, kEmbThreads, smem, st>>>(table, vocab, dim, proj, out_dim, d_tokens, d_mask, seq, nullptr,
                                                                       d_out_f32, (__half*)d_out_f16, d_bad_token, d_bad_flag);
    else
        embed_normalize_first_kernel<<<batch, kEmbThreads, smem, st>>>(table, vocab, dim, proj, out_dim, d_tokens, d_mask, seq, d_out_f32,
                                                                     (__half*)d_out_f16, d_bad_token, d_bad_flag);
    count_launch();
    return cudaGetLastError();
}

}  // namespace mb200
