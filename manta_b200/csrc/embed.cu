// Embedding front end of the score path on the device: gather(token_embedding, tokens) -> @matmul(projection) ->
// masked mean_pool / normalize, producing the f16 query batch the scoring kernels consume without a host hop.
// Arithmetic follows the reference's host math (runtime/backend/tensor_ops.go:981-1011 matmul: f32 products and
// sums rounded separately, k ascending; :1210-1275 masked mean pool: rows added in order, times 1/count;
// :1114-1138 normalize: f64 sum of squares, f32 norm, f32 divide, zero rows untouched).
#include "kernels.h"

namespace mb200 {

constexpr int kEmbThreads = 256;
constexpr int kEmbRows = 8;      // token rows multiplied per pass over the projection matrix
constexpr int kEmbColsPerThread = 4;

// One CTA per batch element.  Thread t owns output columns t, t+256, ...  Valid tokens are processed in order, eight
// at a time: their embedding rows are staged in shared memory as f32 and every thread walks k once per group.
__global__ void __launch_bounds__(kEmbThreads) embed_pooled_kernel(const __half* __restrict__ table, int vocab, int dim,
                                                                   const __half* __restrict__ proj, int out_dim,
                                                                   const int32_t* __restrict__ tokens,
                                                                   const int32_t* __restrict__ mask, int seq, int order,
                                                                   float* __restrict__ out_f32, __half* __restrict__ out_f16,
                                                                   int32_t* __restrict__ bad_token, uint32_t* __restrict__ bad_flag) {
    extern __shared__ __align__(16) unsigned char emb_smem[];
    float* h = reinterpret_cast<float*>(emb_smem);            // [kEmbRows][dim]
    float* proj_rows = h + (size_t)kEmbRows * dim;            // [kEmbRows][out_dim] (order 1) / pooled (order 0)
    int32_t* valid = reinterpret_cast<int32_t*>(proj_rows + (size_t)kEmbRows * out_dim);  // [seq] token ids of valid positions
    __shared__ int s_count;
    __shared__ float s_norm[kEmbRows];
    __shared__ double s_part[kEmbThreads / 32];

    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        int n = 0;
        for (int t = 0; t < seq; ++t) {
            const int32_t tok = tokens[(size_t)b * seq + t];
            if (tok < 0 || tok >= vocab) {  // the reference's gather rejects it whether or not the mask keeps it
                if (atomicExch(bad_flag, 1u) == 0u) *bad_token = tok;
                continue;
            }
            if (mask[(size_t)b * seq + t] != 0) valid[n++] = tok;
        }
        s_count = n;
    }
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
#pragma unroll
        for (int j = 0; j < kEmbColsPerThread; ++j) {
            const int c = tid + j * kEmbThreads;
            if (c >= out_dim) continue;
            float sums[kEmbRows];
#pragma unroll
            for (int r = 0; r < kEmbRows; ++r) sums[r] = 0.0f;
            int k = 0;
            if ((dim & 3) == 0) {  // four k per shared-memory read of each staged row
                for (; k < dim; k += 4) {
                    float p[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) p[u] = __half2float(proj[(size_t)(k + u) * out_dim + c]);
#pragma unroll
                    for (int r = 0; r < kEmbRows; ++r) {
                        const float4 hv = *reinterpret_cast<const float4*>(h + r * dim + k);
                        sums[r] = __fadd_rn(sums[r], __fmul_rn(hv.x, p[0]));
                        sums[r] = __fadd_rn(sums[r], __fmul_rn(hv.y, p[1]));
                        sums[r] = __fadd_rn(sums[r], __fmul_rn(hv.z, p[2]));
                        sums[r] = __fadd_rn(sums[r], __fmul_rn(hv.w, p[3]));
                    }
                }
            }
            for (; k < dim; ++k) {
                const float p = __half2float(proj[(size_t)k * out_dim + c]);
#pragma unroll
                for (int r = 0; r < kEmbRows; ++r) sums[r] = __fadd_rn(sums[r], __fmul_rn(h[r * dim + k], p));
            }
            if (order == 0) {
#pragma unroll
                for (int r = 0; r < kEmbRows; ++r)
                    if (r < rows) pooled[j] = __fadd_rn(pooled[j], sums[r]);
            } else {
#pragma unroll
                for (int r = 0; r < kEmbRows; ++r) proj_rows[(size_t)r * out_dim + c] = sums[r];
            }
        }
        if (order == 1) {
            // normalize each projected row, then add it to the pool
            __syncthreads();
            if (warp < kEmbRows) {
                double ss = 0.0;
                for (int c = lane; c < out_dim; c += 32) {
                    const double v = (double)proj_rows[(size_t)warp * out_dim + c];
                    ss = __dadd_rn(ss, __dmul_rn(v, v));
                }
                for (int off = 16; off > 0; off >>= 1) ss = __dadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, off));
                if (lane == 0) s_norm[warp] = __double2float_rn(__dsqrt_rn(ss));
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
        }
        __syncthreads();
    }
    if (count > 0) {
        const float inv = __fdiv_rn(1.0f, (float)count);
#pragma unroll
        for (int j = 0; j < kEmbColsPerThread; ++j) pooled[j] = __fmul_rn(pooled[j], inv);
    }
    float norm = 0.0f;
    if (order == 0) {
        double ss = 0.0;
#pragma unroll
        for (int j = 0; j < kEmbColsPerThread; ++j) {
            const int c = tid + j * kEmbThreads;
            if (c < out_dim) ss = __dadd_rn(ss, __dmul_rn((double)pooled[j], (double)pooled[j]));
        }
        for (int off = 16; off > 0; off >>= 1) ss = __dadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, off));
        if (lane == 0) s_part[warp] = ss;
        __syncthreads();
        double tot = 0.0;
        for (int w = 0; w < kEmbThreads / 32; ++w) tot = __dadd_rn(tot, s_part[w]);
        norm = __double2float_rn(__dsqrt_rn(tot));
    }
#pragma unroll
    for (int j = 0; j < kEmbColsPerThread; ++j) {
        const int c = tid + j * kEmbThreads;
        if (c >= out_dim) continue;
        float v = pooled[j];
        if (order == 0 && norm != 0.0f) v = __fdiv_rn(v, norm);
        if (out_f32) out_f32[(size_t)b * out_dim + c] = v;
        if (out_f16) out_f16[(size_t)b * out_dim + c] = __float2half_rn(v);
    }
}

size_t embed_smem_bytes(int dim, int out_dim, int seq) {
    return (size_t)kEmbRows * dim * 4 + (size_t)kEmbRows * out_dim * 4 + (size_t)seq * 4;
}

cudaError_t launch_embed_pooled(cudaStream_t st, const void* table_f16, int vocab, int dim, const void* proj_f16, int out_dim,
                                const int32_t* d_tokens, const int32_t* d_mask, int batch, int seq, int order, float* d_out_f32,
                                void* d_out_f16, int32_t* d_bad_token, uint32_t* d_bad_flag) {
    if (out_dim > kEmbThreads * kEmbColsPerThread) return cudaErrorInvalidValue;
    const size_t smem = embed_smem_bytes(dim, out_dim, seq);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(embed_pooled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    embed_pooled_kernel<<<batch, kEmbThreads, smem, st>>>((const __half*)table_f16, vocab, dim, (const __half*)proj_f16, out_dim,
                                                        d_tokens, d_mask, seq, order, d_out_f32, (__half*)d_out_f16, d_bad_token,
                                                        d_bad_flag);
    count_launch();
    return cudaGetLastError();
}

}  // namespace mb200
