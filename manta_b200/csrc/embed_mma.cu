// The per-token projection of the normalize-first embedding order, mean_pool(normalize(gather(table, tokens) @ P)), on
// the tensor cores.  The reference runs that product as an SGEMM over every token row (runtime/backends/cuda/
// native_linux.go:509-549) and normalises each projected row (runtime/backend/tensor_ops.go:1114-1138).
//
// The pool that follows is linear, so only ONE number per token is needed from the big product: the norm of the token's
// projected row.  mean_pool(normalize(Y)) = (1/count) * sum_t y_t / |y_t| = (1/count) * (sum_t a_t / |y_t|) @ P, where a_t
// is the token's embedding row and y_t = a_t @ P.  This file computes |y_t| for every token with tcgen05.mma
// ([128 tokens] x [dim] x [out_dim] per CTA, f16 operands, f32 accumulators in tensor memory) and reads the accumulators
// back only to square and add them; embed.cu then pools the embedding rows with the weights 1/|y_t| and projects one
// row per batch element.
//
// One CTA per 128 tokens, 160 threads: warps 0..3 stage the operands (thread t owns token row t: it gathers the row's
// 128-byte K chunk from the table and copies its share of the projection chunk, both into the 128-byte-swizzled K-major
// layout the tensor core reads) and afterwards read back tensor-memory lanes 32w..32w+31; warp 4 owns the tensor-memory
// allocation and issues the MMAs.  Every wait is bounded; a wait that runs out raises the time-out value in the
// embedder's flag word, every role leaves, tensor memory is released and the kernel returns.
#include "kernels.h"
#include "tc.cuh"

namespace mb200 {

namespace {

constexpr int kTokRows = 128;          // tokens per CTA = M of the MMA
constexpr int kKChunk = 64;            // f16 elements per K chunk = one 128-byte swizzle span
constexpr int kNfThreads = 160;
constexpr int kStageWarps = 4;
constexpr size_t kNfSmemLimit = 232448 - 2048;

struct NormArgs {
    const __half* table;     // [vocab][dim]
    const __half* proj_t;    // [out_dim][dim]: the projection, transposed (K-major rows)
    const int32_t* tokens;   // [n_tokens]
    float* norms;            // [n_tokens]
    uint32_t* flag;          // embedder flag word: 2 = a wait ran out
    int vocab, dim, out_dim, n_tokens, stages;
};

__global__ void __launch_bounds__(kNfThreads, 1) embed_token_norms_kernel(const NormArgs a) {
    extern __shared__ __align__(1024) unsigned char nf_smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = a.stages;
    const int kchunks = a.dim / kKChunk;
    const uint32_t a_bytes = kTokRows * 128, b_bytes = (uint32_t)a.out_dim * 128;
    const uint32_t stage_bytes = a_bytes + b_bytes;
    unsigned char* base = (unsigned char*)(((uintptr_t)nf_smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* p = base + (size_t)S * stage_bytes;
    uint64_t* full = (uint64_t*)p;
    uint64_t* empty = full + 4;
    uint64_t* acc_full = empty + 4;
    uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
    volatile uint32_t* abort_s = tmem_slot + 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], kStageWarps);   // one arrival per staging warp
            mbar_init(&empty[s], 1);            // the MMAs that read the stage have completed
        }
        mbar_init(acc_full, 1);
        *abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) tmem_alloc(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int64_t tok0 = (int64_t)blockIdx.x * kTokRows;

    if (warp < kStageWarps) {
        // ---------------- operand staging, then the read-back ----------------
        const int t = threadIdx.x;   // row of the tile
        const int64_t ti = tok0 + t;
        int32_t tok = (ti < a.n_tokens) ? a.tokens[ti] : 0;
        tok = min(max(tok, 0), a.vocab - 1);   // an out-of-range token is reported by the pooling kernel; here it must only not fault
        const unsigned char* arow = reinterpret_cast<const unsigned char*>(a.table + (size_t)tok * a.dim);
        const unsigned char* pt = reinterpret_cast<const unsigned char*>(a.proj_t);
        const size_t prow_bytes = (size_t)a.dim * 2;
        bool ok = true;
        for (int kc = 0; kc < kchunks && ok; ++kc) {
            const int s = kc % S;
            if (!mbar_wait(&empty[s], (((uint32_t)(kc / S)) & 1u) ^ 1u, abort_s)) { ok = false; break; }
            unsigned char* sa = base + (size_t)s * stage_bytes;
            unsigned char* sb = sa + a_bytes;
            // A: this thread's token row, eight 16-byte pieces, piece j at (j ^ (row % 8)) within the row's 128 bytes
            uint4 va[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) va[j] = __ldg(reinterpret_cast<const uint4*>(arow + (size_t)kc * 128) + j);
#pragma unroll
            for (int j = 0; j < 8; ++j) *reinterpret_cast<uint4*>(sa + (size_t)t * 128 + ((j ^ (t & 7)) << 4)) = va[j];
            // B: out_dim rows of 128 bytes; consecutive threads take consecutive 16-byte pieces (coalesced in global memory)
            const int pieces = a.out_dim * 8;
            for (int i0 = t; i0 < pieces; i0 += 8 * kTokRows) {
                uint4 vb[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = i0 + u * kTokRows;
                    vb[u] = (i < pieces) ? __ldg(reinterpret_cast<const uint4*>(pt + (size_t)(i >> 3) * prow_bytes + (size_t)kc * 128) + (i & 7))
                                         : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = i0 + u * kTokRows;
                    const int r = i >> 3, j = i & 7;
                    if (i < pieces) *reinterpret_cast<uint4*>(sb + (size_t)r * 128 + ((j ^ (r & 7)) << 4)) = vb[u];
                }
            }
            // generic-proxy stores -> visible to the tensor core's async proxy, then one arrival per warp
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
        }
        if (ok && mbar_wait(acc_full, 0u, abort_s)) {
            tc_fence_after();
            // lane t of tensor memory holds token row t: f64 sum of squares of its out_dim f32 values, f32 square root
            const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
            double ss = 0.0;
            for (int c0 = 0; c0 < a.out_dim; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(taddr + (uint32_t)c0, v);
                tmem_ld_wait();
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    const double x = (double)__uint_as_float(v[u]);
                    ss = fma(x, x, ss);
                }
            }
            if (ti < a.n_tokens) a.norms[ti] = __double2float_rn(__dsqrt_rn(ss));
        }
    } else if (lane == 0) {
        // ---------------- MMA issuer ----------------
        // out_dim columns as one instruction of up to 256 columns and, past that, a second one for the rest
        const int n1 = min(a.out_dim, 256), n2 = a.out_dim - n1;
        const uint32_t idesc1 = (1u << 4) | ((uint32_t)(n1 >> 3) << 17) | ((uint32_t)(kTokRows >> 4) << 24);   // f16 x f16 -> f32, K-major both
        const uint32_t idesc2 = (1u << 4) | ((uint32_t)(n2 >> 3) << 17) | ((uint32_t)(kTokRows >> 4) << 24);
        bool ok = true;
        for (int kc = 0; kc < kchunks; ++kc) {
            const int s = kc % S;
            if (!mbar_wait(&full[s], ((uint32_t)(kc / S)) & 1u, abort_s)) { ok = false; break; }
            tc_fence_after();
            const uint32_t a_addr = smem_u32(base + (size_t)s * stage_bytes);
            const uint32_t b_addr = a_addr + a_bytes;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {   // 16 f16 = 32 bytes of K per instruction
                const uint32_t acc = (kc > 0 || ks > 0) ? 1u : 0u;
                tc_mma<false>(tmem_base, smem_desc_sw128(a_addr + ks * 32), smem_desc_sw128(b_addr + ks * 32), idesc1, acc);
                if (n2 > 0)
                    tc_mma<false>(tmem_base + (uint32_t)n1, smem_desc_sw128(a_addr + ks * 32),
                                  smem_desc_sw128(b_addr + (uint32_t)n1 * 128 + ks * 32), idesc2, acc);
            }
            tc_commit(&empty[s]);
        }
        if (ok) tc_commit(acc_full);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *abort_s) atomicMax(a.flag, 2u);
}

// [dim][out_dim] -> [out_dim][dim], once per bound embedder.
__global__ void __launch_bounds__(256) transpose_f16_kernel(const __half* __restrict__ src, int rows, int cols, __half* __restrict__ dst) {
    __shared__ __half tile[32][33];
    const int bx = blockIdx.x * 32, by = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int j = ty; j < 32; j += 8)
        if (by + j < rows && bx + tx < cols) tile[j][tx] = src[(size_t)(by + j) * cols + bx + tx];
    __syncthreads();
    for (int j = ty; j < 32; j += 8)
        if (bx + j < cols && by + tx < rows) dst[(size_t)(bx + j) * rows + by + tx] = tile[tx][j];
}

}  // namespace

bool embed_mma_supported(int dim, int out_dim) {
    return dim >= kKChunk && dim % kKChunk == 0 && out_dim >= 16 && out_dim % 16 == 0 && out_dim <= 512;
}

cudaError_t launch_transpose_f16(cudaStream_t st, const void* src, int rows, int cols, void* dst) {
    dim3 grid((cols + 31) / 32, (rows + 31) / 32);
    transpose_f16_kernel<<<grid, 256, 0, st>>>((const __half*)src, rows, cols, (__half*)dst);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_embed_token_norms(cudaStream_t st, const void* table_f16, int vocab, int dim, const void* proj_t_f16, int out_dim,
                                     const int32_t* d_tokens, int64_t n_tokens, float* d_norms, uint32_t* d_flag) {
    if (!embed_mma_supported(dim, out_dim) || n_tokens <= 0 || n_tokens > (int64_t)kTokRows * 0x7fffff) return cudaErrorInvalidValue;
    NormArgs a;
    a.table = (const __half*)table_f16;
    a.proj_t = (const __half*)proj_t_f16;
    a.tokens = d_tokens;
    a.norms = d_norms;
    a.flag = d_flag;
    a.vocab = vocab;
    a.dim = dim;
    a.out_dim = out_dim;
    a.n_tokens = (int)n_tokens;
    const size_t stage = (size_t)kTokRows * 128 + (size_t)out_dim * 128;
    int stages = (int)((kNfSmemLimit - 1024 - 256) / stage);
    stages = stages > 4 ? 4 : stages;
    if (stages < 2) return cudaErrorInvalidValue;
    a.stages = stages;
    const size_t smem = 1024 + (size_t)stages * stage + 256;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(embed_token_norms_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kNfSmemLimit);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const int grid = (int)((n_tokens + kTokRows - 1) / kTokRows);
    embed_token_norms_kernel<<<grid, kNfThreads, smem, st>>>(a);
    count_launch();
    return cudaGetLastError();
}

}  // namespace mb200
