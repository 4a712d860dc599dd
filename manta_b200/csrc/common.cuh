// Shared declarations of the score/select kernels: parameter blocks, key encoding, small device helpers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/manta_b200.h"

namespace mb200 {

constexpr int kMaxK = 2048;          // largest k the fused pass accepts
constexpr int kMaxCols = 8192;       // largest row width (elements)
constexpr int kThreads = 256;        // threads per CTA of the streaming kernels
constexpr int kWarpsPerCta = kThreads / 32;

// ---- ordering -------------------------------------------------------------------------------------
// A candidate is ranked by "goodness" g: g = score for LARGEST, g = -score for SMALLEST.  ord(g) is a
// monotone map float -> uint32 (0 is below every finite value and marks "empty").  The 64-bit key
// (ord(g) << 32) | ~id is unique per row and orders by goodness descending, then id ascending, which is
// the comparator of topKTensor.
__host__ __device__ inline uint32_t ord_from_float(float g) {
    uint32_t u = __builtin_bit_cast(uint32_t, g);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__host__ __device__ inline float float_from_ord(uint32_t o) {
    uint32_t u = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
    return __builtin_bit_cast(float, u);
}
__host__ __device__ inline uint64_t make_key(float g, int32_t id) {
    return ((uint64_t)ord_from_float(g) << 32) | (uint64_t)(~(uint32_t)id);
}
__host__ __device__ inline int32_t key_id(uint64_t key) { return (int32_t)(~(uint32_t)(key & 0xffffffffu)); }
__host__ __device__ inline float key_goodness(uint64_t key) { return float_from_ord((uint32_t)(key >> 32)); }

// ---- per-query constants produced by the query-prep kernel -----------------------------------------
struct QueryHeader {
    float s_hi;   // scale of the high int8 plane (q8/q4 candidates)
    float s_lo;   // scale of the low int8 plane
    float qn;     // ||q|| (f32 of the f64 root)
    float qinv;   // 1/||q|| (f32 division), 0 for a zero query
    double qn2d;  // ||q||^2 in f64
    double qhat2; // ||s_hi*hi + s_lo*lo||^2 in f64: the squared norm of the query the int8 planes represent
};

// ---- selection workspace ------------------------------------------------------------------------------
// Per query: pool of candidate keys (append-only within a pass), its fill count, the current filter
// threshold (ord space, only ever raised) and one running maximum per bucket (a bucket is a disjoint
// subset of rows; the k-th largest bucket maximum is a valid lower bound of the k-th best score).
struct SelectWs {
    uint64_t* pool;       // [nq][cap]
    uint32_t* count;      // [nq]
    uint32_t* thr;        // [nq]
    uint32_t* bucket;     // [nq][nb]
    uint32_t* flags;      // [0] pool overflow, [1] bounded wait gave up, [2] internal check failed, [3] a peer's list is incomplete
    uint32_t cap;
    uint32_t nb;
};

enum { kFlagOverflow = 0, kFlagTimeout = 1, kFlagInternal = 2, kFlagPeerOverflow = 3, kNumFlags = 4 };

struct CandView {
    const uint8_t* data;     // packed rows
    const void* scales;      // f32 per row (q8) or f16 per block (q4); null for f16
    const void* stats;       // per row: int32 sum code^2 (q8) or f32 sum value^2 (q4, f16)
    int64_t rows;
    int64_t row_base;
    int cols;
    int row_bytes;           // stride between rows in data
    int chunks;              // 16-byte chunks per row that carry data
    int layout;
};

// score epilogues -----------------------------------------------------------------------------------------
// Cosine is finished as t * (qinv * rinv): qinv = 1/||q|| once per query, rinv = 1/||d|| once per row, so a score
// costs multiplications only; either factor is 0 for a zero vector, which yields exactly 0 as the reference does.
// Every operation below is a single correctly rounded IEEE operation in a fixed order, so a CPU model can
// reproduce the bits.

// q8 rows: 1/sqrt(sum code^2) (0 for an all-zero row); the row scale cancels out of the cosine.
__device__ __forceinline__ float q8_row_inv_norm(int nn) {
    return (nn > 0) ? __frcp_rn(__fsqrt_rn((float)nn)) : 0.0f;
}
// f16 / q4 rows: 1/sqrt(||d||^2) from the bind-time statistic.
__device__ __forceinline__ float float_row_inv_norm(float dn2) {
    return (dn2 > 0.0f) ? __frcp_rn(__fsqrt_rn(dn2)) : 0.0f;
}

// q8: t = s_hi*I_hi + s_lo*I_lo is q . codes (without the row scale).  rinv is used by cosine only, nn and sd by
// l2 (sd also by dot).
__device__ __forceinline__ float q8_finish(int metric, int ih, int il, int nn, float rinv, float sd, const QueryHeader& h) {
    float a = __fmul_rn((float)ih, h.s_hi);
    float t = __fmaf_rn((float)il, h.s_lo, a);
    float res;
    if (metric == MANTA_B200_METRIC_DOT) {
        res = __fmul_rn(t, sd);
    } else if (metric == MANTA_B200_METRIC_COSINE) {
        res = __fmul_rn(t, __fmul_rn(h.qinv, rinv));
    } else {
        // ||qhat - d||^2 = ||qhat||^2 + ||d||^2 - 2 qhat.d, combined in f64 so that the cancellation near zero
        // distance costs nothing; qhat is the query the two planes represent (|qhat - q| <= s_lo/2 per element).
        double td = __dadd_rn(__dmul_rn((double)ih, (double)h.s_hi), __dmul_rn((double)il, (double)h.s_lo));
        double dotd = __dmul_rn(td, (double)sd);
        double dn2d = __dmul_rn(__dmul_rn((double)sd, (double)sd), (double)nn);
        double x = __dadd_rn(__dadd_rn(h.qhat2, dn2d), -__dmul_rn(2.0, dotd));
        res = __double2float_rn(__dsqrt_rn(fmax(x, 0.0)));
    }
    return res + 0.0f;  // -0 -> +0 so equal scores have equal bits
}

// float layouts (f16, q4): dotv = q . d, dn2 = ||d||^2 from the bind-time statistics (rinv its inverse root, used
// by cosine only), q2 = squared norm of the query as the kernel sees it (f64).  The l2 combination runs in f64;
// dotv and dn2 carry f32 rounding.
__device__ __forceinline__ float float_finish(int metric, float dotv, float dn2, float rinv, const QueryHeader& h, double q2) {
    float res;
    if (metric == MANTA_B200_METRIC_DOT) {
        res = dotv;
    } else if (metric == MANTA_B200_METRIC_COSINE) {
        res = __fmul_rn(dotv, __fmul_rn(h.qinv, rinv));
    } else {
        double x = __dadd_rn(__dadd_rn(q2, (double)dn2), -__dmul_rn(2.0, (double)dotv));
        res = __double2float_rn(__dsqrt_rn(fmax(x, 0.0)));
    }
    return res + 0.0f;
}

__device__ __forceinline__ uint32_t ld_relaxed_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ void st_relaxed_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v));
}

}  // namespace mb200
