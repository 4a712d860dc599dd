/*
 * manta_oracle.c -- CPU restatement of the reference's host math for the score/select path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links or calls this file; it is the
 * checker that the GPU parity tests, the smoke test and the bench's cpu_baseline leg compare
 * against.  Parity is pinned: the functions below are checked against the reference's own
 * known-answer fixtures (runtime/backend/tensor_ops_test.go:537-684,
 * runtime/runtime_test.go:483-586) by tests/test_oracle_golden.py.
 *
 * Every function cites the reference file:line it follows (paths inside odvcencio/manta).
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (Go on amd64 never fuses a*b+c, so
 * contraction must stay off).  Rows are independent in the reference loops, so OpenMP splits
 * across rows only; the per-row arithmetic order is the reference's.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define MO_OK 0
#define MO_ERR_SHAPE 1
#define MO_ERR_RANGE 2

int mo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void mo_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ---- half <-> float -------------------------------------------------------------------- */

/* runtime/weight_file.go:388-410 (halfToFloat32): exact widening, subnormals normalised. */
float mo_half_to_float(uint16_t bits) {
    uint32_t sign = ((uint32_t)(bits & 0x8000u)) << 16;
    uint32_t exp = (bits >> 10) & 0x1fu;
    uint32_t mant = bits & 0x03ffu;
    uint32_t out;
    if (exp == 0) {
        if (mant == 0) {
            out = sign;
        } else {
            uint32_t exp32 = 127 - 15 + 1;
            while ((mant & 0x0400u) == 0) {
                mant <<= 1;
                exp32--;
            }
            mant &= 0x03ffu;
            out = sign | (exp32 << 23) | (mant << 13);
        }
    } else if (exp == 0x1f) {
        out = sign | 0x7f800000u | (mant << 13);
    } else {
        out = sign | ((exp + (127 - 15)) << 23) | (mant << 13);
    }
    float f;
    memcpy(&f, &out, 4);
    return f;
}

/* f32 -> f16 round-to-nearest-even.  The reference only narrows on disk export
 * (runtime/mll_export.go:876-914, ties half-up); the score path never narrows, so the canonical
 * inputs of this build are produced with IEEE RNE and their bit patterns are the ground truth. */
uint16_t mo_float_to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | ((absx > 0x7f800000u) ? 0x0200u : 0));
    }
    if (absx >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (absx < 0x33000001u) { /* below half of the smallest subnormal -> 0 */
        return (uint16_t)sign;
    }
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x007fffffu) | 0x00800000u;
    uint32_t shift;
    uint32_t base;
    if (e < -14) { /* subnormal half */
        shift = (uint32_t)(13 + (-14 - e));
        base = 0;
    } else {
        shift = 13;
        base = ((uint32_t)(e + 15) << 10) - 0x0400u; /* implicit bit adds 0x400 */
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q++;
    return (uint16_t)(sign | (base + q));
}

void mo_half_to_float_n(const uint16_t* in, float* out, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) out[i] = mo_half_to_float(in[i]);
}

void mo_float_to_half_n(const float* in, uint16_t* out, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) out[i] = mo_float_to_half(in[i]);
}

/* ---- score builtins ---------------------------------------------------------------------- */

/* runtime/backend/tensor_ops.go:1366-1396 (dotRows): f32 sequential accumulate.
 * queries [batches, cols]; docs [rows, cols] when shared != 0 (every query sees the same rows;
 * the build's extension, equal to `batches` independent rank-1 calls) or
 * [batches, rows, cols] when shared == 0 (the reference's batched form). */
int mo_dot_rows(const float* queries, const float* docs, int64_t batches, int64_t rows, int64_t cols,
                int shared, float* out) {
    if (batches <= 0 || rows < 0 || cols < 0) return MO_ERR_SHAPE;
    for (int64_t b = 0; b < batches; b++) {
        const float* q = queries + b * cols;
        const float* dbase = shared ? docs : docs + b * rows * cols;
#pragma omp parallel for schedule(static)
        for (int64_t r = 0; r < rows; r++) {
            float sum = 0.0f;
            const float* d = dbase + r * cols;
            for (int64_t c = 0; c < cols; c++) sum += q[c] * d[c];
            out[b * rows + r] = sum;
        }
    }
    return MO_OK;
}

/* runtime/backend/tensor_ops.go:1398-1456 (cosineRows): f64 accumulate; query norm once;
 * denom = sqrt(qn)*sqrt(dn); exactly 0 when denom == 0; result narrowed to f32. */
int mo_cosine_rows(const float* queries, const float* docs, int64_t batches, int64_t rows, int64_t cols,
                   int shared, float* out) {
    if (batches <= 0 || rows < 0 || cols < 0) return MO_ERR_SHAPE;
    for (int64_t b = 0; b < batches; b++) {
        const float* q = queries + b * cols;
        const float* dbase = shared ? docs : docs + b * rows * cols;
        double query_norm = 0.0;
        for (int64_t c = 0; c < cols; c++) {
            double v = (double)q[c];
            query_norm += v * v;
        }
#pragma omp parallel for schedule(static)
        for (int64_t r = 0; r < rows; r++) {
            double dot = 0.0, doc_norm = 0.0;
            const float* d = dbase + r * cols;
            for (int64_t c = 0; c < cols; c++) {
                double qq = (double)q[c];
                double dd = (double)d[c];
                dot += qq * dd;
                doc_norm += dd * dd;
            }
            double denom = sqrt(query_norm) * sqrt(doc_norm);
            out[b * rows + r] = (denom == 0.0) ? 0.0f : (float)(dot / denom);
        }
    }
    return MO_OK;
}

/* runtime/backend/tensor_ops.go:1458-1490 (l2DistanceRows): difference in f32, squares summed in
 * f64, root narrowed to f32 (the distance, not its square). */
int mo_l2_rows(const float* queries, const float* docs, int64_t batches, int64_t rows, int64_t cols,
               int shared, float* out) {
    if (batches <= 0 || rows < 0 || cols < 0) return MO_ERR_SHAPE;
    for (int64_t b = 0; b < batches; b++) {
        const float* q = queries + b * cols;
        const float* dbase = shared ? docs : docs + b * rows * cols;
#pragma omp parallel for schedule(static)
        for (int64_t r = 0; r < rows; r++) {
            double sum = 0.0;
            const float* d = dbase + r * cols;
            for (int64_t c = 0; c < cols; c++) {
                volatile float df = q[c] - d[c]; /* force the f32 rounding of the difference */
                double diff = (double)df;
                sum += diff * diff;
            }
            out[b * rows + r] = (float)sqrt(sum);
        }
    }
    return MO_OK;
}

/* ---- topk ------------------------------------------------------------------------------- */

typedef struct {
    int64_t idx;
    float val;
} mo_pair;

/* comparator of runtime/backend/tensor_ops.go:1539-1552: value descending, then index ascending */
static int mo_pair_cmp(const void* pa, const void* pb) {
    const mo_pair* a = (const mo_pair*)pa;
    const mo_pair* b = (const mo_pair*)pb;
    if (a->val > b->val) return -1;
    if (a->val < b->val) return 1;
    if (a->idx < b->idx) return -1;
    if (a->idx > b->idx) return 1;
    return 0;
}

/* runtime/backend/tensor_ops.go:1523-1592 (topKTensor): full sort of (index,value) pairs per row
 * of scores[rows, cols]; first k indices as int32; error when k <= 0 or k > cols.
 * smallest != 0 is the build's extension for "k smallest distance": topKTensor on the negated
 * values (ties still resolved towards the lower index). */
int mo_topk(const float* scores, int64_t rows, int64_t cols, int k, int smallest, int32_t* out_idx) {
    if (k <= 0 || k > cols) return MO_ERR_RANGE;
    int rc = MO_OK;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t r = 0; r < rows; r++) {
        mo_pair* pairs = (mo_pair*)malloc((size_t)cols * sizeof(mo_pair));
        if (!pairs) {
            rc = MO_ERR_RANGE;
            continue;
        }
        const float* s = scores + r * cols;
        for (int64_t c = 0; c < cols; c++) {
            pairs[c].idx = c;
            pairs[c].val = smallest ? -s[c] : s[c];
        }
        qsort(pairs, (size_t)cols, sizeof(mo_pair), mo_pair_cmp);
        for (int i = 0; i < k; i++) out_idx[r * k + i] = (int32_t)pairs[i].idx;
        free(pairs);
    }
    return rc;
}

/* runtime/retrieval_eval.go:586-661 (topRetrievalScores): f32 dot + size-k min-heap, then sort of
 * the k survivors.  Ties there break on the string doc ID; integer row ids stand in for it.  The
 * bench times this as the reference's better host algorithm.  One query, docs [rows, cols]. */
static int mo_better(float sa, int64_t ia, float sb, int64_t ib) {
    if (sa > sb) return 1;
    if (sa < sb) return 0;
    return ia < ib;
}

int mo_dot_heap_topk(const float* query, const float* docs, int64_t rows, int64_t cols, int k,
                     int32_t* out_idx, float* out_scores) {
    if (k <= 0 || k > rows) k = (int)rows;
    mo_pair* h = (mo_pair*)malloc((size_t)k * sizeof(mo_pair));
    if (!h) return MO_ERR_RANGE;
    int n = 0;
    for (int64_t r = 0; r < rows; r++) {
        const float* d = docs + r * cols;
        float sum = 0.0f;
        for (int64_t c = 0; c < cols; c++) sum += query[c] * d[c];
        if (n < k) { /* push + sift up; heap root is the worst kept entry */
            int i = n++;
            h[i].idx = r;
            h[i].val = sum;
            while (i > 0) {
                int p = (i - 1) / 2;
                if (mo_better(h[p].val, h[p].idx, h[i].val, h[i].idx)) {
                    mo_pair t = h[p];
                    h[p] = h[i];
                    h[i] = t;
                    i = p;
                } else {
                    break;
                }
            }
            continue;
        }
        if (mo_better(sum, r, h[0].val, h[0].idx)) {
            h[0].idx = r;
            h[0].val = sum;
            int i = 0;
            for (;;) { /* sift down */
                int l = 2 * i + 1, rr = l + 1, w = i;
                if (l < n && mo_better(h[w].val, h[w].idx, h[l].val, h[l].idx)) w = l;
                if (rr < n && mo_better(h[w].val, h[w].idx, h[rr].val, h[rr].idx)) w = rr;
                if (w == i) break;
                mo_pair t = h[w];
                h[w] = h[i];
                h[i] = t;
                i = w;
            }
        }
    }
    qsort(h, (size_t)n, sizeof(mo_pair), mo_pair_cmp);
    for (int i = 0; i < n; i++) {
        out_idx[i] = (int32_t)h[i].idx;
        out_scores[i] = h[i].val;
    }
    free(h);
    return MO_OK;
}

/* ---- gather ----------------------------------------------------------------------------- */

/* runtime/backend/tensor_ops.go:761-827 (gatherTensor, rank-1 and rank-2 tables with rank-1
 * indices): out[i, :] = table[idx[i], :]; any index outside [0, rows) is an error.  elem_bytes is
 * 4 for f32/i32 tables and 8 for i64 tables; cols == 1 is the rank-1 table. */
int mo_gather_rows(const void* table, int64_t rows, int64_t cols, int elem_bytes, const int32_t* idx,
                   int64_t n, void* out, int32_t* bad_index) {
    size_t row_bytes = (size_t)cols * (size_t)elem_bytes;
    for (int64_t i = 0; i < n; i++) {
        if (idx[i] < 0 || (int64_t)idx[i] >= rows) {
            if (bad_index) *bad_index = idx[i];
            return MO_ERR_RANGE;
        }
        memcpy((char*)out + (size_t)i * row_bytes, (const char*)table + (size_t)idx[i] * row_bytes,
               row_bytes);
    }
    return MO_OK;
}

/* ---- quantiser -------------------------------------------------------------------------- */

/* runtime/embedding_trainer.go:3730-3763 (fakeQuantizeDataInPlace): symmetric, one scale per slice,
 * levels = 2^(bits-1)-1, scale = maxAbs/levels, q = Round(v/scale) half away from zero, clamp,
 * value = q*scale; untouched when the slice is all zero. */
void mo_fake_quantize(float* data, int64_t n, int bits) {
    if (bits <= 0 || n == 0) return;
    float max_abs = 0.0f;
    for (int64_t i = 0; i < n; i++) {
        float a = (float)fabs((double)data[i]);
        if (a > max_abs) max_abs = a;
    }
    if (max_abs == 0.0f) return;
    int levels_int = (1 << (bits - 1)) - 1;
    float levels = (float)levels_int;
    if (levels <= 0.0f) return;
    float scale = max_abs / levels;
    if (scale == 0.0f) return;
    for (int64_t i = 0; i < n; i++) {
        volatile float ratio = data[i] / scale;
        float q = (float)round((double)ratio);
        if (q > levels) q = levels;
        if (q < -levels) q = -levels;
        data[i] = q * scale;
    }
}

/* q8-row packing (layout fixed by the build's ABI): the quantiser above applied per row with
 * bits = 8; codes kept as int8 and the scale as one f32 per row.  value = (float)code * scale. */
void mo_pack_q8_rows(const float* src, int64_t rows, int64_t cols, int8_t* codes, float* scales) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
        const float* x = src + r * cols;
        int8_t* q = codes + r * cols;
        float max_abs = 0.0f;
        for (int64_t c = 0; c < cols; c++) {
            float a = (float)fabs((double)x[c]);
            if (a > max_abs) max_abs = a;
        }
        float scale = max_abs / 127.0f;
        if (max_abs == 0.0f || scale == 0.0f) {
            scales[r] = 0.0f;
            for (int64_t c = 0; c < cols; c++) q[c] = 0;
            continue;
        }
        scales[r] = scale;
        for (int64_t c = 0; c < cols; c++) {
            volatile float ratio = x[c] / scale;
            float v = (float)round((double)ratio);
            if (v > 127.0f) v = 127.0f;
            if (v < -127.0f) v = -127.0f;
            q[c] = (int8_t)v;
        }
    }
}

void mo_unpack_q8_rows(const int8_t* codes, const float* scales, int64_t rows, int64_t cols, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
        for (int64_t c = 0; c < cols; c++) {
            volatile float v = (float)codes[r * cols + c] * scales[r];
            out[r * cols + c] = v;
        }
    }
}

/* q4-block32 packing (layout fixed by the build's ABI): per row cols/32 blocks; per block the
 * quantiser above with bits = 4 (levels 7) against the scale AFTER it is rounded to f16, so that
 * pack and unpack agree; 16 bytes per block, element 2j in the low nibble of byte j and element
 * 2j+1 in the high nibble, both as 4-bit two's complement; one f16 scale per block. */
int mo_pack_q4_b32(const float* src, int64_t rows, int64_t cols, uint8_t* codes, uint16_t* scales) {
    if (cols % 32 != 0) return MO_ERR_SHAPE;
    int64_t blocks = cols / 32;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
        for (int64_t b = 0; b < blocks; b++) {
            const float* x = src + r * cols + b * 32;
            uint8_t* out = codes + (r * blocks + b) * 16;
            float max_abs = 0.0f;
            for (int c = 0; c < 32; c++) {
                float a = (float)fabs((double)x[c]);
                if (a > max_abs) max_abs = a;
            }
            uint16_t hs = mo_float_to_half(max_abs / 7.0f);
            float scale = mo_half_to_float(hs);
            if (max_abs == 0.0f || scale == 0.0f) {
                scales[r * blocks + b] = 0;
                memset(out, 0, 16);
                continue;
            }
            scales[r * blocks + b] = hs;
            int8_t q[32];
            for (int c = 0; c < 32; c++) {
                volatile float ratio = x[c] / scale;
                float v = (float)round((double)ratio);
                if (v > 7.0f) v = 7.0f;
                if (v < -7.0f) v = -7.0f;
                q[c] = (int8_t)v;
            }
            for (int j = 0; j < 16; j++) {
                out[j] = (uint8_t)((q[2 * j] & 0x0f) | ((q[2 * j + 1] & 0x0f) << 4));
            }
        }
    }
    return MO_OK;
}

int mo_unpack_q4_b32(const uint8_t* codes, const uint16_t* scales, int64_t rows, int64_t cols, float* out) {
    if (cols % 32 != 0) return MO_ERR_SHAPE;
    int64_t blocks = cols / 32;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
        for (int64_t b = 0; b < blocks; b++) {
            const uint8_t* in = codes + (r * blocks + b) * 16;
            float scale = mo_half_to_float(scales[r * blocks + b]);
            for (int j = 0; j < 16; j++) {
                int lo = in[j] & 0x0f;
                int hi = (in[j] >> 4) & 0x0f;
                if (lo >= 8) lo -= 16;
                if (hi >= 8) hi -= 16;
                volatile float v0 = (float)lo * scale;
                volatile float v1 = (float)hi * scale;
                out[r * cols + b * 32 + 2 * j] = v0;
                out[r * cols + b * 32 + 2 * j + 1] = v1;
            }
        }
    }
    return MO_OK;
}

/* ---- bit-exact model of the packed q8 device arithmetic ------------------------------------
 *
 * The device never widens q8 rows to float.  It splits each f16 query into two int8 planes
 *   q[c] ~= s_hi*hi[c] + s_lo*lo[c],  s_hi = max|q|/127,  s_lo = s_hi/254
 * accumulates I_hi = sum hi*d, I_lo = sum lo*d and nn = sum d*d in int32 (exact, order-free) and
 * finishes in f32 with a fixed sequence of correctly rounded operations.  This model restates that
 * sequence so tests can demand bit equality of the integer accumulators and of the final f32.
 * It is a statement of the build's own arithmetic, not of the reference's; agreement of this
 * arithmetic with the reference's float path (1e-3 relative) is tested separately.
 */
static double mo_butterfly32(double* part) {
    double tmp[32];
    for (int off = 16; off > 0; off >>= 1) {
        for (int l = 0; l < 32; l++) tmp[l] = part[l] + part[l ^ off];
        for (int l = 0; l < 32; l++) part[l] = tmp[l];
    }
    return part[0];
}

void mo_q8_query_planes(const float* q, int64_t cols, int8_t* hi, int8_t* lo, float* s_hi, float* s_lo,
                        float* qn, float* qn2, double* qhat2) {
    float amax = 0.0f;
    /* device order of the f64 sum of squares: 32 lane-strided partial sums, then an xor butterfly */
    double part[32], hpart[32];
    for (int l = 0; l < 32; l++) part[l] = hpart[l] = 0.0;
    for (int64_t c = 0; c < cols; c++) {
        float a = fabsf(q[c]);
        if (a > amax) amax = a;
        double v = (double)q[c];
        part[c & 31] += v * v;
    }
    double n2 = mo_butterfly32(part);
    *qn2 = (float)n2;
    *qn = (float)sqrt(n2);
    if (amax == 0.0f) {
        *s_hi = 0.0f;
        *s_lo = 0.0f;
        *qhat2 = 0.0;
        memset(hi, 0, (size_t)cols);
        memset(lo, 0, (size_t)cols);
        return;
    }
    volatile float sh = amax / 127.0f;
    volatile float sl = sh / 254.0f;
    *s_hi = sh;
    *s_lo = sl;
    for (int64_t c = 0; c < cols; c++) {
        volatile float ratio = q[c] / sh;
        float h = roundf(ratio);
        if (h > 127.0f) h = 127.0f;
        if (h < -127.0f) h = -127.0f;
        float rem = fmaf(-h, sh, q[c]);
        float l = 0.0f;
        if (sl != 0.0f) {
            volatile float r2 = rem / sl;
            l = roundf(r2);
            if (l > 127.0f) l = 127.0f;
            if (l < -127.0f) l = -127.0f;
        }
        hi[c] = (int8_t)h;
        lo[c] = (int8_t)l;
        double v = (double)h * (double)sh + (double)l * (double)sl;
        hpart[c & 31] += v * v;
    }
    *qhat2 = mo_butterfly32(hpart);
}

/* metric: 0 dot, 1 cosine, 2 l2_distance.  acc (optional) receives I_hi, I_lo, nn per row. */
int mo_q8_model_scores(const float* query, const int8_t* codes, const float* scales, int64_t rows,
                       int64_t cols, int metric, float* out, int32_t* acc) {
    int8_t* hi = (int8_t*)malloc((size_t)cols);
    int8_t* lo = (int8_t*)malloc((size_t)cols);
    if (!hi || !lo) return MO_ERR_RANGE;
    float s_hi, s_lo, qn, qn2;
    double qhat2;
    mo_q8_query_planes(query, cols, hi, lo, &s_hi, &s_lo, &qn, &qn2, &qhat2);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
        const int8_t* d = codes + r * cols;
        int32_t ih = 0, il = 0, nn = 0;
        for (int64_t c = 0; c < cols; c++) {
            ih += (int32_t)hi[c] * d[c];
            il += (int32_t)lo[c] * d[c];
            nn += (int32_t)d[c] * d[c];
        }
        if (acc) {
            acc[3 * r + 0] = ih;
            acc[3 * r + 1] = il;
            acc[3 * r + 2] = nn;
        }
        volatile float a = (float)ih * s_hi;
        float t = fmaf((float)il, s_lo, a);
        float sd = scales[r];
        float res;
        if (metric == 0) {
            volatile float p = t * sd;
            res = p;
        } else if (metric == 1) {
            volatile float qinv = (qn > 0.0f) ? 1.0f / qn : 0.0f;
            volatile float root = sqrtf((float)nn);
            volatile float rinv = (nn > 0) ? 1.0f / root : 0.0f;
            volatile float w = qinv * rinv;
            volatile float qv = t * w;
            res = qv + 0.0f;
        } else {
            double td = (double)ih * (double)s_hi + (double)il * (double)s_lo;
            double dotd = td * (double)sd;
            double dn2d = ((double)sd * (double)sd) * (double)nn;
            double x = (qhat2 + dn2d) + -(2.0 * dotd);
            if (!(x > 0.0)) x = 0.0;
            res = (float)sqrt(x);
        }
        out[r] = res + 0.0f; /* -0 -> +0, as the device does */
    }
    free(hi);
    free(lo);
    return MO_OK;
}

/* ---- embedding front end (the callers' side of the score path) ------------------------------------ */

/* gatherTensor on a rank-2 table (runtime/backend/tensor_ops.go:794-827) -> matmulTensor rank-3 x rank-2
 * (:981-1011 and its batched form: f32 sequential accumulate, products and sums rounded separately) ->
 * meanPoolMaskedTensor (:1210-1275: rows with mask != 0 summed in order in f32, times 1/count) and
 * normalizeRows (:1114-1138: f64 sum of squares, f32 norm, f32 divide; zero rows untouched), in either order:
 *   order 0: normalize(mean_pool(x, mask))   (the end-to-end embed+score configuration)
 *   order 1: mean_pool(normalize(x), mask)   (examples/embed_masked_pooled.manta)
 * table [vocab, dim] and proj [dim, out] are f32 (f16-representable values); tokens / mask are [batch, seq].
 * Returns MO_ERR_RANGE for a token outside the table. */
int mo_embed_pooled(const float* table, int64_t vocab, int64_t dim, const float* proj, int64_t out_dim,
                    const int32_t* tokens, const int32_t* mask, int64_t batch, int64_t seq, int order, float* out) {
    for (int64_t i = 0; i < batch * seq; i++)
        if (tokens[i] < 0 || tokens[i] >= vocab) return MO_ERR_RANGE;
    int rc = MO_OK;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t b = 0; b < batch; b++) {
        float* projected = (float*)malloc((size_t)out_dim * sizeof(float));
        float* pooled = out + b * out_dim;
        if (!projected) {
            rc = MO_ERR_RANGE;
            continue;
        }
        for (int64_t c = 0; c < out_dim; c++) pooled[c] = 0.0f;
        int count = 0;
        for (int64_t t = 0; t < seq; t++) {
            if (mask[b * seq + t] == 0) continue; /* unmasked rows never reach the output */
            const float* h = table + (int64_t)tokens[b * seq + t] * dim;
            for (int64_t c = 0; c < out_dim; c++) {
                float sum = 0.0f;
                for (int64_t k = 0; k < dim; k++) {
                    volatile float p = h[k] * proj[k * out_dim + c];
                    sum += p;
                }
                projected[c] = sum;
            }
            if (order == 1) { /* normalizeRows on this row */
                double ss = 0.0;
                for (int64_t c = 0; c < out_dim; c++) ss += (double)projected[c] * (double)projected[c];
                float norm = (float)sqrt(ss);
                if (norm != 0.0f)
                    for (int64_t c = 0; c < out_dim; c++) {
                        volatile float v = projected[c] / norm;
                        projected[c] = v;
                    }
            }
            count++;
            for (int64_t c = 0; c < out_dim; c++) pooled[c] += projected[c];
        }
        if (count > 0) {
            volatile float inv = 1.0f / (float)count;
            for (int64_t c = 0; c < out_dim; c++) {
                volatile float v = pooled[c] * inv;
                pooled[c] = v;
            }
        }
        if (order == 0) {
            double ss = 0.0;
            for (int64_t c = 0; c < out_dim; c++) ss += (double)pooled[c] * (double)pooled[c];
            float norm = (float)sqrt(ss);
            if (norm != 0.0f)
                for (int64_t c = 0; c < out_dim; c++) {
                    volatile float v = pooled[c] / norm;
                    pooled[c] = v;
                }
        }
        free(projected);
    }
    return rc;
}
