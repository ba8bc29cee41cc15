/*
 * CPU oracle for the vector-search hot path (Flat / Int8Flat / IVFPQ search and
 * multi-index merge).  TEST INFRASTRUCTURE ONLY: the product library never links,
 * loads or calls anything in this file; tests and the benchmark's CPU-baseline leg
 * use it as the checker.
 *
 * PARITY UNPINNED: the reference (Ascend/IndexSDK) holds no golden vectors or
 * known-answer files for this path.  Its device operators cannot run off Ascend
 * hardware, its unit tests run on a mock runtime whose operators write zeros
 * (feature_retrieval/opensource/AscendCLMock/acl/simu/AscendSimuSysOperator.cpp:430-447),
 * and its CPU ground truth is the third-party library Faiss (v1.10.0 pinned by
 * build/install_deps.sh:23-27, not vendored).  This file therefore restates the
 * published semantics of Faiss' IndexFlatL2 / IndexFlatIP / IndexIVFPQ in its own
 * code and anchors on the reference's call sites:
 *   - Flat ground truth: examples/TestAscendIndexFlat.cpp:242-250 (faiss::IndexFlat),
 *     self-hit property FR/test/ascend/TestAscendIndexFlat.cpp:117-123
 *   - int8 dot product / squared distance in int32:
 *     FR/ops/tbe/impl/distance_int8_cos_maxs.py:256-284 (accumulate part only; the
 *     build follows the stricter raw-int32 contract, no fp16 rescale)
 *   - IVFPQ: raw-vector or residual PQ encode, exhaustive nearest codeword, first
 *     minimum wins: FR/ascend/impl/AscendIndexIVFPQImpl.cpp:879-910; one ADC table
 *     per query [M][256]: FR/ascenddaemon/impl/IndexIVFPQ.cpp:1681-1704; table entry
 *     semantics FR/ops/ascendc/op_kernel/ascendc_ivfpq_subspace_distance.cpp:222-258;
 *     only non-empty probed lists are scanned: IndexIVFPQ.cpp:2166-2219
 *   - result padding FLT_MAX / -1: FR/ascend/impl/AscendIndexImpl.cpp:628-633
 *   - multi-index layout [index][query][k] and merge: FR/ascend/utils/MergeResUtils.cpp:44-107
 *   (FR = feature_retrieval/src/ascendfaiss)
 *
 * Canonical arithmetic (the GPU path computes the same expressions in the same
 * order, which is what makes fp32 and int8 results bit-comparable):
 *   L2(q,y)  : acc = 0; for i in 0..d-1: t = q[i]-y[i]; acc = fmaf(t,t,acc)
 *   IP(q,y)  : acc = 0; for i in 0..d-1: acc = fmaf(q[i],y[i],acc)
 *   ADC      : acc = 0; for m in 0..M-1: acc = acc + LUT[m][code[m]]   (fp32 adds)
 *   ordering : ascending (key, tie) with key = distance (L2) or -score (IP) and
 *              tie = insertion position (Flat/Int8Flat) or label (IVFPQ, merges).
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_METRIC_IP 0
#define ORC_METRIC_L2 1
#define ORC_METRIC_INT8_COS 2

typedef struct {
    double key;
    int64_t tie;
} orc_item;

static inline int item_less(const orc_item* a, const orc_item* b) {
    return (a->key < b->key) || (a->key == b->key && a->tie < b->tie);
}

/* max-heap on (key, tie): root is the worst of the kept k */
static void heap_sift_down(orc_item* h, int n, int i) {
    for (;;) {
        int l = 2 * i + 1, r = l + 1, m = i;
        if (l < n && item_less(&h[m], &h[l])) m = l;
        if (r < n && item_less(&h[m], &h[r])) m = r;
        if (m == i) return;
        orc_item t = h[i]; h[i] = h[m]; h[m] = t;
        i = m;
    }
}

static void heap_sift_up(orc_item* h, int i) {
    while (i > 0) {
        int p = (i - 1) / 2;
        if (!item_less(&h[p], &h[i])) return;
        orc_item t = h[i]; h[i] = h[p]; h[p] = t;
        i = p;
    }
}

static inline void heap_offer(orc_item* h, int* n, int k, double key, int64_t tie) {
    orc_item it = {key, tie};
    if (*n < k) {
        h[*n] = it;
        heap_sift_up(h, *n);
        (*n)++;
    } else if (item_less(&it, &h[0])) {
        h[0] = it;
        heap_sift_down(h, k, 0);
    }
}

static int item_cmp(const void* a, const void* b) {
    const orc_item* x = (const orc_item*)a;
    const orc_item* y = (const orc_item*)b;
    if (item_less(x, y)) return -1;
    if (item_less(y, x)) return 1;
    return 0;
}

/* write sorted heap content to the output row; pad with FLT_MAX / -1 */
static void heap_emit(orc_item* h, int n, int k, int negate, float* D, int64_t* I) {
    qsort(h, (size_t)n, sizeof(orc_item), item_cmp);
    for (int j = 0; j < k; ++j) {
        if (j < n) {
            D[j] = (float)(negate ? -h[j].key : h[j].key);
            I[j] = h[j].tie;
        } else {
            D[j] = FLT_MAX;
            I[j] = -1;
        }
    }
}

static inline float l2_canon(const float* q, const float* y, int d) {
    float acc = 0.f;
    for (int i = 0; i < d; ++i) {
        float t = q[i] - y[i];
        acc = fmaf(t, t, acc);
    }
    return acc;
}

static inline float ip_canon(const float* q, const float* y, int d) {
    float acc = 0.f;
    for (int i = 0; i < d; ++i) acc = fmaf(q[i], y[i], acc);
    return acc;
}

static inline double l2_f64(const float* q, const float* y, int d) {
    double acc = 0.0;
    for (int i = 0; i < d; ++i) {
        double t = (double)q[i] - (double)y[i];
        acc += t * t;
    }
    return acc;
}

static inline double ip_f64(const float* q, const float* y, int d) {
    double acc = 0.0;
    for (int i = 0; i < d; ++i) acc += (double)q[i] * (double)y[i];
    return acc;
}

/*
 * Blocked forms of the canonical kernels: ORC_B independent accumulator chains side by side
 * (one per query, centroid or codeword of a block, operands transposed to [i][ORC_B]) so that
 * the compiler can use one vector FMA per step.  Each chain performs exactly the operations of
 * l2_canon / ip_canon in the same order, so results are bit-identical to the scalar forms.
 */
#define ORC_B 8
static inline void l2_canon_qblock(const float* qT, const float* y, int d, float* acc) {
    for (int b = 0; b < ORC_B; ++b) acc[b] = 0.f;
    for (int i = 0; i < d; ++i) {
        const float yi = y[i];
#pragma omp simd
        for (int b = 0; b < ORC_B; ++b) {
            float t = qT[i * ORC_B + b] - yi;
            acc[b] = fmaf(t, t, acc[b]);
        }
    }
}
static inline void ip_canon_qblock(const float* qT, const float* y, int d, float* acc) {
    for (int b = 0; b < ORC_B; ++b) acc[b] = 0.f;
    for (int i = 0; i < d; ++i) {
        const float yi = y[i];
#pragma omp simd
        for (int b = 0; b < ORC_B; ++b) acc[b] = fmaf(qT[i * ORC_B + b], yi, acc[b]);
    }
}
/* the same for four base rows at a time: four times as many independent fmaf chains in flight (a
 * single chain over the dimension is bound by the latency of fmaf, not by its throughput) */
#define ORC_R 4
static inline void l2_canon_qblock_rows(const float* qT, const float* y, int d, float acc[ORC_R][ORC_B]) {
    for (int r = 0; r < ORC_R; ++r)
        for (int b = 0; b < ORC_B; ++b) acc[r][b] = 0.f;
    for (int i = 0; i < d; ++i) {
        for (int r = 0; r < ORC_R; ++r) {
            const float yi = y[(size_t)r * d + i];
#pragma omp simd
            for (int b = 0; b < ORC_B; ++b) {
                float t = qT[i * ORC_B + b] - yi;
                acc[r][b] = fmaf(t, t, acc[r][b]);
            }
        }
    }
}
static inline void ip_canon_qblock_rows(const float* qT, const float* y, int d, float acc[ORC_R][ORC_B]) {
    for (int r = 0; r < ORC_R; ++r)
        for (int b = 0; b < ORC_B; ++b) acc[r][b] = 0.f;
    for (int i = 0; i < d; ++i) {
        for (int r = 0; r < ORC_R; ++r) {
            const float yi = y[(size_t)r * d + i];
#pragma omp simd
            for (int b = 0; b < ORC_B; ++b) acc[r][b] = fmaf(qT[i * ORC_B + b], yi, acc[r][b]);
        }
    }
}
/* one query against a block of ORC_B rows stored transposed yT[i][ORC_B] */
static inline void l2_canon_yblock(const float* q, const float* yT, int d, float* acc) {
    for (int b = 0; b < ORC_B; ++b) acc[b] = 0.f;
    for (int i = 0; i < d; ++i) {
        const float qi = q[i];
#pragma omp simd
        for (int b = 0; b < ORC_B; ++b) {
            float t = qi - yT[i * ORC_B + b];
            acc[b] = fmaf(t, t, acc[b]);
        }
    }
}
/* rows [n][d] -> blocks [ceil(n/ORC_B)][d][ORC_B]; rows past n repeat the last row */
static float* transpose_blocks(const float* x, int64_t n, int d) {
    int64_t nb = (n + ORC_B - 1) / ORC_B;
    float* t = (float*)malloc(sizeof(float) * (size_t)nb * d * ORC_B);
    if (!t) return NULL;
    for (int64_t blk = 0; blk < nb; ++blk)
        for (int i = 0; i < d; ++i)
            for (int b = 0; b < ORC_B; ++b) {
                int64_t r = blk * ORC_B + b;
                if (r >= n) r = n - 1;
                t[(blk * d + i) * ORC_B + b] = x[r * d + i];
            }
    return t;
}

/*
 * Exact Flat search.  precise = 0: canonical fp32 arithmetic (bit-comparable with the
 * GPU fp32 mode); precise = 1: fp64 accumulation rounded to fp32 once (used to bound
 * the error of every lower-precision mode).  labels: optional nb entries mapping
 * position -> user id (NULL = identity); ties are broken by position.
 */
int orc_flat_search(int metric, int d, int64_t nb, const float* xb, const int64_t* labels,
                    int64_t nq, const float* xq, int k, int precise, float* D, int64_t* I) {
    if (d <= 0 || nb < 0 || nq < 0 || k <= 0) return -1;
    int fail = 0;
    if (!precise && nq > 0) {
        /* Cache-blocked: the base is walked once per call in blocks of about 1 MB; every block of
         * ORC_B queries (transposed, one SIMD lane per query) meets a base block while it is in
         * cache.  Every (query, row) pair is still the canonical sequential sum, and every query
         * still sees the rows in increasing order, so the results are those of the plain loop. */
        float* qT = transpose_blocks(xq, nq, d);
        if (!qT) return -2;
        const int64_t nblk = (nq + ORC_B - 1) / ORC_B;
        orc_item* heaps = (orc_item*)malloc(sizeof(orc_item) * (size_t)k * (size_t)nblk * ORC_B);
        int* cnt = (int*)calloc((size_t)nblk * ORC_B, sizeof(int));
        if (!heaps || !cnt) { free(qT); free(heaps); free(cnt); return -2; }
        int64_t jb = ((int64_t)1 << 20) / ((int64_t)d * 4);
        if (jb < 64) jb = 64;
        jb = jb / ORC_R * ORC_R;
        const int l2 = metric == ORC_METRIC_L2;
        for (int64_t j0 = 0; j0 < nb; j0 += jb) {
            const int64_t j1 = j0 + jb < nb ? j0 + jb : nb;
#pragma omp parallel for schedule(dynamic, 1)
            for (int64_t blk = 0; blk < nblk; ++blk) {
                orc_item* h = heaps + (size_t)blk * ORC_B * k;
                int* n = cnt + blk * ORC_B;
                const float* qb = qT + blk * d * ORC_B;
                const int live = (int)((nq - blk * ORC_B) < ORC_B ? (nq - blk * ORC_B) : ORC_B);
                float acc4[ORC_R][ORC_B];
                int64_t j = j0;
                for (; j + ORC_R <= j1; j += ORC_R) {
                    if (l2) l2_canon_qblock_rows(qb, xb + j * d, d, acc4);
                    else ip_canon_qblock_rows(qb, xb + j * d, d, acc4);
                    for (int r = 0; r < ORC_R; ++r)
                        for (int b = 0; b < live; ++b)
                            heap_offer(h + (size_t)b * k, &n[b], k, l2 ? (double)acc4[r][b] : -(double)acc4[r][b], j + r);
                }
                for (; j < j1; ++j) {
                    if (l2) l2_canon_qblock(qb, xb + j * d, d, acc4[0]);
                    else ip_canon_qblock(qb, xb + j * d, d, acc4[0]);
                    for (int b = 0; b < live; ++b)
                        heap_offer(h + (size_t)b * k, &n[b], k, l2 ? (double)acc4[0][b] : -(double)acc4[0][b], j);
                }
            }
        }
#pragma omp parallel for schedule(static)
        for (int64_t q = 0; q < nq; ++q) {
            heap_emit(heaps + (size_t)q * k, cnt[q], k, !l2, D + q * k, I + q * k);
            if (labels)
                for (int j = 0; j < k; ++j)
                    if (I[q * k + j] >= 0) I[q * k + j] = labels[I[q * k + j]];
        }
        free(heaps);
        free(cnt);
        free(qT);
        return 0;
    }
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t q = 0; q < nq; ++q) {
        orc_item* h = (orc_item*)malloc(sizeof(orc_item) * (size_t)k);
        if (!h) { fail = 1; continue; }
        int n = 0;
        const float* qv = xq + q * d;
        for (int64_t j = 0; j < nb; ++j) {
            const float* yv = xb + j * d;
            double key;
            if (metric == ORC_METRIC_L2)
                key = precise ? (double)(float)l2_f64(qv, yv, d) : (double)l2_canon(qv, yv, d);
            else
                key = -(precise ? (double)(float)ip_f64(qv, yv, d) : (double)ip_canon(qv, yv, d));
            heap_offer(h, &n, k, key, j);
        }
        heap_emit(h, n, k, metric != ORC_METRIC_L2, D + q * k, I + q * k);
        if (labels)
            for (int j = 0; j < k; ++j)
                if (I[q * k + j] >= 0) I[q * k + j] = labels[I[q * k + j]];
        free(h);
    }
    return fail ? -2 : 0;
}

/* fp32 -> fp16 -> fp32 with round-to-nearest-even, the conversion the reference applies
 * to base and queries on the host (FR/ascend/utils/fp16.cpp:73-93). */
void orc_round_fp16(int64_t n, const float* x, float* out) {
#pragma omp parallel for
    for (int64_t i = 0; i < n; ++i) out[i] = (float)(_Float16)x[i];
}

void orc_round_bf16(int64_t n, const float* x, float* out) {
#pragma omp parallel for
    for (int64_t i = 0; i < n; ++i) {
        uint32_t u;
        memcpy(&u, &x[i], 4);
        uint32_t r = u + 0x7FFFu + ((u >> 16) & 1u);
        r &= 0xFFFF0000u;
        if ((u & 0x7F800000u) == 0x7F800000u) r = u & 0xFFFF0000u; /* inf/nan: truncate */
        memcpy(&out[i], &r, 4);
    }
}


/* ---- fp16 arithmetic for the int8 cosine ---- */

/* float -> fp16 bits, round to nearest even, subnormals and overflow to inf as IEEE 754 */
static uint16_t f2h(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    const uint32_t sign = (u >> 16) & 0x8000u;
    const uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return (uint16_t)(sign | 0x7FFFu);            /* NaN */
    if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);           /* >= 65520 rounds to inf */
    if (a < 0x33000001u) return (uint16_t)sign;                        /* <= 2^-25 rounds to zero */
    int e = (int)(a >> 23) - 127;
    uint32_t m = (a & 0x7FFFFFu) | 0x800000u;                          /* 24-bit significand */
    int shift = e >= -14 ? 13 : 13 + (-14 - e);                        /* bits dropped */
    uint32_t keep = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (keep & 1u))) ++keep;
    /* normal: keep has the hidden bit at 0x400, adding the biased exponent minus one absorbs it
     * (and a carry out of the significand bumps the exponent); subnormal: exponent field 0 */
    const uint32_t h = e >= -14 ? ((uint32_t)(e + 14) << 10) + keep : keep;
    return (uint16_t)(sign | h);
}

static float h2f(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
    uint32_t u;
    if (e == 0x1F) u = sign | 0x7F800000u | (m << 13);
    else if (e) u = sign | ((e + 112u) << 23) | (m << 13);
    else if (!m) u = sign;
    else {
        int sh = 0;
        uint32_t mm = m;
        while (!(mm & 0x400u)) { mm <<= 1; ++sh; }
        u = sign | ((uint32_t)(113 - sh) << 23) | ((mm & 0x3FFu) << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* fp16 product of two fp16 values: the float product of two 11-bit significands is exact */
static uint16_t hmul(uint16_t a, uint16_t b) { return f2h(h2f(a) * h2f(b)); }

/* rnorm(v) = fp16(1 / sqrt(fp16(|v|^2 * 0.01)))
 * (feature_retrieval/src/ascendfaiss/ops/tbe/impl/int8_l2_norm.py:140-183: the squared norms leave
 * the cube unit through a 0.01 dequantisation to fp16, then vec_rsqrt_high_preci) */
static uint16_t cos16_rnorm(int32_t sq) {
    volatile float scaled = (float)sq * 0.01f;
    const float s = h2f(f2h(scaled));
    volatile float root = sqrtf(s);
    volatile float r = 1.0f / root;
    return f2h(r);
}

/* the fp16 score as an integer with the order of the values; NaN below everything
 * (feature_retrieval/src/ascendfaiss/ops/tbe/impl/distance_int8_cos_maxs.py:256-284:
 *  res = (rnorm_x * rnorm_q) in fp16; ip = int32 * 0.01 -> fp16; res = ip * res in fp16) */
static int32_t cos16_score(int32_t dot, uint16_t rx, uint16_t rq) {
    volatile float scaled = (float)dot * 0.01f;
    const uint16_t ip = f2h(scaled);
    const uint16_t r = hmul(ip, hmul(rx, rq));
    if ((r & 0x7FFFu) > 0x7C00u) return -32768;
    const int32_t x = (int16_t)r;
    return x ^ ((x >> 31) & 0x7FFF);
}

static float cos16_value(int32_t s) {
    if (s <= -32768) return -INFINITY;
    return h2f((uint16_t)(s >= 0 ? (uint32_t)s : (0x8000u | (uint32_t)(-1 - s))));
}

/*
 * Exact int8 Flat search, int32 accumulation, no scaling.  IP: score = sum q*x, larger
 * is better; L2: sum (q-x)^2, smaller is better.  Ties -> lower position.  Distances are
 * returned as float (|value| <= 1024*2^14 < 2^24, exactly representable).
 * ORC_METRIC_INT8_COS: the fp16 cosine above, larger is better, NaN last and returned as -inf.
 */
int orc_int8_search(int metric, int d, int64_t nb, const int8_t* xb, const int64_t* labels,
                    int64_t nq, const int8_t* xq, int k, float* D, int64_t* I) {
    if (d <= 0 || nb < 0 || nq < 0 || k <= 0) return -1;
    if (nq == 0) return 0;
    /* cache-blocked like orc_flat_search: base blocks of about 1 MB, all queries against a block
     * while it is in cache; integer arithmetic, so the order of the sums is immaterial */
    orc_item* heaps = (orc_item*)malloc(sizeof(orc_item) * (size_t)k * (size_t)nq);
    int* cnt = (int*)calloc((size_t)nq, sizeof(int));
    uint16_t *rx = NULL, *rq = NULL;
    if (metric == ORC_METRIC_INT8_COS) {
        rx = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)(nb > 0 ? nb : 1));
        rq = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)nq);
        if (!rx || !rq) { free(heaps); free(cnt); free(rx); free(rq); return -2; }
#pragma omp parallel for schedule(static)
        for (int64_t j = 0; j < nb + nq; ++j) {
            const int8_t* v = j < nb ? xb + j * d : xq + (j - nb) * d;
            int32_t sq = 0;
            for (int i = 0; i < d; ++i) sq += (int32_t)v[i] * (int32_t)v[i];
            if (j < nb) rx[j] = cos16_rnorm(sq);
            else rq[j - nb] = cos16_rnorm(sq);
        }
    }
    if (!heaps || !cnt) { free(heaps); free(cnt); free(rx); free(rq); return -2; }
    int64_t jb = ((int64_t)1 << 20) / (int64_t)d;
    if (jb < 64) jb = 64;
    for (int64_t j0 = 0; j0 < nb; j0 += jb) {
        const int64_t j1 = j0 + jb < nb ? j0 + jb : nb;
#pragma omp parallel for schedule(dynamic, 1)
        for (int64_t q = 0; q < nq; ++q) {
            orc_item* h = heaps + (size_t)q * k;
            int* n = cnt + q;
            const int8_t* qv = xq + q * d;
            for (int64_t j = j0; j < j1; ++j) {
                const int8_t* yv = xb + j * d;
                int32_t acc = 0;
                if (metric == ORC_METRIC_INT8_COS) {
                    for (int i = 0; i < d; ++i) acc += (int32_t)qv[i] * (int32_t)yv[i];
                    heap_offer(h, n, k, -(double)cos16_score(acc, rx[j], rq[q]), j);
                } else if (metric == ORC_METRIC_L2) {
                    for (int i = 0; i < d; ++i) {
                        int32_t t = (int32_t)qv[i] - (int32_t)yv[i];
                        acc += t * t;
                    }
                    heap_offer(h, n, k, (double)acc, j);
                } else {
                    for (int i = 0; i < d; ++i) acc += (int32_t)qv[i] * (int32_t)yv[i];
                    heap_offer(h, n, k, -(double)acc, j);
                }
            }
        }
    }
#pragma omp parallel for schedule(static)
    for (int64_t q = 0; q < nq; ++q) {
        heap_emit(heaps + (size_t)q * k, cnt[q], k, metric != ORC_METRIC_L2, D + q * k, I + q * k);
        if (metric == ORC_METRIC_INT8_COS)
            for (int j = 0; j < k; ++j)
                if (I[q * k + j] >= 0) D[q * k + j] = cos16_value((int32_t)D[q * k + j]);
        if (labels)
            for (int j = 0; j < k; ++j)
                if (I[q * k + j] >= 0) I[q * k + j] = labels[I[q * k + j]];
    }
    free(heaps);
    free(cnt);
    free(rx);
    free(rq);
    return 0;
}

/* fp16 helpers exported for the tests of the restatement itself */
uint16_t orc_f2h(float f) { return f2h(f); }
float orc_h2f(uint16_t h) { return h2f(h); }
uint16_t orc_cos16_rnorm(int32_t sq) { return cos16_rnorm(sq); }
float orc_cos16(int32_t dot, int32_t sq_x, int32_t sq_q) {
    return cos16_value(cos16_score(dot, cos16_rnorm(sq_x), cos16_rnorm(sq_q)));
}

/* ---- IVFPQ ---- */

/* nearest centroid under canonical L2, ties -> lower list id */
int orc_ivf_assign(int d, int nlist, const float* centroids, int64_t n, const float* x,
                   int32_t* list_no) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float best = INFINITY;
        int32_t arg = 0;
        for (int l = 0; l < nlist; ++l) {
            float dd = l2_canon(x + i * d, centroids + (int64_t)l * d, d);
            if (dd < best) { best = dd; arg = l; }
        }
        list_no[i] = arg;
    }
    return 0;
}

/*
 * PQ encode: codebooks [M][ksub][dsub]; by_residual subtracts the assigned centroid
 * first.  Exhaustive nearest codeword, first minimum wins.
 */
int orc_pq_encode(int d, int M, int ksub, const float* codebooks, int by_residual,
                  const float* centroids, const int32_t* list_no, int64_t n, const float* x,
                  uint8_t* codes) {
    if (M <= 0 || d % M || ksub > 256) return -1;
    int dsub = d / M;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float r[4096];
        const float* v = x + i * d;
        if (by_residual) {
            const float* c = centroids + (int64_t)list_no[i] * d;
            for (int t = 0; t < d; ++t) r[t] = v[t] - c[t];
            v = r;
        }
        for (int m = 0; m < M; ++m) {
            float best = INFINITY;
            int arg = 0;
            for (int j = 0; j < ksub; ++j) {
                float dd = l2_canon(v + m * dsub, codebooks + ((int64_t)m * ksub + j) * dsub, dsub);
                if (dd < best) { best = dd; arg = j; }
            }
            codes[i * M + m] = (uint8_t)arg;
        }
    }
    return 0;
}

/*
 * IVFPQ search, L2 only (the reference forces L2: AscendIndexIVFPQImpl.cpp:701).
 * Lists are CSR: list_offsets[nlist+1] into codes[ntotal][M] and ids[ntotal].
 * Stage 1: nprobe nearest centroids by canonical L2, ties -> lower list id.
 * Stage 2: by_residual = 0: one table per query, LUT[m][j] = L2(q_m, cb[m][j]);
 *          by_residual = 1: one table per (query, list) on q - centroid[list] (direct form);
 * Stage 3: ADC sum in fp32, m ascending; top-k by (distance, label).
 * coarse_out (optional, nq*nprobe) receives the probed list ids in rank order.
 */
int orc_ivfpq_search(int d, int nlist, int M, int ksub, const float* centroids,
                     const float* codebooks, int by_residual, const int64_t* list_offsets,
                     const uint8_t* codes, const int64_t* ids, int64_t nq, const float* xq,
                     int nprobe, int k, float* D, int64_t* I, int32_t* coarse_out) {
    if (M <= 0 || d % M || nprobe <= 0 || k <= 0 || ksub > 256 || d > 4096) return -1;
    if (nprobe > nlist) nprobe = nlist;
    int dsub = d / M;
    int fail = 0;
    /* transposed copies: centroids in blocks of ORC_B rows, each sub-codebook in blocks of
       ORC_B codewords, so the canonical per-row sums run ORC_B at a time */
    float* cT = transpose_blocks(centroids, nlist, d);
    float* cbT = transpose_blocks(codebooks, (int64_t)M * ksub, dsub);
    if (!cT || !cbT || ksub % ORC_B) { free(cT); free(cbT); return ksub % ORC_B ? -1 : -2; }
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t q = 0; q < nq; ++q) {
        const float* qv = xq + q * d;
        orc_item* ch = (orc_item*)malloc(sizeof(orc_item) * (size_t)nprobe);
        orc_item* h = (orc_item*)malloc(sizeof(orc_item) * (size_t)k);
        float* lut = (float*)malloc(sizeof(float) * (size_t)M * ksub);
        if (!ch || !h || !lut) { fail = 1; free(ch); free(h); free(lut); continue; }
        int cn = 0;
        for (int l0 = 0; l0 < nlist; l0 += ORC_B) {
            float acc[ORC_B];
            l2_canon_yblock(qv, cT + (int64_t)(l0 / ORC_B) * d * ORC_B, d, acc);
            for (int b = 0; b < ORC_B && l0 + b < nlist; ++b) heap_offer(ch, &cn, nprobe, (double)acc[b], l0 + b);
        }
        qsort(ch, (size_t)cn, sizeof(orc_item), item_cmp);
        if (coarse_out)
            for (int p = 0; p < nprobe; ++p) coarse_out[q * nprobe + p] = p < cn ? (int32_t)ch[p].tie : -1;
        int n = 0;
        if (!by_residual) {
            for (int m = 0; m < M; ++m)
                for (int j = 0; j < ksub; j += ORC_B)
                    l2_canon_yblock(qv + m * dsub, cbT + (int64_t)((m * ksub + j) / ORC_B) * dsub * ORC_B, dsub,
                                    lut + m * ksub + j);
        }
        for (int p = 0; p < cn; ++p) {
            int l = (int)ch[p].tie;
            int64_t b = list_offsets[l], e = list_offsets[l + 1];
            if (b == e) continue;
            if (by_residual) {
                float r[4096];
                const float* c = centroids + (int64_t)l * d;
                for (int t = 0; t < d; ++t) r[t] = qv[t] - c[t];
                for (int m = 0; m < M; ++m)
                    for (int j = 0; j < ksub; j += ORC_B)
                        l2_canon_yblock(r + m * dsub, cbT + (int64_t)((m * ksub + j) / ORC_B) * dsub * ORC_B, dsub,
                                        lut + m * ksub + j);
            }
            for (int64_t v = b; v < e; ++v) {
                const uint8_t* c = codes + v * M;
                float acc = 0.f;
                for (int m = 0; m < M; ++m) acc = acc + lut[m * ksub + c[m]];
                heap_offer(h, &n, k, (double)acc, ids[v]);
            }
        }
        heap_emit(h, n, k, 0, D + q * k, I + q * k);
        free(ch); free(h); free(lut);
    }
    free(cT); free(cbT);
    return fail ? -2 : 0;
}

/*
 * Merge nsrc sorted result sets [src][nq][k] into [nq][k] by (key, label); entries with
 * label < 0 are padding.  descending = 1 for inner-product scores.
 */
int orc_merge_topk(int nsrc, int64_t nq, int k, int descending, const float* Din,
                   const int64_t* Iin, float* D, int64_t* I) {
#pragma omp parallel for schedule(static)
    for (int64_t q = 0; q < nq; ++q) {
        orc_item* h = (orc_item*)malloc(sizeof(orc_item) * (size_t)k);
        int n = 0;
        for (int s = 0; s < nsrc; ++s)
            for (int j = 0; j < k; ++j) {
                int64_t off = ((int64_t)s * nq + q) * k + j;
                if (Iin[off] < 0) continue;
                heap_offer(h, &n, k, descending ? -(double)Din[off] : (double)Din[off], Iin[off]);
            }
        heap_emit(h, n, k, descending, D + q * k, I + q * k);
        free(h);
    }
    return 0;
}

/* Sets the OpenMP thread count of the following calls (a launcher may have exported
 * OMP_NUM_THREADS=1 for its worker processes); returns the count now in effect. */
int orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/*
 * Lloyd k-means in the arithmetic the GPU trainer reproduces bit for bit (the reference trains on
 * the NPU with the same structure -- distance operator, arg-min, centroid update --
 * feature_retrieval/src/ascendfaiss/ascenddaemon/impl/IndexIVFPQ.cpp:810-1135; its random choices
 * are not pinned, so this is a restatement of the algorithm, not of its bits):
 *   start   : centroid c = x[(floor(c * n / k) + seed) mod n]
 *   assign  : nearest centroid under the canonical fp32 L2 distance, ties -> lower centroid
 *   update  : mean of the members, summed in fp64 in increasing vector index, rounded to fp32 once;
 *             a centroid without members keeps its value
 */
int orc_kmeans(int d, int64_t n, const float* x, int k, int niter, uint64_t seed, float* cent) {
    if (d <= 0 || n <= 0 || k <= 0 || niter < 0) return -1;
    for (int c = 0; c < k; ++c) {
        int64_t src = (int64_t)(((__int128)c * n) / k);
        src = (int64_t)(((uint64_t)src + seed) % (uint64_t)n);
        memcpy(cent + (int64_t)c * d, x + src * d, sizeof(float) * (size_t)d);
    }
    int32_t* assign = (int32_t*)malloc(sizeof(int32_t) * (size_t)n);
    double* sum = (double*)malloc(sizeof(double) * (size_t)k * d);
    int64_t* cnt = (int64_t*)malloc(sizeof(int64_t) * (size_t)k);
    if (!assign || !sum || !cnt) { free(assign); free(sum); free(cnt); return -2; }
    for (int it = 0; it < niter; ++it) {
        orc_ivf_assign(d, k, cent, n, x, assign);
        memset(sum, 0, sizeof(double) * (size_t)k * d);
        memset(cnt, 0, sizeof(int64_t) * (size_t)k);
        for (int64_t i = 0; i < n; ++i) {          /* increasing vector index: the summation order */
            const int32_t c = assign[i];
            cnt[c] += 1;
            for (int t = 0; t < d; ++t) sum[(int64_t)c * d + t] += (double)x[i * d + t];
        }
        for (int c = 0; c < k; ++c)
            if (cnt[c] > 0)
                for (int t = 0; t < d; ++t) cent[(int64_t)c * d + t] = (float)(sum[(int64_t)c * d + t] / (double)cnt[c]);
    }
    free(assign); free(sum); free(cnt);
    return 0;
}
