// tcgen05 / TMEM / TMA distance GEMM with fused selection epilogues, plus a plain CUDA-core
// variant that shares the epilogue code and serves as an on-device cross-check.
//
// Pipeline of the tcgen05 variant (one persistent CTA per SM, 320 or 576 threads):
//   warp 0 (one lane)  : TMA producer.  Per K chunk of 128 bytes: query box 128 x 128 B and base
//                        box 256 x 128 B into a 4-stage ring of 48 KB stages (SWIZZLE_128B).
//   warp 1 (one lane)  : issues tcgen05.mma 128 x 256 x (32 bytes of K) from shared-memory
//                        descriptors into one of two 256-column TMEM accumulators; commits free
//                        the stage (per chunk) and publish the accumulator (per tile).
//   warps 2-9 / 2-17   : epilogue, two or four warps per scheduler (see epi_warps).  Thread = (query
//                        row = TMEM lane, a half or a quarter of the tile's columns); reads 32
//                        columns at a time with tcgen05.ld (double-buffered) and applies the
//                        selection predicate (after the norm-add where the operands are not folded).
// Work items are (query block, base tile) pairs, query block fastest, so the CTAs running at
// the same time read the same base tiles and HBM sees each base tile about once per pass.
#include "dist_gemm.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "cos16.cuh"

#include <cstring>
#include <type_traits>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace b200 {
namespace {

constexpr int kMaxStages = 8;
// int8 with the fp16 cosine epilogue: a kernel instantiation of its own (chosen by launch_dist_gemm from
// GemmArgs::metric), so that the inner-product / L2 kernels carry none of its code
constexpr int kKindI8Cos = 3;
// int8 inner product: reads no norms, so its epilogue is light enough for sixteen warps of two
// chunks (96 registers) instead of eight of four -- the eight, two per scheduler, cannot hide their
// own instruction latency
constexpr int kKindI8IP = 4;
constexpr int kKindF16IP = 5;   // the same for fp16 operands
constexpr int kKindI8L2 = 6;    // sixteen-warp L2 kinds, see l2_global
constexpr int kKindF16L2 = 7;
__host__ __device__ constexpr bool is_i8(int kind) {
    return kind == kKindI8 || kind == kKindI8Cos || kind == kKindI8IP || kind == kKindI8L2;
}
__host__ __device__ constexpr bool ip_only(int kind) { return kind == kKindI8IP || kind == kKindF16IP; }
// L2 with sixteen epilogue warps as well: the norms are not staged in shared memory (which costs a
// barrier per item and 32 registers per chunk) but read from global memory where they are used --
// the 32 lanes of a warp want the same 32 norms, so a load is one broadcast that hits L1 after the
// first warp of the CTA has asked for it.
__host__ __device__ constexpr bool l2_global(int kind) { return kind == kKindI8L2 || kind == kKindF16L2; }
constexpr int kStageABytes = kTileQ * kChunkBytes;               // 16 KB
constexpr int kStageBBytes = kTileB * kChunkBytes;               // 32 KB
constexpr int kStageBytes = kStageABytes + kStageBBytes;         // 48 KB
constexpr int kGemmSmemBudget = 224 * 1024;                      // dynamic shared memory incl. 1 KB alignment slack
constexpr int kResidentMaxChunks = 4;                            // query tile kept in shared memory up to 64 KB
// Epilogue warps: two per scheduler, each thread draining half of a row's columns, where the
// epilogue is bound by shared-memory norm loads (fp16, int8); four per scheduler and a quarter
// of the columns each for the folded bf16 kind, whose short ALU-only epilogue is latency-bound
// and scales with the number of warps.
__host__ __device__ constexpr int epi_warps(int kind) {
    return (kind == kKindBF16 || ip_only(kind) || l2_global(kind) || kind == kKindI8Cos) ? 16 : 8;
}
// + the producer warp, the MMA warp and, behind the epilogue warps, a second MMA warp and a second
// producer warp (even and odd items have their own issuing threads and their own stage sub-ring)
__host__ __device__ constexpr int gemm_threads(int kind) { return 64 + 32 * epi_warps(kind) + 64; }
__host__ __device__ constexpr int mma2_warp(int kind) { return 2 + epi_warps(kind); }
__host__ __device__ constexpr int prod2_warp(int kind) { return 3 + epi_warps(kind); }
constexpr uint32_t kTmemCols = 512;
// Per-role cycle counters (GemmArgs::prof) exist in development builds only (-DB200IDX_DEV_PROF):
// the epilogue is bound by instruction issue, and even predicated-off clock reads cost slots.
#ifdef B200IDX_DEV_PROF
constexpr bool kDevProf = true;
#else
constexpr bool kDevProf = false;
#endif

template <typename AccT>
struct KeyOps;
template <>
struct KeyOps<float> {
    using Norm = float;
    static __device__ __forceinline__ float from_bits(uint32_t r) { return __uint_as_float(r); }
    static __device__ __forceinline__ float key(float acc, float bn, bool l2) { return l2 ? fmaf(-2.f, acc, bn) : -acc; }
    static __device__ __forceinline__ uint32_t ord(float k) { return float_to_ord(k); }
    static __device__ __forceinline__ float tau(uint32_t o) { return ord_to_float(o); }
    static __device__ __forceinline__ float worst() { return __int_as_float(0x7f800000); }
    // smallest value strictly above t (t itself when t = +inf): key <= t  <=>  key - above(t) < 0
    static __device__ __forceinline__ float above(float t) {
        return t == __int_as_float(0x7f800000) ? t : ord_to_float(float_to_ord(t) + 1u);
    }
    // sign word of (l2 ? bn - 2 acc : -acc) - tup
    static __device__ __forceinline__ uint32_t sign_l2(float acc, float bn, float tup) {
        return __float_as_uint(fmaf(-2.f, acc, bn) - tup);
    }
    static __device__ __forceinline__ uint32_t sign_ip(float acc, float ntup) { return __float_as_uint(ntup - acc); }
    static __device__ __forceinline__ float neg(float v) { return -v; }
};
template <>
struct KeyOps<int32_t> {
    using Norm = int32_t;
    static __device__ __forceinline__ int32_t from_bits(uint32_t r) { return static_cast<int32_t>(r); }
    static __device__ __forceinline__ int32_t key(int32_t acc, int32_t bn, bool l2) { return l2 ? bn - 2 * acc : -acc; }
    static __device__ __forceinline__ uint32_t ord(int32_t k) { return int_to_ord(k); }
    static __device__ __forceinline__ int32_t tau(uint32_t o) { return ord_to_int(o); }
    static __device__ __forceinline__ int32_t worst() { return 0x7fffffff; }
    static __device__ __forceinline__ int32_t above(int32_t t) { return t == 0x7fffffff ? t : t + 1; }
    static __device__ __forceinline__ uint32_t sign_l2(int32_t acc, int32_t bn, int32_t tup) {
        return static_cast<uint32_t>(bn - 2 * acc - tup);
    }
    static __device__ __forceinline__ uint32_t sign_ip(int32_t acc, int32_t ntup) {
        return static_cast<uint32_t>(ntup - acc);
    }
    static __device__ __forceinline__ int32_t neg(int32_t v) { return -v; }
};

constexpr uint32_t kCandBlock = 8;   // candidate slots a thread reserves with one atomic

// Shared-memory side of the epilogue: the tile's base norms, double-buffered with the TMEM
// accumulators (kinds whose operands are not folded).
struct EpiShared {
    uint32_t norm[2][kTileB];
};

// Per-thread (= query row x part of the tile's columns) epilogue state.
//   append mode : a thread reserves kCandBlock consecutive slots of its row's candidate list with
//                 ONE atomicAdd and fills them over as many tiles as it takes -- a CTA walks
//                 consecutive base tiles of the same query block, so the row stays the same.
//                 When the row changes (or the kernel ends) the unused slots of the open block are
//                 written as "invalid"; the consumers skip those.  counts[row] is therefore the
//                 number of RESERVED slots, an upper bound of the candidates.
//   direct mode : every key is written to cand[q][position] (no threshold, no atomics).
//   FOLD        : the operands carry 16 extra K columns (GemmArgs / kFoldCols), so the accumulator
//                 already holds  D = q.y - |y|^2/2 + tau/2  (L2; inner product: q.y + tau).  No
//                 norms are read and "key <= tau" is the sign of D: 32 columns are tested with a
//                 16-instruction AND tree, and the burst minimum of the key is a maximum of D.
// NCH: 32-column chunks a thread handles per tile.
template <typename AccT, int MODE, int BURST, bool FOLD, int NCH, bool COS = false, bool IPONLY = false>
struct RowEpilogue {
    using K = KeyOps<AccT>;
    const GemmArgs& a;
    int q;        // query row, valid when row_ok
    bool row_ok;
    bool l2;
    static constexpr bool cosm = COS;   // int8 cosine: the accumulators are turned into ordered fp16 scores first
    __half2 rq2;              // cosine: the row's query term
    AccT tau, tau_up;
    float tq;                 // FOLD append: the row's threshold, for the approximate key
    int blk_q;                // row of the open candidate block (-1: none)
    uint32_t blk_next, blk_left;
    uint32_t pre_base;        // a second block reserved ahead of need (its atomic is issued at the end of a
    bool pre_ok;              // tile and not read before the open block runs out, so nobody waits for it)
    uint32_t res[NCH * (32 / BURST)];   // burst-min results of this thread's part of the tile

    __device__ __forceinline__ explicit RowEpilogue(const GemmArgs& a_)
        : a(a_), q(-1), row_ok(false), l2(!IPONLY && a_.metric == kMetricL2),
          tau(AccT(0)), tau_up(AccT(0)), tq(0.f),
          blk_q(-1), blk_next(0), blk_left(0), pre_base(0), pre_ok(false) {}

    // 32 filter bits of this row for base positions col0 .. col0 + 31 (col0 is a multiple of 32).
    __device__ __forceinline__ uint32_t mask_word(int64_t col0) const {
        return __ldg(a.qmask + static_cast<int64_t>(q) * a.qmask_stride + (col0 >> 5));
    }

    // Fills what is left of the open block with the "invalid" marker.
    __device__ __forceinline__ void close_block() {
        if (blk_q >= 0) {
            uint64_t* crow = a.cand + static_cast<int64_t>(blk_q) * a.cap;
            for (uint32_t i = 0; i < blk_left; ++i)
                if (blk_next + i < a.cap) crow[blk_next + i] = kCandInvalid;
            if (pre_ok)
                for (uint32_t i = 0; i < kCandBlock; ++i)
                    if (pre_base + i < a.cap) crow[pre_base + i] = kCandInvalid;
        }
        blk_q = -1;
        blk_left = 0;
        pre_ok = false;
    }

    __device__ __forceinline__ void begin_tile(int q_, bool ok) {
        const bool new_row = q_ != q || ok != row_ok;
        if (MODE == kModeAppend && !a.direct && (q_ != blk_q || !ok)) close_block();
        q = q_;
        row_ok = ok;
        if (cosm && ok && new_row) {
            const int qn = a.seg_index ? q % a.nq : q;   // segmented base: candidate row -> query
            rq2 = cos16_query_term(__ldg(a.qnorm_i32 + qn));
        }
        if (MODE == kModeAppend && ok && new_row) {
            // once per run of tiles of the same row: the threshold, and (threshold mode) the first
            // candidate block -- reserved now, while the accumulator is still being computed, so
            // that the first candidate of the run does not wait for the atomic
            const uint32_t to = __ldg(a.tau + q);
            if (!a.direct && blk_q != q) {
                blk_next = atomicAdd(a.counts + q, kCandBlock);
                blk_left = kCandBlock;
                blk_q = q;
            }
            if (FOLD && !a.direct) {
                tq = ord_to_float(to);
            } else {
                tau = K::tau(to);
                tau_up = K::above(tau);
            }
        }
    }

    __device__ __forceinline__ void append(uint64_t e) {
        if (blk_left == 0) {
            if (pre_ok) {
                blk_next = pre_base;
                pre_ok = false;
            } else {
                blk_next = atomicAdd(a.counts + q, kCandBlock);   // first block of a run, or a burst of candidates
            }
            blk_left = kCandBlock;
            blk_q = q;
        }
        if (blk_next < a.cap) a.cand[static_cast<int64_t>(q) * a.cap + blk_next] = e;
        ++blk_next;
        --blk_left;
    }

    // Value of r[c] for a run-time c without indexing registers dynamically (select tree).
    static __device__ __forceinline__ uint32_t pick(const uint32_t (&r)[32], uint32_t c) {
        uint32_t v16[16], v8[8], v4[4], v2[2];
#pragma unroll
        for (int i = 0; i < 16; ++i) v16[i] = (c & 16u) ? r[16 + i] : r[i];
#pragma unroll
        for (int i = 0; i < 8; ++i) v8[i] = (c & 8u) ? v16[8 + i] : v16[i];
#pragma unroll
        for (int i = 0; i < 4; ++i) v4[i] = (c & 4u) ? v8[4 + i] : v8[i];
#pragma unroll
        for (int i = 0; i < 2; ++i) v2[i] = (c & 2u) ? v4[2 + i] : v4[i];
        return (c & 1u) ? v2[1] : v2[0];
    }

    // Folded operands: r holds D for 32 columns.
    // ci: index of the chunk inside this thread's part of the tile (a constant after unrolling)
    __device__ __forceinline__ void chunk_fold(const uint32_t (&r)[32], int64_t col0, int nvalid, int ci, int64_t cbase) {
        if (!row_ok && (MODE == kModeBurstMin || a.direct)) return;
        if (MODE == kModeBurstMin) {
            constexpr int NB = 32 / BURST;
            const float ninf = __int_as_float(0xff800000);
            // min / max and selects share the half-rate integer pipe, which is what bounds this
            // epilogue: the test for rows past the end of the base is kept out of the common path.
            uint32_t keep = nvalid >= 32 ? 0xFFFFFFFFu : ((1u << nvalid) - 1u);   // bit c: column c takes part
            if (a.qmask) keep &= mask_word(col0);
            const bool full = keep == 0xFFFFFFFFu;
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                float v[BURST];
                if (full) {
#pragma unroll
                    for (int j = 0; j < BURST; ++j) v[j] = __uint_as_float(r[b * BURST + j]);
                } else {
#pragma unroll
                    for (int j = 0; j < BURST; ++j) {
                        const int c = b * BURST + j;
                        v[j] = ((keep >> c) & 1u) ? __uint_as_float(r[c]) : ninf;
                    }
                }
#pragma unroll
                for (int w = BURST / 2; w > 0; w >>= 1)
#pragma unroll
                    for (int j = 0; j < w; ++j) v[j] = fmaxf(v[j], v[j + w]);   // NaN never wins
                const float key = l2 ? -2.f * v[0] : -v[0];
                res[ci * NB + b] = float_to_ord(key);
            }
        } else if (a.direct) {
            uint64_t* crow = a.cand + static_cast<int64_t>(q) * a.cap + (col0 - cbase);
            uint32_t keep = nvalid >= 32 ? 0xFFFFFFFFu : ((1u << nvalid) - 1u);
            if (a.qmask) keep &= mask_word(col0);
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                const float dv = __uint_as_float(r[c]);
                const float key = l2 ? -2.f * dv : -dv;
                // NaN keys are left at the buffer's "invalid" fill
                if (((keep >> c) & 1u) && key <= tau) crow[c] = pack_cand(float_to_ord(key), static_cast<uint32_t>(col0 + c));
            }
        } else {
            // (the tcgen05 kernel calls fold_mask / fold_extract itself, with the accumulator handed
            // back in between; this is the path of the CUDA-core variant)
            const uint32_t m = fold_mask(r, col0, nvalid);
            fold_extract(r, m, col0);
        }
    }

    // Folded operands, append mode, split in two so that the accumulator can be handed back between
    // them.  fold_mask: bit (31 - c) of the result = column c of this lane's row passes (D >= 0, a
    // real base row, not filtered out); warp-collective, 0 for everybody when no lane has a hit.
    __device__ __forceinline__ uint32_t fold_mask(const uint32_t (&r)[32], int64_t col0, int nvalid) {
        uint32_t t[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) t[i] = r[2 * i] & r[2 * i + 1];
#pragma unroll
        for (int w = 8; w > 0; w >>= 1)
#pragma unroll
            for (int i = 0; i < w; ++i) t[i] &= t[i + w];
        const bool hit = row_ok && static_cast<int32_t>(t[0]) >= 0;   // not every D negative
        if (!__any_sync(0xFFFFFFFFu, hit)) return 0u;
        uint32_t m0 = 0, m1 = 0;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            m0 = __funnelshift_l(r[c], m0, 1);
            m1 = __funnelshift_l(r[16 + c], m1, 1);
        }
        uint32_t mask = ~((m0 << 16) | (m1 & 0xFFFFu));
        mask &= nvalid >= 32 ? 0xFFFFFFFFu : ~(0xFFFFFFFFu >> nvalid);
        if (a.qmask && row_ok) mask &= __brev(mask_word(col0));
        return hit ? mask : 0u;
    }
    // fold_extract: appends the columns of `mask` from the registers (select tree; no TMEM access).
    __device__ __forceinline__ void fold_extract(const uint32_t (&r)[32], uint32_t mask, int64_t col0) {
        while (mask) {
            const uint32_t c = __clz(mask);
            mask &= ~(0x80000000u >> c);
            const float dv = __uint_as_float(pick(r, c));
            if (!(dv >= 0.f)) continue;   // NaN
            const float key = l2 ? fmaf(-2.f, dv, tq) : tq - dv;
            append(pack_cand(float_to_ord(key), static_cast<uint32_t>(col0 + c)));
        }
    }

    // The same split for an inner product without folded operands and without norms (int8): bit
    // (31 - c) = column c has key = -acc <= tau.
    __device__ __forceinline__ uint32_t ip_mask(const uint32_t (&r)[32], int64_t col0, int nvalid) {
        const AccT ntup = K::neg(tau_up);
        uint32_t m0 = 0, m1 = 0;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            m0 = __funnelshift_l(K::sign_ip(K::from_bits(r[c]), ntup), m0, 1);
            m1 = __funnelshift_l(K::sign_ip(K::from_bits(r[16 + c]), ntup), m1, 1);
        }
        uint32_t mask = (m0 << 16) | (m1 & 0xFFFFu);
        uint32_t valid = nvalid >= 32 ? 0xFFFFFFFFu : ((1u << nvalid) - 1u);
        if (a.qmask && row_ok) valid &= mask_word(col0);
        return row_ok ? (mask & __brev(valid)) : 0u;
    }
    __device__ __forceinline__ void ip_extract(const uint32_t (&r)[32], uint32_t mask, int64_t col0) {
        while (mask) {
            const uint32_t c = __clz(mask);
            mask &= ~(0x80000000u >> c);
            const AccT key = K::neg(K::from_bits(pick(r, c)));
            if (!(key <= tau)) continue;
            append(pack_cand(K::ord(key), static_cast<uint32_t>(col0 + c)));
        }
    }

    // ... and for L2 with the norms taken from global memory (gn: the norms of the chunk's 32 columns)
    __device__ __forceinline__ uint32_t l2_mask(const uint32_t (&r)[32], const uint32_t* gn, int64_t col0, int nvalid) {
        uint32_t m0 = 0, m1 = 0;
        const uint4* g4 = reinterpret_cast<const uint4*>(gn);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const uint4 na = __ldg(g4 + g), nb4 = __ldg(g4 + 4 + g);
            m0 = __funnelshift_l(K::sign_l2(K::from_bits(r[4 * g + 0]), K::from_bits(na.x), tau_up), m0, 1);
            m0 = __funnelshift_l(K::sign_l2(K::from_bits(r[4 * g + 1]), K::from_bits(na.y), tau_up), m0, 1);
            m0 = __funnelshift_l(K::sign_l2(K::from_bits(r[4 * g + 2]), K::from_bits(na.z), tau_up), m0, 1);
            m0 = __funnelshift_l(K::sign_l2(K::from_bits(r[4 * g + 3]), K::from_bits(na.w), tau_up), m0, 1);
            m1 = __funnelshift_l(K::sign_l2(K::from_bits(r[16 + 4 * g + 0]), K::from_bits(nb4.x), tau_up), m1, 1);
            m1 = __funnelshift_l(K::sign_l2(K::from_bits(r[16 + 4 * g + 1]), K::from_bits(nb4.y), tau_up), m1, 1);
            m1 = __funnelshift_l(K::sign_l2(K::from_bits(r[16 + 4 * g + 2]), K::from_bits(nb4.z), tau_up), m1, 1);
            m1 = __funnelshift_l(K::sign_l2(K::from_bits(r[16 + 4 * g + 3]), K::from_bits(nb4.w), tau_up), m1, 1);
        }
        uint32_t mask = (m0 << 16) | (m1 & 0xFFFFu);
        uint32_t valid = nvalid >= 32 ? 0xFFFFFFFFu : ((1u << nvalid) - 1u);
        if (a.qmask && row_ok) valid &= mask_word(col0);
        return row_ok ? (mask & __brev(valid)) : 0u;
    }
    __device__ __forceinline__ void l2_extract(const uint32_t (&r)[32], uint32_t mask, int64_t col0, const uint32_t* gn) {
        while (mask) {
            const uint32_t c = __clz(mask);
            mask &= ~(0x80000000u >> c);
            const AccT key = K::key(K::from_bits(pick(r, c)), K::from_bits(__ldg(gn + c)), true);
            if (!(key <= tau)) continue;   // NaN
            append(pack_cand(K::ord(key), static_cast<uint32_t>(col0 + c)));
        }
    }

    // r: 32 accumulator columns; nb: the matching 32 norms in shared memory; col0: base position
    // of r[0]; nvalid: real base rows among the 32; bslot: first burst slot (burst-min mode);
    // ci: see chunk_fold.  The hot path is straight-line code: the threshold test of the 32
    // columns is folded into a bit mask, and only a non-zero mask (rare) enters the compact
    // candidate loop.
    // cbase: position of the first base row of the segment the tile belongs to (0 without segments)
    __device__ __forceinline__ void chunk(uint32_t (&r)[32], const uint32_t* nb, int64_t col0, int nvalid,
                                          int bslot, int ci, int64_t cbase) {
        if (FOLD) {
            chunk_fold(r, col0, nvalid, ci, cbase);
            return;
        }
        if (!row_ok) return;
        if (cosm) cos_scores(r, nb);
        chunk_keys(r, nb, col0, nvalid, bslot, ci, cbase);
    }

    // nb holds the base rows' fp16 reciprocal norms; the accumulators become ordered scores in place,
    // and from here on they are treated as inner products
    __device__ __forceinline__ void cos_scores(uint32_t (&r)[32], const uint32_t* nb) const {
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
            int32_t s0, s1;
            cos16_pair(static_cast<int32_t>(r[c]), static_cast<int32_t>(r[c + 1]), nb[c], nb[c + 1], rq2, s0, s1);
            r[c] = static_cast<uint32_t>(s0);
            r[c + 1] = static_cast<uint32_t>(s1);
        }
    }

    __device__ __forceinline__ void chunk_keys(const uint32_t (&r)[32], const uint32_t* nb, int64_t col0, int nvalid,
                                               int bslot, int ci, int64_t cbase) {
        // The norms (L2) are taken eight at a time, next to their use: nb may point into shared or
        // into global memory, and 32 of them held in registers beside the 32 accumulator words are
        // what a 96-register kernel cannot afford.
        const uint4* np4 = reinterpret_cast<const uint4*>(nb);
        auto norms8 = [&](int s8, uint32_t (&n8)[8]) {
            if (l2) {
                const uint4 x = np4[2 * s8], y = np4[2 * s8 + 1];
                n8[0] = x.x; n8[1] = x.y; n8[2] = x.z; n8[3] = x.w;
                n8[4] = y.x; n8[5] = y.y; n8[6] = y.z; n8[7] = y.w;
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) n8[j] = 0u;   // +0.0f / 0
            }
        };
        uint32_t valid = nvalid >= 32 ? 0xFFFFFFFFu : ((1u << nvalid) - 1u);
        if (a.qmask) valid &= mask_word(col0);
        if (MODE == kModeBurstMin) {
            uint32_t* dst = a.mins + static_cast<int64_t>(q) * a.mins_stride + bslot;
            const bool full = valid == 0xFFFFFFFFu;
            AccT m[4] = {K::worst(), K::worst(), K::worst(), K::worst()};   // independent chains
#pragma unroll
            for (int s8 = 0; s8 < 4; ++s8) {
                uint32_t n8[8];
                norms8(s8, n8);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int c = s8 * 8 + j;
                    const AccT key = K::key(K::from_bits(r[c]), K::from_bits(n8[j]), l2);
                    if (full || ((valid >> c) & 1u)) m[j & 3] = key < m[j & 3] ? key : m[j & 3];
                }
                if (BURST == 8 || s8 == 3) {   // a burst of 8 ends with every group, a burst of 32 with the last
                    const AccT ma = m[0] < m[1] ? m[0] : m[1], mb = m[2] < m[3] ? m[2] : m[3];
                    dst[BURST == 8 ? s8 : 0] = K::ord(ma < mb ? ma : mb);
#pragma unroll
                    for (int i = 0; i < 4; ++i) m[i] = K::worst();
                }
            }
        } else if (a.direct) {
            uint64_t* crow = a.cand + static_cast<int64_t>(q) * a.cap + (col0 - cbase);
#pragma unroll
            for (int s8 = 0; s8 < 4; ++s8) {
                uint32_t n8[8];
                norms8(s8, n8);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int c = s8 * 8 + j;
                    const AccT key = K::key(K::from_bits(r[c]), K::from_bits(n8[j]), l2);
                    // NaN keys are left at the buffer's "invalid" fill
                    if (((valid >> c) & 1u) && key <= tau) crow[c] = pack_cand(K::ord(key), static_cast<uint32_t>(col0 + c));
                }
            }
        } else {
            // bit (31 - c) of mask = "column c passes": the sign of key - above(tau), shifted in
            // with one funnel shift per column (two independent chains for the scheduler).
            uint32_t m0 = 0, m1 = 0;
            if (l2) {
#pragma unroll
                for (int s8 = 0; s8 < 2; ++s8) {
                    uint32_t na[8], nc[8];
                    norms8(s8, na);
                    norms8(s8 + 2, nc);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        m0 = __funnelshift_l(K::sign_l2(K::from_bits(r[s8 * 8 + j]), K::from_bits(na[j]), tau_up), m0, 1);
                        m1 = __funnelshift_l(K::sign_l2(K::from_bits(r[16 + s8 * 8 + j]), K::from_bits(nc[j]), tau_up), m1, 1);
                    }
                }
            } else {
                const AccT ntup = K::neg(tau_up);
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    m0 = __funnelshift_l(K::sign_ip(K::from_bits(r[c]), ntup), m0, 1);
                    m1 = __funnelshift_l(K::sign_ip(K::from_bits(r[16 + c]), ntup), m1, 1);
                }
            }
            uint32_t mask = (m0 << 16) | (m1 & 0xFFFFu);
            mask &= __brev(valid);   // rows past the end of the base, rows the filter excludes
            while (mask) {
                const uint32_t c = __clz(mask);
                mask &= ~(0x80000000u >> c);
                const AccT key = K::key(K::from_bits(pick(r, c)), K::from_bits(l2 ? nb[c] : 0u), l2);
                if (!(key <= tau)) continue;   // NaN
                append(pack_cand(K::ord(key), static_cast<uint32_t>(col0 + c)));
            }
        }
    }

    // hslot: first burst slot of this thread's part of the tile (burst-min mode)
    __device__ __forceinline__ void end_tile(int hslot) {
        if (MODE == kModeAppend && !a.direct && row_ok && blk_q == q && !pre_ok && blk_left <= kCandBlock / 2) {
            pre_base = atomicAdd(a.counts + q, kCandBlock);
            pre_ok = true;
        }
        if (MODE == kModeBurstMin && FOLD && row_ok) {
            // 16-byte (or 8-byte) stores instead of scattered words
            uint32_t* dst = a.mins + static_cast<int64_t>(q) * a.mins_stride + hslot;
            constexpr int NW = NCH * (32 / BURST);
            if (NW % 4 == 0) {
#pragma unroll
                for (int i = 0; i < NW / 4; ++i)
                    reinterpret_cast<uint4*>(dst)[i] = make_uint4(res[4 * i], res[4 * i + 1], res[4 * i + 2], res[4 * i + 3]);
            } else {
#pragma unroll
                for (int i = 0; i < NW / 2; ++i) reinterpret_cast<uint2*>(dst)[i] = make_uint2(res[2 * i], res[2 * i + 1]);
            }
        }
    }

    __device__ __forceinline__ void finish() {
        if (MODE == kModeAppend && !a.direct) close_block();
    }
};

__device__ __forceinline__ int tile_of(const GemmArgs& a, int sel) {
    if (a.tile_first >= 0) return a.tile_first + sel;   // a contiguous stretch of tiles (whole base: first = 0)
    return static_cast<int>(static_cast<int64_t>(sel) * a.n_tiles_total / a.n_tiles_sel);
}

// Work of one CTA: a contiguous range of the (query block, base tile) items in query-block-major
// order.  Consecutive items of a CTA share the query block, which is what lets the query tile stay
// in shared memory and a thread keep one candidate block open across tiles.  With few query blocks
// and a base larger than L2 the ranges are aligned (see below) so that CTAs of different query
// blocks walk the same base tiles at the same time and a base tile is read from HBM about once;
// otherwise the linearised item list is simply cut into equal pieces.
struct ItemRange {
    int64_t count;       // items of this CTA
    int qb0, sel0;       // first item
    int n_sel;
    __device__ __forceinline__ ItemRange(const GemmArgs& a, int n_qb) {
        n_sel = a.n_tiles_sel;
        const int G = gridDim.x, c = blockIdx.x;
        if (a.aligned_ranges) {
            // one query block per CTA; the CTAs of a query block split the tiles evenly, so CTAs of
            // different query blocks sit on the same stretch of the base at the same time
            const int qb = c % n_qb, j = c / n_qb;
            const int nl = G / n_qb + (qb < G % n_qb ? 1 : 0);
            const int64_t lo = static_cast<int64_t>(n_sel) * j / nl;
            const int64_t hi = static_cast<int64_t>(n_sel) * (j + 1) / nl;
            count = hi - lo;
            qb0 = qb;
            sel0 = static_cast<int>(lo);
        } else {
            const int64_t total = static_cast<int64_t>(n_qb) * n_sel;
            const int64_t lo = total * c / G;
            const int64_t hi = total * (c + 1) / G;
            count = hi - lo;
            qb0 = static_cast<int>(lo / n_sel);
            sel0 = static_cast<int>(lo % n_sel);
        }
    }
};
// Walks a range without divisions (the roles that run one thread deep cannot afford them).
struct ItemCursor {
    int qb, sel;
    int n_sel;
    __device__ __forceinline__ explicit ItemCursor(const ItemRange& r) : qb(r.qb0), sel(r.sel0), n_sel(r.n_sel) {}
    __device__ __forceinline__ void next() {
        if (++sel == n_sel) {
            sel = 0;
            ++qb;
        }
    }
    __device__ __forceinline__ bool last_of_qb() const { return sel + 1 == n_sel; }
};

// ---------------------------------------------------------------------------------------
// tcgen05 variant
// ---------------------------------------------------------------------------------------
// Shared memory is the scarce resource of this kernel: a 128 x 256 x 16 UMMA reads 12 KB of
// operands, and with K of a few hundred every operand byte that TMA writes is read about once, so
// TMA writes and UMMA reads together are bounded by the 128 B/clk of the shared-memory pipe.  When
// the query tile is small enough (a.a_resident) it is therefore loaded once per query block and
// only base chunks (32 KB) travel through the stage ring.
template <int KIND, int MODE, int BURST>
__global__ void __launch_bounds__(gemm_threads(KIND), 1)
dist_gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                    const GemmArgs a) {
    using AccT = typename std::conditional<is_i8(KIND), int32_t, float>::type;
    constexpr int kElemBytes = is_i8(KIND) ? 1 : 2;
    constexpr int kChunkElems = kChunkBytes / kElemBytes;
    constexpr bool FOLD = KIND == kKindBF16;
    constexpr uint32_t kIdesc = is_i8(KIND) ? ptx::umma_idesc(2, 1, kTileQ, kTileB)
                                                : ptx::umma_idesc(1, KIND == kKindBF16 ? 1 : 0, kTileQ, kTileB);

    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[kMaxStages];
    __shared__ uint64_t bar_empty[kMaxStages];
    __shared__ uint64_t bar_acc_full[2];
    __shared__ uint64_t bar_acc_empty[2];
    __shared__ uint64_t bar_a_full;      // resident query tile landed
    __shared__ uint64_t bar_a_free;      // every UMMA that read the resident query tile has completed
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    __shared__ __align__(16) EpiShared epi_sh;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // Packed operands (bf16 kind only): the query tile and a base tile are one contiguous image each;
    // an item is ONE stage of its parity's sub-ring (nst = 1) and ONE hand-off per role.
    const bool packed = KIND == kKindBF16 && a.packed != 0;
    const uint32_t a_img_bytes = static_cast<uint32_t>(kTileQ) * a.d * 2u;
    const int nkc = packed ? 1 : (a.d + kChunkElems - 1) / kChunkElems;
    const bool resident = a.a_resident != 0;
    const int nst = a.n_stages / 2;          // stages per sub-ring (even / odd items)
    const uint32_t stage_bytes = packed ? static_cast<uint32_t>(kTileB) * a.d * 2u : (resident ? kStageBBytes : kStageBytes);
    uint8_t* ring = smem + (packed ? ((a_img_bytes + 1023u) & ~1023u) : (resident ? nkc * kStageABytes : 0));

    if (threadIdx.x == 0) {
        for (int r = 0; r < 2; ++r)
            for (int s = 0; s < nst; ++s) {
                ptx::mbar_init(&bar_full[r * (kMaxStages / 2) + s], 1);
                ptx::mbar_init(&bar_empty[r * (kMaxStages / 2) + s], 1);
            }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(&bar_acc_full[b], 1);
            ptx::mbar_init(&bar_acc_empty[b], epi_warps(KIND));
        }
        ptx::mbar_init(&bar_a_full, 1);
        ptx::mbar_init(&bar_a_free, 2);   // both MMA-issuing threads
        abort_flag = 0;
        ptx::mbar_fence_init();
        if (!packed) {
            ptx::prefetch_tensormap(&mapA);
            ptx::prefetch_tensormap(&mapB);
        }
    }
    if (warp == 1) {
        ptx::tmem_alloc(&tmem_base_slot, kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    const int n_qb = (a.nq + kTileQ - 1) / kTileQ;
    const ItemRange range(a, n_qb);

    if (warp == 0 || warp == prod2_warp(KIND)) {
        if (lane == 0) {
            const uint32_t pidx = warp == 0 ? 0u : 1u;   // this producer serves the items of this parity
            // Two sub-rings of nst / 2 stages: even items travel through the first, odd items through
            // the second, so that each ring's barriers have exactly one consuming thread (a consumer a
            // whole revolution ahead of the other would otherwise read a parity that has not happened).
            // The resident query tile is loaded by producer 0.
            int rs = 0;
            uint32_t rph = 0;
            int cur_qb = -1;
            uint32_t a_loads = 0, t = 0;
            bool ok = true;
            long long pw = 0;
            const bool prof_on = kDevProf && a.prof && pidx == 0;
            const long long k0 = prof_on ? clock64() : 0;
            const uint32_t r = pidx;
            ItemCursor cur(range);
            for (int64_t i = 0; i < range.count && ok; ++i, ++t, cur.next()) {
                const int qb = cur.qb;
                if (resident && pidx == 0 && qb != cur_qb) {
                    // the previous query block's UMMAs must be done with the tile before it is overwritten
                    if (a_loads && !ptx::mbar_wait_bounded(&bar_a_free, (a_loads - 1u) & 1u, &abort_flag)) { ok = false; break; }
                    if (packed) {
                        ptx::mbar_expect_tx(&bar_a_full, a_img_bytes);
                        ptx::bulk_load_1d(smem, static_cast<const uint8_t*>(a.A) + static_cast<size_t>(qb) * a_img_bytes,
                                          a_img_bytes, &bar_a_full);
                    } else {
                        ptx::mbar_expect_tx(&bar_a_full, static_cast<uint32_t>(nkc) * kStageABytes);
                        for (int kc = 0; kc < nkc; ++kc)
                            ptx::tma_load_2d(smem + kc * kStageABytes, &mapA, &bar_a_full, kc * kChunkElems, qb * kTileQ);
                    }
                    ++a_loads;
                    cur_qb = qb;
                }
                if ((t & 1u) != pidx) continue;
                const int tile = tile_of(a, cur.sel);
                for (int kc = 0; kc < nkc; ++kc) {
                    const int s = rs;
                    uint64_t* full = &bar_full[r * (kMaxStages / 2) + s];
                    const long long w0 = prof_on ? clock64() : 0;
                    if (!ptx::mbar_wait_bounded(&bar_empty[r * (kMaxStages / 2) + s], rph ^ 1u, &abort_flag)) { ok = false; break; }
                    if (prof_on) pw += clock64() - w0;
                    ptx::mbar_expect_tx(full, stage_bytes);
                    uint8_t* st = ring + static_cast<size_t>(r * nst + s) * stage_bytes;
                    if (packed) {
                        ptx::bulk_load_1d(st, static_cast<const uint8_t*>(a.B) + static_cast<size_t>(tile) * stage_bytes,
                                          stage_bytes, full);
                        if (++rs == nst) { rs = 0; rph ^= 1u; }
                        continue;
                    }
                    if (!resident) {
                        ptx::tma_load_2d(st, &mapA, full, kc * kChunkElems, qb * kTileQ);
                        st += kStageABytes;
                    }
                    ptx::tma_load_2d(st, &mapB, full, kc * kChunkElems, tile * kTileB);
                    if (++rs == nst) { rs = 0; rph ^= 1u; }
                }
                if (kDevProf && a.trace && blockIdx.x == 0 && t < 64) a.trace[0 * 64 + t] = clock64();
            }
            if (prof_on) {
                atomicAdd(a.prof + 0, static_cast<unsigned long long>(pw));
                atomicAdd(a.prof + 7, static_cast<unsigned long long>(clock64() - k0));
            }
        }
    } else if (warp == 1 || warp == mma2_warp(KIND)) {
        // Two threads issue the UMMAs, one for the even items (accumulator 0) and one for the odd
        // items (accumulator 1), on different schedulers: a single issuing thread, sharing its
        // scheduler with busy epilogue warps, could not keep the tensor pipe fed.  Both walk the
        // whole item list so that their view of the query-block runs agrees; each consumes its own
        // sub-ring of stages.
        if (lane == 0) {
            const uint32_t parity = warp == 1 ? 0u : 1u;
            const bool prof_on = kDevProf && a.prof && parity == 0;
            int s = 0;
            uint32_t ph = 0, t = 0;
            int cur_qb = -1;
            uint32_t a_seen = 0;
            bool ok = true;
            long long mw0 = 0, mw1 = 0;
            // Descriptors differ only in their 14-bit address field: build the constant part once
            // and add byte offsets / 16 (the single issuing thread is on the critical path).
            const uint64_t desc_hi = ptx::umma_desc_k_sw128(0);
            // packed operands: core matrices adjacent along K are 128 bytes apart, 8-row groups a.d / 8 of them
            const uint64_t desc_hi_p = ptx::umma_desc_k_plain(0, 128u, static_cast<uint32_t>(a.d) * 16u);
            const uint32_t a_res_lo = (ptx::smem_u32(smem) & 0x3FFFFu) >> 4;
            const uint32_t ring_lo = (ptx::smem_u32(ring) & 0x3FFFFu) >> 4;
            const uint32_t stage_lo = stage_bytes >> 4;
            const int tail_bytes = a.d * kElemBytes - (nkc - 1) * kChunkBytes;   // bytes of K in the last chunk
            const int tail_nks = tail_bytes >= kChunkBytes ? kChunkBytes / 32 : (tail_bytes + 31) / 32;
            ItemCursor cur(range);
            for (int64_t i = 0; i < range.count && ok; ++i, ++t, cur.next()) {
                const int qb = cur.qb;
                if (resident && qb != cur_qb) {
                    if (!ptx::mbar_wait_bounded(&bar_a_full, a_seen & 1u, &abort_flag)) { ok = false; break; }
                    ++a_seen;
                    cur_qb = qb;
                }
                const bool run_ends = resident && (i + 1 == range.count || cur.last_of_qb());
                if ((t & 1u) != parity) {
                    // the other thread's item (it travels through the other sub-ring)
                    if (run_ends) ptx::umma_commit(&bar_a_free);   // nothing of this run left on this thread
                    continue;
                }
                const uint32_t ab = parity;
                const uint32_t aph = (t >> 1) & 1u;
                long long w0 = prof_on ? clock64() : 0;
                if (!ptx::mbar_wait_bounded(&bar_acc_empty[ab], aph ^ 1u, &abort_flag)) { ok = false; break; }
                if (prof_on) mw0 += clock64() - w0;
                if (kDevProf && a.trace && blockIdx.x == 0 && t < 64) a.trace[1 * 64 + t] = clock64();
                ptx::tc_fence_after();
                const uint32_t tacc = tmem_base + ab * kTileB;
                for (int kc = 0; kc < nkc; ++kc) {
                    w0 = prof_on ? clock64() : 0;
                    if (!ptx::mbar_wait_bounded(&bar_full[parity * (kMaxStages / 2) + s], ph, &abort_flag)) { ok = false; break; }
                    if (prof_on) mw1 += clock64() - w0;
                    if (kDevProf && a.trace && blockIdx.x == 0 && t < 64 && kc + 1 == nkc) a.trace[2 * 64 + t] = clock64();
                    ptx::tc_fence_after();
                    const uint32_t st_lo = ring_lo + (parity * static_cast<uint32_t>(nst) + static_cast<uint32_t>(s)) * stage_lo;
                    if (packed) {
                        // K / 16 steps of one 128 x 256 x 16 UMMA; a step advances both images by two core matrices
                        const int nks_p = a.d >> 4;
                        for (int ks = 0; ks < nks_p; ++ks) {
                            const uint64_t da = desc_hi_p | static_cast<uint64_t>(a_res_lo + ks * 16);
                            const uint64_t db = desc_hi_p | static_cast<uint64_t>(st_lo + ks * 16);
                            ptx::umma_f16(tacc, da, db, kIdesc, ks > 0 ? 1u : 0u);
                        }
                        ptx::umma_commit(&bar_empty[parity * (kMaxStages / 2) + s]);
                        if (++s == nst) { s = 0; ph ^= 1u; }
                        continue;
                    }
                    const uint32_t sa_lo = resident ? a_res_lo + static_cast<uint32_t>(kc) * (kStageABytes >> 4) : st_lo;
                    const uint32_t sb_lo = resident ? st_lo : st_lo + (kStageABytes >> 4);
                    // the last chunk may hold fewer than four 32-byte K steps (the rest is zero fill)
                    const int nks = kc + 1 == nkc ? tail_nks : kChunkBytes / 32;
#pragma unroll
                    for (int ks = 0; ks < kChunkBytes / 32; ++ks) {
                        if (ks >= nks) break;
                        const uint64_t da = desc_hi | static_cast<uint64_t>(sa_lo + ks * 2);
                        const uint64_t db = desc_hi | static_cast<uint64_t>(sb_lo + ks * 2);
                        const uint32_t accum = (kc > 0 || ks > 0) ? 1u : 0u;
                        if (kDevProf && (a.dbg & 4)) continue;
                        if (is_i8(KIND)) ptx::umma_i8(tacc, da, db, kIdesc, accum);
                        else ptx::umma_f16(tacc, da, db, kIdesc, accum);
                    }
                    ptx::umma_commit(&bar_empty[parity * (kMaxStages / 2) + s]);
                    if (++s == nst) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                ptx::umma_commit(&bar_acc_full[ab]);
                if (kDevProf && a.trace && blockIdx.x == 0 && t < 64) a.trace[3 * 64 + t] = clock64();
                // last item of this CTA for the query block: the resident tile may be replaced once
                // everything both threads issued so far has completed
                if (run_ends) ptx::umma_commit(&bar_a_free);
            }
            if (prof_on) {
                atomicAdd(a.prof + 1, static_cast<unsigned long long>(mw0));
                atomicAdd(a.prof + 2, static_cast<unsigned long long>(mw1));
            }
        }
    } else {
        const int quarter = warp & 3;          // TMEM lane quarter this warp may read
        const int half = (warp - 2) >> 2;      // which kCols columns of the tile this warp drains
        const int row_in_tile = quarter * 32 + lane;
        const int et = threadIdx.x - 64;       // epilogue thread index
        constexpr int kCols = kTileB / (epi_warps(KIND) / 4);   // columns per epilogue thread
        RowEpilogue<AccT, MODE, BURST, FOLD, kCols / 32, KIND == kKindI8Cos, ip_only(KIND)> epi(a);
        // FOLD, plain inner products: no norms; sixteen-warp L2: norms read where they are used
        const bool l2 = a.metric == kMetricL2 && !FOLD && !ip_only(KIND) && !l2_global(KIND);
        constexpr bool cosm = KIND == kKindI8Cos;
        const uint32_t* gnorm = static_cast<const uint32_t*>(a.bnorm);
        uint32_t t = 0;
        bool ok = true;
        long long ew = 0, ec = 0, ef = 0, elw = 0, ebar = 0, ecc = 0;
        const bool profiler = kDevProf && a.prof && warp == 2 && lane == 0;
        ItemCursor cur(range);
        for (int64_t i = 0; i < range.count && ok; ++i, ++t, cur.next()) {
            const int qb = cur.qb;
            const int sel = cur.sel;
            const int tile = tile_of(a, sel);
            const uint32_t ab = t & 1u;
            const uint32_t aph = (t >> 1) & 1u;
            const int q_in = qb * kTileQ + row_in_tile;
            const int64_t tile_col0 = static_cast<int64_t>(tile) * kTileB;
            // segmented base: the tile's index decides the candidate row and the valid extent
            int q = q_in;
            int64_t cbase = 0, n_end = a.N;
            if (a.seg_index) {
                q += (__ldg(a.seg_index + tile) - a.seg_first) * a.nq;
                cbase = __ldg(a.seg_col0 + tile);
                n_end = __ldg(a.seg_end + tile);
            }
            const long long e0 = profiler ? clock64() : 0;
            // The tile's norms travel global -> registers while the MMA is still running.
            uint32_t n0 = 0;
            if ((l2 || cosm) && et < kTileB) {
                n0 = __ldg(gnorm + tile_col0 + et);
                if (cosm) n0 = cos16_rnorm_bits(static_cast<int32_t>(n0));
            }
            epi.begin_tile(q, q_in < a.nq);
            if (!ptx::mbar_wait_bounded(&bar_acc_full[ab], aph, &abort_flag)) {
                // leave without stranding a sibling warp at the named barrier below
                if (!FOLD && (l2 || cosm)) asm volatile("bar.arrive 1, %0;" ::"n"(32 * epi_warps(KIND)) : "memory");
                ok = false;
                break;
            }
            const long long e1 = profiler ? clock64() : 0;
            if (kDevProf && a.trace && blockIdx.x == 0 && t < 64 && lane == 0 && (warp == 2 || warp == 2 + epi_warps(KIND) - 1))
                a.trace[(warp == 2 ? 4 : 6) * 64 + t] = clock64();
            ptx::tc_fence_after();
            const long long b0 = profiler ? clock64() : 0;
            if (!FOLD && (l2 || cosm)) {   // inner product: no norms, and no reason to keep the warps in step
                if (et < kTileB) epi_sh.norm[ab][et] = n0;
                asm volatile("bar.sync 1, %0;" ::"n"(32 * epi_warps(KIND)) : "memory");   // the epilogue warps
            }
            if (profiler) ebar += clock64() - b0;
            const uint32_t tacc =
                tmem_base + ab * kTileB + half * kCols + (static_cast<uint32_t>(quarter * 32) << 16);
            const int64_t half_col0 = tile_col0 + half * kCols;
            // sixteen-warp L2: the generic chunk code (sample pass, direct mode) reads the norms from global memory too
            const uint32_t* hnorm = l2_global(KIND) ? gnorm + tile_col0 + half * kCols : &epi_sh.norm[ab][half * kCols];
            const int hslot = sel * (kTileB / BURST) + half * (kCols / BURST);
            uint32_t ra[32], rb[32];
            if (KIND == kKindI8Cos && MODE == kModeAppend && kCols == 64 && !a.direct) {
                // cosine: the accumulators of both chunks become ordered fp16 scores in place (the
                // reciprocal norms staged above are read here, before the buffer goes back), and from
                // there on they are inner products
                ptx::tmem_ld_32x32(tacc, ra);
                ptx::tmem_ld_32x32(tacc + 32, rb);
                ptx::tmem_ld_wait(ra);
                ptx::tmem_ld_wait(rb);
                epi.cos_scores(ra, hnorm);
                epi.cos_scores(rb, hnorm + 32);
                const int64_t rem_a = n_end - half_col0, rem_b = rem_a - 32;
                const uint32_t ma = epi.ip_mask(ra, half_col0, rem_a >= 32 ? 32 : (rem_a > 0 ? static_cast<int>(rem_a) : 0));
                const uint32_t mb = epi.ip_mask(rb, half_col0 + 32, rem_b >= 32 ? 32 : (rem_b > 0 ? static_cast<int>(rem_b) : 0));
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&bar_acc_empty[ab]);
                epi.ip_extract(ra, ma, half_col0);
                epi.ip_extract(rb, mb, half_col0 + 32);
                epi.end_tile(hslot);
                continue;
            }
            if (ip_only(KIND) && MODE == kModeAppend && kCols == 64 && !a.direct) {
                // as below: both chunks, both masks, the accumulator back, then the candidates
                ptx::tmem_ld_32x32(tacc, ra);
                ptx::tmem_ld_32x32(tacc + 32, rb);
                ptx::tmem_ld_wait(ra);
                ptx::tmem_ld_wait(rb);
                const int64_t rem_a = n_end - half_col0, rem_b = rem_a - 32;
                const uint32_t ma = epi.ip_mask(ra, half_col0, rem_a >= 32 ? 32 : (rem_a > 0 ? static_cast<int>(rem_a) : 0));
                const uint32_t mb = epi.ip_mask(rb, half_col0 + 32, rem_b >= 32 ? 32 : (rem_b > 0 ? static_cast<int>(rem_b) : 0));
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&bar_acc_empty[ab]);
                epi.ip_extract(ra, ma, half_col0);
                epi.ip_extract(rb, mb, half_col0 + 32);
                epi.end_tile(hslot);
                continue;
            }
            if (l2_global(KIND) && MODE == kModeAppend && kCols == 64 && !a.direct) {
                ptx::tmem_ld_32x32(tacc, ra);
                ptx::tmem_ld_32x32(tacc + 32, rb);
                ptx::tmem_ld_wait(ra);
                ptx::tmem_ld_wait(rb);
                const uint32_t* gna = gnorm + half_col0;
                const int64_t rem_a = n_end - half_col0, rem_b = rem_a - 32;
                const uint32_t ma = epi.l2_mask(ra, gna, half_col0, rem_a >= 32 ? 32 : (rem_a > 0 ? static_cast<int>(rem_a) : 0));
                const uint32_t mb = epi.l2_mask(rb, gna + 32, half_col0 + 32, rem_b >= 32 ? 32 : (rem_b > 0 ? static_cast<int>(rem_b) : 0));
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&bar_acc_empty[ab]);
                epi.l2_extract(ra, ma, half_col0, gna);
                epi.l2_extract(rb, mb, half_col0 + 32, gna + 32);
                epi.end_tile(hslot);
                continue;
            }
            if (FOLD && MODE == kModeAppend && kCols == 64 && !a.direct && !(kDevProf && a.dbg)) {
                // Both chunks into registers, the pass masks, and the accumulator goes back to the MMA
                // side at once: taking the candidates out (the slow, uneven part -- a warp with three
                // hits would otherwise hold the buffer for all sixteen) happens afterwards, from the
                // registers, while the tensor core already refills the buffer.
                ptx::tmem_ld_32x32(tacc, ra);
                ptx::tmem_ld_32x32(tacc + 32, rb);
                ptx::tmem_ld_wait(ra);
                ptx::tmem_ld_wait(rb);
                const int64_t rem_a = n_end - half_col0, rem_b = rem_a - 32;
                const uint32_t ma = epi.fold_mask(ra, half_col0, rem_a >= 32 ? 32 : (rem_a > 0 ? static_cast<int>(rem_a) : 0));
                const uint32_t mb = epi.fold_mask(rb, half_col0 + 32, rem_b >= 32 ? 32 : (rem_b > 0 ? static_cast<int>(rem_b) : 0));
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&bar_acc_empty[ab]);
                epi.fold_extract(ra, ma, half_col0);
                epi.fold_extract(rb, mb, half_col0 + 32);
                epi.end_tile(hslot);
                continue;
            }
            const bool dbg_no_ld = kDevProf && (a.dbg & 2), dbg_no_chunk = kDevProf && (a.dbg & 3);
            if (!dbg_no_ld) ptx::tmem_ld_32x32(tacc, ra);
            // two chunks per step, the TMEM load of the next chunk in flight behind the current one
            auto step = [&](int c) {
                if (dbg_no_ld) return;
                const long long w0 = profiler ? clock64() : 0;
                ptx::tmem_ld_wait(ra);
                if (profiler) elw += clock64() - w0;
                ptx::tmem_ld_32x32(tacc + (c + 1) * 32, rb);
                {
                    const long long c0 = profiler ? clock64() : 0;
                    const int64_t col0 = half_col0 + c * 32;
                    const int64_t rem = n_end - col0;
                    if (!dbg_no_chunk) epi.chunk(ra, hnorm + c * 32, col0, rem >= 32 ? 32 : (rem > 0 ? static_cast<int>(rem) : 0),
                              hslot + c * (32 / BURST), c, cbase);
                    if (profiler) ecc += clock64() - c0;
                }
                const long long w1 = profiler ? clock64() : 0;
                ptx::tmem_ld_wait(rb);
                if (profiler) elw += clock64() - w1;
                if (c + 2 < kCols / 32) ptx::tmem_ld_32x32(tacc + (c + 2) * 32, ra);
                {
                    const int64_t col0 = half_col0 + (c + 1) * 32;
                    const int64_t rem = n_end - col0;
                    if (!dbg_no_chunk) epi.chunk(rb, hnorm + (c + 1) * 32, col0, rem >= 32 ? 32 : (rem > 0 ? static_cast<int>(rem) : 0),
                              hslot + (c + 1) * (32 / BURST), c + 1, cbase);
                }
            };
            if (FOLD) {   // small body: unrolled, so the chunk index is a constant
#pragma unroll
                for (int c = 0; c < kCols / 32; c += 2) step(c);
            } else {
#pragma unroll 1
                for (int c = 0; c < kCols / 32; c += 2) step(c);
            }
            // accumulator drained: hand the TMEM buffer back before the global stores
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&bar_acc_empty[ab]);
            if (kDevProf && a.trace && blockIdx.x == 0 && t < 64 && lane == 0 && (warp == 2 || warp == 2 + epi_warps(KIND) - 1))
                a.trace[(warp == 2 ? 5 : 7) * 64 + t] = clock64();
            const long long e2 = profiler ? clock64() : 0;
            epi.end_tile(hslot);
            if (profiler) {
                const long long e3 = clock64();
                ew += e1 - e0;
                ec += e2 - e1;
                ef += e3 - e2;
            }
        }
        epi.finish();
        if (profiler) {
            atomicAdd(a.prof + 3, static_cast<unsigned long long>(ew));
            atomicAdd(a.prof + 4, static_cast<unsigned long long>(ec));
            atomicAdd(a.prof + 5, static_cast<unsigned long long>(ef));
            atomicAdd(a.prof + 6, static_cast<unsigned long long>(t));
            atomicAdd(a.prof + 8, static_cast<unsigned long long>(elw));
            atomicAdd(a.prof + 9, static_cast<unsigned long long>(ebar));
            atomicAdd(a.prof + 10, static_cast<unsigned long long>(ecc));
        }
    }

    // Teardown.  After an abort, give copies in flight time to land before the CTA's shared
    // memory is released.
    __syncwarp();
    if (abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000LL) { }
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && abort_flag) atomicOr(a.err, kDevErrPipelineTimeout);
}

// ---------------------------------------------------------------------------------------
// CUDA-core variant: same work decomposition and epilogue, accumulators computed with
// scalar FMAs.  Used to cross-check the tcgen05 variant on device.
// ---------------------------------------------------------------------------------------
template <int KIND>
__device__ __forceinline__ typename std::conditional<is_i8(KIND), int32_t, float>::type
load_elem(const void* p, int64_t idx) {
    if (is_i8(KIND)) return static_cast<int32_t>(static_cast<const int8_t*>(p)[idx]);
    else if (KIND == kKindBF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
    else return __half2float(static_cast<const __half*>(p)[idx]);
}

template <int KIND, int MODE, int BURST>
__global__ void __launch_bounds__(kTileQ)
dist_gemm_simt_kernel(const GemmArgs a) {
    using AccT = typename std::conditional<is_i8(KIND), int32_t, float>::type;
    __shared__ __align__(16) EpiShared epi_sh;
    const int n_qb = (a.nq + kTileQ - 1) / kTileQ;
    const ItemRange range(a, n_qb);
    const bool l2 = a.metric == kMetricL2;
    constexpr bool cosm = KIND == kKindI8Cos;
    const uint32_t* gnorm = static_cast<const uint32_t*>(a.bnorm);
    RowEpilogue<AccT, MODE, BURST, KIND == kKindBF16, kTileB / 32, KIND == kKindI8Cos, ip_only(KIND)> epi(a);
    ItemCursor cur(range);
    for (int64_t i = 0; i < range.count; ++i, cur.next()) {
        const int qb = cur.qb;
        const int sel = cur.sel;
        const int tile = tile_of(a, sel);
        const int q_in = qb * kTileQ + threadIdx.x;
        const bool row_ok = q_in < a.nq;
        const int qc = row_ok ? q_in : a.nq - 1;
        const int64_t tile_col0 = static_cast<int64_t>(tile) * kTileB;
        int q = q_in;
        int64_t cbase = 0, n_end = a.N;
        if (a.seg_index) {
            q += (a.seg_index[tile] - a.seg_first) * a.nq;
            cbase = a.seg_col0[tile];
            n_end = a.seg_end[tile];
        }
        __syncthreads();
        for (int h = 0; h < kTileB; h += kTileQ) {
            uint32_t nv = (l2 || cosm) ? __ldg(gnorm + tile_col0 + h + threadIdx.x) : 0u;
            if (cosm) nv = cos16_rnorm_bits(static_cast<int32_t>(nv));
            epi_sh.norm[0][h + threadIdx.x] = nv;
        }
        __syncthreads();
        epi.begin_tile(q, row_ok);
        for (int c = 0; c < kTileB / 32; ++c) {
            const int64_t col0 = tile_col0 + c * 32;
            int64_t rem = n_end - col0;
            const int nvalid = rem >= 32 ? 32 : (rem > 0 ? static_cast<int>(rem) : 0);
            uint32_t r[32];
            for (int j = 0; j < 32; ++j) {
                const int64_t col = (col0 + j < a.N) ? col0 + j : a.N - 1;
                AccT acc = AccT(0);
                const bool packed = packed_operands(KIND, a.d);
                for (int k = 0; k < a.d; ++k)
                    acc += load_elem<KIND>(a.A, operand_elem(packed, qc, k, a.d, kTileQ)) *
                           load_elem<KIND>(a.B, operand_elem(packed, col, k, a.d, kTileB));
                if (is_i8(KIND)) r[j] = static_cast<uint32_t>(acc);
                else r[j] = __float_as_uint(acc);
            }
            const int bslot = sel * (kTileB / BURST) + c * (32 / BURST);
            epi.chunk(r, &epi_sh.norm[0][c * 32], col0, nvalid, bslot, c, cbase);
        }
        epi.end_tile(sel * (kTileB / BURST));
    }
    epi.finish();
}

template <int KIND, int MODE, int BURST>
cudaError_t launch_one(const GemmLaunch& L, GemmArgs a, const CUtensorMap* mapA, const CUtensorMap* mapB,
                       cudaStream_t stream) {
    const int n_qb = (a.nq + kTileQ - 1) / kTileQ;
    const int64_t total = static_cast<int64_t>(n_qb) * a.n_tiles_sel;
    if (total <= 0) return cudaSuccess;
    if (L.simt) {
        const int grid = static_cast<int>(total < 4LL * L.num_sms ? total : 4LL * L.num_sms);
        dist_gemm_simt_kernel<KIND, MODE, BURST><<<grid, kTileQ, 0, stream>>>(a);
        return cudaGetLastError();
    }
    // shared-memory plan: resident query tile (if it is small) + as many ring stages as fit
    const int elem = is_i8(KIND) ? 1 : 2;
    const int nkc = (a.d * elem + kChunkBytes - 1) / kChunkBytes;
    a.packed = packed_operands(KIND, a.d) ? 1 : 0;
    a.a_resident = (a.packed || nkc <= kResidentMaxChunks) ? 1 : 0;
    const int a_bytes = a.packed ? ((kTileQ * a.d * 2 + 1023) & ~1023) : (a.a_resident ? nkc * kStageABytes : 0);
    const int stage_bytes = a.packed ? kTileB * a.d * 2 : (a.a_resident ? kStageBBytes : kStageBytes);
    int nst = a.packed ? 2 : (kGemmSmemBudget - 1024 - a_bytes) / stage_bytes;   // packed: one whole tile per parity
    if (nst > kMaxStages) nst = kMaxStages;
    nst &= ~1;                       // two sub-rings of equal depth
    if (nst < 2) return cudaErrorInvalidConfiguration;
    a.n_stages = nst;
    const int smem = a_bytes + nst * stage_bytes + 1024;
    if (smem > kGemmSmemBudget) return cudaErrorInvalidConfiguration;
    auto kern = dist_gemm_tc_kernel<KIND, MODE, BURST>;
    // per-device attribute; cheap enough to set on every launch
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBudget);
    if (e != cudaSuccess) return e;
    const int grid = static_cast<int>(total < L.num_sms ? total : L.num_sms);
    // aligned ranges when every query block gets at least one CTA and the split stays balanced
    a.aligned_ranges = 0;
    if (n_qb <= grid && a.n_tiles_sel >= grid / n_qb) {
        const int nl_min = grid / n_qb;
        const double worst = static_cast<double>((a.n_tiles_sel + nl_min - 1) / nl_min);
        const double ideal = static_cast<double>(total) / grid;
        if (worst <= 1.06 * ideal + 1.0) a.aligned_ranges = 1;
    }
    kern<<<grid, gemm_threads(KIND), smem, stream>>>(*mapA, *mapB, a);
    return cudaGetLastError();
}

template <int KIND>
cudaError_t launch_kind(const GemmLaunch& L, const GemmArgs& a, const CUtensorMap* mapA, const CUtensorMap* mapB,
                        cudaStream_t stream) {
    if (L.mode == kModeAppend) return launch_one<KIND, kModeAppend, 32>(L, a, mapA, mapB, stream);
    if (L.burst == 8) return launch_one<KIND, kModeBurstMin, 8>(L, a, mapA, mapB, stream);
    return launch_one<KIND, kModeBurstMin, 32>(L, a, mapA, mapB, stream);
}

}  // namespace

cudaError_t launch_dist_gemm(const GemmLaunch& L, const GemmArgs& a, const CUtensorMap* mapA, const CUtensorMap* mapB,
                             cudaStream_t stream) {
    switch (L.kind) {
        case kKindF16:
            return a.metric == kMetricIP ? launch_kind<kKindF16IP>(L, a, mapA, mapB, stream)
                                         : launch_kind<kKindF16L2>(L, a, mapA, mapB, stream);
        case kKindBF16: return launch_kind<kKindBF16>(L, a, mapA, mapB, stream);
        case kKindI8:
            return a.metric == kMetricCos  ? launch_kind<kKindI8Cos>(L, a, mapA, mapB, stream)
                   : a.metric == kMetricIP ? launch_kind<kKindI8IP>(L, a, mapA, mapB, stream)
                                           : launch_kind<kKindI8L2>(L, a, mapA, mapB, stream);
        default: return cudaErrorInvalidValue;
    }
}

int encode_operand_map(CUtensorMap* out, int kind, const void* base, int64_t rows, int d, int box_rows) {
    if (packed_operands(kind, d)) {   // read with contiguous copies: no tensor map
        std::memset(out, 0, sizeof(*out));
        return 0;
    }
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault, &qres) !=
                cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn)
            return -1;
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    const int elem = kind == kKindI8 ? 1 : 2;
    const CUtensorMapDataType dt = kind == kKindI8    ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                   : kind == kKindBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                       : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    cuuint64_t gdim[2] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(rows)};
    cuuint64_t gstride[1] = {static_cast<cuuint64_t>(d) * elem};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(kChunkBytes / elem), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estride[2] = {1, 1};
    CUresult r = encode(out, dt, 2, const_cast<void*>(base), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

}  // namespace b200
