// tcgen05 / TMEM / TMA distance GEMM with fused selection epilogues, plus a plain CUDA-core
// variant that shares the epilogue code and serves as an on-device cross-check.
//
// Pipeline of the tcgen05 variant (one persistent CTA per SM, 320 threads):
//   warp 0 (one lane)  : TMA producer.  Per K chunk of 128 bytes: query box 128 x 128 B and base
//                        box 256 x 128 B into a 4-stage ring of 48 KB stages (SWIZZLE_128B).
//   warp 1 (one lane)  : issues tcgen05.mma 128 x 256 x (32 bytes of K) from shared-memory
//                        descriptors into one of two 256-column TMEM accumulators; commits free
//                        the stage (per chunk) and publish the accumulator (per tile).
//   warps 2-9          : epilogue, two warps per scheduler.  Thread = (query row = TMEM lane, one
//                        half of the tile's columns); reads 32 columns at a time with tcgen05.ld
//                        (double-buffered) and applies the norm-add and the selection predicate.
// Work items are (query block, base tile) pairs, query block fastest, so the CTAs running at
// the same time read the same base tiles and HBM sees each base tile about once per pass.
#include "dist_gemm.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace b200 {
namespace {

constexpr int kStages = 4;
constexpr int kStageABytes = kTileQ * kChunkBytes;               // 16 KB
constexpr int kStageBBytes = kTileB * kChunkBytes;               // 32 KB
constexpr int kStageBytes = kStageABytes + kStageBBytes;         // 48 KB
constexpr int kGemmSmemBytes = kStages * kStageBytes + 1024;     // + slack for 1024-byte alignment
constexpr int kEpiWarps = 8;                                    // two per scheduler; pairs split the tile's columns
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kGemmThreads = 64 + kEpiThreads;                   // producer warp + MMA warp + epilogue warps
constexpr uint32_t kTmemCols = 512;

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

constexpr int kStageSlots = 8;   // per-row candidate staging slots per tile (shared memory)

// Shared-memory side of the epilogue: the tile's base norms (double-buffered with the TMEM
// accumulators) and a per-row staging area for candidates found in the current tile.
struct EpiShared {
    uint32_t norm[2][kTileB];
    uint64_t stage[kStageSlots][2 * kTileQ];   // one column of slots per epilogue thread
};

// Per-thread (= per query row) epilogue state for one tile.
//   append mode : candidates of the tile are staged in shared memory (thread-private slots, no
//                 atomics) and flushed with ONE global atomicAdd per row per tile, so the
//                 latency of the L2 atomic is paid once per tile instead of once per candidate.
//   direct mode : every key is written to cand[q][position] (no threshold, no atomics).
//   FOLD        : the operands carry 16 extra K columns (see GemmArgs::fold), so the accumulator
//                 already holds  D = q.y - |y|^2/2 + tau/2  (L2; inner product: q.y + tau).  No
//                 norms are read and "key <= tau" is the sign of D: 32 columns are tested with a
//                 16-instruction AND tree, and the burst minimum of the key is a maximum of D.
template <typename AccT, int MODE, int BURST, bool FOLD>
struct RowEpilogue {
    using K = KeyOps<AccT>;
    const GemmArgs& a;
    EpiShared& sh;
    int q;        // query row, valid when row_ok
    int tid;      // row inside the tile, 0..127
    bool row_ok;
    bool l2;
    AccT tau, tau_up;
    uint32_t cnt;

    // tid_: index of this thread's private staging column
    __device__ __forceinline__ RowEpilogue(const GemmArgs& a_, EpiShared& sh_, int tid_)
        : a(a_), sh(sh_), q(0), tid(tid_), row_ok(false), l2(a_.metric == kMetricL2), tau(AccT(0)),
          tau_up(AccT(0)), cnt(0) {}

    __device__ __forceinline__ void begin_tile(int q_, bool ok) {
        q = q_;
        row_ok = ok;
        cnt = 0;
        if (MODE == kModeAppend && ok && (!FOLD || a.direct)) {
            tau = K::tau(__ldg(a.tau + q));
            tau_up = K::above(tau);
        }
    }

    // Folded operands: r holds D for 32 columns.
    __device__ __forceinline__ void chunk_fold(const uint32_t (&r)[32], int64_t col0, int nvalid, int bslot) {
        if (!row_ok) return;
        if (MODE == kModeBurstMin) {
            constexpr int NB = 32 / BURST;
            uint32_t* dst = a.mins + static_cast<int64_t>(q) * a.mins_stride + bslot;
            const float ninf = __int_as_float(0xff800000);
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                float v[BURST];
#pragma unroll
                for (int j = 0; j < BURST; ++j) {
                    const int c = b * BURST + j;
                    v[j] = __uint_as_float(r[c]);
                    if (nvalid < 32 && c >= nvalid) v[j] = ninf;   // rows past the end of the base
                }
#pragma unroll
                for (int w = BURST / 2; w > 0; w >>= 1)
#pragma unroll
                    for (int j = 0; j < w; ++j) v[j] = fmaxf(v[j], v[j + w]);   // NaN never wins
                const float key = l2 ? -2.f * v[0] : -v[0];
                dst[b] = float_to_ord(key);
            }
        } else if (a.direct) {
            uint64_t* crow = a.cand + static_cast<int64_t>(q) * a.cap + col0;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                const float dv = __uint_as_float(r[c]);
                const float key = l2 ? -2.f * dv : -dv;
                // NaN keys are left at the buffer's "invalid" fill
                if (c < nvalid && key <= tau) crow[c] = pack_cand(float_to_ord(key), static_cast<uint32_t>(col0 + c));
            }
        } else {
            uint32_t t[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) t[i] = r[2 * i] & r[2 * i + 1];
#pragma unroll
            for (int w = 8; w > 0; w >>= 1)
#pragma unroll
                for (int i = 0; i < w; ++i) t[i] &= t[i + w];
            if (static_cast<int32_t>(t[0]) < 0) return;   // every D negative: no key <= tau here
            uint32_t m0 = 0, m1 = 0;                      // bit (31 - c): D of column c has its sign set
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                m0 = __funnelshift_l(r[c], m0, 1);
                m1 = __funnelshift_l(r[16 + c], m1, 1);
            }
            uint32_t mask = ~((m0 << 16) | (m1 & 0xFFFFu));
            mask &= nvalid >= 32 ? 0xFFFFFFFFu : ~(0xFFFFFFFFu >> nvalid);
            if (!mask) return;
            const float tq = ord_to_float(__ldg(a.tau + q));
            while (mask) {
                const uint32_t c = __clz(mask);
                mask &= ~(0x80000000u >> c);
                const float dv = __uint_as_float(pick(r, c));
                if (!(dv >= 0.f)) continue;   // NaN
                // approximate key (the fp32 refinement recomputes it): D = (tau' - key) / 2 or tau' - key
                const float key = l2 ? fmaf(-2.f, dv, tq) : tq - dv;
                const uint64_t e = pack_cand(float_to_ord(key), static_cast<uint32_t>(col0 + c));
                if (cnt < kStageSlots) sh.stage[cnt][tid] = e;
                else slow_append(e);
                ++cnt;
            }
        }
    }

    __device__ __forceinline__ void slow_append(uint64_t e) {
        const uint32_t slot = atomicAdd(a.counts + q, 1u);
        if (slot < a.cap) a.cand[static_cast<int64_t>(q) * a.cap + slot] = e;
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

    // r: 32 accumulator columns; nb: the matching 32 norms in shared memory; col0: base position
    // of r[0]; nvalid: real base rows among the 32; bslot: first burst slot (burst-min mode).
    // The hot path is straight-line code: the threshold test of the 32 columns is folded into a
    // bit mask, and only a non-zero mask (rare) enters the compact candidate loop.
    __device__ __forceinline__ void chunk(const uint32_t (&r)[32], const uint32_t* nb, int64_t col0, int nvalid,
                                          int bslot) {
        if (FOLD) {
            chunk_fold(r, col0, nvalid, bslot);
            return;
        }
        if (!row_ok) return;
        uint32_t bnb[32];
        if (l2) {
            const uint4* p = reinterpret_cast<const uint4*>(nb);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint4 v = p[j];
                bnb[4 * j + 0] = v.x;
                bnb[4 * j + 1] = v.y;
                bnb[4 * j + 2] = v.z;
                bnb[4 * j + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) bnb[j] = 0u;   // +0.0f / 0
        }
        const uint32_t valid = nvalid >= 32 ? 0xFFFFFFFFu : ((1u << nvalid) - 1u);
        if (MODE == kModeBurstMin) {
            constexpr int NB = 32 / BURST;
            uint32_t* dst = a.mins + static_cast<int64_t>(q) * a.mins_stride + bslot;
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                AccT m[4] = {K::worst(), K::worst(), K::worst(), K::worst()};   // independent chains
#pragma unroll
                for (int j = 0; j < BURST; ++j) {
                    const int c = b * BURST + j;
                    const AccT key = K::key(K::from_bits(r[c]), K::from_bits(bnb[c]), l2);
                    if ((valid >> c) & 1u) m[j & 3] = key < m[j & 3] ? key : m[j & 3];
                }
                const AccT ma = m[0] < m[1] ? m[0] : m[1], mb = m[2] < m[3] ? m[2] : m[3];
                dst[b] = K::ord(ma < mb ? ma : mb);
            }
        } else if (a.direct) {
            uint64_t* crow = a.cand + static_cast<int64_t>(q) * a.cap + col0;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                const AccT key = K::key(K::from_bits(r[c]), K::from_bits(bnb[c]), l2);
                // NaN keys are left at the buffer's "invalid" fill
                if (((valid >> c) & 1u) && key <= tau) crow[c] = pack_cand(K::ord(key), static_cast<uint32_t>(col0 + c));
            }
        } else {
            // bit (31 - c) of mask = "column c passes": the sign of key - above(tau), shifted in
            // with one funnel shift per column (two independent chains for the scheduler).
            uint32_t m0 = 0, m1 = 0;
            if (l2) {
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    m0 = __funnelshift_l(K::sign_l2(K::from_bits(r[c]), K::from_bits(bnb[c]), tau_up), m0, 1);
                    m1 = __funnelshift_l(K::sign_l2(K::from_bits(r[16 + c]), K::from_bits(bnb[16 + c]), tau_up), m1, 1);
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
            mask &= nvalid >= 32 ? 0xFFFFFFFFu : ~(0xFFFFFFFFu >> nvalid);
            while (mask) {
                const uint32_t c = __clz(mask);
                mask &= ~(0x80000000u >> c);
                const AccT key = K::key(K::from_bits(pick(r, c)), K::from_bits(l2 ? nb[c] : 0u), l2);
                if (!(key <= tau)) continue;   // NaN
                const uint64_t e = pack_cand(K::ord(key), static_cast<uint32_t>(col0 + c));
                if (cnt < kStageSlots) sh.stage[cnt][tid] = e;
                else slow_append(e);
                ++cnt;
            }
        }
    }

    __device__ __forceinline__ void end_tile() {
        if (MODE != kModeAppend || !row_ok || a.direct) return;
        const uint32_t n_st = cnt < kStageSlots ? cnt : kStageSlots;
        if (n_st) {
            const uint32_t slot0 = atomicAdd(a.counts + q, n_st);
            uint64_t* crow = a.cand + static_cast<int64_t>(q) * a.cap;
            for (uint32_t i = 0; i < n_st; ++i)
                if (slot0 + i < a.cap) crow[slot0 + i] = sh.stage[i][tid];
        }
    }
};

__device__ __forceinline__ int tile_of(const GemmArgs& a, int sel) {
    return static_cast<int>(static_cast<int64_t>(sel) * a.n_tiles_total / a.n_tiles_sel);
}

// ---------------------------------------------------------------------------------------
// tcgen05 variant
// ---------------------------------------------------------------------------------------
template <int KIND, int MODE, int BURST>
__global__ void __launch_bounds__(kGemmThreads, 1)
dist_gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                    const GemmArgs a) {
    using AccT = typename std::conditional<KIND == kKindI8, int32_t, float>::type;
    constexpr int kElemBytes = KIND == kKindI8 ? 1 : 2;
    constexpr int kChunkElems = kChunkBytes / kElemBytes;
    constexpr bool FOLD = KIND == kKindBF16;
    constexpr uint32_t kIdesc = KIND == kKindI8 ? ptx::umma_idesc(2, 1, kTileQ, kTileB)
                                                : ptx::umma_idesc(1, KIND == kKindBF16 ? 1 : 0, kTileQ, kTileB);

    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[kStages];
    __shared__ uint64_t bar_empty[kStages];
    __shared__ uint64_t bar_acc_full[2];
    __shared__ uint64_t bar_acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    __shared__ __align__(16) EpiShared epi_sh;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(&bar_full[s], 1);
            ptx::mbar_init(&bar_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(&bar_acc_full[b], 1);
            ptx::mbar_init(&bar_acc_empty[b], kEpiWarps);
        }
        abort_flag = 0;
        ptx::mbar_fence_init();
        ptx::prefetch_tensormap(&mapA);
        ptx::prefetch_tensormap(&mapB);
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
    const int64_t total = static_cast<int64_t>(n_qb) * a.n_tiles_sel;
    const int nkc = (a.d + kChunkElems - 1) / kChunkElems;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            long long pw = 0;
            const long long k0 = a.prof ? clock64() : 0;
            for (int64_t item = blockIdx.x; item < total && ok; item += gridDim.x) {
                const int qb = static_cast<int>(item % n_qb);
                const int tile = tile_of(a, static_cast<int>(item / n_qb));
                for (int kc = 0; kc < nkc; ++kc, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1u;
                    const long long w0 = a.prof ? clock64() : 0;
                    if (!ptx::mbar_wait_bounded(&bar_empty[s], ph ^ 1u, &abort_flag)) { ok = false; break; }
                    if (a.prof) pw += clock64() - w0;
                    ptx::mbar_expect_tx(&bar_full[s], kStageBytes);
                    uint8_t* sa = smem + s * kStageBytes;
                    ptx::tma_load_2d(sa, &mapA, &bar_full[s], kc * kChunkElems, qb * kTileQ);
                    ptx::tma_load_2d(sa + kStageABytes, &mapB, &bar_full[s], kc * kChunkElems, tile * kTileB);
                }
            }
            if (a.prof) {
                atomicAdd(a.prof + 0, static_cast<unsigned long long>(pw));
                atomicAdd(a.prof + 7, static_cast<unsigned long long>(clock64() - k0));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0, t = 0;
            bool ok = true;
            long long mw0 = 0, mw1 = 0;
            for (int64_t item = blockIdx.x; item < total && ok; item += gridDim.x, ++t) {
                const uint32_t ab = t & 1u;
                const uint32_t aph = (t >> 1) & 1u;
                long long w0 = a.prof ? clock64() : 0;
                if (!ptx::mbar_wait_bounded(&bar_acc_empty[ab], aph ^ 1u, &abort_flag)) { ok = false; break; }
                if (a.prof) mw0 += clock64() - w0;
                ptx::tc_fence_after();
                const uint32_t tacc = tmem_base + ab * kTileB;
                for (int kc = 0; kc < nkc; ++kc, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1u;
                    w0 = a.prof ? clock64() : 0;
                    if (!ptx::mbar_wait_bounded(&bar_full[s], ph, &abort_flag)) { ok = false; break; }
                    if (a.prof) mw1 += clock64() - w0;
                    ptx::tc_fence_after();
                    const uint32_t sa = ptx::smem_u32(smem + s * kStageBytes);
                    const uint32_t sb = sa + kStageABytes;
                    // the last chunk may hold fewer than four 32-byte K steps (the rest is zero fill)
                    const int rem_bytes = a.d * kElemBytes - kc * kChunkBytes;
                    const int nks = rem_bytes >= kChunkBytes ? kChunkBytes / 32 : (rem_bytes + 31) / 32;
#pragma unroll
                    for (int ks = 0; ks < kChunkBytes / 32; ++ks) {
                        if (ks >= nks) break;
                        const uint64_t da = ptx::umma_desc_k_sw128(sa + ks * 32);
                        const uint64_t db = ptx::umma_desc_k_sw128(sb + ks * 32);
                        const uint32_t accum = (kc > 0 || ks > 0) ? 1u : 0u;
                        if (KIND == kKindI8) ptx::umma_i8(tacc, da, db, kIdesc, accum);
                        else ptx::umma_f16(tacc, da, db, kIdesc, accum);
                    }
                    ptx::umma_commit(&bar_empty[s]);
                }
                if (ok) ptx::umma_commit(&bar_acc_full[ab]);
            }
            if (a.prof) {
                atomicAdd(a.prof + 1, static_cast<unsigned long long>(mw0));
                atomicAdd(a.prof + 2, static_cast<unsigned long long>(mw1));
            }
        }
    } else {
        const int quarter = warp & 3;          // TMEM lane quarter this warp may read
        const int half = (warp - 2) >> 2;      // which 128 columns of the tile this warp drains
        const int row_in_tile = quarter * 32 + lane;
        const int et = threadIdx.x - 64;       // epilogue thread index, 0..255
        constexpr int kCols = kTileB / 2;      // columns per epilogue thread
        RowEpilogue<AccT, MODE, BURST, FOLD> epi(a, epi_sh, et);
        const bool l2 = a.metric == kMetricL2 && !FOLD;   // FOLD: no norms to fetch
        const uint32_t* gnorm = static_cast<const uint32_t*>(a.bnorm);
        uint32_t t = 0;
        bool ok = true;
        long long ew = 0, ec = 0, ef = 0, elw = 0, ebar = 0, ecc = 0;
        const bool profiler = a.prof && warp == 2 && lane == 0;
        for (int64_t item = blockIdx.x; item < total && ok; item += gridDim.x, ++t) {
            const int qb = static_cast<int>(item % n_qb);
            const int sel = static_cast<int>(item / n_qb);
            const int tile = tile_of(a, sel);
            const uint32_t ab = t & 1u;
            const uint32_t aph = (t >> 1) & 1u;
            const int q = qb * kTileQ + row_in_tile;
            const int64_t tile_col0 = static_cast<int64_t>(tile) * kTileB;
            const long long e0 = profiler ? clock64() : 0;
            // The tile's norms travel global -> registers while the MMA is still running.
            uint32_t n0 = 0;
            if (l2) n0 = __ldg(gnorm + tile_col0 + et);
            epi.begin_tile(q, q < a.nq);
            if (!ptx::mbar_wait_bounded(&bar_acc_full[ab], aph, &abort_flag)) {
                // leave without stranding a sibling warp at the named barrier below
                if (!FOLD) asm volatile("bar.arrive 1, 256;" ::: "memory");
                ok = false;
                break;
            }
            const long long e1 = profiler ? clock64() : 0;
            ptx::tc_fence_after();
            const long long b0 = profiler ? clock64() : 0;
            if (!FOLD) {
                epi_sh.norm[ab][et] = n0;
                asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight epilogue warps
            }
            if (profiler) ebar += clock64() - b0;
            const uint32_t tacc =
                tmem_base + ab * kTileB + half * kCols + (static_cast<uint32_t>(quarter * 32) << 16);
            const int64_t half_col0 = tile_col0 + half * kCols;
            const uint32_t* hnorm = &epi_sh.norm[ab][half * kCols];
            const int hslot = sel * (kTileB / BURST) + half * (kCols / BURST);
            uint32_t ra[32], rb[32];
            ptx::tmem_ld_32x32(tacc, ra);
#pragma unroll 1
            for (int c = 0; c < kCols / 32; c += 2) {
                const long long w0 = profiler ? clock64() : 0;
                ptx::tmem_ld_wait(ra);
                if (profiler) elw += clock64() - w0;
                ptx::tmem_ld_32x32(tacc + (c + 1) * 32, rb);
                {
                    const long long c0 = profiler ? clock64() : 0;
                    const int64_t col0 = half_col0 + c * 32;
                    const int64_t rem = a.N - col0;
                    epi.chunk(ra, hnorm + c * 32, col0, rem >= 32 ? 32 : (rem > 0 ? static_cast<int>(rem) : 0),
                              hslot + c * (32 / BURST));
                    if (profiler) ecc += clock64() - c0;
                }
                const long long w1 = profiler ? clock64() : 0;
                ptx::tmem_ld_wait(rb);
                if (profiler) elw += clock64() - w1;
                if (c + 2 < kCols / 32) ptx::tmem_ld_32x32(tacc + (c + 2) * 32, ra);
                {
                    const int64_t col0 = half_col0 + (c + 1) * 32;
                    const int64_t rem = a.N - col0;
                    epi.chunk(rb, hnorm + (c + 1) * 32, col0, rem >= 32 ? 32 : (rem > 0 ? static_cast<int>(rem) : 0),
                              hslot + (c + 1) * (32 / BURST));
                }
            }
            // accumulator drained: hand the TMEM buffer back before the global flush
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&bar_acc_empty[ab]);
            const long long e2 = profiler ? clock64() : 0;
            epi.end_tile();
            if (profiler) {
                const long long e3 = clock64();
                ew += e1 - e0;
                ec += e2 - e1;
                ef += e3 - e2;
            }
        }
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
__device__ __forceinline__ typename std::conditional<KIND == kKindI8, int32_t, float>::type
load_elem(const void* p, int64_t idx) {
    if (KIND == kKindI8) return static_cast<int32_t>(static_cast<const int8_t*>(p)[idx]);
    else if (KIND == kKindBF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
    else return __half2float(static_cast<const __half*>(p)[idx]);
}

template <int KIND, int MODE, int BURST>
__global__ void __launch_bounds__(kTileQ)
dist_gemm_simt_kernel(const GemmArgs a) {
    using AccT = typename std::conditional<KIND == kKindI8, int32_t, float>::type;
    __shared__ __align__(16) EpiShared epi_sh;
    const int n_qb = (a.nq + kTileQ - 1) / kTileQ;
    const int64_t total = static_cast<int64_t>(n_qb) * a.n_tiles_sel;
    const bool l2 = a.metric == kMetricL2;
    const uint32_t* gnorm = static_cast<const uint32_t*>(a.bnorm);
    RowEpilogue<AccT, MODE, BURST, KIND == kKindBF16> epi(a, epi_sh, threadIdx.x);
    for (int64_t item = blockIdx.x; item < total; item += gridDim.x) {
        const int qb = static_cast<int>(item % n_qb);
        const int sel = static_cast<int>(item / n_qb);
        const int tile = tile_of(a, sel);
        const int q = qb * kTileQ + threadIdx.x;
        const bool row_ok = q < a.nq;
        const int qc = row_ok ? q : a.nq - 1;
        const int64_t tile_col0 = static_cast<int64_t>(tile) * kTileB;
        __syncthreads();
        epi_sh.norm[0][threadIdx.x] = l2 ? __ldg(gnorm + tile_col0 + threadIdx.x) : 0u;
        epi_sh.norm[0][kTileQ + threadIdx.x] = l2 ? __ldg(gnorm + tile_col0 + kTileQ + threadIdx.x) : 0u;
        __syncthreads();
        epi.begin_tile(q, row_ok);
        for (int c = 0; c < kTileB / 32; ++c) {
            const int64_t col0 = tile_col0 + c * 32;
            int64_t rem = a.N - col0;
            const int nvalid = rem >= 32 ? 32 : (rem > 0 ? static_cast<int>(rem) : 0);
            uint32_t r[32];
            for (int j = 0; j < 32; ++j) {
                const int64_t col = (col0 + j < a.N) ? col0 + j : a.N - 1;
                AccT acc = AccT(0);
                for (int k = 0; k < a.d; ++k)
                    acc += load_elem<KIND>(a.A, static_cast<int64_t>(qc) * a.d + k) *
                           load_elem<KIND>(a.B, col * a.d + k);
                if (KIND == kKindI8) r[j] = static_cast<uint32_t>(acc);
                else r[j] = __float_as_uint(acc);
            }
            const int bslot = sel * (kTileB / BURST) + c * (32 / BURST);
            epi.chunk(r, &epi_sh.norm[0][c * 32], col0, nvalid, bslot);
        }
        epi.end_tile();
    }
}

template <int KIND, int MODE, int BURST>
cudaError_t launch_one(const GemmLaunch& L, const GemmArgs& a, const CUtensorMap* mapA, const CUtensorMap* mapB,
                       cudaStream_t stream) {
    const int n_qb = (a.nq + kTileQ - 1) / kTileQ;
    const int64_t total = static_cast<int64_t>(n_qb) * a.n_tiles_sel;
    if (total <= 0) return cudaSuccess;
    if (L.simt) {
        const int grid = static_cast<int>(total < 4LL * L.num_sms ? total : 4LL * L.num_sms);
        dist_gemm_simt_kernel<KIND, MODE, BURST><<<grid, kTileQ, 0, stream>>>(a);
        return cudaGetLastError();
    }
    auto kern = dist_gemm_tc_kernel<KIND, MODE, BURST>;
    // per-device attribute; cheap enough to set on every launch
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes);
    if (e != cudaSuccess) return e;
    const int grid = static_cast<int>(total < L.num_sms ? total : L.num_sms);
    kern<<<grid, kGemmThreads, kGemmSmemBytes, stream>>>(*mapA, *mapB, a);
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
        case kKindF16: return launch_kind<kKindF16>(L, a, mapA, mapB, stream);
        case kKindBF16: return launch_kind<kKindBF16>(L, a, mapA, mapB, stream);
        case kKindI8: return launch_kind<kKindI8>(L, a, mapA, mapB, stream);
        default: return cudaErrorInvalidValue;
    }
}

int encode_operand_map(CUtensorMap* out, int kind, const void* base, int64_t rows, int d, int box_rows) {
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
