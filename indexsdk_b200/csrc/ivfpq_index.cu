// IVFPQ search on one GPU.
//
// Stage 1  coarse quantizer: FlatIndex (fp32 mode) over the nlist centroids with k = nprobe --
//          the same tcgen05 distance GEMM, filter + fp32 refinement, so probe lists and their
//          distances are the canonical fp32 values (replaces DistanceFlatL2MinsAtFP32 +
//          TopkFlatFp32, FR/ascenddaemon/impl/IndexIVFPQ.cpp:2104-2164).
// Stage 2  lookup tables (replaces AscendcIvfpqSubspaceDistance, FR/ops/ascendc/op_kernel/
//          ascendc_ivfpq_subspace_distance.cpp:46-617): never materialised in HBM -- every scan CTA
//          builds its query's [M][256] fp32 table straight into shared memory from a regrouped
//          copy of the codebooks (L2-resident), which costs about 1 % of the scan's instructions.
//            raw encoding      : T[m][j] = |q_m - cb[m][j]|^2
//            residual encoding : T[m][j] = -2 q_m . cb[m][j]; the list-dependent remainder
//              |cb|^2 + 2 c_list . cb is summed over a vector's codes once, at add time, into one
//              float per vector (t2), and |q - c_list|^2 is the coarse distance:
//              |q - c - r|^2 = |q - c|^2 + (|r|^2 + 2 c.r) - 2 q.r.
// Stage 3  code scan (replaces AscendcIvfpqSearchDistanceL2 + TopkIvfpqL3, FR/ops/ascendc/
//          op_kernel/ascendc_ivfpq_search_distance_topk.h:95-810, FR/ops/cpukernel/impl/
//          topk_ivfpq_l3_cpu_kernel.cpp:36-254) as filter + exact refinement:
//            3a  ivfpq_fast_scan_kernel: CTA per (query, probe split), the query's table in shared
//                memory laid out [code][32] (sub-quantizer in the bank index, two replicas) so
//                that lane l, which handles sub-quantizer (s + l) mod 16 at step s, always hits
//                bank l -- no bank conflicts.  Codes are stored rotated by (position mod 16), so
//                byte s of a lane's 128-bit load is exactly the sub-quantizer it needs at step s.
//                The fp32 sum therefore runs in a rotated order; it is used as a FILTER: each warp
//                keeps the k' = 32 * KPT best (approximate distance, position) in registers.
//            3b  ivfpq_refine_kernel: the k' survivors per query are re-computed in the oracle's
//                canonical arithmetic (raw: sum_m |q_m - cb[m][code_m]|^2 in ascending m; residual: the
//                direct form sum_m |(q - c)_m - cb[m][code_m]|^2), ordered by (distance, label),
//                and the result is VERIFIED: it is accepted only if the exact k-th distance lies
//                below (worst kept approximate distance - error bound); otherwise the query is
//                flagged.
//            3c  ivfpq_exact_scan_kernel: flagged queries (heavy ties, more duplicates than k')
//                are re-scanned in canonical arithmetic with a canonical table built in shared
//                memory -- one per query (raw) or one per (query, list) from q - c_list (residual).
//          Results are therefore bit-identical to the CPU oracle for both encodings.
#include "ivfpq_index.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cub/cub.cuh>
#include <unordered_set>

#include "ivfpq_tc_scan.cuh"
#include "kmeans.h"
#include "ptx_sm100.cuh"
#include "select.cuh"

namespace b200 {
namespace {

constexpr int kKsub = 256;
constexpr int kListPad = 32;     // lists are padded to a multiple of this many vectors
constexpr int kScanThreads = 128;
constexpr float kInf = 3.402823466e+38f;   // FLT_MAX used as padding distance
constexpr uint32_t kNoPos = 0xFFFFFFFFu;
constexpr int64_t kNoLabel = 0x7fffffffffffffffll;

// Byte offset of sub-quantizer m inside the stored code of the vector at `pos`.
__device__ __forceinline__ int code_byte(bool rotated, int m, int64_t pos) {
    return rotated ? ((m & ~15) | ((m - static_cast<int>(pos & 15)) & 15)) : m;
}

__global__ void cb_norm_kernel(const float* cb, int M, int dsub, float* out) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= M * kKsub) return;
    const float* c = cb + static_cast<int64_t>(idx) * dsub;
    float acc = 0.f;
    for (int t = 0; t < dsub; ++t) acc = fmaf(c[t], c[t], acc);
    out[idx] = acc;
}

// PQ encode: one warp per (vector, sub-quantizer); exhaustive nearest codeword under the
// canonical fp32 distance, first minimum wins.
__global__ void encode_kernel(const float* x, int64_t n, int d, int M, int dsub, const float* cb, int by_residual,
                              const float* centroids, const int32_t* list_no, uint8_t* codes) {
    const int64_t task = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (task >= n * M) return;
    const int64_t v = task / M;
    const int m = static_cast<int>(task % M);
    const float* xv = x + v * d + m * dsub;
    const float* cv = by_residual ? centroids + static_cast<int64_t>(list_no[v]) * d + m * dsub : nullptr;
    float best = __int_as_float(0x7f800000);
    int arg = 0;
    for (int j = lane; j < kKsub; j += 32) {
        const float* c = cb + (static_cast<int64_t>(m) * kKsub + j) * dsub;
        float acc = 0.f;
        for (int t = 0; t < dsub; ++t) {
            const float r = by_residual ? xv[t] - cv[t] : xv[t];
            const float df = r - c[t];
            acc = fmaf(df, df, acc);
        }
        if (acc < best) {
            best = acc;
            arg = j;
        }
    }
    for (int off = 16; off > 0; off >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, off);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, off);
        if (ob < best || (ob == best && oa < arg)) {
            best = ob;
            arg = oa;
        }
    }
    if (lane == 0) codes[v * M + m] = static_cast<uint8_t>(arg);
}

// t2[v] = sum_m ( |cb[m][code]|^2 + 2 c_list,m . cb[m][code] ), fp32, m ascending (canonical codes).
__global__ void t2_kernel(int64_t n, int d, int M, int dsub, const float* cb, const float* cbnorm,
                          const float* centroids, const int32_t* list_no, const uint8_t* codes, float* t2) {
    const int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (v >= n) return;
    const float* cen = centroids + static_cast<int64_t>(list_no[v]) * d;
    float acc = 0.f;
    for (int m = 0; m < M; ++m) {
        const int j = codes[v * M + m];
        const float* c = cb + (static_cast<int64_t>(m) * kKsub + j) * dsub;
        float dot = 0.f;
        for (int t = 0; t < dsub; ++t) dot = fmaf(cen[m * dsub + t], c[t], dot);
        acc = acc + fmaf(2.f, dot, cbnorm[m * kKsub + j]);
    }
    t2[v] = acc;
}

__global__ void i64_to_i32_kernel(const int64_t* in, int64_t n, int32_t* out) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = static_cast<int32_t>(in[i]);
}

// ---- list maintenance ----
__global__ void hist_kernel(const int32_t* list_no, int64_t n, int64_t* hist) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) atomicAdd(reinterpret_cast<unsigned long long*>(hist + list_no[i]), 1ull);
}
// Lists are stored padded to a multiple of kListPad vectors (the scan kernels read whole
// 32-vector groups without a per-lane bounds check): new length and padded size per list.
__global__ void add_counts_kernel(const int64_t* old_len, const int64_t* new_hist, int nlist, int64_t* new_len,
                                  int64_t* padded) {
    const int l = blockIdx.x * blockDim.x + threadIdx.x;
    if (l < nlist) {
        const int64_t t = old_len[l] + new_hist[l];
        new_len[l] = t;
        padded[l] = (t + kListPad - 1) / kListPad * kListPad;
    }
    if (l == nlist) {
        new_len[l] = 0;
        padded[l] = 0;
    }
}
// Padding slots (and kListPad slots behind the last list): zero codes, label -1, NaN in the
// per-vector term so that a padding slot can never enter a result.
__global__ void fill_pads_kernel(int nlist, const int64_t* off, const int64_t* len, int M, uint8_t* codes,
                                 int64_t* ids, float* t2) {
    const int l = blockIdx.x * (blockDim.x / kListPad) + threadIdx.x / kListPad;
    const int j = threadIdx.x % kListPad;
    if (l > nlist) return;
    const int64_t first = l < nlist ? off[l] + len[l] : off[nlist];
    const int64_t last = l < nlist ? off[l + 1] : off[nlist] + kListPad;
    const int64_t p = first + j;
    if (p >= last) return;
    for (int b = 0; b < M; ++b) codes[p * M + b] = 0;
    ids[p] = -1;
    t2[p] = __int_as_float(0x7fc00000);
}
__global__ void iota_i32_kernel(int32_t* p, int64_t n) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) p[i] = static_cast<int32_t>(i);
}
// Copies one code from position `src` (stored with rotation src_rot) to position `dst`
// (stored with rotation dst & 15 when rotated).
__device__ __forceinline__ void copy_code(const uint8_t* from, uint8_t* to, int M, bool rotated, int64_t src,
                                          int src_rot, int64_t dst) {
    if (!rotated) {
        for (int b = 0; b < M; ++b) to[dst * M + b] = from[src * M + b];
        return;
    }
    const int delta = (static_cast<int>(dst & 15) - src_rot) & 15;
    for (int g = 0; g < M; g += 16)
        for (int s = 0; s < 16; ++s) to[dst * M + g + s] = from[src * M + g + ((s + delta) & 15)];
}
// n_old: old padded size; padding slots of the old layout are skipped.
__global__ void scatter_old_kernel(int64_t n_old, int nlist, const int64_t* old_off, const int64_t* old_len,
                                   const int64_t* new_off, int M, int rotated, const uint8_t* codes, const int64_t* ids,
                                   const float* t2, uint8_t* ncodes, int64_t* nids, float* nt2) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_old) return;
    int lo = 0, hi = nlist;  // largest l with old_off[l] <= i
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (old_off[mid] <= i) lo = mid;
        else hi = mid;
    }
    const int64_t idx = i - old_off[lo];
    if (idx >= old_len[lo]) return;
    const int64_t dst = new_off[lo] + idx;
    copy_code(codes, ncodes, M, rotated != 0, i, static_cast<int>(i & 15), dst);
    nids[dst] = ids[i];
    nt2[dst] = t2[i];
}
__global__ void scatter_new_kernel(int64_t n_new, const int32_t* sorted_list, const int32_t* sorted_src,
                                   const int64_t* old_len, const int64_t* new_off, const int64_t* new_first, int M,
                                   int rotated, const uint8_t* codes, const int64_t* ids, const float* t2,
                                   uint8_t* ncodes, int64_t* nids, float* nt2) {
    const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (j >= n_new) return;
    const int l = sorted_list[j];
    const int64_t src = sorted_src[j];
    const int64_t dst = new_off[l] + old_len[l] + (j - new_first[l]);
    copy_code(codes, ncodes, M, rotated != 0, src, 0, dst);
    nids[dst] = ids[src];
    nt2[dst] = t2 ? t2[src] : 0.f;   // raw encoding: no per-vector term
}

// ---- top-k kept in a warp's registers ----
template <typename L>
__device__ __forceinline__ bool pair_less(float d1, L l1, float d2, L l2) {
    return d1 < d2 || (d1 == d2 && l1 < l2);
}

// Sorted list of 32*KPT (distance, payload) pairs spread over a warp: rank r lives in lane
// r / KPT, slot r % KPT.  Inserting shifts the tail by one with a single shuffle per register.
template <int KPT, typename L>
__device__ __forceinline__ void warp_insert(float (&dk)[KPT], L (&lb)[KPT], float vd, L vl, int lane) {
    const float pd = __shfl_up_sync(0xffffffffu, dk[KPT - 1], 1);
    const L pl = __shfl_up_sync(0xffffffffu, lb[KPT - 1], 1);
    bool ls[KPT];
#pragma unroll
    for (int s = 0; s < KPT; ++s) ls[s] = pair_less<L>(dk[s], lb[s], vd, vl);
    const bool prev_less = lane == 0 ? true : pair_less<L>(pd, pl, vd, vl);
#pragma unroll
    for (int s = KPT - 1; s >= 0; --s) {
        if (!ls[s]) {
            const bool below = s > 0 ? ls[s > 0 ? s - 1 : 0] : prev_less;
            if (below) {
                dk[s] = vd;
                lb[s] = vl;
            } else {
                dk[s] = s > 0 ? dk[s > 0 ? s - 1 : 0] : pd;
                lb[s] = s > 0 ? lb[s > 0 ? s - 1 : 0] : pl;
            }
        }
    }
}

// Bitonic sort of 32 (distance, position) pairs, one per lane, ascending.
__device__ __forceinline__ void warp_sort32(float& d, uint32_t& p, int lane) {
#pragma unroll
    for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            const float od = __shfl_xor_sync(0xffffffffu, d, stride);
            const uint32_t op = __shfl_xor_sync(0xffffffffu, p, stride);
            const bool keep_min = ((lane & stride) == 0) == ((lane & size) == 0);
            const bool other_less = pair_less<uint32_t>(od, op, d, p);
            if (keep_min ? other_less : !other_less) {
                d = od;
                p = op;
            }
        }
    }
}

// First 32 candidates of a warp whose sorted list is still empty: one bitonic sort instead of 32
// insertions.  (d, p): one candidate per lane, (+inf, kNoPos) where the lane has none.
template <int KPT>
__device__ __forceinline__ void warp_fill_sorted(float (&dk)[KPT], uint32_t (&pk)[KPT], float d, uint32_t p, int lane) {
    warp_sort32(d, p, lane);
#pragma unroll
    for (int s = 0; s < KPT; ++s) {
        const int r = lane * KPT + s;          // rank held in this register
        const float fd = __shfl_sync(0xffffffffu, d, r & 31);
        const uint32_t fp = __shfl_sync(0xffffffffu, p, r & 31);
        dk[s] = r < 32 ? fd : __int_as_float(0x7f800000);
        pk[s] = r < 32 ? fp : kNoPos;
    }
}

// (dk, pk) and (od, op): two sorted lists of 32 * KPT pairs in the layout of warp_insert, KPT = 1 or 2.
// Leaves the 32 * KPT smallest of their union, sorted, in (dk, pk): the second list is reversed, the
// element-wise minimum is a bitonic sequence holding the winners, and log2 compare-exchange steps
// sort it.
template <int KPT>
__device__ __forceinline__ void warp_merge_sorted(float (&dk)[KPT], uint32_t (&pk)[KPT], const float (&od)[KPT],
                                                  const uint32_t (&op)[KPT], int lane) {
    static_assert(KPT == 1 || KPT == 2, "register merge is written for k' = 32 and 64");
#pragma unroll
    for (int s = 0; s < KPT; ++s) {
        const float rd = __shfl_sync(0xffffffffu, od[KPT - 1 - s], 31 - lane);
        const uint32_t rp = __shfl_sync(0xffffffffu, op[KPT - 1 - s], 31 - lane);
        if (pair_less<uint32_t>(rd, rp, dk[s], pk[s])) {
            dk[s] = rd;
            pk[s] = rp;
        }
    }
#pragma unroll
    for (int stride = 16; stride > 0; stride >>= 1) {
#pragma unroll
        for (int s = 0; s < KPT; ++s) {
            const float xd = __shfl_xor_sync(0xffffffffu, dk[s], stride);
            const uint32_t xp = __shfl_xor_sync(0xffffffffu, pk[s], stride);
            const bool keep_min = (lane & stride) == 0;
            const bool other_less = pair_less<uint32_t>(xd, xp, dk[s], pk[s]);
            if (keep_min ? other_less : !other_less) {
                dk[s] = xd;
                pk[s] = xp;
            }
        }
    }
    if (KPT == 2) {
        if (pair_less<uint32_t>(dk[KPT - 1], pk[KPT - 1], dk[0], pk[0])) {
            const float td = dk[0];
            const uint32_t tp = pk[0];
            dk[0] = dk[KPT - 1];
            pk[0] = pk[KPT - 1];
            dk[KPT - 1] = td;
            pk[KPT - 1] = tp;
        }
    }
}

// Bitonic sort of E (power of two) pairs held in shared memory, ascending by (distance, payload).
template <typename L>
__device__ __forceinline__ void block_sort_pairs(float* sd, L* sl, int E) {
    for (int size = 2; size <= E; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = threadIdx.x; i < E / 2; i += blockDim.x) {
                const int lo = 2 * i - (i & (stride - 1));
                const int hi = lo + stride;
                const bool up = (lo & size) == 0;
                const float d1 = sd[lo], d2 = sd[hi];
                const L l1 = sl[lo], l2 = sl[hi];
                if (pair_less<L>(d2, l2, d1, l1) == up) {
                    sd[lo] = d2; sd[hi] = d1;
                    sl[lo] = l2; sl[hi] = l1;
                }
            }
            __syncthreads();
        }
    }
}

struct ScanArgs {
    const float* cbT;        // codebooks regrouped [M / 16][256][16][dsub] (fast scan only)
    const int64_t* cI;       // [nq][nprobe] probed list ids (-1 = none)
    const float* cD;         // [nq][nprobe] coarse distances
    int nprobe;
    const int64_t* offsets;  // [nlist + 1] first position of every list (multiples of 32: lists are padded)
    const int64_t* lens;     // [nlist] vectors in every list
    const uint8_t* codes;
    const int64_t* ids;
    const float* t2;
    int by_residual;
    int rotated;
    int k;
    int S;                   // probe splits per query (fast scan)
    int M, d, dsub, nlist;
    int64_t nq;
    const float* xq;         // [nq][d]
    const float* centroids;  // [nlist][d]
    const float* codebooks;  // [M][256][dsub]
    // fast scan output
    float* fd;               // [nq][S][kprime] approximate distances
    uint32_t* fp;            // [nq][S][kprime] positions (kNoPos = empty)
    float* fth;              // [nq][S] worst kept approximate distance when the split's list is full, else +inf
    int kprime;
    float err_rel;           // filter error bound: eps = err_rel * approx + err_abs[q-dependent part]
    float err_abs_c0, err_abs_c1;   // eps_abs = err_abs_c0 * (coarse_max + c1_const) + ... see refine kernel
    float t2_bound;          // bound on |t2|
    float cb_bound;          // sqrt(sum_m max_j |cb|^2)
    // results
    float* outD;             // [nq][k]
    int64_t* outI;
    uint8_t* flag;           // [nq] 1 = not verified, re-scan exactly
    const int32_t* qlist;    // exact scan: indices of the queries to process
    unsigned long long* scanned;
    unsigned int* work;      // persistent scan: next query to hand out (zeroed before the launch)
    unsigned long long* prof;   // development builds (-DB200IDX_DEV_PROF): phase cycle counters, else unused
    // > 0: fd / fth come from the tensor-core filter, which already subtracted the error bound of
    // its fp16 product from every value; only fp32 rounding slack remains (twice the table scan's)
    float tc_rel, tc_abs;
};

// ---------------------------------------------------------------------------------------
// 3a. fast scan (filter)
// ---------------------------------------------------------------------------------------
// Adds the 16 table entries of 16-byte code group G (and the following groups) to acc.
// offb[s]: shared-space byte address of this lane's column in the row of code 0, group 0.
template <int G, int MT>
struct GroupSum {
    static __device__ __forceinline__ void run(const uint4 (&cc)[MT], const uint32_t (&offb)[16], float& acc) {
        const uint32_t w[4] = {cc[G].x, cc[G].y, cc[G].z, cc[G].w};
#pragma unroll
        for (int s = 0; s < 16; ++s) {
            // byte s of the code -> row address code * 128 bytes, + this lane's column
            const uint32_t byte = __byte_perm(w[s >> 2], 0u, 0x4440u + (s & 3));
            const uint32_t addr = byte * 128u + offb[s];
            float val;
            asm("ld.shared.f32 %0, [%1+%2];" : "=f"(val) : "r"(addr), "n"(G * kKsub * 32 * 4));
            acc = acc + val;
        }
        GroupSum<G + 1, MT>::run(cc, offb, acc);
    }
};
template <int MT>
struct GroupSum<MT, MT> {
    static __device__ __forceinline__ void run(const uint4 (&)[MT], const uint32_t (&)[16], float&) {}
};

// Filter table of query q in shared memory, [g][code][32]: entry (m, code) sits in column m % 16 of
// row (m / 16, code) and again 16 columns on.
//   raw encoding      : |q_m - cb[m][code]|^2        residual encoding : -2 q_m . cb[m][code]
// Lane l owns sub-quantizer l % 16; the two half-warps take adjacent codes, so a warp reads 32 * dsub
// contiguous floats of the regrouped codebook per step and its two stores touch 32 distinct banks.
// DS = dsub at compile time (query slice in registers), DS = 0: any dsub.
// pitch: floats per table row (32, or 64 when two queries share a row); warp / nwarps: the
// building warps.
template <int DS>
__device__ __forceinline__ void build_scan_table(const ScanArgs& a, int64_t q, int groups, float* lut, int pitch,
                                                 int warp, int nwarps) {
    const int lane = threadIdx.x & 31;
    const int mm = lane & 15, half = lane >> 4;
    const int dsub = DS > 0 ? DS : a.dsub;
    for (int g = 0; g < groups; ++g) {
        const float* qrow = a.xq + q * a.d + (g * 16 + mm) * dsub;
        float qr[DS > 0 ? DS : 1];
        if (DS > 0) {
#pragma unroll
            for (int t = 0; t < DS; ++t) qr[t] = __ldg(qrow + t);
        }
        if (DS > 0 && DS % 4 == 0) {
            // Four table entries per step, their codeword loads (L2 hits, several hundred cycles
            // each) issued together: entry after entry this loop is one latency chain per entry.
            constexpr int B = 4, V = DS > 0 ? DS / 4 : 1;
            for (int c0 = 2 * warp + half; c0 < kKsub; c0 += 2 * nwarps * B) {
                float4 cv[B][V];
#pragma unroll
                for (int j = 0; j < B; ++j) {
                    const int c = min(c0 + 2 * nwarps * j, kKsub - 1);
                    const float4* cw4 = reinterpret_cast<const float4*>(
                        a.cbT + (static_cast<size_t>(g * kKsub + c) * 16 + mm) * dsub);
#pragma unroll
                    for (int t4 = 0; t4 < V; ++t4) cv[j][t4] = __ldg(cw4 + t4);
                }
#pragma unroll
                for (int j = 0; j < B; ++j) {
                    const int c = c0 + 2 * nwarps * j;
                    if (c >= kKsub) break;
                    float acc = 0.f;
#pragma unroll
                    for (int t4 = 0; t4 < V; ++t4) {
                        const float c4[4] = {cv[j][t4].x, cv[j][t4].y, cv[j][t4].z, cv[j][t4].w};
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            if (a.by_residual) {
                                acc = fmaf(qr[t4 * 4 + u], c4[u], acc);
                            } else {
                                const float df = qr[t4 * 4 + u] - c4[u];
                                acc = fmaf(df, df, acc);
                            }
                        }
                    }
                    if (a.by_residual) acc = -2.f * acc;
                    float* row = lut + (g * kKsub + c) * pitch;
                    row[mm + 16 * half] = acc;
                    row[mm + 16 * (half ^ 1)] = acc;
                }
            }
        } else {
            for (int c = 2 * warp + half; c < kKsub; c += 2 * nwarps) {
                const float* cw = a.cbT + (static_cast<size_t>(g * kKsub + c) * 16 + mm) * dsub;
                float acc = 0.f;
                for (int t = 0; t < dsub; ++t) {
                    const float qt = __ldg(qrow + t);
                    const float ct = __ldg(cw + t);
                    if (a.by_residual) {
                        acc = fmaf(qt, ct, acc);
                    } else {
                        const float df = qt - ct;
                        acc = fmaf(df, df, acc);
                    }
                }
                if (a.by_residual) acc = -2.f * acc;
                float* row = lut + (g * kKsub + c) * pitch;
                row[mm + 16 * half] = acc;
                row[mm + 16 * (half ^ 1)] = acc;
            }
        }
    }
}

// Where a warp gets its probes (inverted lists) from.
//   StaticFeed : probes p_first, p_first + stride, ... in batches of 32 -- lane i fetches the
//                metadata of the batch's i-th probe (list bounds, coarse distance), so the dependent
//                chain probe -> offsets is paid once per batch.
//   SharedFeed : the probes' metadata sits in shared memory and the warps working on the query take
//                them one at a time from a shared counter, so none of them idles while another
//                still has lists to scan.
struct StaticFeed {
    const ScanArgs& a;
    int64_t q;
    int next_p0, stride, lane;
    int li;
    uint32_t my_begin, my_end;
    float my_base;
    unsigned long long& visited;
    __device__ __forceinline__ StaticFeed(const ScanArgs& a_, int64_t q_, int p_first, int p_stride, int lane_,
                                          unsigned long long& visited_)
        : a(a_), q(q_), next_p0(p_first), stride(p_stride), lane(lane_), li(32), my_begin(0), my_end(0),
          my_base(0.f), visited(visited_) {}
    __device__ __forceinline__ bool next(uint32_t& begin, uint32_t& end, float& base) {
        if (li >= 32) {
            if (next_p0 >= a.nprobe) return false;
            my_begin = my_end = 0;
            my_base = 0.f;
            const int p = next_p0 + lane * stride;
            if (p < a.nprobe) {
                const int64_t list = a.cI[q * a.nprobe + p];
                if (list >= 0 && list < a.nlist) {
                    my_begin = static_cast<uint32_t>(a.offsets[list]);
                    my_end = my_begin + static_cast<uint32_t>(a.lens[list]);
                    if (a.by_residual) my_base = a.cD[q * a.nprobe + p];
                }
            }
            visited += my_end - my_begin;   // per lane; all lanes add their share at the end
            next_p0 += 32 * stride;
            li = 0;
        }
        begin = __shfl_sync(0xffffffffu, my_begin, li);
        end = __shfl_sync(0xffffffffu, my_end, li);
        base = __shfl_sync(0xffffffffu, my_base, li);
        ++li;
        return true;
    }
};

// L2 prefetch of the codes (and per-vector terms) of list slots [begin, end): one thread, two bulk
// requests.  begin is a multiple of 32, so both addresses are 128-byte aligned.
__device__ __forceinline__ void prefetch_list_l2(const ScanArgs& a, uint32_t begin, uint32_t end, bool resid) {
    if (end <= begin) return;
    const uint32_t n = end - begin;
    ptx::bulk_prefetch_l2(a.codes + static_cast<size_t>(begin) * a.M, n * static_cast<uint32_t>(a.M));
    if (resid) ptx::bulk_prefetch_l2(a.t2 + begin, ((n + 3u) & ~3u) * 4u);
}

struct SharedFeed {
    const ScanArgs& a;
    const uint32_t* s_begin;   // [nprobe]
    const uint32_t* s_end;
    const float* s_base;
    int* s_next;               // next probe to hand out (starts at 1)
    int nprobe, lane;
    int wslot, nwarps;         // this warp's place among the warps that share the query
    bool resid;
    bool first;
    // The nearest list comes first and is split evenly (in 32-vector groups) over the warps of the
    // query: it is where most of the final neighbours sit, so every warp's kept list -- and with it
    // the bound the warps share -- is tight before the remaining lists are handed out.
    __device__ __forceinline__ bool next(uint32_t& begin, uint32_t& end, float& base) {
        if (first) {
            first = false;
            const uint32_t b = s_begin[0], e = s_end[0];
            const uint32_t groups = (e - b + 31u) >> 5;
            const uint32_t lo = groups * static_cast<uint32_t>(wslot) / static_cast<uint32_t>(nwarps);
            const uint32_t hi = groups * static_cast<uint32_t>(wslot + 1) / static_cast<uint32_t>(nwarps);
            begin = b + 32u * lo;
            end = min(e, b + 32u * hi);
            if (begin > end) begin = end;
            base = s_base[0];
            return true;
        }
        int p = 0;
        if (lane == 0) {
            p = atomicAdd(s_next, 1);
            // the whole list is asked into L2 now; the warp's own loads run a few groups ahead only
            if (p < nprobe) prefetch_list_l2(a, s_begin[p], s_end[p], resid);
        }
        p = __shfl_sync(0xffffffffu, p, 0);
        if (p >= nprobe) return false;
        begin = s_begin[p];
        end = s_end[p];
        base = s_base[p];
        return true;
    }
};

// The filter loop of one warp over the probes its feed hands out.  `sum` adds the table entries of
// one vector's codes to an accumulator; `gth` is the bound shared by the warps that work on the
// same query (float bits, >= 0).  dk / pk: the warp's sorted k' best so far (empty on entry).
// The unit of work is a group of 32 consecutive vectors (lists are stored padded to whole groups);
// U groups, possibly of different lists, form a chunk, and the loads of the next chunk are in flight
// while the current one is processed.  Positions fit 32 bits (an index holds fewer than 2^31
// vectors).  RESID: residual encoding (per-vector term in a.t2, per-list term = coarse distance).
template <int MT, int KPT, bool RESID, typename Sum, typename Feed>
__device__ __forceinline__ void scan_warp_probes(const ScanArgs& a, Feed& feed, int lane, const Sum& sum, int* gth,
                                                 float (&dk)[KPT], uint32_t (&pk)[KPT]) {
    const float kNaN = __int_as_float(0x7fc00000);
    float th_d = __int_as_float(0x7f800000);
    uint32_t th_p = kNoPos;
    bool cold = true;                    // nothing kept yet: the first group is sorted, not inserted
    const uint4* codes4 = reinterpret_cast<const uint4*>(a.codes);
    uint32_t begin = 0, end = 0, v0 = 0;
    float base = 0.f;
    constexpr int U = MT >= 4 ? 1 : 2;   // 32-vector groups per chunk (wide codes: one, the chunk must stay in registers)
    // One chunk in flight: codes, the per-vector term and where it came from.  A padding slot
    // carries NaN in its term (residual encoding: stored in t2; raw encoding: from the list's end),
    // which fails every comparison, so the lookups need no per-lane bounds logic; a group that does
    // not exist (the feed ran dry inside a chunk) is all NaN.
    struct Chunk {
        uint4 c[U][MT];
        float t[U];      // per-vector term (loaded; consumed only when the chunk is processed)
        float bias[U];   // the list's term, or NaN
        uint32_t v0[U];
    };
    // next group of 32 vectors; false when the feed has run dry
    auto next_group = [&](uint32_t& gv0, float& gbias) -> bool {
        while (v0 >= end) {
            if (!feed.next(begin, end, base)) return false;
            v0 = begin;                   // a multiple of 32: lists are stored padded
        }
        gv0 = v0;
        gbias = RESID ? base : ((v0 + lane < end) ? 0.f : kNaN);
        v0 += 32;
        return true;
    };
    auto fetch = [&](Chunk& ch) -> bool {
        bool any = false;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            uint32_t gv0 = u > 0 ? ch.v0[0] : 0u;   // an absent group re-reads a valid address
            float gb = kNaN;
            const bool ok = next_group(gv0, gb);
            if (u == 0 && !ok) return false;
            any = true;
            ch.v0[u] = gv0;
            ch.bias[u] = ok ? gb : kNaN;
            const uint32_t v = gv0 + lane;
            const uint4* cp = codes4 + static_cast<size_t>(v) * MT;
#pragma unroll
            for (int g = 0; g < MT; ++g) ch.c[u][g] = __ldg(cp + g);
            if (RESID) ch.t[u] = __ldg(a.t2 + v);
        }
        return any;
    };
    auto insert_group = [&](float acc, uint32_t v, float lim) {
        const bool pass = acc <= lim && pair_less<uint32_t>(acc, v, th_d, th_p);
        unsigned bal = __ballot_sync(0xffffffffu, pass);
        if constexpr (KPT <= 2) {
            // several candidates at once (the first groups of a near list): sort them and merge the
            // two sorted lists -- a fixed cost, where insertions form one long dependent chain each
            if (__popc(bal) >= 4) {
                float od[KPT];
                uint32_t op[KPT];
                warp_fill_sorted<KPT>(od, op, pass ? acc : __int_as_float(0x7f800000), pass ? v : kNoPos, lane);
                warp_merge_sorted<KPT>(dk, pk, od, op, lane);
                th_d = __shfl_sync(0xffffffffu, dk[KPT - 1], 31);
                th_p = __shfl_sync(0xffffffffu, pk[KPT - 1], 31);
                return;
            }
        }
        while (bal) {
            const int src = __ffs(bal) - 1;
            bal &= bal - 1;
            const float vd = __shfl_sync(0xffffffffu, acc, src);
            const uint32_t vp = __shfl_sync(0xffffffffu, v, src);
            if (pair_less<uint32_t>(vd, vp, th_d, th_p)) {
                warp_insert<KPT, uint32_t>(dk, pk, vd, vp, lane);
                th_d = __shfl_sync(0xffffffffu, dk[KPT - 1], 31);
                th_p = __shfl_sync(0xffffffffu, pk[KPT - 1], 31);
            }
        }
    };
    auto process = [&](const Chunk& ch) {
        // the bound shared with the other warps is read before the lookups and used after them
        const float lim = fminf(th_d, __int_as_float(*reinterpret_cast<volatile int*>(gth)));
        float acc[U];
#pragma unroll
        for (int u = 0; u < U; ++u) acc[u] = RESID ? ch.bias[u] + ch.t[u] : ch.bias[u];
#pragma unroll
        for (int u = 0; u < U; ++u) sum(ch.c[u], acc[u]);
        bool maybe = false;
#pragma unroll
        for (int u = 0; u < U; ++u) maybe |= acc[u] <= lim;
        if (__any_sync(0xffffffffu, maybe)) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t v = ch.v0[u] + lane;   // v & 15 == lane & 15: the stored rotation
                if (u == 0 && cold) {
                    const bool ok = acc[u] <= lim;    // false for NaN
                    warp_fill_sorted<KPT>(dk, pk, ok ? acc[u] : __int_as_float(0x7f800000), ok ? v : kNoPos, lane);
                    th_d = __shfl_sync(0xffffffffu, dk[KPT - 1], 31);
                    th_p = __shfl_sync(0xffffffffu, pk[KPT - 1], 31);
                    cold = false;
                } else {
                    insert_group(acc[u], v, fminf(lim, th_d));
                }
            }
            // a full list bounds what the whole query still needs: publish its worst distance
            // (clamped at 0 so that the integer minimum orders like the float)
            if (lane == 0 && th_d < lim) atomicMin(gth, __float_as_int(fmaxf(th_d, 0.f)));
        }
    };
    Chunk ca, cb;
    bool have = fetch(ca);
    while (have) {
        // the next chunk's loads are in flight while this one is processed
        have = fetch(cb);
        process(ca);
        if (!have) break;
        have = fetch(ca);
        process(cb);
    }
}

// Table lookups of the [g][code][32] layout (128-byte rows): three integer instructions and a load
// per entry.
template <int MT>
struct RowSum128 {
    uint32_t offb[16];   // shared-space byte address of this lane's column in the row of code 0, group 0
    __device__ __forceinline__ void operator()(const uint4 (&c)[MT], float& acc) const {
        GroupSum<0, MT>::run(c, offb, acc);
    }
};

// NT threads per CTA: 128, or 256 when the table (MT x 32 KB) leaves room for only one or two CTAs
// per SM and the warps of a CTA are what hides the load latency.
template <int MT, int KPT, int NT>
// (M = 48: a 96 KB table, two CTAs per SM if each keeps to 128 registers)
__global__ void __launch_bounds__(NT, (MT == 1 && KPT <= 2) ? 6 : ((MT == 3 && KPT <= 8) ? 2 : 1))
ivfpq_fast_scan_kernel(const ScanArgs a) {
    extern __shared__ __align__(16) uint8_t scan_smem[];
    float* lut = reinterpret_cast<float*>(scan_smem);   // [MT][256][32]
    const int64_t q = blockIdx.x;
    const int split = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Smallest "worst kept distance" of any warp of this CTA whose list is full (float bits, >= 0):
    // nothing above it can reach the CTA's k' best, so every warp also filters with it.
    int& s_gth = *reinterpret_cast<int*>(scan_smem + static_cast<size_t>(MT) * kKsub * 32 * 4);
    if (threadIdx.x == 0) s_gth = 0x7f800000;
    switch (a.dsub) {
        case 4: build_scan_table<4>(a, q, MT, lut, 32, warp, NT / 32); break;
        case 8: build_scan_table<8>(a, q, MT, lut, 32, warp, NT / 32); break;
        default: build_scan_table<0>(a, q, MT, lut, 32, warp, NT / 32); break;
    }
    __syncthreads();

    float dk[KPT];
    uint32_t pk[KPT];
#pragma unroll
    for (int s = 0; s < KPT; ++s) {
        dk[s] = __int_as_float(0x7f800000);
        pk[s] = kNoPos;
    }
    unsigned long long visited = 0;

    // Lane l reads sub-quantizer (s + l) mod 16 at step s: its column inside a [code][32] row.
    const uint32_t lut_base = static_cast<uint32_t>(__cvta_generic_to_shared(lut));
    RowSum128<MT> sum;
#pragma unroll
    for (int s = 0; s < 16; ++s) sum.offb[s] = lut_base + 4u * (((s + lane) & 15) + (lane & 16));
    StaticFeed feed(a, q, split + a.S * warp, a.S * (NT / 32), lane, visited);
    if (a.by_residual) scan_warp_probes<MT, KPT, true>(a, feed, lane, sum, &s_gth, dk, pk);
    else scan_warp_probes<MT, KPT, false>(a, feed, lane, sum, &s_gth, dk, pk);
    if (a.scanned && visited) atomicAdd(a.scanned, visited);

    // merge the four warp lists, keep the kprime best of the CTA
    __syncthreads();
    constexpr int E = NT * KPT;
    constexpr int KP = 32 * KPT;
    uint32_t* sp = reinterpret_cast<uint32_t*>(scan_smem);
    float* sd = reinterpret_cast<float*>(scan_smem + static_cast<size_t>(E) * 4);
#pragma unroll
    for (int s = 0; s < KPT; ++s) {
        sd[threadIdx.x * KPT + s] = dk[s];
        sp[threadIdx.x * KPT + s] = pk[s];
    }
    __syncthreads();
    block_sort_pairs<uint32_t>(sd, sp, E);
    float* od = a.fd + (q * a.S + split) * KP;
    uint32_t* op = a.fp + (q * a.S + split) * KP;
    for (int i = threadIdx.x; i < KP; i += NT) {
        od[i] = sd[i];
        op[i] = sp[i];
    }
    if (threadIdx.x == 0) {
        // Everything this CTA dropped has an approximate distance >= the worst kept one; if the
        // kept list is not full nothing was dropped.
        a.fth[q * a.S + split] = sp[KP - 1] != kNoPos ? sd[KP - 1] : __int_as_float(0x7f800000);
    }
}

// ---------------------------------------------------------------------------------------
// 3a'. fast scan for large batches (M = 16): one persistent CTA per SM, four query slots
// ---------------------------------------------------------------------------------------
// A table row of 256 bytes holds the [32]-column rows of TWO queries side by side, and the table
// starts on a 64 KB boundary of the shared window.  The address of an entry is then
//   table | code << 8 | (query half * 128 + 4 * column)
// -- the code value is exactly byte 1 -- so ONE byte-permute of the code word with a per-lane
// constant forms it, against a permute and a multiply-add for 128-byte rows: three instructions
// per lookup instead of four in a loop that is bound by instruction issue.  Two such tables (four
// queries) fit beside the alignment gap; each query slot is worked by six warps, which take the
// next query from a global counter when they are done, so slots never wait for one another.
constexpr int kPsWarpsPerSlot = 6;
constexpr int kPsSlots = 4;
constexpr int kPsSlotThreads = kPsWarpsPerSlot * 32;              // 192
constexpr int kPsThreads = kPsSlots * kPsSlotThreads;             // 768
constexpr int kPsMaxProbe = 256;                                  // probes whose metadata is staged per slot
constexpr int kPsMaxKpt = 2;                                      // k' <= 64 (k <= 48)
constexpr int kPsScratchBytes = 24 * 1024;                        // slot control words, probe metadata, merge buffers
constexpr int kPsSmemBytes = 3 * 65536 + 4096;                    // two aligned tables + gap + room for the scratch

struct RowSum256 {
    uint32_t offb[16];   // table base | (query half * 128 + 4 * this lane's column at step s)
    __device__ __forceinline__ void operator()(const uint4 (&c)[1], float& acc) const {
        const uint32_t w[4] = {c[0].x, c[0].y, c[0].z, c[0].w};
#pragma unroll
        for (int s = 0; s < 16; ++s) {
            // bytes of the address: [offb.0, code byte s, offb.2, offb.3]
            const uint32_t addr = __byte_perm(w[s >> 2], offb[s], 0x7604u | ((s & 3) << 4));
            float val;
            asm("ld.shared.f32 %0, [%1];" : "=f"(val) : "r"(addr));
            acc = acc + val;
        }
    }
};

__device__ __forceinline__ void slot_barrier(int slot) {
    asm volatile("bar.sync %0, %1;" ::"r"(slot + 1), "n"(kPsSlotThreads) : "memory");
}

#ifdef B200IDX_DEV_PROF
// Development build: cycles per phase of the second warp (0-3: table build, wait for the table
// barrier, scan, wait for the scan barrier) and of the first warp (4-8: the same four, then merge and
// output) of every slot, summed over slots; 9: queries.
#define PS_PROF_DECL long long ps_t = clock64(); const int ps_who = tid_s == 32 ? 0 : (tid_s == 0 ? 4 : -1); long long ps_c[5] = {0, 0, 0, 0, 0}; long long ps_n = 0;
#define PS_PROF_MARK(i) do { if (ps_who >= 0) { const long long ps_now = clock64(); ps_c[i] += ps_now - ps_t; ps_t = ps_now; } } while (0)
#define PS_PROF_COUNT() do { ++ps_n; } while (0)
#define PS_PROF_FLUSH() do { if (ps_who >= 0 && a.prof) { for (int i = 0; i < 5; ++i) atomicAdd(a.prof + ps_who + i, static_cast<unsigned long long>(ps_c[i])); if (ps_who == 0) atomicAdd(a.prof + 9, static_cast<unsigned long long>(ps_n)); } } while (0)
#else
#define PS_PROF_DECL
#define PS_PROF_MARK(i) do { } while (0)
#define PS_PROF_COUNT() do { } while (0)
#define PS_PROF_FLUSH() do { } while (0)
#endif

// Per query a slot goes through: table build (all six warps) | barrier | scan | barrier | merge of
// the six kept lists in the registers of the slot's first warp, which also writes the result, while
// the other five warps already build the next query's table.
template <int KPT, bool RESID>
__global__ void __launch_bounds__(kPsThreads, 1)
ivfpq_scan_persist_kernel(const ScanArgs a) {
    extern __shared__ __align__(16) uint8_t ps_smem[];
    const uint32_t base = static_cast<uint32_t>(__cvta_generic_to_shared(ps_smem));
    const uint32_t tab0 = (base + 0xFFFFu) & ~0xFFFFu;      // first 64 KB boundary of the shared window
    const uint32_t gap = tab0 - base;
    uint8_t* tabs = ps_smem + gap;                            // two tables of 64 KB
    uint8_t* scratch = gap >= static_cast<uint32_t>(kPsScratchBytes) ? ps_smem : tabs + 2 * 65536;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slot = warp / kPsWarpsPerSlot, wslot = warp % kPsWarpsPerSlot;
    const int tid_s = threadIdx.x - slot * kPsSlotThreads;
    const int tbl = slot >> 1, half = slot & 1;
    float* lut = reinterpret_cast<float*>(tabs + tbl * 65536) + half * 32;   // this query's half of the rows

    // scratch: per slot {next query, bound, next probe}, the probes' metadata, the kept lists of
    // warps 1 .. 5 of every slot
    constexpr int KP = 32 * KPT;
    unsigned int* s_q = reinterpret_cast<unsigned int*>(scratch);            // [4]
    int* s_gth = reinterpret_cast<int*>(scratch + 16);                       // [4]
    int* s_next = reinterpret_cast<int*>(scratch + 32);                      // [4] next probe of the slot's query
    uint32_t* s_pb = reinterpret_cast<uint32_t*>(scratch + 64) + slot * 3 * kPsMaxProbe;   // list begin
    uint32_t* s_pe = s_pb + kPsMaxProbe;                                                   // list end
    float* s_pbase = reinterpret_cast<float*>(s_pe + kPsMaxProbe);                         // coarse distance
    uint32_t* sp = reinterpret_cast<uint32_t*>(scratch + 64 + kPsSlots * 3 * kPsMaxProbe * 4) +
                   slot * 2 * (kPsWarpsPerSlot - 1) * KP;
    float* sd = reinterpret_cast<float*>(sp + (kPsWarpsPerSlot - 1) * KP);

    unsigned long long visited = 0;
    // the slot's next query is drawn from the global counter one query ahead, so that the round
    // trip of the atomic hides behind the scan
    if (tid_s == 0) {
        s_q[slot] = atomicAdd(a.work, 1u);
        s_gth[slot] = 0x7f800000;
        s_next[slot] = 1;
    }
    slot_barrier(slot);
    PS_PROF_DECL
    bool first_query = true;
    for (;;) {
        const int64_t q = s_q[slot];
        if (q >= a.nq) break;
        PS_PROF_COUNT();
        unsigned int q_next = 0;
        if (tid_s == 0) q_next = atomicAdd(a.work, 1u);
        // the probes' metadata: loads issued here, stored to shared memory after the table is built
        constexpr int kMeta = (kPsMaxProbe + kPsSlotThreads - 1) / kPsSlotThreads;
        uint32_t m_begin[kMeta] = {0, 0};
        uint32_t m_end[kMeta] = {0, 0};
        float m_base[kMeta] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < kMeta; ++j) {
            const int pidx = tid_s + j * kPsSlotThreads;
            if (pidx < a.nprobe) {
                const int64_t list = a.cI[q * a.nprobe + pidx];
                if (list >= 0 && list < a.nlist) {
                    m_begin[j] = static_cast<uint32_t>(a.offsets[list]);
                    m_end[j] = m_begin[j] + static_cast<uint32_t>(a.lens[list]);
                    if (RESID) m_base[j] = a.cD[q * a.nprobe + pidx];
                    // the nearest list is scanned first, by all warps: fetch it while the table is built
                    if (pidx == 0) prefetch_list_l2(a, m_begin[j], m_end[j], RESID);
                }
            }
        }
        // The first warp of the slot is busy merging the previous query's lists (below, at the end of
        // the loop body): the table is built by the other five, by all six for the slot's first query.
        const int bw = first_query ? wslot : wslot - 1;
        const int bn = first_query ? kPsWarpsPerSlot : kPsWarpsPerSlot - 1;
        if (bw >= 0) {
            switch (a.dsub) {
                case 4: build_scan_table<4>(a, q, 1, lut, 64, bw, bn); break;
                case 8: build_scan_table<8>(a, q, 1, lut, 64, bw, bn); break;
                default: build_scan_table<0>(a, q, 1, lut, 64, bw, bn); break;
            }
        }
        first_query = false;
#pragma unroll
        for (int j = 0; j < kMeta; ++j) {
            const int pidx = tid_s + j * kPsSlotThreads;
            if (pidx < a.nprobe) {
                s_pb[pidx] = m_begin[j];
                s_pe[pidx] = m_end[j];
                s_pbase[pidx] = m_base[j];
                visited += m_end[j] - m_begin[j];
            }
        }
        PS_PROF_MARK(0);
        slot_barrier(slot);   // table and metadata complete (and the previous query's merge has read its lists)
        PS_PROF_MARK(1);

        float dk[KPT];
        uint32_t pk[KPT];
#pragma unroll
        for (int s = 0; s < KPT; ++s) {
            dk[s] = __int_as_float(0x7f800000);
            pk[s] = kNoPos;
        }
        // The 16 lookup address constants are formed here, per query, from a value the compiler cannot
        // see through: kept live across the table build they would push its loads out of registers.
        uint32_t lv = static_cast<uint32_t>(lane);
        asm volatile("" : "+r"(lv));
        RowSum256 sum;
#pragma unroll
        for (int s = 0; s < 16; ++s)
            sum.offb[s] = (tab0 + static_cast<uint32_t>(tbl) * 65536u) |
                          (static_cast<uint32_t>(half) * 128u + 4u * (((s + lv) & 15u) + (lv & 16u)));
        SharedFeed feed{a, s_pb, s_pe, s_pbase, &s_next[slot], a.nprobe, lane, wslot, kPsWarpsPerSlot, RESID, true};
        scan_warp_probes<1, KPT, RESID>(a, feed, lane, sum, &s_gth[slot], dk, pk);
        PS_PROF_MARK(2);

        if (wslot > 0) {
#pragma unroll
            for (int s = 0; s < KPT; ++s) {
                sd[(wslot - 1) * KP + lane * KPT + s] = dk[s];
                sp[(wslot - 1) * KP + lane * KPT + s] = pk[s];
            }
        }
        if (tid_s == 0) s_q[slot] = q_next;   // read by everybody after the barrier
        slot_barrier(slot);   // every warp of the slot is done with the table, the bound and the probe counter
        PS_PROF_MARK(3);
        if (wslot == 0) {
            if (lane == 0) {
                s_gth[slot] = 0x7f800000;
                s_next[slot] = 1;
            }
#pragma unroll 1
            for (int w = 0; w < kPsWarpsPerSlot - 1; ++w) {
                float od[KPT];
                uint32_t op[KPT];
#pragma unroll
                for (int s = 0; s < KPT; ++s) {
                    od[s] = sd[w * KP + lane * KPT + s];
                    op[s] = sp[w * KP + lane * KPT + s];
                }
                warp_merge_sorted<KPT>(dk, pk, od, op, lane);
            }
            float* outd = a.fd + q * KP;
            uint32_t* outp = a.fp + q * KP;
#pragma unroll
            for (int s = 0; s < KPT; ++s) {
                outd[lane * KPT + s] = dk[s];
                outp[lane * KPT + s] = pk[s];
            }
            // everything the slot dropped has an approximate distance >= the worst kept one; if the
            // kept list is not full nothing was dropped
            if (lane == 31) a.fth[q] = pk[KPT - 1] != kNoPos ? dk[KPT - 1] : __int_as_float(0x7f800000);
            PS_PROF_MARK(4);
        }
    }
    PS_PROF_FLUSH();
    if (a.scanned && visited) atomicAdd(a.scanned, visited);
}

// Canonical distance of the vector at `pos` (probed through list `list`): sum over m, in
// ascending m, of |(q - c_list)_m - cb[m][code_m]|^2 accumulated with sequential fmaf over the
// sub-vector (c_list = 0 for raw encoding).  Rows are read as float4 where the sub-vector length
// allows: the survivors of a query live in unrelated lists, so every lane streams its own
// centroid row and codewords, and wide loads keep the number of cache transactions down.
__device__ __forceinline__ float exact_distance(const ScanArgs& a, int64_t q, int64_t pos, int64_t list) {
    const uint8_t* code = a.codes + pos * a.M;
    const float* qv = a.xq + q * a.d;
    const float* cen = a.centroids + list * a.d;
    const bool resid = a.by_residual != 0;
    float acc = 0.f;
    if ((a.dsub & 3) == 0) {
        const int d4 = a.dsub >> 2;
        const float4* q4 = reinterpret_cast<const float4*>(qv);
        const float4* c4 = reinterpret_cast<const float4*>(cen);
        for (int m = 0; m < a.M; ++m) {
            const float4* w4 = reinterpret_cast<const float4*>(
                a.codebooks + (static_cast<int64_t>(m) * kKsub + code[code_byte(a.rotated != 0, m, pos)]) * a.dsub);
            float e = 0.f;
            for (int t = 0; t < d4; ++t) {
                float4 r = __ldg(q4 + m * d4 + t);
                if (resid) {
                    const float4 c = __ldg(c4 + m * d4 + t);
                    r.x -= c.x; r.y -= c.y; r.z -= c.z; r.w -= c.w;
                }
                const float4 w = __ldg(w4 + t);
                float df;
                df = r.x - w.x; e = fmaf(df, df, e);
                df = r.y - w.y; e = fmaf(df, df, e);
                df = r.z - w.z; e = fmaf(df, df, e);
                df = r.w - w.w; e = fmaf(df, df, e);
            }
            acc = acc + e;
        }
        return acc;
    }
    for (int m = 0; m < a.M; ++m) {
        const float* cw = a.codebooks +
                          (static_cast<int64_t>(m) * kKsub + code[code_byte(a.rotated != 0, m, pos)]) * a.dsub;
        float e = 0.f;
        for (int t = 0; t < a.dsub; ++t) {
            float r = qv[m * a.dsub + t];
            if (resid) r -= cen[m * a.dsub + t];
            const float df = r - cw[t];
            e = fmaf(df, df, e);
        }
        acc = acc + e;
    }
    return acc;
}

// ---------------------------------------------------------------------------------------
// 3b. exact re-computation of the survivors, ordering by (distance, label), verification
// ---------------------------------------------------------------------------------------
constexpr int kRefMaxProbe = 256;
__global__ void __launch_bounds__(kScanThreads)
ivfpq_refine_kernel(const ScanArgs a, int P) {
    extern __shared__ __align__(16) uint8_t ref_smem[];
    int64_t* sl = reinterpret_cast<int64_t*>(ref_smem);                       // P labels
    float* sd = reinterpret_cast<float*>(ref_smem + static_cast<size_t>(P) * 8);   // P distances
    __shared__ float s_qn2;
    const int64_t q = blockIdx.x;
    const int n_c = a.S * a.kprime;
    // The owning list of a survivor is one of the query's probed lists: their bounds go to shared
    // memory once and the owner is found there, not by a search through the global offsets array.
    __shared__ uint32_t s_lb[kRefMaxProbe], s_le[kRefMaxProbe];
    __shared__ int32_t s_ll[kRefMaxProbe];
    const bool probes_staged = a.by_residual && a.nprobe <= kRefMaxProbe;
    if (probes_staged) {
        for (int p = threadIdx.x; p < a.nprobe; p += kScanThreads) {
            const int64_t list = a.cI[q * a.nprobe + p];
            s_ll[p] = static_cast<int32_t>(list);
            s_lb[p] = list >= 0 ? static_cast<uint32_t>(a.offsets[list]) : 0u;
            s_le[p] = list >= 0 ? s_lb[p] + static_cast<uint32_t>(a.lens[list]) : 0u;
        }
        __syncthreads();
    }
    for (int i = threadIdx.x; i < P; i += kScanThreads) {
        float dist = __int_as_float(0x7f800000);
        int64_t label = kNoLabel;
        if (i < n_c) {
            const uint32_t pos = a.fp[q * n_c + i];
            if (pos != kNoPos) {
                int64_t list = 0;
                if (probes_staged) {
                    for (int p = 0; p < a.nprobe; ++p)
                        if (pos >= s_lb[p] && pos < s_le[p]) list = s_ll[p];
                } else if (a.by_residual) {          // owning list of the position
                    int lo = 0, hi = a.nlist;
                    while (hi - lo > 1) {
                        const int mid = (lo + hi) >> 1;
                        if (a.offsets[mid] <= static_cast<int64_t>(pos)) lo = mid;
                        else hi = mid;
                    }
                    list = lo;
                }
                dist = exact_distance(a, q, pos, list);
                label = a.ids[pos];
            }
        }
        sd[i] = dist;
        sl[i] = label;
    }
    if (threadIdx.x < 32) {   // |q|^2 for the residual error bound
        float s = 0.f;
        if (a.by_residual)
            for (int t = threadIdx.x; t < a.d; t += 32) s = fmaf(a.xq[q * a.d + t], a.xq[q * a.d + t], s);
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (threadIdx.x == 0) s_qn2 = s;
    }
    __syncthreads();
    block_sort_pairs<int64_t>(sd, sl, P);
    for (int i = threadIdx.x; i < a.k; i += kScanThreads) {
        const bool real = i < P && sl[i] != kNoLabel;
        a.outD[q * a.k + i] = real ? sd[i] : kInf;
        a.outI[q * a.k + i] = real ? sl[i] : -1;
    }
    if (threadIdx.x == 0) {
        // Anything a split dropped has approximate distance >= that split's threshold, hence an
        // exact distance >= threshold - eps.  The refined top-k stands if its k-th distance is
        // strictly below that for every split.
        float a_min = __int_as_float(0x7f800000);
        for (int s = 0; s < a.S; ++s) a_min = fminf(a_min, a.fth[q * a.S + s]);
        uint8_t bad = 0;
        if (a_min != __int_as_float(0x7f800000)) {
            float eps = a.err_rel * fabsf(a_min);
            if (a.by_residual) {
                const float coarse_max = a.cD[q * a.nprobe + a.nprobe - 1];
                const float bound = fabsf(coarse_max) + a.t2_bound + 2.f * sqrtf(s_qn2) * a.cb_bound + fabsf(a_min);
                eps = a.err_rel * bound;
                if (a.tc_rel > 0.f) eps = 2.f * eps;   // the kept values are lower bounds already (see ivfpq_tc_scan.cu)
            }
            const int kk = a.k <= P ? a.k : P;
            const bool have_k = sl[kk - 1] != kNoLabel;
            // fewer than k survivors although something was dropped, or the k-th is too close
            if (!have_k || !(sd[kk - 1] < a_min - eps)) bad = 1;
        }
        a.flag[q] = bad;
    }
}

// The same for 32 survivors per query (one split, k' = 32): one WARP per query, a lane per
// survivor, the sort done with shuffles -- no block-wide barriers and four queries per CTA, which
// is what the latency chain survivor -> code -> codewords needs to be hidden by other warps.
constexpr int kRefWarpsPerBlock = 4;
__global__ void __launch_bounds__(kRefWarpsPerBlock * 32)
ivfpq_refine_warp_kernel(const ScanArgs a) {
    __shared__ uint32_t s_lb[kRefWarpsPerBlock][kRefMaxProbe], s_le[kRefWarpsPerBlock][kRefMaxProbe];
    __shared__ int32_t s_ll[kRefWarpsPerBlock][kRefMaxProbe];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t q = static_cast<int64_t>(blockIdx.x) * kRefWarpsPerBlock + warp;
    if (q >= a.nq) return;
    const uint32_t pos = a.fp[q * 32 + lane];
    if (a.by_residual) {
        for (int p = lane; p < a.nprobe; p += 32) {
            const int64_t list = a.cI[q * a.nprobe + p];
            s_ll[warp][p] = static_cast<int32_t>(list);
            const uint32_t b = list >= 0 ? static_cast<uint32_t>(a.offsets[list]) : 0u;
            s_lb[warp][p] = b;
            s_le[warp][p] = list >= 0 ? b + static_cast<uint32_t>(a.lens[list]) : 0u;
        }
        __syncwarp();
    }
    float dist = __int_as_float(0x7f800000);
    int64_t label = kNoLabel;
    if (pos != kNoPos) {
        int64_t list = 0;
        if (a.by_residual)
            for (int p = 0; p < a.nprobe; ++p)
                if (pos >= s_lb[warp][p] && pos < s_le[warp][p]) list = s_ll[warp][p];
        dist = exact_distance(a, q, pos, list);
        label = a.ids[pos];
    }
    float qn2 = 0.f;   // |q|^2 for the residual error bound
    if (a.by_residual)
        for (int t = lane; t < a.d; t += 32) qn2 = fmaf(a.xq[q * a.d + t], a.xq[q * a.d + t], qn2);
    for (int o = 16; o > 0; o >>= 1) qn2 += __shfl_xor_sync(0xffffffffu, qn2, o);
    // bitonic sort of the 32 (distance, label) pairs across the lanes, ascending
    for (int size = 2; size <= 32; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            const float od = __shfl_xor_sync(0xffffffffu, dist, stride);
            const int64_t ol = __shfl_xor_sync(0xffffffffu, label, stride);
            const bool lower = (lane & stride) == 0;              // this lane keeps the smaller of the two ...
            const bool up = (lane & size) == 0;                   // ... in an ascending run
            const bool other_less = pair_less<int64_t>(od, ol, dist, label);
            const bool take = (lower == up) ? other_less : !other_less && !(od == dist && ol == label);
            if (take) {
                dist = od;
                label = ol;
            }
        }
    }
    if (lane < a.k) {
        const bool real = label != kNoLabel;
        a.outD[q * a.k + lane] = real ? dist : kInf;
        a.outI[q * a.k + lane] = real ? label : -1;
    }
    // verification (see ivfpq_refine_kernel): the k-th exact distance against the filter's threshold
    const int kk = a.k <= 32 ? a.k : 32;
    const float dk = __shfl_sync(0xffffffffu, dist, kk - 1);
    const int64_t lk = __shfl_sync(0xffffffffu, label, kk - 1);
    if (lane == 0) {
        const float a_min = a.fth[q];
        uint8_t bad = 0;
        if (a_min != __int_as_float(0x7f800000)) {
            float eps = a.err_rel * fabsf(a_min);
            if (a.by_residual) {
                const float coarse_max = a.cD[q * a.nprobe + a.nprobe - 1];
                const float bound = fabsf(coarse_max) + a.t2_bound + 2.f * sqrtf(qn2) * a.cb_bound + fabsf(a_min);
                eps = a.err_rel * bound;
                if (a.tc_rel > 0.f) eps = 2.f * eps;   // the kept values are lower bounds already (see ivfpq_tc_scan.cu)
            }
            if (lk == kNoLabel || !(dk < a_min - eps)) bad = 1;
        }
        a.flag[q] = bad;
    }
}

// ---------------------------------------------------------------------------------------
// 3c. exact scan (canonical arithmetic), one CTA per listed query.  Residual encoding builds
//     one table per (query, list) in shared memory from q - c_list.
// ---------------------------------------------------------------------------------------
template <int KPT>
__global__ void __launch_bounds__(kScanThreads)
ivfpq_exact_scan_kernel(const ScanArgs a) {
    extern __shared__ __align__(16) uint8_t ex_smem[];
    float* lut = reinterpret_cast<float*>(ex_smem);                  // [M][256] canonical layout
    float* resid = lut + a.M * kKsub;                                // [d]
    const int64_t q = a.qlist ? a.qlist[blockIdx.x] : blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int M = a.M;
    const bool rotated = a.rotated != 0;

    // Canonical table of `resid` (the query, or the query minus a list's centroid): [m][code].
    auto build_table = [&]() {
        for (int i = threadIdx.x; i < M * kKsub; i += kScanThreads) {
            const int m = i / kKsub;
            const float* cw = a.codebooks + static_cast<int64_t>(i) * a.dsub;
            float e = 0.f;
            for (int t = 0; t < a.dsub; ++t) {
                const float df = resid[m * a.dsub + t] - cw[t];
                e = fmaf(df, df, e);
            }
            lut[i] = e;
        }
    };
    if (!a.by_residual) {
        for (int t = threadIdx.x; t < a.d; t += kScanThreads) resid[t] = a.xq[q * a.d + t];
        __syncthreads();
        build_table();
    }
    float dk[KPT];
    int64_t lb[KPT];
#pragma unroll
    for (int s = 0; s < KPT; ++s) {
        dk[s] = __int_as_float(0x7f800000);
        lb[s] = kNoLabel;
    }
    float th_d = __int_as_float(0x7f800000);
    int64_t th_l = kNoLabel;

    for (int p = 0; p < a.nprobe; ++p) {
        const int64_t list = a.cI[q * a.nprobe + p];
        if (list < 0) continue;
        const int64_t begin = a.offsets[list], end = begin + a.lens[list];
        if (begin == end) continue;
        __syncthreads();   // previous list fully scanned before the table changes
        if (a.by_residual) {
            for (int t = threadIdx.x; t < a.d; t += kScanThreads)
                resid[t] = a.xq[q * a.d + t] - a.centroids[list * a.d + t];
            __syncthreads();
            build_table();
        }
        __syncthreads();
        for (int64_t v0 = begin + warp * 32; v0 < end; v0 += kScanThreads) {
            const int64_t v = v0 + lane;
            const bool valid = v < end;
            float acc = 0.f;
            if (valid) {
                const uint8_t* cp = a.codes + v * M;
                for (int m = 0; m < M; ++m) acc = acc + lut[m * kKsub + cp[code_byte(rotated, m, v)]];
            }
            bool pass = valid && acc <= th_d;
            int64_t label = 0;
            if (pass) {
                label = a.ids[v];
                pass = pair_less<int64_t>(acc, label, th_d, th_l);
            }
            unsigned bal = __ballot_sync(0xffffffffu, pass);
            while (bal) {
                const int src = __ffs(bal) - 1;
                bal &= bal - 1;
                const float vd = __shfl_sync(0xffffffffu, acc, src);
                const int64_t vl = __shfl_sync(0xffffffffu, label, src);
                warp_insert<KPT, int64_t>(dk, lb, vd, vl, lane);
                th_d = __shfl_sync(0xffffffffu, dk[KPT - 1], 31);
                th_l = __shfl_sync(0xffffffffu, lb[KPT - 1], 31);
            }
        }
    }
    __syncthreads();
    constexpr int E = kScanThreads * KPT;
    int64_t* sl = reinterpret_cast<int64_t*>(ex_smem);
    float* sd = reinterpret_cast<float*>(ex_smem + static_cast<size_t>(E) * 8);
#pragma unroll
    for (int s = 0; s < KPT; ++s) {
        sd[threadIdx.x * KPT + s] = dk[s];
        sl[threadIdx.x * KPT + s] = lb[s];
    }
    __syncthreads();
    block_sort_pairs<int64_t>(sd, sl, E);
    for (int i = threadIdx.x; i < a.k; i += kScanThreads) {
        const bool real = i < E && sl[i] != kNoLabel;
        a.outD[q * a.k + i] = real ? sd[i] : kInf;
        a.outI[q * a.k + i] = real ? sl[i] : -1;
    }
}

// ---------------------------------------------------------------------------------------
// 3b'. second filter pass for queries the verification turned down.
//      The first pass keeps the k' best approximate distances; when more than k' vectors are (nearly)
//      tied at the boundary -- identical codes: raw encoding of clustered data gives hundreds -- the
//      exact k-th distance cannot be told from the worst kept one and the query is flagged.  The
//      refined result still gives an UPPER bound U of the true k-th distance (k of the kept vectors
//      are at or below it), and every true top-k member has an approximate distance <= U + eps.
//      This pass collects ALL vectors under that fixed threshold (no kept lists, one shared counter),
//      and ivfpq_collect_refine_kernel orders them exactly by (distance, label): ties are then
//      decided by the labels of all tied vectors, as in the exact scan, at the cost of one more
//      filter scan instead of a canonical one.  More than `cap` vectors under the threshold leave
//      the flag set (exact scan).
// ---------------------------------------------------------------------------------------
constexpr int kCollectCap = 1024;

template <int MT>
__global__ void __launch_bounds__(kScanThreads)
ivfpq_collect_kernel(const ScanArgs a, uint32_t* cpos, uint32_t* ccount) {
    extern __shared__ __align__(16) uint8_t col_smem[];
    float* lut = reinterpret_cast<float*>(col_smem);   // [MT][256][32]
    __shared__ unsigned int s_count;
    __shared__ float s_thr;
    const int slot = blockIdx.x;
    const int64_t q = a.qlist[slot];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) s_count = 0;
    switch (a.dsub) {
        case 4: build_scan_table<4>(a, q, MT, lut, 32, warp, kScanThreads / 32); break;
        case 8: build_scan_table<8>(a, q, MT, lut, 32, warp, kScanThreads / 32); break;
        default: build_scan_table<0>(a, q, MT, lut, 32, warp, kScanThreads / 32); break;
    }
    if (warp == 0) {
        float qn2 = 0.f;
        if (a.by_residual)
            for (int t = lane; t < a.d; t += 32) qn2 = fmaf(a.xq[q * a.d + t], a.xq[q * a.d + t], qn2);
        for (int o = 16; o > 0; o >>= 1) qn2 += __shfl_xor_sync(0xffffffffu, qn2, o);
        if (lane == 0) {
            // U: the k-th refined distance of the first pass (+inf when fewer than k were kept)
            const bool have = a.outI[q * a.k + a.k - 1] >= 0;
            const float u = have ? a.outD[q * a.k + a.k - 1] : __int_as_float(0x7f800000);
            float eps = a.err_rel * fabsf(u);
            if (a.by_residual) {
                const float coarse_max = a.cD[q * a.nprobe + a.nprobe - 1];
                eps = a.err_rel * (fabsf(coarse_max) + a.t2_bound + 2.f * sqrtf(qn2) * a.cb_bound + fabsf(u));
            }
            s_thr = u + 2.f * eps;
        }
    }
    __syncthreads();
    const float thr = s_thr;
    RowSum128<MT> sum;
    const uint32_t lut_base = static_cast<uint32_t>(__cvta_generic_to_shared(lut));
#pragma unroll
    for (int s = 0; s < 16; ++s) sum.offb[s] = lut_base + 4u * (((s + lane) & 15) + (lane & 16));
    const uint4* codes4 = reinterpret_cast<const uint4*>(a.codes);
    const unsigned lt = (1u << lane) - 1u;
    for (int p = warp; p < a.nprobe; p += kScanThreads / 32) {
        const int64_t list = a.cI[q * a.nprobe + p];
        if (list < 0 || list >= a.nlist) continue;
        const uint32_t begin = static_cast<uint32_t>(a.offsets[list]);
        const uint32_t end = begin + static_cast<uint32_t>(a.lens[list]);
        const float base = a.by_residual ? a.cD[q * a.nprobe + p] : 0.f;
        for (uint32_t v0 = begin; v0 < end; v0 += 32) {
            const uint32_t v = v0 + lane;          // padded slots carry NaN in t2; raw encoding: bounds test
            uint4 c[MT];
#pragma unroll
            for (int g = 0; g < MT; ++g) c[g] = __ldg(codes4 + static_cast<size_t>(v) * MT + g);
            float acc = a.by_residual ? base + __ldg(a.t2 + v) : (v < end ? 0.f : __int_as_float(0x7fc00000));
            sum(c, acc);
            const bool pass = acc <= thr;
            const unsigned bal = __ballot_sync(0xffffffffu, pass);
            if (bal) {
                unsigned int i0 = 0;
                if (lane == 0) i0 = atomicAdd(&s_count, static_cast<unsigned int>(__popc(bal)));
                i0 = __shfl_sync(0xffffffffu, i0, 0);
                const unsigned int i = i0 + __popc(bal & lt);
                if (pass && i < static_cast<unsigned int>(kCollectCap)) cpos[static_cast<size_t>(slot) * kCollectCap + i] = v;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) ccount[slot] = s_count;
}

// The collected vectors of a flagged query: canonical distances, order by (distance, label), top k.
__global__ void __launch_bounds__(kScanThreads)
ivfpq_collect_refine_kernel(const ScanArgs a, const uint32_t* cpos, const uint32_t* ccount) {
    extern __shared__ __align__(16) uint8_t cr_smem[];
    const int slot = blockIdx.x;
    const int64_t q = a.qlist[slot];
    const unsigned int n = ccount[slot];
    if (n > static_cast<unsigned int>(kCollectCap)) return;   // too many under the threshold: the flag stays set
    int P = 32;
    while (P < static_cast<int>(n)) P <<= 1;
    int64_t* sl = reinterpret_cast<int64_t*>(cr_smem);
    float* sd = reinterpret_cast<float*>(cr_smem + static_cast<size_t>(P) * 8);
    __shared__ uint32_t s_lb[kRefMaxProbe], s_le[kRefMaxProbe];
    __shared__ int32_t s_ll[kRefMaxProbe];
    const bool staged = a.by_residual && a.nprobe <= kRefMaxProbe;
    if (staged) {
        for (int p = threadIdx.x; p < a.nprobe; p += kScanThreads) {
            const int64_t list = a.cI[q * a.nprobe + p];
            const bool ok = list >= 0 && list < a.nlist;
            s_ll[p] = ok ? static_cast<int32_t>(list) : 0;
            s_lb[p] = ok ? static_cast<uint32_t>(a.offsets[list]) : 0u;
            s_le[p] = ok ? s_lb[p] + static_cast<uint32_t>(a.lens[list]) : 0u;
        }
        __syncthreads();
    }
    for (int i = threadIdx.x; i < P; i += kScanThreads) {
        float dist = __int_as_float(0x7f800000);
        int64_t label = kNoLabel;
        if (i < static_cast<int>(n)) {
            const uint32_t pos = cpos[static_cast<size_t>(slot) * kCollectCap + i];
            int64_t list = 0;
            if (staged) {
                for (int p = 0; p < a.nprobe; ++p)
                    if (pos >= s_lb[p] && pos < s_le[p]) list = s_ll[p];
            } else if (a.by_residual) {
                int lo = 0, hi = a.nlist;
                while (hi - lo > 1) {
                    const int mid = (lo + hi) >> 1;
                    if (a.offsets[mid] <= static_cast<int64_t>(pos)) lo = mid;
                    else hi = mid;
                }
                list = lo;
            }
            dist = exact_distance(a, q, pos, list);
            label = a.ids[pos];
        }
        sd[i] = dist;
        sl[i] = label;
    }
    __syncthreads();
    block_sort_pairs<int64_t>(sd, sl, P);
    for (int i = threadIdx.x; i < a.k; i += kScanThreads) {
        const bool real = i < P && sl[i] != kNoLabel;
        a.outD[q * a.k + i] = real ? sd[i] : kInf;
        a.outI[q * a.k + i] = real ? sl[i] : -1;
    }
    if (threadIdx.x == 0) a.flag[q] = 0;
}

template <typename Kern>
cudaError_t set_smem(Kern kern, size_t smem) {
    if (smem > 48 * 1024)
        return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    return cudaSuccess;
}

constexpr int fast_scan_threads(int mt) { return mt >= 2 ? 256 : 128; }

template <int MT>
cudaError_t launch_fast_mt(const ScanArgs& a, int kpt, cudaStream_t st) {
    constexpr int NT = fast_scan_threads(MT);
    // table + the CTA-wide bound; reused for the final merge
    const size_t smem = std::max(static_cast<size_t>(MT) * kKsub * 32 * 4 + 16, static_cast<size_t>(NT) * kpt * 8);
    dim3 grid(static_cast<unsigned>(a.nq), static_cast<unsigned>(a.S));
#define B200_FAST_CASE(KP)                                           \
    case KP: {                                                       \
        auto kern = ivfpq_fast_scan_kernel<MT, KP, NT>;              \
        cudaError_t e = set_smem(kern, smem);                        \
        if (e != cudaSuccess) return e;                              \
        kern<<<grid, NT, smem, st>>>(a);                             \
        return cudaGetLastError();                                   \
    }
    switch (kpt) {
        B200_FAST_CASE(1)
        B200_FAST_CASE(2)
        B200_FAST_CASE(4)
        B200_FAST_CASE(8)
        B200_FAST_CASE(16)
        B200_FAST_CASE(32)
        default: return cudaErrorInvalidValue;
    }
#undef B200_FAST_CASE
}

cudaError_t launch_fast(const ScanArgs& a, int kpt, cudaStream_t st) {
    switch (a.M / 16) {
        case 1: return launch_fast_mt<1>(a, kpt, st);
        case 2: return launch_fast_mt<2>(a, kpt, st);
        case 3: return launch_fast_mt<3>(a, kpt, st);
        case 4: return launch_fast_mt<4>(a, kpt, st);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_persist(const ScanArgs& a, int kpt, int num_sms, cudaStream_t st) {
    cudaError_t e = cudaMemsetAsync(a.work, 0, sizeof(unsigned int), st);
    if (e != cudaSuccess) return e;
#define B200_PS_CASE(KP)                                                                       \
    case KP: {                                                                                 \
        auto kern = a.by_residual ? ivfpq_scan_persist_kernel<KP, true> : ivfpq_scan_persist_kernel<KP, false>; \
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPsSmemBytes); \
        if (e != cudaSuccess) return e;                                                        \
        kern<<<num_sms, kPsThreads, kPsSmemBytes, st>>>(a);                                    \
        return cudaGetLastError();                                                             \
    }
    switch (kpt) {
        B200_PS_CASE(1)
        B200_PS_CASE(2)
        default: return cudaErrorInvalidValue;
    }
#undef B200_PS_CASE
}

cudaError_t launch_exact(const ScanArgs& a, int nq_launch, cudaStream_t st) {
    int kpt = 1;
    while (kpt * 32 < a.k) kpt <<= 1;
    if (kpt > 32) return cudaErrorInvalidValue;
    const size_t smem = std::max(static_cast<size_t>(a.M) * kKsub * 4 + static_cast<size_t>(a.d) * 4,
                                 static_cast<size_t>(kScanThreads) * kpt * 12);
#define B200_EXACT_CASE(KP)                                          \
    case KP: {                                                       \
        auto kern = ivfpq_exact_scan_kernel<KP>;                     \
        cudaError_t e = set_smem(kern, smem);                        \
        if (e != cudaSuccess) return e;                              \
        kern<<<nq_launch, kScanThreads, smem, st>>>(a);              \
        return cudaGetLastError();                                   \
    }
    switch (kpt) {
        B200_EXACT_CASE(1)
        B200_EXACT_CASE(2)
        B200_EXACT_CASE(4)
        B200_EXACT_CASE(8)
        B200_EXACT_CASE(16)
        B200_EXACT_CASE(32)
        default: return cudaErrorInvalidValue;
    }
#undef B200_EXACT_CASE
}

cudaError_t launch_collect(const ScanArgs& a, int nslots, uint32_t* cpos, uint32_t* ccount, cudaStream_t st) {
    const int mt = a.M / 16;
    const size_t smem = static_cast<size_t>(mt) * kKsub * 32 * 4;
    cudaError_t e = cudaSuccess;
#define B200_COLLECT_CASE(MTV)                                                \
    case MTV: {                                                               \
        auto kern = ivfpq_collect_kernel<MTV>;                                \
        e = set_smem(kern, smem);                                             \
        if (e != cudaSuccess) return e;                                       \
        kern<<<nslots, kScanThreads, smem, st>>>(a, cpos, ccount);            \
        break;                                                                \
    }
    switch (mt) {
        B200_COLLECT_CASE(1)
        B200_COLLECT_CASE(2)
        B200_COLLECT_CASE(3)
        B200_COLLECT_CASE(4)
        default: return cudaErrorInvalidValue;
    }
#undef B200_COLLECT_CASE
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    ivfpq_collect_refine_kernel<<<nslots, kScanThreads, static_cast<size_t>(kCollectCap) * 12, st>>>(a, cpos, ccount);
    return cudaGetLastError();
}

inline unsigned blocks_for(int64_t n, int threads) { return static_cast<unsigned>((n + threads - 1) / threads); }
inline int pow2_ceil_int(int v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

}  // namespace

IvfpqIndex::IvfpqIndex(int d, int nlist, int M, int nbits, bool by_residual, int device)
    : d_(d), nlist_(nlist), M_(M), dsub_(d / M), device_(device), by_residual_(by_residual),
      rotated_(M % 16 == 0 && M <= 64) {
    if (nbits != 8) throw std::invalid_argument("IVFPQ supports nbits = 8 only");
    if (M <= 0 || d % M != 0) throw std::invalid_argument("d must be a multiple of M");
    DeviceGuard g(device_);
    B200_CUDA_CHECK(cudaDeviceGetAttribute(&num_sms_, cudaDevAttrMultiProcessorCount, device_));
    coarse_.reset(new FlatIndex(d, kMetricL2, kF32, device));
    offsets_.ensure(static_cast<size_t>(nlist_ + 1) * 8);
    B200_CUDA_CHECK(cudaMemset(offsets_.get(), 0, static_cast<size_t>(nlist_ + 1) * 8));
    offsets_host_.assign(static_cast<size_t>(nlist_ + 1), 0);
    lens_.ensure(static_cast<size_t>(nlist_ + 1) * 8);
    B200_CUDA_CHECK(cudaMemset(lens_.get(), 0, static_cast<size_t>(nlist_ + 1) * 8));
    lens_host_.assign(static_cast<size_t>(nlist_ + 1), 0);
    w_tmp_.ensure(sizeof(unsigned long long));
    B200_CUDA_CHECK(cudaMemset(w_tmp_.get(), 0, sizeof(unsigned long long)));
    const char* e = std::getenv("B200IDX_IVFPQ_EXACT");
    force_exact_ = e && std::strcmp(e, "1") == 0;
#ifdef B200IDX_DEV_PROF
    const char* np = std::getenv("B200IDX_IVFPQ_NO_PERSIST");   // development builds: always the per-query CTAs
    no_persist_ = np && std::strcmp(np, "1") == 0;
#endif
    const char* tc = std::getenv("B200IDX_IVFPQ_TC");
    tc_scan_ = tc && std::strcmp(tc, "1") == 0;
    w_work_.ensure(sizeof(unsigned int));
}

IvfpqIndex::~IvfpqIndex() {
    DeviceGuard g(device_);
    cudaStreamSynchronize(stream());
}

void IvfpqIndex::set_centroids(const float* c) {
    DeviceGuard g(device_);
    coarse_->reset();
    coarse_->add(nlist_, c, false, nullptr, false);
    has_centroids_ = true;
}

void IvfpqIndex::set_codebooks(const float* cb) {
    DeviceGuard g(device_);
    const size_t bytes = static_cast<size_t>(M_) * kKsub * dsub_ * 4;
    codebooks_.ensure(bytes);
    cbnorm_.ensure(static_cast<size_t>(M_) * kKsub * 4);
    B200_CUDA_CHECK(cudaMemcpyAsync(codebooks_.get(), cb, bytes, cudaMemcpyHostToDevice, stream()));
    cb_norm_kernel<<<blocks_for(M_ * kKsub, 256), 256, 0, stream()>>>(codebooks_.as<float>(), M_, dsub_,
                                                                     cbnorm_.as<float>());
    B200_CUDA_CHECK(cudaGetLastError());
    B200_CUDA_CHECK(cudaStreamSynchronize(stream()));
    double acc = 0.0;
    for (int m = 0; m < M_; ++m) {
        double mx = 0.0;
        for (int j = 0; j < kKsub; ++j) {
            double s = 0.0;
            const float* c = cb + (static_cast<size_t>(m) * kKsub + j) * dsub_;
            for (int t = 0; t < dsub_; ++t) s += static_cast<double>(c[t]) * c[t];
            mx = std::max(mx, s);
        }
        acc += mx;
    }
    cb_norm_bound_ = static_cast<float>(std::sqrt(acc) * 1.0001);
    {   // fp16 copy for the tensor-core scan; usable while every entry stays inside the fp16 range
        float amax = 0.f;
        const size_t ne = static_cast<size_t>(M_) * kKsub * dsub_;
        for (size_t i = 0; i < ne; ++i) amax = std::max(amax, std::fabs(cb[i]));
        tc_cb_ok_ = amax < 3.0e4f;
        cb16_.ensure(ne * 2);
        B200_CUDA_CHECK(launch_tc_cb16(codebooks_.as<float>(), static_cast<int64_t>(ne), cb16_.as<uint16_t>(), stream()));
        B200_CUDA_CHECK(cudaStreamSynchronize(stream()));
    }
    if (rotated_) {
        // [M / 16][256][16][dsub]: the 16 codewords (one per sub-quantizer of a group) that share a
        // code value lie together, the order in which the scan kernel builds its table
        std::vector<float> t(static_cast<size_t>(M_) * kKsub * dsub_);
        for (int m = 0; m < M_; ++m)
            for (int j = 0; j < kKsub; ++j)
                std::memcpy(&t[((static_cast<size_t>(m >> 4) * kKsub + j) * 16 + (m & 15)) * dsub_],
                            cb + (static_cast<size_t>(m) * kKsub + j) * dsub_, static_cast<size_t>(dsub_) * 4);
        codebooks_t_.ensure(bytes);
        B200_CUDA_CHECK(cudaMemcpy(codebooks_t_.get(), t.data(), bytes, cudaMemcpyHostToDevice));
    }
    has_codebooks_ = true;
}

namespace {
// sub[i][t] = x[i][m * dsub + t] - (cent ? cent[assign[i]][m * dsub + t] : 0)
__global__ void train_subspace_kernel(const float* x, int64_t n, int d, int m, int dsub, const float* cent,
                                      const int32_t* assign, float* sub) {
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= n * dsub) return;
    const int64_t i = idx / dsub;
    const int t = static_cast<int>(idx % dsub);
    float v = x[i * d + m * dsub + t];
    if (cent) v = v - cent[static_cast<int64_t>(assign[i]) * d + m * dsub + t];
    sub[idx] = v;
}
}  // namespace

void IvfpqIndex::train(int64_t n, const float* x_host, int niter, uint64_t seed) {
    if (n < std::max(nlist_, kKsub)) throw std::invalid_argument("training needs at least max(nlist, 256) vectors");
    DeviceGuard g(device_);
    DeviceBuffer xd, cd, ad, sd, cbd;
    float* x = static_cast<float*>(xd.ensure(static_cast<size_t>(n) * d_ * 4));
    float* cent = static_cast<float*>(cd.ensure(static_cast<size_t>(nlist_) * d_ * 4));
    int32_t* assign = static_cast<int32_t*>(ad.ensure(static_cast<size_t>(n) * 4));
    float* sub = static_cast<float*>(sd.ensure(static_cast<size_t>(n) * dsub_ * 4));
    float* cb = static_cast<float*>(cbd.ensure(static_cast<size_t>(kKsub) * dsub_ * 4));
    B200_CUDA_CHECK(cudaMemcpy(x, x_host, static_cast<size_t>(n) * d_ * 4, cudaMemcpyHostToDevice));
    kmeans_device(device_, d_, n, x, nlist_, niter, seed, cent, assign);   // refuses non-finite input
    std::vector<float> hc(static_cast<size_t>(nlist_) * d_), hcb(static_cast<size_t>(M_) * kKsub * dsub_);
    B200_CUDA_CHECK(cudaMemcpy(hc.data(), cent, hc.size() * 4, cudaMemcpyDeviceToHost));
    for (int m = 0; m < M_; ++m) {
        train_subspace_kernel<<<blocks_for(n * dsub_, 256), 256>>>(x, n, d_, m, dsub_, by_residual_ ? cent : nullptr,
                                                                   assign, sub);
        B200_CUDA_CHECK(cudaGetLastError());
        B200_CUDA_CHECK(cudaDeviceSynchronize());
        kmeans_device(device_, dsub_, n, sub, kKsub, niter, seed + 1 + static_cast<uint64_t>(m), cb, nullptr);
        B200_CUDA_CHECK(cudaMemcpy(hcb.data() + static_cast<size_t>(m) * kKsub * dsub_, cb,
                                   static_cast<size_t>(kKsub) * dsub_ * 4, cudaMemcpyDeviceToHost));
    }
    set_centroids(hc.data());
    set_codebooks(hcb.data());
}

void IvfpqIndex::get_centroids(float* out) const { coarse_->get_base(0, nlist_, out); }

void IvfpqIndex::get_codebooks(float* out) const {
    DeviceGuard g(device_);
    B200_CUDA_CHECK(cudaMemcpy(out, codebooks_.get(), static_cast<size_t>(M_) * kKsub * dsub_ * 4,
                               cudaMemcpyDeviceToHost));
}

void IvfpqIndex::compute_t2(int64_t n, const int32_t* list_no, const uint8_t* codes, float* t2) {
    t2_kernel<<<blocks_for(n, 128), 128, 0, stream()>>>(n, d_, M_, dsub_, codebooks_.as<float>(),
                                                        cbnorm_.as<float>(), coarse_->rows_f32(), list_no, codes, t2);
    B200_CUDA_CHECK(cudaGetLastError());
}

void IvfpqIndex::add(int64_t n, const float* x, const int64_t* ids, bool x_on_device) {
    if (n <= 0) return;
    if (!is_trained()) throw std::invalid_argument("IVFPQ index is not trained (centroids / codebooks missing)");
    DeviceGuard g(device_);
    cudaStream_t st = stream();
    // A vector with a NaN or an infinite component has no nearest centroid (its assignment would be
    // -1): the whole batch is refused before anything changes.
    int* vflag = static_cast<int*>(w_vflag_.ensure(sizeof(int)));
    auto read_flag = [&]() {
        int hf = 0;
        B200_CUDA_CHECK(cudaMemcpyAsync(&hf, vflag, sizeof(int), cudaMemcpyDeviceToHost, st));
        B200_CUDA_CHECK(cudaStreamSynchronize(st));
        return hf;
    };
    if (x_on_device) {
        B200_CUDA_CHECK(cudaMemsetAsync(vflag, 0, sizeof(int), st));
        B200_CUDA_CHECK(launch_check_finite(x, n * d_, vflag, st));
        if (read_flag()) throw std::invalid_argument("add: x holds NaN or infinite values");
    } else {
        const uint32_t* bits = reinterpret_cast<const uint32_t*>(x);
        uint32_t bad = 0;
        for (int64_t i = 0; i < n * d_; ++i) bad |= static_cast<uint32_t>((bits[i] & 0x7f800000u) == 0x7f800000u);
        if (bad) throw std::invalid_argument("add: x holds NaN or infinite values");
    }
    const int64_t chunk = 1 << 20;
    for (int64_t off = 0; off < n; off += chunk) {
        const int64_t m = std::min(chunk, n - off);
        const float* xd;
        if (x_on_device) {
            xd = x + off * d_;
        } else {
            float* buf = static_cast<float*>(w_x_.ensure(static_cast<size_t>(m) * d_ * 4));
            B200_CUDA_CHECK(cudaMemcpyAsync(buf, x + off * d_, static_cast<size_t>(m) * d_ * 4,
                                            cudaMemcpyHostToDevice, st));
            xd = buf;
        }
        float* aD = static_cast<float*>(w_assign_D_.ensure(static_cast<size_t>(m) * 4));
        int64_t* aI = static_cast<int64_t*>(w_assign_I_.ensure(static_cast<size_t>(m) * 8));
        coarse_->search_device(m, xd, false, 1, aD, aI, 1);
        int32_t* ln = static_cast<int32_t*>(w_list_.ensure(static_cast<size_t>(m) * 4));
        i64_to_i32_kernel<<<blocks_for(m, 256), 256, 0, st>>>(aI, m, ln);
        // finite input can still overflow to an infinite distance: no assignment may leave [0, nlist)
        B200_CUDA_CHECK(cudaMemsetAsync(vflag, 0, sizeof(int), st));
        B200_CUDA_CHECK(launch_check_range_i32(ln, m, nlist_, vflag, st));
        if (read_flag()) throw std::invalid_argument("add: a vector could not be assigned to a list (distance overflow)");
        uint8_t* cd = static_cast<uint8_t*>(w_codes_.ensure(static_cast<size_t>(m) * M_));
        encode_kernel<<<blocks_for(m * M_, 8), 256, 0, st>>>(xd, m, d_, M_, dsub_, codebooks_.as<float>(),
                                                             by_residual_ ? 1 : 0, coarse_->rows_f32(), ln, cd);
        B200_CUDA_CHECK(cudaGetLastError());
        float* t2 = nullptr;
        if (by_residual_) {
            t2 = static_cast<float*>(w_t2_.ensure(static_cast<size_t>(m) * 4));
            compute_t2(m, ln, cd, t2);
        }
        int64_t* idd = static_cast<int64_t*>(w_ids_.ensure(static_cast<size_t>(m) * 8));
        if (ids) B200_CUDA_CHECK(cudaMemcpyAsync(idd, ids + off, static_cast<size_t>(m) * 8, cudaMemcpyHostToDevice, st));
        else B200_CUDA_CHECK(launch_iota_i64(idd, m, n_, st));
        merge_new(m, ln, cd, t2, idd);
    }
}

void IvfpqIndex::add_codes(int64_t n, const int32_t* list_no, const uint8_t* codes, const int64_t* ids) {
    if (n <= 0) return;
    if (!is_trained()) throw std::invalid_argument("IVFPQ index is not trained (centroids / codebooks missing)");
    for (int64_t i = 0; i < n; ++i)
        if (list_no[i] < 0 || list_no[i] >= nlist_) throw std::invalid_argument("add_codes: list id out of range");
    DeviceGuard g(device_);
    cudaStream_t st = stream();
    int32_t* ln = static_cast<int32_t*>(w_list_.ensure(static_cast<size_t>(n) * 4));
    uint8_t* cd = static_cast<uint8_t*>(w_codes_.ensure(static_cast<size_t>(n) * M_));
    int64_t* idd = static_cast<int64_t*>(w_ids_.ensure(static_cast<size_t>(n) * 8));
    B200_CUDA_CHECK(cudaMemcpyAsync(ln, list_no, static_cast<size_t>(n) * 4, cudaMemcpyHostToDevice, st));
    B200_CUDA_CHECK(cudaMemcpyAsync(cd, codes, static_cast<size_t>(n) * M_, cudaMemcpyHostToDevice, st));
    if (ids) B200_CUDA_CHECK(cudaMemcpyAsync(idd, ids, static_cast<size_t>(n) * 8, cudaMemcpyHostToDevice, st));
    else B200_CUDA_CHECK(launch_iota_i64(idd, n, n_, st));
    float* t2 = nullptr;
    if (by_residual_) {
        t2 = static_cast<float*>(w_t2_.ensure(static_cast<size_t>(n) * 4));
        compute_t2(n, ln, cd, t2);
    }
    merge_new(n, ln, cd, t2, idd);
}

// Stable merge of a batch into the CSR lists: existing entries keep their order, new entries
// follow in arrival order (the order the reference's per-list append produces).  Codes are
// re-rotated for their new positions on the way.
void IvfpqIndex::merge_new(int64_t n, const int32_t* ln, const uint8_t* cd, const float* t2, const int64_t* idd) {
    cudaStream_t st = stream();
    const int64_t n_new_total = n_ + n;
    // upper bound of the padded size; the exact value is known after the scan below
    const int64_t pad_bound = n_new_total + static_cast<int64_t>(kListPad) * (nlist_ + 1);
    if (pad_bound > 0x7FFFFFF0ll) throw std::invalid_argument("a single-device IVFPQ index holds at most 2^31 - 16 vectors (padding included)");
    DeviceBuffer hist, new_len, padded, new_off, new_first, keys_out, vals_in, vals_out, cub_tmp;
    DeviceBuffer ncodes, nids, nt2;
    int64_t* h = static_cast<int64_t*>(hist.ensure(static_cast<size_t>(nlist_ + 1) * 8));
    B200_CUDA_CHECK(cudaMemsetAsync(h, 0, static_cast<size_t>(nlist_ + 1) * 8, st));
    hist_kernel<<<blocks_for(n, 256), 256, 0, st>>>(ln, n, h);
    int64_t* nlen = static_cast<int64_t*>(new_len.ensure(static_cast<size_t>(nlist_ + 1) * 8));
    int64_t* pad = static_cast<int64_t*>(padded.ensure(static_cast<size_t>(nlist_ + 1) * 8));
    add_counts_kernel<<<blocks_for(nlist_ + 1, 256), 256, 0, st>>>(lens_.as<int64_t>(), h, nlist_, nlen, pad);
    int64_t* noff = static_cast<int64_t*>(new_off.ensure(static_cast<size_t>(nlist_ + 1) * 8));
    int64_t* nfirst = static_cast<int64_t*>(new_first.ensure(static_cast<size_t>(nlist_ + 1) * 8));
    size_t tmp_bytes = 0, tb = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, tmp_bytes, pad, noff, nlist_ + 1, st);
    int32_t* kout = static_cast<int32_t*>(keys_out.ensure(static_cast<size_t>(n) * 4));
    int32_t* vin = static_cast<int32_t*>(vals_in.ensure(static_cast<size_t>(n) * 4));
    int32_t* vout = static_cast<int32_t*>(vals_out.ensure(static_cast<size_t>(n) * 4));
    int end_bit = 1;
    while ((1 << end_bit) < nlist_) ++end_bit;
    cub::DeviceRadixSort::SortPairs(nullptr, tb, ln, kout, vin, vout, static_cast<int>(n), 0, end_bit, st);
    tmp_bytes = std::max(tmp_bytes, tb);
    void* tmp = cub_tmp.ensure(tmp_bytes + 16);
    size_t tsz = tmp_bytes;
    B200_CUDA_CHECK(cub::DeviceScan::ExclusiveSum(tmp, tsz, pad, noff, nlist_ + 1, st));
    tsz = tmp_bytes;
    B200_CUDA_CHECK(cub::DeviceScan::ExclusiveSum(tmp, tsz, h, nfirst, nlist_ + 1, st));
    iota_i32_kernel<<<blocks_for(n, 256), 256, 0, st>>>(vin, n);
    tsz = tmp_bytes;
    B200_CUDA_CHECK(cub::DeviceRadixSort::SortPairs(tmp, tsz, ln, kout, vin, vout, static_cast<int>(n), 0, end_bit, st));
    uint8_t* nc = static_cast<uint8_t*>(ncodes.ensure(static_cast<size_t>(pad_bound) * M_ + 64));
    int64_t* ni = static_cast<int64_t*>(nids.ensure(static_cast<size_t>(pad_bound) * 8));
    float* nt = static_cast<float*>(nt2.ensure(static_cast<size_t>(pad_bound) * 4));
    if (n_pad_ > 0)
        scatter_old_kernel<<<blocks_for(n_pad_, 256), 256, 0, st>>>(n_pad_, nlist_, offsets_.as<int64_t>(),
                                                                    lens_.as<int64_t>(), noff, M_, rotated_ ? 1 : 0,
                                                                    codes_.as<uint8_t>(), ids_.as<int64_t>(),
                                                                    t2_.as<float>(), nc, ni, nt);
    scatter_new_kernel<<<blocks_for(n, 256), 256, 0, st>>>(n, kout, vout, lens_.as<int64_t>(), noff, nfirst, M_,
                                                           rotated_ ? 1 : 0, cd, idd, t2, nc, ni, nt);
    fill_pads_kernel<<<blocks_for(static_cast<int64_t>(nlist_ + 1) * kListPad, 256), 256, 0, st>>>(nlist_, noff, nlen, M_,
                                                                                               nc, ni, nt);
    B200_CUDA_CHECK(cudaGetLastError());
    B200_CUDA_CHECK(cudaMemcpyAsync(offsets_host_.data(), noff, static_cast<size_t>(nlist_ + 1) * 8,
                                    cudaMemcpyDeviceToHost, st));
    B200_CUDA_CHECK(cudaMemcpyAsync(lens_host_.data(), nlen, static_cast<size_t>(nlist_ + 1) * 8,
                                    cudaMemcpyDeviceToHost, st));
    B200_CUDA_CHECK(cudaStreamSynchronize(st));
    offsets_.swap(new_off);
    lens_.swap(new_len);
    codes_.swap(ncodes);
    ids_.swap(nids);
    t2_.swap(nt2);
    n_ = n_new_total;
    n_pad_ = offsets_host_[static_cast<size_t>(nlist_)];
}

void IvfpqIndex::reset() {
    DeviceGuard g(device_);
    cudaStreamSynchronize(stream());
    n_ = 0;
    n_pad_ = 0;
    cudaMemset(offsets_.get(), 0, static_cast<size_t>(nlist_ + 1) * 8);
    cudaMemset(lens_.get(), 0, static_cast<size_t>(nlist_ + 1) * 8);
    offsets_host_.assign(static_cast<size_t>(nlist_ + 1), 0);
    lens_host_.assign(static_cast<size_t>(nlist_ + 1), 0);
}

// codes: n stored codes starting at CSR position first_pos -> canonical byte order, in place.
void IvfpqIndex::unrotate_host(uint8_t* codes, int64_t first_pos, int64_t n) const {
    if (!rotated_) return;
    uint8_t tmp[16];
    for (int64_t i = 0; i < n; ++i) {
        const int rot = static_cast<int>((first_pos + i) & 15);
        for (int g = 0; g < M_; g += 16) {
            uint8_t* c = codes + i * M_ + g;
            for (int m = 0; m < 16; ++m) tmp[m] = c[(m - rot) & 15];
            std::memcpy(c, tmp, 16);
        }
    }
}

int64_t IvfpqIndex::remove_ids(int64_t n, const int64_t* ids) {
    if (n <= 0 || n_ == 0) return 0;
    DeviceGuard g(device_);
    std::vector<int64_t> hid(static_cast<size_t>(n_pad_));
    std::vector<uint8_t> hcodes(static_cast<size_t>(n_pad_) * M_);
    B200_CUDA_CHECK(cudaMemcpy(hid.data(), ids_.get(), hid.size() * 8, cudaMemcpyDeviceToHost));
    B200_CUDA_CHECK(cudaMemcpy(hcodes.data(), codes_.get(), hcodes.size(), cudaMemcpyDeviceToHost));
    unrotate_host(hcodes.data(), 0, n_pad_);
    std::unordered_set<int64_t> rm(ids, ids + n);
    std::vector<int32_t> ln;
    std::vector<int64_t> kid;
    std::vector<uint8_t> kc;
    ln.reserve(hid.size());
    kid.reserve(hid.size());
    kc.reserve(hcodes.size());
    int64_t removed = 0;
    for (int l = 0; l < nlist_; ++l)
        for (int64_t v = offsets_host_[l]; v < offsets_host_[l] + lens_host_[l]; ++v) {
            if (rm.count(hid[static_cast<size_t>(v)])) {
                ++removed;
                continue;
            }
            ln.push_back(l);
            kid.push_back(hid[static_cast<size_t>(v)]);
            kc.insert(kc.end(), hcodes.begin() + v * M_, hcodes.begin() + (v + 1) * M_);
        }
    if (removed == 0) return 0;
    reset();
    if (!ln.empty()) add_codes(static_cast<int64_t>(ln.size()), ln.data(), kc.data(), kid.data());
    return removed;
}

int64_t IvfpqIndex::list_length(int list) const {
    if (list < 0 || list >= nlist_) throw std::invalid_argument("list id out of range");
    return lens_host_[static_cast<size_t>(list)];
}

void IvfpqIndex::get_list(int list, uint8_t* codes, int64_t* ids) const {
    const int64_t len = list_length(list);
    if (len == 0) return;
    DeviceGuard g(device_);
    const int64_t b = offsets_host_[static_cast<size_t>(list)];
    if (codes) {
        B200_CUDA_CHECK(cudaMemcpy(codes, codes_.as<uint8_t>() + b * M_, static_cast<size_t>(len) * M_,
                                   cudaMemcpyDeviceToHost));
        unrotate_host(codes, b, len);
    }
    if (ids) B200_CUDA_CHECK(cudaMemcpy(ids, ids_.as<int64_t>() + b, static_cast<size_t>(len) * 8, cudaMemcpyDeviceToHost));
}

void IvfpqIndex::coarse_device(int64_t nq, const float* xq, float* cD, int64_t* cI) {
    if (nq <= 0) return;
    if (!is_trained()) throw std::invalid_argument("IVFPQ index is not trained (centroids / codebooks missing)");
    DeviceGuard g(device_);
    cudaStream_t st = stream();
    const int nprobe = std::max(1, std::min(nprobe_, nlist_));
    timer_.begin(kStageCoarse, st);
    coarse_->search_device(nq, xq, false, nprobe, cD, cI, nprobe);
    timer_.end(st);
    B200_CUDA_CHECK(cudaStreamSynchronize(st));
    timer_.collect(stats_);
    stats_.kernel_launches += coarse_->stats().kernel_launches;
    stats_.gemm_launches += coarse_->stats().gemm_launches;
    coarse_->stats().kernel_launches = 0;
    coarse_->stats().gemm_launches = 0;
}

void IvfpqIndex::search_device(int64_t nq, const float* xq, int k, float* D, int64_t* I) {
    search_stages(nq, xq, k, D, I, nullptr, nullptr);
}

void IvfpqIndex::search_preassigned_device(int64_t nq, const float* xq, int k, const float* cD, const int64_t* cI,
                                           float* D, int64_t* I) {
    if (!cD || !cI) throw std::invalid_argument("search_preassigned needs the probe lists and their distances");
    search_stages(nq, xq, k, D, I, cD, cI);
}

// pre_cD / pre_cI: [nq][nprobe] probe distances and list ids computed elsewhere (nullptr: run the
// coarse stage here).
void IvfpqIndex::search_stages(int64_t nq, const float* xq, int k, float* D, int64_t* I, const float* pre_cD,
                               const int64_t* pre_cI) {
    if (nq <= 0) return;
    if (!is_trained()) throw std::invalid_argument("IVFPQ index is not trained (centroids / codebooks missing)");
    if (k > 1024) throw std::invalid_argument("IVFPQ search supports k <= 1024");
    DeviceGuard g(device_);
    cudaStream_t st = stream();
    stats_.searches += 1;
    stats_.queries += static_cast<uint64_t>(nq);
    const int nprobe = std::max(1, std::min(nprobe_, nlist_));
    // filter width: k' = 32 * KPT >= k + 16
    int kpt = 1;
    while (kpt * 32 < k + 16) kpt <<= 1;
    const bool fast = rotated_ && !force_exact_ && kpt <= 32;
    const int kprime = 32 * kpt;
    const int64_t page = 16384;
    unsigned long long scanned = stats_.scan_codes;
    const unsigned long long* scanned_src = &scanned;
    bool idle = true;    // the stream has been synchronised and nothing was queued since
    for (int64_t q0 = 0; q0 < nq; q0 += page) {
        const int64_t m = std::min(page, nq - q0);
        const float* xp = xq + q0 * d_;
        const float* cD;
        const int64_t* cI;
        if (pre_cI) {
            cD = pre_cD + q0 * nprobe;
            cI = pre_cI + q0 * nprobe;
        } else {
            float* wD = static_cast<float*>(w_cD_.ensure(static_cast<size_t>(m) * nprobe * 4));
            int64_t* wI = static_cast<int64_t*>(w_cI_.ensure(static_cast<size_t>(m) * nprobe * 8));
            timer_.begin(kStageCoarse, st);
            coarse_->search_device(m, xp, false, nprobe, wD, wI, nprobe);
            timer_.end(st);
            cD = wD;
            cI = wI;
        }

        ScanArgs a{};
        a.cbT = codebooks_t_.as<float>();
        a.cI = cI;
        a.cD = cD;
        a.nprobe = nprobe;
        a.offsets = offsets_.as<int64_t>();
        a.lens = lens_.as<int64_t>();
        a.codes = codes_.as<uint8_t>();
        a.ids = ids_.as<int64_t>();
        a.t2 = t2_.as<float>();
        a.by_residual = by_residual_ ? 1 : 0;
        a.rotated = rotated_ ? 1 : 0;
        a.k = k;
        a.M = M_;
        a.d = d_;
        a.dsub = dsub_;
        a.nlist = nlist_;
        a.nq = m;
        a.xq = xp;
        a.centroids = coarse_->rows_f32();
        a.codebooks = codebooks_.as<float>();
        a.outD = D + q0 * k;
        a.outI = I + q0 * k;
        a.scanned = w_tmp_.as<unsigned long long>();
        a.qlist = nullptr;

        if (!fast) {
            timer_.begin(kStageScan, st);
            B200_CUDA_CHECK(launch_exact(a, static_cast<int>(m), st));
            timer_.end(st);
            stats_.kernel_launches += 2;
            idle = false;
            continue;
        }
        // probe splits: enough CTAs to fill the machine, bounded so that the refine kernel's
        // candidate set (S * k') stays within shared memory
        int S = static_cast<int>((16LL * num_sms_ + m - 1) / m);
        const int scan_warps = fast_scan_threads(M_ / 16) / 32;
        S = std::max(1, std::min(S, (nprobe + scan_warps - 1) / scan_warps));
        S = std::max(1, std::min(S, 4096 / kprime));
        // large batches of 16-byte codes: persistent CTAs, four queries per SM at a time
        const bool persist = M_ == 16 && kpt <= kPsMaxKpt && nprobe <= kPsMaxProbe && m >= 8LL * num_sms_ && !no_persist_;
        if (persist) S = 1;
        a.S = S;
        a.kprime = kprime;
        a.fd = static_cast<float*>(w_fd_.ensure(static_cast<size_t>(m) * S * kprime * 4));
        a.fp = static_cast<uint32_t*>(w_fp_.ensure(static_cast<size_t>(m) * S * kprime * 4));
        a.fth = static_cast<float*>(w_fth_.ensure(static_cast<size_t>(m) * S * 4));
        a.flag = static_cast<uint8_t*>(w_flag_.ensure(static_cast<size_t>(m)));
        // error bound of the filter arithmetic relative to the canonical value:
        //   raw      : re-ordering a sum of M non-negative fp32 terms -> (2M + 8) ulp of the sum
        //   residual : every rounding acts on a partial sum bounded by
        //              B = |coarse| + |t2|max + 2 |q| cbnorm + |result|, about 2M + 2 dsub + 16 of them
        const float ulp = 5.9604645e-08f;
        a.err_rel = by_residual_ ? (2.f * M_ + 2.f * dsub_ + 16.f) * ulp : (2.f * M_ + 8.f) * ulp;
        a.cb_bound = cb_norm_bound_;
        const float cmax = coarse_->raw_view().max_norm;
        a.t2_bound = cb_norm_bound_ * cb_norm_bound_ + 2.f * cmax * cb_norm_bound_;
        // very large batches of residual codes: every probed list is decoded once and multiplied with
        // all of its queries on the tensor cores (ivfpq_tc_scan.cu)
        const bool tc = persist && tc_scan_ && tc_cb_ok_ && by_residual_ && d_ == kTcDim && M_ == kTcM && kpt == 1 &&
                        nprobe >= 16 && m * nprobe < (1LL << 30);
        unsigned int* tc_err = nullptr;
        timer_.begin(kStageScan, st);
        if (tc) {
            const int64_t npairs = m * nprobe;
            int32_t* keys = static_cast<int32_t*>(w_tc_keys_.ensure(static_cast<size_t>(npairs) * 4));
            int32_t* vals = static_cast<int32_t*>(w_tc_vals_.ensure(static_cast<size_t>(npairs) * 4));
            int32_t* keys2 = static_cast<int32_t*>(w_tc_keys2_.ensure(static_cast<size_t>(npairs) * 4));
            int32_t* vals2 = static_cast<int32_t*>(w_tc_vals2_.ensure(static_cast<size_t>(npairs) * 4));
            int32_t* first = static_cast<int32_t*>(w_tc_first_.ensure(static_cast<size_t>(nlist_) * 4));
            int32_t* last = static_cast<int32_t*>(w_tc_last_.ensure(static_cast<size_t>(nlist_) * 4));
            B200_CUDA_CHECK(launch_tc_keys(cI, npairs, nlist_, keys, vals, st));
            int end_bit = 1;
            while ((1 << end_bit) <= nlist_) ++end_bit;
            size_t sort_bytes = 0;
            B200_CUDA_CHECK(cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, keys, keys2, vals, vals2,
                                                            static_cast<int>(npairs), 0, end_bit, st));
            void* sort_tmp = w_tc_sort_.ensure(sort_bytes);
            B200_CUDA_CHECK(cub::DeviceRadixSort::SortPairs(sort_tmp, sort_bytes, keys, keys2, vals, vals2,
                                                            static_cast<int>(npairs), 0, end_bit, st));
            B200_CUDA_CHECK(launch_tc_bounds(keys2, npairs, nlist_, first, last, st));
            // lists with the most probing queries are handed out first, so that no long list is
            // left for the end of the launch
            int32_t* okeys = static_cast<int32_t*>(w_tc_okeys_.ensure(static_cast<size_t>(nlist_) * 16));
            int32_t* ovals = okeys + nlist_;
            int32_t* okeys2 = ovals + nlist_;
            int32_t* order = okeys2 + nlist_;
            B200_CUDA_CHECK(launch_tc_order_keys(first, last, nlist_, okeys, ovals, st));
            size_t osort_bytes = 0;
            B200_CUDA_CHECK(cub::DeviceRadixSort::SortPairs(nullptr, osort_bytes, okeys, okeys2, ovals, order, nlist_, 0, 31, st));
            void* osort_tmp = w_tc_osort_.ensure(osort_bytes);
            B200_CUDA_CHECK(cub::DeviceRadixSort::SortPairs(osort_tmp, osort_bytes, okeys, okeys2, ovals, order, nlist_, 0, 31, st));
            float* tau = static_cast<float*>(w_tc_tau_.ensure(static_cast<size_t>(m) * 4));
            TcScanArgs t{};
            t.cb16 = cb16_.as<uint16_t>();
            t.cbnorm = cbnorm_.as<float>();
            t.xq = xp;
            t.centroids = coarse_->rows_f32();
            t.cD = cD;
            t.nprobe = nprobe;
            t.nlist = nlist_;
            t.nq = m;
            t.sorted_pair = vals2;
            t.first = first;
            t.last = last;
            t.order = order;
            t.offsets = offsets_.as<int64_t>();
            t.lens = lens_.as<int64_t>();
            t.codes = codes_.as<uint8_t>();
            t.tau = tau;
            t.cap = 256;
            t.cb_bound = a.cb_bound;
            t.cand_d = static_cast<float*>(w_tc_cd_.ensure(static_cast<size_t>(m) * t.cap * 4));
            t.cand_p = static_cast<uint32_t*>(w_tc_cp_.ensure(static_cast<size_t>(m) * t.cap * 4));
            t.cand_n = static_cast<unsigned int*>(w_tc_cn_.ensure(static_cast<size_t>(m) * 4));
            t.stage_cap = kTcStageCap;
            t.stage = static_cast<uint4*>(w_tc_stage_.ensure(static_cast<size_t>(num_sms_) * kTcStageCap * 16));
            t.stage_n = static_cast<unsigned int*>(w_tc_stage_n_.ensure(static_cast<size_t>(num_sms_) * 4));
            t.work = w_work_.as<unsigned int>();
            t.scanned = a.scanned;
            if (!w_tc_err_.get()) {
                w_tc_err_.ensure(4);
                B200_CUDA_CHECK(cudaMemsetAsync(w_tc_err_.get(), 0, 4, st));
            }
            t.err = tc_err = w_tc_err_.as<unsigned int>();
#ifdef B200IDX_DEV_PROF
            const char* pe = std::getenv("B200IDX_PROF");
            const bool tc_prof = pe && std::strcmp(pe, "1") == 0;
#else
            const bool tc_prof = false;
#endif
            if (tc_prof) {
                w_tc_prof_.ensure(64 + static_cast<size_t>(m) * 4);
                B200_CUDA_CHECK(cudaMemsetAsync(w_tc_prof_.get(), 0, 64, st));
                t.prof = w_tc_prof_.as<unsigned long long>();
            }
            // threshold: one warp per query over the codes of its nearest list
            B200_CUDA_CHECK(launch_tc_head_tau(t, cI, a.err_rel, a.t2_bound, tau, st));
            B200_CUDA_CHECK(launch_tc_scan(t, num_sms_, st));
            B200_CUDA_CHECK(launch_tc_select(t, a.fd, a.fp, a.fth, st));
            if (tc_prof) {   // development aid: phase cycles of thread 0 (sum over CTAs), candidates per query
                unsigned long long hp[8];
                std::vector<unsigned int> cn(static_cast<size_t>(m));
                B200_CUDA_CHECK(cudaMemcpyAsync(hp, t.prof, 64, cudaMemcpyDeviceToHost, st));
                B200_CUDA_CHECK(cudaMemcpyAsync(cn.data(), t.cand_n, cn.size() * 4, cudaMemcpyDeviceToHost, st));
                B200_CUDA_CHECK(cudaStreamSynchronize(st));
                unsigned long long tot = 0, mx = 0;
                for (unsigned int c : cn) { tot += c; mx = std::max<unsigned long long>(mx, c); }
                std::fprintf(stderr, "[tc scan] per-CTA kcycles: ctx_wait %.0f decode %.0f barrier %.0f issue %.0f mma_wait %.0f "
                             "epilogue %.0f release %.0f; tiles/CTA %.0f; candidates/query avg %.1f max %llu\n",
                             hp[0] / 1e3 / num_sms_, hp[1] / 1e3 / num_sms_, hp[2] / 1e3 / num_sms_, hp[3] / 1e3 / num_sms_,
                             hp[4] / 1e3 / num_sms_, hp[5] / 1e3 / num_sms_, hp[6] / 1e3 / num_sms_,
                             static_cast<double>(hp[7]) / num_sms_, static_cast<double>(tot) / m, mx);
            }
            a.tc_rel = kTcErrRel;
            a.tc_abs = kTcErrAbs;
            stats_.kernel_launches += 8;
        } else if (persist) {
            a.work = w_work_.as<unsigned int>();
#ifdef B200IDX_DEV_PROF
            a.prof = static_cast<unsigned long long*>(w_tc_prof_.ensure(128));
            B200_CUDA_CHECK(cudaMemsetAsync(a.prof, 0, 128, st));
#endif
            B200_CUDA_CHECK(launch_persist(a, kpt, num_sms_, st));
#ifdef B200IDX_DEV_PROF
            {
                unsigned long long hp[16];
                B200_CUDA_CHECK(cudaMemcpyAsync(hp, a.prof, 128, cudaMemcpyDeviceToHost, st));
                B200_CUDA_CHECK(cudaStreamSynchronize(st));
                const double nq_s = hp[9] ? static_cast<double>(hp[9]) : 1.0;
                std::fprintf(stderr, "[persist scan] cycles per query of a slot -- warp 1: build %.0f wait %.0f scan %.0f wait %.0f | "
                             "warp 0: build %.0f wait %.0f scan %.0f wait %.0f merge %.0f\n", hp[0] / nq_s, hp[1] / nq_s,
                             hp[2] / nq_s, hp[3] / nq_s, hp[4] / nq_s, hp[5] / nq_s, hp[6] / nq_s, hp[7] / nq_s, hp[8] / nq_s);
            }
#endif
        } else {
            B200_CUDA_CHECK(launch_fast(a, kpt, st));
        }
        timer_.end(st);
        timer_.begin(kStageMerge, st);
        const int P = pow2_ceil_int(std::max(S * kprime, 32));
        const size_t rsmem = static_cast<size_t>(P) * 12;
        if (S * kprime == 32 && k <= 32 && nprobe <= kRefMaxProbe) {
            ivfpq_refine_warp_kernel<<<blocks_for(m, kRefWarpsPerBlock), kRefWarpsPerBlock * 32, 0, st>>>(a);
        } else {
            B200_CUDA_CHECK(set_smem(ivfpq_refine_kernel, rsmem));
            ivfpq_refine_kernel<<<static_cast<unsigned>(m), kScanThreads, rsmem, st>>>(a, P);
        }
        B200_CUDA_CHECK(cudaGetLastError());
        timer_.end(st);
        stats_.kernel_launches += 3;
        // flags of the page and, behind them, the counter of visited codes: one copy-back and one
        // synchronisation per page
        const size_t cnt_off = (static_cast<size_t>(m) + 7) & ~size_t(7);
        uint8_t* hf = static_cast<uint8_t*>(h_flag_.ensure(cnt_off + 8));
        B200_CUDA_CHECK(cudaMemcpyAsync(hf, a.flag, static_cast<size_t>(m), cudaMemcpyDeviceToHost, st));
        B200_CUDA_CHECK(cudaMemcpyAsync(hf + cnt_off, w_tmp_.get(), 8, cudaMemcpyDeviceToHost, st));
        scanned_src = reinterpret_cast<const unsigned long long*>(hf + cnt_off);
        idle = false;
        unsigned int tc_err_host = 0;
        if (tc_err) B200_CUDA_CHECK(cudaMemcpyAsync(&tc_err_host, tc_err, 4, cudaMemcpyDeviceToHost, st));
        B200_CUDA_CHECK(cudaStreamSynchronize(st));
        idle = true;
        scanned = *scanned_src;
        if (tc_err_host) cudaMemsetAsync(tc_err, 0, 4, st);
        if (tc_err_host & 2u)                       // a staging area overflowed: candidates were lost,
            std::memset(hf, 1, static_cast<size_t>(m));   // every query of the page takes the exact path
        if (tc_err_host & 1u) {
            throw std::runtime_error("IVFPQ tensor-core scan reported error word " + std::to_string(tc_err_host) +
                                     " (bounded wait ran out)");
        }
        std::vector<int32_t> bad;
        for (int64_t i = 0; i < m; ++i)
            if (hf[i]) bad.push_back(static_cast<int32_t>(i));
        if (!bad.empty() && k <= kCollectCap && !(tc_err_host & 2u)) {
            // second filter pass with a fixed threshold for the flagged queries (ties at the k' boundary)
            stats_.second_pass_queries += bad.size();
            int32_t* ql = static_cast<int32_t*>(w_qlist_.ensure(bad.size() * 4));
            B200_CUDA_CHECK(cudaMemcpyAsync(ql, bad.data(), bad.size() * 4, cudaMemcpyHostToDevice, st));
            a.qlist = ql;
            uint32_t* cpos = static_cast<uint32_t*>(w_cpos_.ensure(bad.size() * kCollectCap * 4));
            uint32_t* ccount = static_cast<uint32_t*>(w_ccount_.ensure(bad.size() * 4));
            timer_.begin(kStageScan, st);
            B200_CUDA_CHECK(launch_collect(a, static_cast<int>(bad.size()), cpos, ccount, st));
            timer_.end(st);
            B200_CUDA_CHECK(cudaMemcpyAsync(hf, a.flag, static_cast<size_t>(m), cudaMemcpyDeviceToHost, st));
            B200_CUDA_CHECK(cudaStreamSynchronize(st));
            stats_.kernel_launches += 2;
            std::vector<int32_t> still;
            for (int32_t i : bad)
                if (hf[i]) still.push_back(i);
            bad.swap(still);
        }
        if (!bad.empty()) {
            stats_.fallback_queries += bad.size();
            int32_t* ql = static_cast<int32_t*>(w_qlist_.ensure(bad.size() * 4));
            B200_CUDA_CHECK(cudaMemcpyAsync(ql, bad.data(), bad.size() * 4, cudaMemcpyHostToDevice, st));
            a.qlist = ql;
            B200_CUDA_CHECK(launch_exact(a, static_cast<int>(bad.size()), st));
            B200_CUDA_CHECK(cudaStreamSynchronize(st));
            stats_.kernel_launches += 1;
        }
    }
    if (!idle) {   // (the exact-only path queues its kernels without reading anything back)
        B200_CUDA_CHECK(cudaMemcpyAsync(&scanned, w_tmp_.get(), 8, cudaMemcpyDeviceToHost, st));
        B200_CUDA_CHECK(cudaStreamSynchronize(st));
    }
    timer_.collect(stats_);
    stats_.scan_codes = scanned;
    stats_.kernel_launches += coarse_->stats().kernel_launches;
    stats_.gemm_launches += coarse_->stats().gemm_launches;
    coarse_->stats().kernel_launches = 0;
    coarse_->stats().gemm_launches = 0;
}

void IvfpqIndex::search_host(int64_t nq, const float* xq, int k, float* D, int64_t* I) {
    if (nq <= 0) return;
    DeviceGuard g(device_);
    cudaStream_t st = stream();
    float* dq = static_cast<float*>(w_q_.ensure(static_cast<size_t>(nq) * d_ * 4));
    float* dD = static_cast<float*>(w_D_.ensure(static_cast<size_t>(nq) * k * 4));
    int64_t* dI = static_cast<int64_t*>(w_I_.ensure(static_cast<size_t>(nq) * k * 8));
    B200_CUDA_CHECK(cudaMemcpyAsync(dq, xq, static_cast<size_t>(nq) * d_ * 4, cudaMemcpyHostToDevice, st));
    search_device(nq, dq, k, dD, dI);
    B200_CUDA_CHECK(cudaMemcpyAsync(D, dD, static_cast<size_t>(nq) * k * 4, cudaMemcpyDeviceToHost, st));
    B200_CUDA_CHECK(cudaMemcpyAsync(I, dI, static_cast<size_t>(nq) * k * 8, cudaMemcpyDeviceToHost, st));
    B200_CUDA_CHECK(cudaStreamSynchronize(st));
}

}  // namespace b200
