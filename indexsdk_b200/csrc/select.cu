#include "select.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "cos16.cuh"

#include "common.cuh"
#include "dist_gemm.cuh"

namespace b200 {
namespace {

constexpr int kSelThreads = 256;
constexpr int kSmallSet = 512;   // candidate sets up to this size are sorted in shared memory

// Inclusive scan of a 256-bin histogram held in shared memory; returns through `bucket`/`below`
// the bin that contains rank r (1-based) and the number of elements in lower bins.
__device__ __forceinline__ void find_bucket(uint32_t* hist, uint32_t* scan, uint32_t r, uint32_t* bucket,
                                            uint32_t* below) {
    // 256 threads, one bin each: shuffle scan inside the warp, the eight warp totals through `scan`
    const int t = threadIdx.x, lane = t & 31, w = t >> 5;
    const uint32_t v = hist[t];
    uint32_t incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const uint32_t u = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += u;
    }
    if (lane == 31) scan[w] = incl;
    __syncthreads();
    for (int i = 0; i < w; ++i) incl += scan[i];
    const uint32_t excl = incl - v;
    if (incl >= r && excl < r) {
        *bucket = t;
        *below = excl;
    }
    __syncthreads();
}

// k-th smallest (rank r, 1-based, r <= n) of n keys of KeyT read from global memory.
template <typename KeyT>
__device__ KeyT block_radix_kth(const KeyT* in, uint32_t n, uint32_t r, uint32_t* hist, uint32_t* scan,
                                uint32_t* sh_bucket, uint32_t* sh_below) {
    KeyT prefix = 0, mask = 0;
    for (int shift = static_cast<int>(sizeof(KeyT)) * 8 - 8; shift >= 0; shift -= 8) {
        hist[threadIdx.x] = 0;
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < n; i += kSelThreads) {
            const KeyT v = in[i];
            if ((v & mask) == prefix) atomicAdd(&hist[static_cast<uint32_t>(v >> shift) & 255u], 1u);
        }
        __syncthreads();
        find_bucket(hist, scan, r, sh_bucket, sh_below);
        prefix |= static_cast<KeyT>(*sh_bucket) << shift;
        mask |= static_cast<KeyT>(255) << shift;
        r -= *sh_below;
        __syncthreads();
    }
    return prefix;
}

__global__ void __launch_bounds__(kSelThreads)
kth_threshold_kernel(const uint32_t* mins, int stride, int n, int k, const float* eps, uint32_t tau_all,
                     uint32_t* tau) {
    __shared__ uint32_t hist[256], scan[256], sh_bucket, sh_below;
    const int q = blockIdx.x;
    if (n < k) {
        if (threadIdx.x == 0) tau[q] = tau_all;
        return;
    }
    uint32_t kth = block_radix_kth<uint32_t>(mins + static_cast<int64_t>(q) * stride, n, k, hist, scan, &sh_bucket,
                                             &sh_below);
    if (threadIdx.x == 0) {
        if (eps) {
            float f = ord_to_float(kth);
            f = f + 2.f * eps[q];
            f = f + fabsf(f) * 9.5367431640625e-07f;  // one part in 2^20 against the rounding of the adds
            kth = (f != f) ? tau_all : float_to_ord(f);
            if (kth > tau_all) kth = tau_all;
        }
        tau[q] = kth;
    }
}

// Drops candidates that cannot reach the exact top-k before the (costly) exact refinement.  The
// keys in the list are approximate, |approx - exact| <= eps for every candidate.  With A_k the k-th
// smallest approximate key, k candidates have exact keys <= A_k + eps, so the exact k-th key is
// <= A_k + eps and every member of the exact top-k has an approximate key <= A_k + 2 eps; all
// others are overwritten with the "invalid" marker.  A constant offset common to a row's keys
// cancels out of this argument.
constexpr int kPruneKeys = 4096;    // keys staged in shared memory for the rank search
constexpr int kPruneKeep = 2048;    // survivors staged for the in-place compaction

// Tightens a threshold part-way through the full pass: the candidates found so far (in the tiles
// already visited) contain k keys <= their k-th smallest key A_k, so A_k bounds the final k-th key
// from above and the remaining tiles need only admit keys <= min(tau, A_k (+ 2 eps where keys are
// approximate)).  Rows whose list overflowed or holds fewer than k candidates keep their threshold.
__global__ void __launch_bounds__(kSelThreads)
tighten_tau_kernel(const uint64_t* cand, const uint32_t* counts, uint32_t cap, int k, const float* eps,
                   uint32_t* tau) {
    __shared__ uint32_t hist[256], scan[256], sh_bucket, sh_below;
    __shared__ uint32_t keys[kPruneKeys];
    const int q = blockIdx.x;
    const uint64_t* row = cand + static_cast<int64_t>(q) * cap;
    const uint32_t n = counts[q];
    if (n > cap || n > static_cast<uint32_t>(kPruneKeys) || n < static_cast<uint32_t>(k)) return;
    for (uint32_t i = threadIdx.x; i < n; i += kSelThreads) keys[i] = static_cast<uint32_t>(row[i] >> 32);
    __syncthreads();
    uint32_t kth = block_radix_kth<uint32_t>(keys, n, static_cast<uint32_t>(k), hist, scan, &sh_bucket, &sh_below);
    if (kth == 0xFFFFFFFFu) return;   // fewer than k real candidates (the rest are unused slots)
    if (threadIdx.x == 0) {
        if (eps) {
            float f = ord_to_float(kth);
            f = f + 2.f * eps[q] + eps[q] * 0.125f;
            f = f + fabsf(f) * 9.5367431640625e-07f;
            if (f != f) return;
            kth = float_to_ord(f);
        }
        if (kth < tau[q]) tau[q] = kth;
    }
}

__global__ void __launch_bounds__(kSelThreads)
prune_candidates_kernel(uint64_t* cand, uint32_t* counts, uint32_t cap, int k, const float* eps) {
    __shared__ uint32_t hist[256], scan[256], sh_bucket, sh_below, sh_fill;
    __shared__ uint32_t keys[kPruneKeys];
    __shared__ uint64_t keep[kPruneKeep];
    const int q = blockIdx.x;
    uint64_t* row = cand + static_cast<int64_t>(q) * cap;
    const uint32_t n = counts[q];
    if (n > cap) return;   // overflowed row: left as it is for the selection kernel to flag
    if (n <= static_cast<uint32_t>(k)) return;
    uint32_t kth_ord;
    if (n <= static_cast<uint32_t>(kPruneKeys)) {
        for (uint32_t i = threadIdx.x; i < n; i += kSelThreads) keys[i] = static_cast<uint32_t>(row[i] >> 32);
        __syncthreads();
        kth_ord = block_radix_kth<uint32_t>(keys, n, static_cast<uint32_t>(k), hist, scan, &sh_bucket, &sh_below);
    } else {
        kth_ord = static_cast<uint32_t>(
            block_radix_kth<uint64_t>(row, n, static_cast<uint32_t>(k), hist, scan, &sh_bucket, &sh_below) >> 32);
    }
    if (kth_ord == 0xFFFFFFFFu) return;   // fewer than k real candidates
    float lim = ord_to_float(kth_ord);
    lim = lim + 2.f * eps[q];
    lim = lim + fabsf(lim) * 9.5367431640625e-07f + eps[q] * 0.125f;   // slack for the adds and the accumulation
    if (lim != lim) return;
    const uint32_t lim_ord = float_to_ord(lim);
    if (threadIdx.x == 0) sh_fill = 0;
    __syncthreads();
    // survivors go to shared memory first: the row is compacted in place
    for (uint32_t i = threadIdx.x; i < n; i += kSelThreads) {
        const uint64_t v = row[i];
        if (v != kCandInvalid && static_cast<uint32_t>(v >> 32) <= lim_ord) {
            const uint32_t slot = atomicAdd(&sh_fill, 1u);
            if (slot < static_cast<uint32_t>(kPruneKeep)) keep[slot] = v;
        }
    }
    __syncthreads();
    const uint32_t m = sh_fill;
    if (m <= static_cast<uint32_t>(kPruneKeep)) {
        for (uint32_t i = threadIdx.x; i < m; i += kSelThreads) row[i] = keep[i];
        if (threadIdx.x == 0) counts[q] = m;
    } else {
        // too many to stage: invalidate the losers where they are
        for (uint32_t i = threadIdx.x; i < n; i += kSelThreads) {
            const uint64_t v = row[i];
            if (v != kCandInvalid && static_cast<uint32_t>(v >> 32) > lim_ord) row[i] = kCandInvalid;
        }
    }
}

// The same threshold for short rows (n <= 32 * NPL), one WARP per query: the minima sit in
// registers, NPL per lane, and the k-th smallest is found bit by bit -- per bit every lane counts
// its values that agree with the bits fixed so far and have a 0 there, one warp reduction adds the
// counts.  About a third of the instructions of the block-wide byte-radix version at n = 512.
template <int NPL>
__global__ void __launch_bounds__(128)
kth_threshold_warp_kernel(const uint32_t* mins, int stride, int n, int nq, int k, const float* eps, uint32_t tau_all,
                          uint32_t* tau) {
    const int lane = threadIdx.x & 31;
    const int q = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (q >= nq) return;
    if (n < k) {
        if (lane == 0) tau[q] = tau_all;
        return;
    }
    uint32_t v[NPL];
    const uint32_t* row = mins + static_cast<int64_t>(q) * stride;
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
        const int i = j * 32 + lane;
        v[j] = i < n ? row[i] : 0xFFFFFFFFu;
    }
    uint32_t prefix = 0, mask = 0, r = static_cast<uint32_t>(k);
    for (int bit = 31; bit >= 0; --bit) {
        const uint32_t b = 1u << bit;
        uint32_t c = 0;
#pragma unroll
        for (int j = 0; j < NPL; ++j) c += ((v[j] & (mask | b)) == prefix) ? 1u : 0u;   // agrees so far, bit is 0
        c = __reduce_add_sync(0xffffffffu, c);
        if (r > c) {   // the k-th smallest has a 1 at this bit
            prefix |= b;
            r -= c;
        }
        mask |= b;
    }
    if (lane == 0) {
        uint32_t kth = prefix;
        if (eps) {
            float f = ord_to_float(kth);
            f = f + 2.f * eps[q];
            f = f + fabsf(f) * 9.5367431640625e-07f;  // one part in 2^20 against the rounding of the adds
            kth = (f != f) ? tau_all : float_to_ord(f);
            if (kth > tau_all) kth = tau_all;
        }
        tau[q] = kth;
    }
}

__device__ __forceinline__ void bitonic_sort_u64(uint64_t* s, int P) {
    for (int size = 2; size <= P; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = threadIdx.x; i < P / 2; i += blockDim.x) {
                const int lo = 2 * i - (i & (stride - 1));
                const int hi = lo + stride;
                const bool up = (lo & size) == 0;
                const uint64_t a = s[lo], b = s[hi];
                if ((a > b) == up) {
                    s[lo] = b;
                    s[hi] = a;
                }
            }
            __syncthreads();
        }
    }
}

__global__ void __launch_bounds__(kSelThreads)
select_topk_kernel(const uint64_t* cand, const uint32_t* counts, uint32_t n_fixed, uint32_t cap, int k, int P,
                   uint64_t* out, uint8_t* overflow) {
    extern __shared__ uint64_t sorted[];  // P entries
    __shared__ uint32_t hist[256], scan[256], sh_bucket, sh_below, sh_fill;
    const int q = blockIdx.x;
    const uint64_t* row = cand + static_cast<int64_t>(q) * cap;
    uint32_t n = counts ? counts[q] : n_fixed;
    if (overflow && threadIdx.x == 0) overflow[q] = n > cap ? 1 : 0;
    if (n > cap) n = cap;
    uint64_t* orow_fast = out + static_cast<int64_t>(q) * k;
    if (n <= static_cast<uint32_t>(kSmallSet)) {
        // Small candidate set (the common case after a tight threshold): the real entries (unused
        // reserved slots are dropped) are staged in shared memory and every one is placed by its
        // rank, counted against all others.  Candidates are distinct (positions are unique), so
        // the ranks are a permutation.
        __shared__ uint64_t small[kSmallSet];
        if (threadIdx.x == 0) sh_fill = 0;
        for (int i = threadIdx.x; i < k; i += kSelThreads) orow_fast[i] = kCandInvalid;
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < n; i += kSelThreads) {
            const uint64_t v = row[i];
            if (v != kCandInvalid) small[atomicAdd(&sh_fill, 1u)] = v;
        }
        __syncthreads();
        const uint32_t m = sh_fill;
        for (uint32_t i = threadIdx.x; i < m; i += kSelThreads) {
            const uint64_t v = small[i];
            uint32_t rank = 0;
#pragma unroll 8
            for (uint32_t j = 0; j < m; ++j) rank += small[j] < v ? 1u : 0u;
            if (rank < static_cast<uint32_t>(k)) orow_fast[rank] = v;
        }
        return;
    }
    for (int i = threadIdx.x; i < P; i += kSelThreads) sorted[i] = kCandInvalid;
    if (threadIdx.x == 0) sh_fill = 0;
    __syncthreads();
    uint64_t kth = kCandInvalid;
    if (n > static_cast<uint32_t>(k))
        kth = block_radix_kth<uint64_t>(row, n, static_cast<uint32_t>(k), hist, scan, &sh_bucket, &sh_below);
    for (uint32_t i = threadIdx.x; i < n; i += kSelThreads) {
        const uint64_t v = row[i];
        if (v <= kth && v != kCandInvalid) {
            const uint32_t slot = atomicAdd(&sh_fill, 1u);
            if (slot < static_cast<uint32_t>(P)) sorted[slot] = v;
        }
    }
    __syncthreads();
    bitonic_sort_u64(sorted, P);
    uint64_t* orow = out + static_cast<int64_t>(q) * k;
    for (int i = threadIdx.x; i < k; i += kSelThreads) orow[i] = sorted[i];
}

// Canonical fp32 distances of the candidates (sequential fmaf over the dimensions, the arithmetic
// of the CPU oracle).  The chain of one candidate cannot be split over lanes, so a lane owns a
// candidate -- but the rows are fetched co-operatively: a warp reads the rows of its 32 candidates
// kRefChunk floats at a time, each row as one contiguous 128-byte piece spread over consecutive
// lanes (four cache lines per load instruction instead of 32), parks them in shared memory and
// every lane then walks its own row there.  Rows are padded by 4 floats: 8 consecutive lanes
// reading one float4 each fall into 8 different 16-byte bank groups.
constexpr int kRefChunk = 32;     // small, so that many warps fit an SM: the kernel lives on memory-level parallelism
constexpr int kRefPitch = kRefChunk + 4;
constexpr uint32_t kRefWindow = 512;   // candidate slots compacted at a time
__global__ void __launch_bounds__(128)
refine_f32_kernel(uint64_t* cand, const uint32_t* counts, uint32_t n_fixed, uint32_t cap, int d, int metric,
                  const float* xq, const float* xb, int q_first, int q_mod) {
    extern __shared__ __align__(16) float ref_sm[];
    float* qs = ref_sm;                                              // [d]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* rows = ref_sm + d + warp * (32 * kRefPitch);              // [32][kRefPitch] per warp
    const int q = blockIdx.y;
    // candidate row q_first + q holds the candidates of query (q_first + q) % q_mod (several indexes
    // searched with the same queries) or of query q_first + q (q_mod = 0)
    const int qrow = q_mod > 0 ? (q_first + q) % q_mod : q_first + q;
    uint32_t n = counts ? counts[q] : n_fixed;
    if (n > cap) n = cap;
    if (blockIdx.x * kRefWindow >= n) return;
    for (int i = threadIdx.x; i < d / 4; i += 128)
        reinterpret_cast<float4*>(qs)[i] = __ldg(reinterpret_cast<const float4*>(xq + static_cast<int64_t>(qrow) * d) + i);
    __syncthreads();
    uint64_t* row = cand + static_cast<int64_t>(q) * cap;
    // The list is sparse (reserved but unused slots, see the GEMM's block reservation): a window of
    // slots is compacted into shared memory first, so that every warp pass works on 32 live
    // candidates.  The result goes back to the candidate's own slot: the order of compaction is free.
    __shared__ uint32_t s_slot[kRefWindow];
    __shared__ uint32_t s_pos[kRefWindow];
    __shared__ uint32_t s_cnt;
    for (uint32_t win0 = blockIdx.x * kRefWindow; win0 < n; win0 += gridDim.x * kRefWindow) {
    if (threadIdx.x == 0) s_cnt = 0u;
    __syncthreads();
    const uint32_t win1 = win0 + kRefWindow < n ? win0 + kRefWindow : n;
    for (uint32_t i = win0 + threadIdx.x; i < win1; i += 128) {
        const uint64_t c = row[i];
        if (c != kCandInvalid) {
            const uint32_t j = atomicAdd(&s_cnt, 1u);
            s_slot[j] = i;
            s_pos[j] = static_cast<uint32_t>(c);
        }
    }
    __syncthreads();
    const uint32_t cnt = s_cnt;
    for (uint32_t i0 = warp * 32; i0 < cnt; i0 += 128) {
        const bool live = i0 + lane < cnt;
        const uint32_t i = live ? s_slot[i0 + lane] : 0u;
        const uint32_t pos = live ? s_pos[i0 + lane] : 0u;
        const uint32_t live_mask = __ballot_sync(0xffffffffu, live);
        float acc = 0.f;
        if (d % kRefChunk == 0) {
            // Whole chunks only: a lane stages the same 8 rows in every chunk, so their addresses are
            // formed once per pass, and the loads of the next chunk are in flight while the current
            // one is accumulated from shared memory.
            const int j = lane & 7;
            const float4* src[8];
            uint32_t okm = 0;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int r = it * 4 + (lane >> 3);
                const uint32_t pr = __shfl_sync(0xffffffffu, pos, r);
                src[it] = reinterpret_cast<const float4*>(xb + static_cast<int64_t>(pr) * d) + j;
                okm |= ((live_mask >> r) & 1u) << it;   // rows of unused slots are neither fetched nor read
            }
            float4* dst = reinterpret_cast<float4*>(rows + (lane >> 3) * kRefPitch + 4 * j);
            const float4* mine = reinterpret_cast<const float4*>(rows + lane * kRefPitch);
            float4 v[8];
#pragma unroll
            for (int it = 0; it < 8; ++it)
                if ((okm >> it) & 1u) v[it] = __ldg(src[it]);
            for (int ch0 = 0; ch0 < d; ch0 += kRefChunk) {
#pragma unroll
                for (int it = 0; it < 8; ++it)
                    if ((okm >> it) & 1u) dst[it * kRefPitch] = v[it];   // 4 rows further per step
                __syncwarp();
                if (ch0 + kRefChunk < d) {
#pragma unroll
                    for (int it = 0; it < 8; ++it)
                        if ((okm >> it) & 1u) v[it] = __ldg(src[it] + (ch0 + kRefChunk) / 4);
                }
                const float4* qv = reinterpret_cast<const float4*>(qs + ch0);
                if (live) {
                    if (metric == kMetricL2) {
#pragma unroll
                        for (int jj = 0; jj < kRefChunk / 4; ++jj) {
                            const float4 a = qv[jj], b = mine[jj];
                            float t;
                            t = a.x - b.x; acc = fmaf(t, t, acc);
                            t = a.y - b.y; acc = fmaf(t, t, acc);
                            t = a.z - b.z; acc = fmaf(t, t, acc);
                            t = a.w - b.w; acc = fmaf(t, t, acc);
                        }
                    } else {
#pragma unroll
                        for (int jj = 0; jj < kRefChunk / 4; ++jj) {
                            const float4 a = qv[jj], b = mine[jj];
                            acc = fmaf(a.x, b.x, acc);
                            acc = fmaf(a.y, b.y, acc);
                            acc = fmaf(a.z, b.z, acc);
                            acc = fmaf(a.w, b.w, acc);
                        }
                    }
                }
                __syncwarp();
            }
        } else
        for (int ch0 = 0; ch0 < d; ch0 += kRefChunk) {
            const int w = d - ch0 < kRefChunk ? d - ch0 : kRefChunk;
            const int lpr = w >> 2;                                  // float4 pieces per row
            if (lpr == kRefChunk / 4) {
#pragma unroll
                for (int it = 0; it < 8; ++it) {                     // four of the 32 rows per load instruction
                    const int r = it * 4 + (lane >> 3), j = lane & 7;
                    const uint32_t pr = __shfl_sync(0xffffffffu, pos, r);
                    if ((live_mask >> r) & 1u) {   // rows of unused slots are neither fetched nor read
                        const float4 v = __ldg(reinterpret_cast<const float4*>(xb + static_cast<int64_t>(pr) * d + ch0) + j);
                        *reinterpret_cast<float4*>(rows + r * kRefPitch + 4 * j) = v;
                    }
                }
            } else {
                for (int idx = lane; idx < 32 * lpr; idx += 32) {
                    const int r = idx / lpr, j = idx - r * lpr;
                    const uint32_t pr = __shfl_sync(0xffffffffu, pos, r);
                    const float4 v = __ldg(reinterpret_cast<const float4*>(xb + static_cast<int64_t>(pr) * d + ch0) + j);
                    *reinterpret_cast<float4*>(rows + r * kRefPitch + 4 * j) = v;
                }
            }
            __syncwarp();
            const float4* mine = reinterpret_cast<const float4*>(rows + lane * kRefPitch);
            const float4* qv = reinterpret_cast<const float4*>(qs + ch0);
            if (!live) {
                // nothing to accumulate for an unused slot
            } else if (metric == kMetricL2) {
#pragma unroll 4
                for (int j = 0; j < lpr; ++j) {
                    const float4 a = qv[j], b = mine[j];
                    float t;
                    t = a.x - b.x; acc = fmaf(t, t, acc);
                    t = a.y - b.y; acc = fmaf(t, t, acc);
                    t = a.z - b.z; acc = fmaf(t, t, acc);
                    t = a.w - b.w; acc = fmaf(t, t, acc);
                }
            } else {
#pragma unroll 4
                for (int j = 0; j < lpr; ++j) {
                    const float4 a = qv[j], b = mine[j];
                    acc = fmaf(a.x, b.x, acc);
                    acc = fmaf(a.y, b.y, acc);
                    acc = fmaf(a.z, b.z, acc);
                    acc = fmaf(a.w, b.w, acc);
                }
            }
            __syncwarp();
        }
        if (metric != kMetricL2) acc = -acc;
        if (live) row[i] = pack_cand(float_to_ord(acc), pos);
    }
    __syncthreads();   // the window's lists are reused
    }
}

__global__ void emit_kernel(const EmitArgs e) {
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<int64_t>(e.nq) * e.k) return;
    const int q = static_cast<int>(idx / e.k), j = static_cast<int>(idx % e.k);
    const int orow = e.qmap ? e.qmap[q] : q;
    const int qn = e.q_mod > 0 ? q % e.q_mod : q;   // row of the query norms
    const uint64_t c = e.sel[idx];
    float dist;
    int64_t label;
    if (c == kCandInvalid) {
        dist = 3.402823466e+38f;  // FLT_MAX padding, label -1
        label = -1;
    } else {
        const uint32_t ok = static_cast<uint32_t>(c >> 32), pos = static_cast<uint32_t>(c);
        label = e.labels ? e.labels[pos] : static_cast<int64_t>(pos);
        if (e.mode == 2) {
            int32_t kv = ord_to_int(ok);
            if (e.metric == kMetricL2) dist = static_cast<float>(kv + static_cast<const int32_t*>(e.qnorm)[qn]);
            else if (e.metric == kMetricCos) dist = cos16_value(-kv);
            else dist = static_cast<float>(-kv);
        } else {
            float kv = ord_to_float(ok);
            if (e.metric == kMetricL2) {
                if (e.mode == 0) {
                    kv += static_cast<const float*>(e.qnorm)[qn];
                    kv = kv < 0.f ? 0.f : kv;
                }
                dist = kv;
            } else {
                dist = -kv;
            }
        }
    }
    e.D[static_cast<int64_t>(orow) * e.ldk + j] = dist;
    e.I[static_cast<int64_t>(orow) * e.ldk + j] = label;
}

// One warp per query; heads[] in shared memory.
__global__ void __launch_bounds__(32)
merge_topk_kernel(int nsrc, int64_t nq, int k, int descending, const float* Din, const int64_t* Iin,
                  int64_t src_stride_d, int64_t src_stride_i, float* D, int64_t* I) {
    extern __shared__ int heads[];
    const int64_t q = blockIdx.x;
    const int lane = threadIdx.x;
    for (int s = lane; s < nsrc; s += 32) heads[s] = 0;
    __syncwarp();
    for (int j = 0; j < k; ++j) {
        float bk = 0.f;
        int64_t bl = -1;
        int bs = -1;
        for (int s = lane; s < nsrc; s += 32) {
            const int h = heads[s];
            if (h >= k) continue;
            const int64_t off = q * k + h;
            const int64_t l = Iin[s * src_stride_i + off];
            if (l < 0) {
                heads[s] = k;
                continue;
            }
            const float dv = Din[s * src_stride_d + off];
            const float key = descending ? -dv : dv;
            if (bs < 0 || key < bk || (key == bk && l < bl)) {
                bk = key;
                bl = l;
                bs = s;
            }
        }
        for (int off = 16; off > 0; off >>= 1) {
            const float ok = __shfl_xor_sync(0xffffffffu, bk, off);
            const int64_t ol = __shfl_xor_sync(0xffffffffu, bl, off);
            const int os = __shfl_xor_sync(0xffffffffu, bs, off);
            if (os >= 0 && (bs < 0 || ok < bk || (ok == bk && ol < bl))) {
                bk = ok;
                bl = ol;
                bs = os;
            }
        }
        if (lane == 0) {
            if (bs >= 0) {
                D[q * k + j] = descending ? -bk : bk;
                I[q * k + j] = bl;
                heads[bs] += 1;
            } else {
                D[q * k + j] = 3.402823466e+38f;
                I[q * k + j] = -1;
            }
        }
        __syncwarp();
    }
}

// ---- preparation kernels: one warp per row ----
__device__ __forceinline__ float warp_sum(float v) {
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// Three bf16 terms whose sum reproduces v to 24 significant bits (an infinite v stays in the
// first term).
__device__ __forceinline__ void split3_bf16(float v, __nv_bfloat16* out) {
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    float r = isfinite(v) ? v - __bfloat162float(h) : 0.f;
    const __nv_bfloat16 m = __float2bfloat16_rn(r);
    r -= __bfloat162float(m);
    out[0] = h;
    out[1] = m;
    out[2] = __float2bfloat16_rn(r);
}

// Query operand rows of d + kFoldCols bf16: the query, three ones (they pick up the base row's
// folded norm), three zeros (the threshold terms, written by fold_tau_kernel once the threshold is
// known) and zero padding.
__global__ void prep_queries_f32_kernel(const float* xq, int nq, int d, int metric, float ymax,
                                        __nv_bfloat16* qb, float* qnorm, float* eps) {
    const int q = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (q >= nq) return;
    const int dp = d + kFoldCols;
    const bool packed = packed_operands(kKindBF16, dp);
    float s = 0.f;
    for (int i = lane; i < d; i += 32) {
        const float v = xq[static_cast<int64_t>(q) * d + i];
        s = fmaf(v, v, s);
        qb[operand_elem(packed, q, i, dp, kTileQ)] = __float2bfloat16_rn(v);
    }
    if (lane < kFoldCols) qb[operand_elem(packed, q, d + lane, dp, kTileQ)] = __float2bfloat16_rn(lane < 3 ? 1.f : 0.f);
    s = warp_sum(s);
    if (lane == 0) {
        qnorm[q] = s;
        // Filter slack.  bf16 rounding of both operands perturbs every product by at most
        // 2^-8 (1 + 2^-10) relatively, so |dot~ - dot| <= c |q||y| with the accumulation slack
        // folded into c; the second term covers the fp32 rounding of norms and of the canonical
        // distance itself.
        const float qn = sqrtf(s) * 1.0001f;
        const float c = 0.00390625f * 1.01f + static_cast<float>(d) * 4.76837158203125e-07f;
        const float g = static_cast<float>(d + 4) * 2.384185791015625e-07f;
        float e;
        if (metric == kMetricL2) e = 2.f * c * qn * ymax + g * (qn + ymax) * (qn + ymax);
        else e = c * qn * ymax + g * qn * ymax;
        eps[q] = e;
    }
}

// Writes the threshold terms of the folded query rows: c = tau / 2 (L2) or tau (inner product).
// tau is first raised by a margin for the fp32 accumulation inside the tensor core: d + 16
// additions of terms whose partial sums stay below M = |q||y|max + |y|max^2 / 2 + |tau| perturb a
// key by less than 2^-14.8 M in either pass, and 2^-12 M covers the sample pass, the full pass and
// the threshold's own term together, so no key <= tau is missed.
__global__ void fold_tau_kernel(const uint32_t* tau, const float* qnorm, float ymax, int nq, int d, int metric,
                                __nv_bfloat16* qb) {
    const int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= nq) return;
    const float t = ord_to_float(tau[q]);
    const float m = sqrtf(qnorm[q]) * ymax + 0.5f * ymax * ymax + fabsf(t);
    float c = t + 0.000244140625f * m;
    if (metric == kMetricL2) c *= 0.5f;
    const int dp = d + kFoldCols;
    // columns d + 3 .. d + 5 lie in one 8-column group (d is a multiple of 16), so they are
    // consecutive in the packed layout as well
    split3_bf16(c, qb + operand_elem(packed_operands(kKindBF16, dp), q, d + 3, dp, kTileQ));
}

__global__ void prep_queries_f16_kernel(const __half* xq, int nq, int d, float* qnorm) {
    const int q = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (q >= nq) return;
    float s = 0.f;
    for (int i = lane; i < d; i += 32) {
        const float v = __half2float(xq[static_cast<int64_t>(q) * d + i]);
        s = fmaf(v, v, s);
    }
    s = warp_sum(s);
    if (lane == 0) qnorm[q] = s;
}

__global__ void prep_queries_i8_kernel(const int8_t* xq, int nq, int d, int32_t* qnorm) {
    const int q = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (q >= nq) return;
    int s = 0;
    for (int i = lane; i < d; i += 32) {
        const int v = xq[static_cast<int64_t>(q) * d + i];
        s += v * v;
    }
    s = warp_sum_i(s);
    if (lane == 0) qnorm[q] = s;
}

// Base operand rows of d + kFoldCols bf16: the vector, -|y|^2 / 2 in three terms (zeros for inner
// product), three ones (they pick up the query's threshold terms) and zero padding.
// x, norms: the n rows being added; xb: the whole operand buffer, whose row row0 + r belongs to x's row r.
__global__ void base_prep_f32_kernel(const float* x, int64_t n, int d, int metric, __nv_bfloat16* xb, int64_t row0,
                                     float* norms, float* max_norm_sq) {
    const int64_t r = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (r >= n) return;
    const int dp = d + kFoldCols;
    const bool packed = packed_operands(kKindBF16, dp);
    const int64_t ro = row0 + r;
    float s = 0.f;
    for (int i = lane; i < d; i += 32) {
        const float v = x[r * d + i];
        s = fmaf(v, v, s);
        xb[operand_elem(packed, ro, i, dp, kTileB)] = __float2bfloat16_rn(v);
    }
    s = warp_sum(s);
    if (lane >= 3 && lane < kFoldCols) xb[operand_elem(packed, ro, d + lane, dp, kTileB)] = __float2bfloat16_rn(lane < 6 ? 1.f : 0.f);
    if (lane == 0) {
        split3_bf16(metric == kMetricL2 ? -0.5f * s : 0.f, xb + operand_elem(packed, ro, d, dp, kTileB));
        norms[r] = s;
        atomicMax(reinterpret_cast<unsigned int*>(max_norm_sq), __float_as_uint(s));
    }
}

__global__ void base_prep_f16_kernel(const __half* x, int64_t n, int d, float* norms) {
    const int64_t r = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (r >= n) return;
    float s = 0.f;
    for (int i = lane; i < d; i += 32) {
        const float v = __half2float(x[r * d + i]);
        s = fmaf(v, v, s);
    }
    s = warp_sum(s);
    if (lane == 0) norms[r] = s;
}

__global__ void base_prep_i8_kernel(const int8_t* x, int64_t n, int d, int32_t* norms) {
    const int64_t r = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (r >= n) return;
    int s = 0;
    for (int i = lane; i < d; i += 32) {
        const int v = x[r * d + i];
        s += v * v;
    }
    s = warp_sum_i(s);
    if (lane == 0) norms[r] = s;
}

__global__ void f32_to_f16_kernel(const float* x, int64_t count, __half* out) {
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        out[i] = __float2half_rn(x[i]);
}
__global__ void f16_to_f32_kernel(const __half* x, int64_t count, float* out) {
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        out[i] = __half2float(x[i]);
}

__global__ void fill_u32_kernel(uint32_t* p, int64_t count, uint32_t value) {
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        p[i] = value;
}
__global__ void iota_i64_kernel(int64_t* p, int64_t count, int64_t start) {
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        p[i] = start + i;
}
__global__ void gather_rows_kernel(const uint32_t* src, const int32_t* idx, int n, int row_words, uint32_t* dst) {
    const int r = blockIdx.x;
    if (r >= n) return;
    const uint32_t* s = src + static_cast<int64_t>(idx[r]) * row_words;
    uint32_t* d = dst + static_cast<int64_t>(r) * row_words;
    for (int i = threadIdx.x; i < row_words; i += blockDim.x) d[i] = s[i];
}

inline int next_pow2(int v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

}  // namespace

cudaError_t launch_kth_threshold(const uint32_t* mins, int stride, int n, int nq, int k, const float* eps,
                                 uint32_t tau_all, uint32_t* tau, cudaStream_t stream) {
    if (nq <= 0) return cudaSuccess;
    if (n <= 512)
        kth_threshold_warp_kernel<16><<<(nq + 3) / 4, 128, 0, stream>>>(mins, stride, n, nq, k, eps, tau_all, tau);
    else if (n <= 1024)
        kth_threshold_warp_kernel<32><<<(nq + 3) / 4, 128, 0, stream>>>(mins, stride, n, nq, k, eps, tau_all, tau);
    else
        kth_threshold_kernel<<<nq, kSelThreads, 0, stream>>>(mins, stride, n, k, eps, tau_all, tau);
    return cudaGetLastError();
}

cudaError_t launch_select_topk(const uint64_t* cand, const uint32_t* counts, uint32_t n_fixed, uint32_t cap, int nq,
                               int k, uint64_t* out, uint8_t* overflow, cudaStream_t stream) {
    if (nq <= 0) return cudaSuccess;
    int P = next_pow2(k < 32 ? 32 : k);
    size_t smem = static_cast<size_t>(P) * sizeof(uint64_t);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(select_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem));
        if (e != cudaSuccess) return e;
    }
    select_topk_kernel<<<nq, kSelThreads, smem, stream>>>(cand, counts, n_fixed, cap, k, P, out, overflow);
    return cudaGetLastError();
}

cudaError_t launch_tighten_tau(const uint64_t* cand, const uint32_t* counts, uint32_t cap, int nq, int k,
                               const float* eps, uint32_t* tau, cudaStream_t stream) {
    if (nq <= 0) return cudaSuccess;
    tighten_tau_kernel<<<nq, kSelThreads, 0, stream>>>(cand, counts, cap, k, eps, tau);
    return cudaGetLastError();
}

cudaError_t launch_prune_candidates(uint64_t* cand, uint32_t* counts, uint32_t cap, int nq, int k,
                                    const float* eps, cudaStream_t stream) {
    if (nq <= 0) return cudaSuccess;
    prune_candidates_kernel<<<nq, kSelThreads, 0, stream>>>(cand, counts, cap, k, eps);
    return cudaGetLastError();
}

cudaError_t launch_refine_f32(uint64_t* cand, const uint32_t* counts, uint32_t n_fixed, uint32_t cap, int nq, int d,
                              int metric, const float* xq, const float* xb, cudaStream_t stream, int q_mod) {
    if (nq <= 0) return cudaSuccess;
    uint32_t per_row = counts ? cap : (n_fixed < cap ? n_fixed : cap);
    // Blocks stride over a row's candidates, so a few thousand blocks in total keep the machine
    // busy; one block per 128 candidate SLOTS would mostly launch blocks that find nothing to do.
    int gx = static_cast<int>((per_row + kRefWindow - 1) / kRefWindow);
    const int want = (2048 + nq - 1) / nq;
    if (gx > want) gx = want;
    if (gx > 64) gx = 64;
    if (gx < 1) gx = 1;
    const size_t smem = (static_cast<size_t>(d) + 4 * 32 * kRefPitch) * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(refine_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem));
        if (e != cudaSuccess) return e;
    }
    for (int q0 = 0; q0 < nq; q0 += 65535) {
        const int nqq = nq - q0 < 65535 ? nq - q0 : 65535;
        refine_f32_kernel<<<dim3(gx, nqq), 128, smem, stream>>>(cand + static_cast<int64_t>(q0) * cap,
                                                            counts ? counts + q0 : nullptr, n_fixed, cap, d, metric,
                                                            xq, xb, q0, q_mod);
    }
    return cudaGetLastError();
}

cudaError_t launch_emit(const EmitArgs& e, cudaStream_t stream) {
    const int64_t total = static_cast<int64_t>(e.nq) * e.k;
    if (total <= 0) return cudaSuccess;
    emit_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(e);
    return cudaGetLastError();
}

cudaError_t launch_merge_topk(int nsrc, int64_t nq, int k, int descending, const float* Din, const int64_t* Iin,
                              float* D, int64_t* I, cudaStream_t stream, int64_t src_stride_d, int64_t src_stride_i) {
    if (nq <= 0 || k <= 0) return cudaSuccess;
    if (src_stride_d <= 0) src_stride_d = nq * k;
    if (src_stride_i <= 0) src_stride_i = nq * k;
    merge_topk_kernel<<<static_cast<unsigned>(nq), 32, static_cast<size_t>(nsrc) * sizeof(int), stream>>>(
        nsrc, nq, k, descending, Din, Iin, src_stride_d, src_stride_i, D, I);
    return cudaGetLastError();
}

cudaError_t launch_prep_queries_f32(const float* xq, int nq, int d, int metric, float base_max_norm, void* q_bf16,
                                    float* qnorm, float* eps, cudaStream_t stream) {
    if (nq <= 0) return cudaSuccess;
    prep_queries_f32_kernel<<<(nq + 7) / 8, 256, 0, stream>>>(xq, nq, d, metric, base_max_norm,
                                                              static_cast<__nv_bfloat16*>(q_bf16), qnorm, eps);
    return cudaGetLastError();
}
cudaError_t launch_prep_queries_f16(const void* xq, int nq, int d, float* qnorm, cudaStream_t stream) {
    if (nq <= 0) return cudaSuccess;
    prep_queries_f16_kernel<<<(nq + 7) / 8, 256, 0, stream>>>(static_cast<const __half*>(xq), nq, d, qnorm);
    return cudaGetLastError();
}
cudaError_t launch_prep_queries_i8(const int8_t* xq, int nq, int d, int32_t* qnorm, cudaStream_t stream) {
    if (nq <= 0) return cudaSuccess;
    prep_queries_i8_kernel<<<(nq + 7) / 8, 256, 0, stream>>>(xq, nq, d, qnorm);
    return cudaGetLastError();
}
cudaError_t launch_base_prep_f32(const float* x, int64_t n, int d, int metric, void* x_bf16, int64_t row0,
                                 float* norms, float* max_norm_sq, cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    base_prep_f32_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(
        x, n, d, metric, static_cast<__nv_bfloat16*>(x_bf16), row0, norms, max_norm_sq);
    return cudaGetLastError();
}
cudaError_t launch_fold_tau(const uint32_t* tau, const float* qnorm, float base_max_norm, int nq, int d, int metric,
                            void* q_bf16, cudaStream_t stream) {
    if (nq <= 0) return cudaSuccess;
    fold_tau_kernel<<<(nq + 255) / 256, 256, 0, stream>>>(tau, qnorm, base_max_norm, nq, d, metric,
                                                          static_cast<__nv_bfloat16*>(q_bf16));
    return cudaGetLastError();
}
cudaError_t launch_base_prep_f16(const void* x, int64_t n, int d, float* norms, cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    base_prep_f16_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(static_cast<const __half*>(x), n, d,
                                                                                 norms);
    return cudaGetLastError();
}
cudaError_t launch_base_prep_i8(const int8_t* x, int64_t n, int d, int32_t* norms, cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    base_prep_i8_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(x, n, d, norms);
    return cudaGetLastError();
}
cudaError_t launch_f32_to_f16(const float* x, int64_t count, void* out, cudaStream_t stream) {
    if (count <= 0) return cudaSuccess;
    int grid = static_cast<int>((count + 255) / 256 < 65535 ? (count + 255) / 256 : 65535);
    f32_to_f16_kernel<<<grid, 256, 0, stream>>>(x, count, static_cast<__half*>(out));
    return cudaGetLastError();
}
cudaError_t launch_f16_to_f32(const void* x, int64_t count, float* out, cudaStream_t stream) {
    if (count <= 0) return cudaSuccess;
    int grid = static_cast<int>((count + 255) / 256 < 65535 ? (count + 255) / 256 : 65535);
    f16_to_f32_kernel<<<grid, 256, 0, stream>>>(static_cast<const __half*>(x), count, static_cast<float*>(out));
    return cudaGetLastError();
}

namespace {
// flag |= 1 when x holds a NaN or an infinity
__global__ void check_finite_kernel(const float* x, int64_t count, int* flag) {
    bool bad = false;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        bad |= (__float_as_uint(x[i]) & 0x7f800000u) == 0x7f800000u;
    if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(flag, 1);
}
// flag |= 2 when a value lies outside [0, bound)
__global__ void check_range_i32_kernel(const int32_t* v, int64_t count, int32_t bound, int* flag) {
    bool bad = false;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        bad |= v[i] < 0 || v[i] >= bound;
    if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(flag, 2);
}
}  // namespace
cudaError_t launch_check_finite(const float* x, int64_t count, int* flag, cudaStream_t stream) {
    if (count <= 0) return cudaSuccess;
    int grid = static_cast<int>((count + 255) / 256 < 2048 ? (count + 255) / 256 : 2048);
    check_finite_kernel<<<grid, 256, 0, stream>>>(x, count, flag);
    return cudaGetLastError();
}
cudaError_t launch_check_range_i32(const int32_t* v, int64_t count, int32_t bound, int* flag, cudaStream_t stream) {
    if (count <= 0) return cudaSuccess;
    int grid = static_cast<int>((count + 255) / 256 < 2048 ? (count + 255) / 256 : 2048);
    check_range_i32_kernel<<<grid, 256, 0, stream>>>(v, count, bound, flag);
    return cudaGetLastError();
}

cudaError_t launch_fill_u32(uint32_t* p, int64_t count, uint32_t value, cudaStream_t stream) {
    if (count <= 0) return cudaSuccess;
    int grid = static_cast<int>((count + 255) / 256 < 4096 ? (count + 255) / 256 : 4096);
    fill_u32_kernel<<<grid, 256, 0, stream>>>(p, count, value);
    return cudaGetLastError();
}
cudaError_t launch_iota_i64(int64_t* p, int64_t count, int64_t start, cudaStream_t stream) {
    if (count <= 0) return cudaSuccess;
    int grid = static_cast<int>((count + 255) / 256 < 4096 ? (count + 255) / 256 : 4096);
    iota_i64_kernel<<<grid, 256, 0, stream>>>(p, count, start);
    return cudaGetLastError();
}
cudaError_t launch_gather_rows(const void* src, const int32_t* idx, int n, int row_bytes, void* dst,
                               cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    gather_rows_kernel<<<n, 128, 0, stream>>>(static_cast<const uint32_t*>(src), idx, n, row_bytes / 4,
                                              static_cast<uint32_t*>(dst));
    return cudaGetLastError();
}

}  // namespace b200
