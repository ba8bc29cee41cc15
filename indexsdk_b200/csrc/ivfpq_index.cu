// IVFPQ search on one GPU.
//
// Stage 1  coarse quantizer: FlatIndex (fp32 mode) over the nlist centroids with k = nprobe --
//          the same tcgen05 distance GEMM, filter + fp32 refinement, so probe lists and their
//          distances are the canonical fp32 values (replaces DistanceFlatL2MinsAtFP32 +
//          TopkFlatFp32, FR/ascenddaemon/impl/IndexIVFPQ.cpp:2104-2164).
// Stage 2  lookup tables, one [M][256] fp32 table per query (replaces
//          AscendcIvfpqSubspaceDistance, FR/ops/ascendc/op_kernel/
//          ascendc_ivfpq_subspace_distance.cpp:46-617).
//            raw encoding      : LUT[m][j] = |q_m - cb[m][j]|^2
//            residual encoding : LUT[m][j] = -2 q_m . cb[m][j]; the list-dependent remainder
//              |cb|^2 + 2 c_list . cb is summed over a vector's codes once, at add time, into one
//              float per vector (t2), and |q - c_list|^2 is the coarse distance.  The distance
//              |q - c - r|^2 = |q - c|^2 + (|r|^2 + 2 c.r) - 2 q.r is the same decomposition Faiss
//              uses for its precomputed tables, with the per-list table folded per vector.
// Stage 3  code scan (replaces AscendcIvfpqSearchDistanceL2 + TopkIvfpqL3, FR/ops/ascendc/
//          op_kernel/ascendc_ivfpq_search_distance_topk.h:95-810, FR/ops/cpukernel/impl/
//          topk_ivfpq_l3_cpu_kernel.cpp:36-254): one CTA per (query, probe split); the query's
//          table sits in shared memory; each warp streams the codes of its probed lists with
//          128-bit coalesced loads (one vector per lane), sums M table entries in fp32 in
//          ascending m, and keeps a sorted top-k distributed over the warp's registers; the four
//          warp lists are merged by a shared-memory bitonic sort.
#include "ivfpq_index.h"

#include <algorithm>
#include <cub/cub.cuh>
#include <unordered_set>

#include "select.cuh"

namespace b200 {
namespace {

constexpr int kKsub = 256;
constexpr int kScanThreads = 128;
constexpr int kScanWarps = kScanThreads / 32;

__global__ void cb_norm_kernel(const float* cb, int M, int dsub, float* out) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= M * kKsub) return;
    const float* c = cb + static_cast<int64_t>(idx) * dsub;
    float acc = 0.f;
    for (int t = 0; t < dsub; ++t) acc = fmaf(c[t], c[t], acc);
    out[idx] = acc;
}

// lut[q][m][j]; one thread per entry.
__global__ void lut_kernel(const float* xq, int64_t nq, int d, int M, int dsub, const float* cb, int by_residual,
                           float* lut) {
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= nq * M * kKsub) return;
    const int j = static_cast<int>(idx % kKsub);
    const int m = static_cast<int>((idx / kKsub) % M);
    const int64_t q = idx / (static_cast<int64_t>(kKsub) * M);
    const float* qv = xq + q * d + m * dsub;
    const float* c = cb + (static_cast<int64_t>(m) * kKsub + j) * dsub;
    float acc = 0.f;
    if (by_residual) {
        for (int t = 0; t < dsub; ++t) acc = fmaf(qv[t], c[t], acc);
        acc = -2.f * acc;
    } else {
        for (int t = 0; t < dsub; ++t) {
            const float df = qv[t] - c[t];
            acc = fmaf(df, df, acc);
        }
    }
    lut[idx] = acc;
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

// t2[v] = sum_m ( |cb[m][code]|^2 + 2 c_list,m . cb[m][code] ), fp32, m ascending.
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
__global__ void add_counts_kernel(const int64_t* old_off, const int64_t* new_hist, int nlist, int64_t* total) {
    const int l = blockIdx.x * blockDim.x + threadIdx.x;
    if (l < nlist) total[l] = (old_off[l + 1] - old_off[l]) + new_hist[l];
    if (l == nlist) total[l] = 0;
}
__global__ void iota_i32_kernel(int32_t* p, int64_t n) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) p[i] = static_cast<int32_t>(i);
}
__global__ void scatter_old_kernel(int64_t n_old, int nlist, const int64_t* old_off, const int64_t* new_off, int M,
                                   const uint8_t* codes, const int64_t* ids, const float* t2, uint8_t* ncodes,
                                   int64_t* nids, float* nt2) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_old) return;
    int lo = 0, hi = nlist;  // largest l with old_off[l] <= i
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (old_off[mid] <= i) lo = mid;
        else hi = mid;
    }
    const int64_t dst = new_off[lo] + (i - old_off[lo]);
    for (int b = 0; b < M; ++b) ncodes[dst * M + b] = codes[i * M + b];
    nids[dst] = ids[i];
    if (t2) nt2[dst] = t2[i];
}
__global__ void scatter_new_kernel(int64_t n_new, const int32_t* sorted_list, const int32_t* sorted_src,
                                   const int64_t* old_off, const int64_t* new_off, const int64_t* new_first, int M,
                                   const uint8_t* codes, const int64_t* ids, const float* t2, uint8_t* ncodes,
                                   int64_t* nids, float* nt2) {
    const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (j >= n_new) return;
    const int l = sorted_list[j];
    const int64_t src = sorted_src[j];
    const int64_t dst = new_off[l] + (old_off[l + 1] - old_off[l]) + (j - new_first[l]);
    for (int b = 0; b < M; ++b) ncodes[dst * M + b] = codes[src * M + b];
    nids[dst] = ids[src];
    if (t2) nt2[dst] = t2[src];
}

// ---- scan ----
struct ScanArgs {
    const float* lut;        // [nq][M][256]
    const int64_t* cI;       // [nq][nprobe] probed list ids (-1 = none)
    const float* cD;         // [nq][nprobe] coarse distances
    int nprobe;
    const int64_t* offsets;  // [nlist + 1]
    const uint8_t* codes;
    const int64_t* ids;
    const float* t2;
    int by_residual;
    int k;
    int S;                   // probe splits per query
    int M;
    int64_t nq;
    float* outD;             // [S][nq][k]
    int64_t* outI;
    unsigned long long* scanned;  // statistics: codes visited
};

__device__ __forceinline__ bool pair_less(float d1, int64_t l1, float d2, int64_t l2) {
    return d1 < d2 || (d1 == d2 && l1 < l2);
}

// Sorted top-(32*KPT) list spread over a warp: rank r lives in lane r / KPT, slot r % KPT.
template <int KPT>
__device__ __forceinline__ void warp_insert(float (&dk)[KPT], int64_t (&lb)[KPT], float vd, int64_t vl, int lane) {
    const float pd = __shfl_up_sync(0xffffffffu, dk[KPT - 1], 1);
    const int64_t pl = __shfl_up_sync(0xffffffffu, lb[KPT - 1], 1);
    bool ls[KPT];
#pragma unroll
    for (int s = 0; s < KPT; ++s) ls[s] = pair_less(dk[s], lb[s], vd, vl);
    const bool prev_less = lane == 0 ? true : pair_less(pd, pl, vd, vl);
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

__device__ __forceinline__ float lut_sum_word(const float* lut, int m0, uint32_t w, float acc) {
    acc = acc + lut[(m0 + 0) * kKsub + (w & 255u)];
    acc = acc + lut[(m0 + 1) * kKsub + ((w >> 8) & 255u)];
    acc = acc + lut[(m0 + 2) * kKsub + ((w >> 16) & 255u)];
    acc = acc + lut[(m0 + 3) * kKsub + (w >> 24)];
    return acc;
}

// MT: 16-byte words per code (M = 16 * MT), or 0 for any M (byte loads).
template <int MT, int KPT>
__global__ void __launch_bounds__(kScanThreads)
ivfpq_scan_kernel(const ScanArgs a) {
    extern __shared__ __align__(16) uint8_t scan_smem[];
    float* lut = reinterpret_cast<float*>(scan_smem);
    const int64_t q = blockIdx.x;
    const int split = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int M = MT > 0 ? MT * 16 : a.M;

    {
        const float4* src = reinterpret_cast<const float4*>(a.lut + q * M * kKsub);
        float4* dst = reinterpret_cast<float4*>(lut);
        for (int i = threadIdx.x; i < M * kKsub / 4; i += kScanThreads) dst[i] = __ldg(src + i);
    }
    __syncthreads();

    float dk[KPT];
    int64_t lb[KPT];
#pragma unroll
    for (int s = 0; s < KPT; ++s) {
        dk[s] = __int_as_float(0x7f800000);
        lb[s] = 0x7fffffffffffffffll;
    }
    float th_d = __int_as_float(0x7f800000);
    int64_t th_l = 0x7fffffffffffffffll;
    unsigned long long visited = 0;

    for (int p = split + a.S * warp; p < a.nprobe; p += a.S * kScanWarps) {
        const int64_t list = a.cI[q * a.nprobe + p];
        if (list < 0) continue;
        const int64_t begin = a.offsets[list], end = a.offsets[list + 1];
        const float base = a.by_residual ? a.cD[q * a.nprobe + p] : 0.f;
        visited += static_cast<unsigned long long>(end - begin);
        for (int64_t v0 = begin; v0 < end; v0 += 32) {
            const int64_t v = v0 + lane;
            const bool valid = v < end;
            float acc = base;
            if (valid) {
                if (a.by_residual) acc = acc + a.t2[v];
                if (MT > 0) {
                    const uint4* cp = reinterpret_cast<const uint4*>(a.codes + v * M);
#pragma unroll
                    for (int w = 0; w < MT; ++w) {
                        const uint4 c = __ldg(cp + w);
                        acc = lut_sum_word(lut, w * 16 + 0, c.x, acc);
                        acc = lut_sum_word(lut, w * 16 + 4, c.y, acc);
                        acc = lut_sum_word(lut, w * 16 + 8, c.z, acc);
                        acc = lut_sum_word(lut, w * 16 + 12, c.w, acc);
                    }
                } else {
                    const uint8_t* cp = a.codes + v * M;
                    for (int m = 0; m < M; ++m) acc = acc + lut[m * kKsub + cp[m]];
                }
            }
            bool pass = valid && acc <= th_d;
            int64_t label = 0;
            if (pass) {
                label = a.ids[v];
                pass = pair_less(acc, label, th_d, th_l);
            }
            unsigned bal = __ballot_sync(0xffffffffu, pass);
            while (bal) {
                const int src = __ffs(bal) - 1;
                bal &= bal - 1;
                const float vd = __shfl_sync(0xffffffffu, acc, src);
                const int64_t vl = __shfl_sync(0xffffffffu, label, src);
                warp_insert<KPT>(dk, lb, vd, vl, lane);
                th_d = __shfl_sync(0xffffffffu, dk[KPT - 1], 31);
                th_l = __shfl_sync(0xffffffffu, lb[KPT - 1], 31);
            }
        }
    }
    if (a.scanned && lane == 0 && visited) atomicAdd(a.scanned, visited);

    // merge the warp lists
    __syncthreads();  // everyone is done with the table
    constexpr int E = kScanThreads * KPT;
    int64_t* sl = reinterpret_cast<int64_t*>(scan_smem);
    float* sd = reinterpret_cast<float*>(scan_smem + static_cast<size_t>(E) * 8);
#pragma unroll
    for (int s = 0; s < KPT; ++s) {
        sd[threadIdx.x * KPT + s] = dk[s];
        sl[threadIdx.x * KPT + s] = lb[s];
    }
    __syncthreads();
    for (int size = 2; size <= E; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = threadIdx.x; i < E / 2; i += kScanThreads) {
                const int lo = 2 * i - (i & (stride - 1));
                const int hi = lo + stride;
                const bool up = (lo & size) == 0;
                const float d1 = sd[lo], d2 = sd[hi];
                const int64_t l1 = sl[lo], l2 = sl[hi];
                if (pair_less(d2, l2, d1, l1) == up) {
                    sd[lo] = d2; sd[hi] = d1;
                    sl[lo] = l2; sl[hi] = l1;
                }
            }
            __syncthreads();
        }
    }
    float* oD = a.outD + (static_cast<int64_t>(split) * a.nq + q) * a.k;
    int64_t* oI = a.outI + (static_cast<int64_t>(split) * a.nq + q) * a.k;
    for (int i = threadIdx.x; i < a.k; i += kScanThreads) {
        const bool real = i < E && sl[i] != 0x7fffffffffffffffll;
        oD[i] = real ? sd[i] : 3.402823466e+38f;
        oI[i] = real ? sl[i] : -1;
    }
}

template <int MT>
cudaError_t launch_scan_mt(const ScanArgs& a, int kpt, size_t smem, dim3 grid, cudaStream_t st) {
#define B200_SCAN_CASE(KP)                                                                                      \
    case KP: {                                                                                                   \
        auto kern = ivfpq_scan_kernel<MT, KP>;                                                                   \
        if (smem > 48 * 1024) {                                                                                  \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
            if (e != cudaSuccess) return e;                                                                      \
        }                                                                                                        \
        kern<<<grid, kScanThreads, smem, st>>>(a);                                                               \
        return cudaGetLastError();                                                                               \
    }
    switch (kpt) {
        B200_SCAN_CASE(1)
        B200_SCAN_CASE(2)
        B200_SCAN_CASE(4)
        B200_SCAN_CASE(8)
        B200_SCAN_CASE(16)
        B200_SCAN_CASE(32)
        default: return cudaErrorInvalidValue;
    }
#undef B200_SCAN_CASE
}

cudaError_t launch_scan(const ScanArgs& a, cudaStream_t st) {
    int kpt = 1;
    while (kpt * 32 < a.k) kpt <<= 1;
    if (kpt > 32) return cudaErrorInvalidValue;
    const size_t lut_bytes = static_cast<size_t>(a.M) * kKsub * 4;
    const size_t sort_bytes = static_cast<size_t>(kScanThreads) * kpt * 12;
    const size_t smem = std::max(lut_bytes, sort_bytes);
    dim3 grid(static_cast<unsigned>(a.nq), static_cast<unsigned>(a.S));
    if (a.M % 16 == 0 && a.M <= 64) {
        switch (a.M / 16) {
            case 1: return launch_scan_mt<1>(a, kpt, smem, grid, st);
            case 2: return launch_scan_mt<2>(a, kpt, smem, grid, st);
            case 3: return launch_scan_mt<3>(a, kpt, smem, grid, st);
            case 4: return launch_scan_mt<4>(a, kpt, smem, grid, st);
        }
    }
    return launch_scan_mt<0>(a, kpt, smem, grid, st);
}

inline unsigned blocks_for(int64_t n, int threads) { return static_cast<unsigned>((n + threads - 1) / threads); }

}  // namespace

IvfpqIndex::IvfpqIndex(int d, int nlist, int M, int nbits, bool by_residual, int device)
    : d_(d), nlist_(nlist), M_(M), dsub_(d / M), device_(device), by_residual_(by_residual) {
    if (nbits != 8) throw std::invalid_argument("IVFPQ supports nbits = 8 only");
    if (M <= 0 || d % M != 0) throw std::invalid_argument("d must be a multiple of M");
    DeviceGuard g(device_);
    B200_CUDA_CHECK(cudaDeviceGetAttribute(&num_sms_, cudaDevAttrMultiProcessorCount, device_));
    coarse_.reset(new FlatIndex(d, kMetricL2, kF32, device));
    offsets_.ensure(static_cast<size_t>(nlist_ + 1) * 8);
    B200_CUDA_CHECK(cudaMemset(offsets_.get(), 0, static_cast<size_t>(nlist_ + 1) * 8));
    offsets_host_.assign(static_cast<size_t>(nlist_ + 1), 0);
    w_tmp_.ensure(sizeof(unsigned long long));
    B200_CUDA_CHECK(cudaMemset(w_tmp_.get(), 0, sizeof(unsigned long long)));
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
    has_codebooks_ = true;
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
// follow in arrival order (the order the reference's per-list append produces).
void IvfpqIndex::merge_new(int64_t n, const int32_t* ln, const uint8_t* cd, const float* t2, const int64_t* idd) {
    cudaStream_t st = stream();
    const int64_t n_new_total = n_ + n;
    if (n_new_total > 0x7FFFFFF0ll) throw std::invalid_argument("a single-device IVFPQ index holds at most 2^31 - 16 vectors");
    DeviceBuffer hist, total, new_off, new_first, keys_out, vals_in, vals_out, cub_tmp;
    DeviceBuffer ncodes, nids, nt2;
    int64_t* h = static_cast<int64_t*>(hist.ensure(static_cast<size_t>(nlist_ + 1) * 8));
    B200_CUDA_CHECK(cudaMemsetAsync(h, 0, static_cast<size_t>(nlist_ + 1) * 8, st));
    hist_kernel<<<blocks_for(n, 256), 256, 0, st>>>(ln, n, h);
    int64_t* tot = static_cast<int64_t*>(total.ensure(static_cast<size_t>(nlist_ + 1) * 8));
    add_counts_kernel<<<blocks_for(nlist_ + 1, 256), 256, 0, st>>>(offsets_.as<int64_t>(), h, nlist_, tot);
    int64_t* noff = static_cast<int64_t*>(new_off.ensure(static_cast<size_t>(nlist_ + 1) * 8));
    int64_t* nfirst = static_cast<int64_t*>(new_first.ensure(static_cast<size_t>(nlist_ + 1) * 8));
    size_t tmp_bytes = 0, tb = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, tmp_bytes, tot, noff, nlist_ + 1, st);
    int32_t* kout = static_cast<int32_t*>(keys_out.ensure(static_cast<size_t>(n) * 4));
    int32_t* vin = static_cast<int32_t*>(vals_in.ensure(static_cast<size_t>(n) * 4));
    int32_t* vout = static_cast<int32_t*>(vals_out.ensure(static_cast<size_t>(n) * 4));
    int end_bit = 1;
    while ((1 << end_bit) < nlist_) ++end_bit;
    cub::DeviceRadixSort::SortPairs(nullptr, tb, ln, kout, vin, vout, static_cast<int>(n), 0, end_bit, st);
    tmp_bytes = std::max(tmp_bytes, tb);
    void* tmp = cub_tmp.ensure(tmp_bytes + 16);
    size_t tsz = tmp_bytes;
    B200_CUDA_CHECK(cub::DeviceScan::ExclusiveSum(tmp, tsz, tot, noff, nlist_ + 1, st));
    tsz = tmp_bytes;
    B200_CUDA_CHECK(cub::DeviceScan::ExclusiveSum(tmp, tsz, h, nfirst, nlist_ + 1, st));
    iota_i32_kernel<<<blocks_for(n, 256), 256, 0, st>>>(vin, n);
    tsz = tmp_bytes;
    B200_CUDA_CHECK(cub::DeviceRadixSort::SortPairs(tmp, tsz, ln, kout, vin, vout, static_cast<int>(n), 0, end_bit, st));

    uint8_t* nc = static_cast<uint8_t*>(ncodes.ensure(static_cast<size_t>(n_new_total) * M_ + 64));
    int64_t* ni = static_cast<int64_t*>(nids.ensure(static_cast<size_t>(n_new_total) * 8));
    float* nt = by_residual_ ? static_cast<float*>(nt2.ensure(static_cast<size_t>(n_new_total) * 4)) : nullptr;
    if (n_ > 0)
        scatter_old_kernel<<<blocks_for(n_, 256), 256, 0, st>>>(n_, nlist_, offsets_.as<int64_t>(), noff, M_,
                                                                codes_.as<uint8_t>(), ids_.as<int64_t>(),
                                                                by_residual_ ? t2_.as<float>() : nullptr, nc, ni, nt);
    scatter_new_kernel<<<blocks_for(n, 256), 256, 0, st>>>(n, kout, vout, offsets_.as<int64_t>(), noff, nfirst, M_, cd,
                                                           idd, t2, nc, ni, nt);
    B200_CUDA_CHECK(cudaGetLastError());
    B200_CUDA_CHECK(cudaMemcpyAsync(offsets_host_.data(), noff, static_cast<size_t>(nlist_ + 1) * 8,
                                    cudaMemcpyDeviceToHost, st));
    B200_CUDA_CHECK(cudaStreamSynchronize(st));
    offsets_.swap(new_off);
    codes_.swap(ncodes);
    ids_.swap(nids);
    if (by_residual_) t2_.swap(nt2);
    n_ = n_new_total;
}

void IvfpqIndex::reset() {
    DeviceGuard g(device_);
    cudaStreamSynchronize(stream());
    n_ = 0;
    cudaMemset(offsets_.get(), 0, static_cast<size_t>(nlist_ + 1) * 8);
    offsets_host_.assign(static_cast<size_t>(nlist_ + 1), 0);
}

int64_t IvfpqIndex::remove_ids(int64_t n, const int64_t* ids) {
    if (n <= 0 || n_ == 0) return 0;
    DeviceGuard g(device_);
    std::vector<int64_t> hid(static_cast<size_t>(n_));
    std::vector<uint8_t> hcodes(static_cast<size_t>(n_) * M_);
    B200_CUDA_CHECK(cudaMemcpy(hid.data(), ids_.get(), hid.size() * 8, cudaMemcpyDeviceToHost));
    B200_CUDA_CHECK(cudaMemcpy(hcodes.data(), codes_.get(), hcodes.size(), cudaMemcpyDeviceToHost));
    std::unordered_set<int64_t> rm(ids, ids + n);
    std::vector<int32_t> ln;
    std::vector<int64_t> kid;
    std::vector<uint8_t> kc;
    ln.reserve(hid.size());
    kid.reserve(hid.size());
    kc.reserve(hcodes.size());
    int64_t removed = 0;
    for (int l = 0; l < nlist_; ++l)
        for (int64_t v = offsets_host_[l]; v < offsets_host_[l + 1]; ++v) {
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
    return offsets_host_[static_cast<size_t>(list) + 1] - offsets_host_[static_cast<size_t>(list)];
}

void IvfpqIndex::get_list(int list, uint8_t* codes, int64_t* ids) const {
    const int64_t len = list_length(list);
    if (len == 0) return;
    DeviceGuard g(device_);
    const int64_t b = offsets_host_[static_cast<size_t>(list)];
    if (codes)
        B200_CUDA_CHECK(cudaMemcpy(codes, codes_.as<uint8_t>() + b * M_, static_cast<size_t>(len) * M_,
                                   cudaMemcpyDeviceToHost));
    if (ids) B200_CUDA_CHECK(cudaMemcpy(ids, ids_.as<int64_t>() + b, static_cast<size_t>(len) * 8, cudaMemcpyDeviceToHost));
}

void IvfpqIndex::search_device(int64_t nq, const float* xq, int k, float* D, int64_t* I) {
    if (nq <= 0) return;
    if (!is_trained()) throw std::invalid_argument("IVFPQ index is not trained (centroids / codebooks missing)");
    DeviceGuard g(device_);
    cudaStream_t st = stream();
    stats_.searches += 1;
    stats_.queries += static_cast<uint64_t>(nq);
    const int nprobe = std::max(1, std::min(nprobe_, nlist_));
    const int64_t page = 16384;
    for (int64_t q0 = 0; q0 < nq; q0 += page) {
        const int64_t m = std::min(page, nq - q0);
        const float* xp = xq + q0 * d_;
        float* cD = static_cast<float*>(w_cD_.ensure(static_cast<size_t>(m) * nprobe * 4));
        int64_t* cI = static_cast<int64_t*>(w_cI_.ensure(static_cast<size_t>(m) * nprobe * 8));
        timer_.begin(kStageCoarse, st);
        coarse_->search_device(m, xp, false, nprobe, cD, cI, nprobe);
        timer_.end(st);
        timer_.begin(kStageLut, st);
        float* lut = static_cast<float*>(w_lut_.ensure(static_cast<size_t>(m) * M_ * kKsub * 4));
        lut_kernel<<<blocks_for(m * M_ * kKsub, 256), 256, 0, st>>>(xp, m, d_, M_, dsub_, codebooks_.as<float>(),
                                                                   by_residual_ ? 1 : 0, lut);
        B200_CUDA_CHECK(cudaGetLastError());
        timer_.end(st);
        int S = static_cast<int>((16LL * num_sms_ + m - 1) / m);
        S = std::max(1, std::min(S, (nprobe + kScanWarps - 1) / kScanWarps));
        ScanArgs a{};
        a.lut = lut;
        a.cI = cI;
        a.cD = cD;
        a.nprobe = nprobe;
        a.offsets = offsets_.as<int64_t>();
        a.codes = codes_.as<uint8_t>();
        a.ids = ids_.as<int64_t>();
        a.t2 = t2_.as<float>();
        a.by_residual = by_residual_ ? 1 : 0;
        a.k = k;
        a.S = S;
        a.M = M_;
        a.nq = m;
        a.scanned = w_tmp_.as<unsigned long long>();
        if (S == 1) {
            a.outD = D + q0 * k;
            a.outI = I + q0 * k;
            timer_.begin(kStageScan, st);
            B200_CUDA_CHECK(launch_scan(a, st));
            timer_.end(st);
            stats_.kernel_launches += 2;
        } else {
            a.outD = static_cast<float*>(w_pD_.ensure(static_cast<size_t>(S) * m * k * 4));
            a.outI = static_cast<int64_t*>(w_pI_.ensure(static_cast<size_t>(S) * m * k * 8));
            timer_.begin(kStageScan, st);
            B200_CUDA_CHECK(launch_scan(a, st));
            timer_.end(st);
            timer_.begin(kStageMerge, st);
            B200_CUDA_CHECK(launch_merge_topk(S, m, k, 0, a.outD, a.outI, D + q0 * k, I + q0 * k, st));
            timer_.end(st);
            stats_.kernel_launches += 3;
        }
    }
    unsigned long long scanned = 0;
    B200_CUDA_CHECK(cudaMemcpyAsync(&scanned, w_tmp_.get(), 8, cudaMemcpyDeviceToHost, st));
    B200_CUDA_CHECK(cudaStreamSynchronize(st));
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
