// Lloyd k-means on the device, in an arithmetic that a CPU restatement reproduces bit for bit
// (replaces the reference's NPU training loop, feature_retrieval/src/ascendfaiss/ascenddaemon/impl/
// IndexIVFPQ.cpp:810-1135 -- distance operator, arg-min, centroid update -- and the host-side
// sub-space training of AscendIndexIVFPQImpl.cpp:962-1252):
//   start   : centroid c = x[(floor(c * n / k) + seed) mod n]
//   assign  : nearest centroid under the canonical fp32 L2 distance (sequential fmaf), ties -> lower
//             centroid.  d % 16 == 0: the Flat fp32 search (tcgen05 filter + canonical refinement)
//             with k = 1 on the centroids; otherwise (PQ sub-spaces of a few dimensions) a direct kernel.
//   update  : members grouped by a stable radix sort of (centroid, vector index); one thread per
//             (centroid, dimension) adds its members in increasing vector index in fp64 and rounds
//             the mean to fp32 once.  A centroid without members keeps its value.
#include "kmeans.h"

#include <cub/cub.cuh>

#include <memory>
#include <stdexcept>

#include "common.cuh"
#include "device_mem.h"
#include "flat_index.h"
#include "select.cuh"

namespace b200 {
namespace {

__global__ void km_init_kernel(const float* x, int64_t n, int d, int k, uint64_t seed, float* cent) {
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<int64_t>(k) * d) return;
    const int c = static_cast<int>(idx / d), t = static_cast<int>(idx % d);
    // floor(c * n / k) without a 128-bit product: n / k and n % k
    const int64_t qn = n / k, rn = n % k;
    int64_t src = static_cast<int64_t>(c) * qn + (static_cast<int64_t>(c) * rn) / k;
    src = static_cast<int64_t>((static_cast<uint64_t>(src) + seed) % static_cast<uint64_t>(n));
    cent[idx] = x[src * d + t];
}

// small d: one thread per vector, every centroid, canonical arithmetic
__global__ void km_assign_direct_kernel(const float* x, int64_t n, int d, const float* cent, int k, int32_t* assign) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float best = __int_as_float(0x7f800000);
    int arg = 0;
    for (int c = 0; c < k; ++c) {
        float acc = 0.f;
        for (int t = 0; t < d; ++t) {
            const float df = x[i * d + t] - cent[static_cast<int64_t>(c) * d + t];
            acc = fmaf(df, df, acc);
        }
        if (acc < best) {
            best = acc;
            arg = c;
        }
    }
    assign[i] = arg;
}

__global__ void km_narrow_kernel(const int64_t* in, int64_t n, int32_t* out) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = static_cast<int32_t>(in[i]);
}
__global__ void km_iota_kernel(int32_t* p, int64_t n) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) p[i] = static_cast<int32_t>(i);
}
__global__ void km_hist_kernel(const int32_t* assign, int64_t n, unsigned long long* hist) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) atomicAdd(hist + assign[i], 1ull);
}
// members of centroid c: sorted_idx[off[c] .. off[c + 1]) in increasing vector index
__global__ void km_update_kernel(const float* x, int d, int k, const unsigned long long* off, const int32_t* sorted_idx,
                                 float* cent) {
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<int64_t>(k) * d) return;
    const int c = static_cast<int>(idx / d), t = static_cast<int>(idx % d);
    const unsigned long long b = off[c], e = off[c + 1];
    if (b == e) return;
    double s = 0.0;
    for (unsigned long long j = b; j < e; ++j) s += static_cast<double>(x[static_cast<int64_t>(sorted_idx[j]) * d + t]);
    cent[idx] = static_cast<float>(s / static_cast<double>(e - b));
}

inline unsigned nblk(int64_t n, int t) { return static_cast<unsigned>((n + t - 1) / t); }

}  // namespace

void kmeans_assign_device(FlatIndex* flat, cudaStream_t st, const float* x_dev, int64_t n, int d, const float* cent_dev,
                          int k, int32_t* assign_dev, DeviceBuffer& scratch) {
    if (flat) {
        flat->reset();
        flat->add(k, cent_dev, false, nullptr, true);
        float* D = static_cast<float*>(scratch.ensure(static_cast<size_t>(n) * 12));
        int64_t* I = reinterpret_cast<int64_t*>(D + n + (n & 1));
        flat->search_device(n, x_dev, false, 1, D, I, 1);
        km_narrow_kernel<<<nblk(n, 256), 256, 0, st>>>(I, n, assign_dev);
    } else {
        km_assign_direct_kernel<<<nblk(n, 128), 128, 0, st>>>(x_dev, n, d, cent_dev, k, assign_dev);
    }
    B200_CUDA_CHECK(cudaGetLastError());
}

void kmeans_device(int device, int d, int64_t n, const float* x_dev, int k, int niter, uint64_t seed, float* cent_dev,
                   int32_t* assign_out_dev) {
    if (d <= 0 || n <= 0 || k <= 0 || niter < 0) throw std::invalid_argument("k-means: d, n, k must be > 0, niter >= 0");
    if (n > 0x7FFFFFF0ll) throw std::invalid_argument("k-means: at most 2^31 - 16 training vectors");
    DeviceGuard g(device);
    std::unique_ptr<FlatIndex> flat;
    if (d % 16 == 0 && d <= 4096) flat.reset(new FlatIndex(d, kMetricL2, kF32, device));
    cudaStream_t st = flat ? flat->stream() : nullptr;
    DeviceBuffer assign_own, keys_out, vals_in, vals_out, hist, off, tmp, scratch;
    int32_t* assign = assign_out_dev ? assign_out_dev : static_cast<int32_t*>(assign_own.ensure(static_cast<size_t>(n) * 4));
    int32_t* kout = static_cast<int32_t*>(keys_out.ensure(static_cast<size_t>(n) * 4));
    int32_t* vin = static_cast<int32_t*>(vals_in.ensure(static_cast<size_t>(n) * 4));
    int32_t* vout = static_cast<int32_t*>(vals_out.ensure(static_cast<size_t>(n) * 4));
    unsigned long long* h = static_cast<unsigned long long*>(hist.ensure(static_cast<size_t>(k + 1) * 8));
    unsigned long long* o = static_cast<unsigned long long*>(off.ensure(static_cast<size_t>(k + 1) * 8));
    int end_bit = 1;
    while ((1ll << end_bit) < k) ++end_bit;
    size_t t1 = 0, t2 = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, t1, assign, kout, vin, vout, static_cast<int>(n), 0, end_bit, st);
    cub::DeviceScan::ExclusiveSum(nullptr, t2, h, o, k + 1, st);
    const size_t tbytes = std::max(t1, t2);
    void* tp = tmp.ensure(tbytes + 16);

    // A non-finite training vector has no nearest centroid; an assignment outside [0, k) must never
    // reach the histogram or the update below.
    DeviceBuffer vflag_buf;
    int* vflag = static_cast<int*>(vflag_buf.ensure(sizeof(int)));
    auto read_flag = [&]() {
        int hf = 0;
        B200_CUDA_CHECK(cudaMemcpyAsync(&hf, vflag, sizeof(int), cudaMemcpyDeviceToHost, st));
        B200_CUDA_CHECK(cudaStreamSynchronize(st));
        return hf;
    };
    B200_CUDA_CHECK(cudaMemsetAsync(vflag, 0, sizeof(int), st));
    B200_CUDA_CHECK(launch_check_finite(x_dev, n * d, vflag, st));
    if (read_flag()) throw std::invalid_argument("k-means: the training vectors hold NaN or infinite values");

    km_init_kernel<<<nblk(static_cast<int64_t>(k) * d, 256), 256, 0, st>>>(x_dev, n, d, k, seed, cent_dev);
    km_iota_kernel<<<nblk(n, 256), 256, 0, st>>>(vin, n);
    B200_CUDA_CHECK(cudaGetLastError());
    for (int it = 0; it < niter; ++it) {
        kmeans_assign_device(flat.get(), st, x_dev, n, d, cent_dev, k, assign, scratch);
        B200_CUDA_CHECK(launch_check_range_i32(assign, n, k, vflag, st));
        if (read_flag()) throw std::invalid_argument("k-means: a vector could not be assigned (distance overflow)");
        B200_CUDA_CHECK(cudaMemsetAsync(h, 0, static_cast<size_t>(k + 1) * 8, st));
        km_hist_kernel<<<nblk(n, 256), 256, 0, st>>>(assign, n, h);
        size_t tb = tbytes;
        B200_CUDA_CHECK(cub::DeviceScan::ExclusiveSum(tp, tb, h, o, k + 1, st));
        tb = tbytes;
        B200_CUDA_CHECK(cub::DeviceRadixSort::SortPairs(tp, tb, assign, kout, vin, vout, static_cast<int>(n), 0, end_bit, st));
        km_update_kernel<<<nblk(static_cast<int64_t>(k) * d, 128), 128, 0, st>>>(x_dev, d, k, o, vout, cent_dev);
        B200_CUDA_CHECK(cudaGetLastError());
    }
    if (assign_out_dev) {   // assignment to the FINAL centroids
        kmeans_assign_device(flat.get(), st, x_dev, n, d, cent_dev, k, assign, scratch);
        B200_CUDA_CHECK(launch_check_range_i32(assign, n, k, vflag, st));
        if (read_flag()) throw std::invalid_argument("k-means: a vector could not be assigned (distance overflow)");
    }
    B200_CUDA_CHECK(cudaStreamSynchronize(st));
}

}  // namespace b200
