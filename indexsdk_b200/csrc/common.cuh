// Shared definitions for the search kernels: ordered-key encodings, candidate packing,
// error words, launch helpers.
#pragma once
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <stdexcept>
#include <string>

namespace b200 {

// Status values follow the reference's APP_ERROR numbering
// (feature_retrieval/src/ascendfaiss/common/ErrorCode.h:50-66).
enum Status : int {
    kOk = 0,
    kInvalidParam = 2001,
    kNotImplemented = 2008,
    kInnerError = 2010,
    kTimeout = 2011,
};

// kMetricCos: int8 only -- the fp16 cosine the reference's Int8Flat index computes for
// METRIC_INNER_PRODUCT (see cos16_* below); larger is better, like kMetricIP.
enum Metric : int { kMetricIP = 0, kMetricL2 = 1, kMetricCos = 2 };
enum DType : int { kF32 = 0, kF16 = 1, kBF16 = 2, kI8 = 3 };

// Device error word bits (one int per index, polled by the host after each search).
enum DevErr : int {
    kDevErrPipelineTimeout = 1,  // a bounded mbarrier wait in the GEMM pipeline ran out
    kDevErrBadArgs = 2,
};

struct CudaError : std::runtime_error {
    explicit CudaError(const std::string& m) : std::runtime_error(m) {}
};

#define B200_CUDA_CHECK(expr)                                                                          \
    do {                                                                                               \
        cudaError_t _e = (expr);                                                                       \
        if (_e != cudaSuccess)                                                                         \
            throw ::b200::CudaError(std::string(#expr) + ": " + cudaGetErrorString(_e) + " (" __FILE__ \
                                    ":" + std::to_string(__LINE__) + ")");                             \
    } while (0)

// Monotone float -> uint32 map: a < b  <=>  ord(a) < ord(b) for all non-NaN floats.
__host__ __device__ __forceinline__ uint32_t float_to_ord(float f) {
#ifdef __CUDA_ARCH__
    uint32_t u = __float_as_uint(f);
#else
    uint32_t u;
    memcpy(&u, &f, 4);
#endif
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__host__ __device__ __forceinline__ float ord_to_float(uint32_t o) {
    uint32_t u = (o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o;
#ifdef __CUDA_ARCH__
    return __uint_as_float(u);
#else
    float f;
    memcpy(&f, &u, 4);
    return f;
#endif
}
__host__ __device__ __forceinline__ uint32_t int_to_ord(int32_t v) { return static_cast<uint32_t>(v) ^ 0x80000000u; }
__host__ __device__ __forceinline__ int32_t ord_to_int(uint32_t o) { return static_cast<int32_t>(o ^ 0x80000000u); }

// A candidate is (ordered key, position) packed so that unsigned 64-bit order is
// (key ascending, position ascending).
__host__ __device__ __forceinline__ uint64_t pack_cand(uint32_t ord_key, uint32_t pos) {
    return (static_cast<uint64_t>(ord_key) << 32) | pos;
}

constexpr uint64_t kCandInvalid = 0xFFFFFFFFFFFFFFFFull;

inline int div_up(int64_t a, int64_t b) { return static_cast<int>((a + b - 1) / b); }

}  // namespace b200
