// The fp16 cosine that the reference's int8 Flat index returns for METRIC_INNER_PRODUCT
// (feature_retrieval/src/ascendfaiss/ascend/impl/AscendIndexInt8FlatImpl.cpp:790-793 picks the
// "Cos" index; the arithmetic is ops/tbe/impl/int8_l2_norm.py:140-183 and
// ops/tbe/impl/distance_int8_cos_maxs.py:256-284, the same in
// ops/ascendc/op_kernel/ascendc_dist_int8_flat_cos.cpp:139-141,314-316):
//
//   rnorm(x) = fp16( 1 / sqrt( fp16( |x|^2 * 0.01 ) ) )          ( = 10 / |x| )
//   score    = fp16( fp16( q.x * 0.01 ) * fp16( rnorm(x) * rnorm(q) ) )
//
// with |x|^2 and q.x exact int32 values and every fp16 step rounded to nearest even.  The search
// kernels carry the score as a 32-bit integer that orders like the fp16 value (cos16_order), so
// everything between the accumulator and the result rows treats it as an inner product.
// A score that is NaN (a zero vector: 0 x inf; or a saturated product x 0) ranks below every
// number and is reported as -inf.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace b200 {

constexpr int32_t kCos16NaN = -32768;

// fp16 bits of rnorm from the exact squared norm (< 2^24, so the conversion to float is exact)
__device__ __forceinline__ uint32_t cos16_rnorm_bits(int32_t sq) {
    const __half s = __float2half_rn(__fmul_rn(__int2float_rn(sq), 0.01f));
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__half2float(s)));
    return static_cast<uint32_t>(__half_as_ushort(__float2half_rn(r)));
}

// 16 fp16 bits -> integer with the order of the values (-0 directly below +0)
__device__ __forceinline__ int32_t cos16_order(uint32_t hbits) {
    const int32_t x = static_cast<int16_t>(static_cast<uint16_t>(hbits));
    const int32_t s = x ^ ((x >> 31) & 0x7FFF);
    return (x & 0x7FFF) > 0x7C00 ? kCos16NaN : s;
}

// Two accumulators at once.  n0, n1: rnorm bits of the two base rows (low 16 bits); rq2: the
// query's rnorm in both halves.
__device__ __forceinline__ void cos16_pair(int32_t a0, int32_t a1, uint32_t n0, uint32_t n1, __half2 rq2,
                                           int32_t& s0, int32_t& s1) {
    const __half2 ip = __floats2half2_rn(__fmul_rn(__int2float_rn(a0), 0.01f), __fmul_rn(__int2float_rn(a1), 0.01f));
    const uint32_t nn = (n0 & 0xFFFFu) | (n1 << 16);
    const __half2 w = __hmul2(*reinterpret_cast<const __half2*>(&nn), rq2);
    const __half2 r = __hmul2(ip, w);
    const uint32_t bits = *reinterpret_cast<const uint32_t*>(&r);
    s0 = cos16_order(bits & 0xFFFFu);
    s1 = cos16_order(bits >> 16);
}

__device__ __forceinline__ __half2 cos16_query_term(int32_t qsq) {
    const uint32_t b = cos16_rnorm_bits(qsq);
    const uint32_t bb = b | (b << 16);
    return *reinterpret_cast<const __half2*>(&bb);
}

// ordered integer -> the fp16 value as float
__device__ __forceinline__ float cos16_value(int32_t s) {
    if (s <= kCos16NaN) return __int_as_float(0xff800000);
    const uint32_t h = s >= 0 ? static_cast<uint32_t>(s) : (0x8000u | static_cast<uint32_t>(-1 - s));
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
}

}  // namespace b200
