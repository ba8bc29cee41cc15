// tcgen05 / TMEM / TMA distance GEMM with fused selection epilogues, plus a plain CUDA-core
// variant that shares the epilogue code and serves as an on-device cross-check.
//
// Pipeline of the tcgen05 variant (one persistent CTA per SM, 192 threads):
//   warp 0 (one lane)  : TMA producer.  Per K chunk of 128 bytes: query box 128 x 128 B and base
//                        box 256 x 128 B into a 4-stage ring of 48 KB stages (SWIZZLE_128B).
//   warp 1 (one lane)  : issues tcgen05.mma 128 x 256 x (32 bytes of K) from shared-memory
//                        descriptors into one of two 256-column TMEM accumulators; commits free
//                        the stage (per chunk) and publish the accumulator (per tile).
//   warps 2-5          : epilogue.  Thread = query row = TMEM lane; reads 32 columns at a time
//                        with tcgen05.ld and applies the norm-add and the selection predicate.
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
constexpr int kGemmThreads = 192;
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
};
template <>
struct KeyOps<int32_t> {
    using Norm = int32_t;
    static __device__ __forceinline__ int32_t from_bits(uint32_t r) { return static_cast<int32_t>(r); }
    static __device__ __forceinline__ int32_t key(int32_t acc, int32_t bn, bool l2) { return l2 ? bn - 2 * acc : -acc; }
    static __device__ __forceinline__ uint32_t ord(int32_t k) { return int_to_ord(k); }
    static __device__ __forceinline__ int32_t tau(uint32_t o) { return ord_to_int(o); }
    static __device__ __forceinline__ int32_t worst() { return 0x7fffffff; }
};

// Consumes 32 consecutive accumulator columns of one query row.
//   r       : raw 32-bit accumulators (float or int32 bit patterns)
//   q       : query row (caller guarantees q < nq)
//   col0    : base position of r[0]; nvalid: how many of the 32 columns are real base rows
//   bslot   : first burst slot of this chunk inside the row's mins[] segment (kModeBurstMin)
template <typename AccT, int MODE, int BURST>
__device__ __forceinline__ void epilogue_chunk(const GemmArgs& a, const uint32_t (&r)[32], int q, int64_t col0,
                                               int nvalid, int bslot, AccT tau) {
    using K = KeyOps<AccT>;
    using Norm = typename K::Norm;
    const bool l2 = a.metric == kMetricL2;
    Norm bn[32];
    if (l2) {
        const uint4* p = reinterpret_cast<const uint4*>(static_cast<const Norm*>(a.bnorm) + col0);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint4 v = __ldg(p + j);
            bn[4 * j + 0] = K::from_bits(v.x);
            bn[4 * j + 1] = K::from_bits(v.y);
            bn[4 * j + 2] = K::from_bits(v.z);
            bn[4 * j + 3] = K::from_bits(v.w);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) bn[j] = Norm(0);
    }
    if (MODE == kModeBurstMin) {
        constexpr int NB = 32 / BURST;
        uint32_t out[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            AccT m = K::worst();
#pragma unroll
            for (int j = 0; j < BURST; ++j) {
                const int c = b * BURST + j;
                AccT key = K::key(K::from_bits(r[c]), bn[c], l2);
                if (c < nvalid) m = key < m ? key : m;
            }
            out[b] = K::ord(m);
        }
        uint32_t* dst = a.mins + static_cast<int64_t>(q) * a.mins_stride + bslot;
#pragma unroll
        for (int b = 0; b < NB; ++b) dst[b] = out[b];
    } else {
        uint64_t* crow = a.cand + static_cast<int64_t>(q) * a.cap;
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            AccT key = K::key(K::from_bits(r[c]), bn[c], l2);
            if (key <= tau && c < nvalid) {
                const uint32_t pos = static_cast<uint32_t>(col0 + c);
                uint32_t slot = a.direct ? pos : atomicAdd(a.counts + q, 1u);
                if (slot < a.cap) crow[slot] = pack_cand(K::ord(key), pos);
            }
        }
    }
}

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
    constexpr uint32_t kIdesc = KIND == kKindI8 ? ptx::umma_idesc(2, 1, kTileQ, kTileB)
                                                : ptx::umma_idesc(1, KIND == kKindBF16 ? 1 : 0, kTileQ, kTileB);

    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[kStages];
    __shared__ uint64_t bar_empty[kStages];
    __shared__ uint64_t bar_acc_full[2];
    __shared__ uint64_t bar_acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

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
            ptx::mbar_init(&bar_acc_empty[b], 4);
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
            for (int64_t item = blockIdx.x; item < total && ok; item += gridDim.x) {
                const int qb = static_cast<int>(item % n_qb);
                const int tile = tile_of(a, static_cast<int>(item / n_qb));
                for (int kc = 0; kc < nkc; ++kc, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1u;
                    if (!ptx::mbar_wait_bounded(&bar_empty[s], ph ^ 1u, &abort_flag)) { ok = false; break; }
                    ptx::mbar_expect_tx(&bar_full[s], kStageBytes);
                    uint8_t* sa = smem + s * kStageBytes;
                    ptx::tma_load_2d(sa, &mapA, &bar_full[s], kc * kChunkElems, qb * kTileQ);
                    ptx::tma_load_2d(sa + kStageABytes, &mapB, &bar_full[s], kc * kChunkElems, tile * kTileB);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0, t = 0;
            bool ok = true;
            for (int64_t item = blockIdx.x; item < total && ok; item += gridDim.x, ++t) {
                const uint32_t ab = t & 1u;
                const uint32_t aph = (t >> 1) & 1u;
                if (!ptx::mbar_wait_bounded(&bar_acc_empty[ab], aph ^ 1u, &abort_flag)) { ok = false; break; }
                ptx::tc_fence_after();
                const uint32_t tacc = tmem_base + ab * kTileB;
                for (int kc = 0; kc < nkc; ++kc, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1u;
                    if (!ptx::mbar_wait_bounded(&bar_full[s], ph, &abort_flag)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint32_t sa = ptx::smem_u32(smem + s * kStageBytes);
                    const uint32_t sb = sa + kStageABytes;
#pragma unroll
                    for (int ks = 0; ks < kChunkBytes / 32; ++ks) {
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
        }
    } else {
        const int quarter = warp & 3;  // TMEM lane quarter this warp may read
        const int row_in_tile = quarter * 32 + lane;
        uint32_t t = 0;
        bool ok = true;
        for (int64_t item = blockIdx.x; item < total && ok; item += gridDim.x, ++t) {
            const int qb = static_cast<int>(item % n_qb);
            const int sel = static_cast<int>(item / n_qb);
            const int tile = tile_of(a, sel);
            const uint32_t ab = t & 1u;
            const uint32_t aph = (t >> 1) & 1u;
            const int q = qb * kTileQ + row_in_tile;
            const bool row_ok = q < a.nq;
            AccT tau = AccT(0);
            if (MODE == kModeAppend && row_ok) tau = KeyOps<AccT>::tau(__ldg(a.tau + q));
            if (!ptx::mbar_wait_bounded(&bar_acc_full[ab], aph, &abort_flag)) { ok = false; break; }
            ptx::tc_fence_after();
            const uint32_t tacc = tmem_base + ab * kTileB + (static_cast<uint32_t>(quarter * 32) << 16);
            const int64_t tile_col0 = static_cast<int64_t>(tile) * kTileB;
#pragma unroll 1
            for (int c = 0; c < kTileB / 32; ++c) {
                uint32_t r[32];
                ptx::tmem_ld_32x32(tacc + c * 32, r);
                ptx::tmem_ld_wait();
                const int64_t col0 = tile_col0 + c * 32;
                int64_t rem = a.N - col0;
                const int nvalid = rem >= 32 ? 32 : (rem > 0 ? static_cast<int>(rem) : 0);
                if (row_ok && (nvalid > 0 || MODE == kModeBurstMin)) {
                    const int bslot = sel * (kTileB / BURST) + c * (32 / BURST);
                    epilogue_chunk<AccT, MODE, BURST>(a, r, q, col0, nvalid, bslot, tau);
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&bar_acc_empty[ab]);
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
    const int n_qb = (a.nq + kTileQ - 1) / kTileQ;
    const int64_t total = static_cast<int64_t>(n_qb) * a.n_tiles_sel;
    for (int64_t item = blockIdx.x; item < total; item += gridDim.x) {
        const int qb = static_cast<int>(item % n_qb);
        const int sel = static_cast<int>(item / n_qb);
        const int tile = tile_of(a, sel);
        const int q = qb * kTileQ + threadIdx.x;
        const bool row_ok = q < a.nq;
        const int qc = row_ok ? q : a.nq - 1;
        AccT tau = AccT(0);
        if (MODE == kModeAppend && row_ok) tau = KeyOps<AccT>::tau(__ldg(a.tau + q));
        for (int c = 0; c < kTileB / 32; ++c) {
            const int64_t col0 = static_cast<int64_t>(tile) * kTileB + c * 32;
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
            if (row_ok && (nvalid > 0 || MODE == kModeBurstMin)) {
                const int bslot = sel * (kTileB / BURST) + c * (32 / BURST);
                epilogue_chunk<AccT, MODE, BURST>(a, r, q, col0, nvalid, bslot, tau);
            }
        }
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
