// Distance GEMM with a fused selection epilogue (replaces the reference's distance operators
// DistanceComputeFlatMin64 / DistanceFlatL2 / DistanceFlatIP / DistanceInt8* together with
// the flag-polling AICPU TopkFlat: FR/ops/ascendc/op_kernel/distance_flat_l2.cpp:53-666,
// FR/ops/cpukernel/impl/topk_flat_cpu_kernel.cpp:36-371).  The [nq x N] distance matrix is
// never written: each 128 x 256 accumulator tile is consumed out of TMEM by one of two
// epilogues,
//   kModeBurstMin : per query row, the minimum key of every burst of 32 (or 8) base rows
//   kModeAppend   : per query row, every (key, position) whose key <= tau[row]
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int kTileQ = 128;   // query rows per accumulator tile (TMEM lanes)
constexpr int kTileB = 256;   // base rows per accumulator tile (TMEM columns)
constexpr int kChunkBytes = 128;  // K extent of one pipeline stage, in bytes (one 128-byte swizzle row)

enum GemmKind : int { kKindF16 = 0, kKindBF16 = 1, kKindI8 = 2 };

// bf16 operands are "folded": every row carries kFoldCols extra K columns so that the tensor core
// itself adds the base norm and the query's threshold to the dot product,
//   base row  y : [ y (d) | h0 h1 h2 | 1 1 1 | 0 .. ]   h0 + h1 + h2 = -|y|^2 / 2   (0 for inner product)
//   query row q : [ q (d) | 1  1  1  | t0 t1 t2 | 0 .. ]  t0 + t1 + t2 = tau / 2     (tau for inner product;
//                                                          0 while no threshold is known)
// each value split into three bf16 terms (24 significant bits).  The accumulator then holds
// D = q.y - |y|^2/2 + tau/2 = (tau - key) / 2 with key = |y|^2 - 2 q.y, so the epilogue reads no
// norms: "key <= tau" is "D >= 0", and min(key) over a burst is -2 max(D).
constexpr int kFoldCols = 16;
enum GemmMode : int { kModeBurstMin = 0, kModeAppend = 1 };

// Packed operands.  Folded bf16 operands of at most kPackedMaxCols columns (fp32 indexes up to
// d = 144, the IVFPQ coarse quantizers) are not kept as rows but as the shared-memory image the
// tensor core reads: per tile of R rows (R = kTileQ for queries, kTileB for base rows) a block of
// R * cols bf16 in the UMMA's K-major no-swizzle layout -- "core matrices" of 8 rows x 8 columns
// (128 contiguous bytes, a row's 8 values = 16 bytes), the core matrices of an 8-row group side by
// side along K, the groups one after the other:
//   element (r, k) of the tile sits at bf16 index ((r / 8) * (cols / 8) + k / 8) * 64 + (r % 8) * 8 + k % 8.
// A tile is then ONE contiguous copy into shared memory (cp.async.bulk), K = 144 needs 72 KB per
// base tile instead of three 32 KB swizzle-128 boxes (the third three quarters zero fill), and an
// item of the kernel's work list is one hand-off between its roles instead of three.
constexpr int kPackedMaxCols = 160;
__host__ __device__ constexpr bool packed_operands(int kind, int cols) {
    return kind == kKindBF16 && cols <= kPackedMaxCols && cols % 16 == 0;
}
__host__ __device__ __forceinline__ int64_t packed_elem(int64_t r, int k, int cols, int rows_per_tile) {
    const int64_t tile = r / rows_per_tile;
    const int rr = static_cast<int>(r - tile * rows_per_tile);
    return tile * rows_per_tile * cols + static_cast<int64_t>((rr >> 3) * (cols >> 3) + (k >> 3)) * 64 + (rr & 7) * 8 +
           (k & 7);
}
// bf16 index of (r, k) in an operand buffer, packed or row-major
__host__ __device__ __forceinline__ int64_t operand_elem(bool packed, int64_t r, int k, int cols, int rows_per_tile) {
    return packed ? packed_elem(r, k, cols, rows_per_tile) : r * cols + k;
}

struct GemmArgs {
    const void* A;        // queries [nq, d] in the operand dtype (SIMT variant, packed operands)
    const void* B;        // base    [N, d]  in the operand dtype (SIMT variant, packed operands)
    int d;                // elements per operand row = K extent (bf16 kind: includes the 16 folded columns)
    int nq;
    int64_t N;
    int n_tiles_total;    // ceil(N / kTileB)
    int n_tiles_sel;      // tiles visited by this pass
    int tile_first;       // >= 0: tiles tile_first .. tile_first + n_tiles_sel - 1;
                          // -1: n_tiles_sel tiles spread evenly, tile(i) = i * n_tiles_total / n_tiles_sel
    int metric;           // kMetricIP / kMetricL2 / kMetricCos (i8 only)
    const void* bnorm;    // float* (f16/bf16 kinds) or int32_t* (i8): squared norm per base row, L2 and cosine
    const int32_t* qnorm_i32;   // kMetricCos: squared norm per query
    // kModeBurstMin
    uint32_t* mins;       // [nq][mins_stride] ordered keys
    int mins_stride;      // n_tiles_sel * (kTileB / burst)
    // kModeAppend
    const uint32_t* tau;  // [nq] inclusive threshold on the ordered key
    uint64_t* cand;       // [nq][cap] packed (ordered key, position); reserved but unused slots hold "invalid"
    uint32_t* counts;     // [nq] slots reserved (blocks of 8 per thread and query block run): >= candidates
    uint32_t cap;
    int direct;           // 1: slot = position (cap >= N, no atomics); 0: slot = atomic counter
    // optional per-(query, base row) filter: bit (row % 32) of qmask[q * qmask_stride + row / 32] = 1
    // lets the row take part (nullptr: every row does)
    const uint32_t* qmask;
    int64_t qmask_stride;
    // optional segmented base: the concatenated bases of several indexes that are searched with the
    // same queries in ONE pass (multi-index search).  A tile belongs to exactly one index (segments
    // start on tile boundaries); per tile:
    //   seg_index: which index; the candidates of (index i, query q) go to row
    //              (i - seg_first) * nq + q of cand / tau (direct mode only)
    //   seg_col0 : position of the index's first base row in the concatenated base (the slot of a
    //              candidate is its position minus this)
    //   seg_end  : position one past the index's last real base row
    const int32_t* seg_index;
    int seg_first;        // index of the first member this pass covers
    const int64_t* seg_col0;
    const int64_t* seg_end;
    int* err;             // device error word
    // optional phase profile (nullptr = off): 8 counters of SM cycles summed over CTAs
    //   0 producer wait-empty   1 mma wait-acc-empty   2 mma wait-full   3 epilogue wait-acc-full
    //   4 epilogue chunks       5 epilogue flush       6 items           7 total kernel cycles (per CTA, summed)
    unsigned long long* prof;
    unsigned long long* trace;   // development builds only: [6][64] clock64 stamps of CTA 0's first 64 items
    int dbg;              // development builds only: 1 skip the epilogue's chunk work, 2 also its TMEM loads, 4 skip the UMMAs
    // filled in by launch_dist_gemm (tcgen05 variant): shared-memory plan
    int packed;           // 1: packed operands (see packed_operands), read through A / B with contiguous copies
    int a_resident;       // 1: the query tile stays in shared memory for a whole query block
    int n_stages;         // ring stages (base chunks, or query + base chunks when not resident)
    int aligned_ranges;   // 1: CTA = (query block, even share of the tiles); 0: equal cuts of the item list
};

struct GemmLaunch {
    int kind;     // GemmKind
    int mode;     // GemmMode
    int burst;    // 32 or 8 (kModeBurstMin)
    int simt;     // 1: plain CUDA-core variant (cross-check), 0: tcgen05 pipeline
    int num_sms;
};

// Operands for the tcgen05 variant: row-major [rows, d] tensors with 128-byte swizzled boxes.
cudaError_t launch_dist_gemm(const GemmLaunch& L, const GemmArgs& a, const CUtensorMap* mapA, const CUtensorMap* mapB,
                             cudaStream_t stream);

// Encodes a 2-D row-major tensor map with a {128 bytes, box_rows} box and SWIZZLE_128B.
// Returns 0 on success.
int encode_operand_map(CUtensorMap* out, int kind, const void* base, int64_t rows, int d, int box_rows);

}  // namespace b200
