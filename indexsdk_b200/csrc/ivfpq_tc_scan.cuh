// List-major IVFPQ filter scan on the tensor cores (residual encoding, d = 128, M = 16 x 8 bit).
//
// The table-lookup scan costs M shared-memory lookups per (query, code) pair.  Here every probed
// list is visited ONCE per batch: its codes are decoded to fp16 rows in shared memory (M 16-byte
// codeword lookups per code, not per pair) and multiplied on tcgen05 with the (query - centroid)
// rows of all queries that probe the list, split into two fp16 terms:
//     |q - c - r|^2 = |q - c|^2 + |r|^2 - 2 (q - c) . r
//                   = coarse distance + sum_m |cb[m][code_m]|^2 - 2 * accumulator.
// Every value is turned into a LOWER BOUND of the exact distance by subtracting the error bound of
// the fp16 product for its (query, list) pair, 2 (kTcErrRel |q - c| |r|max + kTcErrAbs (|q - c| +
// |r|max)) -- small for the near lists that hold the neighbours, larger for far lists whose
// distances are far above the threshold anyway.  A per-query threshold (the k'-th smallest upper
// bound over the codes of the query's nearest list, computed directly by one warp per query)
// decides in the epilogue which pairs are written out as candidates; a per-query selection
// keeps the k' smallest lower bounds, and the usual exact refinement + verification
// (ivfpq_index.cu) follows: a result is accepted when its k-th exact distance lies below the
// largest kept lower bound.  Replaces AscendcIvfpqSearchDistanceL2
// (FR/ops/ascendc/op_kernel/ascendc_ivfpq_search_distance_topk.h:95-810) for large batches.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int kTcDim = 128;          // vector dimension this path is built for
constexpr int kTcM = 16;             // sub-quantizers (8 dims each)
constexpr int kTcTile = 128;         // codes per accumulator tile (UMMA M)
constexpr int kTcMaxN = 64;          // queries per chunk (UMMA N, TMEM columns per accumulator)
constexpr int kTcMainThreads = 256;  // decode + epilogue warps (warp 0 lane 0 issues the MMAs)
constexpr int kTcThreads = kTcMainThreads + 96;   // + two warps that prepare the next (list, chunk) + the MMA warp
constexpr int kTcKeep = 32;          // k' of the filter
constexpr int kTcStageCap = 16384;   // candidates one CTA can stage per launch

// Relative and absolute error of the fp16 two-term product against (q - c) . r in exact arithmetic:
//   |err| <= kTcErrRel * |q - c| * |r| + kTcErrAbs * (|q - c| + |r|)
// (fp16 rounding of r: 2^-12 relative, 2^-25 absolute below the normal range; the query side keeps
// 22 bits; fp32 accumulation of 256 products: < 2^-15 relative.)
constexpr float kTcErrRel = 3.1e-4f;      // 2^-12 + 2^-14, rounded up
constexpr float kTcErrAbs = 7.0e-7f;      // 2^-25 * sqrt(128) * 2

struct TcScanArgs {
    const uint16_t* cb16;        // [16][256][8] fp16 bits of the codebooks
    const float* cbnorm;         // [16][256] squared norm of every codeword
    const float* xq;             // [nq][128]
    const float* centroids;      // [nlist][128]
    const float* cD;             // [nq][nprobe] coarse distances (|q - c|^2)
    int nprobe, nlist;
    int64_t nq;
    const int32_t* sorted_pair;  // [nq * nprobe] pair index q * nprobe + p, ordered by list
    const int32_t* first;        // [nlist] first entry of the list's pairs in sorted_pair
    const int32_t* last;         // [nlist] one past its last entry (first == last: not probed)
    const int32_t* order;        // [nlist] lists in the order they are handed out (most queries first), or null
    const int64_t* offsets;      // [nlist + 1] first slot of every list
    const int64_t* lens;         // [nlist] vectors per list
    const uint8_t* codes;        // 16 bytes per slot, rotated by (slot mod 16)
    const float* tau;            // [nq] widened threshold; -inf: the query takes the exact path
    float cb_bound;              // bound on |r| (sqrt of the summed largest codeword norms)
    float* cand_d;               // [nq][cap] approximate distances of the candidates
    uint32_t* cand_p;            // [nq][cap] their slots
    unsigned int* cand_n;        // [nq] candidates found (may exceed cap: overflow)
    int cap;
    uint4* stage;                // [CTAs][stage_cap] (query, slot, distance bits, -) as the epilogues find them
    unsigned int* stage_n;       // [CTAs] entries each CTA produced (beyond stage_cap they went straight to cand_*)
    int stage_cap;
    unsigned int* work;          // next list to hand out (zeroed before the launch)
    unsigned long long* scanned; // += (query, code) pairs visited
    unsigned int* err;           // bit 0: a bounded wait ran out
    unsigned long long* prof;    // optional [8]: cycles of thread 0 per phase, summed over CTAs (development aid)
};

// keys for the (list, pair) sort: key = list id, or nlist for an empty probe slot
cudaError_t launch_tc_keys(const int64_t* cI, int64_t npairs, int nlist, int32_t* keys, int32_t* vals,
                           cudaStream_t st);
// first / last entry of every list in the sorted keys
cudaError_t launch_tc_bounds(const int32_t* sorted_keys, int64_t npairs, int nlist, int32_t* first, int32_t* last,
                             cudaStream_t st);
// tau[q]: an upper bound of the k'-th smallest value the scan will produce for the query, from
// fp16-decoded distances to the codes of its nearest list(s); -inf: exact path (fp16 range)
cudaError_t launch_tc_head_tau(const TcScanArgs& a, const int64_t* cI, float err_rel, float t2_bound, float* tau,
                               cudaStream_t st);
// sort keys that put the lists with the most probing queries first (keys[l] = -queries, vals[l] = l)
cudaError_t launch_tc_order_keys(const int32_t* first, const int32_t* last, int nlist, int32_t* keys, int32_t* vals,
                                 cudaStream_t st);
cudaError_t launch_tc_scan(const TcScanArgs& a, int num_sms, cudaStream_t st);
// per query: the kTcKeep best candidates -> fd / fp ([nq][32]) and fth ([nq])
cudaError_t launch_tc_select(const TcScanArgs& a, float* fd, uint32_t* fp, float* fth, cudaStream_t st);
// fp16 copy of the codebooks ([M][256][dsub] floats -> the same order in fp16)
cudaError_t launch_tc_cb16(const float* cb, int64_t n, uint16_t* out, cudaStream_t st);

}  // namespace b200
