// Selection, refinement and merge kernels around the distance GEMM (the exact replacement of
// the reference's AICPU heap selection and host merges: FR/ops/cpukernel/impl/
// topk_flat_cpu_kernel.cpp:261-369, topk_multisearch_cpu_kernel.cpp:316-430,
// FR/ascend/impl/AscendIndexImpl.cpp:587-642, FR/ascend/utils/MergeResUtils.cpp:44-107).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// tau[q] = k-th smallest (1-based) of mins[q][0..n) as an ordered key; when eps != nullptr the
// key is widened in the float domain by 2*eps[q] (filter-and-refine slack).  n < k gives the
// "accept everything" threshold tau_all.
cudaError_t launch_kth_threshold(const uint32_t* mins, int stride, int n, int nq, int k, const float* eps,
                                 uint32_t tau_all, uint32_t* tau, cudaStream_t stream);

// Per query: the k smallest of cand[q][0..min(counts[q],cap)) in ascending order into
// out[q][0..k), padded with kCandInvalid.  counts == nullptr means every row holds n_fixed
// candidates.  overflow[q] is set to 1 when counts[q] > cap (the row's result is then not
// trustworthy and the caller re-runs it without a threshold).
cudaError_t launch_select_topk(const uint64_t* cand, const uint32_t* counts, uint32_t n_fixed, uint32_t cap, int nq,
                               int k, uint64_t* out, uint8_t* overflow, cudaStream_t stream);

// fp32 refinement: replaces the key of every candidate by the canonical fp32 distance
// (sequential fmaf over the dimension) computed from the fp32 rows; L2 -> distance,
// IP -> negated dot product.
// thresholded path, between two stretches of the full pass: tau[row] = min(tau[row], k-th smallest
// key among the row's candidates so far (+ 2 eps[row] where eps is given: approximate keys))
cudaError_t launch_tighten_tau(const uint64_t* cand, const uint32_t* counts, uint32_t cap, int nq, int k,
                               const float* eps, uint32_t* tau, cudaStream_t stream);
// fp32 index, thresholded path: removes candidates whose approximate key exceeds the k-th smallest
// approximate key of the row by more than 2 eps[row] (they cannot be in the exact top-k); the row
// is compacted and counts[row] updated
cudaError_t launch_prune_candidates(uint64_t* cand, uint32_t* counts, uint32_t cap, int nq, int k,
                                    const float* eps, cudaStream_t stream);
// q_mod > 0: candidate row r belongs to query r % q_mod (rows = [index][query] of a multi-index search)
cudaError_t launch_refine_f32(uint64_t* cand, const uint32_t* counts, uint32_t n_fixed, uint32_t cap, int nq, int d,
                              int metric, const float* xq, const float* xb, cudaStream_t stream, int q_mod = 0);

struct EmitArgs {
    const uint64_t* sel;     // [nq][k] sorted candidates
    int nq, k;
    int metric;
    int mode;                // 0: float key without query norm (add qnorm for L2); 1: refined float key; 2: int key
    const void* qnorm;       // float* (mode 0) or int32_t* (mode 2); L2 only
    const int64_t* labels;   // position -> label, or nullptr for identity
    float* D;                // [nq][ldk] row stride ldk
    int64_t* I;
    int ldk;
    const int32_t* qmap;     // optional: output row = qmap[q] (fallback re-runs scatter into place)
    int q_mod;               // > 0: row q uses the query norm of row q % q_mod (multi-index search)
};
cudaError_t launch_emit(const EmitArgs& e, cudaStream_t stream);

// Merge nsrc sorted lists per query.  Din/Iin: [nsrc][nq][k]; order by (distance ascending or
// score descending, label ascending); label < 0 marks padding.  src_stride_d / src_stride_i: elements
// between the blocks of consecutive sources (0: nq * k, i.e. dense arrays) -- lets the per-rank
// results of one packed all-gather (distances and labels of a rank side by side) be merged in place.
cudaError_t launch_merge_topk(int nsrc, int64_t nq, int k, int descending, const float* Din, const int64_t* Iin,
                              float* D, int64_t* I, cudaStream_t stream, int64_t src_stride_d = 0,
                              int64_t src_stride_i = 0);

// Query preparation.  fp32 queries -> bf16 operand copy (row-major or packed, see dist_gemm.cuh: a
// packed copy needs room for nq rounded up to kTileQ rows), squared norms and the filter slack
// eps[q] (see flat_index.cu); fp16 / int8 queries -> norms only.
cudaError_t launch_prep_queries_f32(const float* xq, int nq, int d, int metric, float base_max_norm, void* q_bf16,
                                    float* qnorm, float* eps, cudaStream_t stream);
cudaError_t launch_prep_queries_f16(const void* xq_f16, int nq, int d, float* qnorm, cudaStream_t stream);
cudaError_t launch_prep_queries_i8(const int8_t* xq, int nq, int d, int32_t* qnorm, cudaStream_t stream);

// Base preparation at add time.
// fp32 index: operand rows are d + kFoldCols bf16 wide, row-major or packed (see dist_gemm.cuh;
// the layout follows from d).  x_bf16 is the whole operand buffer, row0 the position of x's first row
// in it; norms points at the norms of the rows being added.
cudaError_t launch_base_prep_f32(const float* x, int64_t n, int d, int metric, void* x_bf16, int64_t row0,
                                 float* norms, float* max_norm_sq, cudaStream_t stream);
// threshold terms of the folded query rows, from the ordered-key thresholds tau[nq]
cudaError_t launch_fold_tau(const uint32_t* tau, const float* qnorm, float base_max_norm, int nq, int d, int metric,
                            void* q_bf16, cudaStream_t stream);
cudaError_t launch_base_prep_f16(const void* x_f16, int64_t n, int d, float* norms, cudaStream_t stream);
cudaError_t launch_base_prep_i8(const int8_t* x, int64_t n, int d, int32_t* norms, cudaStream_t stream);
cudaError_t launch_f32_to_f16(const float* x, int64_t count, void* out, cudaStream_t stream);
cudaError_t launch_f16_to_f32(const void* x, int64_t count, float* out, cudaStream_t stream);

// Input validation on the device.  *flag (an int the caller zeroed) gets bit 0 when x holds a NaN or
// an infinity, bit 1 when an assignment lies outside [0, bound): a non-finite vector has no nearest
// centroid, and an assignment of -1 must never reach a histogram or a gather.
cudaError_t launch_check_finite(const float* x, int64_t count, int* flag, cudaStream_t stream);
cudaError_t launch_check_range_i32(const int32_t* v, int64_t count, int32_t bound, int* flag, cudaStream_t stream);

// Small utilities.
cudaError_t launch_fill_u32(uint32_t* p, int64_t count, uint32_t value, cudaStream_t stream);
cudaError_t launch_iota_i64(int64_t* p, int64_t count, int64_t start, cudaStream_t stream);
// dst[i] = src[idx[i]] for rows of row_bytes bytes (row_bytes a multiple of 4).
cudaError_t launch_gather_rows(const void* src, const int32_t* idx, int n, int row_bytes, void* dst,
                               cudaStream_t stream);

}  // namespace b200
