// Several small exact indexes of one device searched with the same queries in ONE pass.
//
// The reference's multi-index search does not run one search per index: the blocks of all indexes
// are processed page by page by one distance operator and ONE top-k operator that carries
// (block -> index, label offset) tables (FR/ascendhost/src/index/IndexFlatL2Aicpu.cpp:307-444 driver,
// FR/ops/cpukernel/impl/topk_multisearch_cpu_kernel.cpp:316-430 segmented heap select,
// FR/ascenddaemon/impl/IndexFlat.cpp:813-847 tables); its API admits 10 000 indexes
// (FR/ascend/AscendMultiIndexSearch.cpp:38-41).  Here the bases of the member indexes are kept
// concatenated (every member starts on a tile boundary) beside a tile -> index table, and one
// distance GEMM walks all tiles with every query block: the epilogue sends the keys of a tile to
// the candidate rows of the tile's index.  Refinement, selection and emission then run over
// [index][query] rows, so the number of kernel launches does not depend on the number of indexes.
#pragma once
#include <stdint.h>

#include <vector>

#include "flat_index.h"

namespace b200 {

class FlatGroup {
public:
    explicit FlatGroup(int device) : device_(device) {}
    // Can these members (one device; same d / metric / dtype is the caller's contract) be searched
    // as one group with nq queries?  Small indexes only: every key of a member is written once.
    static bool eligible(const std::vector<FlatIndex*>& members, int64_t nq, int k);
    // xq: device pointer, float rows (kF32 / kF16 members) or int8 rows.  D / I: device pointers
    // [members][nq][k].  Work is queued on `stream`; returns after synchronising it.
    void search_device(const std::vector<FlatIndex*>& members, int64_t nq, const void* xq, int k, float* D, int64_t* I,
                       cudaStream_t stream);
    uint64_t launches() const { return launches_; }   // kernels launched by searches so far
    uint64_t rebuilds() const { return rebuilds_; }   // times the concatenation was (re)built

private:
    void refresh(const std::vector<FlatIndex*>& members, cudaStream_t stream);

    int device_;
    std::vector<const FlatIndex*> cur_;
    std::vector<uint64_t> cur_gen_;
    std::vector<int64_t> seg_start_;      // first position of every member in the concatenation (+ total at the end)
    int64_t total_rows_ = 0;              // padded rows of the concatenation
    uint32_t cap_ = 0;                    // largest padded member
    float max_norm_ = 0.f;
    int d_ = 0, metric_ = 0, dtype_ = 0, op_cols_ = 0, kind_ = 0, num_sms_ = 0;
    bool use_simt_ = false;
    CUtensorMap map_b_;
    DeviceBuffer xop_, x32_, norms_, labels_, seg_index_, seg_col0_, seg_end_;
    DeviceBuffer w_qop_, w_qnorm_, w_eps_, w_tau_, w_cand_, w_sel_, w_err_;
    uint64_t launches_ = 0, rebuilds_ = 0;
};

}  // namespace b200
