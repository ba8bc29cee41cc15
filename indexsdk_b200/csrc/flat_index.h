// Per-device exact index (the counterpart of the reference's per-device IndexFlat /
// IndexInt8Flat objects and their metric-specific search loops:
// FR/ascenddaemon/impl/IndexFlat.cpp:82-125,551-562, FR/ascendhost/src/index/
// IndexFlatL2Aicpu.cpp:157-305, FR/ascenddaemon/impl/IndexInt8Flat.cpp:523-692).
// Storage is one contiguous row-major array per dtype, grown geometrically; there are no
// 262144-row blocks and no fractal layouts.
#pragma once
#include "dist_gemm.cuh"
#include <cuda.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "common.cuh"
#include "device_mem.h"

namespace b200 {

// Stages timed with CUDA events on the index's stream when timing is enabled.
enum Stage : int {
    kStageSample = 0,   // query prep + sample GEMM pass + threshold selection
    kStageFullGemm = 1, // full GEMM pass with the append epilogue
    kStageRefine = 2,   // fp32 re-computation of candidates
    kStageSelect = 3,   // exact top-k of candidates + result emission
    kStageCoarse = 4,   // IVFPQ: whole coarse-quantizer search
    kStageLut = 5,      // IVFPQ: lookup tables
    kStageScan = 6,     // IVFPQ: code scan
    kStageMerge = 7,    // IVFPQ: merge of probe splits
    kNumStages = 8
};

struct SearchStats {
    double stage_ms[kNumStages] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint64_t stage_launches[kNumStages] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint64_t searches = 0;
    uint64_t queries = 0;
    uint64_t fallback_queries = 0;   // queries re-run without a threshold after a candidate overflow (IVFPQ: exact re-scan)
    uint64_t second_pass_queries = 0;   // IVFPQ: queries that took the second (fixed-threshold) filter pass
    uint64_t gemm_launches = 0;
    uint64_t kernel_launches = 0;    // every kernel of this library launched by searches
    uint64_t scan_codes = 0;         // IVFPQ: codes visited
};

// Records begin/end events per stage; elapsed times are folded into SearchStats after the
// stream has been synchronised.  Disabled (no events recorded) unless enable(true) was called.
class StageTimer {
public:
    ~StageTimer() {
        for (auto& r : recs_) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
        for (auto& r : pool_) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
    }
    void enable(bool on) { on_ = on; }
    bool enabled() const { return on_; }
    void begin(int stage, cudaStream_t st) {
        if (!on_) return;
        Rec r;
        if (!pool_.empty()) { r = pool_.back(); pool_.pop_back(); }
        else { cudaEventCreate(&r.a); cudaEventCreate(&r.b); }
        r.stage = stage;
        cudaEventRecord(r.a, st);
        recs_.push_back(r);
        open_ = static_cast<int>(recs_.size()) - 1;
    }
    void end(cudaStream_t st) {
        if (!on_ || open_ < 0) return;
        cudaEventRecord(recs_[open_].b, st);
        open_ = -1;
    }
    // call only after the stream is idle
    void collect(SearchStats& s) {
        for (auto& r : recs_) {
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
                s.stage_ms[r.stage] += ms;
                s.stage_launches[r.stage] += 1;
            } else {
                cudaGetLastError();
            }
            pool_.push_back(r);
        }
        recs_.clear();
    }

private:
    struct Rec { cudaEvent_t a = nullptr, b = nullptr; int stage = 0; };
    std::vector<Rec> recs_, pool_;
    bool on_ = false;
    int open_ = -1;
};

class FlatIndex {
public:
    // dtype: kF32 (fp32 rows + bf16 filter copy, results refined in fp32), kF16 (fp16 rows,
    // fp32 accumulation, results are the GEMM's), kI8 (int8 rows, exact int32).
    FlatIndex(int d, int metric, int dtype, int device);
    ~FlatIndex();

    int d() const { return d_; }
    int metric() const { return metric_; }
    int dtype() const { return dtype_; }
    int device() const { return device_; }
    int64_t ntotal() const { return n_; }
    // changes whenever the stored rows change (add / reset / remove_ids): lets a cached copy notice
    uint64_t generation() const { return generation_; }
    cudaStream_t stream() const { return stream_; }
    SearchStats& stats() { return stats_; }
    StageTimer& timer() { return timer_; }

    // x: host or device pointer in the index's input dtype (float for kF32 and kF16 unless
    // x_is_f16, int8 for kI8).  ids: host pointer or nullptr (labels = ntotal + i).
    void add(int64_t n, const void* x, bool x_is_f16, const int64_t* ids, bool x_on_device);
    void reset();
    int64_t remove_ids(int64_t n, const int64_t* ids);
    // Copies rows [offset, offset + n) to a host buffer: float for kF32, fp16 bits for kF16,
    // int8 for kI8.
    void get_base(int64_t offset, int64_t n, void* out_host) const;
    void get_labels(int64_t offset, int64_t n, int64_t* out_host) const;

    // Device-resident search.  xq: device pointer, rows of float (kF32, kF16 unless q_is_f16) or
    // int8.  D/I: device pointers with row stride ldk >= k.  Work is enqueued on stream();
    // the call synchronises that stream before returning (candidate-overflow check).
    void search_device(int64_t nq, const void* xq, bool q_is_f16, int k, float* D, int64_t* I, int ldk);
    // Host-pointer search: pinned staging, H2D, search_device, D2H.
    void search_host(int64_t nq, const void* xq, bool q_is_f16, int k, float* D, int64_t* I);
    // mask: nq rows of ceil(ntotal / 8) bytes, bit (i % 8) of byte i / 8 = 1 lets base position i take part
    void search_host_masked(int64_t nq, const void* xq, bool q_is_f16, int k, const uint8_t* mask, float* D, int64_t* I);

    // Raw access for composite indexes (IVFPQ coarse quantizer).
    const float* rows_f32() const { return x32_.as<float>(); }

    // Read-only view of the stored arrays (device pointers) for entry points that bring their
    // own scratch memory.
    struct RawView {
        const void* operand;     // bf16 (kF32), fp16 (kF16) or int8 (kI8) rows
        const float* rows_f32;   // kF32 only
        const void* norms;       // float or int32 squared norms
        const int64_t* labels;
        int64_t n;
        float max_norm;
        int num_sms;
        bool use_simt;
    };
    RawView raw_view() const {
        return RawView{xop_.get(), x32_.as<float>(), norms_.get(), labels_.as<int64_t>(), n_, max_norm_, num_sms_,
                       use_simt_};
    }
    int gemm_kind_public() const { return gemm_kind(); }

private:
    struct Plan {
        bool sampled;
        int burst;
        int s_tiles;
        uint32_t cap;
    };
    Plan make_plan(int k, int64_t nq) const;
    void run_page(int nq, const void* xq_raw, const void* xq_op, int k, float* D, int64_t* I, int ldk,
                  const int32_t* qmap_dev, bool force_full);
    void reserve(int64_t n);
    size_t in_elem_bytes() const { return dtype_ == kI8 ? 1 : (dtype_ == kF16 ? 2 : 4); }
    size_t op_elem_bytes() const { return dtype_ == kI8 ? 1 : 2; }
  public:
    // elements per GEMM operand row: fp32 indexes carry the folded norm / threshold columns
    int op_cols() const { return dtype_ == kF32 ? d_ + kFoldCols : d_; }
  private:
    int gemm_kind() const;

    int d_, metric_, dtype_, device_;
    int num_sms_ = 0;
    bool use_simt_ = false;
    int64_t n_ = 0, cap_rows_ = 0;
    // Changes with every mutation; drawn from one process-wide counter, so that no two states of any
    // two indexes share a value (a cache keyed on (address, generation) must not mistake a new index
    // that the allocator placed where a destroyed one lived for the old one).
    static uint64_t next_generation();
    uint64_t generation_ = next_generation();
    int64_t next_auto_id_ = 0;
    cudaStream_t stream_ = nullptr;

    DeviceBuffer x32_;     // kF32: fp32 rows
    // filter of the search in progress (device, one row of mask_stride_ words per query of the current
    // host page; nullptr = none) and the rows of the page run_page is working on
    const uint32_t* mask_dev_ = nullptr;
    const uint32_t* mask_cur_ = nullptr;
    int64_t mask_stride_ = 0;
    DeviceBuffer w_mask_, w_fb_mask_;
    DeviceBuffer xop_;     // GEMM operand rows: bf16 (kF32), fp16 (kF16), int8 (kI8)
    DeviceBuffer norms_;   // float (kF32/kF16) or int32 (kI8), padded to a multiple of 256 rows
    DeviceBuffer labels_;  // int64 per row
    DeviceBuffer maxnorm_; // float: max squared base norm (kF32)
    float max_norm_ = 0.f;
    bool map_b_valid_ = false;
    CUtensorMap map_b_;

    // scratch
    DeviceBuffer w_qop_, w_qraw_, w_qnorm_, w_eps_, w_mins_, w_tau_, w_cand_, w_counts_, w_sel_, w_over_, w_qmap_,
        w_err_, w_stage_in_, w_stage_D_, w_stage_I_, w_fb_q_, w_fb_qop_, w_prof_;
    bool prof_ = false;
    PinnedBuffer h_over_, h_in_, h_D_, h_I_;
    SearchStats stats_;
    StageTimer timer_;
};

}  // namespace b200
