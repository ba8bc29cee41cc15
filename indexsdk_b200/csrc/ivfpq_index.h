// Per-device IVFPQ index (counterpart of the reference's ascend::IndexIVFPQ three-stage search,
// FR/ascenddaemon/impl/IndexIVFPQ.cpp:2104-2411, and of the host-side assignment / PQ encoding
// in FR/ascend/impl/AscendIndexIVFPQImpl.cpp:603-805,879-921).
//
// Layout in HBM: inverted lists are one CSR structure -- list_offsets[nlist + 1], codes[ntotal][M],
// ids[ntotal], and, for residual encoding, one float per vector (the list-dependent part of the
// distance, see ivfpq_index.cu).  When M is a multiple of 16 the 16 code bytes of each 16-byte
// group are stored rotated by (position mod 16): stored[s] = code[(s + position) & 15].  The scan
// kernel walks the sub-quantizers of a vector in that rotated order, which makes its shared-memory
// table reads bank-conflict free; everything that leaves the index (get_list) is un-rotated.
#pragma once
#include <stdint.h>

#include <memory>
#include <vector>

#include "flat_index.h"

namespace b200 {

class IvfpqIndex {
public:
    IvfpqIndex(int d, int nlist, int M, int nbits, bool by_residual, int device);
    ~IvfpqIndex();

    int d() const { return d_; }
    int nlist() const { return nlist_; }
    int M() const { return M_; }
    bool by_residual() const { return by_residual_; }
    int device() const { return device_; }
    int64_t ntotal() const { return n_; }
    int nprobe() const { return nprobe_; }
    void set_nprobe(int p) { nprobe_ = p; }
    bool is_trained() const { return has_centroids_ && has_codebooks_; }
    SearchStats& stats() { return stats_; }
    SearchStats& coarse_stats() { return coarse_->stats(); }
    void set_timing(bool on) {
        timer_.enable(on);
        coarse_->timer().enable(on);
    }
    cudaStream_t stream() const { return coarse_->stream(); }

    void set_centroids(const float* centroids_host);  // [nlist][d]
    void set_codebooks(const float* codebooks_host);  // [M][256][d / M]
    // Trains coarse centroids (k-means, k = nlist) and the M sub-space codebooks (k-means, k = 256, on
    // the residuals to the assigned centroid when the index encodes residuals) on the device.
    void train(int64_t n, const float* x_host, int niter, uint64_t seed);
    void get_centroids(float* out_host) const;
    void get_codebooks(float* out_host) const;

    // Assign + encode on the GPU, then merge into the lists.  x: host or device floats.
    void add(int64_t n, const float* x, const int64_t* ids_host, bool x_on_device);
    // Pre-encoded vectors (list ids, codes, ids on the host), e.g. from a CPU index.
    void add_codes(int64_t n, const int32_t* list_no, const uint8_t* codes, const int64_t* ids);
    void reset();
    int64_t remove_ids(int64_t n, const int64_t* ids);
    int64_t list_length(int list) const;
    void get_list(int list, uint8_t* codes_host, int64_t* ids_host) const;

    void search_device(int64_t nq, const float* xq, int k, float* D, int64_t* I);
    // the two halves of a search: probe selection (k = nprobe on the coarse quantizer), and the
    // code scan + refinement given the probes (device pointers, [nq][nprobe])
    void coarse_device(int64_t nq, const float* xq, float* cD, int64_t* cI);
    void search_preassigned_device(int64_t nq, const float* xq, int k, const float* cD, const int64_t* cI, float* D,
                                   int64_t* I);
    void search_host(int64_t nq, const float* xq, int k, float* D, int64_t* I);

private:
    void merge_new(int64_t n, const int32_t* list_no_dev, const uint8_t* codes_dev, const float* t2_dev,
                   const int64_t* ids_dev);
    void compute_t2(int64_t n, const int32_t* list_no_dev, const uint8_t* codes_dev, float* t2_dev);
    void unrotate_host(uint8_t* codes, int64_t first_pos, int64_t n) const;

    int d_, nlist_, M_, dsub_, device_;
    bool by_residual_;
    bool rotated_;                        // M % 16 == 0: rotated code storage + conflict-free scan
    int nprobe_ = 1;
    int64_t n_ = 0;                       // vectors stored
    int64_t n_pad_ = 0;                   // storage slots in use: every list padded to a multiple of 32
    void search_stages(int64_t nq, const float* xq, int k, float* D, int64_t* I, const float* pre_cD,
                       const int64_t* pre_cI);
    bool has_centroids_ = false, has_codebooks_ = false;
    bool no_persist_ = false;
    bool tc_scan_ = false;                // list-major tensor-core filter scan (large batches, residual encoding)
    bool tc_cb_ok_ = false;               // codebook entries inside the fp16 range
    int num_sms_ = 0;
    float cb_norm_bound_ = 0.f;           // sqrt(sum_m max_j |cb[m][j]|^2), for the filter's error bound
    bool force_exact_ = false;            // B200IDX_IVFPQ_EXACT=1: always use the exact scan kernels

    std::unique_ptr<FlatIndex> coarse_;   // nlist centroids, fp32, L2
    DeviceBuffer codebooks_;              // [M][256][dsub] float
    DeviceBuffer codebooks_t_;            // the same regrouped [M / 16][256][16][dsub] (M % 16 == 0)
    DeviceBuffer cbnorm_;                 // [M][256] float: canonical squared norm of each codeword
    DeviceBuffer cb16_;                   // [M][256][dsub] fp16 bits of the codebooks (tensor-core scan)
    DeviceBuffer offsets_;                // int64 [nlist + 1] first slot of every list (multiples of 32)
    DeviceBuffer lens_;                   // int64 [nlist + 1] vectors per list
    std::vector<int64_t> offsets_host_, lens_host_;
    DeviceBuffer codes_, ids_, t2_;
    // scratch
    DeviceBuffer w_work_, w_cD_, w_cI_, w_fd_, w_fp_, w_fth_, w_flag_, w_qlist_, w_q_, w_D_, w_I_, w_assign_D_,
        w_assign_I_, w_list_, w_codes_, w_t2_, w_ids_, w_x_, w_tmp_, w_vflag_, w_cpos_, w_ccount_;
    DeviceBuffer w_tc_keys_, w_tc_vals_, w_tc_keys2_, w_tc_vals2_, w_tc_first_, w_tc_last_, w_tc_cI0_, w_tc_cD0_,
        w_tc_fd0_, w_tc_fp0_, w_tc_fth0_, w_tc_tau_, w_tc_cd_, w_tc_cp_, w_tc_cn_, w_tc_sort_, w_tc_err_, w_tc_prof_, w_tc_stage_, w_tc_stage_n_, w_tc_okeys_, w_tc_osort_;
    PinnedBuffer h_flag_;
    SearchStats stats_;
    StageTimer timer_;
};

}  // namespace b200
