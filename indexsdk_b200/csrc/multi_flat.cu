#include "multi_flat.h"

#include <algorithm>
#include <stdexcept>
#include <string>

#include "select.cuh"

namespace b200 {
namespace {

constexpr int64_t kMaxMemberRows = 65536;                 // larger members use the thresholded pipeline of their own
constexpr size_t kGroupCandBytes = size_t(2) << 30;       // candidate scratch per pass
constexpr size_t kGroupBaseBytes = size_t(8) << 30;       // concatenated copy
inline int64_t pad_tile(int64_t n) { return (n + kTileB - 1) / kTileB * kTileB; }
inline size_t op_elem(int dtype) { return dtype == kI8 ? 1 : 2; }

}  // namespace

bool FlatGroup::eligible(const std::vector<FlatIndex*>& m, int64_t nq, int k) {
    if (m.size() < 2 || nq <= 0 || nq > 0x7FFFFFFF / static_cast<int64_t>(m.size())) return false;
    int64_t cap = 0, total = 0;
    for (const FlatIndex* ix : m) {
        if (ix->ntotal() <= 0 || ix->ntotal() > kMaxMemberRows) return false;
        cap = std::max(cap, pad_tile(ix->ntotal()));
        total += pad_tile(ix->ntotal());
    }
    if (k > cap) return false;   // (short results are padded by the per-index path)
    const size_t row = static_cast<size_t>(m[0]->op_cols()) * op_elem(m[0]->dtype()) +
                       (m[0]->dtype() == kF32 ? static_cast<size_t>(m[0]->d()) * 4 : 0) + 12;
    if (static_cast<size_t>(total) * row > kGroupBaseBytes) return false;
    // one member's candidate rows must fit a pass (members are paged, queries are not)
    return static_cast<size_t>(nq) * static_cast<size_t>(cap) * 8 <= kGroupCandBytes;
}

void FlatGroup::refresh(const std::vector<FlatIndex*>& members, cudaStream_t st) {
    bool same = cur_.size() == members.size();
    for (size_t i = 0; same && i < members.size(); ++i)
        same = cur_[i] == members[i] && cur_gen_[i] == members[i]->generation();
    if (same) return;
    const FlatIndex* f0 = members[0];
    d_ = f0->d();
    metric_ = f0->metric();
    dtype_ = f0->dtype();
    op_cols_ = f0->op_cols();
    kind_ = f0->gemm_kind_public();
    const FlatIndex::RawView v0 = f0->raw_view();
    num_sms_ = v0.num_sms;
    use_simt_ = v0.use_simt;
    seg_start_.assign(members.size() + 1, 0);
    cap_ = 0;
    max_norm_ = 0.f;
    for (size_t i = 0; i < members.size(); ++i) {
        const int64_t p = pad_tile(members[i]->ntotal());
        seg_start_[i + 1] = seg_start_[i] + p;
        cap_ = std::max<uint32_t>(cap_, static_cast<uint32_t>(p));
        max_norm_ = std::max(max_norm_, members[i]->raw_view().max_norm);
    }
    total_rows_ = seg_start_.back();
    const size_t row_op = static_cast<size_t>(op_cols_) * op_elem(dtype_);
    void* xop = xop_.ensure(static_cast<size_t>(total_rows_) * row_op);
    void* nrm = norms_.ensure(static_cast<size_t>(total_rows_) * 4);
    int64_t* lab = static_cast<int64_t*>(labels_.ensure(static_cast<size_t>(total_rows_) * 8));
    float* x32 = dtype_ == kF32 ? static_cast<float*>(x32_.ensure(static_cast<size_t>(total_rows_) * d_ * 4)) : nullptr;
    // padding rows: zero operands and norms (their keys are never read: the epilogue stops at seg_end)
    B200_CUDA_CHECK(cudaMemsetAsync(xop, 0, static_cast<size_t>(total_rows_) * row_op, st));
    B200_CUDA_CHECK(cudaMemsetAsync(nrm, 0, static_cast<size_t>(total_rows_) * 4, st));
    const int64_t n_tiles = total_rows_ / kTileB;
    std::vector<int32_t> h_idx(static_cast<size_t>(n_tiles));
    std::vector<int64_t> h_col0(static_cast<size_t>(n_tiles)), h_end(static_cast<size_t>(n_tiles));
    for (size_t i = 0; i < members.size(); ++i) {
        const FlatIndex::RawView v = members[i]->raw_view();
        const int64_t s0 = seg_start_[i];
        const size_t n = static_cast<size_t>(v.n);
        // packed operands (fp32 members of few dimensions) are whole-tile images: a member starts on a
        // tile boundary here as in its own buffer, so its tiles are copied as they are
        const size_t n_op = packed_operands(kind_, op_cols_) ? static_cast<size_t>((v.n + kTileB - 1) / kTileB * kTileB) : n;
        B200_CUDA_CHECK(cudaMemcpyAsync(static_cast<uint8_t*>(xop) + static_cast<size_t>(s0) * row_op, v.operand, n_op * row_op,
                                        cudaMemcpyDeviceToDevice, st));
        B200_CUDA_CHECK(cudaMemcpyAsync(static_cast<uint8_t*>(nrm) + static_cast<size_t>(s0) * 4, v.norms, n * 4,
                                        cudaMemcpyDeviceToDevice, st));
        B200_CUDA_CHECK(cudaMemcpyAsync(lab + s0, v.labels, n * 8, cudaMemcpyDeviceToDevice, st));
        if (x32)
            B200_CUDA_CHECK(cudaMemcpyAsync(x32 + static_cast<size_t>(s0) * d_, v.rows_f32, n * d_ * 4,
                                            cudaMemcpyDeviceToDevice, st));
        for (int64_t t = s0 / kTileB; t < seg_start_[i + 1] / kTileB; ++t) {
            h_idx[static_cast<size_t>(t)] = static_cast<int32_t>(i);
            h_col0[static_cast<size_t>(t)] = s0;
            h_end[static_cast<size_t>(t)] = s0 + v.n;
        }
    }
    B200_CUDA_CHECK(cudaMemcpyAsync(seg_index_.ensure(h_idx.size() * 4), h_idx.data(), h_idx.size() * 4,
                                    cudaMemcpyHostToDevice, st));
    B200_CUDA_CHECK(cudaMemcpyAsync(seg_col0_.ensure(h_col0.size() * 8), h_col0.data(), h_col0.size() * 8,
                                    cudaMemcpyHostToDevice, st));
    B200_CUDA_CHECK(cudaMemcpyAsync(seg_end_.ensure(h_end.size() * 8), h_end.data(), h_end.size() * 8,
                                    cudaMemcpyHostToDevice, st));
    if (!w_err_.get()) {
        w_err_.ensure(sizeof(int));
        B200_CUDA_CHECK(cudaMemsetAsync(w_err_.get(), 0, sizeof(int), st));
    }
    B200_CUDA_CHECK(cudaStreamSynchronize(st));   // the host tables above go out of scope
    if (!use_simt_ && encode_operand_map(&map_b_, kind_, xop, total_rows_, op_cols_, kTileB) != 0)
        throw std::runtime_error("cuTensorMapEncodeTiled failed for the concatenated base");
    cur_.assign(members.begin(), members.end());
    cur_gen_.resize(members.size());
    for (size_t i = 0; i < members.size(); ++i) cur_gen_[i] = members[i]->generation();
    ++rebuilds_;
}

void FlatGroup::search_device(const std::vector<FlatIndex*>& members, int64_t nq64, const void* xq, int k, float* D,
                              int64_t* I, cudaStream_t st) {
    DeviceGuard g(device_);
    refresh(members, st);
    const int nq = static_cast<int>(nq64);
    const bool is_int = dtype_ == kI8;
    // query preparation, once for all members
    void* qnorm = w_qnorm_.ensure(static_cast<size_t>(nq) * 4);
    const void* xq_op = xq;
    if (dtype_ == kF32) {
        void* qop = w_qop_.ensure(static_cast<size_t>((nq + kTileQ - 1) / kTileQ * kTileQ) * op_cols_ * 2);   // whole tiles
        float* eps = static_cast<float*>(w_eps_.ensure(static_cast<size_t>(nq) * 4));
        B200_CUDA_CHECK(launch_prep_queries_f32(static_cast<const float*>(xq), nq, d_, metric_, max_norm_, qop,
                                                static_cast<float*>(qnorm), eps, st));
        xq_op = qop;
    } else if (dtype_ == kF16) {
        void* qop = w_qop_.ensure(static_cast<size_t>(nq) * d_ * 2);
        B200_CUDA_CHECK(launch_f32_to_f16(static_cast<const float*>(xq), static_cast<int64_t>(nq) * d_, qop, st));
        B200_CUDA_CHECK(launch_prep_queries_f16(qop, nq, d_, static_cast<float*>(qnorm), st));
        xq_op = qop;
        ++launches_;
    } else {
        B200_CUDA_CHECK(launch_prep_queries_i8(static_cast<const int8_t*>(xq), nq, d_, static_cast<int32_t*>(qnorm), st));
    }
    ++launches_;
    CUtensorMap map_a;
    if (!use_simt_ && encode_operand_map(&map_a, kind_, xq_op, nq, op_cols_, kTileQ) != 0)
        throw std::runtime_error("cuTensorMapEncodeTiled failed for the query operand");

    // members per pass: their [member][query] candidate rows of cap_ slots share the scratch
    const size_t per_member = static_cast<size_t>(nq) * cap_ * 8;
    const size_t per_pass = std::max<size_t>(1, kGroupCandBytes / per_member);
    const size_t nm = members.size();
    const size_t max_rows = std::min(nm, per_pass) * static_cast<size_t>(nq);
    uint64_t* cand = static_cast<uint64_t*>(w_cand_.ensure(max_rows * cap_ * 8));
    uint32_t* tau = static_cast<uint32_t*>(w_tau_.ensure(max_rows * 4));
    uint64_t* sel = static_cast<uint64_t*>(w_sel_.ensure(max_rows * k * 8));
    B200_CUDA_CHECK(launch_fill_u32(tau, static_cast<int64_t>(max_rows), is_int ? 0xFFFFFFFFu : 0xFF800000u, st));
    ++launches_;
    for (size_t m0 = 0; m0 < nm; m0 += per_pass) {
        const size_t m1 = std::min(nm, m0 + per_pass);
        const int rows = static_cast<int>((m1 - m0) * static_cast<size_t>(nq));
        B200_CUDA_CHECK(cudaMemsetAsync(cand, 0xFF, static_cast<size_t>(rows) * cap_ * 8, st));
        GemmArgs a{};
        a.A = xq_op;
        a.B = xop_.get();
        a.d = op_cols_;
        a.nq = nq;
        a.N = total_rows_;
        a.n_tiles_total = static_cast<int>(total_rows_ / kTileB);
        a.tile_first = static_cast<int>(seg_start_[m0] / kTileB);
        a.n_tiles_sel = static_cast<int>((seg_start_[m1] - seg_start_[m0]) / kTileB);
        a.metric = metric_;
        a.bnorm = norms_.get();
        a.qnorm_i32 = dtype_ == kI8 ? static_cast<const int32_t*>(qnorm) : nullptr;
        a.tau = tau;
        a.cand = cand;
        a.counts = nullptr;
        a.cap = cap_;
        a.direct = 1;
        a.seg_index = seg_index_.as<int32_t>();
        a.seg_first = static_cast<int>(m0);
        a.seg_col0 = seg_col0_.as<int64_t>();
        a.seg_end = seg_end_.as<int64_t>();
        a.err = w_err_.as<int>();
        GemmLaunch L{};
        L.kind = kind_;
        L.mode = kModeAppend;
        L.burst = 32;
        L.simt = use_simt_ ? 1 : 0;
        L.num_sms = num_sms_;
        B200_CUDA_CHECK(launch_dist_gemm(L, a, &map_a, &map_b_, st));
        if (dtype_ == kF32) {
            B200_CUDA_CHECK(launch_refine_f32(cand, nullptr, cap_, cap_, rows, d_, metric_, static_cast<const float*>(xq),
                                              x32_.as<float>(), st, nq));
            ++launches_;
        }
        B200_CUDA_CHECK(launch_select_topk(cand, nullptr, cap_, cap_, rows, k, sel, nullptr, st));
        EmitArgs e{};
        e.sel = sel;
        e.nq = rows;
        e.k = k;
        e.metric = metric_;
        e.mode = is_int ? 2 : (dtype_ == kF32 ? 1 : 0);
        e.qnorm = qnorm;
        e.labels = labels_.as<int64_t>();
        e.D = D + m0 * static_cast<size_t>(nq) * k;
        e.I = I + m0 * static_cast<size_t>(nq) * k;
        e.ldk = k;
        e.qmap = nullptr;
        e.q_mod = nq;
        B200_CUDA_CHECK(launch_emit(e, st));
        launches_ += 3;
    }
    int herr = 0;
    B200_CUDA_CHECK(cudaMemcpyAsync(&herr, w_err_.get(), sizeof(int), cudaMemcpyDeviceToHost, st));
    B200_CUDA_CHECK(cudaStreamSynchronize(st));
    if (herr) {
        cudaMemsetAsync(w_err_.get(), 0, sizeof(int), st);
        throw std::runtime_error("device pipeline reported error word " + std::to_string(herr) + " (bounded wait ran out)");
    }
}

}  // namespace b200
