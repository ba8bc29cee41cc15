#include "flat_index.h"

#include <atomic>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <unordered_set>

#include "dist_gemm.cuh"
#include "select.cuh"

namespace b200 {
namespace {

constexpr size_t kCandBudgetBytes = size_t(2) << 30;  // candidate scratch per query page
constexpr uint32_t kTauAllFloat = 0xFF800000u;        // ordered key of +inf
constexpr uint32_t kTauAllInt = 0xFFFFFFFFu;

inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }
inline uint32_t pow2_ceil(uint64_t v) {
    uint32_t p = 1;
    while (p < v) p <<= 1;
    return p;
}

bool env_flag(const char* name, const char* value) {
    const char* e = std::getenv(name);
    return e && std::strcmp(e, value) == 0;
}

bool pointer_on_device(const void* p) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

}  // namespace

uint64_t FlatIndex::next_generation() {
    static std::atomic<uint64_t> counter{0};
    return ++counter;
}

FlatIndex::FlatIndex(int d, int metric, int dtype, int device)
    : d_(d), metric_(metric), dtype_(dtype), device_(device) {
    if (metric != kMetricIP && metric != kMetricL2 && !(metric == kMetricCos && dtype == kI8))
        throw std::invalid_argument("Unsupported metric type");
    DeviceGuard g(device_);
    B200_CUDA_CHECK(cudaDeviceGetAttribute(&num_sms_, cudaDevAttrMultiProcessorCount, device_));
    B200_CUDA_CHECK(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    use_simt_ = env_flag("B200IDX_GEMM", "simt");
#ifdef B200IDX_DEV_PROF
    prof_ = env_flag("B200IDX_PROF", "1");   // development builds: per-role cycle counters of the GEMM kernel
#endif
    if (prof_) {
        w_prof_.ensure((32 + 8 * 64) * 8);
        B200_CUDA_CHECK(cudaMemset(w_prof_.get(), 0, (32 + 8 * 64) * 8));
    }
    w_err_.ensure(sizeof(int));
    B200_CUDA_CHECK(cudaMemset(w_err_.get(), 0, sizeof(int)));
    maxnorm_.ensure(sizeof(float));
    B200_CUDA_CHECK(cudaMemset(maxnorm_.get(), 0, sizeof(float)));
}

FlatIndex::~FlatIndex() {
    DeviceGuard g(device_);
    if (stream_) {
        cudaStreamSynchronize(stream_);
        cudaStreamDestroy(stream_);
    }
}

int FlatIndex::gemm_kind() const {
    return dtype_ == kI8 ? kKindI8 : (dtype_ == kF16 ? kKindF16 : kKindBF16);
}

void FlatIndex::reserve(int64_t n) {
    if (n <= cap_rows_) return;
    int64_t want = std::max<int64_t>(n, cap_rows_ + cap_rows_ / 2);
    want = round_up(want, kTileB);
    const size_t row_op = static_cast<size_t>(op_cols()) * op_elem_bytes();
    if (dtype_ == kF32)
        x32_.grow_keep(static_cast<size_t>(want) * d_ * 4, static_cast<size_t>(n_) * d_ * 4, stream_);
    // whole tiles are kept: a packed operand copy interleaves the rows of a tile
    xop_.grow_keep(static_cast<size_t>(want) * row_op, static_cast<size_t>(std::min(cap_rows_, round_up(n_, kTileB))) * row_op, stream_);
    norms_.grow_keep(static_cast<size_t>(want) * 4, static_cast<size_t>(n_) * 4, stream_);
    labels_.grow_keep(static_cast<size_t>(want) * 8, static_cast<size_t>(n_) * 8, stream_);
    cap_rows_ = want;
    map_b_valid_ = false;
}

void FlatIndex::add(int64_t n, const void* x, bool x_is_f16, const int64_t* ids, bool x_on_device) {
    if (n <= 0) return;
    DeviceGuard g(device_);
    if (n_ + n > 0xFFFFFFF0ll) throw std::invalid_argument("a single-device index holds at most 2^32 - 16 vectors");
    reserve(n_ + n);
    const cudaMemcpyKind kind = x_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    const size_t rows_per_chunk = std::max<size_t>(1, (size_t(256) << 20) / (static_cast<size_t>(d_) * 4));
    for (int64_t off = 0; off < n; off += static_cast<int64_t>(rows_per_chunk)) {
        const int64_t m = std::min<int64_t>(static_cast<int64_t>(rows_per_chunk), n - off);
        const int64_t row0 = n_ + off;
        if (dtype_ == kF32) {
            float* dst = x32_.as<float>() + row0 * d_;
            B200_CUDA_CHECK(cudaMemcpyAsync(dst, static_cast<const float*>(x) + off * d_,
                                            static_cast<size_t>(m) * d_ * 4, kind, stream_));
            B200_CUDA_CHECK(launch_base_prep_f32(dst, m, d_, metric_, xop_.get(), row0, norms_.as<float>() + row0,
                                                 maxnorm_.as<float>(), stream_));
        } else if (dtype_ == kF16) {
            uint16_t* dst = xop_.as<uint16_t>() + row0 * d_;
            if (x_is_f16) {
                B200_CUDA_CHECK(cudaMemcpyAsync(dst, static_cast<const uint16_t*>(x) + off * d_,
                                                static_cast<size_t>(m) * d_ * 2, kind, stream_));
            } else {
                float* st = static_cast<float*>(w_stage_in_.ensure(static_cast<size_t>(m) * d_ * 4));
                B200_CUDA_CHECK(cudaMemcpyAsync(st, static_cast<const float*>(x) + off * d_,
                                                static_cast<size_t>(m) * d_ * 4, kind, stream_));
                B200_CUDA_CHECK(launch_f32_to_f16(st, m * d_, dst, stream_));
            }
            B200_CUDA_CHECK(launch_base_prep_f16(dst, m, d_, norms_.as<float>() + row0, stream_));
        } else {
            int8_t* dst = xop_.as<int8_t>() + row0 * d_;
            B200_CUDA_CHECK(cudaMemcpyAsync(dst, static_cast<const int8_t*>(x) + off * d_,
                                            static_cast<size_t>(m) * d_, kind, stream_));
            B200_CUDA_CHECK(launch_base_prep_i8(dst, m, d_, norms_.as<int32_t>() + row0, stream_));
        }
        B200_CUDA_CHECK(cudaStreamSynchronize(stream_));  // staging buffer and user memory are reusable
    }
    if (ids) {
        B200_CUDA_CHECK(cudaMemcpyAsync(labels_.as<int64_t>() + n_, ids, static_cast<size_t>(n) * 8,
                                        cudaMemcpyDefault, stream_));
    } else {
        B200_CUDA_CHECK(launch_iota_i64(labels_.as<int64_t>() + n_, n, n_, stream_));
    }
    if (dtype_ == kF32) {
        float m2 = 0.f;
        B200_CUDA_CHECK(cudaMemcpyAsync(&m2, maxnorm_.get(), 4, cudaMemcpyDeviceToHost, stream_));
        B200_CUDA_CHECK(cudaStreamSynchronize(stream_));
        max_norm_ = std::sqrt(m2) * 1.0001f;
    }
    B200_CUDA_CHECK(cudaStreamSynchronize(stream_));
    n_ += n;
    generation_ = next_generation();
    map_b_valid_ = false;
}

void FlatIndex::reset() {
    DeviceGuard g(device_);
    cudaStreamSynchronize(stream_);
    n_ = 0;
    generation_ = next_generation();
    max_norm_ = 0.f;
    cudaMemset(maxnorm_.get(), 0, sizeof(float));
    map_b_valid_ = false;
}

int64_t FlatIndex::remove_ids(int64_t n, const int64_t* ids) {
    if (n <= 0 || n_ == 0) return 0;
    DeviceGuard g(device_);
    std::vector<int64_t> lab(static_cast<size_t>(n_));
    B200_CUDA_CHECK(cudaMemcpy(lab.data(), labels_.get(), static_cast<size_t>(n_) * 8, cudaMemcpyDeviceToHost));
    std::unordered_set<int64_t> rm(ids, ids + n);
    std::vector<int64_t> pos;
    for (int64_t i = 0; i < n_; ++i)
        if (rm.count(lab[static_cast<size_t>(i)])) pos.push_back(i);
    // Swap-with-last compaction, highest position first, as the reference's removeIds does
    // (FR/ascenddaemon/impl/Index.cpp:86-140).
    const size_t row_op = static_cast<size_t>(op_cols()) * op_elem_bytes();
    const size_t norm_b = 4;
    int64_t last = n_ - 1;
    for (auto it = pos.rbegin(); it != pos.rend(); ++it, --last) {
        const int64_t p = *it;
        if (p == last) continue;
        if (dtype_ == kF32)
            B200_CUDA_CHECK(cudaMemcpyAsync(x32_.as<float>() + p * d_, x32_.as<float>() + last * d_,
                                            static_cast<size_t>(d_) * 4, cudaMemcpyDeviceToDevice, stream_));
        if (dtype_ == kF32)   // the operand copy may be packed: rewrite the row from its fp32 values
            B200_CUDA_CHECK(launch_base_prep_f32(x32_.as<float>() + p * d_, 1, d_, metric_, xop_.get(), p,
                                                 norms_.as<float>() + p, maxnorm_.as<float>(), stream_));
        else
            B200_CUDA_CHECK(cudaMemcpyAsync(xop_.as<uint8_t>() + p * row_op, xop_.as<uint8_t>() + last * row_op, row_op,
                                            cudaMemcpyDeviceToDevice, stream_));
        B200_CUDA_CHECK(cudaMemcpyAsync(norms_.as<uint8_t>() + p * norm_b, norms_.as<uint8_t>() + last * norm_b,
                                        norm_b, cudaMemcpyDeviceToDevice, stream_));
        B200_CUDA_CHECK(cudaMemcpyAsync(labels_.as<int64_t>() + p, labels_.as<int64_t>() + last, 8,
                                        cudaMemcpyDeviceToDevice, stream_));
    }
    B200_CUDA_CHECK(cudaStreamSynchronize(stream_));
    n_ -= static_cast<int64_t>(pos.size());
    generation_ = next_generation();
    map_b_valid_ = false;
    return static_cast<int64_t>(pos.size());
}

void FlatIndex::get_base(int64_t offset, int64_t n, void* out) const {
    if (n <= 0) return;
    DeviceGuard g(device_);
    if (offset < 0 || offset + n > n_) throw std::invalid_argument("get_base: range outside the index");
    if (dtype_ == kF32)
        B200_CUDA_CHECK(cudaMemcpy(out, x32_.as<float>() + offset * d_, static_cast<size_t>(n) * d_ * 4,
                                   cudaMemcpyDeviceToHost));
    else
        B200_CUDA_CHECK(cudaMemcpy(out, xop_.as<uint8_t>() + offset * d_ * op_elem_bytes(),
                                   static_cast<size_t>(n) * d_ * op_elem_bytes(), cudaMemcpyDeviceToHost));
}

void FlatIndex::get_labels(int64_t offset, int64_t n, int64_t* out) const {
    if (n <= 0) return;
    DeviceGuard g(device_);
    if (offset < 0 || offset + n > n_) throw std::invalid_argument("get_labels: range outside the index");
    B200_CUDA_CHECK(cudaMemcpy(out, labels_.as<int64_t>() + offset, static_cast<size_t>(n) * 8,
                               cudaMemcpyDeviceToHost));
}

// Sampling plan.  A pass over s_tiles evenly spaced base tiles yields per-burst minima; the
// k-th smallest burst minimum bounds the k-th best key from above (k bursts each hold an
// element at or below it), so appending every key <= that bound in the full pass cannot lose a
// true top-k member.  The expected number of appended candidates is about k / (sample
// fraction); cap is four times that.
FlatIndex::Plan FlatIndex::make_plan(int k, int64_t nq) const {
    Plan p{};
    const int64_t n_tiles = (n_ + kTileB - 1) / kTileB;
    const int64_t need = std::max<int64_t>(4LL * k, 1024);
    p.sampled = false;
    if (n_tiles <= 256 && n_tiles >= 8) {
        // Small base (e.g. an IVF coarse quantizer): the "sample" is the whole base, so the k-th
        // smallest burst minimum is a certain upper bound of the k-th smallest key and admits
        // little more than k candidates as long as bursts are plentiful against k (with k / bursts
        // = 1/8 and bursts of 32 about 1.07 k keys pass).  A second cheap GEMM pass is what the
        // refinement and selection kernels then do not pay for.
        const int64_t b32 = n_tiles * (kTileB / 32), b8 = n_tiles * (kTileB / 8);
        if (8LL * k <= b32) {
            p.sampled = true;
            p.burst = 32;
        } else if (4LL * k <= b8) {
            p.sampled = true;
            p.burst = 8;
        }
        if (p.sampled) p.s_tiles = static_cast<int>(n_tiles);
    }
    for (int burst : {32, 8}) {
        if (p.sampled) break;
        const int bpt = kTileB / burst;
        const int64_t s = std::max<int64_t>((n_tiles + 15) / 16, (need + bpt - 1) / bpt);
        if (s * 2 <= n_tiles) {
            p.sampled = true;
            p.burst = burst;
            p.s_tiles = static_cast<int>(s);
            break;
        }
    }
    const int64_t n_pad = round_up(n_, kTileB);
    if (p.sampled) {
        const double inv_f = static_cast<double>(n_tiles) / p.s_tiles;
        uint64_t want = static_cast<uint64_t>(4.0 * k * inv_f);
        // The append epilogue reserves slots in blocks of 8 per (thread, run of tiles of one query
        // block); a row is shared by up to four threads in each of the CTAs that walk its query block, and
        // every one of them may leave a block partly unused.
        const int64_t n_qb = (std::max<int64_t>(nq, 1) + kTileQ - 1) / kTileQ;
        // (four threads per row in the 16-warp epilogue of the bf16 kind)
        const uint64_t owners = 4 * static_cast<uint64_t>((num_sms_ + n_qb - 1) / n_qb + 1);
        want += owners * 32;   // an open block and one reserved ahead, in each of the two stretches of the pass
        p.cap = pow2_ceil(std::max<uint64_t>(p.s_tiles == n_tiles ? 512 : 2048, want));
        if (p.cap >= static_cast<uint64_t>(n_pad)) p.sampled = false;
    }
    if (!p.sampled) {
        p.burst = 32;
        p.s_tiles = 0;
        p.cap = static_cast<uint32_t>(n_pad);
    }
    return p;
}

void FlatIndex::run_page(int nq, const void* xq_raw, const void* xq_op_in, int k, float* D, int64_t* I, int ldk,
                         const int32_t* qmap_dev, bool force_full) {
    const int kind = gemm_kind();
    const bool is_int = dtype_ == kI8;
    const uint32_t tau_all = is_int ? kTauAllInt : kTauAllFloat;

    // 1. query preparation
    timer_.begin(kStageSample, stream_);
    const void* xq_op = xq_op_in;
    float* eps = nullptr;
    void* qnorm = w_qnorm_.ensure(static_cast<size_t>(nq) * 4);
    if (dtype_ == kF32) {
        const size_t qop_bytes = static_cast<size_t>(round_up(nq, kTileQ)) * op_cols() * 2;   // whole tiles (packed copy)
        void* qop = force_full ? w_fb_qop_.ensure(qop_bytes) : w_qop_.ensure(qop_bytes);
        eps = static_cast<float*>(w_eps_.ensure(static_cast<size_t>(nq) * 4));
        B200_CUDA_CHECK(launch_prep_queries_f32(static_cast<const float*>(xq_raw), nq, d_, metric_, max_norm_, qop,
                                                static_cast<float*>(qnorm), eps, stream_));
        xq_op = qop;
    } else if (dtype_ == kF16) {
        B200_CUDA_CHECK(launch_prep_queries_f16(xq_raw, nq, d_, static_cast<float*>(qnorm), stream_));
    } else {
        B200_CUDA_CHECK(launch_prep_queries_i8(static_cast<const int8_t*>(xq_raw), nq, d_,
                                               static_cast<int32_t*>(qnorm), stream_));
    }
    stats_.kernel_launches += 1;

    // 2. operand maps
    CUtensorMap map_a;
    if (!use_simt_) {
        if (!map_b_valid_) {
            if (encode_operand_map(&map_b_, kind, xop_.get(), n_, op_cols(), kTileB) != 0)
                throw std::runtime_error("cuTensorMapEncodeTiled failed for the base operand");
            map_b_valid_ = true;
        }
        if (encode_operand_map(&map_a, kind, xq_op, nq, op_cols(), kTileQ) != 0)
            throw std::runtime_error("cuTensorMapEncodeTiled failed for the query operand");
    }

    Plan plan = make_plan(k, nq);
    if (force_full) {
        plan.sampled = false;
        plan.cap = static_cast<uint32_t>(round_up(n_, kTileB));
    }

    GemmArgs a{};
    a.A = xq_op;
    a.B = xop_.get();
    a.d = op_cols();
    a.nq = nq;
    a.N = n_;
    a.n_tiles_total = static_cast<int>((n_ + kTileB - 1) / kTileB);
    a.metric = metric_;
    a.bnorm = norms_.get();
    a.qnorm_i32 = is_int ? static_cast<const int32_t*>(qnorm) : nullptr;
    a.err = w_err_.as<int>();
    a.qmask = mask_cur_;
    a.qmask_stride = mask_stride_;
    a.prof = nullptr;
#ifdef B200IDX_DEV_PROF
    if (const char* dv = getenv("B200IDX_GEMM_DBG")) a.dbg = atoi(dv);
#endif
    GemmLaunch L{};
    L.kind = kind;
    L.simt = use_simt_ ? 1 : 0;
    L.num_sms = num_sms_;

    uint32_t* tau = static_cast<uint32_t*>(w_tau_.ensure(static_cast<size_t>(nq) * 4));
    uint64_t* cand = static_cast<uint64_t*>(w_cand_.ensure(static_cast<size_t>(nq) * plan.cap * 8));
    uint32_t* counts = static_cast<uint32_t*>(w_counts_.ensure(static_cast<size_t>(nq) * 4));

    if (plan.sampled) {
        // 3a. sample pass -> per-burst minima -> threshold
        const int stride = plan.s_tiles * (kTileB / plan.burst);
        uint32_t* mins = static_cast<uint32_t*>(w_mins_.ensure(static_cast<size_t>(nq) * stride * 4));
        a.n_tiles_sel = plan.s_tiles;
        a.tile_first = plan.s_tiles == a.n_tiles_total ? 0 : -1;
        a.mins = mins;
        a.mins_stride = stride;
        L.mode = kModeBurstMin;
        L.burst = plan.burst;
        a.prof = prof_ ? w_prof_.as<unsigned long long>() : nullptr;
        B200_CUDA_CHECK(launch_dist_gemm(L, a, &map_a, &map_b_, stream_));
        B200_CUDA_CHECK(launch_kth_threshold(mins, stride, stride, nq, k, eps, tau_all, tau, stream_));
        if (dtype_ == kF32) {
            // the full pass tests "key <= tau" inside the GEMM: the threshold joins the query operand
            B200_CUDA_CHECK(launch_fold_tau(tau, static_cast<const float*>(qnorm), max_norm_, nq, d_, metric_,
                                            const_cast<void*>(xq_op), stream_));
            stats_.kernel_launches += 1;
        }
        B200_CUDA_CHECK(cudaMemsetAsync(counts, 0, static_cast<size_t>(nq) * 4, stream_));
        stats_.gemm_launches += 1;
        stats_.kernel_launches += 2;
        a.direct = 0;
    } else {
        B200_CUDA_CHECK(launch_fill_u32(tau, nq, tau_all, stream_));
        B200_CUDA_CHECK(cudaMemsetAsync(cand, 0xFF, static_cast<size_t>(nq) * plan.cap * 8, stream_));
        stats_.kernel_launches += 1;
        a.direct = 1;
    }
    timer_.end(stream_);
    timer_.begin(kStageFullGemm, stream_);
    // 4. full pass: append every key <= tau.  With a threshold from a small sample the pass runs
    //    in two stretches: after the first fifth of the tiles the candidates found so far give a
    //    much tighter threshold for the rest (their k-th smallest key bounds the final k-th key),
    //    which roughly halves the candidates and with them the epilogue's and the refinement's work.
    a.tau = tau;
    a.cand = cand;
    a.counts = counts;
    a.cap = plan.cap;
    L.mode = kModeAppend;
    L.burst = 32;
    a.prof = prof_ ? w_prof_.as<unsigned long long>() + 16 : nullptr;
    const int n_tiles = a.n_tiles_total;
    const bool two_stretches = plan.sampled && !force_full && plan.s_tiles * 4 <= n_tiles && n_tiles >= 512;
    int first_stretch = two_stretches ? std::max(n_tiles / 5, 2 * plan.s_tiles) : n_tiles;
    a.tile_first = 0;
    a.n_tiles_sel = first_stretch;
    B200_CUDA_CHECK(launch_dist_gemm(L, a, &map_a, &map_b_, stream_));
    stats_.gemm_launches += 1;
    stats_.kernel_launches += 1;
    auto report_counts = [&](const char* what) {   // development aid (B200IDX_PROF=1)
        if (!prof_ || !plan.sampled) return;
        std::vector<uint32_t> hc(static_cast<size_t>(nq));
        cudaMemcpyAsync(hc.data(), counts, static_cast<size_t>(nq) * 4, cudaMemcpyDeviceToHost, stream_);
        cudaStreamSynchronize(stream_);
        double sum = 0;
        uint32_t mx = 0;
        for (uint32_t c : hc) { sum += c; mx = std::max(mx, c); }
        fprintf(stderr, "[b200idx prof] reserved candidate slots %s: mean %.1f max %u (cap %u)\n", what, sum / nq, mx, plan.cap);
    };
    report_counts(two_stretches ? "after the first stretch" : "after the full pass");
    if (two_stretches) {
        B200_CUDA_CHECK(launch_tighten_tau(cand, counts, plan.cap, nq, k, eps, tau, stream_));
        if (dtype_ == kF32)
            B200_CUDA_CHECK(launch_fold_tau(tau, static_cast<const float*>(qnorm), max_norm_, nq, d_, metric_,
                                            const_cast<void*>(xq_op), stream_));
        a.tile_first = first_stretch;
        a.n_tiles_sel = n_tiles - first_stretch;
        a.prof = nullptr;
#ifdef B200IDX_DEV_PROF
        if (prof_ && getenv("B200IDX_GEMM_TRACE")) a.trace = w_prof_.as<unsigned long long>() + 32;
#endif
        B200_CUDA_CHECK(launch_dist_gemm(L, a, &map_a, &map_b_, stream_));
        a.trace = nullptr;
        stats_.gemm_launches += 1;
        stats_.kernel_launches += 3;
        report_counts("after the second stretch");
    }
    timer_.end(stream_);

    const uint32_t* counts_arg = plan.sampled ? counts : nullptr;
    const uint32_t n_fixed = static_cast<uint32_t>(n_);
    // 5. fp32 refinement of the candidates
    if (dtype_ == kF32) {
        timer_.begin(kStageRefine, stream_);
        // worth a pass only when the threshold came from a subset of the tiles (about 1 / fraction
        // times more candidates than k)
        if (plan.sampled && static_cast<int64_t>(plan.s_tiles) * 2 <= (n_ + kTileB - 1) / kTileB) {
            B200_CUDA_CHECK(launch_prune_candidates(cand, counts, plan.cap, nq, k, eps, stream_));
            stats_.kernel_launches += 1;
        }
        B200_CUDA_CHECK(launch_refine_f32(cand, counts_arg, n_fixed, plan.cap, nq, d_, metric_,
                                          static_cast<const float*>(xq_raw), x32_.as<float>(), stream_));
        stats_.kernel_launches += 1;
        timer_.end(stream_);
    }
    timer_.begin(kStageSelect, stream_);
    // 6. exact top-k of the candidates, 7. results
    uint64_t* sel = static_cast<uint64_t*>(w_sel_.ensure(static_cast<size_t>(nq) * k * 8));
    uint8_t* over = static_cast<uint8_t*>(w_over_.ensure(static_cast<size_t>(nq)));
    B200_CUDA_CHECK(launch_select_topk(cand, counts_arg, n_fixed, plan.cap, nq, k, sel,
                                       plan.sampled ? over : nullptr, stream_));
    if (!plan.sampled) B200_CUDA_CHECK(cudaMemsetAsync(over, 0, static_cast<size_t>(nq), stream_));
    EmitArgs e{};
    e.sel = sel;
    e.nq = nq;
    e.k = k;
    e.metric = metric_;
    e.mode = is_int ? 2 : (dtype_ == kF32 ? 1 : 0);
    e.qnorm = qnorm;
    e.labels = labels_.as<int64_t>();
    e.D = D;
    e.I = I;
    e.ldk = ldk;
    e.qmap = qmap_dev;
    B200_CUDA_CHECK(launch_emit(e, stream_));
    stats_.kernel_launches += 2;
    timer_.end(stream_);
}

void FlatIndex::search_device(int64_t nq, const void* xq, bool q_is_f16, int k, float* D, int64_t* I, int ldk) {
    if (nq <= 0) return;
    DeviceGuard g(device_);
    stats_.searches += 1;
    stats_.queries += static_cast<uint64_t>(nq);
    if (n_ == 0) {
        // empty index: FLT_MAX / -1 padding
        std::vector<float> dpad(static_cast<size_t>(k), 3.402823466e+38f);
        std::vector<int64_t> ipad(static_cast<size_t>(k), -1);
        for (int64_t q = 0; q < nq; ++q) {
            B200_CUDA_CHECK(cudaMemcpyAsync(D + q * ldk, dpad.data(), k * 4, cudaMemcpyHostToDevice, stream_));
            B200_CUDA_CHECK(cudaMemcpyAsync(I + q * ldk, ipad.data(), k * 8, cudaMemcpyHostToDevice, stream_));
        }
        B200_CUDA_CHECK(cudaStreamSynchronize(stream_));
        return;
    }
    // fp16 index fed float queries: convert once
    const void* xq_in = xq;
    if (dtype_ == kF16 && !q_is_f16) {
        void* st = w_qraw_.ensure(static_cast<size_t>(nq) * d_ * 2);
        B200_CUDA_CHECK(launch_f32_to_f16(static_cast<const float*>(xq), nq * d_, st, stream_));
        stats_.kernel_launches += 1;
        xq_in = st;
    }
    const size_t in_row = static_cast<size_t>(d_) * in_elem_bytes();

    const Plan plan = make_plan(k, nq);
    int64_t page = static_cast<int64_t>(kCandBudgetBytes / (static_cast<size_t>(plan.cap) * 8));
    if (page >= kTileQ) page = page / kTileQ * kTileQ;
    if (page < 1) page = 1;
    std::vector<int32_t> over_idx;
    for (int64_t q0 = 0; q0 < nq; q0 += page) {
        const int nqp = static_cast<int>(std::min<int64_t>(page, nq - q0));
        const uint8_t* xp = static_cast<const uint8_t*>(xq_in) + q0 * in_row;
        mask_cur_ = mask_dev_ ? mask_dev_ + q0 * mask_stride_ : nullptr;
        run_page(nqp, xp, xp, k, D + q0 * ldk, I + q0 * ldk, ldk, nullptr, false);
        uint8_t* h = static_cast<uint8_t*>(h_over_.ensure(static_cast<size_t>(nqp) + sizeof(int)));
        B200_CUDA_CHECK(cudaMemcpyAsync(h, w_over_.get(), static_cast<size_t>(nqp), cudaMemcpyDeviceToHost, stream_));
        B200_CUDA_CHECK(cudaMemcpyAsync(h + nqp, w_err_.get(), sizeof(int), cudaMemcpyDeviceToHost, stream_));
        B200_CUDA_CHECK(cudaStreamSynchronize(stream_));
        timer_.collect(stats_);
        if (prof_) {
            unsigned long long pc[32];
            cudaMemcpy(pc, w_prof_.get(), sizeof(pc), cudaMemcpyDeviceToHost);
            cudaMemset(w_prof_.get(), 0, sizeof(pc));
            if (getenv("B200IDX_GEMM_TRACE")) {
                static unsigned long long tr[8 * 64];
                cudaMemcpy(tr, w_prof_.as<unsigned long long>() + 32, sizeof(tr), cudaMemcpyDeviceToHost);
                unsigned long long t0 = ~0ull;
                for (int i = 0; i < 8 * 64; ++i)
                    if (tr[i] && tr[i] < t0) t0 = tr[i];
                fprintf(stderr, "[b200idx trace] item: loads_issued mma_start mma_last_chunk_in mma_committed | epiA acc_full, released | epiZ acc_full, released\n");
                for (int t = 0; t < 40; ++t)
                    fprintf(stderr, "[b200idx trace] %2d: %7lld %7lld %7lld %7lld | %7lld %7lld | %7lld %7lld\n", t,
                            (long long)(tr[t] - t0), (long long)(tr[64 + t] - t0), (long long)(tr[128 + t] - t0),
                            (long long)(tr[192 + t] - t0), (long long)(tr[256 + t] - t0), (long long)(tr[320 + t] - t0),
                            (long long)(tr[384 + t] - t0), (long long)(tr[448 + t] - t0));
            }
            for (int p = 0; p < 2; ++p) {
                const unsigned long long* c = pc + 16 * p;
                const double items = c[6] ? static_cast<double>(c[6]) : 1.0;
                fprintf(stderr, "[b200idx prof] %s pass: items %.0f per-item cycles: prod_wait_empty %.0f mma_wait_acc_empty %.0f "
                                "mma_wait_full %.0f | epi: wait_acc_full %.0f span %.0f (barrier %.0f, tmem_wait %.0f, chunk calls %.0f) flush %.0f | CTA total %.0f\n",
                        p ? "append" : "sample", items, c[0] / items, c[1] / items, c[2] / items, c[3] / items,
                        c[4] / items, c[9] / items, c[8] / items, c[10] / items, c[5] / items, c[7] / items);
            }
        }
        int err = 0;
        std::memcpy(&err, h + nqp, sizeof(int));
        if (err) {
            cudaMemsetAsync(w_err_.get(), 0, sizeof(int), stream_);
            throw std::runtime_error("device pipeline reported error word " + std::to_string(err) +
                                     " (bounded wait ran out)");
        }
        for (int i = 0; i < nqp; ++i)
            if (h[i]) over_idx.push_back(static_cast<int32_t>(q0 + i));
    }
    if (!over_idx.empty()) {
        // Candidate overflow (heavy ties or an unrepresentative sample): re-run those queries
        // with no threshold, every base row a candidate.
        stats_.fallback_queries += over_idx.size();
        const int64_t n_pad = round_up(n_, kTileB);
        int64_t fpage = static_cast<int64_t>(kCandBudgetBytes / (static_cast<size_t>(n_pad) * 8));
        if (fpage < 1) fpage = 1;
        int32_t* qmap = static_cast<int32_t*>(w_qmap_.ensure(over_idx.size() * 4));
        B200_CUDA_CHECK(cudaMemcpyAsync(qmap, over_idx.data(), over_idx.size() * 4, cudaMemcpyHostToDevice, stream_));
        for (size_t o0 = 0; o0 < over_idx.size(); o0 += static_cast<size_t>(fpage)) {
            const int m = static_cast<int>(std::min<size_t>(static_cast<size_t>(fpage), over_idx.size() - o0));
            void* fq = w_fb_q_.ensure(static_cast<size_t>(m) * in_row);
            B200_CUDA_CHECK(launch_gather_rows(xq_in, qmap + o0, m, static_cast<int>(in_row), fq, stream_));
            stats_.kernel_launches += 1;
            mask_cur_ = nullptr;
            if (mask_dev_) {
                void* fm = w_fb_mask_.ensure(static_cast<size_t>(m) * mask_stride_ * 4);
                B200_CUDA_CHECK(launch_gather_rows(mask_dev_, qmap + o0, m, static_cast<int>(mask_stride_ * 4), fm, stream_));
                mask_cur_ = static_cast<const uint32_t*>(fm);
            }
            run_page(m, fq, fq, k, D, I, ldk, qmap + o0, true);
            B200_CUDA_CHECK(cudaStreamSynchronize(stream_));
            timer_.collect(stats_);
        }
    }
}

void FlatIndex::search_host(int64_t nq, const void* xq, bool q_is_f16, int k, float* D, int64_t* I) {
    search_host_masked(nq, xq, q_is_f16, k, nullptr, D, I);
}

void FlatIndex::search_host_masked(int64_t nq, const void* xq, bool q_is_f16, int k, const uint8_t* mask, float* D,
                                   int64_t* I) {
    if (nq <= 0) return;
    DeviceGuard g(device_);
    // the filter travels as 32-bit words, one row per query, rows padded with zeros to whole tiles
    const size_t mask_bytes = static_cast<size_t>((n_ + 7) / 8);
    const int64_t mstride = round_up(std::max<int64_t>(n_, 1), kTileB) / 32;
    struct MaskScope {   // the members describe the search in progress only
        FlatIndex* self;
        ~MaskScope() { self->mask_dev_ = self->mask_cur_ = nullptr; self->mask_stride_ = 0; }
    } scope{this};
    const size_t in_row = static_cast<size_t>(d_) * ((dtype_ == kI8) ? 1 : (q_is_f16 ? 2 : 4));
    // Page so that staging stays bounded.
    const size_t per_query = std::max<size_t>(std::max<size_t>(in_row, size_t(k) * 12), mask ? static_cast<size_t>(mstride) * 4 : 0);
    const int64_t page = std::max<int64_t>(1, std::min<int64_t>(nq, (size_t(1) << 30) / per_query));
    for (int64_t q0 = 0; q0 < nq; q0 += page) {
        const int64_t m = std::min<int64_t>(page, nq - q0);
        void* dq = w_stage_in_.ensure(static_cast<size_t>(m) * in_row);
        float* dD = static_cast<float*>(w_stage_D_.ensure(static_cast<size_t>(m) * k * 4));
        int64_t* dI = static_cast<int64_t*>(w_stage_I_.ensure(static_cast<size_t>(m) * k * 8));
        B200_CUDA_CHECK(cudaMemcpyAsync(dq, static_cast<const uint8_t*>(xq) + q0 * in_row,
                                        static_cast<size_t>(m) * in_row, cudaMemcpyHostToDevice, stream_));
        if (mask && n_ > 0) {
            void* dm = w_mask_.ensure(static_cast<size_t>(m) * mstride * 4);
            B200_CUDA_CHECK(cudaMemsetAsync(dm, 0, static_cast<size_t>(m) * mstride * 4, stream_));
            B200_CUDA_CHECK(cudaMemcpy2DAsync(dm, static_cast<size_t>(mstride) * 4, mask + q0 * mask_bytes, mask_bytes,
                                              mask_bytes, static_cast<size_t>(m), cudaMemcpyHostToDevice, stream_));
            mask_dev_ = static_cast<const uint32_t*>(dm);
            mask_stride_ = mstride;
        }
        search_device(m, dq, q_is_f16, k, dD, dI, k);
        B200_CUDA_CHECK(cudaMemcpyAsync(D + q0 * k, dD, static_cast<size_t>(m) * k * 4, cudaMemcpyDeviceToHost,
                                        stream_));
        B200_CUDA_CHECK(cudaMemcpyAsync(I + q0 * k, dI, static_cast<size_t>(m) * k * 8, cudaMemcpyDeviceToHost,
                                        stream_));
        B200_CUDA_CHECK(cudaStreamSynchronize(stream_));
    }
}

}  // namespace b200
