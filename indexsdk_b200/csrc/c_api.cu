// extern "C" surface declared in include/b200idx.h: argument checks, exception -> status code
// translation, and the multi-index / multi-device fan-out.
#include "../../include/b200idx.h"

#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "c_api_internal.h"
#include "flat_index.h"
#include "ivfpq_index.h"
#include "select.cuh"

using namespace b200;

struct b200idx_index {
    int kind = 0;  // 0 flat, 1 int8 flat, 2 ivfpq
    std::unique_ptr<FlatIndex> flat;
    std::unique_ptr<IvfpqIndex> ivfpq;
    mutable std::string last_error;
};

namespace {

std::string g_create_error;
std::mutex g_create_mutex;

constexpr int kMaxK = 4096;        // FR/ascend/AscendIndex.h:36
constexpr int64_t kMaxN = 1000000000;  // FR/ascend/AscendIndex.h:35

template <typename F>
int guarded(const b200idx_index* h, F&& f) {
    try {
        f();
        return B200IDX_OK;
    } catch (const std::invalid_argument& e) {
        if (h) h->last_error = e.what();
        return B200IDX_ERR_INVALID_PARAM;
    } catch (const std::exception& e) {
        if (h) h->last_error = e.what();
        const bool timeout = std::strstr(e.what(), "bounded wait") != nullptr;
        cudaGetLastError();
        return timeout ? B200IDX_ERR_TIMEOUT : B200IDX_ERR_INNER;
    } catch (...) {
        if (h) h->last_error = "unknown error";
        return B200IDX_ERR_INNER;
    }
}

template <typename F>
int guarded_create(F&& f) {
    try {
        f();
        return B200IDX_OK;
    } catch (const std::invalid_argument& e) {
        std::lock_guard<std::mutex> l(g_create_mutex);
        g_create_error = e.what();
        return B200IDX_ERR_INVALID_PARAM;
    } catch (const std::exception& e) {
        std::lock_guard<std::mutex> l(g_create_mutex);
        g_create_error = e.what();
        cudaGetLastError();
        return B200IDX_ERR_INNER;
    }
}

void check_common_create(int d, int metric, int device, b200idx_t** out) {
    if (!out) throw std::invalid_argument("out must not be NULL");
    if (d <= 0 || d % 16 != 0 || d > 4096)
        throw std::invalid_argument("Unsupported dims: d must be a multiple of 16 in (0, 4096]");
    if (metric != B200IDX_METRIC_INNER_PRODUCT && metric != B200IDX_METRIC_L2)
        throw std::invalid_argument("Unsupported metric type");
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        cudaGetLastError();
        throw std::runtime_error("no CUDA device is available; this library has no CPU path");
    }
    if (device < 0 || device >= count) throw std::invalid_argument("device ordinal out of range");
}

void check_search_args(const b200idx_index* h, int64_t n, const void* x, int k, const float* D, const int64_t* I) {
    if (!h) throw std::invalid_argument("Invalid handle: nullptr.");
    if (n <= 0 || n >= kMaxN) throw std::invalid_argument("n must be > 0 and < 1e9");
    if (k <= 0 || k > kMaxK) throw std::invalid_argument("k must be > 0 and <= 4096");
    if (!x) throw std::invalid_argument("Invalid x: nullptr.");
    if (!D) throw std::invalid_argument("Invalid distances: nullptr.");
    if (!I) throw std::invalid_argument("Invalid labels: nullptr.");
}

int dev_of(const b200idx_index* h) { return h->kind == 2 ? h->ivfpq->device() : h->flat->device(); }
int dim_of(const b200idx_index* h) { return h->kind == 2 ? h->ivfpq->d() : h->flat->d(); }
size_t query_row_bytes(const b200idx_index* h) {
    return static_cast<size_t>(dim_of(h)) * (h->kind == 1 ? 1 : 4);
}
bool descending_of(const b200idx_index* h) {
    return h->kind != 2 && h->flat->metric() == kMetricIP;
}

}  // namespace

namespace b200_capi {
int guarded(const b200idx_t* h, const std::function<void()>& f) { return ::guarded(h, f); }
b200::FlatIndex* flat_of(b200idx_t* h) { return (h && h->kind != 2) ? h->flat.get() : nullptr; }
}  // namespace b200_capi

extern "C" {

int b200idx_create_flat(int d, int metric, int dtype, int device, b200idx_t** out) {
    return guarded_create([&] {
        check_common_create(d, metric, device, out);
        if (dtype != B200IDX_F32 && dtype != B200IDX_F16) throw std::invalid_argument("Unsupported dtype");
        std::unique_ptr<b200idx_index> h(new b200idx_index);
        h->kind = 0;
        h->flat.reset(new FlatIndex(d, metric, dtype == B200IDX_F32 ? kF32 : kF16, device));
        *out = h.release();
    });
}

int b200idx_create_int8flat(int d, int metric, int device, b200idx_t** out) {
    return guarded_create([&] {
        check_common_create(d, metric, device, out);
        std::unique_ptr<b200idx_index> h(new b200idx_index);
        h->kind = 1;
        h->flat.reset(new FlatIndex(d, metric, kI8, device));
        *out = h.release();
    });
}

int b200idx_create_ivfpq(int d, int metric, int nlist, int M, int nbits, int by_residual, int device,
                         b200idx_t** out) {
    return guarded_create([&] {
        check_common_create(d, metric, device, out);
        if (metric != B200IDX_METRIC_L2) throw std::invalid_argument("Unsupported metric type: IVFPQ supports L2 only");
        if (nlist <= 0) throw std::invalid_argument("Unsupported nlists");
        if (M <= 0 || d % M != 0 || M > 256) throw std::invalid_argument("Unsupported msubs");
        if (nbits != 8) throw std::invalid_argument("Unsupported nbits");
        std::unique_ptr<b200idx_index> h(new b200idx_index);
        h->kind = 2;
        h->ivfpq.reset(new IvfpqIndex(d, nlist, M, nbits, by_residual != 0, device));
        *out = h.release();
    });
}

int b200idx_destroy(b200idx_t* h) {
    delete h;
    return B200IDX_OK;
}

int b200idx_add(b200idx_t* h, int64_t n, const void* x, const int64_t* ids) {
    if (!h) return B200IDX_ERR_INVALID_PARAM;
    return guarded(h, [&] {
        if (n <= 0 || n >= kMaxN) throw std::invalid_argument("n must be > 0 and < 1e9");
        if (!x) throw std::invalid_argument("Invalid x: nullptr.");
        if (h->kind == 2) h->ivfpq->add(n, static_cast<const float*>(x), ids, false);
        else h->flat->add(n, x, false, ids, false);
    });
}

int b200idx_add_f16(b200idx_t* h, int64_t n, const uint16_t* x, const int64_t* ids) {
    if (!h) return B200IDX_ERR_INVALID_PARAM;
    return guarded(h, [&] {
        if (n <= 0 || n >= kMaxN) throw std::invalid_argument("n must be > 0 and < 1e9");
        if (!x) throw std::invalid_argument("Invalid x: nullptr.");
        if (h->kind != 0 || h->flat->dtype() != kF16)
            throw std::invalid_argument("fp16 input is accepted by Flat indexes of dtype F16 only");
        h->flat->add(n, x, true, ids, false);
    });
}

int b200idx_add_device(b200idx_t* h, int64_t n, const void* x_dev, const int64_t* ids_host) {
    if (!h) return B200IDX_ERR_INVALID_PARAM;
    return guarded(h, [&] {
        if (n <= 0 || n >= kMaxN) throw std::invalid_argument("n must be > 0 and < 1e9");
        if (!x_dev) throw std::invalid_argument("Invalid x: nullptr.");
        if (h->kind == 2) h->ivfpq->add(n, static_cast<const float*>(x_dev), ids_host, true);
        else h->flat->add(n, x_dev, false, ids_host, true);
    });
}

int b200idx_search(b200idx_t* h, int64_t n, const void* x, int k, float* D, int64_t* I) {
    return guarded(h, [&] {
        check_search_args(h, n, x, k, D, I);
        if (h->kind == 2) h->ivfpq->search_host(n, static_cast<const float*>(x), k, D, I);
        else h->flat->search_host(n, x, false, k, D, I);
    });
}

int b200idx_search_f16(b200idx_t* h, int64_t n, const uint16_t* x, int k, float* D, int64_t* I) {
    return guarded(h, [&] {
        check_search_args(h, n, x, k, D, I);
        if (h->kind != 0 || h->flat->dtype() != kF16)
            throw std::invalid_argument("fp16 queries are accepted by Flat indexes of dtype F16 only");
        h->flat->search_host(n, x, true, k, D, I);
    });
}

int b200idx_search_with_masks(b200idx_t* h, int64_t n, const void* x, int k, const uint8_t* mask, float* D,
                              int64_t* I) {
    return guarded(h, [&] {
        check_search_args(h, n, x, k, D, I);
        if (h->kind == 2) throw std::invalid_argument("search_with_masks applies to Flat and Int8Flat indexes");
        if (!mask) throw std::invalid_argument("mask can not be nullptr.");
        h->flat->search_host_masked(n, x, false, k, mask, D, I);
    });
}

int b200idx_search_device(b200idx_t* h, int64_t n, const void* x, int k, float* D, int64_t* I) {
    return guarded(h, [&] {
        check_search_args(h, n, x, k, D, I);
        if (h->kind == 2) h->ivfpq->search_device(n, static_cast<const float*>(x), k, D, I);
        else h->flat->search_device(n, x, false, k, D, I, k);
    });
}

int b200idx_search_multi(b200idx_t* const* hs, int nh, int64_t n, const void* x, int k, float* D, int64_t* I,
                         int merged) {
    if (!hs || nh <= 0 || !hs[0]) return B200IDX_ERR_INVALID_PARAM;
    b200idx_index* h0 = hs[0];
    return guarded(h0, [&] {
        if (nh > 10000) throw std::invalid_argument("size of indexes must be > 0 and <= 10000.");
        check_search_args(h0, n, x, k, D, I);
        for (int i = 0; i < nh; ++i) {
            if (!hs[i]) throw std::invalid_argument("Invalid index: nullptr.");
            if (hs[i]->kind != h0->kind || dim_of(hs[i]) != dim_of(h0) ||
                descending_of(hs[i]) != descending_of(h0))
                throw std::invalid_argument("the indexes of a multi-index search must share type, dims and metric");
        }
        const size_t row = query_row_bytes(h0);
        const size_t per = static_cast<size_t>(n) * k;
        const int dev0 = dev_of(h0);
        // per-device groups; one worker thread per device, indexes of a device run back to back
        std::map<int, std::vector<int>> groups;
        for (int i = 0; i < nh; ++i) groups[dev_of(hs[i])].push_back(i);

        float* allD = nullptr;   // [nh][n][k] on dev0 when merged
        int64_t* allI = nullptr;
        {
            DeviceGuard g(dev0);
            if (merged) {
                B200_CUDA_CHECK(cudaMalloc(&allD, per * nh * 4));
                B200_CUDA_CHECK(cudaMalloc(&allI, per * nh * 8));
            }
        }
        std::vector<std::string> errors(groups.size());
        std::vector<std::thread> workers;
        size_t gi = 0;
        for (auto& kv : groups) {
            const int dev = kv.first;
            const std::vector<int>& members = kv.second;
            std::string* err = &errors[gi++];
            auto body = [=, &hs]() {
                try {
                    DeviceGuard g(dev);
                    void* dq = nullptr;
                    float* dD = nullptr;
                    int64_t* dI = nullptr;
                    B200_CUDA_CHECK(cudaMalloc(&dq, static_cast<size_t>(n) * row));
                    B200_CUDA_CHECK(cudaMalloc(&dD, per * 4));
                    B200_CUDA_CHECK(cudaMalloc(&dI, per * 8));
                    B200_CUDA_CHECK(cudaMemcpy(dq, x, static_cast<size_t>(n) * row, cudaMemcpyHostToDevice));
                    for (int i : members) {
                        b200idx_index* h = hs[i];
                        if (h->kind == 2) h->ivfpq->search_device(n, static_cast<const float*>(dq), k, dD, dI);
                        else h->flat->search_device(n, dq, false, k, dD, dI, k);
                        if (merged) {
                            B200_CUDA_CHECK(cudaMemcpy(allD + per * i, dD, per * 4, cudaMemcpyDefault));
                            B200_CUDA_CHECK(cudaMemcpy(allI + per * i, dI, per * 8, cudaMemcpyDefault));
                        } else {
                            B200_CUDA_CHECK(cudaMemcpy(D + per * i, dD, per * 4, cudaMemcpyDeviceToHost));
                            B200_CUDA_CHECK(cudaMemcpy(I + per * i, dI, per * 8, cudaMemcpyDeviceToHost));
                        }
                    }
                    cudaFree(dq);
                    cudaFree(dD);
                    cudaFree(dI);
                } catch (const std::exception& e) {
                    *err = e.what();
                }
            };
            if (groups.size() == 1) body();
            else workers.emplace_back(body);
        }
        for (auto& w : workers) w.join();
        std::string first_err;
        for (auto& e : errors)
            if (!e.empty() && first_err.empty()) first_err = e;
        if (first_err.empty() && merged) {
            DeviceGuard g(dev0);
            float* mD = nullptr;
            int64_t* mI = nullptr;
            B200_CUDA_CHECK(cudaMalloc(&mD, per * 4));
            B200_CUDA_CHECK(cudaMalloc(&mI, per * 8));
            B200_CUDA_CHECK(launch_merge_topk(nh, n, k, descending_of(h0) ? 1 : 0, allD, allI, mD, mI, nullptr));
            B200_CUDA_CHECK(cudaMemcpy(D, mD, per * 4, cudaMemcpyDeviceToHost));
            B200_CUDA_CHECK(cudaMemcpy(I, mI, per * 8, cudaMemcpyDeviceToHost));
            cudaFree(mD);
            cudaFree(mI);
        }
        {
            DeviceGuard g(dev0);
            if (allD) cudaFree(allD);
            if (allI) cudaFree(allI);
        }
        if (!first_err.empty()) throw std::runtime_error(first_err);
    });
}

int b200idx_merge_topk_device(int nsrc, int64_t n, int k, int descending, const float* Din, const int64_t* Iin,
                              float* D, int64_t* I, void* stream) {
    if (nsrc <= 0 || n <= 0 || k <= 0 || !Din || !Iin || !D || !I) return B200IDX_ERR_INVALID_PARAM;
    cudaError_t e = launch_merge_topk(nsrc, n, k, descending, Din, Iin, D, I, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? B200IDX_OK : B200IDX_ERR_INNER;
}

int b200idx_reset(b200idx_t* h) {
    if (!h) return B200IDX_ERR_INVALID_PARAM;
    return guarded(h, [&] {
        if (h->kind == 2) h->ivfpq->reset();
        else h->flat->reset();
    });
}

int b200idx_remove_ids(b200idx_t* h, int64_t n, const int64_t* ids, int64_t* n_removed) {
    if (!h) return B200IDX_ERR_INVALID_PARAM;
    return guarded(h, [&] {
        if (n < 0 || (n > 0 && !ids)) throw std::invalid_argument("Invalid ids: nullptr.");
        int64_t r = h->kind == 2 ? h->ivfpq->remove_ids(n, ids) : h->flat->remove_ids(n, ids);
        if (n_removed) *n_removed = r;
    });
}

int64_t b200idx_ntotal(const b200idx_t* h) {
    if (!h) return -1;
    return h->kind == 2 ? h->ivfpq->ntotal() : h->flat->ntotal();
}
int b200idx_dim(const b200idx_t* h) { return h ? dim_of(h) : -1; }
int b200idx_device(const b200idx_t* h) { return h ? dev_of(h) : -1; }

int b200idx_get_base(const b200idx_t* h, int64_t offset, int64_t n, void* out) {
    if (!h) return B200IDX_ERR_INVALID_PARAM;
    return guarded(h, [&] {
        if (h->kind == 2) throw std::invalid_argument("get_base applies to Flat indexes; use b200idx_ivfpq_get_list");
        if (!out) throw std::invalid_argument("Invalid out: nullptr.");
        h->flat->get_base(offset, n, out);
    });
}

int b200idx_get_ids(const b200idx_t* h, int64_t offset, int64_t n, int64_t* out) {
    if (!h) return B200IDX_ERR_INVALID_PARAM;
    return guarded(h, [&] {
        if (h->kind == 2) throw std::invalid_argument("get_ids applies to Flat indexes; use b200idx_ivfpq_get_list");
        if (!out) throw std::invalid_argument("Invalid out: nullptr.");
        h->flat->get_labels(offset, n, out);
    });
}

#define B200_REQUIRE_IVFPQ(h)                                                         \
    if (!(h)) return B200IDX_ERR_INVALID_PARAM;                                       \
    if ((h)->kind != 2) {                                                             \
        (h)->last_error = "not an IVFPQ index";                                       \
        return B200IDX_ERR_INVALID_PARAM;                                             \
    }

int b200idx_ivfpq_set_centroids(b200idx_t* h, const float* c) {
    B200_REQUIRE_IVFPQ(h)
    return guarded(h, [&] {
        if (!c) throw std::invalid_argument("Invalid centroids: nullptr.");
        if (h->ivfpq->ntotal() > 0) throw std::invalid_argument("centroids cannot change while the index holds vectors");
        h->ivfpq->set_centroids(c);
    });
}
int b200idx_ivfpq_set_codebooks(b200idx_t* h, const float* cb) {
    B200_REQUIRE_IVFPQ(h)
    return guarded(h, [&] {
        if (!cb) throw std::invalid_argument("Invalid codebooks: nullptr.");
        if (h->ivfpq->ntotal() > 0) throw std::invalid_argument("codebooks cannot change while the index holds vectors");
        h->ivfpq->set_codebooks(cb);
    });
}
int b200idx_ivfpq_get_centroids(const b200idx_t* h, float* out) {
    B200_REQUIRE_IVFPQ(h)
    return guarded(h, [&] {
        if (!out || !h->ivfpq->is_trained()) throw std::invalid_argument("index is not trained or out is NULL");
        h->ivfpq->get_centroids(out);
    });
}
int b200idx_ivfpq_get_codebooks(const b200idx_t* h, float* out) {
    B200_REQUIRE_IVFPQ(h)
    return guarded(h, [&] {
        if (!out || !h->ivfpq->is_trained()) throw std::invalid_argument("index is not trained or out is NULL");
        h->ivfpq->get_codebooks(out);
    });
}
int b200idx_ivfpq_add_codes(b200idx_t* h, int64_t n, const int32_t* list_no, const uint8_t* codes,
                            const int64_t* ids) {
    B200_REQUIRE_IVFPQ(h)
    return guarded(h, [&] {
        if (n <= 0 || !list_no || !codes) throw std::invalid_argument("add_codes: n must be > 0, pointers non-NULL");
        h->ivfpq->add_codes(n, list_no, codes, ids);
    });
}
int b200idx_ivfpq_set_nprobe(b200idx_t* h, int nprobe) {
    B200_REQUIRE_IVFPQ(h)
    return guarded(h, [&] {
        if (nprobe <= 0 || nprobe > h->ivfpq->nlist()) throw std::invalid_argument("nprobe must be in [1, nlist]");
        h->ivfpq->set_nprobe(nprobe);
    });
}
int b200idx_ivfpq_get_nprobe(const b200idx_t* h) { return (h && h->kind == 2) ? h->ivfpq->nprobe() : -1; }
int64_t b200idx_ivfpq_list_length(const b200idx_t* h, int list) {
    if (!h || h->kind != 2 || list < 0 || list >= h->ivfpq->nlist()) return -1;
    return h->ivfpq->list_length(list);
}
int b200idx_ivfpq_coarse_device(b200idx_t* h, int64_t n, const float* x, float* cD, int64_t* cI) {
    B200_REQUIRE_IVFPQ(h)
    return guarded(h, [&] {
        if (n <= 0 || !x || !cD || !cI) throw std::invalid_argument("n must be > 0, pointers non-NULL");
        h->ivfpq->coarse_device(n, x, cD, cI);
    });
}
int b200idx_ivfpq_search_preassigned_device(b200idx_t* h, int64_t n, const float* x, int k, const float* cD,
                                            const int64_t* cI, float* D, int64_t* I) {
    B200_REQUIRE_IVFPQ(h)
    return guarded(h, [&] {
        check_search_args(h, n, x, k, D, I);
        h->ivfpq->search_preassigned_device(n, x, k, cD, cI, D, I);
    });
}
int b200idx_ivfpq_get_list(const b200idx_t* h, int list, uint8_t* codes, int64_t* ids) {
    B200_REQUIRE_IVFPQ(h)
    return guarded(h, [&] { h->ivfpq->get_list(list, codes, ids); });
}

int b200idx_stats(b200idx_t* h, b200idx_stats_t* out, int reset) {
    if (!h || !out) return B200IDX_ERR_INVALID_PARAM;
    SearchStats& s = h->kind == 2 ? h->ivfpq->stats() : h->flat->stats();
    for (int i = 0; i < B200IDX_NUM_STAGES; ++i) {
        out->stage_ms[i] = s.stage_ms[i];
        out->stage_launches[i] = s.stage_launches[i];
    }
    if (h->kind == 2) {
        // the coarse quantizer's own stages are reported in slots 0-3
        SearchStats& c = h->ivfpq->coarse_stats();
        for (int i = 0; i < 4; ++i) {
            out->stage_ms[i] = c.stage_ms[i];
            out->stage_launches[i] = c.stage_launches[i];
        }
        if (reset) c = SearchStats();
    }
    out->searches = s.searches;
    out->queries = s.queries;
    out->fallback_queries = s.fallback_queries;
    out->gemm_launches = s.gemm_launches;
    out->kernel_launches = s.kernel_launches;
    out->scan_codes = s.scan_codes;
    if (reset) s = SearchStats();
    return B200IDX_OK;
}

int b200idx_set_timing(b200idx_t* h, int enabled) {
    if (!h) return B200IDX_ERR_INVALID_PARAM;
    if (h->kind == 2) h->ivfpq->set_timing(enabled != 0);
    else h->flat->timer().enable(enabled != 0);
    return B200IDX_OK;
}

void* b200idx_stream(const b200idx_t* h) {
    if (!h) return nullptr;
    return h->kind == 2 ? static_cast<void*>(h->ivfpq->stream()) : static_cast<void*>(h->flat->stream());
}

const char* b200idx_last_error(const b200idx_t* h) {
    if (h) return h->last_error.c_str();
    std::lock_guard<std::mutex> l(g_create_mutex);
    return g_create_error.c_str();
}

const char* b200idx_version(void) { return "b200idx 0.1 (sm_100a)"; }

}  // extern "C"
