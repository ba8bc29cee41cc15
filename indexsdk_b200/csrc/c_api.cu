// extern "C" surface declared in include/b200idx.h: argument checks, exception -> status code
// translation, and the multi-index / multi-device fan-out.
#include "../../include/b200idx.h"

#include <algorithm>
#include <cstdio>
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
#include "kmeans.h"
#include "multi_flat.h"
#include "select.cuh"

using namespace b200;

struct b200idx_index {
    int kind = 0;  // 0 flat, 1 int8 flat, 2 ivfpq
    std::unique_ptr<FlatIndex> flat;
    std::unique_ptr<IvfpqIndex> ivfpq;
    mutable std::string last_error;
    // An index owns ONE stream and ONE set of scratch buffers, so its entry points are not
    // re-entrant: every call on a handle runs under this mutex.  Host threads may share a handle
    // (the reference's MX_INDEX_MULTITHREAD=1 mode lets several threads search one index); their
    // calls are serialised here, calls on different handles run concurrently.
    mutable std::mutex mu;
};

namespace {

std::string g_create_error;
std::mutex g_create_mutex;

constexpr int kMaxK = 4096;        // FR/ascend/AscendIndex.h:36
constexpr int64_t kMaxN = 1000000000;  // FR/ascend/AscendIndex.h:35

// status_of_error: message of a thrown exception -> status code.  A bounded device-side wait that
// ran out is reported by the index classes as a runtime_error whose text contains "bounded wait".
int status_of_error(const char* what) {
    return std::strstr(what, "bounded wait") != nullptr ? B200IDX_ERR_TIMEOUT : B200IDX_ERR_INNER;
}

template <typename F>
int guarded(const b200idx_index* h, F&& f, bool lock = true) {
    std::unique_lock<std::mutex> guard;
    if (h && lock) guard = std::unique_lock<std::mutex>(h->mu);
    try {
        f();
        return B200IDX_OK;
    } catch (const std::invalid_argument& e) {
        if (h) h->last_error = e.what();
        return B200IDX_ERR_INVALID_PARAM;
    } catch (const std::exception& e) {
        if (h) h->last_error = e.what();
        cudaGetLastError();
        return status_of_error(e.what());
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

void check_common_create(int d, int metric, int device, b200idx_t** out, bool allow_cosine = false) {
    if (!out) throw std::invalid_argument("out must not be NULL");
    if (d <= 0 || d % 16 != 0 || d > 4096)
        throw std::invalid_argument("Unsupported dims: d must be a multiple of 16 in (0, 4096]");
    if (metric != B200IDX_METRIC_INNER_PRODUCT && metric != B200IDX_METRIC_L2 &&
        !(allow_cosine && metric == B200IDX_METRIC_INT8_COSINE))
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

// Device buffers of b200idx_search_multi, one set per device, grown on demand and kept.
struct MultiScratch {
    std::mutex mu;           // held for a whole multi-index search that uses this device
    DeviceBuffer q, D, I, allD, allI, mD, mI, gD, gI;
    std::unique_ptr<FlatGroup> group;   // concatenated copy of the small Flat indexes searched together last
};
MultiScratch& multi_scratch(int device) {
    static std::mutex table_mu;
    static std::map<int, std::unique_ptr<MultiScratch>> table;
    std::lock_guard<std::mutex> l(table_mu);
    std::unique_ptr<MultiScratch>& p = table[device];
    if (!p) p.reset(new MultiScratch);
    return *p;
}

int dev_of(const b200idx_index* h) { return h->kind == 2 ? h->ivfpq->device() : h->flat->device(); }
int dim_of(const b200idx_index* h) { return h->kind == 2 ? h->ivfpq->d() : h->flat->d(); }
size_t query_row_bytes(const b200idx_index* h) {
    return static_cast<size_t>(dim_of(h)) * (h->kind == 1 ? 1 : 4);
}
bool descending_of(const b200idx_index* h) {
    return h->kind != 2 && h->flat->metric() != kMetricL2;
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
        check_common_create(d, metric, device, out, true);
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
    // the member handles are locked below (all of them, in address order), not by guarded()
    return guarded(h0, [&] {
        if (nh > 10000) throw std::invalid_argument("size of indexes must be > 0 and <= 10000.");
        check_search_args(h0, n, x, k, D, I);
        for (int i = 0; i < nh; ++i) {
            if (!hs[i]) throw std::invalid_argument("Invalid index: nullptr.");
            if (hs[i]->kind != h0->kind || dim_of(hs[i]) != dim_of(h0) ||
                descending_of(hs[i]) != descending_of(h0))
                throw std::invalid_argument("the indexes of a multi-index search must share type, dims and metric");
        }
        // FR/ascend/AscendMultiIndexSearch.cpp:213-228 takes every index's lock before searching
        std::vector<b200idx_index*> uniq(hs, hs + nh);
        std::sort(uniq.begin(), uniq.end());
        uniq.erase(std::unique(uniq.begin(), uniq.end()), uniq.end());
        std::vector<std::unique_lock<std::mutex>> locks;
        locks.reserve(uniq.size());
        for (b200idx_index* u : uniq) locks.emplace_back(u->mu);

        const size_t row = query_row_bytes(h0);
        const size_t per = static_cast<size_t>(n) * k;
        const int dev0 = dev_of(h0);
        // per-device groups; one worker thread per device, indexes of a device run back to back
        std::map<int, std::vector<int>> groups;
        for (int i = 0; i < nh; ++i) groups[dev_of(hs[i])].push_back(i);

        // Scratch is per device, grow-only and kept between calls (a steady-state call allocates
        // nothing); every buffer is owned by the scratch object, so no exit path leaks.
        MultiScratch& s0 = multi_scratch(dev0);
        std::vector<MultiScratch*> held;
        for (auto& kv : groups) held.push_back(&multi_scratch(kv.first));
        if (std::find(held.begin(), held.end(), &s0) == held.end()) held.push_back(&s0);
        std::sort(held.begin(), held.end());
        std::vector<std::unique_lock<std::mutex>> scratch_locks;
        for (MultiScratch* m : held) scratch_locks.emplace_back(m->mu);

        float* allD = nullptr;   // [nh][n][k] on dev0 when merged
        int64_t* allI = nullptr;
        if (merged) {
            DeviceGuard g(dev0);
            allD = static_cast<float*>(s0.allD.ensure(per * nh * 4));
            allI = static_cast<int64_t*>(s0.allI.ensure(per * nh * 8));
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
                    MultiScratch& sc = multi_scratch(dev);
                    void* dq = sc.q.ensure(static_cast<size_t>(n) * row);
                    float* dD = static_cast<float*>(sc.D.ensure(per * 4));
                    int64_t* dI = static_cast<int64_t*>(sc.I.ensure(per * 8));
                    cudaStream_t st = static_cast<cudaStream_t>(b200idx_stream(hs[members[0]]));
                    B200_CUDA_CHECK(cudaMemcpyAsync(dq, x, static_cast<size_t>(n) * row, cudaMemcpyHostToDevice, st));
                    B200_CUDA_CHECK(cudaStreamSynchronize(st));
                    // Small exact indexes of one device are searched in ONE pass over their
                    // concatenated bases (segmented search): launches do not grow with their number.
                    std::vector<FlatIndex*> fm;
                    bool groupable = members.size() >= 2 && hs[members[0]]->kind != 2;
                    for (size_t j = 0; groupable && j < members.size(); ++j) {
                        FlatIndex* f = hs[members[j]]->flat.get();
                        groupable = f->dtype() == hs[members[0]]->flat->dtype() && f->metric() == hs[members[0]]->flat->metric();
                        fm.push_back(f);
                    }
                    if (groupable && FlatGroup::eligible(fm, n, k)) {
                        if (!sc.group) sc.group.reset(new FlatGroup(dev));
                        const size_t m = members.size();
                        bool contiguous = true;
                        for (size_t j = 1; j < m; ++j) contiguous = contiguous && members[j] == members[0] + static_cast<int>(j);
                        const bool direct = merged && dev == dev0 && contiguous;
                        float* gD = direct ? allD + per * members[0] : static_cast<float*>(sc.gD.ensure(per * m * 4));
                        int64_t* gI = direct ? allI + per * members[0] : static_cast<int64_t*>(sc.gI.ensure(per * m * 8));
                        sc.group->search_device(fm, n, dq, k, gD, gI, st);
                        if (!direct) {
                            const cudaMemcpyKind kind = merged ? cudaMemcpyDefault : cudaMemcpyDeviceToHost;
                            float* dstD = merged ? allD : D;
                            int64_t* dstI = merged ? allI : I;
                            if (contiguous) {
                                B200_CUDA_CHECK(cudaMemcpyAsync(dstD + per * members[0], gD, per * m * 4, kind, st));
                                B200_CUDA_CHECK(cudaMemcpyAsync(dstI + per * members[0], gI, per * m * 8, kind, st));
                            } else {
                                for (size_t j = 0; j < m; ++j) {
                                    B200_CUDA_CHECK(cudaMemcpyAsync(dstD + per * members[j], gD + per * j, per * 4, kind, st));
                                    B200_CUDA_CHECK(cudaMemcpyAsync(dstI + per * members[j], gI + per * j, per * 8, kind, st));
                                }
                            }
                            B200_CUDA_CHECK(cudaStreamSynchronize(st));
                        }
                        return;
                    }
                    for (int i : members) {
                        b200idx_index* h = hs[i];
                        // with merged results on this device the member writes its slice directly
                        float* oD = (merged && dev == dev0) ? allD + per * i : dD;
                        int64_t* oI = (merged && dev == dev0) ? allI + per * i : dI;
                        if (h->kind == 2) h->ivfpq->search_device(n, static_cast<const float*>(dq), k, oD, oI);
                        else h->flat->search_device(n, dq, false, k, oD, oI, k);
                        if (merged && dev != dev0) {
                            B200_CUDA_CHECK(cudaMemcpyAsync(allD + per * i, dD, per * 4, cudaMemcpyDefault, st));
                            B200_CUDA_CHECK(cudaMemcpyAsync(allI + per * i, dI, per * 8, cudaMemcpyDefault, st));
                            B200_CUDA_CHECK(cudaStreamSynchronize(st));
                        } else if (!merged) {
                            B200_CUDA_CHECK(cudaMemcpyAsync(D + per * i, dD, per * 4, cudaMemcpyDeviceToHost, st));
                            B200_CUDA_CHECK(cudaMemcpyAsync(I + per * i, dI, per * 8, cudaMemcpyDeviceToHost, st));
                            B200_CUDA_CHECK(cudaStreamSynchronize(st));
                        }
                    }
                } catch (const std::exception& e) {
                    *err = e.what();
                    cudaGetLastError();
                }
            };
            if (groups.size() == 1) body();
            else workers.emplace_back(body);
        }
        for (auto& w : workers) w.join();
        for (auto& e : errors)
            if (!e.empty()) throw std::runtime_error(e);
        if (merged) {
            DeviceGuard g(dev0);
            cudaStream_t st = static_cast<cudaStream_t>(b200idx_stream(h0));
            float* mD = static_cast<float*>(s0.mD.ensure(per * 4));
            int64_t* mI = static_cast<int64_t*>(s0.mI.ensure(per * 8));
            B200_CUDA_CHECK(launch_merge_topk(nh, n, k, descending_of(h0) ? 1 : 0, allD, allI, mD, mI, st));
            B200_CUDA_CHECK(cudaMemcpyAsync(D, mD, per * 4, cudaMemcpyDeviceToHost, st));
            B200_CUDA_CHECK(cudaMemcpyAsync(I, mI, per * 8, cudaMemcpyDeviceToHost, st));
            B200_CUDA_CHECK(cudaStreamSynchronize(st));
        }
    }, /*lock=*/false);
}

int b200idx_search_multi_stats(int device, uint64_t* group_launches, uint64_t* group_rebuilds) {
    MultiScratch& sc = multi_scratch(device);
    std::lock_guard<std::mutex> l(sc.mu);
    if (group_launches) *group_launches = sc.group ? sc.group->launches() : 0;
    if (group_rebuilds) *group_rebuilds = sc.group ? sc.group->rebuilds() : 0;
    return B200IDX_OK;
}

int b200idx_merge_topk_device(int nsrc, int64_t n, int k, int descending, const float* Din, const int64_t* Iin,
                              float* D, int64_t* I, void* stream) {
    if (nsrc <= 0 || n <= 0 || k <= 0 || !Din || !Iin || !D || !I) return B200IDX_ERR_INVALID_PARAM;
    cudaError_t e = launch_merge_topk(nsrc, n, k, descending, Din, Iin, D, I, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? B200IDX_OK : B200IDX_ERR_INNER;
}

int b200idx_merge_topk_device_strided(int nsrc, int64_t n, int k, int descending, const float* Din, const int64_t* Iin,
                                      int64_t src_stride_bytes, float* D, int64_t* I, void* stream) {
    if (nsrc <= 0 || n <= 0 || k <= 0 || !Din || !Iin || !D || !I) return B200IDX_ERR_INVALID_PARAM;
    if (src_stride_bytes <= 0 || src_stride_bytes % 8 != 0) return B200IDX_ERR_INVALID_PARAM;
    cudaError_t e = launch_merge_topk(nsrc, n, k, descending, Din, Iin, D, I, static_cast<cudaStream_t>(stream),
                                      src_stride_bytes / 4, src_stride_bytes / 8);
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
int b200idx_kmeans(int device, int d, int64_t n, const float* x, int k, int niter, uint64_t seed, float* centroids) {
    return guarded_create([&] {
        if (!x || !centroids) throw std::invalid_argument("x and centroids can not be nullptr.");
        if (d <= 0 || n <= 0 || k <= 0 || niter < 0 || k > n) throw std::invalid_argument("k-means: need d > 0, 0 < k <= n, niter >= 0");
        DeviceGuard g(device);
        DeviceBuffer xd, cd;
        float* xdev = static_cast<float*>(xd.ensure(static_cast<size_t>(n) * d * 4));
        float* cdev = static_cast<float*>(cd.ensure(static_cast<size_t>(k) * d * 4));
        B200_CUDA_CHECK(cudaMemcpy(xdev, x, static_cast<size_t>(n) * d * 4, cudaMemcpyHostToDevice));
        kmeans_device(device, d, n, xdev, k, niter, seed, cdev, nullptr);
        B200_CUDA_CHECK(cudaMemcpy(centroids, cdev, static_cast<size_t>(k) * d * 4, cudaMemcpyDeviceToHost));
    });
}
int b200idx_ivfpq_train(b200idx_t* h, int64_t n, const float* x, int niter, uint64_t seed) {
    B200_REQUIRE_IVFPQ(h)
    return guarded(h, [&] {
        if (n <= 0 || !x) throw std::invalid_argument("n must be > 0, x non-NULL");
        if (niter < 0) throw std::invalid_argument("niter must be >= 0");
        if (h->ivfpq->ntotal() != 0) throw std::invalid_argument("train: the index already holds vectors");
        h->ivfpq->train(n, x, niter, seed);
    });
}
int b200idx_ivfpq_get_list(const b200idx_t* h, int list, uint8_t* codes, int64_t* ids) {
    B200_REQUIRE_IVFPQ(h)
    return guarded(h, [&] { h->ivfpq->get_list(list, codes, ids); });
}

// ---------------------------------------------------------------------------------------
// Native file format (little-endian):
//   "B2IX" | u32 version = 1 | u32 kind (0 Flat, 1 Int8Flat, 2 IVFPQ) | i32 d | i32 metric | i32 dtype | i64 ntotal
//   Flat / Int8Flat : ntotal rows in the index's storage dtype (fp32, fp16 or int8) | ntotal int64 labels
//   IVFPQ           : i32 nlist | i32 M | i32 nbits | i32 by_residual | i32 nprobe | i32 trained |
//                     centroids [nlist][d] fp32 | codebooks [M][256][d/M] fp32 |
//                     per list: i64 length | codes [length][M] (canonical byte order) | ids [length]
// ---------------------------------------------------------------------------------------
}  // extern "C"
namespace {
struct FileCloser {
    void operator()(FILE* f) const { if (f) std::fclose(f); }
};
using FilePtr = std::unique_ptr<FILE, FileCloser>;

void put(FILE* f, const void* p, size_t n) {
    if (n && std::fwrite(p, 1, n, f) != n) throw std::runtime_error("write failed");
}
void get(FILE* f, void* p, size_t n) {
    if (n && std::fread(p, 1, n, f) != n) throw std::runtime_error("file is truncated");
}
template <typename T>
void put_v(FILE* f, T v) { put(f, &v, sizeof(T)); }
template <typename T>
T get_v(FILE* f) { T v; get(f, &v, sizeof(T)); return v; }
size_t storage_elem_bytes(int dtype) { return dtype == kI8 ? 1 : (dtype == kF16 ? 2 : 4); }
}  // namespace
extern "C" {

int b200idx_save(const b200idx_t* h, const char* path) {
    if (!h || !path) return B200IDX_ERR_INVALID_PARAM;
    return guarded(h, [&] {
        FilePtr f(std::fopen(path, "wb"));
        if (!f) throw std::invalid_argument(std::string("cannot open for writing: ") + path);
        put(f.get(), "B2IX", 4);
        put_v<uint32_t>(f.get(), 1u);
        put_v<uint32_t>(f.get(), static_cast<uint32_t>(h->kind));
        if (h->kind != 2) {
            const FlatIndex& ix = *h->flat;
            put_v<int32_t>(f.get(), ix.d());
            put_v<int32_t>(f.get(), ix.metric());
            put_v<int32_t>(f.get(), ix.dtype());
            put_v<int64_t>(f.get(), ix.ntotal());
            const size_t row = static_cast<size_t>(ix.d()) * storage_elem_bytes(ix.dtype());
            const int64_t chunk = std::max<int64_t>(1, (int64_t(64) << 20) / static_cast<int64_t>(row));
            std::vector<uint8_t> buf;
            for (int64_t o = 0; o < ix.ntotal(); o += chunk) {
                const int64_t m = std::min(chunk, ix.ntotal() - o);
                buf.resize(static_cast<size_t>(m) * row);
                ix.get_base(o, m, buf.data());
                put(f.get(), buf.data(), buf.size());
            }
            std::vector<int64_t> ids(static_cast<size_t>(ix.ntotal()));
            if (!ids.empty()) ix.get_labels(0, ix.ntotal(), ids.data());
            put(f.get(), ids.data(), ids.size() * 8);
        } else {
            const IvfpqIndex& ix = *h->ivfpq;
            put_v<int32_t>(f.get(), ix.d());
            put_v<int32_t>(f.get(), B200IDX_METRIC_L2);
            put_v<int32_t>(f.get(), 0);
            put_v<int64_t>(f.get(), ix.ntotal());
            put_v<int32_t>(f.get(), ix.nlist());
            put_v<int32_t>(f.get(), ix.M());
            put_v<int32_t>(f.get(), 8);
            put_v<int32_t>(f.get(), ix.by_residual() ? 1 : 0);
            put_v<int32_t>(f.get(), ix.nprobe());
            put_v<int32_t>(f.get(), ix.is_trained() ? 1 : 0);
            if (ix.is_trained()) {
                std::vector<float> c(static_cast<size_t>(ix.nlist()) * ix.d()), cb(static_cast<size_t>(256) * ix.d());
                ix.get_centroids(c.data());
                ix.get_codebooks(cb.data());
                put(f.get(), c.data(), c.size() * 4);
                put(f.get(), cb.data(), cb.size() * 4);
                std::vector<uint8_t> codes;
                std::vector<int64_t> ids;
                for (int l = 0; l < ix.nlist(); ++l) {
                    const int64_t len = ix.list_length(l);
                    put_v<int64_t>(f.get(), len);
                    codes.resize(static_cast<size_t>(len) * ix.M());
                    ids.resize(static_cast<size_t>(len));
                    if (len) ix.get_list(l, codes.data(), ids.data());
                    put(f.get(), codes.data(), codes.size());
                    put(f.get(), ids.data(), ids.size() * 8);
                }
            }
        }
        if (std::fflush(f.get()) != 0) throw std::runtime_error("write failed");
    });
}

int b200idx_load(const char* path, int device, b200idx_t** out) {
    if (!path || !out) return B200IDX_ERR_INVALID_PARAM;
    *out = nullptr;
    b200idx_t* h = nullptr;
    const int code = guarded_create([&] {
        FilePtr f(std::fopen(path, "rb"));
        if (!f) throw std::invalid_argument(std::string("cannot open for reading: ") + path);
        char magic[4];
        get(f.get(), magic, 4);
        if (std::memcmp(magic, "B2IX", 4) != 0 || get_v<uint32_t>(f.get()) != 1u)
            throw std::invalid_argument("not an index file of this library (or an unknown version)");
        const uint32_t kind = get_v<uint32_t>(f.get());
        const int d = get_v<int32_t>(f.get());
        const int metric = get_v<int32_t>(f.get());
        const int dtype = get_v<int32_t>(f.get());
        const int64_t ntotal = get_v<int64_t>(f.get());
        if (kind > 2 || ntotal < 0) throw std::invalid_argument("corrupt index file");
        int rc;
        if (kind == 0) rc = b200idx_create_flat(d, metric, dtype == kF16 ? B200IDX_F16 : B200IDX_F32, device, &h);
        else if (kind == 1) rc = b200idx_create_int8flat(d, metric, device, &h);
        else {
            const int nlist = get_v<int32_t>(f.get()), M = get_v<int32_t>(f.get()), nbits = get_v<int32_t>(f.get());
            const int by_res = get_v<int32_t>(f.get());
            rc = b200idx_create_ivfpq(d, metric, nlist, M, nbits, by_res, device, &h);
        }
        if (rc != B200IDX_OK) throw std::invalid_argument(std::string("corrupt index file: ") + b200idx_last_error(nullptr));
        if (kind != 2) {
            const size_t row = static_cast<size_t>(d) * storage_elem_bytes(h->flat->dtype());
            const int64_t chunk = std::max<int64_t>(1, (int64_t(64) << 20) / static_cast<int64_t>(row));
            std::vector<uint8_t> rows(static_cast<size_t>(std::min<int64_t>(chunk, std::max<int64_t>(ntotal, 1))) * row);
            // labels follow the rows: read them first
            const long rows_at = std::ftell(f.get());
            if (std::fseek(f.get(), rows_at + static_cast<long>(static_cast<size_t>(ntotal) * row), SEEK_SET) != 0)
                throw std::runtime_error("file is truncated");
            std::vector<int64_t> ids(static_cast<size_t>(ntotal));
            get(f.get(), ids.data(), ids.size() * 8);
            if (std::fseek(f.get(), rows_at, SEEK_SET) != 0) throw std::runtime_error("seek failed");
            for (int64_t o = 0; o < ntotal; o += chunk) {
                const int64_t m = std::min(chunk, ntotal - o);
                get(f.get(), rows.data(), static_cast<size_t>(m) * row);
                h->flat->add(m, rows.data(), h->flat->dtype() == kF16, ids.data() + o, false);
            }
        } else {
            IvfpqIndex& ix = *h->ivfpq;
            ix.set_nprobe(get_v<int32_t>(f.get()));
            const int trained = get_v<int32_t>(f.get());
            if (trained) {
                std::vector<float> c(static_cast<size_t>(ix.nlist()) * d), cb(static_cast<size_t>(256) * d);
                get(f.get(), c.data(), c.size() * 4);
                get(f.get(), cb.data(), cb.size() * 4);
                ix.set_centroids(c.data());
                ix.set_codebooks(cb.data());
                std::vector<uint8_t> codes;
                std::vector<int64_t> ids;
                std::vector<int32_t> ln;
                for (int l = 0; l < ix.nlist(); ++l) {
                    const int64_t len = get_v<int64_t>(f.get());
                    if (len < 0) throw std::invalid_argument("corrupt index file");
                    const size_t at = ln.size();
                    ln.resize(at + static_cast<size_t>(len), l);
                    codes.resize((at + static_cast<size_t>(len)) * ix.M());
                    ids.resize(at + static_cast<size_t>(len));
                    get(f.get(), codes.data() + at * ix.M(), static_cast<size_t>(len) * ix.M());
                    get(f.get(), ids.data() + at, static_cast<size_t>(len) * 8);
                    if (ln.size() >= (size_t(1) << 22) || l + 1 == ix.nlist()) {   // add in batches, list order kept
                        if (!ln.empty()) ix.add_codes(static_cast<int64_t>(ln.size()), ln.data(), codes.data(), ids.data());
                        ln.clear();
                        codes.clear();
                        ids.clear();
                    }
                }
            }
        }
    });
    if (code != B200IDX_OK) {
        if (h) b200idx_destroy(h);
        return code;
    }
    *out = h;
    return B200IDX_OK;
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
    out->second_pass_queries = s.second_pass_queries;
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

int b200idx_status_of_message(const char* message) {
    if (!message) return B200IDX_ERR_INVALID_PARAM;
    return status_of_error(message);
}

const char* b200idx_version(void) { return "b200idx 0.1 (sm_100a)"; }

}  // extern "C"
