// faiss::ascend classes of include/b200/ascend_api.h over the b200idx C ABI: parameter checks
// with the reference's messages, near-even split of added vectors over the device list,
// fan-out / merge through b200idx_search_multi, copyFrom / copyTo against the CPU structs.
// Reference behaviour followed (FR = feature_retrieval/src/ascendfaiss):
//   checks and messages  FR/ascend/impl/AscendIndexImpl.cpp:696-726, AscendIndexImpl.h:216-237,
//                        AscendIndexFlatImpl.cpp:88-93, AscendIndexInt8FlatImpl.cpp:64-75,
//                        AscendIndexIVFPQImpl.cpp:510-525, AscendMultiIndexSearch.cpp:55-69
//   add split            FR/ascend/impl/AscendIndexImpl.cpp:175-200 (calcAddMap)
//   locking              MX_INDEX_MULTITHREAD=1: shared lock for search, exclusive for mutation
//                        (FR/ascend/impl/AscendIndexImpl.h:62,230)
#include "../../../include/b200/ascend_api.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <random>
#include <shared_mutex>
#include <thread>
#include <string>

#include "../../../include/b200idx.h"

namespace faiss {
namespace ascend {
namespace {

bool g_relaxed = false;
bool env_is(const char* name, const char* v) {
    const char* e = std::getenv(name);
    return e && std::strcmp(e, v) == 0;
}
const std::vector<int> kFlatDims = {32, 64, 128, 256, 384, 512, 768, 1024, 1408, 1536, 2048, 3072, 3584, 4096};
const std::vector<int> kInt8Dims = {64, 128, 256, 384, 512, 768, 1024};
const std::vector<uint32_t> kInt8Blocks = {16384, 32768, 65536, 131072, 262144};
const std::vector<int> kPqDims = {128};
const std::vector<int> kPqNlists = {1024, 2048, 4096, 8192, 16384, 262144, 524288};
const std::vector<int> kPqMsubs = {2, 4, 8, 16, 32};
template <typename T>
bool in(const std::vector<T>& v, T x) { return std::find(v.begin(), v.end(), x) != v.end(); }

constexpr int kMaxDim = 4096, kDimDivisor = 16;
constexpr size_t kMaxDevices = 64;
constexpr int64_t kMaxResource = 10240LL * 1024 * 1024;

void check_common(int dims, const std::vector<int>& devices, int64_t resourceSize) {
    FAISS_THROW_IF_NOT_FMT(dims > 0 && dims <= kMaxDim, "Invalid number of dimensions(%d), should be (0, %d]", dims, kMaxDim);
    FAISS_THROW_IF_NOT_FMT(dims % kDimDivisor == 0, "Invalid number of dimensions(%d), should be divisible by %d", dims,
                           kDimDivisor);
    FAISS_THROW_IF_NOT_FMT(!devices.empty() && devices.size() <= kMaxDevices, "device list should be in range (0, %zu]!",
                           kMaxDevices);
    std::vector<int> u(devices);
    std::sort(u.begin(), u.end());
    FAISS_THROW_IF_NOT_MSG(std::adjacent_find(u.begin(), u.end()) == u.end(), "some device IDs are the same");
    FAISS_THROW_IF_NOT_FMT(resourceSize == -1 || (resourceSize >= 0 && resourceSize <= kMaxResource),
                           "resourceSize:%ld should be -1 or in range [0, 10240MB]!", static_cast<long>(resourceSize));
}

int to_abi_metric(MetricType m) { return m == METRIC_L2 ? B200IDX_METRIC_L2 : B200IDX_METRIC_INNER_PRODUCT; }

struct RwGuard {   // no-op unless MX_INDEX_MULTITHREAD=1
    RwGuard(std::shared_mutex& m, bool exclusive) : m_(m), ex_(exclusive), on_(env_is("MX_INDEX_MULTITHREAD", "1")) {
        if (!on_) return;
        if (ex_) m_.lock();
        else m_.lock_shared();
    }
    ~RwGuard() {
        if (!on_) return;
        if (ex_) m_.unlock();
        else m_.unlock_shared();
    }
    std::shared_mutex& m_;
    bool ex_, on_;
};

}  // namespace

void SetRelaxedLimits(bool on) { g_relaxed = on; }
namespace {
bool g_int8_ip_cosine = false;
}
void SetInt8InnerProductAsCosine(bool on) { g_int8_ip_cosine = on; }
bool Int8InnerProductAsCosine() { return g_int8_ip_cosine || env_is("B200IDX_INT8_IP_COSINE", "1"); }
bool RelaxedLimits() { return g_relaxed || env_is("B200IDX_RELAXED", "1"); }

// One object per index: the handles of its device list.
class IndexImplBase {
public:
    virtual ~IndexImplBase() {
        for (b200idx_t* h : handles) b200idx_destroy(h);
    }
    std::vector<int> devices;
    std::vector<b200idx_t*> handles;
    mutable std::shared_mutex mutex;
    int dims = 0;
    MetricType metric = METRIC_L2;

    void rc(int code, b200idx_t* h, const char* what) const {
        if (code != B200IDX_OK) FAISS_THROW_FMT("%s failed (%d): %s", what, code, b200idx_last_error(h));
    }
    // Query-parallel layout (AscendIndexIVFPQConfig::enableQueryParallelSearch, FR/ascend/impl/
    // AscendIndexIVFPQImpl.cpp:323-333 replication, :1305-1328 search): every device holds the WHOLE
    // index and a search splits the QUERIES over the devices instead of the base.
    bool replicated = false;
    idx_t total() const {
        if (replicated) return handles.empty() ? 0 : b200idx_ntotal(handles[0]);
        idx_t t = 0;
        for (b200idx_t* h : handles) t += b200idx_ntotal(h);
        return t;
    }
    // near-even split, the remainder going to the least-loaded devices first
    std::vector<idx_t> split(idx_t n) const {
        const size_t nd = handles.size();
        std::vector<idx_t> cnt(nd, n / static_cast<idx_t>(nd));
        std::vector<size_t> order(nd);
        for (size_t i = 0; i < nd; ++i) order[i] = i;
        std::stable_sort(order.begin(), order.end(),
                         [&](size_t a, size_t b) { return b200idx_ntotal(handles[a]) < b200idx_ntotal(handles[b]); });
        for (idx_t r = 0; r < n % static_cast<idx_t>(nd); ++r) cnt[order[static_cast<size_t>(r)]] += 1;
        return cnt;
    }
    void add_rows(idx_t n, const void* x, size_t row_bytes, const idx_t* ids, bool f16) {
        if (replicated) {
            for (b200idx_t* h : handles)
                rc(f16 ? b200idx_add_f16(h, n, static_cast<const uint16_t*>(x), ids) : b200idx_add(h, n, x, ids), h, "add");
            return;
        }
        const std::vector<idx_t> cnt = split(n);
        idx_t off = 0;
        for (size_t i = 0; i < handles.size(); ++i) {
            if (cnt[i] == 0) continue;
            const uint8_t* xp = static_cast<const uint8_t*>(x) + static_cast<size_t>(off) * row_bytes;
            const int code = f16 ? b200idx_add_f16(handles[i], cnt[i], reinterpret_cast<const uint16_t*>(xp), ids + off)
                                 : b200idx_add(handles[i], cnt[i], xp, ids + off);
            rc(code, handles[i], "add");
            off += cnt[i];
        }
    }
    void search_rows(idx_t n, const void* x, idx_t k, float* D, idx_t* I, bool f16) const {
        if (handles.size() == 1) {
            const int code = f16 ? b200idx_search_f16(handles[0], n, static_cast<const uint16_t*>(x), static_cast<int>(k), D, I)
                                 : b200idx_search(handles[0], n, x, static_cast<int>(k), D, I);
            rc(code, handles[0], "search");
            return;
        }
        // fp16 queries: widened on the host (exact); an fp16-storage index rounds them back to the same bits
        std::vector<float> wide;
        if (f16) {
            const uint16_t* xh = static_cast<const uint16_t*>(x);
            wide.resize(static_cast<size_t>(n) * dims);
            for (size_t i = 0; i < wide.size(); ++i) {
                _Float16 v;
                std::memcpy(&v, xh + i, 2);
                wide[i] = static_cast<float>(v);
            }
            x = wide.data();
        }
        if (replicated) {
            // near-even slices of the queries, one worker per device
            const size_t nd = std::min<size_t>(handles.size(), static_cast<size_t>(n));
            const size_t row = static_cast<size_t>(dims) * row_elem_bytes;
            std::vector<std::string> errs(nd);
            std::vector<std::thread> workers;
            for (size_t i = 0; i < nd; ++i) {
                const idx_t lo = n * static_cast<idx_t>(i) / static_cast<idx_t>(nd);
                const idx_t hi = n * static_cast<idx_t>(i + 1) / static_cast<idx_t>(nd);
                workers.emplace_back([=, &errs] {
                    const int code = b200idx_search(handles[i], hi - lo, static_cast<const uint8_t*>(x) + static_cast<size_t>(lo) * row,
                                                    static_cast<int>(k), D + lo * k, I + lo * k);
                    if (code != B200IDX_OK) errs[i] = b200idx_last_error(handles[i]);
                });
            }
            for (auto& w : workers) w.join();
            for (auto& e : errs)
                if (!e.empty()) FAISS_THROW_FMT("search failed: %s", e.c_str());
            return;
        }
        rc(b200idx_search_multi(handles.data(), static_cast<int>(handles.size()), n, x, static_cast<int>(k), D, I, 1),
           handles[0], "search");
    }
    size_t row_elem_bytes = sizeof(float);   // bytes per query component (1 for the int8 index)
    void reset_all() {
        for (b200idx_t* h : handles) rc(b200idx_reset(h), h, "reset");
    }
    int slot_of(int deviceId) const {
        for (size_t i = 0; i < devices.size(); ++i)
            if (devices[i] == deviceId) return static_cast<int>(i);
        FAISS_THROW_FMT("deviceId %d is not in the device list of this index", deviceId);
    }
};

// All state of a float index lives in AscendIndexImpl (created by the AscendIndex constructor);
// the per-class Impl types the headers name are views onto it.
class AscendIndexImpl : public IndexImplBase {
public:
    bool store_f16 = true;   // Flat: the reference's fp16 storage unless B200IDX_FLAT_FP32=1
    bool ivfpq = false;
    int nlist = 0, nprobe = 64, msubs = 0, nbits = 8;
    bool by_residual = false;
    std::vector<float> centroids, codebooks;
};
class AscendIndexFlatImpl { public: AscendIndexImpl* core = nullptr; };
class AscendIndexIVFImpl { public: AscendIndexImpl* core = nullptr; };
class AscendIndexIVFPQImpl { public: AscendIndexImpl* core = nullptr; };
class AscendIndexInt8Impl : public IndexImplBase {};
class AscendIndexInt8FlatImpl { public: AscendIndexInt8Impl* core = nullptr; };

namespace {
float half_bits_to_float(uint16_t h) {
    _Float16 v;
    std::memcpy(&v, &h, 2);
    return static_cast<float>(v);
}
void check_search_args(idx_t n, const void* x, idx_t k, const float* D, const idx_t* I, bool trained) {
    FAISS_THROW_IF_NOT_FMT((n > 0) && (n < MAX_N), "n must be > 0 and < %ld", static_cast<long>(MAX_N));
    FAISS_THROW_IF_NOT_FMT((k > 0) && (k <= MAX_K), "k must be > 0 and <= %ld", static_cast<long>(MAX_K));
    FAISS_THROW_IF_NOT_MSG(x != nullptr, "x cannot be nullptr.");
    FAISS_THROW_IF_NOT_MSG(D != nullptr, "distance cannot be nullptr.");
    FAISS_THROW_IF_NOT_MSG(I != nullptr, "labels cannot be nullptr.");
    FAISS_THROW_IF_NOT_MSG(trained, "Index not trained");
}
std::vector<idx_t> auto_ids(idx_t start, idx_t n) {
    std::vector<idx_t> ids(static_cast<size_t>(n));
    for (idx_t i = 0; i < n; ++i) ids[static_cast<size_t>(i)] = start + i;
    return ids;
}
}  // namespace

// ------------------------------------------------------------------ AscendIndex
AscendIndex::AscendIndex(int dims, faiss::MetricType metric, AscendIndexConfig config)
    : Index(dims, metric), impl_(std::make_shared<AscendIndexImpl>()) {
    check_common(dims, config.deviceList, config.resourceSize);
    impl_->devices = config.deviceList;
    impl_->dims = dims;
    impl_->metric = metric;
    impl_->store_f16 = !env_is("B200IDX_FLAT_FP32", "1");
}
AscendIndex::~AscendIndex() {}

void AscendIndex::add(idx_t n, const float* x) { add_with_ids(n, x, nullptr); }

void AscendIndex::add_with_ids(idx_t n, const float* x, const idx_t* ids) {
    RwGuard g(impl_->mutex, true);
    FAISS_THROW_IF_NOT_FMT((n > 0) && (n < MAX_N), "n must be > 0 and < %ld", static_cast<long>(MAX_N));
    FAISS_THROW_IF_NOT_MSG(x != nullptr, "x cannot be nullptr.");
    FAISS_THROW_IF_NOT_MSG(is_trained, "Index not trained");
    FAISS_THROW_IF_NOT_FMT(ntotal + n < MAX_N, "ntotal must be < %ld after add", static_cast<long>(MAX_N));
    std::vector<idx_t> gen;
    if (!ids) {
        gen = auto_ids(ntotal, n);
        ids = gen.data();
    }
    impl_->add_rows(n, x, static_cast<size_t>(d) * sizeof(float), ids, false);
    ntotal = impl_->total();
}

void AscendIndex::add(idx_t n, const uint16_t* x) { add_with_ids(n, x, nullptr); }

void AscendIndex::add_with_ids(idx_t n, const uint16_t* x, const idx_t* ids) {
    RwGuard g(impl_->mutex, true);
    FAISS_THROW_IF_NOT_FMT((n > 0) && (n < MAX_N), "n must be > 0 and < %ld", static_cast<long>(MAX_N));
    FAISS_THROW_IF_NOT_MSG(x != nullptr, "x cannot be nullptr.");
    FAISS_THROW_IF_NOT_MSG(!impl_->ivfpq && impl_->store_f16, "fp16 input needs a Flat index with fp16 storage");
    std::vector<idx_t> gen;
    if (!ids) {
        gen = auto_ids(ntotal, n);
        ids = gen.data();
    }
    impl_->add_rows(n, x, static_cast<size_t>(d) * 2, ids, true);
    ntotal = impl_->total();
}

void AscendIndex::search(idx_t n, const float* x, idx_t k, float* distances, idx_t* labels,
                         const SearchParameters*) const {
    RwGuard g(impl_->mutex, false);
    check_search_args(n, x, k, distances, labels, is_trained);
    if (impl_->ivfpq && !RelaxedLimits())
        FAISS_THROW_IF_NOT_FMT(k <= 320, "k must be > 0 and <= %d for IVFPQ", 320);
    impl_->search_rows(n, x, k, distances, labels, false);
}

void AscendIndex::search(idx_t n, const uint16_t* x, idx_t k, float* distances, idx_t* labels) const {
    RwGuard g(impl_->mutex, false);
    check_search_args(n, x, k, distances, labels, is_trained);
    FAISS_THROW_IF_NOT_MSG(!impl_->ivfpq && impl_->store_f16, "fp16 queries need a Flat index with fp16 storage");
    impl_->search_rows(n, x, k, distances, labels, true);
}

size_t AscendIndex::remove_ids(const faiss::IDSelector& sel) {
    RwGuard g(impl_->mutex, true);
    size_t removed = 0;
    for (b200idx_t* h : impl_->handles) {
        std::vector<idx_t> ids;
        if (impl_->ivfpq) {
            for (int l = 0; l < impl_->nlist; ++l) {
                const int64_t len = b200idx_ivfpq_list_length(h, l);
                if (len <= 0) continue;
                std::vector<idx_t> li(static_cast<size_t>(len));
                impl_->rc(b200idx_ivfpq_get_list(h, l, nullptr, li.data()), h, "get_list");
                ids.insert(ids.end(), li.begin(), li.end());
            }
        } else {
            ids.resize(static_cast<size_t>(b200idx_ntotal(h)));
            if (!ids.empty()) impl_->rc(b200idx_get_ids(h, 0, static_cast<int64_t>(ids.size()), ids.data()), h, "get_ids");
        }
        std::vector<idx_t> hit;
        for (idx_t id : ids)
            if (sel.is_member(id)) hit.push_back(id);
        if (hit.empty()) continue;
        int64_t r = 0;
        impl_->rc(b200idx_remove_ids(h, static_cast<int64_t>(hit.size()), hit.data(), &r), h, "remove_ids");
        if (!impl_->replicated || h == impl_->handles[0]) removed += static_cast<size_t>(r);   // replicas hold the same rows
    }
    ntotal = impl_->total();
    return removed;
}

void AscendIndex::reserveMemory(size_t) {}            // storage grows geometrically on add
size_t AscendIndex::reclaimMemory() { return 0; }
void AscendIndex::reset() {
    RwGuard g(impl_->mutex, true);
    impl_->reset_all();
    ntotal = 0;
}
std::vector<int> AscendIndex::getDeviceList() { return impl_->devices; }
IndexImplBase& AscendIndex::GetIndexImplBase() const { return *impl_; }

// ------------------------------------------------------------------ AscendIndexFlat
namespace {
void create_flat_handles(AscendIndexImpl& im) {
    for (int dev : im.devices) {
        b200idx_t* h = nullptr;
        const int code = b200idx_create_flat(im.dims, to_abi_metric(im.metric), im.store_f16 ? B200IDX_F16 : B200IDX_F32,
                                             dev, &h);
        if (code != B200IDX_OK) FAISS_THROW_FMT("create index failed (%d): %s", code, b200idx_last_error(nullptr));
        im.handles.push_back(h);
    }
}
void check_flat_params(int dims, MetricType metric) {
    FAISS_THROW_IF_NOT_MSG(metric == METRIC_L2 || metric == METRIC_INNER_PRODUCT, "Unsupported metric type");
    if (!RelaxedLimits()) FAISS_THROW_IF_NOT_MSG(in(kFlatDims, dims), "Unsupported dims");
}
}  // namespace

AscendIndexFlat::AscendIndexFlat(int dims, faiss::MetricType metric, AscendIndexFlatConfig config)
    : AscendIndex(dims, metric, config), impl_(std::make_shared<AscendIndexFlatImpl>()) {
    check_flat_params(dims, metric);
    impl_->core = AscendIndex::impl_.get();
    create_flat_handles(*impl_->core);
    is_trained = true;
}

AscendIndexFlat::AscendIndexFlat(const faiss::IndexFlat* index, AscendIndexFlatConfig config)
    : AscendIndex(index ? index->d : 128, index ? index->metric_type : METRIC_L2, config),   // 128: let the nullptr check below speak
      impl_(std::make_shared<AscendIndexFlatImpl>()) {
    FAISS_THROW_IF_NOT_MSG(index != nullptr, "Invalid index nullptr.");
    check_flat_params(index->d, index->metric_type);
    impl_->core = AscendIndex::impl_.get();
    create_flat_handles(*impl_->core);
    copyFrom(index);
}

AscendIndexFlat::AscendIndexFlat(const faiss::IndexIDMap* index, AscendIndexFlatConfig config)
    : AscendIndex((index && index->index) ? index->index->d : 128,
                  (index && index->index) ? index->index->metric_type : METRIC_L2, config),
      impl_(std::make_shared<AscendIndexFlatImpl>()) {
    FAISS_THROW_IF_NOT_MSG(index != nullptr && index->index != nullptr, "Invalid index nullptr.");
    check_flat_params(index->index->d, index->index->metric_type);
    impl_->core = AscendIndex::impl_.get();
    create_flat_handles(*impl_->core);
    copyFrom(index);
}

AscendIndexFlat::~AscendIndexFlat() {}

void AscendIndexFlat::copyFrom(const faiss::IndexFlat* index) {
    FAISS_THROW_IF_NOT_MSG(index != nullptr, "Invalid index nullptr.");
    FAISS_THROW_IF_NOT_MSG(index->d == d && index->metric_type == metric_type, "the dim and metric type must be same");
    FAISS_THROW_IF_NOT_FMT((index->ntotal >= 0) && (index->ntotal < MAX_N), "ntotal must be >= 0 and < %ld",
                           static_cast<long>(MAX_N));
    FAISS_THROW_IF_NOT_MSG(index->codes.size() == static_cast<size_t>(index->ntotal) * d * sizeof(float),
                           "The size of xb must be equal to ntotal * dim.\n");
    reset();
    if (index->ntotal > 0) add(index->ntotal, index->get_xb());
}

void AscendIndexFlat::copyFrom(const faiss::IndexIDMap* index) {
    FAISS_THROW_IF_NOT_MSG(index != nullptr && index->index != nullptr, "Invalid index nullptr.");
    const faiss::IndexFlat* flat = dynamic_cast<const faiss::IndexFlat*>(index->index);
    FAISS_THROW_IF_NOT_MSG(flat != nullptr, "Invalid flatIndex nullptr.");
    FAISS_THROW_IF_NOT_MSG(index->id_map.size() == static_cast<size_t>(flat->ntotal),
                           "The size of id_map must be equal to ntotal.\n");
    FAISS_THROW_IF_NOT_MSG(flat->d == d && flat->metric_type == metric_type, "the dim and metric type must be same");
    reset();
    if (flat->ntotal > 0) add_with_ids(flat->ntotal, flat->get_xb(), index->id_map.data());
}

size_t AscendIndexFlat::getBaseSize(int deviceId) const {
    return static_cast<size_t>(b200idx_ntotal(impl_->core->handles[static_cast<size_t>(impl_->core->slot_of(deviceId))]));
}

// floats, [getBaseSize(deviceId)][d]; with fp16 storage they are the stored halves widened
// (lossy by design, as in the reference: FR/ascend/impl/AscendIndexFlatImpl.cpp:394-405)
void AscendIndexFlat::getBase(int deviceId, char* xb) const {
    FAISS_THROW_IF_NOT_MSG(xb != nullptr, "xb cannot be nullptr.");
    b200idx_t* h = impl_->core->handles[static_cast<size_t>(impl_->core->slot_of(deviceId))];
    const int64_t n = b200idx_ntotal(h);
    if (n == 0) return;
    float* out = reinterpret_cast<float*>(xb);
    if (impl_->core->store_f16) {
        std::vector<uint16_t> bits(static_cast<size_t>(n) * d);
        impl_->core->rc(b200idx_get_base(h, 0, n, bits.data()), h, "get_base");
        for (size_t i = 0; i < bits.size(); ++i) out[i] = half_bits_to_float(bits[i]);
    } else {
        impl_->core->rc(b200idx_get_base(h, 0, n, out), h, "get_base");
    }
}

void AscendIndexFlat::getIdxMap(int deviceId, std::vector<idx_t>& idxMap) const {
    b200idx_t* h = impl_->core->handles[static_cast<size_t>(impl_->core->slot_of(deviceId))];
    idxMap.resize(static_cast<size_t>(b200idx_ntotal(h)));
    if (!idxMap.empty()) impl_->core->rc(b200idx_get_ids(h, 0, static_cast<int64_t>(idxMap.size()), idxMap.data()), h, "get_ids");
}

void AscendIndexFlat::copyTo(faiss::IndexFlat* index) const {
    FAISS_THROW_IF_NOT_MSG(index != nullptr, "Invalid index nullptr.");
    index->d = d;
    index->metric_type = metric_type;
    index->code_size = sizeof(float) * d;
    index->reset();
    // rows go back to the slot their label names when the labels are 0..ntotal-1, else device order
    std::vector<float> rows(static_cast<size_t>(ntotal) * d);
    std::vector<idx_t> ids;
    size_t off = 0;
    for (int dev : impl_->core->devices) {
        const size_t n = getBaseSize(dev);
        if (!n) continue;
        getBase(dev, reinterpret_cast<char*>(rows.data() + off * d));
        std::vector<idx_t> m;
        getIdxMap(dev, m);
        ids.insert(ids.end(), m.begin(), m.end());
        off += n;
    }
    std::vector<char> seen(static_cast<size_t>(ntotal), 0);
    bool perm = true;
    for (idx_t id : ids) {
        if (id < 0 || id >= ntotal || seen[static_cast<size_t>(id)]) { perm = false; break; }
        seen[static_cast<size_t>(id)] = 1;
    }
    index->codes.resize(rows.size() * sizeof(float));
    float* dst = index->get_xb();
    for (size_t i = 0; i < ids.size(); ++i) {
        const size_t slot = perm ? static_cast<size_t>(ids[i]) : i;
        std::memcpy(dst + slot * d, rows.data() + i * d, sizeof(float) * d);
    }
    index->ntotal = ntotal;
}

void AscendIndexFlat::copyTo(faiss::IndexIDMap* index) const {
    FAISS_THROW_IF_NOT_MSG(index != nullptr && index->index != nullptr, "Invalid index nullptr.");
    faiss::IndexFlat* flat = dynamic_cast<faiss::IndexFlat*>(index->index);
    FAISS_THROW_IF_NOT_MSG(flat != nullptr, "Invalid flatIndex nullptr.");
    flat->d = d;
    flat->metric_type = metric_type;
    flat->code_size = sizeof(float) * d;
    flat->reset();
    flat->codes.resize(static_cast<size_t>(ntotal) * d * sizeof(float));
    index->id_map.clear();
    size_t off = 0;
    for (int dev : impl_->core->devices) {
        const size_t n = getBaseSize(dev);
        if (!n) continue;
        getBase(dev, reinterpret_cast<char*>(flat->get_xb() + off * d));
        std::vector<idx_t> m;
        getIdxMap(dev, m);
        index->id_map.insert(index->id_map.end(), m.begin(), m.end());
        off += n;
    }
    flat->ntotal = index->ntotal = ntotal;
    index->d = d;
    index->metric_type = metric_type;
}

void AscendIndexFlat::search_with_masks(idx_t n, const float* x, idx_t k, float* distances, idx_t* labels,
                                        const void* mask) const {
    RwGuard g(AscendIndex::impl_->mutex, false);
    check_search_args(n, x, k, distances, labels, is_trained);
    FAISS_THROW_IF_NOT_MSG(mask, "mask can not be nullptr.");
    // bit i of a query's row refers to the i-th vector in add order, which is one device's storage order
    FAISS_THROW_IF_NOT_MSG(AscendIndex::impl_->handles.size() == 1,
                           "search_with_masks is implemented for an index on one device");
    b200idx_t* h = AscendIndex::impl_->handles[0];
    AscendIndex::impl_->rc(b200idx_search_with_masks(h, n, x, static_cast<int>(k), static_cast<const uint8_t*>(mask),
                                                     distances, labels), h, "search_with_masks");
}
// fp16 queries: widened on the host (exact), then the float entry point; an fp16-storage index
// rounds them back to the same bits.
void AscendIndexFlat::search_with_masks(idx_t n, const uint16_t* x, idx_t k, float* distances, idx_t* labels,
                                        const void* mask) const {
    FAISS_THROW_IF_NOT_MSG(x != nullptr, "x cannot be nullptr.");
    FAISS_THROW_IF_NOT_FMT((n > 0) && (n < MAX_N), "n must be > 0 and < %ld", static_cast<long>(MAX_N));
    std::vector<float> xf(static_cast<size_t>(n) * d);
    for (size_t i = 0; i < xf.size(); ++i) xf[i] = half_bits_to_float(x[i]);
    search_with_masks(n, xf.data(), k, distances, labels, mask);
}

AscendIndexFlatL2::AscendIndexFlatL2(faiss::IndexFlatL2* index, AscendIndexFlatConfig config)
    : AscendIndexFlat(index, config) {}
AscendIndexFlatL2::AscendIndexFlatL2(int dims, AscendIndexFlatConfig config)
    : AscendIndexFlat(dims, faiss::METRIC_L2, config) {}
void AscendIndexFlatL2::copyFrom(faiss::IndexFlat* index) { AscendIndexFlat::copyFrom(index); }
void AscendIndexFlatL2::copyTo(faiss::IndexFlat* index) { AscendIndexFlat::copyTo(index); }

// ------------------------------------------------------------------ AscendIndexInt8 / Int8Flat
AscendIndexInt8::AscendIndexInt8(int dims, faiss::MetricType metric, AscendIndexInt8Config config)
    : impl_(std::make_shared<AscendIndexInt8Impl>()) {
    check_common(dims, config.deviceList, config.resourceSize);
    impl_->devices = config.deviceList;
    impl_->dims = dims;
    impl_->metric = metric;
    impl_->row_elem_bytes = 1;
}
AscendIndexInt8::~AscendIndexInt8() {}
void AscendIndexInt8::train(idx_t, const int8_t*) {}                       // a flat index needs no training
void AscendIndexInt8::updateCentroids(idx_t, const int8_t*) { FAISS_THROW_MSG("updateCentroids not implemented"); }
void AscendIndexInt8::updateCentroids(idx_t, const char*) { FAISS_THROW_MSG("updateCentroids not implemented"); }
void AscendIndexInt8::add(idx_t n, const int8_t* x) { add_with_ids(n, x, nullptr); }
void AscendIndexInt8::add(idx_t n, const char* x) { add_with_ids(n, reinterpret_cast<const int8_t*>(x), nullptr); }
void AscendIndexInt8::add_with_ids(idx_t n, const char* x, const idx_t* ids) {
    add_with_ids(n, reinterpret_cast<const int8_t*>(x), ids);
}
void AscendIndexInt8::add_with_ids(idx_t n, const int8_t* x, const idx_t* ids) {
    RwGuard g(impl_->mutex, true);
    FAISS_THROW_IF_NOT_FMT((n > 0) && (n < MAX_N), "n must be > 0 and < %ld", static_cast<long>(MAX_N));
    FAISS_THROW_IF_NOT_MSG(x != nullptr, "x cannot be nullptr.");
    std::vector<idx_t> gen;
    if (!ids) {
        gen = auto_ids(impl_->total(), n);
        ids = gen.data();
    }
    impl_->add_rows(n, x, static_cast<size_t>(impl_->dims), ids, false);
}
size_t AscendIndexInt8::remove_ids(const faiss::IDSelector& sel) {
    RwGuard g(impl_->mutex, true);
    size_t removed = 0;
    for (b200idx_t* h : impl_->handles) {
        std::vector<idx_t> ids(static_cast<size_t>(b200idx_ntotal(h)));
        if (ids.empty()) continue;
        impl_->rc(b200idx_get_ids(h, 0, static_cast<int64_t>(ids.size()), ids.data()), h, "get_ids");
        std::vector<idx_t> hit;
        for (idx_t id : ids)
            if (sel.is_member(id)) hit.push_back(id);
        if (hit.empty()) continue;
        int64_t r = 0;
        impl_->rc(b200idx_remove_ids(h, static_cast<int64_t>(hit.size()), hit.data(), &r), h, "remove_ids");
        removed += static_cast<size_t>(r);
    }
    return removed;
}
void AscendIndexInt8::assign(idx_t n, const int8_t* x, idx_t* labels, idx_t k) {
    std::vector<float> dist(static_cast<size_t>(n * k));
    search(n, x, k, dist.data(), labels);
}
void AscendIndexInt8::search(idx_t n, const int8_t* x, idx_t k, float* distances, idx_t* labels) const {
    RwGuard g(impl_->mutex, false);
    check_search_args(n, x, k, distances, labels, true);
    impl_->search_rows(n, x, k, distances, labels, false);
}
void AscendIndexInt8::search(idx_t n, const char* x, idx_t k, float* distances, idx_t* labels) const {
    search(n, reinterpret_cast<const int8_t*>(x), k, distances, labels);
}
void AscendIndexInt8::reserveMemory(size_t) {}
size_t AscendIndexInt8::reclaimMemory() { return 0; }
IndexImplBase& AscendIndexInt8::GetIndexImplBase() const { return *impl_; }
std::vector<int> AscendIndexInt8::getDeviceList() const { return impl_->devices; }
int AscendIndexInt8::getDim() const { return impl_->dims; }
faiss::idx_t AscendIndexInt8::getNTotal() const { return impl_->total(); }
bool AscendIndexInt8::isTrained() const { return true; }
faiss::MetricType AscendIndexInt8::getMetricType() const { return impl_->metric; }

namespace {
void check_int8_params(int dims, MetricType metric, const AscendIndexInt8FlatConfig& config) {
    FAISS_THROW_IF_NOT_MSG(metric == METRIC_L2 || metric == METRIC_INNER_PRODUCT, "Unsupported metric type");
    if (!RelaxedLimits()) {
        FAISS_THROW_IF_NOT_FMT(in(kInt8Dims, dims), "Unsupported dims %d", dims);
        FAISS_THROW_IF_NOT_FMT(in(kInt8Blocks, config.dBlockSize), " Unsupported blockSize %u! ", config.dBlockSize);
    }
    FAISS_THROW_IF_NOT_MSG(config.dIndexMode != Int8IndexMode::WITHOUT_NORM_MODE || metric == METRIC_L2,
                           "Unsupported metric type, should be METRIC_L2");
}
void create_int8_handles(AscendIndexInt8Impl& im) {
    for (int dev : im.devices) {
        b200idx_t* h = nullptr;
        const int metric = (im.metric == METRIC_INNER_PRODUCT && Int8InnerProductAsCosine()) ? B200IDX_METRIC_INT8_COSINE
                                                                                              : to_abi_metric(im.metric);
        const int code = b200idx_create_int8flat(im.dims, metric, dev, &h);
        if (code != B200IDX_OK) FAISS_THROW_FMT("create index failed (%d): %s", code, b200idx_last_error(nullptr));
        im.handles.push_back(h);
    }
}
}  // namespace

AscendIndexInt8Flat::AscendIndexInt8Flat(int dims, faiss::MetricType metric, AscendIndexInt8FlatConfig config)
    : AscendIndexInt8(dims, metric, config), impl_(std::make_shared<AscendIndexInt8FlatImpl>()) {
    check_int8_params(dims, metric, config);
    impl_->core = AscendIndexInt8::impl_.get();
    create_int8_handles(*impl_->core);
}
AscendIndexInt8Flat::AscendIndexInt8Flat(const faiss::IndexScalarQuantizer* index, AscendIndexInt8FlatConfig config)
    : AscendIndexInt8(index ? index->d : 128, index ? index->metric_type : METRIC_L2, config),
      impl_(std::make_shared<AscendIndexInt8FlatImpl>()) {
    FAISS_THROW_IF_NOT_MSG(index != nullptr, "Invalid index nullptr.");
    check_int8_params(index->d, index->metric_type, config);
    impl_->core = AscendIndexInt8::impl_.get();
    create_int8_handles(*impl_->core);
    copyFrom(index);
}
AscendIndexInt8Flat::AscendIndexInt8Flat(const faiss::IndexIDMap* index, AscendIndexInt8FlatConfig config)
    : AscendIndexInt8((index && index->index) ? index->index->d : 128,
                      (index && index->index) ? index->index->metric_type : METRIC_L2, config),
      impl_(std::make_shared<AscendIndexInt8FlatImpl>()) {
    FAISS_THROW_IF_NOT_MSG(index != nullptr && index->index != nullptr, "Invalid index nullptr.");
    check_int8_params(index->index->d, index->index->metric_type, config);
    impl_->core = AscendIndexInt8::impl_.get();
    create_int8_handles(*impl_->core);
    copyFrom(index);
}
AscendIndexInt8Flat::~AscendIndexInt8Flat() {}

size_t AscendIndexInt8Flat::getBaseSize(int deviceId) const {
    return static_cast<size_t>(b200idx_ntotal(impl_->core->handles[static_cast<size_t>(impl_->core->slot_of(deviceId))]));
}
void AscendIndexInt8Flat::getBase(int deviceId, std::vector<int8_t>& xb) const {
    b200idx_t* h = impl_->core->handles[static_cast<size_t>(impl_->core->slot_of(deviceId))];
    const int64_t n = b200idx_ntotal(h);
    xb.resize(static_cast<size_t>(n) * impl_->core->dims);
    if (n) impl_->core->rc(b200idx_get_base(h, 0, n, xb.data()), h, "get_base");
}
void AscendIndexInt8Flat::getIdxMap(int deviceId, std::vector<idx_t>& idxMap) const {
    b200idx_t* h = impl_->core->handles[static_cast<size_t>(impl_->core->slot_of(deviceId))];
    idxMap.resize(static_cast<size_t>(b200idx_ntotal(h)));
    if (!idxMap.empty()) impl_->core->rc(b200idx_get_ids(h, 0, static_cast<int64_t>(idxMap.size()), idxMap.data()), h, "get_ids");
}
void AscendIndexInt8Flat::reset() {
    RwGuard g(impl_->core->mutex, true);
    impl_->core->reset_all();
}
void AscendIndexInt8Flat::copyFrom(const faiss::IndexScalarQuantizer* index) {
    FAISS_THROW_IF_NOT_MSG(index != nullptr, "Invalid index nullptr.");
    FAISS_THROW_IF_NOT_FMT(index->ntotal >= 0 && index->ntotal < MAX_N, "ntotal must be >= 0 and < %ld", static_cast<long>(MAX_N));
    FAISS_THROW_IF_NOT_MSG(index->codes.size() == static_cast<size_t>(index->ntotal) * getDim(),
                           "The size of codes must be equal to ntotal * dim.\n");
    reset();
    if (index->ntotal > 0) add(index->ntotal, reinterpret_cast<const int8_t*>(index->codes.data()));
}
void AscendIndexInt8Flat::copyFrom(const faiss::IndexIDMap* index) {
    FAISS_THROW_IF_NOT_MSG(index != nullptr && index->index != nullptr, "Invalid index nullptr.");
    const faiss::IndexScalarQuantizer* sq = dynamic_cast<const faiss::IndexScalarQuantizer*>(index->index);
    FAISS_THROW_IF_NOT_MSG(sq != nullptr, "Invalid sqIndex nullptr.");
    FAISS_THROW_IF_NOT_MSG(index->id_map.size() == static_cast<size_t>(sq->ntotal),
                           "The size of id_map must be equal to ntotal.\n");
    reset();
    if (sq->ntotal > 0) add_with_ids(sq->ntotal, reinterpret_cast<const int8_t*>(sq->codes.data()), index->id_map.data());
}
void AscendIndexInt8Flat::copyTo(faiss::IndexScalarQuantizer* index) const {
    FAISS_THROW_IF_NOT_MSG(index != nullptr, "Invalid index nullptr.");
    index->d = getDim();
    index->metric_type = getMetricType();
    index->code_size = index->sq.code_size = static_cast<size_t>(getDim());
    index->sq.d = static_cast<size_t>(getDim());
    index->codes.clear();
    for (int dev : impl_->core->devices) {
        std::vector<int8_t> xb;
        getBase(dev, xb);
        index->codes.insert(index->codes.end(), reinterpret_cast<uint8_t*>(xb.data()),
                            reinterpret_cast<uint8_t*>(xb.data()) + xb.size());
    }
    index->ntotal = getNTotal();
}
void AscendIndexInt8Flat::copyTo(faiss::IndexIDMap* index) const {
    FAISS_THROW_IF_NOT_MSG(index != nullptr && index->index != nullptr, "Invalid index nullptr.");
    faiss::IndexScalarQuantizer* sq = dynamic_cast<faiss::IndexScalarQuantizer*>(index->index);
    FAISS_THROW_IF_NOT_MSG(sq != nullptr, "Invalid sqIndex nullptr.");
    copyTo(sq);
    index->id_map.clear();
    for (int dev : impl_->core->devices) {
        std::vector<idx_t> m;
        getIdxMap(dev, m);
        index->id_map.insert(index->id_map.end(), m.begin(), m.end());
    }
    index->ntotal = sq->ntotal;
}
void AscendIndexInt8Flat::search_with_masks(idx_t n, const int8_t* x, idx_t k, float* distances, idx_t* labels,
                                            const void* mask) const {
    FAISS_THROW_IF_NOT_MSG(n > 0 && x && distances && labels && k > 0, "invalid search arguments");
    FAISS_THROW_IF_NOT_MSG(mask, "mask can not be nullptr.");
    AscendIndexInt8Impl& core = *AscendIndexInt8::impl_;
    RwGuard g(core.mutex, false);
    FAISS_THROW_IF_NOT_MSG(core.handles.size() == 1, "search_with_masks is implemented for an index on one device");
    b200idx_t* h = core.handles[0];
    const int code = b200idx_search_with_masks(h, n, x, static_cast<int>(k), static_cast<const uint8_t*>(mask),
                                               distances, labels);
    if (code != B200IDX_OK) FAISS_THROW_FMT("search_with_masks failed (%d): %s", code, b200idx_last_error(h));
}
void AscendIndexInt8Flat::setPageSize(uint16_t pageBlockNum) {
    FAISS_THROW_IF_NOT_MSG(pageBlockNum > 0 && pageBlockNum <= 144, "pageBlockNum should be in range (0, 144]");
    // no effect: the B200 path streams the whole base in one persistent kernel
}

// ------------------------------------------------------------------ AscendIndexIVF / IVFPQ
namespace {
void create_ivfpq_handles(AscendIndexImpl& im) {
    for (b200idx_t* h : im.handles) b200idx_destroy(h);
    im.handles.clear();
    for (int dev : im.devices) {
        b200idx_t* h = nullptr;
        const int code = b200idx_create_ivfpq(im.dims, B200IDX_METRIC_L2, im.nlist, im.msubs, im.nbits,
                                              im.by_residual ? 1 : 0, dev, &h);
        if (code != B200IDX_OK) FAISS_THROW_FMT("create index failed (%d): %s", code, b200idx_last_error(nullptr));
        im.handles.push_back(h);
        im.rc(b200idx_ivfpq_set_nprobe(h, std::min(im.nprobe, im.nlist)), h, "set_nprobe");
    }
}
void push_trained_state(AscendIndexImpl& im) {
    for (b200idx_t* h : im.handles) {
        im.rc(b200idx_ivfpq_set_centroids(h, im.centroids.data()), h, "set_centroids");
        im.rc(b200idx_ivfpq_set_codebooks(h, im.codebooks.data()), h, "set_codebooks");
    }
}
}  // namespace

AscendIndexIVF::AscendIndexIVF(int dims, faiss::MetricType metric, int nlist, AscendIndexIVFConfig config)
    : AscendIndex(dims, metric, config), impl_(std::make_shared<AscendIndexIVFImpl>()) {
    FAISS_THROW_IF_NOT_MSG(metric == METRIC_L2 || metric == METRIC_INNER_PRODUCT, "Unsupported metric type");
    FAISS_THROW_IF_NOT_FMT(config.cp.niter > 0 && config.cp.niter <= 1000,
                           "ClusteringParameters niter must be in range (0, %d] ", 1000);
    impl_->core = AscendIndex::impl_.get();
    impl_->core->nlist = nlist;
    impl_->core->nprobe = 64;
    is_trained = false;
}
AscendIndexIVF::~AscendIndexIVF() {}
int AscendIndexIVF::getNumLists() const { return impl_->core->nlist; }
void AscendIndexIVF::copyFrom(const faiss::IndexIVF*) { FAISS_THROW_MSG("use the copyFrom of the concrete IVF class"); }
void AscendIndexIVF::copyTo(faiss::IndexIVF*) const { FAISS_THROW_MSG("use the copyTo of the concrete IVF class"); }
void AscendIndexIVF::reset() { AscendIndex::reset(); }   // lists cleared, trained state kept
void AscendIndexIVF::setNumProbes(int nprobes) {
    FAISS_THROW_IF_NOT_MSG(nprobes > 0, "nprobe must be greater than 0");
    FAISS_THROW_IF_NOT_MSG(nprobes <= impl_->core->nlist, "nprobe must be less than or equal to nlist");
    impl_->core->nprobe = nprobes;
    for (b200idx_t* h : impl_->core->handles) impl_->core->rc(b200idx_ivfpq_set_nprobe(h, nprobes), h, "set_nprobe");
}
int AscendIndexIVF::getNumProbes() const { return impl_->core->nprobe; }
void AscendIndexIVF::reserveMemory(size_t numVecs) {
    FAISS_THROW_IF_NOT_FMT((numVecs > 0) && (numVecs <= static_cast<size_t>(MAX_N)), "numVecs must be > 0 and <= %ld",
                           static_cast<long>(MAX_N));
}
size_t AscendIndexIVF::reclaimMemory() { return 0; }
uint32_t AscendIndexIVF::getListLength(int listId) const {
    FAISS_THROW_IF_NOT_FMT(listId >= 0 && listId < impl_->core->nlist, "listId must be in range [0, %d)", impl_->core->nlist);
    uint32_t len = 0;
    for (b200idx_t* h : impl_->core->handles) {
        len += static_cast<uint32_t>(b200idx_ivfpq_list_length(h, listId));
        if (impl_->core->replicated) break;   // every device holds the whole list
    }
    return len;
}
void AscendIndexIVF::getListCodesAndIds(int listId, std::vector<uint8_t>& codes, std::vector<ascend_idx_t>& ids) const {
    FAISS_THROW_IF_NOT_FMT(listId >= 0 && listId < impl_->core->nlist, "listId must be in range [0, %d)", impl_->core->nlist);
    codes.clear();
    ids.clear();
    const size_t M = static_cast<size_t>(impl_->core->msubs);
    for (b200idx_t* h : impl_->core->handles) {
        const int64_t len = b200idx_ivfpq_list_length(h, listId);
        if (len <= 0) continue;
        const size_t o = ids.size();
        codes.resize((o + static_cast<size_t>(len)) * M);
        ids.resize(o + static_cast<size_t>(len));
        impl_->core->rc(b200idx_ivfpq_get_list(h, listId, codes.data() + o * M, reinterpret_cast<int64_t*>(ids.data() + o)),
                        h, "get_list");
        if (impl_->core->replicated) break;   // every device holds the whole list
    }
}

AscendIndexIVFPQ::AscendIndexIVFPQ(int dims, faiss::MetricType metric, int nlist, int msubs, int nbits,
                                   AscendIndexIVFPQConfig config)
    : AscendIndexIVF(dims, metric, nlist, config), impl_(std::make_shared<AscendIndexIVFPQImpl>()) {
    FAISS_THROW_IF_NOT_MSG(metric == METRIC_L2, "Unsupported metric type");
    if (!RelaxedLimits()) {
        FAISS_THROW_IF_NOT_FMT(in(kPqDims, dims), "Unsupported dims: %d\n", dims);
        FAISS_THROW_IF_NOT_FMT(in(kPqNlists, nlist), "Unsupported nlists: %d\n", nlist);
        FAISS_THROW_IF_NOT_FMT(in(kPqMsubs, msubs), "Unsupported msubs: %d\n", msubs);
    } else {
        FAISS_THROW_IF_NOT_FMT(nlist > 0, "Unsupported nlists: %d\n", nlist);
        FAISS_THROW_IF_NOT_FMT(msubs > 0 && dims % msubs == 0, "Unsupported msubs: %d\n", msubs);
    }
    FAISS_THROW_IF_NOT_FMT(nbits == 8, "Unsupported nbits: %d\n", nbits);
    impl_->core = AscendIndex::impl_.get();
    AscendIndexImpl& im = *impl_->core;
    im.ivfpq = true;
    im.msubs = msubs;
    im.nbits = nbits;
    im.by_residual = env_is("B200IDX_IVFPQ_BY_RESIDUAL", "1");   // the reference encodes raw vectors
    im.nprobe = std::min(64, nlist);
    im.replicated = config.enableQueryParallelSearch && im.devices.size() > 1;
    create_ivfpq_handles(im);
}
AscendIndexIVFPQ::~AscendIndexIVFPQ() {}

void AscendIndexIVFPQ::train(idx_t n, const float* x) {
    AscendIndexImpl& im = *impl_->core;
    RwGuard g(im.mutex, true);
    FAISS_THROW_IF_NOT_FMT((n > 0) && (n < MAX_N), "n must be > 0 and < %ld", static_cast<long>(MAX_N));
    FAISS_THROW_IF_NOT_MSG(x != nullptr, "x cannot be nullptr.");
    FAISS_THROW_IF_NOT_FMT(n >= static_cast<idx_t>(im.msubs) * 256 && n >= im.nlist,
                           "training needs at least max(msubs * 256, nlist) = %d vectors",
                           std::max(im.msubs * 256, im.nlist));
    if (is_trained) return;
    // Lloyd k-means for the coarse centroids and for each sub-space codebook runs on the first
    // device (10 iterations, fixed seed); the other devices receive the trained state.
    b200idx_t* h0 = im.handles[0];
    im.rc(b200idx_ivfpq_train(h0, n, x, 10, 1234), h0, "train");
    im.centroids.resize(static_cast<size_t>(im.nlist) * d);
    im.codebooks.resize(static_cast<size_t>(d) * 256);
    im.rc(b200idx_ivfpq_get_centroids(h0, im.centroids.data()), h0, "get_centroids");
    im.rc(b200idx_ivfpq_get_codebooks(h0, im.codebooks.data()), h0, "get_codebooks");
    push_trained_state(im);
    is_trained = true;
}

void AscendIndexIVFPQ::copyFrom(const faiss::IndexIVFPQ* index) {
    AscendIndexImpl& im = *impl_->core;
    RwGuard g(im.mutex, true);
    FAISS_THROW_IF_NOT_MSG(index != nullptr, "Invalid index nullptr.");
    FAISS_THROW_IF_NOT_MSG(index->metric_type == METRIC_L2, "Unsupported metric type");
    FAISS_THROW_IF_NOT_FMT(index->ntotal >= 0 && index->ntotal < MAX_N, "Ntotal must be >= 0 and < %ld", static_cast<long>(MAX_N));
    FAISS_THROW_IF_NOT_MSG(index->d == d && static_cast<int>(index->nlist) == im.nlist &&
                               static_cast<int>(index->pq.M) == im.msubs && index->pq.nbits == 8,
                           "dims, nlist, msubs and nbits of the CPU index must match this index");
    const faiss::IndexFlat* q = dynamic_cast<const faiss::IndexFlat*>(index->quantizer);
    FAISS_THROW_IF_NOT_MSG(q != nullptr && q->ntotal == static_cast<idx_t>(index->nlist), "cpuQuantizer.ntotal must be nlist");
    FAISS_THROW_IF_NOT_MSG(index->invlists != nullptr, "Invalid invlists nullptr.");
    im.centroids.assign(q->get_xb(), q->get_xb() + static_cast<size_t>(im.nlist) * d);
    im.codebooks = index->pq.centroids;
    if (im.by_residual != index->by_residual) {   // handles are created for one encoding
        im.by_residual = index->by_residual;
        create_ivfpq_handles(im);
    } else {
        im.reset_all();
    }
    im.nprobe = static_cast<int>(std::min<size_t>(std::max<size_t>(index->nprobe, 1), index->nlist));
    for (b200idx_t* h : im.handles) im.rc(b200idx_ivfpq_set_nprobe(h, im.nprobe), h, "set_nprobe");
    push_trained_state(im);
    // every list is dealt to the devices in turn, so each device holds a slice of every list
    const size_t nd = im.handles.size(), M = static_cast<size_t>(im.msubs);
    std::vector<std::vector<int32_t>> ln(nd);
    std::vector<std::vector<uint8_t>> cd(nd);
    std::vector<std::vector<idx_t>> id(nd);
    size_t turn = 0;
    for (size_t l = 0; l < index->nlist; ++l) {
        const auto& lc = index->invlists->codes[l];
        const auto& li = index->invlists->ids[l];
        FAISS_THROW_IF_NOT_MSG(lc.size() == li.size() * M, "list codes and ids disagree in size");
        for (size_t v = 0; v < li.size(); ++v, ++turn) {
            for (size_t dv = im.replicated ? 0 : turn % nd; dv < nd; ++dv) {
                ln[dv].push_back(static_cast<int32_t>(l));
                cd[dv].insert(cd[dv].end(), lc.begin() + v * M, lc.begin() + (v + 1) * M);
                id[dv].push_back(li[v]);
                if (!im.replicated) break;
            }
        }
    }
    for (size_t dv = 0; dv < nd; ++dv)
        if (!ln[dv].empty())
            im.rc(b200idx_ivfpq_add_codes(im.handles[dv], static_cast<int64_t>(ln[dv].size()), ln[dv].data(), cd[dv].data(),
                                          id[dv].data()),
                  im.handles[dv], "add_codes");
    ntotal = im.total();
    is_trained = true;
}

void AscendIndexIVFPQ::copyTo(faiss::IndexIVFPQ* index) const {
    const AscendIndexImpl& im = *impl_->core;
    FAISS_THROW_IF_NOT_MSG(index != nullptr, "Invalid index nullptr.");
    FAISS_THROW_IF_NOT_MSG(is_trained, "Index not trained");
    index->d = d;
    index->metric_type = METRIC_L2;
    index->nlist = static_cast<size_t>(im.nlist);
    index->nprobe = static_cast<size_t>(im.nprobe);
    index->by_residual = im.by_residual;
    index->pq = faiss::ProductQuantizer(static_cast<size_t>(d), static_cast<size_t>(im.msubs), 8);
    index->pq.centroids = im.codebooks;
    faiss::IndexFlat* q = dynamic_cast<faiss::IndexFlat*>(index->quantizer);
    if (!q) {
        q = new faiss::IndexFlatL2(d);
        index->quantizer = q;
        index->own_fields = true;
    }
    q->d = d;
    q->code_size = sizeof(float) * d;
    q->reset();
    q->add(im.nlist, im.centroids.data());
    if (index->own_invlists) delete index->invlists;
    index->invlists = new faiss::ArrayInvertedLists(static_cast<size_t>(im.nlist), static_cast<size_t>(im.msubs));
    index->own_invlists = true;
    for (int l = 0; l < im.nlist; ++l) {
        std::vector<uint8_t> codes;
        std::vector<ascend_idx_t> ids;
        getListCodesAndIds(l, codes, ids);
        index->invlists->codes[static_cast<size_t>(l)] = codes;
        index->invlists->ids[static_cast<size_t>(l)].assign(ids.begin(), ids.end());
    }
    index->ntotal = ntotal;
    index->is_trained = true;
}

void AscendIndexIVFPQ::remove_ids(size_t n, const idx_t* ids) {
    AscendIndexImpl& im = *impl_->core;
    RwGuard g(im.mutex, true);
    FAISS_THROW_IF_NOT_MSG(n == 0 || ids != nullptr, "ids cannot be nullptr.");
    for (b200idx_t* h : im.handles) {
        int64_t r = 0;
        im.rc(b200idx_remove_ids(h, static_cast<int64_t>(n), ids, &r), h, "remove_ids");
    }
    ntotal = im.total();
}

std::vector<idx_t> AscendIndexIVFPQ::update(idx_t n, const float* x, const idx_t* ids) {
    FAISS_THROW_IF_NOT_MSG(n > 0, "update vector number must be greater than 0!");
    FAISS_THROW_IF_NOT_MSG(x != nullptr && ids != nullptr, "x and ids cannot be nullptr.");
    remove_ids(static_cast<size_t>(n), ids);       // replace = remove + add under the same ids
    add_with_ids(n, x, ids);
    return std::vector<idx_t>(ids, ids + n);
}

// ------------------------------------------------------------------ multi-index batch search
namespace {
constexpr size_t kMaxIndexCount = 10000;
constexpr idx_t kMultiMaxN = 1024, kMultiMaxK = 1024;

void check_multi(size_t count, idx_t n, const void* x, idx_t k, const float* D, const idx_t* I) {
    FAISS_THROW_IF_NOT_FMT(count > 0 && count <= kMaxIndexCount, "size of indexes (%zu) must be > 0 and <= %zu.", count,
                           kMaxIndexCount);
    if (!RelaxedLimits()) {
        FAISS_THROW_IF_NOT_FMT((n > 0) && (n <= kMultiMaxN), "n must be > 0 and <= %ld", static_cast<long>(kMultiMaxN));
        FAISS_THROW_IF_NOT_FMT((k > 0) && (k <= kMultiMaxK), "k must be > 0 and <= %ld", static_cast<long>(kMultiMaxK));
    } else {
        FAISS_THROW_IF_NOT_FMT((n > 0) && (n < MAX_N), "n must be > 0 and < %ld", static_cast<long>(MAX_N));
        FAISS_THROW_IF_NOT_FMT((k > 0) && (k <= MAX_K), "k must be > 0 and <= %ld", static_cast<long>(MAX_K));
    }
    FAISS_THROW_IF_NOT_MSG(x != nullptr, "Invalid x: nullptr.");
    FAISS_THROW_IF_NOT_MSG(D != nullptr, "Invalid distances: nullptr.");
    FAISS_THROW_IF_NOT_MSG(I != nullptr, "Invalid labels: nullptr.");
}

// impls: one per index.  merged: one list over everything; else layout [index][n][k].
void multi_search(const std::vector<const IndexImplBase*>& impls, idx_t n, const void* x, idx_t k, float* D, idx_t* I,
                  bool merged) {
    for (const IndexImplBase* im : impls) {
        FAISS_THROW_IF_NOT_MSG(im->metric == impls[0]->metric, "the metric type must be same");
        FAISS_THROW_IF_NOT_MSG(im->dims == impls[0]->dims, "the dim must be same.");
        if (!RelaxedLimits()) {
            FAISS_THROW_IF_NOT_FMT(im->devices.size() == 1, "the number of deviceList (%zu) must be 1.", im->devices.size());
            FAISS_THROW_IF_NOT_MSG(im->devices == impls[0]->devices, "the deviceList must be same.");
        }
    }
    std::vector<b200idx_t*> all;
    bool single = true;
    for (const IndexImplBase* im : impls) {
        single = single && im->handles.size() == 1;
        all.insert(all.end(), im->handles.begin(), im->handles.end());
    }
    if (merged || single) {
        const int code = b200idx_search_multi(all.data(), static_cast<int>(all.size()), n, x, static_cast<int>(k), D, I,
                                              merged ? 1 : 0);
        if (code != B200IDX_OK) FAISS_THROW_FMT("multi-index search failed (%d): %s", code, b200idx_last_error(all[0]));
        return;
    }
    const size_t per = static_cast<size_t>(n) * static_cast<size_t>(k);
    for (size_t i = 0; i < impls.size(); ++i) {   // multi-device indexes: merge inside each index
        const IndexImplBase* im = impls[i];
        const int code = b200idx_search_multi(im->handles.data(), static_cast<int>(im->handles.size()), n, x,
                                              static_cast<int>(k), D + per * i, I + per * i, 1);
        if (code != B200IDX_OK) FAISS_THROW_FMT("multi-index search failed (%d): %s", code, b200idx_last_error(im->handles[0]));
    }
}
}  // namespace

void Search(std::vector<AscendIndex*> indexes, idx_t n, const float* x, idx_t k, float* distances, idx_t* labels,
            bool merged) {
    check_multi(indexes.size(), n, x, k, distances, labels);
    std::vector<const IndexImplBase*> impls;
    for (AscendIndex* ix : indexes) {
        FAISS_THROW_IF_NOT_MSG(ix != nullptr, "Invalid index nullptr.");
        FAISS_THROW_IF_NOT_MSG(ix->is_trained, "Index not trained");
        impls.push_back(&ix->GetIndexImplBase());
    }
    multi_search(impls, n, x, k, distances, labels, merged);
}

void Search(std::vector<Index*> indexes, idx_t n, const float* x, idx_t k, float* distances, idx_t* labels, bool merged) {
    FAISS_THROW_IF_NOT_FMT(indexes.size() > 0 && indexes.size() <= kMaxIndexCount,
                           "size of indexes (%zu) must be > 0 and <= 10000.", indexes.size());
    std::vector<AscendIndex*> cast;
    for (Index* ix : indexes) {
        AscendIndex* a = dynamic_cast<AscendIndex*>(ix);
        FAISS_THROW_IF_NOT_MSG(a != nullptr, "Invalid index nullptr.");
        cast.push_back(a);
    }
    Search(cast, n, x, k, distances, labels, merged);
}

void Search(std::vector<AscendIndexInt8*> indexes, idx_t n, const int8_t* x, idx_t k, float* distances, idx_t* labels,
            bool merged) {
    check_multi(indexes.size(), n, x, k, distances, labels);
    std::vector<const IndexImplBase*> impls;
    for (AscendIndexInt8* ix : indexes) {
        FAISS_THROW_IF_NOT_MSG(ix != nullptr, "Invalid index nullptr.");
        impls.push_back(&ix->GetIndexImplBase());
    }
    multi_search(impls, n, x, k, distances, labels, merged);
}

// ------------------------------------------------------------------ cloner
// FR/ascend/AscendCloner.cpp:64-99 (to CPU), :159-196 (to the devices), :232-281 (entry points).
faiss::Index* index_ascend_to_cpu(const faiss::Index* ascend_index) {
    FAISS_THROW_IF_NOT_MSG(ascend_index != nullptr, "Invalid index nullptr.");
    faiss::Index* res = nullptr;
    try {
        if (auto flat = dynamic_cast<const AscendIndexFlat*>(ascend_index)) {
            faiss::IndexFlat* cpu = new faiss::IndexFlat(flat->d, flat->metric_type);
            faiss::IndexIDMap* map = new faiss::IndexIDMap(cpu);
            res = map;
            map->own_fields = true;
            flat->copyTo(map);
            return res;
        }
        if (auto pq = dynamic_cast<const AscendIndexIVFPQ*>(ascend_index)) {
            faiss::IndexIVFPQ* cpu = new faiss::IndexIVFPQ();
            res = cpu;
            pq->copyTo(cpu);
            return res;
        }
    } catch (const std::exception& e) {
        delete res;
        FAISS_THROW_FMT("clone from ascend to cpu failed, %s", e.what());
    }
    FAISS_THROW_MSG("clone from ascend to cpu not supported for this type of Index");
}

faiss::Index* index_cpu_to_ascend(std::vector<int> devices, const faiss::Index* index, const AscendClonerOptions* options) {
    FAISS_THROW_IF_NOT_MSG(index != nullptr, "Invalid index nullptr.");
    const int64_t res = options ? options->resourceSize : -1;
    if (auto flat = dynamic_cast<const faiss::IndexFlat*>(index)) {
        AscendIndexFlatConfig config(devices);
        if (res >= 0) config.resourceSize = res;
        return new AscendIndexFlat(flat, config);
    }
    if (auto pq = dynamic_cast<const faiss::IndexIVFPQ*>(index)) {
        AscendIndexIVFPQConfig config(devices);
        if (res >= 0) config.resourceSize = res;
        std::unique_ptr<AscendIndexIVFPQ> out(new AscendIndexIVFPQ(pq->d, pq->metric_type, static_cast<int>(pq->nlist),
                                                                   static_cast<int>(pq->pq.M), static_cast<int>(pq->pq.nbits),
                                                                   config));
        out->copyFrom(pq);
        return out.release();
    }
    if (auto map = dynamic_cast<const faiss::IndexIDMap*>(index)) {
        FAISS_THROW_IF_NOT_MSG(dynamic_cast<const faiss::IndexFlat*>(map->index) != nullptr,
                               "clone from cpu to ascend not supported for this type of Index");
        AscendIndexFlatConfig config(devices);
        if (res >= 0) config.resourceSize = res;
        return new AscendIndexFlat(map, config);
    }
    FAISS_THROW_MSG("clone from cpu to ascend not supported for this type of Index");
}
faiss::Index* index_cpu_to_ascend(std::initializer_list<int> devices, const faiss::Index* index,
                                  const AscendClonerOptions* options) {
    return index_cpu_to_ascend(std::vector<int>(devices), index, options);
}

faiss::Index* index_int8_ascend_to_cpu(const AscendIndexInt8* index) {
    FAISS_THROW_IF_NOT_MSG(index != nullptr, "Invalid index nullptr.");
    if (auto flat = dynamic_cast<const AscendIndexInt8Flat*>(index)) {
        faiss::IndexScalarQuantizer* sq = new faiss::IndexScalarQuantizer();
        faiss::IndexIDMap* map = new faiss::IndexIDMap(sq);
        map->own_fields = true;
        try {
            flat->copyTo(map);
        } catch (const std::exception& e) {
            delete map;
            FAISS_THROW_FMT("clone from ascend to cpu failed, %s", e.what());
        }
        return map;
    }
    FAISS_THROW_MSG("clone from ascend to cpu not supported for this type of Index");
}
AscendIndexInt8* index_int8_cpu_to_ascend(std::vector<int> devices, const faiss::Index* index,
                                          const AscendClonerOptions* options) {
    FAISS_THROW_IF_NOT_MSG(index != nullptr, "Invalid index nullptr.");
    AscendIndexInt8FlatConfig config(devices);
    if (options && options->resourceSize >= 0) config.resourceSize = options->resourceSize;
    if (auto sq = dynamic_cast<const faiss::IndexScalarQuantizer*>(index)) return new AscendIndexInt8Flat(sq, config);
    if (auto map = dynamic_cast<const faiss::IndexIDMap*>(index)) {
        FAISS_THROW_IF_NOT_MSG(dynamic_cast<const faiss::IndexScalarQuantizer*>(map->index) != nullptr,
                               "clone from cpu to ascend not supported for this type of Index");
        return new AscendIndexInt8Flat(map, config);
    }
    FAISS_THROW_MSG("clone from cpu to ascend not supported for this type of Index");
}
AscendIndexInt8* index_int8_cpu_to_ascend(std::initializer_list<int> devices, const faiss::Index* index,
                                          const AscendClonerOptions* options) {
    return index_int8_cpu_to_ascend(std::vector<int>(devices), index, options);
}

}  // namespace ascend
}  // namespace faiss
