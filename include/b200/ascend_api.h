// faiss::ascend index classes with the reference's public API, implemented on the b200idx C ABI
// (include/b200idx.h).  Names, namespaces, parameter lists, config fields and defaults follow
//   FR/ascend/AscendIndex.h:33-111, AscendIndexFlat.h:33-118, AscendIndexInt8.h:36-128,
//   AscendIndexInt8Flat.h:32-109, AscendIndexIVF.h:35-119, AscendIndexIVFPQ.h:32-96,
//   AscendMultiIndexSearch.h:34-56            (FR = feature_retrieval/src/ascendfaiss)
// so that code written against those headers compiles unchanged.  deviceList entries are CUDA
// device ordinals; resourceSize is accepted and range-checked but scratch memory is grow-only.
// Members the hot path does not need (reserveMemory, reclaimMemory, GetIndexImplBase, train on
// device, update, search_with_masks) are declared; the ones not built yet throw
// FaissException("not implemented ...").
#pragma once
#include <cstdint>
#include <initializer_list>
#include <memory>
#include <vector>

#include <faiss/Clustering.h>
#include <faiss/Index.h>
#include <faiss/IndexFlat.h>
#include <faiss/IndexIVFPQ.h>
#include <faiss/IndexScalarQuantizer.h>
#include <faiss/MetaIndexes.h>
#include <faiss/impl/FaissAssert.h>

namespace faiss {
namespace ascend {
using rpcContext = void*;
using ascend_idx_t = uint64_t;

const idx_t MAX_N = 1e9;
const idx_t MAX_K = 4096;
const int64_t INDEX_DEFAULT_MEM = 0x2000000;
const int64_t INDEX_MAX_MEM = 0x280000000;
const uint32_t DEFAULT_BLOCK_SIZE = 16384 * 16;
const int64_t FLAT_DEFAULT_MEM = 0x8000000;
const int64_t INDEX_INT8_DEFAULT_MEM = 0x2000000;
const int64_t INT8_FLAT_DEFAULT_MEM = 0x8000000;
const int64_t IVF_DEFAULT_MEM = 0x8000000;
const uint32_t BLOCK_SIZE = 16384 * 16;

struct AscendIndexConfig {
    AscendIndexConfig() : deviceList({0}), resourceSize(INDEX_DEFAULT_MEM), dBlockSize(DEFAULT_BLOCK_SIZE) {}
    AscendIndexConfig(std::initializer_list<int> devices, int64_t resources = INDEX_DEFAULT_MEM,
                      uint32_t blockSize = DEFAULT_BLOCK_SIZE)
        : deviceList(devices), resourceSize(resources), dBlockSize(blockSize) {}
    AscendIndexConfig(std::vector<int> devices, int64_t resources = INDEX_DEFAULT_MEM,
                      uint32_t blockSize = DEFAULT_BLOCK_SIZE)
        : deviceList(devices), resourceSize(resources), dBlockSize(blockSize) {}
    std::vector<int> deviceList;
    int64_t resourceSize;
    bool slim = false;
    bool filterable = false;
    uint32_t dBlockSize = DEFAULT_BLOCK_SIZE;
};

class AscendIndexImpl;   // shared state of every float index: one b200idx handle per device
class IndexImplBase;

class AscendIndex : public faiss::Index {
public:
    AscendIndex(int dims, faiss::MetricType metric, AscendIndexConfig config);
    virtual ~AscendIndex();
    void add(idx_t n, const float* x) override;
    void add_with_ids(idx_t n, const float* x, const idx_t* ids) override;
    size_t remove_ids(const faiss::IDSelector& sel) override;
    void search(idx_t n, const float* x, idx_t k, float* distances, idx_t* labels,
                const SearchParameters* params = nullptr) const override;
    virtual void reserveMemory(size_t numVecs);
    virtual size_t reclaimMemory();
    void reset() override;
    std::vector<int> getDeviceList();
    IndexImplBase& GetIndexImplBase() const;
    AscendIndex(const AscendIndex&) = delete;
    AscendIndex& operator=(const AscendIndex&) = delete;
    void add(idx_t n, const uint16_t* x);
    void add_with_ids(idx_t n, const uint16_t* x, const idx_t* ids);
    void search(idx_t n, const uint16_t* x, idx_t k, float* distances, idx_t* labels) const;

protected:
    std::shared_ptr<AscendIndexImpl> impl_;
};

struct AscendIndexFlatConfig : public AscendIndexConfig {
    AscendIndexFlatConfig() {}
    AscendIndexFlatConfig(std::initializer_list<int> devices, int64_t resourceSize = FLAT_DEFAULT_MEM)
        : AscendIndexConfig(devices, resourceSize) {}
    AscendIndexFlatConfig(std::vector<int> devices, int64_t resourceSize = FLAT_DEFAULT_MEM)
        : AscendIndexConfig(devices, resourceSize) {}
};

class AscendIndexFlatImpl;
class AscendIndexFlat : public AscendIndex {
public:
    AscendIndexFlat(const faiss::IndexFlat* index, AscendIndexFlatConfig config = AscendIndexFlatConfig());
    AscendIndexFlat(const faiss::IndexIDMap* index, AscendIndexFlatConfig config = AscendIndexFlatConfig());
    AscendIndexFlat(int dims, faiss::MetricType metric, AscendIndexFlatConfig config = AscendIndexFlatConfig());
    virtual ~AscendIndexFlat();
    void copyFrom(const faiss::IndexFlat* index);
    void copyFrom(const faiss::IndexIDMap* index);
    void copyTo(faiss::IndexFlat* index) const;
    void copyTo(faiss::IndexIDMap* index) const;
    size_t getBaseSize(int deviceId) const;
    void getBase(int deviceId, char* xb) const;
    void getIdxMap(int deviceId, std::vector<idx_t>& idxMap) const;
    void search_with_masks(idx_t n, const float* x, idx_t k, float* distances, idx_t* labels, const void* mask) const;
    void search_with_masks(idx_t n, const uint16_t* x, idx_t k, float* distances, idx_t* labels,
                           const void* mask) const;
    AscendIndexFlat(const AscendIndexFlat&) = delete;
    AscendIndexFlat& operator=(const AscendIndexFlat&) = delete;

protected:
    std::shared_ptr<AscendIndexFlatImpl> impl_;
};

class AscendIndexFlatL2 : public AscendIndexFlat {
public:
    AscendIndexFlatL2(faiss::IndexFlatL2* index, AscendIndexFlatConfig config = AscendIndexFlatConfig());
    AscendIndexFlatL2(int dims, AscendIndexFlatConfig config = AscendIndexFlatConfig());
    virtual ~AscendIndexFlatL2() {}
    void copyFrom(faiss::IndexFlat* index);
    void copyTo(faiss::IndexFlat* index);
    AscendIndexFlatL2(const AscendIndexFlatL2&) = delete;
    AscendIndexFlatL2& operator=(const AscendIndexFlatL2&) = delete;
};

// ---- int8 ----
struct AscendIndexInt8Config {
    AscendIndexInt8Config() : deviceList({0}), resourceSize(INDEX_INT8_DEFAULT_MEM) {}
    AscendIndexInt8Config(std::initializer_list<int> devices, int64_t resources = INDEX_INT8_DEFAULT_MEM)
        : deviceList(devices), resourceSize(resources) {}
    AscendIndexInt8Config(std::vector<int> devices, int64_t resources = INDEX_INT8_DEFAULT_MEM)
        : deviceList(devices), resourceSize(resources) {}
    std::vector<int> deviceList;
    int64_t resourceSize;
};

class AscendIndexInt8Impl;
class AscendIndexInt8 {
public:
    AscendIndexInt8(int dims, faiss::MetricType metric, AscendIndexInt8Config config);
    virtual ~AscendIndexInt8();
    virtual void train(idx_t n, const int8_t* x);
    virtual void updateCentroids(idx_t n, const int8_t* x);
    virtual void updateCentroids(idx_t n, const char* x);
    void add(idx_t n, const int8_t* x);
    void add_with_ids(idx_t n, const int8_t* x, const idx_t* ids);
    void add(idx_t n, const char* x);
    void add_with_ids(idx_t n, const char* x, const idx_t* ids);
    size_t remove_ids(const faiss::IDSelector& sel);
    void assign(idx_t n, const int8_t* x, idx_t* labels, idx_t k = 1);
    void search(idx_t n, const int8_t* x, idx_t k, float* distances, idx_t* labels) const;
    void search(idx_t n, const char* x, idx_t k, float* distances, idx_t* labels) const;
    virtual void reserveMemory(size_t numVecs);
    virtual size_t reclaimMemory();
    IndexImplBase& GetIndexImplBase() const;
    std::vector<int> getDeviceList() const;
    AscendIndexInt8(const AscendIndexInt8&) = delete;
    AscendIndexInt8& operator=(const AscendIndexInt8&) = delete;
    int getDim() const;
    faiss::idx_t getNTotal() const;
    bool isTrained() const;
    faiss::MetricType getMetricType() const;

public:
    bool verbose = false;

protected:
    std::shared_ptr<AscendIndexInt8Impl> impl_;
};

enum class Int8IndexMode { DEFAULT_MODE = 0, PIPE_SEARCH_MODE, WITHOUT_NORM_MODE };

struct AscendIndexInt8FlatConfig : public AscendIndexInt8Config {
    AscendIndexInt8FlatConfig(uint32_t blockSize = BLOCK_SIZE, Int8IndexMode indexMode = Int8IndexMode::DEFAULT_MODE)
        : dBlockSize(blockSize), dIndexMode(indexMode) {}
    AscendIndexInt8FlatConfig(std::initializer_list<int> devices, int64_t resourceSize = INT8_FLAT_DEFAULT_MEM,
                              uint32_t blockSize = BLOCK_SIZE, Int8IndexMode indexMode = Int8IndexMode::DEFAULT_MODE)
        : AscendIndexInt8Config(devices, resourceSize), dBlockSize(blockSize), dIndexMode(indexMode) {}
    AscendIndexInt8FlatConfig(std::vector<int> devices, int64_t resourceSize = INT8_FLAT_DEFAULT_MEM,
                              uint32_t blockSize = BLOCK_SIZE, Int8IndexMode indexMode = Int8IndexMode::DEFAULT_MODE)
        : AscendIndexInt8Config(devices, resourceSize), dBlockSize(blockSize), dIndexMode(indexMode) {}
    uint32_t dBlockSize;
    Int8IndexMode dIndexMode;
};

class AscendIndexInt8FlatImpl;
class AscendIndexInt8Flat : public AscendIndexInt8 {
public:
    AscendIndexInt8Flat(int dims, faiss::MetricType metric = faiss::METRIC_L2,
                        AscendIndexInt8FlatConfig config = AscendIndexInt8FlatConfig());
    AscendIndexInt8Flat(const faiss::IndexScalarQuantizer* index,
                        AscendIndexInt8FlatConfig config = AscendIndexInt8FlatConfig());
    AscendIndexInt8Flat(const faiss::IndexIDMap* index, AscendIndexInt8FlatConfig config = AscendIndexInt8FlatConfig());
    virtual ~AscendIndexInt8Flat();
    size_t getBaseSize(int deviceId) const;
    void getBase(int deviceId, std::vector<int8_t>& xb) const;
    void getIdxMap(int deviceId, std::vector<idx_t>& idxMap) const;
    void reset();
    void copyFrom(const faiss::IndexScalarQuantizer* index);
    void copyFrom(const faiss::IndexIDMap* index);
    void copyTo(faiss::IndexScalarQuantizer* index) const;
    void copyTo(faiss::IndexIDMap* index) const;
    void search_with_masks(idx_t n, const int8_t* x, idx_t k, float* distances, idx_t* labels, const void* mask) const;
    void setPageSize(uint16_t pageBlockNum);
    AscendIndexInt8Flat(const AscendIndexInt8Flat&) = delete;
    AscendIndexInt8Flat& operator=(const AscendIndexInt8Flat&) = delete;

protected:
    std::shared_ptr<AscendIndexInt8FlatImpl> impl_;
};

// ---- IVF / IVFPQ ----
struct AscendIndexIVFConfig : public AscendIndexConfig {
    AscendIndexIVFConfig() : AscendIndexConfig({0}, IVF_DEFAULT_MEM), useKmeansPP(false) { SetDefaultClusteringConfig(); }
    AscendIndexIVFConfig(std::initializer_list<int> devices, int64_t resourceSize = IVF_DEFAULT_MEM)
        : AscendIndexConfig(devices, resourceSize), useKmeansPP(false) { SetDefaultClusteringConfig(); }
    AscendIndexIVFConfig(std::vector<int> devices, int64_t resourceSize = IVF_DEFAULT_MEM)
        : AscendIndexConfig(devices, resourceSize), useKmeansPP(false) { SetDefaultClusteringConfig(); }
    void SetDefaultClusteringConfig() { cp.niter = 10; }
    AscendIndexConfig flatConfig;
    bool useKmeansPP;
    ClusteringParameters cp;
};

class AscendIndexIVFImpl;
class AscendIndexIVF : public AscendIndex {
public:
    AscendIndexIVF(int dims, faiss::MetricType metric, int nlist, AscendIndexIVFConfig config = AscendIndexIVFConfig());
    virtual ~AscendIndexIVF();
    int getNumLists() const;
    void copyFrom(const faiss::IndexIVF* index);
    void copyTo(faiss::IndexIVF* index) const;
    void reset() override;
    virtual void setNumProbes(int nprobes);
    int getNumProbes() const;
    void reserveMemory(size_t numVecs) override;
    size_t reclaimMemory() override;
    virtual uint32_t getListLength(int listId) const;
    virtual void getListCodesAndIds(int listId, std::vector<uint8_t>& codes, std::vector<ascend_idx_t>& ids) const;
    AscendIndexIVF(const AscendIndexIVF&) = delete;
    AscendIndexIVF& operator=(const AscendIndexIVF&) = delete;

protected:
    std::shared_ptr<AscendIndexIVFImpl> impl_;
};

struct AscendIndexIVFPQConfig : public AscendIndexIVFConfig {
    AscendIndexIVFPQConfig() : AscendIndexIVFConfig({0}, IVF_DEFAULT_MEM) {}
    explicit AscendIndexIVFPQConfig(std::initializer_list<int> devices, int64_t resourceSize = IVF_DEFAULT_MEM)
        : AscendIndexIVFConfig(devices, resourceSize) {}
    explicit AscendIndexIVFPQConfig(std::vector<int> devices, int64_t resourceSize = IVF_DEFAULT_MEM)
        : AscendIndexIVFConfig(devices, resourceSize) {}
    int trainSamplesPerList = 40;
    int maxTrainSamples = 10000000;
    int pqNiter = -1;
    bool useDistributedCoarse = false;
    bool enableQueryParallelSearch = false;
};

class AscendIndexIVFPQImpl;
class AscendIndexIVFPQ : public AscendIndexIVF {
public:
    AscendIndexIVFPQ(int dims, faiss::MetricType metric, int nlist, int msubs, int nbits,
                     AscendIndexIVFPQConfig config = AscendIndexIVFPQConfig());
    void copyFrom(const faiss::IndexIVFPQ* index);
    void copyTo(faiss::IndexIVFPQ* index) const;
    virtual ~AscendIndexIVFPQ();
    AscendIndexIVFPQ(const AscendIndexIVFPQ&) = delete;
    AscendIndexIVFPQ& operator=(const AscendIndexIVFPQ&) = delete;
    void train(idx_t n, const float* x) override;
    void remove_ids(size_t n, const idx_t* ids);
    std::vector<idx_t> update(idx_t n, const float* x, const idx_t* ids);

protected:
    std::shared_ptr<AscendIndexIVFPQImpl> impl_;
};

// ---- multi-index batch search ----
void Search(std::vector<Index*> indexes, idx_t n, const float* x, idx_t k, float* distances, idx_t* labels, bool merged);
void Search(std::vector<AscendIndex*> indexes, idx_t n, const float* x, idx_t k, float* distances, idx_t* labels,
            bool merged);
void Search(std::vector<AscendIndexInt8*> indexes, idx_t n, const int8_t* x, idx_t k, float* distances, idx_t* labels,
            bool merged);

// ---- cloner: CPU index <-> index on the devices (ascend/AscendCloner.h, AscendClonerOptions.h of
//      the reference).  Covered: IndexFlat / IndexIDMap(IndexFlat) <-> AscendIndexFlat,
//      IndexIVFPQ <-> AscendIndexIVFPQ, IndexScalarQuantizer / IndexIDMap(IndexScalarQuantizer)
//      <-> AscendIndexInt8Flat; other index types raise "not supported". ----
struct AscendClonerOptions {
    AscendClonerOptions() : reserveVecs(0), verbose(false), resourceSize(-1), indexMode(0), blockSize(0) {}
    long reserveVecs;
    bool verbose;
    int64_t resourceSize;
    bool slim = false;         // (scalar-quantizer indexes of the reference; not used here)
    bool filterable = false;
    uint32_t indexMode;
    uint32_t blockSize;
};
faiss::Index* index_ascend_to_cpu(const faiss::Index* ascend_index);
faiss::Index* index_cpu_to_ascend(std::initializer_list<int> devices, const faiss::Index* index,
                                  const AscendClonerOptions* options = nullptr);
faiss::Index* index_cpu_to_ascend(std::vector<int> devices, const faiss::Index* index,
                                  const AscendClonerOptions* options = nullptr);
// the int8 index does not derive from faiss::Index
faiss::Index* index_int8_ascend_to_cpu(const AscendIndexInt8* index);
AscendIndexInt8* index_int8_cpu_to_ascend(std::initializer_list<int> devices, const faiss::Index* index,
                                          const AscendClonerOptions* options = nullptr);
AscendIndexInt8* index_int8_cpu_to_ascend(std::vector<int> devices, const faiss::Index* index,
                                          const AscendClonerOptions* options = nullptr);

// Relaxed mode (env B200IDX_RELAXED=1 or this switch): lifts the reference's whitelists (dims,
// nlist, msubs, k <= 320 for IVFPQ, same-device rule and n, k <= 1024 of multi-index search) to
// the limits of the C ABI.  Off by default: the reference's checks and messages apply.
void SetRelaxedLimits(bool on);
bool RelaxedLimits();

// What METRIC_INNER_PRODUCT means on an AscendIndexInt8Flat created from now on.  Off (default):
// the exact int32 dot product, returned as float.  On (this switch or env B200IDX_INT8_IP_COSINE=1):
// the fp16 cosine the reference computes for that metric (its "Cos" index,
// FR/ascend/impl/AscendIndexInt8FlatImpl.cpp:790-793) -- B200IDX_METRIC_INT8_COSINE of the C ABI.
void SetInt8InnerProductAsCosine(bool on);
bool Int8InnerProductAsCosine();

#define VALUE_UNUSED(x) (void)(x)
}  // namespace ascend
}  // namespace faiss
