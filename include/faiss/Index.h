// Minimal stand-in for faiss::Index (NOT Faiss): the virtual interface the Ascend-style classes
// derive from -- add / add_with_ids / search / reset / remove_ids / train.
#pragma once
#include <cstddef>
#include "MetricType.h"
#include "impl/FaissAssert.h"
#include "impl/IDSelector.h"
namespace faiss {
struct SearchParameters {
    virtual ~SearchParameters() {}
};
struct Index {
    int d;
    idx_t ntotal = 0;
    bool verbose = false;
    bool is_trained = true;
    MetricType metric_type;
    explicit Index(idx_t dim = 0, MetricType metric = METRIC_L2) : d(static_cast<int>(dim)), metric_type(metric) {}
    virtual ~Index() {}
    virtual void train(idx_t /*n*/, const float* /*x*/) {}
    virtual void add(idx_t n, const float* x) = 0;
    virtual void add_with_ids(idx_t, const float*, const idx_t*) { FAISS_THROW_MSG("add_with_ids not implemented"); }
    virtual void search(idx_t n, const float* x, idx_t k, float* distances, idx_t* labels,
                        const SearchParameters* params = nullptr) const = 0;
    virtual void reset() = 0;
    virtual size_t remove_ids(const IDSelector&) { FAISS_THROW_MSG("remove_ids not implemented"); }
};
}  // namespace faiss
