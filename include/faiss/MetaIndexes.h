// Minimal stand-in for faiss::IndexIDMap (NOT Faiss): a wrapped index plus its id_map.
#pragma once
#include <vector>
#include "Index.h"
namespace faiss {
struct IndexIDMap : Index {
    Index* index = nullptr;
    bool own_fields = false;
    std::vector<idx_t> id_map;
    explicit IndexIDMap(Index* sub = nullptr) : Index(sub ? sub->d : 0, sub ? sub->metric_type : METRIC_L2), index(sub) {
        if (sub) ntotal = sub->ntotal;
    }
    ~IndexIDMap() override {
        if (own_fields) delete index;
    }
    void add(idx_t, const float*) override { FAISS_THROW_MSG("add does not make sense with IndexIDMap, use add_with_ids"); }
    void add_with_ids(idx_t n, const float* x, const idx_t* ids) override {
        index->add(n, x);
        id_map.insert(id_map.end(), ids, ids + n);
        ntotal = index->ntotal;
    }
    void search(idx_t n, const float* x, idx_t k, float* D, idx_t* I, const SearchParameters* p = nullptr) const override {
        index->search(n, x, k, D, I, p);
        for (idx_t i = 0; i < n * k; ++i)
            if (I[i] >= 0) I[i] = id_map[static_cast<size_t>(I[i])];
    }
    void reset() override {
        index->reset();
        id_map.clear();
        ntotal = 0;
    }
};
}  // namespace faiss
