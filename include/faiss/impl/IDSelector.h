// Minimal stand-in for Faiss' IDSelector family (NOT Faiss).
#pragma once
#include <unordered_set>
#include "../MetricType.h"
namespace faiss {
struct IDSelector {
    virtual bool is_member(idx_t id) const = 0;
    virtual ~IDSelector() {}
};
struct IDSelectorRange : IDSelector {
    idx_t imin, imax;
    IDSelectorRange(idx_t lo, idx_t hi) : imin(lo), imax(hi) {}
    bool is_member(idx_t id) const override { return id >= imin && id < imax; }
};
struct IDSelectorBatch : IDSelector {
    std::unordered_set<idx_t> set;
    IDSelectorBatch(size_t n, const idx_t* ids) : set(ids, ids + n) {}
    bool is_member(idx_t id) const override { return set.count(id) != 0; }
};
}  // namespace faiss
