// Minimal stand-in for faiss::IndexIVF / IndexIVFPQ (NOT Faiss): the fields copyFrom / copyTo
// exchange -- coarse quantizer, nlist, nprobe, product quantizer centroids, inverted lists.
#pragma once
#include <cstdint>
#include <vector>
#include "IndexFlat.h"
namespace faiss {
struct ProductQuantizer {
    size_t d = 0, M = 0, nbits = 8, dsub = 0, ksub = 256, code_size = 0;
    std::vector<float> centroids;   // [M][ksub][dsub]
    ProductQuantizer() {}
    ProductQuantizer(size_t d_, size_t M_, size_t nbits_) : d(d_), M(M_), nbits(nbits_) {
        dsub = M ? d / M : 0;
        ksub = size_t(1) << nbits;
        code_size = (nbits * M + 7) / 8;
        centroids.resize(d * ksub);
    }
};
struct ArrayInvertedLists {
    size_t nlist = 0, code_size = 0;
    std::vector<std::vector<uint8_t>> codes;
    std::vector<std::vector<idx_t>> ids;
    ArrayInvertedLists(size_t nlist_ = 0, size_t code_size_ = 0) : nlist(nlist_), code_size(code_size_), codes(nlist_), ids(nlist_) {}
    size_t list_size(size_t l) const { return ids[l].size(); }
};
struct IndexIVF : Index {
    Index* quantizer = nullptr;
    size_t nlist = 0, nprobe = 1;
    bool own_fields = false;
    ArrayInvertedLists* invlists = nullptr;
    bool own_invlists = false;
    IndexIVF(Index* q, size_t d_, size_t nlist_, MetricType m) : Index(d_, m), quantizer(q), nlist(nlist_) {}
    ~IndexIVF() override {
        if (own_invlists) delete invlists;
        if (own_fields) delete quantizer;
    }
};
struct IndexIVFPQ : IndexIVF {
    bool by_residual = true;
    ProductQuantizer pq;
    IndexIVFPQ() : IndexIVF(nullptr, 0, 0, METRIC_L2) { is_trained = false; }
    IndexIVFPQ(Index* q, size_t d_, size_t nlist_, size_t M, size_t nbits, MetricType m = METRIC_L2)
        : IndexIVF(q, d_, nlist_, m), pq(d_, M, nbits) {
        invlists = new ArrayInvertedLists(nlist_, pq.code_size);
        own_invlists = true;
        is_trained = false;
    }
    void add(idx_t, const float*) override { FAISS_THROW_MSG("not supported by this stand-in"); }
    void search(idx_t, const float*, idx_t, float*, idx_t*, const SearchParameters* = nullptr) const override {
        FAISS_THROW_MSG("not supported by this stand-in");
    }
    void reset() override {
        if (!invlists) return;
        for (auto& c : invlists->codes) c.clear();
        for (auto& i : invlists->ids) i.clear();
        ntotal = 0;
    }
};
}  // namespace faiss
