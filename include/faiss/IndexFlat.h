// Minimal stand-in for faiss::IndexFlat / IndexFlatL2 / IndexFlatIP (NOT Faiss): a CPU container
// of raw float rows (the `codes` byte vector of the published struct) used by copyFrom / copyTo.
// search() is a plain exhaustive scan so that examples that compare against a CPU index work.
#pragma once
#include <cstdint>
#include <cstring>
#include <vector>
#include "Index.h"
namespace faiss {
struct IndexFlat : Index {
    size_t code_size;
    std::vector<uint8_t> codes;   // ntotal * d floats
    explicit IndexFlat(idx_t d = 0, MetricType metric = METRIC_L2) : Index(d, metric), code_size(sizeof(float) * d) {}
    float* get_xb() { return reinterpret_cast<float*>(codes.data()); }
    const float* get_xb() const { return reinterpret_cast<const float*>(codes.data()); }
    void add(idx_t n, const float* x) override {
        const size_t old = codes.size();
        codes.resize(old + static_cast<size_t>(n) * code_size);
        std::memcpy(codes.data() + old, x, static_cast<size_t>(n) * code_size);
        ntotal += n;
    }
    void reset() override {
        codes.clear();
        ntotal = 0;
    }
    void search(idx_t n, const float* x, idx_t k, float* D, idx_t* I, const SearchParameters* = nullptr) const override;
};
struct IndexFlatL2 : IndexFlat {
    explicit IndexFlatL2(idx_t d = 0) : IndexFlat(d, METRIC_L2) {}
};
struct IndexFlatIP : IndexFlat {
    explicit IndexFlatIP(idx_t d = 0) : IndexFlat(d, METRIC_INNER_PRODUCT) {}
};
inline void IndexFlat::search(idx_t n, const float* x, idx_t k, float* D, idx_t* I, const SearchParameters*) const {
    const float* xb = get_xb();
    const bool l2 = metric_type == METRIC_L2;
    for (idx_t q = 0; q < n; ++q) {
        for (idx_t j = 0; j < k; ++j) {
            D[q * k + j] = 3.402823466e+38f;
            I[q * k + j] = -1;
        }
        for (idx_t i = 0; i < ntotal; ++i) {
            float acc = 0.f;
            for (int t = 0; t < d; ++t) {
                if (l2) {
                    const float df = x[q * d + t] - xb[i * d + t];
                    acc += df * df;
                } else {
                    acc += x[q * d + t] * xb[i * d + t];
                }
            }
            const float key = l2 ? acc : -acc;
            idx_t pos = k;
            while (pos > 0 && (I[q * k + pos - 1] < 0 || key < (l2 ? D[q * k + pos - 1] : -D[q * k + pos - 1]))) --pos;
            if (pos < k) {
                for (idx_t j = k - 1; j > pos; --j) {
                    D[q * k + j] = D[q * k + j - 1];
                    I[q * k + j] = I[q * k + j - 1];
                }
                D[q * k + pos] = acc;
                I[q * k + pos] = i;
            }
        }
    }
}
}  // namespace faiss
