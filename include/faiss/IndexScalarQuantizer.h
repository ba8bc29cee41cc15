// Minimal stand-in for faiss::IndexScalarQuantizer (NOT Faiss): for the int8 index it is only a
// container of ntotal * d code bytes (the reference mirrors its int8 base into one for
// persistence, examples/TestAscendIndexInt8FlatWithCPU.cpp:81-89).
#pragma once
#include <cstdint>
#include <vector>
#include "Index.h"
namespace faiss {
struct ScalarQuantizer {
    enum QuantizerType { QT_8bit = 0, QT_8bit_uniform = 2, QT_8bit_direct = 6 };
    QuantizerType qtype = QT_8bit;
    size_t d = 0, code_size = 0;
};
struct IndexScalarQuantizer : Index {
    ScalarQuantizer sq;
    std::vector<uint8_t> codes;
    size_t code_size = 0;
    IndexScalarQuantizer(int d_, ScalarQuantizer::QuantizerType qt, MetricType m = METRIC_L2) : Index(d_, m) {
        sq.qtype = qt;
        sq.d = d_;
        sq.code_size = code_size = d_;
    }
    IndexScalarQuantizer() : Index(0, METRIC_L2) {}
    void add(idx_t, const float*) override { FAISS_THROW_MSG("not supported by this stand-in"); }
    void search(idx_t, const float*, idx_t, float*, idx_t*, const SearchParameters* = nullptr) const override {
        FAISS_THROW_MSG("not supported by this stand-in");
    }
    void reset() override {
        codes.clear();
        ntotal = 0;
    }
};
}  // namespace faiss
