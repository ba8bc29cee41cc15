// Minimal stand-in for Faiss' MetricType.h (NOT Faiss: only what the B200 search path's C++
// classes touch).  A build that has the real Faiss puts its include directory first.
#pragma once
#include <cstdint>
namespace faiss {
using idx_t = int64_t;
enum MetricType { METRIC_INNER_PRODUCT = 0, METRIC_L2 = 1 };
}  // namespace faiss
