// Minimal stand-in for <faiss/MetricType.h>, used ONLY when a real FAISS
// installation is not on the include path.  Written from the names the
// reference uses (include/faiss-metal/MetalIndexFlat.h:3-5,
// src/MetalIndexFlat.mm:9,167-171); it is not FAISS source.
#pragma once
#include <cstdint>

namespace faiss {

using idx_t = int64_t;

enum MetricType {
    METRIC_INNER_PRODUCT = 0,
    METRIC_L2 = 1,
};

}  // namespace faiss
