// Minimal stand-in for <faiss/IndexFlat.h> (see MetricType.h in this directory).
// A host-memory flat index with the members the converters need
// (get_xb(), add, search, ntotal, d, metric_type: src/MetalIndexFlat.mm:552-587).
// Its search is a plain loop, good enough for conversion round-trip tests; it is
// not a code path of the GPU index.
#pragma once
#include <vector>

#include "Index.h"

namespace faiss {

struct IndexFlat : Index {
    std::vector<float> xb;

    explicit IndexFlat(idx_t d_ = 0, MetricType metric = METRIC_L2) : Index(d_, metric) {}

    void add(idx_t n, const float* x) override;
    void search(idx_t n, const float* x, idx_t k, float* distances, idx_t* labels,
                const SearchParameters* params = nullptr) const override;
    void reset() override;
    void reconstruct(idx_t key, float* recons) const override;

    float* get_xb() { return xb.data(); }
    const float* get_xb() const { return xb.data(); }
};

struct IndexFlatL2 : IndexFlat {
    explicit IndexFlatL2(idx_t d_ = 0) : IndexFlat(d_, METRIC_L2) {}
};

struct IndexFlatIP : IndexFlat {
    explicit IndexFlatIP(idx_t d_ = 0) : IndexFlat(d_, METRIC_INNER_PRODUCT) {}
};

}  // namespace faiss
