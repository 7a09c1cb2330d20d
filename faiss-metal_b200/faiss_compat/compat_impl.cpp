// Out-of-line members of the FAISS stand-in headers in this directory.
// Compiled into the library only when real FAISS headers are unavailable.
#include <algorithm>
#include <cmath>
#include <limits>
#include <utility>
#include <vector>

#include "faiss/IndexFlat.h"
#include "faiss/impl/FaissAssert.h"

namespace faiss {

void Index::reconstruct(idx_t, float*) const {
    FAISS_THROW_MSG("reconstruct not implemented for this type of index");
}

void IndexFlat::add(idx_t n, const float* x) {
    if (n <= 0) return;
    xb.insert(xb.end(), x, x + (size_t)n * d);
    ntotal += n;
}

void IndexFlat::reset() {
    xb.clear();
    ntotal = 0;
}

void IndexFlat::reconstruct(idx_t key, float* recons) const {
    FAISS_THROW_IF_NOT_MSG(key >= 0 && key < ntotal, "reconstruct: key out of range");
    std::copy(xb.begin() + (size_t)key * d, xb.begin() + (size_t)(key + 1) * d, recons);
}

void IndexFlat::search(idx_t n, const float* x, idx_t k, float* distances, idx_t* labels,
                       const SearchParameters*) const {
    FAISS_THROW_IF_NOT_MSG(k > 0, "k must be > 0");
    const bool l2 = metric_type == METRIC_L2;
    const float pad = l2 ? std::numeric_limits<float>::infinity()
                         : -std::numeric_limits<float>::infinity();
    std::vector<std::pair<float, idx_t>> cand;
    for (idx_t i = 0; i < n; i++) {
        cand.clear();
        const float* q = x + (size_t)i * d;
        for (idx_t j = 0; j < ntotal; j++) {
            const float* v = xb.data() + (size_t)j * d;
            float s = 0.f;
            if (l2) {
                for (int t = 0; t < d; t++) { float df = q[t] - v[t]; s += df * df; }
            } else {
                for (int t = 0; t < d; t++) s += q[t] * v[t];
                s = -s;
            }
            cand.emplace_back(s, j);
        }
        const idx_t kk = std::min<idx_t>(k, ntotal);
        std::partial_sort(cand.begin(), cand.begin() + kk, cand.end());
        for (idx_t j = 0; j < k; j++) {
            if (j < kk) {
                distances[i * k + j] = l2 ? cand[j].first : -cand[j].first;
                labels[i * k + j] = cand[j].second;
            } else {
                distances[i * k + j] = pad;
                labels[i * k + j] = -1;
            }
        }
    }
}

}  // namespace faiss
