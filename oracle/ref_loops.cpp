// Harness around the reference's OWN CPU code for this path -- TEST INFRASTRUCTURE ONLY.
//
// The reference project holds exactly one CPU implementation of the flat k-NN arithmetic: the
// inline loops of its unit tests (tests/test_metal_distance.mm:46-54,85-93 squared norms,
// :141-153 squared L2, :193-204 inner product, :207-227 inner-product top-1) together with the
// seeded std::mt19937 input generators in front of them (:23-31, :65-72, :105-115, :164-174)
// and the generator of the index tests (tests/test_metal_flat.mm:64-70).  None of those lines
// is copied here.  The Makefile beside this file cuts them out of the reference tree, where
// they lie, into _ref/*.inc (not tracked), and this file #includes them verbatim between its
// own scaffolding, so what runs is the reference's text compiled as it stands.
//
// The loops compare a GPU result with the CPU value inside an assert.  Here the "GPU result"
// is a recorder: subtracting the CPU value from one of its cells stores that value and yields
// zero, so the assert holds and the CPU values come out in an array.
//
// Output: one raw little-endian file per array in the directory given as argv[1], and one
// manifest line per array on stdout: "<name> <dtype> <dim0> [<dim1>]".
#include <cassert>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <string>
#include <vector>

namespace {

struct Recorder {
    std::vector<float> v;
    explicit Recorder(size_t n) : v(n, 0.0f) {}
    struct Cell {
        float* p;
        operator float() const { return *p; }
    };
    Cell operator[](size_t i) {
        if (i >= v.size()) {
            std::fprintf(stderr, "recorder index %zu out of range %zu\n", i, v.size());
            std::exit(2);
        }
        return Cell{&v[i]};
    }
};
// "gpu[i] - cpu" inside the reference's loops: keep the CPU value, report no difference
inline float operator-(Recorder::Cell c, float cpu) {
    *c.p = cpu;
    return 0.0f;
}

std::string g_dir;

template <typename T>
void dump(const std::string& name, const char* dtype, const T* data, size_t d0, size_t d1) {
    const std::string path = g_dir + "/" + name + ".bin";
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f) {
        std::perror(path.c_str());
        std::exit(2);
    }
    const size_t n = d0 * (d1 ? d1 : 1);
    if (std::fwrite(data, sizeof(T), n, f) != n) std::exit(2);
    std::fclose(f);
    if (d1) std::printf("%s %s %zu %zu\n", name.c_str(), dtype, d0, d1);
    else std::printf("%s %s %zu\n", name.c_str(), dtype, d0);
}

void norm_case_small() {
#include "_ref/norm_small_setup.inc"
    Recorder metalNorms(n);
#include "_ref/norm_small_loop.inc"
    dump("norm_small_x", "f32", data.data(), n, d);
    dump("norm_small_out", "f32", metalNorms.v.data(), n, 0);
}

void norm_case_large_dim() {
#include "_ref/norm_large_setup.inc"
    Recorder metalNorms(n);
#include "_ref/norm_large_loop.inc"
    dump("norm_large_x", "f32", data.data(), n, d);
    dump("norm_large_out", "f32", metalNorms.v.data(), n, 0);
}

void l2_case() {
#include "_ref/l2_setup.inc"
    Recorder metalDist(nq * nv);
#include "_ref/l2_loop.inc"
    dump("l2_q", "f32", queries.data(), nq, d);
    dump("l2_x", "f32", vectors.data(), nv, d);
    dump("l2_out", "f32", metalDist.v.data(), nq, nv);
}

void ip_case() {
#include "_ref/ip_setup.inc"
    Recorder metalDist(nq * nv);
#include "_ref/ip_loop.inc"
    // the top-1 block ends in assert(metalBest == cpuBest): record what the CPU side found
    std::vector<int64_t> top1(nq, -1);
#undef assert
#define assert(expr) (top1[i] = (int64_t)cpuBest)
#include "_ref/ip_top1.inc"
#undef assert
#define assert(expr) ((expr) ? (void)0 : (std::fprintf(stderr, "assert failed: %s\n", #expr), std::exit(3)))
    dump("ip_q", "f32", queries.data(), nq, d);
    dump("ip_x", "f32", vectors.data(), nv, d);
    dump("ip_out", "f32", metalDist.v.data(), nq, nv);
    dump("ip_top1", "i64", top1.data(), nq, 0);
}

// Shapes of the index tests (tests/test_metal_flat.mm:477-490): the reference's generator, then
// the reference's distance loops over what it generated.  The CPU side of those tests is CPU
// FAISS (absent); the loops above are the same arithmetic in the reference's own words.
void flat_case(const char* tag, size_t nv, size_t nq, size_t d, size_t k, bool ip) {
#include "_ref/flat_gen.inc"
    Recorder metalDist(nq * nv);
    (void)k;
    if (ip) {
#include "_ref/ip_loop.inc"
    } else {
#include "_ref/l2_loop.inc"
    }
    // inputs are large: only their first and last values and a checksum are kept, the tests
    // regenerate them from the seed and verify these
    uint64_t h = 1469598103934665603ull;
    auto mix = [&](const std::vector<float>& a) {
        const unsigned char* b = reinterpret_cast<const unsigned char*>(a.data());
        for (size_t i = 0; i < a.size() * sizeof(float); i++) {
            h ^= b[i];
            h *= 1099511628211ull;
        }
    };
    mix(vectors);
    mix(queries);
    const int64_t meta[5] = {(int64_t)nv, (int64_t)nq, (int64_t)d, (int64_t)k, (int64_t)(h >> 1)};
    const std::string t(tag);
    dump(t + "_meta", "i64", meta, 5, 0);
    dump(t + "_out", "f32", metalDist.v.data(), nq, nv);
}

}  // namespace

int main(int argc, char** argv) {
    if (argc < 2) {
        std::fprintf(stderr, "usage: %s <output directory>\n", argv[0]);
        return 2;
    }
    g_dir = argv[1];
    norm_case_small();
    norm_case_large_dim();
    l2_case();
    ip_case();
    flat_case("flat_l2_1000x32", 1000, 10, 32, 5, false);
    flat_case("flat_l2_1000x128", 1000, 10, 128, 10, false);
    flat_case("flat_l2_500x768", 500, 5, 768, 5, false);
    flat_case("flat_l2_500x1536", 500, 5, 1536, 5, false);
    flat_case("flat_l2_100x32", 100, 1, 32, 1, false);
    flat_case("flat_ip_1000x128", 1000, 10, 128, 10, true);
    return 0;
}
