// Contract test of the C++ plugin classes, written the way the reference's own test
// binary is (tests/test_metal_flat.mm): a faiss::Index* holder, the CPU IndexFlat as the
// comparison, std::mt19937(42) + uniform(-1, 1) data.  Exits non-zero on the first failure.
#include <b200_flat.h>
#include <faiss-b200/faiss_b200.h>
#include <faiss/IndexFlat.h>
#include <faiss/impl/FaissAssert.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <random>
#include <vector>

using namespace faiss_b200;

#define CHECK(cond)                                                              \
    do {                                                                         \
        if (!(cond)) {                                                           \
            std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond);          \
            std::exit(1);                                                        \
        }                                                                        \
    } while (0)

static std::vector<float> randomVectors(size_t n, size_t d, std::mt19937& rng) {
    std::uniform_real_distribution<float> dist(-1.0f, 1.0f);
    std::vector<float> v(n * d);
    for (auto& x : v) x = dist(rng);
    return v;
}

// top-1 equal, every distance within tol (tests/test_metal_flat.mm:16-59 asserts the first,
// only warns about the second; both are asserted here)
static void compare(faiss::idx_t n, faiss::idx_t k, const float* gd, const faiss::idx_t* gl,
                    const float* cd, const faiss::idx_t* cl, float tol) {
    for (faiss::idx_t i = 0; i < n; i++) {
        CHECK(gl[i * k] == cl[i * k]);
        for (faiss::idx_t j = 0; j < k; j++) {
            float rel = std::fabs(gd[i * k + j] - cd[i * k + j]) / std::max(std::fabs(cd[i * k + j]), 1e-2f);
            CHECK(rel <= tol);
        }
    }
}

static void testFlat(std::shared_ptr<B200Resources> res, size_t nv, size_t nq, size_t d, size_t k,
                     faiss::MetricType metric, StorageType storage, float tol) {
    std::mt19937 rng(42);
    auto vectors = randomVectors(nv, d, rng);
    auto queries = randomVectors(nq, d, rng);
    faiss::IndexFlat cpu(d, metric);
    cpu.add(nv, vectors.data());
    std::vector<float> cd(nq * k), gd(nq * k);
    std::vector<faiss::idx_t> cl(nq * k), gl(nq * k);
    cpu.search(nq, queries.data(), k, cd.data(), cl.data());

    std::unique_ptr<faiss::Index> gpu(new B200IndexFlat(res, (int)d, metric, storage));  // used through the base class
    CHECK(gpu->is_trained && gpu->ntotal == 0 && gpu->d == (int)d && gpu->metric_type == metric);
    gpu->add(nv, vectors.data());
    CHECK(gpu->ntotal == (faiss::idx_t)nv);
    gpu->search(nq, queries.data(), k, gd.data(), gl.data());
    compare(nq, k, gd.data(), gl.data(), cd.data(), cl.data(), tol);
    std::printf("flat nv=%zu nq=%zu d=%zu k=%zu metric=%d storage=%d PASS\n", nv, nq, d, k, (int)metric,
                (int)storage);
}

static void testConversion(std::shared_ptr<B200Resources> res) {
    // tests/test_metal_flat.mm:132-176
    const size_t nv = 500, d = 128, nq = 10, k = 5;
    std::mt19937 rng(42);
    auto vectors = randomVectors(nv, d, rng);
    auto queries = randomVectors(nq, d, rng);
    faiss::IndexFlatL2 cpu(d);
    cpu.add(nv, vectors.data());
    auto gpu = index_cpu_to_gpu(res, &cpu);
    CHECK(gpu->ntotal == (faiss::idx_t)nv && gpu->d == (int)d);
    CHECK(gpu->getStorageType() == StorageType::Float32 && !gpu->isFloat16Storage() && !gpu->isBFloat16Storage());
    const float* mirror = gpu->getVectorsData();
    CHECK(mirror != nullptr);
    for (size_t i = 0; i < nv * d; i++) CHECK(mirror[i] == vectors[i]);
    auto back = index_gpu_to_cpu(gpu.get());
    CHECK(back->ntotal == (faiss::idx_t)nv && back->d == (int)d);
    std::vector<float> d1(nq * k), d2(nq * k);
    std::vector<faiss::idx_t> l1(nq * k), l2(nq * k);
    cpu.search(nq, queries.data(), k, d1.data(), l1.data());
    back->search(nq, queries.data(), k, d2.data(), l2.data());
    for (size_t i = 0; i < nq * k; i++) {
        CHECK(l1[i] == l2[i]);
        CHECK(std::fabs(d1[i] - d2[i]) <= 1e-5f);
    }
    // 16-bit storage: converter with a storage argument, bulk read back
    auto gpu16 = index_cpu_to_gpu(res, &cpu, StorageType::BFloat16);
    CHECK(gpu16->isBFloat16Storage() && gpu16->getVectorsData() == nullptr);
    auto back16 = index_gpu_to_cpu(gpu16.get());
    CHECK(back16->ntotal == (faiss::idx_t)nv);
    for (size_t i = 0; i < nv * d; i++) CHECK(std::fabs(back16->get_xb()[i] - vectors[i]) <= 4e-3f);
    std::printf("conversion PASS\n");
}

static void testErrorsAndTokens(std::shared_ptr<B200Resources> res) {
    B200IndexFlat idx(res, 32, faiss::METRIC_L2);
    std::mt19937 rng(1);
    auto v = randomVectors(100, 32, rng);
    idx.add(100, v.data());
    std::vector<float> dd(5);
    std::vector<faiss::idx_t> ll(5);
    bool threw = false;
    try { idx.search(1, v.data(), 0, dd.data(), ll.data()); } catch (const faiss::FaissException&) { threw = true; }
    CHECK(threw);  // k must be > 0 (src/MetalIndexFlat.mm:321)
    threw = false;
    try { idx.reconstruct(100, dd.data()); } catch (const faiss::FaissException&) { threw = true; }
    CHECK(threw);  // src/MetalIndexFlat.mm:509-511
    // token: move-only, waits in the destructor, moved-from token throws
    {
        B200SearchToken t = idx.searchAsync(1, v.data(), 5, dd.data(), ll.data());
        B200SearchToken u = std::move(t);
        threw = false;
        try { t.wait(); } catch (const faiss::FaissException&) { threw = true; }
        CHECK(threw);  // src/MetalIndexFlat.mm:50
        u.wait();
        CHECK(ll[0] == 0 && dd[0] <= 1e-5f);
        u.wait();  // second wait is a no-op
    }
    {
        std::vector<float> d2(5);
        std::vector<faiss::idx_t> l2(5, -7);
        { B200SearchToken t = idx.searchAsync(1, v.data() + 32, 5, d2.data(), l2.data()); }  // destructor waits
        CHECK(l2[0] == 1);
    }
    // several tokens in flight at once, then a second round: the second round's buffers come
    // out of the resources' pools (no fresh allocation), results stay right
    {
        auto* sres = dynamic_cast<StandardB200Resources*>(res.get());
        CHECK(sres != nullptr);
        for (int round = 0; round < 2; round++) {
            const size_t missesBefore = sres->tempPoolMisses();
            std::vector<std::vector<float>> ds(4, std::vector<float>(3 * 5));
            std::vector<std::vector<faiss::idx_t>> ls(4, std::vector<faiss::idx_t>(3 * 5, -7));
            std::vector<B200SearchToken> tokens;
            for (int i = 0; i < 4; i++)
                tokens.push_back(idx.searchAsync(3, v.data() + (size_t)(10 * i) * 32, 5, ds[i].data(), ls[i].data()));
            for (int i = 0; i < 4; i++) {
                tokens[i].wait();
                for (int q = 0; q < 3; q++) CHECK(ls[i][q * 5] == 10 * i + q);
            }
            if (round == 1) CHECK(sres->tempPoolMisses() == missesBefore);
        }
        CHECK(sres->tempPoolHits() > 0);
    }
    idx.reset();
    CHECK(idx.ntotal == 0);
    idx.add(50, v.data());
    CHECK(idx.ntotal == 50);  // tests/test_metal_flat.mm:178-196
    std::printf("errors/tokens PASS\n");
}

// The sharded index through a faiss::Index*: S shards (all on the one GPU a test box is sure to
// have: the exchange then runs on device copies; on different GPUs when the box has them:
// NCCL), rows placed block-cyclically over several add() calls, results bit-equal to the
// unsharded index, labels global.
static void testSharded(std::vector<std::shared_ptr<B200Resources>> shardRes, std::shared_ptr<B200Resources> res,
                        StorageType storage, faiss::MetricType metric, size_t k, const char* what) {
    const size_t nv = 5000, nq = 37, d = 48;
    std::mt19937 rng(7);
    auto vectors = randomVectors(nv, d, rng);
    auto queries = randomVectors(nq, d, rng);
    for (size_t i = 100; i < 140; i++)   // exact duplicates that land on different shards
        for (size_t j = 0; j < d; j++) vectors[i * d + j] = vectors[(3000 + i) * d + j];
    B200IndexFlat plain(res, (int)d, metric, storage);
    plain.add(nv, vectors.data());
    std::vector<float> pd(nq * k), gd(nq * k);
    std::vector<faiss::idx_t> pl(nq * k), gl(nq * k);
    plain.search(nq, queries.data(), k, pd.data(), pl.data());

    std::unique_ptr<faiss::Index> gpu(new B200ShardedIndexFlat(shardRes, (int)d, metric, storage, 64));
    CHECK(gpu->is_trained && gpu->ntotal == 0);
    gpu->add(10, vectors.data());                        // partial block
    gpu->add(1990, vectors.data() + 10 * d);             // finishes it, many whole blocks
    gpu->add(nv - 2000, vectors.data() + 2000 * d);
    CHECK(gpu->ntotal == (faiss::idx_t)nv);
    gpu->search(nq, queries.data(), k, gd.data(), gl.data());
    for (size_t i = 0; i < nq * k; i++) {
        CHECK(gl[i] == pl[i]);
        CHECK(gd[i] == pd[i]);
    }
    std::vector<float> row(d);
    for (faiss::idx_t key : {0, 63, 64, 65, 1999, 2000, 4999}) {
        gpu->reconstruct(key, row.data());
        std::vector<float> want(d);
        plain.reconstruct(key, want.data());
        for (size_t j = 0; j < d; j++) CHECK(row[j] == want[j]);
    }
    bool threw = false;
    try {
        gpu->reconstruct(nv, row.data());
    } catch (const faiss::FaissException&) {
        threw = true;
    }
    CHECK(threw);
    gpu->reset();
    CHECK(gpu->ntotal == 0);
    gpu->add(300, vectors.data());
    gpu->search(nq, queries.data(), 5, gd.data(), gl.data());
    for (size_t i = 0; i < nq; i++) CHECK(gl[i * 5] >= 0 && gl[i * 5] < 300);
    std::printf("sharded %s shards=%zu storage=%d metric=%d k=%zu PASS\n", what, shardRes.size(), (int)storage,
                (int)metric, k);
}

static void testShardedAll(std::shared_ptr<B200Resources> res) {
    // one GPU, several shards
    for (size_t S : {1, 3, 8}) {
        std::vector<std::shared_ptr<B200Resources>> same(S, res);
        testSharded(same, res, StorageType::BFloat16, faiss::METRIC_L2, 10, "one-gpu");
        testSharded(same, res, StorageType::Float32, faiss::METRIC_INNER_PRODUCT, 100, "one-gpu");
    }
    // one process per GPU with a world of one: the rank form without a communicator
    {
        auto local = std::make_shared<B200IndexFlat>(res, 32, faiss::METRIC_L2, StorageType::Float16);
        std::mt19937 rng(9);
        auto v = randomVectors(2000, 32, rng);
        local->add(2000, v.data());
        local->setLabelBase(500);
        B200CommId id{};
        B200ShardedIndexFlat sh(local, 0, 1, id);
        std::vector<float> d1(4 * 7), d2(4 * 7);
        std::vector<faiss::idx_t> l1(4 * 7), l2(4 * 7);
        local->search(4, v.data(), 7, d1.data(), l1.data());
        sh.search(4, v.data(), 7, d2.data(), l2.data());
        for (int i = 0; i < 28; i++) CHECK(l1[i] == l2[i] && d1[i] == d2[i]);
        CHECK(l2[0] == 500);
        sh.search(4, v.data(), 7, nullptr, nullptr);   // a rank that wants no result
        std::printf("sharded rank-form world=1 PASS\n");
    }
    // every GPU of the box, when there are several
    int ndev = 0;
    if (b200f_device_count(&ndev) == B200F_OK && ndev >= 2) {
        std::vector<std::shared_ptr<B200Resources>> all;
        for (int i = 0; i < ndev; i++) all.push_back(std::make_shared<StandardB200Resources>(i));
        testSharded(all, all[0], StorageType::BFloat16, faiss::METRIC_L2, 10, "multi-gpu");
        testSharded(all, all[0], StorageType::Float16, faiss::METRIC_INNER_PRODUCT, 100, "multi-gpu");
        // a plain index on the LAST device of the process: per-device kernel attributes
        testFlat(all.back(), 3000, 200, 128, 10, faiss::METRIC_L2, StorageType::BFloat16, 5e-2f);
        testFlat(all.back(), 3000, 200, 96, 100, faiss::METRIC_L2, StorageType::Float32, 1e-3f);
    } else {
        std::printf("sharded multi-gpu SKIPPED (one device)\n");
    }
}

int main() {
    std::shared_ptr<B200Resources> res;
    try {
        res = std::make_shared<StandardB200Resources>();
    } catch (const std::exception& e) {
        std::printf("no usable device: %s\n", e.what());
        return 77;
    }
    std::printf("%s\n", describeCapabilities(res->getCapabilities()).c_str());
    // the reference's list (tests/test_metal_flat.mm:477-490)
    const size_t cases[5][4] = {{1000, 10, 32, 5}, {1000, 10, 128, 10}, {500, 5, 768, 5}, {500, 5, 1536, 5}, {100, 1, 32, 1}};
    for (auto& c : cases) testFlat(res, c[0], c[1], c[2], c[3], faiss::METRIC_L2, StorageType::Float32, 1e-3f);
    testFlat(res, 1000, 10, 128, 10, faiss::METRIC_INNER_PRODUCT, StorageType::Float32, 1e-2f);
    testFlat(res, 1000, 10, 128, 10, faiss::METRIC_L2, StorageType::Float16, 5e-2f);
    testFlat(res, 500, 5, 768, 5, faiss::METRIC_L2, StorageType::Float16, 5e-2f);
    testFlat(res, 1000, 10, 128, 10, faiss::METRIC_L2, StorageType::BFloat16, 5e-2f);
    testConversion(res);
    testErrorsAndTokens(res);
    testShardedAll(res);
    std::printf("ALL PASS\n");
    return 0;
}
