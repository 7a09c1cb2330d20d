// Handle-based C mirror of the plugin class for bindings that cannot hold a C++
// object (ctypes, cgo, JNI).  Every function catches C++ exceptions and returns a
// status code; the message is kept per thread for b200f_last_error().
#include <cuda_runtime.h>
#include <faiss/impl/FaissAssert.h>

#include <cstring>
#include <memory>
#include <new>
#include <vector>
#include <stdexcept>
#include <string>

#include "../../include/b200_flat.h"
#include "../include/faiss-b200/faiss_b200.h"

using namespace faiss_b200;

struct B200FResources {
    std::shared_ptr<StandardB200Resources> res;
};
struct B200FIndex {
    std::shared_ptr<B200IndexFlat> index;   // shared with a sharded index built over it
};
struct B200FSharded {
    std::unique_ptr<B200ShardedIndexFlat> index;
};
struct B200FToken {
    std::unique_ptr<B200SearchToken> token;
};

namespace {

thread_local std::string g_last_error;

int fail(int code, const std::string& msg) {
    g_last_error = msg;
    return code;
}

// Every exception the host layer throws carries its status code (B200Exception.h); the
// bare base classes can only come from outside it (a user-supplied resources object, the
// FAISS headers) and map to the generic code of their kind.
#define B200F_GUARD_BEGIN try {
#define B200F_GUARD_END                                                        \
    }                                                                          \
    catch (const B200ArgumentError& e) {                                       \
        return fail(e.status(), e.what());                                     \
    }                                                                          \
    catch (const B200RuntimeError& e) {                                        \
        return fail(e.status(), e.what());                                     \
    }                                                                          \
    catch (const faiss::FaissException& e) {                                   \
        return fail(B200F_ERR_BAD_ARG, e.what());                              \
    }                                                                          \
    catch (const std::bad_alloc& e) {                                          \
        return fail(B200F_ERR_OOM, e.what());                                  \
    }                                                                          \
    catch (const std::exception& e) {                                          \
        return fail(B200F_ERR_CUDA, e.what());                                 \
    }                                                                          \
    catch (...) {                                                              \
        return fail(B200F_ERR_CUDA, "unknown exception");                      \
    }

}  // namespace

extern "C" {

const char* b200f_last_error(void) { return g_last_error.c_str(); }

int b200f_debug_raise(int status) {
    B200F_GUARD_BEGIN
    switch (status) {
        case B200F_OK: return B200F_OK;
        case B200F_ERR_BAD_ARG:
        case B200F_ERR_UNSUPPORTED:
        case B200F_ERR_RANGE:
        case B200F_ERR_STATE:
            throw B200ArgumentError(status, std::string("raised for the test: ") + b200f_status_string(status));
        case -1: throw faiss::FaissException("a bare FaissException");
        case -2: throw std::runtime_error("a bare runtime_error");
        case -3: throw std::bad_alloc();
        default:
            throw B200RuntimeError(status, std::string("raised for the test: ") + b200f_status_string(status));
    }
    B200F_GUARD_END
}

int b200f_resources_create(int device, B200FResources** out) {
    if (!out) return fail(B200F_ERR_BAD_ARG, "null output pointer");
    *out = nullptr;
    B200F_GUARD_BEGIN
    std::unique_ptr<B200FResources> h(new B200FResources);
    h->res = std::make_shared<StandardB200Resources>(device);
    *out = h.release();
    return B200F_OK;
    B200F_GUARD_END
}

void b200f_resources_destroy(B200FResources* res) { delete res; }

int b200f_resources_device(const B200FResources* res) { return res ? res->res->getDevice() : -1; }

void* b200f_resources_stream(const B200FResources* res) {
    return res ? static_cast<void*>(res->res->getDefaultStream()) : nullptr;
}

int b200f_resources_wait_stream(B200FResources* res, void* producer_stream) {
    if (!res) return fail(B200F_ERR_BAD_ARG, "null resources");
    B200F_GUARD_BEGIN
    res->res->waitStream(static_cast<StreamHandle>(producer_stream));
    return B200F_OK;
    B200F_GUARD_END
}

size_t b200f_resources_scratch_bytes(const B200FResources* res) {
    return res ? res->res->getScratchSize() : 0;
}

int b200f_index_create(B200FResources* res, int d, int metric, int storage, B200FIndex** out) {
    if (!out) return fail(B200F_ERR_BAD_ARG, "null output pointer");
    *out = nullptr;
    if (!res) return fail(B200F_ERR_BAD_ARG, "null resources");
    if (metric != B200F_METRIC_L2 && metric != B200F_METRIC_INNER_PRODUCT)
        return fail(B200F_ERR_BAD_ARG, "metric must be L2 or inner product");
    if (storage < 0 || storage > 2) return fail(B200F_ERR_BAD_ARG, "invalid storage type");
    B200F_GUARD_BEGIN
    std::unique_ptr<B200FIndex> h(new B200FIndex);
    h->index.reset(new B200IndexFlat(res->res, d,
                                     metric == B200F_METRIC_L2 ? faiss::METRIC_L2
                                                               : faiss::METRIC_INNER_PRODUCT,
                                     static_cast<StorageType>(storage)));
    *out = h.release();
    return B200F_OK;
    B200F_GUARD_END
}

void b200f_index_destroy(B200FIndex* index) { delete index; }

int b200f_index_add(B200FIndex* index, int64_t n, const float* x) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->add(n, x);
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_index_reserve(B200FIndex* index, int64_t n) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->reserve(n);
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_index_search(const B200FIndex* index, int64_t n, const float* x, int64_t k,
                       float* distances, int64_t* labels) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->search(n, x, k, distances, reinterpret_cast<faiss::idx_t*>(labels));
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_index_search_enqueue(const B200FIndex* index, int64_t n, const float* x, int64_t k,
                               float* distances, int64_t* labels) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->searchDeviceEnqueue(n, x, k, distances, reinterpret_cast<faiss::idx_t*>(labels));
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_index_synchronize(const B200FIndex* index) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->synchronize();
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_index_search_async(const B200FIndex* index, int64_t n, const float* x, int64_t k,
                             float* distances, int64_t* labels, B200FToken** out) {
    if (!out) return fail(B200F_ERR_BAD_ARG, "null output pointer");
    *out = nullptr;
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    std::unique_ptr<B200FToken> h(new B200FToken);
    h->token.reset(new B200SearchToken(
            index->index->searchAsync(n, x, k, distances, reinterpret_cast<faiss::idx_t*>(labels))));
    *out = h.release();
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_token_wait(B200FToken* token) {
    if (!token || !token->token) return fail(B200F_ERR_STATE, "null or consumed token");
    B200F_GUARD_BEGIN
    token->token->wait();
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_token_is_ready(const B200FToken* token, int* ready) {
    if (!token || !token->token || !ready) return fail(B200F_ERR_STATE, "null or consumed token");
    B200F_GUARD_BEGIN
    *ready = token->token->isReady() ? 1 : 0;
    return B200F_OK;
    B200F_GUARD_END
}

void b200f_token_destroy(B200FToken* token) { delete token; }

int b200f_index_reset(B200FIndex* index) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->reset();
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_index_reconstruct(const B200FIndex* index, int64_t key, float* recons) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->reconstruct(key, recons);
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_index_reconstruct_n(const B200FIndex* index, int64_t first, int64_t n, float* out) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->reconstruct_n(first, n, out);
    return B200F_OK;
    B200F_GUARD_END
}

int64_t b200f_index_ntotal(const B200FIndex* index) { return index ? index->index->ntotal : -1; }
int b200f_index_d(const B200FIndex* index) { return index ? index->index->d : -1; }
int b200f_index_metric(const B200FIndex* index) {
    if (!index) return -1;
    return index->index->metric_type == faiss::METRIC_L2 ? B200F_METRIC_L2 : B200F_METRIC_INNER_PRODUCT;
}
int b200f_index_storage(const B200FIndex* index) {
    return index ? (int)index->index->getStorageType() : -1;
}

int b200f_index_set_path(B200FIndex* index, int path) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->setForcePath(path);
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_index_set_label_base(B200FIndex* index, int64_t base) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->setLabelBase(base);
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_index_set_growth_mode(B200FIndex* index, int mode) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->setGrowthMode(mode);
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_index_set_fp32_planes(B200FIndex* index, int format) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->setFp32PlaneFormat(format);
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_index_fp32_planes(const B200FIndex* index) { return index ? index->index->getFp32PlaneFormat() : -1; }

int b200f_index_set_use_graphs(B200FIndex* index, int on) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->setUseGraphs(on != 0);
    return B200F_OK;
    B200F_GUARD_END
}

const void* b200f_index_device_rows(const B200FIndex* index) {
    return index ? index->index->getDeviceRows() : nullptr;
}

int b200f_index_last_device_status(const B200FIndex* index) {
    return index ? index->index->lastDeviceStatus() : -1;
}

int b200f_index_debug_wait_expiry(B200FIndex* index, int64_t limit_cycles) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->debugWaitExpiry(limit_cycles);
    return B200F_OK;
    B200F_GUARD_END
}

// ---- sharded index ------------------------------------------------------------------------

int b200f_comm_id_create(void* id128) {
    if (!id128) return fail(B200F_ERR_BAD_ARG, "null output pointer");
    B200F_GUARD_BEGIN
    const B200CommId id = createCommId();
    std::memcpy(id128, id.bytes, sizeof(id.bytes));
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_sharded_create(B200FResources* const* res, int nshards, int d, int metric, int storage,
                         int64_t block_rows, B200FSharded** out) {
    if (!out) return fail(B200F_ERR_BAD_ARG, "null output pointer");
    *out = nullptr;
    if (!res || nshards < 1) return fail(B200F_ERR_BAD_ARG, "at least one resources handle is needed");
    if (metric != B200F_METRIC_L2 && metric != B200F_METRIC_INNER_PRODUCT)
        return fail(B200F_ERR_BAD_ARG, "metric must be L2 or inner product");
    if (storage < 0 || storage > 2) return fail(B200F_ERR_BAD_ARG, "invalid storage type");
    B200F_GUARD_BEGIN
    std::vector<std::shared_ptr<B200Resources>> rs;
    for (int i = 0; i < nshards; i++) {
        if (!res[i]) return fail(B200F_ERR_BAD_ARG, "null resources");
        rs.push_back(res[i]->res);
    }
    std::unique_ptr<B200FSharded> h(new B200FSharded);
    h->index.reset(new B200ShardedIndexFlat(std::move(rs), d,
                                            metric == B200F_METRIC_L2 ? faiss::METRIC_L2 : faiss::METRIC_INNER_PRODUCT,
                                            static_cast<StorageType>(storage), block_rows));
    *out = h.release();
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_sharded_create_rank(B200FIndex* local, int rank, int world, const void* id128, B200FSharded** out) {
    if (!out) return fail(B200F_ERR_BAD_ARG, "null output pointer");
    *out = nullptr;
    if (!local) return fail(B200F_ERR_BAD_ARG, "null index");
    if (world > 1 && !id128) return fail(B200F_ERR_BAD_ARG, "null communicator id");
    B200F_GUARD_BEGIN
    B200CommId id;
    std::memset(id.bytes, 0, sizeof(id.bytes));
    if (id128) std::memcpy(id.bytes, id128, sizeof(id.bytes));
    std::unique_ptr<B200FSharded> h(new B200FSharded);
    h->index.reset(new B200ShardedIndexFlat(local->index, rank, world, id));
    *out = h.release();
    return B200F_OK;
    B200F_GUARD_END
}

void b200f_sharded_destroy(B200FSharded* index) { delete index; }

int b200f_sharded_add(B200FSharded* index, int64_t n, const float* x) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->add(n, x);
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_sharded_search(const B200FSharded* index, int64_t n, const float* x, int64_t k, float* distances,
                         int64_t* labels) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->search(n, x, k, distances, reinterpret_cast<faiss::idx_t*>(labels));
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_sharded_search_enqueue(const B200FSharded* index, int64_t n, const float* x, int64_t k, float* distances,
                                 int64_t* labels) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->searchDeviceEnqueue(n, x, k, distances, reinterpret_cast<faiss::idx_t*>(labels));
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_sharded_synchronize(const B200FSharded* index) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->synchronize();
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_sharded_reset(B200FSharded* index) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->reset();
    return B200F_OK;
    B200F_GUARD_END
}

int b200f_sharded_reconstruct(const B200FSharded* index, int64_t key, float* recons) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->reconstruct(key, recons);
    return B200F_OK;
    B200F_GUARD_END
}

int64_t b200f_sharded_ntotal(const B200FSharded* index) { return index ? index->index->ntotal : -1; }
int b200f_sharded_num_shards(const B200FSharded* index) { return index ? index->index->numShards() : -1; }

int b200f_sharded_set_use_graphs(B200FSharded* index, int on) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    index->index->setUseGraphs(on != 0);
    return B200F_OK;
}

int b200f_sharded_trace(B200FSharded* index, int on) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    index->index->setTrace(on != 0);
    return B200F_OK;
}

int64_t b200f_sharded_trace_read(const B200FSharded* index, float* enqueue_us, float* wait_us, int64_t capacity) {
    if (!index || capacity < 0) return -1;
    return (int64_t)index->index->readTrace(enqueue_us, wait_us, (size_t)capacity);
}

int b200f_sharded_set_path(B200FSharded* index, int path) {
    if (!index) return fail(B200F_ERR_BAD_ARG, "null index");
    B200F_GUARD_BEGIN
    index->index->setForcePath(path);
    return B200F_OK;
    B200F_GUARD_END
}

}  // extern "C"
