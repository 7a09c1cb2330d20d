// B200ShardedIndexFlat: row shards over the GPUs of one box, NCCL all-gather of the per-GPU
// candidates issued directly on the resources' streams, k-way merge kernel.
// The reference is single-device (src/StandardMetalResources.mm:17-23); the per-shard search is
// the path of src/MetalIndexFlat.mm:313-401, the exchange and merge have no counterpart there.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <chrono>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>

#include "../../include/b200_flat.h"
#include "../include/faiss-b200/B200Exception.h"
#include "../include/faiss-b200/B200Resources.h"
#include "../include/faiss-b200/B200ShardedIndexFlat.h"

namespace faiss_b200 {

namespace {

constexpr int64_t kFusedBatch = 16384;   // queries per launch, k <= B200F_LIST_MAX_K
constexpr int64_t kSelectBatch = 1024;   // beyond: few rows, wide column chunks
constexpr size_t kSmallQueryBytes = 64 * 1024;
constexpr int64_t kGraphMaxQueries = 8;  // searches this small are replayed from a CUDA graph
constexpr size_t kMaxGraphs = 8;

size_t alignUp(size_t x, size_t a) { return (x + a - 1) / a * a; }

void cudaCheck(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        std::string msg = std::string("faiss-b200: ") + what + ": " + cudaGetErrorString(e);
        (void)cudaGetLastError();
        throw B200RuntimeError(e == cudaErrorMemoryAllocation ? B200F_ERR_OOM : B200F_ERR_CUDA, msg);
    }
}

void abiCheck(int rc, const char* what) {
    if (rc == B200F_OK) return;
    std::string msg = std::string("faiss-b200: ") + what + ": " + b200f_status_string(rc);
    if (rc == B200F_ERR_BAD_ARG || rc == B200F_ERR_UNSUPPORTED || rc == B200F_ERR_RANGE || rc == B200F_ERR_STATE)
        throw B200ArgumentError(rc, msg);
    throw B200RuntimeError(rc, msg);
}

bool isDevicePointer(const void* p) {
    if (!p) return false;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) cudaCheck(cudaSetDevice(dev), "cudaSetDevice");
    }
    ~DeviceGuard() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) (void)cudaSetDevice(prev);
    }
};

// NCCL is looked up at run time (the copy already loaded into the process, else the system
// one): the library keeps no link-time dependency on it, and a single-GPU user never loads it.
struct NcclApi {
    decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&ncclCommInitRank) CommInitRank = nullptr;
    decltype(&ncclCommInitAll) CommInitAll = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclAllGather) AllGather = nullptr;
    decltype(&ncclGroupStart) GroupStart = nullptr;
    decltype(&ncclGroupEnd) GroupEnd = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;

    static const NcclApi& get() {
        static NcclApi api;
        static std::once_flag once;
        static std::string error;
        std::call_once(once, [] {
            void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
            if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
            if (!h) {
                error = std::string("NCCL library not found: ") + dlerror();
                return;
            }
#define B200F_NCCL_SYM(NAME)                                                        \
    api.NAME = reinterpret_cast<decltype(api.NAME)>(dlsym(h, "nccl" #NAME));          \
    if (!api.NAME) error = "NCCL symbol nccl" #NAME " not found";
            B200F_NCCL_SYM(GetUniqueId)
            B200F_NCCL_SYM(CommInitRank)
            B200F_NCCL_SYM(CommInitAll)
            B200F_NCCL_SYM(CommDestroy)
            B200F_NCCL_SYM(AllGather)
            B200F_NCCL_SYM(GroupStart)
            B200F_NCCL_SYM(GroupEnd)
            B200F_NCCL_SYM(GetErrorString)
#undef B200F_NCCL_SYM
        });
        if (!error.empty()) throw B200RuntimeError(B200F_ERR_CUDA, "faiss-b200: " + error);
        return api;
    }
};

void ncclCheck(ncclResult_t r, const char* what) {
    if (r != ncclSuccess)
        throw B200RuntimeError(B200F_ERR_CUDA, std::string("faiss-b200: ") + what + ": " +
                                                       NcclApi::get().GetErrorString(r));
}

}  // namespace

B200CommId createCommId() {
    static_assert(sizeof(ncclUniqueId) == sizeof(B200CommId), "communicator id is 128 bytes");
    ncclUniqueId id;
    ncclCheck(NcclApi::get().GetUniqueId(&id), "ncclGetUniqueId");
    B200CommId out;
    std::memcpy(out.bytes, &id, sizeof(id));
    return out;
}

// ---------------------------------------------------------------------------------------
struct B200ShardedIndexFlat::Impl {
    enum class Exchange { None, Nccl, SameDevice };
    bool ranks = false;            // one process per GPU
    Exchange exchange = Exchange::None;
    int rank = 0, world = 1;
    int64_t blockRows = 65536;
    int d = 0;
    bool l2 = true;
    std::vector<std::shared_ptr<B200Resources>> res;   // per shard of this process
    std::vector<std::shared_ptr<B200IndexFlat>> shards;
    std::vector<ncclComm_t> comms;                     // per shard of this process (Exchange::Nccl)

    // grow-only device buffers per shard: queries of all parts, this process's view of all
    // parts' candidates ([distances | labels] per part), merged result staging
    struct Buffers {
        void* queries = nullptr;
        size_t queryBytes = 0;
        void* cand = nullptr;
        size_t candBytes = 0;
        void* out = nullptr;
        size_t outBytes = 0;
    };
    std::vector<Buffers> buf;

    // One process per GPU, host buffers, at most kGraphMaxQueries queries: the whole call
    // (query upload, shard search, candidate all-gather, merge, result download) is captured
    // into a CUDA graph the second time a shape is seen and replayed afterwards.  A graph owns
    // every buffer it touches and is tied to the local index as it was (generation).
    struct CallGraph {
        int64_t n = 0, k = 0;
        bool wantResult = false;
        int selectMode = 0;
        uint64_t generation = 0;
        void* dev = nullptr;        // queries | candidates of all parts | merged result | search scratch
        uint8_t* host = nullptr;    // pinned: queries | distances | labels
        size_t hostDistOff = 0, hostLabOff = 0;
        cudaGraph_t graph = nullptr;
        cudaGraphExec_t exec = nullptr;
        uint64_t lastUse = 0;
    };
    std::vector<CallGraph> graphs;
    std::vector<std::pair<int64_t, int64_t>> seenShapes;
    uint64_t useCounter = 0;
    bool useGraphs = true;

    // Host-side trace of the calls (off by default): microseconds from entry until everything
    // was enqueued, and from there until the stream had drained.  A rank whose enqueue time is
    // large was late on the host; large waits with small enqueue times on every rank point at
    // the device or the exchange.
    bool trace = false;
    std::vector<float> traceEnqueueUs, traceWaitUs;

    void destroyGraph(CallGraph& g) {
        if (g.exec) (void)cudaGraphExecDestroy(g.exec);
        if (g.graph) (void)cudaGraphDestroy(g.graph);
        if (g.dev) res[0]->deallocBuffer(g.dev);
        if (g.host) res[0]->releasePinnedTemp(g.host);
        g = CallGraph{};
    }
    bool searchFromGraph(int64_t n, const float* x, int64_t k, float* distances, faiss::idx_t* labels);

    int localShards() const { return (int)shards.size(); }
    int parts() const { return ranks ? world : localShards(); }   // lists merged per query
    int partOf(int s) const { return ranks ? rank : s; }
    cudaStream_t stream(int s) const { return reinterpret_cast<cudaStream_t>(res[s]->getDefaultStream()); }
    // with every shard on one device the shards share buffers: each writes its part in place
    int bufOf(int s) const { return exchange == Exchange::SameDevice ? 0 : s; }

    void* grow(int s, void*& p, size_t& have, size_t want) {
        if (want > have) {
            DeviceGuard g(res[s]->getDevice());
            cudaCheck(cudaStreamSynchronize(stream(s)), "synchronize");
            if (p) res[s]->deallocBuffer(p);
            p = nullptr;
            have = 0;
            p = res[s]->allocBuffer(want);
            have = want;
        }
        return p;
    }

    void destroy() {
        if (!graphs.empty()) {
            try {
                DeviceGuard g(res[0]->getDevice());
                (void)cudaStreamSynchronize(stream(0));
                for (auto& gr : graphs) destroyGraph(gr);
            } catch (...) {
            }
            graphs.clear();
        }
        for (size_t s = 0; s < buf.size(); s++) {
            if (!res[s]) continue;
            try {
                DeviceGuard g(res[s]->getDevice());
                (void)cudaStreamSynchronize(stream((int)s));
                if (buf[s].queries) res[s]->deallocBuffer(buf[s].queries);
                if (buf[s].cand) res[s]->deallocBuffer(buf[s].cand);
                if (buf[s].out) res[s]->deallocBuffer(buf[s].out);
            } catch (...) {
            }
        }
        buf.clear();
        for (ncclComm_t c : comms)
            if (c) (void)NcclApi::get().CommDestroy(c);
        comms.clear();
    }

    // One all-gather per local shard: part p of `data` (count elements of `bytesPer` bytes,
    // starting at part * partBytes) is sent, every part is received in place.
    void allGather(void* const* data, size_t partBytes) const {
        if (exchange != Exchange::Nccl) return;
        const NcclApi& nccl = NcclApi::get();
        const int S = localShards();
        if (S > 1) ncclCheck(nccl.GroupStart(), "ncclGroupStart");
        for (int s = 0; s < S; s++) {
            DeviceGuard g(res[s]->getDevice());
            uint8_t* base = static_cast<uint8_t*>(data[s]);
            ncclCheck(nccl.AllGather(base + (size_t)partOf(s) * partBytes, base, partBytes, ncclUint8, comms[s], stream(s)),
                      "ncclAllGather");
        }
        if (S > 1) ncclCheck(nccl.GroupEnd(), "ncclGroupEnd");
    }

    // One batch: queries onto every GPU, shard searches, candidate exchange, merge.  Everything
    // is enqueued; the caller decides whether to wait.  outDist / outLabels: device pointers on
    // the merging shard's GPU, or nullptr for "no result wanted here".
    void enqueueBatch(int64_t nq, const float* x, bool xOnDevice, int64_t k, float* outDist, faiss::idx_t* outLabels);
};

// ---------------------------------------------------------------------------------------
B200ShardedIndexFlat::B200ShardedIndexFlat(std::vector<std::shared_ptr<B200Resources>> resources, int d_,
                                           faiss::MetricType metric, StorageType storage, int64_t blockRows)
        : faiss::Index(d_, metric), impl_(new Impl) {
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, !resources.empty(), "at least one resources object is needed");
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, blockRows >= 1, "blockRows must be >= 1");
    for (auto& r : resources) B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, r != nullptr, "resources must not be null");
    Impl& im = *impl_;
    im.blockRows = blockRows;
    im.d = d_;
    im.l2 = metric == faiss::METRIC_L2;
    const int S = (int)resources.size();
    bool sameDevice = true, distinct = true;
    for (int i = 0; i < S; i++)
        for (int j = i + 1; j < S; j++) {
            if (resources[i]->getDevice() == resources[j]->getDevice()) distinct = false;
            else sameDevice = false;
        }
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, S == 1 || distinct || sameDevice,
                          "shards must be on pairwise different GPUs, or all on one GPU");
    if (S > 1 && sameDevice) {
        // every shard runs on the first resources' stream: one stream orders everything
        for (int i = 0; i < S; i++) im.res.push_back(resources[0]);
        im.exchange = Impl::Exchange::SameDevice;
    } else {
        im.res = std::move(resources);
        im.exchange = S > 1 ? Impl::Exchange::Nccl : Impl::Exchange::None;
    }
    for (int i = 0; i < S; i++) im.shards.push_back(std::make_shared<B200IndexFlat>(im.res[i], d_, metric, storage));
    im.buf.resize(S);
    if (im.exchange == Impl::Exchange::Nccl) {
        std::vector<int> devs;
        for (auto& r : im.res) devs.push_back(r->getDevice());
        im.comms.assign(S, nullptr);
        ncclCheck(NcclApi::get().CommInitAll(im.comms.data(), S, devs.data()), "ncclCommInitAll");
    }
    is_trained = true;
    ntotal = 0;
}

B200ShardedIndexFlat::B200ShardedIndexFlat(std::shared_ptr<B200IndexFlat> local, int rank, int world,
                                           const B200CommId& id)
        : faiss::Index(local ? local->d : 1, local ? local->metric_type : faiss::METRIC_L2), impl_(new Impl) {
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, local != nullptr, "local index must not be null");
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, world >= 1 && rank >= 0 && rank < world, "rank outside [0, world)");
    Impl& im = *impl_;
    im.ranks = true;
    im.rank = rank;
    im.world = world;
    im.d = local->d;
    im.l2 = local->metric_type == faiss::METRIC_L2;
    im.res.push_back(local->getResources());
    im.shards.push_back(std::move(local));
    im.buf.resize(1);
    im.exchange = world > 1 ? Impl::Exchange::Nccl : Impl::Exchange::None;
    if (world > 1) {
        DeviceGuard g(im.res[0]->getDevice());
        ncclUniqueId nid;
        std::memcpy(&nid, id.bytes, sizeof(nid));
        im.comms.assign(1, nullptr);
        ncclCheck(NcclApi::get().CommInitRank(&im.comms[0], world, nid, rank), "ncclCommInitRank");
    }
    is_trained = true;
    ntotal = im.shards[0]->ntotal;   // this rank's rows
}

B200ShardedIndexFlat::~B200ShardedIndexFlat() {
    if (impl_) impl_->destroy();
}

int B200ShardedIndexFlat::numShards() const { return impl_->localShards(); }
int B200ShardedIndexFlat::rank() const { return impl_->rank; }
int B200ShardedIndexFlat::world() const { return impl_->world; }
const B200IndexFlat* B200ShardedIndexFlat::shard(int i) const {
    B200_THROW_ARG_IF_NOT(B200F_ERR_RANGE, i >= 0 && i < impl_->localShards(), "shard number out of range");
    return impl_->shards[(size_t)i].get();
}
void B200ShardedIndexFlat::setForcePath(int path) {
    for (auto& s : impl_->shards) s->setForcePath(path);
}

// ---------------------------------------------------------------------------------------
void B200ShardedIndexFlat::add(faiss::idx_t n, const float* x) {
    if (n == 0) return;
    Impl& im = *impl_;
    B200_THROW_ARG_IF_NOT(B200F_ERR_STATE, !im.ranks,
                          "one process per GPU: add this rank's rows to its local index instead");
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, n > 0 && x != nullptr, "add: invalid arguments");
    const int S = im.localShards();
    const int64_t B = im.blockRows;
    // runs of rows that fall into one block, in global order; shard s takes every S-th block
    struct Run {
        const float* src;
        int64_t rows;
    };
    std::vector<std::vector<Run>> runs((size_t)S);
    for (int64_t g = ntotal; g < ntotal + n;) {
        const int64_t blockEnd = (g / B + 1) * B;
        const int64_t take = std::min<int64_t>(blockEnd, ntotal + n) - g;
        runs[(size_t)((g / B) % S)].push_back(Run{x + (size_t)(g - ntotal) * d, take});
        g += take;
    }
    // the shards ingest in parallel: each GPU has its own PCIe link and its own ingest pipeline
    std::vector<std::exception_ptr> errors((size_t)S);
    auto work = [&](int s) {
        try {
            for (const Run& r : runs[(size_t)s]) im.shards[(size_t)s]->add(r.rows, r.src);
        } catch (...) {
            errors[(size_t)s] = std::current_exception();
        }
    };
    if (im.exchange == Impl::Exchange::Nccl) {
        std::vector<std::thread> threads;
        for (int s = 1; s < S; s++) threads.emplace_back(work, s);
        work(0);
        for (auto& t : threads) t.join();
    } else {
        for (int s = 0; s < S; s++) work(s);   // one device, one stream: nothing to overlap
    }
    for (auto& e : errors)
        if (e) std::rethrow_exception(e);
    ntotal += n;
}

void B200ShardedIndexFlat::reset() {
    for (auto& s : impl_->shards) s->reset();
    ntotal = 0;
}

void B200ShardedIndexFlat::reconstruct(faiss::idx_t key, float* recons) const {
    const Impl& im = *impl_;
    B200_THROW_ARG_IF_NOT(B200F_ERR_STATE, !im.ranks, "one process per GPU: reconstruct from the rank's local index");
    B200_THROW_ARG_IF_NOT(B200F_ERR_RANGE, key >= 0 && key < ntotal,
                          "reconstruct: key " + std::to_string(key) + " out of range [0, " + std::to_string(ntotal) + ")");
    const int64_t B = im.blockRows, S = im.localShards();
    im.shards[(size_t)((key / B) % S)]->reconstruct((key / (B * S)) * B + key % B, recons);
}

// ---------------------------------------------------------------------------------------
namespace {
void checkSearchArgs(faiss::idx_t n, const float* x, faiss::idx_t k) {
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, k > 0, "k must be > 0");
    B200_THROW_ARG_IF_NOT(B200F_ERR_UNSUPPORTED, k <= B200F_MAX_K,
                          "k = " + std::to_string(k) + " exceeds the maximum of " + std::to_string(B200F_MAX_K));
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, n >= 0, "n must be >= 0");
    if (n > 0) B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, x != nullptr, "search: null queries");
}
}  // namespace

void B200ShardedIndexFlat::search(faiss::idx_t n, const float* x, faiss::idx_t k, float* distances,
                                  faiss::idx_t* labels, const faiss::SearchParameters*) const {
    checkSearchArgs(n, x, k);
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, (distances == nullptr) == (labels == nullptr),
                          "search: distances and labels must both be given or both be null");
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, impl_->ranks || distances != nullptr, "search: null outputs");
    if (n == 0) return;
    Impl& im = *impl_;
    const bool xOnDevice = isDevicePointer(x);
    const bool wantResult = distances != nullptr;
    const bool outOnDevice = wantResult && isDevicePointer(distances);
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, !wantResult || outOnDevice == isDevicePointer(labels),
                          "search: distances and labels must live in the same memory space");
    const int64_t batch = std::min<int64_t>(n, k <= B200F_LIST_MAX_K ? kFusedBatch : kSelectBatch);
    const int m = 0;   // merging shard
    DeviceGuard g(im.res[m]->getDevice());
    const auto t0 = std::chrono::steady_clock::now();
    if (im.ranks && im.useGraphs && n <= kGraphMaxQueries && !xOnDevice && !outOnDevice &&
        im.searchFromGraph(n, x, k, distances, labels))
        return;
    for (int64_t q0 = 0; q0 < n; q0 += batch) {
        const int64_t nq = std::min<int64_t>(batch, n - q0);
        float* dOut = nullptr;
        faiss::idx_t* lOut = nullptr;
        if (wantResult) {
            if (outOnDevice) {
                dOut = distances + (size_t)q0 * k;
                lOut = labels + (size_t)q0 * k;
            } else {
                Impl::Buffers& b = im.buf[(size_t)im.bufOf(m)];
                const size_t distBytes = alignUp((size_t)nq * k * 4, 256);
                uint8_t* out = static_cast<uint8_t*>(im.grow(m, b.out, b.outBytes, distBytes + (size_t)nq * k * 8));
                dOut = reinterpret_cast<float*>(out);
                lOut = reinterpret_cast<faiss::idx_t*>(out + distBytes);
            }
        }
        im.enqueueBatch(nq, x + (size_t)q0 * d, xOnDevice, k, dOut, lOut);
        if (wantResult && !outOnDevice) {
            cudaStream_t st = im.stream(m);
            cudaCheck(cudaMemcpyAsync(distances + (size_t)q0 * k, dOut, (size_t)nq * k * 4, cudaMemcpyDeviceToHost, st),
                      "search: device to host copy of distances");
            cudaCheck(cudaMemcpyAsync(labels + (size_t)q0 * k, lOut, (size_t)nq * k * 8, cudaMemcpyDeviceToHost, st),
                      "search: device to host copy of labels");
        }
        // host buffers are the caller's again on return, and the next batch reuses the staging
        const auto t1 = std::chrono::steady_clock::now();
        synchronize();
        if (im.trace && im.traceEnqueueUs.size() < (size_t)1 << 20) {
            const auto t2 = std::chrono::steady_clock::now();
            im.traceEnqueueUs.push_back(std::chrono::duration<float, std::micro>(t1 - t0).count());
            im.traceWaitUs.push_back(std::chrono::duration<float, std::micro>(t2 - t1).count());
        }
    }
}

// The rank form's small search through a captured graph.  First call with a shape: ordinary
// path (it also performs every lazy set-up of this library and of NCCL for that message size,
// none of which belongs inside a capture); second call: capture; afterwards: one memcpy into
// the pinned slot, one graph launch, one synchronisation, one memcpy out.  Every rank takes
// the same decisions, because every rank sees the same sequence of (n, k); a rank whose capture
// fails falls back to the ordinary path for good, which issues the same collective.
bool B200ShardedIndexFlat::Impl::searchFromGraph(int64_t n, const float* x, int64_t k, float* distances,
                                                 faiss::idx_t* labels) {
    const auto t0 = std::chrono::steady_clock::now();
    Impl& im = *this;
    cudaStream_t st = im.stream(0);
    const bool wantResult = distances != nullptr;
    const int selectMode = b200f_get_selection_mode();
    const uint64_t gen = im.shards[0]->generation();
    CallGraph* g = nullptr;
    for (size_t i = 0; i < im.graphs.size();) {
        if (im.graphs[i].generation != gen) {   // the local index changed: stale
            cudaCheck(cudaStreamSynchronize(st), "search: synchronize");
            im.destroyGraph(im.graphs[i]);
            im.graphs.erase(im.graphs.begin() + (long)i);
            continue;
        }
        if (im.graphs[i].n == n && im.graphs[i].k == k && im.graphs[i].wantResult == wantResult &&
            im.graphs[i].selectMode == selectMode)
            g = &im.graphs[i];
        i++;
    }
    if (!g) {
        const std::pair<int64_t, int64_t> shape(n, k);
        if (std::find(im.seenShapes.begin(), im.seenShapes.end(), shape) == im.seenShapes.end()) {
            if (im.seenShapes.size() >= 64) im.seenShapes.clear();
            im.seenShapes.push_back(shape);
            return false;
        }
        if (im.graphs.size() >= kMaxGraphs) {
            size_t oldest = 0;
            for (size_t i = 1; i < im.graphs.size(); i++)
                if (im.graphs[i].lastUse < im.graphs[oldest].lastUse) oldest = i;
            cudaCheck(cudaStreamSynchronize(st), "search: synchronize");
            im.destroyGraph(im.graphs[oldest]);
            im.graphs.erase(im.graphs.begin() + (long)oldest);
        }
        const int P = im.parts();
        const int d = im.d;
        const size_t qBytes = alignUp((size_t)n * d * 4, 256);
        const size_t distBytes = alignUp((size_t)n * k * 4, 16);
        const size_t partBytes = alignUp(distBytes + (size_t)n * k * 8, 16);
        const size_t candBytes = alignUp((size_t)P * partBytes, 256);
        const size_t outDist = alignUp((size_t)n * k * 4, 256);
        const size_t outBytes = outDist + alignUp((size_t)n * k * 8, 256);
        const size_t scratchBytes = im.shards[0]->searchScratchBytes(n, k);
        CallGraph e;
        e.n = n;
        e.k = k;
        e.wantResult = wantResult;
        e.selectMode = selectMode;
        e.generation = gen;
        e.hostDistOff = qBytes;
        e.hostLabOff = qBytes + outDist;
        try {
            e.dev = im.res[0]->allocBuffer(qBytes + candBytes + outBytes + scratchBytes);
            e.host = static_cast<uint8_t*>(im.res[0]->acquirePinnedTemp(qBytes + outBytes));
            if (!e.host) throw B200RuntimeError(B200F_ERR_OOM, "faiss-b200: pinned allocation failed");
            uint8_t* dev = static_cast<uint8_t*>(e.dev);
            float* q = reinterpret_cast<float*>(dev);
            uint8_t* cand = dev + qBytes;
            uint8_t* mine = cand + (size_t)im.rank * partBytes;
            float* outD = reinterpret_cast<float*>(dev + qBytes + candBytes);
            faiss::idx_t* outL = reinterpret_cast<faiss::idx_t*>(dev + qBytes + candBytes + outDist);
            void* scratch = dev + qBytes + candBytes + outBytes;
            // relaxed: NCCL may make calls of its own while its collective is being captured
            cudaCheck(cudaStreamBeginCapture(st, cudaStreamCaptureModeRelaxed), "search: begin capture");
            bool ok = true;
            try {
                cudaCheck(cudaMemcpyAsync(q, e.host, (size_t)n * d * 4, cudaMemcpyHostToDevice, st), "capture: upload");
                float* dLoc = reinterpret_cast<float*>(mine);
                faiss::idx_t* lLoc = reinterpret_cast<faiss::idx_t*>(mine + distBytes);
                if (P == 1) {
                    dLoc = outD;
                    lLoc = outL;
                }
                im.shards[0]->searchDeviceEnqueue(n, q, k, dLoc, lLoc, scratch, scratchBytes);
                if (P > 1) {
                    ncclCheck(NcclApi::get().AllGather(mine, cand, partBytes, ncclUint8, im.comms[0], st), "ncclAllGather");
                    if (wantResult)
                        abiCheck(b200f_merge_lists_strided(reinterpret_cast<const float*>(cand),
                                                           reinterpret_cast<const int64_t*>(cand + distBytes),
                                                           (int64_t)(partBytes / 4), (int64_t)(partBytes / 8), P, n, (int)k,
                                                           im.l2 ? B200F_METRIC_L2 : B200F_METRIC_INNER_PRODUCT, outD,
                                                           reinterpret_cast<int64_t*>(outL), st),
                                 "merge lists");
                }
                if (wantResult) {
                    cudaCheck(cudaMemcpyAsync(e.host + e.hostDistOff, outD, (size_t)n * k * 4, cudaMemcpyDeviceToHost, st),
                              "capture: download");
                    cudaCheck(cudaMemcpyAsync(e.host + e.hostLabOff, outL, (size_t)n * k * 8, cudaMemcpyDeviceToHost, st),
                              "capture: download");
                }
            } catch (...) {
                ok = false;
            }
            const cudaError_t ee = cudaStreamEndCapture(st, &e.graph);   // always ends the capture
            if (!ok || ee != cudaSuccess || !e.graph || cudaGraphInstantiate(&e.exec, e.graph, 0) != cudaSuccess) {
                (void)cudaGetLastError();
                im.destroyGraph(e);
                im.useGraphs = false;   // cannot capture here: the ordinary path from now on
                return false;
            }
        } catch (...) {
            im.destroyGraph(e);
            throw;
        }
        im.graphs.push_back(e);
        g = &im.graphs.back();
    }
    g->lastUse = ++im.useCounter;
    std::memcpy(g->host, x, (size_t)n * im.d * 4);
    cudaCheck(cudaGraphLaunch(g->exec, st), "search: graph launch");
    const auto t1 = std::chrono::steady_clock::now();
    im.shards[0]->synchronize();   // waits, and reports the search's device status word
    if (wantResult) {
        std::memcpy(distances, g->host + g->hostDistOff, (size_t)n * k * 4);
        std::memcpy(labels, g->host + g->hostLabOff, (size_t)n * k * 8);
    }
    if (im.trace && im.traceEnqueueUs.size() < (size_t)1 << 20) {
        const auto t2 = std::chrono::steady_clock::now();
        im.traceEnqueueUs.push_back(std::chrono::duration<float, std::micro>(t1 - t0).count());
        im.traceWaitUs.push_back(std::chrono::duration<float, std::micro>(t2 - t1).count());
    }
    return true;
}

void B200ShardedIndexFlat::setUseGraphs(bool on) { impl_->useGraphs = on; }

void B200ShardedIndexFlat::setTrace(bool on) {
    impl_->trace = on;
    impl_->traceEnqueueUs.clear();
    impl_->traceWaitUs.clear();
}

size_t B200ShardedIndexFlat::readTrace(float* enqueueUs, float* waitUs, size_t capacity) const {
    const size_t n = std::min(capacity, impl_->traceEnqueueUs.size());
    for (size_t i = 0; i < n; i++) {
        if (enqueueUs) enqueueUs[i] = impl_->traceEnqueueUs[i];
        if (waitUs) waitUs[i] = impl_->traceWaitUs[i];
    }
    return impl_->traceEnqueueUs.size();
}

void B200ShardedIndexFlat::searchDeviceEnqueue(faiss::idx_t n, const float* x, faiss::idx_t k, float* distances,
                                               faiss::idx_t* labels) const {
    checkSearchArgs(n, x, k);
    if (n == 0) return;
    const int64_t batch = k <= B200F_LIST_MAX_K ? kFusedBatch : kSelectBatch;
    B200_THROW_ARG_IF_NOT(B200F_ERR_UNSUPPORTED, n <= batch, "searchDeviceEnqueue: too many queries for one launch");
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, (distances == nullptr) == (labels == nullptr),
                          "searchDeviceEnqueue: distances and labels must both be given or both be null");
    DeviceGuard g(impl_->res[0]->getDevice());
    impl_->enqueueBatch(n, x, true, k, distances, labels);
}

void B200ShardedIndexFlat::synchronize() const {
    std::exception_ptr first;
    for (auto& s : impl_->shards) {
        try {
            s->synchronize();
        } catch (...) {
            if (!first) first = std::current_exception();
        }
    }
    if (first) std::rethrow_exception(first);
}

void B200ShardedIndexFlat::Impl::enqueueBatch(int64_t nq, const float* x, bool xOnDevice, int64_t k, float* outDist,
                                              faiss::idx_t* outLabels) {
    Impl& im = *this;
    const int S = im.localShards();
    const int P = im.parts();
    const int d = im.d;
    const int64_t slice = (nq + P - 1) / P;                          // query rows per part
    const size_t sliceBytes = alignUp((size_t)slice * d * 4, 16);
    const size_t distBytes = alignUp((size_t)nq * k * 4, 16);
    const size_t partBytes = alignUp(distBytes + (size_t)nq * k * 8, 16);   // [distances | labels] of one part
    // Host queries are normally uploaded in slices and all-gathered; a query block this small is
    // cheaper to upload whole on every GPU (one 5 us copy each) than to all-gather (a collective
    // launch on the critical path of a single-query search).
    const bool exchangeQueries = !xOnDevice && P > 1 && (size_t)nq * d * 4 > kSmallQueryBytes;

    // 1. queries: every GPU needs all of them.  From host memory each part's GPU takes one
    //    slice over PCIe and the slices are all-gathered over NVLink; device queries are
    //    already whole where this process's first shard lives.
    std::vector<const float*> q((size_t)S, nullptr);
    std::vector<void*> qbase((size_t)S, nullptr);
    if (xOnDevice && im.exchange == Impl::Exchange::Nccl && !im.ranks) {
        // the peer copies below read x on the first GPU: they start once its stream got here
        cudaEvent_t ev = reinterpret_cast<cudaEvent_t>(im.res[0]->acquireEvent());
        cudaError_t e = cudaEventRecord(ev, im.stream(0));
        for (int s = 1; s < S && e == cudaSuccess; s++) e = cudaStreamWaitEvent(im.stream(s), ev, 0);
        im.res[0]->releaseEvent(reinterpret_cast<EventHandle>(ev));
        cudaCheck(e, "search: order peer copies");
    }
    for (int s = 0; s < S; s++) {
        const int b = im.bufOf(s);
        if (xOnDevice && (s == 0 || im.exchange == Impl::Exchange::SameDevice)) {
            q[(size_t)s] = x;
            continue;
        }
        Impl::Buffers& bf = im.buf[(size_t)b];
        DeviceGuard g(im.res[s]->getDevice());
        uint8_t* base = static_cast<uint8_t*>(im.grow(s, bf.queries, bf.queryBytes, (size_t)P * sliceBytes));
        qbase[(size_t)s] = base;
        q[(size_t)s] = reinterpret_cast<const float*>(base);
        if (xOnDevice) {
            // several GPUs in one process, queries on the first: a plain peer copy each
            cudaCheck(cudaMemcpyPeerAsync(base, im.res[s]->getDevice(), x, im.res[0]->getDevice(), (size_t)nq * d * 4,
                                          im.stream(s)),
                      "search: peer copy of queries");
            continue;
        }
        if (im.exchange == Impl::Exchange::SameDevice && s > 0) continue;   // shard 0 copied all of it
        const bool whole = !exchangeQueries || im.exchange == Impl::Exchange::SameDevice;
        const int64_t r0 = whole ? 0 : std::min<int64_t>(nq, (int64_t)im.partOf(s) * slice);
        const int64_t r1 = whole ? nq : std::min<int64_t>(nq, r0 + slice);
        if (r1 > r0)
            cudaCheck(cudaMemcpyAsync(base + (whole ? 0 : (size_t)im.partOf(s) * sliceBytes), x + (size_t)r0 * d,
                                      (size_t)(r1 - r0) * d * 4, cudaMemcpyHostToDevice, im.stream(s)),
                      "search: host to device copy of queries");
    }
    if (exchangeQueries && im.exchange == Impl::Exchange::Nccl) {
        // slices are sliceBytes apart; the gathered rows are contiguous only if that equals the
        // payload, which alignUp(.., 16) guarantees whenever slice * d * 4 is a multiple of 16
        if (sliceBytes != (size_t)slice * d * 4) {
            // odd row size: fall back to copying everything to every GPU
            for (int s = 0; s < S; s++) {
                DeviceGuard g(im.res[s]->getDevice());
                cudaCheck(cudaMemcpyAsync(qbase[(size_t)s], x, (size_t)nq * d * 4, cudaMemcpyHostToDevice, im.stream(s)),
                          "search: host to device copy of queries");
            }
        } else {
            im.allGather(qbase.data(), sliceBytes);
        }
    }

    // 2. shard-local searches into this process's view of all parts' candidates
    std::vector<void*> cand((size_t)S, nullptr);
    for (int s = 0; s < S; s++) {
        const int b = im.bufOf(s);
        Impl::Buffers& bf = im.buf[(size_t)b];
        DeviceGuard g(im.res[s]->getDevice());
        uint8_t* base = static_cast<uint8_t*>(im.grow(s, bf.cand, bf.candBytes, (size_t)P * partBytes));
        cand[(size_t)s] = base;
        uint8_t* mine = base + (size_t)im.partOf(s) * partBytes;
        float* dLoc = reinterpret_cast<float*>(mine);
        faiss::idx_t* lLoc = reinterpret_cast<faiss::idx_t*>(mine + distBytes);
        if (P == 1 && outDist) {   // nothing to merge: straight into the output
            dLoc = outDist;
            lLoc = outLabels;
        }
        im.shards[(size_t)s]->searchDeviceEnqueue(nq, q[(size_t)s], k, dLoc, lLoc);
        if (!im.ranks && S > 1)
            abiCheck(b200f_remap_labels_block_cyclic(reinterpret_cast<int64_t*>(lLoc), nq * k, im.blockRows, S, s,
                                                     im.stream(s)),
                     "remap labels");
    }
    if (P == 1) return;

    // 3. exchange: one all-gather of [distances | labels] per shard, in place
    im.allGather(cand.data(), partBytes);

    // 4. k-way merge straight out of the gathered buffer, where a result is wanted
    if (outDist) {
        const int m = 0;
        DeviceGuard g(im.res[m]->getDevice());
        const uint8_t* base = static_cast<const uint8_t*>(cand[(size_t)m]);
        abiCheck(b200f_merge_lists_strided(reinterpret_cast<const float*>(base),
                                           reinterpret_cast<const int64_t*>(base + distBytes), (int64_t)(partBytes / 4),
                                           (int64_t)(partBytes / 8), P, nq, (int)k,
                                           im.l2 ? B200F_METRIC_L2 : B200F_METRIC_INNER_PRODUCT, outDist,
                                           reinterpret_cast<int64_t*>(outLabels), im.stream(m)),
                 "merge lists");
    }
}

}  // namespace faiss_b200
