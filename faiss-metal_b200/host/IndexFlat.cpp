// B200IndexFlat: storage growth, conversion on add, search orchestration, async
// tokens, reconstruct and the cpu<->gpu converters.
// Counterpart of src/MetalIndexFlat.mm (add :185-311, search :313-401,
// searchAsync :403-490, token :17-78, reset :492-506, reconstruct :508-527,
// converters :552-587).  All device work goes through the C-ABI in
// include/b200_flat.h; nothing here computes distances on the host.
#include <cuda_runtime.h>
#include <faiss/impl/FaissAssert.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <future>
#include <limits>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "../../include/b200_flat.h"
#include "../include/faiss-b200/B200Exception.h"
#include "../include/faiss-b200/B200IndexFlat.h"
#include "../include/faiss-b200/B200Resources.h"
#include "GrowableArray.h"

namespace faiss_b200 {

namespace {

constexpr size_t kStageBytes = 32ull << 20;   // fp32 staging chunk of add / reconstruct_n (two in flight)
constexpr int64_t kGraphMaxQueries = 8;        // searches this small are replayed from a CUDA graph
constexpr size_t kMaxGraphs = 8;               // graphs kept per index (least recently used goes)
constexpr int64_t kFusedBatch = 16384;        // queries per launch, k <= 1024 (fused kernel, lists)
constexpr int64_t kSelectBatch = 1024;        // queries per launch beyond: few rows, wide column chunks

void cudaCheck(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        std::string msg = std::string("faiss-b200: ") + what + ": " + cudaGetErrorString(e);
        (void)cudaGetLastError();
        throw B200RuntimeError(e == cudaErrorMemoryAllocation ? B200F_ERR_OOM : B200F_ERR_CUDA, msg);
    }
}

// A status code of the op-level C-ABI becomes the exception class the reference would have
// thrown (argument errors: faiss::FaissException; everything else: std::runtime_error), with
// the code kept inside.
void abiCheck(int rc, const char* what) {
    if (rc == B200F_OK) return;
    std::string msg = std::string("faiss-b200: ") + what + ": " + b200f_status_string(rc);
    if (rc == B200F_ERR_BAD_ARG || rc == B200F_ERR_UNSUPPORTED || rc == B200F_ERR_RANGE || rc == B200F_ERR_STATE)
        throw B200ArgumentError(rc, msg);
    throw B200RuntimeError(rc, msg);
}

// Device status word of a search (B200FSearchArgs::status[0]): bit 1 = a bounded wait ran out,
// any other bit = a self-check of a kernel failed.
[[noreturn]] void throwDeviceStatus(int word, const char* what) {
    const int code = (word & 1) ? B200F_ERR_DEVICE_WAIT : B200F_ERR_DEVICE_CHECK;
    throw B200RuntimeError(code, std::string("faiss-b200: ") + what + " reported device status " +
                                         std::to_string(word) + " (" + b200f_status_string(code) + ")");
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

enum class PtrKind { Pageable, Pinned, Device };

PtrKind pointerKind(const void* p) {
    if (!p) return PtrKind::Pageable;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return PtrKind::Pageable;
    }
    if (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) return PtrKind::Device;
    return attr.type == cudaMemoryTypeHost ? PtrKind::Pinned : PtrKind::Pageable;
}

bool isDevicePointer(const void* p) { return pointerKind(p) == PtrKind::Device; }

// Host copy into / out of pinned staging.  One thread moves ~10 GB/s, well under what the
// copy engine takes from pinned memory, so large blocks are split over a few threads.
void hostCopy(void* dst, const void* src, size_t bytes) {
    constexpr size_t kPerThread = 4ull << 20;
    const unsigned hw = std::thread::hardware_concurrency();
    size_t nthreads = std::min<size_t>({bytes / kPerThread, (size_t)8, (size_t)(hw > 1 ? hw - 1 : 1)});
    if (nthreads <= 1) {
        std::memcpy(dst, src, bytes);
        return;
    }
    const size_t per = ((bytes / nthreads) + 63) & ~(size_t)63;
    std::vector<std::future<void>> parts;
    for (size_t t = 1; t < nthreads; t++) {
        const size_t off = t * per;
        if (off >= bytes) break;
        const size_t len = std::min(per, bytes - off);
        parts.push_back(std::async(std::launch::async, [=] {
            std::memcpy(static_cast<uint8_t*>(dst) + off, static_cast<const uint8_t*>(src) + off, len);
        }));
    }
    std::memcpy(dst, src, std::min(per, bytes));
    for (auto& f : parts) f.get();
}

// B200F_NO_VMM=1 in the environment makes allocate-copy-free growth the default (read once).
bool growthByCopyDefault() {
    static const bool v = [] {
        const char* off = std::getenv("B200F_NO_VMM");
        return off && off[0] == '1';
    }();
    return v;
}

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }
int64_t roundUp(int64_t a, int64_t b) { return (a + b - 1) / b * b; }

size_t elemBytes(StorageType s) { return s == StorageType::Float32 ? 4 : 2; }

}  // namespace

// ---------------------------------------------------------------------------------------
struct B200IndexFlat::Impl {
    std::shared_ptr<B200Resources> res;
    StorageType storage = StorageType::Float32;
    int d = 0;
    bool l2 = true;
    int64_t pitch = 0;       // elements per stored row
    int64_t planePitch = 0;  // fp32 storage: elements per bf16 split-plane row
    void* rows = nullptr;
    uint16_t* planes = nullptr;
    float* norms = nullptr;
    int64_t capacity = 0;
    int32_t* status = nullptr;    // device int32[4]
    float* oneRow = nullptr;      // device fp32[d] for reconstruct
    int32_t* hostStatus = nullptr;  // pinned int32[4]
    int forcePath = B200F_PATH_AUTO;
    int64_t labelBase = 0;
    mutable std::vector<float> mirror;
    mutable bool mirrorValid = false;
    mutable int lastStatus = 0;

    cudaStream_t stream() const { return reinterpret_cast<cudaStream_t>(res->getDefaultStream()); }
    int storageCode() const { return (int)storage; }

    // Storage that grows in place (address range reserved once, memory mapped in as rows are
    // added; see GrowableArray.h).  When the driver calls are not available, or
    // B200F_NO_VMM=1 is set in the environment (testing), plain allocations with the
    // reference's allocate-copy-free growth are used instead.
    GrowableDeviceArray vRows, vPlanes, vNorms;
    bool inPlace = false;
    int64_t maxRows = 0;          // rows the reserved ranges can hold
    int64_t planeStrideFixed = 0;  // elements between split planes when inPlace

    int64_t planeStride() const { return inPlace ? planeStrideFixed : capacity * planePitch; }
    int growthMode = -1;           // -1: process default, 0: in place, 1: allocate-copy-free

    // FP32 storage: format of the split planes (B200F_PLANES_*).  An index starts with two fp16
    // planes (half the tensor work of three bf16 planes) unless told otherwise, takes its
    // power-of-two scale from the first rows it sees, and re-splits itself into three bf16 planes
    // the moment a row does not fit fp16's range (the conversion kernel raises a flag).
    int planeFormat = B200F_PLANES_FP16X2;
    int planeFormatWanted = B200F_PLANES_FP16X2;
    int planeScaleLog2 = 0;
    bool planeScaleKnown = false;
    int planesBacked() const { return planeFormat == B200F_PLANES_FP16X2 ? 2 : 3; }
    int32_t* rangeFlag() const { return status + 8; }   // device word beside the status words

    // Small searches (n <= kGraphMaxQueries, host buffers) replayed from CUDA graphs.  A graph
    // holds the whole call: host-to-device copy of the queries out of its pinned slot, the
    // search, and the copies of distances, labels and status word back into the slot.  It is
    // tied to the addresses and sizes it was captured with: `generation` changes whenever the
    // stored rows, the label base or the forced path change, and stale graphs are dropped.
    struct SearchGraph {
        int64_t n = 0, k = 0;
        int selectMode = 0;
        void* region = nullptr;      // device: queries, outputs, scratch (owned by the graph)
        uint8_t* host = nullptr;     // pinned: queries | distances | labels | status
        size_t hostDistOff = 0, hostLabOff = 0, hostStatusOff = 0;
        cudaGraph_t graph = nullptr;
        cudaGraphExec_t exec = nullptr;
        uint64_t lastUse = 0;
    };
    mutable std::vector<SearchGraph> graphs;
    mutable std::vector<std::pair<int64_t, int64_t>> seenShapes;  // (n, k) searched once without a graph
    mutable uint64_t useCounter = 0;
    bool useGraphs = true;

    void destroyGraph(SearchGraph& g) const {
        if (g.exec) (void)cudaGraphExecDestroy(g.exec);
        if (g.graph) (void)cudaGraphDestroy(g.graph);
        if (g.region) res->releaseDeviceTemp(g.region);
        if (g.host) res->releasePinnedTemp(g.host);
        g = SearchGraph{};
    }
    // The stored rows / label base / path changed: nothing captured so far is valid.
    mutable uint64_t generation = 1;   // bumped with every change that makes captured work stale
    void invalidateGraphs() const {
        generation++;
        if (graphs.empty() && seenShapes.empty()) return;
        (void)cudaStreamSynchronize(stream());
        for (auto& g : graphs) destroyGraph(g);
        graphs.clear();
        seenShapes.clear();
    }

    void freeStorage() {
        if (inPlace) {
            vRows.release();
            vPlanes.release();
            vNorms.release();
            inPlace = false;
        } else {
            if (rows) res->deallocBuffer(rows);
            if (planes) res->deallocBuffer(planes);
            if (norms) res->deallocBuffer(norms);
        }
        rows = nullptr;
        planes = nullptr;
        norms = nullptr;
        capacity = 0;
    }

    // First allocation of an empty index: reserve the address ranges.  Returns false (nothing
    // reserved) when in-place growth cannot be used.
    bool reserveInPlace() {
        if (growthMode == 1 || (growthMode < 0 && growthByCopyDefault())) return false;
        const int dev = res->getDevice();
        if (!GrowableDeviceArray::supported(dev)) return false;
        const size_t es = elemBytes(storage);
        const size_t rowBytes = (size_t)pitch * es;
        // no shard can hold more rows than fit the device memory (or the int32 row numbers)
        size_t freeB = 0, totalB = 0;
        if (cudaMemGetInfo(&freeB, &totalB) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
        int64_t cap = (int64_t)(totalB / rowBytes);
        cap = std::min<int64_t>(cap, B200DeviceCapabilities::kMaxVectorsPerShard);
        cap = std::max<int64_t>(cap, 1024);
        // planes start on 2 MiB multiples of a common stride, so that each one is backed on its own
        const size_t planeBytes = roundUp((int64_t)((size_t)cap * planePitch * 2), 2ll << 20);
        bool ok = vRows.reserve(dev, (size_t)cap * rowBytes);
        if (ok && storage == StorageType::Float32) ok = vPlanes.reserve(dev, 3 * planeBytes);
        if (ok && l2) ok = vNorms.reserve(dev, (size_t)cap * 4);
        if (!ok) {
            vRows.release();
            vPlanes.release();
            vNorms.release();
            return false;
        }
        maxRows = cap;
        planeStrideFixed = (int64_t)(planeBytes / 2);
        rows = vRows.data();
        planes = storage == StorageType::Float32 ? static_cast<uint16_t*>(vPlanes.data()) : nullptr;
        norms = l2 ? static_cast<float*>(vNorms.data()) : nullptr;
        inPlace = true;
        return true;
    }

    // Grow to hold at least `want` rows; keeps the first `keep` rows.
    void grow(int64_t want, int64_t keep) {
        if (want <= capacity) return;
        if (capacity == 0 && !rows && !inPlace) (void)reserveInPlace();
        if (inPlace) {
            if (want > maxRows)
                throw B200RuntimeError(B200F_ERR_OOM, "faiss-b200: the index cannot hold " + std::to_string(want) +
                                                              " rows on this device");
            const size_t es = elemBytes(storage);
            vRows.back(0, (size_t)want * pitch * es);
            if (planes)
                for (int p = 0; p < planesBacked(); p++)
                    vPlanes.back((size_t)p * planeStrideFixed * 2, (size_t)want * planePitch * 2);
            if (norms) vNorms.back(0, (size_t)want * 4);
            capacity = want;
            return;
        }
        const size_t es = elemBytes(storage);
        void* newRows = res->allocBuffer((size_t)want * pitch * es);
        uint16_t* newPlanes = nullptr;
        float* newNorms = nullptr;
        try {
            if (storage == StorageType::Float32)
                newPlanes = static_cast<uint16_t*>(res->allocBuffer((size_t)3 * want * planePitch * 2));
            if (l2) newNorms = static_cast<float*>(res->allocBuffer((size_t)want * 4));
        } catch (...) {
            res->deallocBuffer(newRows);
            if (newPlanes) res->deallocBuffer(newPlanes);
            throw;
        }
        cudaStream_t st = stream();
        if (keep > 0) {
            cudaCheck(cudaMemcpyAsync(newRows, rows, (size_t)keep * pitch * es, cudaMemcpyDeviceToDevice, st),
                      "copy rows");
            if (newPlanes)
                for (int p = 0; p < 3; p++)
                    cudaCheck(cudaMemcpyAsync(newPlanes + (size_t)p * want * planePitch,
                                              planes + (size_t)p * capacity * planePitch,
                                              (size_t)keep * planePitch * 2, cudaMemcpyDeviceToDevice, st),
                              "copy planes");
            if (newNorms)
                cudaCheck(cudaMemcpyAsync(newNorms, norms, (size_t)keep * 4, cudaMemcpyDeviceToDevice, st),
                          "copy norms");
            cudaCheck(cudaStreamSynchronize(st), "grow sync");
        }
        freeStorage();
        rows = newRows;
        planes = newPlanes;
        norms = newNorms;
        capacity = want;
    }

    void fillArgs(B200FSearchArgs& a, int64_t ntotal) const {
        std::memset(&a, 0, sizeof(a));
        a.d = d;
        a.storage = storageCode();
        a.rows = rows;
        a.row_pitch = pitch;
        a.planes = planes;
        a.plane_pitch = planePitch;
        a.plane_stride = planeStride();
        a.plane_format = planeFormat;
        a.plane_scale_log2 = planeScaleLog2;
        a.norms = norms;
        a.nb = ntotal;
        a.metric = l2 ? B200F_METRIC_L2 : B200F_METRIC_INNER_PRODUCT;
        a.label_base = labelBase;
        a.status = status;
        a.stream = stream();
        a.path = forcePath;
        a.norm_cols = l2 ? 1 : 0;
    }
};

// layout of one search call inside a device region
namespace {
struct CallLayout {
    size_t offQueries, offDist, offLabels, offScratch, scratchBytes, total;
};
CallLayout makeLayout(int64_t nOut, int64_t nBatch, int d, int64_t k, bool stageQueries, int64_t nQueriesStaged,
                      bool stageOutputs, size_t scratchBytes) {
    CallLayout L{};
    size_t off = 0;
    L.offQueries = off;
    if (stageQueries) off += align256((size_t)nQueriesStaged * d * 4);
    L.offDist = off;
    if (stageOutputs) off += align256((size_t)nOut * k * 4);
    L.offLabels = off;
    if (stageOutputs) off += align256((size_t)nOut * k * 8);
    L.offScratch = off;
    L.scratchBytes = scratchBytes;
    off += align256(scratchBytes);
    L.total = off;
    (void)nBatch;
    return L;
}
}  // namespace

// ---------------------------------------------------------------------------------------
B200IndexFlat::B200IndexFlat(std::shared_ptr<B200Resources> resources, int d_,
                             faiss::MetricType metric, bool useFloat16Storage)
        : B200IndexFlat(std::move(resources), d_, metric,
                        useFloat16Storage ? StorageType::Float16 : StorageType::Float32) {}

B200IndexFlat::B200IndexFlat(std::shared_ptr<B200Resources> resources, int d_,
                             faiss::MetricType metric, StorageType storage)
        : faiss::Index(d_, metric), impl_(new Impl) {
    FAISS_THROW_IF_NOT_MSG(resources != nullptr, "resources must not be null");
    FAISS_THROW_IF_NOT_MSG(d_ > 0, "d must be > 0");
    FAISS_THROW_IF_NOT_MSG(metric == faiss::METRIC_L2 || metric == faiss::METRIC_INNER_PRODUCT,
                           "only METRIC_L2 and METRIC_INNER_PRODUCT are supported");
    FAISS_THROW_IF_NOT_MSG((int)storage >= 0 && (int)storage <= 2, "invalid storage type");
    impl_->res = std::move(resources);
    impl_->storage = storage;
    impl_->d = d_;
    impl_->l2 = metric == faiss::METRIC_L2;
    // L2: the 16-bit row (or split plane 0) carries 8 norm columns after round_up(d, 8)
    const int64_t normCols = impl_->l2 ? 8 : 0;
    impl_->pitch = storage == StorageType::Float32 ? roundUp(d_, 4) : roundUp(d_, 8) + normCols;
    impl_->planePitch = roundUp(d_, 8) + normCols;
    DeviceGuard g(impl_->res->getDevice());
    impl_->status = static_cast<int32_t*>(impl_->res->allocBuffer(256));
    impl_->oneRow = static_cast<float*>(impl_->res->allocBuffer((size_t)d_ * 4));
    impl_->hostStatus = static_cast<int32_t*>(alloc_pinned(64));
    if (!impl_->hostStatus) throw B200RuntimeError(B200F_ERR_OOM, "faiss-b200: pinned allocation failed");
    cudaCheck(cudaMemsetAsync(impl_->status, 0, 256, impl_->stream()), "memset status");
    is_trained = true;
    ntotal = 0;
}

B200IndexFlat::~B200IndexFlat() {
    if (!impl_) return;
    try {
        DeviceGuard g(impl_->res->getDevice());
        (void)cudaStreamSynchronize(impl_->stream());
        impl_->invalidateGraphs();
        impl_->freeStorage();
        impl_->res->deallocBuffer(impl_->status);
        impl_->res->deallocBuffer(impl_->oneRow);
        free_pinned(impl_->hostStatus);
    } catch (...) {
    }
}

void B200IndexFlat::reserve(faiss::idx_t n) {
    DeviceGuard g(impl_->res->getDevice());
    if (n > impl_->capacity) {
        impl_->invalidateGraphs();
        impl_->grow(n, ntotal);
    }
}

void B200IndexFlat::setGrowthMode(int mode) {
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, mode == 0 || mode == 1, "growth mode must be 0 (in place) or 1 (copy)");
    B200_THROW_ARG_IF_NOT(B200F_ERR_STATE, impl_->capacity == 0 && !impl_->rows,
                          "the growth mode can only be chosen on an index that holds no storage yet");
    impl_->growthMode = mode;
}

void B200IndexFlat::setFp32PlaneFormat(int format) {
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, format == B200F_PLANES_BF16X3 || format == B200F_PLANES_FP16X2,
                          "plane format must be B200F_PLANES_BF16X3 or B200F_PLANES_FP16X2");
    B200_THROW_ARG_IF_NOT(B200F_ERR_STATE, ntotal == 0 && impl_->capacity == 0,
                          "the plane format can only be chosen on an index that holds no storage yet");
    impl_->planeFormatWanted = format;
    impl_->planeFormat = format;
}
int B200IndexFlat::getFp32PlaneFormat() const { return impl_->planeFormat; }

void B200IndexFlat::setUseGraphs(bool on) {
    if (!on) {
        DeviceGuard g(impl_->res->getDevice());
        impl_->invalidateGraphs();
    }
    impl_->useGraphs = on;
}

void B200IndexFlat::add(faiss::idx_t n, const float* x) {
    if (n == 0) return;  // src/MetalIndexFlat.mm:186
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, n > 0 && x != nullptr, "add: invalid arguments");
    const int64_t newTotal = ntotal + n;
    B200_THROW_ARG_IF_NOT(B200F_ERR_UNSUPPORTED, newTotal <= B200DeviceCapabilities::kMaxVectorsPerShard,
                          "B200IndexFlat holds at most 2^31-1 vectors per shard (int32 row numbers)");
    DeviceGuard g(impl_->res->getDevice());
    impl_->invalidateGraphs();
    if (newTotal > impl_->capacity) {
        // growth rule of the reference: max(newTotal, 2 * capacity, 1024)
        // (src/MetalIndexFlat.mm:196-197,272-273)
        int64_t newCap = std::max<int64_t>(newTotal, impl_->capacity * 2);
        newCap = std::max<int64_t>(newCap, 1024);
        impl_->grow(newCap, ntotal);
    }
    cudaStream_t st = impl_->stream();
    const size_t es = elemBytes(impl_->storage);
    const bool fp32 = impl_->storage == StorageType::Float32;
    if (fp32) cudaCheck(cudaMemsetAsync(impl_->rangeFlag(), 0, 4, st), "add: clear range flag");
    auto store = [&](const float* src, int64_t r0, int64_t nr) {
        const int64_t row = ntotal + r0;
        if (!fp32) {
            abiCheck(b200f_store_rows(
                             src, nr, d, impl_->storageCode(),
                             static_cast<uint8_t*>(impl_->rows) + (size_t)row * impl_->pitch * es, impl_->pitch, nullptr, 0,
                             0, impl_->norms ? impl_->norms + row : nullptr, impl_->l2 ? 1 : 0, st),
                     "add: store rows");
            return;
        }
        if (impl_->planeFormat == B200F_PLANES_FP16X2 && !impl_->planeScaleKnown) {
            // the index's scale: the largest element of the first rows it is given goes to [2^6, 2^7)
            uint32_t* bits = reinterpret_cast<uint32_t*>(impl_->rangeFlag() + 1);
            abiCheck(b200f_rows_absmax(src, nr, d, d, bits, st), "add: rows absmax");
            cudaCheck(cudaMemcpyAsync(impl_->hostStatus + 8, bits, 4, cudaMemcpyDeviceToHost, st), "add: absmax copy");
            cudaCheck(cudaStreamSynchronize(st), "add: synchronize");
            float amax;
            std::memcpy(&amax, impl_->hostStatus + 8, 4);
            int e = 0;
            if (amax > 0.f) (void)std::frexp(amax, &e);
            impl_->planeScaleLog2 = amax > 0.f ? std::max(-120, std::min(120, 7 - e)) : 0;
            impl_->planeScaleKnown = amax > 0.f;   // all-zero rows say nothing: ask the next block again
        }
        abiCheck(b200f_store_rows_fp32(src, d, nr, d, static_cast<float*>(impl_->rows) + (size_t)row * impl_->pitch,
                                       impl_->pitch, impl_->planes + (size_t)row * impl_->planePitch, impl_->planePitch,
                                       impl_->planeStride(), impl_->planeFormat, impl_->planeScaleLog2,
                                       impl_->rangeFlag(), impl_->norms ? impl_->norms + row : nullptr,
                                       impl_->l2 ? 1 : 0, st),
                 "add: store rows");
    };
    const PtrKind kind = pointerKind(x);
    if (kind == PtrKind::Device) {
        store(x, 0, n);
    } else {
        // Ingest pipeline.  The input is cut into chunks of kStageBytes; chunk i is copied host to
        // device on the upload stream into one of two device staging buffers while the
        // conversion kernel of chunk i - 1 runs on the search stream.  Pageable input goes through
        // two pinned staging buffers first (filled by host threads while the previous chunk is
        // on the bus); pinned input is copied straight from where it lies.  One host
        // synchronisation, at the end.
        const int64_t rowsPerChunk = std::max<int64_t>(1, (int64_t)(kStageBytes / ((size_t)d * 4)));
        const size_t chunkBytes = align256((size_t)std::min<int64_t>(rowsPerChunk, n) * d * 4);
        const int nbuf = n > rowsPerChunk ? 2 : 1;
        uint8_t* dev = static_cast<uint8_t*>(impl_->res->getScratch(nbuf * chunkBytes));
        uint8_t* pin = kind == PtrKind::Pageable
                               ? static_cast<uint8_t*>(impl_->res->getPinnedStaging(nbuf * chunkBytes))
                               : nullptr;
        cudaStream_t up = reinterpret_cast<cudaStream_t>(impl_->res->getAuxStream(B200Resources::kUploadStream));
        cudaEvent_t copied[2] = {nullptr, nullptr}, consumed[2] = {nullptr, nullptr};
        cudaEvent_t start = reinterpret_cast<cudaEvent_t>(impl_->res->acquireEvent());
        for (int i = 0; i < nbuf; i++) {
            copied[i] = reinterpret_cast<cudaEvent_t>(impl_->res->acquireEvent());
            consumed[i] = reinterpret_cast<cudaEvent_t>(impl_->res->acquireEvent());
        }
        auto releaseEvents = [&] {
            impl_->res->releaseEvent(start);
            for (int i = 0; i < nbuf; i++) {
                impl_->res->releaseEvent(copied[i]);
                impl_->res->releaseEvent(consumed[i]);
            }
        };
        try {
            // the staging region may still be in use by work queued earlier on the search stream
            cudaCheck(cudaEventRecord(start, st), "add: event record");
            cudaCheck(cudaStreamWaitEvent(up, start, 0), "add: stream wait");
            int64_t chunk = 0;
            for (int64_t r0 = 0; r0 < n; r0 += rowsPerChunk, chunk++) {
                const int64_t nr = std::min<int64_t>(rowsPerChunk, n - r0);
                const size_t bytes = (size_t)nr * d * 4;
                const int b = (int)(chunk % nbuf);
                const float* src = x + (size_t)r0 * d;
                if (chunk >= nbuf) {
                    // device buffer b: the conversion of chunk - 2 has to be done with it
                    cudaCheck(cudaStreamWaitEvent(up, consumed[b], 0), "add: stream wait");
                    // pinned buffer b: its copy to the device has to be complete
                    if (pin) cudaCheck(cudaEventSynchronize(copied[b]), "add: event synchronize");
                }
                if (pin) {
                    hostCopy(pin + (size_t)b * chunkBytes, src, bytes);
                    src = reinterpret_cast<const float*>(pin + (size_t)b * chunkBytes);
                }
                cudaCheck(cudaMemcpyAsync(dev + (size_t)b * chunkBytes, src, bytes, cudaMemcpyHostToDevice, up),
                          "add: host to device copy");
                cudaCheck(cudaEventRecord(copied[b], up), "add: event record");
                cudaCheck(cudaStreamWaitEvent(st, copied[b], 0), "add: stream wait");
                store(reinterpret_cast<const float*>(dev + (size_t)b * chunkBytes), r0, nr);
                cudaCheck(cudaEventRecord(consumed[b], st), "add: event record");
            }
        } catch (...) {
            (void)cudaStreamSynchronize(up);
            (void)cudaStreamSynchronize(st);
            releaseEvents();
            throw;
        }
        releaseEvents();
    }
    // the caller may free x as soon as add returns
    if (fp32 && impl_->planeFormat == B200F_PLANES_FP16X2)
        cudaCheck(cudaMemcpyAsync(impl_->hostStatus + 9, impl_->rangeFlag(), 4, cudaMemcpyDeviceToHost, st),
                  "add: range flag copy");
    cudaCheck(cudaStreamSynchronize(st), "add: synchronize");
    ntotal = newTotal;
    impl_->mirrorValid = false;
    if (fp32 && impl_->planeFormat == B200F_PLANES_FP16X2 && impl_->hostStatus[9] != 0) {
        // a row of this add does not fit fp16's range at the index's scale: three bf16 planes
        // from now on, re-split from the stored fp32 rows
        impl_->planeFormat = B200F_PLANES_BF16X3;
        if (impl_->inPlace)
            impl_->vPlanes.back((size_t)2 * impl_->planeStrideFixed * 2, (size_t)impl_->capacity * impl_->planePitch * 2);
        abiCheck(b200f_store_rows_fp32(static_cast<const float*>(impl_->rows), impl_->pitch, ntotal, d,
                                       static_cast<float*>(impl_->rows), impl_->pitch, impl_->planes, impl_->planePitch,
                                       impl_->planeStride(), B200F_PLANES_BF16X3, 0, nullptr, impl_->norms,
                                       impl_->l2 ? 1 : 0, st),
                 "add: re-split rows");
        cudaCheck(cudaStreamSynchronize(st), "add: synchronize");
    }
}

void B200IndexFlat::reset() {
    DeviceGuard g(impl_->res->getDevice());
    cudaCheck(cudaStreamSynchronize(impl_->stream()), "reset: synchronize");
    impl_->invalidateGraphs();
    impl_->freeStorage();
    impl_->planeFormat = impl_->planeFormatWanted;
    impl_->planeScaleKnown = false;
    impl_->planeScaleLog2 = 0;
    impl_->mirror.clear();
    impl_->mirror.shrink_to_fit();
    impl_->mirrorValid = false;
    ntotal = 0;
}

void B200IndexFlat::reconstruct_n(faiss::idx_t first, faiss::idx_t n, float* out) const {
    if (!(first >= 0 && n >= 0 && first + n <= ntotal))
        throw B200ArgumentError(B200F_ERR_RANGE, "faiss-b200: reconstruct_n: range [" + std::to_string(first) + ", " +
                                                         std::to_string(first + n) + ") outside [0, " +
                                                         std::to_string(ntotal) + ")");
    if (n == 0) return;
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, out != nullptr, "reconstruct_n: null output");
    DeviceGuard g(impl_->res->getDevice());
    cudaStream_t st = impl_->stream();
    const size_t es = elemBytes(impl_->storage);
    auto load = [&](int64_t r0, int64_t nr, float* dst) {
        abiCheck(b200f_load_rows(static_cast<const uint8_t*>(impl_->rows) + (size_t)(first + r0) * impl_->pitch * es,
                                 impl_->storageCode(), nr, d, impl_->pitch, dst, st),
                 "reconstruct_n: load rows");
    };
    const PtrKind kind = pointerKind(out);
    if (kind == PtrKind::Device) {
        load(0, n, out);
        cudaCheck(cudaStreamSynchronize(st), "reconstruct_n: synchronize");
        return;
    }
    // The ingest pipeline backwards: chunk i is dequantised on the search stream into one of two
    // device buffers while chunk i - 1 crosses the bus on the download stream (into pinned
    // staging for pageable output, else straight into `out`) and the host threads copy chunk
    // i - 2 out of the staging.
    const int64_t rowsPerChunk = std::max<int64_t>(1, (int64_t)(kStageBytes / ((size_t)d * 4)));
    const size_t chunkBytes = align256((size_t)std::min<int64_t>(rowsPerChunk, n) * d * 4);
    const int nbuf = n > rowsPerChunk ? 2 : 1;
    uint8_t* dev = static_cast<uint8_t*>(impl_->res->getScratch(nbuf * chunkBytes));
    uint8_t* pin = kind == PtrKind::Pageable ? static_cast<uint8_t*>(impl_->res->getPinnedStaging(nbuf * chunkBytes))
                                             : nullptr;
    cudaStream_t down = reinterpret_cast<cudaStream_t>(impl_->res->getAuxStream(B200Resources::kDownloadStream));
    cudaEvent_t loaded[2] = {nullptr, nullptr}, landed[2] = {nullptr, nullptr};
    for (int i = 0; i < nbuf; i++) {
        loaded[i] = reinterpret_cast<cudaEvent_t>(impl_->res->acquireEvent());
        landed[i] = reinterpret_cast<cudaEvent_t>(impl_->res->acquireEvent());
    }
    auto releaseEvents = [&] {
        for (int i = 0; i < nbuf; i++) {
            impl_->res->releaseEvent(loaded[i]);
            impl_->res->releaseEvent(landed[i]);
        }
    };
    // host side of chunk c (pageable output only): wait for its copy, move it out of the staging
    auto finish = [&](int64_t c) {
        if (!pin) return;
        const int64_t r0 = c * rowsPerChunk;
        const int64_t nr = std::min<int64_t>(rowsPerChunk, n - r0);
        cudaCheck(cudaEventSynchronize(landed[c % nbuf]), "reconstruct_n: event synchronize");
        hostCopy(out + (size_t)r0 * d, pin + (size_t)(c % nbuf) * chunkBytes, (size_t)nr * d * 4);
    };
    try {
        int64_t chunk = 0;
        for (int64_t r0 = 0; r0 < n; r0 += rowsPerChunk, chunk++) {
            const int64_t nr = std::min<int64_t>(rowsPerChunk, n - r0);
            const int b = (int)(chunk % nbuf);
            // device buffer b is free once the copy of chunk - 2 has left it
            if (chunk >= nbuf) cudaCheck(cudaStreamWaitEvent(st, landed[b], 0), "reconstruct_n: stream wait");
            load(r0, nr, reinterpret_cast<float*>(dev + (size_t)b * chunkBytes));
            cudaCheck(cudaEventRecord(loaded[b], st), "reconstruct_n: event record");
            cudaCheck(cudaStreamWaitEvent(down, loaded[b], 0), "reconstruct_n: stream wait");
            // pinned buffer b was emptied by finish(chunk - 2) in the previous round
            void* dst = pin ? static_cast<void*>(pin + (size_t)b * chunkBytes) : static_cast<void*>(out + (size_t)r0 * d);
            cudaCheck(cudaMemcpyAsync(dst, dev + (size_t)b * chunkBytes, (size_t)nr * d * 4, cudaMemcpyDeviceToHost, down),
                      "reconstruct_n: device to host copy");
            cudaCheck(cudaEventRecord(landed[b], down), "reconstruct_n: event record");
            if (chunk >= 1) finish(chunk - 1);
        }
        finish(chunk - 1);
        cudaCheck(cudaStreamSynchronize(down), "reconstruct_n: synchronize");
        cudaCheck(cudaStreamSynchronize(st), "reconstruct_n: synchronize");
    } catch (...) {
        (void)cudaStreamSynchronize(down);
        (void)cudaStreamSynchronize(st);
        releaseEvents();
        throw;
    }
    releaseEvents();
}

void B200IndexFlat::reconstruct(faiss::idx_t key, float* recons) const {
    // range check of the reference: src/MetalIndexFlat.mm:509-511
    B200_THROW_ARG_IF_NOT(B200F_ERR_RANGE, key >= 0 && key < ntotal,
                          "reconstruct: key " + std::to_string(key) + " out of range [0, " + std::to_string(ntotal) + ")");
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, recons != nullptr, "reconstruct: null output");
    DeviceGuard g(impl_->res->getDevice());
    cudaStream_t st = impl_->stream();
    const size_t es = elemBytes(impl_->storage);
    abiCheck(b200f_load_rows(static_cast<const uint8_t*>(impl_->rows) + (size_t)key * impl_->pitch * es,
                             impl_->storageCode(), 1, d, impl_->pitch, impl_->oneRow, st),
             "reconstruct: load row");
    cudaCheck(cudaMemcpyAsync(recons, impl_->oneRow, (size_t)d * 4,
                              isDevicePointer(recons) ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, st),
              "reconstruct: copy");
    cudaCheck(cudaStreamSynchronize(st), "reconstruct: synchronize");
}

const float* B200IndexFlat::getVectorsData() const {
    if (impl_->storage != StorageType::Float32) return nullptr;  // include/faiss-metal/MetalIndexFlat.h:92-94
    if (ntotal == 0) return nullptr;
    if (!impl_->mirrorValid) {
        impl_->mirror.resize((size_t)ntotal * d);
        reconstruct_n(0, ntotal, impl_->mirror.data());
        impl_->mirrorValid = true;
    }
    return impl_->mirror.data();
}

bool B200IndexFlat::isFloat16Storage() const { return impl_->storage == StorageType::Float16; }
bool B200IndexFlat::isBFloat16Storage() const { return impl_->storage == StorageType::BFloat16; }
StorageType B200IndexFlat::getStorageType() const { return impl_->storage; }
void B200IndexFlat::setForcePath(int path) {
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, path >= B200F_PATH_AUTO && path <= B200F_PATH_TENSOR, "invalid path");
    if (path != impl_->forcePath) {
        DeviceGuard g(impl_->res->getDevice());
        impl_->invalidateGraphs();
    }
    impl_->forcePath = path;
}
void B200IndexFlat::setLabelBase(faiss::idx_t base) {
    if (base != impl_->labelBase) {
        DeviceGuard g(impl_->res->getDevice());
        impl_->invalidateGraphs();
    }
    impl_->labelBase = base;
}
const void* B200IndexFlat::getDeviceRows() const { return impl_->rows; }
std::shared_ptr<B200Resources> B200IndexFlat::getResources() const { return impl_->res; }
int B200IndexFlat::lastDeviceStatus() const { return impl_->lastStatus; }
void B200IndexFlat::debugWaitExpiry(int64_t limitCycles) {
    DeviceGuard g(impl_->res->getDevice());
    abiCheck(b200f_debug_wait_expiry(impl_->status, limitCycles, impl_->stream()), "debugWaitExpiry");
}

// ---------------------------------------------------------------------------------------
// search
// ---------------------------------------------------------------------------------------
namespace {

void checkSearchArgs(faiss::idx_t n, const float* x, faiss::idx_t k, const float* distances,
                     const faiss::idx_t* labels, faiss::idx_t ntotal) {
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, k > 0, "k must be > 0");  // src/MetalIndexFlat.mm:321
    B200_THROW_ARG_IF_NOT(B200F_ERR_UNSUPPORTED, k <= B200F_MAX_K,
                          "k = " + std::to_string(k) + " exceeds the maximum of " +
                                  std::to_string(B200F_MAX_K));  // src/MetalSelect.mm:65-70
    B200_THROW_ARG_IF_NOT(B200F_ERR_UNSUPPORTED, ntotal <= B200DeviceCapabilities::kMaxVectorsPerShard,
                          "B200IndexFlat supports at most 2^31-1 vectors per shard (int32 row numbers)");
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, n >= 0, "n must be >= 0");
    if (n > 0) B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, x && distances && labels, "search: null pointer");
}

}  // namespace

void B200IndexFlat::search(faiss::idx_t n, const float* x, faiss::idx_t k, float* distances,
                           faiss::idx_t* labels, const faiss::SearchParameters* /*params*/) const {
    checkSearchArgs(n, x, k, distances, labels, ntotal);
    if (n == 0) return;
    DeviceGuard g(impl_->res->getDevice());
    cudaStream_t st = impl_->stream();
    const bool qOnDevice = isDevicePointer(x);
    const bool dOnDevice = isDevicePointer(distances);
    const bool lOnDevice = isDevicePointer(labels);
    if (n <= kGraphMaxQueries && impl_->useGraphs && !qOnDevice && !dOnDevice && !lOnDevice &&
        searchFromGraph(n, x, k, distances, labels))
        return;
    const int64_t batch = std::min<int64_t>(n, k <= B200F_LIST_MAX_K ? kFusedBatch : kSelectBatch);
    const size_t scratchBytes =
            b200f_search_scratch_bytes(batch, ntotal, d, (int)k, impl_->storageCode(), impl_->forcePath);
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, scratchBytes > 0, "search: cannot plan this shape");
    CallLayout L = makeLayout(batch, batch, d, k, !qOnDevice, batch, true, scratchBytes);
    uint8_t* region = static_cast<uint8_t*>(impl_->res->getScratch(L.total));
    impl_->lastStatus = 0;

    for (int64_t q0 = 0; q0 < n; q0 += batch) {
        const int64_t nq = std::min<int64_t>(batch, n - q0);
        const float* dq = x + (size_t)q0 * d;
        if (!qOnDevice) {
            cudaCheck(cudaMemcpyAsync(region + L.offQueries, dq, (size_t)nq * d * 4,
                                      cudaMemcpyHostToDevice, st),
                      "search: host to device copy of queries");
            dq = reinterpret_cast<const float*>(region + L.offQueries);
        }
        float* dDist = dOnDevice ? distances + (size_t)q0 * k : reinterpret_cast<float*>(region + L.offDist);
        int64_t* dLab = lOnDevice ? reinterpret_cast<int64_t*>(labels) + (size_t)q0 * k
                                  : reinterpret_cast<int64_t*>(region + L.offLabels);
        B200FSearchArgs a;
        impl_->fillArgs(a, ntotal);
        a.queries = dq;
        a.nq = nq;
        a.k = (int)k;
        a.out_dist = dDist;
        a.out_labels = dLab;
        a.scratch = region + L.offScratch;
        a.scratch_bytes = L.scratchBytes;
        abiCheck(b200f_search(&a), "search");
        if (!dOnDevice)
            cudaCheck(cudaMemcpyAsync(distances + (size_t)q0 * k, dDist, (size_t)nq * k * 4,
                                      cudaMemcpyDeviceToHost, st),
                      "search: device to host copy of distances");
        if (!lOnDevice)
            cudaCheck(cudaMemcpyAsync(labels + (size_t)q0 * k, dLab, (size_t)nq * k * 8,
                                      cudaMemcpyDeviceToHost, st),
                      "search: device to host copy of labels");
        cudaCheck(cudaMemcpyAsync(impl_->hostStatus, impl_->status, 16, cudaMemcpyDeviceToHost, st),
                  "search: status copy");
        cudaCheck(cudaStreamSynchronize(st), "search: synchronize");
        if (impl_->hostStatus[0] != 0) {
            impl_->lastStatus = impl_->hostStatus[0];
            throwDeviceStatus(impl_->hostStatus[0], "search");
        }
    }
}

// Small search with host buffers through a captured graph.  The first call with a shape runs
// the ordinary path (which also performs every lazy one-time set-up of the library, none of
// which may happen inside a capture); the second call captures; later calls replay: one memcpy
// into the pinned slot, one graph launch, one stream synchronisation, one memcpy out.
// Returns false when the ordinary path should serve the call.
bool B200IndexFlat::searchFromGraph(faiss::idx_t n, const float* x, faiss::idx_t k, float* distances,
                                    faiss::idx_t* labels) const {
    Impl& im = *impl_;
    cudaStream_t st = im.stream();
    const int selectMode = b200f_get_selection_mode();
    Impl::SearchGraph* g = nullptr;
    for (auto& e : im.graphs)
        if (e.n == n && e.k == k && e.selectMode == selectMode) g = &e;
    if (!g) {
        const std::pair<int64_t, int64_t> shape(n, k);
        if (std::find(im.seenShapes.begin(), im.seenShapes.end(), shape) == im.seenShapes.end()) {
            if (im.seenShapes.size() >= 64) im.seenShapes.clear();
            im.seenShapes.push_back(shape);
            return false;
        }
        const size_t scratchBytes = b200f_search_scratch_bytes(n, ntotal, d, (int)k, im.storageCode(), im.forcePath);
        if (scratchBytes == 0) return false;
        if (im.graphs.size() >= kMaxGraphs) {
            size_t oldest = 0;
            for (size_t i = 1; i < im.graphs.size(); i++)
                if (im.graphs[i].lastUse < im.graphs[oldest].lastUse) oldest = i;
            cudaCheck(cudaStreamSynchronize(st), "search: synchronize");
            im.destroyGraph(im.graphs[oldest]);
            im.graphs.erase(im.graphs.begin() + (long)oldest);
        }
        Impl::SearchGraph e;
        e.n = n;
        e.k = k;
        e.selectMode = selectMode;
        CallLayout L = makeLayout(n, n, d, k, true, n, true, scratchBytes);
        size_t hoff = align256((size_t)n * d * 4);
        e.hostDistOff = hoff;
        hoff += align256((size_t)n * k * 4);
        e.hostLabOff = hoff;
        hoff += align256((size_t)n * k * 8);
        e.hostStatusOff = hoff;
        hoff += 256;
        try {
            e.region = im.res->acquireDeviceTemp(L.total);
            e.host = static_cast<uint8_t*>(im.res->acquirePinnedTemp(hoff));
            if (!e.host) throw B200RuntimeError(B200F_ERR_OOM, "faiss-b200: pinned allocation failed");
            uint8_t* region = static_cast<uint8_t*>(e.region);
            B200FSearchArgs a;
            im.fillArgs(a, ntotal);
            a.queries = reinterpret_cast<const float*>(region + L.offQueries);
            a.nq = n;
            a.k = (int)k;
            a.out_dist = reinterpret_cast<float*>(region + L.offDist);
            a.out_labels = reinterpret_cast<int64_t*>(region + L.offLabels);
            a.scratch = region + L.offScratch;
            a.scratch_bytes = L.scratchBytes;
            cudaCheck(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal), "search: begin capture");
            cudaError_t ce = cudaMemcpyAsync(region + L.offQueries, e.host, (size_t)n * d * 4, cudaMemcpyHostToDevice, st);
            int rc = ce == cudaSuccess ? b200f_search(&a) : B200F_ERR_CUDA;
            if (rc == B200F_OK) {
                ce = cudaMemcpyAsync(e.host + e.hostDistOff, a.out_dist, (size_t)n * k * 4, cudaMemcpyDeviceToHost, st);
                if (ce == cudaSuccess)
                    ce = cudaMemcpyAsync(e.host + e.hostLabOff, a.out_labels, (size_t)n * k * 8, cudaMemcpyDeviceToHost, st);
                if (ce == cudaSuccess)
                    ce = cudaMemcpyAsync(e.host + e.hostStatusOff, im.status, 16, cudaMemcpyDeviceToHost, st);
                if (ce != cudaSuccess) rc = B200F_ERR_CUDA;
            }
            cudaError_t ee = cudaStreamEndCapture(st, &e.graph);   // always ends the capture
            if (rc != B200F_OK || ee != cudaSuccess || !e.graph ||
                cudaGraphInstantiate(&e.exec, e.graph, 0) != cudaSuccess) {
                (void)cudaGetLastError();
                im.destroyGraph(e);
                im.useGraphs = false;   // this build / driver cannot capture the search: stop trying
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
    std::memcpy(g->host, x, (size_t)n * d * 4);
    cudaCheck(cudaGraphLaunch(g->exec, st), "search: graph launch");
    cudaCheck(cudaStreamSynchronize(st), "search: synchronize");
    std::memcpy(distances, g->host + g->hostDistOff, (size_t)n * k * 4);
    std::memcpy(labels, g->host + g->hostLabOff, (size_t)n * k * 8);
    const int32_t word = *reinterpret_cast<const int32_t*>(g->host + g->hostStatusOff);
    im.lastStatus = word;
    if (word != 0) throwDeviceStatus(word, "search");
    return true;
}

size_t B200IndexFlat::searchScratchBytes(faiss::idx_t n, faiss::idx_t k) const {
    return align256(b200f_search_scratch_bytes(n, ntotal, d, (int)k, impl_->storageCode(), impl_->forcePath));
}

uint64_t B200IndexFlat::generation() const { return impl_->generation; }

void B200IndexFlat::searchDeviceEnqueue(faiss::idx_t n, const float* x, faiss::idx_t k,
                                        float* distances, faiss::idx_t* labels, void* scratch,
                                        size_t scratchSize) const {
    checkSearchArgs(n, x, k, distances, labels, ntotal);
    if (n == 0) return;
    const int64_t batch = k <= B200F_LIST_MAX_K ? kFusedBatch : kSelectBatch;
    B200_THROW_ARG_IF_NOT(B200F_ERR_UNSUPPORTED, n <= batch, "searchDeviceEnqueue: too many queries for one launch");
    DeviceGuard g(impl_->res->getDevice());
    const size_t scratchBytes =
            b200f_search_scratch_bytes(n, ntotal, d, (int)k, impl_->storageCode(), impl_->forcePath);
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, scratchBytes > 0, "searchDeviceEnqueue: cannot plan this shape");
    if (scratch) B200_THROW_ARG_IF_NOT(B200F_ERR_SCRATCH, scratchSize >= align256(scratchBytes), "scratch too small");
    // the caller's scratch (a captured graph must own what it touches), else the shared arena
    uint8_t* region = scratch ? static_cast<uint8_t*>(scratch)
                              : static_cast<uint8_t*>(impl_->res->getScratch(align256(scratchBytes)));
    B200FSearchArgs a;
    impl_->fillArgs(a, ntotal);
    a.queries = x;
    a.nq = n;
    a.k = (int)k;
    a.out_dist = distances;
    a.out_labels = reinterpret_cast<int64_t*>(labels);
    a.scratch = region;
    a.scratch_bytes = align256(scratchBytes);
    abiCheck(b200f_search(&a), "searchDeviceEnqueue");
}

void B200IndexFlat::synchronize() const {
    DeviceGuard g(impl_->res->getDevice());
    cudaStream_t st = impl_->stream();
    cudaCheck(cudaMemcpyAsync(impl_->hostStatus, impl_->status, 16, cudaMemcpyDeviceToHost, st),
              "synchronize: status copy");
    cudaCheck(cudaStreamSynchronize(st), "synchronize");
    if (impl_->hostStatus[0] != 0) {
        impl_->lastStatus = impl_->hostStatus[0];
        throwDeviceStatus(impl_->hostStatus[0], "search");
    }
}

// ---------------------------------------------------------------------------------------
// async search
// ---------------------------------------------------------------------------------------
struct B200SearchToken::Impl {
    std::shared_ptr<B200Resources> res;
    void* region = nullptr;       // device: queries, outputs, scratch
    int32_t* status = nullptr;    // device int32[4 * nbatches]
    uint8_t* host = nullptr;      // pinned: staged queries, result staging, status
    size_t hostDistOff = 0, hostLabOff = 0, hostStatusOff = 0;
    int64_t n = 0, k = 0;
    int nbatches = 0;
    float* userDist = nullptr;
    faiss::idx_t* userLabels = nullptr;
    bool distOnDevice = false, labelsOnDevice = false;
    cudaEvent_t done = nullptr;
    bool waited = false;

    // Buffers go back to the resources' pools, where the next token may take them at once:
    // nothing queued may still use them.  `finished` is set once the token's event was waited for.
    bool finished = false;
    void release() {
        if (res) {
            int prev = -1;
            (void)cudaGetDevice(&prev);
            (void)cudaSetDevice(res->getDevice());
            if (!finished && (region || status || host)) {
                // dropped before its work was waited for: everything of this token is in front of `done`
                if (!done || cudaEventSynchronize(done) != cudaSuccess) {
                    (void)cudaGetLastError();
                    (void)cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(res->getDefaultStream()));
                    (void)cudaStreamSynchronize(
                            reinterpret_cast<cudaStream_t>(res->getAuxStream(B200Resources::kDownloadStream)));
                }
            }
            if (done) res->releaseEvent(reinterpret_cast<EventHandle>(done));
            if (region) res->releaseDeviceTemp(region);
            if (status) res->releaseDeviceTemp(status);
            if (host) res->releasePinnedTemp(host);
            if (prev >= 0) (void)cudaSetDevice(prev);
        } else {
            free_pinned(host);
        }
        done = nullptr;
        region = nullptr;
        status = nullptr;
        host = nullptr;
    }
    ~Impl() { release(); }
};

B200SearchToken::B200SearchToken(std::unique_ptr<Impl> impl) : impl_(std::move(impl)) {}
B200SearchToken::B200SearchToken(B200SearchToken&&) noexcept = default;
B200SearchToken& B200SearchToken::operator=(B200SearchToken&& o) noexcept {
    if (this != &o) {
        if (impl_ && !impl_->waited) {
            try { wait(); } catch (...) {}
        }
        impl_ = std::move(o.impl_);
    }
    return *this;
}

B200SearchToken::~B200SearchToken() {
    // wait if the caller never did (src/MetalIndexFlat.mm:41-47)
    if (impl_ && !impl_->waited) {
        try { wait(); } catch (...) {}
    }
}

void B200SearchToken::wait() {
    B200_THROW_ARG_IF_NOT(B200F_ERR_STATE, impl_ != nullptr, "wait() on a moved-from search token");  // :50
    if (impl_->waited) return;
    impl_->waited = true;
    if (impl_->done) {
        DeviceGuard g(impl_->res->getDevice());
        cudaCheck(cudaEventSynchronize(impl_->done), "token wait");
        impl_->finished = true;
        if (!impl_->distOnDevice)
            std::memcpy(impl_->userDist, impl_->host + impl_->hostDistOff, (size_t)impl_->n * impl_->k * 4);
        if (!impl_->labelsOnDevice)
            std::memcpy(impl_->userLabels, impl_->host + impl_->hostLabOff, (size_t)impl_->n * impl_->k * 8);
        const int32_t* hs = reinterpret_cast<const int32_t*>(impl_->host + impl_->hostStatusOff);
        int bad = 0;
        for (int b = 0; b < impl_->nbatches; b++) bad |= hs[4 * b];
        impl_->release();
        if (bad)
            throwDeviceStatus(bad, "async search");
    }
}

bool B200SearchToken::isReady() const {
    B200_THROW_ARG_IF_NOT(B200F_ERR_STATE, impl_ != nullptr, "isReady() on a moved-from search token");  // :75
    if (impl_->waited || !impl_->done) return true;
    cudaError_t e = cudaEventQuery(impl_->done);
    if (e == cudaSuccess) return true;
    if (e == cudaErrorNotReady) {
        (void)cudaGetLastError();
        return false;
    }
    cudaCheck(e, "token isReady");
    return false;
}

B200SearchToken B200IndexFlat::searchAsync(faiss::idx_t n, const float* x, faiss::idx_t k,
                                           float* distances, faiss::idx_t* labels,
                                           const faiss::SearchParameters* /*params*/) const {
    checkSearchArgs(n, x, k, distances, labels, ntotal);
    std::unique_ptr<B200SearchToken::Impl> t(new B200SearchToken::Impl);
    if (n == 0) {  // ready token, nothing to write (src/MetalIndexFlat.mm:423-433)
        t->waited = true;
        return B200SearchToken(std::move(t));
    }
    DeviceGuard g(impl_->res->getDevice());
    cudaStream_t st = impl_->stream();
    t->res = impl_->res;
    t->n = n;
    t->k = k;
    t->userDist = distances;
    t->userLabels = labels;
    t->distOnDevice = isDevicePointer(distances);
    t->labelsOnDevice = isDevicePointer(labels);
    const bool qOnDevice = isDevicePointer(x);
    const int64_t batch = std::min<int64_t>(n, k <= B200F_LIST_MAX_K ? kFusedBatch : kSelectBatch);
    t->nbatches = (int)((n + batch - 1) / batch);
    const size_t scratchBytes =
            b200f_search_scratch_bytes(batch, ntotal, d, (int)k, impl_->storageCode(), impl_->forcePath);
    B200_THROW_ARG_IF_NOT(B200F_ERR_BAD_ARG, scratchBytes > 0, "searchAsync: cannot plan this shape");
    // per-call buffers: the token owns them (src/MetalIndexFlat.mm:441-476)
    CallLayout L = makeLayout(n, batch, d, k, !qOnDevice, n, true, scratchBytes);
    t->region = impl_->res->acquireDeviceTemp(L.total);
    t->status = static_cast<int32_t*>(impl_->res->acquireDeviceTemp(align256((size_t)t->nbatches * 16)));
    size_t hoff = 0;
    const size_t hostQOff = hoff;
    if (!qOnDevice) hoff += align256((size_t)n * d * 4);
    t->hostDistOff = hoff;
    hoff += align256((size_t)n * k * 4);
    t->hostLabOff = hoff;
    hoff += align256((size_t)n * k * 8);
    t->hostStatusOff = hoff;
    hoff += align256((size_t)t->nbatches * 16);
    t->host = static_cast<uint8_t*>(impl_->res->acquirePinnedTemp(hoff));
    if (!t->host) throw B200RuntimeError(B200F_ERR_OOM, "faiss-b200: pinned allocation failed");
    uint8_t* region = static_cast<uint8_t*>(t->region);

    // Three streams: the queries go up on the upload stream, the kernels run on the search
    // stream, the results come down on the download stream.  The tokens' kernels still run one
    // after the other, but the copies of a token overlap the kernels of its neighbours:
    // H2D(q[i+1]) | search(q[i]) | D2H(r[i-1]).  Each token has its own buffers, so only the
    // three hand-overs of one token need ordering (events).
    cudaStream_t up = reinterpret_cast<cudaStream_t>(impl_->res->getAuxStream(B200Resources::kUploadStream));
    cudaStream_t down = reinterpret_cast<cudaStream_t>(impl_->res->getAuxStream(B200Resources::kDownloadStream));
    t->done = reinterpret_cast<cudaEvent_t>(impl_->res->acquireEvent());
    const float* dqAll = x;
    if (!qOnDevice) {
        // the caller's array is only read during this call
        std::memcpy(t->host + hostQOff, x, (size_t)n * d * 4);
        cudaCheck(cudaMemcpyAsync(region + L.offQueries, t->host + hostQOff, (size_t)n * d * 4,
                                  cudaMemcpyHostToDevice, up),
                  "searchAsync: host to device copy of queries");
        if (up != st) {
            cudaCheck(cudaEventRecord(t->done, up), "searchAsync: event record");
            cudaCheck(cudaStreamWaitEvent(st, t->done, 0), "searchAsync: stream wait");
        }
        dqAll = reinterpret_cast<const float*>(region + L.offQueries);
    }
    float* dDistAll = t->distOnDevice ? distances : reinterpret_cast<float*>(region + L.offDist);
    int64_t* dLabAll = t->labelsOnDevice ? reinterpret_cast<int64_t*>(labels)
                                         : reinterpret_cast<int64_t*>(region + L.offLabels);
    for (int b = 0; b < t->nbatches; b++) {
        const int64_t q0 = (int64_t)b * batch;
        const int64_t nq = std::min<int64_t>(batch, n - q0);
        B200FSearchArgs a;
        impl_->fillArgs(a, ntotal);
        a.queries = dqAll + (size_t)q0 * d;
        a.nq = nq;
        a.k = (int)k;
        a.out_dist = dDistAll + (size_t)q0 * k;
        a.out_labels = dLabAll + (size_t)q0 * k;
        a.scratch = region + L.offScratch;
        a.scratch_bytes = L.scratchBytes;
        a.status = t->status + 4 * b;
        abiCheck(b200f_search(&a), "searchAsync");
    }
    if (down != st) {
        cudaCheck(cudaEventRecord(t->done, st), "searchAsync: event record");
        cudaCheck(cudaStreamWaitEvent(down, t->done, 0), "searchAsync: stream wait");
    }
    if (!t->distOnDevice)
        cudaCheck(cudaMemcpyAsync(t->host + t->hostDistOff, dDistAll, (size_t)n * k * 4,
                                  cudaMemcpyDeviceToHost, down),
                  "searchAsync: distances copy");
    if (!t->labelsOnDevice)
        cudaCheck(cudaMemcpyAsync(t->host + t->hostLabOff, dLabAll, (size_t)n * k * 8,
                                  cudaMemcpyDeviceToHost, down),
                  "searchAsync: labels copy");
    cudaCheck(cudaMemcpyAsync(t->host + t->hostStatusOff, t->status, (size_t)t->nbatches * 16,
                              cudaMemcpyDeviceToHost, down),
              "searchAsync: status copy");
    cudaCheck(cudaEventRecord(t->done, down), "event record");
    return B200SearchToken(std::move(t));
}

// ---------------------------------------------------------------------------------------
// converters (src/MetalIndexFlat.mm:552-587)
// ---------------------------------------------------------------------------------------
std::unique_ptr<B200IndexFlat> index_cpu_to_gpu(std::shared_ptr<B200Resources> resources,
                                                const faiss::IndexFlat* cpu_index,
                                                StorageType storage) {
    FAISS_THROW_IF_NOT_MSG(cpu_index != nullptr, "index_cpu_to_gpu: null index");
    std::unique_ptr<B200IndexFlat> out(
            new B200IndexFlat(std::move(resources), cpu_index->d, cpu_index->metric_type, storage));
    if (cpu_index->ntotal > 0) {
        out->reserve(cpu_index->ntotal);
        out->add(cpu_index->ntotal, cpu_index->get_xb());
    }
    return out;
}

std::unique_ptr<faiss::IndexFlat> index_gpu_to_cpu(const B200IndexFlat* gpu_index) {
    FAISS_THROW_IF_NOT_MSG(gpu_index != nullptr, "index_gpu_to_cpu: null index");
    std::unique_ptr<faiss::IndexFlat> out(new faiss::IndexFlat(gpu_index->d, gpu_index->metric_type));
    const faiss::idx_t n = gpu_index->ntotal;
    if (n > 0) {
        // one bulk dequantising read for every storage type (the reference loops
        // per vector for 16-bit storage, :574-580)
        const faiss::idx_t chunk = std::max<faiss::idx_t>(1, (faiss::idx_t)((256ull << 20) / ((size_t)gpu_index->d * 4)));
        std::vector<float> buf;
        for (faiss::idx_t r0 = 0; r0 < n; r0 += chunk) {
            const faiss::idx_t nr = std::min<faiss::idx_t>(chunk, n - r0);
            buf.resize((size_t)nr * gpu_index->d);
            gpu_index->reconstruct_n(r0, nr, buf.data());
            out->add(nr, buf.data());
        }
    }
    return out;
}

}  // namespace faiss_b200
