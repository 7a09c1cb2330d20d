// StandardB200Resources: device, stream, buffers, grow-only scratch and pinned staging.
// Counterpart of src/StandardMetalResources.mm:10-91 and
// src/MetalDeviceCapabilities.mm:8-124.
#include <cuda_runtime.h>

#include <mutex>
#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/b200_flat.h"
#include "../include/faiss-b200/B200Exception.h"
#include "../include/faiss-b200/StandardB200Resources.h"

namespace faiss_b200 {

namespace {

void check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        std::string msg = std::string("faiss-b200: ") + what + ": " + cudaGetErrorString(e);
        (void)cudaGetLastError();
        throw B200RuntimeError(e == cudaErrorMemoryAllocation ? B200F_ERR_OOM : B200F_ERR_CUDA, msg);
    }
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) check(cudaSetDevice(dev), "cudaSetDevice");
    }
    ~DeviceGuard() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) (void)cudaSetDevice(prev);
    }
};

}  // namespace

void* alloc_pinned(size_t bytes) {
    void* p = nullptr;
    if (cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocDefault) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    return p;
}

void free_pinned(void* ptr) {
    if (ptr) (void)cudaFreeHost(ptr);
}

EventHandle B200Resources::acquireEvent() {
    cudaEvent_t ev = nullptr;
    check(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate");
    return ev;
}

void B200Resources::releaseEvent(EventHandle ev) {
    if (ev) (void)cudaEventDestroy(ev);
}

B200DeviceCapabilities queryDeviceCapabilities(int device) {
    B200FCaps c;
    int rc = b200f_device_caps(device, &c);
    if (rc != B200F_OK)
        throw B200RuntimeError(rc, std::string("faiss-b200: cannot query device: ") + b200f_status_string(rc));
    B200DeviceCapabilities caps;
    caps.device = c.device;
    caps.ccMajor = c.cc_major;
    caps.ccMinor = c.cc_minor;
    caps.smCount = c.sm_count;
    caps.maxSharedMemPerBlock = c.max_smem_per_block;
    caps.l2Bytes = c.l2_bytes;
    caps.hbmBytes = c.hbm_bytes;
    caps.smClockKHz = c.sm_clock_khz;
    caps.memClockKHz = c.mem_clock_khz;
    caps.supported = c.supported != 0;
    caps.name = c.name;
    return caps;
}

std::string describeCapabilities(const B200DeviceCapabilities& caps) {
    std::ostringstream os;
    os << "device " << caps.device << ": " << caps.name << " (sm_" << caps.ccMajor << caps.ccMinor
       << "), " << caps.smCount << " SMs, " << (caps.hbmBytes >> 20) << " MiB HBM, "
       << (caps.l2Bytes >> 20) << " MiB L2, " << caps.maxSharedMemPerBlock
       << " B shared memory per block, SM clock " << caps.smClockKHz / 1000 << " MHz, "
       << (caps.supported ? "supported" : "NOT supported (needs sm_100)");
    return os.str();
}

namespace {

// Blocks handed out and taken back whole; idle blocks are kept for the next request of a
// similar size.  `Alloc` / `Free` are the raw allocator of the memory kind.
class BlockPool {
   public:
    static constexpr size_t kMaxIdle = 8;
    static constexpr size_t kGranule = 1u << 20;

    template <typename Alloc>
    void* acquire(size_t size, Alloc alloc) {
        const size_t need = ((size ? size : 1) + kGranule - 1) / kGranule * kGranule;
        {
            std::lock_guard<std::mutex> g(mu_);
            int best = -1;
            for (size_t i = 0; i < idle_.size(); i++)
                if (idle_[i].second >= need && idle_[i].second <= 2 * need &&
                    (best < 0 || idle_[i].second < idle_[(size_t)best].second))
                    best = (int)i;
            if (best >= 0) {
                std::pair<void*, size_t> blk = idle_[(size_t)best];
                idle_.erase(idle_.begin() + best);
                busy_.push_back(blk);
                hits_++;
                return blk.first;
            }
            misses_++;
        }
        void* p = alloc(need);
        if (p) {
            std::lock_guard<std::mutex> g(mu_);
            busy_.emplace_back(p, need);
        }
        return p;
    }

    template <typename Free>
    void release(void* p, Free free_fn) {
        if (!p) return;
        void* evict = nullptr;
        {
            std::lock_guard<std::mutex> g(mu_);
            size_t size = 0;
            for (size_t i = 0; i < busy_.size(); i++)
                if (busy_[i].first == p) {
                    size = busy_[i].second;
                    busy_.erase(busy_.begin() + (long)i);
                    break;
                }
            if (size == 0) {  // not ours: hand it straight back
                evict = p;
            } else {
                idle_.emplace_back(p, size);
                if (idle_.size() > kMaxIdle) {  // drop the block that has been idle longest
                    evict = idle_.front().first;
                    idle_.erase(idle_.begin());
                }
            }
        }
        if (evict) free_fn(evict);
    }

    template <typename Free>
    void clear(Free free_fn) {
        std::lock_guard<std::mutex> g(mu_);
        for (auto& b : idle_) free_fn(b.first);
        for (auto& b : busy_) free_fn(b.first);
        idle_.clear();
        busy_.clear();
    }

    size_t hits() const { return hits_; }
    size_t misses() const { return misses_; }

   private:
    std::mutex mu_;
    std::vector<std::pair<void*, size_t>> idle_, busy_;
    size_t hits_ = 0, misses_ = 0;
};

}  // namespace

struct StandardB200Resources::Impl {
    int device = 0;
    cudaStream_t stream = nullptr;
    cudaStream_t aux[2] = {nullptr, nullptr};
    std::mutex evMu;
    std::vector<cudaEvent_t> idleEvents;
    B200DeviceCapabilities caps;
    void* scratch = nullptr;
    size_t scratchBytes = 0;
    void* pinned = nullptr;
    size_t pinnedBytes = 0;
    BlockPool devicePool, pinnedPool;
};

StandardB200Resources::StandardB200Resources(int device) : impl_(new Impl) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        (void)cudaGetLastError();
        throw B200RuntimeError(B200F_ERR_NO_DEVICE,
                               "faiss-b200: no CUDA device available (this backend has no CPU fallback)");
    }
    if (device < 0) check(cudaGetDevice(&device), "cudaGetDevice");
    if (device >= count)
        throw B200RuntimeError(B200F_ERR_NO_DEVICE, "faiss-b200: device ordinal out of range");
    impl_->device = device;
    impl_->caps = queryDeviceCapabilities(device);
    if (!impl_->caps.supported)
        throw B200RuntimeError(B200F_ERR_NO_DEVICE, "faiss-b200: device is not sm_100 (" + impl_->caps.name +
                                                            "); kernels are built for sm_100a only");
    DeviceGuard g(device);
    check(cudaStreamCreateWithFlags(&impl_->stream, cudaStreamNonBlocking), "cudaStreamCreate");
    for (int i = 0; i < 2; i++)
        check(cudaStreamCreateWithFlags(&impl_->aux[i], cudaStreamNonBlocking), "cudaStreamCreate");
}

StandardB200Resources::~StandardB200Resources() {
    if (!impl_) return;
    int prev = -1;
    (void)cudaGetDevice(&prev);
    (void)cudaSetDevice(impl_->device);
    for (int i = 0; i < 2; i++)
        if (impl_->aux[i]) {
            (void)cudaStreamSynchronize(impl_->aux[i]);
            (void)cudaStreamDestroy(impl_->aux[i]);
        }
    if (impl_->stream) {
        (void)cudaStreamSynchronize(impl_->stream);
        (void)cudaStreamDestroy(impl_->stream);
    }
    for (cudaEvent_t ev : impl_->idleEvents) (void)cudaEventDestroy(ev);
    if (impl_->scratch) (void)cudaFree(impl_->scratch);
    if (impl_->pinned) (void)cudaFreeHost(impl_->pinned);
    impl_->devicePool.clear([](void* p) { (void)cudaFree(p); });
    impl_->pinnedPool.clear([](void* p) { (void)cudaFreeHost(p); });
    if (prev >= 0) (void)cudaSetDevice(prev);
    (void)cudaGetLastError();
}

const B200DeviceCapabilities& StandardB200Resources::getCapabilities() const { return impl_->caps; }
int StandardB200Resources::getDevice() const { return impl_->device; }
StreamHandle StandardB200Resources::getDefaultStream() const { return impl_->stream; }
StreamHandle StandardB200Resources::getAuxStream(int which) const {
    return (which == kUploadStream || which == kDownloadStream) ? impl_->aux[which] : impl_->stream;
}

EventHandle StandardB200Resources::acquireEvent() {
    {
        std::lock_guard<std::mutex> g(impl_->evMu);
        if (!impl_->idleEvents.empty()) {
            cudaEvent_t ev = impl_->idleEvents.back();
            impl_->idleEvents.pop_back();
            return ev;
        }
    }
    DeviceGuard g(impl_->device);
    cudaEvent_t ev = nullptr;
    check(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate");
    return ev;
}

void StandardB200Resources::releaseEvent(EventHandle ev) {
    if (!ev) return;
    std::lock_guard<std::mutex> g(impl_->evMu);
    if (impl_->idleEvents.size() < 64) {
        impl_->idleEvents.push_back(ev);
        return;
    }
    (void)cudaEventDestroy(ev);
}

void StandardB200Resources::waitStream(StreamHandle producer) {
    DeviceGuard g(impl_->device);
    cudaEvent_t ev = acquireEvent();
    cudaError_t e = cudaEventRecord(ev, producer);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(impl_->stream, ev, 0);
    releaseEvent(ev);   // the wait has captured the record; the event may be recorded again
    check(e, "waitStream");
}

void* StandardB200Resources::allocBuffer(size_t size) {
    DeviceGuard g(impl_->device);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, size ? size : 256);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        throw B200RuntimeError(e == cudaErrorMemoryAllocation ? B200F_ERR_OOM : B200F_ERR_CUDA,
                               "faiss-b200: failed to allocate device buffer of " + std::to_string(size) +
                                       " bytes: " + cudaGetErrorString(e));
    }
    return p;
}

void StandardB200Resources::deallocBuffer(void* buf) {
    if (!buf) return;
    DeviceGuard g(impl_->device);
    (void)cudaFree(buf);
}

void* StandardB200Resources::acquireDeviceTemp(size_t size) {
    DeviceGuard g(impl_->device);
    void* p = impl_->devicePool.acquire(size, [](size_t n) -> void* {
        void* q = nullptr;
        if (cudaMalloc(&q, n) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        return q;
    });
    if (!p)
        throw B200RuntimeError(B200F_ERR_OOM,
                               "faiss-b200: failed to allocate device buffer of " + std::to_string(size) + " bytes");
    return p;
}

void StandardB200Resources::releaseDeviceTemp(void* buf) {
    if (!buf) return;
    DeviceGuard g(impl_->device);
    impl_->devicePool.release(buf, [](void* p) { (void)cudaFree(p); });
}

void* StandardB200Resources::acquirePinnedTemp(size_t size) {
    return impl_->pinnedPool.acquire(size, [](size_t n) -> void* { return alloc_pinned(n); });
}

void StandardB200Resources::releasePinnedTemp(void* buf) {
    impl_->pinnedPool.release(buf, [](void* p) { free_pinned(p); });
}

size_t StandardB200Resources::tempPoolHits() const { return impl_->devicePool.hits() + impl_->pinnedPool.hits(); }
size_t StandardB200Resources::tempPoolMisses() const {
    return impl_->devicePool.misses() + impl_->pinnedPool.misses();
}

void* StandardB200Resources::getScratch(size_t bytes) {
    if (bytes > impl_->scratchBytes) {
        DeviceGuard g(impl_->device);
        // work already queued on the stream may still use the old region
        check(cudaStreamSynchronize(impl_->stream), "cudaStreamSynchronize");
        if (impl_->scratch) (void)cudaFree(impl_->scratch);
        impl_->scratch = nullptr;
        impl_->scratchBytes = 0;
        size_t want = bytes + (bytes >> 3);  // a little headroom against regrowth
        want = (want + 255) & ~(size_t)255;
        cudaError_t e = cudaMalloc(&impl_->scratch, want);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            want = (bytes + 255) & ~(size_t)255;
            check(cudaMalloc(&impl_->scratch, want), "cudaMalloc(scratch)");
        }
        impl_->scratchBytes = want;
    }
    return impl_->scratch;
}

size_t StandardB200Resources::getScratchSize() const { return impl_->scratchBytes; }

void* StandardB200Resources::getPinnedStaging(size_t bytes) {
    if (bytes > impl_->pinnedBytes) {
        DeviceGuard g(impl_->device);
        check(cudaStreamSynchronize(impl_->stream), "cudaStreamSynchronize");
        if (impl_->pinned) (void)cudaFreeHost(impl_->pinned);
        impl_->pinned = nullptr;
        impl_->pinnedBytes = 0;
        check(cudaHostAlloc(&impl_->pinned, bytes, cudaHostAllocDefault), "cudaHostAlloc(staging)");
        impl_->pinnedBytes = bytes;
    }
    return impl_->pinned;
}

}  // namespace faiss_b200
