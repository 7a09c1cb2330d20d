// Resource manager interface of the B200 backend.
// Counterpart of include/faiss-metal/MetalResources.h:20-54: device handle,
// default queue (a CUDA stream here), buffer allocation, and page-aligned host
// allocation for staging (pinned memory here).
#pragma once
#include <cstddef>
#include <memory>

#include "B200DeviceCapabilities.h"

struct CUstream_st;
struct CUevent_st;

namespace faiss_b200 {

typedef CUstream_st* StreamHandle;  // == cudaStream_t
typedef CUevent_st* EventHandle;    // == cudaEvent_t

/// Pinned host memory suitable for asynchronous copies; the analogue of the
/// reference's alloc_aligned / free_aligned (MetalResources.h:20-34).
/// Returns nullptr on failure.
void* alloc_pinned(size_t bytes);
void free_pinned(void* ptr);

class B200Resources {
   public:
    virtual ~B200Resources() = default;

    virtual const B200DeviceCapabilities& getCapabilities() const = 0;
    virtual int getDevice() const = 0;
    virtual StreamHandle getDefaultStream() const = 0;

    /// Side streams for copies that should overlap the kernels on the default stream:
    /// 0 = host-to-device (queries of the next search, the next chunk of an add),
    /// 1 = device-to-host (results of the previous search, reconstructed rows).  Work on them
    /// is ordered against the default stream with events only.  An implementation without side
    /// streams returns the default stream: everything then serialises, results are the same.
    enum { kUploadStream = 0, kDownloadStream = 1 };
    virtual StreamHandle getAuxStream(int /*which*/) const { return getDefaultStream(); }

    /// Timing-disabled events for the ordering above and for search tokens.  Recycled by the
    /// standard implementation, so that an asynchronous search creates nothing per call.
    virtual EventHandle acquireEvent();
    virtual void releaseEvent(EventHandle ev);

    /// Device buffer (throws std::runtime_error on failure,
    /// src/StandardMetalResources.mm:68-76).
    virtual void* allocBuffer(size_t size) = 0;
    virtual void deallocBuffer(void* buf) = 0;

    /// Buffers of in-flight asynchronous searches (device memory and pinned host memory).  Same
    /// contract as allocBuffer / alloc_pinned, but an implementation may recycle them: a
    /// released buffer must no longer be in use by any queued work.  The reference allocates
    /// fresh MTLBuffers per searchAsync call (src/MetalIndexFlat.mm:441-476); on CUDA that would
    /// put a cudaMalloc / cudaFree (a device-wide synchronisation) into every call.
    virtual void* acquireDeviceTemp(size_t size) { return allocBuffer(size); }
    virtual void releaseDeviceTemp(void* buf) { deallocBuffer(buf); }
    virtual void* acquirePinnedTemp(size_t size) { return alloc_pinned(size); }  ///< nullptr on failure
    virtual void releasePinnedTemp(void* buf) { free_pinned(buf); }

    /// Grow-only scratch region shared by the synchronous searches of every index
    /// that uses these resources (src/MetalIndexFlat.mm:102-142 kept one per index).
    /// The pointer stays valid until the next call with a larger size; work using it
    /// must be ordered on the default stream.
    virtual void* getScratch(size_t bytes) = 0;
    virtual size_t getScratchSize() const = 0;
    /// Grow-only pinned staging region (same lifetime rule as getScratch).
    virtual void* getPinnedStaging(size_t bytes) = 0;
};

}  // namespace faiss_b200
