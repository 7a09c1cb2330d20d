// Default resource manager: one device, one stream, grow-only scratch arena.
// Counterpart of include/faiss-metal/StandardMetalResources.h:9-32.
#pragma once
#include "B200Resources.h"

namespace faiss_b200 {

class StandardB200Resources : public B200Resources {
   public:
    /// device < 0 selects the calling thread's current CUDA device.
    /// Throws std::runtime_error when there is no sm_100 device: there is no
    /// CPU fallback (src/StandardMetalResources.mm:17-44 throws likewise).
    explicit StandardB200Resources(int device = -1);
    ~StandardB200Resources() override;

    const B200DeviceCapabilities& getCapabilities() const override;
    int getDevice() const override;
    StreamHandle getDefaultStream() const override;
    void* allocBuffer(size_t size) override;
    void deallocBuffer(void* buf) override;
    void* getScratch(size_t bytes) override;
    size_t getScratchSize() const override;
    void* getPinnedStaging(size_t bytes) override;
    StreamHandle getAuxStream(int which) const override;
    EventHandle acquireEvent() override;
    void releaseEvent(EventHandle ev) override;
    /// Makes the default stream wait for everything queued so far on `producer` (a stream of
    /// the same device; nullptr = the legacy default stream).  No host synchronisation.
    void waitStream(StreamHandle producer);

    /// Recycling pools (at most 8 idle blocks each; a request takes the smallest idle block of
    /// at least its size and at most twice its size, else allocates).
    void* acquireDeviceTemp(size_t size) override;
    void releaseDeviceTemp(void* buf) override;
    void* acquirePinnedTemp(size_t size) override;
    void releasePinnedTemp(void* buf) override;
    /// Requests served from idle blocks / by a fresh allocation since construction.
    size_t tempPoolHits() const;
    size_t tempPoolMisses() const;

   private:
    struct Impl;
    std::unique_ptr<Impl> impl_;
};

}  // namespace faiss_b200
