// Device capabilities of the B200 backend.
// Counterpart of include/faiss-metal/MetalDeviceCapabilities.h:13-69: the
// reference's chip-generation dispatch matrix does not exist here (one target,
// sm_100a); what remains is the description of the device the resources own.
#pragma once
#include <cstdint>
#include <string>

namespace faiss_b200 {

struct B200DeviceCapabilities {
    int device = -1;
    int ccMajor = 0, ccMinor = 0;
    int smCount = 0;
    int maxSharedMemPerBlock = 0;
    int l2Bytes = 0;
    int64_t hbmBytes = 0;
    int smClockKHz = 0;
    int memClockKHz = 0;
    bool supported = false;  // true on sm_100
    std::string name;

    // Limits of the search path (README.md:218-219 of the reference: k <= 4096,
    // 2^31-1 vectors per index; here per shard).
    static constexpr int kMaxK = 4096;
    static constexpr int64_t kMaxVectorsPerShard = 2147483647LL;
};

/// Query the capabilities of a CUDA device (src/MetalDeviceCapabilities.mm:8-96).
B200DeviceCapabilities queryDeviceCapabilities(int device);

/// Human-readable summary (src/MetalDeviceCapabilities.mm:98-124).
std::string describeCapabilities(const B200DeviceCapabilities& caps);

}  // namespace faiss_b200
