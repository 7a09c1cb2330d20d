// Device array that grows in place: a virtual address range is reserved once for the largest
// size the array may ever reach, and physical memory is mapped into it piece by piece as rows
// are added (CUDA virtual memory management: address reserve / create / map / set access).
// The base address never changes and nothing is copied when the array grows, so an index
// of tens of gigabytes does not need a second copy of itself to take one more add(), and
// tensor maps built over the base stay valid.
//
// The reference grows its row buffer by allocating a new MTLBuffer of twice the size and
// copying (src/MetalIndexFlat.mm:196-208, 272-285); this class replaces that step.
#pragma once
#include <cstddef>
#include <cstdint>
#include <vector>

namespace faiss_b200 {

class GrowableDeviceArray {
   public:
    GrowableDeviceArray() = default;
    ~GrowableDeviceArray();
    GrowableDeviceArray(const GrowableDeviceArray&) = delete;
    GrowableDeviceArray& operator=(const GrowableDeviceArray&) = delete;

    /// True when the driver offers the virtual memory management calls on `device`.
    static bool supported(int device);

    /// Reserves `maxBytes` of address space on `device` (nothing is backed yet).  Returns false
    /// (and stays empty) when the reservation cannot be made; the caller then falls back to
    /// plain allocations.
    bool reserve(int device, size_t maxBytes);

    /// Backs every byte of [offset, offset + bytes) that is not backed yet.  Ranges may be
    /// touched in any order (an array of several planes backs the used part of each plane).
    /// Throws std::runtime_error when the device is out of memory or the range is outside
    /// the reservation; on failure the ranges backed before stay backed.
    void back(size_t offset, size_t bytes);

    /// Unmaps and frees everything, including the address range.
    void release();

    void* data() const { return reinterpret_cast<void*>(base_); }
    bool valid() const { return base_ != 0; }
    size_t reservedBytes() const { return reserved_; }
    size_t backedBytes() const { return backedBytes_; }

   private:
    struct Piece {
        size_t offset, size;
        unsigned long long handle;
    };
    int device_ = -1;
    uintptr_t base_ = 0;
    size_t reserved_ = 0;
    size_t granule_ = 0;
    size_t backedBytes_ = 0;
    std::vector<Piece> pieces_;       // mapped pieces
    std::vector<uint8_t> backed_;     // one flag per granule
};

}  // namespace faiss_b200
