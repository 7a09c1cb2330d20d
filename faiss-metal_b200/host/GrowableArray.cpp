// GrowableDeviceArray: see GrowableArray.h.  The driver entry points are looked up through the
// runtime (cudaGetDriverEntryPoint), so the library does not link against the driver library.
#include "GrowableArray.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <stdexcept>
#include <string>

namespace faiss_b200 {

namespace {

typedef CUresult (*GranularityFn)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
typedef CUresult (*ReserveFn)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
typedef CUresult (*CreateFn)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
typedef CUresult (*MapFn)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
typedef CUresult (*SetAccessFn)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
typedef CUresult (*UnmapFn)(CUdeviceptr, size_t);
typedef CUresult (*ReleaseFn)(CUmemGenericAllocationHandle);
typedef CUresult (*AddressFreeFn)(CUdeviceptr, size_t);

struct DriverApi {
    GranularityFn granularity = nullptr;
    ReserveFn reserve = nullptr;
    CreateFn create = nullptr;
    MapFn map = nullptr;
    SetAccessFn setAccess = nullptr;
    UnmapFn unmap = nullptr;
    ReleaseFn release = nullptr;
    AddressFreeFn addressFree = nullptr;
    bool ok = false;
};

void* lookup(const char* name) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    return fn;
}

const DriverApi& api() {
    static DriverApi a;
    static std::once_flag once;
    std::call_once(once, [] {
        a.granularity = reinterpret_cast<GranularityFn>(lookup("cuMemGetAllocationGranularity"));
        a.reserve = reinterpret_cast<ReserveFn>(lookup("cuMemAddressReserve"));
        a.create = reinterpret_cast<CreateFn>(lookup("cuMemCreate"));
        a.map = reinterpret_cast<MapFn>(lookup("cuMemMap"));
        a.setAccess = reinterpret_cast<SetAccessFn>(lookup("cuMemSetAccess"));
        a.unmap = reinterpret_cast<UnmapFn>(lookup("cuMemUnmap"));
        a.release = reinterpret_cast<ReleaseFn>(lookup("cuMemRelease"));
        a.addressFree = reinterpret_cast<AddressFreeFn>(lookup("cuMemAddressFree"));
        a.ok = a.granularity && a.reserve && a.create && a.map && a.setAccess && a.unmap && a.release &&
               a.addressFree;
    });
    return a;
}

CUmemAllocationProp deviceProp(int device) {
    CUmemAllocationProp prop = {};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    return prop;
}

}  // namespace

bool GrowableDeviceArray::supported(int device) {
    if (!api().ok) return false;
    int vmm = 0;
    if (cudaDeviceGetAttribute(&vmm, cudaDevAttrMemoryPoolsSupported, device) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    // every device with memory pools has virtual memory management; the granularity query
    // below is the real test
    const CUmemAllocationProp prop = deviceProp(device);
    size_t g = 0;
    return vmm != 0 && api().granularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS &&
           g > 0;
}

GrowableDeviceArray::~GrowableDeviceArray() { release(); }

bool GrowableDeviceArray::reserve(int device, size_t maxBytes) {
    release();
    if (!api().ok || maxBytes == 0) return false;
    const CUmemAllocationProp prop = deviceProp(device);
    size_t g = 0;
    if (api().granularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || g == 0)
        return false;
    const size_t size = (maxBytes + g - 1) / g * g;
    CUdeviceptr p = 0;
    if (api().reserve(&p, size, 0, 0, 0) != CUDA_SUCCESS || p == 0) return false;
    device_ = device;
    base_ = static_cast<uintptr_t>(p);
    reserved_ = size;
    granule_ = g;
    backedBytes_ = 0;
    backed_.assign(size / g, 0);
    return true;
}

void GrowableDeviceArray::back(size_t offset, size_t bytes) {
    if (bytes == 0) return;
    if (!valid() || offset + bytes > reserved_)
        throw std::runtime_error("faiss-b200: growable array: range outside the reserved address space");
    const size_t g0 = offset / granule_;
    const size_t g1 = (offset + bytes + granule_ - 1) / granule_;
    const CUmemAllocationProp prop = deviceProp(device_);
    CUmemAccessDesc access = {};
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = device_;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    size_t g = g0;
    while (g < g1) {
        if (backed_[g]) {
            g++;
            continue;
        }
        size_t e = g;
        while (e < g1 && !backed_[e]) e++;
        // one physical allocation for the run of granules [g, e)
        const size_t off = g * granule_, size = (e - g) * granule_;
        CUmemGenericAllocationHandle h = 0;
        CUresult r = api().create(&h, size, &prop, 0);
        if (r != CUDA_SUCCESS)
            throw std::runtime_error("faiss-b200: failed to allocate " + std::to_string(size) +
                                     " bytes of device memory for the index (driver error " +
                                     std::to_string((int)r) + ")");
        r = api().map(static_cast<CUdeviceptr>(base_ + off), size, 0, h, 0);
        if (r == CUDA_SUCCESS) {
            r = api().setAccess(static_cast<CUdeviceptr>(base_ + off), size, &access, 1);
            if (r != CUDA_SUCCESS) (void)api().unmap(static_cast<CUdeviceptr>(base_ + off), size);
        }
        if (r != CUDA_SUCCESS) {
            (void)api().release(h);
            throw std::runtime_error("faiss-b200: failed to map device memory for the index (driver error " +
                                     std::to_string((int)r) + ")");
        }
        pieces_.push_back(Piece{off, size, static_cast<unsigned long long>(h)});
        for (size_t i = g; i < e; i++) backed_[i] = 1;
        backedBytes_ += size;
        g = e;
    }
}

void GrowableDeviceArray::release() {
    if (!valid()) return;
    for (const Piece& p : pieces_) {
        (void)api().unmap(static_cast<CUdeviceptr>(base_ + p.offset), p.size);
        (void)api().release(static_cast<CUmemGenericAllocationHandle>(p.handle));
    }
    (void)api().addressFree(static_cast<CUdeviceptr>(base_), reserved_);
    pieces_.clear();
    backed_.clear();
    base_ = 0;
    reserved_ = 0;
    backedBytes_ = 0;
    device_ = -1;
}

}  // namespace faiss_b200
