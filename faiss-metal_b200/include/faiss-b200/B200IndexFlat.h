// Flat (brute-force) k-NN index on a B200 GPU: the drop-in for
// faiss_metal::MetalIndexFlat (include/faiss-metal/MetalIndexFlat.h:13-120).
// Same constructors, overrides, async token, storage enum and converters.
#pragma once

#include <faiss/Index.h>
#include <faiss/IndexFlat.h>
#include <faiss/MetricType.h>

#include <cstdint>
#include <memory>

namespace faiss_b200 {

class B200Resources;
class B200IndexFlat;

/// Move-only token returned by B200IndexFlat::searchAsync()
/// (MetalSearchToken, include/faiss-metal/MetalIndexFlat.h:15-36).
/// Owns every per-call buffer, so several searches may be in flight.
class B200SearchToken {
   public:
    B200SearchToken(B200SearchToken&&) noexcept;
    B200SearchToken& operator=(B200SearchToken&&) noexcept;
    ~B200SearchToken();  // waits if the caller never did

    B200SearchToken(const B200SearchToken&) = delete;
    B200SearchToken& operator=(const B200SearchToken&) = delete;

    /// Block until the GPU has finished, then copy results to the caller's arrays.
    void wait();
    /// Non-blocking: true once the GPU has finished.
    bool isReady() const;

   private:
    friend class B200IndexFlat;
    struct Impl;
    std::unique_ptr<Impl> impl_;
    explicit B200SearchToken(std::unique_ptr<Impl> impl);
};

/// Vector storage precision (include/faiss-metal/MetalIndexFlat.h:39-43).
enum class StorageType : uint8_t {
    Float32 = 0,
    Float16 = 1,
    BFloat16 = 2,
};

class B200IndexFlat : public faiss::Index {
   public:
    B200IndexFlat(std::shared_ptr<B200Resources> resources, int d,
                  faiss::MetricType metric = faiss::METRIC_L2, bool useFloat16Storage = false);
    B200IndexFlat(std::shared_ptr<B200Resources> resources, int d, faiss::MetricType metric,
                  StorageType storage);
    ~B200IndexFlat() override;

    // --- faiss::Index interface ---
    /// x: fp32 [n][d] in host memory or device memory of this index's GPU.
    void add(faiss::idx_t n, const float* x) override;
    /// x / distances / labels may each be host or device pointers.
    void search(faiss::idx_t n, const float* x, faiss::idx_t k, float* distances,
                faiss::idx_t* labels,
                const faiss::SearchParameters* params = nullptr) const override;
    void reset() override;
    void reconstruct(faiss::idx_t key, float* recons) const override;

    B200SearchToken searchAsync(faiss::idx_t n, const float* x, faiss::idx_t k, float* distances,
                                faiss::idx_t* labels,
                                const faiss::SearchParameters* params = nullptr) const;

    /// Host copy of the stored vectors for Float32 storage (refreshed lazily after
    /// add / reset), nullptr for 16-bit storage.  The reference returned a pointer
    /// into unified memory (MetalIndexFlat.h:94); discrete HBM needs the mirror.
    const float* getVectorsData() const;
    bool isFloat16Storage() const;
    bool isBFloat16Storage() const;
    StorageType getStorageType() const;

    /// Test knob in the place of setForceMPS (MetalIndexFlat.h:106):
    /// 0 = choose by (nq, k), 1 = streaming scan, 2 = tensor-core GEMM.
    void setForcePath(int path);

    // --- additions needed by a discrete, multi-GPU device ---
    /// Make room for n vectors in total without the x2 growth copies.
    void reserve(faiss::idx_t n);
    /// 0: grow in place (address range reserved once, memory mapped behind the rows; default
    /// where the driver supports it), 1: the reference's allocate-copy-free growth
    /// (src/MetalIndexFlat.mm:196-222).  Only before the first add / reserve.
    void setGrowthMode(int mode);
    /// FP32 storage only: which split planes the tensor path multiplies (B200F_PLANES_BF16X3: three
    /// bf16 planes, six products; B200F_PLANES_FP16X2: two fp16 planes of the rows scaled by a power of
    /// two the index picks from its first rows, three products).  The default is FP16X2; an index
    /// whose rows stop fitting fp16's range re-splits itself into BF16X3 during that add().  Both
    /// hold the 1e-4 contract.  Only on an empty index.
    void setFp32PlaneFormat(int format);
    int getFp32PlaneFormat() const;
    /// Searches of at most 8 queries with host buffers are replayed from a CUDA graph captured
    /// on their second occurrence (default on).  Off: every search is enqueued call by call.
    void setUseGraphs(bool on);
    /// Rows [first, first + n) as fp32 into out (host or device pointer).
    void reconstruct_n(faiss::idx_t first, faiss::idx_t n, float* out) const;
    /// Labels returned by search are local row number + this base (row shards).
    void setLabelBase(faiss::idx_t base);
    /// Device pointers of the shard (rows in storage precision).
    const void* getDeviceRows() const;
    /// The resources this index was built on.
    std::shared_ptr<B200Resources> getResources() const;
    /// Enqueue a search whose queries and outputs are all DEVICE pointers on the resources'
    /// stream and return without synchronising (single batch: n <= 16384 for k <= 32,
    /// n <= 1024 otherwise).  The multi-GPU layer chains the candidate exchange and the merge
    /// behind it on the same stream; call synchronize() before reading results on the host.
    /// `scratch` (device, searchScratchBytes(n, k) bytes): used instead of the resources' shared
    /// scratch arena, for callers that capture the call into a CUDA graph of their own.
    void searchDeviceEnqueue(faiss::idx_t n, const float* x, faiss::idx_t k, float* distances,
                             faiss::idx_t* labels, void* scratch = nullptr, size_t scratchSize = 0) const;
    size_t searchScratchBytes(faiss::idx_t n, faiss::idx_t k) const;
    /// Changes whenever stored rows, label base or forced path change: work captured against an
    /// older value must not be replayed.
    uint64_t generation() const;
    /// Wait for the resources' stream and throw if a search reported a device-side error.
    void synchronize() const;
    /// Device status word of the most recent synchronous search (0 = fine).
    int lastDeviceStatus() const;
    /// Test aid: queues a one-CTA kernel that waits, with the library's bounded-wait helper and a
    /// limit of `limitCycles` SM clocks, on a barrier nothing signals; it gives up, marks this
    /// index's status word and returns.  The next synchronize() then throws the device-wait
    /// error; the search after that clears the word and runs normally.
    void debugWaitExpiry(int64_t limitCycles);

   private:
    struct Impl;
    std::unique_ptr<Impl> impl_;
    bool searchFromGraph(faiss::idx_t n, const float* x, faiss::idx_t k, float* distances,
                         faiss::idx_t* labels) const;
};

/// CPU IndexFlat -> GPU index (index_cpu_to_metal, MetalIndexFlat.h:114).  The
/// reference always created Float32 storage; the storage argument is an addition.
std::unique_ptr<B200IndexFlat> index_cpu_to_gpu(std::shared_ptr<B200Resources> resources,
                                                const faiss::IndexFlat* cpu_index,
                                                StorageType storage = StorageType::Float32);

/// GPU index -> CPU IndexFlat (index_metal_to_cpu, MetalIndexFlat.h:119).
std::unique_ptr<faiss::IndexFlat> index_gpu_to_cpu(const B200IndexFlat* gpu_index);

}  // namespace faiss_b200
