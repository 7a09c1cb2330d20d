// Flat k-NN index whose rows are sharded over the GPUs of one box, behind the same
// faiss::Index surface as B200IndexFlat (include/faiss-metal/MetalIndexFlat.h:47-111 is the
// contract; the reference itself is single-device, src/StandardMetalResources.mm:17-23).
//
// Every GPU searches its own rows with the single-GPU path; the per-GPU (distance, label)
// candidate lists are exchanged with one ncclAllGather issued by this class, on the
// resources' own stream, between the shard search and the k-way merge kernel: no other
// library and no extra stream sits in that sequence.
//
// Two ways to run it:
//  * one process drives several GPUs (constructor over a list of resources): add() places rows
//    block-cyclically, global row g on shard (g / B) % S, so any sequence of add() calls stays
//    balanced and label <-> (shard, local row) is a closed form;
//  * one process per GPU (constructor over a rank's own B200IndexFlat): the caller adds each
//    rank's rows to its local index and sets its label base; search() is a collective call.
// Queries cross PCIe once: GPU i receives the i-th slice of the query matrix and the slices are
// all-gathered over NVLink; only the caller that passes output arrays gets results copied back.
#pragma once

#include <cstdint>
#include <memory>
#include <vector>

#include "B200IndexFlat.h"

namespace faiss_b200 {

/// The 128 bytes every rank of a one-process-per-GPU group needs to join the same NCCL
/// communicator (an ncclUniqueId).  Rank 0 creates it and hands it to the others by any means
/// it has (a file, a socket, torch.distributed's store).
struct B200CommId {
    char bytes[128];
};
B200CommId createCommId();

class B200ShardedIndexFlat : public faiss::Index {
   public:
    /// One process, several GPUs: one resources object per GPU (several shards on ONE device are
    /// accepted too and exchange with device copies: a single-GPU rehearsal of the same code).
    B200ShardedIndexFlat(std::vector<std::shared_ptr<B200Resources>> resources, int d,
                         faiss::MetricType metric = faiss::METRIC_L2,
                         StorageType storage = StorageType::Float32, int64_t blockRows = 65536);
    /// One process per GPU: `local` holds this rank's rows (label base set by the caller).
    /// world == 1 needs no communicator and ignores `id`.
    B200ShardedIndexFlat(std::shared_ptr<B200IndexFlat> local, int rank, int world, const B200CommId& id);
    ~B200ShardedIndexFlat() override;

    // --- faiss::Index interface ---
    void add(faiss::idx_t n, const float* x) override;   ///< several-GPU form only
    /// x host or device (device: on the first shard's GPU / this rank's GPU, complete on the
    /// resources' stream).  One process per GPU: a collective call with identical n, k and x on
    /// every rank; distances / labels may both be nullptr on ranks that do not want the result.
    void search(faiss::idx_t n, const float* x, faiss::idx_t k, float* distances, faiss::idx_t* labels,
                const faiss::SearchParameters* params = nullptr) const override;
    void reset() override;
    void reconstruct(faiss::idx_t key, float* recons) const override;   ///< several-GPU form only

    /// Device-pointer, enqueue-only form (x holds all n queries on the first shard's GPU / this
    /// rank's GPU; outputs on the same GPU): returns without a host synchronisation.
    void searchDeviceEnqueue(faiss::idx_t n, const float* x, faiss::idx_t k, float* distances,
                             faiss::idx_t* labels) const;
    /// Waits for every shard's stream; throws if a search reported a device-side error.
    void synchronize() const;

    int numShards() const;
    int rank() const;    ///< one process per GPU: this rank; else 0
    int world() const;   ///< one process per GPU: ranks in the group; else 1
    const B200IndexFlat* shard(int i) const;
    void setForcePath(int path);
    /// One process per GPU: searches of at most 8 queries with host buffers are replayed from a
    /// CUDA graph that holds the whole call, exchange included (default on).
    void setUseGraphs(bool on);
    /// Host-side trace of search() calls: per call, microseconds until everything was enqueued
    /// and microseconds waiting for the device after that.  setTrace clears the record.
    void setTrace(bool on);
    size_t readTrace(float* enqueueUs, float* waitUs, size_t capacity) const;   ///< returns the number recorded

   private:
    struct Impl;
    std::unique_ptr<Impl> impl_;
};

}  // namespace faiss_b200
