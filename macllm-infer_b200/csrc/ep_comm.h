// Expert-parallel communicator: one rank per GPU, NCCL over NVLink / NVSwitch.
//
// The reference serves a sparse-MoE model from one device and runs the experts one after another
// (SparseMoeFeedForward::forward, src/decoder.rs:394-441).  Here the expert banks can be split over `size` processes:
// every rank runs the same ticks on the same tokens, computes the contributions of the experts it holds, and the
// per-rank partial sums are exchanged with one all-gather per MoE layer and added in rank order, so that every rank
// ends the layer with the same bits.
//
// NCCL is resolved at run time (dlopen of libnccl.so.2), so the library loads on hosts without it and a
// single-GPU process never touches it.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace mk {

constexpr int kEpUniqueIdBytes = 128;

class EpComm {
public:
    // Rank 0 creates the id and hands it to the other ranks out of band (a file, a store, a socket).
    static void unique_id(uint8_t out[kEpUniqueIdBytes]);
    // Collective over all `size` ranks; the calling thread's current device is the rank's GPU.
    EpComm(int rank, int size, const uint8_t id[kEpUniqueIdBytes]);
    ~EpComm();
    EpComm(const EpComm&) = delete;
    EpComm& operator=(const EpComm&) = delete;

    int rank() const { return rank_; }
    int size() const { return size_; }
    // recv[r * count + i] = rank r's send[i], enqueued on `s`.
    void all_gather_f32(const float* send, float* recv, size_t count, cudaStream_t s);

private:
    void* comm_ = nullptr;
    int rank_ = 0, size_ = 1;
};

}  // namespace mk
