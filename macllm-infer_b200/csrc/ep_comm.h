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
constexpr int kEpMaxRanks = 8;

// The exchange area of the fused combine kernel, as every rank sees it.  Each rank owns one cudaMalloc'd block, mapped
// into the other processes through CUDA IPC (NVLink peer stores land in it):
//   gather[p]: rank p's block viewed as floats [2][ranks][slot_floats]: buffer b, slot q holds rank q's partial rows
//   flags[p]:  rank p's block viewed as u32    [2][ranks][max_tokens]:  the epoch in which slot q's row t was filled
// gather[rank] / flags[rank] are this process's own block.
struct EpPeers {
    float* gather[kEpMaxRanks] = {};
    uint32_t* flags[kEpMaxRanks] = {};
    int rank = 0, ranks = 1, max_tokens = 0;
    int64_t slot_floats = 0;
};

// The exchange area of expert parallelism with data-parallel lanes (see ep_dispatch.cu), as every rank sees it: base[p]
// is rank p's block (this rank's own for p = rank; the others mapped through CUDA IPC).  Inside a block, for buffer
// b = epoch & 1:
//   rows_in   f16 [2][ranks][cap_rows][hidden]  rows sent by each source for this rank's experts
//   off_in    i32 [2][ranks][local_experts + 1] the source's own positions of those rows, per local expert
//   flag_in   u32 [2][ranks]                    epoch in which the source's rows were complete
//   out_back  f32 [2][cap_rows][hidden]         expert outputs of this rank's routed rows, in its own grouped order
//   flag_back u32 [2][ranks]                    epoch in which a destination's outputs were complete
struct EpDispatch {
    uint8_t* base[kEpMaxRanks] = {};
    int rank = 0, ranks = 1, local_experts = 0, hidden = 0;
    int64_t cap_rows = 0;
    int64_t rows_in_off = 0, off_in_off = 0, flag_in_off = 0, out_back_off = 0, flag_back_off = 0;
};

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

    // Collective: allocates this rank's exchange block for `max_tokens` rows of `row_floats` floats, publishes its IPC
    // handle to the other ranks (through an all-gather) and maps theirs.  Throws when a peer's block cannot be mapped.
    void open_exchange(int max_tokens, int row_floats, cudaStream_t s);
    bool has_exchange() const { return exchange_ != nullptr; }
    // Collective: the same for the dispatch / return exchange of data-parallel lanes: every source may send up to cap_rows
    // rows of `hidden` halves to every destination per exchange.
    void open_dispatch(int64_t cap_rows, int hidden, int local_experts, cudaStream_t s);
    bool has_dispatch() const { return dispatch_block_ != nullptr; }
    const EpDispatch& dispatch() const { return dispatch_; }
    const EpPeers& peers() const { return peers_; }
    // Every rank calls this once per exchange, in the same order: the epoch names the exchange, its parity the buffer.
    uint32_t next_epoch() { return ++epoch_; }

private:
    void* comm_ = nullptr;
    int rank_ = 0, size_ = 1;
    // Collective: allocates and zeroes `bytes` on this rank, exchanges the IPC handles, maps the peers' blocks and
    // returns once every rank has mapped every block.
    void* open_block(size_t bytes, cudaStream_t s, void* (&bases)[kEpMaxRanks], void* (&mapped)[kEpMaxRanks]);
    void* exchange_ = nullptr;
    void* mapped_[kEpMaxRanks] = {};
    void* dispatch_block_ = nullptr;
    void* dispatch_mapped_[kEpMaxRanks] = {};
    EpDispatch dispatch_;
    EpPeers peers_;
    uint32_t epoch_ = 0;
};

}  // namespace mk
