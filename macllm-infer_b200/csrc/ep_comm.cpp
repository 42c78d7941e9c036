// NCCL binding of the expert-parallel communicator (see ep_comm.h).
#include "ep_comm.h"

#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>

namespace mk {

namespace {

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

template <class F>
void bind(void* lib, const char* name, F& fn) {
    fn = reinterpret_cast<F>(dlsym(lib, name));
    if (fn == nullptr) throw std::runtime_error(std::string("libnccl.so.2 has no symbol ") + name);
}

const NcclApi& nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        // a copy the process already holds (for instance the one bundled with a Python package) wins over the system's
        void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
        if (lib == nullptr) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (lib == nullptr) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
        if (lib == nullptr) throw std::runtime_error("expert parallelism needs NCCL: libnccl.so.2 could not be loaded");
        bind(lib, "ncclGetUniqueId", api.GetUniqueId);
        bind(lib, "ncclCommInitRank", api.CommInitRank);
        bind(lib, "ncclCommDestroy", api.CommDestroy);
        bind(lib, "ncclAllGather", api.AllGather);
        bind(lib, "ncclGetErrorString", api.GetErrorString);
    });
    return api;
}

void check(ncclResult_t r, const char* what) {
    if (r != ncclSuccess) throw std::runtime_error(std::string(what) + ": " + nccl().GetErrorString(r));
}

static_assert(sizeof(ncclUniqueId) == kEpUniqueIdBytes, "NCCL unique id size");

}  // namespace

void EpComm::unique_id(uint8_t out[kEpUniqueIdBytes]) {
    ncclUniqueId id;
    check(nccl().GetUniqueId(&id), "ncclGetUniqueId");
    memcpy(out, &id, sizeof id);
}

EpComm::EpComm(int rank, int size, const uint8_t id_bytes[kEpUniqueIdBytes]) : rank_(rank), size_(size) {
    if (size < 2 || rank < 0 || rank >= size) throw std::runtime_error("expert-parallel rank / size out of range");
    ncclUniqueId id;
    memcpy(&id, id_bytes, sizeof id);
    ncclComm_t c = nullptr;
    check(nccl().CommInitRank(&c, size, id, rank), "ncclCommInitRank");
    comm_ = c;
}

EpComm::~EpComm() {
    for (void* p : mapped_)
        if (p != nullptr) cudaIpcCloseMemHandle(p);
    for (void* p : dispatch_mapped_)
        if (p != nullptr) cudaIpcCloseMemHandle(p);
    if (exchange_ != nullptr) cudaFree(exchange_);
    if (dispatch_block_ != nullptr) cudaFree(dispatch_block_);
    if (comm_ != nullptr) nccl().CommDestroy(static_cast<ncclComm_t>(comm_));
}

namespace {
void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        cudaGetLastError();
        throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
    }
}
}  // namespace

void* EpComm::open_block(size_t bytes, cudaStream_t s, void* (&bases)[kEpMaxRanks], void* (&mapped)[kEpMaxRanks]) {
    if (size_ > kEpMaxRanks) throw std::runtime_error("the expert exchange serves at most 8 ranks");
    void* block = nullptr;
    cuda_check(cudaMalloc(&block, bytes), "cudaMalloc of an expert exchange block");
    cuda_check(cudaMemsetAsync(block, 0, bytes, s), "cudaMemsetAsync");
    // the handles travel through the communicator itself; nobody can store into a block before its owner has
    // zeroed it, because the owner's all-gather is ordered after the memset on the same stream
    cudaIpcMemHandle_t mine;
    cuda_check(cudaIpcGetMemHandle(&mine, block), "cudaIpcGetMemHandle");
    static_assert(sizeof(cudaIpcMemHandle_t) % 4 == 0, "handle size");
    constexpr size_t HF = sizeof(cudaIpcMemHandle_t) / 4;
    float* stage = nullptr;
    cuda_check(cudaMalloc(&stage, (size_t)(size_ + 1) * HF * 4), "cudaMalloc");
    cudaIpcMemHandle_t all[kEpMaxRanks];
    try {
        cuda_check(cudaMemcpyAsync(stage, &mine, sizeof mine, cudaMemcpyHostToDevice, s), "cudaMemcpyAsync");
        all_gather_f32(stage, stage + HF, HF, s);
        cuda_check(cudaMemcpyAsync(all, stage + HF, (size_t)size_ * sizeof mine, cudaMemcpyDeviceToHost, s), "cudaMemcpyAsync");
        cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    } catch (...) {
        cudaFree(stage);
        throw;
    }
    cudaFree(stage);
    for (int p = 0; p < size_; ++p) {
        void* base = block;
        if (p != rank_) {
            cuda_check(cudaIpcOpenMemHandle(&base, all[p], cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle of a peer's expert exchange block");
            mapped[p] = base;
        }
        bases[p] = base;
    }
    // leave together: once this returns, every rank has mapped every block
    float* fence = nullptr;
    cuda_check(cudaMalloc(&fence, (size_t)(size_ + 1) * 4), "cudaMalloc");
    try {
        all_gather_f32(fence, fence + 1, 1, s);
        cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    } catch (...) {
        cudaFree(fence);
        throw;
    }
    cudaFree(fence);
    return block;
}

void EpComm::open_exchange(int max_tokens, int row_floats, cudaStream_t s) {
    if (exchange_ != nullptr) throw std::runtime_error("expert exchange opened twice");
    const int64_t slot_floats = (int64_t)max_tokens * row_floats;
    const size_t gather_bytes = (size_t)2 * size_ * slot_floats * 4;
    const size_t flag_bytes = (size_t)2 * size_ * max_tokens * 4;
    void* bases[kEpMaxRanks] = {};
    exchange_ = open_block(gather_bytes + flag_bytes, s, bases, mapped_);
    peers_ = EpPeers{};
    peers_.rank = rank_;
    peers_.ranks = size_;
    peers_.max_tokens = max_tokens;
    peers_.slot_floats = slot_floats;
    for (int p = 0; p < size_; ++p) {
        peers_.gather[p] = static_cast<float*>(bases[p]);
        peers_.flags[p] = reinterpret_cast<uint32_t*>(static_cast<char*>(bases[p]) + gather_bytes);
    }
}

void EpComm::open_dispatch(int64_t cap_rows, int hidden, int local_experts, cudaStream_t s) {
    if (dispatch_block_ != nullptr) throw std::runtime_error("expert dispatch exchange opened twice");
    if (hidden % 8 != 0 || cap_rows <= 0 || local_experts <= 0) throw std::runtime_error("expert dispatch exchange: bad geometry");
    auto up = [](int64_t v) { return (v + 255) / 256 * 256; };
    EpDispatch d;
    d.rank = rank_;
    d.ranks = size_;
    d.local_experts = local_experts;
    d.hidden = hidden;
    d.cap_rows = cap_rows;
    int64_t at = 0;
    d.rows_in_off = at;
    at = up(at + (int64_t)2 * size_ * cap_rows * hidden * 2);
    d.off_in_off = at;
    at = up(at + (int64_t)2 * size_ * (local_experts + 1) * 4);
    d.flag_in_off = at;
    at = up(at + (int64_t)2 * size_ * 4);
    d.out_back_off = at;
    at = up(at + (int64_t)2 * cap_rows * hidden * 4);
    d.flag_back_off = at;
    at = up(at + (int64_t)2 * size_ * 4);
    void* bases[kEpMaxRanks] = {};
    dispatch_block_ = open_block((size_t)at, s, bases, dispatch_mapped_);
    for (int p = 0; p < size_; ++p) d.base[p] = static_cast<uint8_t*>(bases[p]);
    dispatch_ = d;
}

void EpComm::all_gather_f32(const float* send, float* recv, size_t count, cudaStream_t s) {
    check(nccl().AllGather(send, recv, count, ncclFloat32, static_cast<ncclComm_t>(comm_), s), "ncclAllGather");
}

}  // namespace mk
