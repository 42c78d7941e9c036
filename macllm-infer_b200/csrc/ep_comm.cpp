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
    if (comm_ != nullptr) nccl().CommDestroy(static_cast<ncclComm_t>(comm_));
}

void EpComm::all_gather_f32(const float* send, float* recv, size_t count, cudaStream_t s) {
    check(nccl().AllGather(send, recv, count, ncclFloat32, static_cast<ncclComm_t>(comm_), s), "ncclAllGather");
}

}  // namespace mk
