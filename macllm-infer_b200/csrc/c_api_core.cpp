// C ABI, part 0: error slot, version, device probe, and the host-only helpers that need no GPU.
#include "../../include/macllm_b200.h"
#include "c_api_util.h"
#include "seed_model.h"
#include "device_util.h"
#include "sha256.h"
#include "host_sampler.h"
#include <cstring>

namespace mk {

std::string& last_error_slot() {
    static thread_local std::string slot;
    return slot;
}

void require_device() {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        cudaGetLastError();
        throw std::runtime_error("no usable CUDA device: this library has no CPU fallback");
    }
}

}  // namespace mk

using namespace mk;

extern "C" {

const char* mk_last_error(void) { return last_error_slot().c_str(); }

const char* mk_version(void) { return "macllm_b200 0.1 (sm_100a)"; }

int32_t mk_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int32_t mk_sha256(const uint8_t* data, int64_t n, uint8_t out[32]) {
    return guarded([&] {
        Sha256 h;
        h.update(data, (size_t)n);
        auto d = h.finish();
        memcpy(out, d.data(), 32);
    });
}

int32_t mk_seed_tensor(uint64_t seed, uint64_t stream, float std_dev, int32_t type, int64_t rows, int64_t cols, void* out) {
    return guarded([&] { seed_tensor(seed, stream, std_dev, type, rows, cols, out); });
}

int64_t mk_row_bytes(int32_t type, int64_t cols) { return seed_row_bytes(type, cols); }

int32_t mk_decode_rows(int32_t type, const void* src, int64_t rows, int64_t cols, float* out) {
    return guarded([&] {
        if (src == nullptr || out == nullptr || rows <= 0 || cols <= 0) throw std::runtime_error("mk_decode_rows: bad arguments");
        decode_rows_host(type, src, rows, cols, out);
    });
}

int32_t mk_unpermute_qk_rows(const void* src, int64_t rows, int64_t row_bytes, int32_t heads, void* dst) {
    return guarded([&] {
        if (src == nullptr || dst == nullptr || row_bytes <= 0) throw std::runtime_error("mk_unpermute_qk_rows: bad arguments");
        unpermute_qk_rows_host(static_cast<const uint8_t*>(src), rows, row_bytes, heads, static_cast<uint8_t*>(dst));
    });
}

int32_t mk_host_sample_greedy(float* logits, int32_t vocab, const uint32_t* history, int32_t n_history, float repetition_penalty,
                              const uint32_t* generated, int32_t n_generated, float presence_penalty, float frequency_penalty,
                              uint32_t* token) {
    return guarded([&] {
        apply_penalties(logits, vocab, history, n_history, repetition_penalty, generated, n_generated, presence_penalty,
                        frequency_penalty);
        *token = (uint32_t)argmax_first(logits, vocab);
    });
}

}  // extern "C"
