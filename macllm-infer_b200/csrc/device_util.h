// Small RAII helpers for device and pinned host memory.
#pragma once
#include "common.cuh"
#include <vector>

namespace mk {

class DevBuf {
public:
    DevBuf() = default;
    explicit DevBuf(size_t bytes) { alloc(bytes); }
    ~DevBuf() { release(); }
    DevBuf(const DevBuf&) = delete;
    DevBuf& operator=(const DevBuf&) = delete;
    DevBuf(DevBuf&& o) noexcept : p_(o.p_), n_(o.n_) { o.p_ = nullptr; o.n_ = 0; }
    DevBuf& operator=(DevBuf&& o) noexcept {
        if (this != &o) { release(); p_ = o.p_; n_ = o.n_; o.p_ = nullptr; o.n_ = 0; }
        return *this;
    }
    void alloc(size_t bytes) {
        release();
        if (bytes == 0) return;
        MK_CUDA(cudaMalloc(&p_, bytes));
        n_ = bytes;
    }
    void ensure(size_t bytes) { if (bytes > n_) alloc(bytes); }
    void release() { if (p_) cudaFree(p_); p_ = nullptr; n_ = 0; }
    void zero(cudaStream_t s = nullptr) { if (p_) MK_CUDA(cudaMemsetAsync(p_, 0, n_, s)); }
    template <typename T> T* as() const { return reinterpret_cast<T*>(p_); }
    void* ptr() const { return p_; }
    size_t size() const { return n_; }
    void upload(const void* src, size_t bytes, cudaStream_t s = nullptr) {
        ensure(bytes);
        if (bytes) MK_CUDA(cudaMemcpyAsync(p_, src, bytes, cudaMemcpyHostToDevice, s));
    }
    void download(void* dst, size_t bytes, cudaStream_t s = nullptr) const {
        if (bytes) MK_CUDA(cudaMemcpyAsync(dst, p_, bytes, cudaMemcpyDeviceToHost, s));
    }
private:
    void* p_ = nullptr;
    size_t n_ = 0;
};

class PinnedBuf {
public:
    PinnedBuf() = default;
    ~PinnedBuf() { if (p_) cudaFreeHost(p_); }
    PinnedBuf(const PinnedBuf&) = delete;
    PinnedBuf& operator=(const PinnedBuf&) = delete;
    void ensure(size_t bytes) {
        if (bytes <= n_) return;
        if (p_) cudaFreeHost(p_);
        p_ = nullptr;
        MK_CUDA(cudaMallocHost(&p_, bytes));
        n_ = bytes;
    }
    template <typename T> T* as() const { return reinterpret_cast<T*>(p_); }
    size_t size() const { return n_; }
private:
    void* p_ = nullptr;
    size_t n_ = 0;
};

// The f16 image of one weight matrix [rows][cols] plus the TMA descriptor of its 128-row x 64-column
// boxes (see hgemm_tc.h).  Built once at load time from the device copy of the quantised matrix.
struct HalfWeight {
    DevBuf values;               // rows * cols halves, row-major
    int64_t rows = 0, cols = 0;
    alignas(64) unsigned char tmap[128] = {};  // CUtensorMap (opaque here, 64-byte aligned)
    bool ready = false;
};

// A weight matrix uploaded to HBM in the layout the kernels read (see QWeight).
struct DeviceWeight {
    QWeight w;
    DevBuf b0, b1, b2, b3;
    HalfWeight half;  // optional second copy for wide batches
    int file_type = -1;  // the GGML type in the file when the matrix was decoded at load (w.type is then F32), else -1
};

// Upload `rows` x `cols` weights stored in GGUF block format `type` at host pointer `src`.
// Q6_K and Q8_0 blocks (210 and 34 bytes, only 2-byte aligned in the file) are split into aligned
// planes on the way; Q4_K and F32/F16 are uploaded as they are (F16 is widened to F32).
void upload_weight(int type, const void* src, int64_t rows, int64_t cols, DeviceWeight& out, cudaStream_t s = nullptr);

// Bytes of one row of `cols` weights in GGUF storage (src/gguf.rs:386-408 of the reference).
int64_t gguf_row_bytes(int type, int64_t cols);
// Block formats without a kernel of their own (Q4_0, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K, BF16): upload_weight decodes them on the
// host into a dense f32 matrix.  decode_rows_host is that decoder (host only, no GPU).
bool decoded_at_load(int type);
void decode_rows_host(int type, const void* src, int64_t rows, int64_t cols, float* out);
// llama.cpp stores Llama Q/K rows pair-interleaved per head; the loader puts them back in half-split order so that the
// half-split rotation applies: source row head*d + 2*pair + lane -> destination row head*d + lane*d/2 + pair, rows moved
// as opaque byte strings so block formats stay compressed (inverse_permute_quantized_rows, src/gguf.rs:1888-1924).
void unpermute_qk_rows_host(const uint8_t* src, int64_t rows, int64_t row_bytes, int heads, uint8_t* dst);

}  // namespace mk
