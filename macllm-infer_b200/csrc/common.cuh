// Shared definitions for the sm_100a kernels of the continuous-batching step.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <cstdio>
#include <string>
#include <stdexcept>
#include <cstdlib>
#include <utility>

namespace mk {

// GGML tensor type ids as stored in GGUF files (the reference's src/gguf.rs:283-297 table).
// GGML tensor types (src/gguf.rs:283-345 of the reference).  The kernels read F32, Q8_0, Q4_K and Q6_K in place; the other
// block formats are decoded once at load into a dense matrix (weights.cpp) and served by the dense f16 GEMM.
enum QType : int { QT_F32 = 0, QT_F16 = 1, QT_Q4_0 = 2, QT_Q5_0 = 6, QT_Q5_1 = 7, QT_Q8_0 = 8, QT_Q2_K = 10, QT_Q3_K = 11, QT_Q4_K = 12,
                   QT_Q5_K = 13, QT_Q6_K = 14, QT_BF16 = 30 };

// Activation block formats produced by the quantising kernels.
enum ActKind : int { ACT_Q8K = 0, ACT_Q80 = 1 };

// A weight matrix [rows = out, cols = in] resident in HBM.
//  Q4_K : p0 = raw 144-byte blocks, row-major (16-byte aligned, header 16 B + 128 B of nibbles)
//  Q6_K : split into aligned planes: p0 = ql [rows*nb][128], p1 = qh [rows*nb][64],
//         p2 = scales [rows*nb][16] (int8), p3 = d [rows*nb] (f16)
//  Q8_0 : p0 = qs [rows][cols] (int8), p1 = d [rows][cols/32] (f16)
//  F32  : p0 = values
struct QWeight {
    int type = QT_F32;
    int64_t rows = 0, cols = 0;
    const void* p0 = nullptr;
    const void* p1 = nullptr;
    const void* p2 = nullptr;
    const void* p3 = nullptr;
    int64_t bytes = 0;  // algorithmic bytes of the matrix as stored in the file
};

// Quantised activations for T rows of width K.
//  ACT_Q8K: qs [T][K] int8, d [T][K/256] f32, bsums [T][K/16] int16
//  ACT_Q80: qs [T][K] int8, d [T][K/32] f32 (value already rounded through f16), bsums unused
//  xh (optional): [T][K] f16, the dequantised activation d*q rounded once - the operand of the
//  tensor-core path, so both paths multiply the weights by the same quantised activations.
struct ActQ {
    int8_t* qs = nullptr;
    float* d = nullptr;
    int16_t* bsums = nullptr;
    __half* xh = nullptr;
};

struct CudaError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

inline void cuda_check(cudaError_t e, const char* what, const char* file, int line) {
    if (e != cudaSuccess) {
        char buf[512];
        snprintf(buf, sizeof buf, "%s failed: %s (%s:%d)", what, cudaGetErrorString(e), file, line);
        throw CudaError(buf);
    }
}
#define MK_CUDA(x) ::mk::cuda_check((x), #x, __FILE__, __LINE__)
#define MK_LAUNCH_CHECK() ::mk::cuda_check(cudaGetLastError(), "kernel launch", __FILE__, __LINE__)

// Index of the (block, layer) page of a paged KV pool whose pages are [kv_heads][block_tokens][head_dim].
// pool_blocks > 0: layer-major pool [layers][pool_blocks] - one layer's pages are contiguous, so the attention
// of a layer walks one compact region (this is how the model lays its pools out); pool_blocks == 0: block-major
// pool [blocks][layers] (the layout of host-provided pools in the kernel-level entry points).
__host__ __device__ __forceinline__ int64_t kv_page_index(int64_t blk, int layer, int layers, int64_t pool_blocks) {
    return pool_blocks > 0 ? (int64_t)layer * pool_blocks + blk : blk * layers + layer;
}

// Programmatic dependent launch: a kernel launched through launch_pdl may start (be scheduled, run its
// prologue) while the previous kernel of the stream is still running; pdl_wait() blocks until that kernel has
// completed and its writes are visible, so it must precede the first access to anything the predecessor wrote
// or still reads.  pdl_trigger() lets the next kernel of the stream begin its own launch early.  Both are no-ops
// for kernels launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device attribute of a kernel: opt `func` in for `bytes` of
// dynamic shared memory on the current device, once per (kernel, device) and again only when more is asked for.
// Safe to call from several host threads.
void ensure_dynamic_smem(const void* func, size_t bytes);
// Streaming multiprocessors of the current device (cached per device).
int device_sm_count();

#ifdef __CUDACC__
inline bool pdl_enabled() {
    static const bool on = [] { const char* e = std::getenv("MACLLM_B200_PDL"); return e == nullptr || e[0] != '0'; }();
    return on;
}
// Launch `kernel`, which calls pdl_wait() before it touches global memory, with programmatic stream serialisation.
template <typename... Params, typename... Args>
inline void launch_pdl(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    cuda_check(cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...), "kernel launch", __FILE__, __LINE__);
}
#endif

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum for blockDim.x <= 1024 (multiple of 32); `red` is 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

}  // namespace mk
