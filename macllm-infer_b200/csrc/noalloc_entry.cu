// An allocation-free variant of the tensor-core quantised matmul.
//
// Who needs it: hosts that embed this library inside a process whose GPU memory is owned by someone
// else - an inference server that hands out device buffers from its own arena and forbids cudaMalloc
// on the request path (an allocation there can stall every stream of the context or fragment the
// arena), or a plugin running inside a sandbox whose allocator hooks reject foreign allocations.  Such
// a caller can still pass device pointers for the weights, the activations and the result, but the
// kernel's own working storage (the 8-bit/f16 image of the activations, the split-K partial sums and
// the status word) has to live somewhere: here it lives in file-scope device arrays that are part of
// the library image, about 10 MiB on every GPU that loads the library, held until the process exits.
//
// Consequences the caller must know:
//   * sizes are capped (see the MK_NOALLOC_* constants); larger problems are refused with a message;
//   * every call uses the same arrays, which keep whatever the previous call left in them - the status
//     word is cleared at the start of each call, the rest is fully overwritten before it is read;
//   * two calls that overlap on the GPU (different streams, or different host threads) race on the
//     arrays and corrupt each other's results - serialise them;
//   * the first call on a device resolves the arrays' device addresses (cudaGetSymbolAddress with that
//     device current); make that first call before starting any stream capture;
//   * every call synchronises its stream and copies a status word back to the host before it returns.
#include "../../include/macllm_b200.h"
#include "c_api_util.h"
#include "kernels.h"
#include "qgemm_tc.h"
#include <mutex>

using namespace mk;

namespace {

constexpr size_t ACT_ELEMS = MK_NOALLOC_MAX_ACT_ELEMS;        // T * cols
constexpr size_t PARTIAL_FLOATS = MK_NOALLOC_MAX_PARTIAL;     // splits * T * rows
constexpr int MAX_DEVICES = 64;

// Working storage inside the library image.  In host code these names are only stand-ins for the
// symbols; the addresses a kernel can use come from cudaGetSymbolAddress below.
static __device__ __align__(256) int8_t g_act_qs[ACT_ELEMS];
static __device__ __align__(256) __half g_act_f16[ACT_ELEMS];
static __device__ __align__(256) float g_act_scale[ACT_ELEMS / 256];
static __device__ __align__(256) int16_t g_act_bsums[ACT_ELEMS / 16];
static __device__ __align__(256) float g_partial[PARTIAL_FLOATS];
static __device__ __align__(256) int32_t g_status[64];

struct Resolved {
    bool ready = false;
    int8_t* qs = nullptr;
    __half* f16 = nullptr;
    float* scale = nullptr;
    int16_t* bsums = nullptr;
    float* partial = nullptr;
    int32_t* status = nullptr;
};

Resolved g_resolved[MAX_DEVICES];
std::mutex g_resolve_mutex;

// Once per device, with that device current.
const Resolved& resolve_for_current_device() {
    int dev = -1;
    MK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) throw std::runtime_error("device ordinal out of range for the allocation-free entry point");
    std::lock_guard<std::mutex> lock(g_resolve_mutex);
    Resolved& r = g_resolved[dev];
    if (!r.ready) {
        MK_CUDA(cudaGetSymbolAddress((void**)&r.qs, g_act_qs));
        MK_CUDA(cudaGetSymbolAddress((void**)&r.f16, g_act_f16));
        MK_CUDA(cudaGetSymbolAddress((void**)&r.scale, g_act_scale));
        MK_CUDA(cudaGetSymbolAddress((void**)&r.bsums, g_act_bsums));
        MK_CUDA(cudaGetSymbolAddress((void**)&r.partial, g_partial));
        MK_CUDA(cudaGetSymbolAddress((void**)&r.status, g_status));
        r.ready = true;
    }
    return r;
}

}  // namespace

extern "C" int32_t mk_k_q4k_matmul_tc_noalloc_dev(const void* w_q4k_dev, int64_t rows, int64_t cols, const float* x_dev, int32_t T,
                                                  float* y_dev, void* cuda_stream) {
    return guarded([&] {
        require_device();
        if (w_q4k_dev == nullptr || x_dev == nullptr || y_dev == nullptr) throw std::runtime_error("mk_k_q4k_matmul_tc_noalloc_dev: null pointer");
        if (rows <= 0 || T <= 0 || cols <= 0 || cols % 256 != 0)
            throw std::runtime_error("mk_k_q4k_matmul_tc_noalloc_dev: rows and T must be positive and cols a positive multiple of 256");
        if (rows > INT32_MAX) throw std::runtime_error("mk_k_q4k_matmul_tc_noalloc_dev: rows must fit a 32-bit integer");
        if (((uintptr_t)w_q4k_dev & 15) != 0) throw std::runtime_error("mk_k_q4k_matmul_tc_noalloc_dev: weights must be 16-byte aligned");
        if ((size_t)T * (size_t)cols > ACT_ELEMS)
            throw std::runtime_error("mk_k_q4k_matmul_tc_noalloc_dev: T * cols = " + std::to_string((size_t)T * cols) +
                                     " exceeds the built-in activation scratch of " + std::to_string(ACT_ELEMS) + " elements");
        QWeight W;
        W.type = QT_Q4_K;
        W.rows = rows;
        W.cols = cols;
        W.p0 = w_q4k_dev;
        W.bytes = rows * (cols / 256) * 144;
        size_t need = qgemm_tc_partial_floats(W, T);
        if (need > PARTIAL_FLOATS)
            throw std::runtime_error("mk_k_q4k_matmul_tc_noalloc_dev: the split-K partial sums need " + std::to_string(need) +
                                     " floats, more than the built-in scratch of " + std::to_string(PARTIAL_FLOATS));
        const Resolved& r = resolve_for_current_device();
        cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
        MK_CUDA(cudaMemsetAsync(r.status, 0, sizeof(int32_t), s));  // the only word that must start at zero
        ActQ act;
        act.qs = r.qs;
        act.d = r.scale;
        act.bsums = r.bsums;
        act.xh = r.f16;
        NormQuantArgs q;
        q.h = const_cast<float*>(x_dev);  // read only: no residual, no norm, no write-back
        q.rows = T;
        q.dim = (int)cols;
        q.act_kind = ACT_Q8K;
        q.out = act;
        launch_add_norm_quant(q, s);
        launch_qgemm_tc_scratch(W, act, T, y_dev, (int)rows, 1.0f, 0.f, r.partial, r.status, s);
        int32_t status = 0;
        MK_CUDA(cudaMemcpyAsync(&status, r.status, sizeof status, cudaMemcpyDeviceToHost, s));
        MK_CUDA(cudaStreamSynchronize(s));
        if (status != 0) throw std::runtime_error("mk_k_q4k_matmul_tc_noalloc_dev: a bounded wait inside the kernel gave up (status " + std::to_string(status) + ")");
    });
}
