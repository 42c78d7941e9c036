// On-device token selection and MoE routing.
//
// Greedy selection restates argmax of src/sampling.rs:425-433: a total order on f32 bit patterns,
// the earliest index winning ties.  The reference reads the whole [lanes, vocab] logits back to the
// host every tick (src/engine.rs:2388-2392); here only one u32 per lane crosses PCIe.
// Routing restates selected_softmax_routes (src/decoder.rs:448-554): the k largest router logits in
// (value descending, index ascending) order, then a softmax over those k only.
#include "kernels.h"

namespace mk {

namespace {

__device__ __forceinline__ int total_key(float f) {
    int b = __float_as_int(f);
    return b ^ (int)(((unsigned)(b >> 31)) >> 1);
}

// grid (rows, chunks): every CTA scans one chunk of one row, folds its best (key, index) into the row's packed
// 64-bit slot with atomicMax (key in the high word, 2^32-1 - index in the low word, so the larger packed value
// is the larger key and, among equal keys, the lower index - an order-independent reduction), and the CTA that
// arrives last at the row's counter writes the token and restores slot and counter to zero for the next call.
constexpr int ARGMAX_THREADS = 256;
constexpr int ARGMAX_CHUNKS = 16;

__global__ void __launch_bounds__(ARGMAX_THREADS) argmax_kernel(const float* logits, int vocab, uint32_t* out,
                                                                unsigned long long* slots, int32_t* counters) {
    __shared__ unsigned long long s_best[ARGMAX_THREADS / 32];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const float* row = logits + (int64_t)r * vocab;
    const int per = ((vocab + gridDim.y - 1) / gridDim.y + 3) / 4 * 4;
    const int lo = blockIdx.y * per, hi = min(vocab, lo + per);
    unsigned long long best = 0;
    auto consider = [&](float f, int i) {
        unsigned long long p = ((unsigned long long)((uint32_t)total_key(f) ^ 0x80000000u) << 32) | (0xFFFFFFFFu - (uint32_t)i);
        best = p > best ? p : best;
    };
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        int i = lo + threadIdx.x * 4;
        for (; i + 3 < hi; i += ARGMAX_THREADS * 4) {
            float4 v = *reinterpret_cast<const float4*>(row + i);
            consider(v.x, i);
            consider(v.y, i + 1);
            consider(v.z, i + 2);
            consider(v.w, i + 3);
        }
        for (; i < hi; ++i) consider(row[i], i);  // at most one ragged group per row, in the last chunk
    } else {
        for (int i = lo + threadIdx.x; i < hi; i += ARGMAX_THREADS) consider(row[i], i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) s_best[w] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int k = 1; k < ARGMAX_THREADS / 32; ++k) best = s_best[k] > best ? s_best[k] : best;
        atomicMax(&slots[r], best);
        __threadfence();
        int prev = atomicAdd(&counters[r], 1);
        if (prev == (int)gridDim.y - 1) {
            __threadfence();
            unsigned long long win = atomicExch(&slots[r], 0ull);
            counters[r] = 0;
            out[r] = 0xFFFFFFFFu - (uint32_t)(win & 0xFFFFFFFFull);
        }
    }
}

// One warp per token row; experts <= 1024.  Repeated selection of the best remaining candidate.
__global__ void __launch_bounds__(128) moe_route_kernel(const float* logits, int T, int experts, int k,
                                                        int32_t* sel_experts, float* sel_weights) {
    int t = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (t >= T) return;
    int lane = threadIdx.x & 31;
    const float* row = logits + (int64_t)t * experts;
    constexpr int MAX_PER_LANE = 32;
    float v[MAX_PER_LANE];
    int cnt = 0;
    for (int e = lane; e < experts && cnt < MAX_PER_LANE; e += 32, ++cnt) v[cnt] = row[e];
    unsigned taken = 0;  // bit c set when this lane's c-th candidate was selected
    float mx = -INFINITY;
    for (int i = 0; i < k; ++i) {
        float bv = -INFINITY;
        int be = INT_MAX;
        for (int c = 0; c < cnt; ++c) {
            if (taken >> c & 1u) continue;
            int e = lane + 32 * c;
            if (v[c] > bv || (v[c] == bv && e < be)) { bv = v[c]; be = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (oe != INT_MAX && (be == INT_MAX || ov > bv || (ov == bv && oe < be))) { bv = ov; be = oe; }
        }
        if ((be & 31) == lane) taken |= 1u << (be >> 5);
        if (i == 0) mx = bv;  // the first pick is the maximum of the selected set
        if (lane == 0) { sel_experts[(int64_t)t * k + i] = be; sel_weights[(int64_t)t * k + i] = bv; }
    }
    __syncwarp();
    // softmax over the selected logits: exp(l - max) / sum in selection order
    if (lane == 0) {
        float den = 0.f;
        for (int i = 0; i < k; ++i) den += expf(sel_weights[(int64_t)t * k + i] - mx);
        for (int i = 0; i < k; ++i) sel_weights[(int64_t)t * k + i] = expf(sel_weights[(int64_t)t * k + i] - mx) / den;
    }
}

}  // namespace

size_t argmax_scratch_bytes(int B) { return (size_t)B * 16; }

void launch_argmax(const float* logits, int B, int vocab, uint32_t* out, void* scratch, cudaStream_t s) {
    if (B <= 0) return;
    unsigned long long* slots = reinterpret_cast<unsigned long long*>(scratch);
    int32_t* counters = reinterpret_cast<int32_t*>(slots + B);
    int chunks = vocab >= 4096 ? ARGMAX_CHUNKS : 1;
    dim3 grid((unsigned)B, (unsigned)chunks);
    launch_pdl(argmax_kernel, grid, dim3(ARGMAX_THREADS), 0, s, logits, vocab, out, slots, counters);
    MK_LAUNCH_CHECK();
}

void launch_moe_route(const float* logits, int T, int experts, int k, int32_t* sel_experts, float* sel_weights,
                      cudaStream_t s) {
    if (T <= 0) return;
    if (experts > 1024) throw std::runtime_error("launch_moe_route: more than 1024 experts");
    moe_route_kernel<<<(T + 3) / 4, 128, 0, s>>>(logits, T, experts, k, sel_experts, sel_weights);
    MK_LAUNCH_CHECK();
}

}  // namespace mk
