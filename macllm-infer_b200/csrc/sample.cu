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

__global__ void __launch_bounds__(1024) argmax_kernel(const float* logits, int vocab, uint32_t* out) {
    __shared__ int s_key[32];
    __shared__ int s_idx[32];
    const float* row = logits + (int64_t)blockIdx.x * vocab;
    int best_key = INT_MIN, best_idx = INT_MAX;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        int k = total_key(row[i]);
        if (k > best_key || (k == best_key && i < best_idx)) { best_key = k; best_idx = i; }
    }
    auto better = [](int k1, int i1, int k2, int i2) { return k1 > k2 || (k1 == k2 && i1 < i2); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        int ok = __shfl_xor_sync(0xffffffffu, best_key, o);
        int oi = __shfl_xor_sync(0xffffffffu, best_idx, o);
        if (better(ok, oi, best_key, best_idx)) { best_key = ok; best_idx = oi; }
    }
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) { s_key[w] = best_key; s_idx[w] = best_idx; }
    __syncthreads();
    if (w == 0) {
        int nw = blockDim.x >> 5;
        best_key = lane < nw ? s_key[lane] : INT_MIN;
        best_idx = lane < nw ? s_idx[lane] : INT_MAX;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            int ok = __shfl_xor_sync(0xffffffffu, best_key, o);
            int oi = __shfl_xor_sync(0xffffffffu, best_idx, o);
            if (better(ok, oi, best_key, best_idx)) { best_key = ok; best_idx = oi; }
        }
        if (lane == 0) out[blockIdx.x] = (uint32_t)best_idx;
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

void launch_argmax(const float* logits, int B, int vocab, uint32_t* out, cudaStream_t s) {
    if (B <= 0) return;
    argmax_kernel<<<B, 1024, 0, s>>>(logits, vocab, out);
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
