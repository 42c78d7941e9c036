// Sparse-MoE dispatch helpers around the expert-grouped matmuls.
//
// The reference runs the experts one after another on index-selected rows and index_adds each
// weighted contribution back (SparseMoeFeedForward::forward, src/decoder.rs:394-441).  Here the
// (token, choice) pairs of the whole batch are grouped by expert once, the grouped matmul kernels
// walk each expert's rows, and the combine kernel adds a token's contributions in ascending expert
// order - the order index_add produces - so the sum is bit-identical for identical contributions.
#include "kernels.h"

namespace mk {

namespace {

constexpr int MAX_EXPERTS = 1024;

// One CTA.  Counting sort of pairs by expert; positions inside an expert follow pair order.
__global__ void __launch_bounds__(1024) moe_group_kernel(const int32_t* sel, int pairs, int k, int experts, int32_t* offsets,
                                                         int32_t* pos_of_pair, int32_t* token_of_pos) {
    __shared__ int32_t count[MAX_EXPERTS];
    __shared__ int32_t start[MAX_EXPERTS + 1];
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&count[sel[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < experts; ++e) { start[e] = acc; acc += count[e]; }
        start[experts] = acc;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = start[e];
    // deterministic placement: expert e's positions are assigned in increasing pair order by one thread per expert
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        if (count[e] == 0) continue;
        int pos = start[e];
        for (int p = 0; p < pairs; ++p) {
            if (sel[p] == e) {
                pos_of_pair[p] = pos;
                token_of_pos[pos] = p / k;
                ++pos;
            }
        }
    }
}

// Only choices whose expert lies in [e_lo, e_hi) contribute (the whole range on one GPU, a rank's share under
// expert parallelism).
__global__ void moe_combine_kernel(const float* expert_out, const int32_t* sel, const float* w, const int32_t* pos_of_pair, int k,
                                   int hidden, int e_lo, int e_hi, float* out) {
    int t = blockIdx.x;
    // choices sorted by expert index (k <= 32)
    __shared__ int order[32];
    if (threadIdx.x == 0) {
        for (int i = 0; i < k; ++i) order[i] = i;
        for (int i = 1; i < k; ++i) {
            int o = order[i], j = i - 1;
            while (j >= 0 && sel[t * k + order[j]] > sel[t * k + o]) { order[j + 1] = order[j]; --j; }
            order[j + 1] = o;
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float acc = 0.f;
        for (int i = 0; i < k; ++i) {
            int choice = order[i];
            int e = sel[t * k + choice];
            if (e < e_lo || e >= e_hi) continue;
            float v = expert_out[(int64_t)pos_of_pair[t * k + choice] * hidden + c];
            acc = __fadd_rn(acc, __fmul_rn(v, w[t * k + choice]));
        }
        out[(int64_t)t * hidden + c] = acc;
    }
}

// out[i] = ((g[0][i] + g[1][i]) + g[2][i]) + ... : the same order on every rank, so every rank gets the same bits.
__global__ void ep_sum_kernel(const float4* gathered, int ranks, int64_t count4, float4* out) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count4; i += (int64_t)gridDim.x * blockDim.x) {
        float4 a = gathered[i];
        for (int r = 1; r < ranks; ++r) {
            float4 b = gathered[(int64_t)r * count4 + i];
            a.x = __fadd_rn(a.x, b.x);
            a.y = __fadd_rn(a.y, b.y);
            a.z = __fadd_rn(a.z, b.z);
            a.w = __fadd_rn(a.w, b.w);
        }
        out[i] = a;
    }
}

}  // namespace

void launch_moe_group(const int32_t* sel_experts, int T, int k, int experts, int32_t* offsets, int32_t* pos_of_pair,
                      int32_t* token_of_pos, cudaStream_t s) {
    if (T <= 0) return;
    if (experts > MAX_EXPERTS) throw std::runtime_error("launch_moe_group: more than 1024 experts");
    moe_group_kernel<<<1, 1024, 0, s>>>(sel_experts, T * k, k, experts, offsets, pos_of_pair, token_of_pos);
    MK_LAUNCH_CHECK();
}

void launch_moe_combine(const float* expert_out, const int32_t* sel_experts, const float* sel_weights,
                        const int32_t* pos_of_pair, int T, int k, int hidden, int e_lo, int e_hi, float* out, cudaStream_t s) {
    if (T <= 0) return;
    if (k > 32) throw std::runtime_error("launch_moe_combine: more than 32 experts per token");
    moe_combine_kernel<<<T, 256, 0, s>>>(expert_out, sel_experts, sel_weights, pos_of_pair, k, hidden, e_lo, e_hi, out);
    MK_LAUNCH_CHECK();
}

void launch_ep_sum(const float* gathered, int ranks, int64_t count, float* out, cudaStream_t s) {
    if (count <= 0) return;
    if (count % 4 != 0) throw std::runtime_error("launch_ep_sum: count must be a multiple of 4");
    int64_t c4 = count / 4;
    int grid = (int)std::min<int64_t>((c4 + 255) / 256, 148 * 8);
    ep_sum_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const float4*>(gathered), ranks, c4, reinterpret_cast<float4*>(out));
    MK_LAUNCH_CHECK();
}

}  // namespace mk
