// Sparse-MoE dispatch helpers around the expert-grouped matmuls.
//
// The reference runs the experts one after another on index-selected rows and index_adds each
// weighted contribution back (SparseMoeFeedForward::forward, src/decoder.rs:394-441).  Here the
// (token, choice) pairs of the whole batch are grouped by expert once, the grouped matmul kernels
// walk each expert's rows, and the combine kernel adds a token's contributions in ascending expert
// order - the order index_add produces - so the sum is bit-identical for identical contributions.
#include "kernels.h"

#include <climits>

namespace mk {

namespace {

constexpr int MAX_EXPERTS = 1024;

// Counting sort of the (token, choice) pairs by expert; positions inside an expert follow pair order.  CTA b owns the
// experts [32 b, 32 b + 32), one warp each.  Every CTA counts all experts for itself (the start of its own experts needs
// the counts of all earlier ones); then each warp walks the pairs 32 at a time and gives the pairs of its expert their
// positions from a ballot: the rank of a pair among its expert's pairs is the number of earlier pairs of that expert.
__global__ void __launch_bounds__(1024) moe_group_kernel(const int32_t* __restrict__ sel, int pairs, int k, int experts, int32_t* offsets,
                                                         int32_t* pos_of_pair, int32_t* token_of_pos) {
    __shared__ int32_t count[MAX_EXPERTS];
    __shared__ int32_t start[MAX_EXPERTS + 1];
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    // a choice outside [0, experts) cannot come from the routing kernel; if one ever does it is left out of every group
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = sel[p];
        if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
        else if (blockIdx.x == 0) pos_of_pair[p] = -1;
    }
    __syncthreads();
    if (threadIdx.x < 32) {  // exclusive scan of the counts by one warp, 32 experts at a time
        int carry = 0;
        for (int base = 0; base < experts; base += 32) {
            const int e = base + (int)threadIdx.x;
            const int c = e < experts ? count[e] : 0;
            int inc = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, inc, o);
                if ((int)threadIdx.x >= o) inc += v;
            }
            if (e < experts) start[e] = carry + inc - c;
            carry += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (threadIdx.x == 0) start[experts] = carry;
    }
    __syncthreads();
    if (blockIdx.x == 0)
        for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = start[e];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = (int)blockIdx.x * 32 + warp;
    if (e >= experts || count[e] == 0) return;
    int pos = start[e];
    const unsigned below = (1u << lane) - 1u;
    for (int base = 0; base < pairs; base += 128) {  // four independent loads in flight per lane
        int mine[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int p = base + 32 * j + lane;
            mine[j] = p < pairs ? sel[p] : -1;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const unsigned m = __ballot_sync(0xffffffffu, mine[j] == e);
            if (mine[j] == e) {
                const int p = base + 32 * j + lane, at = pos + __popc(m & below);
                pos_of_pair[p] = at;
                token_of_pos[at] = p / k;
            }
            pos += __popc(m);
        }
    }
}

// Only choices whose expert lies in [e_lo, e_hi) contribute (the whole range on one GPU, a rank's share under
// expert parallelism).
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ expert_out, const int32_t* __restrict__ sel,
                                                          const float* __restrict__ w, const int32_t* __restrict__ pos_of_pair, int k,
                                                          int hidden, int e_lo, int e_hi, float* __restrict__ out) {
    const int t = blockIdx.x;
    // the token's choices held here, sorted by expert index (k <= 32): row position and weight of each
    __shared__ int s_pos[32], n_here;
    __shared__ float s_w[32];
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        const int e = lane < k ? sel[t * k + lane] : INT_MAX;
        const bool here = lane < k && e >= e_lo && e < e_hi;
        // rank among the choices held here: experts of one token are distinct, so the expert index orders them
        int rank = 0;
        for (int j = 0; j < k; ++j) {
            const int ej = __shfl_sync(0xffffffffu, e, j);
            const bool hj = ej >= e_lo && ej < e_hi;
            if (hj && (ej < e || (ej == e && j < lane))) ++rank;
        }
        if (here) {
            s_pos[rank] = pos_of_pair[t * k + lane];
            s_w[rank] = w[t * k + lane];
        }
        const unsigned m = __ballot_sync(0xffffffffu, here);
        if (lane == 0) n_here = __popc(m);
    }
    __syncthreads();
    const int n = n_here;
    if (hidden % 4 == 0) {
        const int h4 = hidden / 4;
        for (int c = threadIdx.x; c < h4; c += blockDim.x) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int base = 0; base < n; base += 8) {  // eight rows in flight, then added in order
                float4 v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (base + i < n) v[i] = reinterpret_cast<const float4*>(expert_out + (int64_t)s_pos[base + i] * hidden)[c];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (base + i < n) {
                        const float wt = s_w[base + i];
                        acc.x = __fadd_rn(acc.x, __fmul_rn(v[i].x, wt));
                        acc.y = __fadd_rn(acc.y, __fmul_rn(v[i].y, wt));
                        acc.z = __fadd_rn(acc.z, __fmul_rn(v[i].z, wt));
                        acc.w = __fadd_rn(acc.w, __fmul_rn(v[i].w, wt));
                    }
            }
            reinterpret_cast<float4*>(out + (int64_t)t * hidden)[c] = acc;
        }
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            float acc = 0.f;
            for (int i = 0; i < n; ++i) acc = __fadd_rn(acc, __fmul_rn(expert_out[(int64_t)s_pos[i] * hidden + c], s_w[i]));
            out[(int64_t)t * hidden + c] = acc;
        }
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


__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Expert-parallel combine and exchange in one kernel (ranks run it at the same point of the same forward, one per
// GPU).  Pass 1, for each of the CTA's tokens: the weighted sum of the token's choices held by this rank, in ascending
// expert order, is stored into slot `rank` of buffer `buf` in this GPU's block AND, with peer stores over NVLink, in
// every other rank's block; after a system-scope fence the row's flag in each block is set to `epoch`.  Pass 2: wait
// (bounded) until the flags of all other ranks' rows carry `epoch`, then add the slots in rank order - all local
// reads.  No CTA waits before it has published all of its rows, so two GPUs can never wait on each other's
// unscheduled CTAs.  Buffers alternate with the epoch: a rank can reach exchange e+2 only after every peer has set
// its flags of exchange e+1, which a peer does only after it has finished reading exchange e.
__global__ void __launch_bounds__(256) moe_combine_exchange_kernel(const float* __restrict__ expert_out, const int32_t* __restrict__ sel,
                                                                   const float* __restrict__ w, const int32_t* __restrict__ pos_of_pair,
                                                                   int T, int k, int hidden, int e_lo, int e_hi, EpPeers P, uint32_t epoch,
                                                                   uint64_t wait_ns, float* __restrict__ out, int32_t* status) {
    __shared__ int order[32];
    __shared__ int lost;
    const int R = P.ranks, me = P.rank, buf = (int)(epoch & 1u);
    const int h4 = hidden / 4;
    if (threadIdx.x == 0) lost = 0;
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int i = 0; i < k; ++i) order[i] = i;
            for (int i = 1; i < k; ++i) {
                int o = order[i], j = i - 1;
                while (j >= 0 && sel[t * k + order[j]] > sel[t * k + o]) { order[j + 1] = order[j]; --j; }
                order[j + 1] = o;
            }
        }
        __syncthreads();
        const int64_t row4 = ((int64_t)(buf * R + me) * P.slot_floats + (int64_t)t * hidden) / 4;
        for (int c = threadIdx.x; c < h4; c += blockDim.x) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int i = 0; i < k; ++i) {
                int choice = order[i];
                int e = sel[t * k + choice];
                if (e < e_lo || e >= e_hi) continue;
                float wt = w[t * k + choice];
                float4 v = reinterpret_cast<const float4*>(expert_out + (int64_t)pos_of_pair[t * k + choice] * hidden)[c];
                acc.x = __fadd_rn(acc.x, __fmul_rn(v.x, wt));
                acc.y = __fadd_rn(acc.y, __fmul_rn(v.y, wt));
                acc.z = __fadd_rn(acc.z, __fmul_rn(v.z, wt));
                acc.w = __fadd_rn(acc.w, __fmul_rn(v.w, wt));
            }
            for (int p = 0; p < R; ++p) reinterpret_cast<float4*>(P.gather[p])[row4 + c] = acc;
        }
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x < R && threadIdx.x != me)
            st_release_sys(P.flags[threadIdx.x] + (int64_t)(buf * R + me) * P.max_tokens + t, epoch);
    }
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
        if (threadIdx.x < R && threadIdx.x != me) {
            const uint32_t* f = P.flags[me] + (int64_t)(buf * R + threadIdx.x) * P.max_tokens + t;
            const uint64_t t0 = global_ns();
            while (ld_acquire_sys(f) != epoch) {
                if (global_ns() - t0 > wait_ns) {
                    atomicExch(status, 0x4550000 | (int)threadIdx.x);
                    lost = 1;
                    break;
                }
                __nanosleep(200);
            }
        }
        __syncthreads();
        if (lost) return;  // the host reads the status word and fails the forward
        const float4* g = reinterpret_cast<const float4*>(P.gather[me]);
        for (int c = threadIdx.x; c < h4; c += blockDim.x) {
            float4 a = __ldcg(g + ((int64_t)(buf * R) * P.slot_floats + (int64_t)t * hidden) / 4 + c);
            for (int r = 1; r < R; ++r) {
                float4 b = __ldcg(g + ((int64_t)(buf * R + r) * P.slot_floats + (int64_t)t * hidden) / 4 + c);
                a.x = __fadd_rn(a.x, b.x);
                a.y = __fadd_rn(a.y, b.y);
                a.z = __fadd_rn(a.z, b.z);
                a.w = __fadd_rn(a.w, b.w);
            }
            reinterpret_cast<float4*>(out + (int64_t)t * hidden)[c] = a;
        }
    }
}

}  // namespace

void launch_moe_combine_exchange(const float* expert_out, const int32_t* sel_experts, const float* sel_weights,
                                 const int32_t* pos_of_pair, int T, int k, int hidden, int e_lo, int e_hi, const EpPeers& peers,
                                 uint32_t epoch, float* out, int32_t* status, cudaStream_t s, uint64_t wait_ns) {
    if (T <= 0) return;
    if (k > 32) throw std::runtime_error("launch_moe_combine_exchange: more than 32 experts per token");
    if (hidden % 4 != 0 || (int64_t)T * hidden > peers.slot_floats || T > peers.max_tokens)
        throw std::runtime_error("launch_moe_combine_exchange: batch does not fit the exchange block");
    // one CTA per SM at most: every CTA is resident, so pass 1 of all tokens runs without waiting on anything
    int grid = std::min(T, 148);
    moe_combine_exchange_kernel<<<grid, 256, 0, s>>>(expert_out, sel_experts, sel_weights, pos_of_pair, T, k, hidden, e_lo, e_hi, peers,
                                                     epoch, wait_ns, out, status);
    MK_LAUNCH_CHECK();
}

namespace {

__global__ void gather_rows_half_kernel(const uint4* x, const int32_t* token_of_pos, int P, int chunks, uint4* out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)P * chunks) return;
    const int p = (int)(i / chunks), c = (int)(i - (int64_t)p * chunks);
    out[i] = x[(int64_t)token_of_pos[p] * chunks + c];
}

}  // namespace

void launch_gather_rows_half(const __half* x, const int32_t* token_of_pos, int P, int width, __half* out, cudaStream_t s) {
    if (P <= 0) return;
    if (width % 8 != 0) throw std::runtime_error("launch_gather_rows_half: rows must be multiples of 16 bytes");
    const int chunks = width / 8;
    const int64_t n = (int64_t)P * chunks;
    gather_rows_half_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(reinterpret_cast<const uint4*>(x), token_of_pos, P, chunks, reinterpret_cast<uint4*>(out));
    MK_LAUNCH_CHECK();
}

void launch_moe_group(const int32_t* sel_experts, int T, int k, int experts, int32_t* offsets, int32_t* pos_of_pair,
                      int32_t* token_of_pos, cudaStream_t s) {
    if (T <= 0) return;
    if (experts > MAX_EXPERTS) throw std::runtime_error("launch_moe_group: more than 1024 experts");
    moe_group_kernel<<<(experts + 31) / 32, 1024, 0, s>>>(sel_experts, T * k, k, experts, offsets, pos_of_pair, token_of_pos);
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
