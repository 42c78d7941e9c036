// On-device token selection and MoE routing.
//
// Greedy selection restates argmax of src/sampling.rs:425-433: a total order on f32 bit patterns,
// the earliest index winning ties.  The reference reads the whole [lanes, vocab] logits back to the
// host every tick (src/engine.rs:2388-2392); here only one u32 per lane crosses PCIe.
// Routing restates selected_softmax_routes (src/decoder.rs:448-554): the k largest router logits in
// (value descending, index ascending) order, then a softmax over those k only.
#include "kernels.h"
#include "sampling_math.h"

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

// ---- temperature / top-k / top-p on the device ------------------------------------------------------------------
// One CTA of 1024 threads per lane.  A lane with temperature <= 0 takes the first-index argmax.  Otherwise the rule of
// Sampler::sample_stochastic (src/sampling.rs:145-169,337-390), for 1 <= top_k <= 1024, with the uniform draw supplied
// by the host (the random stream stays host-side, so the same request draws the same numbers on either path):
//   1. keys of value / temperature in the (value descending, index ascending) order; a four-pass radix select finds the
//      key of the top_k-th candidate, one more pass over the row collects the candidates above it and, in index order,
//      as many of its equals as are still needed;
//   2. the candidates are sorted (bitonic, shared memory); softmax numerators with det_expf against the first one;
//   3. sorted by index, one thread adds the numerators in index order - the order in which the reference adds the whole
//      row, whose other entries are zero - and every candidate is divided by that sum;
//   4. sorted by (probability descending, index ascending), one thread walks the running sum to the top_p cut;
//   5. sorted by index again, one thread adds the survivors, scales the draw and walks to the token.
// The host sampler (sample_top_k_top_p) performs the same operations in the same order, so both return the same token.
constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_MAX_K = 1024;

__device__ __forceinline__ void bitonic_sort_desc(uint64_t* a, int tid) {
    // 1024 keys, 1024 threads; every thread owns the compare-exchange whose lower partner it is
    for (int size = 2; size <= SAMPLE_MAX_K; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            const int partner = tid ^ stride;
            if (partner > tid) {
                const uint64_t x = a[tid], y = a[partner];
                const bool descending = (tid & size) == 0;
                if ((x < y) == descending) { a[tid] = y; a[partner] = x; }
            }
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const float* logits, int vocab, const LaneSampling* params, uint32_t* out,
                                                                 int32_t* status) {
    __shared__ uint64_t keys[SAMPLE_MAX_K];
    __shared__ float prob[SAMPLE_MAX_K];       // indexed like keys after the latest sort
    __shared__ uint32_t hist[256];
    __shared__ uint32_t scan[SAMPLE_THREADS / 32];
    __shared__ uint32_t s_prefix, s_need, s_count, s_keep;
    __shared__ float s_max, s_sum;
    pdl_trigger();
    pdl_wait();
    const int lane_id = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (int64_t)lane_id * vocab;
    const LaneSampling sp = params[lane_id];
    if (!(sp.temperature > 0.f)) {
        // greedy: first-index argmax under the total order
        uint64_t best = 0;
        for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
            const uint64_t k = rank_key(row[i], (uint32_t)i);
            best = k > best ? k : best;
        }
        keys[tid] = best;
        __syncthreads();
        for (int s = SAMPLE_THREADS / 2; s > 0; s >>= 1) {
            if (tid < s && keys[tid + s] > keys[tid]) keys[tid] = keys[tid + s];
            __syncthreads();
        }
        if (tid == 0) out[lane_id] = rank_key_index(keys[0]);
        return;
    }
    const int k = min(min(sp.top_k, SAMPLE_MAX_K), vocab);
    const float temperature = sp.temperature;
    // ---- 1. radix select of the k-th largest 32-bit order key
    uint32_t prefix = 0, mask = 0, need = (uint32_t)k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
            const uint32_t key = f32_order_key(row[i] / temperature);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            uint32_t acc = 0;
            int d = 255;
            for (; d > 0; --d) {
                if (acc + hist[d] >= need) break;
                acc += hist[d];
            }
            s_prefix = prefix | ((uint32_t)d << shift);
            s_need = need - acc;
        }
        __syncthreads();
        prefix = s_prefix;
        need = s_need;
        mask |= 255u << shift;
        __syncthreads();
    }
    // prefix is the key of the k-th candidate; `need` of its equals are taken, lowest indices first
    if (tid == 0) s_count = 0;
    keys[tid] = 0;
    __syncthreads();
    const int chunk = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int lo = min(vocab, tid * chunk), hi = min(vocab, lo + chunk);
    uint32_t equals = 0;
    for (int i = lo; i < hi; ++i) {
        const float v = row[i] / temperature;
        const uint32_t key = f32_order_key(v);
        if (key > prefix) keys[atomicAdd(&s_count, 1u)] = rank_key(v, (uint32_t)i);
        else if (key == prefix) ++equals;
    }
    // exclusive scan of `equals` over the threads (= over index ranges in order)
    uint32_t incl = equals;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
        if ((tid & 31) >= o) incl += t;
    }
    if ((tid & 31) == 31) scan[tid >> 5] = incl;
    __syncthreads();
    if (tid < 32) {
        uint32_t w = scan[tid];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, w, o);
            if (tid >= o) w += t;
        }
        scan[tid] = w;
    }
    __syncthreads();
    uint32_t rank = incl - equals + ((tid >> 5) > 0 ? scan[(tid >> 5) - 1] : 0u);
    const uint32_t greater = (uint32_t)k - need;  // == s_count once every thread has appended
    if (equals > 0 && rank < need) {
        for (int i = lo; i < hi && rank < need; ++i) {
            const float v = row[i] / temperature;
            if (f32_order_key(v) == prefix) { keys[greater + rank] = rank_key(v, (uint32_t)i); ++rank; }
        }
    }
    __syncthreads();
    // ---- 2. rank order, softmax numerators
    bitonic_sort_desc(keys, tid);
    if (tid == 0) s_max = row[rank_key_index(keys[0])] / temperature;
    __syncthreads();
    float p = 0.f;
    uint32_t idx = 0;
    if (tid < k) {
        idx = rank_key_index(keys[tid]);
        p = det_expf(row[idx] / temperature - s_max);
    }
    __syncthreads();
    // ---- 3. index order: the sum of the numerators, then the probabilities
    keys[tid] = tid < k ? (((uint64_t)(0xFFFFFFFFu - idx)) << 32) | (uint64_t)f32_bits(p) : 0ull;
    bitonic_sort_desc(keys, tid);
    if (tid == 0) {
        float sum = 0.f;
        for (int i = 0; i < k; ++i) sum += bits_f32((uint32_t)(keys[i] & 0xFFFFFFFFull));
        s_sum = sum;
    }
    __syncthreads();
    const float sum = s_sum;
    if (!(sum > 0.f) || !isfinite(sum)) {  // "sampling distribution is empty"
        if (tid == 0) { atomicCAS(status, 0, kSampleEmptyStatus | (lane_id & 0xFFFF)); out[lane_id] = 0; }
        return;
    }
    if (tid < k) {
        idx = 0xFFFFFFFFu - (uint32_t)(keys[tid] >> 32);
        p = bits_f32((uint32_t)(keys[tid] & 0xFFFFFFFFull)) / sum;
    }
    __syncthreads();
    // ---- 4. probability order: the top_p cut
    keys[tid] = tid < k ? rank_key(p, idx) : 0ull;
    bitonic_sort_desc(keys, tid);
    if (tid < k) {
        // probabilities travel with their keys: the order key of a non-negative float is its bit pattern with the top bit set
        prob[tid] = bits_f32((uint32_t)(keys[tid] >> 32) & 0x7FFFFFFFu);
    }
    __syncthreads();
    if (tid == 0) {
        uint32_t keep = (uint32_t)k;
        if (sp.top_p >= 0.f && sp.top_p < 1.f) {
            float cumulative = 0.f;
            keep = 0;
            for (int i = 0; i < k; ++i) {
                cumulative += prob[i];
                ++keep;
                if (cumulative >= sp.top_p) break;
            }
        }
        s_keep = keep;
    }
    __syncthreads();
    const uint32_t keep = s_keep;
    const uint32_t best_index = rank_key_index(keys[0]);
    if (tid < k) {
        idx = rank_key_index(keys[tid]);
        p = (uint32_t)tid < keep ? prob[tid] : 0.f;
    }
    __syncthreads();
    // ---- 5. index order again: total, target, walk
    keys[tid] = tid < k ? (((uint64_t)(0xFFFFFFFFu - idx)) << 32) | (uint64_t)f32_bits(p) : 0ull;
    bitonic_sort_desc(keys, tid);
    if (tid == 0) {
        float total = 0.f;
        for (int i = 0; i < k; ++i) total += bits_f32((uint32_t)(keys[i] & 0xFFFFFFFFull));
        const float target = sp.u * total;
        float cumulative = 0.f;
        uint32_t token = best_index;
        for (int i = 0; i < k; ++i) {
            const float q = bits_f32((uint32_t)(keys[i] & 0xFFFFFFFFull));
            if (q <= 0.f) continue;
            cumulative += q;
            if (target < cumulative) { token = 0xFFFFFFFFu - (uint32_t)(keys[i] >> 32); break; }
        }
        out[lane_id] = token;
    }
}

// One warp per token row; experts <= 1024.  Repeated selection of the best remaining candidate.
//
// The reference refuses a row with a non-finite logit ("router produced non-finite logits for token row N",
// src/decoder.rs:474-483).  Here such a row records kMoeRouteStatus | row in *status, which fails the forward at its
// completion barrier, and the offending values compete as the lowest finite number, so that the k choices written
// are always k distinct experts in range and nothing downstream indexes out of bounds.
__global__ void __launch_bounds__(128) moe_route_kernel(const float* logits, int T, int experts, int k,
                                                        int32_t* sel_experts, float* sel_weights, int32_t* status) {
    int t = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (t >= T) return;
    int lane = threadIdx.x & 31;
    const float* row = logits + (int64_t)t * experts;
    constexpr int MAX_PER_LANE = 32;
    float v[MAX_PER_LANE];
    int cnt = 0;
    bool bad = false;
    for (int e = lane; e < experts && cnt < MAX_PER_LANE; e += 32, ++cnt) {
        float x = row[e];
        if (!isfinite(x)) { bad = true; x = -3.402823466e38f; }
        v[cnt] = x;
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0 && status != nullptr) atomicCAS(status, 0, kMoeRouteStatus | (t & 0xFFFF));
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

bool device_sampling_covers(float temperature, int top_k, int vocab) {
    return !(temperature > 0.f) || (top_k >= 1 && top_k <= SAMPLE_MAX_K && top_k <= vocab);
}

void launch_sample(const float* logits, int B, int vocab, const LaneSampling* params_dev, uint32_t* out, int32_t* status, cudaStream_t s) {
    if (B <= 0) return;
    launch_pdl(sample_kernel, dim3((unsigned)B), dim3(SAMPLE_THREADS), 0, s, logits, vocab, params_dev, out, status);
    MK_LAUNCH_CHECK();
}

void launch_moe_route(const float* logits, int T, int experts, int k, int32_t* sel_experts, float* sel_weights,
                      int32_t* status, cudaStream_t s) {
    if (T <= 0) return;
    if (experts > 1024) throw std::runtime_error("launch_moe_route: more than 1024 experts");
    if (k <= 0 || k > experts) throw std::runtime_error("experts per token " + std::to_string(k) + " must be in 1..=" + std::to_string(experts));  // src/decoder.rs:456-458
    moe_route_kernel<<<(T + 3) / 4, 128, 0, s>>>(logits, T, experts, k, sel_experts, sel_weights, status);
    MK_LAUNCH_CHECK();
}

}  // namespace mk
