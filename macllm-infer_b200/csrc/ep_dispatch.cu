// Expert parallelism with data-parallel lanes: every rank runs its own sequences through attention, router and norms,
// holds the experts [rank * EL, (rank + 1) * EL) and, once per MoE layer, sends the token rows routed to another rank's
// experts there and gets the expert outputs back (SparseMoeFeedForward::forward, src/decoder.rs:394-441, spread over
// ranks; the reference itself runs every expert on one device).
//
// The routed rows of a rank are already grouped by expert (moe_group_kernel), so the rows bound for rank d are one
// contiguous run of the grouped f16 activations.  Per MoE layer and rank:
//   dispatch  - that run is stored into rank d's receive area (peer stores over NVLink; d = this rank is a local copy),
//               together with the per-expert row positions; the CTA that finishes last publishes the exchange's epoch in
//               d's flag;
//   regroup   - waits (bounded) for the flags of all sources, merges the sources' rows expert by expert into one
//               contiguous run per local expert and writes the row ranges the grouped matmuls read;
//   (the two expert-grouped matmuls run on those rows)
//   return    - every output row goes back into its source's result area at the position the source's own grouping gave
//               it, one CTA per (source, local expert); the last CTA of a source publishes the epoch in its return flag;
//   wait_back - waits (bounded) for the return flags of all destinations; the ordinary combine kernel then adds a token's
//               choices in ascending expert order from the result area.
// Buffers alternate with the epoch's parity: a rank can reach exchange e + 2 only after every peer has returned its rows
// of exchange e + 1, which a peer does after it has finished reading exchange e.  Every wait gives up after wait_ns and
// leaves 0x4550000 | peer in the status word; nothing traps and nothing spins without a limit.
#include "ep_comm.h"
#include "kernels.h"

namespace mk {

namespace {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t now_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Once a wait of this forward has given up (the status word is set) the later ones do not wait again: a broken exchange
// costs one limit, not one per layer.
__device__ bool wait_flag(const uint32_t* flag, uint32_t epoch, uint64_t wait_ns, const int32_t* status) {
    const uint64_t t0 = now_ns();
    while (ld_acquire_sys(flag) != epoch) {
        if (*reinterpret_cast<const volatile int32_t*>(status) != 0 || now_ns() - t0 > wait_ns) return false;
        __nanosleep(100);
    }
    return true;
}

__device__ __forceinline__ __half* rows_in(const EpDispatch& D, int p, int buf, int src) {
    return reinterpret_cast<__half*>(D.base[p] + D.rows_in_off) + ((int64_t)(buf * D.ranks + src) * D.cap_rows) * D.hidden;
}
__device__ __forceinline__ int32_t* off_in(const EpDispatch& D, int p, int buf, int src) {
    return reinterpret_cast<int32_t*>(D.base[p] + D.off_in_off) + (int64_t)(buf * D.ranks + src) * (D.local_experts + 1);
}
__device__ __forceinline__ uint32_t* flag_in(const EpDispatch& D, int p, int buf, int src) {
    return reinterpret_cast<uint32_t*>(D.base[p] + D.flag_in_off) + buf * D.ranks + src;
}
__device__ __forceinline__ float* out_back(const EpDispatch& D, int p, int buf) {
    return reinterpret_cast<float*>(D.base[p] + D.out_back_off) + (int64_t)buf * D.cap_rows * D.hidden;
}
__device__ __forceinline__ uint32_t* flag_back(const EpDispatch& D, int p, int buf, int dst) {
    return reinterpret_cast<uint32_t*>(D.base[p] + D.flag_back_off) + buf * D.ranks + dst;
}

constexpr int EPD_SLICES = 64;  // CTAs per destination of the dispatch copy
constexpr int EPD_PARTS = 1;    // CTAs per (source, local expert) segment of the regroup and return copies
constexpr int EPD_COPY_THREADS = 1024;  // threads of those CTAs: few CTAs poll the flags, many threads carry the copies

// Part `part` of `parts` of a copy of n 16-byte pieces by one CTA, four loads in flight per thread (a wide tick moves
// hundreds of megabytes per layer through these copies; one load at a time would leave them latency-bound).
template <typename V>
__device__ __forceinline__ void copy_part(V* __restrict__ to, const V* __restrict__ from, int64_t n, int part, int parts) {
    const int64_t stride = (int64_t)parts * blockDim.x;
    int64_t i = (int64_t)part * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < n; i += 4 * stride) {
        const V a = from[i], b = from[i + stride], c = from[i + 2 * stride], d = from[i + 3 * stride];
        to[i] = a;
        to[i + stride] = b;
        to[i + 2 * stride] = c;
        to[i + 3 * stride] = d;
    }
    for (; i < n; i += stride) to[i] = from[i];
}

// grid (ranks * EPD_SLICES).  x: this rank's routed rows grouped by expert, f16 [P][hidden]; off: [experts + 1].
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ off, EpDispatch D, uint32_t epoch,
                                                          int32_t* done, int32_t* status) {
    const int d = blockIdx.x / EPD_SLICES, slice = blockIdx.x % EPD_SLICES;
    const int EL = D.local_experts, me = D.rank, buf = (int)(epoch & 1u);
    const int r0 = off[d * EL];
    int n = off[(d + 1) * EL] - r0;
    if (n > D.cap_rows) {  // cannot happen while the batch respects max_batch_tokens; recorded, never overrun
        if (threadIdx.x == 0) atomicCAS(status, 0, 0x4551000 | d);
        n = (int)D.cap_rows;
    }
    const int chunks = D.hidden / 8;  // 16-byte pieces per row
    uint4* dst = reinterpret_cast<uint4*>(rows_in(D, d, buf, me));
    const uint4* src = x + (int64_t)r0 * chunks;
    copy_part(dst, src, (int64_t)n * chunks, slice, EPD_SLICES);
    if (slice == 0)
        for (int le = threadIdx.x; le <= EL; le += blockDim.x) off_in(D, d, buf, me)[le] = off[d * EL + le];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(&done[d], 1) == EPD_SLICES - 1) {  // every slice's rows are out
            done[d] = 0;
            __threadfence_system();
            st_release_sys(flag_in(D, d, buf, me), epoch);
        }
    }
}

// grid (ranks * local_experts * EPD_PARTS): the CTAs (src, le, part) move that source's rows for local expert le to their
// place in the merged run.  comb_off [EL + 1]: row ranges per local expert in the merged run; src_start [ranks][EL]: where each source's
// rows of an expert begin in it.
__global__ void __launch_bounds__(EPD_COPY_THREADS) ep_regroup_kernel(EpDispatch D, uint32_t epoch, uint64_t wait_ns, uint4* __restrict__ merged,
                                                         int32_t* __restrict__ comb_off, int32_t* __restrict__ src_start, int32_t* status) {
    __shared__ int ok;
    __shared__ int32_t s_n[kEpMaxRanks * 128], s_start[kEpMaxRanks * 128], s_comb[129];
    const int EL = D.local_experts, N = D.ranks, me = D.rank, buf = (int)(epoch & 1u);
    if (threadIdx.x == 0) ok = 1;
    __syncthreads();
    if ((int)threadIdx.x < N && !wait_flag(flag_in(D, me, buf, threadIdx.x), epoch, wait_ns, status)) {
        atomicCAS(status, 0, 0x4550000 | (int)threadIdx.x);
        ok = 0;
    }
    __syncthreads();
    if (!ok) {  // a source never delivered: publish empty ranges so that nothing downstream reads rows that are not there
        if (blockIdx.x == 0)
            for (int le = threadIdx.x; le <= EL; le += blockDim.x) comb_off[le] = 0;
        return;
    }
    for (int i = threadIdx.x; i < N * EL; i += blockDim.x) {
        const int src = i / EL, le = i - src * EL;
        const int32_t* o = off_in(D, me, buf, src);
        s_n[i] = o[le + 1] - o[le];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int le = 0; le < EL; ++le) {
            s_comb[le] = acc;
            for (int src = 0; src < N; ++src) {
                s_start[src * EL + le] = acc;
                acc += s_n[src * EL + le];
            }
        }
        s_comb[EL] = acc;
    }
    __syncthreads();
    if (blockIdx.x == 0) {
        for (int le = threadIdx.x; le <= EL; le += blockDim.x) comb_off[le] = s_comb[le];
        for (int i = threadIdx.x; i < N * EL; i += blockDim.x) src_start[i] = s_start[i];
    }
    const int seg = blockIdx.x / EPD_PARTS, part = blockIdx.x % EPD_PARTS, src = seg / EL, le = seg - src * EL;
    const int n = s_n[seg];
    if (n <= 0) return;
    const int chunks = D.hidden / 8;
    const int32_t* o = off_in(D, me, buf, src);
    const uint4* from = reinterpret_cast<const uint4*>(rows_in(D, me, buf, src)) + (int64_t)(o[le] - o[0]) * chunks;
    uint4* to = merged + (int64_t)s_start[seg] * chunks;
    copy_part(to, from, (int64_t)n * chunks, part, EPD_PARTS);
}

// grid (ranks * local_experts * EPD_PARTS): the CTAs (src, le, part) send the outputs of that source's rows of local expert le back to the
// positions the source's own grouping gave them.  out: expert outputs of the merged run, f32 [rows][hidden].  The CTA
// that finishes last among a source's CTAs publishes the epoch in the source's return flag.
__global__ void __launch_bounds__(EPD_COPY_THREADS) ep_return_kernel(const float4* __restrict__ out, const int32_t* __restrict__ src_start, EpDispatch D,
                                                        uint32_t epoch, int32_t* done) {
    const int EL = D.local_experts, me = D.rank, buf = (int)(epoch & 1u);
    const int seg = blockIdx.x / EPD_PARTS, part = blockIdx.x % EPD_PARTS, src = seg / EL, le = seg - src * EL;
    const int chunks = D.hidden / 4;
    const int32_t* o = off_in(D, me, buf, src);  // the source's own positions of its rows for my experts
    const int at = o[le], n = o[le + 1] - at;
    if (n > 0) {
        const float4* from = out + (int64_t)src_start[src * EL + le] * chunks;
        float4* to = reinterpret_cast<float4*>(out_back(D, src, buf)) + (int64_t)at * chunks;
        copy_part(to, from, (int64_t)n * chunks, part, EPD_PARTS);
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(&done[src], 1) == EL * EPD_PARTS - 1) {
            done[src] = 0;
            __threadfence_system();
            st_release_sys(flag_back(D, src, buf, me), epoch);
        }
    }
}

// Stand-in for the expert matmuls when the exchange is checked by itself: out = x * (first_expert + local expert + 1).
__global__ void ep_scale_rows_kernel(const __half* __restrict__ x, const int32_t* __restrict__ comb_off, int EL, int first_expert, int hidden,
                                     float* __restrict__ out) {
    const int le = blockIdx.x;
    const int64_t lo = (int64_t)comb_off[le] * hidden, hi = (int64_t)comb_off[le + 1] * hidden;
    const float f = (float)(first_expert + le + 1);
    for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) out[i] = __half2float(x[i]) * f;
}

__global__ void ep_wait_back_kernel(EpDispatch D, uint32_t epoch, uint64_t wait_ns, int32_t* status) {
    const int buf = (int)(epoch & 1u);
    if ((int)threadIdx.x < D.ranks && !wait_flag(flag_back(D, D.rank, buf, threadIdx.x), epoch, wait_ns, status)) atomicCAS(status, 0, 0x4550000 | (int)threadIdx.x);
}

}  // namespace

void launch_ep_dispatch(const __half* grouped_rows, const int32_t* offsets, const EpDispatch& D, uint32_t epoch, int32_t* done, int32_t* status,
                        cudaStream_t s) {
    ep_dispatch_kernel<<<D.ranks * EPD_SLICES, 256, 0, s>>>(reinterpret_cast<const uint4*>(grouped_rows), offsets, D, epoch, done, status);
    MK_LAUNCH_CHECK();
}

void launch_ep_regroup(const EpDispatch& D, uint32_t epoch, __half* merged, int32_t* comb_off, int32_t* src_start, int32_t* status, cudaStream_t s,
                       uint64_t wait_ns) {
    if (D.ranks * D.local_experts > kEpMaxRanks * 128 || D.local_experts > 128) throw std::runtime_error("expert dispatch: more than 128 local experts");
    ep_regroup_kernel<<<D.ranks * D.local_experts * EPD_PARTS, EPD_COPY_THREADS, 0, s>>>(D, epoch, wait_ns, reinterpret_cast<uint4*>(merged), comb_off, src_start, status);
    MK_LAUNCH_CHECK();
}

void launch_ep_return(const float* expert_out, const int32_t* src_start, const EpDispatch& D, uint32_t epoch, int32_t* done, cudaStream_t s) {
    ep_return_kernel<<<D.ranks * D.local_experts * EPD_PARTS, EPD_COPY_THREADS, 0, s>>>(reinterpret_cast<const float4*>(expert_out), src_start, D, epoch, done);
    MK_LAUNCH_CHECK();
}

void launch_ep_wait_back(const EpDispatch& D, uint32_t epoch, int32_t* status, cudaStream_t s, uint64_t wait_ns) {
    ep_wait_back_kernel<<<1, 32, 0, s>>>(D, epoch, wait_ns, status);
    MK_LAUNCH_CHECK();
}

void launch_ep_scale_rows(const __half* merged, const int32_t* comb_off, int local_experts, int first_expert, int hidden, float* out, cudaStream_t s) {
    ep_scale_rows_kernel<<<local_experts, 256, 0, s>>>(merged, comb_off, local_experts, first_expert, hidden, out);
    MK_LAUNCH_CHECK();
}

const float* ep_result_area(const EpDispatch& D, uint32_t epoch) {
    return reinterpret_cast<const float*>(D.base[D.rank] + D.out_back_off) + (int64_t)(epoch & 1u) * D.cap_rows * D.hidden;
}

}  // namespace mk
