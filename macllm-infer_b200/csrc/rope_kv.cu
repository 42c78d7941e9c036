// Fused per-head QK RMSNorm + half-split RoPE + paged-KV scatter.
//
// Replaces, per layer, SelfAttention::project_packed_qkv's per-head norms (src/decoder.rs:1137-1154,
// applied BEFORE the rotation), RotaryEmbedding::apply (src/decoder.rs:203-257, half-split layout on
// the first rotary_dim dims) and PagedKvBatchReservation::write_layer
// (crates/macllm-kv/src/cache.rs:2543-2643): K is stored after the rotation, V unmodified, both at
// KV-head cardinality, token at slot block*block_tokens + row.
// One warp per (token, head); the head vector is staged in shared memory so any head_dim works.
#include "kernels.h"
#include "rope_head.cuh"

namespace mk {

namespace {

constexpr int RK_WARPS = 4;

template <typename KV>
__device__ __forceinline__ KV to_kv(float v);
template <>
__device__ __forceinline__ float to_kv<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half to_kv<__half>(float v) { return __float2half_rn(v); }

template <typename KV>
__global__ void __launch_bounds__(RK_WARPS * 32) rope_kv_kernel(RopeKvArgs a) {
    __shared__ float buf[RK_WARPS][RK_MAX_D];
    pdl_trigger();
    pdl_wait();
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int heads_total = a.q_heads + 2 * a.kv_heads;
    int head = blockIdx.y * RK_WARPS + warp;
    int t = blockIdx.x;
    if (head >= heads_total) return;
    const int d = a.d;
    float* x = buf[warp];

    int kind, hh;  // 0 = q, 1 = k, 2 = v
    if (head < a.q_heads) { kind = 0; hh = head; }
    else if (head < a.q_heads + a.kv_heads) { kind = 1; hh = head - a.q_heads; }
    else { kind = 2; hh = head - a.q_heads - a.kv_heads; }
    rope_head_prepare(a, kind, hh, t, kind != 2 && a.cos_t != nullptr ? a.positions[t] : 0, x, lane);
    if (kind == 0) {
        float* dst = a.q_out != nullptr ? a.q_out + (int64_t)t * a.ldq_out + hh * d : a.q + (int64_t)t * a.ldq + hh * d;
        for (int i = lane; i < d; i += 32) dst[i] = x[i];
    } else {
        int64_t slot = a.slots[t];
        int64_t blk = slot / a.block_tokens, row = slot % a.block_tokens;
        int64_t base = ((kv_page_index(blk, a.layer, a.layers, a.pool_blocks) * a.kv_heads + hh) * a.block_tokens + row) * (int64_t)d;
        KV* pool = reinterpret_cast<KV*>(kind == 1 ? a.k_pool : a.v_pool);
        for (int i = lane; i < d; i += 32) pool[base + i] = to_kv<KV>(x[i]);
    }
}

template <typename KV>
__global__ void cow_copy_kernel(KV* k_pool, KV* v_pool, int64_t src_block, int64_t dst_block, int rows, int layers, int64_t pool_blocks,
                                int kv_heads, int block_tokens, int d) {
    // one CTA per (layer, kv_head)
    int layer = blockIdx.x / kv_heads, h = blockIdx.x % kv_heads;
    int64_t s = ((kv_page_index(src_block, layer, layers, pool_blocks) * kv_heads + h) * block_tokens) * (int64_t)d;
    int64_t t = ((kv_page_index(dst_block, layer, layers, pool_blocks) * kv_heads + h) * block_tokens) * (int64_t)d;
    for (int i = threadIdx.x; i < rows * d; i += blockDim.x) {
        k_pool[t + i] = k_pool[s + i];
        v_pool[t + i] = v_pool[s + i];
    }
}

}  // namespace

void launch_rope_kv(const RopeKvArgs& a, cudaStream_t s) {
    if (a.T <= 0) return;
    if (a.d > RK_MAX_D) throw std::runtime_error("launch_rope_kv: head_dim above 256 is not supported");
    int heads_total = a.q_heads + 2 * a.kv_heads;
    dim3 grid((unsigned)a.T, (unsigned)((heads_total + RK_WARPS - 1) / RK_WARPS));
    if (a.kv_f16)
        launch_pdl(rope_kv_kernel<__half>, grid, dim3(RK_WARPS * 32), 0, s, a);
    else
        launch_pdl(rope_kv_kernel<float>, grid, dim3(RK_WARPS * 32), 0, s, a);
    MK_LAUNCH_CHECK();
}

void launch_cow_copy(void* k_pool, void* v_pool, int kv_f16, int64_t src_block, int64_t dst_block, int rows, int layers,
                     int64_t pool_blocks, int kv_heads, int block_tokens, int d, cudaStream_t s) {
    if (rows <= 0) return;
    unsigned grid = (unsigned)(layers * kv_heads);
    if (kv_f16)
        cow_copy_kernel<__half><<<grid, 128, 0, s>>>((__half*)k_pool, (__half*)v_pool, src_block, dst_block, rows,
                                                     layers, pool_blocks, kv_heads, block_tokens, d);
    else
        cow_copy_kernel<float><<<grid, 128, 0, s>>>((float*)k_pool, (float*)v_pool, src_block, dst_block, rows, layers,
                                                    pool_blocks, kv_heads, block_tokens, d);
    MK_LAUNCH_CHECK();
}

}  // namespace mk
