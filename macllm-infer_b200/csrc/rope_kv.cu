// Fused per-head QK RMSNorm + half-split RoPE + paged-KV scatter.
//
// Replaces, per layer, SelfAttention::project_packed_qkv's per-head norms (src/decoder.rs:1137-1154,
// applied BEFORE the rotation), RotaryEmbedding::apply (src/decoder.rs:203-257, half-split layout on
// the first rotary_dim dims) and PagedKvBatchReservation::write_layer
// (crates/macllm-kv/src/cache.rs:2543-2643): K is stored after the rotation, V unmodified, both at
// KV-head cardinality, token at slot block*block_tokens + row.
// One warp per (token, head); the head vector is staged in shared memory so any head_dim works.
#include "kernels.h"

namespace mk {

namespace {

constexpr int RK_WARPS = 4;
constexpr int RK_MAX_D = 256;

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

    int kind;  // 0 = q, 1 = k, 2 = v
    const float* src;
    int hh;
    if (head < a.q_heads) { kind = 0; hh = head; src = a.q + (int64_t)t * a.ldq + hh * d; }
    else if (head < a.q_heads + a.kv_heads) { kind = 1; hh = head - a.q_heads; src = a.k + (int64_t)t * a.ldk + hh * d; }
    else { kind = 2; hh = head - a.q_heads - a.kv_heads; src = a.v + (int64_t)t * a.ldv + hh * d; }

    const int n_parts = kind == 2 ? a.v_splits : a.qk_splits;
    const int64_t part_stride = kind == 2 ? a.v_split_stride : a.qk_split_stride;
    if ((d & 127) == 0 && ((reinterpret_cast<uintptr_t>(src) | (uintptr_t)(part_stride * 4)) & 15) == 0) {
        for (int i = lane * 4; i < d; i += 128) {
            float4 v = *reinterpret_cast<const float4*>(src + i);
#pragma unroll 4
            for (int sp = 1; sp < n_parts; ++sp) {
                float4 w = *reinterpret_cast<const float4*>(src + (int64_t)sp * part_stride + i);
                v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
            }
            *reinterpret_cast<float4*>(x + i) = v;
        }
    } else {
        for (int i = lane; i < d; i += 32) {
            float v = src[i];
            for (int sp = 1; sp < n_parts; ++sp) v += src[(int64_t)sp * part_stride + i];
            x[i] = v;
        }
    }
    __syncwarp();

    const float* nw = kind == 0 ? a.q_norm_w : (kind == 1 ? a.k_norm_w : nullptr);
    if (nw != nullptr) {
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) ss += x[i] * x[i];
        ss = warp_sum(ss);
        float m = sqrtf(ss / (float)d + a.norm_eps);
        for (int i = lane; i < d; i += 32) x[i] = x[i] / m * nw[i];
        __syncwarp();
    }
    if (kind != 2 && a.cos_t != nullptr) {
        int half = a.rotary_dim / 2;
        const float* c = a.cos_t + (int64_t)a.positions[t] * half;
        const float* s = a.sin_t + (int64_t)a.positions[t] * half;
        float r1[RK_MAX_D / 64], r2[RK_MAX_D / 64];
        int cnt = 0;
        for (int i = lane; i < half; i += 32, ++cnt) {
            float x1 = x[i], x2 = x[i + half];
            r1[cnt] = __fsub_rn(__fmul_rn(x1, c[i]), __fmul_rn(x2, s[i]));
            r2[cnt] = __fadd_rn(__fmul_rn(x1, s[i]), __fmul_rn(x2, c[i]));
        }
        __syncwarp();
        cnt = 0;
        for (int i = lane; i < half; i += 32, ++cnt) { x[i] = r1[cnt]; x[i + half] = r2[cnt]; }
        __syncwarp();
    }
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
