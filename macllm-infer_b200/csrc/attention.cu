// Variable-length paged grouped-query attention (full causal and sliding window, optional tanh
// softcap) reading K/V straight from the paged pool.
//
// Replaces macllm_kernels::paged_attention_batch (crates/macllm-kernels/src/paged_attention.rs:
// 614-709 is its scalar CPU form; metal/paged_decode.metal:189-489 the Metal forms) and the dense
// fallback the CPU/CUDA backends take (dense_causal_attention, src/decoder.rs:4580-4670, with the
// visibility rule of src/decoder.rs:4515-4532: key j is visible to the query at absolute position p
// iff j <= p and, on sliding layers, p - j < window).  One query tile of one lane and one KV head
// per CTA, so the K/V pages of that head are loaded once for the whole query group (all q heads that
// map to the KV head, query head h reads KV head h / groups).  Scores, softmax and the weighted sum
// are f32; the softmax is the online (running max / running sum) form.
#include "kernels.h"

namespace mk {

namespace {

constexpr int AT_WARPS = 8;
constexpr int AT_KEYS = 32;      // keys per shared-memory tile (one per lane)
constexpr int AT_MAX_ITEMS = 64; // (query row, q head) pairs per CTA
constexpr int AT_IPW = AT_MAX_ITEMS / AT_WARPS;
constexpr int AT_MAX_D = 256;
constexpr int AT_DPL = AT_MAX_D / 32;

template <typename KV>
__device__ __forceinline__ float kv_to_float(KV v);
template <>
__device__ __forceinline__ float kv_to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float kv_to_float<__half>(__half v) { return __half2float(v); }

template <typename KV>
__global__ void __launch_bounds__(AT_WARPS * 32) attn_tile_kernel(AttnArgs a) {
    extern __shared__ float smem[];
    const int d = a.d;
    const int kstride = d + 4;
    float* Qs = smem;                               // [AT_MAX_ITEMS][d]
    float* Ks = Qs + AT_MAX_ITEMS * d;              // [AT_KEYS][d+4]
    float* Vs = Ks + AT_KEYS * kstride;             // [AT_KEYS][d]

    const int tile = blockIdx.x, kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lane_id = a.batch.tile_lane[tile];
    const int row0 = a.batch.tile_row0[tile];
    const LaneHeader hdr = a.batch.hdr[lane_id];
    const int q_off = a.batch.cu_seqlens[lane_id];
    const int n_rows = min(a.q_tile, hdr.n_tokens - row0);
    const int g = a.q_heads / a.kv_heads;
    const int items = n_rows * g;
    const int ldq = a.ldq > 0 ? a.ldq : a.q_heads * d;
    const int ldo = a.q_heads * d;

    for (int i = threadIdx.x; i < items * d; i += blockDim.x) {
        int item = i / d, k = i - item * d;
        int r = item / g, hq = item - r * g;
        Qs[item * d + k] = a.q[(int64_t)(q_off + row0 + r) * ldq + (kvh * g + hq) * d + k];
    }

    const int p_first = hdr.start_pos + row0;
    const int p_last = p_first + n_rows - 1;
    int k_begin = 0;
    if (a.window > 0) k_begin = max(0, p_first - a.window + 1);
    k_begin = (k_begin / AT_KEYS) * AT_KEYS;
    const int k_end = p_last + 1;

    float m_run[AT_IPW], l_run[AT_IPW], acc[AT_IPW][AT_DPL];
#pragma unroll
    for (int i = 0; i < AT_IPW; ++i) {
        m_run[i] = -INFINITY;
        l_run[i] = 0.f;
#pragma unroll
        for (int j = 0; j < AT_DPL; ++j) acc[i][j] = 0.f;
    }

    const KV* kp = reinterpret_cast<const KV*>(a.k_pool);
    const KV* vp = reinterpret_cast<const KV*>(a.v_pool);

    for (int kt = k_begin; kt < k_end; kt += AT_KEYS) {
        __syncthreads();
        // stage 32 keys and values (zero beyond k_end)
        for (int i = threadIdx.x; i < AT_KEYS * (d / 4); i += blockDim.x) {
            int key = i / (d / 4), c = (i - key * (d / 4)) * 4;
            int pos = kt + key;
            float4 kv4 = make_float4(0.f, 0.f, 0.f, 0.f), vv4 = kv4;
            if (pos < k_end) {
                int64_t blk = a.batch.tables[hdr.table_off + pos / a.block_tokens];
                int64_t base = ((kv_page_index(blk, a.layer, a.layers, a.pool_blocks) * a.kv_heads + kvh) * a.block_tokens + pos % a.block_tokens) *
                                   (int64_t)d + c;
                kv4 = make_float4(kv_to_float<KV>(kp[base]), kv_to_float<KV>(kp[base + 1]), kv_to_float<KV>(kp[base + 2]),
                                  kv_to_float<KV>(kp[base + 3]));
                vv4 = make_float4(kv_to_float<KV>(vp[base]), kv_to_float<KV>(vp[base + 1]), kv_to_float<KV>(vp[base + 2]),
                                  kv_to_float<KV>(vp[base + 3]));
            }
            *reinterpret_cast<float4*>(Ks + key * kstride + c) = kv4;
            *reinterpret_cast<float4*>(Vs + key * d + c) = vv4;
        }
        __syncthreads();

#pragma unroll
        for (int ii = 0; ii < AT_IPW; ++ii) {
            int item = warp + AT_WARPS * ii;
            if (item >= items) continue;
            int r = item / g;
            int p = p_first + r;
            int key = kt + lane;
            bool visible = key <= p && (a.window == 0 || p - key < a.window);
            float s = -INFINITY;
            if (visible) {
                const float4* qv = reinterpret_cast<const float4*>(Qs + item * d);
                const float4* kv = reinterpret_cast<const float4*>(Ks + lane * kstride);
                float dot = 0.f;
                for (int c = 0; c < d / 4; ++c) {
                    float4 x = qv[c], y = kv[c];
                    dot += x.x * y.x;
                    dot += x.y * y.y;
                    dot += x.z * y.z;
                    dot += x.w * y.w;
                }
                s = dot * a.scale;
                if (a.softcap != 0.f) s = tanhf(s / a.softcap) * a.softcap;
            }
            float tmax = warp_max(s);
            if (tmax == -INFINITY) continue;  // nothing visible in this tile for this row
            float m_new = fmaxf(m_run[ii], tmax);
            float alpha = (m_run[ii] == -INFINITY) ? 0.f : expf(m_run[ii] - m_new);
            float pj = visible ? expf(s - m_new) : 0.f;
            float psum = warp_sum(pj);
            l_run[ii] = l_run[ii] * alpha + psum;
            m_run[ii] = m_new;
#pragma unroll
            for (int j = 0; j < AT_DPL; ++j) acc[ii][j] *= alpha;
            for (int kk = 0; kk < AT_KEYS; ++kk) {
                float pk = __shfl_sync(0xffffffffu, pj, kk);
                if (pk != 0.f) {
#pragma unroll
                    for (int j = 0; j < AT_DPL; ++j) {
                        int c = lane + 32 * j;
                        if (c < d) acc[ii][j] += pk * Vs[kk * d + c];
                    }
                }
            }
        }
    }

#pragma unroll
    for (int ii = 0; ii < AT_IPW; ++ii) {
        int item = warp + AT_WARPS * ii;
        if (item >= items) continue;
        int r = item / g, hq = item - r * g;
        float* o = a.out + (int64_t)(q_off + row0 + r) * ldo + (kvh * g + hq) * d;
        float inv = 1.0f / l_run[ii];
#pragma unroll
        for (int j = 0; j < AT_DPL; ++j) {
            int c = lane + 32 * j;
            if (c < d) o[c] = acc[ii][j] * inv;
        }
    }
}

}  // namespace

int attention_q_tile(int q_heads, int kv_heads) {
    int g = q_heads / kv_heads;
    int t = AT_MAX_ITEMS / g;
    return t < 1 ? 1 : t;
}

void launch_paged_attention(const AttnArgs& a, cudaStream_t s) {
    if (a.batch.max_tiles <= 0) return;
    if (a.d > AT_MAX_D || a.d % 4 != 0) throw std::runtime_error("launch_paged_attention: head_dim must be a multiple of 4, at most 256");
    if (a.q_heads % a.kv_heads != 0 || a.q_heads / a.kv_heads > AT_MAX_ITEMS)
        throw std::runtime_error("launch_paged_attention: unsupported query group size");
    size_t smem = (size_t)(AT_MAX_ITEMS * a.d + AT_KEYS * (a.d + 4) + AT_KEYS * a.d) * sizeof(float);
    dim3 grid((unsigned)a.batch.max_tiles, (unsigned)a.kv_heads);
    if (a.kv_f16) {
        ensure_dynamic_smem(reinterpret_cast<const void*>(&attn_tile_kernel<__half>), smem);
        attn_tile_kernel<__half><<<grid, AT_WARPS * 32, smem, s>>>(a);
    } else {
        ensure_dynamic_smem(reinterpret_cast<const void*>(&attn_tile_kernel<float>), smem);
        attn_tile_kernel<float><<<grid, AT_WARPS * 32, smem, s>>>(a);
    }
    MK_LAUNCH_CHECK();
}

}  // namespace mk
