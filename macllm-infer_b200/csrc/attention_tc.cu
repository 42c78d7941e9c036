// Tensor-core varlen paged GQA attention for f16 KV pools: prefill chunks and (split over the keys)
// decode lanes.
//
// Same operator as attention.cu (the replacement of macllm_kernels::paged_attention_batch,
// crates/macllm-kernels/src/paged_attention.rs:614-709, and of dense_causal_attention,
// src/decoder.rs:4580-4670; visibility rule src/decoder.rs:4515-4532), restructured for bandwidth:
// one CTA owns 16*WARPS (query row, query head) items that all read ONE KV head, so every K/V page
// is fetched once for the whole query group; pages travel global -> shared with 16-byte cp.async in a
// two-stage pipeline; Q.K^T and P.V run on the tensor cores (mma.sync m16n8k16, f16 operands, f32
// accumulators) and the online softmax stays in f32 registers.  One-token lanes run attn_decode_kernel: the
// keys are shared out over the four warps of a CTA (warp-private cp.async rings, merge in shared memory) and,
// when few lanes have long histories, over several CTAs as well (scratch: unnormalised partial outputs +
// running max / sum per head, merged by attn_combine_kernel).  Queries are rounded to f16 once; K/V are read
// as stored.
#include "kernels.h"
#include "attention_tc.h"
#include "rope_head.cuh"
#include "quant_blocks.cuh"
#include <algorithm>

namespace mk {

namespace {

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    int bytes = valid ? 16 : 0;  // src-size 0 zero-fills the 16 destination bytes
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float x, float y) {
    __half2 h = __floats2half2_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&h);
}

// One CTA.  D = head_dim, WARPS warps of 16 items each, KT keys per shared-memory tile.
// SPLIT = false: work item = tiles[blockIdx.x] = (lane, first query row); the CTA walks every visible key
//                and writes normalised outputs.
// SPLIT = true : work item = entries[blockIdx.x] = (lane, split, n_splits) of a one-token lane; the CTA walks
//                its share of the keys and writes an unnormalised partial.
template <int D, int WARPS, int KT, bool SPLIT>
__global__ void __launch_bounds__(WARPS * 32) attn_tc_kernel(AttnTcArgs a) {
    constexpr int DP = D + 8;              // padded row (halves): conflict-free ldmatrix
    constexpr int M = 16 * WARPS;
    constexpr int NT_S = KT / 8;           // score n-tiles per warp
    constexpr int NT_O = D / 8;            // output n-tiles per warp
    constexpr int CHUNKS = D / 8;          // 16-byte chunks per K or V row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* Qs = reinterpret_cast<__half*>(smem_raw);          // [M][DP]
    __half* Ks = Qs + M * DP;                                   // [2][KT][DP]
    __half* Vs = Ks + 2 * KT * DP;                              // [2][KT][DP]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, tq = lane & 3;
    const int kvh = blockIdx.y;
    const int g = a.q_heads / a.kv_heads;
    pdl_trigger();
    pdl_wait();

    int lane_id, row0, rows_per_head, split = 0, n_splits = 1;
    if (SPLIT) {
        lane_id = a.entries[3 * blockIdx.x];
        split = a.entries[3 * blockIdx.x + 1];
        n_splits = a.entries[3 * blockIdx.x + 2];
        row0 = 0;
        rows_per_head = 1;
    } else {
        lane_id = a.tiles[2 * blockIdx.x];
        row0 = a.tiles[2 * blockIdx.x + 1];
        rows_per_head = M / g;
    }
    const LaneHeader hdr = a.hdr[lane_id];
    const int q_off = a.cu_seqlens[lane_id];
    const int n_rows = SPLIT ? 1 : min(rows_per_head, hdr.n_tokens - row0);
    const int ldq = a.ldq > 0 ? a.ldq : a.q_heads * D;
    const int ldo = a.q_heads * D;

    // item i of the CTA: head-in-group i / rows_per_head, query row i % rows_per_head
    for (int i = tid; i < M * CHUNKS; i += WARPS * 32) {
        int item = i / CHUNKS, c = (i - item * CHUNKS) * 8;
        int hq = item / rows_per_head, r = item - hq * rows_per_head;
        __half2 h[4];
        if (hq < g && r < n_rows) {
            const float* src = a.q + (int64_t)(q_off + row0 + r) * ldq + (kvh * g + hq) * D + c;
            float4 x0 = *reinterpret_cast<const float4*>(src), x1 = *reinterpret_cast<const float4*>(src + 4);
            h[0] = __floats2half2_rn(x0.x, x0.y);
            h[1] = __floats2half2_rn(x0.z, x0.w);
            h[2] = __floats2half2_rn(x1.x, x1.y);
            h[3] = __floats2half2_rn(x1.z, x1.w);
        } else {
            h[0] = h[1] = h[2] = h[3] = __floats2half2_rn(0.f, 0.f);
        }
        *reinterpret_cast<uint4*>(Qs + item * DP + c) = *reinterpret_cast<uint4*>(h);
    }

    // key range of this CTA
    const int p_first = hdr.start_pos + row0, p_last = p_first + n_rows - 1;
    int k_lo = a.window > 0 ? max(0, p_first - a.window + 1) : 0;
    int k_hi = p_last + 1;
    if (SPLIT) {
        int len = k_hi - k_lo;
        int chunk = ((len + n_splits - 1) / n_splits + 15) / 16 * 16;
        k_lo = k_lo + split * chunk;
        k_hi = min(k_hi, k_lo + chunk);
    }
    const int k_begin = k_lo / 16 * 16;  // page aligned
    const int n_tiles = k_hi > k_begin ? (k_hi - k_begin + KT - 1) / KT : 0;

    const __half* kp = reinterpret_cast<const __half*>(a.k_pool);
    const __half* vp = reinterpret_cast<const __half*>(a.v_pool);
    auto load_tile = [&](int t, int stage) {
        __half* kd = Ks + stage * KT * DP;
        __half* vd = Vs + stage * KT * DP;
        for (int i = tid; i < KT * CHUNKS; i += WARPS * 32) {
            int key = i / CHUNKS, c = (i - key * CHUNKS) * 8;
            int pos = k_begin + t * KT + key;
            bool valid = pos < k_hi;
            int64_t base = 0;
            if (valid) {
                int64_t blk = a.tables[hdr.table_off + (pos >> a.bt_shift)];
                base = ((kv_page_index(blk, a.layer, a.layers, a.pool_blocks) * a.kv_heads + kvh) * a.block_tokens +
                        (pos & (a.block_tokens - 1))) * (int64_t)D + c;
            }
            cp_async16(kd + key * DP + c, kp + base, valid);
            cp_async16(vd + key * DP + c, vp + base, valid);
        }
    };

    float o_acc[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) o_acc[j][0] = o_acc[j][1] = o_acc[j][2] = o_acc[j][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    // the two accumulator rows of this thread: items warp*16 + gid and + 8
    int item_r[2] = {warp * 16 + gid, warp * 16 + gid + 8};
    int pos_r[2];
    bool live_r[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        int hq = item_r[h] / rows_per_head, r = item_r[h] - hq * rows_per_head;
        live_r[h] = hq < g && r < n_rows;
        pos_r[h] = p_first + r;
    }

    if (n_tiles > 0) load_tile(0, 0);
    cp_async_commit();
    for (int t = 0; t < n_tiles; ++t) {
        if (t + 1 < n_tiles) load_tile(t + 1, (t + 1) & 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const __half* kt = Ks + (t & 1) * KT * DP;
        const __half* vt = Vs + (t & 1) * KT * DP;

        // S = Q K^T
        float s[NT_S][4];
#pragma unroll
        for (int j = 0; j < NT_S; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            uint32_t af[4];
            ldmatrix_x4(af, Qs + (warp * 16 + (lane & 15)) * DP + kk * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int j = 0; j < NT_S; j += 2) {
                uint32_t bf[4];
                ldmatrix_x4(bf, kt + (j * 8 + (lane & 7) + (lane >> 4) * 8) * DP + kk * 16 + ((lane >> 3) & 1) * 8);
                mma16816(s[j], af, bf[0], bf[1]);
                mma16816(s[j + 1], af, bf[2], bf[3]);
            }
        }
        // scale, softcap, mask, online softmax (f32)
        const int tile_pos = k_begin + t * KT;
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < NT_S; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int h = e >> 1;
                int pos = tile_pos + j * 8 + 2 * tq + (e & 1);
                float v = s[j][e] * a.scale;
                if (a.softcap != 0.f) v = tanhf(v / a.softcap) * a.softcap;
                bool vis = live_r[h] && pos >= k_lo && pos < k_hi && pos <= pos_r[h] && (a.window == 0 || pos_r[h] - pos < a.window);
                v = vis ? v : -INFINITY;
                s[j][e] = v;
                tmax[h] = fmaxf(tmax[h], v);
            }
        }
        float alpha[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
            tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
            float m_new = fmaxf(m_run[h], tmax[h]);
            m_use[h] = m_new == -INFINITY ? 0.f : m_new;
            alpha[h] = m_run[h] == -INFINITY ? 0.f : __expf(m_run[h] - m_use[h]);
            m_run[h] = m_new;
        }
        float psum[2] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < NT_S; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int h = e >> 1;
                float p = s[j][e] == -INFINITY ? 0.f : __expf(s[j][e] - m_use[h]);
                s[j][e] = p;
                psum[h] += p;
            }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 1);
            psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 2);
            l_run[h] = l_run[h] * alpha[h] + psum[h];
        }
#pragma unroll
        for (int j = 0; j < NT_O; ++j) {
            o_acc[j][0] *= alpha[0];
            o_acc[j][1] *= alpha[0];
            o_acc[j][2] *= alpha[1];
            o_acc[j][3] *= alpha[1];
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
            uint32_t pf[4] = {pack_half2(s[2 * kk][0], s[2 * kk][1]), pack_half2(s[2 * kk][2], s[2 * kk][3]),
                              pack_half2(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_half2(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
            for (int j = 0; j < NT_O; j += 2) {
                uint32_t bf[4];
                ldmatrix_x4_trans(bf, vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * DP + j * 8 + (lane >> 4) * 8);
                mma16816(o_acc[j], pf, bf[0], bf[1]);
                mma16816(o_acc[j + 1], pf, bf[2], bf[3]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

    if (!SPLIT) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (!live_r[h]) continue;
            int hq = item_r[h] / rows_per_head, r = item_r[h] - hq * rows_per_head;
            float inv = 1.0f / l_run[h];
            const int64_t at = (int64_t)(q_off + row0 + r) * ldo + (kvh * g + hq) * D;
            if (a.out != nullptr) {
#pragma unroll
                for (int j = 0; j < NT_O; ++j)
                    *reinterpret_cast<float2*>(a.out + at + j * 8 + 2 * tq) = make_float2(o_acc[j][2 * h] * inv, o_acc[j][2 * h + 1] * inv);
            }
            if (a.out_h != nullptr) {
#pragma unroll
                for (int j = 0; j < NT_O; ++j)
                    *reinterpret_cast<__half2*>(a.out_h + at + j * 8 + 2 * tq) =
                        __floats2half2_rn(o_acc[j][2 * h] * inv, o_acc[j][2 * h + 1] * inv);
            }
        }
    } else {
        // unnormalised partial of this key share: [entry][kv head][16 items][D], plus (max, sum) per item
        int64_t slot = ((int64_t)blockIdx.x * a.kv_heads + kvh) * 16;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            int item = gid + 8 * h;
            if (item >= g) continue;  // only the group's heads are live in a one-token lane
            float* o = a.part_o + (slot + item) * D;
#pragma unroll
            for (int j = 0; j < NT_O; ++j)
                *reinterpret_cast<float2*>(o + j * 8 + 2 * tq) = make_float2(o_acc[j][2 * h], o_acc[j][2 * h + 1]);
            if (tq == 0) {
                a.part_ml[(slot + item) * 2] = m_run[h];
                a.part_ml[(slot + item) * 2 + 1] = l_run[h];
            }
        }
    }
}

// One-token lanes.  Work item = entries[blockIdx.x] = (lane, share, n_shares) x KV head.  The four warps of the
// CTA take the 16-key tiles of the share round-robin, each through its own ring of cp.async stages (no
// block-wide barrier inside the loop), keep their own running max / sum / output, and merge through shared
// memory at the end.  n_shares == 1: the CTA writes the normalised output.  Otherwise it writes its unnormalised
// partial, and the CTA that arrives last at the lane's counter merges the shares.
// LOW8: at most eight query heads per KV head, so rows 8-15 of the A operand are zero and everything that concerns
// them (half of the softmax and of the accumulator rescaling) is skipped.
template <int D, int STAGES, bool LOW8>
__global__ void __launch_bounds__(128) attn_decode_kernel(AttnTcArgs a) {
    constexpr int NH = LOW8 ? 1 : 2;  // accumulator row halves that can hold live rows
    constexpr int DP = D + 8;
    constexpr int KT = 16;
    constexpr int NT_O = D / 8;
    constexpr int CHUNKS = D / 8;
    constexpr int RING_HALVES = STAGES * 2 * KT * DP;  // per warp: STAGES x (K tile + V tile)
    static_assert(RING_HALVES * 2 >= 16 * D * 4 + 16 * 2 * 4, "a warp's ring must hold its partial result");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* Qs = reinterpret_cast<__half*>(smem_raw);  // [16][DP]
    __half* rings = Qs + 16 * DP;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, tq = lane & 3;
    const int kvh = blockIdx.y;
    const int g = a.q_heads / a.kv_heads;
    pdl_trigger();
    pdl_wait();
    // one 32-byte record per work item, so that nothing but the block table and the queries is a dependent load
    const int4 e0 = reinterpret_cast<const int4*>(a.entries)[2 * blockIdx.x];
    const int4 e1 = reinterpret_cast<const int4*>(a.entries)[2 * blockIdx.x + 1];
    const int lane_id = e0.x, split = e0.y, n_splits = e0.z, start_pos = e0.w, table_off = e1.x, q_off = e1.y, first_entry = e1.z;
    const int ldq = a.ldq > 0 ? a.ldq : a.q_heads * D;

    // Rows straight from the projection's output (see AttnTcArgs::fused_rope): one warp per head, the head vector staged
    // in f32; the group's query heads, and in the CTA that walks the lane's newest keys also the new K and V rows, which
    // reach the pool before any tile is requested (block-wide barrier below).
    __shared__ __align__(16) float head_stage[4][D];
    auto prepare_head = [&](int kind, int item) {  // kind 0: query head `item` of the group; 1 / 2: the new K / V row
        float* xs = head_stage[warp];
        rope_head_prepare(a.rk, kind, kind == 0 ? kvh * g + item : kvh, q_off, start_pos, xs, lane);
        if (kind == 0) {
            for (int i = lane; i < D; i += 32) Qs[item * DP + i] = __float2half_rn(xs[i]);
        } else {
            const int64_t blk = a.tables[table_off + (start_pos >> a.bt_shift)];
            const int64_t base = ((kv_page_index(blk, a.layer, a.layers, a.pool_blocks) * a.kv_heads + kvh) * a.block_tokens +
                                  (start_pos & (a.block_tokens - 1))) * (int64_t)D;
            __half* pool = reinterpret_cast<__half*>(kind == 1 ? a.rk.k_pool : a.rk.v_pool);
            for (int i = lane; i < D; i += 32) pool[base + i] = __float2half_rn(xs[i]);
        }
        __syncwarp();
    };
    if (a.fused_rope) {
        for (int i = tid; i < (16 - g) * CHUNKS; i += 128) {
            int item = g + i / CHUNKS, c = (i % CHUNKS) * 8;
            *reinterpret_cast<uint4*>(Qs + item * DP + c) = make_uint4(0u, 0u, 0u, 0u);
        }
        const int n_heads = g + (split == n_splits - 1 ? 2 : 0);
        for (int h = warp; h < n_heads; h += 4) prepare_head(h < g ? 0 : (h == g ? 1 : 2), h);
        __syncthreads();  // the new K / V rows are visible to every tile load of this CTA
    } else {
    // the group's query heads -> rows 0..g-1 of the A operand, the rest zero
    for (int i = tid; i < 16 * CHUNKS; i += 128) {
        int item = i / CHUNKS, c = (i - item * CHUNKS) * 8;
        __half2 h[4];
        if (item < g) {
            const float* src = a.q + (int64_t)q_off * ldq + (kvh * g + item) * D + c;
            float4 x0 = *reinterpret_cast<const float4*>(src), x1 = *reinterpret_cast<const float4*>(src + 4);
            h[0] = __floats2half2_rn(x0.x, x0.y);
            h[1] = __floats2half2_rn(x0.z, x0.w);
            h[2] = __floats2half2_rn(x1.x, x1.y);
            h[3] = __floats2half2_rn(x1.z, x1.w);
        } else {
            h[0] = h[1] = h[2] = h[3] = __floats2half2_rn(0.f, 0.f);
        }
        *reinterpret_cast<uint4*>(Qs + item * DP + c) = *reinterpret_cast<uint4*>(h);
    }
    }

    const int p = start_pos;  // the query's position
    int k_lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
    int k_hi = p + 1;
    {
        int len = k_hi - k_lo;
        int chunk = ((len + n_splits - 1) / n_splits + 15) / 16 * 16;
        k_lo = k_lo + split * chunk;
        k_hi = min(k_hi, k_lo + chunk);
    }
    const int k_begin = k_lo / 16 * 16;
    const int n_tiles = k_hi > k_begin ? (k_hi - k_begin + KT - 1) / KT : 0;
    const int my_tiles = n_tiles > warp ? (n_tiles - warp + 3) / 4 : 0;  // tiles warp, warp + 4, ...

    const __half* kp = reinterpret_cast<const __half*>(a.k_pool);
    const __half* vp = reinterpret_cast<const __half*>(a.v_pool);
    __half* ring = rings + warp * RING_HALVES;
    uint32_t tile_blk = 0;
    auto load_tile = [&](int i) {  // the warp's i-th tile into stage i % STAGES (called with i = 0, 1, 2, ... in order)
        __half* kd = ring + (i % STAGES) * 2 * KT * DP;
        __half* vd = kd + KT * DP;
        // 16 keys starting at a multiple of 16 lie in one page (block_tokens is a multiple of 16): one table
        // lookup, then the tile is one contiguous run of 16 * D halves in each pool
        const int pos0 = k_begin + (warp + 4 * i) * KT;
        // the page ids of the warp's next 32 tiles sit in the lanes (fetched together, off the critical path)
        if ((i & 31) == 0) {
            const int t = i + lane;
            tile_blk = t < my_tiles ? a.tables[table_off + ((k_begin + (warp + 4 * t) * KT) >> a.bt_shift)] : 0u;
        }
        const int64_t blk = __shfl_sync(0xffffffffu, tile_blk, i & 31);
        const int64_t src0 = ((kv_page_index(blk, a.layer, a.layers, a.pool_blocks) * a.kv_heads + kvh) * a.block_tokens +
                              (pos0 & (a.block_tokens - 1))) * (int64_t)D;
        const int n_valid = k_hi - pos0;  // keys of the tile inside the share
#pragma unroll
        for (int j = lane; j < KT * CHUNKS; j += 32) {
            const int key = j / CHUNKS, c = (j % CHUNKS) * 8;
            const bool valid = key < n_valid;
            const int64_t src = valid ? src0 + (int64_t)j * 8 : 0;
            cp_async16(kd + key * DP + c, kp + src, valid);
            cp_async16(vd + key * DP + c, vp + src, valid);
        }
    };

    float o_acc[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) o_acc[j][0] = o_acc[j][1] = o_acc[j][2] = o_acc[j][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const bool live_r[2] = {gid < g, gid + 8 < g};

#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) {
        if (i < my_tiles) load_tile(i);
        cp_async_commit();
    }
    __syncthreads();  // Qs complete
    constexpr bool Q_IN_REGS = D <= 128;
    uint32_t qf[Q_IN_REGS ? D / 16 : 1][4];
    if (Q_IN_REGS) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) ldmatrix_x4(qf[Q_IN_REGS ? kk : 0], Qs + (lane & 15) * DP + kk * 16 + (lane >> 4) * 8);
    }

    for (int i = 0; i < my_tiles; ++i) {
        if (i + STAGES - 1 < my_tiles) load_tile(i + STAGES - 1);
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncwarp();
        const __half* kt = ring + (i % STAGES) * 2 * KT * DP;
        const __half* vt = kt + KT * DP;

        float sc[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            uint32_t af[4], bf[4];
            if (!Q_IN_REGS) ldmatrix_x4(af, Qs + (lane & 15) * DP + kk * 16 + (lane >> 4) * 8);
            ldmatrix_x4(bf, kt + ((lane & 7) + (lane >> 4) * 8) * DP + kk * 16 + ((lane >> 3) & 1) * 8);
            mma16816(sc[0], Q_IN_REGS ? qf[Q_IN_REGS ? kk : 0] : af, bf[0], bf[1]);
            mma16816(sc[1], Q_IN_REGS ? qf[Q_IN_REGS ? kk : 0] : af, bf[2], bf[3]);
        }
        const int tile_pos = k_begin + (warp + 4 * i) * KT;
        // a tile that lies wholly inside the share needs no masking (rows without a query head hold zeros and are
        // never stored)
        const bool full_tile = tile_pos >= k_lo && tile_pos + KT <= k_hi;
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int e = 0; e < 2 * NH; ++e) {
                int h = e >> 1;
                int pos = tile_pos + j * 8 + 2 * tq + (e & 1);
                float v = sc[j][e] * a.scale;
                if (a.softcap != 0.f) v = tanhf(v / a.softcap) * a.softcap;
                bool vis = full_tile || (live_r[h] && pos >= k_lo && pos < k_hi);  // k_lo / k_hi carry causality and the window
                v = vis ? v : -INFINITY;
                sc[j][e] = v;
                tmax[h] = fmaxf(tmax[h], v);
            }
        }
        float alpha[2] = {1.f, 1.f}, m_use[2] = {0.f, 0.f};
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
            tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
            float m_new = fmaxf(m_run[h], tmax[h]);
            m_use[h] = m_new == -INFINITY ? 0.f : m_new;
            alpha[h] = m_run[h] == -INFINITY ? 0.f : __expf(m_run[h] - m_use[h]);
            m_run[h] = m_new;
        }
        float psum[2] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int e = 0; e < 2 * NH; ++e) {
                int h = e >> 1;
                float pe = sc[j][e] == -INFINITY ? 0.f : __expf(sc[j][e] - m_use[h]);
                sc[j][e] = pe;
                psum[h] += pe;
            }
            if (LOW8) sc[j][2] = sc[j][3] = 0.f;
        }
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 1);
            psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 2);
            l_run[h] = l_run[h] * alpha[h] + psum[h];
        }
#pragma unroll
        for (int j = 0; j < NT_O; ++j) {
            o_acc[j][0] *= alpha[0];
            o_acc[j][1] *= alpha[0];
            if (!LOW8) {
                o_acc[j][2] *= alpha[1];
                o_acc[j][3] *= alpha[1];
            }
        }
        uint32_t pf[4] = {pack_half2(sc[0][0], sc[0][1]), LOW8 ? 0u : pack_half2(sc[0][2], sc[0][3]), pack_half2(sc[1][0], sc[1][1]),
                          LOW8 ? 0u : pack_half2(sc[1][2], sc[1][3])};
#pragma unroll
        for (int j = 0; j < NT_O; j += 2) {
            uint32_t bf[4];
            ldmatrix_x4_trans(bf, vt + ((lane & 7) + ((lane >> 3) & 1) * 8) * DP + j * 8 + (lane >> 4) * 8);
            mma16816(o_acc[j], pf, bf[0], bf[1]);
            mma16816(o_acc[j + 1], pf, bf[2], bf[3]);
        }
        __syncwarp();  // the stage is refilled by the next iteration's load
    }
    cp_async_wait<0>();
    __syncwarp();

    // each warp leaves (max, sum, output) of its live rows in its own ring, then everyone merges
    float* w_o = reinterpret_cast<float*>(ring);            // [16][D]
    float* w_ml = w_o + 16 * D;                              // [16][2]
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        int item = gid + 8 * h;
        if (item >= g) continue;
#pragma unroll
        for (int j = 0; j < NT_O; ++j)
            *reinterpret_cast<float2*>(w_o + item * D + j * 8 + 2 * tq) = make_float2(o_acc[j][2 * h], o_acc[j][2 * h + 1]);
        if (tq == 0) {
            w_ml[item * 2] = m_run[h];
            w_ml[item * 2 + 1] = l_run[h];
        }
    }
    __syncthreads();
    const int64_t slot = ((int64_t)blockIdx.x * a.kv_heads + kvh) * 16;
    // merged, normalised outputs of this (lane, KV head): g * D consecutive values of the lane's output row
    // (all threads of the CTA call this together; the query tile is dead by now and lends its shared memory: g * D
    // floats fit in it for up to eight query heads per KV head)
    float* stage = reinterpret_cast<float*>(Qs);
    auto finish = [&](auto&& value_of) {
        const int64_t row = q_off;
        const int col0 = kvh * g * D;
        const bool fuse_quant = a.qout.qs != nullptr;  // uniform
        if (!fuse_quant) {
            for (int idx = tid; idx < g * D; idx += 128) {
                float v = value_of(idx);
                if (a.out != nullptr) a.out[row * a.q_heads * D + col0 + idx] = v;
                if (a.out_h != nullptr) a.out_h[row * a.q_heads * D + col0 + idx] = __float2half_rn(v);
            }
            return;
        }
        for (int idx = tid; idx < g * D; idx += 128) {
            float v = value_of(idx);
            stage[idx] = v;
            if (a.out != nullptr) a.out[row * a.q_heads * D + col0 + idx] = v;
        }
        __syncthreads();
        // one warp per 256-wide group, eight consecutive values per lane (g * D is a multiple of 256 here)
        for (int grp = warp; grp < g * D / 256; grp += 4) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = stage[grp * 256 + lane * 8 + i];
            quant_group(v, lane, a.qkind, a.qout, row, a.q_heads * D, col0 / 256 + grp);
        }
    };
    auto merged_local = [&](int idx, float& m_out, float& l_out) {
        int item = idx / D, c = idx - item * D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, reinterpret_cast<const float*>(rings + w * RING_HALVES)[16 * D + item * 2]);
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float* ro = reinterpret_cast<const float*>(rings + w * RING_HALVES);
            float mw = ro[16 * D + item * 2];
            if (mw != -INFINITY) {
                float f = __expf(mw - m);
                l += ro[16 * D + item * 2 + 1] * f;
                o += ro[item * D + c] * f;
            }
        }
        m_out = m;
        l_out = l;
        return o;
    };
    if (n_splits == 1) {
        finish([&](int idx) {
            float m, l;
            float o = merged_local(idx, m, l);
            return o / l;
        });
    } else {
        for (int idx = tid; idx < g * D; idx += 128) {
            int item = idx / D, c = idx - item * D;
            float m, l;
            float o = merged_local(idx, m, l);
            a.part_o[(slot + item) * D + c] = o;
            if (c == 0) {
                a.part_ml[(slot + item) * 2] = m;
                a.part_ml[(slot + item) * 2 + 1] = l;
            }
        }
        // The lane's keys were shared out over several CTAs: the CTA that arrives last at the lane's counter adds
        // the shares in share order (so the result does not depend on which one that is) and resets the counter.
        __shared__ int s_last;
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            int prev = atomicAdd(&a.counters[lane_id * a.kv_heads + kvh], 1);
            s_last = prev == n_splits - 1 ? 1 : 0;
            if (prev == n_splits - 1) a.counters[lane_id * a.kv_heads + kvh] = 0;
        }
        __syncthreads();
        if (s_last) {
            __threadfence();
            finish([&](int idx) {
                int item = idx / D, c = idx - item * D;
                float m = -INFINITY;
                for (int sp = 0; sp < n_splits; ++sp)
                    m = fmaxf(m, __ldcg(a.part_ml + (((int64_t)(first_entry + sp) * a.kv_heads + kvh) * 16 + item) * 2));
                float l = 0.f, o = 0.f;
                for (int sp = 0; sp < n_splits; ++sp) {
                    const int64_t ps = ((int64_t)(first_entry + sp) * a.kv_heads + kvh) * 16 + item;
                    float ms = __ldcg(a.part_ml + ps * 2);
                    if (ms != -INFINITY) {
                        float f = __expf(ms - m);
                        l += __ldcg(a.part_ml + ps * 2 + 1) * f;
                        o += __ldcg(a.part_o + ps * D + c) * f;
                    }
                }
                return o / l;
            });
        }
    }
}

// Merge the key shares of one-token lanes: grid (decode lane, kv head), one warp per query head of the group.
__global__ void attn_combine_kernel(AttnTcArgs a, int D) {
    pdl_trigger();
    pdl_wait();
    const int dl = blockIdx.x, kvh = blockIdx.y;
    const int lane_id = a.dec_lanes[3 * dl], first = a.dec_lanes[3 * dl + 1], n_splits = a.dec_lanes[3 * dl + 2];
    const int g = a.q_heads / a.kv_heads;
    const int hq = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (hq >= g) return;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, a.part_ml[(((int64_t)(first + s) * a.kv_heads + kvh) * 16 + hq) * 2]);
    float l = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float* ml = a.part_ml + (((int64_t)(first + s) * a.kv_heads + kvh) * 16 + hq) * 2;
        if (ml[0] != -INFINITY) l += ml[1] * __expf(ml[0] - m);
    }
    const int q_off = a.cu_seqlens[lane_id];
    float* o = a.out + (int64_t)q_off * a.q_heads * D + (kvh * g + hq) * D;
    for (int c = lane; c < D; c += 32) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            int64_t slot = ((int64_t)(first + s) * a.kv_heads + kvh) * 16 + hq;
            float ms = a.part_ml[slot * 2];
            if (ms != -INFINITY) acc += a.part_o[slot * D + c] * __expf(ms - m);
        }
        o[c] = acc / l;
    }
}

template <int D, int WARPS, int KT, bool SPLIT>
void launch_variant(const AttnTcArgs& a, int n_work, cudaStream_t s) {
    constexpr size_t smem = (size_t)(16 * WARPS + 4 * KT) * (D + 8) * sizeof(__half);
    ensure_dynamic_smem(reinterpret_cast<const void*>(&attn_tc_kernel<D, WARPS, KT, SPLIT>), smem);
    dim3 grid((unsigned)n_work, (unsigned)a.kv_heads);
    launch_pdl(attn_tc_kernel<D, WARPS, KT, SPLIT>, grid, dim3(WARPS * 32), smem, s, a);
    MK_LAUNCH_CHECK();
}

template <int D>
void launch_for_dim(const AttnTcArgs& a, int warps, cudaStream_t s) {
    if (a.n_tiles > 0) {
        if (warps == 8) launch_variant<D, 8, 64, false>(a, a.n_tiles, s);
        else launch_variant<D, 4, 32, false>(a, a.n_tiles, s);  // 32-key tiles: half the shared memory, twice the CTAs per SM (measured +0.4 % on the whole benchmark)
    }
    if (a.n_entries > 0) {
        constexpr int STAGES = D >= 256 ? 2 : 3;
        constexpr size_t smem = (size_t)(16 + 4 * STAGES * 2 * 16) * (D + 8) * sizeof(__half);
        ensure_dynamic_smem(reinterpret_cast<const void*>(&attn_decode_kernel<D, STAGES, true>), smem);
        ensure_dynamic_smem(reinterpret_cast<const void*>(&attn_decode_kernel<D, STAGES, false>), smem);
        dim3 grid((unsigned)a.n_entries, (unsigned)a.kv_heads);
        if (a.q_heads / a.kv_heads <= 8) launch_pdl(attn_decode_kernel<D, STAGES, true>, grid, dim3(128), smem, s, a);
        else launch_pdl(attn_decode_kernel<D, STAGES, false>, grid, dim3(128), smem, s, a);
        MK_LAUNCH_CHECK();
    }
    if (a.n_dec_lanes > 0) {  // lanes whose keys were shared out over several CTAs
        dim3 grid((unsigned)a.n_dec_lanes, (unsigned)a.kv_heads);
        launch_pdl(attn_combine_kernel, grid, dim3(32 * (a.q_heads / a.kv_heads)), 0, s, a, (int)D);
        MK_LAUNCH_CHECK();
    }
}

}  // namespace

bool attention_tc_supported(int q_heads, int kv_heads, int head_dim, int block_tokens, bool kv_f16) {
    int g = kv_heads > 0 ? q_heads / kv_heads : 0;
    if (block_tokens < 16 || (block_tokens & (block_tokens - 1)) != 0) return false;  // pages hold whole 16-key tiles
    return kv_f16 && (head_dim == 64 || head_dim == 128 || head_dim == 256) && (g == 1 || g == 2 || g == 4 || g == 8) &&
           q_heads == g * kv_heads;
}

// Eight warps (128 (row, head) items per CTA) for groups of eight query heads, else four: with four heads per group
// eight warps measured slower (fewer, longer CTAs) than four.
int attention_tc_warps(int q_heads, int kv_heads) { return q_heads / kv_heads == 8 ? 8 : 4; }

int attention_tc_tile_rows(int q_heads, int kv_heads) { return 16 * attention_tc_warps(q_heads, kv_heads) / (q_heads / kv_heads); }

int attention_tc_max_entries(int lanes, int kv_heads) { return std::max(lanes + lanes / 2, kAttnTargetCtas / std::max(1, kv_heads)) + 1; }

void plan_attention_tc(const int32_t* start_pos, const int32_t* n_tokens, const int32_t* n_blocks, int lanes, int q_heads,
                       int kv_heads, AttnTcPlan& plan) {
    plan.tiles.clear();
    plan.entries.clear();
    plan.dec_lanes.clear();
    const int tile_rows = attention_tc_tile_rows(q_heads, kv_heads);
    // One-token lanes: every CTA should walk about the same number of keys, and all CTAs should fit on the GPU at
    // once.  Share size = total keys / CTA slots per KV head, raised until the shares of all lanes fit.
    int n_dec = 0;
    int64_t total_keys = 0;
    for (int i = 0; i < lanes; ++i)
        if (n_tokens[i] == 1) { ++n_dec; total_keys += start_pos[i] + 1; }
    // Once the lanes alone give every SM a CTA, sharing keys out only adds merge work and repeated query preparation
    // (measured at 64 lanes x 4 KV heads with histories within twice their mean: +1.4 % on the whole benchmark
    // without shares).  Then only a lane more than twice as long as the mean is cut, so that one long history among
    // many short ones does not set the length of the launch.
    const bool filled = n_dec * kv_heads >= kPlanSms;
    const int slots = filled ? n_dec + n_dec / 2 : std::max(n_dec, kAttnTargetCtas / std::max(1, kv_heads));
    int share = (int)std::max<int64_t>(kAttnMinSplitKeys, filled ? 2 * (total_keys / std::max(1, n_dec)) : (total_keys + slots - 1) / std::max(1, slots));
    share = (share + 63) / 64 * 64;
    auto shares_of = [&](int ctx) { return std::max(1, std::min(kAttnMaxSplits, (ctx + share - 1) / share)); };
    for (;;) {
        int64_t ctas = 0;
        for (int i = 0; i < lanes; ++i)
            if (n_tokens[i] == 1) ctas += shares_of(start_pos[i] + 1);
        if (ctas <= slots || share > (1 << 20)) break;
        share += 64;
    }
    int q_off = 0, table_off = 0;
    for (int i = 0; i < lanes; q_off += n_tokens[i], table_off += n_blocks[i], ++i) {
        if (n_tokens[i] == 1) {
            const int splits = shares_of(start_pos[i] + 1);
            const int first = plan.n_entries();
            for (int sidx = 0; sidx < splits; ++sidx) {
                const int32_t rec[8] = {i, sidx, splits, start_pos[i], table_off, q_off, first, 0};
                plan.entries.insert(plan.entries.end(), rec, rec + 8);
            }
        } else {
            for (int r0 = 0; r0 < n_tokens[i]; r0 += tile_rows) {
                plan.tiles.push_back(i);
                plan.tiles.push_back(r0);
            }
        }
    }
}

int launch_paged_attention_tc(const AttnTcArgs& a_in, cudaStream_t s) {
    AttnTcArgs a = a_in;
    if (!attention_tc_supported(a.q_heads, a.kv_heads, a.d, a.block_tokens, true))
        throw std::runtime_error("launch_paged_attention_tc: unsupported shape");
    if (a.out == nullptr && a.out_h == nullptr && a.qout.qs == nullptr) throw std::runtime_error("launch_paged_attention_tc: no output");
    if (a.out == nullptr && a.n_dec_lanes > 0) throw std::runtime_error("launch_paged_attention_tc: the separate merge pass writes f32 rows");
    a.bt_shift = 0;
    while ((1 << a.bt_shift) < a.block_tokens) ++a.bt_shift;
    int warps = attention_tc_warps(a.q_heads, a.kv_heads);
    switch (a.d) {
        case 64: launch_for_dim<64>(a, warps, s); break;
        case 128: launch_for_dim<128>(a, warps, s); break;
        case 256: launch_for_dim<256>(a, warps, s); break;
        default: throw std::runtime_error("launch_paged_attention_tc: unsupported head_dim");
    }
    return (a.n_tiles > 0 ? 1 : 0) + (a.n_entries > 0 ? 1 : 0) + (a.n_dec_lanes > 0 ? 1 : 0);
}

}  // namespace mk
