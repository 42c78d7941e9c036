// Activation preparation kernels: residual add + RMSNorm + 8-bit block quantisation, and the
// gated-activation product of the feed-forward, both ending in the block format the integer
// matmul kernels consume.
//
// The quantisation rule restates the published GGML activation formats used by the reference's
// CPU matmul (LinearOp::forward, src/model_weights.rs:346-377, which hands an f32 row to the
// quantised matmul): blocks of 256 with an f32 scale chosen so the element of largest magnitude
// maps to -128 (clamped to 127) for K-quant weights, blocks of 32 with an f16 scale amax/127 for
// Q8_0 weights.  RMSNorm follows src/model_weights.rs:563-565: x / sqrt(mean(x^2) + eps) * w.
#include "kernels.h"
#include "quant_blocks.cuh"

namespace mk {

namespace {

constexpr int NQ_THREADS = 256;

// Quantise the row held in shared memory `row[0..dim)`.
__device__ void quantize_row_q8k(const float* row, int dim, int8_t* qs, float* d, int16_t* bsums, __half* xh) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int b = warp; b < dim / 256; b += nw) {
        const float* xb = row + b * 256 + lane * 8;
        float v[8];
        float amax = 0.f;
        int idx = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = xb[i];
            float ax = fabsf(v[i]);
            if (ax > amax) { amax = ax; idx = lane * 8 + i; }
        }
        // largest magnitude, lowest index on ties
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float oa = __shfl_xor_sync(0xffffffffu, amax, o);
            int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (oa > amax || (oa == amax && oi < idx)) { amax = oa; idx = oi; }
        }
        int8_t q[8];
        int sum = 0;
        float dd = 0.f;
        if (amax == 0.f) {
#pragma unroll
            for (int i = 0; i < 8; ++i) q[i] = 0;
        } else {
            float mx = row[b * 256 + idx];
            float iscale = -128.f / mx;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float r = roundf(iscale * v[i]);
                q[i] = (int8_t)(r > 127.f ? 127.f : r);
                sum += q[i];
            }
            dd = 1.0f / iscale;
        }
        int2 packed;
        packed.x = (uint8_t)q[0] | ((uint8_t)q[1] << 8) | ((uint8_t)q[2] << 16) | ((uint32_t)(uint8_t)q[3] << 24);
        packed.y = (uint8_t)q[4] | ((uint8_t)q[5] << 8) | ((uint8_t)q[6] << 16) | ((uint32_t)(uint8_t)q[7] << 24);
        *reinterpret_cast<int2*>(qs + b * 256 + lane * 8) = packed;
        if (xh != nullptr) {
            __half2 hv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                hv[i] = __floats2half2_rn(__fmul_rn(dd, (float)q[2 * i]), __fmul_rn(dd, (float)q[2 * i + 1]));
            *reinterpret_cast<uint4*>(xh + b * 256 + lane * 8) = *reinterpret_cast<uint4*>(hv);
        }
        int pair = sum + __shfl_xor_sync(0xffffffffu, sum, 1);
        if ((lane & 1) == 0) bsums[b * 16 + (lane >> 1)] = (int16_t)pair;
        if (lane == 0) d[b] = dd;
    }
}

__device__ void quantize_row_q80(const float* row, int dim, int8_t* qs, float* d, __half* xh) {
    // 8 lanes per 32-element block, 4 elements per lane
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int b0 = warp * 4; b0 < dim / 32; b0 += nw * 4) {
        int b = b0 + (lane >> 3);
        bool live = b < dim / 32;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        float amax = 0.f;
        if (live) {
#pragma unroll
            for (int i = 0; i < 4; ++i) { v[i] = row[b * 32 + (lane & 7) * 4 + i]; amax = fmaxf(amax, fabsf(v[i])); }
        }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        float dd = amax / 127.f;
        float id = dd != 0.f ? 1.0f / dd : 0.f;
        if (live) {
            uint32_t p = 0;
            float ddh = __half2float(__float2half_rn(dd));
            __half2 hv[2];
            int8_t qv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { qv[i] = (int8_t)roundf(v[i] * id); p |= (uint32_t)(uint8_t)qv[i] << (8 * i); }
            *reinterpret_cast<uint32_t*>(qs + b * 32 + (lane & 7) * 4) = p;
            if (xh != nullptr) {
                hv[0] = __floats2half2_rn(__fmul_rn(ddh, (float)qv[0]), __fmul_rn(ddh, (float)qv[1]));
                hv[1] = __floats2half2_rn(__fmul_rn(ddh, (float)qv[2]), __fmul_rn(ddh, (float)qv[3]));
                *reinterpret_cast<uint2*>(xh + b * 32 + (lane & 7) * 4) = *reinterpret_cast<uint2*>(hv);
            }
            if ((lane & 7) == 0) d[b] = ddh;
        }
    }
}

__device__ __forceinline__ void quantize_row(const float* row, int dim, int kind, const ActQ& out, int r) {
    if (out.qs == nullptr) return;
    if (kind == ACT_Q8K)
        quantize_row_q8k(row, dim, out.qs + (int64_t)r * dim, out.d + (int64_t)r * (dim / 256),
                         out.bsums + (int64_t)r * (dim / 16), out.xh ? out.xh + (int64_t)r * dim : nullptr);
    else
        quantize_row_q80(row, dim, out.qs + (int64_t)r * dim, out.d + (int64_t)r * (dim / 32),
                         out.xh ? out.xh + (int64_t)r * dim : nullptr);
}

__global__ void __launch_bounds__(NQ_THREADS) add_norm_quant_kernel(NormQuantArgs a) {
    extern __shared__ float smem[];
    float* row = smem;                 // [dim]
    __shared__ float red[32];
    int r = blockIdx.x;
    int src = a.row_index ? a.row_index[r] : r;
    float* h = a.h + (int64_t)src * a.dim;
    const int dim = a.dim;

    if (a.a != nullptr) {
        const float* av = a.a + (int64_t)src * dim;
        auto a_at = [&](int k) {
            float x = av[k];
            for (int sp = 1; sp < a.a_splits; ++sp) x += av[(int64_t)sp * a.a_split_stride + k];
            return x;
        };
        float post_m = 1.f;
        if (a.post_w != nullptr) {
            float ss = 0.f;
            for (int k = threadIdx.x; k < dim; k += blockDim.x) { float x = a_at(k); ss += x * x; }
            ss = block_sum(ss, red);
            post_m = sqrtf(ss / (float)dim + a.eps);
        }
        for (int k = threadIdx.x; k < dim; k += blockDim.x) {
            float x = a_at(k);
            if (a.post_w != nullptr) x = x / post_m * a.post_w[k];
            float hv = h[k] + x * a.a_scale;
            row[k] = hv;
            if (a.row_index == nullptr) h[k] = hv;
        }
    } else {
        for (int k = threadIdx.x; k < dim; k += blockDim.x) row[k] = h[k];
    }
    __syncthreads();
    if (a.norm_w != nullptr) {
        float ss = 0.f;
        for (int k = threadIdx.x; k < dim; k += blockDim.x) { float x = row[k]; ss += x * x; }
        ss = block_sum(ss, red);
        float m = sqrtf(ss / (float)dim + a.eps);
        for (int k = threadIdx.x; k < dim; k += blockDim.x) row[k] = row[k] / m * a.norm_w[k];
        __syncthreads();
    }
    if (a.normed_out != nullptr)
        for (int k = threadIdx.x; k < dim; k += blockDim.x) a.normed_out[(int64_t)r * dim + k] = row[k];
    quantize_row(row, dim, a.act_kind, a.out, r);
}

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float gelu_tanh_f(float v) {
    return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * v * (1.0f + 0.044715f * v * v)));
}

__global__ void __launch_bounds__(NQ_THREADS) actmul_quant_kernel(const float* gate, const float* up, int ld, int F,
                                                                   int act, int kind, ActQ out, float* f32_out) {
    extern __shared__ float smem[];
    float* row = smem;
    int r = blockIdx.x;
    const float* g = gate + (int64_t)r * ld;
    const float* u = up + (int64_t)r * ld;
    for (int k = threadIdx.x; k < F; k += blockDim.x) {
        float gv = g[k];
        float a = act == 0 ? silu_f(gv) : gelu_tanh_f(gv);
        float v = a * u[k];
        row[k] = v;
        if (f32_out) f32_out[(int64_t)r * F + k] = v;
    }
    __syncthreads();
    quantize_row(row, F, kind, out, r);
}

__global__ void add_inplace_kernel(float* h, const float* a, float scale, int64_t n) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) h[i] = h[i] + a[i] * scale;
}


// One CTA per row, NG groups of 256 per warp held in registers (dim <= 8 warps * NG * 256).
template <int NG>
__global__ void __launch_bounds__(NQ_THREADS) add_norm_quant_fast_kernel(NormQuantArgs a) {
    __shared__ float red[32];
    pdl_trigger();
    const int r = blockIdx.x;
    const int dim = a.dim, groups = dim / 256;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // the norm weights never depend on the predecessor kernel: fetch them while it finishes
    float nw[NG][8], pw[NG][8];
#pragma unroll
    for (int g = 0; g < NG; ++g) {
        const int grp = warp + g * 8;
        if (grp < groups && a.norm_w != nullptr) load8(a.norm_w + grp * 256 + lane * 8, nw[g]);
        if (grp < groups && a.post_w != nullptr && a.a != nullptr) load8(a.post_w + grp * 256 + lane * 8, pw[g]);
    }
    pdl_wait();
    const int src = a.row_index ? a.row_index[r] : r;
    float* h = a.h + (int64_t)src * dim;
    float x[NG][8];
    bool live[NG];
#pragma unroll
    for (int g = 0; g < NG; ++g) {
        int grp = warp + g * 8;
        live[g] = grp < groups;
        if (live[g]) load8(h + grp * 256 + lane * 8, x[g]);
        else {
#pragma unroll
            for (int i = 0; i < 8; ++i) x[g][i] = 0.f;
        }
    }
    if (a.a != nullptr) {
        const float* av = a.a + (int64_t)src * dim;
        float y[NG][8];
        float ss = 0.f;
#pragma unroll
        for (int g = 0; g < NG; ++g) {
            if (live[g]) {
                load8(av + (warp + g * 8) * 256 + lane * 8, y[g]);
#pragma unroll 4
                for (int sp = 1; sp < a.a_splits; ++sp) {
                    float part[8];
                    load8(av + (int64_t)sp * a.a_split_stride + (warp + g * 8) * 256 + lane * 8, part);
#pragma unroll
                    for (int i = 0; i < 8; ++i) y[g][i] += part[i];
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) y[g][i] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += y[g][i] * y[g][i];
        }
        float post_m = 1.f;
        if (a.post_w != nullptr) {
            ss = block_sum(ss, red);
            post_m = sqrtf(ss / (float)dim + a.eps);
        }
#pragma unroll
        for (int g = 0; g < NG; ++g) {
            if (!live[g]) continue;
            int base = (warp + g * 8) * 256 + lane * 8;
            if (a.post_w != nullptr) {
#pragma unroll
                for (int i = 0; i < 8; ++i) y[g][i] = y[g][i] / post_m * pw[g][i];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) x[g][i] = x[g][i] + y[g][i] * a.a_scale;
            if (a.row_index == nullptr) store8(h + base, x[g]);
        }
    }
    if (a.norm_w != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int g = 0; g < NG; ++g)
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += x[g][i] * x[g][i];
        ss = block_sum(ss, red);
        float m = sqrtf(ss / (float)dim + a.eps);
#pragma unroll
        for (int g = 0; g < NG; ++g) {
            if (!live[g]) continue;
#pragma unroll
            for (int i = 0; i < 8; ++i) x[g][i] = x[g][i] / m * nw[g][i];
        }
    }
#pragma unroll
    for (int g = 0; g < NG; ++g) {
        if (!live[g]) continue;  // uniform per warp
        int grp = warp + g * 8;
        if (a.normed_out != nullptr) store8(a.normed_out + (int64_t)r * dim + grp * 256 + lane * 8, x[g]);
        quant_group(x[g], lane, a.act_kind, a.out, r, dim, grp);
    }
}

// Rows that need no row-wide statistic: one warp per (row, 256-value group), any number of rows.
__global__ void __launch_bounds__(NQ_THREADS) quant_groups_kernel(const float* x, int ld, int rows, int dim, int kind, ActQ out) {
    const int groups = dim / 256;
    pdl_trigger();
    pdl_wait();
    const int64_t wid = (int64_t)blockIdx.x * (NQ_THREADS / 32) + (threadIdx.x >> 5);
    if (wid >= (int64_t)rows * groups) return;
    const int r = (int)(wid / groups), grp = (int)(wid - (int64_t)r * groups), lane = threadIdx.x & 31;
    float v[8];
    load8(x + (int64_t)r * ld + grp * 256 + lane * 8, v);
    quant_group(v, lane, kind, out, r, dim, grp);
}

__global__ void __launch_bounds__(NQ_THREADS) actmul_quant_groups_kernel(const float* gate, const float* up, int ld, int rows, int F,
                                                                          int act, int kind, ActQ out, float* f32_out, int splits,
                                                                          int64_t split_stride) {
    const int groups = F / 256;
    pdl_trigger();
    pdl_wait();
    const int64_t wid = (int64_t)blockIdx.x * (NQ_THREADS / 32) + (threadIdx.x >> 5);
    if (wid >= (int64_t)rows * groups) return;
    const int r = (int)(wid / groups), grp = (int)(wid - (int64_t)r * groups), lane = threadIdx.x & 31;
    float g[8], u[8], v[8];
    load8(gate + (int64_t)r * ld + grp * 256 + lane * 8, g);
    load8(up + (int64_t)r * ld + grp * 256 + lane * 8, u);
#pragma unroll 4
    for (int sp = 1; sp < splits; ++sp) {
        float pg[8], pu[8];
        load8(gate + sp * split_stride + (int64_t)r * ld + grp * 256 + lane * 8, pg);
        load8(up + sp * split_stride + (int64_t)r * ld + grp * 256 + lane * 8, pu);
#pragma unroll
        for (int i = 0; i < 8; ++i) { g[i] += pg[i]; u[i] += pu[i]; }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (act == 0 ? silu_f(g[i]) : gelu_tanh_f(g[i])) * u[i];
    if (f32_out) store8(f32_out + (int64_t)r * F + grp * 256 + lane * 8, v);
    quant_group(v, lane, kind, out, r, F, grp);
}

}  // namespace

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

void launch_add_norm_quant(const NormQuantArgs& a, cudaStream_t s) {
    if (a.rows <= 0) return;
    const bool vec_ok = a.dim % 256 == 0 && aligned16(a.h) && aligned16(a.a) && aligned16(a.post_w) && aligned16(a.norm_w) &&
                        aligned16(a.normed_out) && aligned16(a.out.xh) && (reinterpret_cast<uintptr_t>(a.out.qs) & 7) == 0;
    if (vec_ok && a.a == nullptr && a.norm_w == nullptr && a.row_index == nullptr && a.normed_out == nullptr) {
        // plain quantisation: no row-wide dependency
        int64_t warps = (int64_t)a.rows * (a.dim / 256);
        launch_pdl(quant_groups_kernel, dim3((unsigned)((warps + 7) / 8)), dim3(NQ_THREADS), 0, s, (const float*)a.h, a.dim, a.rows, a.dim, a.act_kind, a.out);
        MK_LAUNCH_CHECK();
        return;
    }
    if (vec_ok && a.dim <= 8 * 4 * 256) {
        int ng = (a.dim / 256 + 7) / 8;
        if (ng == 1) launch_pdl(add_norm_quant_fast_kernel<1>, dim3(a.rows), dim3(NQ_THREADS), 0, s, a);
        else if (ng == 2) launch_pdl(add_norm_quant_fast_kernel<2>, dim3(a.rows), dim3(NQ_THREADS), 0, s, a);
        else launch_pdl(add_norm_quant_fast_kernel<4>, dim3(a.rows), dim3(NQ_THREADS), 0, s, a);
        MK_LAUNCH_CHECK();
        return;
    }
    size_t smem = (size_t)a.dim * sizeof(float);
    ensure_dynamic_smem(reinterpret_cast<const void*>(&add_norm_quant_kernel), smem);
    add_norm_quant_kernel<<<a.rows, NQ_THREADS, smem, s>>>(a);
    MK_LAUNCH_CHECK();
}

void launch_actmul_quant(const float* gate, const float* up, int ld, int T, int F, int act, int act_kind, ActQ out,
                         float* f32_out, cudaStream_t s, int splits, int64_t split_stride) {
    if (T <= 0) return;
    if (splits > 1 && !(F % 256 == 0 && ld % 4 == 0 && split_stride % 4 == 0 && aligned16(gate) && aligned16(up)))
        throw std::runtime_error("launch_actmul_quant: split inputs need 256-wide, 16-byte aligned rows");
    if (F % 256 == 0 && ld % 4 == 0 && aligned16(gate) && aligned16(up) && aligned16(f32_out) && aligned16(out.xh) &&
        (reinterpret_cast<uintptr_t>(out.qs) & 7) == 0) {
        int64_t warps = (int64_t)T * (F / 256);
        launch_pdl(actmul_quant_groups_kernel, dim3((unsigned)((warps + 7) / 8)), dim3(NQ_THREADS), 0, s, gate, up, ld, T, F, act, act_kind, out,
                   f32_out, splits, split_stride);
        MK_LAUNCH_CHECK();
        return;
    }
    size_t smem = (size_t)F * sizeof(float);
    ensure_dynamic_smem(reinterpret_cast<const void*>(&actmul_quant_kernel), smem);
    actmul_quant_kernel<<<T, NQ_THREADS, smem, s>>>(gate, up, ld, F, act, act_kind, out, f32_out);
    MK_LAUNCH_CHECK();
}

void launch_add_inplace(float* h, const float* a, float scale, int64_t n, cudaStream_t s) {
    if (n <= 0) return;
    add_inplace_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(h, a, scale, n);
    MK_LAUNCH_CHECK();
}

}  // namespace mk
