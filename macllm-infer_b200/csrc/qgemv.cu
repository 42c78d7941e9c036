// Quantised matrix-vector kernels for decode rows: y[t][n] = sum_k x[t][k] * W[n][k].
//
// Replaces, on this path, the reference's LinearOp::Quantized forward
// (src/model_weights.rs:346-377 -> candle QMatMul): weights stay in their GGUF block format in
// HBM (block sizes src/gguf.rs:386-408), activations arrive as 8-bit blocks, and every block dot
// product is an exact integer sum (dp4a) scaled in f32 - the arithmetic of the reference's CPU path.
//
// Memory plan: one warp owns one output row and streams that row's blocks with 128-bit (Q4_K,
// Q8_0) or 64-bit (Q6_K planes) loads, eight lanes per 256-weight block, so a warp consumes whole
// 128-byte lines; activations (T*K bytes) are re-read from L1/L2.  Each weight byte leaves HBM once
// per call when T <= ROWS_PER_PASS; larger T re-walks the row from cache in passes.
#include "kernels.h"

namespace mk {

namespace {

constexpr int GEMV_WARPS = 4;
constexpr int NT = 8;  // activation rows per pass

// Optional expert grouping: blockIdx.y selects the expert, whose output rows are [offsets[e], offsets[e+1]).
struct Group {
    const int32_t* offsets = nullptr;
    const int32_t* src_row = nullptr;
};
__device__ __forceinline__ void group_range(const Group& g, int T, int& t_begin, int& t_end) {
    if (g.offsets != nullptr) { t_begin = g.offsets[blockIdx.y]; t_end = g.offsets[blockIdx.y + 1]; }
    else { t_begin = 0; t_end = T; }
}
__device__ __forceinline__ int src_of(const Group& g, int t) { return g.src_row != nullptr ? g.src_row[t] : t; }

__device__ __forceinline__ void q4k_scale_min(const uint8_t* s, int j, int& sc, int& mn) {
    if (j < 4) {
        sc = s[j] & 63;
        mn = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4);
        mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

template <int ROWS>
__device__ __forceinline__ void finish_rows(float (&acc)[NT], int n, int t0, int T, float* y, int ldy, float out_scale,
                                            float softcap) {
#pragma unroll
    for (int t = 0; t < ROWS; ++t) {
        float v = warp_sum(acc[t]);
        if ((threadIdx.x & 31) == 0 && t0 + t < T) {
            v *= out_scale;
            if (softcap != 0.f) v = tanhf(v * (1.0f / softcap)) * softcap;
            y[(int64_t)(t0 + t) * ldy + n] = v;
        }
    }
}

// ---------------------------------------------------------------- Q4_K
__global__ void __launch_bounds__(GEMV_WARPS * 32) qgemv_q4k_kernel(const uint8_t* __restrict__ W, int nb, int out,
                                                                    const int8_t* __restrict__ xq,
                                                                    const float* __restrict__ xd,
                                                                    const int16_t* __restrict__ xbs, int T,
                                                                    float* __restrict__ y, int ldy, float out_scale,
                                                                    float softcap, Group grp) {
    int n = blockIdx.x * GEMV_WARPS + (threadIdx.x >> 5);
    if (n >= out) return;
    int lane = threadIdx.x & 31;
    int part = lane & 7;       // 16-byte slice of the 128 nibble bytes
    int j = part >> 1;         // 64-weight chunk
    int h = part & 1;          // half of the chunk's 32 bytes
    const int K = nb * 256;
    const uint8_t* wrow = W + ((int64_t)blockIdx.y * out + n) * nb * 144;
    int t_first;
    group_range(grp, T, t_first, T);

    for (int t0 = t_first; t0 < T; t0 += NT) {
        float acc[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t] = 0.f;
        int rows = min(NT, T - t0);
        for (int ib = lane >> 3; ib < nb; ib += 4) {
            const uint8_t* blk = wrow + (int64_t)ib * 144;
            uint4 q = *reinterpret_cast<const uint4*>(blk + 16 + 16 * part);
            uint32_t dm = *reinterpret_cast<const uint32_t*>(blk);
            float d = __half2float(__ushort_as_half((unsigned short)(dm & 0xFFFF)));
            float dmin = __half2float(__ushort_as_half((unsigned short)(dm >> 16)));
            int sc_lo, m_lo, sc_hi, m_hi;
            q4k_scale_min(blk + 4, 2 * j, sc_lo, m_lo);
            q4k_scale_min(blk + 4, 2 * j + 1, sc_hi, m_hi);
            uint32_t ql[4] = {q.x & 0x0F0F0F0Fu, q.y & 0x0F0F0F0Fu, q.z & 0x0F0F0F0Fu, q.w & 0x0F0F0F0Fu};
            uint32_t qh[4] = {(q.x >> 4) & 0x0F0F0F0Fu, (q.y >> 4) & 0x0F0F0F0Fu, (q.z >> 4) & 0x0F0F0F0Fu,
                              (q.w >> 4) & 0x0F0F0F0Fu};
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                if (t < rows) {
                    const int64_t xrow = src_of(grp, t0 + t);
                    const int8_t* xr = xq + xrow * K + ib * 256 + 64 * j + 16 * h;
                    int4 xl = *reinterpret_cast<const int4*>(xr);
                    int4 xh = *reinterpret_cast<const int4*>(xr + 32);
                    int s_lo = __dp4a((int)ql[0], xl.x, 0);
                    s_lo = __dp4a((int)ql[1], xl.y, s_lo);
                    s_lo = __dp4a((int)ql[2], xl.z, s_lo);
                    s_lo = __dp4a((int)ql[3], xl.w, s_lo);
                    int s_hi = __dp4a((int)qh[0], xh.x, 0);
                    s_hi = __dp4a((int)qh[1], xh.y, s_hi);
                    s_hi = __dp4a((int)qh[2], xh.z, s_hi);
                    s_hi = __dp4a((int)qh[3], xh.w, s_hi);
                    const int16_t* bs = xbs + xrow * (K / 16) + ib * 16 + 4 * j + h;
                    int isum = sc_lo * s_lo + sc_hi * s_hi;
                    int msum = m_lo * (int)bs[0] + m_hi * (int)bs[2];
                    acc[t] += xd[xrow * nb + ib] * (d * (float)isum - dmin * (float)msum);
                }
            }
        }
        finish_rows<NT>(acc, n, t0, T, y, ldy, out_scale, softcap);
    }
}

// ---------------------------------------------------------------- Q6_K (planar layout)
__global__ void __launch_bounds__(GEMV_WARPS * 32) qgemv_q6k_kernel(const uint8_t* __restrict__ ql_p,
                                                                    const uint8_t* __restrict__ qh_p,
                                                                    const int8_t* __restrict__ sc_p,
                                                                    const __half* __restrict__ d_p, int nb, int out,
                                                                    const int8_t* __restrict__ xq,
                                                                    const float* __restrict__ xd, int T,
                                                                    float* __restrict__ y, int ldy, float out_scale,
                                                                    float softcap, Group grp) {
    int n = blockIdx.x * GEMV_WARPS + (threadIdx.x >> 5);
    if (n >= out) return;
    int lane = threadIdx.x & 31;
    int part = lane & 7;
    int half = part >> 2;          // 128-weight half of the block
    int l0 = (part & 3) * 8;       // eight consecutive positions inside the half
    const int K = nb * 256;
    int64_t row_blk = ((int64_t)blockIdx.y * out + n) * nb;
    int t_first;
    group_range(grp, T, t_first, T);

    for (int t0 = t_first; t0 < T; t0 += NT) {
        float acc[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t] = 0.f;
        int rows = min(NT, T - t0);
        for (int ib = lane >> 3; ib < nb; ib += 4) {
            int64_t b = row_blk + ib;
            uint2 qa = *reinterpret_cast<const uint2*>(ql_p + b * 128 + half * 64 + l0);
            uint2 qb = *reinterpret_cast<const uint2*>(ql_p + b * 128 + half * 64 + 32 + l0);
            uint2 qhh = *reinterpret_cast<const uint2*>(qh_p + b * 64 + half * 32 + l0);
            const int8_t* sc = sc_p + b * 16 + half * 8 + (l0 >> 4);
            int s0 = sc[0], s1 = sc[2], s2 = sc[4], s3 = sc[6];
            float d = __half2float(d_p[b]);
            // four groups of eight 6-bit values, re-centred to [-32, 31]
            uint32_t g[4][2];
            g[0][0] = __vsub4((qa.x & 0x0F0F0F0Fu) | (((qhh.x >> 0) & 0x03030303u) << 4), 0x20202020u);
            g[0][1] = __vsub4((qa.y & 0x0F0F0F0Fu) | (((qhh.y >> 0) & 0x03030303u) << 4), 0x20202020u);
            g[1][0] = __vsub4((qb.x & 0x0F0F0F0Fu) | (((qhh.x >> 2) & 0x03030303u) << 4), 0x20202020u);
            g[1][1] = __vsub4((qb.y & 0x0F0F0F0Fu) | (((qhh.y >> 2) & 0x03030303u) << 4), 0x20202020u);
            g[2][0] = __vsub4(((qa.x >> 4) & 0x0F0F0F0Fu) | (((qhh.x >> 4) & 0x03030303u) << 4), 0x20202020u);
            g[2][1] = __vsub4(((qa.y >> 4) & 0x0F0F0F0Fu) | (((qhh.y >> 4) & 0x03030303u) << 4), 0x20202020u);
            g[3][0] = __vsub4(((qb.x >> 4) & 0x0F0F0F0Fu) | (((qhh.x >> 6) & 0x03030303u) << 4), 0x20202020u);
            g[3][1] = __vsub4(((qb.y >> 4) & 0x0F0F0F0Fu) | (((qhh.y >> 6) & 0x03030303u) << 4), 0x20202020u);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                if (t < rows) {
                    const int64_t xrow = src_of(grp, t0 + t);
                    const int8_t* xr = xq + xrow * K + ib * 256 + half * 128 + l0;
                    int2 x0 = *reinterpret_cast<const int2*>(xr);
                    int2 x1 = *reinterpret_cast<const int2*>(xr + 32);
                    int2 x2 = *reinterpret_cast<const int2*>(xr + 64);
                    int2 x3 = *reinterpret_cast<const int2*>(xr + 96);
                    int i0 = __dp4a((int)g[0][1], x0.y, __dp4a((int)g[0][0], x0.x, 0));
                    int i1 = __dp4a((int)g[1][1], x1.y, __dp4a((int)g[1][0], x1.x, 0));
                    int i2 = __dp4a((int)g[2][1], x2.y, __dp4a((int)g[2][0], x2.x, 0));
                    int i3 = __dp4a((int)g[3][1], x3.y, __dp4a((int)g[3][0], x3.x, 0));
                    int isum = s0 * i0 + s1 * i1 + s2 * i2 + s3 * i3;
                    acc[t] += xd[xrow * nb + ib] * (d * (float)isum);
                }
            }
        }
        finish_rows<NT>(acc, n, t0, T, y, ldy, out_scale, softcap);
    }
}

// ---------------------------------------------------------------- Q8_0 (planar layout)
__global__ void __launch_bounds__(GEMV_WARPS * 32) qgemv_q80_kernel(const int8_t* __restrict__ qs_p,
                                                                    const __half* __restrict__ d_p, int K, int out,
                                                                    const int8_t* __restrict__ xq,
                                                                    const float* __restrict__ xd, int T,
                                                                    float* __restrict__ y, int ldy, float out_scale,
                                                                    float softcap, Group grp) {
    int n = blockIdx.x * GEMV_WARPS + (threadIdx.x >> 5);
    if (n >= out) return;
    int lane = threadIdx.x & 31;
    int nb = K / 32;
    const int8_t* wq = qs_p + ((int64_t)blockIdx.y * out + n) * K;
    const __half* wd = d_p + ((int64_t)blockIdx.y * out + n) * nb;
    int t_first;
    group_range(grp, T, t_first, T);
    for (int t0 = t_first; t0 < T; t0 += NT) {
        float acc[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t] = 0.f;
        int rows = min(NT, T - t0);
        for (int b = lane; b < nb; b += 32) {
            int4 w0 = *reinterpret_cast<const int4*>(wq + b * 32);
            int4 w1 = *reinterpret_cast<const int4*>(wq + b * 32 + 16);
            float d = __half2float(wd[b]);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                if (t < rows) {
                    const int64_t xrow = src_of(grp, t0 + t);
                    const int8_t* xr = xq + xrow * K + b * 32;
                    int4 x0 = *reinterpret_cast<const int4*>(xr);
                    int4 x1 = *reinterpret_cast<const int4*>(xr + 16);
                    int s = __dp4a(w0.x, x0.x, 0);
                    s = __dp4a(w0.y, x0.y, s);
                    s = __dp4a(w0.z, x0.z, s);
                    s = __dp4a(w0.w, x0.w, s);
                    s = __dp4a(w1.x, x1.x, s);
                    s = __dp4a(w1.y, x1.y, s);
                    s = __dp4a(w1.z, x1.z, s);
                    s = __dp4a(w1.w, x1.w, s);
                    acc[t] += (float)s * (d * xd[xrow * nb + b]);
                }
            }
        }
        finish_rows<NT>(acc, n, t0, T, y, ldy, out_scale, softcap);
    }
}

// ---------------------------------------------------------------- F32 (router)
constexpr int F32_GEMV_ROWS = 8;
// y[t][n] = sum_k x[t][k] * W[n][k] for a small f32 matrix (the MoE router).  One warp per output n and run of
// F32_GEMV_ROWS rows of x (blockIdx.y): the rows' sums advance side by side, so a warp has a row's worth of independent
// loads in flight per step instead of one chain.  The sum of one (row, output) pair is always formed the same way -
// lane-strided partial sums in ascending k, then the warp tree - whatever the grid or the number of rows.
__global__ void __launch_bounds__(GEMV_WARPS * 32) f32_gemv_kernel(const float* __restrict__ W, int out, int in,
                                                                   const float* __restrict__ x, int T,
                                                                   float* __restrict__ y) {
    int n = blockIdx.x * GEMV_WARPS + (threadIdx.x >> 5);
    if (n >= out) return;
    int lane = threadIdx.x & 31;
    const float* w = W + (int64_t)n * in;
    const int t0 = (int)blockIdx.y * F32_GEMV_ROWS;
    const int rows = min(F32_GEMV_ROWS, T - t0);
    const float* xr = x + (int64_t)t0 * in;
    float acc[F32_GEMV_ROWS];
#pragma unroll
    for (int r = 0; r < F32_GEMV_ROWS; ++r) acc[r] = 0.f;
    if (rows == F32_GEMV_ROWS) {
#pragma unroll 4
        for (int k = lane; k < in; k += 32) {
            const float wv = w[k];
#pragma unroll
            for (int r = 0; r < F32_GEMV_ROWS; ++r) acc[r] += xr[(int64_t)r * in + k] * wv;
        }
    } else {
        for (int k = lane; k < in; k += 32) {
            const float wv = w[k];
#pragma unroll
            for (int r = 0; r < F32_GEMV_ROWS; ++r)
                if (r < rows) acc[r] += xr[(int64_t)r * in + k] * wv;
        }
    }
#pragma unroll
    for (int r = 0; r < F32_GEMV_ROWS; ++r) {
        const float v = warp_sum(acc[r]);
        if (lane == 0 && r < rows) y[(int64_t)(t0 + r) * out + n] = v;
    }
}

}  // namespace

static void launch_qgemv_impl(const QWeight& W, const ActQ& x, int T, float* y, int ldy, float out_scale, float softcap,
                              int experts, Group grp, cudaStream_t s) {
    dim3 grid((unsigned)((W.rows + GEMV_WARPS - 1) / GEMV_WARPS), (unsigned)experts);
    switch (W.type) {
        case QT_Q4_K:
            qgemv_q4k_kernel<<<grid, GEMV_WARPS * 32, 0, s>>>((const uint8_t*)W.p0, (int)(W.cols / 256), (int)W.rows, x.qs,
                                                              x.d, x.bsums, T, y, ldy, out_scale, softcap, grp);
            break;
        case QT_Q6_K:
            qgemv_q6k_kernel<<<grid, GEMV_WARPS * 32, 0, s>>>((const uint8_t*)W.p0, (const uint8_t*)W.p1,
                                                              (const int8_t*)W.p2, (const __half*)W.p3,
                                                              (int)(W.cols / 256), (int)W.rows, x.qs, x.d, T, y, ldy,
                                                              out_scale, softcap, grp);
            break;
        case QT_Q8_0:
            qgemv_q80_kernel<<<grid, GEMV_WARPS * 32, 0, s>>>((const int8_t*)W.p0, (const __half*)W.p1, (int)W.cols,
                                                              (int)W.rows, x.qs, x.d, T, y, ldy, out_scale, softcap, grp);
            break;
        default:
            throw std::runtime_error("launch_qgemv: unsupported weight type");
    }
    MK_LAUNCH_CHECK();
}

void launch_qgemv(const QWeight& W, const ActQ& x, int T, float* y, int ldy, float out_scale, float softcap,
                  cudaStream_t s) {
    if (T <= 0 || W.rows <= 0) return;
    launch_qgemv_impl(W, x, T, y, ldy, out_scale, softcap, 1, Group{}, s);
}

void launch_qgemv_grouped(const QWeight& W, int experts, const int32_t* offsets, const int32_t* src_row, const ActQ& x,
                          float* y, int ldy, cudaStream_t s) {
    if (experts <= 0 || W.rows <= 0) return;
    Group g;
    g.offsets = offsets;
    g.src_row = src_row;
    launch_qgemv_impl(W, x, 0, y, ldy, 1.0f, 0.f, experts, g, s);
}

void launch_f32_gemv(const float* W, int out, int in, const float* x, int T, float* y, cudaStream_t s) {
    if (T <= 0) return;
    dim3 grid((unsigned)((out + GEMV_WARPS - 1) / GEMV_WARPS), (unsigned)((T + F32_GEMV_ROWS - 1) / F32_GEMV_ROWS));
    f32_gemv_kernel<<<grid, GEMV_WARPS * 32, 0, s>>>(W, out, in, x, T, y);
    MK_LAUNCH_CHECK();
}

}  // namespace mk
