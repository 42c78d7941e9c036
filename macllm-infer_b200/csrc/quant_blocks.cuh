// Register-resident 8-bit block quantisation of activations, shared by the activation kernels and by kernels that
// quantise their own output.  The rule restates the published GGML activation formats used by the reference's CPU
// matmul (see quantize.cu): blocks of 256 with an f32 scale chosen so the element of largest magnitude maps to -128
// (clamped to 127) for K-quant weights, blocks of 32 with an f16 scale amax/127 for Q8_0 weights.
#pragma once
#include "common.cuh"

namespace mk {

// ---- rows whose width is a multiple of 256 -----------------------------------------------------------
// One warp owns one 256-element group at a time and each lane eight consecutive values of it, so a K-quant
// activation block (256) or eight Q8_0 blocks (32 = four lanes) are quantised from registers with
// shuffles only.  Same arithmetic as quantize_row_q8k / quantize_row_q80 in quantize.cu.

__device__ __forceinline__ void quant8_q8k(const float (&v)[8], int lane, int8_t* qs, float* d, int16_t* bsums, __half* xh) {
    float amax = 0.f, mx = 0.f;
    int idx = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float ax = fabsf(v[i]);
        if (ax > amax) { amax = ax; idx = lane * 8 + i; mx = v[i]; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float oa = __shfl_xor_sync(0xffffffffu, amax, o);
        int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        float om = __shfl_xor_sync(0xffffffffu, mx, o);
        if (oa > amax || (oa == amax && oi < idx)) { amax = oa; idx = oi; mx = om; }
    }
    int8_t q[8];
    int sum = 0;
    float dd = 0.f;
    if (amax == 0.f) {
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = 0;
    } else {
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
    *reinterpret_cast<int2*>(qs + lane * 8) = packed;
    if (xh != nullptr) {
        __half2 hv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) hv[i] = __floats2half2_rn(__fmul_rn(dd, (float)q[2 * i]), __fmul_rn(dd, (float)q[2 * i + 1]));
        *reinterpret_cast<uint4*>(xh + lane * 8) = *reinterpret_cast<uint4*>(hv);
    }
    int pair = sum + __shfl_xor_sync(0xffffffffu, sum, 1);
    if ((lane & 1) == 0) bsums[lane >> 1] = (int16_t)pair;
    if (lane == 0) *d = dd;
}

__device__ __forceinline__ void quant8_q80(const float (&v)[8], int lane, int8_t* qs, float* d, __half* xh) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    float dd = amax / 127.f;
    float id = dd != 0.f ? 1.0f / dd : 0.f;
    float ddh = __half2float(__float2half_rn(dd));
    int8_t q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = (int8_t)roundf(v[i] * id);
    int2 packed;
    packed.x = (uint8_t)q[0] | ((uint8_t)q[1] << 8) | ((uint8_t)q[2] << 16) | ((uint32_t)(uint8_t)q[3] << 24);
    packed.y = (uint8_t)q[4] | ((uint8_t)q[5] << 8) | ((uint8_t)q[6] << 16) | ((uint32_t)(uint8_t)q[7] << 24);
    *reinterpret_cast<int2*>(qs + lane * 8) = packed;
    if (xh != nullptr) {
        __half2 hv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) hv[i] = __floats2half2_rn(__fmul_rn(ddh, (float)q[2 * i]), __fmul_rn(ddh, (float)q[2 * i + 1]));
        *reinterpret_cast<uint4*>(xh + lane * 8) = *reinterpret_cast<uint4*>(hv);
    }
    if ((lane & 3) == 0) d[lane >> 2] = ddh;
}

// Quantise group `grp` (256 values, eight per lane) of output row r.
__device__ __forceinline__ void quant_group(const float (&v)[8], int lane, int kind, const ActQ& out, int64_t r, int dim, int grp) {
    if (out.qs == nullptr) return;
    int8_t* qs = out.qs + r * dim + grp * 256;
    __half* xh = out.xh ? out.xh + r * dim + grp * 256 : nullptr;
    if (kind == ACT_Q8K) {
        quant8_q8k(v, lane, qs, out.d + r * (dim / 256) + grp, out.bsums + r * (dim / 16) + grp * 16, xh);
    }
    else quant8_q80(v, lane, qs, out.d + r * (dim / 32) + grp * 8, xh);
}

__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

}  // namespace mk
