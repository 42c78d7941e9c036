// One head vector of one token on its way from the projection to the attention: summation of split-K shares, the
// optional per-head RMSNorm (SelfAttention::project_packed_qkv, src/decoder.rs:1137-1154, applied BEFORE the rotation)
// and the half-split rotation (RotaryEmbedding::apply, src/decoder.rs:203-257).  Shared by the stand-alone
// RoPE + KV-scatter kernel and by the decode attention kernel that prepares its own rows, so that both produce the
// same bits.
#pragma once
#include "kernels.h"

namespace mk {

constexpr int RK_MAX_D = 256;

// One warp.  kind: 0 = q, 1 = k, 2 = v; hh = head index within its kind; t = packed token row; x = the warp's d floats
// of shared memory, holding the finished head on return (after a __syncwarp).
__device__ __forceinline__ void rope_head_prepare(const RopeKvArgs& a, int kind, int hh, int t, int position, float* x, int lane) {
    const int d = a.d;
    const float* src = kind == 0 ? a.q + (int64_t)t * a.ldq + hh * d : (kind == 1 ? a.k + (int64_t)t * a.ldk + hh * d : a.v + (int64_t)t * a.ldv + hh * d);
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
        const float* c = a.cos_t + (int64_t)position * half;
        const float* s = a.sin_t + (int64_t)position * half;
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
}

}  // namespace mk
