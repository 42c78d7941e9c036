// Token-embedding row gather straight from quantised storage.
//
// Replaces TokenEmbedding::forward_validated (src/model_weights.rs:489-502) and the embedding scale
// of src/decoder.rs:3194-3197: the selected rows are dequantised to f32 and multiplied by the scale.
// One CTA per token; a row is hidden*bits/8 bytes, read once.
#include "kernels.h"

namespace mk {

namespace {

__device__ __forceinline__ void q4k_scale_min(const uint8_t* s, int j, int& sc, int& mn) {
    if (j < 4) {
        sc = s[j] & 63;
        mn = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4);
        mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

__global__ void embed_kernel(QWeight W, const uint32_t* ids, float scale, float* out) {
    int t = blockIdx.x;
    int64_t row = ids[t];
    int cols = (int)W.cols;
    float* o = out + (int64_t)t * cols;
    for (int k = threadIdx.x; k < cols; k += blockDim.x) {
        float v;
        if (W.type == QT_F32) {
            v = ((const float*)W.p0)[row * cols + k];
        } else if (W.type == QT_Q8_0) {
            int nb = cols / 32;
            v = __half2float(((const __half*)W.p1)[row * nb + k / 32]) * (float)((const int8_t*)W.p0)[row * cols + k];
        } else if (W.type == QT_Q4_K) {
            int nb = cols / 256;
            const uint8_t* blk = (const uint8_t*)W.p0 + (row * nb + k / 256) * 144;
            int e = k & 255;
            int j = e >> 6, within = e & 63;
            int sub = 2 * j + (within >> 5);
            int sc, mn;
            q4k_scale_min(blk + 4, sub, sc, mn);
            uint8_t byte = blk[16 + 32 * j + (within & 31)];
            int q = (within >> 5) ? (byte >> 4) : (byte & 0xF);
            float d = __half2float(*(const __half*)blk), dmin = __half2float(*(const __half*)(blk + 2));
            v = __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)mn));
        } else {  // Q6_K planes
            int nb = cols / 256;
            int64_t b = row * nb + k / 256;
            int e = k & 255;
            int half = e >> 7, r = e & 127;
            int grp = r >> 5, l = r & 31;  // grp 0..3 -> +0, +32, +64, +96
            const uint8_t* ql = (const uint8_t*)W.p0 + b * 128 + half * 64;
            const uint8_t* qh = (const uint8_t*)W.p1 + b * 64 + half * 32;
            uint8_t lo = ql[(grp & 1) * 32 + l];
            int nib = (grp >> 1) ? (lo >> 4) : (lo & 0xF);
            int q = (nib | (((qh[l] >> (2 * grp)) & 3) << 4)) - 32;
            int sc = ((const int8_t*)W.p2)[b * 16 + half * 8 + (l >> 4) + 2 * grp];
            float d = __half2float(((const __half*)W.p3)[b]);
            v = __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
        }
        o[k] = scale == 1.0f ? v : __fmul_rn(v, scale);
    }
}

}  // namespace

void launch_embed(const QWeight& W, const uint32_t* ids, int T, float scale, float* out, cudaStream_t s) {
    if (T <= 0) return;
    embed_kernel<<<T, 256, 0, s>>>(W, ids, scale, out);
    MK_LAUNCH_CHECK();
}

}  // namespace mk
