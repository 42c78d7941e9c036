// Arithmetic shared by the host sampler and the device sampling kernel, so that both pick the same token for the same
// uniform draw: a total order on f32 bit patterns and an exponential built from fused multiply-adds only (fmaf is
// exactly rounded on the host and on the device, library exp functions differ by an ulp between the two).
//
// The sampling rule itself is Sampler::sample_stochastic / nucleus_probabilities / sample_from_probabilities of the
// reference (src/sampling.rs:145-169,337-390).
#pragma once
#include <cstdint>
#include <cstring>
#include <cmath>

#ifdef __CUDACC__
#define MK_HD __host__ __device__ __forceinline__
#else
#define MK_HD inline
#endif

namespace mk {

MK_HD uint32_t f32_bits(float f) {
#ifdef __CUDA_ARCH__
    return __float_as_uint(f);
#else
    uint32_t b;
    memcpy(&b, &f, 4);
    return b;
#endif
}
MK_HD float bits_f32(uint32_t b) {
#ifdef __CUDA_ARCH__
    return __uint_as_float(b);
#else
    float f;
    memcpy(&f, &b, 4);
    return f;
#endif
}

// f32::total_cmp as an unsigned key: a larger key is a larger value (src/sampling.rs:425-433 uses total_cmp).
MK_HD uint32_t f32_order_key(float f) {
    const uint32_t b = f32_bits(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// (value descending, index ascending) as one 64-bit key, larger first.
MK_HD uint64_t rank_key(float value, uint32_t index) {
    return ((uint64_t)f32_order_key(value) << 32) | (uint64_t)(0xFFFFFFFFu - index);
}
MK_HD uint32_t rank_key_index(uint64_t k) { return 0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull); }

// exp(x) for x <= 0 (softmax numerators): n = round(x log2 e), r = x - n ln 2 in two fused steps, a degree-6 polynomial
// in r, then scaling by 2^n through the exponent field (in two exact steps when the result is subnormal).  About 1 ulp
// from exp; the same bits on the host and on the device.  x below -104 (and -inf) gives 0, x > 0 is treated as 0.
MK_HD float det_expf(float x) {
    if (!(x > -104.0f)) return 0.0f;  // also NaN
    if (x > 0.0f) x = 0.0f;
    const float n = nearbyintf(x * 1.44269504088896341f);
    float r = fmaf(n, -0.693145751953125f, x);            // ln 2, high part (exact product for |n| < 2^11)
    r = fmaf(n, -1.42860682030941723212e-6f, r);          // ln 2, low part
    float p = 1.38888888e-3f;                             // 1/720
    p = fmaf(p, r, 8.33333377e-3f);
    p = fmaf(p, r, 4.16666679e-2f);
    p = fmaf(p, r, 1.66666672e-1f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    const int e = (int)n;                                  // -151 .. 0
    if (e >= -126) return p * bits_f32((uint32_t)(e + 127) << 23);
    return (p * bits_f32((uint32_t)(e + 64 + 127) << 23)) * bits_f32((uint32_t)(-64 + 127) << 23);
}

}  // namespace mk
