// Per-thread steps of the recurrent mixers (Gated DeltaNet, Mamba2 selective scan, short convolution), written once for the
// device kernels of recurrent.cu and for a host build of the same source (the tests compile this header with a C++ compiler
// and walk the "threads" in a loop, so the arithmetic and the state indexing are checked where no GPU is at hand).
//
// Rounding: every product and every sum is rounded on its own, in the order the reference's CPU operators take them
// (crates/macllm-kernels/src/gated_delta.rs:396-431, crates/macllm-kernels/src/mamba2.rs:255-289, src/decoder.rs:1466-1481),
// so that given equal controls the recurrences agree with the reference bit for bit.  On the device that takes the
// explicit round-to-nearest intrinsics: the compiler would otherwise contract a product and a sum into one fused operation.
#pragma once
#include <cmath>

#if defined(__CUDACC__)
#define MK_HD __host__ __device__ __forceinline__
#else
#define MK_HD inline
#endif

namespace mk {
namespace recurrent {

MK_HD float mul(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fmul_rn(a, b);
#else
    return a * b;
#endif
}

MK_HD float add(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fadd_rn(a, b);
#else
    return a + b;
#endif
}

MK_HD float sub(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fsub_rn(a, b);
#else
    return a - b;
#endif
}

// max(x, 0) + ln(1 + exp(-|x|)): finite for any finite x
MK_HD float softplus_stable(float x) { return add(fmaxf(x, 0.f), log1pf(expf(-fabsf(x)))); }

// exp(softplus(alpha + time_bias) * state_decay)   (gated_delta.rs:96-104)
MK_HD float gated_delta_decay(float alpha, float time_bias, float state_decay) {
    return expf(mul(softplus_stable(add(alpha, time_bias)), state_decay));
}

// One token of one (head, value column): `state` walks the column's key_dim entries `stride` floats apart.
//   memory = sum_k S[k] * decay * key[k];  delta = (value - memory) * beta;
//   S[k] = S[k] * decay + key[k] * delta;  returns sum_k S[k] * query[k]
MK_HD float gated_delta_step(float* state, int stride, int key_dim, const float* key, const float* query, float decay, float beta,
                             float value) {
    float memory = 0.f;
    for (int k = 0; k < key_dim; ++k) memory = add(memory, mul(mul(state[(long long)k * stride], decay), key[k]));
    const float delta = mul(sub(value, memory), beta);
    float projected = 0.f;
    for (int k = 0; k < key_dim; ++k) {
        const float next = add(mul(state[(long long)k * stride], decay), mul(key[k], delta));
        state[(long long)k * stride] = next;
        projected = add(projected, mul(next, query[k]));
    }
    return projected;
}

// The same step on a column held in registers (KD known at compile time).
template <int KD>
MK_HD float gated_delta_step_reg(float (&state)[KD], const float* key, const float* query, float decay, float beta, float value) {
    float memory = 0.f;
#pragma unroll
    for (int k = 0; k < KD; ++k) memory = add(memory, mul(mul(state[k], decay), key[k]));
    const float delta = mul(sub(value, memory), beta);
    float projected = 0.f;
#pragma unroll
    for (int k = 0; k < KD; ++k) {
        const float next = add(mul(state[k], decay), mul(key[k], delta));
        state[k] = next;
        projected = add(projected, mul(next, query[k]));
    }
    return projected;
}

// The controls of one (token, head) of the Mamba2 scan: delta = softplus(dt + dt_bias), decay = exp(delta * a).
MK_HD void mamba2_controls(float raw_dt, float dt_bias, float a, float* delta, float* decay) {
    *delta = softplus_stable(add(raw_dt, dt_bias));
    *decay = expf(mul(*delta, a));
}

// One token of one (head, position): S[n] = decay * S[n] + delta * x * B[n]; returns sum_n S[n] * C[n] + d * x.
MK_HD float mamba2_step(float* state, int state_size, const float* B, const float* C, float decay, float delta, float x, float skip) {
    const float dx = mul(delta, x);
    float projected = 0.f;
    for (int n = 0; n < state_size; ++n) {
        const float next = add(mul(decay, state[n]), mul(dx, B[n]));
        state[n] = next;
        projected = add(projected, mul(next, C[n]));
    }
    return add(projected, mul(skip, x));
}

template <int N>
MK_HD float mamba2_step_reg(float (&state)[N], const float* B, const float* C, float decay, float delta, float x, float skip) {
    const float dx = mul(delta, x);
    float projected = 0.f;
#pragma unroll
    for (int n = 0; n < N; ++n) {
        const float next = add(mul(decay, state[n]), mul(dx, B[n]));
        state[n] = next;
        projected = add(projected, mul(next, C[n]));
    }
    return add(projected, mul(skip, x));
}

// One output of the short convolution: `window` holds the channel's last K values of B * x, oldest first (zeros or the tail
// before the lane's first row); the taps are summed from the oldest on and the sum is gated by C.
MK_HD float short_conv_tap_sum(const float* window, const float* taps, int K, float gate) {
    float sum = mul(window[0], taps[0]);
    for (int j = 1; j < K; ++j) sum = add(sum, mul(window[j], taps[j]));
    return mul(gate, sum);
}

}  // namespace recurrent
}  // namespace mk
