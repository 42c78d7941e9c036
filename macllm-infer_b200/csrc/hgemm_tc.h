// Wide-batch matmul over an f16 image of the weights kept resident in HBM (see hgemm_tc.cu).
#pragma once
#include "common.cuh"
#include "device_util.h"

namespace mk {

// Bytes an f16 image of W takes.
inline size_t half_weight_bytes(const QWeight& W) { return (size_t)W.rows * (size_t)W.cols * 2; }

// Whether the f16 GEMM covers this matrix (Q4_K / Q6_K / Q8_0 / F32 sources, cols a multiple of 64).
bool hgemm_tc_supported(const QWeight& W);

// Dequantise W (device layout of QWeight) into out.values and encode its descriptor.
void build_half_weight(const QWeight& W, HalfWeight& out, cudaStream_t s);

// y[t][n] = scale * sum_k xh[t][k] * Wh[n][k] (then the optional soft cap), t < T, n < rows.
// xh is [T][cols] f16, 16-byte aligned.  `status` receives a non-zero code when a bounded wait gave up.
void launch_hgemm_tc(const HalfWeight& W, const __half* xh, int T, float* y, int ldy, float out_scale, float softcap,
                     int32_t* status, cudaStream_t s);

}  // namespace mk
