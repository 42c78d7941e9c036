// Tensor-core (tcgen05) quantised GEMM for prefill chunks and wide decode batches.
#pragma once
#include "device_util.h"

namespace mk {

// Split-K partial sums live here between the MMA kernel and the ordered reduction.
struct QgemmWorkspace {
    DevBuf partial;      // [splits][T][out] f32
    DevBuf status;       // [1] int32: non-zero when a bounded wait inside the kernel gave up
};

// True when the tensor-core path is the better choice for this matrix and row count.
bool qgemm_tc_preferred(const QWeight& W, int T);

// y[t][n] = (sum_k xh[t][k] * dequant(W)[n][k]) * out_scale, optional tanh softcap.
// Needs x.xh (f16 dequantised activations).  K must be a multiple of 256 (128 for Q8_0).
void launch_qgemm_tc(const QWeight& W, const ActQ& x, int act_kind, int T, float* y, int ldy, float out_scale,
                     float softcap, QgemmWorkspace& ws, cudaStream_t s);

// Same, with caller-owned scratch (no allocation inside): `partial` must hold
// qgemm_tc_partial_floats(W, T) floats, `status` one int32.
size_t qgemm_tc_partial_floats(const QWeight& W, int T);
void launch_qgemm_tc_scratch(const QWeight& W, const ActQ& x, int T, float* y, int ldy, float out_scale, float softcap,
                             float* partial, int32_t* status, cudaStream_t s);

}  // namespace mk
