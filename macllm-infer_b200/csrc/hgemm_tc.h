// Wide-batch matmul over an f16 image of the weights kept resident in HBM (see hgemm_tc.cu).
#pragma once
#include "common.cuh"
#include "device_util.h"

namespace mk {

// Encodes a 2-D tiled TMA descriptor (128 bytes at out_map, 64-byte aligned) over a row-major matrix of bytes or
// halves: `inner` elements per row, `outer` rows, boxes of box_inner x box_outer, optional 128-byte swizzle, zero
// fill outside the matrix.
void encode_tma_2d(void* out_map, bool bytes_not_halves, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                   uint32_t box_inner, uint32_t box_outer, bool swizzle_128b);

// Bytes an f16 image of W takes.
inline size_t half_weight_bytes(const QWeight& W) { return (size_t)W.rows * (size_t)W.cols * 2; }

// Whether the f16 GEMM covers this matrix (Q4_K / Q6_K / Q8_0 / F32 sources, cols a multiple of 64).
bool hgemm_tc_supported(const QWeight& W);

// Dequantise W (device layout of QWeight) into out.values and encode its descriptor.
void build_half_weight(const QWeight& W, HalfWeight& out, cudaStream_t s);

// Dequantise several matrices with the same number of columns into one image, stacked by rows (fused
// projections: one GEMM then produces the concatenated outputs).
void build_half_weight_stacked(const QWeight* const* parts, int n_parts, HalfWeight& out, cudaStream_t s);

// The gate and up projections of a gated feed-forward in one image with their rows interleaved (row 2j = gate row j,
// row 2j+1 = up row j), for launch_hgemm_tc_gated.
void build_half_weight_interleaved(const QWeight& gate, const QWeight& up, HalfWeight& out, cudaStream_t s);

// How a call is cut into work items (see hgemm_tc.cu); partial_floats is the scratch a split call needs.
struct HgemmPlan {
    int bn = 0, row_tiles = 0, n_tiles = 0, splits = 1, kb_per_split = 0;
    size_t partial_floats = 0;
};
HgemmPlan hgemm_tc_plan(int64_t rows, int64_t cols, int T, int max_splits);

// Device scratch of the GEMM: split-K partial sums and the status word that receives a non-zero code when
// a bounded wait gave up.
struct HgemmScratch {
    float* partial = nullptr;
    size_t partial_floats = 0;
    int32_t* status = nullptr;
};

// y[t][n] = scale * sum_k xh[t][k] * Wh[n][k] (then the optional soft cap), t < T, n < rows.
// xh is [T][cols] f16, 16-byte aligned.  Returns the number of K shares S the call was cut into.  S = 1: y holds
// the result.  S > 1 (only when max_splits > 1, scale = 1 and no soft cap): y is NOT written; share s left its
// partial sums at ws.partial[(s * T + t) * rows + n] and the consumer adds them for s = 0 .. S-1 in that order.
int launch_hgemm_tc(const HalfWeight& W, const __half* xh, int T, float* y, int ldy, float out_scale, float softcap,
                    const HgemmScratch& ws, cudaStream_t s, int max_splits = 1);

// Gated feed-forward front half in one kernel: with W an interleaved gate/up image (2F rows),
// yh[t][j] = f16(act(sum_k xh[t][k] gate[j][k]) * sum_k xh[t][k] up[j][k]), j < F; act 0 = SiLU, otherwise tanh GELU.
// The two sums are the f32 accumulators of the plain GEMM and the activation is evaluated like the separate SwiGLU
// kernel does, so the halves written equal the ones that kernel derives from the plain GEMM's output.
void launch_hgemm_tc_gated(const HalfWeight& W, const __half* xh, int T, int act, __half* yh, int ldyh, const HgemmScratch& ws,
                           cudaStream_t s);

}  // namespace mk
