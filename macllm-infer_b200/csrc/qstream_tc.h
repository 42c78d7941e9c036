// Narrow-batch (decode tick) matmul that streams Q4_K blocks from HBM once (see qstream_tc.cu).
#pragma once
#include "common.cuh"
#include "device_util.h"

namespace mk {

// A Q4_K matrix [rows][cols] re-tiled for the streamed matmul: (128-row tile, 256-column block) units one after the
// other, each 128 rows x 144 raw block bytes, so that a unit is one contiguous 18 KiB copy.  A second copy of the
// matrix (the row-major blocks stay where the other kernels read them).
struct QStreamWeight {
    DevBuf tiled;
    int64_t rows = 0, cols = 0;
    alignas(64) unsigned char tmap[128] = {};  // TMA descriptor of the copy as rows of 128 bytes, boxes of one unit
    bool ready = false;
};

constexpr int kQStreamMaxRows = 64;  // activation rows per call

// q4k_blocks: device pointer to the row-major blocks (16-byte aligned).
void build_qstream_weight(const void* q4k_blocks, int64_t rows, int64_t cols, QStreamWeight& out, cudaStream_t s);

// (row tile, 256-column block) units are shared out evenly over `ctas` persistent CTAs; `slots` is the most pieces
// any row tile is cut into (1: results complete in y).
struct QStreamPlan {
    int bn = 0, row_tiles = 0, units = 0, ctas = 0, slots = 1;
    size_t partial_floats = 0;
};
QStreamPlan qstream_plan(int64_t rows, int64_t cols, int T, int max_splits);

// y[t][n] = sum_k xh[t][k] * dequant(W)[n][k] for T <= kQStreamMaxRows rows of f16 activations [T][cols]; gs holds the
// per-group sums of those activations (ActQ::gs).
// Returns the number of partial-sum slots S.  S = 1: y (row stride ldy) holds the result.  S > 1 (only when
// max_splits > 1, and never more than that): y is not written; the pieces of every row tile were left at
// partial[(s * T + t) * rows + n], unused slots zeroed, and the consumer adds them for s = 0 .. S-1 in that order.  `status` receives a non-zero code when a bounded wait gave up.
int launch_qstream_tc(const QStreamWeight& W, const __half* xh, const __half* gs, int T, float* y, int ldy, float* partial,
                      size_t partial_floats, int32_t* status, cudaStream_t s, int max_splits);

}  // namespace mk
