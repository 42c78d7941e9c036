// Narrow-batch (decode tick) matmul that streams Q4_K blocks from HBM once (see qstream_tc.cu).
#pragma once
#include "common.cuh"
#include "device_util.h"

namespace mk {

// A Q4_K matrix [rows][cols] (raw 144-byte blocks, row-major, 16-byte aligned) with the TMA descriptor of its
// 128-row x one-block boxes.  `base` is borrowed: it points into a DeviceWeight (or into a buffer that stacks
// several of them by rows).
struct QStreamWeight {
    const void* base = nullptr;
    int64_t rows = 0, cols = 0;
    alignas(64) unsigned char tmap[128] = {};
    bool ready = false;
};

constexpr int kQStreamMaxRows = 64;  // activation rows per call

void build_qstream_weight(const void* q4k_blocks, int64_t rows, int64_t cols, QStreamWeight& out);

struct QStreamPlan {
    int bn = 0, row_tiles = 0, splits = 1, blocks_per_split = 0;
    size_t partial_floats = 0;
};
QStreamPlan qstream_plan(int64_t rows, int64_t cols, int T, int max_splits);

// y[t][n] = sum_k xh[t][k] * dequant(W)[n][k] for T <= kQStreamMaxRows rows of f16 activations [T][cols]; gs holds the
// per-group sums of those activations (ActQ::gs).
// Returns the number of K shares S.  S = 1: y (row stride ldy) holds the result.  S > 1 (only when max_splits > 1):
// y is not written; share s left its partial sums at partial[(s * T + t) * rows + n] and the consumer adds them
// for s = 0 .. S-1 in that order.  `status` receives a non-zero code when a bounded wait gave up.
int launch_qstream_tc(const QStreamWeight& W, const __half* xh, const __half* gs, int T, float* y, int ldy, float* partial,
                      size_t partial_floats, int32_t* status, cudaStream_t s, int max_splits);

}  // namespace mk
