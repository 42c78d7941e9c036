// Narrow-batch (decode tick) matmul that streams Q4_K / Q6_K blocks from HBM once (see qstream_tc.cu).
#pragma once
#include "common.cuh"
#include "device_util.h"

namespace mk {

// A Q4_K or Q6_K matrix [rows][cols] re-tiled for the streamed matmul: (128-row tile, 256-column block) units one after
// the other, so that a unit is one contiguous bulk copy (Q4_K: 128 rows x 144 raw block bytes = 18 KiB; Q6_K: the ql,
// qh, scales and d planes of the 128 rows = 26.25 KiB).  A second copy of the matrix (the row-major blocks stay where
// the other kernels read them).
struct QStreamWeight {
    DevBuf tiled;
    int64_t rows = 0, cols = 0;
    int row_tiles = 0;
    int fmt = 0;          // 0 = Q4_K, 1 = Q6_K
    bool gated = false;   // rows interleaved: row 2f = gate row f, row 2f + 1 = up row f
    bool ready = false;
};

constexpr int kQStreamMaxRows = 64;  // activation rows per call
constexpr size_t kSplitScratchBytes = (size_t)24 << 20;  // partial sums of one matmul launch (three slots of 64 x 22016 floats fit)

// q4k_blocks: device pointer to the row-major blocks (16-byte aligned).  interleave > 0: the source is `interleave` gate
// rows followed by as many up rows, stored with their rows interleaved for the gated form of the matmul.
void build_qstream_weight(const void* q4k_blocks, int64_t rows, int64_t cols, QStreamWeight& out, cudaStream_t s, int64_t interleave = 0);
// The same for a Q6_K matrix in the plane layout of QWeight.
void build_qstream_weight_q6k(const QWeight& w, QStreamWeight& out, cudaStream_t s);

// R row tiles form a group, (group, block) is an item; items are shared out evenly over `ctas` persistent CTAs;
// `slots` is the most pieces any group is cut into (1: results complete in y).
struct QStreamPlan {
    int bn = 0, R = 1, row_tiles = 0, groups = 0, items = 0, ctas = 0, slots = 1;
    bool whole_groups = false;
    size_t partial_floats = 0;
};
QStreamPlan qstream_plan(int row_tiles, int n_blocks, int64_t rows, int T, int max_splits, bool whole_groups, int sms = 148);

// y[t][n] = sum_k xh[t][k] * dequant(W)[n][k] for T <= kQStreamMaxRows rows of f16 activations [T][cols].  W2, when
// given, is a second matrix of the same width whose rows follow W's (W.rows a multiple of 128): one launch computes the
// stacked result, e.g. [wq; wk] in Q4_K followed by wv in Q6_K.
// Returns the number of partial-sum slots S.  S = 1: y (row stride ldy) holds the result.  S > 1 (only when
// max_splits > 1, and never more than that): y is not written; the pieces were left at
// partial[(s * T + t) * rows + n], unused slots zeroed, and the consumer adds them for s = 0 .. S-1 in that order.
// gated_act >= 0 (W built with interleave): nothing of the above is written; instead
// yh[t * ldyh + f] = f16(act(gate_f . x_t) * (up_f . x_t)), act 0 = SiLU, 1 = tanh GELU, and the call returns 1.
// `status` receives a non-zero code when a bounded wait gave up.
int launch_qstream_tc(const QStreamWeight& W, const __half* xh, int T, float* y, int ldy, float* partial, size_t partial_floats,
                      int32_t* status, cudaStream_t s, int max_splits, const QStreamWeight* W2 = nullptr, int gated_act = -1,
                      __half* yh = nullptr, int ldyh = 0);

// Expert-grouped form: W is a bank of `experts` matrices stacked by rows (each a whole number of 128-row tiles);
// activation rows [offsets[e], offsets[e + 1]) of xh [rows_total][cols] (grouped by expert, device array of experts + 1
// row numbers) are multiplied by expert e's matrix: y[r][n] for those rows r and n < rows per expert, or, gated,
// yh[r][f].  max_rows_per_expert picks the chunk width (16, 32 or 64 rows): an expert's rows are processed a chunk at a
// time, each chunk one pass over the expert's matrix, so any width is correct for any row count.  The kernel reads the
// row ranges on the device: no host round trip.  rows_known = false: rows_total is only the extent of xh (the true row
// count lives on the device); the host then cannot bound the jobs per CTA, and a launch that overflows the kernel's job
// table reports status 30 instead of an exception here.
int launch_qstream_tc_grouped(const QStreamWeight& W, int experts, const int32_t* offsets_dev, const __half* xh, int rows_total,
                              int max_rows_per_expert, float* y, int ldy, int32_t* status, cudaStream_t s, int gated_act = -1,
                              __half* yh = nullptr, int ldyh = 0, bool rows_known = true);

// Measuring aid: when set (a device buffer of 40 int64), CTA 0 of every following launch records the cycles its roles
// spent waiting: rows weight loader, MMA issuer, activation loader, first converter warp, first epilogue warp; columns
// total, wait sites 0-3, items.  nullptr switches it off.
void qstream_set_profile_buffer(long long* dev_buffer);

}  // namespace mk
