// Tensor-core paged attention (see attention_tc.cu).
#pragma once
#include "kernels.h"
#include <vector>

namespace mk {

struct AttnTcArgs {
    const float* q = nullptr;   // [T] rows of q_heads*d f32 values, row stride ldq
    int ldq = 0;                // 0 = q_heads*d
    float* out = nullptr;       // [T][q_heads*d] f32
    __half* out_h = nullptr;    // optional: the same rows rounded to f16 (what an f16 GEMM of the output projection reads);
                                // with out_h set, `out` may be null
    const void* k_pool = nullptr;  // f16 pages [kv_heads][block_tokens][d], page order per kv_page_index
    const void* v_pool = nullptr;
    const LaneHeader* hdr = nullptr;
    const uint32_t* tables = nullptr;
    const int32_t* cu_seqlens = nullptr;
    // work lists (device): prefill tiles (lane, first row); decode entries, 8 ints each, 32-byte aligned
    // (lane, share, n_shares, start_pos, table offset, first packed row, first entry of the lane, 0);
    // one-token lanes with more than one share (lane, first entry, n_splits)
    const int32_t* tiles = nullptr;
    const int32_t* entries = nullptr;
    const int32_t* dec_lanes = nullptr;
    int n_tiles = 0, n_entries = 0, n_dec_lanes = 0;
    float* part_o = nullptr;    // [n_entries][kv_heads][16][d]
    float* part_ml = nullptr;   // [n_entries][kv_heads][16][2]
    // optional: one-token lanes also leave their output rows quantised (8-bit blocks, f16 image) for the
    // matmul that follows; needs (q_heads / kv_heads) * d to be a multiple of 256.  With qout set, `out` may be null.
    ActQ qout;
    int qkind = ACT_Q8K;
    // optional (ticks of one-token lanes only): the kernel prepares its own rows from the projection's output - share
    // summation, per-head norm and rotation of the group's query heads, and, in the CTA that walks the lane's last keys,
    // of the new K and V rows, which it writes to the pools (rk.k_pool / rk.v_pool) before it fetches any tile - so no
    // separate RoPE + scatter launch is needed.  `q` is not read then.
    int fused_rope = 0;
    RopeKvArgs rk;
    int32_t* counters = nullptr;  // [lanes][kv_heads], zero before the first call; every call leaves them zero
    int q_heads = 0, kv_heads = 0, d = 0, block_tokens = 16, layers = 0, layer = 0;
    int64_t pool_blocks = 0;  // see kv_page_index
    int bt_shift = 0;         // log2(block_tokens), filled in by the launcher
    float scale = 1.f, softcap = 0.f;
    int window = 0;
};

// f16 pools, head_dim 64/128/256, 1/2/4/8 query heads per KV head, block_tokens a power of two >= 16.
bool attention_tc_supported(int q_heads, int kv_heads, int head_dim, int block_tokens, bool kv_f16);
// Query rows of one prefill tile (the CTA covers rows x group heads = 16 * warps items).
int attention_tc_tile_rows(int q_heads, int kv_heads);
int attention_tc_warps(int q_heads, int kv_heads);

// Host-side work lists of one tick (the same for every layer): lanes with more than one token are cut
// into query tiles; one-token lanes split their keys over up to kAttnMaxSplits CTAs (four warps each), at
// least kAttnMinSplitKeys keys each, until about kAttnTargetCtas CTAs are in flight - unless the lanes alone already
// give every SM a CTA, in which case no lane is split.
constexpr int kPlanSms = 148;  // the work lists are planned on the host, without a device, for a B200's SM count
constexpr int kAttnTargetCtas = kPlanSms * 2;
constexpr int kAttnMaxSplits = 16;
constexpr int kAttnMinSplitKeys = 512;  // a share costs a partial write, a counter and a merge: below this a lane stays whole (measured at 4 lanes x 333 keys: +8 % without shares)
struct AttnTcPlan {
    std::vector<int32_t> tiles, entries, dec_lanes;
    int n_tiles() const { return (int)tiles.size() / 2; }
    int n_entries() const { return (int)entries.size() / 8; }
    int n_dec_lanes() const { return (int)dec_lanes.size() / 3; }
};
// n_blocks[i] = entries of lane i's block table (tables are concatenated in lane order, tokens packed in lane order).
void plan_attention_tc(const int32_t* start_pos, const int32_t* n_tokens, const int32_t* n_blocks, int lanes, int q_heads,
                       int kv_heads, AttnTcPlan& plan);
// Upper bound of plan.n_entries() for a tick of at most `lanes` lanes.
int attention_tc_max_entries(int lanes, int kv_heads);

// Returns the number of kernels launched.
int launch_paged_attention_tc(const AttnTcArgs& a, cudaStream_t s);

}  // namespace mk
