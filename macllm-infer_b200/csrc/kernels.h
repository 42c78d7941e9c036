// Host-side launchers of the sm_100a kernels.  All pointers are device pointers unless noted.
#pragma once
#include "common.cuh"
#include "ep_comm.h"

namespace mk {

// ---- activation preparation -------------------------------------------------------------
// Row-wise residual add, RMSNorm and 8-bit activation quantisation in one pass:
//   a' = post_w ? rmsnorm(a, post_w) : a          (Gemma-style sandwich norm)
//   h  = h + a_scale * a'                          (skipped when a == nullptr)
//   n  = norm_w ? rmsnorm(h, norm_w) : h
//   normed_out (optional f32) = n ; quantised blocks of n -> out (optional)
// When row_index != nullptr, row r reads h[row_index[r]] and no residual is written back
// (used to gather the last token of each sequence before the output projection).
struct NormQuantArgs {
    float* h = nullptr;
    const float* a = nullptr;
    // a may arrive as a_splits partial sums a_split_stride floats apart (split-K matmul output); they are
    // added in index order before anything else
    int a_splits = 1;
    int64_t a_split_stride = 0;
    float a_scale = 1.f;
    const float* post_w = nullptr;
    const float* norm_w = nullptr;
    float eps = 1e-5f;
    int rows = 0, dim = 0;
    float* normed_out = nullptr;
    const int32_t* row_index = nullptr;
    int act_kind = ACT_Q8K;
    ActQ out;
};
void launch_add_norm_quant(const NormQuantArgs& a, cudaStream_t s);

// out = quantise(act(gate) * up) ; act 0 = SiLU, 1 = tanh-GELU.  gate/up are [T][F] with row stride ld.
// gate/up may arrive as `splits` partial sums `split_stride` floats apart (split-K matmul output), added in index
// order on the way in.
void launch_actmul_quant(const float* gate, const float* up, int ld, int T, int F, int act, int act_kind,
                         ActQ out, float* f32_out, cudaStream_t s, int splits = 1, int64_t split_stride = 0);

// ---- quantised matmul ---------------------------------------------------------------------
// y[t][n] = (sum_k x[t][k] W[n][k]) * out_scale, then optional tanh softcap; integer block dots
// against 8-bit activation blocks (CUDA-core path, any T; best for T <= 8).
void launch_qgemv(const QWeight& W, const ActQ& x, int T, float* y, int ldy, float out_scale, float softcap,
                  cudaStream_t s);
// Expert-grouped form: W holds `experts` matrices of W.rows x W.cols back to back; output rows
// [offsets[e], offsets[e+1]) are computed with expert e's matrix.  Output row p reads activation row
// src_row[p] (identity when src_row is null).
void launch_qgemv_grouped(const QWeight& W, int experts, const int32_t* offsets, const int32_t* src_row, const ActQ& x,
                          float* y, int ldy, cudaStream_t s);
// F32 weight matrix (MoE router): y[t][n] = sum_k x[t][k] W[n][k], f32 activations.
void launch_f32_gemv(const float* W, int out, int in, const float* x, int T, float* y, cudaStream_t s);

// ---- embedding ------------------------------------------------------------------------------
void launch_embed(const QWeight& W, const uint32_t* ids, int T, float scale, float* out, cudaStream_t s);

// ---- batch descriptor -----------------------------------------------------------------------
// Per-lane header uploaded by the host each tick.
struct LaneHeader {
    int32_t start_pos;    // absolute position of the lane's first token in this tick
    int32_t n_tokens;     // tokens of this lane in the tick
    int32_t table_off;    // offset of the lane's block table inside the concatenated table array
    int32_t n_blocks;     // entries of that table
};
struct BatchDesc {
    int lanes = 0, T = 0, max_tiles = 0;
    const LaneHeader* hdr = nullptr;   // [lanes]
    const uint32_t* tables = nullptr;  // concatenated block ids
    int32_t* cu_seqlens = nullptr;     // [lanes+1]
    int32_t* positions = nullptr;      // [T]
    int32_t* token_lane = nullptr;     // [T]
    int64_t* slots = nullptr;          // [T]  block*block_tokens + row
    int32_t* last_index = nullptr;     // [lanes] packed index of each lane's last token
    int32_t* tile_lane = nullptr;      // [max_tiles] attention query tiles: lane
    int32_t* tile_row0 = nullptr;      // [max_tiles] first query row (within the lane's chunk)
    int32_t* n_tiles = nullptr;        // [1]
    int32_t* error_flag = nullptr;     // [1] set non-zero when an index is out of range
};
void launch_build_batch(const BatchDesc& b, int block_tokens, int q_tile, cudaStream_t s);

// ---- RoPE + QK-norm + paged KV scatter --------------------------------------------------------
struct RopeKvArgs {
    float* q = nullptr;            // [T][q_heads*d]  rotated in place
    const float* k = nullptr;      // [T][kv_heads*d]
    const float* v = nullptr;      // [T][kv_heads*d]
    int ldq = 0, ldk = 0, ldv = 0;
    // q and k may arrive as qk_splits partial sums qk_split_stride floats apart (split-K matmul output), added in
    // index order on the way in; the rotated q is then written to q_out (row stride ldq_out) instead of in place
    int qk_splits = 1;
    int64_t qk_split_stride = 0;
    int v_splits = 1;              // the same for v
    int64_t v_split_stride = 0;
    float* q_out = nullptr;
    int ldq_out = 0;
    const float* q_norm_w = nullptr;  // [d] or null
    const float* k_norm_w = nullptr;  // [d] or null
    float norm_eps = 1e-6f;
    const float* cos_t = nullptr;  // [capacity][rotary_dim/2], null on NoPE layers
    const float* sin_t = nullptr;
    int rotary_dim = 0;
    const int32_t* positions = nullptr;  // [T]
    const int64_t* slots = nullptr;      // [T]
    void* k_pool = nullptr;        // [blocks][layers][kv_heads][block_tokens][d]
    void* v_pool = nullptr;
    int kv_f16 = 1;
    int T = 0, q_heads = 0, kv_heads = 0, d = 0, block_tokens = 16, layers = 0, layer = 0;
    int64_t pool_blocks = 0;  // see kv_page_index
};
void launch_rope_kv(const RopeKvArgs& a, cudaStream_t s);

// Copy `rows` token rows of every layer and head from block src to block dst (copy-on-write).
void launch_cow_copy(void* k_pool, void* v_pool, int kv_f16, int64_t src_block, int64_t dst_block, int rows,
                     int layers, int64_t pool_blocks, int kv_heads, int block_tokens, int d, cudaStream_t s);

// ---- attention ---------------------------------------------------------------------------------
struct AttnArgs {
    const float* q = nullptr;  // [T] rows of q_heads*d values, row stride ldq
    int ldq = 0;               // 0 = q_heads*d
    float* out = nullptr;      // [T][q_heads*d]
    const void* k_pool = nullptr;
    const void* v_pool = nullptr;
    int kv_f16 = 1;
    BatchDesc batch;
    int q_heads = 0, kv_heads = 0, d = 0, block_tokens = 16, layers = 0, layer = 0;
    int64_t pool_blocks = 0;  // see kv_page_index
    float scale = 1.f, softcap = 0.f;
    int window = 0;  // 0 = full causal
    int q_tile = 0;
};
void launch_paged_attention(const AttnArgs& a, cudaStream_t s);
int attention_q_tile(int q_heads, int kv_heads);

// ---- sampling ------------------------------------------------------------------------------------
// First-index argmax of each row of logits [B][vocab].  `scratch` is argmax_scratch_bytes(B) bytes of device
// memory that is zero before the first call; every call leaves it zero again.
size_t argmax_scratch_bytes(int B);
void launch_argmax(const float* logits, int B, int vocab, uint32_t* out, void* scratch, cudaStream_t s);

// Per-lane sampling of one tick: temperature <= 0 selects the first-index argmax; otherwise temperature / top-k / top-p
// with the uniform draw u in [0, 1) supplied by the host (Sampler::sample_stochastic, src/sampling.rs:145-169,337-390).
struct LaneSampling {
    float temperature;
    int32_t top_k;
    float top_p;
    float u;
};
// Whether the device kernel covers these settings (greedy, or 1 <= top_k <= 1024); the rest is sampled on the host.
bool device_sampling_covers(float temperature, int top_k, int vocab);
// One token per row of logits [B][vocab].  A row whose kept candidates add up to nothing leaves
// kSampleEmptyStatus | (row & 0xFFFF) in *status ("sampling distribution is empty", src/sampling.rs:352-355).
constexpr int32_t kSampleEmptyStatus = 0x534D0000;
void launch_sample(const float* logits, int B, int vocab, const LaneSampling* params_dev, uint32_t* out, int32_t* status, cudaStream_t s);

// ---- MoE -------------------------------------------------------------------------------------------
// Top-k routing with (logit desc, index asc) order and softmax over the selected k.  A row with a non-finite logit
// leaves kMoeRouteStatus | (row & 0xFFFF) in *status (when it is still zero); the choices written stay in range.
constexpr int32_t kMoeRouteStatus = 0x524F0000;
void launch_moe_route(const float* logits, int T, int experts, int k, int32_t* sel_experts, float* sel_weights,
                      int32_t* status, cudaStream_t s);

// Groups the (token, choice) pairs of a routed batch by expert: offsets [experts+1], pos_of_pair [T*k],
// token_of_pos [T*k] (the activation row each grouped position reads).
void launch_moe_group(const int32_t* sel_experts, int T, int k, int experts, int32_t* offsets, int32_t* pos_of_pair,
                      int32_t* token_of_pos, cudaStream_t s);
// out[t] = sum over the token's k choices in ascending expert order of weight * expert_out[pos]
// (the index_add order of SparseMoeFeedForward::forward, src/decoder.rs:424-439).  Only experts in [e_lo, e_hi) are
// read and added: the whole range on one GPU, one rank's experts under expert parallelism.
void launch_moe_combine(const float* expert_out, const int32_t* sel_experts, const float* sel_weights,
                        const int32_t* pos_of_pair, int T, int k, int hidden, int e_lo, int e_hi, float* out, cudaStream_t s);
// Expert parallelism: out[i] = sum over ranks r = 0, 1, ... (in that order) of gathered[r * count + i].
void launch_ep_sum(const float* gathered, int ranks, int64_t count, float* out, cudaStream_t s);
// Expert parallelism, fused: launch_moe_combine of this rank's experts, the exchange of the partial rows with the other
// ranks through peer stores into their exchange blocks (EpComm::open_exchange), and the sum in rank order, in one
// kernel.  All ranks call it with the same epoch.  A peer that does not deliver within wait_ns (5 s unless told
// otherwise) leaves a non-zero code (0x4550000 | peer) in *status and the forward's result is not to be used.
constexpr uint64_t kEpWaitNs = 5ull * 1000 * 1000 * 1000;
void launch_moe_combine_exchange(const float* expert_out, const int32_t* sel_experts, const float* sel_weights,
                                 const int32_t* pos_of_pair, int T, int k, int hidden, int e_lo, int e_hi, const EpPeers& peers,
                                 uint32_t epoch, float* out, int32_t* status, cudaStream_t s, uint64_t wait_ns = kEpWaitNs);

// Expert parallelism with data-parallel lanes (ep_dispatch.cu): the four steps around the expert matmuls of one MoE layer.
// `done` is ranks ints of device memory, zero before the first call (every call leaves it zero).  All ranks call these
// with the same epoch, in the same order.
void launch_ep_dispatch(const __half* grouped_rows, const int32_t* offsets, const EpDispatch& D, uint32_t epoch, int32_t* done, int32_t* status,
                        cudaStream_t s);
void launch_ep_regroup(const EpDispatch& D, uint32_t epoch, __half* merged, int32_t* comb_off, int32_t* src_start, int32_t* status, cudaStream_t s,
                       uint64_t wait_ns = kEpWaitNs);
void launch_ep_return(const float* expert_out, const int32_t* src_start, const EpDispatch& D, uint32_t epoch, int32_t* done, cudaStream_t s);
void launch_ep_wait_back(const EpDispatch& D, uint32_t epoch, int32_t* status, cudaStream_t s, uint64_t wait_ns = kEpWaitNs);
// Test stand-in for the expert matmuls: out[row] = merged[row] * (first_expert + local expert of the row + 1).
void launch_ep_scale_rows(const __half* merged, const int32_t* comb_off, int local_experts, int first_expert, int hidden, float* out, cudaStream_t s);
// This rank's result area of the exchange `epoch`: expert outputs of its routed rows in its own grouped order.
const float* ep_result_area(const EpDispatch& D, uint32_t epoch);

// out[p] = x[token_of_pos[p]] for p < P: rows of `width` halves (a multiple of 8) gathered into grouped order.
void launch_gather_rows_half(const __half* x, const int32_t* token_of_pos, int P, int width, __half* out, cudaStream_t s);

// Small helpers
void launch_add_inplace(float* h, const float* a, float scale, int64_t n, cudaStream_t s);

}  // namespace mk
