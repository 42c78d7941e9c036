// The decoder on the B200: GGUF weights resident in HBM in the layouts the kernels read, one
// contiguous paged K/V arena, and the per-tick graph of kernel launches on one CUDA stream.
// Mirrors DecoderModel of the reference (src/decoder.rs: load :2980-3105, forward_inner_batch
// :3146-3358) for the attention-only families llama, smollm3, qwen3, qwen3moe and gemma2.
#pragma once
#include "device_util.h"
#include "gguf_file.h"
#include "kernels.h"
#include "paged_lm.h"
#include "qgemm_tc.h"
#include "hgemm_tc.h"
#include "qstream_tc.h"
#include "attention_tc.h"
#include "ep_comm.h"

namespace mk {

struct LayerSpec {
    bool sliding = false;
    int window = 0;
    bool rope = true;
    double theta = 10000.0;
    bool qk_norm = false;
    int act = 0;           // 0 SiLU, 1 tanh-GELU
    bool sandwich = false; // Gemma-style post norms
    bool moe = false;
    float scale = 1.f;
    float softcap = 0.f;
};

struct ModelSpec {
    std::string arch;
    int vocab = 0, max_context = 0, layers = 0, hidden = 0, q_heads = 0, kv_heads = 0, head_dim = 0, ffn = 0, rotary_dim = 0;
    float eps = 1e-5f, embedding_scale = 1.f, final_logit_scale = 1.f, final_softcap = 0.f;
    bool tied = false, permute_qk = false;
    int experts = 0, experts_used = 0, expert_ffn = 0;
    std::vector<float> rope_factors;  // GGUF `rope_freqs.weight`: per-frequency divisors (Llama profile only), else empty
    std::vector<LayerSpec> layer;
};

// Reads the family spec from GGUF metadata (the reference's src/gguf_model.rs:1298-1461,1816-2533).
ModelSpec model_spec_from_gguf(const GgufFile& f);

// What validate_decoder_tensors found: the matrices and vectors the forward pass uploads.
struct GgufAudit {
    int64_t tensors_in_file = 0, matrices = 0, vectors = 0, matrix_bytes = 0;
};
// Every tensor of the spec present with the expected shape and a readable block format, nothing of another layer kind
// (src/gguf_model.rs:3388-3776); throws with the reference's wording on the first violation.  Host only.
GgufAudit validate_decoder_tensors(const GgufFile& f, const ModelSpec& s);

struct ModelConfig {
    int device = 0;
    int block_tokens = 16, slab_blocks = 8;
    int64_t kv_capacity_tokens = 4096, prefix_capacity_tokens = 0;
    bool kv_f16 = true;
    int max_batch_tokens = 2048, max_batch_lanes = 64;
    // 0 auto (integer GEMV for a few rows, in-kernel dequant GEMM for tens of rows, f16-image GEMM for wide
    // ticks when the image fits), 1 integer GEMV only, 2 in-kernel dequant GEMM whenever the shape allows,
    // 3 f16-image GEMM whenever more than 8 rows share a matrix, 4 like 0 but nothing falls back to the in-kernel
    // dequant GEMM (f16 images for wide ticks, streamed Q4_K / Q6_K blocks for 1..64 rows)
    int matmul_path = 0;
    // expert parallelism of a sparse-MoE model: this process holds experts [ep_rank, ep_rank + 1) * experts / ep_size
    // and exchanges per-layer partial sums with the other ranks; ep_size <= 1 keeps every expert here
    int ep_rank = 0, ep_size = 1;
    // 0: all ranks run the same ticks on the same tokens (partial sums exchanged); 1: every rank schedules its own
    // sequences and each MoE layer sends the routed rows to the experts' ranks and the outputs back (ep_dispatch.cu)
    int ep_mode = 0;
};

class Model : public PagedLm {
public:
    Model(const std::string& gguf_path, const ModelConfig& cfg);
    ~Model() override;

    const ModelSpec& model_spec() const { return ms_; }
    // Joins the expert-parallel group (collective over all ep_size ranks; `id` is EpComm::unique_id from rank 0).
    void ep_init(const uint8_t* id);
    // ep_mode 1: the exchanges of one tick for a rank that has no lane to run (it serves the other ranks' rows).
    void ep_idle_tick();
    bool device_sampling_covers(float temperature, int top_k) const override { return mk::device_sampling_covers(temperature, top_k, ms_.vocab); }
    float last_forward_ms() const override;
    int64_t launch_count() const override { return launches_; }
    int64_t h2d_bytes() const override { return h2d_bytes_; }
    int64_t d2h_bytes() const override { return d2h_bytes_; }
    void profile_enable(bool on) override;
    std::vector<KernelProfile> profile_query() override;

protected:
    void run_forward(const std::vector<LmLane>& lanes, KvReservation& r, uint32_t flags) override;
    void fetch_output(float* logits, uint32_t* tokens) override;
    void device_synchronize() override;

private:
    struct LayerWeights {
        DevBuf attn_norm, ffn_norm, post_attn_norm, post_ffn_norm, q_norm, k_norm, router;
        HalfWeight qkv_half, gu_half;  // f16 images of [wq; wk; wv] and [gate; up] stacked by rows
        // Q4_K matrices streamed by the narrow-batch matmul: [wq; wk] and [gate; up] share one buffer each
        DevBuf qk_raw, gu_raw;
        QStreamWeight qs_qk, qs_v, qs_o, qs_gu, qs_down;  // qs_gu: rows interleaved when the gated form is on
        DeviceWeight wq, wk, wv, wo, gate, up, down;  // dense FFN, or expert banks for MoE layers
    };
    void load_weights(const GgufFile& f);
    int ep_local_experts() const { return ms_.experts / std::max(cfg_.ep_size, 1); }
    int ep_first_expert() const { return cfg_.ep_size > 1 ? cfg_.ep_rank * ep_local_experts() : 0; }
    void upload_expert_bank(const GgufFile& f, const std::string& name, int experts, int64_t rows, int64_t cols, DeviceWeight& out);
    void upload_matrix(const GgufFile& f, const std::string& name, int64_t rows, int64_t cols, DeviceWeight& out, bool permute_heads,
                       int heads);
    void upload_f32(const GgufFile& f, const std::string& name, int64_t n, DevBuf& out);
    void matmul(const DeviceWeight& DW, const ActQ& x, int T, float* y, int ldy, float scale, float softcap);
    ActQ act_view(DevBuf& qs, DevBuf& d, DevBuf& bs, DevBuf& xh, int T, int dim, int kind, bool want_f16);
    bool tensor_path(const QWeight& W, int T) const;
    void rope_tables_for(double theta, const float*& cos_t, const float*& sin_t);

    ModelSpec ms_;
    ModelConfig cfg_;
    cudaStream_t stream_ = nullptr;
    cudaEvent_t ev_start_ = nullptr, ev_stop_ = nullptr;
    bool timed_ = false;
    int64_t launches_ = 0, h2d_bytes_ = 0, d2h_bytes_ = 0;
    // profiling: one event pair per launch group, resolved after the tick's barrier
    enum KClass { KC_GEMM_TC = 0, KC_HGEMM, KC_QSTREAM, KC_GEMV, KC_ATTN, KC_NORM_QUANT, KC_ROPE_KV, KC_ACTMUL, KC_EMBED, KC_BATCH, KC_SAMPLE, KC_MOE, KC_HGEMM_NARROW, KC_EP, KC_COUNT };
    struct ProfSpan { int cls; double bytes, flops; cudaEvent_t a, b; };
    bool profiling_ = false;
    std::vector<ProfSpan> spans_;
    std::vector<cudaEvent_t> event_pool_;
    KernelProfile prof_[KC_COUNT];
    void prof_begin(int cls, double bytes, double flops);
    void prof_end();
    void prof_resolve();

    std::vector<LayerWeights> lw_;
    DeviceWeight token_embd_, output_;
    DevBuf output_norm_;
    struct RopeTable { double theta; DevBuf cos_t, sin_t; };
    std::vector<std::unique_ptr<RopeTable>> rope_;

    DevBuf k_pool_, v_pool_;
    // per-tick staging
    PinnedBuf stage_host_;
    DevBuf stage_dev_;
    DevBuf cu_, pos_, tok_lane_, slots_, last_, tile_lane_, tile_row_, ntiles_, err_;
    // tensor-core attention: split-KV partials of one-token lanes
    DevBuf attn_part_o_, attn_part_ml_, attn_counters_;
    bool attn_tc_ = false;
    // f16 weight images for wide ticks
    DevBuf argmax_scratch_;
    bool half_cache_ = false;
    int hgemm_min_rows_ = 33;
    int64_t half_cache_bytes_ = 0;
    void build_half_cache();
    void build_qstream();
    bool qstream_ = false;
    bool qstream_gated_ = false;   // gate|up streamed with act(gate) * up in its epilogue
    bool qstream_qkv_ = false;     // [wq; wk] and wv go in one streamed launch
    bool qstream_moe_ = false;     // expert banks re-tiled for the expert-grouped form of the streamed matmul
    DevBuf e_xh_;                  // routed rows grouped by expert, f16 [T * experts_used][hidden]
    QStreamWeight qs_head_;        // output projection for narrow batches
    DevBuf v_partial_;  // split-K shares of the V projection on streamed ticks
    bool dense_matrices_ = false;  // some matrix is F32 / F16 / BF16 or was decoded at load: the f16 GEMM serves every row count
    void half_cache_refused(const char* why) const;
    int qstream_min_rows_ = 1;  // measured: from one row up the streamed kernel is level with the integer GEMV on 2-6 MB matrices and ahead above
    int matmul_stream(const QStreamWeight& W, const ActQ& x, int T, float* y, int ldy, int max_splits, const QStreamWeight* W2 = nullptr);
    HgemmScratch hgemm_scratch() const;
    // Returns the number of K shares; more than one means the result is the sum of that many partials in the
    // split-K scratch (see launch_hgemm_tc) and y was not written.
    int matmul_half(const HalfWeight& W, const ActQ& x, int T, float* y, int ldy, float scale, float softcap, int max_splits = 1,
                    float* partial = nullptr, size_t partial_floats = 0);
    int attn_max_entries_ = 0;
    AttnTcPlan attn_plan_;
    std::vector<int32_t> plan_sp_, plan_nt_, plan_nb_;
    // activations
    // qkv_: [T][AW + 2 KW] (q | k | v per row); gu_: [T][2 ffn] (gate | up per row)
    DevBuf h_, qkv_, attn_, proj_, gu_, down_, normed_, logits_, tokens_;
    DevBuf a_qs_, a_d_, a_bs_, a_xh_;   // quantised activations of width hidden / attention width
    DevBuf f_qs_, f_d_, f_bs_, f_xh_;   // quantised activations of width ffn
    DevBuf l_qs_, l_d_, l_bs_, l_xh_;   // last-token rows for the output projection
    // MoE
    DevBuf router_logits_, sel_e_, sel_w_, grp_off_, pos_of_pair_, tok_of_pos_, e_gate_, e_up_, e_down_;
    // expert parallelism: this rank's partial layer output [T][hidden] and all ranks' partials [ep_size][T][hidden]
    std::unique_ptr<EpComm> ep_;
    DevBuf ep_partial_, ep_gather_;
    // ep_mode 1: rows of all sources merged per local expert (f16 inputs, f16 gated activations, f32 outputs), their row
    // ranges, where each source's rows start, the completion counters of the two exchange kernels, and an all-zero
    // range table for a tick without rows
    DevBuf ep_merged_xh_, ep_merged_act_, ep_merged_out_, ep_comb_off_, ep_src_start_, ep_done_, ep_zero_off_;
    uint64_t ep_wait_ns_ = kEpWaitNs;
    const float* ep_exchange_layer(LayerWeights& w, const LayerSpec& ls, const __half* grouped_rows, const int32_t* offsets, int T);
    QgemmWorkspace tc_ws_;
    PinnedBuf out_host_;
    int out_lanes_ = 0;
    uint32_t out_flags_ = 0;
};

}  // namespace mk
