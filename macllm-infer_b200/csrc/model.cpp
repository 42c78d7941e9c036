// See model.h.  Line references are into the reference's sources.
#include "model.h"
#include <algorithm>
#include <cmath>
#include <cstring>

namespace mk {


namespace {

bool starts_with(const std::string& s, const std::string& p) { return s.compare(0, p.size(), p) == 0; }

}  // namespace

ModelSpec model_spec_from_gguf(const GgufFile& f) {
    ModelSpec s;
    s.arch = f.get_string("general.architecture");
    const std::string a = s.arch;
    if (a != "llama" && a != "smollm3" && a != "qwen3" && a != "qwen3moe" && a != "gemma2")
        throw std::runtime_error("GGUF architecture `" + a + "` is not supported on this path");
    s.layers = (int)f.get_int(a + ".block_count");
    s.hidden = (int)f.get_int(a + ".embedding_length");
    s.q_heads = (int)f.get_int(a + ".attention.head_count");
    s.kv_heads = (int)f.get_int_or(a + ".attention.head_count_kv", s.q_heads);
    s.head_dim = (int)f.get_int_or(a + ".attention.key_length", s.hidden / s.q_heads);
    if (f.has(a + ".attention.value_length") && f.get_int(a + ".attention.value_length") != s.head_dim)
        throw std::runtime_error("different key/value head widths are not supported");
    s.ffn = (int)f.get_int_or(a + ".feed_forward_length", 0);
    s.eps = (float)f.get_float(a + ".attention.layer_norm_rms_epsilon");
    s.max_context = (int)f.get_int(a + ".context_length");
    if (s.max_context <= 0 || s.max_context > (1 << 20)) throw std::runtime_error("GGUF context length is out of range");  // gguf_model.rs:63
    const GgufTensor& emb = f.require("token_embd.weight");
    s.vocab = (int)f.get_int_or(a + ".vocab_size", emb.dims[0]);
    if (emb.dims.size() != 2 || emb.dims[0] != s.vocab || emb.dims[1] != s.hidden)
        throw std::runtime_error("token_embd.weight shape does not match the model spec");
    s.tied = f.tensor("output.weight") == nullptr;  // gguf.rs:1203-1210
    s.rotary_dim = (int)f.get_int_or(a + ".rope.dimension_count", s.head_dim);
    double theta = f.get_float_or(a + ".rope.freq_base", 10000.0);
    s.permute_qk = (a == "llama" || a == "smollm3");  // gguf_model.rs:454-460
    if (const GgufTensor* rf = f.tensor("rope_freqs.weight")) {
        // only the Llama profile reads frequency factors (gguf_model.rs:1855,2015-2033); the others refuse the tensor
        // (gguf_model.rs:1302,2138,2244,2402)
        if (a == "gemma2") throw std::runtime_error("GGUF Gemma 2 RoPE frequency-factor tensors are not supported");
        if (a != "llama") throw std::runtime_error("GGUF " + a + " rope frequency factors are not supported yet");
        if (rf->type != QT_F32) throw std::runtime_error("GGUF `rope_freqs.weight` must be F32");
        if (rf->elements() != s.head_dim / 2)
            throw std::runtime_error("GGUF `rope_freqs.weight` has " + std::to_string(rf->elements()) + " factors, expected " +
                                     std::to_string(s.head_dim / 2) + " for head dimension " + std::to_string(s.head_dim));
        s.rope_factors.resize((size_t)rf->elements());
        memcpy(s.rope_factors.data(), rf->data, s.rope_factors.size() * 4);
        for (float v : s.rope_factors)
            if (!std::isfinite(v) || !(v > 0.f)) throw std::runtime_error("GGUF `rope_freqs.weight` factors must be finite and positive");
        if (s.rotary_dim != s.head_dim) throw std::runtime_error("partial Llama RoPE is not supported");  // gguf_model.rs:1851-1854
    }
    if (a == "smollm3" && s.layers != 36 && !f.has("macllm.allow_scaled_layers"))
        throw std::runtime_error("GGUF SmolLM3 must have exactly 36 layers");  // gguf_model.rs:2251-2254
    if (a == "qwen3moe") {
        s.experts = (int)f.get_int("qwen3moe.expert_count");
        s.experts_used = (int)f.get_int("qwen3moe.expert_used_count");
        s.expert_ffn = (int)f.get_int("qwen3moe.expert_feed_forward_length");
    }
    if (a == "gemma2") {
        if (!s.tied) throw std::runtime_error("Gemma 2 requires a tied output head and does not support `output.weight`");
        s.embedding_scale = (float)std::sqrt((double)s.hidden);  // gguf_model.rs:1345
        s.final_softcap = (float)f.get_float_or("gemma2.final_logit_softcapping", 0.0);
        s.rotary_dim = s.head_dim;
    }
    s.layer.resize((size_t)s.layers);
    for (int l = 0; l < s.layers; ++l) {
        LayerSpec& ls = s.layer[(size_t)l];
        ls.theta = theta;
        ls.scale = (float)(1.0 / std::sqrt((double)s.head_dim));
        ls.qk_norm = (a == "qwen3" || a == "qwen3moe");
        ls.moe = (a == "qwen3moe");
        if (a == "smollm3") ls.rope = ((l + 1) % 4) != 0;  // gguf_model.rs:2313-2324
        if (a == "gemma2") {                                 // gguf_model.rs:1400-1461
            int window = (int)f.get_int_or("gemma2.attention.sliding_window", 4096);
            ls.sliding = (l % 2 == 0);                       // gguf_model.rs:1491-1494
            ls.window = ls.sliding ? window : 0;
            ls.theta = ls.sliding ? f.get_float_or("gemma2.rope.freq_base_swa", theta) : theta;
            ls.softcap = (float)f.get_float("gemma2.attn_logit_softcapping");
            ls.act = 1;
            ls.sandwich = true;
            if (s.layers == 46) ls.scale = (float)(1.0 / std::sqrt((double)(s.hidden / s.q_heads)));
        }
    }
    return s;
}

// ---------------------------------------------------------------------------- load

Model::Model(const std::string& gguf_path, const ModelConfig& cfg) : cfg_(cfg) {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) {
        cudaGetLastError();
        throw std::runtime_error("no usable CUDA device: this library has no CPU fallback");
    }
    if (cfg.device < 0 || cfg.device >= ndev) throw std::runtime_error("device ordinal out of range");
    MK_CUDA(cudaSetDevice(cfg.device));
    GgufFile f(gguf_path);
    ms_ = model_spec_from_gguf(f);
    validate_decoder_tensors(f, ms_);  // before any device memory is touched
    if (cfg.ep_size > 1) {
        if (ms_.experts <= 0) throw std::runtime_error("expert parallelism asked for a model without experts");
        if (cfg.ep_rank < 0 || cfg.ep_rank >= cfg.ep_size) throw std::runtime_error("ep_rank out of range");
        if (ms_.experts % cfg.ep_size != 0) throw std::runtime_error("expert count is not a multiple of ep_size");
    }
    if (ms_.head_dim > 256 || ms_.head_dim % 4 != 0) throw std::runtime_error("head_dim must be a multiple of 4, at most 256");
    spec_.vocab = ms_.vocab;
    spec_.max_context = ms_.max_context;
    spec_.layers = ms_.layers;
    spec_.hidden = ms_.hidden;
    if (f.has("tokenizer.ggml.eos_token_id")) spec_.stop_ids.push_back((uint32_t)f.get_int("tokenizer.ggml.eos_token_id"));
    bool any_sliding = false;
    for (const LayerSpec& l : ms_.layer) any_sliding |= l.sliding;
    init_pool(cfg.block_tokens, cfg.slab_blocks, cfg.kv_capacity_tokens, cfg.prefix_capacity_tokens, !any_sliding);

    MK_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    MK_CUDA(cudaEventCreate(&ev_start_));
    MK_CUDA(cudaEventCreate(&ev_stop_));
    load_weights(f);

    const int64_t esz = cfg.kv_f16 ? 2 : 4;
    const int64_t block_elems = (int64_t)ms_.layers * ms_.kv_heads * cfg.block_tokens * ms_.head_dim;
    const int64_t pool_bytes = pool_->max_blocks() * block_elems * esz;
    k_pool_.alloc((size_t)pool_bytes);
    v_pool_.alloc((size_t)pool_bytes);
    k_pool_.zero(stream_);
    v_pool_.zero(stream_);
    spec_.kv_bytes_per_token = 2 * (int64_t)ms_.layers * ms_.kv_heads * ms_.head_dim * esz;

    const int T = cfg.max_batch_tokens, B = cfg.max_batch_lanes;
    const int AW = ms_.q_heads * ms_.head_dim, KW = ms_.kv_heads * ms_.head_dim;
    const int aw = std::max(ms_.hidden, AW);
    const bool moe = ms_.experts > 0;
    const int64_t P = moe ? (int64_t)T * ms_.experts_used : 0;
    const int fw = moe ? ms_.expert_ffn : ms_.ffn;
    const int64_t frows = moe ? P : T;
    cu_.alloc((size_t)(B + 1) * 4);
    pos_.alloc((size_t)T * 4);
    tok_lane_.alloc((size_t)T * 4);
    slots_.alloc((size_t)T * 8);
    last_.alloc((size_t)B * 4);
    tile_lane_.alloc((size_t)(T + B) * 4);
    tile_row_.alloc((size_t)(T + B) * 4);
    ntiles_.alloc(4);
    err_.alloc(4);
    err_.zero(stream_);
    h_.alloc((size_t)T * ms_.hidden * 4);
    qkv_.alloc((size_t)T * (AW + 2 * KW) * 4);
    attn_.alloc((size_t)T * AW * 4);
    proj_.alloc((size_t)T * ms_.hidden * 4);
    down_.alloc((size_t)T * ms_.hidden * 4);
    if (!moe) {
        gu_.alloc((size_t)T * 2 * ms_.ffn * 4);
    } else {
        normed_.alloc((size_t)T * ms_.hidden * 4);
        router_logits_.alloc((size_t)T * ms_.experts * 4);
        sel_e_.alloc((size_t)P * 4);
        sel_w_.alloc((size_t)P * 4);
        grp_off_.alloc((size_t)(ms_.experts + 1) * 4);
        pos_of_pair_.alloc((size_t)P * 4);
        tok_of_pos_.alloc((size_t)P * 4);
        e_gate_.alloc((size_t)P * fw * 4);
        e_up_.alloc((size_t)P * fw * 4);
        e_down_.alloc((size_t)P * ms_.hidden * 4);
        if (cfg_.ep_size > 1) {
            // rows of experts held elsewhere are never written here; keep them finite for the row-wise kernels
            e_gate_.zero(stream_);
            e_up_.zero(stream_);
            ep_partial_.alloc((size_t)T * ms_.hidden * 4);
            ep_gather_.alloc((size_t)cfg_.ep_size * T * ms_.hidden * 4);
        }
    }
    logits_.alloc((size_t)B * ms_.vocab * 4);
    tokens_.alloc((size_t)B * 4);
    argmax_scratch_.alloc(argmax_scratch_bytes(B));
    argmax_scratch_.zero(stream_);
    a_qs_.alloc((size_t)T * aw);
    a_d_.alloc((size_t)T * (aw / 32 + 1) * 4);
    a_bs_.alloc((size_t)T * (aw / 16 + 1) * 2);
    a_xh_.alloc((size_t)T * aw * 2);
    f_qs_.alloc((size_t)frows * fw);
    f_d_.alloc((size_t)frows * (fw / 32 + 1) * 4);
    f_bs_.alloc((size_t)frows * (fw / 16 + 1) * 2);
    f_xh_.alloc((size_t)frows * fw * 2);
    l_qs_.alloc((size_t)B * ms_.hidden);
    l_d_.alloc((size_t)B * (ms_.hidden / 32 + 1) * 4);
    l_bs_.alloc((size_t)B * (ms_.hidden / 16 + 1) * 2);
    l_xh_.alloc((size_t)B * ms_.hidden * 2);
    tc_ws_.status.alloc(4);
    tc_ws_.status.zero(stream_);
    // the largest split-K scratch any matmul of this model can ask for
    size_t partial = 0;
    auto consider = [&](const QWeight& w, int rows_t) {
        if (w.type == QT_Q4_K || w.type == QT_Q6_K || w.type == QT_Q8_0)
            for (int t : {9, 32, 64, 128, rows_t}) if (t <= rows_t && t > 0) partial = std::max(partial, qgemm_tc_partial_floats(w, t));
    };
    for (const LayerWeights& lw : lw_) {
        consider(lw.wq.w, T); consider(lw.wk.w, T); consider(lw.wv.w, T); consider(lw.wo.w, T);
        if (!moe) { consider(lw.gate.w, T); consider(lw.up.w, T); consider(lw.down.w, T); }
    }
    consider(ms_.tied ? token_embd_.w : output_.w, B);
    tc_ws_.partial.alloc(std::max<size_t>(partial, 1) * 4);
    size_t stage_bytes = (size_t)B * sizeof(LaneHeader) + (size_t)(pool_->max_blocks() + B) * 4 + (size_t)T * 4 + 64 +
                         (size_t)B * sizeof(LaneSampling) + 16;
    attn_tc_ = attention_tc_supported(ms_.q_heads, ms_.kv_heads, ms_.head_dim, cfg_.block_tokens, cfg_.kv_f16);
    if (attn_tc_) {
        attn_max_entries_ = attention_tc_max_entries(B, ms_.kv_heads);
        attn_part_o_.alloc((size_t)attn_max_entries_ * ms_.kv_heads * 16 * ms_.head_dim * 4);
        attn_part_ml_.alloc((size_t)attn_max_entries_ * ms_.kv_heads * 16 * 2 * 4);
        attn_counters_.alloc((size_t)B * ms_.kv_heads * 4);
        attn_counters_.zero(stream_);
        // work lists: key-share entries (8 ints), prefill tiles (2 ints), split one-token lanes (3 ints)
        stage_bytes += ((size_t)(T + B) * 2 + (size_t)attn_max_entries_ * 8 + (size_t)B * 3) * 4 + 16;
    }
    stage_host_.ensure(stage_bytes);
    stage_dev_.alloc(stage_bytes);
    out_host_.ensure((size_t)B * ms_.vocab * 4 + (size_t)B * 4 + 16);
    MK_CUDA(cudaStreamSynchronize(stream_));
    build_half_cache();
    build_qstream();
}

Model::~Model() {
    if (stream_) cudaStreamSynchronize(stream_);
    if (ev_start_) cudaEventDestroy(ev_start_);
    if (ev_stop_) cudaEventDestroy(ev_stop_);
    if (stream_) cudaStreamDestroy(stream_);
}

void Model::upload_f32(const GgufFile& f, const std::string& name, int64_t n, DevBuf& out) {
    const GgufTensor& t = f.require(name);
    if (t.type != QT_F32 || t.elements() != n) throw std::runtime_error("tensor `" + name + "` must be F32 with " + std::to_string(n) + " elements");
    out.upload(t.data, (size_t)n * 4, stream_);
    MK_CUDA(cudaStreamSynchronize(stream_));
}

void Model::upload_matrix(const GgufFile& f, const std::string& name, int64_t rows, int64_t cols, DeviceWeight& out,
                          bool permute_heads, int heads) {
    const GgufTensor& t = f.require(name);
    int64_t total_rows = t.elements() / t.dims.back();
    if (t.dims.back() != cols || total_rows != rows)
        throw std::runtime_error("tensor `" + name + "` has shape that does not match the model spec");  // validate_decoder_tensors, gguf_model.rs:3388-3420
    if (!permute_heads) {
        upload_weight(t.type, t.data, rows, cols, out, stream_);
    } else {
        // llama.cpp stores Q/K rows pair-interleaved; undo it so the half-split rotation applies
        // (src/gguf.rs:1888-1924): source row head*d + 2*pair + lane -> dest head*d + lane*d/2 + pair.
        int64_t rb = gguf_row_bytes(t.type, cols);
        std::vector<uint8_t> tmp((size_t)(rb * rows));
        unpermute_qk_rows_host(t.data, rows, rb, heads, tmp.data());
        upload_weight(t.type, tmp.data(), rows, cols, out, stream_);
    }
    spec_.weight_bytes += out.w.bytes;
}

// An expert bank [experts * rows][cols]; with expert parallelism only this rank's contiguous share of the experts
// is uploaded (expert e lives on rank e / (experts / ep_size)).
void Model::upload_expert_bank(const GgufFile& f, const std::string& name, int experts, int64_t rows, int64_t cols, DeviceWeight& out) {
    const GgufTensor& t = f.require(name);
    int64_t total_rows = t.elements() / t.dims.back();
    if (t.dims.back() != cols || total_rows != rows * experts)
        throw std::runtime_error("tensor `" + name + "` has shape that does not match the model spec");
    int64_t rb = gguf_row_bytes(t.type, cols);
    int local = ep_local_experts();
    upload_weight(t.type, t.data + (int64_t)ep_first_expert() * rows * rb, rows * local, cols, out, stream_);
    spec_.weight_bytes += out.w.bytes;
}

void Model::ep_init(const uint8_t* id) {
    if (cfg_.ep_size <= 1) throw std::runtime_error("mk_model_ep_init on a model loaded without expert parallelism");
    MK_CUDA(cudaSetDevice(cfg_.device));
    ep_ = std::make_unique<EpComm>(cfg_.ep_rank, cfg_.ep_size, id);
    // MACLLM_B200_EP_FUSED=0 keeps the exchange on NCCL (all-gather + a sum kernel) instead of the fused kernel
    const char* fused = getenv("MACLLM_B200_EP_FUSED");
    if (cfg_.ep_mode == 1) {
        if (!qstream_moe_) throw std::runtime_error("expert parallelism with data-parallel lanes needs Q4_K / Q6_K expert banks of whole 128-row tiles");
        if (cfg_.ep_size > kEpMaxRanks) throw std::runtime_error("expert parallelism with data-parallel lanes: at most 8 ranks");
        const int EL = ep_local_experts(), N = cfg_.ep_size;
        const int64_t cap = (int64_t)cfg_.max_batch_tokens * ms_.experts_used;
        ep_->open_dispatch(cap, ms_.hidden, EL, stream_);
        // how long a rank waits for a peer's rows before it reports the peer missing (MACLLM_B200_EP_WAIT_MS, default 5 s)
        if (const char* e = std::getenv("MACLLM_B200_EP_WAIT_MS")) ep_wait_ns_ = (uint64_t)std::max(1, atoi(e)) * 1000000ull;
        ep_merged_xh_.alloc((size_t)N * cap * ms_.hidden * 2);
        ep_merged_act_.alloc((size_t)N * cap * ms_.expert_ffn * 2);
        ep_merged_out_.alloc((size_t)N * cap * ms_.hidden * 4);
        ep_comb_off_.alloc((size_t)(EL + 1) * 4);
        ep_src_start_.alloc((size_t)N * EL * 4);
        ep_done_.alloc((size_t)2 * kEpMaxRanks * 4);
        ep_zero_off_.alloc((size_t)(ms_.experts + 1) * 4);
        MK_CUDA(cudaMemsetAsync(ep_done_.ptr(), 0, (size_t)2 * kEpMaxRanks * 4, stream_));
        MK_CUDA(cudaMemsetAsync(ep_zero_off_.ptr(), 0, (size_t)(ms_.experts + 1) * 4, stream_));
        MK_CUDA(cudaMemsetAsync(ep_comb_off_.ptr(), 0, (size_t)(EL + 1) * 4, stream_));
        MK_CUDA(cudaStreamSynchronize(stream_));
        return;
    }
    if ((fused == nullptr || strcmp(fused, "0") != 0) && cfg_.ep_size <= kEpMaxRanks)
        ep_->open_exchange(cfg_.max_batch_tokens, ms_.hidden, stream_);
}

// The column width the expert-grouped matmuls are launched with: rows of one expert are processed in chunks of that many,
// and a chunk costs the same whether it is full or not, so a tick whose experts see a handful of rows each runs narrow
// chunks (an expert with more rows than one chunk takes a second pass over its weights), a wide tick runs full ones.
// MACLLM_B200_MOE_CHUNK=16|32|64 pins it.
static int moe_chunk_rows(int T, int k, int experts) {
    static const int pinned = [] { const char* e = std::getenv("MACLLM_B200_MOE_CHUNK"); return e ? atoi(e) : 0; }();
    if (pinned == 16 || pinned == 32 || pinned == 64) return pinned;
    const double avg = (double)T * k / std::max(experts, 1);
    return avg <= 6.0 ? 16 : (avg <= 14.0 ? 32 : 64);
}

// One MoE layer's experts under data-parallel expert parallelism: this rank's routed rows (grouped by expert, f16) go to
// the ranks that hold the experts, the rows this rank received run through its expert banks, and the outputs go back.
// Returns the area that holds the outputs of this rank's own rows in its own grouped order.
const float* Model::ep_exchange_layer(LayerWeights& w, const LayerSpec& ls, const __half* grouped_rows, const int32_t* offsets, int T) {
    const EpDispatch& D = ep_->dispatch();
    const int EL = ep_local_experts(), H = ms_.hidden, F = ms_.expert_ffn;
    const int capacity = (int)std::min<int64_t>((int64_t)D.ranks * D.cap_rows, INT32_MAX);
    const uint32_t epoch = ep_->next_epoch();
    int32_t* status = tc_ws_.status.as<int32_t>();
    // the other ranks' row counts are not known on the host (a peer may run a prefill chunk while this rank decodes), and
    // a narrow chunk under many rows costs a pass over the expert's weights per chunk: always the full width
    (void)T;
    const int chunk = kQStreamMaxRows;
    // the time of the two exchange halves includes waiting for the slowest peer; rows are not known on the host, so the
    // profile's byte counts are the weights alone
    prof_begin(KC_EP, 0, 0);
    launch_ep_dispatch(grouped_rows, offsets, D, epoch, ep_done_.as<int32_t>(), status, stream_);
    launch_ep_regroup(D, epoch, ep_merged_xh_.as<__half>(), ep_comb_off_.as<int32_t>(), ep_src_start_.as<int32_t>(), status, stream_, ep_wait_ns_);
    prof_end();
    prof_begin(KC_QSTREAM, (double)w.qs_gu.rows * (double)(w.qs_gu.cols / 256) * 144.0, 0);
    launch_qstream_tc_grouped(w.qs_gu, EL, ep_comb_off_.as<int32_t>(), ep_merged_xh_.as<__half>(), capacity, chunk, nullptr, 0, status,
                              stream_, ls.act, ep_merged_act_.as<__half>(), F, false);
    prof_end();
    prof_begin(KC_QSTREAM, (double)w.qs_down.rows * (double)(w.qs_down.cols / 256) * (w.qs_down.fmt ? 210.0 : 144.0), 0);
    launch_qstream_tc_grouped(w.qs_down, EL, ep_comb_off_.as<int32_t>(), ep_merged_act_.as<__half>(), capacity, chunk,
                              ep_merged_out_.as<float>(), H, status, stream_, -1, nullptr, 0, false);
    prof_end();
    prof_begin(KC_EP, 0, 0);
    launch_ep_return(ep_merged_out_.as<float>(), ep_src_start_.as<int32_t>(), D, epoch, ep_done_.as<int32_t>() + kEpMaxRanks, stream_);
    launch_ep_wait_back(D, epoch, status, stream_, ep_wait_ns_);
    prof_end();
    launches_ += 6;
    return ep_result_area(D, epoch);
}

void Model::ep_idle_tick() {
    if (cfg_.ep_mode != 1 || !ep_ || !ep_->has_dispatch()) throw std::runtime_error("ep_idle_tick needs a model in data-parallel expert parallelism after mk_model_ep_init");
    MK_CUDA(cudaSetDevice(cfg_.device));
    for (int l = 0; l < ms_.layers; ++l)
        if (ms_.layer[(size_t)l].moe) ep_exchange_layer(lw_[(size_t)l], ms_.layer[(size_t)l], e_xh_.as<__half>(), ep_zero_off_.as<int32_t>(), 0);
}

void Model::load_weights(const GgufFile& f) {
    const int H = ms_.hidden, AW = ms_.q_heads * ms_.head_dim, KW = ms_.kv_heads * ms_.head_dim;
    upload_matrix(f, "token_embd.weight", ms_.vocab, H, token_embd_, false, 0);
    if (!ms_.tied) upload_matrix(f, "output.weight", ms_.vocab, H, output_, false, 0);
    upload_f32(f, "output_norm.weight", H, output_norm_);
    int64_t per_token = (ms_.tied ? token_embd_.w.bytes : output_.w.bytes);
    lw_.resize((size_t)ms_.layers);
    for (int l = 0; l < ms_.layers; ++l) {
        LayerWeights& w = lw_[(size_t)l];
        const LayerSpec& ls = ms_.layer[(size_t)l];
        std::string p = "blk." + std::to_string(l) + ".";
        upload_f32(f, p + "attn_norm.weight", H, w.attn_norm);
        upload_matrix(f, p + "attn_q.weight", AW, H, w.wq, ms_.permute_qk, ms_.q_heads);
        upload_matrix(f, p + "attn_k.weight", KW, H, w.wk, ms_.permute_qk, ms_.kv_heads);
        upload_matrix(f, p + "attn_v.weight", KW, H, w.wv, false, 0);
        upload_matrix(f, p + "attn_output.weight", H, AW, w.wo, false, 0);
        per_token += w.wq.w.bytes + w.wk.w.bytes + w.wv.w.bytes + w.wo.w.bytes;
        if (ls.qk_norm) {
            upload_f32(f, p + "attn_q_norm.weight", ms_.head_dim, w.q_norm);
            upload_f32(f, p + "attn_k_norm.weight", ms_.head_dim, w.k_norm);
        }
        upload_f32(f, p + "ffn_norm.weight", H, w.ffn_norm);
        if (ls.sandwich) {
            upload_f32(f, p + "post_attention_norm.weight", H, w.post_attn_norm);
            upload_f32(f, p + "post_ffw_norm.weight", H, w.post_ffn_norm);
        }
        if (!ls.moe) {
            upload_matrix(f, p + "ffn_gate.weight", ms_.ffn, H, w.gate, false, 0);
            upload_matrix(f, p + "ffn_up.weight", ms_.ffn, H, w.up, false, 0);
            upload_matrix(f, p + "ffn_down.weight", H, ms_.ffn, w.down, false, 0);
            per_token += w.gate.w.bytes + w.up.w.bytes + w.down.w.bytes;
        } else {
            const int E = ms_.experts, F = ms_.expert_ffn;
            upload_f32(f, p + "ffn_gate_inp.weight", (int64_t)E * H, w.router);
            upload_expert_bank(f, p + "ffn_gate_exps.weight", E, F, H, w.gate);
            upload_expert_bank(f, p + "ffn_up_exps.weight", E, F, H, w.up);
            upload_expert_bank(f, p + "ffn_down_exps.weight", E, H, F, w.down);
            per_token += (w.gate.w.bytes + w.up.w.bytes + w.down.w.bytes) / ep_local_experts() * ms_.experts_used + (int64_t)E * H * 4;
            // the grouped kernels address one expert's matrix at a time
            w.gate.w.rows = F;
            w.up.w.rows = F;
            w.down.w.rows = H;
        }
    }
    spec_.weight_bytes_per_token = per_token;
}

void Model::rope_tables_for(double theta, const float*& cos_t, const float*& sin_t) {
    for (auto& r : rope_)
        if (r->theta == theta) { cos_t = r->cos_t.as<float>(); sin_t = r->sin_t.as<float>(); return; }
    // RotaryEmbedding::new / tables (src/decoder.rs:136-201): inverse frequencies in f64 then f32,
    // angle = f32(position) * inv_freq, cos/sin in f32.
    int half = ms_.rotary_dim / 2;
    int64_t capacity = std::min<int64_t>(ms_.max_context, std::max<int64_t>(pool_->max_blocks() * pool_->block_tokens(), 256));
    std::vector<float> inv((size_t)half), c((size_t)(capacity * half)), s((size_t)(capacity * half));
    for (int i = 0; i < half; ++i) {
        double base = 1.0 / std::pow(theta, (double)(2 * i) / (double)ms_.rotary_dim);
        inv[(size_t)i] = ms_.rope_factors.empty() ? (float)base : (float)(base / (double)ms_.rope_factors[(size_t)i]);
    }
    for (int64_t p = 0; p < capacity; ++p)
        for (int i = 0; i < half; ++i) {
            float a = (float)p * inv[(size_t)i];
            c[(size_t)(p * half + i)] = cosf(a);
            s[(size_t)(p * half + i)] = sinf(a);
        }
    auto t = std::make_unique<RopeTable>();
    t->theta = theta;
    t->cos_t.upload(c.data(), c.size() * 4, stream_);
    t->sin_t.upload(s.data(), s.size() * 4, stream_);
    MK_CUDA(cudaStreamSynchronize(stream_));
    cos_t = t->cos_t.as<float>();
    sin_t = t->sin_t.as<float>();
    rope_.push_back(std::move(t));
}

// ---------------------------------------------------------------------------- profiling

static const char* kclass_names[] = {"qgemm_tc", "hgemm_tc", "qstream_tc", "qgemv", "paged_attention", "add_norm_quant", "rope_kv_scatter", "actmul_quant",
                                     "embed", "build_batch", "argmax", "moe", "hgemm_tc_splitk", "ep_exchange"};

void Model::profile_enable(bool on) {
    profiling_ = on;
    if (on) for (int i = 0; i < KC_COUNT; ++i) { prof_[i] = KernelProfile{}; prof_[i].name = kclass_names[i]; }
}

void Model::prof_begin(int cls, double bytes, double flops) {
    if (!profiling_) return;
    ProfSpan sp;
    sp.cls = cls;
    sp.bytes = bytes;
    sp.flops = flops;
    for (cudaEvent_t* e : {&sp.a, &sp.b}) {
        if (event_pool_.empty()) {
            MK_CUDA(cudaEventCreate(e));
        } else {
            *e = event_pool_.back();
            event_pool_.pop_back();
        }
    }
    MK_CUDA(cudaEventRecord(sp.a, stream_));
    spans_.push_back(sp);
}

void Model::prof_end() {
    if (!profiling_ || spans_.empty()) return;
    MK_CUDA(cudaEventRecord(spans_.back().b, stream_));
}

void Model::prof_resolve() {
    for (ProfSpan& sp : spans_) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, sp.a, sp.b) == cudaSuccess) {
            KernelProfile& k = prof_[sp.cls];
            ++k.launches;
            k.ms += ms;
            k.bytes += sp.bytes;
            k.flops += sp.flops;
        } else {
            cudaGetLastError();
        }
        event_pool_.push_back(sp.a);
        event_pool_.push_back(sp.b);
    }
    spans_.clear();
}

std::vector<PagedLm::KernelProfile> Model::profile_query() {
    std::vector<KernelProfile> out;
    for (int i = 0; i < KC_COUNT; ++i) if (prof_[i].launches > 0) out.push_back(prof_[i]);
    return out;
}

// ---------------------------------------------------------------------------- forward

bool Model::tensor_path(const QWeight& W, int T) const {
    if (cfg_.matmul_path == 1) return false;
    if (W.type != QT_Q4_K && W.type != QT_Q6_K && W.type != QT_Q8_0) return false;
    if (W.cols % 256 != 0) return false;
    return cfg_.matmul_path == 2 ? true : T > 8;
}

ActQ Model::act_view(DevBuf& qs, DevBuf& d, DevBuf& bs, DevBuf& xh, int, int, int, bool want_f16) {
    ActQ a;
    a.qs = qs.as<int8_t>();
    a.d = d.as<float>();
    a.bsums = bs.as<int16_t>();
    a.xh = want_f16 ? xh.as<__half>() : nullptr;
    return a;
}

HgemmScratch Model::hgemm_scratch() const {
    HgemmScratch ws;
    ws.partial = tc_ws_.partial.as<float>();
    ws.partial_floats = tc_ws_.partial.size() / 4;
    ws.status = tc_ws_.status.as<int32_t>();
    return ws;
}

int Model::matmul_half(const HalfWeight& W, const ActQ& x, int T, float* y, int ldy, float scale, float softcap, int max_splits,
                       float* partial, size_t partial_floats) {
    // narrow ticks run the 64-token instantiation with K shared out over CTAs: a weight-streaming kernel, accounted apart
    prof_begin(T <= 64 ? KC_HGEMM_NARROW : KC_HGEMM, 2.0 * (double)W.rows * (double)W.cols + 2.0 * T * W.cols + 4.0 * T * W.rows,
               2.0 * T * (double)W.rows * (double)W.cols);
    HgemmScratch ws = hgemm_scratch();
    if (partial != nullptr) {
        ws.partial = partial;
        ws.partial_floats = partial_floats;
    }
    int splits = launch_hgemm_tc(W, x.xh, T, y, ldy, scale, softcap, ws, stream_, max_splits);
    prof_end();
    ++launches_;
    return splits;
}

void Model::matmul(const DeviceWeight& DW, const ActQ& x, int T, float* y, int ldy, float scale, float softcap) {
    const QWeight& W = DW.w;
    if (DW.half.ready && T >= hgemm_min_rows_ && x.xh != nullptr) {
        matmul_half(DW.half, x, T, y, ldy, scale, softcap);
        return;
    }
    if (W.type == QT_F32) throw std::runtime_error("a dense matrix reached the quantised matmul paths (its f16 image is missing)");
    const bool tc = tensor_path(W, T) && x.xh != nullptr;
    // algorithmic traffic of one call: the matrix as stored, the activation rows as consumed, the f32 result
    const double act_bytes = tc ? 2.0 * T * W.cols : 1.0 * T * W.cols;
    prof_begin(tc ? KC_GEMM_TC : KC_GEMV, (double)W.bytes + act_bytes + 4.0 * T * W.rows, 2.0 * T * (double)W.rows * (double)W.cols);
    struct End { Model* m; ~End() { m->prof_end(); } } end{this};
    if (tc) {
        size_t need = qgemm_tc_partial_floats(W, T);
        tc_ws_.partial.ensure(need * 4);
        launch_qgemm_tc_scratch(W, x, T, y, ldy, scale, softcap, tc_ws_.partial.as<float>(), tc_ws_.status.as<int32_t>(), stream_);
        launches_ += need > 0 ? 2 : 1;
    } else {
        launch_qgemv(W, x, T, y, ldy, scale, softcap, stream_);
        ++launches_;
    }
}

// The f16 images of the dense layer matrices (2 bytes per weight), built when the configuration asks for
// them and, in automatic mode, only when they fit beside everything else with room to spare.
void Model::build_half_cache() {
    // Matrices without a quantised kernel - F32 / F16 / BF16 in the file, or a block format decoded at load - are dense
    // (the reference multiplies them without quantising the activations, src/model_weights.rs:346-377): the f16 GEMM
    // serves them at every row count, so their images are not optional and every matmul of the model takes that route.
    DeviceWeight& head_first = ms_.tied ? token_embd_ : output_;
    dense_matrices_ = head_first.w.type == QT_F32;
    for (size_t l = 0; l < lw_.size(); ++l) {
        LayerWeights& w = lw_[l];
        for (DeviceWeight* dw : {&w.wq, &w.wk, &w.wv, &w.wo}) dense_matrices_ |= dw->w.type == QT_F32;
        if (!ms_.layer[l].moe)
            for (DeviceWeight* dw : {&w.gate, &w.up, &w.down}) dense_matrices_ |= dw->w.type == QT_F32;
    }
    if (dense_matrices_ && cfg_.matmul_path != 0 && cfg_.matmul_path != 3 && cfg_.matmul_path != 4)
        throw std::runtime_error("this checkpoint has dense matrices (F32 / F16 / BF16, or a block format decoded at load): they need the f16 "
                                 "images, which matmul_path " + std::to_string(cfg_.matmul_path) + " does not build");
    if (cfg_.matmul_path != 0 && cfg_.matmul_path != 3 && cfg_.matmul_path != 4) return;
    hgemm_min_rows_ = dense_matrices_ ? 1 : (cfg_.matmul_path == 0 ? 33 : 9);
    size_t total = 0;
    for (size_t l = 0; l < lw_.size(); ++l) {
        LayerWeights& w = lw_[l];
        for (DeviceWeight* dw : {&w.wq, &w.wk, &w.wv, &w.wo}) {
            if (!hgemm_tc_supported(dw->w)) { half_cache_refused("a layer matrix the f16 GEMM does not take"); return; }  // all or nothing: the forward pass takes one route per tick
            total += half_weight_bytes(dw->w);
        }
        if (!ms_.layer[l].moe)
            for (DeviceWeight* dw : {&w.gate, &w.up, &w.down}) {
                if (!hgemm_tc_supported(dw->w)) { half_cache_refused("a layer matrix the f16 GEMM does not take"); return; }
                total += half_weight_bytes(dw->w);
            }
    }
    // the output head joins when batches of lanes can be wide enough to use it
    DeviceWeight& head_dw = ms_.tied ? token_embd_ : output_;
    const bool head_half = hgemm_tc_supported(head_dw.w) && cfg_.max_batch_lanes >= hgemm_min_rows_;
    if (head_half) total += half_weight_bytes(head_dw.w);
    if (cfg_.matmul_path == 0) {
        if (cfg_.max_batch_tokens < hgemm_min_rows_) return;
        size_t free_b = 0, total_b = 0;
        MK_CUDA(cudaMemGetInfo(&free_b, &total_b));
        if (total + (size_t(4) << 30) > free_b) { half_cache_refused("not enough free device memory for the f16 images"); return; }  // keep 4 GiB of headroom
    }
    if (dense_matrices_ && !head_half) half_cache_refused("an output matrix the f16 GEMM does not take");
    if (head_half) build_half_weight(head_dw.w, head_dw.half, stream_);
    for (size_t l = 0; l < lw_.size(); ++l) {
        LayerWeights& w = lw_[l];
        const QWeight* qkv[3] = {&w.wq.w, &w.wk.w, &w.wv.w};
        build_half_weight_stacked(qkv, 3, w.qkv_half, stream_);
        build_half_weight(w.wo.w, w.wo.half, stream_);
        build_half_weight(w.wv.w, w.wv.half, stream_);  // V alone, for ticks whose Q and K come from the streamed matmul
        if (!ms_.layer[l].moe) {
            // gate and up rows interleaved: the GEMM that uses this image finishes the gated activation itself
            build_half_weight_interleaved(w.gate.w, w.up.w, w.gu_half, stream_);
            build_half_weight(w.down.w, w.down.half, stream_);
        }
    }
    tc_ws_.partial.ensure(kSplitScratchBytes);
    MK_CUDA(cudaStreamSynchronize(stream_));
    half_cache_ = true;
    half_cache_bytes_ = (int64_t)total;
}

// Quantised models simply stay on the integer paths without the images; a model with dense matrices cannot run.
void Model::half_cache_refused(const char* why) const {
    if (dense_matrices_) throw std::runtime_error(std::string("this checkpoint has dense matrices, which need the f16 images: ") + why);
}

// Re-tiled copies for the narrow-batch matmul over raw Q4_K / Q6_K blocks.  [wq; wk] and [gate; up] are moved into one
// buffer each (rows stacked) so that one launch covers both; nothing of the row-major blocks is duplicated.
void Model::build_qstream() {
    if (cfg_.matmul_path != 0 && cfg_.matmul_path != 4) return;
    if (!half_cache_) return;  // wide ticks ride on the f16 images
    auto q4k = [](const DeviceWeight& d) { return d.w.type == QT_Q4_K && d.w.cols % 256 == 0; };
    auto kq = [](const DeviceWeight& d) { return (d.w.type == QT_Q4_K || d.w.type == QT_Q6_K) && d.w.cols % 256 == 0; };
    auto stack = [&](DeviceWeight& a, DeviceWeight& b, DevBuf& out) {
        out.alloc((size_t)(a.w.bytes + b.w.bytes));
        MK_CUDA(cudaMemcpyAsync(out.ptr(), a.w.p0, (size_t)a.w.bytes, cudaMemcpyDeviceToDevice, stream_));
        MK_CUDA(cudaMemcpyAsync(out.as<uint8_t>() + a.w.bytes, b.w.p0, (size_t)b.w.bytes, cudaMemcpyDeviceToDevice, stream_));
        MK_CUDA(cudaStreamSynchronize(stream_));
        a.b0.release();
        b.b0.release();
        a.w.p0 = out.ptr();
        b.w.p0 = out.as<uint8_t>() + a.w.bytes;
    };
    auto retile = [&](const QWeight& w, QStreamWeight& out) {
        if (w.type == QT_Q4_K) build_qstream_weight(w.p0, w.rows, w.cols, out, stream_);
        else build_qstream_weight_q6k(w, out, stream_);
    };
    bool qkv_one = true;
    const bool moe = ms_.experts > 0;
    if (moe && ((2 * ms_.expert_ffn) % 128 != 0 || ms_.hidden % 128 != 0)) return;  // experts are whole row tiles
    for (size_t l = 0; l < lw_.size(); ++l) {
        LayerWeights& w = lw_[l];
        if (ms_.layer[l].moe != moe) return;
        if (!q4k(w.wq) || !q4k(w.wk) || !kq(w.wo) || !q4k(w.gate) || !q4k(w.up) || !kq(w.down)) return;
        if (!w.wv.half.ready) return;
        // one launch for q | k | v needs the Q4_K part to end on a row-tile boundary
        if (!kq(w.wv) || (w.wq.w.rows + w.wk.w.rows) % 128 != 0) qkv_one = false;
    }
    // act(gate) * up in the epilogue of the streamed gate|up matmul (rows interleaved); MACLLM_B200_QS_GATED=0 keeps the
    // plain form with the separate activation kernel
    { const char* e = std::getenv("MACLLM_B200_QS_GATED"); qstream_gated_ = moe || e == nullptr || e[0] != '0'; }
    for (size_t l = 0; l < lw_.size(); ++l) {
        LayerWeights& w = lw_[l];
        stack(w.wq, w.wk, w.qk_raw);
        stack(w.gate, w.up, w.gu_raw);
        build_qstream_weight(w.qk_raw.ptr(), w.wq.w.rows + w.wk.w.rows, w.wq.w.cols, w.qs_qk, stream_);
        if (qkv_one) retile(w.wv.w, w.qs_v);
        retile(w.wo.w, w.qs_o);
        if (!moe) {
            build_qstream_weight(w.gu_raw.ptr(), w.gate.w.rows + w.up.w.rows, w.gate.w.cols, w.qs_gu, stream_, qstream_gated_ ? w.gate.w.rows : 0);
            retile(w.down.w, w.qs_down);
        } else {
            // expert banks (this rank's experts): [gate bank; up bank] with the rows of every expert interleaved, and the
            // down bank; w.rows holds the rows of ONE expert
            const int64_t EL = ep_local_experts();
            build_qstream_weight(w.gu_raw.ptr(), 2 * EL * w.gate.w.rows, w.gate.w.cols, w.qs_gu, stream_, EL * w.gate.w.rows);
            QWeight bank = w.down.w;
            bank.rows = EL * w.down.w.rows;
            retile(bank, w.qs_down);
        }
    }
    if (moe) {
        e_xh_.alloc((size_t)cfg_.max_batch_tokens * ms_.experts_used * ms_.hidden * 2);
        qstream_moe_ = true;
    }
    qstream_qkv_ = qkv_one;
    // the output projection of narrow batches (no scale, no soft cap: those stay on the other paths)
    DeviceWeight& head = ms_.tied ? token_embd_ : output_;
    if (kq(head) && ms_.final_logit_scale == 1.f && ms_.final_softcap == 0.f) retile(head.w, qs_head_);
    v_partial_.alloc((size_t)16 * kQStreamMaxRows * ms_.kv_heads * ms_.head_dim * 4);
    MK_CUDA(cudaStreamSynchronize(stream_));
    if (const char* e = std::getenv("MACLLM_B200_STREAM_MIN_ROWS")) qstream_min_rows_ = std::max(1, atoi(e));
    qstream_ = true;
}

int Model::matmul_stream(const QStreamWeight& W, const ActQ& x, int T, float* y, int ldy, int max_splits, const QStreamWeight* W2) {
    const double rows = (double)W.rows + (W2 ? (double)W2->rows : 0.0);
    const double wbytes = (double)W.rows * (double)(W.cols / 256) * (W.fmt ? 210.0 : 144.0) +
                          (W2 ? (double)W2->rows * (double)(W2->cols / 256) * (W2->fmt ? 210.0 : 144.0) : 0.0);
    prof_begin(KC_QSTREAM, wbytes + 2.0 * T * W.cols + 4.0 * T * rows, 2.0 * T * rows * (double)W.cols);
    int splits = launch_qstream_tc(W, x.xh, T, y, ldy, tc_ws_.partial.as<float>(), tc_ws_.partial.size() / 4,
                                   tc_ws_.status.as<int32_t>(), stream_, max_splits, W2);
    prof_end();
    ++launches_;
    return splits;
}

static int act_kind_of(const QWeight& w) { return w.type == QT_Q8_0 ? ACT_Q80 : ACT_Q8K; }

void Model::run_forward(const std::vector<LmLane>& lanes, KvReservation& r, uint32_t flags) {
    MK_CUDA(cudaSetDevice(cfg_.device));
    const int B = (int)lanes.size();
    int T = 0;
    for (const LmLane& l : lanes) T += l.n_tokens;
    if (B > cfg_.max_batch_lanes) throw std::runtime_error("batch has more lanes than max_batch_lanes");
    if (T > cfg_.max_batch_tokens) throw std::runtime_error("batch has more tokens than max_batch_tokens");
    const int H = ms_.hidden, AW = ms_.q_heads * ms_.head_dim, KW = ms_.kv_heads * ms_.head_dim, d = ms_.head_dim;
    const int QKVW = AW + 2 * KW;
    const int bt = pool_->block_tokens();
    const int q_tile = attention_q_tile(ms_.q_heads, ms_.kv_heads);

    // ---- stage the per-lane headers, block tables and token ids in one pinned buffer, one copy
    uint8_t* hp = stage_host_.as<uint8_t>();
    LaneHeader* hdr = reinterpret_cast<LaneHeader*>(hp);
    size_t off_tables = (size_t)B * sizeof(LaneHeader);
    uint32_t* tab = reinterpret_cast<uint32_t*>(hp + off_tables);
    int n_tab = 0, tiles = 0;
    for (int i = 0; i < B; ++i) {
        const std::vector<KvBlockId>& blocks = r.lane_blocks((size_t)i);
        hdr[i].start_pos = lanes[(size_t)i].start_pos;
        hdr[i].n_tokens = lanes[(size_t)i].n_tokens;
        hdr[i].table_off = n_tab;
        hdr[i].n_blocks = (int32_t)blocks.size();
        for (const KvBlockId& b : blocks) tab[n_tab++] = b.slot;
        tiles += (lanes[(size_t)i].n_tokens + q_tile - 1) / q_tile;
    }
    size_t off_ids = off_tables + (size_t)n_tab * 4;
    uint32_t* ids = reinterpret_cast<uint32_t*>(hp + off_ids);
    int tpos = 0;
    for (const LmLane& l : lanes) {
        memcpy(ids + tpos, l.ids, (size_t)l.n_tokens * 4);
        tpos += l.n_tokens;
    }
    size_t stage_bytes = off_ids + (size_t)T * 4;
    // per-lane sampling settings, only when some lane does not take the plain argmax
    bool any_stochastic = false;
    for (const LmLane& l : lanes) any_stochastic |= l.temperature > 0.f;
    size_t off_sampling = 0;
    if (any_stochastic && (flags & FWD_WANT_TOKENS)) {
        off_sampling = (stage_bytes + 15) / 16 * 16;
        LaneSampling* sp = reinterpret_cast<LaneSampling*>(hp + off_sampling);
        for (int i = 0; i < B; ++i) {
            const LmLane& l = lanes[(size_t)i];
            if (!mk::device_sampling_covers(l.temperature, l.top_k, ms_.vocab))
                throw std::runtime_error("the device sampler covers greedy selection and 1 <= top_k <= 1024");
            sp[i] = LaneSampling{l.temperature, l.top_k, l.top_p, l.u};
        }
        stage_bytes = off_sampling + (size_t)B * sizeof(LaneSampling);
    }
    // work lists of the tensor-core attention (the same for every layer of the tick)
    size_t off_tiles = 0, off_entries = 0, off_dec = 0;
    int n_attn_tiles = 0, n_attn_entries = 0, n_attn_dec = 0;
    if (attn_tc_) {
        plan_sp_.resize((size_t)B);
        plan_nt_.resize((size_t)B);
        plan_nb_.resize((size_t)B);
        for (int i = 0; i < B; ++i) {
            plan_sp_[(size_t)i] = lanes[(size_t)i].start_pos;
            plan_nt_[(size_t)i] = lanes[(size_t)i].n_tokens;
            plan_nb_[(size_t)i] = hdr[i].n_blocks;
        }
        plan_attention_tc(plan_sp_.data(), plan_nt_.data(), plan_nb_.data(), B, ms_.q_heads, ms_.kv_heads, attn_plan_);
        n_attn_tiles = attn_plan_.n_tiles();
        n_attn_entries = attn_plan_.n_entries();
        n_attn_dec = attn_plan_.n_dec_lanes();
        if (n_attn_entries > attn_max_entries_) throw std::runtime_error("attention work list exceeds its scratch");
        off_entries = (stage_bytes + 15) / 16 * 16;  // 32-byte records read as two 16-byte loads
        off_tiles = off_entries + attn_plan_.entries.size() * 4;
        off_dec = off_tiles + attn_plan_.tiles.size() * 4;
        stage_bytes = off_dec + attn_plan_.dec_lanes.size() * 4;
        if (stage_bytes > stage_host_.size()) throw std::runtime_error("tick staging buffer is too small");
        if (n_attn_tiles) memcpy(hp + off_tiles, attn_plan_.tiles.data(), attn_plan_.tiles.size() * 4);
        if (n_attn_entries) memcpy(hp + off_entries, attn_plan_.entries.data(), attn_plan_.entries.size() * 4);
        if (n_attn_dec) memcpy(hp + off_dec, attn_plan_.dec_lanes.data(), attn_plan_.dec_lanes.size() * 4);
    }
    if (stage_bytes > stage_dev_.size()) throw std::runtime_error("tick staging buffer is too small");
    MK_CUDA(cudaEventRecord(ev_start_, stream_));
    MK_CUDA(cudaMemcpyAsync(stage_dev_.ptr(), hp, stage_bytes, cudaMemcpyHostToDevice, stream_));
    h2d_bytes_ += (int64_t)stage_bytes;
    uint8_t* dp = stage_dev_.as<uint8_t>();

    BatchDesc bd;
    bd.lanes = B;
    bd.T = T;
    bd.max_tiles = tiles;
    bd.hdr = reinterpret_cast<const LaneHeader*>(dp);
    bd.tables = reinterpret_cast<const uint32_t*>(dp + off_tables);
    bd.cu_seqlens = cu_.as<int32_t>();
    bd.positions = pos_.as<int32_t>();
    bd.token_lane = tok_lane_.as<int32_t>();
    bd.slots = slots_.as<int64_t>();
    bd.last_index = last_.as<int32_t>();
    bd.tile_lane = tile_lane_.as<int32_t>();
    bd.tile_row0 = tile_row_.as<int32_t>();
    bd.n_tiles = ntiles_.as<int32_t>();
    bd.error_flag = err_.as<int32_t>();
    prof_begin(KC_BATCH, 0, 0);
        launch_build_batch(bd, bt, q_tile, stream_);
        prof_end();
    ++launches_;
    const uint32_t* ids_dev = reinterpret_cast<const uint32_t*>(dp + off_ids);

    // ---- copy-on-write page copies of shared partial tails (cache.rs:3042-3089)
    for (const KvCowCopy& c : r.cow_copies()) {
        launch_cow_copy(k_pool_.ptr(), v_pool_.ptr(), cfg_.kv_f16 ? 1 : 0, c.src_slot, c.dst_slot, c.rows, ms_.layers, pool_->max_blocks(), ms_.kv_heads, bt,
                        d, stream_);
        ++launches_;
    }

    // ---- embedding (src/decoder.rs:3194-3197)
    prof_begin(KC_EMBED, 4.0 * T * H, 0);
        launch_embed(token_embd_.w, ids_dev, T, ms_.embedding_scale, h_.as<float>(), stream_);
        prof_end();
    ++launches_;

    const bool f16_T = dense_matrices_ || (cfg_.matmul_path != 1 && (cfg_.matmul_path == 2 || T > 8 || (qstream_ && T >= qstream_min_rows_)));
    const float* pending = nullptr;        // branch output not yet added to the residual stream
    const float* pending_post = nullptr;   // its sandwich post-norm weight, if any
    int pending_splits = 1;                // > 1: `pending` is that many split-K partials, T * H floats apart
    const bool fuse_rope_enabled = [] { const char* e = getenv("MACLLM_B200_FUSE_ROPE"); return e == nullptr || strcmp(e, "0") != 0; }();
    for (int l = 0; l < ms_.layers; ++l) {
        LayerWeights& w = lw_[(size_t)l];
        const LayerSpec& ls = ms_.layer[(size_t)l];
        // residual add of the previous layer's FFN + attention norm + quantise
        int kind = act_kind_of(w.wq.w);
        const bool stream_T = qstream_ && T >= qstream_min_rows_ && T <= kQStreamMaxRows && f16_T;
        ActQ xa = act_view(a_qs_, a_d_, a_bs_, a_xh_, T, H, kind, f16_T);
        NormQuantArgs na;
        na.h = h_.as<float>();
        na.a = pending;
        na.a_splits = pending_splits;
        na.a_split_stride = (int64_t)T * H;
        na.post_w = pending_post;
        na.norm_w = w.attn_norm.as<float>();
        na.eps = ms_.eps;
        na.rows = T;
        na.dim = H;
        na.act_kind = kind;
        na.out = xa;
        prof_begin(KC_NORM_QUANT, 9.0 * T * H, 0);
        launch_add_norm_quant(na, stream_);
        prof_end();
        ++launches_;
        // projections (src/decoder.rs:1099-1161)
        float* qp = qkv_.as<float>();
        float* kp = qp + AW;
        float* vp = kp + KW;
        const bool stream = stream_T;
        const int kMaxShares = 16;
        int qk_splits = 1, v_splits = 1;
        bool qkv_joint = false;
        // Narrow ticks: which projections leave the streamed Q4_K matmul for the f16 images with split-K.  Measured on
        // 64-lane decode ticks of the 3 B shape: [q; k; v] as ONE launch over the stacked image beats the streamed
        // Q|K launch plus a separate V launch, and the long-K down projection is a little faster on its image; the
        // output projection and gate|up stay on the streamed blocks (a quarter of the bytes).  Bit 8 applies from 33 rows.
        // MACLLM_B200_DECODE_HALF_MASK overrides: 1 q|k|v, 2 attention output, 4 gate|up (implies 8), 8 down.
        static const int half_mask = [] {
            const char* e = getenv("MACLLM_B200_DECODE_HALF_MASK");
            int m = e != nullptr ? atoi(e) : 0;
            return (m & 4) ? (m | 8) : m;
        }();
        const bool stream_o = stream && !(half_mask & 2), stream_gu = stream && !(half_mask & 4), stream_down = stream && !((half_mask & 8) && T >= 33);  // with a handful of lanes the streamed blocks win (measured at 4 lanes)
        if (stream && (half_mask & 1) && w.qkv_half.ready) {
            qk_splits = v_splits = matmul_half(w.qkv_half, xa, T, qp, QKVW, 1.f, 0.f, kMaxShares);
            qkv_joint = qk_splits > 1;
        } else if (stream && qstream_qkv_) {
            // [wq; wk] in Q4_K and wv in its own format, one launch: the rows of q | k | v side by side
            qk_splits = v_splits = matmul_stream(w.qs_qk, xa, T, qp, QKVW, kMaxShares, &w.qs_v);
            qkv_joint = qk_splits > 1;
        } else if (stream) {
            qk_splits = matmul_stream(w.qs_qk, xa, T, qp, QKVW, kMaxShares);
            v_splits = matmul_half(w.wv.half, xa, T, vp, QKVW, 1.f, 0.f, kMaxShares, v_partial_.as<float>(), v_partial_.size() / 4);
        } else if (w.qkv_half.ready && T >= hgemm_min_rows_ && xa.xh != nullptr) {
            // a tick of a hundred rows has fewer output tiles than SMs: the plan may share K out, the consumer adds the shares
            qk_splits = v_splits = matmul_half(w.qkv_half, xa, T, qp, QKVW, 1.f, 0.f, kMaxShares);
            qkv_joint = qk_splits > 1;
        } else if (w.qk_raw.size() > 0) {
            // [wq; wk] share one buffer: one launch for both (their outputs are adjacent columns of the row)
            DeviceWeight qk;
            qk.w = w.wq.w;
            qk.w.rows = w.wq.w.rows + w.wk.w.rows;
            qk.w.bytes = w.wq.w.bytes + w.wk.w.bytes;
            matmul(qk, xa, T, qp, QKVW, 1.f, 0.f);
            matmul(w.wv, xa, T, vp, QKVW, 1.f, 0.f);
        } else {
            matmul(w.wq, xa, T, qp, QKVW, 1.f, 0.f);
            matmul(w.wk, xa, T, kp, QKVW, 1.f, 0.f);
            matmul(w.wv, xa, T, vp, QKVW, 1.f, 0.f);
        }
        // per-head norms, rotation, paged write
        RopeKvArgs ra;
        ra.q = qp;
        ra.k = kp;
        ra.v = vp;
        ra.ldq = ra.ldk = ra.ldv = QKVW;
        if (qkv_joint) {
            // shares of whole [q | k | v] rows in the split-K scratch
            ra.q = tc_ws_.partial.as<float>();
            ra.k = ra.q + AW;
            ra.v = ra.k + KW;
            ra.qk_splits = ra.v_splits = qk_splits;
            ra.qk_split_stride = ra.v_split_stride = (int64_t)T * QKVW;
            ra.q_out = qp;
            ra.ldq_out = QKVW;
        } else if (qk_splits > 1) {
            // shares of [q | k] rows of width AW + KW in the split-K scratch; the rotated q goes to its usual place
            ra.q = tc_ws_.partial.as<float>();
            ra.k = ra.q + AW;
            ra.ldq = ra.ldk = AW + KW;
            ra.qk_splits = qk_splits;
            ra.qk_split_stride = (int64_t)T * (AW + KW);
            ra.q_out = qp;
            ra.ldq_out = QKVW;
        }
        if (!qkv_joint && v_splits > 1) {
            ra.v = v_partial_.as<float>();
            ra.ldv = KW;
            ra.v_splits = v_splits;
            ra.v_split_stride = (int64_t)T * KW;
        }
        if (ls.qk_norm) { ra.q_norm_w = w.q_norm.as<float>(); ra.k_norm_w = w.k_norm.as<float>(); }
        ra.norm_eps = ms_.eps;
        if (ls.rope) { rope_tables_for(ls.theta, ra.cos_t, ra.sin_t); ra.rotary_dim = ms_.rotary_dim; }
        ra.positions = bd.positions;
        ra.slots = bd.slots;
        ra.k_pool = k_pool_.ptr();
        ra.v_pool = v_pool_.ptr();
        ra.kv_f16 = cfg_.kv_f16 ? 1 : 0;
        ra.T = T;
        ra.q_heads = ms_.q_heads;
        ra.kv_heads = ms_.kv_heads;
        ra.d = d;
        ra.block_tokens = bt;
        ra.layers = ms_.layers;
        ra.pool_blocks = pool_->max_blocks();
        ra.layer = l;
        // ticks of one-token lanes only: the attention kernel prepares its own query rows and writes the new K / V rows
        // itself (same arithmetic, see rope_head.cuh), so the separate launch is dropped.  MACLLM_B200_FUSE_ROPE=0 keeps it.
        const bool fuse_rope = attn_tc_ && cfg_.kv_f16 && n_attn_tiles == 0 && n_attn_entries > 0 && n_attn_dec == 0 && fuse_rope_enabled;
        if (!fuse_rope) {
            prof_begin(KC_ROPE_KV, 4.0 * T * (2 * AW + 2 * KW) + (cfg_.kv_f16 ? 2.0 : 4.0) * 2 * T * KW, 0);
            launch_rope_kv(ra, stream_);
            prof_end();
            ++launches_;
        }
        // the quantised image of the attention output feeds the output projection; on a tick of one-token lanes only,
        // the attention kernel writes it itself
        const int okind = act_kind_of(w.wo.w);
        ActQ xo = act_view(a_qs_, a_d_, a_bs_, a_xh_, T, AW, okind, f16_T);
        const bool fuse_attn_quant = attn_tc_ && n_attn_tiles == 0 && n_attn_entries > 0 && (AW / ms_.kv_heads) % 256 == 0;
        // wide ticks: the output projection is an f16 GEMM that reads nothing but the f16 rows, so the attention kernels
        // write those and the separate quantisation pass is dropped
        const bool attn_half_out = attn_tc_ && !fuse_attn_quant && !stream_o && w.wo.half.ready &&
                                   T >= hgemm_min_rows_ && xo.xh != nullptr && n_attn_dec == 0;
        AttnArgs at;
        at.q = qp;
        at.ldq = QKVW;
        at.out = attn_.as<float>();
        at.k_pool = k_pool_.ptr();
        at.v_pool = v_pool_.ptr();
        at.kv_f16 = ra.kv_f16;
        at.batch = bd;
        at.q_heads = ms_.q_heads;
        at.kv_heads = ms_.kv_heads;
        at.d = d;
        at.block_tokens = bt;
        at.layers = ms_.layers;
        at.pool_blocks = pool_->max_blocks();
        at.layer = l;
        at.scale = ls.scale;
        at.softcap = ls.softcap;
        at.window = ls.window;
        at.q_tile = q_tile;
        {
            // algorithmic traffic: each lane's visible K/V history once, plus queries and outputs
            double kv_tokens = 0;
            for (const LmLane& ln : lanes) {
                double ctx = (double)ln.start_pos + ln.n_tokens;
                kv_tokens += ls.window > 0 ? std::min<double>(ctx, (double)ls.window + ln.n_tokens) : ctx;
            }
            double esz = cfg_.kv_f16 ? 2.0 : 4.0;
            double flops = 0;
            for (const LmLane& ln : lanes) flops += 4.0 * ms_.q_heads * d * ((double)ln.n_tokens * ln.start_pos + 0.5 * ln.n_tokens * ln.n_tokens);
            prof_begin(KC_ATTN, kv_tokens * 2 * KW * esz + 8.0 * T * AW, flops);
        }
        if (attn_tc_) {
            AttnTcArgs ta;
            ta.q = at.q;
            ta.ldq = at.ldq;
            ta.out = at.out;
            ta.k_pool = at.k_pool;
            ta.v_pool = at.v_pool;
            ta.hdr = bd.hdr;
            ta.tables = bd.tables;
            ta.cu_seqlens = bd.cu_seqlens;
            ta.tiles = reinterpret_cast<const int32_t*>(dp + off_tiles);
            ta.entries = reinterpret_cast<const int32_t*>(dp + off_entries);
            ta.dec_lanes = reinterpret_cast<const int32_t*>(dp + off_dec);
            ta.n_tiles = n_attn_tiles;
            ta.n_entries = n_attn_entries;
            ta.n_dec_lanes = n_attn_dec;
            ta.part_o = attn_part_o_.as<float>();
            ta.part_ml = attn_part_ml_.as<float>();
            ta.counters = attn_counters_.as<int32_t>();
            ta.q_heads = ms_.q_heads;
            ta.kv_heads = ms_.kv_heads;
            ta.d = d;
            ta.block_tokens = bt;
            ta.layers = ms_.layers;
            ta.pool_blocks = at.pool_blocks;
            ta.layer = l;
            ta.scale = ls.scale;
            ta.softcap = ls.softcap;
            ta.window = ls.window;
            if (fuse_rope) {
                ta.fused_rope = 1;
                ta.rk = ra;
            }
            if (fuse_attn_quant) {
                ta.qout = xo;
                ta.qkind = okind;
                ta.out = nullptr;  // nothing reads the f32 rows of a pure decode tick
            } else if (attn_half_out) {
                ta.out_h = xo.xh;
                ta.out = nullptr;
            }
            launches_ += launch_paged_attention_tc(ta, stream_);
        } else {
            launch_paged_attention(at, stream_);
            ++launches_;
        }
        prof_end();
        // output projection
        if (!fuse_attn_quant && !attn_half_out) {
            NormQuantArgs no;
            no.h = attn_.as<float>();
            no.rows = T;
            no.dim = AW;
            no.act_kind = okind;
            no.out = xo;
            prof_begin(KC_NORM_QUANT, 5.0 * T * AW, 0);
            launch_add_norm_quant(no, stream_);
            prof_end();
            ++launches_;
        }
        // split-K shares of the two long-K projections are summed by the residual kernel that consumes them
        int wo_splits = 1;
        if (stream_o) wo_splits = matmul_stream(w.qs_o, xo, T, proj_.as<float>(), H, kMaxShares);
        else if (w.wo.half.ready && T >= hgemm_min_rows_ && xo.xh != nullptr) wo_splits = matmul_half(w.wo.half, xo, T, proj_.as<float>(), H, 1.f, 0.f, kMaxShares);
        else matmul(w.wo, xo, T, proj_.as<float>(), H, 1.f, 0.f);
        // residual add + FFN norm + quantise (finish_mixer, src/decoder.rs:2684-2699)
        int fkind = act_kind_of(w.gate.w);
        const bool ep_dp = cfg_.ep_size > 1 && cfg_.ep_mode == 1 && ls.moe;  // the exchange moves f16 rows at every width
        ActQ xf = act_view(a_qs_, a_d_, a_bs_, a_xh_, T, H, fkind, f16_T || ep_dp);
        NormQuantArgs nf;
        nf.h = h_.as<float>();
        nf.a = wo_splits > 1 ? tc_ws_.partial.as<float>() : proj_.as<float>();
        nf.a_splits = wo_splits;
        nf.a_split_stride = (int64_t)T * H;
        nf.post_w = ls.sandwich ? w.post_attn_norm.as<float>() : nullptr;
        nf.norm_w = w.ffn_norm.as<float>();
        nf.eps = ms_.eps;
        nf.rows = T;
        nf.dim = H;
        nf.act_kind = fkind;
        nf.out = xf;
        nf.normed_out = ls.moe ? normed_.as<float>() : nullptr;
        prof_begin(KC_NORM_QUANT, 13.0 * T * H, 0);
        launch_add_norm_quant(nf, stream_);
        prof_end();
        ++launches_;
        if (!ls.moe) {
            // dense feed-forward (src/decoder.rs:298-305)
            float* gp = gu_.as<float>();
            float* up = gp + ms_.ffn;
            int gu_splits = 1;
            // wide ticks: one GEMM over the interleaved gate/up image writes act(gate) * up as f16, which is all the
            // f16 GEMM of the down projection reads; no f32 gate|up round trip and no separate activation kernel
            const bool gated_gemm = !stream_gu && w.gu_half.ready && w.down.half.ready && T >= hgemm_min_rows_ && xf.xh != nullptr && f16_T;
            // narrow ticks, gated form: act(gate) * up leaves the streamed matmul as f16, which is what the streamed down
            // projection reads (the activation is the f16 rounding of the f32 value, not an 8-bit block image)
            const bool gated_stream = stream_gu && qstream_gated_ && stream_down;
            if (gated_stream) {
                const QStreamWeight& W = w.qs_gu;
                prof_begin(KC_QSTREAM, (double)W.rows * (double)(W.cols / 256) * 144.0 + 2.0 * T * W.cols + 2.0 * T * ms_.ffn,
                           2.0 * T * (double)W.rows * (double)W.cols);
                launch_qstream_tc(W, xf.xh, T, nullptr, 0, nullptr, 0, tc_ws_.status.as<int32_t>(), stream_, 1, nullptr, ls.act,
                                  f_xh_.as<__half>(), ms_.ffn);
                prof_end();
                ++launches_;
            } else if (gated_gemm) {
                prof_begin(KC_HGEMM, 2.0 * (double)w.gu_half.rows * (double)w.gu_half.cols + 2.0 * T * H + 2.0 * T * ms_.ffn,
                           2.0 * T * (double)w.gu_half.rows * (double)w.gu_half.cols);
                launch_hgemm_tc_gated(w.gu_half, xf.xh, T, ls.act, f_xh_.as<__half>(), ms_.ffn, hgemm_scratch(), stream_);
                prof_end();
                ++launches_;
            } else if (stream_gu) {
                if (qstream_gated_) throw std::runtime_error("the interleaved gate|up copy serves the gated form only");
                gu_splits = matmul_stream(w.qs_gu, xf, T, gp, 2 * ms_.ffn, kMaxShares);
            } else if (w.gu_raw.size() > 0) {
                DeviceWeight gu;  // [gate; up] share one buffer: one launch for both
                gu.w = w.gate.w;
                gu.w.rows = w.gate.w.rows + w.up.w.rows;
                gu.w.bytes = w.gate.w.bytes + w.up.w.bytes;
                matmul(gu, xf, T, gp, 2 * ms_.ffn, 1.f, 0.f);
            } else {
                matmul(w.gate, xf, T, gp, 2 * ms_.ffn, 1.f, 0.f);
                matmul(w.up, xf, T, up, 2 * ms_.ffn, 1.f, 0.f);
            }
            int dkind = act_kind_of(w.down.w);
            ActQ xd = act_view(f_qs_, f_d_, f_bs_, f_xh_, T, ms_.ffn, dkind, f16_T);
            if (!gated_gemm && !gated_stream) {
                prof_begin(KC_ACTMUL, 9.0 * T * ms_.ffn, 0);
                if (gu_splits > 1) {
                    const float* pg = tc_ws_.partial.as<float>();
                    launch_actmul_quant(pg, pg + ms_.ffn, 2 * ms_.ffn, T, ms_.ffn, ls.act, dkind, xd, nullptr, stream_, gu_splits,
                                        (int64_t)T * 2 * ms_.ffn);
                } else {
                    launch_actmul_quant(gp, up, 2 * ms_.ffn, T, ms_.ffn, ls.act, dkind, xd, nullptr, stream_);
                }
                prof_end();
                ++launches_;
            }
            if (stream_down) pending_splits = matmul_stream(w.qs_down, xd, T, down_.as<float>(), H, kMaxShares);
            else if (w.down.half.ready && T >= hgemm_min_rows_ && xd.xh != nullptr) pending_splits = matmul_half(w.down.half, xd, T, down_.as<float>(), H, 1.f, 0.f, kMaxShares);
            else { matmul(w.down, xd, T, down_.as<float>(), H, 1.f, 0.f); pending_splits = 1; }
        } else {
            // sparse MoE (src/decoder.rs:394-554)
            const int E = ms_.experts, K = ms_.experts_used, F = ms_.expert_ffn, P = T * K;
            prof_begin(KC_MOE, 4.0 * E * H + 4.0 * T * H + 4.0 * T * E, 2.0 * T * E * H);
            launch_f32_gemv(w.router.as<float>(), E, H, normed_.as<float>(), T, router_logits_.as<float>(), stream_);
            prof_end();
            prof_begin(KC_MOE, 4.0 * T * E + 8.0 * P, 0);
            launch_moe_route(router_logits_.as<float>(), T, E, K, sel_e_.as<int32_t>(), sel_w_.as<float>(), tc_ws_.status.as<int32_t>(), stream_);
            prof_end();
            prof_begin(KC_MOE, 12.0 * P, 0);
            launch_moe_group(sel_e_.as<int32_t>(), T, K, E, grp_off_.as<int32_t>(), pos_of_pair_.as<int32_t>(), tok_of_pos_.as<int32_t>(),
                             stream_);
            prof_end();
            ActQ xq = xf;
            xq.xh = nullptr;
            const bool moe_stream = qstream_moe_ && xf.xh != nullptr && (ep_dp || (f16_T && T >= qstream_min_rows_));
            // expert parallelism: only the experts [e0, e0 + EL) live here; their rows of the grouped layout are
            // computed and combined into a partial sum, and the partials of all ranks are added in rank order
            const bool ep = cfg_.ep_size > 1;
            if (ep && !ep_) throw std::runtime_error("expert-parallel model used before mk_model_ep_init");
            const int e0 = ep_first_expert(), EL = ep_local_experts();
            const int32_t* off = grp_off_.as<int32_t>() + e0;
            if (ep_dp) {
                if (!ep_->has_dispatch() || !moe_stream) throw std::runtime_error("data-parallel expert parallelism: the dispatch exchange is not open");
                prof_begin(KC_MOE, 4.0 * P * H, 0);
                launch_gather_rows_half(xf.xh, tok_of_pos_.as<int32_t>(), P, H, e_xh_.as<__half>(), stream_);
                prof_end();
                const float* back = ep_exchange_layer(w, ls, e_xh_.as<__half>(), grp_off_.as<int32_t>(), T);
                launch_moe_combine(back, sel_e_.as<int32_t>(), sel_w_.as<float>(), pos_of_pair_.as<int32_t>(), T, K, H, 0, E, down_.as<float>(),
                                   stream_);
            } else if (moe_stream) {
                // the routed rows grouped by expert as f16, then the expert-grouped tensor-core matmuls: gate|up with the
                // activation in its epilogue (f16 out), down on those rows.  Every expert's weights are read once per 64
                // of its rows; the row ranges stay on the device.
                prof_begin(KC_MOE, 4.0 * P * H, 0);
                launch_gather_rows_half(xf.xh, tok_of_pos_.as<int32_t>(), P, H, e_xh_.as<__half>(), stream_);
                prof_end();
                const double gu_bytes = (double)w.qs_gu.rows * (double)(w.qs_gu.cols / 256) * 144.0;
                prof_begin(KC_QSTREAM, gu_bytes + 2.0 * P * H + 2.0 * P * F, 2.0 * P * 2.0 * F * H);
                launch_qstream_tc_grouped(w.qs_gu, EL, off, e_xh_.as<__half>(), P, moe_chunk_rows(T, K, E), nullptr, 0, tc_ws_.status.as<int32_t>(), stream_,
                                          ls.act, f_xh_.as<__half>(), F);
                prof_end();
                const double dn_bytes = (double)w.qs_down.rows * (double)(w.qs_down.cols / 256) * (w.qs_down.fmt ? 210.0 : 144.0);
                prof_begin(KC_QSTREAM, dn_bytes + 2.0 * P * F + 4.0 * P * H, 2.0 * P * (double)F * H);
                launch_qstream_tc_grouped(w.qs_down, EL, off, f_xh_.as<__half>(), P, moe_chunk_rows(T, K, E), e_down_.as<float>(), H,
                                          tc_ws_.status.as<int32_t>(), stream_);
                prof_end();
            } else {
                launch_qgemv_grouped(w.gate.w, EL, off, tok_of_pos_.as<int32_t>(), xq, e_gate_.as<float>(), F, stream_);
                launch_qgemv_grouped(w.up.w, EL, off, tok_of_pos_.as<int32_t>(), xq, e_up_.as<float>(), F, stream_);
                int dkind = act_kind_of(w.down.w);
                ActQ xd = act_view(f_qs_, f_d_, f_bs_, f_xh_, P, F, dkind, false);
                launch_actmul_quant(e_gate_.as<float>(), e_up_.as<float>(), F, P, F, ls.act, dkind, xd, nullptr, stream_);
                launch_qgemv_grouped(w.down.w, EL, off, nullptr, xd, e_down_.as<float>(), H, stream_);
            }
            // replicated lanes (or one GPU): this rank's expert outputs are combined here, the partial sums exchanged
            if (ep_dp) {
                // combined above from the result area of the exchange
            } else if (ep && ep_->has_exchange()) {
                launch_moe_combine_exchange(e_down_.as<float>(), sel_e_.as<int32_t>(), sel_w_.as<float>(), pos_of_pair_.as<int32_t>(), T, K,
                                            H, e0, e0 + EL, ep_->peers(), ep_->next_epoch(), down_.as<float>(),
                                            tc_ws_.status.as<int32_t>(), stream_);
            } else {
                prof_begin(KC_MOE, 4.0 * P * H + 4.0 * T * H, 2.0 * P * H);
                launch_moe_combine(e_down_.as<float>(), sel_e_.as<int32_t>(), sel_w_.as<float>(), pos_of_pair_.as<int32_t>(), T, K, H,
                                   e0, e0 + EL, ep ? ep_partial_.as<float>() : down_.as<float>(), stream_);
                prof_end();
            }
            if (!ep_dp && ep && !ep_->has_exchange()) {
                ep_->all_gather_f32(ep_partial_.as<float>(), ep_gather_.as<float>(), (size_t)T * H, stream_);
                launch_ep_sum(ep_gather_.as<float>(), cfg_.ep_size, (int64_t)T * H, down_.as<float>(), stream_);
                launches_ += 2;
            }
            launches_ += 8;
        }
        if (ls.moe) pending_splits = 1;
        pending = pending_splits > 1 ? tc_ws_.partial.as<float>() : down_.as<float>();
        pending_post = ls.sandwich ? w.post_ffn_norm.as<float>() : nullptr;
    }
    // last residual add
    {
        NormQuantArgs nl;
        nl.h = h_.as<float>();
        nl.a = pending;
        nl.a_splits = pending_splits;
        nl.a_split_stride = (int64_t)T * H;
        nl.post_w = pending_post;
        nl.eps = ms_.eps;
        nl.rows = T;
        nl.dim = H;
        prof_begin(KC_NORM_QUANT, 12.0 * T * H, 0);
        launch_add_norm_quant(nl, stream_);
        prof_end();
        ++launches_;
    }
    // logits tail (src/decoder.rs:3333-3356): last rows -> final norm -> output projection -> scale -> softcap
    const DeviceWeight& head_dw = ms_.tied ? token_embd_ : output_;
    const QWeight& head = head_dw.w;
    {
        const bool f16_B = dense_matrices_ || (cfg_.matmul_path != 1 && (cfg_.matmul_path == 2 || B > 8));
        int kind = act_kind_of(head);
        ActQ xl = act_view(l_qs_, l_d_, l_bs_, l_xh_, B, H, kind, f16_B);
        NormQuantArgs ng;
        ng.h = h_.as<float>();
        ng.norm_w = output_norm_.as<float>();
        ng.eps = ms_.eps;
        ng.rows = B;
        ng.dim = H;
        ng.row_index = bd.last_index;
        ng.act_kind = kind;
        ng.out = xl;
        prof_begin(KC_NORM_QUANT, 5.0 * B * H, 0);
        launch_add_norm_quant(ng, stream_);
        prof_end();
        ++launches_;
        if (qs_head_.ready && f16_B && B >= qstream_min_rows_ && B <= kQStreamMaxRows && xl.xh != nullptr)
            matmul_stream(qs_head_, xl, B, logits_.as<float>(), ms_.vocab, 1);
        else
            matmul(head_dw, xl, B, logits_.as<float>(), ms_.vocab, ms_.final_logit_scale, ms_.final_softcap);
    }
    if (flags & FWD_WANT_TOKENS) {
        prof_begin(KC_SAMPLE, 4.0 * B * ms_.vocab, 0);
        if (off_sampling != 0)
            launch_sample(logits_.as<float>(), B, ms_.vocab, reinterpret_cast<const LaneSampling*>(dp + off_sampling), tokens_.as<uint32_t>(),
                          tc_ws_.status.as<int32_t>(), stream_);
        else
            launch_argmax(logits_.as<float>(), B, ms_.vocab, tokens_.as<uint32_t>(), argmax_scratch_.ptr(), stream_);
        prof_end();
        ++launches_;
    }
    // results travel to pinned host memory on the same stream; the barrier is in fetch_output
    uint8_t* oh = out_host_.as<uint8_t>();
    size_t tok_off = (size_t)B * ms_.vocab * 4;
    if (flags & FWD_WANT_LOGITS) MK_CUDA(cudaMemcpyAsync(oh, logits_.ptr(), tok_off, cudaMemcpyDeviceToHost, stream_));
    if (flags & FWD_WANT_TOKENS) MK_CUDA(cudaMemcpyAsync(oh + tok_off, tokens_.ptr(), (size_t)B * 4, cudaMemcpyDeviceToHost, stream_));
    MK_CUDA(cudaMemcpyAsync(oh + tok_off + (size_t)B * 4, err_.ptr(), 4, cudaMemcpyDeviceToHost, stream_));
    MK_CUDA(cudaMemcpyAsync(oh + tok_off + (size_t)B * 4 + 4, tc_ws_.status.ptr(), 4, cudaMemcpyDeviceToHost, stream_));
    d2h_bytes_ += 8 + ((flags & FWD_WANT_LOGITS) ? (int64_t)tok_off : 0) + ((flags & FWD_WANT_TOKENS) ? (int64_t)B * 4 : 0);
    MK_CUDA(cudaEventRecord(ev_stop_, stream_));
    timed_ = true;
    out_lanes_ = B;
    out_flags_ = flags;
}

void Model::fetch_output(float* logits, uint32_t* tokens) {
    MK_CUDA(cudaStreamSynchronize(stream_));
    if (profiling_) prof_resolve();
    const int B = out_lanes_;
    uint8_t* oh = out_host_.as<uint8_t>();
    size_t tok_off = (size_t)B * ms_.vocab * 4;
    int32_t flags[2];
    memcpy(flags, oh + tok_off + (size_t)B * 4, 8);
    if (flags[0] != 0) throw std::runtime_error("batch descriptor index out of range on the device (flag " + std::to_string(flags[0]) + ")");
    if (flags[1] != 0) {
        // the status word is sticky on the device: clear it so that the next forward starts clean
        cudaMemsetAsync(tc_ws_.status.ptr(), 0, 4, stream_);
        if ((flags[1] & 0xFFFF0000) == kSampleEmptyStatus)
            throw std::runtime_error("sampling distribution is empty (lane " + std::to_string(flags[1] & 0xFFFF) + ")");  // src/sampling.rs:352-355
        if ((flags[1] & 0xFFFF0000) == kMoeRouteStatus)
            throw std::runtime_error("router produced non-finite logits for token row " + std::to_string(flags[1] & 0xFFFF));  // src/decoder.rs:474-483
        throw std::runtime_error("a bounded wait inside a kernel gave up (tensor-core matmul pipeline or expert exchange; status " + std::to_string(flags[1]) + ")");
    }
    if (logits) {
        if (!(out_flags_ & FWD_WANT_LOGITS)) throw std::runtime_error("logits were not requested for this forward");
        memcpy(logits, oh, tok_off);
    }
    if (tokens) {
        if (!(out_flags_ & FWD_WANT_TOKENS)) throw std::runtime_error("tokens were not requested for this forward");
        memcpy(tokens, oh + tok_off, (size_t)B * 4);
    }
}

void Model::device_synchronize() { MK_CUDA(cudaStreamSynchronize(stream_)); }

float Model::last_forward_ms() const {
    if (!timed_) return 0.f;
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, ev_start_, ev_stop_) != cudaSuccess) {
        cudaGetLastError();
        return 0.f;
    }
    return ms;
}

}  // namespace mk
