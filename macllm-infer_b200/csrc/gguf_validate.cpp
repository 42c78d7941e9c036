// Host-only audit of a GGUF checkpoint against the family spec read from its metadata: every tensor the forward
// pass will upload must be present with the expected shape and a block format the kernels read, and tensors that
// belong to a layer kind this path does not run must be absent.  Follows the rules of the reference's loader
// (validate_decoder_tensors / validate_decoder_layer_tensors, src/gguf_model.rs:3388-3776; expect_shape :3778-3788),
// restricted to the five families of this path; projection and MLP biases, which the reference accepts for other
// families, are refused here instead of being ignored.
#include "model.h"

#include <sstream>

namespace mk {

namespace {

std::string shape_text(const std::vector<int64_t>& dims) {
    std::ostringstream o;
    o << "[";
    for (size_t i = 0; i < dims.size(); ++i) o << (i ? ", " : "") << dims[i];
    o << "]";
    return o.str();
}

const GgufTensor& expect_shape(const GgufFile& f, const std::string& name, const std::vector<int64_t>& expected) {
    const GgufTensor* t = f.tensor(name);
    if (t == nullptr) throw std::runtime_error("required GGUF tensor `" + name + "` is missing");
    if (t->dims != expected)
        throw std::runtime_error("GGUF tensor `" + name + "` has shape " + shape_text(t->dims) + ", expected " + shape_text(expected));
    return *t;
}

void expect_f32(const GgufTensor& t) {
    if (t.type != QT_F32) throw std::runtime_error("GGUF tensor `" + t.name + "` must be F32 (norm and router weights are not quantised)");
}

// Matrices: Q4_K / Q6_K / Q8_0 go through the quantised kernels; the other block formats of the reference's loader
// (src/gguf.rs:283-345) are decoded at load.  K-quants need rows of whole 256-blocks, the others of whole 32-blocks.
void expect_matrix_type(const GgufTensor& t) {
    const int64_t cols = t.dims.back();
    switch (t.type) {
        case QT_F32:
        case QT_F16:
        case QT_BF16: return;
        case QT_Q8_0:
        case QT_Q4_0:
        case QT_Q5_0:
        case QT_Q5_1:
            if (cols % 32 != 0) throw std::runtime_error("GGUF tensor `" + t.name + "`: rows of 32-weight blocks must be a multiple of 32 wide");
            return;
        case QT_Q4_K:
        case QT_Q6_K:
        case QT_Q2_K:
        case QT_Q3_K:
        case QT_Q5_K:
            if (cols % 256 != 0) throw std::runtime_error("GGUF tensor `" + t.name + "`: K-quant rows must be a multiple of 256 wide");
            return;
        default:
            // the wording of GgmlType::from_tag (src/gguf.rs:345-349)
            throw std::runtime_error("GGUF tensor `" + t.name + "`: unsupported GGML tensor type " + std::to_string(t.type) +
                                     "; this runtime currently supports F32 (0), F16 (1), Q4_0 (2), Q5_0 (6), Q5_1 (7), Q8_0 (8), Q2_K (10), "
                                     "Q3_K (11), Q4_K (12), Q5_K (13), Q6_K (14), and BF16 (30)");
    }
}

void expect_absent(const GgufFile& f, const std::string& prefix, std::initializer_list<const char*> suffixes, const std::string& why) {
    for (const char* s : suffixes)
        if (f.tensor(prefix + s) != nullptr) throw std::runtime_error(why + " `" + s + "`");
}

}  // namespace

GgufAudit validate_decoder_tensors(const GgufFile& f, const ModelSpec& s) {
    GgufAudit audit;
    auto matrix = [&](const std::string& name, const std::vector<int64_t>& shape) {
        const GgufTensor& t = expect_shape(f, name, shape);
        expect_matrix_type(t);
        // expert banks are read in place by the expert-grouped kernels; the formats decoded at load have no grouped form
        if (shape.size() == 3 && t.type != QT_Q4_K && t.type != QT_Q6_K && t.type != QT_Q8_0)
            throw std::runtime_error("GGUF tensor `" + t.name + "`: expert banks must be Q4_K, Q6_K or Q8_0 (GGML type " + std::to_string(t.type) +
                                     " has no expert-grouped kernel)");
        ++audit.matrices;
        audit.matrix_bytes += gguf_row_bytes(t.type, t.dims.back()) * (t.elements() / t.dims.back());
    };
    auto vector_f32 = [&](const std::string& name, const std::vector<int64_t>& shape) {
        expect_f32(expect_shape(f, name, shape));
        ++audit.vectors;
    };
    if (s.layers <= 0 || s.hidden <= 0 || s.q_heads <= 0 || s.kv_heads <= 0 || s.head_dim <= 0 || s.vocab <= 0)
        throw std::runtime_error("GGUF model spec has a non-positive dimension");
    if (s.q_heads % s.kv_heads != 0) throw std::runtime_error("query heads must be a multiple of KV heads");
    if (s.experts > 0 && (s.experts_used <= 0 || s.experts_used > s.experts || s.expert_ffn <= 0))
        throw std::runtime_error("sparse-MoE spec is inconsistent (expert_used_count / expert_feed_forward_length)");
    if (s.experts == 0 && s.ffn <= 0) throw std::runtime_error("GGUF metadata key `" + s.arch + ".feed_forward_length` is missing");

    const int64_t H = s.hidden, AW = (int64_t)s.q_heads * s.head_dim, KW = (int64_t)s.kv_heads * s.head_dim;
    matrix("token_embd.weight", {s.vocab, H});
    vector_f32("output_norm.weight", {H});
    if (!s.tied) matrix("output.weight", {s.vocab, H});
    for (int l = 0; l < s.layers; ++l) {
        const LayerSpec& ls = s.layer[(size_t)l];
        const std::string p = "blk." + std::to_string(l) + ".";
        const std::string where = "layer " + std::to_string(l);
        vector_f32(p + "attn_norm.weight", {H});
        vector_f32(p + "ffn_norm.weight", {H});
        if (ls.sandwich) {
            vector_f32(p + "post_attention_norm.weight", {H});
            vector_f32(p + "post_ffw_norm.weight", {H});
        }
        if (ls.qk_norm) {
            vector_f32(p + "attn_q_norm.weight", {s.head_dim});
            vector_f32(p + "attn_k_norm.weight", {s.head_dim});
        }
        matrix(p + "attn_q.weight", {AW, H});
        matrix(p + "attn_k.weight", {KW, H});
        matrix(p + "attn_v.weight", {KW, H});
        matrix(p + "attn_output.weight", {H, AW});
        expect_absent(f, p,
                      {"shortconv.conv.weight", "shortconv.in_proj.weight", "shortconv.out_proj.weight", "attn_qkv.weight", "attn_gate.weight",
                       "ssm_conv1d.weight", "ssm_dt.bias", "ssm_a", "ssm_beta.weight", "ssm_alpha.weight", "ssm_norm.weight", "ssm_out.weight"},
                      "attention " + where + " contains a tensor of another sequence mixer:");
        expect_absent(f, p, {"attn_q.bias", "attn_k.bias", "attn_v.bias", "attn_output.bias", "ffn_gate.bias", "ffn_up.bias", "ffn_down.bias"},
                      where + " carries a bias tensor, which this path does not apply:");
        if (!ls.moe) {
            matrix(p + "ffn_gate.weight", {s.ffn, H});
            matrix(p + "ffn_up.weight", {s.ffn, H});
            matrix(p + "ffn_down.weight", {H, s.ffn});
            expect_absent(f, p, {"ffn_gate_inp.weight", "ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight"},
                          "dense " + where + " contains incompatible sparse-MoE tensor");
        } else {
            vector_f32(p + "ffn_gate_inp.weight", {s.experts, H});
            matrix(p + "ffn_gate_exps.weight", {s.experts, s.expert_ffn, H});
            matrix(p + "ffn_up_exps.weight", {s.experts, s.expert_ffn, H});
            matrix(p + "ffn_down_exps.weight", {s.experts, H, s.expert_ffn});
            expect_absent(f, p, {"ffn_gate.weight", "ffn_up.weight", "ffn_down.weight"},
                          "sparse-MoE " + where + " contains unsupported dense tensor");
        }
    }
    // quantised payloads are only defined for quantisation version 2 (validate_quantization_metadata, src/gguf.rs:1019-1037)
    bool quantised = false;
    for (const GgufTensor& t : f.tensors()) quantised |= (t.type != QT_F32 && t.type != QT_F16 && t.type != QT_BF16);
    if (quantised) {
        if (!f.has("general.quantization_version")) throw std::runtime_error("quantized GGUF tensors require general.quantization_version");
        const int64_t v = f.get_int("general.quantization_version");
        if (v != 2) throw std::runtime_error("unsupported GGUF quantization version " + std::to_string(v) + "; expected version 2");
    }
    audit.tensors_in_file = (int64_t)f.tensors().size();
    return audit;
}

}  // namespace mk
