// C ABI, part 2: model / session / reservation / engine handles and the host-only KV pool and
// prefix-cache handles.
#include "../../include/macllm_b200.h"
#include "c_api_util.h"
#include "engine.h"
#include "model.h"
#include "prefix_cache.h"
#include <cstring>

using namespace mk;

struct mk_model {
    std::unique_ptr<PagedLm> lm;
    std::vector<mk_lane_sampling> sampling;  // settings of the next forward (mk_forward_set_sampling)
};
struct mk_session { std::unique_ptr<LmSession> s; };
struct mk_reservation { std::unique_ptr<LmReservation> r; };
struct mk_engine { std::unique_ptr<Engine> e; };
struct mk_kvpool { std::shared_ptr<KvPool> p; };
struct mk_kvtable { std::unique_ptr<KvTable> t; };
struct mk_prefix_cache { std::unique_ptr<TokenPrefixCache<int64_t>> c; };

namespace {

template <typename F>
int32_t guarded_kv(F&& f) {
    try {
        f();
        return 0;
    } catch (const KvPoolExhausted& e) {
        last_error_slot() = e.what();
        return MK_KV_EXHAUSTED;
    } catch (const std::exception& e) {
        last_error_slot() = e.what();
        return -1;
    } catch (...) {
        last_error_slot() = "unknown error";
        return -1;
    }
}

void fill_pool_stats(const KvPoolStats& s, mk_pool_stats* out) {
    out->allocated_blocks = s.allocated_blocks;
    out->free_blocks = s.free_blocks;
    out->live_blocks = s.live_blocks;
    out->reserved_blocks = s.reserved_blocks;
    out->retired_blocks = s.retired_blocks;
    out->shared_blocks = s.shared_blocks;
    out->live_references = s.live_references;
    out->slabs = s.slabs;
    out->submitted_epoch = (int64_t)s.submitted_epoch;
    out->completed_epoch = (int64_t)s.completed_epoch;
}

std::vector<LmLane> to_lanes(const mk_lane* lanes, int32_t n) {
    std::vector<LmLane> v;
    for (int32_t i = 0; i < n; ++i) {
        if (lanes[i].session == nullptr) throw std::runtime_error("lane has no session");
        v.push_back(LmLane{lanes[i].session->s.get(), lanes[i].input_ids, lanes[i].n_tokens, lanes[i].start_pos});
    }
    return v;
}

ModelConfig to_model_config(const mk_load_config* cfg) {
    ModelConfig c;
    if (cfg == nullptr) return c;
    c.device = cfg->device_ordinal;
    if (cfg->block_tokens > 0) c.block_tokens = cfg->block_tokens;
    if (cfg->slab_blocks > 0) c.slab_blocks = cfg->slab_blocks;
    if (cfg->kv_capacity_tokens > 0) c.kv_capacity_tokens = cfg->kv_capacity_tokens;
    c.prefix_capacity_tokens = cfg->prefix_capacity_tokens;
    if (cfg->kv_dtype != MK_TYPE_F16 && cfg->kv_dtype != MK_TYPE_F32 && cfg->kv_dtype != 0)
        throw std::runtime_error("kv_dtype must be MK_TYPE_F16 or MK_TYPE_F32");
    c.kv_f16 = cfg->kv_dtype != MK_TYPE_F32;
    if (cfg->max_batch_tokens > 0) c.max_batch_tokens = cfg->max_batch_tokens;
    if (cfg->max_batch_lanes > 0) c.max_batch_lanes = cfg->max_batch_lanes;
    c.matmul_path = cfg->matmul_path;
    if (cfg->ep_size > 1) {
        c.ep_size = cfg->ep_size;
        c.ep_rank = cfg->ep_rank;
        c.ep_mode = cfg->ep_mode;
        if (c.ep_mode != 0 && c.ep_mode != 1) throw std::runtime_error("ep_mode must be 0 or 1");
    }
    return c;
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------------------------------ model

int32_t mk_gguf_inspect(const char* path, mk_gguf_summary* out) {
    return guarded([&] {
        if (path == nullptr || out == nullptr) throw std::runtime_error("mk_gguf_inspect: null argument");
        GgufFile f(path);
        ModelSpec s = model_spec_from_gguf(f);
        GgufAudit a = validate_decoder_tensors(f, s);
        memset(out, 0, sizeof *out);
        strncpy(out->architecture, s.arch.c_str(), sizeof out->architecture - 1);
        out->n_layers = s.layers;
        out->hidden_size = s.hidden;
        out->q_heads = s.q_heads;
        out->kv_heads = s.kv_heads;
        out->head_dim = s.head_dim;
        out->rotary_dim = s.rotary_dim;
        out->ffn_size = s.ffn;
        out->vocab_size = s.vocab;
        out->max_context = s.max_context;
        out->experts = s.experts;
        out->experts_used = s.experts_used;
        out->expert_ffn_size = s.expert_ffn;
        out->tied_embeddings = s.tied ? 1 : 0;
        for (const LayerSpec& l : s.layer) {
            out->sliding_layers += l.sliding ? 1 : 0;
            out->nope_layers += l.rope ? 0 : 1;
            out->qk_norm |= l.qk_norm ? 1 : 0;
        }
        out->tensors_in_file = a.tensors_in_file;
        out->matrices = a.matrices;
        out->vectors = a.vectors;
        out->matrix_bytes = a.matrix_bytes;
    });
}

int32_t mk_model_load_gguf(const char* path, const mk_load_config* cfg, mk_model** out) {
    return guarded([&] {
        require_device();
        auto m = std::make_unique<mk_model>();
        m->lm = std::make_unique<Model>(path, to_model_config(cfg));
        *out = m.release();
    });
}

int32_t mk_model_new_fake(int32_t vocab, int32_t max_context, const mk_load_config* cfg, int64_t fail_forward_at, mk_model** out) {
    return guarded([&] {
        ModelConfig c = to_model_config(cfg);
        auto fake = std::make_unique<FakeLm>(vocab, max_context, c.block_tokens, c.slab_blocks, c.kv_capacity_tokens,
                                             c.prefix_capacity_tokens);
        if (fail_forward_at >= 0) fake->fail_forward_at(fail_forward_at);
        auto m = std::make_unique<mk_model>();
        m->lm = std::move(fake);
        *out = m.release();
    });
}

int32_t mk_model_fake_inject(mk_model* m, int32_t site, int64_t index) {
    return guarded([&] {
        FakeLm* fake = dynamic_cast<FakeLm*>(m->lm.get());
        if (fake == nullptr) throw std::runtime_error("failure injection is only available on the host-only fake model");
        fake->inject_failure(site, index);
    });
}

int32_t mk_model_fake_on_barrier(mk_model* m, void (*cb)(void*), void* user) {
    return guarded([&] {
        FakeLm* fake = dynamic_cast<FakeLm*>(m->lm.get());
        if (fake == nullptr) throw std::runtime_error("the barrier hook is only available on the host-only fake model");
        fake->on_next_barrier(cb, user);
    });
}

int32_t mk_model_free(mk_model* m) {
    return guarded([&] { delete m; });
}

int32_t mk_ep_unique_id(uint8_t* id_out) {
    return guarded([&] {
        require_device();
        EpComm::unique_id(id_out);
    });
}

int32_t mk_model_ep_init(mk_model* m, const uint8_t* id) {
    return guarded([&] {
        Model* model = dynamic_cast<Model*>(m->lm.get());
        if (model == nullptr) throw std::runtime_error("mk_model_ep_init needs a GGUF model");
        model->ep_init(id);
    });
}

int32_t mk_model_ep_idle_tick(mk_model* m) {
    return guarded([&] {
        Model* model = dynamic_cast<Model*>(m->lm.get());
        if (model == nullptr) throw std::runtime_error("mk_model_ep_idle_tick needs a GGUF model");
        model->ep_idle_tick();
    });
}

int32_t mk_model_spec(mk_model* m, mk_runtime_spec* out) {
    return guarded([&] {
        const LmRuntimeSpec& s = m->lm->spec();
        memset(out, 0, sizeof *out);
        out->vocab_size = s.vocab;
        out->max_context = s.max_context;
        out->n_layers = s.layers;
        out->hidden_size = s.hidden;
        out->n_stop_tokens = (int32_t)std::min<size_t>(s.stop_ids.size(), 8);
        for (int i = 0; i < out->n_stop_tokens; ++i) out->stop_token_ids[i] = s.stop_ids[(size_t)i];
        out->weight_bytes = s.weight_bytes;
        out->weight_bytes_per_token = s.weight_bytes_per_token;
        out->kv_bytes_per_token = s.kv_bytes_per_token;
    });
}

int32_t mk_session_new(mk_model* m, mk_session** out) {
    return guarded([&] {
        auto s = std::make_unique<mk_session>();
        s->s = m->lm->new_session();
        *out = s.release();
    });
}

int32_t mk_session_fork_prefix(mk_model* m, mk_session* src, int64_t logical_len, mk_session** out) {
    return guarded([&] {
        auto s = std::make_unique<mk_session>();
        s->s = m->lm->fork_session_prefix(*src->s, logical_len);
        *out = s.release();
    });
}

int32_t mk_session_free(mk_session* s) {
    return guarded([&] { delete s; });
}

int32_t mk_session_clear(mk_session* s) {
    return guarded([&] { s->s->owner->clear_session(*s->s); });
}

int32_t mk_session_len(mk_session* s, int64_t* out) {
    return guarded([&] { *out = s->s->logical_len; });
}

int32_t mk_session_block_table(mk_session* s, uint32_t* slots, uint64_t* generations, int32_t* n) {
    return guarded([&] {
        const std::vector<KvBlockId>& b = s->s->table->blocks();
        if ((int32_t)b.size() > *n) throw std::runtime_error("block table buffer is too small");
        for (size_t i = 0; i < b.size(); ++i) {
            if (slots) slots[i] = b[i].slot;
            if (generations) generations[i] = b[i].generation;
        }
        *n = (int32_t)b.size();
    });
}

int32_t mk_reset_session_for_prompt(mk_model* m, mk_session* s, const uint32_t* tokens, int32_t n, int64_t* cached_tokens) {
    return guarded([&] { *cached_tokens = m->lm->reset_session_for_prompt(*s->s, tokens, (size_t)n); });
}

int32_t mk_publish_prompt_prefix(mk_model* m, mk_session* s, const uint32_t* tokens, int32_t n) {
    return guarded([&] { m->lm->publish_prompt_prefix(*s->s, tokens, (size_t)n); });
}

int32_t mk_kv_capacity_query(mk_model* m, mk_kv_capacity* out) {
    return guarded([&] {  // kv_cache_capacity, src/decoder.rs:3682-3694
        KvPoolStats st = m->lm->pool_stats();
        out->block_tokens = st.block_tokens;
        out->total_blocks = st.max_blocks;
        out->free_blocks = st.free_blocks + (st.max_blocks - st.allocated_blocks);
        out->retired_blocks = st.retired_blocks;
    });
}

int32_t mk_pool_stats_query(mk_model* m, mk_pool_stats* out) {
    return guarded([&] { fill_pool_stats(m->lm->pool_stats(), out); });
}

int32_t mk_prefix_diagnostics_query(mk_model* m, mk_prefix_diagnostics* out) {
    return guarded([&] {
        memset(out, 0, sizeof *out);
        auto d = m->lm->prefix_diagnostics();
        if (!d) return;
        out->entries = d->entries;
        out->cached_blocks = d->cached_blocks;
        out->capacity_blocks = d->capacity_blocks;
        out->hits = d->hits;
        out->misses = d->misses;
        out->matched_tokens = d->matched_tokens;
        out->insertions = d->insertions;
        out->evictions = d->evictions;
    });
}

int32_t mk_reserve_batch(mk_model* m, const mk_lane* lanes, int32_t n_lanes, mk_reservation** out) {
    return guarded_kv([&] {
        auto r = std::make_unique<mk_reservation>();
        r->r = m->lm->reserve_batch(to_lanes(lanes, n_lanes));
        *out = r.release();
    });
}

int32_t mk_reservation_drop(mk_reservation* r) {
    return guarded([&] { delete r; });
}

int32_t mk_forward_set_sampling(mk_model* m, const mk_lane_sampling* lanes, int32_t n_lanes) {
    return guarded([&] {
        if (n_lanes < 0 || (n_lanes > 0 && lanes == nullptr)) throw std::runtime_error("mk_forward_set_sampling: bad arguments");
        for (int32_t i = 0; i < n_lanes; ++i) {
            if (!m->lm->device_sampling_covers(lanes[i].temperature, lanes[i].top_k))
                throw std::runtime_error("mk_forward_set_sampling: the device sampler covers greedy selection and 1 <= top_k <= 1024");
            if (lanes[i].temperature > 0.f && !(lanes[i].top_p > 0.f && lanes[i].top_p <= 1.f))
                throw std::runtime_error("mk_forward_set_sampling: top_p must be in (0, 1]");
            if (!(lanes[i].u >= 0.f && lanes[i].u < 1.f)) throw std::runtime_error("mk_forward_set_sampling: the draw must be in [0, 1)");
        }
        m->sampling.assign(lanes, lanes + n_lanes);
    });
}

int32_t mk_forward_batch_reserved(mk_model* m, const mk_lane* lanes, int32_t n_lanes, mk_reservation* r, uint32_t flags) {
    return guarded([&] {
        if (r == nullptr) throw std::runtime_error("forward needs a KV reservation");
        std::unique_ptr<LmReservation> res = std::move(r->r);
        delete r;  // consumed
        std::vector<LmLane> ll = to_lanes(lanes, n_lanes);
        std::vector<mk_lane_sampling> sampling = std::move(m->sampling);  // one forward only
        m->sampling.clear();
        if (!sampling.empty()) {
            if ((int32_t)sampling.size() != n_lanes) throw std::runtime_error("sampling settings cover another number of lanes than the forward");
            for (int32_t i = 0; i < n_lanes; ++i) {
                ll[(size_t)i].temperature = sampling[(size_t)i].temperature;
                ll[(size_t)i].top_k = sampling[(size_t)i].top_k;
                ll[(size_t)i].top_p = sampling[(size_t)i].top_p;
                ll[(size_t)i].u = sampling[(size_t)i].u;
            }
        }
        m->lm->forward_batch_reserved(ll, std::move(res), flags);
    });
}

int32_t mk_read_output(mk_model* m, float* logits, uint32_t* tokens) {
    return guarded([&] { m->lm->read_output(logits, tokens); });
}

int32_t mk_synchronize(mk_model* m) {
    return guarded([&] { m->lm->synchronize(); });
}

int32_t mk_last_forward_ms(mk_model* m, float* out) {
    return guarded([&] { *out = m->lm->last_forward_ms(); });
}

int32_t mk_launch_count(mk_model* m, int64_t* out) {
    return guarded([&] { *out = m->lm->launch_count(); });
}

int32_t mk_transfer_bytes(mk_model* m, int64_t* h2d, int64_t* d2h) {
    return guarded([&] {
        if (h2d) *h2d = m->lm->h2d_bytes();
        if (d2h) *d2h = m->lm->d2h_bytes();
    });
}

int32_t mk_profile_enable(mk_model* m, int32_t on) {
    return guarded([&] { m->lm->profile_enable(on != 0); });
}

int32_t mk_profile_query(mk_model* m, mk_kernel_profile* out, int32_t* n) {
    return guarded([&] {
        auto v = m->lm->profile_query();
        if (out != nullptr) {
            if ((int32_t)v.size() > *n) throw std::runtime_error("profile buffer is too small");
            for (size_t i = 0; i < v.size(); ++i) {
                memset(&out[i], 0, sizeof out[i]);
                strncpy(out[i].name, v[i].name.c_str(), sizeof out[i].name - 1);
                out[i].launches = v[i].launches;
                out[i].ms = v[i].ms;
                out[i].bytes = v[i].bytes;
                out[i].flops = v[i].flops;
            }
        }
        *n = (int32_t)v.size();
    });
}

// ------------------------------------------------------------------------------------------ engine

int32_t mk_engine_new(mk_model* m, const mk_engine_config* cfg, mk_engine** out) {
    return guarded([&] {
        EngineConfig c;
        c.max_active_sequences = cfg->max_active_sequences;
        c.scheduler_token_budget = cfg->scheduler_token_budget;
        c.prefill_token_quantum = cfg->prefill_token_quantum;
        c.queue_capacity = cfg->queue_capacity;
        c.record_logits = cfg->record_logits != 0;
        c.host_sampling = cfg->host_sampling != 0;
        auto e = std::make_unique<mk_engine>();
        e->e = std::make_unique<Engine>(*m->lm, c);
        *out = e.release();
    });
}

int32_t mk_engine_free(mk_engine* e) {
    return guarded([&] { delete e; });
}

int32_t mk_engine_submit(mk_engine* e, const mk_request* reqs, int32_t n, int32_t atomic_batch, int32_t* ids) {
    return guarded([&] {
        std::vector<EngineRequest> v;
        for (int32_t i = 0; i < n; ++i) {
            EngineRequest r;
            r.prompt.assign(reqs[i].prompt, reqs[i].prompt + reqs[i].n_prompt);
            r.max_new_tokens = reqs[i].max_new_tokens;
            r.ignore_stop_tokens = reqs[i].ignore_stop_tokens != 0;
            r.publish_prompt_prefix = reqs[i].no_prefix_publication == 0;
            r.event_capacity = reqs[i].event_capacity;
            r.event_send_timeout_ms = reqs[i].event_send_timeout_ms;
            r.temperature = reqs[i].temperature;
            r.top_k = reqs[i].top_k;
            r.top_p = reqs[i].top_p;
            r.repetition_penalty = reqs[i].repetition_penalty;
            r.presence_penalty = reqs[i].presence_penalty;
            r.frequency_penalty = reqs[i].frequency_penalty;
            r.seed = reqs[i].seed;
            v.push_back(std::move(r));
        }
        std::vector<int> out = e->e->submit(v, atomic_batch != 0);
        for (int32_t i = 0; i < n; ++i) ids[i] = out[(size_t)i];
    });
}

int32_t mk_engine_step(mk_engine* e, int32_t* ran_lanes) {
    return guarded([&] {
        int lanes = e->e->step();
        if (ran_lanes) *ran_lanes = lanes;
    });
}

int32_t mk_engine_run(mk_engine* e) {
    return guarded([&] { e->e->run(); });
}

int32_t mk_engine_pending(mk_engine* e, int32_t* out) {
    return guarded([&] { *out = e->e->pending(); });
}

int32_t mk_engine_result(mk_engine* e, int32_t request_id, uint32_t* tokens, int32_t* n, int32_t* finished, int64_t* cached_tokens) {
    return guarded([&] {
        const EngineResult& r = e->e->result(request_id);
        if (tokens != nullptr) {
            if ((int32_t)r.tokens.size() > *n) throw std::runtime_error("token buffer is too small");
            memcpy(tokens, r.tokens.data(), r.tokens.size() * 4);
        }
        *n = (int32_t)r.tokens.size();
        if (finished) *finished = (int32_t)r.state;
        if (cached_tokens) *cached_tokens = r.cached_tokens;
        if (r.state == FinishState::Failed) last_error_slot() = r.message;
    });
}

int32_t mk_engine_request_metrics(mk_engine* e, int32_t request_id, mk_request_metrics* out) {
    return guarded([&] {
        const EngineResult& r = e->e->result(request_id);
        out->prompt_tokens = r.prompt_tokens;
        out->cached_prompt_tokens = (int32_t)r.cached_tokens;
        out->generated_tokens = (int32_t)r.tokens.size();
        out->decode_steps = r.decode_steps;
        out->finish_reason = r.finish_reason == "length" ? 1 : r.finish_reason == "stop" ? 2 : r.finish_reason == "cancelled" ? 3 : 0;
        out->reserved_ = 0;
        out->suffix_prefill_ms = r.suffix_prefill_ms;
        out->first_token_ms = r.first_token_ms;
        out->prefill_ms = r.suffix_prefill_ms + r.first_token_ms;
        out->decode_ms = r.decode_ms;
    });
}

int32_t mk_model_fake_script(mk_model* m, const uint32_t* stop_ids, int32_t n_stop, const float* logits_row, int32_t n_logits) {
    return guarded([&] {
        FakeLm* fake = dynamic_cast<FakeLm*>(m->lm.get());
        if (fake == nullptr) throw std::runtime_error("scripting is only available on the host-only fake model");
        fake->script(stop_ids, n_stop, logits_row, n_logits);
    });
}

int32_t mk_engine_logits(mk_engine* e, int32_t request_id, float* out, int32_t* n_rows) {
    return guarded([&] {
        const EngineResult& r = e->e->result(request_id);
        // rows are vocab wide; the caller sizes the buffer from the token count
        if (out != nullptr) memcpy(out, r.logits.data(), r.logits.size() * 4);
        *n_rows = r.logit_rows;
    });
}

int32_t mk_engine_trace(mk_engine* e, int64_t tick, mk_tick_lane* lanes, int32_t* n) {
    return guarded([&] {
        const auto& tr = e->e->trace();
        if (tick < 0 || tick >= (int64_t)tr.size()) throw std::runtime_error("tick index out of range");
        const auto& t = tr[(size_t)tick];
        if (lanes != nullptr) {
            if ((int32_t)t.size() > *n) throw std::runtime_error("trace buffer is too small");
            for (size_t i = 0; i < t.size(); ++i) lanes[i] = mk_tick_lane{t[i].request_id, t[i].start_pos, t[i].n_tokens, t[i].phase};
        }
        *n = (int32_t)t.size();
    });
}

int32_t mk_engine_tick_info(mk_engine* e, int64_t tick, mk_tick_info* out) {
    return guarded([&] {
        const TickInfo& t = e->e->tick_info(tick);
        out->kind = (int32_t)t.kind;
        out->lane_count = t.lane_count;
        out->input_tokens = t.input_tokens;
        out->reserved_ = 0;
        out->model_ms = t.model_ms;
    });
}

int32_t mk_engine_batch_trace(mk_engine* e, int32_t member_request_id, mk_batch_trace* out, int64_t* forward_ticks, int32_t* n_forward_ticks) {
    return guarded([&] {
        int terminal = 0;
        const BatchTrace& b = e->e->batch_trace(member_request_id, &terminal);
        out->expected_members = (int32_t)b.members.size();
        out->admitted_members = b.admitted_members;
        out->terminal_members = terminal;
        out->rejected_members = b.rejected_members;
        out->admission_active_sequences = b.admission_active_sequences;
        out->packed_forwards = (int32_t)b.packed_forwards.size();
        out->complete = b.admission_complete && terminal == (int)b.members.size();
        out->reserved_ = 0;
        out->suffix_prefill_ms = b.suffix_prefill_ms;
        out->first_token_ms = b.first_token_ms;
        out->decode_ms = b.decode_ms;
        out->mixed_ms = b.mixed_ms;
        if (forward_ticks != nullptr) {
            if (n_forward_ticks == nullptr || *n_forward_ticks < (int32_t)b.packed_forwards.size())
                throw std::runtime_error("forward tick buffer is too small");
            for (size_t i = 0; i < b.packed_forwards.size(); ++i) forward_ticks[i] = b.packed_forwards[i];
        }
        if (n_forward_ticks != nullptr) *n_forward_ticks = (int32_t)b.packed_forwards.size();
    });
}

int32_t mk_engine_stats_query(mk_engine* e, mk_engine_stats* out) {
    return guarded([&] {
        const EngineStats& s = e->e->stats();
        out->ticks = s.ticks;
        out->prefill_tokens = s.prefill_tokens;
        out->decode_tokens = s.decode_tokens;
        out->completed_requests = s.completed;
        out->failed_requests = s.failed;
        out->kv_shrinks = s.kv_shrinks;
        out->device_ms = s.device_ms;
        out->cleanup_drains = s.cleanup_drains;
        out->device_sampled = s.device_sampled;
        out->cancelled_requests = s.cancelled;
        out->suffix_prefill_ms = s.suffix_prefill_ms;
        out->first_token_ms = s.first_token_ms;
        out->decode_ms = s.decode_ms;
        out->mixed_ms = s.mixed_ms;
    });
}

int32_t mk_engine_status(mk_engine* e, int32_t* status) {
    return guarded([&] { *status = (int32_t)e->e->status(); });
}

int32_t mk_engine_step_at(mk_engine* e, double now_ms, int32_t* ran_lanes) {
    return guarded([&] {
        int lanes = e->e->step_at(now_ms);
        if (ran_lanes != nullptr) *ran_lanes = lanes;
    });
}

int32_t mk_engine_consume_events(mk_engine* e, int32_t request_id, int32_t n) {
    return guarded([&] { e->e->consume_events(request_id, n); });
}

int32_t mk_engine_keep_trace(mk_engine* e, int32_t keep) {
    return guarded([&] { e->e->keep_trace(keep != 0); });
}

int32_t mk_engine_release_request(mk_engine* e, int32_t request_id) {
    return guarded([&] { e->e->release_request(request_id); });
}

int32_t mk_engine_cancel(mk_engine* e, int32_t request_id) {
    return guarded([&] { e->e->cancel(request_id); });
}

int32_t mk_engine_failure_kind(mk_engine* e, int32_t request_id, int32_t* kind) {
    return guarded([&] { *kind = (int32_t)e->e->result(request_id).kind; });
}

// ------------------------------------------------------------------------------------------ host-only pool

int32_t mk_kvpool_new(int32_t block_tokens, int32_t slab_blocks, int64_t max_blocks, mk_kvpool** out) {
    return guarded([&] {
        auto p = std::make_unique<mk_kvpool>();
        p->p = std::make_shared<KvPool>(block_tokens, slab_blocks, max_blocks);
        *out = p.release();
    });
}

int32_t mk_kvpool_free(mk_kvpool* p) {
    return guarded([&] { delete p; });
}

int32_t mk_kvpool_stats(mk_kvpool* p, mk_pool_stats* out) {
    return guarded([&] { fill_pool_stats(p->p->stats(), out); });
}

int32_t mk_kvtable_new(mk_kvpool* p, mk_kvtable** out) {
    return guarded([&] {
        auto t = std::make_unique<mk_kvtable>();
        t->t = std::make_unique<KvTable>(p->p, (int64_t)1 << 40);
        *out = t.release();
    });
}

int32_t mk_kvtable_free(mk_kvtable* t) {
    return guarded([&] { delete t; });
}

int32_t mk_kvtable_len(mk_kvtable* t, int64_t* out) {
    return guarded([&] { *out = t->t->logical_len(); });
}

int32_t mk_kvtable_blocks(mk_kvtable* t, uint32_t* slots, uint64_t* generations, int32_t* n) {
    return guarded([&] {
        const auto& b = t->t->blocks();
        if ((int32_t)b.size() > *n) throw std::runtime_error("block table buffer is too small");
        for (size_t i = 0; i < b.size(); ++i) {
            if (slots) slots[i] = b[i].slot;
            if (generations) generations[i] = b[i].generation;
        }
        *n = (int32_t)b.size();
    });
}

int32_t mk_kvtable_clear(mk_kvtable* t) {
    return guarded([&] { t->t->clear(); });
}

int32_t mk_kvtable_fork_prefix(mk_kvtable* t, int64_t tokens, mk_kvtable** out) {
    return guarded([&] {
        auto f = std::make_unique<mk_kvtable>();
        f->t = t->t->fork_prefix(tokens);
        *out = f.release();
    });
}

int32_t mk_kvtable_attach_prefix(mk_kvtable* t, mk_kvtable* src, int64_t tokens) {
    return guarded([&] { t->t->attach_prefix(*src->t, tokens); });
}

int32_t mk_kvpool_append_batch(mk_kvpool* p, mk_kvtable** tables, const int32_t* n_tokens, int32_t n, int32_t commit,
                               int64_t* copies_out, int32_t* n_copies) {
    return guarded_kv([&] {
        std::vector<KvTable*> tv;
        std::vector<int64_t> nv;
        for (int32_t i = 0; i < n; ++i) { tv.push_back(tables[i]->t.get()); nv.push_back(n_tokens[i]); }
        auto r = p->p->reserve_batch(tv, nv);
        if (n_copies != nullptr) {
            const auto& cows = r->cow_copies();
            if (copies_out != nullptr) {
                if ((int32_t)cows.size() > *n_copies) throw std::runtime_error("copy buffer is too small");
                for (size_t i = 0; i < cows.size(); ++i) {
                    copies_out[3 * i] = cows[i].src_slot;
                    copies_out[3 * i + 1] = cows[i].dst_slot;
                    copies_out[3 * i + 2] = cows[i].rows;
                }
            }
            *n_copies = (int32_t)cows.size();
        }
        if (commit == 1) {
            r->mark_all_used();
            r->commit();
        } else if (commit == 2) {
            // a forward that failed after it had touched its pages: what it wrote or read stays quarantined until the epoch
            // completes (cache.rs:1214-1276)
            r->mark_all_used();
            r->rollback();
        } else {
            r->rollback();
        }
    });
}

int32_t mk_kvpool_page_table(mk_kvpool* p, mk_kvtable** tables, const int32_t* n_tokens, int32_t n, uint32_t* pages, int32_t* n_rows,
                             int32_t* lane_offsets, int32_t* lane_counts, int32_t* lane_lens) {
    return guarded_kv([&] {
        std::vector<KvTable*> tv;
        std::vector<int64_t> nv;
        for (int32_t i = 0; i < n; ++i) { tv.push_back(tables[i]->t.get()); nv.push_back(n_tokens[i]); }
        auto r = p->p->reserve_batch(tv, nv);
        std::vector<uint32_t> pg;
        std::vector<int32_t> lo, lc, ll;
        r->page_table(pg, lo, lc, ll);
        if ((int32_t)(pg.size() / 2) > *n_rows) throw std::runtime_error("page table buffer is too small");
        memcpy(pages, pg.data(), pg.size() * 4);
        *n_rows = (int32_t)(pg.size() / 2);
        for (int32_t i = 0; i < n; ++i) { lane_offsets[i] = lo[(size_t)i]; lane_counts[i] = lc[(size_t)i]; lane_lens[i] = ll[(size_t)i]; }
        r->rollback();
    });
}

int32_t mk_kvpool_submit_epoch(mk_kvpool* p, int64_t* epoch) {
    return guarded([&] { *epoch = (int64_t)p->p->submitted_epoch(); });
}

int32_t mk_kvpool_complete_epoch(mk_kvpool* p, int64_t epoch) {
    return guarded([&] { p->p->mark_completed_through((uint64_t)epoch); });
}

// ------------------------------------------------------------------------------------------ prefix cache

int32_t mk_prefix_cache_new(int32_t block_tokens, int64_t capacity_blocks, mk_prefix_cache** out) {
    return guarded([&] {
        auto c = std::make_unique<mk_prefix_cache>();
        c->c = std::make_unique<TokenPrefixCache<int64_t>>((size_t)block_tokens, (size_t)capacity_blocks);
        *out = c.release();
    });
}

int32_t mk_prefix_cache_free(mk_prefix_cache* c) {
    return guarded([&] { delete c; });
}

int32_t mk_prefix_cache_insert(mk_prefix_cache* c, const uint32_t* tokens, int32_t n, int64_t value, int64_t cost, int64_t* evicted_out,
                               int32_t* n_evicted) {
    return guarded([&] {
        std::vector<TokenPrefixCache<int64_t>::Evicted> ev;
        bool ok = c->c->insert(std::vector<uint32_t>(tokens, tokens + n), value, (size_t)cost, &ev);
        if (n_evicted != nullptr) {
            if (evicted_out != nullptr) {
                if ((int32_t)ev.size() > *n_evicted) throw std::runtime_error("eviction buffer is too small");
                for (size_t i = 0; i < ev.size(); ++i) evicted_out[i] = ev[i].snapshot;
            }
            *n_evicted = (int32_t)ev.size();
        }
        if (!ok) throw std::runtime_error(n == 0 ? "prefix-cache entries must contain tokens" : "prefix-cache entry cost exceeds the configured budget");
    });
}

int32_t mk_prefix_cache_lookup(mk_prefix_cache* c, const uint32_t* tokens, int32_t n, int64_t* value, int64_t* matched_tokens) {
    return guarded([&] {
        auto hit = c->c->lookup_aligned_common_prefix(tokens, (size_t)n, (size_t)n);
        *value = hit ? *hit->snapshot : -1;
        *matched_tokens = hit ? (int64_t)hit->matched_tokens : 0;
    });
}

int32_t mk_prefix_cache_lookup_bounded(mk_prefix_cache* c, int32_t exact, const uint32_t* tokens, int32_t n, int64_t exclusive_max_tokens,
                                       int64_t* value, int64_t* matched_tokens, int64_t* snapshot_tokens) {
    return guarded([&] {
        const size_t limit = exclusive_max_tokens < 0 ? SIZE_MAX : (size_t)exclusive_max_tokens;
        auto hit = exact != 0 ? c->c->lookup(tokens, (size_t)n, limit) : c->c->lookup_aligned_common_prefix(tokens, (size_t)n, limit);
        *value = hit ? *hit->snapshot : -1;
        *matched_tokens = hit ? (int64_t)hit->matched_tokens : 0;
        if (snapshot_tokens != nullptr) *snapshot_tokens = hit ? (int64_t)hit->snapshot_tokens : 0;
    });
}

int32_t mk_prefix_cache_set_max_cost(mk_prefix_cache* c, int64_t max_cost, int64_t* evicted_out, int32_t* n_evicted) {
    return guarded([&] {
        if (max_cost < 0) throw std::runtime_error("prefix-cache budget must not be negative");
        std::vector<TokenPrefixCache<int64_t>::Evicted> ev;
        c->c->set_max_cost((size_t)max_cost, &ev);
        if (evicted_out != nullptr && n_evicted != nullptr) {
            if ((int32_t)ev.size() > *n_evicted) throw std::runtime_error("eviction buffer is too small");
            for (size_t i = 0; i < ev.size(); ++i) evicted_out[i] = ev[i].snapshot;
        }
        if (n_evicted != nullptr) *n_evicted = (int32_t)ev.size();
    });
}

int32_t mk_prefix_cache_force_collisions(mk_prefix_cache* c) {
    return guarded([&] { c->c->force_collisions_for_tests(); });
}

int32_t mk_prefix_cache_evict_lru(mk_prefix_cache* c, int64_t* value) {
    return guarded([&] {
        auto ev = c->c->evict_lru();
        *value = ev ? ev->snapshot : -1;
    });
}

int32_t mk_prefix_cache_diagnostics(mk_prefix_cache* c, mk_prefix_diagnostics* out) {
    return guarded([&] {
        PrefixCacheStats st = c->c->stats();
        out->entries = (int64_t)st.entries;
        out->cached_blocks = (int64_t)st.cost;
        out->capacity_blocks = (int64_t)st.max_cost;
        out->hits = (int64_t)st.hits;
        out->misses = (int64_t)st.misses;
        out->matched_tokens = (int64_t)st.matched_tokens;
        out->insertions = (int64_t)st.insertions;
        out->evictions = (int64_t)st.evictions;
    });
}

int32_t mk_prefix_block_digests(int32_t block_tokens, const uint32_t* tokens, int32_t n, uint8_t* digests, int32_t* n_blocks) {
    return guarded([&] {
        int32_t full = n / block_tokens;
        if (full > *n_blocks) throw std::runtime_error("digest buffer is too small");
        PromptHashPlan plan(tokens, (size_t)n, (size_t)block_tokens);
        for (int32_t b = 0; b < full; ++b) {
            PrefixDigest d = plan.endpoint((size_t)(b + 1) * block_tokens);
            memcpy(digests + 32 * b, d.data(), 32);
        }
        *n_blocks = full;
    });
}

}  // extern "C"
