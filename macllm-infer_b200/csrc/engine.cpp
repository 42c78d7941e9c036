// See engine.h.  Line references are into the reference's src/engine.rs and src/generation.rs.
#include "engine.h"
#include <chrono>
#include <thread>
#include "host_sampler.h"
#include <algorithm>
#include <cmath>
#include <numeric>

namespace mk {

Engine::Engine(PagedLm& model, const EngineConfig& cfg) : model_(model), cfg_(cfg) {
    // EngineConfig::validate (engine.rs:350-367): the same checks in the same order with the same wording
    if (cfg.queue_capacity <= 0) throw std::runtime_error("queue capacity must be positive");
    if (cfg.max_active_sequences <= 0) throw std::runtime_error("maximum active sequences must be positive");
    if (cfg.scheduler_token_budget <= 0) throw std::runtime_error("scheduler token budget must be positive");
    if (cfg.prefill_token_quantum <= 0) throw std::runtime_error("prefill token quantum must be positive");
    if (cfg.prefill_token_quantum > cfg.scheduler_token_budget) throw std::runtime_error("prefill token quantum cannot exceed the scheduler token budget");
    // worker_main creates every reusable session up front (engine.rs:1336-1360)
    for (int i = 0; i < cfg.max_active_sequences; ++i) sessions_.push_back(model_.new_session());
}

Engine::~Engine() {
    // sequences release their pages before the sessions' tables go away
    active_.clear();
    sessions_.clear();
}

std::vector<int> Engine::submit(const std::vector<EngineRequest>& reqs, bool atomic_batch) {
    // submit_batch_with_policy (engine.rs:976-1053) in its order and wording (engine.rs:394-426): empty, larger than the atomic
    // admission limit min(queue capacity, active limit) (engine.rs:876), worker unavailable, queue full - the batch is
    // queued whole or not at all
    if (reqs.empty()) throw std::runtime_error("inference batch must not be empty");
    const int maximum_atomic_batch = std::min(cfg_.queue_capacity, cfg_.max_active_sequences);
    if (atomic_batch && (int)reqs.size() > maximum_atomic_batch)
        throw std::runtime_error("inference batch contains " + std::to_string(reqs.size()) + " requests, but the atomic admission limit is " +
                                 std::to_string(maximum_atomic_batch));
    if (poisoned_) throw std::runtime_error("inference worker is unavailable (Poisoned)");
    if ((int)(queue_.size() + reqs.size()) > cfg_.queue_capacity) throw std::runtime_error("inference queue is full");
    std::vector<int> ids;
    int batch = atomic_batch ? next_batch_++ : -1;
    if (atomic_batch) batches_.emplace_back();
    for (const EngineRequest& r : reqs) {
        Job j;
        j.id = next_id_++;
        j.req = r;
        j.batch = batch;
        j.batch_size = atomic_batch ? (int)reqs.size() : 0;
        results_[j.id] = EngineResult{};
        if (atomic_batch) {
            batches_[(size_t)batch].members.push_back(j.id);
            batch_of_request_[j.id] = batch;
        }
        ids.push_back(j.id);
        queue_.push_back(std::move(j));
    }
    return ids;
}

const EngineResult& Engine::result(int id) const {
    auto it = results_.find(id);
    if (it == results_.end()) throw std::runtime_error("unknown request id " + std::to_string(id));
    return it->second;
}

const TickInfo& Engine::tick_info(int64_t tick) const {
    if (tick < 0 || tick >= (int64_t)tick_info_.size()) throw std::runtime_error("tick index out of range");
    return tick_info_[(size_t)tick];
}

void Engine::keep_trace(bool keep) {
    keep_trace_ = keep;
    if (!keep) {
        trace_.clear();
        trace_.shrink_to_fit();
        tick_info_.clear();
        tick_info_.shrink_to_fit();
    }
}

void Engine::release_request(int id) {
    auto it = results_.find(id);
    if (it == results_.end()) throw std::runtime_error("unknown request id " + std::to_string(id));
    if (it->second.state == FinishState::Running) throw std::runtime_error("request " + std::to_string(id) + " is still running");
    for (const auto& slot : active_)
        if (slot->id == id) throw std::runtime_error("request " + std::to_string(id) + " still has events to deliver");
    results_.erase(it);
    auto b = batch_of_request_.find(id);
    if (b != batch_of_request_.end()) {   // the batch's trace goes with its last member
        const int batch = b->second;
        batch_of_request_.erase(b);
        bool any = false;
        for (int member : batches_[(size_t)batch].members) any = any || batch_of_request_.count(member) != 0;
        if (!any) batches_[(size_t)batch] = BatchTrace{};
    }
}

const BatchTrace& Engine::batch_trace(int member_id, int* terminal) const {
    auto it = batch_of_request_.find(member_id);
    if (it == batch_of_request_.end()) throw std::runtime_error("request " + std::to_string(member_id) + " was not submitted in an atomic batch");
    const BatchTrace& b = batches_[(size_t)it->second];
    int ended = 0;
    for (int id : b.members) {
        auto r = results_.find(id);
        ended += r == results_.end() || r->second.state != FinishState::Running;   // a released result had ended
    }
    if (terminal != nullptr) *terminal = ended;
    return b;
}

void Engine::fail_request(int id, const std::string& message, FailureKind kind) {
    EngineResult& r = results_[id];
    if (r.state != FinishState::Running) return;  // a terminal event is delivered once
    r.state = FinishState::Failed;
    r.message = message;
    r.kind = kind;
    ++stats_.failed;
}

void Engine::cancel(int id) {
    if (id < 0 || id >= next_id_.load()) throw std::runtime_error("unknown request id");
    std::lock_guard<std::mutex> lock(cancel_mu_);
    cancelled_.insert(id);
    any_cancelled_.store(true, std::memory_order_release);
}

bool Engine::is_cancelled(int id) {
    if (!any_cancelled_.load(std::memory_order_acquire)) return false;  // the common tick takes no lock
    std::lock_guard<std::mutex> lock(cancel_mu_);
    return cancelled_.count(id) != 0;
}

// Flags of requests that have ended are dropped, so that the set stays as small as the work in flight and the common tick
// goes back to taking no lock.  A flag set for a request that had already ended is dropped here as well.
void Engine::forget_settled_cancellations() {
    if (!any_cancelled_.load(std::memory_order_acquire)) return;
    std::lock_guard<std::mutex> lock(cancel_mu_);
    for (auto it = cancelled_.begin(); it != cancelled_.end();) {
        auto r = results_.find(*it);
        if (r == results_.end() || r->second.state != FinishState::Running) it = cancelled_.erase(it);   // ended, or already released
        else ++it;
    }
    if (cancelled_.empty()) any_cancelled_.store(false, std::memory_order_release);
}

// A cancelled request gets no terminal event in the reference (its receiver is gone); here its result says so.
void Engine::finish_cancelled(int id) {
    EngineResult& r = results_[id];
    if (r.state != FinishState::Running) return;
    r.state = FinishState::Cancelled;
    r.finish_reason = "cancelled";
    ++stats_.cancelled;
}

// ServingScheduler::poison (engine.rs:2719-2770): drain what was submitted, fail every active slot, every member of
// a pending atomic batch and every queued job with kind Fatal, drop the sequences and all reusable sessions.
void Engine::poison(std::string message) {
    poisoned_ = true;
    if (forward_needs_drain_) {
        forward_needs_drain_ = false;
        ++stats_.cleanup_drains;
        try {
            model_.synchronize();
        } catch (const std::exception& e) {
            message += std::string("; forward-error cleanup synchronization also failed: ") + e.what();
        }
    }
    if (orphan_ >= 0) fail_request(orphan_, message, FailureKind::Fatal);
    orphan_ = -1;
    for (auto& slot : active_) fail_request(slot->id, message, FailureKind::Fatal);
    active_.clear();    // sequences go without a completion barrier of their own (discard_session_without_synchronize)
    sessions_.clear();
    for (Job& j : pending_atomic_) fail_request(j.id, message, FailureKind::Fatal);
    pending_atomic_.clear();
    for (Job& j : queue_) fail_request(j.id, message, FailureKind::Fatal);
    queue_.clear();
    round_visits_remaining_ = round_budget_remaining_ = 0;
    poison_message_ = std::move(message);
}

void Engine::admit(Job job) {  // admit_with_diagnostic_refresh, engine.rs:1654-1808
    if ((int)active_.size() >= cfg_.max_active_sequences) throw std::runtime_error("scheduler attempted to exceed the active sequence limit");
    // a request given up while it queued is skipped before preflight and model work: no validation message, no session
    // taken, no prefix lookup (engine.rs:1671-1674,1715-1718)
    if (is_cancelled(job.id)) return finish_cancelled(job.id);
    const EngineRequest& rq = job.req;
    // reject_preflight (engine.rs:3027-3040): the request fails alone; a traced batch counts it as a rejected member
    auto fail_request = [&](int id, const std::string& message, FailureKind kind = FailureKind::InvalidRequest) {
        this->fail_request(id, message, kind);
        if (job.batch >= 0) ++batches_[(size_t)job.batch].rejected_members;
    };
    const LmRuntimeSpec& spec = model_.spec();
    // prepare_request for EngineInput::TokenIds (engine.rs:2976-3021): empty prompt, vocabulary, context - in that order,
    // with the reference's wording (the context message leads with the phrase clients recognise an overflow by)
    if (rq.prompt.empty()) return fail_request(job.id, "raw token prompt must not be empty");
    for (size_t i = 0; i < rq.prompt.size(); ++i)
        if ((int64_t)rq.prompt[i] >= spec.vocab)
            return fail_request(job.id, "raw prompt token " + std::to_string(rq.prompt[i]) + " at index " + std::to_string(i) +
                                            " exceeds model vocabulary " + std::to_string(spec.vocab));
    int64_t required = (int64_t)rq.prompt.size() + std::max(rq.max_new_tokens - 1, 0);
    if (required > spec.max_context)
        return fail_request(job.id, "This model's maximum context length is " + std::to_string(spec.max_context) + " tokens; the prompt (" +
                                        std::to_string(rq.prompt.size()) + " tokens) plus requested output (" +
                                        std::to_string(rq.max_new_tokens) + " tokens) exceeds it");
    // EngineRequest::sampler -> Sampler::new + set_penalties (sampling.rs:43-79), reported as in prepare_request (engine.rs:3022-3032)
    {
        const char* why = nullptr;
        if (!(std::isfinite(rq.temperature) && rq.temperature >= 0.f)) why = "temperature must be finite and non-negative";
        else if (!(std::isfinite(rq.top_p) && rq.top_p > 0.f && rq.top_p <= 1.f)) why = "top_p must be finite and in (0, 1]";
        else if (!(std::isfinite(rq.repetition_penalty) && rq.repetition_penalty > 0.f)) why = "repetition_penalty must be finite and positive";
        else if (!(std::isfinite(rq.presence_penalty) && rq.presence_penalty >= -2.f && rq.presence_penalty <= 2.f)) why = "invalid presence_penalty";
        else if (!(std::isfinite(rq.frequency_penalty) && rq.frequency_penalty >= -2.f && rq.frequency_penalty <= 2.f)) why = "invalid frequency_penalty";
        if (why != nullptr) return fail_request(job.id, std::string("invalid sampling parameters: ") + why);
    }
    // kv_capacity_rejection (engine.rs:2839-2863)
    {
        KvPoolStats st = model_.pool_stats();
        int64_t max_cached = rq.max_new_tokens == 0 ? 0 : (int64_t)rq.prompt.size() + rq.max_new_tokens - 1;
        if (max_cached > st.max_blocks * st.block_tokens)
            return fail_request(job.id,
                                "request requires up to " + std::to_string(max_cached) +
                                    " cached tokens, exceeding the configured shared KV capacity of " + std::to_string(st.max_blocks) +
                                    " blocks \xc3\x97 " + std::to_string(st.block_tokens) + " tokens",
                                FailureKind::ResourceExhausted);
    }
    if (sessions_.empty()) throw std::runtime_error("active slot has no reusable inference session");
    auto seq = std::make_unique<Sequence>();
    seq->id = job.id;
    seq->req = rq;
    seq->session = std::move(sessions_.back());  // LIFO (engine.rs:1719-1722)
    sessions_.pop_back();
    seq->history = rq.prompt;
    seq->prompt_tokens = (int)rq.prompt.size();
    seq->rng = rq.seed * 0x9E3779B97F4A7C15ull + 0xD1B54A32D192ED03ull;
    // GenerationCore::new (generation.rs:787-832): prefix lookup + block-table attach happen at admission
    int64_t cached = 0;
    try {
        cached = model_.reset_session_for_prompt(*seq->session, seq->history.data(), seq->history.size());
        if (cached >= (int64_t)seq->history.size())
            throw std::runtime_error("prefix cache must leave at least one prompt token for first-token logits");
    } catch (...) {
        sessions_.push_back(std::move(seq->session));  // the slot's session is not lost with the failed admission
        orphan_ = job.id;                              // neither queued nor active any more: poison() answers it
        throw;
    }
    seq->cursor = (int)cached;
    seq->batch = job.batch;
    results_[job.id].cached_tokens = cached;
    results_[job.id].prompt_tokens = seq->prompt_tokens;
    if (job.batch >= 0) ++batches_[(size_t)job.batch].admitted_members;  // record_admitted, engine.rs:1800-1803
    active_.push_back(std::move(seq));
}

bool Engine::admit_pending_atomic() {  // engine.rs:1886-1936
    if (pending_atomic_.empty()) return false;
    int available = cfg_.max_active_sequences - (int)active_.size();
    if ((int)pending_atomic_.size() > available) return false;
    std::vector<Job> batch = std::move(pending_atomic_);
    pending_atomic_.clear();
    const int batch_id = batch.front().batch;
    for (Job& j : batch) admit(std::move(j));
    BatchTrace& bt = batches_[(size_t)batch_id];  // finish_admission, engine.rs:1926-1934
    bt.admission_active_sequences = (int)active_.size();
    bt.admission_complete = true;
    return true;
}

bool Engine::try_admit_available() {  // engine.rs:1810-1881
    bool admitted = admit_pending_atomic();
    if (!pending_atomic_.empty()) return admitted;
    while ((int)active_.size() < cfg_.max_active_sequences && !queue_.empty()) {
        Job job = std::move(queue_.front());
        queue_.pop_front();
        if (job.batch < 0) {
            admit(std::move(job));
            admitted = true;
            continue;
        }
        int batch = job.batch, size = job.batch_size;
        pending_atomic_.push_back(std::move(job));
        while ((int)pending_atomic_.size() < size) {
            if (queue_.empty() || queue_.front().batch != batch)
                throw std::runtime_error("atomic batch jobs were not contiguous in the inference queue");
            pending_atomic_.push_back(std::move(queue_.front()));
            queue_.pop_front();
        }
        admit_pending_atomic();
        admitted = true;
        if (!pending_atomic_.empty()) break;
    }
    return admitted;
}

void Engine::reclaim(Sequence& s) {  // reclaim_slot_sequence_after_completion_barrier, engine.rs:2676-2690
    if (s.reclaimed) return;
    model_.clear_session(*s.session);
    s.reclaimed = std::move(s.session);
}

static inline uint64_t next_u64(uint64_t& state) {
    state += 0x9E3779B97F4A7C15ull;
    uint64_t z = state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// One uniform draw in [0, 1) per sampled token, the same stream whether the token is picked on the host or on the device.
static inline float next_uniform(uint64_t& state) { return (float)(next_u64(state) >> 40) * (1.0f / 16777216.0f); }

uint32_t Engine::sample(Sequence& s, float* row) {  // Sampler::sample_with_generated, sampling.rs:95-169
    const int vocab = model_.spec().vocab;
    const EngineRequest& rq = s.req;
    const uint32_t* generated = s.history.data() + (s.history.size() - (size_t)s.generated);
    apply_penalties(row, vocab, s.history.data(), (int64_t)s.history.size(), rq.repetition_penalty, generated, s.generated,
                    rq.presence_penalty, rq.frequency_penalty);
    if (rq.temperature <= 0.f) return (uint32_t)argmax_first(row, vocab);
    // temperature / top-k / top-p (sampling.rs:145-169,337-390).  The draw uses this library's own
    // counter-based generator: the reference's ChaCha8 stream is a third-party detail that is not
    // restated, so stochastic sampling is not token-comparable with the reference.
    return sample_top_k_top_p(row, vocab, rq.temperature, rq.top_k, rq.top_p, next_uniform(s.rng));
}

int Engine::step() {
    const double now_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
    return step_at(now_ms);
}

void Engine::consume_events(int id, int n) {
    if (n < 0) throw std::runtime_error("cannot take a negative number of events");
    for (auto& slot : active_)
        if (slot->id == id) {
            slot->in_channel = std::max(0, slot->in_channel - n);
            return;
        }
    if (results_.find(id) == results_.end()) throw std::runtime_error("unknown request id " + std::to_string(id));
    // a request that has left the scheduler has no channel any more: nothing to do
}

// ActiveSequence::flush_pending (engine.rs:1408-1465): move waiting events into the channel while it has room.  A full channel
// blocks the slot; the wait is timed from the moment THIS event first met a full channel - polling does not restart it, a
// successful send does - and a wait of event_send_timeout gives the request up like a cancellation.
Engine::Flush Engine::flush_pending(Sequence& s, double now_ms) {
    if (is_cancelled(s.id)) {
        s.pending_events = 0;
        return Flush::Abandoned;
    }
    if (s.req.event_capacity <= 0) {
        s.pending_events = 0;
        return Flush::Drained;
    }
    while (s.pending_events > 0) {
        if (s.in_channel < s.req.event_capacity) {
            ++s.in_channel;
            --s.pending_events;
            s.blocked_since = -1.0;
            continue;
        }
        if (s.blocked_since < 0.0) s.blocked_since = now_ms;
        if (now_ms - s.blocked_since >= s.req.event_send_timeout_ms) {
            cancel(s.id);
            s.pending_events = 0;
            return Flush::Abandoned;
        }
        return Flush::Blocked;
    }
    return Flush::Drained;
}

int Engine::step_at(double now_ms) {  // one turn of ServingScheduler::run, engine.rs:1577-1647
    if (poisoned_) return 0;
    try {
        return drive_once(now_ms);
    } catch (const std::exception& e) {
        poison(std::string("inference worker failed: ") + e.what());
    } catch (...) {
        poison("inference worker panicked and was poisoned");
    }
    return 0;
}

int Engine::drive_once(double now_ms) {  // engine.rs:1938-1964
    blocked_last_tick_ = 0;
    try_admit_available();
    if (active_.empty()) {
        forget_settled_cancellations();
        return 0;
    }
    if (round_visits_remaining_ == 0 || round_budget_remaining_ == 0) {
        round_visits_remaining_ = (int)active_.size();
        round_budget_remaining_ = cfg_.scheduler_token_budget;
    }

    // ---- collect_visits (engine.rs:2005-2095)
    const int visit_limit = std::min(round_visits_remaining_, (int)active_.size());
    std::vector<Visit> actions;
    int token_budget = round_budget_remaining_;
    for (int index = 0; index < visit_limit; ++index) {
        if (token_budget == 0) break;
        Sequence& s = *active_[(size_t)index];
        Visit v;
        const Flush initial = flush_pending(s, now_ms);
        if (initial == Flush::Abandoned) {  // engine.rs:1409-1417,2024-2029: leaves before the peers' forward
            v.kind = Visit::Remove;
            actions.push_back(v);
            continue;
        }
        if (initial == Flush::Blocked) {    // engine.rs:2030-2032: the slot keeps its place and runs nothing this tick
            ++blocked_last_tick_;
            v.kind = Visit::Keep;
            actions.push_back(v);
            continue;
        }
        if (s.delivering) {
            v.kind = Visit::Remove;
            actions.push_back(v);
            continue;
        }
        const int step_budget = std::min(cfg_.prefill_token_quantum, token_budget);
        // GenerationCore::preview (generation.rs:876-943)
        if (s.phase == Phase::Finished || s.req.max_new_tokens == 0) {
            v.kind = Visit::Complete;
            v.finished = true;
            actions.push_back(v);
            continue;
        }
        if (s.phase == Phase::Failed) throw std::runtime_error("generation sequence cannot resume after a failed step");
        if (s.phase == Phase::Prefill) {
            int remaining = s.prompt_tokens - s.cursor;
            if (remaining <= 0) throw std::runtime_error("generation prefill cursor is already complete");
            v.start_pos = s.cursor;
            v.n_tokens = std::min(remaining, step_budget);
            v.was_prefill = true;
        } else {
            v.start_pos = s.prompt_tokens + std::max(s.generated - 1, 0);
            v.n_tokens = 1;
        }
        if (s.session->logical_len != v.start_pos)
            throw std::runtime_error("generation session cache length " + std::to_string(s.session->logical_len) +
                                     " does not match expected position " + std::to_string(v.start_pos));
        v.kind = Visit::Preview;
        token_budget -= v.n_tokens;
        actions.push_back(v);
    }
    const int visits = (int)actions.size();
    for (int i = 0; i < visits; ++i)  // reclaim_collected_removals (engine.rs:1995-2003)
        if (actions[(size_t)i].kind == Visit::Remove) {
            reclaim(*active_[(size_t)i]);
            // only now is the cancelled request answered: if clearing its session fails, it is still a slot of the
            // scheduler and gets the fatal message with its peers (engine.rs:5640-5682)
            if (is_cancelled(active_[(size_t)i]->id)) finish_cancelled(active_[(size_t)i]->id);
        }

    // ---- reserve_and_prepare_visits (engine.rs:2097-2167)
    std::vector<int> candidates;
    for (int i = 0; i < visits; ++i)
        if (actions[(size_t)i].kind == Visit::Preview) candidates.push_back(i);
    std::unique_ptr<LmReservation> reservation;
    int input_tokens = 0;
    size_t selected = candidates.size();
    if (!candidates.empty()) {
        for (;;) {
            std::vector<LmLane> lanes;
            for (size_t c = 0; c < selected; ++c) {
                Sequence& s = *active_[(size_t)candidates[c]];
                const Visit& v = actions[(size_t)candidates[c]];
                lanes.push_back(LmLane{s.session.get(), nullptr, v.n_tokens, v.start_pos});
            }
            try {
                // a failed allocation may leave storage initialisation work behind; Exhausted and success reset the
                // obligation to drain (engine.rs:2131-2152)
                forward_needs_drain_ = true;
                reservation = model_.reserve_batch(lanes);
                break;
            } catch (const KvPoolExhausted& e) {
                forward_needs_drain_ = false;
                if (selected > 1) {  // drop the LAST candidate and retry (engine.rs:2145-2149)
                    --selected;
                    ++stats_.kv_shrinks;
                    continue;
                }
                // one irreducible lane fails only that request (fail_kv_exhausted_visit, engine.rs:2205-2231)
                for (int idx : candidates) actions[(size_t)idx].kind = Visit::Keep;
                Sequence& s = *active_[(size_t)candidates[0]];
                fail_request(s.id, e.what(), FailureKind::ResourceExhausted);
                ++s.pending_events;   // EngineEvent::Failed (engine.rs:2218-2221)
                s.delivering = true;
                reclaim(s);
                selected = 0;
                break;
            }
        }
        for (size_t c = selected; c < candidates.size(); ++c) actions[(size_t)candidates[c]].kind = Visit::Keep;
        // prepare_reserved_visits (engine.rs:2169-2203): GenerationCore::prepare (generation.rs:1003-1102)
        for (size_t c = 0; c < selected; ++c) {
            Visit& v = actions[(size_t)candidates[c]];
            Sequence& s = *active_[(size_t)candidates[c]];
            v.ready_to_sample = !v.was_prefill || v.start_pos + v.n_tokens == s.prompt_tokens;
            v.kind = Visit::Forward;
            input_tokens += v.n_tokens;
        }
    }

    // ---- execute_prepared_visits (engine.rs:2233-2269)
    int lane_count = 0;
    for (const Visit& v : actions) lane_count += v.kind == Visit::Forward;
    if (lane_count > 0) {
        std::vector<LmLane> lanes;
        std::vector<TickLaneTrace> tick;
        // tokens are picked on the device unless some lane needs what only the host sampler has: penalties (they read
        // the request's history), an unbounded or very wide top-k, or recorded logits
        bool device_greedy = !cfg_.host_sampling && !cfg_.record_logits;
        for (int i = 0; i < visits; ++i) {
            const Visit& v = actions[(size_t)i];
            if (v.kind != Visit::Forward) continue;
            Sequence& s = *active_[(size_t)i];
            const uint32_t* ids = v.was_prefill ? s.history.data() + v.start_pos : &s.decode_token;
            lanes.push_back(LmLane{s.session.get(), ids, v.n_tokens, v.start_pos});
            const ForwardKind phase = !v.was_prefill ? ForwardKind::Decode : (v.ready_to_sample ? ForwardKind::FirstToken : ForwardKind::SuffixPrefill);
            tick.push_back(TickLaneTrace{s.id, v.start_pos, v.n_tokens, (int32_t)phase});
            const EngineRequest& rq = s.req;
            if (v.ready_to_sample && (std::fabs(rq.repetition_penalty - 1.f) >= 1.1920929e-07f || rq.presence_penalty != 0.f ||
                                      rq.frequency_penalty != 0.f || !model_.device_sampling_covers(rq.temperature, rq.top_k)))
                device_greedy = false;
            if (v.was_prefill) stats_.prefill_tokens += v.n_tokens; else stats_.decode_tokens += v.n_tokens;
        }
        if (device_greedy) {
            // one uniform draw per stochastic token, taken from the request's stream exactly as the host sampler would
            size_t li = 0;
            for (int i = 0; i < visits; ++i) {
                const Visit& v = actions[(size_t)i];
                if (v.kind != Visit::Forward) continue;
                Sequence& s = *active_[(size_t)i];
                LmLane& l = lanes[li++];
                if (v.ready_to_sample && s.req.temperature > 0.f) {
                    l.temperature = s.req.temperature;
                    l.top_k = s.req.top_k;
                    l.top_p = s.req.top_p;
                    l.u = next_uniform(s.rng);
                    ++stats_.device_sampled;
                }
            }
        }
        uint32_t flags = device_greedy ? FWD_WANT_TOKENS : FWD_WANT_LOGITS;
        forward_needs_drain_ = true;  // engine.rs:2294
        model_.forward_batch_reserved(lanes, std::move(reservation), flags);
        // validate every lane's cache length BEFORE sampling (engine.rs:2258-2265)
        for (const LmLane& l : lanes)
            if (l.session->logical_len != (int64_t)l.start_pos + l.n_tokens)
                throw std::runtime_error("model advanced generation cache to an unexpected length");
        // complete_mixed_forward (engine.rs:2378-2409): the completion barrier
        const int vocab = model_.spec().vocab;
        forward_needs_drain_ = false;  // the read-back is the barrier; a failure inside it is not drained again (engine.rs:2388-2391)
        if (device_greedy) {
            tokens_host_.resize((size_t)lane_count);
            model_.read_output(nullptr, tokens_host_.data());
        } else {
            logits_host_.resize((size_t)lane_count * vocab);
            model_.read_output(logits_host_.data(), nullptr);
        }
        const double tick_ms = model_.last_forward_ms();   // read once: the device time of this packed forward
        stats_.device_ms += tick_ms;
        {   // collect_pending_benchmark_forwards + record_packed_forward (engine.rs:2306-2375,2394-2405,601-619)
            TickInfo info;
            info.kind = (ForwardKind)tick.front().phase;
            for (const TickLaneTrace& l : tick)
                if (l.phase != tick.front().phase) info.kind = ForwardKind::Mixed;
            info.lane_count = lane_count;
            info.input_tokens = input_tokens;
            info.model_ms = tick_ms;
            auto bucket = [&](double& suffix, double& first, double& decode, double& mixed) -> double& {
                switch (info.kind) {
                    case ForwardKind::SuffixPrefill: return suffix;
                    case ForwardKind::FirstToken: return first;
                    case ForwardKind::Decode: return decode;
                    default: return mixed;
                }
            };
            bucket(stats_.suffix_prefill_ms, stats_.first_token_ms, stats_.decode_ms, stats_.mixed_ms) += info.model_ms;
            std::vector<int> seen;  // every traced batch with a member in this forward records the whole forward once
            for (int i = 0; i < visits; ++i) {
                if (actions[(size_t)i].kind != Visit::Forward) continue;
                const int b = active_[(size_t)i]->batch;
                if (b < 0 || std::find(seen.begin(), seen.end(), b) != seen.end()) continue;
                seen.push_back(b);
                BatchTrace& bt = batches_[(size_t)b];
                bucket(bt.suffix_prefill_ms, bt.first_token_ms, bt.decode_ms, bt.mixed_ms) += info.model_ms;
                if (keep_trace_) bt.packed_forwards.push_back((int64_t)trace_.size());   // the index of this forward among the kept records
            }
            if (keep_trace_) tick_info_.push_back(info);
        }
        ++stats_.ticks;
        if (keep_trace_) trace_.push_back(std::move(tick));
        // complete_mixed_rows (engine.rs:2411-2523)
        int row = 0;
        for (int i = 0; i < visits; ++i) {
            Visit& v = actions[(size_t)i];
            if (v.kind != Visit::Forward) continue;
            Sequence& s = *active_[(size_t)i];
            const int next_cache_len = v.start_pos + v.n_tokens;
            // publish after every completed prefill chunk that ends inside the prompt, before sampling
            // (generation.rs:505-509,768-773)
            if (s.req.publish_prompt_prefix && v.was_prefill && next_cache_len > 0 && next_cache_len <= s.prompt_tokens)
                model_.publish_prompt_prefix(*s.session, s.history.data(), (size_t)next_cache_len);
            v.kind = Visit::Complete;
            v.finished = false;
            // GenerationCore::complete (generation.rs:1159-1266): the forward's time is the sequence's before anything else
            {
                EngineResult& res = results_[s.id];
                const double t = tick_ms;
                if (!v.was_prefill) { res.decode_ms += t; ++res.decode_steps; }
                else if (v.ready_to_sample) res.first_token_ms += t;
                else res.suffix_prefill_ms += t;
            }
            if (is_cancelled(s.id)) {  // given up while the forward ran: the row is dropped, the peers' rows keep their places
                s.phase = Phase::Finished;
                finish_cancelled(s.id);
                v.finished = true;
                ++row;
                continue;
            }
            if (!v.ready_to_sample) {
                s.phase = Phase::Prefill;
                s.cursor = next_cache_len;
                ++row;
                continue;
            }
            uint32_t token;
            if (device_greedy) {
                token = tokens_host_[(size_t)row];
            } else {
                float* lrow = logits_host_.data() + (size_t)row * vocab;
                if (cfg_.record_logits) {
                    EngineResult& r = results_[s.id];
                    r.logits.insert(r.logits.end(), lrow, lrow + vocab);
                    ++r.logit_rows;
                }
                token = sample(s, lrow);
            }
            ++row;
            EngineResult& res = results_[s.id];
            const std::vector<uint32_t>& stops = model_.spec().stop_ids;
            if (!s.req.ignore_stop_tokens && std::find(stops.begin(), stops.end(), token) != stops.end()) {
                s.phase = Phase::Finished;
                res.finish_reason = "stop";
                v.finished = true;
                continue;
            }
            bool reaches_budget = s.generated + 1 == s.req.max_new_tokens;
            ++s.generated;
            s.history.push_back(token);
            res.tokens.push_back(token);
            ++s.pending_events;   // EngineEvent::Text with its token evidence (engine.rs:2459-2470)
            if (reaches_budget) {
                s.phase = Phase::Finished;
                res.finish_reason = "length";
                v.finished = true;
                continue;
            }
            s.phase = Phase::Decode;
            s.decode_token = token;
        }
    } else {
        reservation.reset();
        forward_needs_drain_ = false;
    }

    // ---- finalize_visits (engine.rs:2525-2614)
    for (int i = 0; i < visits; ++i) {
        Visit& v = actions[(size_t)i];
        Sequence& s = *active_[(size_t)i];
        if (v.kind == Visit::Complete) {
            if (v.finished) {  // apply_slot_step with final metrics (engine.rs:2618-2671)
                EngineResult& res = results_[s.id];
                if (res.state == FinishState::Running) {
                    res.state = FinishState::Done;
                    if (res.finish_reason.empty()) res.finish_reason = "length";
                    ++stats_.completed;
                    ++s.pending_events;   // EngineEvent::Finished (engine.rs:2663-2669)
                }
                reclaim(s);
                s.delivering = true;
            }
            v.kind = Visit::Keep;
        }
    }
    for (int i = 0; i < visits; ++i) {
        Visit& v = actions[(size_t)i];
        Sequence& s = *active_[(size_t)i];
        if (v.kind == Visit::Remove) continue;
        // the flush after the batch (engine.rs:2559-2580): a finished slot leaves once its last event is in the channel; one
        // whose channel timed out leaves now if its session is already back, else at its next visit
        const Flush final_flush = flush_pending(s, now_ms);
        if (final_flush == Flush::Drained && s.delivering) { reclaim(s); v.kind = Visit::Remove; }
        else if (final_flush == Flush::Abandoned) v.kind = s.reclaimed ? Visit::Remove : Visit::Keep;
    }
    for (int i = 0; i < visits; ++i) {
        std::unique_ptr<Sequence> slot = std::move(active_.front());
        active_.pop_front();
        if (actions[(size_t)i].kind == Visit::Remove) {
            if (!slot->reclaimed) throw std::runtime_error("removed slot has no reclaimed session");
            sessions_.push_back(std::move(slot->reclaimed));
        } else {
            active_.push_back(std::move(slot));
        }
    }
    round_visits_remaining_ -= visits;
    round_budget_remaining_ -= input_tokens;
    if (active_.empty()) {
        round_visits_remaining_ = 0;
        round_budget_remaining_ = 0;
    }
    forget_settled_cancellations();
    return lane_count;
}

void Engine::run() {
    int idle = 0;
    while (pending() > 0 && !poisoned_) {
        int lanes = step();
        if (lanes == 0 && blocked_last_tick_ > 0) {
            // every runnable slot waits for its channel: the wait ends by the host taking events or by the send timeout, so
            // this is time passing, not a scheduler that makes no progress
            std::this_thread::sleep_for(std::chrono::microseconds(200));
            continue;
        }
        idle = lanes > 0 ? 0 : idle + 1;
        if (idle > 4 * (cfg_.max_active_sequences + 4)) throw std::runtime_error("scheduler made no progress");
    }
}

}  // namespace mk
