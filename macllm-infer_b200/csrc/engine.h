// The continuous-batching engine: FIFO admission (with atomic batches), the round-robin scheduler
// tick with its token budget and prefill quantum, KV-pressure batch shrinking, and the per-sequence
// prefill/decode phase machine.  Restates ServingScheduler (src/engine.rs:1578-2770) and
// GenerationCore (src/generation.rs:787-1266) of the reference, minus the HTTP-facing event plumbing:
// results are collected per request instead of streamed.
#pragma once
#include "paged_lm.h"
#include <atomic>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <vector>

namespace mk {

struct EngineConfig {  // src/engine.rs:309-384
    int max_active_sequences = 2;
    int scheduler_token_budget = 256;
    int prefill_token_quantum = 128;
    int queue_capacity = 8;
    bool record_logits = false;
    bool host_sampling = false;
};

struct EngineRequest {
    std::vector<uint32_t> prompt;
    int max_new_tokens = 0;
    bool ignore_stop_tokens = false;
    float temperature = 0.f;
    int top_k = 0;
    float top_p = 1.f;
    float repetition_penalty = 1.f, presence_penalty = 0.f, frequency_penalty = 0.f;
    uint64_t seed = 0;
    bool publish_prompt_prefix = true;
    // The request's event channel (src/engine.rs:755-767, mpsc::channel(event_capacity)): at most `event_capacity` events - one
    // per token, one for the terminal outcome - may wait for the host to take them (Engine::consume_events); a request whose
    // channel stays full pauses, and one that stays full for `event_send_timeout_ms` is given up.  0 = no bound.
    int event_capacity = 0;
    double event_send_timeout_ms = 0.0;
};

// Cancelled: the caller gave the request up (EngineTicket::cancel / a closed event channel, src/engine.rs:1136-1145); the
// scheduler answers nothing more for it, the tokens produced so far stay readable
enum class FinishState : int { Running = 0, Done = 1, Failed = 2, Cancelled = 3 };
// EngineFailureKind (src/engine.rs:268-273)
enum class FailureKind : int { None = 0, InvalidRequest = 1, ResourceExhausted = 2, Internal = 3, Fatal = 4 };
// EngineStatus (src/engine.rs:281-288); this engine is driven by its caller's thread, so Starting never shows
enum class EngineStatus : int { Starting = 0, Ready = 1, Busy = 2, Poisoned = 3, Stopped = 4 };

struct EngineResult {
    std::vector<uint32_t> tokens;
    FinishState state = FinishState::Running;
    std::string message;        // failure message
    FailureKind kind = FailureKind::None;
    std::string finish_reason;  // "length", "stop", "cancelled"
    int64_t cached_tokens = 0;
    std::vector<float> logits;  // record_logits: one row per sampled position
    int logit_rows = 0;
    // GenerationMetrics (src/generation.rs:35-58), the model-side part: every packed forward the sequence joined adds its
    // whole device time to the sequence's bucket for the phase its lane was in (src/generation.rs:1185-1199)
    int prompt_tokens = 0, decode_steps = 0;
    double suffix_prefill_ms = 0.0, first_token_ms = 0.0, decode_ms = 0.0;
};

// Whole-forward classification of the reference's benchmark traces (BenchmarkForwardKind, src/engine.rs:430-439): a lane is
// a prefill chunk that ends inside the prompt (SuffixPrefill), the chunk that ends the prompt and samples (FirstToken) or
// a decode step (src/generation.rs:757-766); a packed forward whose lanes differ is Mixed, and its time goes to that
// bucket alone.
enum class ForwardKind : int32_t { SuffixPrefill = 0, FirstToken = 1, Decode = 2, Mixed = 3 };

struct TickLaneTrace {
    int32_t request_id, start_pos, n_tokens;
    int32_t phase;  // ForwardKind of the lane, never Mixed
};

struct TickInfo {  // BenchmarkPackedForwardRecord (src/engine.rs:452-460)
    ForwardKind kind = ForwardKind::Mixed;
    int lane_count = 0, input_tokens = 0;
    double model_ms = 0.0;
};

// EngineBatchTrace (src/engine.rs:462-484) of one atomic batch, minus the host-side wall-clock splits of admission.
struct BatchTrace {
    std::vector<int> members;
    int admitted_members = 0, rejected_members = 0, admission_active_sequences = 0;
    bool admission_complete = false;
    double suffix_prefill_ms = 0.0, first_token_ms = 0.0, decode_ms = 0.0, mixed_ms = 0.0;
    std::vector<int64_t> packed_forwards;  // tick numbers of the forwards that carried at least one member
};

struct EngineStats {
    int64_t ticks = 0, prefill_tokens = 0, decode_tokens = 0, completed = 0, failed = 0, kv_shrinks = 0, cleanup_drains = 0, device_sampled = 0, cancelled = 0;
    double device_ms = 0.0;
    // device time by whole-forward kind: every forward's time is in exactly one bucket (src/engine.rs:601-619)
    double suffix_prefill_ms = 0.0, first_token_ms = 0.0, decode_ms = 0.0, mixed_ms = 0.0;
};

class Engine {
public:
    Engine(PagedLm& model, const EngineConfig& cfg);
    ~Engine();

    // EngineHandle::submit / submit_batch: returns request ids.  An atomic batch is admitted only when
    // every member fits into the active set at once.  Throws when the queue is full.
    std::vector<int> submit(const std::vector<EngineRequest>& reqs, bool atomic_batch);
    // One turn of ServingScheduler::run (src/engine.rs:1577-1647): admission and drive_once.  Returns the number of
    // lanes of the packed forward (0 when none ran).  Any error that escapes the tick poisons the engine: every active,
    // pending and queued request fails with kind Fatal, the sessions are dropped, later submissions are refused.
    int step();
    // The same with the caller's clock (drive_once(now), src/engine.rs:1938): `now_ms` is what back-pressure timeouts are
    // measured against, for this tick's flush before the forward and the one after it alike.
    int step_at(double now_ms);
    // The host took `n` events of the request out of its channel (the receiver side of src/engine.rs:1420-1447).
    void consume_events(int id, int n);
    // EngineTicket::cancel (src/engine.rs:1136-1145): a sticky flag the scheduler reads - a queued request is skipped
    // before any validation or model work, an active one leaves at its next visit (its pages are back before the peers'
    // forward), one cancelled while its forward ran drops its row after the completion barrier.  The one entry that may be
    // called from another thread while step() runs.
    void cancel(int id);
    EngineStatus status() const { return poisoned_ ? EngineStatus::Poisoned : (pending() > 0 ? EngineStatus::Busy : EngineStatus::Ready); }
    const std::string& poison_message() const { return poison_message_; }
    void run();
    int pending() const { return (int)(queue_.size() + pending_atomic_.size() + active_.size()); }
    const EngineResult& result(int id) const;
    const std::vector<std::vector<TickLaneTrace>>& trace() const { return trace_; }
    const TickInfo& tick_info(int64_t tick) const;
    // A long-lived host (a server) turns the per-tick records off - the reference captures them only for benchmark
    // submissions (capture_benchmark_trace, src/engine.rs:1037-1053) - and releases each request once it has read the result.
    void keep_trace(bool keep);
    void release_request(int id);
    // The trace of the atomic batch `member_id` was submitted in; *terminal receives how many of its members have ended
    // (done, failed, rejected or cancelled).  The trace is complete once admission ran and every member is terminal.
    const BatchTrace& batch_trace(int member_id, int* terminal) const;
    const EngineStats& stats() const { return stats_; }

private:
    enum class Phase { Prefill, Decode, Finished, Failed };
    struct Job {
        int id;
        EngineRequest req;
        int batch = -1;       // atomic batch id
        int batch_size = 0;
    };
    struct Sequence {
        int id = 0;
        EngineRequest req;
        std::unique_ptr<LmSession> session;
        std::unique_ptr<LmSession> reclaimed;
        std::vector<uint32_t> history;
        int prompt_tokens = 0;
        int batch = -1;
        Phase phase = Phase::Prefill;
        int cursor = 0;
        uint32_t decode_token = 0;
        int generated = 0;
        bool delivering = false;
        uint64_t rng = 0;
        int pending_events = 0;      // produced, not yet in the channel (ActiveSequence::pending)
        int in_channel = 0;          // in the channel, not yet taken by the host
        double blocked_since = -1.0; // when the channel was first found full for the event now waiting; < 0: not blocked
    };
    struct Visit {
        enum Kind { Keep, Remove, Preview, Forward, Complete } kind = Keep;
        int start_pos = 0, n_tokens = 0;
        bool ready_to_sample = false;
        bool was_prefill = false;
        bool finished = false;  // Complete: the step carried final metrics
    };

    bool try_admit_available();
    bool admit_pending_atomic();
    void admit(Job job);
    enum class Flush { Drained, Blocked, Abandoned };
    Flush flush_pending(Sequence& s, double now_ms);
    int drive_once(double now_ms);
    void poison(std::string message);
    void fail_request(int id, const std::string& message, FailureKind kind = FailureKind::InvalidRequest);
    void reclaim(Sequence& s);
    bool is_cancelled(int id);
    void finish_cancelled(int id);
    void forget_settled_cancellations();
    uint32_t sample(Sequence& s, float* row);

    PagedLm& model_;
    EngineConfig cfg_;
    std::deque<Job> queue_;
    std::vector<Job> pending_atomic_;
    std::deque<std::unique_ptr<Sequence>> active_;
    std::vector<std::unique_ptr<LmSession>> sessions_;
    std::map<int, EngineResult> results_;
    std::vector<std::vector<TickLaneTrace>> trace_;
    std::vector<TickInfo> tick_info_;
    std::vector<BatchTrace> batches_;       // indexed by atomic batch id
    std::map<int, int> batch_of_request_;
    EngineStats stats_;
    std::atomic<int> next_id_{0};
    int next_batch_ = 0;
    int round_visits_remaining_ = 0, round_budget_remaining_ = 0;
    std::vector<float> logits_host_;
    std::vector<uint32_t> tokens_host_;
    bool poisoned_ = false;
    bool keep_trace_ = true;
    int blocked_last_tick_ = 0;   // slots found waiting for their event channel in the last tick
    int orphan_ = -1;                   // request whose admission threw
    bool forward_needs_drain_ = false;  // a reservation or forward was submitted and no completion barrier ran yet
    std::string poison_message_;
    std::atomic<bool> any_cancelled_{false};
    std::mutex cancel_mu_;
    std::set<int> cancelled_;  // sticky: ids stay until the request's result is final
};

}  // namespace mk
