// The model/session/KV-reservation boundary the scheduler talks to, shaped like the reference's
// CausalLm / CausalLmSession / CausalLmKvReservation traits (src/architecture.rs:803-1246), with the
// shared host-side glue of the reference's DecoderModel: sessions over one paged KV pool, the
// exact-token prefix cache (src/decoder.rs:3392-3431,3494-3603) and transactional reservations
// (src/decoder.rs:3696-3758,4125-4201).  Device work is supplied by the subclass.
#pragma once
#include "kv_pool.h"
#include "prefix_cache.h"
#include <memory>
#include <optional>
#include <string>
#include <vector>

namespace mk {

class PagedLm;

struct LmSession {
    PagedLm* owner = nullptr;
    std::unique_ptr<KvTable> table;
    int64_t logical_len = 0;
};

struct LmLane {
    LmSession* session = nullptr;
    const uint32_t* ids = nullptr;
    int32_t n_tokens = 0;
    int32_t start_pos = 0;
    // how FWD_WANT_TOKENS picks this lane's token: temperature <= 0 = first-index argmax; otherwise temperature /
    // top-k / top-p with the uniform draw u supplied by the caller (see LaneSampling in kernels.h)
    float temperature = 0.f;
    int32_t top_k = 0;
    float top_p = 1.f;
    float u = 0.f;
};

struct LmReservation {
    PagedLm* owner = nullptr;
    std::vector<LmSession*> sessions;
    std::vector<int32_t> start_pos, n_tokens;
    std::unique_ptr<KvReservation> paged;
};

struct LmRuntimeSpec {
    int vocab = 0, max_context = 0, layers = 0, hidden = 0;
    std::vector<uint32_t> stop_ids;
    int64_t weight_bytes = 0, weight_bytes_per_token = 0, kv_bytes_per_token = 0;
};

struct LmPrefixDiagnostics {
    int64_t entries = 0, cached_blocks = 0, capacity_blocks = 0, hits = 0, misses = 0, matched_tokens = 0, insertions = 0,
            evictions = 0;
};

constexpr uint32_t FWD_WANT_LOGITS = 1u, FWD_WANT_TOKENS = 2u;

class PagedLm {
public:
    virtual ~PagedLm() = default;

    const LmRuntimeSpec& spec() const { return spec_; }
    KvPool& pool() { return *pool_; }

    // CausalLm::new_session
    std::unique_ptr<LmSession> new_session();
    // A new session sharing the first logical_len tokens of s (PagedKvBlockTable::fork_prefix, cache.rs:1565-1571).
    std::unique_ptr<LmSession> fork_session_prefix(LmSession& s, int64_t logical_len);
    // CausalLm::reset_session_for_prompt: clears the session, then attaches the longest cached
    // block-aligned prefix strictly shorter than the prompt.  Returns the cached token count.
    int64_t reset_session_for_prompt(LmSession& s, const uint32_t* tokens, size_t n);
    // CausalLm::publish_prompt_prefix: best effort, never fails the request.
    void publish_prompt_prefix(LmSession& s, const uint32_t* tokens, size_t n);
    // CausalLmSession::clear_cache
    void clear_session(LmSession& s);
    // CausalLm::reserve_batch_kv: host only.  Throws KvPoolExhausted after evicting every prefix
    // snapshot that could have relieved the pressure.
    std::unique_ptr<LmReservation> reserve_batch(const std::vector<LmLane>& lanes);
    // CausalLm::forward_batch_tokens_reserved: validates every lane before any mutation, consumes the
    // reservation, enqueues the tick and commits the block tables.
    void forward_batch_reserved(const std::vector<LmLane>& lanes, std::unique_ptr<LmReservation> reservation, uint32_t flags);
    // CausalLm::read_output_to_cpu: completion barrier; retired pages become free.
    void read_output(float* logits, uint32_t* tokens);
    // CausalLm::synchronize
    void synchronize();

    KvPoolStats pool_stats() const { return pool_->stats(); }
    std::optional<LmPrefixDiagnostics> prefix_diagnostics() const;
    int last_lanes() const { return last_lanes_; }
    // Whether FWD_WANT_TOKENS can pick a token with these settings on the device (else the caller reads logits back).
    virtual bool device_sampling_covers(float temperature, int top_k) const { return !(temperature > 0.f) && top_k >= 0; }
    virtual float last_forward_ms() const { return 0.f; }
    virtual int64_t launch_count() const { return 0; }
    // Host<->device bytes moved by forwards since load.
    virtual int64_t h2d_bytes() const { return 0; }
    virtual int64_t d2h_bytes() const { return 0; }
    // Per-kernel-class device timing (CUDA events on the launching stream); off by default.
    struct KernelProfile {
        std::string name;
        int64_t launches = 0;
        double ms = 0, bytes = 0, flops = 0;
    };
    virtual void profile_enable(bool) {}
    virtual std::vector<KernelProfile> profile_query() { return {}; }
    void validate_session(const LmSession& s) const;

protected:
    void init_pool(int block_tokens, int slab_blocks, int64_t capacity_tokens, int64_t prefix_capacity_tokens, bool allow_prefix_cache);
    // Enqueue the device work of one tick.  `r` holds the provisional block tables of every lane.
    virtual void run_forward(const std::vector<LmLane>& lanes, KvReservation& r, uint32_t flags) = 0;
    // Wait for the tick and copy the requested outputs to the host.
    virtual void fetch_output(float* logits, uint32_t* tokens) = 0;
    virtual void device_synchronize() {}
    virtual void on_reset_session() {}  // test hook: the fake model injects admission failures here
    virtual void on_clear_session() {}  // test hook: the fake model injects session-clearing failures here

    LmRuntimeSpec spec_;
    std::shared_ptr<KvPool> pool_;
    using Snapshot = std::unique_ptr<KvTable>;
    std::unique_ptr<TokenPrefixCache<Snapshot>> prefix_cache_;
    int last_lanes_ = 0;
    uint32_t last_flags_ = 0;
    bool forward_unread_ = false;  // a forward was enqueued and neither read_output nor synchronize has run since
};

// Host-only model with deterministic one-hot logits, used to exercise the scheduler, the KV pool and
// the prefix cache without a GPU (the role of FakeModel in the reference's tests,
// src/engine.rs:3107-3300).  The next token after feeding token t at position p is
// (31 * t + 7 * p + 3) mod vocab.
class FakeLm : public PagedLm {
public:
    FakeLm(int vocab, int max_context, int block_tokens, int slab_blocks, int64_t capacity_tokens, int64_t prefix_capacity_tokens);
    // Fail the forward numbered `index` (0-based) with an exception, to test rollback.
    void fail_forward_at(int64_t index) { fail_at_ = index; }
    // The same for the completion barrier (site 1), prompt admission (site 2), the cleanup drain (site 3) and the clearing
    // of a session (site 4; panic_clear_session, src/engine.rs:5640-5682), like
    // fail_completion_barrier_at and friends of the reference's FakeModel (src/engine.rs:3107-3300).
    void inject_failure(int site, int64_t index);
    int64_t drains() const { return drains_; }
    // Stop token ids of the runtime spec, and (n_logits > 0) one logits row that every lane of every forward returns instead
    // of the one-hot row - FakeModel::with_logits of the reference's generation tests (src/generation.rs:1633-1640).
    void script(const uint32_t* stop_ids, int n_stop, const float* logits_row, int n_logits);
    // A made-up, exactly representable duration (0.25 ms + tokens / 1024 ms) so that time buckets can be checked.
    float last_forward_ms() const override { return 0.25f + (float)last_tokens_ / 1024.f; }
    // Calls cb(user) once, inside the next completion barrier: the place where the reference's FakeModel flips
    // cancel_on_completion_barrier (src/engine.rs:3143,3575-3583), i.e. "the client gave up while the forward ran".
    void on_next_barrier(void (*cb)(void*), void* user) { barrier_cb_ = cb; barrier_user_ = user; }

protected:
    void run_forward(const std::vector<LmLane>& lanes, KvReservation& r, uint32_t flags) override;
    void fetch_output(float* logits, uint32_t* tokens) override;
    void device_synchronize() override;
    void on_reset_session() override;
    void on_clear_session() override;

private:
    std::vector<uint32_t> next_;
    std::vector<float> fixed_row_;
    int64_t forwards_ = 0, fail_at_ = -1, last_tokens_ = 0;
    void (*barrier_cb_)(void*) = nullptr;
    void* barrier_user_ = nullptr;
    int64_t reads_ = 0, fail_read_at_ = -1, resets_ = 0, fail_reset_at_ = -1, drains_ = 0, fail_drain_at_ = -1, clears_ = 0, fail_clear_at_ = -1;
};

}  // namespace mk
