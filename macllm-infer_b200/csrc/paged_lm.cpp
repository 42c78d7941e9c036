// See paged_lm.h.  Line references are into the reference's src/decoder.rs unless noted.
#include "paged_lm.h"
#include <algorithm>

namespace mk {

void PagedLm::init_pool(int block_tokens, int slab_blocks, int64_t capacity_tokens, int64_t prefix_capacity_tokens,
                        bool allow_prefix_cache) {
    if (block_tokens <= 0 || slab_blocks <= 0 || capacity_tokens <= 0)
        throw std::runtime_error("KV pool configuration must be positive");
    int64_t max_blocks = (capacity_tokens + block_tokens - 1) / block_tokens;  // src/runtime.rs:194
    pool_ = std::make_shared<KvPool>(block_tokens, slab_blocks, max_blocks);
    if (prefix_capacity_tokens > 0) {
        if (!allow_prefix_cache)  // :4352-4372: rejected for models with a sliding-window layer
            throw std::runtime_error("the automatic prefix cache is not supported for models with sliding-window layers");
        int64_t budget = std::min((prefix_capacity_tokens + block_tokens - 1) / block_tokens, max_blocks);  // :3403-3412
        prefix_cache_ = std::make_unique<TokenPrefixCache<Snapshot>>((size_t)block_tokens, (size_t)budget);
    }
}

std::unique_ptr<LmSession> PagedLm::new_session() {  // :3433-3477
    auto s = std::make_unique<LmSession>();
    s->owner = this;
    s->table = std::make_unique<KvTable>(pool_, spec_.max_context);
    return s;
}

std::unique_ptr<LmSession> PagedLm::fork_session_prefix(LmSession& s, int64_t logical_len) {
    validate_session(s);
    if (s.table->logical_len() != s.logical_len) throw std::runtime_error("decoder session block table disagrees with its sequence length");
    auto f = std::make_unique<LmSession>();
    f->owner = this;
    f->table = s.table->fork_prefix(logical_len);
    f->logical_len = logical_len;
    return f;
}

void PagedLm::validate_session(const LmSession& s) const {  // :3479-3492
    if (s.owner != this) throw std::runtime_error("decoder session belongs to a different model instance");
}

void PagedLm::clear_session(LmSession& s) {  // :3804-3818
    on_clear_session();
    int64_t old_len = s.table->logical_len();
    s.table->clear();
    if (old_len != 0 && s.table->logical_len() != 0) return;  // a reservation keeps the table locked
    s.logical_len = 0;
}

int64_t PagedLm::reset_session_for_prompt(LmSession& s, const uint32_t* tokens, size_t n) {  // :3494-3532
    validate_session(s);
    on_reset_session();
    clear_session(s);
    if (s.logical_len != 0 || s.table->logical_len() != 0)
        throw std::runtime_error("decoder session did not become empty before prompt admission");
    if (!prefix_cache_) return 0;
    auto hit = prefix_cache_->lookup_aligned_common_prefix(tokens, n, n);
    if (!hit) return 0;
    s.table->attach_prefix(**hit->snapshot, (int64_t)hit->matched_tokens);  // restore_into
    s.logical_len = (int64_t)hit->matched_tokens;
    return s.logical_len;
}

void PagedLm::publish_prompt_prefix(LmSession& s, const uint32_t* tokens, size_t n) {  // :3534-3603
    if (!prefix_cache_ || s.owner != this) return;
    size_t bt = prefix_cache_->block_tokens();
    size_t snapshot_tokens = n / bt * bt;
    if (snapshot_tokens == 0 || (size_t)s.logical_len < snapshot_tokens) return;
    Snapshot fork;
    try {
        fork = s.table->fork_prefix((int64_t)snapshot_tokens);
    } catch (...) {
        return;
    }
    size_t cost = std::max<size_t>((size_t)fork->owned_blocks(), 1);
    std::vector<uint32_t> key(tokens, tokens + snapshot_tokens);
    prefix_cache_->insert(std::move(key), std::move(fork), cost);
}

std::optional<LmPrefixDiagnostics> PagedLm::prefix_diagnostics() const {  // :3605-3632
    if (!prefix_cache_) return std::nullopt;
    PrefixCacheStats st = prefix_cache_->stats();
    LmPrefixDiagnostics d;
    d.entries = (int64_t)st.entries;
    d.cached_blocks = (int64_t)st.cost;
    d.capacity_blocks = (int64_t)st.max_cost;
    d.hits = (int64_t)st.hits;
    d.misses = (int64_t)st.misses;
    d.matched_tokens = (int64_t)st.matched_tokens;
    d.insertions = (int64_t)st.insertions;
    d.evictions = (int64_t)st.evictions;
    return d;
}

std::unique_ptr<LmReservation> PagedLm::reserve_batch(const std::vector<LmLane>& lanes) {  // :3696-3758
    if (lanes.empty()) throw std::runtime_error("paged KV reservation batch cannot be empty");
    std::vector<KvTable*> tables;
    std::vector<int64_t> counts;
    auto r = std::make_unique<LmReservation>();
    r->owner = this;
    for (const LmLane& l : lanes) {
        if (l.session == nullptr) throw std::runtime_error("reservation lane has no session");
        validate_session(*l.session);
        if (l.n_tokens <= 0) throw std::runtime_error("input sequence cannot be empty");  // validate_session_geometry :3878-3899
        if (l.session->logical_len != l.start_pos)
            throw std::runtime_error("start_pos " + std::to_string(l.start_pos) + " does not match decoder sequence length " +
                                     std::to_string(l.session->logical_len));
        if (l.session->table->logical_len() != l.session->logical_len)
            throw std::runtime_error("decoder session block table disagrees with its sequence length");
        tables.push_back(l.session->table.get());
        counts.push_back(l.n_tokens);
        r->sessions.push_back(l.session);
        r->start_pos.push_back(l.start_pos);
        r->n_tokens.push_back(l.n_tokens);
    }
    for (;;) {
        try {
            r->paged = pool_->reserve_batch(tables, counts);
            break;
        } catch (const KvPoolExhausted& e) {
            if (prefix_cache_ && prefix_cache_->evict_lru()) continue;  // dropping the evicted snapshot releases its pages
            // classify_reservation_error (src/decoder.rs:3970-3994): what the scheduler is told is the pool's state now
            const KvPoolStats st = pool_->stats();
            const int64_t free_now = st.free_blocks + (st.max_blocks - st.allocated_blocks);
            throw KvPoolExhausted(e.requested, e.free_blocks, e.unallocated,
                                  "KV cache requires " + std::to_string(e.requested) + " additional blocks, but only " + std::to_string(free_now) +
                                      " of " + std::to_string(st.max_blocks) + " are free (" + std::to_string(st.retired_blocks) + " retired, " +
                                      std::to_string(st.block_tokens) + " tokens/block)");
        }
    }
    return r;
}

void PagedLm::forward_batch_reserved(const std::vector<LmLane>& lanes, std::unique_ptr<LmReservation> reservation,
                                     uint32_t flags) {  // :4203-4269, :4125-4201
    if (lanes.empty()) throw std::runtime_error("mixed-sequence batch cannot be empty");
    // one tick in flight: the staging buffers and the output buffer of a tick are reused by the next one
    if (forward_unread_)
        throw std::runtime_error("previous forward was not read: call read_output or synchronize before the next forward");
    if (!reservation || reservation->owner != this || !reservation->paged)
        throw std::runtime_error("forward needs a KV reservation made by this model");
    if (reservation->sessions.size() != lanes.size())
        throw std::runtime_error("KV reservation covers " + std::to_string(reservation->sessions.size()) + " lanes, forward has " +
                                 std::to_string(lanes.size()));
    for (size_t i = 0; i < lanes.size(); ++i) {
        const LmLane& l = lanes[i];
        if (l.session == nullptr || l.ids == nullptr) throw std::runtime_error("forward lane is missing its session or tokens");
        validate_session(*l.session);
        if (l.n_tokens <= 0) throw std::runtime_error("input sequence cannot be empty");
        for (int t = 0; t < l.n_tokens; ++t)
            if ((int64_t)l.ids[t] >= spec_.vocab) throw std::runtime_error("input contains a token ID outside the model vocabulary");
        if (l.session->logical_len != l.start_pos)
            throw std::runtime_error("start_pos " + std::to_string(l.start_pos) + " does not match decoder sequence length " +
                                     std::to_string(l.session->logical_len));
        if (reservation->sessions[i] != l.session || reservation->start_pos[i] != l.start_pos ||
            reservation->n_tokens[i] != l.n_tokens)
            throw std::runtime_error("paged KV reservation lane " + std::to_string(i) +
                                     " does not match session, order, start or token count");  // src/decoder.rs:4076-4090
    }
    KvReservation& paged = *reservation->paged;
    paged.mark_all_used();
    run_forward(lanes, paged, flags);  // a throw leaves every session untouched; the reservation rolls back
    forward_unread_ = true;
    paged.commit();
    for (const LmLane& l : lanes) l.session->logical_len = (int64_t)l.start_pos + l.n_tokens;
    last_lanes_ = (int)lanes.size();
    last_flags_ = flags;
}

void PagedLm::read_output(float* logits, uint32_t* tokens) {  // :3779-3783
    if (!forward_unread_) throw std::runtime_error("no forward is waiting to be read");
    forward_unread_ = false;  // a failed barrier is not retried (src/engine.rs:2388-2391)
    fetch_output(logits, tokens);
    pool_->mark_completed_through(pool_->submitted_epoch());
}

void PagedLm::synchronize() {  // :3785-3788
    forward_unread_ = false;
    device_synchronize();
    pool_->mark_completed_through(pool_->submitted_epoch());
}

// ---------------------------------------------------------------------------- FakeLm

FakeLm::FakeLm(int vocab, int max_context, int block_tokens, int slab_blocks, int64_t capacity_tokens,
               int64_t prefix_capacity_tokens) {
    spec_.vocab = vocab;
    spec_.max_context = max_context;
    spec_.layers = 1;
    spec_.hidden = 1;
    init_pool(block_tokens, slab_blocks, capacity_tokens, prefix_capacity_tokens, true);
}

void FakeLm::run_forward(const std::vector<LmLane>& lanes, KvReservation&, uint32_t) {
    if (forwards_++ == fail_at_) throw std::runtime_error("injected forward failure");
    next_.clear();
    last_tokens_ = 0;
    for (const LmLane& l : lanes) {
        last_tokens_ += l.n_tokens;
        uint64_t t = l.ids[l.n_tokens - 1];
        uint64_t p = (uint64_t)(l.start_pos + l.n_tokens - 1);
        next_.push_back((uint32_t)((31 * t + 7 * p + 3) % (uint64_t)spec_.vocab));
    }
}

void FakeLm::script(const uint32_t* stop_ids, int n_stop, const float* logits_row, int n_logits) {
    if (n_logits > spec_.vocab) throw std::runtime_error("scripted logits row is wider than the vocabulary");
    spec_.stop_ids.assign(stop_ids, stop_ids + std::max(n_stop, 0));
    fixed_row_.assign((size_t)(n_logits > 0 ? spec_.vocab : 0), 0.f);
    for (int i = 0; i < n_logits; ++i) fixed_row_[(size_t)i] = logits_row[i];
}

void FakeLm::inject_failure(int site, int64_t index) {
    switch (site) {
        case 0: fail_at_ = index; break;
        case 1: fail_read_at_ = index; break;
        case 2: fail_reset_at_ = index; break;
        case 3: fail_drain_at_ = index; break;
        case 4: fail_clear_at_ = clears_ + index; break;   // counted from now: admissions clear sessions too
        default: throw std::runtime_error("unknown failure site");
    }
}

void FakeLm::device_synchronize() {
    if (drains_++ == fail_drain_at_) throw std::runtime_error("injected synchronize failure");
}

void FakeLm::on_clear_session() {
    if (clears_++ == fail_clear_at_) throw std::runtime_error("injected session clearing failure");
}

void FakeLm::on_reset_session() {
    if (resets_++ == fail_reset_at_) throw std::runtime_error("injected admission failure");
}

void FakeLm::fetch_output(float* logits, uint32_t* tokens) {
    if (reads_++ == fail_read_at_) throw std::runtime_error("injected completion barrier failure");
    if (barrier_cb_ != nullptr) {
        void (*cb)(void*) = barrier_cb_;
        barrier_cb_ = nullptr;
        cb(barrier_user_);
    }
    for (size_t i = 0; i < next_.size(); ++i) {
        if (!fixed_row_.empty()) {  // scripted logits: the greedy token is the row's first maximum
            if (tokens) tokens[i] = (uint32_t)(std::max_element(fixed_row_.begin(), fixed_row_.end()) - fixed_row_.begin());
            if (logits) std::copy(fixed_row_.begin(), fixed_row_.end(), logits + i * (size_t)spec_.vocab);
            continue;
        }
        if (tokens) tokens[i] = next_[i];
        if (logits) {
            float* row = logits + i * (size_t)spec_.vocab;
            std::fill(row, row + spec_.vocab, 0.f);
            row[next_[i]] = 1.f;
        }
    }
}

}  // namespace mk
