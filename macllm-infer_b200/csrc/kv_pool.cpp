// See kv_pool.h.  Line references are into crates/macllm-kv/src/cache.rs of the reference.
#include "kv_pool.h"
#include <algorithm>

namespace mk {

namespace {
struct KvInvalid : std::runtime_error {
    using std::runtime_error::runtime_error;
};
inline int64_t div_ceil(int64_t a, int64_t b) { return (a + b - 1) / b; }
}  // namespace

KvPool::KvPool(int block_tokens, int slab_blocks, int64_t max_blocks)
    : block_tokens_(block_tokens), slab_blocks_(slab_blocks), max_blocks_(max_blocks) {
    // PagedKvPoolConfig::new (:126-147) with the display form of InvalidConfig (:67)
    if (block_tokens <= 0) throw KvInvalid("invalid paged KV config: block_tokens must be positive");
    if (slab_blocks <= 0) throw KvInvalid("invalid paged KV config: slab_blocks must be positive");
    if (max_blocks <= 0) throw KvInvalid("invalid paged KV config: max_blocks must be positive");
    if (max_blocks > (int64_t)UINT32_MAX) throw KvInvalid("invalid paged KV config: max_blocks exceeds the generational block-ID range");
    slots_.reserve((size_t)std::min<int64_t>(max_blocks, 1 << 20));
}

KvPoolStats KvPool::stats() const {  // :1321-1347
    KvPoolStats s;
    s.block_tokens = block_tokens_;
    s.slab_blocks = slab_blocks_;
    s.max_blocks = max_blocks_;
    s.allocated_blocks = (int64_t)slots_.size();
    s.free_blocks = free_blocks();
    s.reserved_blocks = reserved_;
    s.live_blocks = live_;
    s.live_references = live_refs_;
    s.shared_blocks = shared_;
    s.retired_blocks = retired_;
    s.slabs = slabs_;
    s.submitted_epoch = submitted_epoch_;
    s.completed_epoch = completed_epoch_;
    return s;
}

void KvPool::ensure_free_blocks(int64_t requested) {  // :649-715
    int64_t free_now = free_blocks();
    int64_t unallocated = max_blocks_ - (int64_t)slots_.size();
    if (requested > free_now + unallocated) throw KvPoolExhausted(requested, free_now, unallocated);
    int64_t missing = requested - free_now;
    if (missing <= 0) return;
    int64_t planned = 0;
    while (planned < missing) {
        int64_t remaining = max_blocks_ - (int64_t)slots_.size();
        int64_t blocks = std::min<int64_t>(slab_blocks_, remaining);
        if (blocks == 0) throw KvPoolExhausted(requested, free_now, unallocated);
        for (int64_t i = 0; i < blocks; ++i) {
            Slot s;
            s.last_use = completed_epoch_;
            slots_.push_back(s);
        }
        ++slabs_;
        planned += blocks;
    }
}

void KvPool::begin_transaction(uint64_t& transaction, uint64_t& epoch) {  // :717-733
    if (active_transaction_ != 0)
        throw KvInvalid("paged KV transaction " + std::to_string(active_transaction_) + " is still active");
    transaction = ++next_transaction_;
    active_transaction_ = transaction;
    epoch = ++submitted_epoch_;
}

std::vector<KvBlockId> KvPool::reserve_blocks(int64_t count, uint64_t transaction) {  // :735-809
    if (active_transaction_ != transaction) throw KvInvalid("transaction is not the active paged KV transaction");
    std::vector<KvBlockId> ids;
    if (count == 0) return ids;
    ensure_free_blocks(count);
    ids.reserve((size_t)count);
    // lowest-index free slots first
    for (size_t i = 0; i < slots_.size() && (int64_t)ids.size() < count; ++i)
        if (slots_[i].state == State::Free) ids.push_back(KvBlockId{(uint32_t)i, slots_[i].generation + 1});
    if ((int64_t)ids.size() != count) throw KvInvalid("reserved fewer free blocks than preflighted");
    for (const KvBlockId& id : ids) {
        Slot& s = slots_[id.slot];
        s.generation = id.generation;
        s.state = State::Reserved;
        s.transaction = transaction;
        s.last_use = completed_epoch_;
    }
    reserved_ += count;
    return ids;
}

const KvPool::Slot& KvPool::slot(const KvBlockId& id) const {  // :811-828
    if (id.slot >= slots_.size() || slots_[id.slot].generation != id.generation)
        throw KvInvalid("stale paged KV block id for slot " + std::to_string(id.slot));
    return slots_[id.slot];
}
KvPool::Slot& KvPool::slot_mut(const KvBlockId& id) { return const_cast<Slot&>(slot(id)); }

void KvPool::validate_owned(const KvBlockId& id, uint64_t transaction) const {  // :851-871
    const Slot& s = slot(id);
    bool ok = s.state == State::Live || (s.state == State::Reserved && transaction != 0 && s.transaction == transaction);
    if (!ok) throw KvInvalid("block " + std::to_string(id.slot) + " is not owned by the append transaction");
}

int64_t KvPool::live_references(const KvBlockId& id) const {  // :915-924
    const Slot& s = slot(id);
    if (s.state != State::Live) throw KvInvalid("block " + std::to_string(id.slot) + " is not live");
    return s.references;
}

void KvPool::retain_live(const std::vector<KvBlockId>& ids) {  // :929-983, all-or-nothing
    for (const KvBlockId& id : ids)
        if (slot(id).state != State::Live) throw KvInvalid("block " + std::to_string(id.slot) + " is not live");
    for (const KvBlockId& id : ids) {
        Slot& s = slots_[id.slot];
        if (s.references == 1) ++shared_;
        ++s.references;
    }
    live_refs_ += (int64_t)ids.size();
}

void KvPool::release_live(const std::vector<KvBlockId>& ids) {  // :987-1100, all-or-nothing
    std::vector<std::pair<uint32_t, int64_t>> plan;
    for (const KvBlockId& id : ids) {
        if (slot(id).state != State::Live) throw KvInvalid("block " + std::to_string(id.slot) + " is not live");
        plan.emplace_back(id.slot, 1);
    }
    std::sort(plan.begin(), plan.end());
    std::vector<std::pair<uint32_t, int64_t>> merged;
    for (auto& p : plan) {
        if (!merged.empty() && merged.back().first == p.first) merged.back().second += p.second;
        else merged.push_back(p);
    }
    for (auto& p : merged)
        if (slots_[p.first].references < p.second) throw KvInvalid("block has fewer references than the release requires");
    for (auto& p : merged) {
        Slot& s = slots_[p.first];
        int64_t remaining = s.references - p.second;
        live_refs_ -= p.second;
        if (s.references > 1 && remaining <= 1) --shared_;
        if (remaining == 0) {
            --live_;
            if (s.last_use <= completed_epoch_) {
                s.state = State::Free;
            } else {
                s.state = State::Retired;
                s.until = s.last_use;
                ++retired_;
            }
            s.references = 0;
        } else {
            s.references = remaining;
        }
    }
}

void KvPool::mark_use(const std::vector<KvBlockId>& ids, uint64_t transaction, uint64_t epoch) {  // :1127-1146
    if (active_transaction_ != transaction) throw KvInvalid("transaction is not the active paged KV transaction");
    for (const KvBlockId& id : ids) validate_owned(id, transaction);
    for (const KvBlockId& id : ids) {
        Slot& s = slots_[id.slot];
        s.last_use = std::max(s.last_use, epoch);
    }
}

void KvPool::commit_reserved_replacing(const std::vector<KvBlockId>& ids, const std::vector<KvBlockId>& superseded,
                                       uint64_t transaction) {  // :1152-1212
    if (active_transaction_ != transaction) throw KvInvalid("transaction is not the active paged KV transaction");
    for (const KvBlockId& id : ids) {
        const Slot& s = slot(id);
        if (s.state != State::Reserved || s.transaction != transaction)
            throw KvInvalid("block " + std::to_string(id.slot) + " is not reserved by this transaction");
    }
    for (const KvBlockId& id : superseded)
        if (slot(id).state != State::Live) throw KvInvalid("superseded block is not live");
    for (const KvBlockId& id : ids) {
        Slot& s = slots_[id.slot];
        s.state = State::Live;
        s.references = 1;
    }
    reserved_ -= (int64_t)ids.size();
    live_ += (int64_t)ids.size();
    live_refs_ += (int64_t)ids.size();
    release_live(superseded);
    active_transaction_ = 0;
}

void KvPool::rollback_reserved(const std::vector<KvBlockId>& ids, uint64_t transaction) {  // :1214-1276
    if (active_transaction_ != transaction) return;
    for (size_t i = 0; i < ids.size(); ++i) {
        const KvBlockId& id = ids[i];
        if (std::find(ids.begin(), ids.begin() + (long)i, id) != ids.begin() + (long)i) continue;
        if (id.slot >= slots_.size() || slots_[id.slot].generation != id.generation) continue;
        Slot& s = slots_[id.slot];
        if (s.state != State::Reserved || s.transaction != transaction) continue;
        --reserved_;
        if (s.last_use <= completed_epoch_) {
            s.state = State::Free;
        } else {
            s.state = State::Retired;
            s.until = s.last_use;
            ++retired_;
        }
    }
    active_transaction_ = 0;
}

void KvPool::mark_completed_through(uint64_t epoch) {  // :1278-1319
    if (active_transaction_ != 0) throw KvInvalid("cannot publish device completion while a paged KV transaction is active");
    if (epoch < completed_epoch_ || epoch > submitted_epoch_)
        throw KvInvalid("invalid completion epoch " + std::to_string(epoch));
    completed_epoch_ = epoch;
    for (Slot& s : slots_) {
        if (s.state == State::Retired && s.until <= epoch) {
            s.state = State::Free;
            --retired_;
        }
    }
}

// ---------------------------------------------------------------------------- tables

KvTable::KvTable(std::shared_ptr<KvPool> pool, int64_t limit) : pool_(std::move(pool)), limit_(limit) {
    if (limit <= 0) throw KvInvalid("sequence table limit must be positive");  // :1449-1454
}

KvTable::~KvTable() {  // Drop, :1855-1865
    try {
        pool_->release_live(blocks_);
    } catch (...) {
    }
}

void KvTable::attach_prefix(const KvTable& source, int64_t logical_len) {  // :1486-1563
    if (&source == this) throw KvInvalid("a paged KV table cannot attach itself as a prefix");
    if (source.pool_.get() != pool_.get()) throw KvInvalid("prefix source belongs to another paged KV pool");
    if (in_flight_ != 0 || !blocks_.empty() || logical_len_ != 0)
        throw KvInvalid("prefix destination must be a live, empty, unlocked table");
    if (source.in_flight_ != 0) throw KvInvalid("prefix source must be live and unlocked");
    if (logical_len > source.logical_len_) throw KvInvalid("prefix length exceeds source length");
    if (logical_len > limit_) throw KvInvalid("prefix length exceeds the context limit");
    int bt = pool_->block_tokens();
    if ((int64_t)source.blocks_.size() != div_ceil(source.logical_len_, bt))
        throw KvInvalid("prefix source block table disagrees with its logical length");
    for (const KvBlockId& id : source.blocks_) pool_->validate_owned(id, 0);
    int64_t prefix_blocks = div_ceil(logical_len, bt);
    std::vector<KvBlockId> prefix(source.blocks_.begin(), source.blocks_.begin() + prefix_blocks);
    pool_->retain_live(prefix);
    blocks_ = std::move(prefix);
    logical_len_ = logical_len;
}

std::unique_ptr<KvTable> KvTable::fork_prefix(int64_t logical_len) const {  // :1567-1571
    auto fork = std::make_unique<KvTable>(pool_, limit_);
    fork->attach_prefix(*this, logical_len);
    return fork;
}

bool KvTable::clear() {  // :1840-1852
    if (in_flight_ != 0) return false;
    try {
        pool_->release_live(blocks_);
    } catch (...) {
        return false;
    }
    blocks_.clear();
    logical_len_ = 0;
    return true;
}

// ---------------------------------------------------------------------------- reservations

std::unique_ptr<KvReservation> KvPool::reserve_batch(const std::vector<KvTable*>& tables,
                                                     const std::vector<int64_t>& new_tokens) {  // :2216-2445
    if (tables.empty()) throw KvInvalid("paged KV reservation batch cannot be empty");
    if (tables.size() != new_tokens.size()) throw KvInvalid("reservation lane arrays differ in length");
    if (active_transaction_ != 0)
        throw KvInvalid("paged KV transaction " + std::to_string(active_transaction_) + " is still active");
    std::unique_ptr<KvReservation> r(new KvReservation());
    r->pool_ = shared_from_this();
    int64_t total_reserved = 0;
    for (size_t i = 0; i < tables.size(); ++i) {  // prepare_batch_lanes
        KvTable* t = tables[i];
        if (t == nullptr || t->pool_.get() != this) throw KvInvalid("lane table belongs to another paged KV pool");
        if (t->in_flight_ != 0) throw KvInvalid("lane table is unavailable or already reserved");
        for (size_t j = 0; j < i; ++j)
            if (tables[j] == t) throw KvInvalid("lane " + std::to_string(i) + " duplicates an earlier table");
        if (new_tokens[i] <= 0) throw KvInvalid("lane append token count must be positive");
        for (const KvBlockId& id : t->blocks_) validate_owned(id, 0);
        if ((int64_t)t->blocks_.size() != div_ceil(t->logical_len_, block_tokens_))
            throw KvInvalid("lane block table disagrees with its logical length");
        KvReservation::Lane lane;
        lane.table = t;
        if (t->logical_len_ % block_tokens_ != 0) {
            KvBlockId source = t->blocks_.back();
            if (live_references(source) > 1) {
                lane.cow = true;
                lane.cow_index = t->blocks_.size() - 1;
                lane.cow_source = source;
                lane.cow_valid = (int32_t)(t->logical_len_ % block_tokens_);
            }
        }
        int64_t new_len = t->logical_len_ + new_tokens[i];
        if (new_len > t->limit_)
            throw KvInvalid("sequence of " + std::to_string(new_len) + " tokens exceeds the context limit " +
                            std::to_string(t->limit_));
        int64_t required = div_ceil(new_len, block_tokens_);
        lane.old_len = t->logical_len_;
        lane.new_len = new_len;
        lane.new_tokens = new_tokens[i];
        lane.growth_blocks = std::max<int64_t>(0, required - (int64_t)t->blocks_.size());
        lane.reserved_blocks = lane.growth_blocks + (lane.cow ? 1 : 0);
        lane.provisional = t->blocks_;
        total_reserved += lane.reserved_blocks;
        r->lanes_.push_back(std::move(lane));
    }
    ensure_free_blocks(total_reserved);  // Exhausted is raised before any epoch is published
    uint64_t transaction = 0, epoch = 0;
    begin_transaction(transaction, epoch);
    try {
        r->reserved_ = reserve_blocks(total_reserved, transaction);
    } catch (...) {
        rollback_reserved({}, transaction);
        throw;
    }
    r->transaction_ = transaction;
    r->epoch_ = epoch;
    size_t off = 0;
    for (KvReservation::Lane& lane : r->lanes_) {  // copy-on-write replacement first, then growth
        size_t growth_off = 0;
        if (lane.cow) {
            KvBlockId replacement = r->reserved_[off];
            lane.provisional[lane.cow_index] = replacement;
            r->superseded_.push_back(lane.cow_source);
            r->cows_.push_back(KvCowCopy{lane.cow_source.slot, replacement.slot, lane.cow_valid});
            growth_off = 1;
        }
        for (int64_t g = 0; g < lane.growth_blocks; ++g) lane.provisional.push_back(r->reserved_[off + growth_off + (size_t)g]);
        off += (size_t)lane.reserved_blocks;
    }
    for (KvReservation::Lane& lane : r->lanes_) lane.table->in_flight_ = transaction;
    return r;
}

KvReservation::~KvReservation() { rollback(); }

void KvReservation::mark_all_used() {  // build_attention_batch, :2768-2772 (and the writes of :3091-3127)
    std::vector<KvBlockId> ids;
    for (const Lane& l : lanes_) ids.insert(ids.end(), l.provisional.begin(), l.provisional.end());
    for (const KvCowCopy& c : cows_) (void)c;
    // copy-on-write sources are read by the page copy as well
    for (const KvBlockId& id : superseded_) ids.push_back(id);
    pool_->mark_use(ids, transaction_, epoch_);
}

void KvReservation::page_table(std::vector<uint32_t>& pages, std::vector<int32_t>& lane_offsets,
                               std::vector<int32_t>& lane_counts, std::vector<int32_t>& lane_lens) {  // :2707-2851
    pages.clear();
    lane_offsets.clear();
    lane_counts.clear();
    lane_lens.clear();
    std::vector<int32_t> remap((size_t)pool_->slabs_, -1);
    int32_t next = 0;
    int32_t rows = 0;
    for (const Lane& l : lanes_) {
        if ((int64_t)l.provisional.size() != div_ceil(l.new_len, pool_->block_tokens()))
            throw KvInvalid("provisional block table length disagrees with logical length");
        lane_offsets.push_back(rows);
        lane_counts.push_back((int32_t)l.provisional.size());
        lane_lens.push_back((int32_t)l.new_len);
        for (const KvBlockId& id : l.provisional) {
            pool_->validate_owned(id, transaction_);
            int slab = pool_->slab_of(id.slot);
            if (remap[(size_t)slab] < 0) remap[(size_t)slab] = next++;
            pages.push_back((uint32_t)remap[(size_t)slab]);
            pages.push_back((uint32_t)pool_->slab_offset_of(id.slot));
            ++rows;
        }
    }
    std::vector<KvBlockId> ids;
    for (const Lane& l : lanes_) ids.insert(ids.end(), l.provisional.begin(), l.provisional.end());
    pool_->mark_use(ids, transaction_, epoch_);
}

uint64_t KvReservation::commit() {  // :2947-2979
    if (finalized_) throw KvInvalid("paged KV reservation was already finalized");
    for (const Lane& l : lanes_) {
        if (l.table->in_flight_ != transaction_ || l.table->logical_len_ != l.old_len)
            throw KvInvalid("lane table changed after its reservation");
    }
    pool_->commit_reserved_replacing(reserved_, superseded_, transaction_);
    for (Lane& l : lanes_) {
        l.table->blocks_ = std::move(l.provisional);
        l.table->logical_len_ = l.new_len;
        l.table->in_flight_ = 0;
    }
    finalized_ = true;
    return epoch_;
}

void KvReservation::rollback() {  // :2985-2998
    if (finalized_) return;
    pool_->rollback_reserved(reserved_, transaction_);
    for (Lane& l : lanes_)
        if (l.table->in_flight_ == transaction_) l.table->in_flight_ = 0;
    finalized_ = true;
}

}  // namespace mk
